// Attention whose heads talk before the softmax: the scores of all heads for one (query, key)
// pair are mixed by a matrix T [heads][heads] before the window's softmax,
//     s^g_ij = (q^g_i . k_j) * scale,   s'^h_ij = sum_g T[h][g] s^g_ij,
//     j visible from i iff 0 <= i - j < window (window 0: every j <= i),
//     o^h_i = sum_j softmax_j(s'^h_ij) v_j,  times sigmoid(gate[i][h]) if a gate is given.
// So a block cannot own one head: it owns a query with ALL its heads and walks the visible keys in
// tiles of 32.  Per tile: (A) raw scores of every head, a thread per (key/value head, key) doing the
// dot products of that head's group of query heads; (B) the mix, a thread per (head, key); (C) the
// running softmax, a warp per head; (D) the value sums, a thread per output element.  Scores,
// mixing and softmax are float32 in both precisions.
//
// Keys and values come either from the step's own packed rows (position j of batch row b at token
// cu_seqlens[b] + j) or from the paged cache ([page][kv head][64][width], position p at p % ring
// when the group is a ring).  With `splits` > 1 a query's keys are cut into that many stretches, each
// a block of its own that leaves (max, sum, unnormalised values) per head in scratch memory, and
// talk_combine merges them: single queries over long windows then fill the GPU.
//
//   value_mix     v <- (1 - lam) v + lam v_first on the float32 projection rows, before the
//                 values are rounded and cached
#include "common.cuh"

#define TA_KEYS 32
#define TA_THREADS 128
#define TA_MAX_ACC 32          // output elements a thread may own: heads * vd <= 32 * TA_THREADS

template <typename T> struct TaVec;
template <> struct TaVec<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct TaVec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

struct TalkArgs {
    const void* q;            // [rows][heads][hd]
    const void* k;            // packed [tokens][n_kv][hd] or pages [page][n_kv][64][hd]
    const void* v;            // packed [tokens][n_kv][vd] or pages [page][n_kv][64][vd]
    const int* row_seq;       // [rows] batch row of each query
    const int* row_pos;       // [rows] absolute position of each query
    const int* cu_seqlens;    // packed source
    const int* page_table;    // paged source
    int table_stride, ring;
    const float* talk;        // [heads][heads]
    const float* gate;        // raw gate: gate[row * gate_width + gate_off + head], or null
    long long gate_width;
    int gate_off;
    void* out;                // [rows][heads * vd]
    float* scratch;           // splits > 1: [rows][splits][heads][vd + 2]
    int rows, heads, n_kv, hd, vd, window, splits;
    float scale;
    // the tiled kernel only: the queries' row starts, the rows, the most 16-query tiles a row has,
    // the cluster's size and the most key/value heads one block of it reads
    const int* q_cu;
    int n_seq, max_q_tiles, cluster, nkv, raw_bufs;
};

template <typename T, bool PAGED, bool VEC, int NACC>
__global__ void __launch_bounds__(TA_THREADS) talk_attention_kernel(TalkArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float ta_smem[];
    const int H = a.heads, G = a.n_kv, hd = a.hd, vd = a.vd, R = H / G;
    float* q_s = ta_smem;                       // [H][hd], scaled
    float* talk_s = q_s + H * hd;               // [H][H]
    float* raw_s = talk_s + H * H;              // [H][33]
    float* p_s = raw_s + H * (TA_KEYS + 1);     // [H][33]
    float* m_s = p_s + H * (TA_KEYS + 1);       // [H]
    float* l_s = m_s + H;                       // [H]
    float* alpha_s = l_s + H;                   // [H]
    const int n_floats = H * hd + H * H + 2 * H * (TA_KEYS + 1) + 3 * H;
    long long* base_s = reinterpret_cast<long long*>(ta_smem + n_floats + (n_floats & 1));   // [32]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x, split = blockIdx.y;
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    const long long packed0 = PAGED ? 0 : (long long)a.cu_seqlens[b];
    for (int i = tid; i < H * H; i += TA_THREADS) talk_s[i] = a.talk[i];
    for (int i = tid; i < H; i += TA_THREADS) { m_s[i] = -INFINITY; l_s[i] = 0.f; alpha_s[i] = 0.f; }
    pdl_wait();
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    int hi = pos + 1;
    if (a.splits > 1) {
        const int per = (((hi - lo + a.splits - 1) / a.splits + TA_KEYS - 1) / TA_KEYS) * TA_KEYS;
        lo = lo + split * per;
        hi = min(hi, lo + per);
    }
    const T* qg = (const T*)a.q + (size_t)row * H * hd;
    for (int i = tid; i < H * hd; i += TA_THREADS) q_s[i] = to_f32(qg[i]) * a.scale;
    const T* kbase = (const T*)a.k;
    const T* vbase = (const T*)a.v;
    const long long head_rows = PAGED ? MF_PAGE : 1;    // rows between two kv heads of one position

    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

    for (int j0 = lo; j0 < hi; j0 += TA_KEYS) {
        const int n_here = min(TA_KEYS, hi - j0);
        __syncthreads();                                   // the tile before is used up
        if (tid < TA_KEYS) {
            const int j = j0 + tid;
            long long base = 0;
            if (tid < n_here) {
                if (PAGED) {
                    const int p_eff = a.ring > 0 ? j % a.ring : j;
                    const int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
                    base = (long long)page * G * MF_PAGE + (p_eff & (MF_PAGE - 1));
                } else {
                    base = (packed0 + j) * G;
                }
            }
            base_s[tid] = base;
        }
        __syncthreads();
        // (A) raw scores: a thread per (kv head, key), the group's query heads four at a time
        for (int item = tid; item < G * TA_KEYS; item += TA_THREADS) {
            const int c = item / TA_KEYS, jj = item - c * TA_KEYS;
            if (jj < n_here) {
                const T* kr = kbase + (base_s[jj] + c * head_rows) * hd;
                for (int r0 = 0; r0 < R; r0 += 4) {
                    float dot[4] = {0.f, 0.f, 0.f, 0.f};
                    const float* qh = q_s + (size_t)(c * R + r0) * hd;
                    if (VEC) {
                        for (int d = 0; d < hd; d += TaVec<T>::N) {
                            float kv[TaVec<T>::N];
                            TaVec<T>::load(kr + d, kv);
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                if (r0 + r < R) {
#pragma unroll
                                    for (int e = 0; e < TaVec<T>::N; ++e)
                                        dot[r] = fmaf(qh[r * hd + d + e], kv[e], dot[r]);
                                }
                            }
                        }
                    } else {
                        for (int d = 0; d < hd; ++d) {
                            const float kv = to_f32(kr[d]);
#pragma unroll
                            for (int r = 0; r < 4; ++r)
                                if (r0 + r < R) dot[r] = fmaf(qh[r * hd + d], kv, dot[r]);
                        }
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        if (r0 + r < R) raw_s[(c * R + r0 + r) * (TA_KEYS + 1) + jj] = dot[r];
                }
            }
        }
        __syncthreads();
        // (B) the heads talk: a thread per (head, key)
        for (int item = tid; item < H * TA_KEYS; item += TA_THREADS) {
            const int h = item / TA_KEYS, jj = item - h * TA_KEYS;
            float s = -INFINITY;
            if (jj < n_here) {
                s = 0.f;
                for (int g = 0; g < H; ++g) s = fmaf(talk_s[h * H + g], raw_s[g * (TA_KEYS + 1) + jj], s);
            }
            p_s[h * (TA_KEYS + 1) + jj] = s;
        }
        __syncthreads();
        // (C) running softmax: a warp per head
        for (int h = warp; h < H; h += TA_THREADS / 32) {
            const float s = p_s[h * (TA_KEYS + 1) + lane];
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float corr = expf(m_old - m_new);        // 0 on the first tile
            const float p = lane < n_here ? expf(s - m_new) : 0.f;
            const float sum = warp_sum(p);
            p_s[h * (TA_KEYS + 1) + lane] = p;
            if (lane == 0) { m_s[h] = m_new; l_s[h] = l_s[h] * corr + sum; alpha_s[h] = corr; }
        }
        __syncthreads();
        // (D) values: a thread per output element (head, value dimension)
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int idx = tid + i * TA_THREADS;
            if (idx < H * vd) {
                const int h = idx / vd, dv = idx - h * vd;
                const int c = h / R;
                float s = acc[i] * alpha_s[h];
                const float* ph = p_s + h * (TA_KEYS + 1);
                for (int jj = 0; jj < n_here; ++jj)
                    s = fmaf(ph[jj], to_f32(vbase[(base_s[jj] + c * head_rows) * vd + dv]), s);
                acc[i] = s;
            }
        }
    }
    __syncthreads();
    if (a.splits > 1) {
        float* sc = a.scratch + ((size_t)row * a.splits + split) * H * (vd + 2);
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int idx = tid + i * TA_THREADS;
            if (idx < H * vd) {
                const int h = idx / vd, dv = idx - h * vd;
                sc[(size_t)h * (vd + 2) + dv] = acc[i];
            }
        }
        for (int h = tid; h < H; h += TA_THREADS) {
            sc[(size_t)h * (vd + 2) + vd] = m_s[h];
            sc[(size_t)h * (vd + 2) + vd + 1] = l_s[h];
        }
        return;
    }
    T* o = (T*)a.out + (size_t)row * H * vd;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int idx = tid + i * TA_THREADS;
        if (idx < H * vd) {
            const int h = idx / vd;
            float g = 1.0f;
            if (a.gate) g = 1.0f / (1.0f + expf(-a.gate[(size_t)row * a.gate_width + a.gate_off + h]));
            o[idx] = from_f32<T>(acc[i] / l_s[h] * g);
        }
    }
}

// merges the stretches of a query: a thread per output element
template <typename T>
__global__ void __launch_bounds__(256) talk_combine_kernel(TalkArgs a) {
    pdl_prologue();
    const int H = a.heads, vd = a.vd;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)a.rows * H * vd) return;
    const int row = (int)(idx / (H * vd));
    const int rem = (int)(idx - (long long)row * H * vd);
    const int h = rem / vd, dv = rem - h * vd;
    const float* sc = a.scratch + (size_t)row * a.splits * H * (vd + 2) + (size_t)h * (vd + 2);
    const size_t step = (size_t)H * (vd + 2);
    float m = -INFINITY;
    for (int s = 0; s < a.splits; ++s) m = fmaxf(m, sc[s * step + vd]);
    float l = 0.f, o = 0.f;
    for (int s = 0; s < a.splits; ++s) {
        const float ms = sc[s * step + vd];
        if (ms == -INFINITY) continue;                   // a stretch without keys
        const float w = expf(ms - m);
        l = fmaf(sc[s * step + vd + 1], w, l);
        o = fmaf(sc[s * step + dv], w, o);
    }
    float g = 1.0f;
    if (a.gate) g = 1.0f / (1.0f + expf(-a.gate[(size_t)row * a.gate_width + a.gate_off + h]));
    ((T*)a.out)[idx] = from_f32<T>(o / l * g);
}

static size_t talk_smem(const TalkArgs& a) {
    const size_t floats = (size_t)a.heads * a.hd + (size_t)a.heads * a.heads
                          + 2 * (size_t)a.heads * (TA_KEYS + 1) + 3 * (size_t)a.heads + 1;
    return floats * sizeof(float) + TA_KEYS * sizeof(long long);
}

template <typename T, bool PAGED, bool VEC, int NACC>
static void talk_launch_one(const TalkArgs& a, size_t smem, cudaStream_t stream) {
    static bool raised = false;          // once, outside any capture (a shape's first step)
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute(talk_attention_kernel<T, PAGED, VEC, NACC>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        raised = true;
    }
    mf_launch(talk_attention_kernel<T, PAGED, VEC, NACC>, dim3(a.rows, a.splits), dim3(TA_THREADS),
              smem, stream, a);
}

template <typename T, bool PAGED>
static int talk_launch(const TalkArgs& a, cudaStream_t stream) {
    const size_t smem = talk_smem(a);
    if (smem > 160 * 1024) return MF_ERR_UNSUPPORTED;
    const int per_thread = (a.heads * a.vd + TA_THREADS - 1) / TA_THREADS;
    if (per_thread > TA_MAX_ACC) return MF_ERR_UNSUPPORTED;
    const bool vec = a.hd % TaVec<T>::N == 0;
#define MF_TALK(NACC) \
    do { \
        if (vec) talk_launch_one<T, PAGED, true, NACC>(a, smem, stream); \
        else talk_launch_one<T, PAGED, false, NACC>(a, smem, stream); \
    } while (0)
    if (per_thread <= 4) MF_TALK(4);
    else if (per_thread <= 16) MF_TALK(16);
    else MF_TALK(TA_MAX_ACC);
#undef MF_TALK
    if (a.splits > 1) {
        const long long n = (long long)a.rows * a.heads * a.vd;
        mf_launch(talk_combine_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, a);
    }
    return MF_LAUNCH_CHECK();
}

// floats of scratch a call with `splits` stretches needs
extern "C" long long mf_talk_attention_scratch(int rows, int heads, int vd, int splits) {
    return splits > 1 ? (long long)rows * splits * heads * (vd + 2) : 0;
}

extern "C" int mf_talk_attention(const TalkArgs* args, int paged, int dtype, cudaStream_t stream) {
    TalkArgs a = *args;
    if (a.rows <= 0) return 0;
    if (a.heads < 1 || a.n_kv < 1 || a.heads % a.n_kv != 0 || a.window < 0 || a.splits < 1)
        return MF_ERR_ARGUMENT;
    if (a.hd < 1 || a.vd < 1) return MF_ERR_UNSUPPORTED;
    if (a.splits > 1 && a.scratch == nullptr) return MF_ERR_ARGUMENT;
    if (paged && a.page_table == nullptr) return MF_ERR_ARGUMENT;
    if (!paged && a.cu_seqlens == nullptr) return MF_ERR_ARGUMENT;
    if (dtype == MF_DTYPE_F32)
        return paged ? talk_launch<float, true>(a, stream) : talk_launch<float, false>(a, stream);
    if (dtype == MF_DTYPE_BF16)
        return paged ? talk_launch<__nv_bfloat16, true>(a, stream)
                     : talk_launch<__nv_bfloat16, false>(a, stream);
    return MF_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------
// v <- (1 - lam) v + lam v_first over `width` columns of float32 rows (lam read on the device)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
value_mix_kernel(float* __restrict__ v, long long v_width, int v_off,
                 const float* __restrict__ first, long long first_width, int first_off,
                 const float* __restrict__ lam, long long total, int width) {
    pdl_launch_dependents();
    const float l = lam[0];
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / width;
        const int c = (int)(i - t * width);
        float* p = v + t * v_width + v_off + c;
        *p = (1.0f - l) * *p + l * first[t * first_width + first_off + c];
    }
}

extern "C" int mf_value_mix(float* v, long long v_width, int v_off, const float* first,
                            long long first_width, int first_off, const float* lam, int n_tokens,
                            int width, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return 0;
    const long long total = (long long)n_tokens * width;
    const long long want = (total + 255) / 256, cap = (long long)mf_sm_count() * 8;
    mf_launch(value_mix_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, v,
              v_width, v_off, first, first_width, first_off, lam, total, width);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// Rows of several tokens, bfloat16: tiles of 16 queries on the tensor cores, the heads spread
// over a thread-block cluster.
//
// The mix needs every head's raw score of a (query, key) pair, but one block cannot hold the
// queries and the output sums of all heads.  So a cluster of CS blocks shares a tile of 16 queries:
// block r owns the heads [r H/CS, (r + 1) H/CS).  Per tile of 32 keys it
//   (1) computes the raw scores of its own heads (mma.sync m16n8k16, bfloat16 in, float32 out) into
//       its shared memory, which the whole cluster can read;
//   (2) after a cluster barrier, mixes for its own heads: 8 threads a query, 4 keys a thread, a
//       loop over all heads g whose raw scores come from the owner's shared memory (ld.shared::cluster),
//       then the window's mask and the running softmax, all in float32; the weights go to shared
//       memory as bfloat16, the second operand of the value product;
//   (3) adds weights x values to the output sums it keeps in registers (mma.sync again).
// Raw scores have two buffers, so one cluster barrier a tile is enough: a block that overwrites
// buffer t % 2 has passed the barrier of tile t - 1, which every block reaches only after its mix
// of tile t - 2.  Keys and values of the next tile arrive by cp.async (zero-filled outside the
// visible stretch) while the current one is worked on.
// With `splits` > 1 the key tiles are dealt to that many clusters, which leave (sums, max, sum) in
// scratch memory for talk_combine, as the kernel above does.
// ------------------------------------------------------------------------------------------
#define TT_BM 16
#define TT_BN 32
#define TT_THREADS 128
#define TT_WARPS 4
#define TT_MAX_NT 16            // tiles of 8 output columns a warp may own
#define TT_RAW_LD (TT_BN + 8)   // floats: rows 8 banks apart, so a half warp's float2 stores do not collide
#define TT_P_LD (TT_BN + 8)     // bfloat16
#define TT_MAX_SMEM (200 * 1024)

__device__ __forceinline__ uint32_t tt_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void tt_ldsm(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void tt_ldsm_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void tt_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes, or zeros when bytes == 0 (the source must still be an address that exists)
__device__ __forceinline__ void tt_cp16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ uint32_t tt_mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 tt_ld_cluster(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void tt_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// bytes of shared memory a block needs
__host__ __device__ inline size_t talk_tile_smem(int H, int cs, int nkv, int hd, int vd, int raw_bufs) {
    const size_t hpc = H / cs, hpcp = (hpc + 3) & ~(size_t)3;
    size_t b = hpc * TT_BM * (hd + 8) * 2;                       // queries
    b += 2 * (size_t)nkv * TT_BN * (hd + 8) * 2;                 // keys, two stages
    b += 2 * (size_t)nkv * TT_BN * (vd + 8) * 2;                 // values, two stages
    b += hpc * TT_BM * TT_P_LD * 2;                              // weights
    b += raw_bufs * hpc * TT_BM * TT_RAW_LD * 4;                 // raw scores, one or two buffers
    b += (size_t)H * hpcp * 4;                                   // the own heads' rows of T, transposed
    b += 3 * hpc * TT_BM * 4;                                    // max, sum, correction
    b += TT_BM * 4 + 2 * TT_BN * 8;                              // positions, key bases
    b += hpcp * 4;                                               // the own heads' key/value heads
    return b;
}

// HPC_T: the heads a block owns when known at compile time (4, the usual share), else 0
template <bool PAGED, int HPC_T>
__global__ void __launch_bounds__(TT_THREADS) talk_tile_kernel(TalkArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char tt_smem[];
    typedef __nv_bfloat16 bf16;
    const int H = a.heads, G = a.n_kv, R = H / G, hd = a.hd, vd = a.vd;
    const int CS = a.cluster, HPC = HPC_T ? HPC_T : H / CS, HPCP = (HPC + 3) & ~3, NKV = a.nkv;
    const int q_ld = hd + 8, v_ld = vd + 8;
    bf16* q_s = reinterpret_cast<bf16*>(tt_smem);                      // [HPC][16][q_ld]
    bf16* k_s = q_s + (size_t)HPC * TT_BM * q_ld;                      // [2][NKV][32][q_ld]
    bf16* v_s = k_s + 2 * (size_t)NKV * TT_BN * q_ld;                  // [2][NKV][32][v_ld]
    bf16* p_s = v_s + 2 * (size_t)NKV * TT_BN * v_ld;                  // [HPC][16][TT_P_LD]
    float* raw_s = reinterpret_cast<float*>(p_s + (size_t)HPC * TT_BM * TT_P_LD);   // [2][HPC][16][TT_RAW_LD]
    float* tt_s = raw_s + (size_t)a.raw_bufs * HPC * TT_BM * TT_RAW_LD;   // [H][HPCP]: T[h0 + hl][g] * scale
    float* m_s = tt_s + (size_t)H * HPCP;                              // [HPC][16]
    float* l_s = m_s + HPC * TT_BM;
    float* alpha_s = l_s + HPC * TT_BM;
    int* pos_s = reinterpret_cast<int*>(alpha_s + HPC * TT_BM);        // [16]
    long long* base_s = reinterpret_cast<long long*>(pos_s + TT_BM);   // [2][32], -1: not visible
    int* kvh_s = reinterpret_cast<int*>(base_s + 2 * TT_BN);           // [HPC] key/value head - c_lo

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rank = blockIdx.x;                      // the cluster runs along x and is the grid's x
    // the last tiles of a row see the most keys: they start first
    const int tile = a.max_q_tiles - 1 - blockIdx.y / a.splits, split = blockIdx.y % a.splits;
    const int b = blockIdx.z;
    const int h0 = rank * HPC;
    const int c_lo = h0 / R, c_hi = (h0 + HPC - 1) / R;

    for (int i = tid; i < H * HPCP; i += TT_THREADS) {
        const int g = i / HPCP, hl = i - g * HPCP;
        tt_s[i] = hl < HPC ? a.talk[(size_t)(h0 + hl) * H + g] * a.scale : 0.f;
    }
    for (int i = tid; i < HPC * TT_BM; i += TT_THREADS) { m_s[i] = -INFINITY; l_s[i] = 0.f; alpha_s[i] = 0.f; }
    for (int i = tid; i < HPC; i += TT_THREADS) kvh_s[i] = (h0 + i) / R - c_lo;
    pdl_wait();
    const int q0 = a.q_cu[b] + tile * TT_BM, q_end = a.q_cu[b + 1];
    if (q0 >= q_end) return;                          // the whole cluster leaves
    const int nq = min(TT_BM, q_end - q0);
    if (tid < TT_BM) pos_s[tid] = a.row_pos[q0 + min(tid, nq - 1)];
    {
        const bf16* qg = reinterpret_cast<const bf16*>(a.q);
        const int c8 = hd >> 3;
        for (int idx = tid; idx < HPC * TT_BM * c8; idx += TT_THREADS) {
            const int hl = idx / (TT_BM * c8), rem = idx - hl * TT_BM * c8;
            const int i = rem / c8, ch = rem - i * c8;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (i < nq) val = *reinterpret_cast<const uint4*>(qg + ((size_t)(q0 + i) * H + h0 + hl) * hd + ch * 8);
            *reinterpret_cast<uint4*>(q_s + ((size_t)hl * TT_BM + i) * q_ld + ch * 8) = val;
        }
    }
    __syncthreads();
    const int pos_first = pos_s[0], pos_last = pos_s[TT_BM - 1];
    const int lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    const int hi = pos_last + 1;
    const int lo_t = lo & ~(TT_BN - 1);
    const int n_tiles = (hi - lo_t + TT_BN - 1) / TT_BN;
    int t_begin = 0, t_end = n_tiles;
    if (a.splits > 1) {
        const int per = (n_tiles + a.splits - 1) / a.splits;
        t_begin = split * per;
        t_end = min(n_tiles, t_begin + per);
    }
    const long long packed0 = PAGED ? 0 : (long long)a.cu_seqlens[b];
    const long long head_rows = PAGED ? MF_PAGE : 1;
    const bf16* kbase = reinterpret_cast<const bf16*>(a.k);
    const bf16* vbase = reinterpret_cast<const bf16*>(a.v);

    auto key_base = [&](int j) -> long long {
        if (j < lo || j >= hi) return -1;
        if (PAGED) {
            const int p_eff = a.ring > 0 ? j % a.ring : j;
            const int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
            return (long long)page * G * MF_PAGE + (p_eff & (MF_PAGE - 1));
        }
        return (packed0 + j) * G;
    };
    auto issue = [&](int stage) {
        const long long* bs = base_s + stage * TT_BN;
        const int nkv_here = c_hi - c_lo + 1;
        const int c8 = hd >> 3, cv8 = vd >> 3;
        // a row of keys and of values a warp at a time, its 16-byte pieces over the lanes
        for (int r = warp; r < nkv_here * TT_BN; r += TT_WARPS) {
            const int cl = r / TT_BN, jj = r - cl * TT_BN;
            const long long base = bs[jj];
            const int bytes = base >= 0 ? 16 : 0;
            const bf16* ksrc = base >= 0 ? kbase + (base + (c_lo + cl) * head_rows) * hd : kbase;
            const bf16* vsrc = base >= 0 ? vbase + (base + (c_lo + cl) * head_rows) * vd : vbase;
            const uint32_t kd = tt_u32(k_s + (((size_t)stage * NKV + cl) * TT_BN + jj) * q_ld);
            const uint32_t vdst = tt_u32(v_s + (((size_t)stage * NKV + cl) * TT_BN + jj) * v_ld);
            for (int ch = lane; ch < c8; ch += 32) tt_cp16(kd + ch * 16, base >= 0 ? ksrc + ch * 8 : ksrc, bytes);
            for (int ch = lane; ch < cv8; ch += 32) tt_cp16(vdst + ch * 16, base >= 0 ? vsrc + ch * 8 : vsrc, bytes);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // the output sums: this warp's share of the block's (head, 8 columns) tiles
    const int NTV = vd >> 3, n_out = HPC * NTV, out_per = (n_out + TT_WARPS - 1) / TT_WARPS;
    const int out_first = warp * out_per, out_cnt = max(0, min(out_per, n_out - out_first));
    const int out_hl0 = out_first / NTV, out_nt0 = out_first - out_hl0 * NTV;
    float o[TT_MAX_NT][4];
#pragma unroll
    for (int u = 0; u < TT_MAX_NT; ++u) { o[u][0] = 0.f; o[u][1] = 0.f; o[u][2] = 0.f; o[u][3] = 0.f; }

    if (t_begin < t_end) {
        if (tid < TT_BN) base_s[tid] = key_base(lo_t + t_begin * TT_BN + tid);
        __syncthreads();
        issue(0);
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int s = (t - t_begin) & 1;
        const int sr = a.raw_bufs > 1 ? s : 0;           // the raw scores' buffer
        if (t + 1 < t_end && tid < TT_BN)
            base_s[(s ^ 1) * TT_BN + tid] = key_base(lo_t + (t + 1) * TT_BN + tid);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                  // tile t is here; the other stage and its bases are free
        if (t + 1 < t_end) issue(s ^ 1);
        // (1) raw scores of the own heads: a warp per head, 16 queries x 32 keys
        for (int hl = warp; hl < HPC; hl += TT_WARPS) {
            const int cl = kvh_s[hl];
            float sc[4][4];
#pragma unroll
            for (int n = 0; n < 4; ++n) { sc[n][0] = 0.f; sc[n][1] = 0.f; sc[n][2] = 0.f; sc[n][3] = 0.f; }
            const uint32_t qa = tt_u32(q_s + ((size_t)hl * TT_BM + (lane & 15)) * q_ld + (lane >> 4) * 8);
            const uint32_t ka = tt_u32(k_s + (((size_t)s * NKV + cl) * TT_BN + (lane >> 4) * 8 + (lane & 7)) * q_ld
                                       + ((lane >> 3) & 1) * 8);
#pragma unroll 2
            for (int ks = 0; ks < (hd >> 4); ++ks) {
                uint32_t af[4], b0[4], b1[4];
                tt_ldsm(qa + ks * 32, af);
                tt_ldsm(ka + ks * 32, b0);                              // keys 0 .. 15
                tt_ldsm(ka + 16 * q_ld * 2 + ks * 32, b1);              // keys 16 .. 31
                tt_mma(sc[0], af, b0[0], b0[1]);
                tt_mma(sc[1], af, b0[2], b0[3]);
                tt_mma(sc[2], af, b1[0], b1[1]);
                tt_mma(sc[3], af, b1[2], b1[3]);
            }
            float* rw = raw_s + ((size_t)sr * HPC + hl) * TT_BM * TT_RAW_LD;
            const int r = lane >> 2, c = 2 * (lane & 3);
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                *reinterpret_cast<float2*>(rw + r * TT_RAW_LD + n * 8 + c) = make_float2(sc[n][0], sc[n][1]);
                *reinterpret_cast<float2*>(rw + (r + 8) * TT_RAW_LD + n * 8 + c) = make_float2(sc[n][2], sc[n][3]);
            }
        }
        tt_cluster_sync();                // every block's raw scores of tile t can be read
        // (2) the mix, the mask and the running softmax of the own heads
        {
            const int i = tid >> 3, jq = tid & 7;
            const int jb = lo_t + t * TT_BN + 4 * jq;
            const int pos_i = pos_s[i];
            bool vis[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = jb + e;
                vis[e] = i < nq && j <= pos_i && (a.window == 0 || pos_i - j < a.window);
            }
            const uint32_t mine = tt_u32(raw_s + ((size_t)sr * HPC * TT_BM + i) * TT_RAW_LD + 4 * jq);
            for (int hc = 0; hc < HPCP; hc += 4) {
                float acc[4][4];
#pragma unroll
                for (int x = 0; x < 4; ++x) { acc[x][0] = 0.f; acc[x][1] = 0.f; acc[x][2] = 0.f; acc[x][3] = 0.f; }
#pragma unroll 2
                for (int src = 0; src < CS; ++src) {
                    const uint32_t ra = tt_mapa(mine, (uint32_t)src);
                    const float* tt = tt_s + (size_t)src * HPC * HPCP + hc;
#pragma unroll 4
                    for (int gl = 0; gl < HPC; ++gl) {
                        const float4 rv = tt_ld_cluster(ra + gl * TT_BM * TT_RAW_LD * 4);
                        const float4 tv = *reinterpret_cast<const float4*>(tt + gl * HPCP);
                        const float tw[4] = {tv.x, tv.y, tv.z, tv.w};
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            acc[x][0] = fmaf(tw[x], rv.x, acc[x][0]);
                            acc[x][1] = fmaf(tw[x], rv.y, acc[x][1]);
                            acc[x][2] = fmaf(tw[x], rv.z, acc[x][2]);
                            acc[x][3] = fmaf(tw[x], rv.w, acc[x][3]);
                        }
                    }
                }
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int hl = hc + x;
                    if (hl < HPC) {                                   // the same for every thread
                        const float m_old = m_s[hl * TT_BM + i];
                        float sv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) sv[e] = vis[e] ? acc[x][e] : -INFINITY;
                        float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        const float m_new = fmaxf(m_old, mx);
                        const float m_use = m_new == -INFINITY ? 0.f : m_new;   // no key seen yet
                        const float corr = __expf(m_old - m_use);
                        float pv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) pv[e] = __expf(sv[e] - m_use);
                        float sum = (pv[0] + pv[1]) + (pv[2] + pv[3]);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                        __nv_bfloat162 p01 = __floats2bfloat162_rn(pv[0], pv[1]);
                        __nv_bfloat162 p23 = __floats2bfloat162_rn(pv[2], pv[3]);
                        uint2 pk;
                        pk.x = *reinterpret_cast<uint32_t*>(&p01);
                        pk.y = *reinterpret_cast<uint32_t*>(&p23);
                        *reinterpret_cast<uint2*>(p_s + ((size_t)hl * TT_BM + i) * TT_P_LD + 4 * jq) = pk;
                        if (jq == 0) {
                            m_s[hl * TT_BM + i] = m_new;
                            l_s[hl * TT_BM + i] = l_s[hl * TT_BM + i] * corr + sum;
                            alpha_s[hl * TT_BM + i] = corr;
                        }
                    }
                }
            }
        }
        if (a.raw_bufs > 1) __syncthreads();
        else tt_cluster_sync();           // one buffer: nobody may still read it when it is written again
        // (3) weights x values into the output sums
        if (HPC_T == TT_WARPS && NTV == TT_MAX_NT) {
            // the usual share: head `warp`, all 16 column tiles
            uint32_t pa0[4], pa1[4];
            const uint32_t pa = tt_u32(p_s + ((size_t)warp * TT_BM + (lane & 15)) * TT_P_LD + (lane >> 4) * 8);
            tt_ldsm(pa, pa0);
            tt_ldsm(pa + 32, pa1);
            const float al0 = alpha_s[warp * TT_BM + (lane >> 2)];
            const float al1 = alpha_s[warp * TT_BM + (lane >> 2) + 8];
            const uint32_t v_head = tt_u32(v_s + (((size_t)s * NKV + kvh_s[warp]) * TT_BN + lane) * v_ld);
#pragma unroll
            for (int u = 0; u < TT_MAX_NT; ++u) {
                uint32_t vb[4];
                tt_ldsm_t(v_head + u * 16, vb);
                o[u][0] *= al0; o[u][1] *= al0; o[u][2] *= al1; o[u][3] *= al1;
                tt_mma(o[u], pa0, vb[0], vb[1]);
                tt_mma(o[u], pa1, vb[2], vb[3]);
            }
        } else {
            int cur = -1, hl = out_hl0, nt = out_nt0;
            uint32_t pa0[4], pa1[4];
            float al0 = 1.f, al1 = 1.f;
            const uint32_t p_lane = tt_u32(p_s + (lane & 15) * TT_P_LD + (lane >> 4) * 8);
            const uint32_t v_lane = tt_u32(v_s + ((size_t)s * NKV * TT_BN + lane) * v_ld);
            const uint32_t v_head_bytes = (uint32_t)(TT_BN * v_ld * 2);
            uint32_t v_head = v_lane;
#pragma unroll
            for (int u = 0; u < TT_MAX_NT; ++u) {
                if (u < out_cnt) {
                    if (hl != cur) {
                        const uint32_t pa = p_lane + (uint32_t)hl * (TT_BM * TT_P_LD * 2);
                        v_head = v_lane + (uint32_t)kvh_s[hl] * v_head_bytes;
                        tt_ldsm(pa, pa0);
                        tt_ldsm(pa + 32, pa1);
                        al0 = alpha_s[hl * TT_BM + (lane >> 2)];
                        al1 = alpha_s[hl * TT_BM + (lane >> 2) + 8];
                        cur = hl;
                    }
                    uint32_t vb[4];
                    tt_ldsm_t(v_head + (uint32_t)nt * 16, vb);
                    o[u][0] *= al0; o[u][1] *= al0; o[u][2] *= al1; o[u][3] *= al1;
                    tt_mma(o[u], pa0, vb[0], vb[1]);
                    tt_mma(o[u], pa1, vb[2], vb[3]);
                    if (++nt == NTV) { nt = 0; ++hl; }
                }
            }
        }
    }
    tt_cluster_sync();                    // nobody reads this block's raw scores any more
    {
        const int r = lane >> 2, c2 = 2 * (lane & 3);
        int hl = out_hl0, nt = out_nt0;
#pragma unroll
        for (int u = 0; u < TT_MAX_NT; ++u) {
            if (u < out_cnt) {
                const int h = h0 + hl, col = nt * 8 + c2;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int i = r + 8 * half;
                    if (i < nq) {
                        const size_t row = (size_t)(q0 + i);
                        const float v0 = o[u][2 * half], v1 = o[u][2 * half + 1];
                        if (a.splits > 1) {
                            float* sc = a.scratch + ((row * a.splits + split) * H + h) * (vd + 2);
                            sc[col] = v0;
                            sc[col + 1] = v1;
                        } else {
                            float g = 1.0f;
                            if (a.gate) g = 1.0f / (1.0f + expf(-a.gate[row * a.gate_width + a.gate_off + h]));
                            const float inv = g / l_s[hl * TT_BM + i];
                            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(a.out) + (row * H + h) * vd + col)
                                = __floats2bfloat162_rn(v0 * inv, v1 * inv);
                        }
                    }
                }
                if (++nt == NTV) { nt = 0; ++hl; }
            }
        }
        if (a.splits > 1) {
            for (int idx = tid; idx < HPC * TT_BM; idx += TT_THREADS) {
                const int hl = idx / TT_BM, i = idx - hl * TT_BM;
                if (i < nq) {
                    float* sc = a.scratch + (((size_t)(q0 + i) * a.splits + split) * H + h0 + hl) * (vd + 2);
                    sc[vd] = m_s[idx];
                    sc[vd + 1] = l_s[idx];
                }
            }
        }
    }
}

// the cluster's size for a shape: the most blocks that still leave each at least 4 heads;
// 0 when the tiled kernel does not take the shape
static int talk_tile_cluster(int heads, int n_kv, int hd, int vd, int* nkv_out) {
    if (heads < 1 || n_kv < 1 || heads % n_kv != 0 || hd < 16 || hd % 16 != 0 || vd < 8 || vd % 8 != 0)
        return 0;
    int cs = 1;
    for (int c = 8; c >= 1; c >>= 1)
        if (heads % c == 0 && heads / c >= 4) { cs = c; break; }
    const int hpc = heads / cs, R = heads / n_kv;
    if (hpc * (vd / 8) > TT_MAX_NT * TT_WARPS) return 0;
    int nkv = 1;
    for (int r = 0; r < cs; ++r) {
        const int span = (r * hpc + hpc - 1) / R - (r * hpc) / R + 1;
        if (span > nkv) nkv = span;
    }
    if (talk_tile_smem(heads, cs, nkv, hd, vd, 1) > TT_MAX_SMEM) return 0;
    if (nkv_out) *nkv_out = nkv;
    return cs;
}

// blocks of the cluster that tiles of 16 queries run on for this shape, 0: not taken
extern "C" int mf_talk_tile_cluster(int heads, int n_kv, int hd, int vd) {
    return talk_tile_cluster(heads, n_kv, hd, vd, nullptr);
}

template <bool PAGED, int HPC_T>
static int talk_tile_launch(const TalkArgs& a, size_t smem, cudaStream_t stream) {
    static bool raised = false;          // once, outside any capture (a shape's first step)
    if (!raised) {
        cudaFuncSetAttribute(talk_tile_kernel<PAGED, HPC_T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             TT_MAX_SMEM);
        raised = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.cluster, a.max_q_tiles * a.splits, a.n_seq);
    cfg.blockDim = dim3(TT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = a.cluster;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, talk_tile_kernel<PAGED, HPC_T>, a);
    if (a.splits > 1) {
        const long long n = (long long)a.rows * a.heads * a.vd;
        mf_launch(talk_combine_kernel<__nv_bfloat16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                  stream, a);
    }
    return MF_LAUNCH_CHECK();
}

// bfloat16 only; the rows' queries are tokens q_cu[b] .. q_cu[b + 1] with consecutive positions
extern "C" int mf_talk_attention_tile(const TalkArgs* args, int paged, cudaStream_t stream) {
    TalkArgs a = *args;
    if (a.rows <= 0 || a.n_seq <= 0 || a.max_q_tiles <= 0) return 0;
    if (a.window < 0 || a.splits < 1 || a.q_cu == nullptr) return MF_ERR_ARGUMENT;
    if (a.splits > 1 && a.scratch == nullptr) return MF_ERR_ARGUMENT;
    if (paged && a.page_table == nullptr) return MF_ERR_ARGUMENT;
    if (!paged && a.cu_seqlens == nullptr) return MF_ERR_ARGUMENT;
    int nkv = 0;
    const int cs = talk_tile_cluster(a.heads, a.n_kv, a.hd, a.vd, &nkv);
    if (cs == 0) return MF_ERR_UNSUPPORTED;
    if ((long long)a.max_q_tiles * a.splits > 65535 || a.n_seq > 65535) return MF_ERR_UNSUPPORTED;
    a.cluster = cs;
    a.nkv = nkv;
    // two buffers of raw scores save a cluster barrier a tile; one, when that lets another block
    // live on the SM (three at most, by registers)
    const size_t smem2 = talk_tile_smem(a.heads, cs, nkv, a.hd, a.vd, 2);
    const size_t smem1 = talk_tile_smem(a.heads, cs, nkv, a.hd, a.vd, 1);
    const size_t per_sm = 227 * 1024;
    const size_t occ2 = smem2 > TT_MAX_SMEM ? 0 : (per_sm / (smem2 + 1024) < 3 ? per_sm / (smem2 + 1024) : 3);
    const size_t occ1 = per_sm / (smem1 + 1024) < 3 ? per_sm / (smem1 + 1024) : 3;
    a.raw_bufs = occ1 > occ2 ? 1 : 2;
    const size_t smem = a.raw_bufs == 1 ? smem1 : smem2;
    if (a.heads / cs == 4)
        return paged ? talk_tile_launch<true, 4>(a, smem, stream) : talk_tile_launch<false, 4>(a, smem, stream);
    return paged ? talk_tile_launch<true, 0>(a, smem, stream) : talk_tile_launch<false, 0>(a, smem, stream);
}
