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
