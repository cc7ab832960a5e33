// Attention whose scores are changed before the softmax and whose softmax has a sink.
//
// For query head h (key/value head h / (n_heads / n_kv)), a query at position i and a key at
// position j:
//     s_ij = (q_i . k_j) * scale - r1[h] * ln(1 + r2[h] * (i - j))        (r1 == nullptr: no bias)
//     j is visible from i  iff  j <= i
//                          and  i - j < window                 (window > 0)
//                          and  floor(i / chunk) == floor(j / chunk)   (chunk > 0; counted from
//                                                               position 0 of the sequence)
//     w_ij = exp(s_ij) / (sink + sum over visible j' of exp(s_ij'))       (sink is 0 or 1: a key
//                                                               of score 0 that has no value)
// Two further changes of the score, both optional: a soft cap, s <- cap * tanh(s / cap), applied
// to (q . k) * scale before the bias (cap > 0), and a learned score of the sink per head
// (sink_logit[h] instead of 0: the denominator holds exp(sink_logit[h]) once).
//     o_i = sum_j w_ij v_j
// Keys have `hd` elements a head, values `vd`; the two differ freely.  Scores, the bias, the
// running maximum and sum, and the weighted sum are float32.
//
// Kernels here:
//   * unit_norm_kvstore: a fused q|k|v projection's float32 output (or its K splits) ->
//     q and k divided by their root mean square per head (no weight), v as it is; written
//     as the step's packed q, k, v and into the paged cache.
//   * sink_attention_generic: any sizes, float32 or bfloat16, keys from the step's packed
//     rows (whole prompts) or from the paged cache; one warp per (query, head).
//   * sink_attention_mma (further down): prompts and their portions, bfloat16 on tensor cores.
//   * sink_attention_decode (further down): single tokens over the cache, bfloat16 on tensor
//     cores, the query heads of a key/value head as the rows of the product.
#include "common.cuh"

#define SA_WARPS 4
#define SA_MAX_D 256
#define SA_GEN_MAX_D 640      // the generic kernel alone takes keys and values this wide

// ------------------------------------------------------------------------------------------
// q and k to unit root mean square per head, cache write
// ------------------------------------------------------------------------------------------
// NI: 32-element groups of a head a lane may hold (sizes up to 32 * NI)
template <typename T, int NI>
__global__ void __launch_bounds__(SA_WARPS * 32)
unit_norm_kvstore_kernel(const float* __restrict__ qkv, int n_partials, int n_tokens,
                         const int* __restrict__ positions, const int* __restrict__ token_row,
                         const int* __restrict__ seq_end, T* __restrict__ q_out,
                         T* __restrict__ k_out, T* __restrict__ v_out, T* __restrict__ k_cache,
                         T* __restrict__ v_cache, const int* __restrict__ page_table,
                         int table_stride, int ring, int n_heads, int n_kv, int hd, int vd,
                         float eps, int norm_qk, unsigned* __restrict__ status) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int b = token_row[t];
    // where this token's keys and values go in the cache: page and place in the page
    int page = -1;
    if (k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (ring > 0) {
            keep = pos >= seq_end[b] - ring;
            p_eff = pos % ring;
        }
        if (keep) {
            page = page_table[(size_t)b * table_stride + (p_eff >> 6)];
            if (page < 0 && threadIdx.x == 0 && blockIdx.y == 0)
                atomicOr(status, MF_STATUS_BAD_POSITION);
        }
    }
    pdl_wait();
    const size_t in_width = (size_t)(n_heads + n_kv) * hd + (size_t)n_kv * vd;
    const float* in = qkv + (size_t)t * in_width;
    const size_t plane = (size_t)n_tokens * in_width;
    const int n_items = n_heads + 2 * n_kv;
    // a warp takes a head: q heads, then k heads, then v heads
    for (int item = blockIdx.y * SA_WARPS + warp; item < n_items; item += gridDim.y * SA_WARPS) {
        const bool is_q = item < n_heads, is_v = item >= n_heads + n_kv;
        const int width = is_v ? vd : hd;
        const int hk = is_v ? item - n_heads - n_kv : item - n_heads;
        const size_t col0 = is_q ? (size_t)item * hd
                                 : (is_v ? (size_t)(n_heads + n_kv) * hd + (size_t)hk * vd
                                         : (size_t)(n_heads + hk) * hd);
        float val[NI];
        float ss = 0.0f;
        if (n_partials <= 1) {                           // the projection's whole sums (prompts)
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int d = lane + 32 * i;
                val[i] = d < width ? in[col0 + d] : 0.0f;
            }
        } else if (n_partials <= 16) {
            // all splits' loads of a head in flight at once (a split beyond n_partials reads the
            // last one again and adds nothing); the sums keep the split order
            const int last_split = max(n_partials, 1) - 1;
            float part[16][NI];
#pragma unroll
            for (int sp = 0; sp < 16; ++sp) {
                const float* src = in + (size_t)min(sp, last_split) * plane + col0;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int d = lane + 32 * i;
                    part[sp][i] = d < width ? src[d] : 0.0f;
                }
            }
#pragma unroll
            for (int i = 0; i < NI; ++i) val[i] = 0.0f;
#pragma unroll
            for (int sp = 0; sp < 16; ++sp) {
#pragma unroll
                for (int i = 0; i < NI; ++i) val[i] += sp <= last_split ? part[sp][i] : 0.0f;
            }
        } else {
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int d = lane + 32 * i;
                float v = 0.0f;
                if (d < width) {
                    v = in[col0 + d];
                    for (int sp = 1; sp < n_partials; ++sp) v += in[sp * plane + col0 + d];
                }
                val[i] = v;
            }
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) ss = fmaf(val[i], val[i], ss);
        float f = 1.0f;
        if (!is_v && norm_qk) {
            ss = warp_sum(ss);
            f = 1.0f / sqrtf(ss / (float)width + eps);
        }
        T* dst0 = nullptr;
        T* dst1 = nullptr;
        if (is_q) {
            dst0 = q_out + ((size_t)t * n_heads + item) * hd;
        } else {
            T* step_out = is_v ? v_out : k_out;
            if (step_out != nullptr) dst0 = step_out + ((size_t)t * n_kv + hk) * width;
            if (page >= 0)
                dst1 = (is_v ? v_cache : k_cache) +
                       (((size_t)page * n_kv + hk) * MF_PAGE + (pos & (MF_PAGE - 1))) * width;
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = lane + 32 * i;
            if (d < width) {
                const T y = from_f32<T>(val[i] * f);
                if (dst0) dst0[d] = y;
                if (dst1) dst1[d] = y;
            }
        }
    }
}

extern "C" int mf_unit_norm_kvstore(const float* qkv, int n_partials, const int* positions,
                                    const int* token_row, const int* seq_end, void* q_out,
                                    void* k_out, void* v_out, void* k_cache, void* v_cache,
                                    const int* page_table, int table_stride, int ring,
                                    int n_tokens, int n_heads, int n_kv, int hd, int vd, float eps,
                                    int norm_qk, int dtype, unsigned* status,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd < 1 || hd > SA_MAX_D || vd < 1 || vd > SA_MAX_D || n_partials < 0) return MF_ERR_UNSUPPORTED;
    if ((k_cache == nullptr) != (v_cache == nullptr)) return MF_ERR_ARGUMENT;
    if (k_cache != nullptr && page_table == nullptr) return MF_ERR_ARGUMENT;
    const int n_items = n_heads + 2 * n_kv;
    int by = 1;
    if (n_tokens < 2 * mf_sm_count()) {                  // few tokens: spread a token's heads
        by = (n_items + SA_WARPS - 1) / SA_WARPS;
        if (by > 16) by = 16;
    }
    dim3 grid(n_tokens, by);
#define MF_UNK(T, NI) \
    mf_launch(unit_norm_kvstore_kernel<T, NI>, grid, dim3(SA_WARPS * 32), 0, stream, qkv, n_partials, \
              n_tokens, positions, token_row, seq_end, (T*)q_out, (T*)k_out, (T*)v_out, \
              (T*)k_cache, (T*)v_cache, page_table, table_stride, ring, n_heads, n_kv, hd, vd, eps, \
              norm_qk, status)
#define MF_UNK_SIZES(T) \
    do { \
        if (widest <= 32) MF_UNK(T, 1); else if (widest <= 64) MF_UNK(T, 2); \
        else if (widest <= 128) MF_UNK(T, 4); else MF_UNK(T, 8); \
    } while (0)
    const int widest = hd > vd ? hd : vd;
    if (dtype == MF_DTYPE_F32) MF_UNK_SIZES(float);
    else if (dtype == MF_DTYPE_BF16) MF_UNK_SIZES(__nv_bfloat16);
    else return MF_ERR_UNSUPPORTED;
#undef MF_UNK_SIZES
#undef MF_UNK
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// the generic kernel: one warp per (query, head)
// ------------------------------------------------------------------------------------------
struct SinkArgs {
    const void* q;            // [rows][n_heads][hd]
    const void* k;            // packed keys [tokens][n_kv][hd]      (PAGED: [pages][n_kv][64][hd])
    const void* v;            // packed values [tokens][n_kv][vd]    (PAGED: [pages][n_kv][64][vd])
    const int* row_seq;       // [rows] batch row of each query
    const int* row_pos;       // [rows] absolute position of each query
    const int* cu_seqlens;    // [B+1] packed source only
    const int* page_table;    // paged source only
    int table_stride;
    int ring;                 // paged source: 0 = linear, else ring length in positions
    void* out;                // [rows][n_heads * vd]
    const float* r1;          // [n_heads] or nullptr
    const float* r2;          // [n_heads]
    int rows, n_heads, n_kv, hd, vd;
    int window, chunk, sink;
    float scale;
    const float* sink_logit;  // [n_heads] score of the sink, or nullptr for 0
    float softcap;            // > 0: s <- softcap * tanh(s / softcap) before the bias
    int keep_first;           // > 0: keys at positions below it stay visible beyond the window
};

// tanh through one exponential: 1 - 2 / (exp(2y) + 1); exact at both ends (exp -> inf or 0)
__device__ __forceinline__ float sink_tanh(float y) {
    return 1.0f - __fdividef(2.0f, __expf(2.0f * y) + 1.0f);
}

// first visible key of a query at `pos`
__device__ __forceinline__ int sink_first_key(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    return lo;
}

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
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

// VEC: hd is a multiple of the 16-byte vector (rows of keys then start on 16-byte boundaries)
// NACC: 32-element groups of a value vector a lane accumulates (values up to 32 * NACC wide)
template <typename T, bool PAGED, bool VEC, int NACC>
__global__ void __launch_bounds__(SA_WARPS * 32) sink_attention_generic_kernel(SinkArgs a) {
    pdl_launch_dependents();
    __shared__ float q_s[SA_WARPS][SA_GEN_MAX_D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long item = (long long)blockIdx.x * SA_WARPS + warp;
    if (item >= (long long)a.rows * a.n_heads) return;      // no block-wide barrier below
    const int head = (int)(item % a.n_heads);
    const int row = (int)(item / a.n_heads);
    const int hd = a.hd, vd = a.vd;
    const int hk = head / (a.n_heads / a.n_kv);
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    const int lo = sink_first_key(pos, a.window, a.chunk);
    const float r1 = a.r1 ? a.r1[head] : 0.0f;
    const float r2 = a.r1 ? a.r2[head] : 0.0f;
    const float sink_score = (a.sink && a.sink_logit) ? a.sink_logit[head] : 0.0f;
    const float cap = a.softcap, inv_cap = a.softcap > 0.0f ? 1.0f / a.softcap : 0.0f;
    const long long packed0 = PAGED ? 0 : (long long)a.cu_seqlens[b];
    pdl_wait();

    const T* q = (const T*)a.q + ((size_t)row * a.n_heads + head) * hd;
    for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(q[d]) * a.scale;
    __syncwarp();

    const T* kbase = (const T*)a.k;
    const T* vbase = (const T*)a.v;
    // the sink is a key without a value: its score starts the running maximum and sum
    float m = a.sink ? sink_score : -INFINITY, l = a.sink ? 1.0f : 0.0f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;

    // two stretches of keys: the kept first ones the window no longer covers, then the window
    const int kept_hi = min(a.keep_first, lo);
    for (int seg = kept_hi > 0 ? 0 : 1; seg < 2; ++seg)
    for (int j0 = seg == 0 ? 0 : lo, hi = seg == 0 ? kept_hi : pos + 1; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < hi;
        long long krow = 0;                           // index of key j's row: [..][hk][j]
        if (valid) {
            if (PAGED) {
                const int p_eff = a.ring > 0 ? j % a.ring : j;
                const int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
                krow = ((long long)page * a.n_kv + hk) * MF_PAGE + (j & (MF_PAGE - 1));
            } else {
                krow = (packed0 + j) * a.n_kv + hk;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = kbase + krow * hd;
            float dot = 0.0f;
            if (VEC) {
                for (int d = 0; d < hd; d += Vec16<T>::N) {
                    float kv[Vec16<T>::N];
                    Vec16<T>::load(kr + d, kv);
#pragma unroll
                    for (int e = 0; e < Vec16<T>::N; ++e) dot = fmaf(q_s[warp][d + e], kv[e], dot);
                }
            } else {
                for (int d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], to_f32(kr[d]), dot);
            }
            s = dot;
            if (cap > 0.0f) s = cap * tanhf(s * inv_cap);
            if (a.r1) s -= r1 * log1pf(r2 * (float)(pos - j));
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);           // 0 on the first tile without a sink
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        const int n_here = min(32, hi - j0);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vrow = __shfl_sync(0xffffffffu, krow, jj);
            const T* vr = vbase + vrow * vd;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* o = (T*)a.out + ((size_t)row * a.n_heads + head) * vd;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) o[d] = from_f32<T>(acc[i] * inv);
    }
}

static int sink_check(const SinkArgs& a, int dtype) {
    if (dtype != MF_DTYPE_F32 && dtype != MF_DTYPE_BF16) return MF_ERR_UNSUPPORTED;
    if (a.hd < 1 || a.hd > SA_GEN_MAX_D || a.vd < 1 || a.vd > SA_GEN_MAX_D) return MF_ERR_UNSUPPORTED;
    if (a.n_kv < 1 || a.n_heads % a.n_kv != 0) return MF_ERR_ARGUMENT;
    if (a.window < 0 || a.chunk < 0 || a.softcap < 0.0f || a.keep_first < 0) return MF_ERR_ARGUMENT;
    if (a.keep_first > 0 && a.chunk > 0) return MF_ERR_UNSUPPORTED;
    return 0;
}

template <bool PAGED>
static int sink_generic_launch(const SinkArgs& a, int dtype, cudaStream_t stream) {
    if (a.rows <= 0) return 0;
    const long long items = (long long)a.rows * a.n_heads;
    dim3 grid((unsigned)((items + SA_WARPS - 1) / SA_WARPS)), block(SA_WARPS * 32);
#define MF_SINK_GEN(T, VEC) \
    do { \
        if (a.vd <= SA_MAX_D) mf_launch(sink_attention_generic_kernel<T, PAGED, VEC, SA_MAX_D / 32>, grid, block, 0, stream, a); \
        else mf_launch(sink_attention_generic_kernel<T, PAGED, VEC, SA_GEN_MAX_D / 32>, grid, block, 0, stream, a); \
    } while (0)
    if (dtype == MF_DTYPE_F32) {
        if (a.hd % 4 == 0) MF_SINK_GEN(float, true);
        else MF_SINK_GEN(float, false);
    } else {
        if (a.hd % 8 == 0) MF_SINK_GEN(__nv_bfloat16, true);
        else MF_SINK_GEN(__nv_bfloat16, false);
    }
#undef MF_SINK_GEN
    return MF_LAUNCH_CHECK();
}

static SinkArgs sink_args(const void* q, const void* k, const void* v, const int* row_seq,
                          const int* row_pos, const int* cu_seqlens, const int* page_table,
                          int table_stride, int ring, void* out, const float* r1, const float* r2,
                          int rows, int n_heads, int n_kv, int hd, int vd, int window, int chunk,
                          int sink, float scale, const float* sink_logit, float softcap,
                          int keep_first = 0) {
    SinkArgs a;
    a.q = q; a.k = k; a.v = v; a.row_seq = row_seq; a.row_pos = row_pos; a.cu_seqlens = cu_seqlens;
    a.page_table = page_table; a.table_stride = table_stride; a.ring = ring; a.out = out;
    a.r1 = r1; a.r2 = r2; a.rows = rows; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.vd = vd;
    a.window = window; a.chunk = chunk; a.sink = sink ? 1 : 0; a.scale = scale;
    a.sink_logit = sink_logit; a.softcap = softcap; a.keep_first = keep_first;
    return a;
}

// keys and values are the step's own packed rows: position j of batch row b lies at token
// cu_seqlens[b] + j (whole prompts)
extern "C" int mf_sink_attention_packed(const void* q, const void* k, const void* v,
                                        const int* row_seq, const int* row_pos,
                                        const int* cu_seqlens, void* out, const float* r1,
                                        const float* r2, int rows, int n_heads, int n_kv, int hd,
                                        int vd, int window, int chunk, int sink, float scale,
                                        const float* sink_logit, float softcap, int keep_first,
                                        int dtype, cudaStream_t stream) {
    SinkArgs a = sink_args(q, k, v, row_seq, row_pos, cu_seqlens, nullptr, 0, 0, out, r1, r2, rows,
                           n_heads, n_kv, hd, vd, window, chunk, sink, scale, sink_logit, softcap,
                           keep_first);
    const int bad = sink_check(a, dtype);
    if (bad) return bad;
    return sink_generic_launch<false>(a, dtype, stream);
}

// keys and values come from the paged cache, the step's own among them
extern "C" int mf_sink_attention_paged(const void* q, const void* k_cache, const void* v_cache,
                                       const int* row_seq, const int* row_pos,
                                       const int* page_table, int table_stride, int ring,
                                       void* out, const float* r1, const float* r2, int rows,
                                       int n_heads, int n_kv, int hd, int vd, int window,
                                       int chunk, int sink, float scale,
                                       const float* sink_logit, float softcap, int keep_first,
                                       int dtype, cudaStream_t stream) {
    SinkArgs a = sink_args(q, k_cache, v_cache, row_seq, row_pos, nullptr, page_table,
                           table_stride, ring, out, r1, r2, rows, n_heads, n_kv, hd, vd, window,
                           chunk, sink, scale, sink_logit, softcap, keep_first);
    if (keep_first > 0 && ring > 0) return MF_ERR_ARGUMENT;       // a ring forgets the first keys
    const int bad = sink_check(a, dtype);
    if (bad) return bad;
    if (page_table == nullptr) return MF_ERR_ARGUMENT;
    return sink_generic_launch<true>(a, dtype, stream);
}

// ------------------------------------------------------------------------------------------
// Prompts and portions of prompts on tensor cores (bfloat16; key and value sizes multiples of
// 8 up to 128, padded with zeros in shared memory to 64 or 128).
//
// A CTA owns 64 queries of one head of one sequence and walks the keys its queries can see in
// tiles of 64 absolute positions (a page of the cache, or 64 packed rows) with an online
// softmax in base 2: S = Q K^T and O += P V are m16n8k16 bf16 MMAs with float32
// accumulation; K and V tiles are double-buffered in shared memory by cp.async with an XOR
// swizzle; fragments come out by ldmatrix (transposed for V).  The queries are the step's
// packed rows; row i of a sequence is at position start + i, start = seq_end - rows (0 for
// whole prompts).  The distance bias in base-2 units, r1 log2(1 + r2 d), comes from a table in
// shared memory when the reach is bounded (a chunk or a window of up to 4,096), else it is
// computed per score.  The sink enters at the end: l += 2^(-m) with m >= 0 from the start.
// ------------------------------------------------------------------------------------------
#define SM_WARPS 4
#define SM_ROWS 64
#define SM_KEYS 64
#define SM_MAX_TAB 4096

struct SinkMmaArgs {
    const __nv_bfloat16* q;   // [tokens][n_heads][hd]
    const __nv_bfloat16* k;   // packed [tokens][n_kv][hd], or the cache [pages][n_kv][64][hd]
    const __nv_bfloat16* v;   // packed [tokens][n_kv][vd], or the cache [pages][n_kv][64][vd]
    const int* cu_seqlens;    // [rows + 1] tokens each sequence brings in this step
    const int* seq_end;       // [rows] length after the step (paged source; null: start at 0)
    const int* page_table;
    int table_stride, ring;
    __nv_bfloat16* out;       // [tokens][n_heads * vd]
    const float* r1;          // [n_heads] or null
    const float* r2;
    int n_heads, n_kv, hd, vd, window, chunk, sink;
    int keep_first;           // > 0: keys at positions below it stay visible beyond the window
    int tab_n;                // entries of the bias table (0: the bias is computed per score)
    float scale_log2;         // scale * log2(e)
    const float* sink_logit;  // [n_heads] score of the sink, or null for 0
    float cap_log2;           // soft cap * log2(e); 0: no cap
    float scale_over_cap;     // scale / soft cap
};

__device__ __forceinline__ void sm_mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sm_pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void sm_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                           uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sm_ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                 uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// Copies `n_rows` rows (ROWS at most) of `d` elements each, `row_stride` elements apart, into a
// swizzled [ROWS][DP] tile; rows at or beyond `n_valid` and the columns from `d` to DP are
// filled with zeros.  A thread always copies the same 16-byte column.
template <int DP, int ROWS, int THREADS>
struct SinkTileCopy {
    static constexpr int CPR = DP / 8;                    // 16-byte chunks per padded row
    static constexpr int RPP = THREADS / CPR;             // rows per pass
    int r0;
    uint32_t dst_off;
    int src_col;
    bool col_ok;
    __device__ __forceinline__ SinkTileCopy(int tid, int d) {
        r0 = tid / CPR;
        const int c = tid % CPR;
        dst_off = (uint32_t)((r0 * CPR + (c ^ (r0 & 7))) * 16);
        src_col = c * 8;
        col_ok = src_col < d;
    }
    __device__ __forceinline__ void load(uint32_t tile, const __nv_bfloat16* base,
                                         long long row_stride, int n_valid) const {
        const __nv_bfloat16* src = base + (long long)r0 * row_stride + src_col;
#pragma unroll
        for (int j = 0; j < ROWS / RPP; ++j) {
            const bool ok = col_ok && r0 + j * RPP < n_valid;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         ::"r"(tile + dst_off + (uint32_t)(j * RPP * CPR * 16)),
                           "l"(ok ? src + (long long)j * RPP * row_stride : base), "r"(ok ? 16 : 0)
                         : "memory");
        }
    }
};

template <int HDP, int VDP, bool PAGED>
__global__ void __launch_bounds__(SM_WARPS * 32, (HDP + VDP > 128) ? 2 : 3)
sink_attention_mma_kernel(SinkMmaArgs a) {
    pdl_launch_dependents();
    constexpr int CPRK = HDP / 8, CPRV = VDP / 8;
    extern __shared__ __align__(128) uint8_t sm_smem[];
    const uint32_t k_s = (uint32_t)__cvta_generic_to_shared(sm_smem);           // [2][64][HDP]
    const uint32_t v_s = k_s + 2 * 64 * HDP * 2;                                 // [2][64][VDP]
    float* tab = (float*)(sm_smem + 2 * 64 * (HDP + VDP) * 2);                   // [tab_n]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int tok0 = a.cu_seqlens[seq];
    const int n_new = a.cu_seqlens[seq + 1] - tok0;
    // heavy (late) query tiles first: they have the most keys
    const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int q0 = q_tile * SM_ROWS;
    if (q0 >= n_new) return;
    const int end = a.seq_end != nullptr ? a.seq_end[seq] : n_new;
    const int start = end - n_new;
    const int hk = head / (a.n_heads / a.n_kv);
    const int hd = a.hd, vd = a.vd;
    const bool has_bias = a.r1 != nullptr;
    const float r1 = has_bias ? a.r1[head] : 0.0f, r2 = has_bias ? a.r2[head] : 0.0f;
    // the bias table of this head (weights: before the wait)
    for (int d = tid; d < a.tab_n; d += SM_WARPS * 32) tab[d] = r1 * log2f(fmaf(r2, (float)d, 1.0f));
    pdl_wait();

    const int pos0 = start + q0;                                   // position of the tile's first query
    const int pos_last = start + min(q0 + SM_ROWS, n_new) - 1;
    const int kt_begin = sink_first_key(pos0, a.window, a.chunk) / SM_KEYS;
    const int kt_end = pos_last / SM_KEYS;                         // inclusive

    const SinkTileCopy<HDP, 64, SM_WARPS * 32> copy_k(tid, hd);
    const SinkTileCopy<VDP, 64, SM_WARPS * 32> copy_v(tid, vd);
    auto load_tile = [&](int kt, int buf) {
        const int key0 = kt * SM_KEYS;
        const __nv_bfloat16 *kb, *vb;
        long long ks, vs;
        if (PAGED) {
            const int p_eff = a.ring > 0 ? key0 % a.ring : key0;
            int page = a.page_table[(size_t)seq * a.table_stride + (p_eff >> 6)];
            if (page < 0) page = 0;                                // (masked anyway: beyond the end)
            kb = a.k + ((long long)page * a.n_kv + hk) * MF_PAGE * hd;
            vb = a.v + ((long long)page * a.n_kv + hk) * MF_PAGE * vd;
            ks = hd; vs = vd;
        } else {
            kb = a.k + ((long long)(tok0 + key0) * a.n_kv + hk) * hd;
            vb = a.v + ((long long)(tok0 + key0) * a.n_kv + hk) * vd;
            ks = (long long)a.n_kv * hd; vs = (long long)a.n_kv * vd;
        }
        copy_k.load(k_s + (uint32_t)(buf * 64 * HDP * 2), kb, ks, end - key0);
        copy_v.load(v_s + (uint32_t)(buf * 64 * VDP * 2), vb, vs, end - key0);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // the key tiles a CTA walks: those of the kept first keys that lie before the window's first
    // tile, then the window's
    const int kept_tiles = a.keep_first > 0 ? min((a.keep_first + SM_KEYS - 1) / SM_KEYS, kt_begin) : 0;
    const int n_iter = kept_tiles + kt_end - kt_begin + 1;
    auto tile_of = [&](int it) { return it < kept_tiles ? it : kt_begin + (it - kept_tiles); };
    load_tile(tile_of(0), 0);

    // the sink starts the running maximum at its score (0, or the head's learned one)
    const float sink2 = (a.sink && a.sink_logit) ? a.sink_logit[head] * 1.4426950408889634f : 0.0f;
    float m_r[2], l_r[2] = {0.0f, 0.0f};
    m_r[0] = m_r[1] = a.sink ? sink2 : -INFINITY;
    float o[VDP / 8][4];
#pragma unroll
    for (int i = 0; i < VDP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const int qi = q0 + warp * 16 + g;                            // this thread's queries: qi, qi + 8
    int row_p[2], row_lo[2];
    row_p[0] = start + qi; row_p[1] = row_p[0] + 8;
    row_lo[0] = sink_first_key(row_p[0], a.window, a.chunk);
    row_lo[1] = sink_first_key(row_p[1], a.window, a.chunk);
    const int warp_lo_max = sink_first_key(pos0 + warp * 16 + 15, a.window, a.chunk);
    // query fragments straight from global memory (rows beyond the end and columns beyond hd: 0)
    uint32_t qa[HDP / 16][4];
    {
        const __nv_bfloat16* q_lo = a.q + ((long long)(tok0 + qi) * a.n_heads + head) * hd + 2 * t;
        const __nv_bfloat16* q_hi = q_lo + 8 * (long long)a.n_heads * hd;
        const bool lo_ok = qi < n_new, hi_ok = qi + 8 < n_new;
#pragma unroll
        for (int ks = 0; ks < HDP / 16; ++ks) {
            const bool c0 = 16 * ks + 2 * t < hd, c1 = 16 * ks + 8 + 2 * t < hd;
            qa[ks][0] = lo_ok && c0 ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks) : 0u;
            qa[ks][1] = hi_ok && c0 ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks) : 0u;
            qa[ks][2] = lo_ok && c1 ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + 8) : 0u;
            qa[ks][3] = hi_ok && c1 ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + 8) : 0u;
        }
    }
    const uint32_t k_lane = (uint32_t)((((lane >> 4) * 8 + (lane & 7)) * CPRK) * 16);
    const uint32_t v_lane = (uint32_t)(((((lane >> 3) & 1) * 8 + (lane & 7)) * CPRV) * 16);
    uint32_t k_col[HDP / 16], v_col[VDP / 16];
#pragma unroll
    for (int i = 0; i < HDP / 16; ++i) k_col[i] = (uint32_t)(((2 * i + ((lane >> 3) & 1)) ^ (lane & 7)) * 16);
#pragma unroll
    for (int i = 0; i < VDP / 16; ++i) v_col[i] = (uint32_t)(((2 * i + (lane >> 4)) ^ (lane & 7)) * 16);

    for (int it = 0; it < n_iter; ++it) {
        const int kt = tile_of(it);
        const int buf = it & 1;
        if (it + 1 < n_iter) {                                    // prefetch the next tile
            load_tile(tile_of(it + 1), buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();

        // S[16][64] = Q K^T
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
        const uint32_t ks_base = k_s + (uint32_t)(buf * 64 * HDP * 2) + k_lane;
#pragma unroll
        for (int ks = 0; ks < HDP / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {                      // pairs of 8-key tiles
                uint32_t b0, b1, b2, b3;
                sm_ldsm_x4(ks_base + k_col[ks] + (uint32_t)(np * 16 * CPRK * 16), b0, b1, b2, b3);
                sm_mma16816(s[2 * np], qa[ks], b0, b1);
                sm_mma16816(s[2 * np + 1], qa[ks], b2, b3);
            }
        }

        // scale, bias by distance, mask by position
        const int key0 = kt * SM_KEYS;
        const bool all_visible = key0 >= warp_lo_max && key0 + SM_KEYS - 1 <= pos0 + warp * 16;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nt * 8 + 2 * t + (e & 1);
                const int r = e >> 1;
                const int d = row_p[r] - key;
                float x = a.cap_log2 > 0.0f ? a.cap_log2 * sink_tanh(s[nt][e] * a.scale_over_cap)
                                            : s[nt][e] * a.scale_log2;
                const bool vis = all_visible || (d >= 0 && (key >= row_lo[r] || key < a.keep_first));
                if (has_bias && vis)
                    x -= a.tab_n > 0 ? tab[d] : r1 * __log2f(fmaf(r2, (float)d, 1.0f));
                s[nt][e] = vis ? x : -INFINITY;
            }
        }
        // online softmax (base 2)
        float m_new[2] = {m_r[0], m_r[1]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            m_new[0] = fmaxf(m_new[0], fmaxf(s[nt][0], s[nt][1]));
            m_new[1] = fmaxf(m_new[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            // a row with nothing visible yet keeps m = -inf; 0 as its offset gives
            // exp2(-inf - 0) = 0 and no inf - inf
            m_use[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r];
            corr[r] = m_r[r] == -INFINITY ? 0.0f : exp2f(m_r[r] - m_use[r]);
            m_r[r] = m_new[r];
            l_r[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < VDP / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        uint32_t pa[4][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = exp2f(s[nt][e] - m_use[e >> 1]);
                l_r[e >> 1] += p[e];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = sm_pack2(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = sm_pack2(p[2], p[3]);
        }
        // O += P V
        const uint32_t vs_base = v_s + (uint32_t)(buf * 64 * VDP * 2) + v_lane;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int np = 0; np < VDP / 16; ++np) {
                uint32_t r0, r1_, r2_, r3;
                sm_ldsm_x4_trans(vs_base + v_col[np] + (uint32_t)(ks * 16 * CPRV * 16), r0, r1_, r2_, r3);
                sm_mma16816(o[2 * np], pa[ks], r0, r1_);
                sm_mma16816(o[2 * np + 1], pa[ks], r2_, r3);
            }
        }
        __syncthreads();                                          // the buffer may be refilled now
    }

    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
        if (a.sink) l_r[r] += exp2f(sink2 - m_r[r]);
        inv[r] = 1.0f / l_r[r];
    }
#pragma unroll
    for (int nt = 0; nt < VDP / 8; ++nt) {
        const int d = nt * 8 + 2 * t;
        if (d < vd) {
            if (qi < n_new)
                *reinterpret_cast<uint32_t*>(a.out + ((long long)(tok0 + qi) * a.n_heads + head) * vd + d) =
                    sm_pack2(o[nt][0] * inv[0], o[nt][1] * inv[0]);
            if (qi + 8 < n_new)
                *reinterpret_cast<uint32_t*>(a.out + ((long long)(tok0 + qi + 8) * a.n_heads + head) * vd + d) =
                    sm_pack2(o[nt][2] * inv[1], o[nt][3] * inv[1]);
        }
    }
}

template <int HDP, int VDP, bool PAGED>
static int launch_sink_mma(const SinkMmaArgs& a, int n_seqs, int max_new, cudaStream_t stream) {
    const int smem = 2 * 64 * (HDP + VDP) * 2 + a.tab_n * 4;
    static int configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(sink_attention_mma_kernel<HDP, VDP, PAGED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             2 * 64 * (HDP + VDP) * 2 + SM_MAX_TAB * 4);
        if (e != cudaSuccess) return (int)e;
        configured = 2 * 64 * (HDP + VDP) * 2 + SM_MAX_TAB * 4;
    }
    dim3 grid((max_new + SM_ROWS - 1) / SM_ROWS, a.n_heads, n_seqs);
    mf_launch(sink_attention_mma_kernel<HDP, VDP, PAGED>, grid, dim3(SM_WARPS * 32), (size_t)smem,
              stream, a);
    return MF_LAUNCH_CHECK();
}

// 1 if the tensor-core kernels take these sizes (bfloat16 only)
extern "C" int mf_sink_attention_mma_supported(int hd, int vd) {
    return hd >= 8 && vd >= 8 && hd <= 128 && vd <= 128 && hd % 8 == 0 && vd % 8 == 0;
}

// q [tokens][n_heads][hd] bfloat16, the step's packed rows; sequence b brings the tokens
// cu_seqlens[b] .. cu_seqlens[b+1]-1.  `page_table` null: keys and values are the step's own
// packed rows and every sequence starts at position 0; else they come from the cache and
// sequence b ends at seq_end[b] after this step.
extern "C" int mf_sink_attention_mma(const void* q, const void* k, const void* v,
                                     const int* cu_seqlens, const int* seq_end,
                                     const int* page_table, int table_stride, int ring, void* out,
                                     const float* r1, const float* r2, int n_seqs, int max_new,
                                     int n_heads, int n_kv, int hd, int vd, int window, int chunk,
                                     int sink, float scale, const float* sink_logit, float softcap,
                                     int keep_first, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (keep_first < 0 || (keep_first > 0 && (ring > 0 || chunk > 0 || r1 != nullptr))) return MF_ERR_UNSUPPORTED;
    if (softcap < 0.0f) return MF_ERR_ARGUMENT;
    if (!mf_sink_attention_mma_supported(hd, vd) || n_kv <= 0 || n_heads % n_kv != 0) return MF_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_seqs > 65535 || window < 0 || chunk < 0) return MF_ERR_UNSUPPORTED;
    if ((page_table == nullptr) != (seq_end == nullptr)) return MF_ERR_ARGUMENT;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15)) return MF_ERR_UNSUPPORTED;
    SinkMmaArgs a;
    a.q = (const __nv_bfloat16*)q; a.k = (const __nv_bfloat16*)k; a.v = (const __nv_bfloat16*)v;
    a.cu_seqlens = cu_seqlens; a.seq_end = seq_end; a.page_table = page_table;
    a.table_stride = table_stride; a.ring = ring; a.out = (__nv_bfloat16*)out; a.r1 = r1; a.r2 = r2;
    a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.vd = vd; a.window = window; a.chunk = chunk;
    a.sink = sink ? 1 : 0;
    a.keep_first = window > 0 ? keep_first : 0;
    int reach = 0;
    if (chunk > 0) reach = chunk;
    if (window > 0 && (reach == 0 || window < reach)) reach = window;
    a.tab_n = (r1 != nullptr && reach > 0 && reach <= SM_MAX_TAB) ? reach : 0;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.sink_logit = sink_logit;
    a.cap_log2 = softcap * 1.4426950408889634f;
    a.scale_over_cap = softcap > 0.0f ? scale / softcap : 0.0f;
    const bool paged = page_table != nullptr;
#define MF_SINK_MMA(H, V) \
    (paged ? launch_sink_mma<H, V, true>(a, n_seqs, max_new, stream) \
           : launch_sink_mma<H, V, false>(a, n_seqs, max_new, stream))
    if (hd <= 64) return vd <= 64 ? MF_SINK_MMA(64, 64) : MF_SINK_MMA(64, 128);
    return vd <= 64 ? MF_SINK_MMA(128, 64) : MF_SINK_MMA(128, 128);
#undef MF_SINK_MMA
}

// ------------------------------------------------------------------------------------------
// Single queries over the paged cache on tensor cores (bfloat16; sizes as above; the query
// heads of a key/value head in blocks of up to 16).
//
// One CTA owns (key split, key/value head, query).  The query heads of the key/value head are
// the 16 rows of an m16n8k16 MMA, so a key or value is read once for the whole group.  The
// keys a query sees, [first visible, position], are cut into tiles of 32 absolute positions (a
// tile lies in one page); a CTA takes `tiles_per_cta` consecutive tiles, its four warps take
// every fourth of them, each with a double buffer of its own in shared memory (cp.async, XOR
// swizzle) and its own running maximum, sum and output.  The warps' results are merged in
// shared memory in warp order.  One split: the output is written (the sink added).  Several:
// a partial (maximum, sum, output) per split, merged by sink_decode_combine_kernel in split
// order, which adds the sink.  Base-2 exponentials throughout.
// ------------------------------------------------------------------------------------------
#define SD_WARPS 4
#define SD_KEYS 32

struct SinkDecodeArgs {
    const __nv_bfloat16* q;   // [rows][n_heads][hd]
    const __nv_bfloat16* k;   // cache [pages][n_kv][64][hd]
    const __nv_bfloat16* v;   // cache [pages][n_kv][64][vd]
    const int* row_seq;       // [rows] batch row of each query
    const int* row_pos;       // [rows] absolute position of each query
    const int* page_table;
    int table_stride, ring;
    __nv_bfloat16* out;       // [rows][n_heads * vd]
    float* partial;           // [rows][n_heads][n_splits][vd + 2]   (n_splits > 1)
    const float* r1;
    const float* r2;
    int n_heads, n_kv, hd, vd, window, chunk, sink;
    int keep_first;           // > 0: keys at positions below it stay visible beyond the window
    int tiles_per_cta, n_splits;
    int n_bufs;               // buffers a warp has: 2, or 1 when it takes one tile only
    float scale_log2;
    const float* sink_logit;  // [n_heads] score of the sink, or null for 0
    float cap_log2;           // soft cap * log2(e); 0: no cap
    float scale_over_cap;     // scale / soft cap
};

// a warp copies 32 rows of `d` elements (row r at base + r * d) into its swizzled [32][DP] tile
template <int DP>
__device__ __forceinline__ void sd_copy_tile(uint32_t tile, const __nv_bfloat16* base, int d,
                                             int lane) {
    constexpr int CPR = DP / 8;
#pragma unroll
    for (int i = 0; i < CPR; ++i) {
        const int idx = lane + 32 * i;
        const int r = idx / CPR, c = idx % CPR;
        const bool ok = c * 8 < d;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                     ::"r"(tile + (uint32_t)((r * CPR + (c ^ (r & 7))) * 16)),
                       "l"(ok ? base + (long long)r * d + c * 8 : base), "r"(ok ? 16 : 0)
                     : "memory");
    }
}

template <int HDP, int VDP>
__global__ void __launch_bounds__(SD_WARPS * 32) sink_attention_decode_kernel(SinkDecodeArgs a) {
    pdl_launch_dependents();
    constexpr int CPRK = HDP / 8, CPRV = VDP / 8;
    constexpr int TILE_BYTES = SD_KEYS * (HDP + VDP) * 2;          // one buffer: K then V
    constexpr int OS = VDP + 4;                                    // padded row of a warp's output
    extern __shared__ __align__(128) uint8_t sd_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // a group of more than 16 query heads is taken in blocks of 16, a CTA each
    const int G = a.n_heads / a.n_kv;
    const int gblocks = (G + 15) >> 4;
    const int split = blockIdx.x, hk = blockIdx.y / gblocks, g0 = (blockIdx.y % gblocks) << 4;
    const int row = blockIdx.z;
    const int Gb = min(16, G - g0);
    const int hd = a.hd, vd = a.vd;
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    const int lo = sink_first_key(pos, a.window, a.chunk);
    // the tiles a query sees, numbered in the order they are walked: those of the kept first keys
    // that lie before the window's first tile, then the window's
    const int first_tile = lo / SD_KEYS;
    const int kept_tiles = a.keep_first > 0 ? min((a.keep_first + SD_KEYS - 1) / SD_KEYS, first_tile) : 0;
    auto real_tile = [&](int vt) { return vt < kept_tiles ? vt : first_tile + (vt - kept_tiles); };
    const int tile_lo = split * a.tiles_per_cta;                  // this CTA's first tile (in that order)
    const int tile_hi = min(kept_tiles + pos / SD_KEYS - first_tile, tile_lo + a.tiles_per_cta - 1);   // inclusive
    const bool has_bias = a.r1 != nullptr;
    // this thread's two rows of the product are the group's heads g and g + 8
    float r1v[2] = {0.0f, 0.0f}, r2v[2] = {0.0f, 0.0f};
    if (has_bias) {
        if (g < Gb) { r1v[0] = a.r1[hk * G + g0 + g]; r2v[0] = a.r2[hk * G + g0 + g]; }
        if (g + 8 < Gb) { r1v[1] = a.r1[hk * G + g0 + g + 8]; r2v[1] = a.r2[hk * G + g0 + g + 8]; }
    }
    pdl_wait();

    const uint32_t my_s = (uint32_t)__cvta_generic_to_shared(sd_smem) + (uint32_t)(warp * a.n_bufs * TILE_BYTES);
    auto load_tile = [&](int tile, int buf) {
        const int key0 = tile * SD_KEYS;
        const int p_eff = a.ring > 0 ? key0 % a.ring : key0;
        int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
        if (page < 0) page = 0;                                    // (a tile beyond the end: masked)
        const long long r0 = ((long long)page * a.n_kv + hk) * MF_PAGE + (key0 & (MF_PAGE - 1));
        const uint32_t dst = my_s + (uint32_t)(buf * TILE_BYTES);
        sd_copy_tile<HDP>(dst, a.k + r0 * hd, hd, lane);
        sd_copy_tile<VDP>(dst + SD_KEYS * HDP * 2, a.v + r0 * vd, vd, lane);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int tile = tile_lo + warp;
    if (tile <= tile_hi) load_tile(real_tile(tile), 0);

    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    float o[VDP / 8][4];
#pragma unroll
    for (int i = 0; i < VDP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    uint32_t qa[HDP / 16][4];
    {
        const __nv_bfloat16* q_lo = a.q + ((long long)row * a.n_heads + hk * G + g0 + g) * hd + 2 * t;
        const __nv_bfloat16* q_hi = q_lo + 8 * (long long)hd;
        const bool lo_ok = g < Gb, hi_ok = g + 8 < Gb;
#pragma unroll
        for (int ks = 0; ks < HDP / 16; ++ks) {
            const bool c0 = 16 * ks + 2 * t < hd, c1 = 16 * ks + 8 + 2 * t < hd;
            qa[ks][0] = lo_ok && c0 ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks) : 0u;
            qa[ks][1] = hi_ok && c0 ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks) : 0u;
            qa[ks][2] = lo_ok && c1 ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + 8) : 0u;
            qa[ks][3] = hi_ok && c1 ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + 8) : 0u;
        }
    }
    const uint32_t k_lane = (uint32_t)((((lane >> 4) * 8 + (lane & 7)) * CPRK) * 16);
    const uint32_t v_lane = (uint32_t)(((((lane >> 3) & 1) * 8 + (lane & 7)) * CPRV) * 16);
    uint32_t k_col[HDP / 16], v_col[VDP / 16];
#pragma unroll
    for (int i = 0; i < HDP / 16; ++i) k_col[i] = (uint32_t)(((2 * i + ((lane >> 3) & 1)) ^ (lane & 7)) * 16);
#pragma unroll
    for (int i = 0; i < VDP / 16; ++i) v_col[i] = (uint32_t)(((2 * i + (lane >> 4)) ^ (lane & 7)) * 16);

    for (int it = 0; tile <= tile_hi; tile += SD_WARPS, ++it) {
        const int buf = it & 1;
        if (tile + SD_WARPS <= tile_hi) {
            load_tile(real_tile(tile + SD_WARPS), buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        // S[16][32] = Q K^T
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
        const uint32_t ks_base = my_s + (uint32_t)(buf * TILE_BYTES) + k_lane;
#pragma unroll
        for (int ks = 0; ks < HDP / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b0, b1, b2, b3;
                sm_ldsm_x4(ks_base + k_col[ks] + (uint32_t)(np * 16 * CPRK * 16), b0, b1, b2, b3);
                sm_mma16816(s[2 * np], qa[ks], b0, b1);
                sm_mma16816(s[2 * np + 1], qa[ks], b2, b3);
            }
        }
        const int key0 = real_tile(tile) * SD_KEYS;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nt * 8 + 2 * t + (e & 1);
                const int d = pos - key;
                const bool vis = d >= 0 && (key >= lo || key < a.keep_first);
                float x = a.cap_log2 > 0.0f ? a.cap_log2 * sink_tanh(s[nt][e] * a.scale_over_cap)
                                            : s[nt][e] * a.scale_log2;
                if (has_bias && vis) x -= r1v[e >> 1] * __log2f(fmaf(r2v[e >> 1], (float)d, 1.0f));
                s[nt][e] = vis ? x : -INFINITY;
            }
        }
        float m_new[2] = {m_r[0], m_r[1]};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            m_new[0] = fmaxf(m_new[0], fmaxf(s[nt][0], s[nt][1]));
            m_new[1] = fmaxf(m_new[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            m_use[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r];
            corr[r] = m_r[r] == -INFINITY ? 0.0f : exp2f(m_r[r] - m_use[r]);
            m_r[r] = m_new[r];
            l_r[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < VDP / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        uint32_t pa[2][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = exp2f(s[nt][e] - m_use[e >> 1]);
                l_r[e >> 1] += p[e];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = sm_pack2(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = sm_pack2(p[2], p[3]);
        }
        const uint32_t vs_base = my_s + (uint32_t)(buf * TILE_BYTES + SD_KEYS * HDP * 2) + v_lane;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
            for (int np = 0; np < VDP / 16; ++np) {
                uint32_t x0, x1, x2, x3;
                sm_ldsm_x4_trans(vs_base + v_col[np] + (uint32_t)(ks * 16 * CPRV * 16), x0, x1, x2, x3);
                sm_mma16816(o[2 * np], pa[ks], x0, x1);
                sm_mma16816(o[2 * np + 1], pa[ks], x2, x3);
            }
        }
        __syncwarp();                                             // the buffer may be refilled now
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
    }
    // ---- the four warps' results, merged in warp order ------------------------------------------
    __syncthreads();                                              // every warp is done with its tiles
    float* o_s = (float*)sd_smem;                                 // [SD_WARPS][16][OS]
    float* ml_s = o_s + SD_WARPS * 16 * OS;                       // [SD_WARPS][16][2]
#pragma unroll
    for (int nt = 0; nt < VDP / 8; ++nt) {
        float* p0 = o_s + ((size_t)warp * 16 + g) * OS + nt * 8 + 2 * t;
        p0[0] = o[nt][0]; p0[1] = o[nt][1];
        p0[8 * OS] = o[nt][2]; p0[8 * OS + 1] = o[nt][3];
    }
    if (t == 0) {
        ml_s[(warp * 16 + g) * 2] = m_r[0];     ml_s[(warp * 16 + g) * 2 + 1] = l_r[0];
        ml_s[(warp * 16 + g + 8) * 2] = m_r[1]; ml_s[(warp * 16 + g + 8) * 2 + 1] = l_r[1];
    }
    __syncthreads();
    for (int idx = tid; idx < Gb * VDP; idx += SD_WARPS * 32) {
        const int r = idx / VDP, d = idx - r * VDP;
        if (d >= vd) continue;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < SD_WARPS; ++w) m = fmaxf(m, ml_s[(w * 16 + r) * 2]);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < SD_WARPS; ++w) {
            const float mw = ml_s[(w * 16 + r) * 2];
            if (mw > -INFINITY) {
                const float f = exp2f(mw - m);
                l = fmaf(ml_s[(w * 16 + r) * 2 + 1], f, l);
                acc = fmaf(o_s[((size_t)w * 16 + r) * OS + d], f, acc);
            }
        }
        const int head = hk * G + g0 + r;
        if (a.n_splits > 1) {
            float* part = a.partial + (((size_t)row * a.n_heads + head) * a.n_splits + split) * (vd + 2);
            if (d == 0) { part[0] = m; part[1] = l; }
            part[2 + d] = acc;
        } else {
            float mf = m;
            if (a.sink) {                                         // the sink: a key without a value
                const float sink2 = a.sink_logit ? a.sink_logit[head] * 1.4426950408889634f : 0.0f;
                mf = fmaxf(m, sink2);
                const float f = m > -INFINITY ? exp2f(m - mf) : 0.0f;
                l = l * f + exp2f(sink2 - mf);
                acc *= f;
            }
            a.out[((size_t)row * a.n_heads + head) * vd + d] = __float2bfloat16_rn(acc / l);
        }
    }
}

// merges the splits of one (query, head) in split order and adds the sink
__global__ void sink_decode_combine_kernel(const float* __restrict__ partial,
                                           __nv_bfloat16* __restrict__ out, int n_splits, int vd,
                                           int sink, const float* __restrict__ sink_logit,
                                           int n_heads) {
    pdl_prologue();
    const size_t rh = blockIdx.x;
    const size_t stride = (size_t)(vd + 2);
    const float* p = partial + rh * n_splits * stride;
    const float sink2 = (sink && sink_logit) ? sink_logit[rh % n_heads] * 1.4426950408889634f : 0.0f;
    float m = sink ? sink2 : -INFINITY;
    for (int c = 0; c < n_splits; ++c) m = fmaxf(m, p[c * stride]);
    float l = sink ? exp2f(sink2 - m) : 0.0f;
    for (int c = 0; c < n_splits; ++c) {
        const float mc = p[c * stride];
        if (mc > -INFINITY) l = fmaf(p[c * stride + 1], exp2f(mc - m), l);
    }
    const float inv = 1.0f / l;
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
        float acc = 0.0f;
        for (int c = 0; c < n_splits; ++c) {
            const float mc = p[c * stride];
            if (mc > -INFINITY) acc = fmaf(p[c * stride + 2 + d], exp2f(mc - m), acc);
        }
        out[rh * vd + d] = __float2bfloat16_rn(acc * inv);
    }
}

// How the keys of single queries are cut: (tiles of 32 keys per CTA, splits), from the sizes
// only.  `n_kv`: key/value heads times the blocks of 16 query heads on each.  `reach_keys`: the
// most keys a query sees (its reach, or the longest sequence).
extern "C" int mf_sink_decode_plan(int rows, int n_kv, int reach_keys, int* tiles_per_cta,
                                   int* n_splits) {
    const int n_tiles = reach_keys / SD_KEYS + 2;                  // the range need not start on a tile
    int splits = (2 * mf_sm_count() + rows * n_kv - 1) / (rows * n_kv > 0 ? rows * n_kv : 1);
    const int most = (n_tiles + SD_WARPS - 1) / SD_WARPS;
    if (splits > most) splits = most;
    if (splits < 1) splits = 1;
    int tpc = (n_tiles + splits - 1) / splits;
    tpc = ((tpc + SD_WARPS - 1) / SD_WARPS) * SD_WARPS;
    *tiles_per_cta = tpc;
    *n_splits = (n_tiles + tpc - 1) / tpc;
    return 0;
}

template <int HDP, int VDP>
static int launch_sink_decode(const SinkDecodeArgs& a, int rows, cudaStream_t stream) {
    constexpr int most = SD_WARPS * 2 * SD_KEYS * (HDP + VDP) * 2;
    constexpr int merge = SD_WARPS * 16 * (VDP + 4) * 4 + SD_WARPS * 16 * 2 * 4;
    // a warp with one tile needs one buffer: half the shared memory, twice the CTAs on an SM
    const int tiles = SD_WARPS * a.n_bufs * SD_KEYS * (HDP + VDP) * 2;
    const int smem = tiles > merge ? tiles : merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sink_attention_decode_kernel<HDP, VDP>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             most > merge ? most : merge);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int gblocks = (a.n_heads / a.n_kv + 15) / 16;
    mf_launch(sink_attention_decode_kernel<HDP, VDP>, dim3(a.n_splits, a.n_kv * gblocks, rows),
              dim3(SD_WARPS * 32), (size_t)smem, stream, a);
    return MF_LAUNCH_CHECK();
}

// Every row of q [rows][n_heads][hd] (bfloat16) is a query at row_pos over the paged cache.
// `reach_keys`: the most keys a query sees (chunk, window, or the longest sequence's length).
// `partial`: float32 scratch of rows * n_heads * splits * (vd + 2) floats when the plan has
// more than one split (mf_sink_decode_plan), else unused.
extern "C" int mf_sink_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                        const int* row_seq, const int* row_pos,
                                        const int* page_table, int table_stride, int ring,
                                        void* out, float* partial, const float* r1,
                                        const float* r2, int rows, int n_heads, int n_kv, int hd,
                                        int vd, int window, int chunk, int sink, float scale,
                                        int reach_keys, const float* sink_logit, float softcap,
                                        int keep_first, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (keep_first < 0 || (keep_first > 0 && (ring > 0 || chunk > 0))) return MF_ERR_UNSUPPORTED;
    if (softcap < 0.0f) return MF_ERR_ARGUMENT;
    if (!mf_sink_attention_mma_supported(hd, vd) || n_kv <= 0 || n_heads % n_kv != 0) return MF_ERR_UNSUPPORTED;
    const int head_blocks = n_kv * ((n_heads / n_kv + 15) / 16);      // CTAs per (split, query)
    if (head_blocks > 65535 || rows > 65535) return MF_ERR_UNSUPPORTED;
    if (page_table == nullptr || window < 0 || chunk < 0) return MF_ERR_ARGUMENT;
    SinkDecodeArgs a;
    a.q = (const __nv_bfloat16*)q; a.k = (const __nv_bfloat16*)k_cache;
    a.v = (const __nv_bfloat16*)v_cache; a.row_seq = row_seq; a.row_pos = row_pos;
    a.page_table = page_table; a.table_stride = table_stride; a.ring = ring;
    a.out = (__nv_bfloat16*)out; a.partial = partial; a.r1 = r1; a.r2 = r2;
    a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.vd = vd; a.window = window; a.chunk = chunk;
    a.sink = sink ? 1 : 0;
    a.keep_first = window > 0 ? keep_first : 0;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.sink_logit = sink_logit;
    a.cap_log2 = softcap * 1.4426950408889634f;
    a.scale_over_cap = softcap > 0.0f ? scale / softcap : 0.0f;
    mf_sink_decode_plan(rows, head_blocks, reach_keys, &a.tiles_per_cta, &a.n_splits);
    a.n_bufs = a.tiles_per_cta > SD_WARPS ? 2 : 1;
    if (a.n_splits > 1 && partial == nullptr) return MF_ERR_ARGUMENT;
    int e;
    if (hd <= 64) e = vd <= 64 ? launch_sink_decode<64, 64>(a, rows, stream)
                               : launch_sink_decode<64, 128>(a, rows, stream);
    else e = vd <= 64 ? launch_sink_decode<128, 64>(a, rows, stream)
                      : launch_sink_decode<128, 128>(a, rows, stream);
    if (e || a.n_splits == 1) return e;
    mf_launch_ex(false, sink_decode_combine_kernel, dim3(rows * n_heads), dim3(vd <= 64 ? 64 : 128), 0,
                 stream, (const float*)partial, (__nv_bfloat16*)out, a.n_splits, vd, a.sink, sink_logit,
                 n_heads);
    return MF_LAUNCH_CHECK();
}
