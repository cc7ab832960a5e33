// What attention mixers do between their input projection and the attention itself, for layouts
// the fused rotary kernel does not take, and the small per-head products of latent attention.
//
//   qk_prepare     One block per token (several when tokens are few: each forms the norms' sums
//                  itself and takes a share of the elements).  From the projection's float32 row it takes a query
//                  segment (n_heads heads of qw) and a key segment (n_kv heads of kw), optionally
//                  RMS-norms the first q_norm_n / k_norm_n elements of each segment AS A WHOLE
//                  (all heads at once: x / sqrt(mean(x^2) + eps) * weight), rotates `rot_dims`
//                  dimensions of every head starting at q_rot_off / k_rot_off (pairs (i, i + R/2)
//                  or (2i, 2i + 1), angle position * inv_freq[i] formed in float64, cosine and
//                  sine times `rot_mag`), and writes q, the step's k and v, and the cache's pages.
//                  Values are a segment of their own (n_kv heads of vw) or, with v_from_k, the
//                  first vw elements of each prepared key head (a latent shared by both); the
//                  places for such values may be null, for a caller that reads them from the keys.
//   head_linear    y[t][h][j] = sum_d W[h][j][d] x[t][h][x_off + d] for every head h, optionally
//                  times sigmoid(gate[t][h * J + j]), optionally followed by a copy of `tail`
//                  elements x[t][h][x_tail_off ..] behind the J outputs.  float32 accumulation;
//                  bfloat16 on tensor cores (mma.sync), float32 on the FP32 pipe.
#include "common.cuh"

struct PrepArgs {
    const float* proj;        // [tokens][in_width]
    long long in_width;
    const int* positions;
    const int* token_row;
    const int* seq_end;
    const double* inv_freq;   // [rot_dims / 2] or null
    const float* q_norm_w;    // [q_norm_n] or null
    const float* k_norm_w;    // [k_norm_n] or null
    void* q_out;              // [tokens][n_heads][qw]
    void* k_out;              // [tokens][n_kv][kw] or null
    void* v_out;              // [tokens][n_kv][vw] or null
    void* k_cache;            // [pages][n_kv][64][kw] or null
    void* v_cache;            // [pages][n_kv][64][vw] or null
    const int* page_table;
    int table_stride, ring;
    int q_off, n_heads, qw, q_norm_n, q_rot_off;
    int k_off, n_kv, kw, k_norm_n, k_rot_off;
    int v_off, vw, v_from_k;
    int rot_dims, rot_style;  // style 0: pairs (i, i + R/2); 1: pairs (2i, 2i + 1)
    float rot_mag, eps;
    unsigned* status;
};

// element d of a head after norm and rotation; `seg` points at the segment's first element,
// `e` = head * width + d is the element's place in the segment
__device__ __forceinline__ float prep_value(const float* seg, const float* norm_w, int norm_n,
                                            float rinv, int width, int d, int e, int rot_off,
                                            const PrepArgs& a, const float* cs) {
    auto normed = [&](int at) {
        const float v = seg[at];
        return at < norm_n ? v * rinv * norm_w[at] : v;
    };
    const float v = normed(e);
    const int r = d - rot_off;
    if (a.rot_dims <= 0 || r < 0 || r >= a.rot_dims) return v;
    const int half = a.rot_dims >> 1;
    int pair, partner;
    bool first;
    if (a.rot_style == 0) {
        first = r < half;
        pair = first ? r : r - half;
        partner = first ? e + half : e - half;
    } else {
        first = (r & 1) == 0;
        pair = r >> 1;
        partner = first ? e + 1 : e - 1;
    }
    const float other = normed(partner);
    const float c = cs[2 * pair], s = cs[2 * pair + 1];
    return first ? v * c - other * s : v * c + other * s;
}

template <typename T>
__global__ void __launch_bounds__(256) qk_prepare_kernel(PrepArgs a) {
    pdl_launch_dependents();
    extern __shared__ float pr_cs[];                  // [rot_dims / 2][2] cosine, sine
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int pos = a.positions[t];
    const int b = a.token_row[t];
    for (int i = threadIdx.x; i < (a.rot_dims >> 1); i += blockDim.x) {
        double ang = (double)pos * a.inv_freq[i];
        ang -= 6.283185307179586476925286766559 * floor(ang * 0.15915494309189533576888376337251);
        float s, c;
        sincosf((float)ang, &s, &c);
        pr_cs[2 * i] = c * a.rot_mag;
        pr_cs[2 * i + 1] = s * a.rot_mag;
    }
    int page = -1;
    if (a.k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (a.ring > 0) {
            keep = pos >= a.seq_end[b] - a.ring;
            p_eff = pos % a.ring;
        }
        if (keep) {
            page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
            if (page < 0 && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(a.status, MF_STATUS_BAD_POSITION);
        }
    }
    pdl_wait();
    const float* row = a.proj + (size_t)t * a.in_width;
    const float* qs = row + a.q_off;
    const float* ks = row + a.k_off;
    float q_rinv = 1.0f, k_rinv = 1.0f;
    if (a.q_norm_n > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < a.q_norm_n; i += blockDim.x) ss = fmaf(qs[i], qs[i], ss);
        ss = block_sum(ss, scratch);
        q_rinv = 1.0f / sqrtf(ss / (float)a.q_norm_n + a.eps);
    }
    if (a.k_norm_n > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < a.k_norm_n; i += blockDim.x) ss = fmaf(ks[i], ks[i], ss);
        ss = block_sum(ss, scratch);
        k_rinv = 1.0f / sqrtf(ss / (float)a.k_norm_n + a.eps);
    }
    __syncthreads();                                  // the cosines and sines are written
    T* q_out = (T*)a.q_out + (size_t)t * a.n_heads * a.qw;
    const int nq = a.n_heads * a.qw;
    const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int e = first; e < nq; e += stride) {
        const int d = e % a.qw;
        q_out[e] = from_f32<T>(prep_value(qs, a.q_norm_w, a.q_norm_n, q_rinv, a.qw, d, e, a.q_rot_off, a, pr_cs));
    }
    const int in_page = pos & (MF_PAGE - 1);
    const int nk = a.n_kv * a.kw;
    for (int e = first; e < nk; e += stride) {
        const int hk = e / a.kw, d = e - hk * a.kw;
        const T y = from_f32<T>(prep_value(ks, a.k_norm_w, a.k_norm_n, k_rinv, a.kw, d, e, a.k_rot_off, a, pr_cs));
        if (a.k_out) ((T*)a.k_out)[(size_t)t * nk + e] = y;
        if (page >= 0)
            ((T*)a.k_cache)[(((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.kw + d] = y;
        if (a.v_from_k && d < a.vw) {
            if (a.v_out) ((T*)a.v_out)[((size_t)t * a.n_kv + hk) * a.vw + d] = y;
            if (page >= 0 && a.v_cache)
                ((T*)a.v_cache)[(((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.vw + d] = y;
        }
    }
    if (!a.v_from_k) {
        const float* vs = row + a.v_off;
        const int nv = a.n_kv * a.vw;
        for (int e = first; e < nv; e += stride) {
            const int hk = e / a.vw, d = e - hk * a.vw;
            const T y = from_f32<T>(vs[e]);
            if (a.v_out) ((T*)a.v_out)[(size_t)t * nv + e] = y;
            if (page >= 0)
                ((T*)a.v_cache)[(((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.vw + d] = y;
        }
    }
}

// ---- the same with 16-byte accesses, for layouts in which every offset and width is a multiple of 4
template <typename T> struct PrepStore4;
template <> struct PrepStore4<float> {
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct PrepStore4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&lo);
        u.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

// four consecutive elements of a segment from element `e` on (a multiple of 4), after norm and
// rotation, into out[0..3]
__device__ __forceinline__ void prep_group(const float* seg, const float* norm_w, int norm_n, float rinv,
                                           int d, int e, int rot_off, const PrepArgs& a, const float* cs,
                                           float* out) {
    auto load = [&](int at, float* v) {
        const float4 x = *reinterpret_cast<const float4*>(seg + at);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        if (at < norm_n) {
            const float4 w = *reinterpret_cast<const float4*>(norm_w + at);
            v[0] *= rinv * w.x; v[1] *= rinv * w.y; v[2] *= rinv * w.z; v[3] *= rinv * w.w;
        }
    };
    float v[4];
    load(e, v);
    const int r = d - rot_off;
    if (a.rot_dims <= 0 || r < 0 || r >= a.rot_dims) {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[k] = v[k];
        return;
    }
    if (a.rot_style == 0) {
        const int half = a.rot_dims >> 1;
        const bool first = r < half;
        const int pair = first ? r : r - half;
        float o[4];
        load(first ? e + half : e - half, o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float c = cs[2 * (pair + k)], sn = cs[2 * (pair + k) + 1];
            out[k] = first ? v[k] * c - o[k] * sn : v[k] * c + o[k] * sn;
        }
    } else {
        const int pair = r >> 1;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float c = cs[2 * (pair + k)], sn = cs[2 * (pair + k) + 1];
            out[2 * k] = v[2 * k] * c - v[2 * k + 1] * sn;
            out[2 * k + 1] = v[2 * k + 1] * c + v[2 * k] * sn;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) qk_prepare_vec_kernel(PrepArgs a) {
    pdl_launch_dependents();
    extern __shared__ float pr_cs[];                  // [rot_dims / 2][2] cosine, sine
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int pos = a.positions[t];
    const int b = a.token_row[t];
    for (int i = threadIdx.x; i < (a.rot_dims >> 1); i += blockDim.x) {
        double ang = (double)pos * a.inv_freq[i];
        ang -= 6.283185307179586476925286766559 * floor(ang * 0.15915494309189533576888376337251);
        float s, c;
        sincosf((float)ang, &s, &c);
        pr_cs[2 * i] = c * a.rot_mag;
        pr_cs[2 * i + 1] = s * a.rot_mag;
    }
    int page = -1;
    if (a.k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (a.ring > 0) {
            keep = pos >= a.seq_end[b] - a.ring;
            p_eff = pos % a.ring;
        }
        if (keep) {
            page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
            if (page < 0 && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(a.status, MF_STATUS_BAD_POSITION);
        }
    }
    pdl_wait();
    const float* row = a.proj + (size_t)t * a.in_width;
    const float* qs = row + a.q_off;
    const float* ks = row + a.k_off;
    float q_rinv = 1.0f, k_rinv = 1.0f;
    if (a.q_norm_n > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x * 4; i < a.q_norm_n; i += blockDim.x * 4) {
            const float4 x = *reinterpret_cast<const float4*>(qs + i);
            ss = fmaf(x.x, x.x, ss); ss = fmaf(x.y, x.y, ss); ss = fmaf(x.z, x.z, ss); ss = fmaf(x.w, x.w, ss);
        }
        ss = block_sum(ss, scratch);
        q_rinv = 1.0f / sqrtf(ss / (float)a.q_norm_n + a.eps);
    }
    if (a.k_norm_n > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x * 4; i < a.k_norm_n; i += blockDim.x * 4) {
            const float4 x = *reinterpret_cast<const float4*>(ks + i);
            ss = fmaf(x.x, x.x, ss); ss = fmaf(x.y, x.y, ss); ss = fmaf(x.z, x.z, ss); ss = fmaf(x.w, x.w, ss);
        }
        ss = block_sum(ss, scratch);
        k_rinv = 1.0f / sqrtf(ss / (float)a.k_norm_n + a.eps);
    }
    __syncthreads();                                  // the cosines and sines are written
    const int first = (blockIdx.y * blockDim.x + threadIdx.x) * 4, stride = gridDim.y * blockDim.x * 4;
    T* q_out = (T*)a.q_out + (size_t)t * a.n_heads * a.qw;
    const int nq = a.n_heads * a.qw;
    for (int e = first; e < nq; e += stride) {
        float y[4];
        prep_group(qs, a.q_norm_w, a.q_norm_n, q_rinv, e % a.qw, e, a.q_rot_off, a, pr_cs, y);
        PrepStore4<T>::store(q_out + e, y);
    }
    const int in_page = pos & (MF_PAGE - 1);
    const int nk = a.n_kv * a.kw;
    for (int e = first; e < nk; e += stride) {
        const int hk = e / a.kw, d = e - hk * a.kw;
        float y[4];
        prep_group(ks, a.k_norm_w, a.k_norm_n, k_rinv, d, e, a.k_rot_off, a, pr_cs, y);
        if (a.k_out) PrepStore4<T>::store((T*)a.k_out + (size_t)t * nk + e, y);
        if (page >= 0)
            PrepStore4<T>::store((T*)a.k_cache + (((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.kw + d, y);
        if (a.v_from_k && d < a.vw) {
            if (a.v_out) PrepStore4<T>::store((T*)a.v_out + ((size_t)t * a.n_kv + hk) * a.vw + d, y);
            if (page >= 0 && a.v_cache)
                PrepStore4<T>::store((T*)a.v_cache + (((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.vw + d, y);
        }
    }
    if (!a.v_from_k) {
        const float* vs = row + a.v_off;
        const int nv = a.n_kv * a.vw;
        for (int e = first; e < nv; e += stride) {
            const int hk = e / a.vw, d = e - hk * a.vw;
            const float4 x = *reinterpret_cast<const float4*>(vs + e);
            const float y[4] = {x.x, x.y, x.z, x.w};
            if (a.v_out) PrepStore4<T>::store((T*)a.v_out + (size_t)t * nv + e, y);
            if (page >= 0)
                PrepStore4<T>::store((T*)a.v_cache + (((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.vw + d, y);
        }
    }
}

extern "C" int mf_qk_prepare(const PrepArgs* args, int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const PrepArgs a = *args;
    if (a.rot_dims < 0 || (a.rot_dims & 1) || (a.rot_dims > 0 && a.inv_freq == nullptr)) return MF_ERR_ARGUMENT;
    if (a.q_rot_off + a.rot_dims > a.qw || a.k_rot_off + a.rot_dims > a.kw) return MF_ERR_ARGUMENT;
    if (a.q_norm_n > a.n_heads * a.qw || a.k_norm_n > a.n_kv * a.kw) return MF_ERR_ARGUMENT;
    // (values taken from the keys need no place of their own: the caller may use the keys)
    if (!a.v_from_k && (a.k_cache == nullptr) != (a.v_cache == nullptr)) return MF_ERR_ARGUMENT;
    if (a.k_cache != nullptr && a.page_table == nullptr) return MF_ERR_ARGUMENT;
    if (a.v_from_k && a.vw > a.kw) return MF_ERR_ARGUMENT;
    const size_t smem = (size_t)(a.rot_dims > 0 ? a.rot_dims : 2) * sizeof(float);
    // few tokens: a token's elements are spread over up to 8 blocks
    int by = 1;
    if (n_tokens < 2 * mf_sm_count()) {
        const int widest = a.n_heads * a.qw > a.n_kv * a.kw ? a.n_heads * a.qw : a.n_kv * a.kw;
        by = (widest + 511) / 512;
        if (by > 8) by = 8;
        if (by < 1) by = 1;
    }
    dim3 grid(n_tokens, by);
    // the form with 16-byte accesses: every offset and width a multiple of 4 (8 for the half of a
    // rotation in pairs (i, i + R/2)), every tensor on a 16-byte boundary
    const int all = a.in_width | a.q_off | a.qw | a.q_norm_n | a.q_rot_off | a.k_off | a.kw | a.k_norm_n |
                    a.k_rot_off | a.vw | (a.v_from_k ? 0 : a.v_off) | a.rot_dims |
                    (a.rot_style == 0 ? a.rot_dims >> 1 : 0);
    const uintptr_t ptrs = (uintptr_t)a.proj | (uintptr_t)a.q_norm_w | (uintptr_t)a.k_norm_w | (uintptr_t)a.q_out |
                           (uintptr_t)a.k_out | (uintptr_t)a.v_out | (uintptr_t)a.k_cache | (uintptr_t)a.v_cache;
    static int scalar = -1;             // MINFER_B200_QK_PREPARE=scalar: the element-by-element form always
    if (scalar < 0) { const char* e = getenv("MINFER_B200_QK_PREPARE"); scalar = (e && e[0] == 's') ? 1 : 0; }
    const bool vec = (all & 3) == 0 && (ptrs & 15) == 0 && !scalar;
    if (vec && dtype == MF_DTYPE_F32)
        mf_launch(qk_prepare_vec_kernel<float>, grid, dim3(256), smem, stream, a);
    else if (vec && dtype == MF_DTYPE_BF16)
        mf_launch(qk_prepare_vec_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, a);
    else if (dtype == MF_DTYPE_F32)
        mf_launch(qk_prepare_kernel<float>, grid, dim3(256), smem, stream, a);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(qk_prepare_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, a);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// per-head products
// ------------------------------------------------------------------------------------------
#define HL_TT 64          // tokens per block
#define HL_TJ 64          // outputs per block
#define HL_TD 32          // reduction chunk

struct HeadLinearArgs {
    const void* x;            // [tokens][x_row] elements; head h starts at h * x_head
    const void* w;            // [heads][J][D]
    void* y;                  // [tokens][y_row]; head h starts at h * y_head
    const float* gate;        // [tokens][gate_row] float32 at column gate_off + h * J + j, or null
    long long x_row, y_row, gate_row;
    int x_head, x_off, y_head, gate_off;
    int n_tokens, heads, J, D;
    int tail, x_tail_off;     // copy x[t][h][x_tail_off .. + tail) to y[t][h][J ..)
};

// a thread owns 4 x 4 results: tokens ty + 16 i, outputs tx + 16 j
template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(HeadLinearArgs a) {
    pdl_prologue();
    __shared__ float xs[HL_TT][HL_TD + 1];
    __shared__ float ws[HL_TJ][HL_TD + 1];
    const int h = blockIdx.z;
    const int t0 = blockIdx.x * HL_TT, j0 = blockIdx.y * HL_TJ;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const T* x = (const T*)a.x;
    const T* w = (const T*)a.w + (size_t)h * a.J * a.D;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int d0 = 0; d0 < a.D; d0 += HL_TD) {
        for (int i = tid; i < HL_TT * HL_TD; i += 256) {
            const int r = i >> 5, d = i & 31;
            const int tok = t0 + r;
            xs[r][d] = (tok < a.n_tokens && d0 + d < a.D)
                ? to_f32(x[(size_t)tok * a.x_row + (size_t)h * a.x_head + a.x_off + d0 + d]) : 0.0f;
            const int j = j0 + r;
            ws[r][d] = (j < a.J && d0 + d < a.D) ? to_f32(w[(size_t)j * a.D + d0 + d]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < HL_TD; ++d) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { xv[i] = xs[ty + 16 * i][d]; wv[i] = ws[tx + 16 * i][d]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
    T* y = (T*)a.y;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int tok = t0 + ty + 16 * i;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int j = j0 + tx + 16 * jj;
            if (tok < a.n_tokens && j < a.J) {
                float v = acc[i][jj];
                if (a.gate) {
                    const float gv = a.gate[(size_t)tok * a.gate_row + a.gate_off + (size_t)h * a.J + j];
                    v *= 1.0f / (1.0f + expf(-gv));
                }
                y[(size_t)tok * a.y_row + (size_t)h * a.y_head + j] = from_f32<T>(v);
            }
        }
    }
    if (a.tail > 0 && blockIdx.y == 0) {
        for (int i = tid; i < HL_TT * a.tail; i += 256) {
            const int r = i / a.tail, d = i - r * a.tail;
            const int tok = t0 + r;
            if (tok < a.n_tokens)
                y[(size_t)tok * a.y_row + (size_t)h * a.y_head + a.J + d] =
                    x[(size_t)tok * a.x_row + (size_t)h * a.x_head + a.x_tail_off + d];
        }
    }
}

// The same for bfloat16 on tensor cores: a block of four warps owns 64 tokens x 64 outputs of one
// head, a warp 16 tokens x 64 outputs as eight m16n8k16 products per 16 elements of the reduction
// (float32 accumulation).  x and W go through shared memory in chunks of HM_KC elements with rows
// padded by 8 (fragments are read as 32-bit words without bank conflicts); elements beyond D, J or
// the last token are zeros.
#define HM_KC 64
#define HM_LD (HM_KC + 8)

__device__ __forceinline__ void hm_mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128) head_linear_mma_kernel(HeadLinearArgs a) {
    pdl_prologue();
    __shared__ __align__(16) __nv_bfloat16 xs[64 * HM_LD];
    __shared__ __align__(16) __nv_bfloat16 ws[64 * HM_LD];
    const int h = blockIdx.z;
    const int t0 = blockIdx.x * 64, j0 = blockIdx.y * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* x = (const __nv_bfloat16*)a.x;
    const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)h * a.J * a.D;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }
    // 16-byte copies where every row of x and of W starts on a 16-byte boundary
    const bool vec = (a.x_row & 7) == 0 && (a.x_head & 7) == 0 && (a.x_off & 7) == 0 && (a.D & 7) == 0 &&
                     (((uintptr_t)a.x | (uintptr_t)a.w) & 15) == 0;
    for (int d0 = 0; d0 < a.D; d0 += HM_KC) {
        if (vec) {
            for (int i = tid; i < 64 * (HM_KC / 8); i += 128) {
                const int r = i / (HM_KC / 8), d = (i - r * (HM_KC / 8)) * 8;
                const int tok = t0 + r, j = j0 + r;
                const bool d_ok = d0 + d < a.D;
                uint4 xv = make_uint4(0u, 0u, 0u, 0u), wv = make_uint4(0u, 0u, 0u, 0u);
                if (tok < a.n_tokens && d_ok)
                    xv = *reinterpret_cast<const uint4*>(x + (size_t)tok * a.x_row + (size_t)h * a.x_head + a.x_off + d0 + d);
                if (j < a.J && d_ok) wv = *reinterpret_cast<const uint4*>(w + (size_t)j * a.D + d0 + d);
                *reinterpret_cast<uint4*>(xs + r * HM_LD + d) = xv;
                *reinterpret_cast<uint4*>(ws + r * HM_LD + d) = wv;
            }
        } else {
            for (int i = tid; i < 64 * HM_KC; i += 128) {
                const int r = i / HM_KC, d = i - r * HM_KC;
                const int tok = t0 + r, j = j0 + r;
                const bool d_ok = d0 + d < a.D;
                xs[r * HM_LD + d] = (tok < a.n_tokens && d_ok)
                    ? x[(size_t)tok * a.x_row + (size_t)h * a.x_head + a.x_off + d0 + d] : zero;
                ws[r * HM_LD + d] = (j < a.J && d_ok) ? w[(size_t)j * a.D + d0 + d] : zero;
            }
        }
        __syncthreads();
        const int k_end = min(HM_KC, ((a.D - d0 + 15) / 16) * 16);
        for (int k0 = 0; k0 < k_end; k0 += 16) {
            uint32_t af[4];
            const __nv_bfloat16* xr = xs + (warp * 16 + g) * HM_LD + k0 + 2 * t;
            af[0] = *reinterpret_cast<const uint32_t*>(xr);
            af[1] = *reinterpret_cast<const uint32_t*>(xr + 8 * HM_LD);
            af[2] = *reinterpret_cast<const uint32_t*>(xr + 8);
            af[3] = *reinterpret_cast<const uint32_t*>(xr + 8 * HM_LD + 8);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const __nv_bfloat16* wr = ws + (nt * 8 + g) * HM_LD + k0 + 2 * t;
                hm_mma16816(acc[nt], af, *reinterpret_cast<const uint32_t*>(wr),
                            *reinterpret_cast<const uint32_t*>(wr + 8));
            }
        }
        __syncthreads();
    }
    __nv_bfloat16* y = (__nv_bfloat16*)a.y;
    // a thread's two neighbouring outputs as one 4-byte store where they start on an even element
    const bool pairs = (a.y_row & 1) == 0 && (a.y_head & 1) == 0 && (a.J & 1) == 0 && ((uintptr_t)a.y & 3) == 0;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int tok = t0 + warp * 16 + g + half * 8;
            const int j = j0 + nt * 8 + 2 * t;
            if (tok >= a.n_tokens || j >= a.J) continue;
            float v0 = acc[nt][2 * half], v1 = acc[nt][2 * half + 1];
            if (a.gate) {
                const float* gp = a.gate + (size_t)tok * a.gate_row + a.gate_off + (size_t)h * a.J + j;
                v0 *= 1.0f / (1.0f + expf(-gp[0]));
                if (j + 1 < a.J) v1 *= 1.0f / (1.0f + expf(-gp[1]));
            }
            __nv_bfloat16* dst = y + (size_t)tok * a.y_row + (size_t)h * a.y_head + j;
            if (pairs) {
                *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
            } else {
                dst[0] = __float2bfloat16_rn(v0);
                if (j + 1 < a.J) dst[1] = __float2bfloat16_rn(v1);
            }
        }
    }
    if (a.tail > 0 && blockIdx.y == 0) {
        for (int i = tid; i < 64 * a.tail; i += 128) {
            const int r = i / a.tail, d = i - r * a.tail;
            const int tok = t0 + r;
            if (tok < a.n_tokens)
                y[(size_t)tok * a.y_row + (size_t)h * a.y_head + a.J + d] =
                    x[(size_t)tok * a.x_row + (size_t)h * a.x_head + a.x_tail_off + d];
        }
    }
}

extern "C" int mf_head_linear(const HeadLinearArgs* args, int dtype, cudaStream_t stream) {
    const HeadLinearArgs a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.heads < 1 || a.J < 1 || a.D < 1 || a.tail < 0) return MF_ERR_ARGUMENT;
    dim3 grid((a.n_tokens + HL_TT - 1) / HL_TT, (a.J + HL_TJ - 1) / HL_TJ, a.heads);
    static int simt = -1;              // MINFER_B200_HEAD_LINEAR=simt: the FP32-pipe kernel for bfloat16 too
    if (simt < 0) { const char* e = getenv("MINFER_B200_HEAD_LINEAR"); simt = (e && e[0] == 's') ? 1 : 0; }
    if (dtype == MF_DTYPE_F32) mf_launch(head_linear_kernel<float>, grid, dim3(256), 0, stream, a);
    else if (dtype == MF_DTYPE_BF16 && !simt) mf_launch(head_linear_mma_kernel, grid, dim3(128), 0, stream, a);
    else if (dtype == MF_DTYPE_BF16) mf_launch(head_linear_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, a);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// head_prepare: what qk_prepare does, head by head.  A warp owns one head of one token: a query
// head, or a key head together with its value head.  Each query and key head is optionally
// RMS-normed by itself (x / sqrt(mean(x^2) + eps) * weight, one weight of the head's width shared
// by all heads), `rot_dims` dimensions from the head's start are rotated, and the result is
// multiplied by q_mul / k_mul.  Outputs are bfloat16 or float32; a caller that keeps no cache and
// reads its values from the projection passes null for the places it does not want.
// ------------------------------------------------------------------------------------------
struct HeadPrepArgs {
    const float* proj;        // [tokens][in_width]
    long long in_width;
    const int* positions;
    const int* token_row;
    const int* seq_end;
    const double* inv_freq;   // [rot_dims / 2] or null
    const float* q_norm_w;    // [qw] or null
    const float* k_norm_w;    // [kw] or null
    void* q_out;              // [tokens][n_heads][qw]
    void* k_out;              // [tokens][n_kv][kw] or null
    void* v_out;              // [tokens][n_kv][vw] or null
    void* k_cache;            // [pages][n_kv][64][kw] or null
    void* v_cache;            // [pages][n_kv][64][vw] or null
    const int* page_table;
    int table_stride, ring;
    int q_off, n_heads, qw, k_off, n_kv, kw, v_off, vw;
    int rot_dims, rot_style;
    float rot_mag, eps, q_mul, k_mul;
    unsigned* status;
};

// the head at `seg` (width w) normed, rotated and scaled; element d goes to dst[d] and, if page_dst
// is not null, to page_dst[d]
template <typename T>
__device__ __forceinline__ void head_prep_one(const float* seg, int w, const float* norm_w, float mul,
                                              int pos, const HeadPrepArgs& a, T* dst, T* page_dst,
                                              int lane) {
    float rinv = 1.0f;
    if (norm_w != nullptr) {
        float ss = 0.0f;
        for (int d = lane; d < w; d += 32) ss = fmaf(seg[d], seg[d], ss);
        ss = warp_sum(ss);
        rinv = 1.0f / sqrtf(ss / (float)w + a.eps);
    }
    const int half = a.rot_dims >> 1;
    for (int d = lane; d < w; d += 32) {
        float v = seg[d] * rinv;
        if (norm_w != nullptr) v *= norm_w[d];
        if (d < a.rot_dims) {
            int pair, partner;
            bool first;
            if (a.rot_style == 0) { first = d < half; pair = first ? d : d - half; partner = first ? d + half : d - half; }
            else { first = (d & 1) == 0; pair = d >> 1; partner = first ? d + 1 : d - 1; }
            float other = seg[partner] * rinv;
            if (norm_w != nullptr) other *= norm_w[partner];
            double ang = (double)pos * a.inv_freq[pair];
            ang -= 6.283185307179586476925286766559 * floor(ang * 0.15915494309189533576888376337251);
            float s, c;
            sincosf((float)ang, &s, &c);
            c *= a.rot_mag; s *= a.rot_mag;
            v = first ? v * c - other * s : v * c + other * s;
        }
        const T y = from_f32<T>(v * mul);
        if (dst) dst[d] = y;
        if (page_dst) page_dst[d] = y;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) head_prepare_kernel(HeadPrepArgs a, long long items) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int per_token = a.n_heads + a.n_kv;
    const int t = (int)(item / per_token);
    const int h = (int)(item - (long long)t * per_token);
    const int pos = a.positions[t];
    pdl_wait();
    const float* row = a.proj + (size_t)t * a.in_width;
    if (h < a.n_heads) {
        head_prep_one<T>(row + a.q_off + (size_t)h * a.qw, a.qw, a.q_norm_w, a.q_mul, pos, a,
                         (T*)a.q_out + ((size_t)t * a.n_heads + h) * a.qw, (T*)nullptr, lane);
        return;
    }
    const int hk = h - a.n_heads;
    int page = -1;
    if (a.k_cache != nullptr) {
        const int b = a.token_row[t];
        bool keep = true;
        int p_eff = pos;
        if (a.ring > 0) {
            keep = pos >= a.seq_end[b] - a.ring;
            p_eff = pos % a.ring;
        }
        if (keep) {
            page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
            if (page < 0 && lane == 0) atomicOr(a.status, MF_STATUS_BAD_POSITION);
        }
    }
    const int in_page = pos & (MF_PAGE - 1);
    T* k_dst = a.k_out ? (T*)a.k_out + ((size_t)t * a.n_kv + hk) * a.kw : nullptr;
    T* k_page = page >= 0 ? (T*)a.k_cache + (((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.kw : nullptr;
    head_prep_one<T>(row + a.k_off + (size_t)hk * a.kw, a.kw, a.k_norm_w, a.k_mul, pos, a, k_dst, k_page, lane);
    if (a.v_out == nullptr && (page < 0 || a.v_cache == nullptr)) return;
    const float* vs = row + a.v_off + (size_t)hk * a.vw;
    T* v_dst = a.v_out ? (T*)a.v_out + ((size_t)t * a.n_kv + hk) * a.vw : nullptr;
    T* v_page = (page >= 0 && a.v_cache) ? (T*)a.v_cache + (((size_t)page * a.n_kv + hk) * MF_PAGE + in_page) * a.vw : nullptr;
    for (int d = lane; d < a.vw; d += 32) {
        const T y = from_f32<T>(vs[d]);
        if (v_dst) v_dst[d] = y;
        if (v_page) v_page[d] = y;
    }
}

extern "C" int mf_head_prepare(const HeadPrepArgs* args, int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const HeadPrepArgs a = *args;
    if (a.rot_dims < 0 || (a.rot_dims & 1) || (a.rot_dims > 0 && a.inv_freq == nullptr)) return MF_ERR_ARGUMENT;
    if (a.rot_dims > a.qw || a.rot_dims > a.kw || a.n_heads < 1 || a.n_kv < 0) return MF_ERR_ARGUMENT;
    if ((a.k_cache == nullptr) != (a.v_cache == nullptr)) return MF_ERR_ARGUMENT;
    if (a.k_cache != nullptr && a.page_table == nullptr) return MF_ERR_ARGUMENT;
    const long long items = (long long)n_tokens * (a.n_heads + a.n_kv);
    dim3 grid((unsigned)((items + 7) / 8)), block(256);
    if (dtype == MF_DTYPE_F32) mf_launch(head_prepare_kernel<float>, grid, block, 0, stream, a, items);
    else if (dtype == MF_DTYPE_BF16) mf_launch(head_prepare_kernel<__nv_bfloat16>, grid, block, 0, stream, a, items);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}
