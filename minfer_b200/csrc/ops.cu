// Row-wise and element-wise kernels of the step: embedding lookup, RMSNorm, the fused
// rotary + cache write, SwiGLU, row gather, casts.  All reductions are in float32.
//
// Formulas follow the reference's CPU backend: get_rows src/graph/cpu_backend.rs:249-291,
// rms_norm src/vec_ops.rs:500-522 (x * 1/sqrt(mean(x^2)+eps) * w), rotary
// src/graph/cpu_backend.rs:403-434, KV store src/graph/cpu_backend.rs:118-149, silu
// src/vec_ops.rs:131-146.  Its CUDA versions (src/cuda_kernels.cu:531-668) launch one
// kernel per op and one thread per block for the KV store; here bias, rotation and both
// cache writes are one pass over the projection's output.
#include "common.cuh"

// ------------------------------------------------------------------------------------
// embedding: out[t][:] = table[ids[t]][:] * scale  (float32 out: the residual stream is
// float32; scale is 1 for architectures that do not multiply their embeddings)
// ------------------------------------------------------------------------------------
// `rows` (may be null): a second table [n_rows_table][width] of which row row_idx[t] is added,
// unscaled (learned position vectors: row_idx = the tokens' positions); an index outside it sets
// MF_STATUS_BAD_POSITION and adds nothing.
template <typename T, typename TR>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int width, int vocab, float scale,
                             const TR* __restrict__ rows, const int* __restrict__ row_idx,
                             int n_rows_table, unsigned* __restrict__ status) {
    pdl_prologue();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * width;
    const TR* extra = nullptr;
    if (rows != nullptr) {
        const int r = row_idx[t];
        if (r < 0 || r >= n_rows_table) {
            if (threadIdx.x == 0) atomicOr(status, MF_STATUS_BAD_POSITION);
        } else {
            extra = rows + (size_t)r * width;
        }
    }
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, MF_STATUS_BAD_TOKEN);
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * width;
    if (extra != nullptr) {
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            o[i] = fmaf(to_f32(row[i]), scale, 0.0f) + to_f32(extra[i]);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32(row[i]) * scale;
    }
}

extern "C" int mf_embed_rows(const void* table, int table_dtype, const int* ids, float* out,
                             int n_tokens, int width, int vocab, float scale, const void* rows,
                             int rows_dtype, const int* row_idx, int n_rows_table,
                             unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rows != nullptr && row_idx == nullptr) return MF_ERR_ARGUMENT;
    const int threads = width >= 1024 ? 256 : 128;
#define MF_EMBED(T, TR) \
    mf_launch(embed_kernel<T, TR>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)table, ids, out, \
              width, vocab, scale, (const TR*)rows, row_idx, n_rows_table, status)
    const bool rows_f32 = rows == nullptr || rows_dtype == MF_DTYPE_F32;
    if (rows != nullptr && rows_dtype != MF_DTYPE_F32 && rows_dtype != MF_DTYPE_BF16) return MF_ERR_UNSUPPORTED;
    if (table_dtype == MF_DTYPE_F32) {
        if (rows_f32) MF_EMBED(float, float); else MF_EMBED(float, __nv_bfloat16);
    } else if (table_dtype == MF_DTYPE_BF16) {
        if (rows_f32) MF_EMBED(__nv_bfloat16, float); else MF_EMBED(__nv_bfloat16, __nv_bfloat16);
    } else {
        return MF_ERR_UNSUPPORTED;
    }
#undef MF_EMBED
    return MF_LAUNCH_CHECK();
}

extern "C" int mf_embed(const void* table, int table_dtype, const int* ids, float* out,
                        int n_tokens, int width, int vocab, float scale, unsigned* status,
                        cudaStream_t stream) {
    return mf_embed_rows(table, table_dtype, ids, out, n_tokens, width, vocab, scale, nullptr, 0,
                         nullptr, 0, status, stream);
}

// ------------------------------------------------------------------------------------
// RMSNorm over rows of the float32 residual stream; optional row gather (rows[r] names the
// input row of output row r).  y = x * rsqrt(mean(x^2) + eps) * w
// ------------------------------------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ rows, TO* __restrict__ y, int width,
                               float eps) {
    pdl_prologue();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) yr[i] = from_f32<TO>(xr[i] * scale * w[i]);
}

// four neighbouring outputs in one store
template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<unsigned*>(&lo);
        v.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};

// the same with float4 accesses and the row kept in registers (one pass over memory), for
// widths that are multiples of 4 up to 16384
template <typename TO>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                   const int* __restrict__ rows, TO* __restrict__ y, int width, float eps) {
    // the norm's weights (and the row to take, an input of the step) are fetched while the
    // kernel before this one still runs
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int nv = width >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * width);
    float4 g[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) g[j] = reinterpret_cast<const float4*>(w)[i];
    }
    pdl_wait();
    float4 row[4];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = xr[i];
            row[j] = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = row[j];
            Pack4<TO>::store(yr + 4 * i, v.x * scale * g[j].x, v.y * scale * g[j].y,
                             v.z * scale * g[j].z, v.w * scale * g[j].w);
        }
    }
}

extern "C" int mf_rmsnorm(const float* x, const float* w, const int* rows, void* y, int out_dtype,
                          int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 4 == 0 && width <= 16384 && (out_dtype == MF_DTYPE_F32 || out_dtype == MF_DTYPE_BF16)) {
        // up to four float4 a thread: fewer warps to sum over, more rows on an SM at once
        // (2,048 rows of 3,584: 6.1 us with 256 threads, 13.1 us with 1,024)
        int threads = 32;
        while (threads < 1024 && threads * 16 < width) threads <<= 1;
        if (out_dtype == MF_DTYPE_F32)
            mf_launch(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows,
                      (float*)y, width, eps);
        else
            mf_launch(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, w,
                      rows, (__nv_bfloat16*)y, width, eps);
        return MF_LAUNCH_CHECK();
    }
    // the block size is a function of the width only, so a row's sum never depends on the batch
    int threads = 32;
    while (threads < 512 && threads * 4 < width) threads <<= 1;
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows, (float*)y, width, eps);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows, (__nv_bfloat16*)y,
                                                                      width, eps);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Residual add + RMSNorm in one pass: h[r] += bias + sum_s partial[s][r] (the K splits of the
// projection before it, added in split order), then y[r] = rmsnorm(h[r]) * w.  Saves the
// separate reduction kernel and one round trip of h.
// ------------------------------------------------------------------------------------
template <typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ partial,
                                   int n_partials, const float* __restrict__ bias,
                                   const float* __restrict__ w, TO* __restrict__ y, int n_rows,
                                   int width, float eps) {
    pdl_prologue();
    extern __shared__ float row_s[];                  // the updated row
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * width;
    const size_t plane = (size_t)n_rows * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float add = 0.0f;
        for (int s = 0; s < n_partials; ++s) add += partial[s * plane + (size_t)r * width + i];
        if (bias) add += bias[i];
        const float v = hr[i] + add;
        hr[i] = v;
        row_s[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) yr[i] = from_f32<TO>(row_s[i] * scale * w[i]);
}

// the same for widths that are multiples of 4 up to 4 * 4 * 1024: float4 accesses, the row
// kept in registers, all loads of a thread independent of each other
#define ARN_MAXV 4
template <typename TO, int MAXV>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ partial, int n_partials,
                       const float* __restrict__ bias, const float* __restrict__ w,
                       TO* __restrict__ y, int n_rows, int width, float eps) {
    // the norm's weights are fetched while the kernel before this one still runs
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int nv = width >> 2;                         // float4 per row
    float4* hr = reinterpret_cast<float4*>(h + (size_t)r * width);
    const size_t plane4 = ((size_t)n_rows * width) >> 2;
    const float4* pr = reinterpret_cast<const float4*>(partial) + ((size_t)r * width >> 2);
    float4 g[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) g[j] = reinterpret_cast<const float4*>(w)[i];
    }
    pdl_wait();
    float4 row[MAXV];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            float4 v;
            if (MAXV == 1) v = hr[i];                 // in flight together with the splits
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll (MAXV == 1 ? 10 : 4)
            for (int s = 0; s < n_partials; ++s) {
                const float4 p = pr[s * plane4 + i];
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
            }
            if (bias) {
                const float4 b = reinterpret_cast<const float4*>(bias)[i];
                acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
            }
            if (MAXV != 1) v = hr[i];
            v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
            hr[i] = v;
            row[j] = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = row[j];
            Pack4<TO>::store(yr + 4 * i, v.x * scale * g[j].x, v.y * scale * g[j].y,
                             v.z * scale * g[j].z, v.w * scale * g[j].w);
        }
    }
}

extern "C" int mf_add_rmsnorm(float* h, const float* partial, int n_partials, const float* bias,
                              const float* w, void* y, int out_dtype, int n_rows, int width,
                              float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_partials < 0 || (n_partials > 0 && partial == nullptr)) return MF_ERR_ARGUMENT;
    if (width % 4 == 0 && width <= 4 * ARN_MAXV * 1024 && (out_dtype == MF_DTYPE_F32 ||
                                                            out_dtype == MF_DTYPE_BF16)) {
        // one thread per float4 where that fits; the block size depends on the width only
        int threads = 32;
        while (threads < 1024 && threads * 4 < width) threads <<= 1;
        if (out_dtype == MF_DTYPE_F32)
            mf_launch(add_rmsnorm_vec_kernel<float, ARN_MAXV>, dim3(n_rows), dim3(threads), 0, stream,
                h, partial, n_partials, bias, w, (float*)y, n_rows, width, eps);
        else if (width <= 4 * 1024)        // one float4 a thread: more splits in flight at once
            mf_launch(add_rmsnorm_vec_kernel<__nv_bfloat16, 1>, dim3(n_rows), dim3(threads), 0, stream,
                h, partial, n_partials, bias, w, (__nv_bfloat16*)y, n_rows, width, eps);
        else
            mf_launch(add_rmsnorm_vec_kernel<__nv_bfloat16, ARN_MAXV>, dim3(n_rows), dim3(threads), 0, stream,
                h, partial, n_partials, bias, w, (__nv_bfloat16*)y, n_rows, width, eps);
        return MF_LAUNCH_CHECK();
    }
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return MF_ERR_UNSUPPORTED;
    int threads = 32;
    while (threads < 512 && threads * 4 < width) threads <<= 1;
    if (out_dtype == MF_DTYPE_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mf_launch(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, h, partial, n_partials, bias, w,
                                                                    (float*)y, n_rows, width, eps);
    } else if (out_dtype == MF_DTYPE_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mf_launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, 
            h, partial, n_partials, bias, w, (__nv_bfloat16*)y, n_rows, width, eps);
    } else {
        return MF_ERR_UNSUPPORTED;
    }
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// rotary + cache write.  Input: the fused projection's float32 output qkv[t] =
// [q (n_heads*hd) | k (n_kv*hd) | v (n_kv*hd)], bias already added.  Rotates q and k by
// the token's position (angle pos * inv_freq[i] formed and reduced mod 2 pi in double, its sine
// and cosine in float32), writes
//   q_out[t][h][:]              (activation type)
//   k_out[t][hk][:], v_out[..]  (activation type; the step's own keys and values, which
//                                prefill attention reads; may be null)
//   cache pages                 (if k_cache is not null): position p of batch row b lies in
//                                page page_table[b*table_stride + (p' / 64)], p' = p % ring
//                                for a ring of `ring` positions, else p; inside the page at
//                                [kv_head][p % 64][:].
// A ring holds only the last `ring` positions: a prompt longer than the ring writes just
// those (seq_end[b] is the sequence's length after this step).
// style: 0 = pairs (i, i + R/2) ("NeoX", the reference's NonInterleaved), 1 = pairs
// (2i, 2i+1); R = rotary_dim <= hd, dimensions beyond R pass through; inv_freq null = no
// rotation at all.
// n_partials > 0: `qkv` holds [n_partials][tokens][width] K splits of the projection, which
// are added here in split order together with `bias` (else bias must already be inside).
// ------------------------------------------------------------------------------------
// The angle pos * inv_freq reduced to [0, 2 pi): product and reduction in double (a float32
// product is off by 1e-4 rad at position 2,000 and by 2e-3 rad at 32,000), sine and cosine of
// the small remainder in float32.
__device__ __forceinline__ float rotary_angle(int pos, double inv_freq) {
    const double two_pi = 6.283185307179586476925286766559;
    const double th = (double)pos * inv_freq;
    return (float)(th - two_pi * floor(th / two_pi));
}

template <typename T>
__global__ void rope_kvstore_kernel(const float* __restrict__ qkv, int n_partials, int n_tokens,
                                    const float* __restrict__ bias,
                                    const int* __restrict__ positions,
                                    const int* __restrict__ token_row,
                                    const int* __restrict__ seq_end,
                                    const double* __restrict__ inv_freq, T* __restrict__ q_out,
                                    T* __restrict__ k_out, T* __restrict__ v_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache,
                                    const int* __restrict__ page_table, int table_stride, int ring,
                                    int n_heads, int n_kv, int hd, int rotary_dim, int style,
                                    unsigned* __restrict__ status) {
    pdl_prologue();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int b = token_row[t];
    const int half = hd >> 1;
    const int rhalf = rotary_dim >> 1;
    const int n_slots = (n_heads + 2 * n_kv) * half;
    const size_t in_width = (size_t)(n_heads + 2 * n_kv) * hd;
    const float* in = qkv + (size_t)t * in_width;
    const size_t plane = (size_t)n_tokens * in_width;
    // value of element `col` of this token's projection
    auto value = [&](int col) -> float {
        float v = in[col];
        for (int sp = 1; sp < n_partials; ++sp) v += in[sp * plane + col];
        if (bias != nullptr) v += bias[col];
        return v;
    };

    // where this token's keys and values go in the cache
    long long cache_row = -1;     // element offset of [kv_head 0][pos%64][0] in the page, or -1
    if (k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (ring > 0) {
            keep = pos >= seq_end[b] - ring;
            p_eff = pos % ring;
        }
        if (keep) {
            const int page = page_table[(size_t)b * table_stride + (p_eff >> 6)];
            if (page < 0) {
                if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, MF_STATUS_BAD_POSITION);
            } else {
                cache_row = ((long long)page * n_kv * MF_PAGE + (pos & (MF_PAGE - 1))) * hd;
            }
        }
    }

    // the token's rotation (cos, sin) per pair, once per block: every head uses the same
    __shared__ float2 cs_table[128];
    if (inv_freq != nullptr) {
        for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
            float sn, cs;
            sincosf(rotary_angle(pos, inv_freq[i]), &sn, &cs);
            cs_table[i] = make_float2(cs, sn);
        }
    }
    __syncthreads();
    // blockIdx.y spreads a token's pairs over several blocks when there are few tokens
    for (int s = blockIdx.y * blockDim.x + threadIdx.x; s < n_slots; s += gridDim.y * blockDim.x) {
        const int head = s / half;      // 0..n_heads-1: q, then k heads, then v heads
        const int i = s - head * half;
        const int hbase = head * hd;
        int d0, d1;
        float x0, x1;
        const bool is_v = head >= n_heads + n_kv;
        if (!is_v && inv_freq != nullptr && i < rhalf) {
            if (style == 0) { d0 = i; d1 = i + rhalf; } else { d0 = 2 * i; d1 = 2 * i + 1; }
            const float a = value(hbase + d0), c = value(hbase + d1);
            const float cs = cs_table[i].x, sn = cs_table[i].y;
            x0 = a * cs - c * sn;
            x1 = a * sn + c * cs;
        } else {
            // pass-through pair: for rotated heads the dimensions beyond R, else (2i, 2i+1)
            const int j = (!is_v && inv_freq != nullptr) ? rotary_dim + 2 * (i - rhalf) : 2 * i;
            d0 = j; d1 = j + 1;
            x0 = value(hbase + d0);
            x1 = value(hbase + d1);
        }
        const T y0 = from_f32<T>(x0), y1 = from_f32<T>(x1);
        if (head < n_heads) {
            T* o = q_out + ((size_t)t * n_heads + head) * hd;
            o[d0] = y0; o[d1] = y1;
        } else {
            const int hk = is_v ? head - n_heads - n_kv : head - n_heads;
            T* step_out = is_v ? v_out : k_out;
            if (step_out != nullptr) {
                T* o = step_out + ((size_t)t * n_kv + hk) * hd;
                o[d0] = y0; o[d1] = y1;
            }
            if (cache_row >= 0) {
                T* c = (is_v ? v_cache : k_cache) + cache_row + (long long)hk * MF_PAGE * hd;
                c[d0] = y0; c[d1] = y1;
            }
        }
    }
}

// The common case in wide accesses: pairs (i, i + hd/2), the whole head rotated, head sizes
// that are multiples of 8.  A thread takes 4 neighbouring pairs of a q or k head (two float4
// loads per split, two 4-element stores per destination) or 8 elements of a v head.
// SPLIT: the input holds K splits of the projection (decoding: few tokens, every load of a
// thread in flight at once); without it the kernel keeps few registers, so that many CTAs of
// a long prompt share an SM and hide each other's loads.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(128)
rope_kvstore_vec_kernel(const float* __restrict__ qkv, int n_partials, int n_tokens,
                        const float* __restrict__ bias, const int* __restrict__ positions,
                        const int* __restrict__ token_row, const int* __restrict__ seq_end,
                        const double* __restrict__ inv_freq, T* __restrict__ q_out,
                        T* __restrict__ k_out, T* __restrict__ v_out, T* __restrict__ k_cache,
                        T* __restrict__ v_cache, const int* __restrict__ page_table,
                        int table_stride, int ring, int n_heads, int n_kv, int hd,
                        unsigned* __restrict__ status) {
    // Positions, rows, page tables, inverse frequencies and the bias are the step's inputs
    // (copied to the device before its first kernel) or weights: they are read, and the
    // angles' sines and cosines formed, while the projection before this kernel still runs.
    pdl_launch_dependents();
    __shared__ float2 cs_table[128];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int b = token_row[t];
    const int half = hd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(rotary_angle(pos, inv_freq[i]), &sn, &cs);
        cs_table[i] = make_float2(cs, sn);
    }
    const size_t in_width = (size_t)(n_heads + 2 * n_kv) * hd;
    const float* in = qkv + (size_t)t * in_width;
    const size_t plane = (size_t)n_tokens * in_width;
    // the sums of two columns at once: all loads of up to 8 splits are issued before the first
    // addition (splits are added in split order, as everywhere)
    auto load_pair = [&](int col_a, int col_c, float4& a, float4& c) {
        a = *reinterpret_cast<const float4*>(in + col_a);
        c = *reinterpret_cast<const float4*>(in + col_c);
        for (int s0 = 1; SPLIT && s0 < n_partials; s0 += 8) {
            float4 pa[8], pc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_partials) {
                    pa[j] = *reinterpret_cast<const float4*>(in + (s0 + j) * plane + col_a);
                    pc[j] = *reinterpret_cast<const float4*>(in + (s0 + j) * plane + col_c);
                }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_partials) {
                    a.x += pa[j].x; a.y += pa[j].y; a.z += pa[j].z; a.w += pa[j].w;
                    c.x += pc[j].x; c.y += pc[j].y; c.z += pc[j].z; c.w += pc[j].w;
                }
        }
        if (bias != nullptr) {
            const float4 ba = *reinterpret_cast<const float4*>(bias + col_a);
            const float4 bc = *reinterpret_cast<const float4*>(bias + col_c);
            a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
            c.x += bc.x; c.y += bc.y; c.z += bc.z; c.w += bc.w;
        }
    };
    long long cache_row = -1;
    if (k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (ring > 0) {
            keep = pos >= seq_end[b] - ring;
            p_eff = pos % ring;
        }
        if (keep) {
            const int page = page_table[(size_t)b * table_stride + (p_eff >> 6)];
            if (page < 0) {
                if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, MF_STATUS_BAD_POSITION);
            } else {
                cache_row = ((long long)page * n_kv * MF_PAGE + (pos & (MF_PAGE - 1))) * hd;
            }
        }
    }
    __syncthreads();
    pdl_wait();                    // from here on: the projection's sums
    const int upr = half >> 2;                         // units per rotated head
    const int n_rot = (n_heads + n_kv) * upr;
    const int upv = hd >> 3;                           // units per value head
    const int n_units = n_rot + n_kv * upv;
    for (int u = blockIdx.y * blockDim.x + threadIdx.x; u < n_units; u += gridDim.y * blockDim.x) {
        if (u < n_rot) {
            const int head = u / upr;
            const int i0 = (u - head * upr) << 2;
            float4 a, c;
            load_pair(head * hd + i0, head * hd + half + i0, a, c);
            const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
            float lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float cs = cs_table[i0 + j].x, sn = cs_table[i0 + j].y;
                lo[j] = av[j] * cs - cv[j] * sn;
                hi[j] = av[j] * sn + cv[j] * cs;
            }
            if (head < n_heads) {
                T* o = q_out + ((size_t)t * n_heads + head) * hd + i0;
                Pack4<T>::store(o, lo[0], lo[1], lo[2], lo[3]);
                Pack4<T>::store(o + half, hi[0], hi[1], hi[2], hi[3]);
            } else {
                const int hk = head - n_heads;
                if (k_out != nullptr) {
                    T* o = k_out + ((size_t)t * n_kv + hk) * hd + i0;
                    Pack4<T>::store(o, lo[0], lo[1], lo[2], lo[3]);
                    Pack4<T>::store(o + half, hi[0], hi[1], hi[2], hi[3]);
                }
                if (cache_row >= 0) {
                    T* o = k_cache + cache_row + (long long)hk * MF_PAGE * hd + i0;
                    Pack4<T>::store(o, lo[0], lo[1], lo[2], lo[3]);
                    Pack4<T>::store(o + half, hi[0], hi[1], hi[2], hi[3]);
                }
            }
        } else {
            const int idx = u - n_rot;
            const int hk = idx / upv;
            const int e0 = (idx - hk * upv) << 3;
            const int col = (n_heads + n_kv + hk) * hd + e0;
            float4 a, c;
            load_pair(col, col + 4, a, c);
            if (v_out != nullptr) {
                T* o = v_out + ((size_t)t * n_kv + hk) * hd + e0;
                Pack4<T>::store(o, a.x, a.y, a.z, a.w);
                Pack4<T>::store(o + 4, c.x, c.y, c.z, c.w);
            }
            if (cache_row >= 0) {
                T* o = v_cache + cache_row + (long long)hk * MF_PAGE * hd + e0;
                Pack4<T>::store(o, a.x, a.y, a.z, a.w);
                Pack4<T>::store(o + 4, c.x, c.y, c.z, c.w);
            }
        }
    }
}

extern "C" int mf_rope_kvstore(const float* qkv, int n_partials, const float* bias,
                               const int* positions, const int* token_row,
                               const int* seq_end, const double* inv_freq, void* q_out, void* k_out,
                               void* v_out, void* k_cache, void* v_cache, const int* page_table,
                               int table_stride, int ring, int n_tokens, int n_heads, int n_kv,
                               int hd, int rotary_dim, int style, int dtype, unsigned* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 2 != 0 || rotary_dim % 2 != 0 || rotary_dim > hd || rotary_dim < 0 || rotary_dim > 256)
        return MF_ERR_UNSUPPORTED;
    if (ring % MF_PAGE != 0) return MF_ERR_ARGUMENT;
    const int n_slots = (n_heads + 2 * n_kv) * (hd / 2);
    const int threads = 128;
    // enough blocks to fill the GPU even for a handful of tokens
    int gy = (592 + n_tokens - 1) / n_tokens;
    const int gy_max = (n_slots + threads - 1) / threads;
    if (gy > gy_max) gy = gy_max;
    if (gy < 1) gy = 1;
    const dim3 grid(n_tokens, gy);
    if (inv_freq != nullptr && style == 0 && rotary_dim == hd && hd % 8 == 0 &&
        (dtype == MF_DTYPE_F32 || dtype == MF_DTYPE_BF16)) {
        const int n_units = (n_heads + n_kv) * (hd / 8) + n_kv * (hd / 8);
        int vy = (592 + n_tokens - 1) / n_tokens;
        const int vy_max = (n_units + threads - 1) / threads;
        if (vy > vy_max) vy = vy_max;
        if (vy < 1) vy = 1;
        const dim3 vgrid(n_tokens, vy);
#define MF_ROPE_VEC(T, SPLIT)                                                                    \
    mf_launch(rope_kvstore_vec_kernel<T, SPLIT>, vgrid, dim3(threads), 0, stream, qkv, n_partials, \
              n_tokens, bias, positions, token_row, seq_end, inv_freq, (T*)q_out, (T*)k_out,       \
              (T*)v_out, (T*)k_cache, (T*)v_cache, page_table, table_stride, ring, n_heads, n_kv,  \
              hd, status)
        if (dtype == MF_DTYPE_F32) {
            if (n_partials > 1) MF_ROPE_VEC(float, true); else MF_ROPE_VEC(float, false);
        } else {
            if (n_partials > 1) MF_ROPE_VEC(__nv_bfloat16, true); else MF_ROPE_VEC(__nv_bfloat16, false);
        }
#undef MF_ROPE_VEC
        return MF_LAUNCH_CHECK();
    }
    if (dtype == MF_DTYPE_F32)
        mf_launch(rope_kvstore_kernel<float>, dim3(grid), dim3(threads), 0, stream, 
            qkv, n_partials, n_tokens, bias, positions, token_row, seq_end, inv_freq, (float*)q_out, (float*)k_out,
            (float*)v_out, (float*)k_cache, (float*)v_cache, page_table, table_stride, ring,
            n_heads, n_kv, hd, rotary_dim, style, status);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(rope_kvstore_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, 
            qkv, n_partials, n_tokens, bias, positions, token_row, seq_end, inv_freq, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache, page_table, table_stride, ring, n_heads, n_kv, hd,
            rotary_dim, style, status);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// SwiGLU over the fused gate|up projection, silu(z) = z / (1 + exp(-z)), in float32:
//   layout 0 (gate rows then up rows):   out[t][j] = silu(gu[t][j])  * gu[t][nf + j]
//   layout 1 (rows alternate gate, up):  out[t][j] = silu(gu[t][2j]) * gu[t][2j + 1]
// ------------------------------------------------------------------------------------
// activation of the gate: 0 silu, 1 the tanh form of gelu
__device__ __forceinline__ float gate_activation(float g, int act) {
    if (act == 1) {
        const float inner = 0.7978845608028654f * fmaf(0.044715f * g, g * g, g);
        return 0.5f * g * (1.0f + tanhf(inner));
    }
    return g / (1.0f + expf(-g));
}

template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int nf,
                              long long total, int interleaved, int act) {
    pdl_prologue();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / nf;
        const int j = (int)(idx - t * nf);
        const float g = to_f32(gu[t * 2 * nf + (interleaved ? 2 * j : j)]);
        const float u = to_f32(gu[t * 2 * nf + (interleaved ? 2 * j + 1 : nf + j)]);
        out[idx] = from_f32<TO>(gate_activation(g, act) * u);
    }
}

extern "C" int mf_swiglu(const void* gu, int in_dtype, void* out, int out_dtype, int n_rows, int nf,
                         int interleaved, int act, cudaStream_t stream) {
    if (act != 0 && act != 1) return MF_ERR_ARGUMENT;
    const long long total = (long long)n_rows * nf;
    if (total <= 0) return 0;
    const int threads = 256;
    const long long cap = (long long)mf_sm_count() * 16;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
#define MF_SWIGLU(TI, TO) \
    mf_launch(swiglu_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)gu, (TO*)out, nf, total, \
                                                          interleaved, act)
    if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_F32) MF_SWIGLU(float, float);
    else if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_BF16) MF_SWIGLU(float, __nv_bfloat16);
    else if (in_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_BF16)
        MF_SWIGLU(__nv_bfloat16, __nv_bfloat16);
    else return MF_ERR_UNSUPPORTED;
#undef MF_SWIGLU
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// row gather of the float32 residual stream: out[r][:] = x[rows[r]][:]
// ------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int width) {
    pdl_prologue();
    const float* xr = x + (size_t)rows[blockIdx.x] * width;
    float* o = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = xr[i];
}

extern "C" int mf_gather_rows(const float* x, const int* rows, float* out, int n_rows, int width,
                              cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    mf_launch(gather_rows_kernel, dim3(n_rows), dim3(256), 0, stream, x, rows, out, width);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// cast between float32 and bfloat16 (round to nearest even)
// ------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(in[i]));
}

extern "C" int mf_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                       cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const long long cap = (long long)mf_sm_count() * 16;
    const int blocks = (int)(want < cap ? want : cap);
    if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_BF16)
        mf_launch(cast_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            (const float*)in, (__nv_bfloat16*)out, n);
    else if (in_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_F32)
        mf_launch(cast_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)in, (float*)out, n);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// a table row added to every row of the float32 residual stream: h[t][:] += table[idx[t]][:]
// (learned position vectors: idx = the tokens' positions).  An index outside the table sets a
// status bit and adds nothing.
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rows_kernel(float* __restrict__ h, const T* __restrict__ table,
                                const int* __restrict__ idx, int width, int n_table,
                                unsigned* __restrict__ status) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int r = idx[t];                       // an input of the step
    pdl_wait();
    if (r < 0 || r >= n_table) {
        if (threadIdx.x == 0) atomicOr(status, MF_STATUS_BAD_POSITION);
        return;
    }
    const T* row = table + (size_t)r * width;
    float* o = h + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] += to_f32(row[i]);
}

extern "C" int mf_add_rows(float* h, const void* table, int table_dtype, const int* idx,
                           int n_rows, int width, int n_table, unsigned* status,
                           cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == MF_DTYPE_F32)
        mf_launch(add_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, h,
                  (const float*)table, idx, width, n_table, status);
    else if (table_dtype == MF_DTYPE_BF16)
        mf_launch(add_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, h,
                  (const __nv_bfloat16*)table, idx, width, n_table, status);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// RMSNorm followed by a token shift, in float32:
//     n_t = x_t * rsqrt(mean(x_t^2) + eps) * w        y_t = n_t + (n_{t-1} - n_t) * s
// n_{t-1} is the normed row of the sequence's position before: the row above in the step, or,
// for the first token a sequence brings, what the sequence's state holds (zeros at position
// 0).  The state takes n of the last token a sequence brings.  A row that brings one token
// reads and writes its state in the same threads; for rows that bring more the state is
// written by norm_shift_save_kernel, launched behind this one (the block of a row's first
// token reads the state while the block of its last would write it).
// ------------------------------------------------------------------------------------
// `partial` (may be null): the K splits [n_partials][tokens][width] of the projection before,
// which this kernel adds into x first, with `bias`, in split order (x is then complete in
// memory).  Only in steps in which every sequence brings one token: a row with a row above it
// in the step would need that row complete too, which only its own block makes it.
// SPLITS: compiled with the addition of the K splits (kept out of the form for prompts, which
// then needs few registers and shares an SM among several rows).
template <typename TO, bool SPLITS>
__global__ void norm_shift_kernel(float* x, const float* __restrict__ partial, int n_partials,
                                  const float* __restrict__ bias, int n_tokens,
                                  const float* __restrict__ w, const float* __restrict__ shift,
                                  const int* __restrict__ positions,
                                  const int* __restrict__ token_row,
                                  const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ slots, float* __restrict__ state,
                                  TO* __restrict__ y, int width, float eps) {
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int b = token_row[t];
    const int pos = positions[t];
    const bool first = t == cu_seqlens[b];
    const bool last = t == cu_seqlens[b + 1] - 1;
    float* st = state + (size_t)slots[b] * width;
    pdl_wait();
    float* xr = x + (size_t)t * width;
    const float* xp = xr - width;                       // the row above (used unless first)
    float ss = 0.0f, sp = 0.0f;
    if (SPLITS && n_partials > 0) {
        // every split's load of an element is in flight at once (a split beyond n_partials
        // reads the last one again and adds nothing); the sums keep the split order
        const size_t plane = (size_t)n_tokens * width;
        const float* pr = partial + (size_t)t * width;
        const int last_split = n_partials - 1;
        if ((width & 3) == 0 && n_partials <= 16) {
            for (int i = threadIdx.x; i < (width >> 2); i += blockDim.x) {
                float4 v = reinterpret_cast<const float4*>(xr)[i];
                float4 pv[16];
#pragma unroll
                for (int s = 0; s < 16; ++s)
                    pv[s] = reinterpret_cast<const float4*>(pr + (size_t)min(s, last_split) * plane)[i];
                if (bias != nullptr) {
                    const float4 bv = reinterpret_cast<const float4*>(bias)[i];
                    v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
                }
#pragma unroll
                for (int s = 0; s < 16; ++s) {
                    if (s < n_partials) { v.x += pv[s].x; v.y += pv[s].y; v.z += pv[s].z; v.w += pv[s].w; }
                }
                reinterpret_cast<float4*>(xr)[i] = v;       // read again below
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
                ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            __syncthreads();                                // other threads read these elements below
        } else {
            for (int i = threadIdx.x; i < width; i += blockDim.x) {
                float v = xr[i];
                if (bias != nullptr) v += bias[i];
                for (int s = 0; s < n_partials; ++s) v += pr[s * plane + i];
                xr[i] = v;                                  // read again below by this same thread
                ss = fmaf(v, v, ss);
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = xr[i];
            ss = fmaf(v, v, ss);
            if (!first) {
                const float u = xp[i];
                sp = fmaf(u, u, sp);
            }
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    float scale_p = 0.0f;
    if (!first) {
        sp = block_sum(sp, scratch);
        scale_p = 1.0f / sqrtf(sp / (float)width + eps);
    }
    TO* yr = y + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float g = w[i];
        const float n = xr[i] * scale * g;
        float before;
        if (!first) before = xp[i] * scale_p * g;
        else before = pos > 0 ? st[i] : 0.0f;
        yr[i] = from_f32<TO>(n + (before - n) * shift[i]);
        if (first && last) st[i] = n;
    }
}

// the form for prompts: float4 accesses, the row and the row above (or the state) kept in
// registers, one pass over memory; widths that are multiples of 4 up to 8 * blockDim
template <typename TO>
__global__ void __launch_bounds__(1024)
norm_shift_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                      const float* __restrict__ shift, const int* __restrict__ positions,
                      const int* __restrict__ token_row, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ slots, float* __restrict__ state,
                      TO* __restrict__ y, int width, float eps) {
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int b = token_row[t];
    const int pos = positions[t];
    const bool first = t == cu_seqlens[b];
    const bool last = t == cu_seqlens[b + 1] - 1;
    float4* st = reinterpret_cast<float4*>(state + (size_t)slots[b] * width);
    const int nv = width >> 2;
    float4 g[2], sh[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            g[j] = reinterpret_cast<const float4*>(w)[i];
            sh[j] = reinterpret_cast<const float4*>(shift)[i];
        }
    }
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)t * width);
    const float4* xp = xr - nv;                         // the row above (used unless first)
    float4 row[2], prev[2];
    float ss = 0.0f, sp = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = xr[i];
            row[j] = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            if (!first) {
                const float4 u = xp[i];
                prev[j] = u;
                sp = fmaf(u.x, u.x, sp); sp = fmaf(u.y, u.y, sp);
                sp = fmaf(u.z, u.z, sp); sp = fmaf(u.w, u.w, sp);
            } else {
                prev[j] = pos > 0 ? st[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    float scale_p = 1.0f;
    if (!first) {
        sp = block_sum(sp, scratch);
        scale_p = 1.0f / sqrtf(sp / (float)width + eps);
    }
    TO* yr = y + (size_t)t * width;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = row[j], u = prev[j], gg = g[j], s4 = sh[j];
            const float n0 = v.x * scale * gg.x, n1 = v.y * scale * gg.y;
            const float n2 = v.z * scale * gg.z, n3 = v.w * scale * gg.w;
            // the state already holds normed values; a row above is normed here
            const float b0 = first ? u.x : u.x * scale_p * gg.x, b1 = first ? u.y : u.y * scale_p * gg.y;
            const float b2 = first ? u.z : u.z * scale_p * gg.z, b3 = first ? u.w : u.w * scale_p * gg.w;
            Pack4<TO>::store(yr + 4 * i, n0 + (b0 - n0) * s4.x, n1 + (b1 - n1) * s4.y,
                             n2 + (b2 - n2) * s4.z, n3 + (b3 - n3) * s4.w);
            if (first && last) st[i] = make_float4(n0, n1, n2, n3);
        }
    }
}

__global__ void norm_shift_save_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                       const int* __restrict__ cu_seqlens,
                                       const int* __restrict__ slots, float* __restrict__ state,
                                       int width, float eps) {
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int b = blockIdx.x;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
    if (hi - lo < 2) return;                            // nothing, or done by the kernel before
    float* st = state + (size_t)slots[b] * width;
    pdl_wait();
    const float* xr = x + (size_t)(hi - 1) * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) st[i] = xr[i] * scale * w[i];
}

// `multi`: some row may bring more than one token (then the second kernel runs too, and no
// partial sums are taken)
extern "C" int mf_norm_shift(float* x, const float* partial, int n_partials, const float* bias,
                             const float* w, const float* shift,
                             const int* positions, const int* token_row, const int* cu_seqlens,
                             const int* slots, float* state, void* y, int out_dtype, int n_tokens,
                             int n_rows, int width, float eps, int multi, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_partials < 0 || (n_partials > 0 && (multi || partial == nullptr))) return MF_ERR_ARGUMENT;
    // the block size is a function of the width only, so a row's sum never depends on the batch
    int threads = 32;
    while (threads < 512 && threads * 4 < width) threads <<= 1;
    if (n_partials == 0 && (width & 3) == 0 && width <= 8192 && ((uintptr_t)x & 15) == 0 &&
        ((uintptr_t)state & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
        (out_dtype == MF_DTYPE_F32 || out_dtype == MF_DTYPE_BF16) && multi) {
        int vt = 32;
        while (vt < 1024 && vt * 8 < width) vt <<= 1;
        if (out_dtype == MF_DTYPE_F32)
            mf_launch(norm_shift_vec_kernel<float>, dim3(n_tokens), dim3(vt), 0, stream, (const float*)x, w,
                      shift, positions, token_row, cu_seqlens, slots, state, (float*)y, width, eps);
        else
            mf_launch(norm_shift_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(vt), 0, stream,
                      (const float*)x, w, shift, positions, token_row, cu_seqlens, slots, state,
                      (__nv_bfloat16*)y, width, eps);
        mf_launch(norm_shift_save_kernel, dim3(n_rows), dim3(threads), 0, stream, (const float*)x, w,
                  cu_seqlens, slots, state, width, eps);
        return MF_LAUNCH_CHECK();
    }
#define MF_NORM_SHIFT(TO, SPLITS) \
    mf_launch(norm_shift_kernel<TO, SPLITS>, dim3(n_tokens), dim3(threads), 0, stream, x, partial, \
              n_partials, bias, n_tokens, w, shift, positions, token_row, cu_seqlens, slots, state, \
              (TO*)y, width, eps)
    if (out_dtype == MF_DTYPE_F32) {
        if (n_partials > 0) MF_NORM_SHIFT(float, true); else MF_NORM_SHIFT(float, false);
    } else if (out_dtype == MF_DTYPE_BF16) {
        if (n_partials > 0) MF_NORM_SHIFT(__nv_bfloat16, true); else MF_NORM_SHIFT(__nv_bfloat16, false);
    } else {
        return MF_ERR_UNSUPPORTED;
    }
#undef MF_NORM_SHIFT
    if (multi)
        mf_launch(norm_shift_save_kernel, dim3(n_rows), dim3(threads), 0, stream, (const float*)x, w,
                  cu_seqlens, slots, state, width, eps);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// xIELU, element by element in float32, with two learned numbers a = (a0, a1):
//     z > 0:   softplus(a0) z^2 + z/2
//     z <= 0:  (1/2 + softplus(a1)) (exp(z) - 1 - z) + z/2
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f32(float x) {
    return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.0f);
}
__device__ __forceinline__ float xielu_f32(float z, float cp, float cn) {
    return z > 0.0f ? fmaf(cp * z, z, 0.5f * z) : fmaf(cn, expm1f(z) - z, 0.5f * z);
}

template <typename TI, typename TO>
__global__ void xielu_kernel(const TI* __restrict__ in, TO* __restrict__ out,
                             const float* __restrict__ a, long long total) {
    pdl_launch_dependents();
    const float cp = softplus_f32(a[0]), cn = 0.5f + softplus_f32(a[1]);      // weights
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(xielu_f32(to_f32(in[i]), cp, cn));
}

extern "C" int mf_xielu(const void* in, int in_dtype, void* out, int out_dtype, const float* a,
                        long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    const long long cap = (long long)mf_sm_count() * 16;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
#define MF_XIELU(TI, TO) \
    mf_launch(xielu_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)in, (TO*)out, a, total)
    if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_F32) MF_XIELU(float, float);
    else if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_BF16) MF_XIELU(float, __nv_bfloat16);
    else if (in_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_BF16)
        MF_XIELU(__nv_bfloat16, __nv_bfloat16);
    else return MF_ERR_UNSUPPORTED;
#undef MF_XIELU
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// soft cap: x <- cap * tanh(x / cap), in place, float32 (logits)
// ------------------------------------------------------------------------------------
__global__ void tanh_cap_kernel(float* __restrict__ x, long long n, float cap, float inv_cap) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv_cap);
}

extern "C" int mf_tanh_cap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.0f)) return MF_ERR_ARGUMENT;
    const long long cap_blocks = (long long)mf_sm_count() * 16;
    const long long want = (n + 255) / 256;
    mf_launch(tanh_cap_kernel, dim3((unsigned)(want < cap_blocks ? want : cap_blocks)), dim3(256), 0,
              stream, x, n, cap, 1.0f / cap);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// h[t][:] += other[t][:] (optional) + vec[:] (optional): what a pass of a layer loop adds to
// the residual stream before its first layer
// ------------------------------------------------------------------------------------
template <typename TV>
__global__ void add_stream_kernel(float* __restrict__ h, const float* __restrict__ other,
                                  const TV* __restrict__ vec, long long total, int width) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float v = h[i];
        if (other) v += other[i];
        if (vec) v += to_f32(vec[i % width]);
        h[i] = v;
    }
}

extern "C" int mf_add_stream(float* h, const float* other, const void* vec, int vec_dtype,
                             int n_rows, int width, cudaStream_t stream) {
    const long long total = (long long)n_rows * width;
    if (total <= 0) return 0;
    const long long cap_blocks = (long long)mf_sm_count() * 16;
    const long long want = (total + 255) / 256;
    dim3 grid((unsigned)(want < cap_blocks ? want : cap_blocks));
    if (vec_dtype == MF_DTYPE_F32)
        mf_launch(add_stream_kernel<float>, grid, dim3(256), 0, stream, h, other, (const float*)vec, total, width);
    else if (vec_dtype == MF_DTYPE_BF16)
        mf_launch(add_stream_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, h, other,
                  (const __nv_bfloat16*)vec, total, width);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// PolyNorm: y = a rms(z) + b rms(z^2) + c rms(z^3) + e over a row of float32 values, powers
// element by element, rms(u) = u / sqrt(mean(u^2) + eps); coef = (a, b, c, e) on the device.
// One block a row: a pass for the three sums of squares, a pass to write.
// ------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
poly_norm_kernel(const float* __restrict__ z, const float* __restrict__ coef, TO* __restrict__ out,
                 int width, float eps) {
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];
    pdl_wait();
    const float* zr = z + (size_t)blockIdx.x * width;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v2 * v2, v2, s6);
    }
    s2 = block_sum(s2, scratch);
    s4 = block_sum(s4, scratch);
    s6 = block_sum(s6, scratch);
    const float inv_w = 1.0f / (float)width;
    const float r1 = a / sqrtf(s2 * inv_w + eps), r2 = b / sqrtf(s4 * inv_w + eps),
                r3 = c / sqrtf(s6 * inv_w + eps);
    TO* o = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        o[i] = from_f32<TO>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))));
    }
}

extern "C" int mf_poly_norm(const float* z, const float* coef, void* out, int out_dtype, int n_rows,
                            int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(poly_norm_kernel<float>, dim3(n_rows), dim3(256), 0, stream, z, coef, (float*)out,
                  width, eps);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(poly_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, z, coef,
                  (__nv_bfloat16*)out, width, eps);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Depth-weighted average of the residual streams kept so far:
//     out[r][:] = sum_{j < n_hist} w[j] hist[j][rows ? rows[r] : r][:] + w[n_hist] last[r][:]
// `hist` [n_hist][hist_rows][width]; `last` (the newest stream) has the output's rows already.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
depth_mix_kernel(const float* __restrict__ hist, long long hist_stride, int n_hist,
                 const int* __restrict__ rows, const float* __restrict__ last,
                 const float* __restrict__ w, float* __restrict__ out, int n_rows, int width) {
    pdl_prologue();
    const long long total = (long long)n_rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / width), c = (int)(i - (long long)r * width);
        const long long src = (long long)(rows ? rows[r] : r) * width + c;
        float acc = 0.f;
        for (int j = 0; j < n_hist; ++j) acc = fmaf(w[j], hist[(size_t)j * hist_stride + src], acc);
        out[i] = fmaf(w[n_hist], last[i], acc);
    }
}

extern "C" int mf_depth_mix(const float* hist, long long hist_stride, int n_hist, const int* rows,
                            const float* last, const float* w, float* out, int n_rows, int width,
                            cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    if (n_hist < 0) return MF_ERR_ARGUMENT;
    const long long total = (long long)n_rows * width;
    const long long want = (total + 255) / 256, cap = (long long)mf_sm_count() * 16;
    mf_launch(depth_mix_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, hist,
              hist_stride, n_hist, rows, last, w, out, n_rows, width);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// norm_add: h[t][:] += mult * y[t][:] / sqrt(mean(y[t]^2) + eps) * w[:], the residual add of a
// layer that norms a sublayer's OUTPUT.  y = `base` [rows][width] (may be null) plus the K splits of
// a product, `partial` [n_partials][rows][width] (may be null), added in split order, plus an
// optional bias.  A block per row; the row's y is kept in shared memory between the two passes.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
norm_add_kernel(float* __restrict__ h, const float* __restrict__ base, const float* __restrict__ partial,
                int n_partials, long long split_stride, const float* __restrict__ bias,
                const float* __restrict__ w, int width, float eps, float mult,
                __nv_bfloat16* __restrict__ x_out) {
    pdl_prologue();
    __shared__ float scratch[33];
    extern __shared__ float na_row[];
    const size_t at = (size_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = base ? base[at + i] : 0.0f;
        const float* p = partial + at + i;
        int s = 0;
        for (; s + 4 <= n_partials; s += 4) {          // four loads in flight; added in split order
            const float p0 = p[(size_t)s * split_stride], p1 = p[(size_t)(s + 1) * split_stride];
            const float p2 = p[(size_t)(s + 2) * split_stride], p3 = p[(size_t)(s + 3) * split_stride];
            v = (((v + p0) + p1) + p2) + p3;
        }
        for (; s < n_partials; ++s) v += p[(size_t)s * split_stride];
        if (bias) v += bias[i];
        na_row[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float f = mult / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float y = h[at + i] + na_row[i] * f * w[i];
        h[at + i] = y;
        if (x_out) x_out[at + i] = __float2bfloat16_rn(y);
    }
}

// `x_out` (may be null): the stream after the add, rounded to bfloat16, for the product that reads
// it next.
extern "C" int mf_norm_add(float* h, const float* base, const float* partial, int n_partials,
                           const float* bias, const float* w, int n_rows, int width, float eps,
                           float mult, void* x_out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width < 1 || (size_t)width * sizeof(float) > 200 * 1024) return MF_ERR_UNSUPPORTED;
    if ((base == nullptr && n_partials <= 0) || (n_partials > 0 && partial == nullptr)) return MF_ERR_ARGUMENT;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(norm_add_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // few rows: a row's elements spread over as many threads as the block may have
    int threads = 256;
    if (n_rows < 2 * mf_sm_count()) while (threads < 1024 && threads * 2 <= width) threads *= 2;
    mf_launch(norm_add_kernel, dim3(n_rows), dim3(threads), smem, stream, h, base, partial, n_partials,
              (long long)n_rows * width, bias, w, width, eps, mult, (__nv_bfloat16*)x_out);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Activations on float32 products, written in the activation type.
//   unary_act    kind 0: the erf form of gelu, 0.5 z (1 + erf(z / sqrt 2))
//   row_gate_mul o[t][:] <- o[t][:] * sigmoid(gate[t * gate_stride]), in place: one number a row
//   gated_act    from rows [gate (ff) | up (ff)] (or, interleaved, gate, up, gate, up, ..): kind 0 silu(g) u; kind 1 gelu_tanh(g) u;
//                kind 2 the clamped form g' sigmoid(alpha g') (u' + 1), g' = min(g, limit),
//                u' = clamp(u, -limit, limit); optionally times sigmoid of one number per row
//                (row_gate[t * row_gate_stride])
//   gate_mul     o[t][c] <- o[t][c] * sigmoid(gate[t * gate_width + gate_off + c]) * mul, in place
//   table_gate   out[t][d] = gelu_tanh(a[t][d]) * table[token(t)][off + d]: a per-token input
//                looked up by token id (token(t) = ids[rows[t]] when the step kept only some rows)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float act_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TO>
__global__ void unary_act_kernel(const float* __restrict__ z, TO* __restrict__ out, long long n, int kind) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = z[i];
        out[i] = from_f32<TO>(0.5f * v * (1.0f + erff(v * 0.7071067811865476f)));
    }
}

static inline dim3 mf_flat_grid(long long n) {
    const long long cap_blocks = (long long)mf_sm_count() * 16;
    const long long want = (n + 255) / 256;
    return dim3((unsigned)(want < cap_blocks ? want : cap_blocks));
}

extern "C" int mf_unary_act(const float* z, void* out, int out_dtype, long long n, int kind,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind != 0) return MF_ERR_ARGUMENT;
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(unary_act_kernel<float>, mf_flat_grid(n), dim3(256), 0, stream, z, (float*)out, n, kind);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(unary_act_kernel<__nv_bfloat16>, mf_flat_grid(n), dim3(256), 0, stream, z,
                  (__nv_bfloat16*)out, n, kind);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

template <typename TO>
__global__ void gated_act_kernel(const float* __restrict__ gu, TO* __restrict__ out, long long total, int ff,
                                 int kind, float limit, float alpha, const float* __restrict__ row_gate,
                                 long long row_gate_stride, int interleaved) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / ff;
        const int f = (int)(i - t * ff);
        float g = gu[(size_t)t * 2 * ff + (interleaved ? 2 * f : f)];
        float u = gu[(size_t)t * 2 * ff + (interleaved ? 2 * f + 1 : ff + f)];
        float v;
        if (kind == 0) v = g / (1.0f + expf(-g)) * u;
        else if (kind == 1) v = act_gelu_tanh(g) * u;
        else {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            v = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
        }
        if (row_gate) v *= 1.0f / (1.0f + expf(-row_gate[(size_t)t * row_gate_stride]));
        out[i] = from_f32<TO>(v);
    }
}

extern "C" int mf_gated_act(const float* gu, void* out, int out_dtype, int n_rows, int ff, int kind,
                            float limit, float alpha, const float* row_gate, long long row_gate_stride,
                            int interleaved, cudaStream_t stream) {
    const long long total = (long long)n_rows * ff;
    if (total <= 0) return 0;
    if (kind < 0 || kind > 2) return MF_ERR_ARGUMENT;
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(gated_act_kernel<float>, mf_flat_grid(total), dim3(256), 0, stream, gu, (float*)out,
                  total, ff, kind, limit, alpha, row_gate, row_gate_stride, interleaved);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(gated_act_kernel<__nv_bfloat16>, mf_flat_grid(total), dim3(256), 0, stream, gu,
                  (__nv_bfloat16*)out, total, ff, kind, limit, alpha, row_gate, row_gate_stride, interleaved);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ o, const float* __restrict__ gate, long long gate_width,
                                int gate_off, long long total, int width, float mul) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / width;
        const int c = (int)(i - t * width);
        const float z = gate[(size_t)t * gate_width + gate_off + c];
        o[i] = from_f32<T>(to_f32(o[i]) * (mul / (1.0f + expf(-z))));
    }
}

extern "C" int mf_gate_mul(void* o, int dtype, const float* gate, long long gate_width, int gate_off,
                           int n_rows, int width, float mul, cudaStream_t stream) {
    const long long total = (long long)n_rows * width;
    if (total <= 0) return 0;
    if (dtype == MF_DTYPE_F32)
        mf_launch(gate_mul_kernel<float>, mf_flat_grid(total), dim3(256), 0, stream, (float*)o, gate,
                  gate_width, gate_off, total, width, mul);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(gate_mul_kernel<__nv_bfloat16>, mf_flat_grid(total), dim3(256), 0, stream,
                  (__nv_bfloat16*)o, gate, gate_width, gate_off, total, width, mul);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

template <typename T>
__global__ void row_gate_mul_kernel(T* __restrict__ o, const float* __restrict__ gate, long long gate_stride,
                                    long long total, int width) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const float z = gate[(size_t)(i / width) * gate_stride];
        o[i] = from_f32<T>(to_f32(o[i]) / (1.0f + expf(-z)));
    }
}

extern "C" int mf_row_gate_mul(void* o, int dtype, const float* gate, long long gate_stride, int n_rows,
                               int width, cudaStream_t stream) {
    const long long total = (long long)n_rows * width;
    if (total <= 0) return 0;
    if (dtype == MF_DTYPE_F32)
        mf_launch(row_gate_mul_kernel<float>, mf_flat_grid(total), dim3(256), 0, stream, (float*)o, gate,
                  gate_stride, total, width);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(row_gate_mul_kernel<__nv_bfloat16>, mf_flat_grid(total), dim3(256), 0, stream,
                  (__nv_bfloat16*)o, gate, gate_stride, total, width);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

template <typename TT, typename TO>
__global__ void table_gate_kernel(const float* __restrict__ a, const TT* __restrict__ table, long long table_width,
                                  int off, const int* __restrict__ ids, const int* __restrict__ rows,
                                  TO* __restrict__ out, long long total, int dim, int vocab,
                                  unsigned* __restrict__ status) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / dim;
        const int d = (int)(i - t * dim);
        int id = ids[rows ? rows[t] : t];
        if (id < 0 || id >= vocab) { atomicOr(status, MF_STATUS_BAD_TOKEN); id = 0; }
        out[i] = from_f32<TO>(act_gelu_tanh(a[i]) * to_f32(table[(size_t)id * table_width + off + d]));
    }
}

extern "C" int mf_table_gate(const float* a, const void* table, int table_dtype, long long table_width,
                             int off, const int* ids, const int* rows, void* out, int out_dtype,
                             int n_rows, int dim, int vocab, unsigned* status, cudaStream_t stream) {
    const long long total = (long long)n_rows * dim;
    if (total <= 0) return 0;
#define MF_TG(TT, TO) \
    mf_launch(table_gate_kernel<TT, TO>, mf_flat_grid(total), dim3(256), 0, stream, a, (const TT*)table, \
              table_width, off, ids, rows, (TO*)out, total, dim, vocab, status)
    if (table_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_F32) MF_TG(float, float);
    else if (table_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_BF16) MF_TG(__nv_bfloat16, __nv_bfloat16);
    else if (table_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_BF16) MF_TG(float, __nv_bfloat16);
    else if (table_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_F32) MF_TG(__nv_bfloat16, float);
    else return MF_ERR_UNSUPPORTED;
#undef MF_TG
    return MF_LAUNCH_CHECK();
}
