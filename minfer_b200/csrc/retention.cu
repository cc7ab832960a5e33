// Retention: linear attention with a fixed decay per head and no softmax.
//
//   retention_scan    per (row, head): S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, tokens one
//                     after another from the state the row's slot holds (float32 [slots][heads][Dv][D]),
//                     which takes the row's last state.  q and k come prepared (rotated, scaled) as
//                     float32 [tokens][heads][D]; v is read from the projection's float32 rows.
//                     A block owns up to RT_TV value columns of one head of one row; NS threads (8, or
//                     32 for keys of 64 and wider) share a column and keep its D state elements in
//                     registers (d = lane + NS * i);
//                     tokens are staged through shared memory RT_TC at a time by cp.async, the next
//                     chunk travelling while this one is walked, four tokens' sums side by side.
//   unit_norm_gate    each head's output divided by its root mean square (eps inside the root, no
//                     weight), times silu or sigmoid of a gate read from the projection, times a
//                     constant, written in the activation type.
// Tokens are packed row after row (row b: tokens cu_seqlens[b] .. cu_seqlens[b + 1]); a step may
// bring any number of tokens per row.  All arithmetic is float32.
#include "common.cuh"

#define RT_NS 8             // threads that share a value column
#define RT_TV 32            // value columns per block
#define RT_TC 16            // tokens staged together
#define RT_MAX_D 256

struct RetentionArgs {
    const float* q;          // [tokens][heads][D]
    const float* k;          // [tokens][heads][D]
    const float* v;          // v[t * v_width + v_off + head * Dv + j]
    long long v_width;
    int v_off;
    const float* decay;      // [heads]
    float* state;            // [slots][heads][Dv][D]
    const int* cu_seqlens;
    const int* slots;
    float* out;              // [tokens][heads * Dv]
    int n_rows, heads, D, Dv;
};

__device__ __forceinline__ void rt_cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rt_cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

#define RT_TU 4             // tokens whose sums are formed side by side

// blockDim.x = TV * NS with TV (value columns of the block) 32, 16 or 8: fewer columns a block
// when the blocks would not fill the GPU otherwise.  `tc` tokens are staged together, in two
// buffers (the next chunk travels while this one is walked); a chunk's outputs meet in shared
// memory and are written row by row.
// NS: threads that share a value column, 8 or 32 (wide keys: a thread then holds D / 32 state
// elements and a sequence has four times the warps, which is what hides the latency of a chain
// that goes token by token).
template <int NREG, int NS>
__global__ void __launch_bounds__(256) retention_scan_kernel(RetentionArgs a, int tc) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float rt_smem[];
    const int D = a.D, Dv = a.Dv;
    const int TV = blockDim.x / NS;
    const int buf_floats = tc * (2 * D + TV);
    float* o_s = rt_smem + 2 * buf_floats;          // [tc][TV]
    const int tiles = (Dv + TV - 1) / TV;
    const int h = blockIdx.x / tiles, tile = blockIdx.x - h * tiles;
    const int b = blockIdx.y;
    const int tid = threadIdx.x, l = tid % NS, c = tid / NS;
    const int j0 = tile * TV, j = j0 + c;
    const int n_cols = min(TV, Dv - j0);
    const bool live = c < n_cols;
    const int t0 = a.cu_seqlens[b], n_b = a.cu_seqlens[b + 1] - t0;
    const int slot = a.slots[b];
    const float decay = a.decay[h];
    const bool d16 = (D & 3) == 0;
    pdl_wait();
    auto fetch = [&](int c0, int buf) {
        const int nc = min(tc, n_b - c0);
        float* q_s = rt_smem + buf * buf_floats;
        float* k_s = q_s + tc * D;
        float* v_s = k_s + tc * D;
        if (d16) {
            const int qn = D >> 2;
            for (int i = tid; i < nc * qn; i += blockDim.x) {
                const int tt = i / qn, d = (i - tt * qn) << 2;
                const size_t at = ((size_t)(t0 + c0 + tt) * a.heads + h) * D + d;
                rt_cp_async16(q_s + tt * D + d, a.q + at);
                rt_cp_async16(k_s + tt * D + d, a.k + at);
            }
        } else {
            for (int i = tid; i < nc * D; i += blockDim.x) {
                const int tt = i / D, d = i - tt * D;
                const size_t at = ((size_t)(t0 + c0 + tt) * a.heads + h) * D + d;
                rt_cp_async4(q_s + tt * D + d, a.q + at);
                rt_cp_async4(k_s + tt * D + d, a.k + at);
            }
        }
        for (int i = tid; i < nc * n_cols; i += blockDim.x) {
            const int tt = i / n_cols, cc = i - tt * n_cols;
            rt_cp_async4(v_s + tt * TV + cc,
                         a.v + (size_t)(t0 + c0 + tt) * a.v_width + a.v_off + (size_t)h * Dv + j0 + cc);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n_b > 0) fetch(0, 0);
    float* st = a.state + (((size_t)slot * a.heads + h) * Dv + (live ? j : 0)) * D;
    float S[NREG];
#pragma unroll
    for (int i = 0; i < NREG; ++i) {
        const int d = l + NS * i;
        S[i] = (live && d < D) ? st[d] : 0.0f;
    }
    for (int c0 = 0, buf = 0; c0 < n_b; c0 += tc, buf ^= 1) {
        const int nc = min(tc, n_b - c0);
        if (c0 + tc < n_b) {
            fetch(c0 + tc, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                 // the chunk has arrived; the last chunk's outputs are written
        const float* q_s = rt_smem + buf * buf_floats;
        const float* k_s = q_s + tc * D;
        const float* v_s = k_s + tc * D;
        int tt = 0;
        for (; tt + RT_TU <= nc; tt += RT_TU) {
            float vj[RT_TU], acc[RT_TU];
#pragma unroll
            for (int u = 0; u < RT_TU; ++u) { vj[u] = live ? v_s[(tt + u) * TV + c] : 0.0f; acc[u] = 0.0f; }
#pragma unroll
            for (int i = 0; i < NREG; ++i) {
                const int d = l + NS * i;
                if (d < D) {
#pragma unroll
                    for (int u = 0; u < RT_TU; ++u) {
                        S[i] = fmaf(decay, S[i], k_s[(tt + u) * D + d] * vj[u]);
                        acc[u] = fmaf(S[i], q_s[(tt + u) * D + d], acc[u]);
                    }
                }
            }
#pragma unroll
            for (int o = NS / 2; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < RT_TU; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
            }
            if (l == 0) {
#pragma unroll
                for (int u = 0; u < RT_TU; ++u) o_s[(tt + u) * TV + c] = acc[u];
            }
        }
        for (; tt < nc; ++tt) {
            const float vj = live ? v_s[tt * TV + c] : 0.0f;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NREG; ++i) {
                const int d = l + NS * i;
                if (d < D) {
                    S[i] = fmaf(decay, S[i], k_s[tt * D + d] * vj);
                    acc = fmaf(S[i], q_s[tt * D + d], acc);
                }
            }
#pragma unroll
            for (int o = NS / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (l == 0) o_s[tt * TV + c] = acc;
        }
        __syncthreads();                 // the chunk's outputs are complete; its buffer may be refilled
        for (int i = tid; i < nc * n_cols; i += blockDim.x) {
            const int t2 = i / n_cols, cc = i - t2 * n_cols;
            a.out[(size_t)(t0 + c0 + t2) * a.heads * Dv + (size_t)h * Dv + j0 + cc] = o_s[t2 * TV + cc];
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NREG; ++i) {
            const int d = l + NS * i;
            if (d < D) st[d] = S[i];
        }
    }
}

extern "C" int mf_retention_scan(const RetentionArgs* args, cudaStream_t stream) {
    const RetentionArgs a = *args;
    if (a.n_rows <= 0) return 0;
    if (a.D < 1 || a.D > RT_MAX_D || a.Dv < 1 || a.heads < 1) return MF_ERR_UNSUPPORTED;
    if (a.n_rows > 65535) return MF_ERR_UNSUPPORTED;
    // wide keys: 32 threads a column, 8 columns a block; else 8 threads a column and fewer columns a
    // block while the blocks do not fill the GPU
    const int ns = a.D >= 64 ? 32 : RT_NS;
    int tv = ns == 32 ? 8 : RT_TV;
    while (ns == RT_NS && tv > 8 &&
           (long long)a.heads * ((a.Dv + tv - 1) / tv) * a.n_rows < 2LL * mf_sm_count()) tv >>= 1;
    while (tv > 8 && tv / 2 >= a.Dv) tv >>= 1;
    const int tiles = (a.Dv + tv - 1) / tv;
    dim3 grid(a.heads * tiles, a.n_rows), block(tv * ns);
    const int tc = a.D > 128 ? 8 : RT_TC;
    const size_t smem = (size_t)(2 * tc * (2 * a.D + tv) + tc * tv) * sizeof(float);
    const int nreg = (a.D + ns - 1) / ns;
#define MF_RT(N, S) mf_launch(retention_scan_kernel<N, S>, grid, block, smem, stream, a, tc)
    if (ns == 32) {
        if (nreg <= 2) MF_RT(2, 32);
        else if (nreg <= 4) MF_RT(4, 32);
        else MF_RT(8, 32);
    } else {
        if (nreg <= 2) MF_RT(2, RT_NS);
        else if (nreg <= 4) MF_RT(4, RT_NS);
        else MF_RT(8, RT_NS);
    }
#undef MF_RT
    return MF_LAUNCH_CHECK();
}

template <typename TO>
__global__ void __launch_bounds__(256)
unit_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long gate_width,
                      int gate_off, TO* __restrict__ out, long long items, int heads, int Dv, float eps,
                      int act, float mul) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const long long t = item / heads;
    const int h = (int)(item - t * heads);
    const float* orow = o + (size_t)item * Dv;
    const float* grow = gate + (size_t)t * gate_width + gate_off + (size_t)h * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) ss = fmaf(orow[j], orow[j], ss);
    ss = warp_sum(ss);
    const float inv = mul / sqrtf(ss / (float)Dv + eps);
    for (int j = lane; j < Dv; j += 32) {
        const float z = grow[j];
        const float sg = 1.0f / (1.0f + expf(-z));
        out[(size_t)item * Dv + j] = from_f32<TO>(orow[j] * inv * (act == 0 ? z * sg : sg));
    }
}

// act 0: silu, 1: sigmoid
extern "C" int mf_unit_norm_gate(const float* o, const float* gate, long long gate_width, int gate_off,
                                 void* out, int out_dtype, int n_tokens, int heads, int Dv, float eps,
                                 int act, float mul, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (act != 0 && act != 1) return MF_ERR_ARGUMENT;
    const long long items = (long long)n_tokens * heads;
    dim3 grid((unsigned)((items + 7) / 8)), block(256);
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(unit_norm_gate_kernel<float>, grid, block, 0, stream, o, gate, gate_width, gate_off,
                  (float*)out, items, heads, Dv, eps, act, mul);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(unit_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, o, gate, gate_width,
                  gate_off, (__nv_bfloat16*)out, items, heads, Dv, eps, act, mul);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}
