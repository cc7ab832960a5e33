// Retention: linear attention with a fixed decay per head and no softmax.
//
//   retention_scan    per (row, head): S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, tokens one
//                     after another from the state the row's slot holds (float32 [slots][heads][Dv][D]),
//                     which takes the row's last state.  q and k come prepared (rotated, scaled) as
//                     float32 [tokens][heads][D]; v is read from the projection's float32 rows.
//                     A block owns RT_TV value columns of one head of one row; RT_NS threads share a
//                     column and keep its D state elements in registers (d = lane + RT_NS * i);
//                     tokens are staged through shared memory RT_TC at a time.
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

template <int NREG>
__global__ void __launch_bounds__(RT_TV * RT_NS) retention_scan_kernel(RetentionArgs a) {
    pdl_launch_dependents();
    extern __shared__ float rt_smem[];
    const int D = a.D, Dv = a.Dv;
    float* q_s = rt_smem;                       // [RT_TC][D]
    float* k_s = q_s + RT_TC * D;               // [RT_TC][D]
    float* v_s = k_s + RT_TC * D;               // [RT_TC][RT_TV]
    const int tiles = (Dv + RT_TV - 1) / RT_TV;
    const int h = blockIdx.x / tiles, tile = blockIdx.x - h * tiles;
    const int b = blockIdx.y;
    const int l = threadIdx.x % RT_NS, c = threadIdx.x / RT_NS;
    const int j = tile * RT_TV + c;
    const bool live = j < Dv;
    const int t0 = a.cu_seqlens[b], t1 = a.cu_seqlens[b + 1];
    const int slot = a.slots[b];
    const float decay = a.decay[h];
    pdl_wait();
    float* st = a.state + (((size_t)slot * a.heads + h) * Dv + (live ? j : 0)) * D;
    float S[NREG];
#pragma unroll
    for (int i = 0; i < NREG; ++i) {
        const int d = l + RT_NS * i;
        S[i] = (live && d < D) ? st[d] : 0.0f;
    }
    for (int tc = t0; tc < t1; tc += RT_TC) {
        const int n_here = min(RT_TC, t1 - tc);
        __syncthreads();
        for (int i = threadIdx.x; i < n_here * D; i += blockDim.x) {
            const int tt = i / D, d = i - tt * D;
            const size_t at = ((size_t)(tc + tt) * a.heads + h) * D + d;
            q_s[tt * D + d] = a.q[at];
            k_s[tt * D + d] = a.k[at];
        }
        for (int i = threadIdx.x; i < n_here * RT_TV; i += blockDim.x) {
            const int tt = i / RT_TV, cc = i - tt * RT_TV;
            const int jj = tile * RT_TV + cc;
            v_s[i] = jj < Dv ? a.v[(size_t)(tc + tt) * a.v_width + a.v_off + (size_t)h * Dv + jj] : 0.0f;
        }
        __syncthreads();
        for (int tt = 0; tt < n_here; ++tt) {
            const float vj = v_s[tt * RT_TV + c];
            const float* qr = q_s + tt * D;
            const float* kr = k_s + tt * D;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NREG; ++i) {
                const int d = l + RT_NS * i;
                if (d < D) {
                    S[i] = fmaf(decay, S[i], kr[d] * vj);
                    acc = fmaf(S[i], qr[d], acc);
                }
            }
#pragma unroll
            for (int o = RT_NS / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (l == 0 && live) a.out[(size_t)(tc + tt) * a.heads * Dv + (size_t)h * Dv + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NREG; ++i) {
            const int d = l + RT_NS * i;
            if (d < D) st[d] = S[i];
        }
    }
}

extern "C" int mf_retention_scan(const RetentionArgs* args, cudaStream_t stream) {
    const RetentionArgs a = *args;
    if (a.n_rows <= 0) return 0;
    if (a.D < 1 || a.D > RT_MAX_D || a.Dv < 1 || a.heads < 1) return MF_ERR_UNSUPPORTED;
    const int tiles = (a.Dv + RT_TV - 1) / RT_TV;
    if (a.n_rows > 65535) return MF_ERR_UNSUPPORTED;
    dim3 grid(a.heads * tiles, a.n_rows), block(RT_TV * RT_NS);
    const size_t smem = (size_t)(2 * RT_TC * a.D + RT_TC * RT_TV) * sizeof(float);
    const int nreg = (a.D + RT_NS - 1) / RT_NS;
#define MF_RT(N) mf_launch(retention_scan_kernel<N>, grid, block, smem, stream, a)
    if (nreg <= 2) MF_RT(2);
    else if (nreg <= 4) MF_RT(4);
    else if (nreg <= 8) MF_RT(8);
    else if (nreg <= 16) MF_RT(16);
    else MF_RT(32);
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
