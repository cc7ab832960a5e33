// Kernels of a gated delta-rule mixer: a matrix-valued state per head that every token first
// decays, then corrects towards its value along its key, then reads with its query.
//
// Per head (key size D, value size Dv, state S of D x Dv, float32, zero for a new sequence),
// token by token:
//     S <- diag(g) S          g: one number a head, or one per key channel (`per_channel`)
//     u  = beta (v - S^T k)
//     S <- S + k u^T
//     o  = S^T q
// with q and k made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times D^(-1/2),
// beta = sigmoid(raw), g = exp(-exp(A_log) softplus(raw + dt_bias)).  Because the read comes after
// the write, o = (g S)^T q + (q . k) u: both products with the decayed state are taken in one pass
// and a token costs one reduction.
//
//   delta_scan        a block owns (row, head, a tile of value columns); 8 threads share a column
//                     and hold its D state elements in registers as float4 groups s, s + 8, ..
//                     (state kept per slot as [head][column][D]: a column's elements are
//                     contiguous); tokens come in chunks of 16 that the block prepares together
//                     (unit vectors, decays, beta, q . k) in shared memory
//   delta_prepare     (rows of several tokens) a warp per (token, query/key head): the unit vectors,
//                     q . k, beta and the decays of every token at once, so that the scan's
//                     blocks, which are few and run long, only stream them (two cp.async buffers)
//   head_norm_gate    each head's output divided by its root mean square (eps inside the root),
//                     times a weight shared by the heads, times silu or sigmoid of a gate
// Tokens are packed row after row (row b: tokens cu_seqlens[b] .. cu_seqlens[b + 1]); a row goes
// on from what its slot's state holds, so a step may bring any number of tokens per row.
// All arithmetic is float32.
#include "common.cuh"

#define DR_NS 8             // threads that share a value column
#define DR_TC 16            // tokens prepared together
#define DR_MAX_D 256

struct DeltaArgs {
    const float* u;          // [tokens][u_width]: q | k | v after convolution and silu
    long long u_width;
    int q_off, k_off, v_off;
    const float* beta;       // raw beta: beta[t * beta_width + beta_off + head]
    long long beta_width;
    int beta_off;
    const float* decay;      // raw decay input: [t * decay_width + decay_off + head] or, per
    long long decay_width;   //   channel, [.. + decay_off + head * D + d]
    int decay_off;
    const float* dt_bias;    // [heads] or [heads * D]
    const float* a_log;      // [heads]
    float* state;            // [slots][heads][Dv][D]
    const int* cu_seqlens;
    const int* slots;
    float* out;              // [tokens][heads * Dv]
    float* prep;             // [tokens][prep_width]: what delta_prepare leaves (rows of several tokens)
    long long prep_width;
    int n_rows, heads, kv_heads, D, Dv, per_channel;
};

// Columns of a prepared row: unit q (times D^(-1/2)) and unit k per query/key head, q . k per
// query/key head, beta and the decay per head, and, per channel, the decays per head and channel
// (from a multiple of 4 on).
struct DeltaPrepCols {
    int q, k, qk, beta, g, gch, width;
    __host__ __device__ DeltaPrepCols(int heads, int kv_heads, int D, int per_channel) {
        q = 0; k = kv_heads * D; qk = 2 * kv_heads * D; beta = qk + kv_heads; g = beta + heads;
        gch = (g + heads + 3) & ~3;
        width = (gch + (per_channel ? heads * D : 0) + 3) & ~3;
    }
};

__device__ __forceinline__ float dr_softplus(float v) {
    return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v)));
}
__device__ __forceinline__ float dr_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

// One token of a column's recurrence on the D state elements this thread holds (float4 groups
// s, s + 8, ..): decay, w = beta (v - k . S), S += k w; returns w and leaves q . (decayed S) in p2.
// The two dot products run as four chains each (one per component) and are summed over the 8
// threads of the column.
template <int NV4>
__device__ __forceinline__ float dr_token(float4 (&S)[NV4], const float* krow, const float* qrow,
                                          const float* grow, float g, float beta, float v,
                                          int per_channel, int s, float& p2) {
    const float4* k4 = reinterpret_cast<const float4*>(krow);
    const float4* q4 = reinterpret_cast<const float4*>(qrow);
    const float4* g4 = reinterpret_cast<const float4*>(grow);
    float4 kk[NV4];
    float4 a1 = make_float4(0.f, 0.f, 0.f, 0.f), a2 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        kk[i] = k4[s + DR_NS * i];
        const float4 qq = q4[s + DR_NS * i];
        if (per_channel) {
            const float4 gg = g4[s + DR_NS * i];
            S[i].x *= gg.x; S[i].y *= gg.y; S[i].z *= gg.z; S[i].w *= gg.w;
        } else {
            S[i].x *= g; S[i].y *= g; S[i].z *= g; S[i].w *= g;
        }
        a1.x = fmaf(kk[i].x, S[i].x, a1.x); a1.y = fmaf(kk[i].y, S[i].y, a1.y);
        a1.z = fmaf(kk[i].z, S[i].z, a1.z); a1.w = fmaf(kk[i].w, S[i].w, a1.w);
        a2.x = fmaf(qq.x, S[i].x, a2.x); a2.y = fmaf(qq.y, S[i].y, a2.y);
        a2.z = fmaf(qq.z, S[i].z, a2.z); a2.w = fmaf(qq.w, S[i].w, a2.w);
    }
    float p1 = (a1.x + a1.y) + (a1.z + a1.w);
    p2 = (a2.x + a2.y) + (a2.z + a2.w);
#pragma unroll
    for (int o = 1; o < DR_NS; o <<= 1) {
        p1 += __shfl_xor_sync(0xffffffffu, p1, o);
        p2 += __shfl_xor_sync(0xffffffffu, p2, o);
    }
    const float uj = beta * (v - p1);
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        S[i].x = fmaf(kk[i].x, uj, S[i].x); S[i].y = fmaf(kk[i].y, uj, S[i].y);
        S[i].z = fmaf(kk[i].z, uj, S[i].z); S[i].w = fmaf(kk[i].w, uj, S[i].w);
    }
    return uj;
}

// NV4: float4 groups of a column's state a thread holds (D <= 32 * NV4)
template <int NV4>
__global__ void __launch_bounds__(256) delta_scan_kernel(DeltaArgs a) {
    pdl_launch_dependents();
    constexpr int DP = NV4 * 32;                       // padded key size
    extern __shared__ __align__(16) float dr_smem[];
    const int ct = blockDim.x / DR_NS;                  // value columns of this block
    float* qs = dr_smem;                                // [TC][DP]
    float* ks = qs + DR_TC * DP;                        // [TC][DP]
    float* gs = ks + DR_TC * DP;                        // [TC][DP] (per channel only)
    float* rest = gs + (a.per_channel ? DR_TC * DP : 0);
    float* beta_s = rest;                               // [TC]
    float* g_s = beta_s + DR_TC;                        // [TC]
    float* qk_s = g_s + DR_TC;                          // [TC]
    float* vs = qk_s + DR_TC;                           // [TC][ct]
    float* os = vs + DR_TC * ct;                        // [TC][ct]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int s = tid & (DR_NS - 1), jl = tid / DR_NS;
    const int head = blockIdx.y, b = blockIdx.z;
    const int j = blockIdx.x * ct + jl;
    const bool col_ok = j < a.Dv;
    const int D = a.D, Dv = a.Dv;
    const int kvh = head / (a.heads / a.kv_heads);
    const int t0 = a.cu_seqlens[b], t1 = a.cu_seqlens[b + 1];
    const int slot = a.slots[b];
    const float rate = expf(a.a_log[head]);
    const float q_scale = 1.0f / sqrtf((float)D);
    pdl_wait();
    if (t1 <= t0) return;

    // the column's state, elements 4 (s + 8 i) .. + 3
    float4 S[NV4];
    float* st = a.state + (((size_t)slot * a.heads + head) * Dv + (col_ok ? j : 0)) * D;
    const bool vec = (D & 3) == 0;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const int d = 4 * (s + DR_NS * i);
        S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col_ok) {
            if (vec) {
                if (d < D) S[i] = *reinterpret_cast<const float4*>(st + d);
            } else {
                if (d < D) S[i].x = st[d];
                if (d + 1 < D) S[i].y = st[d + 1];
                if (d + 2 < D) S[i].z = st[d + 2];
                if (d + 3 < D) S[i].w = st[d + 3];
            }
        }
    }

    for (int c0 = t0; c0 < t1; c0 += DR_TC) {
        const int nt = min(DR_TC, t1 - c0);
        __syncthreads();                                // the chunk before is read and written out
        // ---- prepare the chunk: a warp per token ------------------------------------------
        for (int t = warp; t < nt; t += n_warps) {
            const float* ur = a.u + (size_t)(c0 + t) * a.u_width;
            float qv[NV4], kv[NV4];
            float sq = 0.f, sk = 0.f, dot = 0.f;
#pragma unroll
            for (int i = 0; i < NV4; ++i) {
                const int d = lane + 32 * i;
                qv[i] = d < D ? ur[a.q_off + kvh * D + d] : 0.f;
                kv[i] = d < D ? ur[a.k_off + kvh * D + d] : 0.f;
                sq = fmaf(qv[i], qv[i], sq);
                sk = fmaf(kv[i], kv[i], sk);
                dot = fmaf(qv[i], kv[i], dot);
            }
            sq = warp_sum(sq); sk = warp_sum(sk); dot = warp_sum(dot);
            const float qn = q_scale / sqrtf(sq + 1e-6f), kn = 1.0f / sqrtf(sk + 1e-6f);
#pragma unroll
            for (int i = 0; i < NV4; ++i) {
                const int d = lane + 32 * i;
                qs[t * DP + d] = qv[i] * qn;
                ks[t * DP + d] = kv[i] * kn;
            }
            if (a.per_channel) {
                const float* dr = a.decay + (size_t)(c0 + t) * a.decay_width + a.decay_off + head * D;
#pragma unroll
                for (int i = 0; i < NV4; ++i) {
                    const int d = lane + 32 * i;
                    gs[t * DP + d] = d < D ? expf(-rate * dr_softplus(dr[d] + a.dt_bias[head * D + d]))
                                           : 1.0f;
                }
            }
            if (lane == 0) {
                beta_s[t] = dr_sigmoid(a.beta[(size_t)(c0 + t) * a.beta_width + a.beta_off + head]);
                qk_s[t] = dot * qn * kn;
                g_s[t] = a.per_channel ? 1.0f
                    : expf(-rate * dr_softplus(a.decay[(size_t)(c0 + t) * a.decay_width + a.decay_off + head]
                                               + a.dt_bias[head]));
            }
        }
        for (int i = tid; i < nt * ct; i += blockDim.x) {
            const int t = i / ct, c = i - t * ct;
            const int col = blockIdx.x * ct + c;
            vs[i] = col < Dv ? a.u[(size_t)(c0 + t) * a.u_width + a.v_off + head * Dv + col] : 0.f;
        }
        __syncthreads();
        // ---- the recurrence over the chunk's tokens ---------------------------------------
        for (int t = 0; t < nt; ++t) {
            float p2;
            const float uj = dr_token<NV4>(S, ks + t * DP, qs + t * DP, gs + t * DP, g_s[t],
                                           beta_s[t], vs[t * ct + jl], a.per_channel, s, p2);
            if (s == 0) os[t * ct + jl] = fmaf(qk_s[t], uj, p2);
        }
        __syncthreads();
        for (int i = tid; i < nt * ct; i += blockDim.x) {
            const int t = i / ct, c = i - t * ct;
            const int col = blockIdx.x * ct + c;
            if (col < Dv) a.out[(size_t)(c0 + t) * a.heads * Dv + head * Dv + col] = os[i];
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < NV4; ++i) {
            const int d = 4 * (s + DR_NS * i);
            if (vec) {
                if (d < D) *reinterpret_cast<float4*>(st + d) = S[i];
            } else {
                if (d < D) st[d] = S[i].x;
                if (d + 1 < D) st[d + 1] = S[i].y;
                if (d + 2 < D) st[d + 2] = S[i].z;
                if (d + 3 < D) st[d + 3] = S[i].w;
            }
        }
    }
}


// ------------------------------------------------------------------------------------------
// Rows of several tokens: everything of a token that does not depend on the state, for all
// tokens at once.  A warp per (token, query/key head).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaArgs a, int n_tokens) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * a.kv_heads) return;
    const int tok = (int)(item / a.kv_heads), kvh = (int)(item - (long long)tok * a.kv_heads);
    const int D = a.D, R = a.heads / a.kv_heads;
    const DeltaPrepCols col(a.heads, a.kv_heads, D, a.per_channel);
    const float* ur = a.u + (size_t)tok * a.u_width;
    float* pr = a.prep + (size_t)tok * a.prep_width;
    float qv[DR_MAX_D / 32], kv[DR_MAX_D / 32];
    float sq = 0.f, sk = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < DR_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < D ? ur[a.q_off + kvh * D + d] : 0.f;
        kv[i] = d < D ? ur[a.k_off + kvh * D + d] : 0.f;
        sq = fmaf(qv[i], qv[i], sq);
        sk = fmaf(kv[i], kv[i], sk);
        dot = fmaf(qv[i], kv[i], dot);
    }
    sq = warp_sum(sq); sk = warp_sum(sk); dot = warp_sum(dot);
    const float qn = (1.0f / sqrtf((float)D)) / sqrtf(sq + 1e-6f), kn = 1.0f / sqrtf(sk + 1e-6f);
#pragma unroll
    for (int i = 0; i < DR_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
            pr[col.q + kvh * D + d] = qv[i] * qn;
            pr[col.k + kvh * D + d] = kv[i] * kn;
        }
    }
    if (lane == 0) pr[col.qk + kvh] = dot * qn * kn;
    for (int r = 0; r < R; ++r) {
        const int head = kvh * R + r;
        const float rate = expf(a.a_log[head]);
        if (a.per_channel) {
            const float* dr = a.decay + (size_t)tok * a.decay_width + a.decay_off + head * D;
            for (int d = lane; d < D; d += 32)
                pr[col.gch + head * D + d] = expf(-rate * dr_softplus(dr[d] + a.dt_bias[head * D + d]));
        }
        if (lane == 0) {
            pr[col.beta + head] = dr_sigmoid(a.beta[(size_t)tok * a.beta_width + a.beta_off + head]);
            pr[col.g + head] = a.per_channel ? 1.0f
                : expf(-rate * dr_softplus(a.decay[(size_t)tok * a.decay_width + a.decay_off + head]
                                           + a.dt_bias[head]));
        }
    }
}

__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// The scan over prepared rows: as delta_scan_kernel, but a chunk's unit vectors, decays and
// values arrive by cp.async in one of two buffers while the chunk before is walked.
template <int NV4>
__global__ void __launch_bounds__(256) delta_scan_stream_kernel(DeltaArgs a) {
    pdl_launch_dependents();
    constexpr int DP = NV4 * 32;
    extern __shared__ __align__(16) float dr_smem[];
    const int ct = blockDim.x / DR_NS;
    const int n_vec = a.per_channel ? 3 : 2;
    const int buf_floats = DR_TC * DP * n_vec + 4 * DR_TC + DR_TC * ct;   // q k (g) | beta g qk pad | v
    float* os = dr_smem + 2 * buf_floats;                                 // [TC][ct]

    const int tid = threadIdx.x;
    const int s = tid & (DR_NS - 1), jl = tid / DR_NS;
    const int head = blockIdx.y, b = blockIdx.z;
    const int j = blockIdx.x * ct + jl;
    const bool col_ok = j < a.Dv;
    const int D = a.D, Dv = a.Dv;
    const int kvh = head / (a.heads / a.kv_heads);
    const DeltaPrepCols col(a.heads, a.kv_heads, D, a.per_channel);
    const bool vec = (D & 3) == 0;
    // columns beyond D stay zero in both buffers: the copies never touch them
    for (int i = tid; i < 2 * buf_floats; i += blockDim.x) dr_smem[i] = 0.f;
    pdl_wait();
    const int t0 = a.cu_seqlens[b], t1 = a.cu_seqlens[b + 1];
    const int slot = a.slots[b];
    if (t1 <= t0) return;
    __syncthreads();

    float4 S[NV4];
    float* st = a.state + (((size_t)slot * a.heads + head) * Dv + (col_ok ? j : 0)) * D;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const int d = 4 * (s + DR_NS * i);
        S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col_ok) {
            if (vec) {
                if (d < D) S[i] = *reinterpret_cast<const float4*>(st + d);
            } else {
                if (d < D) S[i].x = st[d];
                if (d + 1 < D) S[i].y = st[d + 1];
                if (d + 2 < D) S[i].z = st[d + 2];
                if (d + 3 < D) S[i].w = st[d + 3];
            }
        }
    }

    auto issue = [&](int c0, int buf) {
        const int nt = min(DR_TC, t1 - c0);
        float* base = dr_smem + buf * buf_floats;
        float* sc = base + DR_TC * DP * n_vec;                // beta [TC] | g [TC] | qk [TC]
        float* vs = sc + 4 * DR_TC;
        const int src_off[3] = {col.q + kvh * D, col.k + kvh * D, col.gch + head * D};
        for (int w = 0; w < n_vec; ++w) {
            float* dst = base + w * DR_TC * DP;
            if (vec) {
                const int per = D >> 2;
                for (int i = tid; i < nt * per; i += blockDim.x) {
                    const int t = i / per, c = i - t * per;
                    dr_cp16(dst + t * DP + 4 * c, a.prep + (size_t)(c0 + t) * a.prep_width + src_off[w] + 4 * c);
                }
            } else {
                for (int i = tid; i < nt * D; i += blockDim.x) {
                    const int t = i / D, d = i - t * D;
                    dr_cp4(dst + t * DP + d, a.prep + (size_t)(c0 + t) * a.prep_width + src_off[w] + d);
                }
            }
        }
        for (int i = tid; i < 3 * nt; i += blockDim.x) {
            const int w = i / nt, t = i - w * nt;
            const int c = w == 0 ? col.beta + head : w == 1 ? col.g + head : col.qk + kvh;
            dr_cp4(sc + w * DR_TC + t, a.prep + (size_t)(c0 + t) * a.prep_width + c);
        }
        for (int i = tid; i < nt * ct; i += blockDim.x) {
            const int t = i / ct, c = i - t * ct;
            const int cj = blockIdx.x * ct + c;
            if (cj < Dv) dr_cp4(vs + i, a.u + (size_t)(c0 + t) * a.u_width + a.v_off + head * Dv + cj);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    issue(t0, 0);
    int buf = 0;
    for (int c0 = t0; c0 < t1; c0 += DR_TC, buf ^= 1) {
        const int nt = min(DR_TC, t1 - c0);
        if (c0 + DR_TC < t1) {
            issue(c0 + DR_TC, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                  // the chunk is here; os of the last is out
        const float* base = dr_smem + buf * buf_floats;
        const float* qs = base;
        const float* ks = base + DR_TC * DP;
        const float* gs = base + (a.per_channel ? 2 * DR_TC * DP : 0);
        const float* sc = base + DR_TC * DP * n_vec;
        const float* vs = sc + 4 * DR_TC;
        for (int t = 0; t < nt; ++t) {
            float p2;
            const float uj = dr_token<NV4>(S, ks + t * DP, qs + t * DP, gs + t * DP, sc[DR_TC + t],
                                           sc[t], vs[t * ct + jl], a.per_channel, s, p2);
            if (s == 0) os[t * ct + jl] = fmaf(sc[2 * DR_TC + t], uj, p2);
        }
        __syncthreads();                                  // the buffer may be refilled, os is whole
        for (int i = tid; i < nt * ct; i += blockDim.x) {
            const int t = i / ct, c = i - t * ct;
            const int cj = blockIdx.x * ct + c;
            if (cj < Dv) a.out[(size_t)(c0 + t) * a.heads * Dv + head * Dv + cj] = os[i];
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < NV4; ++i) {
            const int d = 4 * (s + DR_NS * i);
            if (vec) {
                if (d < D) *reinterpret_cast<float4*>(st + d) = S[i];
            } else {
                if (d < D) st[d] = S[i].x;
                if (d + 1 < D) st[d + 1] = S[i].y;
                if (d + 2 < D) st[d + 2] = S[i].z;
                if (d + 3 < D) st[d + 3] = S[i].w;
            }
        }
    }
}

extern "C" int mf_delta_prep_width(int heads, int kv_heads, int D, int per_channel) {
    return DeltaPrepCols(heads, kv_heads, D, per_channel).width;
}

extern "C" int mf_delta_scan(const DeltaArgs* args, int max_row_tokens, int n_tokens,
                             cudaStream_t stream) {
    DeltaArgs a = *args;
    if (a.n_rows <= 0) return 0;
    if (a.D < 1 || a.D > DR_MAX_D || a.Dv < 1) return MF_ERR_UNSUPPORTED;
    if (a.kv_heads < 1 || a.heads % a.kv_heads != 0) return MF_ERR_ARGUMENT;
    const int nv4 = a.D <= 32 ? 1 : a.D <= 64 ? 2 : a.D <= 128 ? 4 : 8;
    // columns a block: as few as still fill the GPU's SMs with blocks, at least 8 (two warps)
    int ct = 32;
    while (ct > 8 && (long long)a.n_rows * a.heads * ((a.Dv + ct - 1) / ct) < 2LL * mf_sm_count())
        ct >>= 1;
    while (ct > 8 && ct / 2 >= a.Dv) ct >>= 1;
    const int dp = nv4 * 32;
    const size_t smem = sizeof(float) * ((size_t)DR_TC * dp * (a.per_channel ? 3 : 2) + 3 * DR_TC
                                         + 2 * (size_t)DR_TC * ct);
    dim3 grid((a.Dv + ct - 1) / ct, a.heads, a.n_rows), block(ct * DR_NS);
    // long rows: blocks run long, so they are placed only when the kernel before has ended
    const bool early = max_row_tokens <= 1;
    if (a.prep != nullptr) {
        if (a.prep_width != DeltaPrepCols(a.heads, a.kv_heads, a.D, a.per_channel).width)
            return MF_ERR_ARGUMENT;
        const long long items = (long long)n_tokens * a.kv_heads;
        mf_launch(delta_prepare_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, stream, a,
                  n_tokens);
        const size_t smem2 = sizeof(float) * (2 * ((size_t)DR_TC * dp * (a.per_channel ? 3 : 2)
                                                   + 4 * DR_TC + (size_t)DR_TC * ct)
                                              + (size_t)DR_TC * ct);
#define MF_DELTA_STREAM(N) \
    do { \
        static bool raised = false;      /* once, outside any capture (a shape's first step) */ \
        if (smem2 > 48 * 1024 && !raised) { \
            cudaFuncSetAttribute(delta_scan_stream_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024); \
            raised = true; \
        } \
        mf_launch_ex(false, delta_scan_stream_kernel<N>, grid, block, smem2, stream, a); \
    } while (0)
        if (nv4 == 1) MF_DELTA_STREAM(1);
        else if (nv4 == 2) MF_DELTA_STREAM(2);
        else if (nv4 == 4) MF_DELTA_STREAM(4);
        else MF_DELTA_STREAM(8);
#undef MF_DELTA_STREAM
        return MF_LAUNCH_CHECK();
    }
#define MF_DELTA(N) \
    do { \
        static bool raised = false;      /* once, outside any capture (a shape's first step) */ \
        if (smem > 48 * 1024 && !raised) { \
            cudaFuncSetAttribute(delta_scan_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); \
            raised = true; \
        } \
        mf_launch_ex(early, delta_scan_kernel<N>, grid, block, smem, stream, a); \
    } while (0)
    if (nv4 == 1) MF_DELTA(1);
    else if (nv4 == 2) MF_DELTA(2);
    else if (nv4 == 4) MF_DELTA(4);
    else MF_DELTA(8);
#undef MF_DELTA
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// out[t][h][j] = o[t][h][j] / sqrt(mean_j o[t][h][j]^2 + eps) * w[j] * act(gate[t][h][j]);
// a warp per (token, head); act 0: silu, 1: sigmoid
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                      long long gate_width, int gate_off, const float* __restrict__ w,
                      TO* __restrict__ out, long long items, int heads, int Dv, float eps, int act) {
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
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int j = lane; j < Dv; j += 32) {
        const float z = grow[j];
        const float sg = dr_sigmoid(z);
        out[(size_t)item * Dv + j] = from_f32<TO>(orow[j] * inv * w[j] * (act == 0 ? z * sg : sg));
    }
}

extern "C" int mf_head_norm_gate(const float* o, const float* gate, long long gate_width,
                                 int gate_off, const float* w, void* out, int out_dtype,
                                 int n_tokens, int heads, int Dv, float eps, int act,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (act != 0 && act != 1) return MF_ERR_ARGUMENT;
    const long long items = (long long)n_tokens * heads;
    dim3 grid((unsigned)((items + 7) / 8)), block(256);
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, gate, gate_width,
                  gate_off, w, (float*)out, items, heads, Dv, eps, act);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, o, gate, gate_width,
                  gate_off, w, (__nv_bfloat16*)out, items, heads, Dv, eps, act);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}
