// Routed feed-forward (a mixture of small gated experts): the router's choice and the experts'
// products for steps of few tokens.
//
//   router_logits  the router's product in float32, a warp per (token, output)
//   moe_route_scored   the router that scores with a softmax over all outputs (see there)
//   moe_route      per token: the `top` largest of its float32 router logits (ties: the lower
//                  index), weights = softmax over the chosen logits only; a warp per token
//   moe_up         hidden[t][k][f] = act(Wg_e x_t)[f] * (Wu_e x_t)[f] for token t's k-th expert e: a
//                  block per (token, choice, tile of rows), a warp per row pair, x_t in shared memory
//   moe_down       h[t][c] += sum_k w[t][k] (Wd_e hidden[t][k])[c], added into the float32 residual;
//                  one warp owns (t, c) and adds the choices in order, so the sum is reproducible
//   moe_counts, moe_offsets, moe_place, moe_gather, moe_combine   for steps of many tokens the
//                  (token, choice) pairs are grouped by expert and each expert runs as dense
//                  products over its rows: count the pairs per expert, turn the counts into
//                  offsets, give every pair its row (pairs of an expert keep their order), gather
//                  the tokens' rows, and add the experts' weighted rows back into the residual
// The act(..) of moe_up is silu (act 0) or the clamped form (act 2): g' sigmoid(alpha g') (u' + 1) with
// g' = min(g, limit), u' = clamp(u, -limit, limit).  Choices e >= n_real name experts without
// weights whose output is the token's input itself: moe_up skips them, moe_down adds w x_t.
// Expert weights are stacked: gate and up [experts][ff][width] each or, rows alternating, as one
// [experts][2 ff][width]; down [experts][width][ff].
// Dot products accumulate in float32; `hidden` is in the activation type.
#include "common.cuh"

#define MOE_MAX_TOP 16

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int* __restrict__ idx, float* __restrict__ wts,
                 int n_tokens, int experts, int top) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const float* z = logits + (size_t)t * experts;
    float chosen_v[MOE_MAX_TOP];
    int chosen_i[MOE_MAX_TOP];
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int p = 0; p < k; ++p) taken |= chosen_i[p] == e;
            const float v = z[e];
            if (!taken && (v > best || (v == best && e < best_i))) { best = v; best_i = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        chosen_v[k] = best;
        chosen_i[k] = best_i;
    }
    if (lane == 0) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += expf(chosen_v[k] - chosen_v[0]);
        for (int k = 0; k < top; ++k) {
            idx[(size_t)t * top + k] = chosen_i[k];
            wts[(size_t)t * top + k] = expf(chosen_v[k] - chosen_v[0]) / sum;
        }
    }
}

extern "C" int mf_moe_route(const float* logits, int* idx, float* wts, int n_tokens, int experts,
                            int top, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP || top > experts) return MF_ERR_UNSUPPORTED;
    mf_launch(moe_route_kernel, dim3((n_tokens + 7) / 8), dim3(256), 0, stream, logits, idx, wts,
              n_tokens, experts, top);
    return MF_LAUNCH_CHECK();
}

// The router's product: logits[t][e] = bias[e] + sum_i x[t][i] W[e][i] with W and the sums in
// float32 (x float32 or bfloat16).  A router has few outputs and a wide input: a warp owns one
// (token, output) pair, its lanes stride over the input 16 bytes at a time; the tokens of a
// block share the rows of W in L1.
template <typename TX>
__global__ void __launch_bounds__(256)
router_logits_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                     float* __restrict__ logits, long long pairs, int outputs, int width) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const long long t = pair / outputs;
    const int e = (int)(pair - t * outputs);
    const TX* xr = x + (size_t)t * width;
    const float* wr = w + (size_t)e * width;
    float s = 0.f;
    if ((width & 3) == 0) {
        for (int i = lane * 4; i < width; i += 128) {
            const float4 wv = *reinterpret_cast<const float4*>(wr + i);
            s = fmaf(to_f32(xr[i]), wv.x, s);
            s = fmaf(to_f32(xr[i + 1]), wv.y, s);
            s = fmaf(to_f32(xr[i + 2]), wv.z, s);
            s = fmaf(to_f32(xr[i + 3]), wv.w, s);
        }
    } else {
        for (int i = lane; i < width; i += 32) s = fmaf(to_f32(xr[i]), wr[i], s);
    }
    s = warp_sum(s);
    if (lane == 0) logits[pair] = s + (bias ? bias[e] : 0.f);
}

extern "C" int mf_router_logits(const void* x, int x_dtype, const float* w, const float* bias,
                                float* logits, int n_tokens, int outputs, int width,
                                cudaStream_t stream) {
    if (n_tokens <= 0 || outputs <= 0) return 0;
    if (((uintptr_t)w & 15) != 0) return MF_ERR_UNSUPPORTED;
    const long long pairs = (long long)n_tokens * outputs;
    dim3 grid((unsigned)((pairs + 7) / 8)), block(256);
    if (x_dtype == MF_DTYPE_F32)
        mf_launch(router_logits_kernel<float>, grid, block, 0, stream, (const float*)x, w, bias, logits,
                  pairs, outputs, width);
    else if (x_dtype == MF_DTYPE_BF16)
        mf_launch(router_logits_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, w,
                  bias, logits, pairs, outputs, width);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// The other way to route: scores = softmax over ALL router outputs; the `top` outputs with the
// largest score + correction (ties: the lower index) are chosen; their weights are the scores
// themselves (no correction, not renormalized).  `stride` floats separate the rows of `logits`
// (a row may carry more columns than `experts`).  A warp per token.
__global__ void __launch_bounds__(256)
moe_route_scored_kernel(const float* __restrict__ logits, long long stride,
                        const float* __restrict__ correction, int* __restrict__ idx,
                        float* __restrict__ wts, int n_tokens, int experts, int top) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const float* z = logits + (size_t)t * stride;
    float zmax = -INFINITY;
    for (int e = lane; e < experts; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) sum += expf(z[e] - zmax);
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    int chosen_i[MOE_MAX_TOP];
    float chosen_s[MOE_MAX_TOP];
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, best_s = 0.f;
        int best_i = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int p = 0; p < k; ++p) taken |= chosen_i[p] == e;
            const float s = expf(z[e] - zmax) * inv;
            const float v = s + (correction ? correction[e] : 0.f);
            if (!taken && (v > best || (v == best && e < best_i))) { best = v; best_i = e; best_s = s; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; best_s = os; }
        }
        chosen_i[k] = best_i;
        chosen_s[k] = best_s;
    }
    if (lane == 0) {
        for (int k = 0; k < top; ++k) {
            idx[(size_t)t * top + k] = chosen_i[k];
            wts[(size_t)t * top + k] = chosen_s[k];
        }
    }
}

extern "C" int mf_moe_route_scored(const float* logits, long long stride, const float* correction,
                                   int* idx, float* wts, int n_tokens, int experts, int top,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP || top > experts) return MF_ERR_UNSUPPORTED;
    mf_launch(moe_route_scored_kernel, dim3((n_tokens + 7) / 8), dim3(256), 0, stream, logits, stride,
              correction, idx, wts, n_tokens, experts, top);
    return MF_LAUNCH_CHECK();
}

__device__ __forceinline__ float moe_dot(const float* w, const float* x, int n, int lane) {
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s = fmaf(w[i], x[i], s);
    return s;
}
__device__ __forceinline__ float moe_dot(const __nv_bfloat16* w, const float* x, int n, int lane) {
    float s = 0.f;
    if ((n & 7) == 0) {
        for (int i = lane * 8; i < n; i += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(w + i);
            const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s = fmaf(__uint_as_float(u[e] << 16), x[i + 2 * e], s);
                s = fmaf(__uint_as_float(u[e] & 0xffff0000u), x[i + 2 * e + 1], s);
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) s = fmaf(__bfloat162float(w[i]), x[i], s);
    }
    return s;
}

#define MOE_ROWS 32            // rows of gate and up a block of moe_up takes

template <typename TX, typename TW>
__global__ void __launch_bounds__(256)
moe_up_kernel(const TX* __restrict__ x, const TW* __restrict__ wg, const TW* __restrict__ wu,
              long long w_row, long long w_expert, const int* __restrict__ idx,
              TX* __restrict__ hidden, int width, int ff, int top, int n_real, int act, float limit,
              float alpha) {
    pdl_launch_dependents();
    extern __shared__ float moe_x[];
    // pairs run along x, the fastest: the blocks of one tile of rows are placed together, so pairs
    // that chose the same expert find its rows in L2
    const int pair = blockIdx.x;                   // token * top + choice
    const int t = pair / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    pdl_wait();
    for (int i = threadIdx.x; i < width; i += blockDim.x) moe_x[i] = to_f32(x[(size_t)t * width + i]);
    const int e = idx[pair];
    __syncthreads();
    if (e >= n_real) return;                       // an expert without weights: it hands its input on
    const int f_end = min(ff, (int)(blockIdx.y + 1) * MOE_ROWS);
    for (int f = blockIdx.y * MOE_ROWS + warp; f < f_end; f += n_warps) {
        const size_t wrow = (size_t)e * w_expert + (size_t)f * w_row;
        const float g = warp_sum(moe_dot(wg + wrow, moe_x, width, lane));
        const float u = warp_sum(moe_dot(wu + wrow, moe_x, width, lane));
        if (lane == 0) {
            float v;
            if (act == 0) v = g / (1.0f + expf(-g)) * u;
            else {
                const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
                v = gc / (1.0f + expf(-alpha * gc)) * (uc + 1.0f);
            }
            hidden[(size_t)pair * ff + f] = from_f32<TX>(v);
        }
    }
}

#define MOE_COLS 32            // output columns a block of moe_down takes

template <typename TX, typename TW>
__global__ void __launch_bounds__(256)
moe_down_kernel(const TX* __restrict__ hidden, const TW* __restrict__ wd, const int* __restrict__ idx,
                const float* __restrict__ wts, float* __restrict__ h, int width, int ff, int top,
                int n_real, const TX* __restrict__ x) {
    pdl_launch_dependents();
    extern __shared__ float moe_hid[];             // [top][ff]
    const int t = blockIdx.x;                      // tokens along x, as the pairs above
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    pdl_wait();
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x)
        moe_hid[i] = to_f32(hidden[(size_t)t * top * ff + i]);
    __syncthreads();
    const int c_end = min(width, (int)(blockIdx.y + 1) * MOE_COLS);
    for (int c = blockIdx.y * MOE_COLS + warp; c < c_end; c += n_warps) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = idx[(size_t)t * top + k];
            const float d = e >= n_real ? to_f32(x[(size_t)t * width + c])
                : warp_sum(moe_dot(wd + ((size_t)e * width + c) * ff, moe_hid + k * ff, ff, lane));
            sum = fmaf(wts[(size_t)t * top + k], d, sum);
        }
        if (lane == 0) h[(size_t)t * width + c] += sum;
    }
}

// gate and up rows of expert e, row f, start at wg / wu + e * w_expert + f * w_row elements (two
// stacks [experts][ff][width], or one with alternating rows [experts][2 ff][width])
extern "C" int mf_moe_experts(const void* x, int x_dtype, const void* wg, const void* wu,
                              long long w_row, long long w_expert,
                              const void* wd, int w_dtype, const int* idx, const float* wts,
                              void* hidden, float* h, int n_tokens, int width, int ff, int top,
                              int n_real, int act, float limit, float alpha, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP || (act != 0 && act != 2)) return MF_ERR_UNSUPPORTED;
    const size_t smem_up = (size_t)width * sizeof(float), smem_dn = (size_t)top * ff * sizeof(float);
    if (smem_up > 48 * 1024 || smem_dn > 48 * 1024) return MF_ERR_UNSUPPORTED;
    if ((ff + MOE_ROWS - 1) / MOE_ROWS > 65535 || (width + MOE_COLS - 1) / MOE_COLS > 65535)
        return MF_ERR_UNSUPPORTED;
    dim3 grid_up(n_tokens * top, (ff + MOE_ROWS - 1) / MOE_ROWS);
    dim3 grid_dn(n_tokens, (width + MOE_COLS - 1) / MOE_COLS);
#define MF_MOE(TX, TW) \
    do { \
        mf_launch(moe_up_kernel<TX, TW>, grid_up, dim3(256), smem_up, stream, (const TX*)x, \
                  (const TW*)wg, (const TW*)wu, w_row, w_expert, idx, (TX*)hidden, width, ff, top, n_real, \
                  act, limit, alpha); \
        mf_launch(moe_down_kernel<TX, TW>, grid_dn, dim3(256), smem_dn, stream, (const TX*)hidden, \
                  (const TW*)wd, idx, wts, h, width, ff, top, n_real, (const TX*)x); \
    } while (0)
    if (x_dtype == MF_DTYPE_F32 && w_dtype == MF_DTYPE_F32) MF_MOE(float, float);
    else if (x_dtype == MF_DTYPE_BF16 && w_dtype == MF_DTYPE_BF16) MF_MOE(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == MF_DTYPE_BF16 && w_dtype == MF_DTYPE_F32) MF_MOE(__nv_bfloat16, float);
    else return MF_ERR_UNSUPPORTED;
#undef MF_MOE
    return MF_LAUNCH_CHECK();
}

// ---- many tokens: grouping by expert --------------------------------------------------------
// counts[e] = number of (token, choice) pairs that chose expert e (counts zeroed by the caller)
__global__ void moe_counts_kernel(const int* __restrict__ idx, int* __restrict__ counts, int n_pairs) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_pairs) atomicAdd(&counts[idx[i]], 1);
}

extern "C" int mf_moe_counts(const int* idx, int* counts, int n_pairs, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    mf_launch(moe_counts_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0, stream, idx, counts, n_pairs);
    return MF_LAUNCH_CHECK();
}

// offsets[e] = counts[0] + .. + counts[e - 1], offsets[experts] = all pairs; one block
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets,
                                   int experts) {
    pdl_prologue();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) {
        int sum = 0;
        for (int i = 0; i < e; ++i) sum += counts[i];
        offsets[e] = sum;
    }
}

// a block per expert walks all pairs in order: pair i of expert e gets row
// where[i] = offsets[e] + (pairs of e before i), and order[where[i]] = i
__global__ void __launch_bounds__(256)
moe_place_kernel(const int* __restrict__ idx, const int* __restrict__ offsets,
                 int* __restrict__ order, int* __restrict__ where, int n_pairs) {
    pdl_prologue();
    __shared__ int warp_total[8];
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int base = offsets[e];
    for (int i0 = 0; i0 < n_pairs; i0 += 256) {
        const int i = i0 + threadIdx.x;
        const bool mine = i < n_pairs && idx[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_total[warp] = __popc(ballot);
        __syncthreads();
        int before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            if (w < warp) before += warp_total[w];
            total += warp_total[w];
        }
        if (mine) {
            const int pos = base + before + __popc(ballot & ((1u << lane) - 1u));
            order[pos] = i;
            where[i] = pos;
        }
        base += total;
        __syncthreads();
    }
}

extern "C" int mf_moe_place(const int* idx, const int* counts, int* offsets, int* order, int* where,
                            int n_pairs, int experts, cudaStream_t stream) {
    if (n_pairs <= 0 || experts <= 0) return 0;
    mf_launch(moe_offsets_kernel, dim3(1), dim3(256), 0, stream, counts, offsets, experts);
    mf_launch(moe_place_kernel, dim3(experts), dim3(256), 0, stream, idx, (const int*)offsets, order,
              where, n_pairs);
    return MF_LAUNCH_CHECK();
}

// rows of x (any type) picked by `pairs[i] / top` into a packed tensor of the same type
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ pairs,
                                  T* __restrict__ out, int width, int top) {
    pdl_prologue();
    const T* xr = x + (size_t)(pairs[blockIdx.x] / top) * width;
    T* o = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = xr[i];
}

extern "C" int mf_moe_gather(const void* x, int dtype, const int* pairs, void* out, int n, int width,
                             int top, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == MF_DTYPE_F32)
        mf_launch(moe_gather_kernel<float>, dim3(n), dim3(256), 0, stream, (const float*)x, pairs,
                  (float*)out, width, top);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(moe_gather_kernel<__nv_bfloat16>, dim3(n), dim3(256), 0, stream,
                  (const __nv_bfloat16*)x, pairs, (__nv_bfloat16*)out, width, top);
    else return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// h[t][:] += sum over the token's choices k, in order, of wts[t][k] * y[where[t * top + k]][:],
// `where` the row of pair (t, k) in the experts' packed output; one thread owns an element
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ where,
                   const float* __restrict__ wts, float* __restrict__ h, int n_tokens, int width,
                   int top) {
    pdl_prologue();
    const long long total = (long long)n_tokens * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / width), c = (int)(i - (long long)t * width);
        float sum = 0.f;
        for (int k = 0; k < top; ++k)
            sum = fmaf(wts[(size_t)t * top + k], y[(size_t)where[(size_t)t * top + k] * width + c], sum);
        h[i] += sum;
    }
}

extern "C" int mf_moe_combine(const float* y, const int* where, const float* wts, float* h,
                              int n_tokens, int width, int top, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const long long total = (long long)n_tokens * width;
    const long long want = (total + 255) / 256, cap = (long long)mf_sm_count() * 16;
    mf_launch(moe_combine_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, y,
              where, wts, h, n_tokens, width, top);
    return MF_LAUNCH_CHECK();
}
