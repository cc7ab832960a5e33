// Kernels of a selective state-space mixer (Mamba-2 form): short causal convolution with its
// state, the recurrence with its state, and the gated group norm behind it.
//
// The input projection's float32 output `proj` [tokens][in_width] holds, per token,
//     [ z : inner | x : inner | B : groups * N | C : groups * N | dt : heads ],   inner = heads * P.
// Tokens are packed row after row (row b: tokens cu_seqlens[b] .. cu_seqlens[b + 1]); a row goes
// on from what its slot's state holds, so a step may bring any number of tokens per row.
//
//   conv_silu         u[t][c] = silu(bias[c] + sum_j taps[c][j] * in[t - (T - 1 - j)][c]) over the
//                     channels c of x | B | C; inputs before the row's first token come from the
//                     slot's state (the last T - 1 inputs, oldest first; zeros for a new sequence)
//                     (a thread per token and channel for single tokens; for longer rows a
//                     thread walks a run of tokens with the history in registers)
//   conv_state        the state after the step (a kernel of its own unless every row brings one
//                     token: a row's first block reads what its last would write)
//   ssm_scan          per (row, head): dt = softplus(raw + dt_bias), a = exp(-exp(A_log) dt),
//                     S <- a S + dt B x^T (S is N x P, float32, kept per slot as [P][N]),
//                     y = S^T C + D x; tokens of a row one after another
//   gated_group_norm  v = y * silu(z); each of `groups` equal parts of v divided by its root mean
//                     square (eps inside the root), times a weight
// All arithmetic is float32.
#include "common.cuh"

#define RC_MAX_TAPS 8

__device__ __forceinline__ float rc_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float rc_softplus(float v) {
    return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v)));
}

// ------------------------------------------------------------------------------------------
// convolution
// ------------------------------------------------------------------------------------------
// one thread per (token, channel); `single`: every row brings one token and the thread also
// writes the state
__global__ void __launch_bounds__(256)
conv_silu_kernel(const float* __restrict__ proj, long long in_width, int x_off, int channels,
                 int taps, const float* __restrict__ w, const float* __restrict__ bias,
                 float* __restrict__ state, const int* __restrict__ token_row,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                 float* __restrict__ out, long long total, int single) {
    pdl_launch_dependents();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx / channels), c = (int)(idx - (long long)t * channels);
    float wt[RC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.0f;
    float acc = bias ? bias[c] : 0.0f;
    const int b = token_row[t];
    const int i = t - cu_seqlens[b];
    const int slot = slots[b];
    pdl_wait();
    float* st = state + ((size_t)slot * channels + c) * (taps - 1);
    float in_cur = 0.0f;
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j) {
        if (j < taps) {
            const int s = i - (taps - 1 - j);
            const float v = s >= 0 ? proj[(size_t)(t - (i - s)) * in_width + x_off + c]
                                   : st[taps - 1 + s];
            acc = fmaf(wt[j], v, acc);
            if (j == taps - 1) in_cur = v;
        }
    }
    out[idx] = rc_silu(acc);
    if (single && taps > 1) {
        // this thread alone owns the (slot, channel): shift and append
        float old[RC_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS; ++j) old[j] = j < taps - 1 ? st[j] : 0.0f;
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS; ++j)
            if (j < taps - 1) st[j] = j + 1 < taps - 1 ? old[j + 1] : in_cur;
    }
}

// Steps that bring more than one token a row: a thread owns a channel over a run of RC_CONV_TB
// packed tokens and keeps the last taps - 1 inputs in registers, so every input is read once;
// at the run's first token and at every first token of a row the history is fetched again (from
// the row's earlier tokens or from the slot's state).
#define RC_CONV_TB 16
__global__ void __launch_bounds__(256)
conv_silu_run_kernel(const float* __restrict__ proj, long long in_width, int x_off, int channels,
                     int taps, const float* __restrict__ w, const float* __restrict__ bias,
                     const float* __restrict__ state, const int* __restrict__ token_row,
                     const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                     float* __restrict__ out, int n_tokens) {
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int t_lo = blockIdx.y * RC_CONV_TB, t_hi = min(n_tokens, t_lo + RC_CONV_TB);
    float wt[RC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.0f;
    const float bv = bias ? bias[c] : 0.0f;
    pdl_wait();
    float hist[RC_MAX_TAPS];                     // hist[j]: the input taps - 1 - j tokens back
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j) hist[j] = 0.0f;
    for (int t = t_lo; t < t_hi; ++t) {
        const int b = token_row[t];
        const int i = t - cu_seqlens[b];
        if (t == t_lo || i == 0) {
            const float* st = state + ((size_t)slots[b] * channels + c) * (taps - 1);
#pragma unroll
            for (int j = 0; j < RC_MAX_TAPS; ++j) {
                if (j < taps - 1) {
                    const int s = i - (taps - 1 - j);
                    hist[j] = s >= 0 ? proj[(size_t)(t - (i - s)) * in_width + x_off + c]
                                     : st[taps - 1 + s];
                }
            }
        }
        const float v = proj[(size_t)t * in_width + x_off + c];
        float acc = bv;
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS; ++j)
            if (j < taps - 1) acc = fmaf(wt[j], hist[j], acc);
        acc = fmaf(wt[taps - 1], v, acc);
        out[(size_t)t * channels + c] = rc_silu(acc);
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS - 1; ++j)
            if (j < taps - 1) hist[j] = j + 1 < taps - 1 ? hist[j + 1] : v;
    }
}

// one thread per (row, channel): the state after the row's tokens
__global__ void __launch_bounds__(256)
conv_state_kernel(const float* __restrict__ proj, long long in_width, int x_off, int channels,
                  int taps, float* __restrict__ state, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ slots, long long total) {
    pdl_launch_dependents();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int b = (int)(idx / channels), c = (int)(idx - (long long)b * channels);
    const int t0 = cu_seqlens[b], n_b = cu_seqlens[b + 1] - t0;
    const int slot = slots[b];
    pdl_wait();
    float* st = state + ((size_t)slot * channels + c) * (taps - 1);
    float fresh[RC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j) {
        fresh[j] = 0.0f;
        if (j < taps - 1) {
            const int s = n_b - (taps - 1) + j;            // place in the row of the j-th kept input
            fresh[j] = s >= 0 ? proj[(size_t)(t0 + s) * in_width + x_off + c] : st[j + n_b];
        }
    }
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j)
        if (j < taps - 1) st[j] = fresh[j];
}

extern "C" int mf_conv_silu(const float* proj, long long in_width, int x_off, int channels, int taps,
                            const float* w, const float* bias, float* state, const int* token_row,
                            const int* cu_seqlens, const int* slots, float* out, int n_tokens,
                            int n_rows, int single, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (taps < 1 || taps > RC_MAX_TAPS || channels < 1) return MF_ERR_UNSUPPORTED;
    const long long total = (long long)n_tokens * channels;
    if (single || n_tokens < RC_CONV_TB)
        mf_launch(conv_silu_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, proj,
                  in_width, x_off, channels, taps, w, bias, state, token_row, cu_seqlens, slots, out,
                  total, single);
    else
        mf_launch(conv_silu_run_kernel, dim3((channels + 255) / 256, (n_tokens + RC_CONV_TB - 1) / RC_CONV_TB),
                  dim3(256), 0, stream, proj, in_width, x_off, channels, taps, w, bias, (const float*)state,
                  token_row, cu_seqlens, slots, out, n_tokens);
    if (!single && taps > 1) {
        const long long per_row = (long long)n_rows * channels;
        mf_launch(conv_state_kernel, dim3((unsigned)((per_row + 255) / 256)), dim3(256), 0, stream,
                  proj, in_width, x_off, channels, taps, state, cu_seqlens, slots, per_row);
    }
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// the recurrence
// ------------------------------------------------------------------------------------------
// A block owns one head of one row and up to RC_PB of its P columns.  NS = 8 or 16 threads share a
// column p: thread (p, s) keeps NREG elements of the column's state in registers, and the NS
// partial sums of y meet by shuffles.  Which elements: with VEC (N a multiple of 4) the float4
// groups s, s + NS, s + 2 NS, .. (n = 4 (s + NS j) + e), else the single elements s, s + NS, ..
// (n = s + NS r): either way the threads of a column read consecutive words of B and C in
// shared memory (no bank conflicts; the other columns' threads read the same words) and
// consecutive words of the state in memory.  Tokens come in chunks of RC_TC through two buffers in
// shared memory filled by cp.async: the next chunk travels while this one is walked.
#define RC_NS 8
#define RC_PB 32
#define RC_TC 32

struct ScanArgs {
    const float* u;           // [tokens][channels] conv output: x | B | C
    const float* proj;        // [tokens][in_width]: dt at column dt_off + head
    long long in_width;
    int dt_off, channels;
    const float* dt_bias;     // [heads]
    const float* a_log;       // [heads]
    const float* d_skip;      // [heads]
    float* state;             // [slots][heads][P][N]
    const int* cu_seqlens;
    const int* slots;
    float* y;                 // [tokens][heads * P]
    int heads, P, N, groups;
};

__device__ __forceinline__ void rc_cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rc_cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

#define RC_TU 4

// TU consecutive tokens of a chunk, from token `tt` on: S <- da S + dt x B, y = S . C + D x for
// each in turn (S carries over), the TU sums reduced over a column's NS threads together.
template <int NREG, bool VEC, int TU, int NS>
__device__ __forceinline__ void rc_walk(float (&S)[NREG], const float* xs, const float* Bs, const float* Cs,
                                        const float* dts, const float* das, int tt, int N, int s, int pl,
                                        bool p_ok, float dsk, float* y_col, int inner) {
    float xv[TU], da[TU], dtx[TU], acc[TU];
#pragma unroll
    for (int u = 0; u < TU; ++u) {
        xv[u] = p_ok ? xs[(tt + u) * RC_PB + pl] : 0.0f;
        da[u] = das[tt + u];
        dtx[u] = dts[tt + u] * xv[u];
        acc[u] = 0.0f;
    }
    if (VEC) {
#pragma unroll
        for (int j = 0; j < NREG / 4; ++j) {
            const int n = 4 * (s + NS * j);
            if (n < N) {
#pragma unroll
                for (int u = 0; u < TU; ++u) {
                    const float4 bv = *reinterpret_cast<const float4*>(Bs + (tt + u) * N + n);
                    const float4 cv = *reinterpret_cast<const float4*>(Cs + (tt + u) * N + n);
                    S[4 * j] = fmaf(da[u], S[4 * j], dtx[u] * bv.x);
                    S[4 * j + 1] = fmaf(da[u], S[4 * j + 1], dtx[u] * bv.y);
                    S[4 * j + 2] = fmaf(da[u], S[4 * j + 2], dtx[u] * bv.z);
                    S[4 * j + 3] = fmaf(da[u], S[4 * j + 3], dtx[u] * bv.w);
                    acc[u] += fmaf(S[4 * j + 3], cv.w,
                                   fmaf(S[4 * j + 2], cv.z, fmaf(S[4 * j + 1], cv.y, S[4 * j] * cv.x)));
                }
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < NREG; ++r) {
            const int n = s + NS * r;
            if (n < N) {
#pragma unroll
                for (int u = 0; u < TU; ++u) {
                    S[r] = fmaf(da[u], S[r], dtx[u] * Bs[(tt + u) * N + n]);
                    acc[u] = fmaf(S[r], Cs[(tt + u) * N + n], acc[u]);
                }
            }
        }
    }
#pragma unroll
    for (int o = 1; o < NS; o <<= 1) {
#pragma unroll
        for (int u = 0; u < TU; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
    }
    if (s == 0 && p_ok) {
#pragma unroll
        for (int u = 0; u < TU; ++u) y_col[(size_t)(tt + u) * inner] = fmaf(dsk, xv[u], acc[u]);
    }
}

template <int NREG, bool VEC, int NS>
__global__ void __launch_bounds__(RC_PB * NS) ssm_scan_kernel(ScanArgs a) {
    // (the kernel behind this one is let in only after the walk, further down: a block here runs
    // for as long as its row is, and blocks of the next kernel that wait beside it on the same SM
    // slowed it down: a prompt of 2,048 tokens through six layer runs 3.54 ms against 2.89 ms
    // without early launches)
    extern __shared__ __align__(16) float rc_smem[];
    const int b = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * RC_PB;
    const int tid = threadIdx.x, s = tid & (NS - 1), pl = tid / NS;
    const int p = p0 + pl;
    const int n_p = min(RC_PB, a.P - p0);
    const bool p_ok = pl < n_p;
    const int N = a.N, P = a.P;
    // two buffers of a chunk's x, B and C (the next chunk travels while this one is walked),
    // then the chunks' step sizes and decays
    const int buf_floats = RC_TC * (RC_PB + 2 * N);
    float* dts = rc_smem + 2 * buf_floats;        // [2][TC]
    float* das = dts + 2 * RC_TC;                 // [2][TC]
    const int g = h / (a.heads / a.groups);
    const float bias = a.dt_bias[h];
    const float rate = expf(a.a_log[h]);
    const float dsk = a.d_skip[h];
    const int t0 = a.cu_seqlens[b], n_b = a.cu_seqlens[b + 1] - t0;
    const int slot = a.slots[b];
    const int inner = a.heads * P;
    // element r of this thread's registers is state element n_of(r) of its column
    auto n_of = [&](int r) { return VEC ? 4 * (s + NS * (r >> 2)) + (r & 3) : s + NS * r; };
    // x may be copied 16 bytes at a time when its rows and this block's columns start on
    // 16-byte boundaries
    const bool x16 = VEC && (a.channels & 3) == 0 && ((h * P + p0) & 3) == 0 && (n_p & 3) == 0;
    pdl_wait();
    auto fetch = [&](int c0, int buf) {
        const int nc = min(RC_TC, n_b - c0);
        float* xs = rc_smem + buf * buf_floats;
        float* Bs = xs + RC_TC * RC_PB;
        float* Cs = Bs + RC_TC * N;
        const float* base = a.u + (size_t)(t0 + c0) * a.channels;
        if (x16) {
            const int q = n_p >> 2;
            for (int i = tid; i < nc * q; i += blockDim.x) {
                const int tt = i / q, pp = (i - tt * q) << 2;
                rc_cp_async16(xs + tt * RC_PB + pp, base + (size_t)tt * a.channels + h * P + p0 + pp);
            }
        } else {
            for (int i = tid; i < nc * n_p; i += blockDim.x) {
                const int tt = i / n_p, pp = i - tt * n_p;
                rc_cp_async4(xs + tt * RC_PB + pp, base + (size_t)tt * a.channels + h * P + p0 + pp);
            }
        }
        if (VEC && (a.channels & 3) == 0 && ((inner + g * N) & 3) == 0) {
            const int q = N >> 2;
            for (int i = tid; i < nc * q; i += blockDim.x) {
                const int tt = i / q, n = (i - tt * q) << 2;
                const float* row = base + (size_t)tt * a.channels + inner + g * N + n;
                rc_cp_async16(Bs + tt * N + n, row);
                rc_cp_async16(Cs + tt * N + n, row + (size_t)a.groups * N);
            }
        } else {
            for (int i = tid; i < nc * N; i += blockDim.x) {
                const int tt = i / N, n = i - tt * N;
                const float* row = base + (size_t)tt * a.channels + inner + g * N + n;
                rc_cp_async4(Bs + tt * N + n, row);
                rc_cp_async4(Cs + tt * N + n, row + (size_t)a.groups * N);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (tid < nc) {
            const float dt = rc_softplus(a.proj[(size_t)(t0 + c0 + tid) * a.in_width + a.dt_off + h] + bias);
            dts[buf * RC_TC + tid] = dt;
            das[buf * RC_TC + tid] = expf(-rate * dt);
        }
    };
    if (n_b > 0) fetch(0, 0);
    float* st = a.state + (((size_t)slot * a.heads + h) * P + (p_ok ? p : p0)) * N;
    float S[NREG];
    if (VEC) {
#pragma unroll
        for (int j = 0; j < NREG / 4; ++j) {
            const int n = 4 * (s + NS * j);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p_ok && n < N) v = *reinterpret_cast<const float4*>(st + n);
            S[4 * j] = v.x; S[4 * j + 1] = v.y; S[4 * j + 2] = v.z; S[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < NREG; ++r) S[r] = (p_ok && n_of(r) < N) ? st[n_of(r)] : 0.0f;
    }
    int buf = 0;
    for (int c0 = 0; c0 < n_b; c0 += RC_TC, buf ^= 1) {
        const int nc = min(RC_TC, n_b - c0);
        if (c0 + RC_TC < n_b) {
            fetch(c0 + RC_TC, buf ^ 1);           // (that buffer's walk ended at the barrier below)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* xs = rc_smem + buf * buf_floats;
        const float* Bs = xs + RC_TC * RC_PB;
        const float* Cs = Bs + RC_TC * N;
        // RC_TU tokens an iteration: a token's chain (products, the column's threads' sums by
        // shuffles, the store) is long and the next token only waits for S, so the chains of
        // RC_TU tokens are issued side by side; the tokens left over go one by one
        int tt = 0;
        for (; tt + RC_TU <= nc; tt += RC_TU)
            rc_walk<NREG, VEC, RC_TU, NS>(S, xs, Bs, Cs, dts + buf * RC_TC, das + buf * RC_TC, tt, N, s, pl, p_ok,
                                      dsk, a.y + (size_t)(t0 + c0) * inner + h * P + p, inner);
        for (; tt < nc; ++tt)
            rc_walk<NREG, VEC, 1, NS>(S, xs, Bs, Cs, dts + buf * RC_TC, das + buf * RC_TC, tt, N, s, pl, p_ok,
                                  dsk, a.y + (size_t)(t0 + c0) * inner + h * P + p, inner);
        __syncthreads();                          // the buffer may be refilled now
    }
    pdl_launch_dependents();
    if (p_ok) {
        if (VEC) {
#pragma unroll
            for (int j = 0; j < NREG / 4; ++j) {
                const int n = 4 * (s + NS * j);
                if (n < N)
                    *reinterpret_cast<float4*>(st + n) =
                        make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
            }
        } else {
#pragma unroll
            for (int r = 0; r < NREG; ++r)
                if (n_of(r) < N) st[n_of(r)] = S[r];
        }
    }
}

extern "C" int mf_ssm_scan(const float* u, const float* proj, long long in_width, int dt_off,
                           int channels, const float* dt_bias, const float* a_log,
                           const float* d_skip, float* state, const int* cu_seqlens,
                           const int* slots, float* y, int n_tokens, int n_rows, int heads, int P,
                           int N, int groups, cudaStream_t stream) {
    if (n_rows <= 0 || n_tokens <= 0) return 0;
    if (heads < 1 || P < 1 || N < 1 || N > RC_NS * 32) return MF_ERR_UNSUPPORTED;
    if (groups < 1 || heads % groups != 0) return MF_ERR_ARGUMENT;
    ScanArgs a;
    a.u = u; a.proj = proj; a.in_width = in_width; a.dt_off = dt_off; a.channels = channels;
    a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip; a.state = state;
    a.cu_seqlens = cu_seqlens; a.slots = slots; a.y = y; a.heads = heads; a.P = P; a.N = N;
    a.groups = groups;
    const int pb = P < RC_PB ? P : RC_PB;
    // float4 groups need rows of B, C (in shared memory) and of the state on 16-byte boundaries
    const bool vec = N % 4 == 0 && ((uintptr_t)state & 15) == 0 && ((uintptr_t)u & 15) == 0;
    // threads that share a column: 8; 16 for states of 128 and more when rows are long and the
    // grid gives an SM one block at most (one prompt on few heads): the kernel then waits on its
    // chains of dependent loads, products and shuffles, and twice the warps hide more of them.
    // With more blocks an SM it is bound by issue slots, and 16 threads a column execute more
    // instructions in all.  Measured inside a model's step (width 2,048 / 4,096: 64 / 128 heads
    // of 64 columns, state 128), 8 -> 16: a prompt of 2,048 tokens 4.48 -> 4.38 ms and 8.19 ->
    // 9.13 ms, a decode step of 8 sequences 0.639 -> 0.663 ms and 1.022 -> 1.078 ms.
    // MINFER_B200_SCAN_THREADS=8|16 forces one form (for comparison).
    static int forced = -1;
    if (forced < 0) { const char* e = getenv("MINFER_B200_SCAN_THREADS"); forced = e ? atoi(e) : 0; }
    const long long n_blocks = (long long)n_rows * heads * ((P + RC_PB - 1) / RC_PB);
    int ns = (vec && N >= 128 && (long long)n_tokens >= 64LL * n_rows && n_blocks <= mf_sm_count()) ? 16 : RC_NS;
    if (vec && N >= 64 && (forced == 8 || forced == 16)) ns = forced;
    dim3 grid(n_rows, heads, (P + RC_PB - 1) / RC_PB), block(((pb * ns + 31) / 32) * 32);
    size_t smem = (size_t)(2 * RC_TC * (RC_PB + 2 * N + 2)) * sizeof(float);
    // A block runs for as long as its row is, so the blocks must lie evenly over the SMs.  Launched
    // early (programmatic dependent launch), they are placed while the kernel before still holds
    // most SMs, and several land on one SM although others will be free in a moment (a prompt of
    // 2,048 tokens through six layer runs: 3.5 ms against 2.9 ms without early launches).  So a
    // block asks for so much shared memory that no SM takes more than its even share.
    {
        const long long blocks = (long long)n_rows * heads * ((P + RC_PB - 1) / RC_PB);
        const long long share = (blocks + mf_sm_count() - 1) / mf_sm_count();       // blocks an SM, evenly
        const size_t most = 227 * 1024;                // shared memory of an SM that blocks can have
        const size_t pad = most / (size_t)(share + 1) + 1024;
        if (pad > smem && pad <= most - 1024) smem = pad;
    }
    const int nreg = vec ? 4 * ((N / 4 + ns - 1) / ns) : (N + ns - 1) / ns;
#define MF_SCAN(NR, V, S_) \
    do { \
        if (smem > 48 * 1024) \
            cudaFuncSetAttribute(ssm_scan_kernel<NR, V, S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        mf_launch(ssm_scan_kernel<NR, V, S_>, grid, block, smem, stream, a); \
    } while (0)
    if (vec && ns == 16) {
        if (nreg <= 8) MF_SCAN(8, true, 16);
        else MF_SCAN(16, true, 16);
    } else if (vec) {
        if (nreg <= 4) MF_SCAN(4, true, 8);
        else if (nreg <= 8) MF_SCAN(8, true, 8);
        else if (nreg <= 16) MF_SCAN(16, true, 8);
        else MF_SCAN(32, true, 8);
    } else {
        if (nreg <= 2) MF_SCAN(2, false, 8);
        else if (nreg <= 4) MF_SCAN(4, false, 8);
        else if (nreg <= 8) MF_SCAN(8, false, 8);
        else if (nreg <= 16) MF_SCAN(16, false, 8);
        else MF_SCAN(32, false, 8);
    }
#undef MF_SCAN
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// gate, then group norm
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ proj,
                        long long in_width, int z_off, const float* __restrict__ w,
                        TO* __restrict__ out, int inner, int groups, float eps) {
    pdl_prologue();
    __shared__ float scratch[33];
    const int t = blockIdx.x, grp = blockIdx.y;
    const int gs = inner / groups;
    const float* yr = y + (size_t)t * inner + grp * gs;
    const float* zr = proj + (size_t)t * in_width + z_off + grp * gs;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = yr[i] * rc_silu(zr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float f = 1.0f / sqrtf(ss / (float)gs + eps);
    TO* o = out + (size_t)t * inner + grp * gs;
    for (int i = threadIdx.x; i < gs; i += blockDim.x)
        o[i] = from_f32<TO>(yr[i] * rc_silu(zr[i]) * f * w[grp * gs + i]);
}

template <typename T> struct RcStore4;
template <> struct RcStore4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct RcStore4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<unsigned*>(&lo);
        v.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};

// the same with float4 accesses, one pass over memory (a thread keeps up to MAXV float4 of the
// gated row in registers, all of its loads in flight together), for parts that are multiples of
// 4 up to 4 * MAXV * blockDim
#define GN_MAXV 4
template <typename TO>
__global__ void __launch_bounds__(1024)
gated_group_norm_vec_kernel(const float* __restrict__ y, const float* __restrict__ proj,
                            long long in_width, int z_off, const float* __restrict__ w,
                            TO* __restrict__ out, int inner, int groups, float eps) {
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int t = blockIdx.x, grp = blockIdx.y;
    const int gs = inner / groups, nv = gs >> 2;
    const float4* wr = reinterpret_cast<const float4*>(w + grp * gs);
    float4 g[GN_MAXV];
#pragma unroll
    for (int j = 0; j < GN_MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) g[j] = wr[i];
    }
    pdl_wait();
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * inner + grp * gs);
    const float4* zr = reinterpret_cast<const float4*>(proj + (size_t)t * in_width + z_off + grp * gs);
    float4 v[GN_MAXV], z[GN_MAXV];
#pragma unroll
    for (int j = 0; j < GN_MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) { v[j] = yr[i]; z[j] = zr[i]; }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < GN_MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            v[j].x *= rc_silu(z[j].x); v[j].y *= rc_silu(z[j].y);
            v[j].z *= rc_silu(z[j].z); v[j].w *= rc_silu(z[j].w);
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float f = 1.0f / sqrtf(ss / (float)gs + eps);
    TO* o = out + (size_t)t * inner + grp * gs;
#pragma unroll
    for (int j = 0; j < GN_MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv)
            RcStore4<TO>::store(o + 4 * i, v[j].x * f * g[j].x, v[j].y * f * g[j].y, v[j].z * f * g[j].z,
                                v[j].w * f * g[j].w);
    }
}

extern "C" int mf_gated_group_norm(const float* y, const float* proj, long long in_width, int z_off,
                                   const float* w, void* out, int out_dtype, int n_tokens,
                                   int inner, int groups, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (groups < 1 || inner % groups != 0) return MF_ERR_ARGUMENT;
    if (out_dtype != MF_DTYPE_F32 && out_dtype != MF_DTYPE_BF16) return MF_ERR_UNSUPPORTED;
    dim3 grid(n_tokens, groups);
    const int gs = inner / groups;
    // float4 accesses want every part of every row on a 16-byte boundary
    const bool vec = gs % 4 == 0 && in_width % 4 == 0 && z_off % 4 == 0 && gs / 4 <= GN_MAXV * 1024 &&
                     (((uintptr_t)y | (uintptr_t)proj | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (vec) {
        int threads = ((gs / 4 + GN_MAXV - 1) / GN_MAXV + 31) / 32 * 32;
        // few tokens: as many threads as float4, so that a row is one round trip
        if (n_tokens * groups < 2 * mf_sm_count()) threads = (gs / 4 + 31) / 32 * 32;
        if (threads > 1024) threads = 1024;
        if (threads < 32) threads = 32;
        if (out_dtype == MF_DTYPE_F32)
            mf_launch(gated_group_norm_vec_kernel<float>, grid, dim3(threads), 0, stream, y, proj, in_width,
                      z_off, w, (float*)out, inner, groups, eps);
        else
            mf_launch(gated_group_norm_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, y, proj,
                      in_width, z_off, w, (__nv_bfloat16*)out, inner, groups, eps);
        return MF_LAUNCH_CHECK();
    }
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(gated_group_norm_kernel<float>, grid, dim3(256), 0, stream, y, proj, in_width, z_off,
                  w, (float*)out, inner, groups, eps);
    else
        mf_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, y, proj, in_width,
                  z_off, w, (__nv_bfloat16*)out, inner, groups, eps);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// selective_scan: the recurrence of the first Mamba form, a state of n_state numbers per CHANNEL
// with a decay of its own per (channel, state):
//     dt = softplus(dt_raw[t][c]);  S[c][n] <- exp(dt * A[c][n]) S[c][n] + dt u[t][c] B[t][n],
//     A = -exp(A_log);  y = sum_n S[c][n] C[t][n] + D[c] u[t][c];  out = y * silu(z[t][c]) * mul
// A block owns up to SL_CH channels of one row; SL_NS threads share a channel and keep its states
// (n = lane + SL_NS * i) and decays' rates in registers; tokens are staged SL_TC at a time by
// cp.async, the next chunk travelling while this one is walked, four tokens' sums side by side.
// The state is float32 [slots][channels][n_state] and takes the row's last state.
// ------------------------------------------------------------------------------------------
#define SL_NS 8
#define SL_CH 32
#define SL_TC 16
#define SL_MAX_N 256

struct SelectiveArgs {
    const float* u;          // [tokens][channels]
    const float* dt_raw;     // [tokens][channels]
    const float* bc;         // B at bc[t * bc_width + b_off + n], C at bc[t * bc_width + c_off + n]
    long long bc_width;
    int b_off, c_off;
    const float* z;          // z[t * z_width + z_off + c]
    long long z_width;
    int z_off;
    const float* a_log;      // [channels][n_state]
    const float* d_skip;     // [channels]
    float* state;            // [slots][channels][n_state]
    const int* cu_seqlens;
    const int* slots;
    void* out;               // [tokens][channels]
    int n_rows, channels, n_state;
    float mul;
};

__device__ __forceinline__ float sl_softplus(float x) {
    return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.0f);
}

#define SL_TU 4             // tokens whose sums are formed side by side

// blockDim.x = CH * SL_NS with CH (channels of the block) 32, 16 or 8.  `tc` tokens are staged
// together by cp.async, in two buffers; the step sizes pass through softplus in shared memory;
// a chunk's outputs meet in shared memory and are gated and written row by row.
template <typename TO, int NREG>
__global__ void __launch_bounds__(SL_CH * SL_NS) selective_scan_kernel(SelectiveArgs a, int tc) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float sl_smem[];
    const int N = a.n_state, C = a.channels;
    const int CH = blockDim.x / SL_NS;
    const int buf_floats = tc * (2 * N + 3 * CH);    // B, C, dt, u, z of a chunk
    float* o_s = sl_smem + 2 * buf_floats;           // [tc][CH]
    const int b = blockIdx.y;
    const int tid = threadIdx.x, l = tid % SL_NS, cc = tid / SL_NS;
    const int ch0 = blockIdx.x * CH, ch = ch0 + cc;
    const int n_ch = min(CH, C - ch0);
    const bool live = cc < n_ch;
    const int t0 = a.cu_seqlens[b], n_b = a.cu_seqlens[b + 1] - t0;
    const int slot = a.slots[b];
    float A[NREG], S[NREG];
#pragma unroll
    for (int i = 0; i < NREG; ++i) {
        const int n = l + SL_NS * i;
        A[i] = (live && n < N) ? -expf(a.a_log[(size_t)ch * N + n]) : 0.0f;
    }
    const float dsk = live ? a.d_skip[ch] : 0.0f;
    pdl_wait();
    auto fetch = [&](int c0, int buf) {
        const int nc = min(tc, n_b - c0);
        float* b_s = sl_smem + buf * buf_floats;
        float* c_s = b_s + tc * N;
        float* dt_s = c_s + tc * N;
        float* u_s = dt_s + tc * CH;
        float* z_s = u_s + tc * CH;
        for (int i = tid; i < nc * N; i += blockDim.x) {
            const int tt = i / N, n = i - tt * N;
            const float* row = a.bc + (size_t)(t0 + c0 + tt) * a.bc_width;
            rc_cp_async4(b_s + i, row + a.b_off + n);
            rc_cp_async4(c_s + i, row + a.c_off + n);
        }
        for (int i = tid; i < nc * n_ch; i += blockDim.x) {
            const int tt = i / n_ch, c2 = i - tt * n_ch;
            const size_t t = (size_t)(t0 + c0 + tt);
            rc_cp_async4(dt_s + tt * CH + c2, a.dt_raw + t * C + ch0 + c2);
            rc_cp_async4(u_s + tt * CH + c2, a.u + t * C + ch0 + c2);
            rc_cp_async4(z_s + tt * CH + c2, a.z + t * a.z_width + a.z_off + ch0 + c2);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n_b > 0) fetch(0, 0);
    float* st = a.state + ((size_t)slot * C + (live ? ch : 0)) * N;
#pragma unroll
    for (int i = 0; i < NREG; ++i) {
        const int n = l + SL_NS * i;
        S[i] = (live && n < N) ? st[n] : 0.0f;
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
        float* b_s = sl_smem + buf * buf_floats;
        float* c_s = b_s + tc * N;
        float* dt_s = c_s + tc * N;
        float* u_s = dt_s + tc * CH;
        float* z_s = u_s + tc * CH;
        for (int i = tid; i < nc * n_ch; i += blockDim.x) {
            const int tt = i / n_ch, c2 = i - tt * n_ch;
            dt_s[tt * CH + c2] = sl_softplus(dt_s[tt * CH + c2]);
        }
        __syncthreads();
        int tt = 0;
        for (; tt + SL_TU <= nc; tt += SL_TU) {
            float dt[SL_TU], uu[SL_TU], du[SL_TU], acc[SL_TU];
#pragma unroll
            for (int u = 0; u < SL_TU; ++u) {
                dt[u] = live ? dt_s[(tt + u) * CH + cc] : 0.0f;
                uu[u] = live ? u_s[(tt + u) * CH + cc] : 0.0f;
                du[u] = dt[u] * uu[u];
                acc[u] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < NREG; ++i) {
                const int n = l + SL_NS * i;
                if (n < N) {
#pragma unroll
                    for (int u = 0; u < SL_TU; ++u) {
                        S[i] = fmaf(expf(dt[u] * A[i]), S[i], du[u] * b_s[(tt + u) * N + n]);
                        acc[u] = fmaf(S[i], c_s[(tt + u) * N + n], acc[u]);
                    }
                }
            }
#pragma unroll
            for (int o = SL_NS / 2; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < SL_TU; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
            }
            if (l == 0) {
#pragma unroll
                for (int u = 0; u < SL_TU; ++u) o_s[(tt + u) * CH + cc] = fmaf(dsk, uu[u], acc[u]);
            }
        }
        for (; tt < nc; ++tt) {
            const float dt = live ? dt_s[tt * CH + cc] : 0.0f, uu = live ? u_s[tt * CH + cc] : 0.0f;
            const float du = dt * uu;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NREG; ++i) {
                const int n = l + SL_NS * i;
                if (n < N) {
                    S[i] = fmaf(expf(dt * A[i]), S[i], du * b_s[tt * N + n]);
                    acc = fmaf(S[i], c_s[tt * N + n], acc);
                }
            }
#pragma unroll
            for (int o = SL_NS / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (l == 0) o_s[tt * CH + cc] = fmaf(dsk, uu, acc);
        }
        __syncthreads();                 // the chunk's outputs are complete
        for (int i = tid; i < nc * n_ch; i += blockDim.x) {
            const int t2 = i / n_ch, c2 = i - t2 * n_ch;
            const float y = o_s[t2 * CH + c2], zz = z_s[t2 * CH + c2];
            ((TO*)a.out)[(size_t)(t0 + c0 + t2) * C + ch0 + c2] = from_f32<TO>(y * zz / (1.0f + expf(-zz)) * a.mul);
        }
        __syncthreads();                 // the gate's inputs lie in the buffer the next round fetches into
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NREG; ++i) {
            const int n = l + SL_NS * i;
            if (n < N) st[n] = S[i];
        }
    }
}

extern "C" int mf_selective_scan(const SelectiveArgs* args, int out_dtype, cudaStream_t stream) {
    const SelectiveArgs a = *args;
    if (a.n_rows <= 0) return 0;
    if (a.n_state < 1 || a.n_state > SL_MAX_N || a.channels < 1 || a.n_rows > 65535) return MF_ERR_UNSUPPORTED;
    // fewer channels a block while the blocks do not fill the GPU
    int chb = SL_CH;
    while (chb > 8 && (long long)((a.channels + chb - 1) / chb) * a.n_rows < 2LL * mf_sm_count()) chb >>= 1;
    while (chb > 8 && chb / 2 >= a.channels) chb >>= 1;
    dim3 grid((a.channels + chb - 1) / chb, a.n_rows), block(chb * SL_NS);
    const int tc = a.n_state <= 64 ? SL_TC : (a.n_state <= 128 ? 8 : 4);
    const size_t smem = (size_t)(2 * tc * (2 * a.n_state + 3 * chb) + tc * chb) * sizeof(float);
    const int nreg = (a.n_state + SL_NS - 1) / SL_NS;
#define MF_SL2(TO, N) mf_launch(selective_scan_kernel<TO, N>, grid, block, smem, stream, a, tc)
#define MF_SL(TO) \
    do { \
        if (nreg <= 1) MF_SL2(TO, 1); else if (nreg <= 2) MF_SL2(TO, 2); else if (nreg <= 4) MF_SL2(TO, 4); \
        else if (nreg <= 8) MF_SL2(TO, 8); else if (nreg <= 16) MF_SL2(TO, 16); else MF_SL2(TO, 32); \
    } while (0)
    if (out_dtype == MF_DTYPE_F32) MF_SL(float);
    else if (out_dtype == MF_DTYPE_BF16) MF_SL(__nv_bfloat16);
    else return MF_ERR_UNSUPPORTED;
#undef MF_SL
#undef MF_SL2
    return MF_LAUNCH_CHECK();
}
