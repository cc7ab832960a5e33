"""Attention whose scores are changed before the softmax, with a sink, as a mixer.

    q, k, v = Wq u, Wk u, Wv u (no biases; v of its own width ``value_dim``)
    q, k divided by their root mean square per head, no weight           (``qk_norm``)
    s_ij = (q_i . k_j) * scale - r1_h ln(1 + r2_h (i - j))               (``distance_bias``)
    j visible from i iff j <= i, floor(i / chunk) == floor(j / chunk)    (``chunk`` > 0, counted
    from position 0 of the sequence), i - j < window                      (``window`` > 0)
    w_ij = exp(s_ij) / (1 + sum_j' exp(s_ij'))                           (``sink``)
    out = Wo concat_h(sum_j w_ij v_j)

Every size, constant and switch is a parameter; the tensors' names are too (behind
``prefix + tensor_prefix``).  One packed product gives q|k|v in float32; one kernel norms q and
k and writes the step's keys and values and the cache's pages; attention runs over the step's
own keys for whole prompts and over the cache otherwise; Wo adds into the residual stream.

A query never looks further back than its chunk's start (or its window), so the cache keeps a
ring of that many positions plus what a step may add, as for a windowed layer.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CacheRequest, CallBinding, Mixer, StepContext, settle_pending
from .linear import Linear


# MINFER_B200_SINK_ATTENTION_GENERIC=1: every step takes the generic kernel (for comparison)
FORCE_GENERIC = os.environ.get("MINFER_B200_SINK_ATTENTION_GENERIC", "0") == "1"
# a step that is neither whole prompts nor one token a row runs the query-tile kernel over the
# cache's pages from this many tokens on; below, every token is a row of the kernel for single
# queries
PAGED_PROMPT_MIN_TOKENS = int(os.environ.get("MINFER_B200_SINK_PAGED_PROMPT_MIN_TOKENS", "48"))


# tiles of 128 queries pay from this many tokens on (as for the other attention mixer)
PAGED_TCGEN05_MIN_TOKENS = int(os.environ.get("MINFER_B200_SINK_PAGED_TCGEN05_MIN_TOKENS", "160"))
# "tcgen05" (tensor memory, where the sizes allow) or "mma" (the mma.sync kernel) for prompts
PROMPT_KERNEL = os.environ.get("MINFER_B200_SINK_PROMPT_KERNEL", "tcgen05")


@dataclass
class ScoreSpec:
    """Sizes and score modifiers of one attention: what ``scored_attention`` runs.  ``sink``: a
    key without a value in the softmax, of score 0 or of ``sink_logit[h]`` (float32 per head);
    ``softcap`` > 0: scores pass through cap * tanh(s / cap) before the bias; ``r1``, ``r2``: the
    logarithmic distance bias per head."""

    n_heads: int
    n_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: int = 0
    chunk: int = 0
    sink: bool = False
    r1: Optional[torch.Tensor] = None
    r2: Optional[torch.Tensor] = None
    sink_logit: Optional[torch.Tensor] = None
    softcap: float = 0.0
    keep_first: int = 0       # > 0: keys at positions below it stay visible beyond the window

    def reach(self) -> int:
        """Positions a query may look back, itself included (0: no bound)."""
        if self.keep_first > 0:
            return 0
        bounds = [b for b in (self.chunk, self.window) if b > 0]
        return min(bounds) if bounds else 0


def decode_reach(spec: ScoreSpec, max_end: int) -> int:
    """The most keys a single query sees: its reach, the window plus the kept first keys (and a
    tile's worth for the two stretches' ragged ends), or the longest sequence."""
    reach = spec.reach()
    if reach > 0:
        return reach
    if spec.window > 0 and spec.keep_first > 0:
        return min(max_end, spec.window + spec.keep_first + 64)
    return max_end


def scored_attention(spec: ScoreSpec, q: torch.Tensor, k_step: Optional[torch.Tensor],
                     v_step: Optional[torch.Tensor], cache, ctx: StepContext, o: torch.Tensor) -> None:
    """o = attention of the step's queries ``q`` [tokens, heads, head_dim] (already normed,
    rotated, whatever the mixer does to them): over the step's own packed keys and values for
    whole prompts (``ctx.from_start``), over the cache's pages otherwise (it holds the step's
    keys by then; every token is a query at its own position).  Picks the kernel by precision,
    sizes and the shape of the step; every choice computes the same function."""
    nh, nk, hd, vd = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.value_dim
    act = q.dtype
    own_kv = ctx.from_start
    r1, r2 = spec.r1, spec.r2
    cap, sl = spec.softcap, spec.sink_logit
    keep = spec.keep_first if spec.window > 0 else 0
    if keep > 0 and (spec.chunk > 0 or r1 is not None or (cache is not None and cache.ring)):
        raise K.KernelError("kept first tokens go with a window on a cache that keeps every position, "
                            "without a chunk mask or a distance bias")
    tensor_cores = K.sink_attention_mma_supported(act, hd, vd) and not FORCE_GENERIC
    # prompts: the tcgen05 kernel where keys and values have one size it takes, else mma.sync
    tcgen05 = (tensor_cores and PROMPT_KERNEL != "mma" and spec.scale > 0.0
               and K.sink_attention_tc_supported(act, hd, vd))
    if own_kv and tcgen05:
        K.sink_attention_tc(q, k_step, v_step, ctx.cu_seqlens, None, None, 0, 0, o, r1, r2,
                            ctx.n_rows, ctx.max_row_tokens, nh, nk, hd, spec.window, spec.chunk,
                            spec.sink, spec.scale, ctx.status, sink_logit=sl, softcap=cap,
                            keep_first=keep)
        return
    if own_kv and tensor_cores:
        K.sink_attention_mma(q, k_step, v_step, ctx.cu_seqlens, None, None, 0, 0, o, r1, r2,
                             ctx.n_rows, ctx.max_row_tokens, nh, nk, hd, vd, spec.window,
                             spec.chunk, spec.sink, spec.scale, sink_logit=sl, softcap=cap,
                             keep_first=keep)
        return
    if own_kv:
        K.sink_attention_packed(q, k_step, v_step, ctx.token_row, ctx.positions, ctx.cu_seqlens, o,
                                r1, r2, nh, nk, hd, vd, spec.window, spec.chunk, spec.sink,
                                spec.scale, sink_logit=spec.sink_logit, softcap=spec.softcap,
                                keep_first=keep)
        return
    reach = spec.reach()
    if cache.ring and ctx.max_row_tokens > cache.ring - reach + 1:
        raise K.KernelError(
            f"a sequence brings {ctx.max_row_tokens} tokens, but a ring of {cache.ring} "
            f"positions with a reach of {reach} takes {cache.ring - reach + 1} a step "
            f"(the engine runs longer rows in portions)")
    if tcgen05 and not ctx.single_token and ctx.n_tokens >= PAGED_TCGEN05_MIN_TOKENS:
        K.sink_attention_tc(q, cache.k, cache.v, ctx.cu_seqlens, ctx.seq_end, cache.page_table,
                            cache.table_stride, cache.ring, o, r1, r2, ctx.n_rows,
                            ctx.max_row_tokens, nh, nk, hd, spec.window, spec.chunk, spec.sink,
                            spec.scale, ctx.status, sink_logit=sl, softcap=cap, keep_first=keep)
        return
    if tensor_cores and not ctx.single_token and ctx.n_tokens >= PAGED_PROMPT_MIN_TOKENS:
        # rows of several tokens: query tiles of the step's rows over the cache's pages
        K.sink_attention_mma(q, cache.k, cache.v, ctx.cu_seqlens, ctx.seq_end, cache.page_table,
                             cache.table_stride, cache.ring, o, r1, r2, ctx.n_rows,
                             ctx.max_row_tokens, nh, nk, hd, vd, spec.window, spec.chunk,
                             spec.sink, spec.scale, sink_logit=sl, softcap=cap, keep_first=keep)
        return
    if tensor_cores:
        # single queries: the heads of a key/value head are the rows of the product
        K.sink_attention_decode(q, cache.k, cache.v, ctx.token_row, ctx.positions,
                                cache.page_table, cache.table_stride, cache.ring, o, r1, r2, nh,
                                nk, hd, vd, spec.window, spec.chunk, spec.sink, spec.scale,
                                decode_reach(spec, ctx.max_end), sink_logit=sl, softcap=cap,
                                keep_first=keep)
        return
    K.sink_attention_paged(q, cache.k, cache.v, ctx.token_row, ctx.positions, cache.page_table,
                           cache.table_stride, cache.ring, o, r1, r2, nh, nk, hd, vd, spec.window,
                           spec.chunk, spec.sink, spec.scale, sink_logit=spec.sink_logit,
                           softcap=spec.softcap, keep_first=keep)


def project_out(out: Linear, o: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
    """residual += out(o), in whichever of three ways fits the step: completed here with the next
    norm's input prepared (``ctx.extras["prepare_for"]``), left as K splits for the next kernel to
    add (``Pending``), or added by the product's epilogue.  A caller whose ``residual`` is a buffer
    of its own that holds nothing yet says so with ``ctx.extras["fresh_output"]``: the product then
    stores instead of adding, and K splits left pending are marked as all there is
    (``ctx.extras["pending_only"]``), so the buffer is never read."""
    fresh = ctx.extras.pop("fresh_output", False)
    target = ctx.extras.pop("prepare_for", None)
    if target is not None and not fresh:
        # the product completes the residual and prepares the next norm's input
        settle_pending(ctx, residual)
        prepared = out.accumulate_prepared(o, residual, target)
        if prepared is not None:
            ctx.extras["prepared"] = prepared
            return
    pending = out.partial_sums(o)
    if pending is None:
        out.forward(o, torch.float32, out=residual, accumulate=not fresh)
    else:
        settle_pending(ctx, residual)          # never two at once
        ctx.extras["pending"] = pending
        if fresh:
            ctx.extras["pending_only"] = True


class SinkAttention(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        libs = ["ops", "attention_sink"]
        if dtype == torch.bfloat16:
            libs.append("gemm_tc")
            if K.sink_attention_tc_supported(dtype, self.head_dim, self.value_dim):
                libs.append("attention_prefill_tc")
        else:
            libs.append("gemm_simt")
        return libs

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, norm_eps: float, chunk: int = 0, window: int = 0,
                 sink: bool = True, qk_norm: bool = True, distance_bias: bool = True,
                 tensor_prefix: str = "mix.", init_std: float = 0.02):
        if n_kv_heads < 1 or n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} heads do not divide into {n_kv_heads} key/value heads")
        for what, d in (("key", head_dim), ("value", value_dim)):
            if not 1 <= d <= 256:
                raise ValueError(f"{what} size {d} is not supported: the kernels take 1 to 256")
        if chunk < 0 or window < 0:
            raise ValueError("chunk and window must not be negative")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim)
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.chunk = int(chunk)
        self.window = int(window)
        self.sink = bool(sink)
        self.qk_norm = bool(qk_norm)
        self.distance_bias = bool(distance_bias)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.r1: Optional[torch.Tensor] = None
        self.r2: Optional[torch.Tensor] = None

    # ---- how far back a query may look ----------------------------------------------------
    def reach(self) -> int:
        """Positions a query may look back, itself included (0: no bound)."""
        return self.scores().reach()

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nk, nv = (self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim,
                      self.n_kv_heads * self.value_dim)
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{p}q", (nq, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}k", (nk, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}v", (nv, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}o", (self.hidden_size, self.n_heads * self.value_dim), MATRIX, init)]
        if self.distance_bias:
            specs += [TensorSpec(f"{p}r1", (self.n_heads,), VECTOR, Init(0.5, 0.1)),
                      TensorSpec(f"{p}r2", (self.n_heads,), VECTOR, Init(0.5, 0.1))]
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        parts = [weights[f"{p}{n}"] for n in "qkv"]
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        self.qkv = Linear(torch.cat(parts, dim=0).contiguous())
        self.out = Linear(weights[f"{p}o"])
        if self.distance_bias:
            self.r1, self.r2 = weights[f"{p}r1"], weights[f"{p}r2"]
        # the projection of q|k|v can apply a norm's 1/rms itself (bfloat16 on tensor cores)
        self.accepts_row_scale = self.qkv.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nk = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        nv = self.n_kv_heads * self.value_dim
        out = {f"{p}q": self.qkv.weight[:nq], f"{p}k": self.qkv.weight[nq:nq + nk],
               f"{p}v": self.qkv.weight[nq + nk:nq + nk + nv], f"{p}o": self.out.weight}
        if self.distance_bias:
            out[f"{p}r1"], out[f"{p}r2"] = self.r1, self.r2
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(self.n_kv_heads, self.head_dim, self.reach(),
                            self.value_dim if self.value_dim != self.head_dim else 0)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n = x.shape[0]
        nh, nk, hd, vd = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        dev, act = x.device, ctx.act_dtype
        cache = binding.cache
        if cache is None:
            raise K.KernelError("the attention mixer was given no cache entry")
        if cache.k.dtype != act:
            raise K.KernelError("the cache and the activations must share one dtype")
        # the K splits of a small projection are added by the kernel that norms q and k
        split = self.qkv.partial_sums(x, row_scale=ctx.input_scale)
        if split is not None:
            qkv, n_partials = split.partial, split.partial.shape[0]
        else:
            qkv, n_partials = self.qkv.forward(x, torch.float32, row_scale=ctx.input_scale), 0
        q = torch.empty((n, nh, hd), dtype=act, device=dev)
        write = binding.writes_cache
        own_kv = ctx.from_start
        k_step = v_step = None
        if own_kv and write:
            k_step = torch.empty((n, nk, hd), dtype=act, device=dev)
            v_step = torch.empty((n, nk, vd), dtype=act, device=dev)
            if binding.has_readers:
                ctx.extras[("step_kv", binding.entry)] = (k_step, v_step)
        elif own_kv:
            k_step, v_step = ctx.extras[("step_kv", binding.entry)]
        K.unit_norm_kvstore(qkv, ctx.positions, ctx.token_row, ctx.seq_end, q,
                            k_step if write else None, v_step if write else None,
                            cache.k if write else None, cache.v if write else None,
                            cache.page_table if write else None, cache.table_stride, cache.ring,
                            nh, nk, hd, vd, self.norm_eps, self.qk_norm, ctx.status,
                            n_partials=n_partials)
        o = torch.empty((n, nh * vd), dtype=act, device=dev)
        scored_attention(self.scores(), q, k_step, v_step, cache, ctx, o)
        self._project_out(o, ctx, residual)

    def scores(self) -> "ScoreSpec":
        return ScoreSpec(n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                         value_dim=self.value_dim, scale=self.scale, window=self.window,
                         chunk=self.chunk, sink=self.sink, r1=self.r1, r2=self.r2)

    def _project_out(self, o: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        project_out(self.out, o, ctx, residual)
