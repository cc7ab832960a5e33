"""Grouped-query attention whose queries and keys are normed as a whole and whose scores are
soft-capped, as a mixer.

    q, k, v = Wq u + bq, Wk u + bk, Wv u + bv          (``bias``; v of its own width ``value_dim``)
    q <- q / sqrt(mean(q^2) + eps) * wq over ALL heads of q at once, k likewise    (``qk_norm``;
        with ``norm_scope`` "head": over each head by itself, one weight of the head's width)
    a rotation of the first ``rotary_dim`` dimensions of every head of q and k      (``position``)
    s_ij = (q_i . k_j) * scale;  s_ij <- softcap * tanh(s_ij / softcap)              (``softcap`` > 0)
    j visible from i iff j <= i and (i - j < window or j < keep_first)   (``window`` > 0; with
        ``keep_first`` the first tokens of a sequence stay visible, at their true positions)
    o = concat_h(softmax_j(s_ij) v_j);  o <- o * sigmoid(Wg u)                     (``gate``)
    out = Wo (o * out_scale)

Every size, constant and switch is a parameter, and so are the tensors' names (behind ``prefix +
tensor_prefix``: ``q``, ``k``, ``v``, ``o``, biases ``<name>.b``, norm weights ``q.norm``,
``k.norm``, the gate ``g``).  One packed product gives q|k|v(|g) in float32 (bias added by the product); one kernel
norms, rotates and writes the step's keys and values and the cache's pages; the attention is
``parts.sink_attention.scored_attention``; Wo adds into the residual stream.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import PartSpec
from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CacheRequest, CallBinding, Mixer, StepContext
from .linear import Linear
from .sink_attention import ScoreSpec, project_out, scored_attention


class QkNormAttention(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture
    stores_fresh_output = True     # its last product goes through ``project_out``

    def libraries(self, dtype: torch.dtype) -> List[str]:
        libs = ["ops", "mixer_prep", "attention_sink"]
        libs.append("gemm_tc" if dtype == torch.bfloat16 else "gemm_simt")
        if K.sink_attention_tc_supported(dtype, self.head_dim, self.value_dim):
            libs.append("attention_prefill_tc")
        return libs

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, norm_eps: float, softcap: float = 0.0,
                 window: int = 0, qk_norm: bool = True, bias: bool = True,
                 position: Optional[PartSpec] = None, tensor_prefix: str = "mix.",
                 init_std: float = 0.02, norm_scope: str = "all", keep_first: int = 0,
                 gate: bool = False, out_scale: float = 1.0):
        from ..registry import build_part
        if n_kv_heads < 1 or n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} heads do not divide into {n_kv_heads} key/value heads")
        for what, d in (("key", head_dim), ("value", value_dim)):
            if not 1 <= d <= 640:
                raise ValueError(f"{what} size {d} is not supported: the kernels take 1 to 640")
        if softcap < 0 or window < 0 or keep_first < 0:
            raise ValueError("softcap, window and keep_first must not be negative")
        if norm_scope not in ("all", "head"):
            raise ValueError(f"norm_scope is \"all\" or \"head\", got {norm_scope!r}")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim)
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.softcap = float(softcap)
        self.window = int(window)
        self.qk_norm = bool(qk_norm)
        self.bias = bool(bias)
        self.norm_scope = norm_scope
        self.keep_first = int(keep_first) if window > 0 else 0
        self.gate = bool(gate)
        self.out_scale = float(out_scale)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.position = build_part("position", position) if position is not None else None
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None

    def _widths(self):
        return (self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim,
                self.n_kv_heads * self.value_dim)

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nk, nv = self._widths()
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{p}q", (nq, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}k", (nk, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}v", (nv, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}o", (self.hidden_size, self.n_heads * self.value_dim), MATRIX, init)]
        if self.bias:
            specs += [TensorSpec(f"{p}q.b", (nq,), VECTOR, init),
                      TensorSpec(f"{p}k.b", (nk,), VECTOR, init),
                      TensorSpec(f"{p}v.b", (nv,), VECTOR, init)]
        if self.qk_norm:
            per_head = self.norm_scope == "head"
            specs += [TensorSpec(f"{p}q.norm", (self.head_dim if per_head else nq,), VECTOR, Init(1.0, 0.0)),
                      TensorSpec(f"{p}k.norm", (self.head_dim if per_head else nk,), VECTOR, Init(1.0, 0.0))]
        if self.gate:
            specs.append(TensorSpec(f"{p}g", (self.n_heads * self.value_dim, self.hidden_size), MATRIX, init))
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        parts = [weights[f"{p}{n}"] for n in ("qkvg" if self.gate else "qkv")]
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        b = None
        if self.bias:
            biases = [weights[f"{p}{n}.b"] for n in "qkv"]
            if self.gate:          # the gate has no bias of its own
                biases.append(torch.zeros(self.n_heads * self.value_dim, dtype=biases[0].dtype,
                                          device=biases[0].device))
            b = torch.cat(biases).contiguous()
        self.qkv = Linear(torch.cat(parts, dim=0).contiguous(), b)
        self.out = Linear(weights[f"{p}o"])
        if self.qk_norm:
            self.q_norm, self.k_norm = weights[f"{p}q.norm"], weights[f"{p}k.norm"]
        # the projection of q|k|v can apply a norm's 1/rms itself (bfloat16 on tensor cores)
        self.accepts_row_scale = self.qkv.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nk, nv = self._widths()
        out = {f"{p}o": self.out.weight}
        for name, lo, hi in (("q", 0, nq), ("k", nq, nq + nk), ("v", nq + nk, nq + nk + nv)):
            out[f"{p}{name}"] = self.qkv.weight[lo:hi]
            if self.bias:
                out[f"{p}{name}.b"] = self.qkv.bias[lo:hi]
        if self.qk_norm:
            out[f"{p}q.norm"], out[f"{p}k.norm"] = self.q_norm, self.k_norm
        if self.gate:
            out[f"{p}g"] = self.qkv.weight[nq + nk + nv:]
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def cache_request(self) -> Optional[CacheRequest]:
        # kept first tokens stay visible for ever: such a layer keeps every position, not a ring
        return CacheRequest(self.n_kv_heads, self.head_dim, 0 if self.keep_first > 0 else self.window,
                            self.value_dim if self.value_dim != self.head_dim else 0)

    def scores(self) -> ScoreSpec:
        return ScoreSpec(n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                         value_dim=self.value_dim, scale=self.scale, window=self.window,
                         softcap=self.softcap, keep_first=self.keep_first)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n = x.shape[0]
        nh, nk, hd, vd = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        nq_w, nk_w, _ = self._widths()
        dev, act = x.device, ctx.act_dtype
        cache = binding.cache
        if cache is None:
            raise K.KernelError("the attention mixer was given no cache entry")
        if cache.k.dtype != act:
            raise K.KernelError("the cache and the activations must share one dtype")
        qkv = self.qkv.forward(x, torch.float32, row_scale=ctx.input_scale)
        inv_freq, rot_dims, style, magnitude = None, 0, 0, 1.0
        if self.position is not None and getattr(self.position, "rotary_dim", 0) > 0:
            inv_freq, rot_dims, style = self.position.tables(dev)
            magnitude = self.position.magnitude()
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
        if self.norm_scope == "head":
            K.head_prepare(qkv, ctx.positions, ctx.token_row, ctx.seq_end, q,
                           k_step if write else None, v_step if write else None,
                           cache.k if write else None, cache.v if write else None,
                           cache.page_table if write else None, cache.table_stride, cache.ring,
                           q_off=0, n_heads=nh, q_width=hd, k_off=nq_w, n_kv=nk, k_width=hd,
                           v_off=nq_w + nk_w, v_width=vd, q_norm=self.q_norm, k_norm=self.k_norm,
                           eps=self.norm_eps, inv_freq=inv_freq, rot_dims=rot_dims, rot_style=style,
                           rot_magnitude=magnitude, q_mul=1.0, k_mul=1.0, status=ctx.status)
        else:
            K.qk_prepare(qkv, ctx.positions, ctx.token_row, ctx.seq_end, q,
                         k_step if write else None, v_step if write else None,
                         cache.k if write else None, cache.v if write else None,
                         cache.page_table if write else None, cache.table_stride, cache.ring,
                         q_off=0, n_heads=nh, q_width=hd, k_off=nq_w, n_kv=nk, k_width=hd,
                         v_off=nq_w + nk_w, v_width=vd, v_from_k=False,
                         q_norm=self.q_norm, k_norm=self.k_norm, eps=self.norm_eps,
                         inv_freq=inv_freq, rot_dims=rot_dims, rot_style=style,
                         rot_magnitude=magnitude, q_rot_off=0, k_rot_off=0, status=ctx.status)
        o = torch.empty((n, nh * vd), dtype=act, device=dev)
        scored_attention(self.scores(), q, k_step, v_step, cache, ctx, o)
        if self.gate:
            K.gate_mul(o, qkv, nq_w + nk_w + self.n_kv_heads * vd, self.out_scale)
        elif self.out_scale != 1.0:
            raise K.KernelError("an output scale rides on the output gate; this attention has none")
        project_out(self.out, o, ctx, residual)
