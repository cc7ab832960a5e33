"""Retention as a mixer: linear attention with a fixed decay per head, no softmax and no
denominator, with per-sequence state instead of cached keys.

    q, k, v, g = Wq u, Wk u, Wv u, Wg u          heads of ``head_dim`` (q, k) and ``value_dim`` (v, g)
    the first ``rotary_dim`` dimensions of every head of q and k rotated           (``position``)
    k <- k * head_dim^(-1/2)
    per head h:  S_t = decay_h S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t
    o <- o / sqrt(mean(o^2) + eps) per head (no weight);  out = Wo (o * silu(g))

State per sequence (float32, zeroed when a slot is handed out): S of every head.  A step may
bring any number of tokens per sequence; the recurrence walks them in order, so the result does
not depend on how a sequence is cut.  Everything between the two products is float32 in both
engines.  One packed product gives q|k|v|g in float32; one kernel rotates and scales q and k;
the scan reads v from the product's rows; one kernel norms, gates and rounds; Wo adds into the
residual stream.  Tensor names behind ``prefix + tensor_prefix``: ``q``, ``k``, ``v``, ``g``, ``o``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config.base import PartSpec
from ..kernels import api as K
from ..weights.spec import MATRIX, Init, TensorSpec
from .base import CallBinding, Mixer, StateRequest, StepContext
from .linear import Linear
from .sink_attention import project_out

RETENTION_STATE = "retention.state"


class Retention(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture
    stores_fresh_output = True     # its last product goes through ``project_out``

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "mixer_prep", "retention", "gemm_tc" if dtype == torch.bfloat16 else "gemm_simt"]

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, value_dim: int,
                 decay: Sequence[float], norm_eps: float, position: Optional[PartSpec] = None,
                 out_scale: float = 1.0, tensor_prefix: str = "mix.", init_std: float = 0.02):
        from ..registry import build_part
        if min(n_heads, head_dim, value_dim) < 1:
            raise ValueError("retention: every size must be at least 1")
        if head_dim > 256:
            raise ValueError("retention: the kernel takes keys up to 256 wide")
        if len(decay) != n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {n_heads} heads")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim)
        self.decay = [float(d) for d in decay]
        self.norm_eps = float(norm_eps)
        self.out_scale = float(out_scale)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.position = build_part("position", position) if position is not None else None
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self._decay: Optional[torch.Tensor] = None

    def _widths(self):
        return self.n_heads * self.head_dim, self.n_heads * self.value_dim

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nv = self._widths()
        init = Init(0.0, self.init_std)
        return [TensorSpec(f"{p}q", (nq, self.hidden_size), MATRIX, init),
                TensorSpec(f"{p}k", (nq, self.hidden_size), MATRIX, init),
                TensorSpec(f"{p}v", (nv, self.hidden_size), MATRIX, init),
                TensorSpec(f"{p}g", (nv, self.hidden_size), MATRIX, init),
                TensorSpec(f"{p}o", (self.hidden_size, nv), MATRIX, init)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        parts = [weights[f"{p}{n}"] for n in "qkvg"]
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        self.proj = Linear(torch.cat(parts, dim=0).contiguous())
        self.out = Linear(weights[f"{p}o"])
        self._decay = torch.tensor(self.decay, dtype=torch.float32, device=self.out.weight.device)

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nv = self._widths()
        w = self.proj.weight
        return {f"{p}q": w[:nq], f"{p}k": w[nq:2 * nq], f"{p}v": w[2 * nq:2 * nq + nv],
                f"{p}g": w[2 * nq + nv:], f"{p}o": self.out.weight}

    # ---- what it keeps per sequence -----------------------------------------------------
    def state_request(self) -> Sequence[StateRequest]:
        return (StateRequest(RETENTION_STATE, (self.n_heads, self.value_dim, self.head_dim),
                             torch.float32),)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n, dev = x.shape[0], x.device
        nh, hd, vd = self.n_heads, self.head_dim, self.value_dim
        nq, nv = self._widths()
        proj = self.proj.forward(x, torch.float32, row_scale=ctx.input_scale)
        inv_freq, rot_dims, style, magnitude = None, 0, 0, 1.0
        if self.position is not None and getattr(self.position, "rotary_dim", 0) > 0:
            inv_freq, rot_dims, style = self.position.tables(dev)
            magnitude = self.position.magnitude()
        q = torch.empty((n, nh, hd), dtype=torch.float32, device=dev)
        k = torch.empty((n, nh, hd), dtype=torch.float32, device=dev)
        K.head_prepare(proj, ctx.positions, ctx.token_row, ctx.seq_end, q, k, None, None, None, None,
                       0, 0, q_off=0, n_heads=nh, q_width=hd, k_off=nq, n_kv=nh, k_width=hd,
                       v_off=2 * nq, v_width=vd, q_norm=None, k_norm=None, eps=self.norm_eps,
                       inv_freq=inv_freq, rot_dims=rot_dims, rot_style=style,
                       rot_magnitude=magnitude, q_mul=1.0, k_mul=hd ** -0.5, status=ctx.status)
        o = torch.empty((n, nv), dtype=torch.float32, device=dev)
        K.retention_scan(q, k, proj, 2 * nq, self._decay, binding.state[RETENTION_STATE],
                         ctx.cu_seqlens, ctx.slots, o, ctx.n_rows)
        gated = torch.empty((n, nv), dtype=ctx.act_dtype, device=dev)
        K.unit_norm_gate(o, proj, 2 * nq + nv, gated, nh, self.norm_eps, "silu", self.out_scale)
        project_out(self.out, gated, ctx, residual)
