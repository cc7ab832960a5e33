"""Routed feed-forward: a token's output is the weighted sum of a few small gated experts that a
linear router picks for it.

    z = Wr u + br                          float32 (the router's matrix is held in float32)
    the ``top`` experts with the largest z; their weights = softmax over the chosen z only
    expert e:  Wd_e (act(Wg_e u) * (Wu_e u)),  act = silu;  no biases
    out = sum over the chosen e of weight_e * expert_e(u)

Every size is a parameter, and so are the tensors' names (behind the layer's prefix):
``router_name``, ``router_bias_name`` (None: no bias) and ``expert_name`` with ``{e}`` for the
expert's number, followed by ``.gate``, ``.up``, ``.down``.  The experts' matrices are stacked at
load ([experts, ff, width] and [experts, width, ff]).

Two ways through a step.  Few tokens (decoding; always inside a CUDA graph capture): one kernel
per half, a block per (token, choice), the expert's rows read by index; nothing is read back.  Many
tokens: the (token, choice) pairs are grouped by expert on the device, the offsets come back to the
host (one small read), and each expert runs as two dense products over its rows, the gate's
activation in the first one's epilogue; the weighted rows are then added into the residual token by
token, the choices in order, so the sum does not depend on the batch.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import FeedForward, StepContext, settle_pending
from .linear import Linear

# steps of up to this many tokens run the per-token kernels
PER_TOKEN_MAX = int(os.environ.get("MINFER_B200_MOE_PER_TOKEN_MAX", "48"))


class RoutedExperts(FeedForward):
    capturable = True      # the per-token path launches kernels only; captures always take it

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "moe", "gemm_simt"] + (["gemm_tc"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, intermediate_size: int, n_experts: int, top: int,
                 activation: str = "silu", router_name: str = "mlp.router",
                 router_bias_name: Optional[str] = "mlp.router.b",
                 expert_name: str = "mlp.e{e}", init_std: float = 0.02, router_std: float = 0.5):
        if activation != "silu":
            raise ValueError(f"the experts' gate has the activation silu, got {activation!r}")
        if not 1 <= top <= n_experts:
            raise ValueError(f"a token cannot use {top} of {n_experts} experts")
        if top > 16:
            raise ValueError("the router's kernel takes up to 16 experts a token")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.n_experts = int(n_experts)
        self.top = int(top)
        self.activation = activation
        self.router_name, self.router_bias_name = router_name, router_bias_name
        self.expert_name = expert_name
        self.init_std, self.router_std = float(init_std), float(router_std)
        self.router: Optional[Linear] = None
        self.w_gate: Optional[torch.Tensor] = None       # [experts, ff, width]
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None       # [experts, width, ff]
        self.w_gate_up: Optional[torch.Tensor] = None    # [experts, 2 ff, width], rows gate, up, ..
        # (``w_gate`` and ``w_up`` are its even and odd rows)

    def _expert(self, prefix: str, e: int) -> str:
        return f"{prefix}{self.expert_name.format(e=e)}"

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        init = Init(0.0, self.init_std)
        ff, w = self.intermediate_size, self.hidden_size
        # the router's matrix and bias take part in a 32-bit product: held in float32
        specs = [TensorSpec(f"{prefix}{self.router_name}", (self.n_experts, w), VECTOR,
                            Init(0.0, self.router_std))]
        if self.router_bias_name is not None:
            specs.append(TensorSpec(f"{prefix}{self.router_bias_name}", (self.n_experts,), VECTOR,
                                    Init(0.0, self.router_std)))
        for e in range(self.n_experts):
            p = self._expert(prefix, e)
            specs += [TensorSpec(f"{p}.gate", (ff, w), MATRIX, init),
                      TensorSpec(f"{p}.up", (ff, w), MATRIX, init),
                      TensorSpec(f"{p}.down", (w, ff), MATRIX, init)]
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        bias = (weights[f"{prefix}{self.router_bias_name}"] if self.router_bias_name is not None
                else None)
        self.router = Linear(weights[f"{prefix}{self.router_name}"], bias)
        names = [self._expert(prefix, e) for e in range(self.n_experts)]
        mats = [weights[f"{p}.{half}"] for p in names for half in ("gate", "up", "down")]
        dtype = mats[0].dtype if len({t.dtype for t in mats}) == 1 else torch.float32
        gate = torch.stack([weights[f"{p}.gate"].to(dtype) for p in names])
        up = torch.stack([weights[f"{p}.up"].to(dtype) for p in names])
        # one stack whose rows alternate gate, up: the per-token kernel reads either half by its
        # stride, and the tensor-core product of a grouped step finds a pair in neighbouring lanes
        # of its epilogue
        self.w_gate_up = torch.stack([gate, up], dim=2).reshape(
            self.n_experts, 2 * self.intermediate_size, self.hidden_size).contiguous()
        pairs = self.w_gate_up.view(self.n_experts, self.intermediate_size, 2, self.hidden_size)
        self.w_gate, self.w_up = pairs[:, :, 0], pairs[:, :, 1]
        self.w_down = torch.stack([weights[f"{p}.down"].to(dtype) for p in names]).contiguous()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        out = {f"{prefix}{self.router_name}": self.router.weight}
        if self.router_bias_name is not None:
            out[f"{prefix}{self.router_bias_name}"] = self.router.bias
        for e in range(self.n_experts):
            p = self._expert(prefix, e)
            out[f"{p}.gate"], out[f"{p}.up"] = self.w_gate[e], self.w_up[e]
            out[f"{p}.down"] = self.w_down[e]
        return out

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        ctx.extras.pop("prepare_for", None)
        settle_pending(ctx, residual)              # the experts add into the complete stream
        n, dev = x.shape[0], x.device
        if n == 0:
            return
        logits = self.router.forward(x, torch.float32)
        idx = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        wts = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        K.moe_route(logits, idx, wts, self.top)
        if n <= PER_TOKEN_MAX or torch.cuda.is_current_stream_capturing():
            hidden = torch.empty((n, self.top, self.intermediate_size), dtype=x.dtype, device=dev)
            K.moe_experts(x, self.w_gate, self.w_up, self.w_down, idx, wts, hidden, residual)
            return
        self._grouped(x, idx, wts, residual)

    def _grouped(self, x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor,
                 residual: torch.Tensor) -> None:
        from ..kernels import gemm
        n, dev = x.shape[0], x.device
        ff, width, top = self.intermediate_size, self.hidden_size, self.top
        n_pairs = n * top
        counts = torch.zeros(self.n_experts, dtype=torch.int32, device=dev)
        offsets = torch.empty(self.n_experts + 1, dtype=torch.int32, device=dev)
        order = torch.empty(n_pairs, dtype=torch.int32, device=dev)
        where = torch.empty((n, top), dtype=torch.int32, device=dev)
        K.moe_counts(idx, counts)
        K.moe_place(idx, counts, offsets, order, where)
        first = offsets.tolist()                   # the one read of the step: rows per expert
        xg = torch.empty((n_pairs, width), dtype=x.dtype, device=dev)
        K.moe_gather(x, order, xg, top)
        act = torch.empty((n_pairs, ff), dtype=x.dtype, device=dev)
        y = torch.empty((n_pairs, width), dtype=torch.float32, device=dev)
        fused = (self.w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
                 and gemm.use_tensor_cores()
                 and K.gemm_tc_supported(xg, self.w_gate_up[0]))
        for e in range(self.n_experts):
            lo, hi = first[e], first[e + 1]
            if hi <= lo:
                continue
            xe, ae = xg[lo:hi], act[lo:hi]
            if fused:
                K.gemm_tc(xe, self.w_gate_up[e], None, ae, K.gated_epilogue("silu"),
                          gemm.status_word(dev))
            else:
                gu = torch.empty((hi - lo, 2 * ff), dtype=torch.float32, device=dev)
                K.gemm_simt(xe, self.w_gate_up[e], None, gu)
                K.swiglu(gu, ae, True, "silu")
            Linear(self.w_down[e]).forward(ae, torch.float32, out=y[lo:hi])
        K.moe_combine(y, where, wts, residual)
