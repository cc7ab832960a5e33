"""Routed feed-forward: a token's output is the weighted sum of a few small gated experts that a
linear router picks for it.

    z = Wr u + br                          float32 (the router's matrix is held in float32)
    the ``top`` experts with the largest z; their weights = softmax over the chosen z only
    expert e:  Wd_e (act(Wg_e u) * (Wu_e u)),  act = silu;  no biases
    out = sum over the chosen e of weight_e * expert_e(u)

Options for designs that route otherwise (each a parameter):

    scoring "softmax_all"   scores s = softmax(z) over ALL router outputs; the ``top`` outputs with the
                            largest s + correction are chosen (``correction_name``: a tensor of one
                            number per output; None: none); the weights are the chosen s themselves,
                            not renormalized
    identity                the last ``identity`` router outputs (beyond the ``n_experts`` experts with
                            weights) stand for experts that return the token's input: weight * u
    activation "clamped_swish"   y = g' sigmoid(1.702 g') (u' + 1), g' = min(Wg u, limit),
                            u' = clamp(Wu u, -limit, limit)
    shared                  {"ff", "limit", "name", "gate_name"}: one more expert of the same form that
                            every token uses, times sigmoid(Ws u) (one number per token), added

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
                 expert_name: str = "mlp.e{e}", init_std: float = 0.02, router_std: float = 0.5,
                 scoring: str = "softmax_top", correction_name: Optional[str] = None,
                 identity: int = 0, limit: float = 0.0, shared: Optional[dict] = None):
        if activation not in K.EXPERT_ACTIVATIONS:
            raise ValueError(f"the experts' activation is one of {sorted(K.EXPERT_ACTIVATIONS)}, got "
                             f"{activation!r}")
        if scoring not in ("softmax_top", "softmax_all"):
            raise ValueError(f"scoring is softmax_top or softmax_all, got {scoring!r}")
        if identity < 0 or (identity > 0 and scoring != "softmax_all"):
            raise ValueError("experts without weights need the scoring softmax_all")
        if shared is not None and scoring != "softmax_all":
            raise ValueError("a shared expert needs the scoring softmax_all")
        if activation == "clamped_swish" and not limit > 0.0:
            raise ValueError("the clamped activation needs a positive limit")
        if not 1 <= top <= n_experts + identity:
            raise ValueError(f"a token cannot use {top} of {n_experts + identity} experts")
        if top > 16:
            raise ValueError("the router's kernel takes up to 16 experts a token")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.n_experts = int(n_experts)
        self.top = int(top)
        self.activation = activation
        self.scoring, self.correction_name = scoring, correction_name
        self.identity = int(identity)
        self.n_outputs = self.n_experts + self.identity          # what the router chooses among
        self.limit = float(limit)
        self.alpha = 1.702 if activation == "clamped_swish" else 1.0
        self.shared = dict(shared) if shared is not None else None
        if self.shared is not None:
            self.shared.setdefault("name", "mlp.shared")
            self.shared.setdefault("gate_name", "mlp.shared.sg")
            self.shared.setdefault("limit", self.limit)
        self.correction: Optional[torch.Tensor] = None
        self.shared_interleaved = False
        self.shared_gate_up: Optional[Linear] = None
        self.shared_down: Optional[Linear] = None
        self.router_name, self.router_bias_name = router_name, router_bias_name
        self.expert_name = expert_name
        self.init_std, self.router_std = float(init_std), float(router_std)
        # the per-token kernels keep a token's input and its experts' hidden values in shared memory;
        # sizes beyond that always take the grouped path, which reads a few numbers back on the host
        # and so cannot be part of a CUDA graph
        self.per_token_fits = (4 * self.hidden_size <= 48 * 1024
                               and 4 * self.top * self.intermediate_size <= 48 * 1024)
        self.capturable = self.per_token_fits
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
        specs = [TensorSpec(f"{prefix}{self.router_name}", (self.n_outputs, w), VECTOR,
                            Init(0.0, self.router_std))]
        if self.router_bias_name is not None:
            specs.append(TensorSpec(f"{prefix}{self.router_bias_name}", (self.n_outputs,), VECTOR,
                                    Init(0.0, self.router_std)))
        if self.correction_name is not None:
            specs.append(TensorSpec(f"{prefix}{self.correction_name}", (self.n_outputs,), VECTOR,
                                    Init(0.0, 0.05)))
        if self.shared is not None:
            p, sff = f"{prefix}{self.shared['name']}", int(self.shared["ff"])
            specs += [TensorSpec(f"{p}.gate", (sff, w), MATRIX, init),
                      TensorSpec(f"{p}.up", (sff, w), MATRIX, init),
                      TensorSpec(f"{p}.down", (w, sff), MATRIX, init),
                      # one more row of the router's float32 product
                      TensorSpec(f"{prefix}{self.shared['gate_name']}", (1, w), VECTOR,
                                 Init(0.0, self.router_std))]
        for e in range(self.n_experts):
            p = self._expert(prefix, e)
            specs += [TensorSpec(f"{p}.gate", (ff, w), MATRIX, init),
                      TensorSpec(f"{p}.up", (ff, w), MATRIX, init),
                      TensorSpec(f"{p}.down", (w, ff), MATRIX, init)]
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        bias = (weights[f"{prefix}{self.router_bias_name}"] if self.router_bias_name is not None
                else None)
        router = weights[f"{prefix}{self.router_name}"]
        if self.correction_name is not None:
            self.correction = weights[f"{prefix}{self.correction_name}"]
        if self.shared is not None:
            # the shared expert's gate is one more row of the router's product
            p = f"{prefix}{self.shared['name']}"
            router = torch.cat([router, weights[f"{prefix}{self.shared['gate_name']}"].to(router.dtype)],
                               dim=0).contiguous()
            if bias is not None:
                bias = torch.cat([bias, torch.zeros(1, dtype=bias.dtype, device=bias.device)])
            sg, su = weights[f"{p}.gate"], weights[f"{p}.up"]
            if sg.dtype != su.dtype:
                sg, su = sg.to(torch.float32), su.to(torch.float32)
            # bfloat16: rows alternate gate, up for the product's gated epilogue; else gates first
            self.shared_interleaved = sg.dtype == torch.bfloat16
            if self.shared_interleaved:
                packed = torch.stack([sg, su], dim=1).reshape(2 * sg.shape[0], sg.shape[1])
            else:
                packed = torch.cat([sg, su], dim=0)
            self.shared_gate_up = Linear(packed.contiguous())
            self.shared_down = Linear(weights[f"{p}.down"])
        self.router = Linear(router, bias)
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
        out = {f"{prefix}{self.router_name}": self.router.weight[:self.n_outputs]}
        if self.router_bias_name is not None:
            out[f"{prefix}{self.router_bias_name}"] = self.router.bias[:self.n_outputs]
        if self.correction is not None:
            out[f"{prefix}{self.correction_name}"] = self.correction
        if self.shared is not None:
            p, sff = f"{prefix}{self.shared['name']}", int(self.shared["ff"])
            out[f"{prefix}{self.shared['gate_name']}"] = self.router.weight[self.n_outputs:]
            sw = self.shared_gate_up.weight
            if self.shared_interleaved:
                pairs = sw.view(sff, 2, self.hidden_size)
                out[f"{p}.gate"], out[f"{p}.up"] = pairs[:, 0], pairs[:, 1]
            else:
                out[f"{p}.gate"], out[f"{p}.up"] = sw[:sff], sw[sff:]
            out[f"{p}.down"] = self.shared_down.weight
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
        w = self.router.weight
        if w.dtype == torch.float32 and w.is_contiguous():
            logits = torch.empty((n, w.shape[0]), dtype=torch.float32, device=dev)
            K.router_logits(x, w, self.router.bias, logits)
        else:
            logits = self.router.forward(x, torch.float32)
        idx = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        wts = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        if self.scoring == "softmax_all":
            K.moe_route_scored(logits, self.correction, idx, wts, self.top, self.n_outputs)
        else:
            K.moe_route(logits, idx, wts, self.top)
        if self.per_token_fits and (n <= PER_TOKEN_MAX or torch.cuda.is_current_stream_capturing()):
            hidden = torch.empty((n, self.top, self.intermediate_size), dtype=x.dtype, device=dev)
            K.moe_experts(x, self.w_gate, self.w_up, self.w_down, idx, wts, hidden, residual,
                          self.activation, self.limit, self.alpha)
        else:
            self._grouped(x, idx, wts, residual)
        if self.shared is not None:
            # act(gate, up) * sigmoid(the router product's extra column), then down into the stream
            from ..kernels import gemm
            sff = int(self.shared["ff"])
            act = torch.empty((n, sff), dtype=x.dtype, device=dev)
            row_gate = logits[:, self.n_outputs]
            sw = self.shared_gate_up.weight
            if (self.shared_interleaved and x.dtype == torch.bfloat16 and gemm.use_tensor_cores()
                    and K.gemm_tc_supported(x, sw)):
                K.gemm_tc_gated(x, sw, act, self.activation, float(self.shared["limit"]), self.alpha,
                                gemm.status_word(dev))
                K.row_gate_mul(act, row_gate)
            else:
                gu = self.shared_gate_up.forward(x, torch.float32)
                K.gated_act(gu, act, self.activation, float(self.shared["limit"]), self.alpha,
                            row_gate=row_gate, interleaved=self.shared_interleaved)
            self.shared_down.forward(act, torch.float32, out=residual, accumulate=True)

    def _grouped(self, x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor,
                 residual: torch.Tensor) -> None:
        from ..kernels import gemm
        n, dev = x.shape[0], x.device
        ff, width, top = self.intermediate_size, self.hidden_size, self.top
        n_pairs = n * top
        counts = torch.zeros(self.n_outputs, dtype=torch.int32, device=dev)
        offsets = torch.empty(self.n_outputs + 1, dtype=torch.int32, device=dev)
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
        for e in range(self.n_outputs):
            lo, hi = first[e], first[e + 1]
            if hi <= lo:
                continue
            if e >= self.n_experts:                # an expert without weights hands its input on
                if xg.dtype == y.dtype:
                    y[lo:hi].copy_(xg[lo:hi])      # (a device copy)
                else:
                    K.cast(xg[lo:hi], y[lo:hi])
                continue
            xe, ae = xg[lo:hi], act[lo:hi]
            if fused:
                # the activation rides on the product's epilogue
                K.gemm_tc_gated(xe, self.w_gate_up[e], ae, self.activation, self.limit, self.alpha,
                                gemm.status_word(dev))
            else:
                gu = torch.empty((hi - lo, 2 * ff), dtype=torch.float32, device=dev)
                if self.activation == "silu":
                    K.gemm_simt(xe, self.w_gate_up[e], None, gu)
                    K.swiglu(gu, ae, True, "silu")
                else:
                    # gates first, then ups: the two strided halves of the stack as two products
                    Linear(self.w_gate[e]).forward(xe, torch.float32, out=gu[:, :ff])
                    Linear(self.w_up[e]).forward(xe, torch.float32, out=gu[:, ff:])
                    K.gated_act(gu, ae, self.activation, self.limit, self.alpha)
            Linear(self.w_down[e]).forward(ae, torch.float32, out=y[lo:hi])
        K.moe_combine(y, where, wts, residual)
