"""Gated feed-forward: down( act(gate(x)) * up(x) ), no biases; act is silu or the tanh form of
gelu.

The reference builds it as silu + mul that its fusion pass folds into SwiGLU
(src/models/qwen2/graph.rs:154-175, src/graph/fusion.rs:37-87), with
silu(z) = z / (1 + exp(-z)) (src/vec_ops.rs:131-146); its Metal path packs gate|up into
one matrix (src/models/qwen2/graph.rs:148-169).  Here gate|up is always one product and
the down projection adds into the residual stream in its epilogue.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import FeedForward, StepContext, settle_pending
from .linear import Linear


class GatedMlp(FeedForward):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "gemm_tc"] if dtype == torch.bfloat16 else ["ops", "gemm_simt"]

    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 init_std: float = 0.02, gate_name: str = "mlp.gate_proj.weight",
                 up_name: str = "mlp.up_proj.weight", down_name: str = "mlp.down_proj.weight"):
        """``activation`` of the gate: "silu", or "gelu_tanh" = 0.5 z (1 + tanh(sqrt(2/pi) (z +
        0.044715 z^3))).  The tensors' names (behind the layer's prefix) are parameters."""
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"the gated feed-forward has the activations {self.ACTIVATIONS}, got "
                             f"{activation!r}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.activation = activation
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.init_std = float(init_std)
        self.interleaved = False
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        init = Init(0.0, self.init_std)
        return [TensorSpec(f"{prefix}{self.gate_name}", (self.intermediate_size, self.hidden_size),
                           MATRIX, init),
                TensorSpec(f"{prefix}{self.up_name}", (self.intermediate_size, self.hidden_size),
                           MATRIX, init),
                TensorSpec(f"{prefix}{self.down_name}", (self.hidden_size, self.intermediate_size),
                           MATRIX, init)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        g, u = weights[f"{prefix}{self.gate_name}"], weights[f"{prefix}{self.up_name}"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        # bfloat16: rows alternate gate, up so that the tensor-core kernel's epilogue finds a
        # pair in neighbouring lanes and writes silu(gate) * up directly; float32: gates first
        self.interleaved = g.dtype == torch.bfloat16
        if self.interleaved:
            packed = torch.stack([g, u], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            packed = torch.cat([g, u], dim=0)
        self.gate_up = Linear(packed.contiguous())
        self.down = Linear(weights[f"{prefix}{self.down_name}"])
        self.accepts_row_scale = self.interleaved and self.gate_up.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        w = self.gate_up.weight
        if self.interleaved:
            pairs = w.view(self.intermediate_size, 2, self.hidden_size)
            gate, up = pairs[:, 0], pairs[:, 1]
        else:
            gate, up = w[:self.intermediate_size], w[self.intermediate_size:]
        return {f"{prefix}{self.gate_name}": gate, f"{prefix}{self.up_name}": up,
                f"{prefix}{self.down_name}": self.down.weight}

    def forward_add(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        from ..kernels import gemm
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=ctx.act_dtype,
                          device=x.device)
        w = self.gate_up.weight
        rs = ctx.input_scale                       # the norm's 1/rms, if this product is to apply it
        if (self.interleaved and x.shape[0] > 0 and gemm.use_tensor_cores()
                and K.gemm_tc_supported(x, w)):
            epi = K.gated_epilogue(self.activation)
            if rs is not None:
                K.gemm_tc_fused(x, w, None, act, epi, gemm.status_word(x.device), row_scale=rs)
            else:
                K.gemm_tc(x, w, None, act, epi, gemm.status_word(x.device))
        else:
            if rs is not None:
                raise K.KernelError("a row scale needs the tensor-core product")
            gu = self.gate_up.forward(x, ctx.act_dtype)
            K.swiglu(gu, act, self.interleaved, self.activation)
        target = ctx.extras.pop("prepare_for", None)
        if target is not None:
            settle_pending(ctx, residual)
            prepared = self.down.accumulate_prepared(act, residual, target)
            if prepared is not None:
                ctx.extras["prepared"] = prepared
                return
        pending = self.down.partial_sums(act)
        if pending is None:
            self.down.forward(act, torch.float32, out=residual, accumulate=True)
        else:
            settle_pending(ctx, residual)          # never two at once
            ctx.extras["pending"] = pending


# MINFER_B200_FUSE_ACTIVATION=0: the dense feed-forward's activation runs as a kernel of its own
FUSE_ACTIVATION = os.environ.get("MINFER_B200_FUSE_ACTIVATION", "1") != "0"


class DenseMlp(FeedForward):
    """Feed-forward without a gate: down( act(up(x)) ), no biases.  ``activation``:

    ``"xielu"``  with two learned numbers a = (a0, a1) in the tensor ``act_name``:
                 z > 0: softplus(a0) z^2 + z/2;  z <= 0: (1/2 + softplus(a1)) (exp(z) - 1 - z) + z/2,
                 evaluated in float32 on the product's float32 sums.

    ``"poly_norm"``  with four learned numbers (a, b, c, e): a N(z) + b N(z^2) + c N(z^3) + e,
                 powers element by element, N(u) = u / sqrt(mean(u^2) + eps) over a token's
                 feed-forward values (``norm_eps``), in float32 on the product's float32 sums.

    ``"gelu"``   the erf form 0.5 z (1 + erf(z / sqrt 2)), no learned numbers (and no tensor
                 ``act_name``), in float32 on the product's float32 sums.

    Tensor names are parameters (``up_name``, ``down_name``, ``act_name``, each behind the
    layer's prefix)."""

    capturable = True      # launches kernels only; safe inside a CUDA graph capture
    stores_fresh_output = True     # its last product goes through ``project_out``
    ACTIVATIONS = ("xielu", "poly_norm", "gelu")
    ACT_NUMBERS = {"xielu": 2, "poly_norm": 4, "gelu": 0}

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "gemm_tc"] if dtype == torch.bfloat16 else ["ops", "gemm_simt"]

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu",
                 up_name: str = "mlp.up", down_name: str = "mlp.down", act_name: str = "mlp.act",
                 init_std: float = 0.02, norm_eps: float = 1e-6):
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"the dense feed-forward has the activations {self.ACTIVATIONS}, got "
                             f"{activation!r}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.activation = activation
        self.norm_eps = float(norm_eps)
        self.up_name, self.down_name, self.act_name = up_name, down_name, act_name
        self.init_std = float(init_std)
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.act_params: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{prefix}{self.up_name}", (self.intermediate_size, self.hidden_size),
                            MATRIX, init),
                 TensorSpec(f"{prefix}{self.down_name}", (self.hidden_size, self.intermediate_size),
                            MATRIX, init)]
        if self.ACT_NUMBERS[self.activation]:
            specs.append(TensorSpec(f"{prefix}{self.act_name}", (self.ACT_NUMBERS[self.activation],),
                                    VECTOR, Init(0.0, 0.5)))
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.up = Linear(weights[f"{prefix}{self.up_name}"])
        self.down = Linear(weights[f"{prefix}{self.down_name}"])
        self.act_params = (weights[f"{prefix}{self.act_name}"] if self.ACT_NUMBERS[self.activation]
                           else None)
        self.accepts_row_scale = self.up.takes_row_scale()
        if self.activation != "xielu":
            return
        # the activation's two coefficients, once, for the product whose epilogue applies it
        a = self.act_params.detach().to("cpu", torch.float64)
        sp = torch.log1p(torch.exp(-a.abs())) + torch.clamp(a, min=0)
        self._act_p, self._act_n = float(sp[0]), 0.5 + float(sp[1])

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        out = {f"{prefix}{self.up_name}": self.up.weight, f"{prefix}{self.down_name}": self.down.weight}
        if self.act_params is not None:
            out[f"{prefix}{self.act_name}"] = self.act_params
        return out

    def forward_add(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        from ..kernels import gemm
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=ctx.act_dtype, device=x.device)
        if self.activation == "poly_norm":
            # a row's three sums come before any of its outputs: the activation is a kernel of
            # its own on the product's float32 rows
            z = self.up.forward(x, torch.float32, row_scale=ctx.input_scale)
            K.poly_norm(z, self.act_params, act, self.norm_eps)
        elif self.activation == "gelu":
            z = self.up.forward(x, torch.float32, row_scale=ctx.input_scale)
            K.unary_act(z, act, "gelu")
        elif (x.shape[0] > 0 and self.up.takes_row_scale() and x.dtype == torch.bfloat16
                and K.gemm_tc_supported(x, self.up.weight) and FUSE_ACTIVATION):
            # the activation rides on the up projection's epilogue
            K.gemm_tc_xielu(x, self.up.weight, act, self._act_p, self._act_n,
                            gemm.status_word(x.device), row_scale=ctx.input_scale)
        else:
            z = self.up.forward(x, torch.float32, row_scale=ctx.input_scale)
            K.xielu(z, self.act_params, act)
        from .sink_attention import project_out
        project_out(self.down, act, ctx, residual)
