"""A selective state-space mixer in the first Mamba form (a state of ``n_state`` numbers per
channel, a decay of its own per channel and state), with per-sequence state instead of cached keys.

    [u | z] = W_in x                                        ``inner`` channels each
    u <- silu(conv(u) + b_conv)         causal, per channel, ``conv`` taps, the last tap on the
                                        current token, zeros before the start
    [r | B | C] = W_x u                 r: ``dt_rank``; B, C: ``n_state`` each
    dt = softplus(W_dt r + b_dt)        one per channel;  A = -exp(A_log), [inner, n_state]
    per channel c, state n:  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n
    y_c = sum_n S[c, n] C_n + D_c u_c;   out = W_o (y * silu(z))

State per sequence (float32, zeroed when a slot is handed out): S and the last ``conv`` - 1 inputs
of the convolution.  A step may bring any number of tokens per sequence; the recurrence walks them
in order.  Between the in- and out-projections everything is float32 in both engines except the
operand of W_x, which is rounded to the activation type; the step-size product W_dt r runs on the
FP32 pipe with float32 operands.  Tensor names behind ``prefix + tensor_prefix``: ``in``, ``conv``,
``conv.b``, ``x``, ``dt``, ``dt.b``, ``A_log``, ``D``, ``o``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CallBinding, Mixer, StateRequest, StepContext
from .linear import Linear
from .sink_attention import project_out

SCAN_STATE = "scan.state"
SCAN_CONV = "scan.conv"


class SelectiveScan(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture
    stores_fresh_output = True     # its last product goes through ``project_out``

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "recurrent", "gemm_simt"] + (["gemm_tc"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, inner: int, n_state: int, dt_rank: int, conv: int,
                 out_scale: float = 1.0, tensor_prefix: str = "mix.", init_std: float = 0.02):
        if min(inner, n_state, dt_rank, conv) < 1:
            raise ValueError("selective scan: every size must be at least 1")
        if conv > 8 or n_state > 256:
            raise ValueError("selective scan: the kernels take up to 8 taps and a state of up to 256")
        self.hidden_size = int(hidden_size)
        self.inner = int(inner)
        self.n_state = int(n_state)
        self.dt_rank = int(dt_rank)
        self.conv = int(conv)
        self.out_scale = float(out_scale)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.in_proj: Optional[Linear] = None
        self.x_proj: Optional[Linear] = None
        self.dt_proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.w: Dict[str, torch.Tensor] = {}

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        init = Init(0.0, self.init_std)
        c, n, r = self.inner, self.n_state, self.dt_rank
        return [TensorSpec(f"{p}in", (2 * c, self.hidden_size), MATRIX, init),
                # small per-channel tensors and the step-size product are held in float32
                TensorSpec(f"{p}conv", (c, self.conv), VECTOR, Init(0.0, 0.3)),
                TensorSpec(f"{p}conv.b", (c,), VECTOR, Init(0.0, 0.1)),
                TensorSpec(f"{p}x", (r + 2 * n, c), MATRIX, init),
                TensorSpec(f"{p}dt", (c, r), VECTOR, Init(0.0, 0.3)),
                TensorSpec(f"{p}dt.b", (c,), VECTOR, Init(-1.0, 0.5)),
                TensorSpec(f"{p}A_log", (c, n), VECTOR, Init(0.0, 0.5)),
                TensorSpec(f"{p}D", (c,), VECTOR, Init(1.0, 0.2)),
                TensorSpec(f"{p}o", (self.hidden_size, c), MATRIX, init)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        self.in_proj = Linear(weights[f"{p}in"])
        self.x_proj = Linear(weights[f"{p}x"])
        self.dt_proj = Linear(weights[f"{p}dt"], weights[f"{p}dt.b"])
        self.out = Linear(weights[f"{p}o"])
        self.w = {n: weights[f"{p}{n}"] for n in ("conv", "conv.b", "A_log", "D")}

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        out = {f"{p}in": self.in_proj.weight, f"{p}x": self.x_proj.weight, f"{p}dt": self.dt_proj.weight,
               f"{p}dt.b": self.dt_proj.bias, f"{p}o": self.out.weight}
        out.update({f"{p}{n}": t for n, t in self.w.items()})
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def state_request(self) -> Sequence[StateRequest]:
        return (StateRequest(SCAN_STATE, (self.inner, self.n_state), torch.float32),
                StateRequest(SCAN_CONV, (self.inner, self.conv - 1), torch.float32))

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n, dev = x.shape[0], x.device
        c, ns, r = self.inner, self.n_state, self.dt_rank
        proj = self.in_proj.forward(x, torch.float32, row_scale=ctx.input_scale)      # [u | z]
        u = torch.empty((n, c), dtype=torch.float32, device=dev)
        K.conv_silu(proj, 0, c, self.w["conv"], self.w["conv.b"], binding.state[SCAN_CONV],
                    ctx.token_row, ctx.cu_seqlens, ctx.slots, u, ctx.n_rows, single=ctx.single_token)
        if ctx.act_dtype == torch.float32:
            u_act = u
        else:
            u_act = torch.empty((n, c), dtype=ctx.act_dtype, device=dev)
            K.cast(u, u_act)
        rbc = self.x_proj.forward(u_act, torch.float32)                                # [r | B | C]
        low = rbc[:, :r]                                           # rows may be strided
        dt_raw = self.dt_proj.forward(low, torch.float32)          # float32 operands: the FP32 pipe
        y = torch.empty((n, c), dtype=ctx.act_dtype, device=dev)
        K.selective_scan(u, dt_raw, rbc, r, r + ns, proj, c, self.w["A_log"], self.w["D"],
                         binding.state[SCAN_STATE], ctx.cu_seqlens, ctx.slots, y, ctx.n_rows,
                         mul=self.out_scale)
        project_out(self.out, y, ctx, residual)
