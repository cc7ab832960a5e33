"""A gated delta-rule mixer: a matrix-valued state per head, carried from token to token, that each
token first decays, then corrects along its key towards its value, then reads with its query.

    q, k = Wq u, Wk u  (kv_heads x key_dim),  v = Wv u  (heads x value_dim);  no biases
    each of q, k, v <- silu(conv(.)): causal, per channel, ``conv`` taps, the last tap on the
    current token, zeros before the start, no bias
    q, k <- x / sqrt(sum(x^2) + 1e-6) per head;  q <- q * key_dim^(-1/2)
    beta = sigmoid(Wb u) per head
    decay per head (``decay="head"``):       g = exp(-exp(A_log_h) softplus(Wa u + dt_bias))
    decay per key channel (``"channel"``):   g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 u) + dt_bias)),
                                             heads x key_dim, on the state's rows
    per head h (q, k of head floor(h / (heads / kv_heads))), S of key_dim x value_dim from zero:
        S <- diag(g) S;  w = beta (v - S^T k);  S <- S + k w^T;  o = S^T q
    o <- o / sqrt(mean(o^2) + eps) per head, times a weight [value_dim] shared by the heads, times
    the output gate: silu(Wg u) (``gate="silu"``) or sigmoid(Wg2 (Wg1 u)) (``"sigmoid"``,
    low rank), heads x value_dim;  out = Wo o

State per sequence (float32, zeroed when a slot is handed out): S of every head and the last
``conv`` - 1 inputs of the convolutions.  A step may bring any number of tokens per sequence; the
recurrence walks them in order, so the result does not depend on how a sequence is cut.  One packed
product gives q | k | v | beta | decay input | gate input in float32; everything between it and
the output product is float32 in both engines.  Tensor names behind ``prefix + tensor_prefix``:
``q``, ``k``, ``v`` (each with ``.conv``), ``b``, ``A_log``, ``dt_bias``, ``norm``, ``o``, and ``a``,
``g`` or their low-rank pairs ``a1``, ``a2``, ``g1``, ``g2``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CallBinding, Mixer, StateRequest, StepContext
from .linear import Linear
from .sink_attention import project_out

DELTA_STATE = "delta.state"
CONV_STATE = "delta.conv"


class GatedDeltaRule(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "recurrent", "delta_rule", "gemm_simt"] + (
            ["gemm_tc"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, key_dim: int,
                 value_dim: int, conv: int, norm_eps: float, decay: str = "head",
                 gate: str = "silu", decay_rank: int = 0, gate_rank: int = 0,
                 tensor_prefix: str = "mix.", init_std: float = 0.02):
        """``decay_rank`` / ``gate_rank`` > 0: that projection is a pair of matrices through so
        many numbers (``a1``, ``a2`` / ``g1``, ``g2``); 0: one matrix (``a`` / ``g``)."""
        if min(n_heads, n_kv_heads, key_dim, value_dim, conv) < 1:
            raise ValueError("delta rule: every size must be at least 1")
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"delta rule: {n_heads} heads do not divide into {n_kv_heads} "
                             f"query/key heads")
        if decay not in ("head", "channel") or gate not in K.HEAD_GATES:
            raise ValueError("delta rule: decay is 'head' or 'channel', gate 'silu' or 'sigmoid'")
        if conv > 8 or key_dim > 256:
            raise ValueError("delta rule: the kernels take up to 8 taps and keys up to 256 wide")
        if decay_rank < 0 or gate_rank < 0:
            raise ValueError("delta rule: a rank cannot be negative")
        self.hidden_size = int(hidden_size)
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)
        self.key_dim, self.value_dim = int(key_dim), int(value_dim)
        self.conv = int(conv)
        self.norm_eps = float(norm_eps)
        self.decay, self.gate = decay, gate
        self.decay_rank, self.gate_rank = int(decay_rank), int(gate_rank)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.qk_width = self.n_kv_heads * self.key_dim
        self.v_width = self.n_heads * self.value_dim
        self.channels = 2 * self.qk_width + self.v_width
        self.n_decay = self.n_heads * (self.key_dim if decay == "channel" else 1)
        self.in_proj: Optional[Linear] = None
        self.decay_up: Optional[torch.Tensor] = None       # a2, if the decay's projection is a pair
        self.gate_up: Optional[torch.Tensor] = None        # g2
        self.out: Optional[Linear] = None
        self.conv_w: Optional[torch.Tensor] = None         # [channels, taps]: q | k | v
        self.w: Dict[str, torch.Tensor] = {}

    # ---- the packed projection's columns --------------------------------------------------
    def _segments(self):
        """(name of the tensor, rows) in the order of the packed projection."""
        a = ("a1", self.decay_rank) if self.decay_rank else ("a", self.n_decay)
        g = ("g1", self.gate_rank) if self.gate_rank else ("g", self.v_width)
        return [("q", self.qk_width), ("k", self.qk_width), ("v", self.v_width),
                ("b", self.n_heads), a, g]

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{p}{n}", (rows, self.hidden_size), MATRIX, init)
                 for n, rows in self._segments()]
        if self.decay_rank:
            specs.append(TensorSpec(f"{p}a2", (self.n_decay, self.decay_rank), MATRIX, init))
        if self.gate_rank:
            specs.append(TensorSpec(f"{p}g2", (self.v_width, self.gate_rank), MATRIX, init))
        # small per-channel and per-head tensors are held in float32 (role VECTOR)
        specs += [TensorSpec(f"{p}q.conv", (self.qk_width, self.conv), VECTOR, Init(0.0, 0.3)),
                  TensorSpec(f"{p}k.conv", (self.qk_width, self.conv), VECTOR, Init(0.0, 0.3)),
                  TensorSpec(f"{p}v.conv", (self.v_width, self.conv), VECTOR, Init(0.0, 0.3)),
                  TensorSpec(f"{p}A_log", (self.n_heads,), VECTOR, Init(0.0, 0.5)),
                  TensorSpec(f"{p}dt_bias", (self.n_decay,), VECTOR, Init(-1.0, 0.5)),
                  TensorSpec(f"{p}norm", (self.value_dim,), VECTOR, Init(1.0, 0.0)),
                  TensorSpec(f"{p}o", (self.hidden_size, self.v_width), MATRIX, init)]
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        parts = [weights[f"{p}{n}"] for n, _ in self._segments()]
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        self.in_proj = Linear(torch.cat(parts, dim=0).contiguous())
        self.decay_up = weights[f"{p}a2"] if self.decay_rank else None
        self.gate_up = weights[f"{p}g2"] if self.gate_rank else None
        self.out = Linear(weights[f"{p}o"])
        self.conv_w = torch.cat([weights[f"{p}{n}.conv"] for n in "qkv"], dim=0).contiguous()
        self.w = {n: weights[f"{p}{n}"] for n in ("A_log", "dt_bias", "norm")}
        self.accepts_row_scale = self.in_proj.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        out, at = {}, 0
        for n, rows in self._segments():
            out[f"{p}{n}"] = self.in_proj.weight[at:at + rows]
            at += rows
        if self.decay_rank:
            out[f"{p}a2"] = self.decay_up
        if self.gate_rank:
            out[f"{p}g2"] = self.gate_up
        qk = self.qk_width
        out[f"{p}q.conv"], out[f"{p}k.conv"] = self.conv_w[:qk], self.conv_w[qk:2 * qk]
        out[f"{p}v.conv"] = self.conv_w[2 * qk:]
        out.update({f"{p}{n}": t for n, t in self.w.items()})
        out[f"{p}o"] = self.out.weight
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def state_request(self) -> Sequence[StateRequest]:
        # a column of S (one value channel, all key channels) is contiguous: a thread of the
        # recurrence's kernel keeps a stretch of it in registers
        req = [StateRequest(DELTA_STATE, (self.n_heads, self.value_dim, self.key_dim), torch.float32)]
        if self.conv > 1:
            req.append(StateRequest(CONV_STATE, (self.channels, self.conv - 1), torch.float32))
        return tuple(req)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n, dev = x.shape[0], x.device
        qk, vw, nh = self.qk_width, self.v_width, self.n_heads
        proj = self.in_proj.forward(x, torch.float32, row_scale=ctx.input_scale)
        conv_state = binding.state.get(CONV_STATE)
        if conv_state is None:
            conv_state = torch.empty((1, self.channels, 0), dtype=torch.float32, device=dev)
        u = torch.empty((n, self.channels), dtype=torch.float32, device=dev)
        K.conv_silu(proj, 0, self.channels, self.conv_w, None, conv_state, ctx.token_row,
                    ctx.cu_seqlens, ctx.slots, u, ctx.n_rows, single=ctx.single_token)
        beta_off = self.channels
        a_off = beta_off + nh
        g_off = a_off + (self.decay_rank or self.n_decay)
        decay, decay_off = proj, a_off
        if self.decay_rank:
            decay = torch.empty((n, self.n_decay), dtype=torch.float32, device=dev)
            K.gemm_simt(proj[:, a_off:a_off + self.decay_rank], self.decay_up, None, decay)
            decay_off = 0
        gate, gate_off = proj, g_off
        if self.gate_rank:
            gate = torch.empty((n, vw), dtype=torch.float32, device=dev)
            K.gemm_simt(proj[:, g_off:g_off + self.gate_rank], self.gate_up, None, gate)
            gate_off = 0
        o = torch.empty((n, vw), dtype=torch.float32, device=dev)
        K.delta_scan(u, 0, qk, 2 * qk, proj, beta_off, decay, decay_off, self.w["dt_bias"],
                     self.w["A_log"], binding.state[DELTA_STATE], ctx.cu_seqlens, ctx.slots, o,
                     ctx.n_rows, ctx.max_row_tokens, nh, self.n_kv_heads, self.key_dim,
                     self.value_dim, self.decay == "channel")
        gated = torch.empty((n, vw), dtype=ctx.act_dtype, device=dev)
        K.head_norm_gate(o, gate, gate_off, self.w["norm"], gated, nh, self.value_dim,
                         self.norm_eps, self.gate)
        project_out(self.out, gated, ctx, residual)
