"""Attention whose heads talk before the softmax, as a mixer: the scores of all heads for a
(query, key) pair are mixed by a learned matrix, so no head's softmax can be taken alone.

    q, k, v = Wq u, Wk u, Wv u   (heads x head_dim, kv_heads x head_dim, kv_heads x value_dim; no
                                  biases; no rotation: positions enter through the mask only)
    s^g_ij = (q^g_i . k_j) * scale;   s'^h_ij = sum_g T[h][g] s^g_ij        (``talk``: T [heads, heads])
    j visible from i iff 0 <= i - j < window (``window`` 0: every j <= i);  softmax over the visible
    values blended across layers (``value_mix``): the first such layer of a model is the "source",
    every later one is a "blend": v <- (1 - lam) v + lam v_source with v_source the source layer's
    values of the same token and lam a learned number; the blended v is what the cache keeps
    head h's output times sigmoid(Wg u)_h, one number per head          (``gate``)
    out = Wo concat_h(..)

One packed product gives q | k | v | gate in float32; the blend runs on those rows; one kernel
writes the step's q, k, v and the cache's pages; the attention kernel takes all heads of a query
together, over the step's own keys for whole prompts and over the cache otherwise.  Scores, their
mix and the softmax are float32 in both engines.  Tensor names behind ``prefix + tensor_prefix``:
``q``, ``k``, ``v``, ``o``, ``talk``, ``g``, ``vmix`` (a scalar; present in a source layer too, unused).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CacheRequest, CallBinding, Mixer, StepContext
from .linear import Linear
from .sink_attention import project_out

VALUE_SOURCE = "value_mix.source"      # in ``StepContext.extras``: (projection rows, column of v)
VALUE_MIXES = ("none", "source", "blend")


class TalkingAttention(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "mixer_prep", "attention_talk",
                "gemm_tc" if dtype == torch.bfloat16 else "gemm_simt"]

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, window: int = 0, talk: bool = True,
                 gate: bool = True, value_mix: str = "none", tensor_prefix: str = "mix.",
                 init_std: float = 0.02):
        if n_kv_heads < 1 or n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} heads do not divide into {n_kv_heads} key/value heads")
        if head_dim < 1 or value_dim < 1 or window < 0:
            raise ValueError("talking attention: sizes must be positive, the window not negative")
        if value_mix not in VALUE_MIXES:
            raise ValueError(f"value_mix is one of {VALUE_MIXES}, got {value_mix!r}")
        if n_heads * value_dim > 32 * 128:
            raise ValueError("talking attention: the kernel takes up to 4096 output values a token")
        self.hidden_size = int(hidden_size)
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale = float(scale)
        self.window = int(window)
        self.talk = bool(talk)
        self.gate = bool(gate)
        self.value_mix = value_mix
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.talk_w: Optional[torch.Tensor] = None
        self.lam: Optional[torch.Tensor] = None

    def _widths(self):
        return (self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim,
                self.n_kv_heads * self.value_dim, self.n_heads if self.gate else 0)

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nk, nv, ng = self._widths()
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{p}q", (nq, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}k", (nk, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}v", (nv, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}o", (self.hidden_size, self.n_heads * self.value_dim), MATRIX, init)]
        if self.talk:
            # scores, their mix and the softmax are 32-bit: the matrix is held in float32
            specs.append(TensorSpec(f"{p}talk", (self.n_heads, self.n_heads), VECTOR, Init(0.0, 0.5)))
        if self.gate:
            specs.append(TensorSpec(f"{p}g", (ng, self.hidden_size), MATRIX, init))
        if self.value_mix != "none":
            specs.append(TensorSpec(f"{p}vmix", (), VECTOR, Init(0.5, 0.1)))
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        parts = [weights[f"{p}{n}"] for n in "qkv"] + ([weights[f"{p}g"]] if self.gate else [])
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        self.proj = Linear(torch.cat(parts, dim=0).contiguous())
        self.out = Linear(weights[f"{p}o"])
        if self.talk:
            self.talk_w = weights[f"{p}talk"]
        else:
            self.talk_w = torch.eye(self.n_heads, dtype=torch.float32, device=self.out.weight.device)
        self.lam = weights[f"{p}vmix"] if self.value_mix != "none" else None
        self.accepts_row_scale = self.proj.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, nk, nv, _ = self._widths()
        w = self.proj.weight
        out = {f"{p}q": w[:nq], f"{p}k": w[nq:nq + nk], f"{p}v": w[nq + nk:nq + nk + nv],
               f"{p}o": self.out.weight}
        if self.talk:
            out[f"{p}talk"] = self.talk_w
        if self.gate:
            out[f"{p}g"] = w[nq + nk + nv:]
        if self.value_mix != "none":
            out[f"{p}vmix"] = self.lam
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(self.n_kv_heads, self.head_dim, self.window,
                            self.value_dim if self.value_dim != self.head_dim else 0)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n = x.shape[0]
        nh, nk, hd, vd = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        nq, nkw, nv, _ = self._widths()
        dev, act = x.device, ctx.act_dtype
        cache = binding.cache
        if cache is None:
            raise K.KernelError("the attention mixer was given no cache entry")
        if cache.k.dtype != act:
            raise K.KernelError("the cache and the activations must share one dtype")
        if not binding.writes_cache:
            raise K.KernelError("talking attention writes its own keys and values")
        proj = self.proj.forward(x, torch.float32, row_scale=ctx.input_scale)
        v_off = nq + nkw
        if self.value_mix == "source":
            ctx.extras[VALUE_SOURCE] = (proj, v_off, nv)
        elif self.value_mix == "blend":
            source = ctx.extras.get(VALUE_SOURCE)
            if source is None:
                raise K.KernelError("a layer blends values, but no layer before it gave its own")
            first, first_off, first_width = source
            if first_width != nv:
                raise K.KernelError(f"values of width {nv} cannot be blended with values of width "
                                    f"{first_width}")
            K.value_mix(proj, v_off, first, first_off, self.lam, nv)
        q = torch.empty((n, nh, hd), dtype=act, device=dev)
        own_kv = ctx.from_start
        k_step = v_step = None
        if own_kv:
            k_step = torch.empty((n, nk, hd), dtype=act, device=dev)
            v_step = torch.empty((n, nk, vd), dtype=act, device=dev)
        K.qk_prepare(proj, ctx.positions, ctx.token_row, ctx.seq_end, q, k_step, v_step,
                     cache.k, cache.v, cache.page_table, cache.table_stride, cache.ring,
                     q_off=0, n_heads=nh, q_width=hd, k_off=nq, n_kv=nk, k_width=hd,
                     v_off=v_off, v_width=vd, v_from_k=False, q_norm=None, k_norm=None, eps=0.0,
                     inv_freq=None, rot_dims=0, rot_style=0, rot_magnitude=1.0, q_rot_off=0,
                     k_rot_off=0, status=ctx.status)
        o = torch.empty((n, nh * vd), dtype=act, device=dev)
        gate = proj if self.gate else None
        gate_off = v_off + nv
        if own_kv:
            K.talk_attention(q, k_step, v_step, ctx.token_row, ctx.positions, ctx.cu_seqlens, None,
                             0, 0, self.talk_w, gate, gate_off, o, nh, nk, hd, vd, self.window,
                             self.scale, q_cu_seqlens=ctx.cu_seqlens, n_seq=ctx.n_rows,
                             max_row_tokens=ctx.max_row_tokens)
        else:
            if cache.ring and ctx.max_row_tokens > cache.ring - self.window + 1:
                raise K.KernelError(
                    f"a sequence brings {ctx.max_row_tokens} tokens, but a ring of {cache.ring} "
                    f"positions with a window of {self.window} takes "
                    f"{cache.ring - self.window + 1} a step (the engine runs longer rows in portions)")
            reach = min(self.window, ctx.max_end) if self.window > 0 else ctx.max_end
            K.talk_attention(q, cache.k, cache.v, ctx.token_row, ctx.positions, None,
                             cache.page_table, cache.table_stride, cache.ring, self.talk_w, gate,
                             gate_off, o, nh, nk, hd, vd, self.window, self.scale, reach_keys=reach,
                             q_cu_seqlens=ctx.cu_seqlens, n_seq=ctx.n_rows,
                             max_row_tokens=ctx.max_row_tokens)
        project_out(self.out, o, ctx, residual)
