"""Pre-norm block with two residual adds: h += mixer(norm1(h)); h += ffn(norm2(h))
(src/models/qwen2/graph.rs:59-64, 137, 154-155, 176).

Two options: a layer without a feed-forward (``LayerSpec.feed_forward`` None: the second half
is left out, norm and all), and a token shift between the first norm and the mixer
(``token_shift``: the parameters of ``parts.shift.TokenShift``), whose per-sequence state the
block asks the cache for beside the mixer's own."""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Sequence

import torch

from ..config.base import LayerSpec
from .base import Block, CallBinding, Part, StateRequest, StepContext, settle_pending


class PreNormBlock(Block):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def __init__(self, layer: LayerSpec, token_shift: Optional[Mapping[str, Any]] = None):
        from ..registry import build_part
        self.prefix = layer.prefix
        self.mixer_norm = build_part("norm", layer.mixer_norm)
        self.mixer = build_part("mixer", layer.mixer)
        self.feed_forward_norm = self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm)
            self.feed_forward = build_part("feed_forward", layer.feed_forward)
        self.shift = None
        if token_shift is not None:
            from .shift import TokenShift
            self.shift = TokenShift(**token_shift)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.shift, self.mixer, self.feed_forward_norm,
                                 self.feed_forward) if p is not None)

    def state_request(self) -> Sequence[StateRequest]:
        own = tuple(self.shift.state_request()) if self.shift is not None else ()
        return tuple(self.mixer.state_request()) + own

    def tensor_specs(self, prefix: str = "") -> List:
        specs = []
        for part in self.parts():
            specs += part.tensor_specs(self.prefix)
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(self.prefix, weights)

    def export(self, prefix: str = "") -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for part in self.parts():
            out.update(part.export(self.prefix))
        return out

    accepts_pending = True     # its norms add a pending projection output while reading h

    def entry_norm(self):
        if self.shift is not None:
            return None            # the shift mixes normed rows: the norm cannot ride on a product
        if self.mixer_norm.foldable() is not None and getattr(self.mixer, "accepts_row_scale", False):
            return self.mixer_norm
        return None

    @staticmethod
    def _normed(norm, h: torch.Tensor, ctx: StepContext, consumer):
        """The norm's output for ``consumer``, as (x, row scale): a prepared input if the product
        before left one for this very norm and the consumer can apply the scale, else the norm
        as a kernel (which also adds a pending projection output into ``h``)."""
        prepared = ctx.extras.pop("prepared", None)
        if (prepared is not None and prepared.norm is norm
                and getattr(consumer, "accepts_row_scale", False)):
            return prepared.x, prepared.scale
        pending = ctx.extras.pop("pending", None)
        if pending is not None:
            return norm.forward_settling(h, pending, ctx.act_dtype), None
        return norm.forward(h, ctx.act_dtype), None

    def _call(self, part, x, scale, ctx, target, *args) -> None:
        ctx.input_scale = scale
        if target is not None and getattr(part, "accepts_row_scale", False):
            ctx.extras["prepare_for"] = target
        try:
            part.forward_add(x, ctx, *args)
        finally:
            ctx.input_scale = None
            ctx.extras.pop("prepare_for", None)

    def mix(self, h: torch.Tensor, ctx: StepContext, binding: CallBinding) -> None:
        if self.shift is not None:
            ctx.extras.pop("prepared", None)
            x, scale = self.shift.norm_and_shift(self.mixer_norm, h, ctx, binding.state), None
        else:
            x, scale = self._normed(self.mixer_norm, h, ctx, self.mixer)
        # the mixer's last product may prepare the input of the norm before the feed-forward,
        # unless the engine drops rows of h between the two
        target = None
        if (self.feed_forward is not None and ctx.extras.get("rows_stay", True)
                and self.feed_forward_norm.foldable() is not None
                and getattr(self.feed_forward, "accepts_row_scale", False)):
            target = self.feed_forward_norm
        self._call(self.mixer, x, scale, ctx, target, binding, h)

    def feed(self, h: torch.Tensor, ctx: StepContext) -> None:
        if self.feed_forward is None:
            return
        x, scale = self._normed(self.feed_forward_norm, h, ctx, self.feed_forward)
        # the feed-forward's last product may prepare the input of the norm that reads h next
        # (the next block's first, or the model's last), which the engine names
        self._call(self.feed_forward, x, scale, ctx, ctx.extras.get("next_norm"), h)


class TokenSide(Part):
    """A per-layer input looked up by token id, added to the stream after the feed-forward:

        e = table[token][offset : offset + dim];   y = Wp (gelu_tanh(Wa x) * e)
        x += mult * y / sqrt(mean(y^2) + eps) * w

    ``table`` ([vocab, layers * dim]) is one tensor of the whole model, named without the layer's
    prefix and shared by every layer's part; ``Wa`` [dim, width], ``Wp`` [width, dim] and the norm
    weight ``w`` are the layer's own."""

    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "gemm_simt"] + (["gemm_tc"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, vocab_size: int, dim: int, offset: int, table_width: int,
                 eps: float, mult: float = 1.0, table_name: str = "side.embed",
                 gate_name: str = "side.gate", proj_name: str = "side.proj",
                 norm_name: str = "side.norm", init_std: float = 0.02):
        if dim < 1 or offset < 0 or offset + dim > table_width:
            raise ValueError(f"columns [{offset}, {offset + dim}) do not lie within a table of {table_width}")
        self.hidden_size, self.vocab_size = int(hidden_size), int(vocab_size)
        self.dim, self.offset, self.table_width = int(dim), int(offset), int(table_width)
        self.eps, self.mult = float(eps), float(mult)
        self.table_name, self.gate_name = table_name, gate_name
        self.proj_name, self.norm_name = proj_name, norm_name
        self.init_std = float(init_std)
        self.table = self.gate = self.proj = self.norm = None

    def tensor_specs(self, prefix: str) -> List:
        from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
        init = Init(0.0, self.init_std)
        return [TensorSpec(self.table_name, (self.vocab_size, self.table_width), MATRIX, init),
                TensorSpec(f"{prefix}{self.gate_name}", (self.dim, self.hidden_size), MATRIX, init),
                TensorSpec(f"{prefix}{self.proj_name}", (self.hidden_size, self.dim), MATRIX, init),
                TensorSpec(f"{prefix}{self.norm_name}", (self.hidden_size,), VECTOR, Init(1.0, 0.0))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        from .linear import Linear
        self.table = weights[self.table_name]
        self.gate = Linear(weights[f"{prefix}{self.gate_name}"])
        self.proj = Linear(weights[f"{prefix}{self.proj_name}"])
        self.norm = weights[f"{prefix}{self.norm_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {self.table_name: self.table, f"{prefix}{self.gate_name}": self.gate.weight,
                f"{prefix}{self.proj_name}": self.proj.weight, f"{prefix}{self.norm_name}": self.norm}

    def add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        """``x``: the stream ``h`` in the activation type; the rows are the step's tokens or, after
        the engine dropped rows, those that ``ctx.extras["kept_rows"]`` names."""
        from ..kernels import api as K
        n = h.shape[0]
        a = self.gate.forward(x, torch.float32)
        g = torch.empty((n, self.dim), dtype=ctx.act_dtype, device=h.device)
        K.table_gate(a, self.table, self.offset, ctx.token_ids, ctx.extras.get("kept_rows"), g, ctx.status)
        y = self.proj.forward(g, torch.float32)
        K.norm_add(h, y, self.norm, self.eps, self.mult, x_out=OutputNormBlock._rounded(h, ctx))


class OutputNormBlock(Block):
    """A block whose norms sit on the sublayers' OUTPUTS, the sublayers reading the stream itself:

        h += mult * norm1(mixer(h));   h += mult * norm2(ffn(h))   (the second half optional)

    followed, with ``side`` (the parameters of ``TokenSide``), by that part's per-token input."""

    capturable = True      # launches kernels only; safe inside a CUDA graph capture
    accepts_pending = False

    def __init__(self, layer: LayerSpec, mult: float = 1.0, side: Optional[Mapping[str, Any]] = None):
        from ..registry import build_part
        self.prefix = layer.prefix
        self.mult = float(mult)
        self.mixer_norm = build_part("norm", layer.mixer_norm)
        self.mixer = build_part("mixer", layer.mixer)
        self.feed_forward_norm = self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm)
            self.feed_forward = build_part("feed_forward", layer.feed_forward)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and norm.foldable() is None:
                raise ValueError("this block adds y / rms(y) * w itself: its norms must be RMS norms")
        self.side = TokenSide(mult=self.mult, **side) if side is not None else None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                 self.feed_forward, self.side) if p is not None)

    tensor_specs = PreNormBlock.tensor_specs
    load = PreNormBlock.load
    export = PreNormBlock.export

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def _input(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """The stream as the sublayers' products take it: the rounded copy the last add into this
        very tensor left (``_rounded``), else a cast."""
        if ctx.act_dtype == torch.float32:
            return h
        left = ctx.extras.pop("rounded_stream", None)
        if left is not None and left[0] is h:
            return left[1]
        from ..kernels import api as K
        x = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
        K.cast(h, x)
        return x

    @staticmethod
    def _rounded(h: torch.Tensor, ctx: StepContext) -> Optional[torch.Tensor]:
        """A place for the stream rounded to the activation type, which the add that completes ``h``
        fills for whoever reads ``h`` next (None in the float32 engine: ``h`` itself is read)."""
        if ctx.act_dtype != torch.bfloat16:
            return None
        x = torch.empty(h.shape, dtype=torch.bfloat16, device=h.device)
        ctx.extras["rounded_stream"] = (h, x)
        return x

    @staticmethod
    def _output_buffer(part, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """The buffer a sublayer adds its output into: zeros, or, for a part whose last product can
        store (``stores_fresh_output``), memory that holds nothing yet."""
        if getattr(part, "stores_fresh_output", False):
            ctx.extras["fresh_output"] = True
            return torch.empty_like(h)
        return torch.zeros_like(h)

    def _add_normed(self, h: torch.Tensor, y: torch.Tensor, norm, ctx: StepContext) -> None:
        """h += mult * norm(y + whatever the sublayer's last product left pending)."""
        from ..kernels import api as K
        weight, eps, _ = norm.foldable()
        ctx.extras.pop("fresh_output", None)
        pending = ctx.extras.pop("pending", None)
        only = ctx.extras.pop("pending_only", False)
        x_out = self._rounded(h, ctx)
        if pending is None:
            K.norm_add(h, y, weight, eps, self.mult, x_out=x_out)
        else:
            K.norm_add(h, None if only else y, weight, eps, self.mult, partial=pending.partial,
                       bias=pending.bias, x_out=x_out)

    def mix(self, h: torch.Tensor, ctx: StepContext, binding: CallBinding) -> None:
        ctx.extras.pop("prepared", None)
        ctx.extras.pop("prepare_for", None)
        ctx.input_scale = None
        y = self._output_buffer(self.mixer, h, ctx)
        self.mixer.forward_add(self._input(h, ctx), ctx, binding, y)
        self._add_normed(h, y, self.mixer_norm, ctx)

    def feed(self, h: torch.Tensor, ctx: StepContext) -> None:
        ctx.extras.pop("prepared", None)
        ctx.extras.pop("prepare_for", None)
        if self.feed_forward is not None:
            y = self._output_buffer(self.feed_forward, h, ctx)
            self.feed_forward.forward_add(self._input(h, ctx), ctx, y)
            self._add_normed(h, y, self.feed_forward_norm, ctx)
        if self.side is not None:
            self.side.add(h, self._input(h, ctx), ctx)
