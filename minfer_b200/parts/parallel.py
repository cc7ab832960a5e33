"""Two mixers side by side on the same input: out = left_scale * left(x) + right_scale * right(x).

Each side is any registered mixer that takes an ``out_scale`` (the constant it multiplies the
operand of its last product with), so both sides add their scaled outputs into the same stream
and no kernel of this part's own runs.  At most one side may keep cached keys; the per-sequence
state of the two sides is kept side by side under the names ``left.<name>`` / ``right.<name>``.
Tensor names: the sides' own, behind ``prefix + tensor_prefix + "left." / "right."``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config.base import PartSpec
from .base import CacheRequest, CallBinding, Mixer, StateRequest, StepContext, settle_pending


class ParallelMixer(Mixer):
    stores_fresh_output = True     # answers ``ctx.extras["fresh_output"]`` (see ``project_out``)

    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0, tensor_prefix: str = "mix."):
        from ..registry import build_part
        self.tensor_prefix = tensor_prefix
        self.sides = []
        for name, spec, scale in (("left", left, left_scale), ("right", right, right_scale)):
            part = build_part("mixer", spec.with_params(out_scale=float(scale),
                                                        tensor_prefix=f"{tensor_prefix}{name}."))
            if not hasattr(part, "out_scale"):
                raise ValueError(f"the {name} mixer ({spec.kind}) takes no output scale")
            self.sides.append((name, part))
        if sum(1 for _, p in self.sides if p.cache_request() is not None) > 1:
            raise ValueError("only one side of a parallel mixer may keep cached keys")
        self.capturable = all(getattr(p, "capturable", False) for _, p in self.sides)

    def libraries(self, dtype: torch.dtype) -> List[str]:
        libs: List[str] = []
        for _, part in self.sides:
            libs += [n for n in part.libraries(dtype) if n not in libs]
        return libs

    def tensor_specs(self, prefix: str):
        return [s for _, part in self.sides for s in part.tensor_specs(prefix)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        for _, part in self.sides:
            part.load(prefix, weights)

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for _, part in self.sides:
            out.update(part.export(prefix))
        return out

    def cache_request(self) -> Optional[CacheRequest]:
        for _, part in self.sides:
            req = part.cache_request()
            if req is not None:
                return req
        return None

    def state_request(self) -> Sequence[StateRequest]:
        return tuple(StateRequest(f"{name}.{r.name}", r.shape, r.dtype)
                     for name, part in self.sides for r in part.state_request())

    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        ctx.extras.pop("prepare_for", None)        # neither side's product completes the stream alone
        fresh = ctx.extras.pop("fresh_output", False)
        for i, (name, part) in enumerate(self.sides):
            if fresh and i == 0:
                ctx.extras["fresh_output"] = True  # the first side stores, the second adds
            own = {k[len(name) + 1:]: t for k, t in binding.state.items() if k.startswith(name + ".")}
            side = CallBinding(cache=binding.cache if part.cache_request() is not None else None,
                               writes_cache=binding.writes_cache, entry=binding.entry,
                               has_readers=binding.has_readers, state=own)
            part.forward_add(x, ctx, side, residual)
            if i == 0:
                # never two pending products at once; K splits of a first side that stored nothing
                # become the buffer's content
                pending = ctx.extras.pop("pending", None)
                if pending is not None:
                    from ..kernels import api as K
                    K.splitk_reduce(pending.partial, pending.bias, residual,
                                    accumulate=not ctx.extras.pop("pending_only", False))
