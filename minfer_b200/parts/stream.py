"""Parts of role "model" that work on the residual stream or the logits around the blocks:

``EmbeddingNorm``    an RMS norm of the embedding rows as they enter the residual stream
``LogitSoftcap``     logits <- cap * tanh(logits / cap)
``PassInjection``    what a pass of a layer loop adds to the residual stream right before its first
                     layer: the embedding output (every pass but the first) and a learned vector
                     per pass, the rows of a table [passes, width]
``DepthAverage``     what goes on after entry i of the run order is a learned mix of the embedding
                     output and the results of entries 0 .. i: sum_j c_i[j] X_j
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import ModelPart, StepContext


class EmbeddingNorm(ModelPart):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, width: int, eps: float, tensor_name: str = "embed.norm"):
        self.width = int(width)
        self.eps = float(eps)
        self.tensor_name = tensor_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.tensor_name}", (self.width,), VECTOR, Init(1.0, 0.0))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.weight = weights[f"{prefix}{self.tensor_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.tensor_name}": self.weight}

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = torch.empty_like(x)
        K.rmsnorm(x, self.weight, self.eps, out)
        return out

    def forward_inplace(self, x: torch.Tensor, ctx: StepContext) -> None:
        x.copy_(self.forward(x, ctx))


class LogitSoftcap(ModelPart):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, cap: float):
        if not cap > 0.0:
            raise ValueError(f"a soft cap must be positive, got {cap}")
        self.cap = float(cap)

    def forward_inplace(self, x: torch.Tensor, ctx: StepContext) -> None:
        K.tanh_cap(x, self.cap)


class PassInjection(ModelPart):
    """``add(h, ctx, pass_index, embedding_output)``: h += embedding_output (pass_index > 0, if
    ``add_embedding``) + table[pass_index]."""

    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, width: int, passes: int, tensor_name: str = "loop.step",
                 add_embedding: bool = True, init_std: float = 0.02):
        self.width = int(width)
        self.passes = int(passes)
        self.tensor_name = tensor_name
        self.add_embedding = bool(add_embedding)
        self.init_std = float(init_std)
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.tensor_name}", (self.passes, self.width), MATRIX,
                           Init(0.0, self.init_std))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.table = weights[f"{prefix}{self.tensor_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.tensor_name}": self.table}

    def needs_embedding(self) -> bool:
        return self.add_embedding and self.passes > 1

    def add(self, h: torch.Tensor, ctx: StepContext, pass_index: int,
            embedding_output: Optional[torch.Tensor]) -> None:
        if not 0 <= pass_index < self.passes:
            raise K.KernelError(f"pass {pass_index} is outside the table of {self.passes} passes")
        other = embedding_output if (self.add_embedding and pass_index > 0) else None
        K.add_stream(h, other, self.table[pass_index])


class DepthAverage(ModelPart):
    """With X_0 the embedding output and X_(i+1) what entry i of the run order leaves (its input
    plus its mixer's and feed-forward's outputs), the stream that goes on to entry i + 1 (after
    the last one: to the final norm) is sum_{j <= i+1} c_i[j] X_j.  ``names[i]`` is the tensor of
    c_i, i + 2 numbers, held in float32.

    The engine keeps the X_j of a step side by side (``begin``), lets entry i work in place on the
    slot the mix before it was written to (so X_(i+1) lies where it belongs without a copy), and
    calls ``mix`` after the entry; after the last one only the wanted rows may be left, which
    ``rows`` then names in the kept streams."""

    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, width: int, names: List[str], init_std: float = 0.0):
        self.width = int(width)
        self.names = list(names)
        self.init_std = float(init_std)
        self.weights: List[torch.Tensor] = []

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        # by default every entry hands on its own result unchanged: c_i = (0, .., 0, 1)
        return [TensorSpec(f"{prefix}{name}", (i + 2,), VECTOR, Init(1.0 / (i + 2), self.init_std))
                for i, name in enumerate(self.names)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.weights = [weights[f"{prefix}{name}"] for name in self.names]
        self._one = torch.ones(1, dtype=torch.float32, device=self.weights[0].device)

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{name}": w for name, w in zip(self.names, self.weights)}

    def begin(self, h: torch.Tensor, ctx: StepContext) -> tuple:
        """Takes the embedding output; returns (the kept streams [entries + 1, tokens, width],
        the stream entry 0 works on)."""
        n = len(self.names)
        history = torch.empty((n + 1, h.shape[0], self.width), dtype=torch.float32, device=h.device)
        K.depth_mix(history, 0, None, h, self._one, history[0])
        if n > 0:
            K.depth_mix(history, 0, None, h, self._one, history[1])
        return history, history[1] if n > 0 else history[0]

    def mix(self, history: torch.Tensor, index: int, last: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """After entry ``index``: ``last`` is X_(index+1) (all rows: slot index + 1 of ``history``;
        or only the rows ``rows`` of the step).  Returns the stream that goes on."""
        if index + 2 < history.shape[0] and rows is None:
            out = history[index + 2]
        else:
            out = torch.empty_like(last)
        K.depth_mix(history, index + 1, rows, last, self.weights[index], out)
        return out
