"""RMSNorm with the residual add folded in.

`x <- x + delta` (the pending term of the previous sublayer), then `h = w * (x / sqrt(mean(x^2) + eps))`
(fusezap/serve/models/llama.py:500-503, 508-523: `mean = sum * (1/D)`, the fused kernel also writes the residual
stream). The residual stream x is float32 in both dtypes; the sum of squares, the scale and the weight product are
computed in 32-bit and h is rounded once to the activation dtype. With `groups` > 1 the vector is normed in that many
equal consecutive parts, each by its own mean square; the weight still spans the whole vector. With `offset` the
multiplier is `offset + w` (a weight stored as its distance from one has offset 1), added in float32 once at load.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, groups: int = 1, name: str = "weight", scalar: bool = False,
                 offset: float = 0.0):
        """groups: the vector is split into this many equal consecutive parts and each is divided by its own root mean
        square (1: the whole vector). name: the weight's tensor name relative to the part ("" when the part's prefix is
        the whole name). scalar: the weight is one number for all coordinates (a tensor without dimensions). offset: the
        row is multiplied by `offset + weight` (random weights are then drawn around zero)."""
        if groups <= 0 or size % groups:
            raise ValueError(f"a norm over {size} values cannot be split into {groups} equal groups")
        self.size, self.eps, self.groups, self.name, self.scalar = size, float(eps), int(groups), name, bool(scalar)
        self.offset = float(offset)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec(() if self.scalar else (self.size,), role="vector", init="normal" if self.offset else "ones")}

    def bind(self, tensors, ops) -> None:
        self.weight = tensors[self.name]
        if self.offset:
            self.weight = (self.weight.float() + self.offset).contiguous()
        if self.scalar:      # the kernels take a weight per coordinate
            self.weight = self.weight.float().reshape(1).expand(self.size).contiguous()

    def forward(self, ctx, x, delta, rows=None, n_rows=None):
        n = x.shape[0] if rows is None else (n_rows if n_rows is not None else rows.shape[0])
        h = ctx.ws.get("norm_h" if rows is None else "norm_h_rows", (n, self.size), ctx.ops.dtype)
        self._run(ctx, x, delta, h, rows)
        return h

    def forward_into(self, ctx, x, h) -> None:
        """h = norm(x), into a buffer of the caller's (a second norm of the same x needs one of its own)."""
        self._run(ctx, x, None, h, None)

    def _run(self, ctx, x, delta, h, rows) -> None:
        if hasattr(delta, "fold_into_norm"):       # a pending operation on the stream that this norm can take in its pass
            if self.groups == 1 and delta.fold_into_norm(ctx, x, self.weight, self.eps, h, rows):
                return
            if rows is not None:
                raise NotImplementedError("a pending operation on the stream cannot be resolved for selected rows only")
            delta = delta.resolve(ctx, x)
        if self.groups == 1:
            ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, h, rows)
        else:
            ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, h, rows, groups=self.groups)
