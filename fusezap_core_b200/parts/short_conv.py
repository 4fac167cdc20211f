"""A short causal convolution over time, per channel, with the inputs it still needs kept as per-request state.

`y_t = sum_j w[:, j] * h_(t - taps + 1 + j)`, j = 0 .. taps-1, with zeros before the sequence's start (so `w[:, taps-1]`
multiplies the token's own input). A step may bring any portion of a sequence: the last `taps - 1` inputs of the
sequence so far live in a state slot `(taps - 1, size)` (oldest first, zero when the request gets its slot), are read
for the first rows of the portion and replaced by the portion's last inputs afterwards. The sum is in 32-bit, taps in
rising j, and rounded once.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import Part


class ShortConv(Part):
    def __init__(self, size: int, taps: int, name: str = "weight", residual: bool = True, activation: str | None = None,
                 bias: str | None = None):
        """residual: the result is `h + conv(h)` (what a block hands on in place of h); False: `conv(h)` alone.
        activation: None, or "silu" (`z * sigmoid(z)` of the 32-bit sum, before the one rounding). bias: the name (after
        the weight's) of a bias per channel, added to the 32-bit sum after the taps; None: the convolution has none."""
        if activation not in (None, "silu"):
            raise ValueError(f"activation {activation!r} is not one of None, 'silu'")
        self.activation = activation
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.size, self.taps, self.name, self.residual = size, int(taps), name, bool(residual)
        self.bias_name = None if bias is None else (f"{name}.{bias}" if name else bias)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def tensors(self) -> dict[str, ParamSpec]:
        out = {self.name: ParamSpec((self.size, self.taps))}
        if self.bias_name is not None:
            out[self.bias_name] = ParamSpec((self.size,), role="vector")
        return out

    def bind(self, tensors, ops) -> None:
        self.weight = tensors[self.name]
        if self.bias_name is not None:
            self.bias = tensors[self.bias_name].float().contiguous()

    def state_need(self) -> dict:
        return {"conv": (self.taps - 1, self.size)} if self.taps > 1 else {}

    def forward(self, ctx, h: torch.Tensor, state: torch.Tensor | None, tag: str = "conv_out") -> torch.Tensor:
        """h: (N, size) T; state: (slots, taps - 1, size) float32 (None when taps == 1). Returns (N, size) T and leaves
        the state of every portion's request at the portion's end."""
        out = ctx.ws.get(tag, tuple(h.shape), h.dtype)
        if self.bias is not None:
            ctx.ops.short_conv(h, self.weight, state, ctx.meta, out, self.residual, self.activation, bias=self.bias)
        elif self.activation is None:
            ctx.ops.short_conv(h, self.weight, state, ctx.meta, out, self.residual)
        else:
            ctx.ops.short_conv(h, self.weight, state, ctx.meta, out, self.residual, self.activation)
        return out
