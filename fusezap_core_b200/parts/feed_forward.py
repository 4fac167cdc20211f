"""Gated feed-forward: `down(act(gate(h)) * up(h))`, act = silu (SwiGLU) or the tanh form of gelu.

One product with the rows [gate; up] stacked at load (fusezap/serve/models/llama.py:327, 746-749), `silu(g) = g / (1 +
exp(-g))` in 32-bit (fusezap/serve/cuda.py:284-303), then the down product (llama.py:752), whose result is the residual
term. Optional biases are taken when the checkpoint has them (gate and up together; down). Where the kernel table has
a fused kernel, the gate/up product and the activation run as one launch and the (N, 2 I) intermediate never exists.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import FeedForward, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int,
                 names: tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj"), suffix: str = ".weight",
                 activation: str = "silu"):
        """suffix: what follows a matrix's name in the checkpoint ("" where the name alone is the tensor). activation:
        what the gate passes through, "silu" or "gelu_tanh" (`0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))`)."""
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"activation {activation!r} is not one of 'silu', 'gelu_tanh'")
        self.D, self.I, self.names, self.suffix, self.activation = hidden_size, intermediate_size, tuple(names), suffix, activation
        self.wgu = self.bgu = self.wd = self.bd = self.packed = None

    def tensors(self) -> dict[str, ParamSpec]:
        g, u, d = self.names
        sx = self.suffix
        return {
            f"{g}{sx}": ParamSpec((self.I, self.D)), f"{u}{sx}": ParamSpec((self.I, self.D)),
            f"{d}{sx}": ParamSpec((self.D, self.I)),
            f"{g}.bias": ParamSpec((self.I,), role="vector", group="gate_up_bias"),
            f"{u}.bias": ParamSpec((self.I,), role="vector", group="gate_up_bias"),
            f"{d}.bias": ParamSpec((self.D,), role="vector", group="down_bias"),
        }

    def bind(self, tensors, ops) -> None:
        g, u, d = self.names
        sx = self.suffix
        # the kernel table may want gate and up in a layout of its own for a fused product + activation
        self.packed = ops.pack_gate_up(tensors[f"{g}{sx}"], tensors[f"{u}{sx}"], tensors.get(f"{g}.bias"),
                                       tensors.get(f"{u}.bias"))
        if self.packed is None:
            self.wgu = torch.cat([tensors[f"{g}{sx}"], tensors[f"{u}{sx}"]], 0).contiguous()
            if f"{g}.bias" in tensors:
                self.bgu = torch.cat([tensors[f"{g}.bias"].float(), tensors[f"{u}.bias"].float()], 0).contiguous()
        self.wd = tensors[f"{d}{sx}"]
        self.bd = tensors[f"{d}.bias"].float() if f"{d}.bias" in tensors else None

    def forward(self, ctx, h: torch.Tensor, tag: str = "") -> torch.Tensor:
        """tag: a prefix for the names of its scratch buffers (a feed-forward that runs inside another one)."""
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        a = ws.get(tag + "act", (n, self.I), ops.dtype)
        other = {} if self.activation == "silu" else {"activation": self.activation}
        if self.packed is not None:
            ops.linear_swiglu(h, self.packed, a, **other)
        else:
            gu = ws.get(tag + "gate_up", (n, 2 * self.I), ops.dtype)
            ops.linear(h, self.wgu, self.bgu, gu)
            ops.swiglu(gu, a, **other)
        delta = ws.get(tag + "delta", (n, self.D), torch.float32)
        ops.linear(a, self.wd, self.bd, delta)
        return delta
