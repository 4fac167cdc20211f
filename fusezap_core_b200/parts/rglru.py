"""Real-gated linear recurrent unit: a recurrent mixer with one 32-bit number of state per channel.

Two branches of `width` channels read the input h:

    y = gelu_tanh(W_y h + b_y)
    u = conv(W_x h + b_x)            a short causal convolution per channel (`taps` wide, with a bias, no activation)

u is cut into `blocks` equal parts; in part b, with square matrices per part,

    r = sigmoid(W_ra[b] u_b + b_ra[b])        the recurrence gate
    i = sigmoid(W_ri[b] u_b + b_ri[b])        the input gate
    a = exp(-sharpness * r * softplus(lam))   per channel, in (0, 1)
    S <- a * S + sqrt(1 - a^2) * (i * u)      from S = 0 at a request's start, the first token like every other

and the result is `W_o (S * y)`. S (float32, zero when a request gets its slot) and the convolution's last `taps - 1`
inputs are request state. Gates, softplus, exponentials, the square root and the recurrence are 32-bit in both dtypes;
the two input products, the convolution and the gelu run in the activation dtype with 32-bit sums, the gates' products
read u in the activation dtype and leave float32.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer
from .short_conv import ShortConv

_NAMES = {"gate_branch": "y_proj", "in": "x_proj", "conv": "conv", "recur_gate": "a_gate", "input_gate": "i_gate",
          "decay": "a_param", "out": "o_proj", "bias": "bias"}


@register_mixer("rglru")
class RGLRU(Mixer):
    def __init__(self, hidden_size: int, width: int, blocks: int, taps: int, sharpness: float = 8.0,
                 names: dict | None = None):
        if width <= 0 or blocks <= 0 or width % blocks:
            raise ValueError(f"{width} channels cannot be cut into {blocks} equal parts")
        self.D, self.W, self.B, self.sharpness = hidden_size, int(width), int(blocks), float(sharpness)
        self.names = {**_NAMES, **(names or {})}
        self.conv = ShortConv(self.W, taps, name="", residual=False, bias=self.names["bias"])
        self.w_in = self.b_in = self.w_gates = self.b_gates = self.lam = self.wo = None

    def children(self):
        return ((self.names["conv"], self.conv),)

    def tensors(self) -> dict[str, ParamSpec]:
        n, D, W, B = self.names, self.D, self.W, self.B
        bw = W // B
        b = "." + n["bias"]
        out = {n["gate_branch"]: ParamSpec((W, D)), n["gate_branch"] + b: ParamSpec((W,), role="vector"),
               n["in"]: ParamSpec((W, D)), n["in"] + b: ParamSpec((W,), role="vector")}
        out.update({(f"{n['conv']}.{k}" if k else n["conv"]): v for k, v in self.conv.tensors().items()})
        out.update({n["recur_gate"]: ParamSpec((B, bw, bw)), n["recur_gate"] + b: ParamSpec((B, bw), role="vector"),
                    n["input_gate"]: ParamSpec((B, bw, bw)), n["input_gate"] + b: ParamSpec((B, bw), role="vector"),
                    n["decay"]: ParamSpec((W,), role="vector"), n["out"]: ParamSpec((D, W))})
        return out

    def bind(self, tensors, ops) -> None:
        n = self.names
        b = "." + n["bias"]
        # one product for both branches: columns [y | x]
        self.w_in = torch.cat([tensors[n["gate_branch"]], tensors[n["in"]]], 0).contiguous()
        self.b_in = torch.cat([tensors[n["gate_branch"] + b].float(), tensors[n["in"] + b].float()], 0).contiguous()
        pre = n["conv"]
        self.conv.bind({k[len(pre) + 1:]: v for k, v in tensors.items() if k == pre or k.startswith(pre + ".")}, ops)
        # one product per part for both gates: rows [recurrence gate | input gate] of part b
        self.w_gates = torch.cat([tensors[n["recur_gate"]], tensors[n["input_gate"]]], 1).contiguous()       # (B, 2 bw, bw)
        self.b_gates = torch.cat([tensors[n["recur_gate"] + b].float(), tensors[n["input_gate"] + b].float()], 1).contiguous()
        self.lam = tensors[n["decay"]].float().contiguous()
        self.wo = tensors[n["out"]]

    def state_need(self) -> dict:
        return {"S": (self.W,), **self.conv.state_need()}

    def step_needs(self) -> tuple[str, ...]:
        return ("portions",)      # the scan is launched differently for long portions: the longest is part of a step's shape

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        W, B = self.W, self.B
        yx = ws.get("rglru_in", (n, 2 * W), torch.float32)
        ops.linear(h, self.w_in, self.b_in, yx)
        y = ws.get("rglru_y", (n, W), ops.dtype)
        ops.activate(yx, 0, "gelu_tanh", y)
        x = ws.get("rglru_x", (n, W), ops.dtype)
        ops.activate(yx, W, "identity", x)                                  # the convolution's input, rounded once
        u = self.conv.forward(ctx, x, cache.state.get("conv"), tag="rglru_u")
        gates = ws.get("rglru_gates", (n, B, 2 * (W // B)), torch.float32)
        ops.linear_heads(u.view(n, B, W // B), 0, W // B, self.w_gates, gates, 0)
        o = ws.get("rglru_o", (n, W), ops.dtype)
        ops.rglru_scan(u, gates, self.b_gates, self.lam, y, self.sharpness, cache.state["S"], ctx.meta, o)
        delta = ws.get("rglru_delta", (n, self.D), torch.float32)
        ops.linear(o, self.wo, None, delta)
        return delta
