"""Parallel block with gated sublayers: `x += g1 * mixer(h1') + g2 * ffn(h2)`, both sublayers reading the same x.

`h1 = norm1(x)`, `h2 = norm2(x)`; the mixer reads `h1' = h1 + conv(h1)` when the block has a short convolution
(`taps` >= 1; see `short_conv.ShortConv`; with one tap it is a per-channel scale and keeps no state), else h1; with `gated` each sublayer's result is multiplied element by element by
`sigmoid(W_g h + b_g)` of its own norm's output (before the convolution). A layer without a feed-forward has only the
first term (and neither norm2 nor the second gate). The pending term of the previous layer is added by norm1, in the
same pass over the row; gates, their sigmoid and the sum of the two terms are 32-bit.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import Block, FeedForward, LayerCache, Mixer, register_block
from .short_conv import ShortConv

_NAMES = {"norm1": "norm1", "norm2": "norm2", "mixer": "mixer", "ffn": "ffn", "conv": "conv", "gate1": "gate1",
          "gate2": "gate2", "bias": "bias"}


@register_block("parallel_gated")
class ParallelGatedBlock(Block):
    def __init__(self, mixer: Mixer, ffn: FeedForward | None, make_norm, hidden_size: int, taps: int = 0,
                 gated: bool = True, norms: tuple = (None, None), names: dict | None = None):
        self.mixer, self.ffn, self.D, self.gated = mixer, ffn, hidden_size, bool(gated)
        self.names = {**_NAMES, **(names or {})}
        self.norm1 = make_norm(norms[0]) if norms[0] is not None else make_norm()
        self.norm2 = None
        if ffn is not None:
            self.norm2 = make_norm(norms[1]) if norms[1] is not None else make_norm()
        self.conv = ShortConv(hidden_size, taps, name="") if taps >= 1 else None      # taps 0: no convolution
        self.wg1 = self.bg1 = self.wg2 = self.bg2 = None

    def children(self):
        n = self.names
        out = [(n["norm1"], self.norm1), (n["mixer"], self.mixer)]
        if self.conv is not None:
            out.append((n["conv"], self.conv))
        if self.ffn is not None:
            out += [(n["norm2"], self.norm2), (n["ffn"], self.ffn)]
        return tuple(out)

    def state_need(self) -> dict:
        return {**self.mixer.state_need(), **(self.conv.state_need() if self.conv is not None else {})}

    def tensors(self) -> dict[str, ParamSpec]:
        out = {(f"{prefix}.{k}" if k else prefix): v for prefix, part in self.children() for k, v in part.tensors().items()}
        n, D = self.names, self.D
        if self.gated:
            for g in ("gate1", "gate2") if self.ffn is not None else ("gate1",):
                out[n[g]] = ParamSpec((D, D))
                out[f"{n[g]}.{n['bias']}"] = ParamSpec((D,), role="vector", init="zeros")
        if self.ffn is None:      # what belongs to the absent feed-forward is passed over if a checkpoint carries it
            out[n["norm2"]] = ParamSpec((D,), role="vector", ignore=True)
            out[n["gate2"]] = ParamSpec((D, D), ignore=True)
            out[f"{n['gate2']}.{n['bias']}"] = ParamSpec((D,), role="vector", ignore=True)
        return out

    def bind(self, tensors, ops) -> None:
        for prefix, part in self.children():
            own = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k == prefix or k.startswith(prefix + ".")}
            part.bind(own, ops)
        if self.gated:
            n = self.names
            self.wg1, self.bg1 = tensors[n["gate1"]], tensors[f"{n['gate1']}.{n['bias']}"].float()
            if self.ffn is not None:
                self.wg2, self.bg2 = tensors[n["gate2"]], tensors[f"{n['gate2']}.{n['bias']}"].float()

    def forward(self, ctx, x, delta, cache: LayerCache):
        n, ops, ws = x.shape[0], ctx.ops, ctx.ws
        h1 = self.norm1.forward(ctx, x, delta)                      # x += pending term; h1 = norm1(x)
        g1 = g2 = None
        if self.gated:
            g1 = ws.get("gate1", (n, self.D), torch.float32)
            ops.linear(h1, self.wg1, self.bg1, g1)
        hm = self.conv.forward(ctx, h1, cache.state.get("conv")) if self.conv is not None else h1
        a = self.mixer.forward(ctx, hm, cache)
        f, f_terms, f_weight = None, 1, 1.0
        if self.ffn is not None:
            h2 = ws.get("norm_h2", (n, self.D), ops.dtype)
            self.norm2.forward_into(ctx, x, h2)
            if self.gated:
                g2 = ws.get("gate2", (n, self.D), torch.float32)
                ops.linear(h2, self.wg2, self.bg2, g2)
            f = self.ffn.forward(ctx, h2)
            if isinstance(f, tuple):          # (terms (N * k, D), k, weight): the feed-forward leaves its sum to the block
                f, f_terms, f_weight = f
        if not self.gated and f is None:
            return x, a
        out = ws.get("block_delta", (n, self.D), torch.float32)
        ops.gated_sum(a, g1, f, g2, out, f_terms, f_weight)
        return x, out


@register_block("parallel_shared")
class ParallelSharedBlock(Block):
    """`h = norm(x); x += m * (mixer(h) + ffn(h))`: one norm whose output both sublayers read, and one multiplier m
    (`residual_mult`) on their sum. A layer without a feed-forward has `x += m * mixer(h)`. The pending term of the
    layer before is added by the norm, in the same pass over the row; the sum and the product with m are 32-bit. A
    feed-forward that can take the mixer's result and m into its own last kernel (`forward(ctx, h, add=, scale=)`, marked
    by `takes_sum`) does so; otherwise the block adds the two terms up itself."""
    def __init__(self, mixer: Mixer, ffn: FeedForward | None, make_norm, hidden_size: int, residual_mult: float = 1.0,
                 norm=None, names: tuple = ("norm", "mixer", "ffn")):
        self.mixer, self.ffn, self.D, self.mult = mixer, ffn, hidden_size, float(residual_mult)
        self.names = tuple(names)
        self.norm = make_norm(norm) if norm is not None else make_norm()

    def children(self):
        out = [(self.names[0], self.norm), (self.names[1], self.mixer)]
        if self.ffn is not None:
            out.append((self.names[2], self.ffn))
        return tuple(out)

    def tensors(self) -> dict[str, ParamSpec]:
        return {(f"{prefix}.{k}" if k else prefix): v for prefix, part in self.children() for k, v in part.tensors().items()}

    def bind(self, tensors, ops) -> None:
        for prefix, part in self.children():
            part.bind({k[len(prefix) + 1:]: v for k, v in tensors.items() if k == prefix or k.startswith(prefix + ".")}, ops)

    def forward(self, ctx, x, delta, cache: LayerCache):
        h = self.norm.forward(ctx, x, delta)                          # x += pending term; h = norm(x)
        a = self.mixer.forward(ctx, h, cache)
        if self.ffn is not None and getattr(self.ffn, "takes_sum", False):
            return x, self.ffn.forward(ctx, h, add=a, scale=self.mult)
        out = ctx.ws.get("block_delta", (x.shape[0], self.D), torch.float32)
        if self.ffn is None:
            if self.mult == 1.0:
                return x, a
            ctx.ops.weighted_sum([a], [self.mult], out)
        else:
            ctx.ops.weighted_sum([a, self.ffn.forward(ctx, h)], [self.mult, self.mult], out)
        return x, out
