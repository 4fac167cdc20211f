"""Depth-averaged layers: what a layer reads is a learned weighted sum of the results of all layers before it.

With X_0 the embeddings and X_(i+1) the result of layer i (the inner block's residual stream after its sublayers), the
stream that layer i + 1 (or the model's last norm) reads is

    x = sum_j c_i[j] X_j,    j = 0 .. i + 1,

c_i being layer i's tensor `name` of i + 2 numbers. The block wraps any other block (`inner`), which computes X_(i+1)
from x as it would without the averaging. The X_j of a step live in one scratch buffer (rows, depths + 1, width) that the
layers of the model share; sums and products are 32-bit, the terms added in rising j. The sum is handed on unevaluated
(`PendingDepthAverage`) so that the next norm takes it in its own pass over the row, as it takes a pending residual term.
"""
from __future__ import annotations
import torch

from dataclasses import dataclass

from ..config import PartSpec
from ..weights import ParamSpec
from .base import BLOCKS, Block, LayerCache, register_block


@dataclass
class PendingDepthAverage:
    """What a depth-averaged layer hands on in place of a pending residual term: the sum has not been taken yet, so that
    the norm that reads the stream next can take it in the same pass (`Norm` parts look for `fold_into_norm`). A
    consumer that cannot fold it calls `resolve`, which runs the plain operation."""
    streams: torch.Tensor
    depth: int
    coef: torch.Tensor
    delta: torch.Tensor | None

    def fold_into_norm(self, ctx, x, weight, eps, h, rows) -> bool:
        return bool(ctx.ops.depth_average_rmsnorm(self.streams, self.depth, self.coef, x, self.delta, weight, eps, h, rows))

    def resolve(self, ctx, x) -> None:
        ctx.ops.depth_average(self.streams, self.depth, self.coef, x, self.delta)


@register_block("depth_average")
class DepthAverageBlock(Block):
    def __init__(self, mixer, ffn, make_norm, inner: PartSpec, depth: int, depths: int, hidden_size: int,
                 name: str = "depth_weights"):
        """inner: the block that arranges the layer's norms, mixer and feed-forward. depth: this layer's index i among the
        `depths` averaged layers of the model."""
        if inner.kind not in BLOCKS:
            raise NotImplementedError(f"block kind {inner.kind!r} is not registered (have {sorted(BLOCKS)})")
        if not 0 <= depth < depths:
            raise ValueError(f"depth {depth} is outside the model's {depths} averaged layers")
        self.inner = BLOCKS[inner.kind](mixer, ffn, make_norm, **inner.params)
        self.mixer, self.ffn = mixer, ffn
        self.depth, self.depths, self.D, self.name = int(depth), int(depths), hidden_size, name
        self.coef: torch.Tensor | None = None

    def children(self):
        return self.inner.children()

    def state_need(self):
        return self.inner.state_need()

    def tensors(self) -> dict[str, ParamSpec]:
        return {**self.inner.tensors(), self.name: ParamSpec((self.depth + 2,), role="vector", init="ones")}

    def bind(self, tensors, ops) -> None:
        self.inner.bind({k: v for k, v in tensors.items() if k != self.name}, ops)
        self.coef = tensors[self.name].float().contiguous()

    def forward(self, ctx, x, delta, cache: LayerCache):
        ops = ctx.ops
        hist = ctx.ws.get("depth_streams", (x.shape[0], self.depths + 1, self.D), torch.float32)
        if self.depth == 0:
            if hasattr(delta, "resolve"):
                delta = delta.resolve(ctx, x)
            ops.depth_average(hist, -1, None, x, delta)      # X_0: the stream as the embedding left it
            delta = None
        x, delta = self.inner.forward(ctx, x, delta, cache)
        return x, PendingDepthAverage(hist, self.depth, self.coef, delta)
