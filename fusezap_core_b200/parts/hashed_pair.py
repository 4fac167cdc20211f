"""Hashed pair embedding: a second table whose row is chosen by a hash of (previous token, token).

For the token t at position p of its request, with u the token before it:

    x += table[(u * mul_prev + t * mul_cur) mod buckets]      p > 0
    x += table[buckets]                                       p = 0 (the table's last row, which no hash reaches)

The table has buckets + 1 rows. Inside a portion the previous token is the row before; for a portion's first token it
is the request's state, one int32 that holds the last token of the portion before (so a prompt may be cut anywhere). The
sum is 32-bit; the hash is computed in 64-bit integers.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import EmbedExtra, register_embed_extra


@register_embed_extra("hashed_pair")
class HashedPairEmbedding(EmbedExtra):
    def __init__(self, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, name: str = "pair_embed"):
        if buckets <= 0 or mul_prev < 0 or mul_cur < 0:
            raise ValueError(f"a hashed pair embedding needs positive buckets and multipliers that are not negative, got "
                             f"{buckets}, {mul_prev}, {mul_cur}")
        self.D, self.buckets, self.mul_prev, self.mul_cur, self.name = hidden_size, int(buckets), int(mul_prev), int(mul_cur), name
        self.table: torch.Tensor | None = None

    def tensors(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.buckets + 1, self.D))}

    def bind(self, tensors, ops) -> None:
        self.table = tensors[self.name]

    def step_needs(self) -> tuple[str, ...]:
        return ("token_ids",)

    def state_need(self) -> dict:
        return {self.name + ".prev": ((1,), torch.int32)}

    def weight_tensors(self) -> list:
        return []       # a step gathers one row per token

    def forward(self, ctx, x: torch.Tensor, state: dict) -> None:
        ctx.ops.hashed_pair_embed(self.table, ctx.token_ids, ctx.meta, state[self.name + ".prev"], self.buckets,
                                  self.mul_prev, self.mul_cur, x)
