"""Rotary position encoding: rotate-half on query and key heads, values untouched.

Inverse frequencies in float32 as the reference computes them (fusezap/serve/models/llama.py:102-120):
`inv[j] = 1 / theta^(2j/hd)`; `linear`: `inv / factor`; `llama3`: with `wl = 2*pi/inv`, frequencies whose wavelength
exceeds `old/low` are divided by `factor`, those between `old/high` and `old/low` are blended with
`smooth = (old/wl - low) / (high - low)`. Tables `cos(p * inv[j])`, `sin(...)` of shape (max_len, hd/2) in float32
(llama.py:122-130); the rotation itself (llama.py:524-527): `out = cat(x1*cos - x2*sin, x2*cos + x1*sin)` with
`x1 = x[..., :hd/2]`, `x2 = x[..., hd/2:]`, the row of the token's own position. The angles and the rotation are computed in
32-bit in both dtypes; the result is rounded once to the cache's dtype.
"""
from __future__ import annotations
import math

import numpy as np
import torch

from .base import LayerCache, PositionEncoding, register_position


def inverse_frequencies(head_dim: int, theta: float, kind: str = "default", factor: float = 1.0,
                        low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                        original_max_position_embeddings: int = 0) -> np.ndarray:
    d = head_dim
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, d, 2, dtype=np.int64).astype(np.float32) / np.float32(d)))).astype(np.float32)
    if kind == "linear":
        inv = (inv / np.float32(factor)).astype(np.float32)
    elif kind == "llama3":
        old, lo, hi = original_max_position_embeddings, low_freq_factor, high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (old / wl - lo) / (hi - lo)
        out = np.where(wl > old / lo, inv / factor, inv)
        mid = (wl <= old / lo) & (wl >= old / hi)
        inv = np.where(mid, (1 - smooth) * out / factor + smooth * out, out).astype(np.float32)
    elif kind != "default":
        raise NotImplementedError(f"rope kind {kind!r}")
    return inv


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, kind: str = "default", factor: float = 1.0,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 0, precise: bool = False, turns_fast: float = 32.0,
                 turns_slow: float = 1.0, magnitude: float = 1.0):
        """precise: frequencies theta^(-2j/head_dim) and angles p * f_j are computed in 64-bit and the cosines and sines
        rounded once to float32 (default: in float32 throughout, as the dense decoder's reference does). The tables
        serve any pairing of dimensions: a mixer that rotates in its own kernels (neighbouring dimensions paired, only
        the first dimensions of a head rotated) reads `cos` / `sin` (max_len, head_dim / 2) by pair index.
        kind "yarn" (factor, original_max_position_embeddings, turns_fast, turns_slow): see below; `magnitude`
        multiplies both tables (1: plain cosines and sines)."""
        if head_dim % 2:
            raise ValueError(f"rope needs an even head_dim, got {head_dim}")
        self.head_dim, self.precise = head_dim, bool(precise)
        if precise and kind not in ("default", "llama3", "yarn"):
            raise NotImplementedError("precise angles are computed for unscaled, llama3-scaled and yarn-scaled frequencies only")
        if kind == "yarn" and not precise:
            raise NotImplementedError("yarn-scaled frequencies are computed in 64-bit only (precise=True)")
        self.magnitude = float(magnitude)
        self.inv_freq64 = np.float64(theta) ** (-np.arange(0, head_dim, 2, dtype=np.float64) / np.float64(head_dim))
        if precise and kind == "llama3":
            # by wavelength l = 2 pi / f: short ones (l < old / high) stay, long ones (l > old / low) are divided by
            # `factor`, those between are blended with s = (old / l - low) / (high - low); all in 64-bit
            f, old = self.inv_freq64, float(original_max_position_embeddings)
            wl = 2 * math.pi / f
            s = (old / wl - low_freq_factor) / (high_freq_factor - low_freq_factor)
            self.inv_freq64 = np.where(wl < old / high_freq_factor, f,
                                       np.where(wl > old / low_freq_factor, f / factor, (1 - s) * f / factor + s * f))
        if kind == "yarn":
            # by the pair index at which a frequency makes `turns` full turns over the original length,
            # dim(t) = head_dim ln(old / (2 pi t)) / (2 ln theta): pairs below dim(turns_fast) keep their frequency,
            # pairs above dim(turns_slow) are divided by `factor`, those between are blended linearly in the index
            old = float(original_max_position_embeddings)
            def pair_of(turns: float) -> float:
                return head_dim * math.log(old / (2 * math.pi * turns)) / (2 * math.log(theta))
            lo = max(math.floor(pair_of(turns_fast)), 0)
            hi = min(math.ceil(pair_of(turns_slow)), head_dim - 1)
            ramp = np.clip((np.arange(head_dim // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            self.inv_freq64 = self.inv_freq64 / factor * ramp + self.inv_freq64 * (1.0 - ramp)
        self.inv_freq = None if kind == "yarn" else inverse_frequencies(
            head_dim, theta, kind, factor, low_freq_factor, high_freq_factor, original_max_position_embeddings)
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None

    def prepare(self, max_len: int, device: torch.device) -> None:
        if self.precise:
            fr = np.arange(max_len, dtype=np.float64)[:, None] * self.inv_freq64[None, :]
        else:
            fr = np.arange(max_len, dtype=np.float32)[:, None] * self.inv_freq[None, :]
        self.cos = torch.from_numpy((np.cos(fr) * self.magnitude).astype(np.float32)).to(device)
        self.sin = torch.from_numpy((np.sin(fr) * self.magnitude).astype(np.float32)).to(device)

    def weight_tensors(self) -> list:
        return []       # a step gathers one row of the tables per token; they are not streamed like weights

    def rotate_and_store(self, ctx, qkv: torch.Tensor, q_out: torch.Tensor, cache: LayerCache,
                         num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if head_dim != self.head_dim:
            raise ValueError(f"rope was built for head_dim {self.head_dim}, the mixer has {head_dim}")
        ctx.ops.rope_kv_write(qkv, self.cos, self.sin, ctx.meta, cache, q_out, num_heads, num_kv_heads, head_dim)

    def project_rotate_store(self, ctx, h, w, bias, q_out, cache, num_heads, num_kv_heads, head_dim) -> bool:
        if head_dim != self.head_dim:
            raise ValueError(f"rope was built for head_dim {self.head_dim}, the mixer has {head_dim}")
        fused = getattr(ctx.ops, "linear_rope_kv_write", None)      # an optional entry of the kernel table
        return bool(fused is not None and fused(h, w, bias, self.cos, self.sin, ctx.meta, cache, q_out, num_heads,
                                                num_kv_heads, head_dim))
