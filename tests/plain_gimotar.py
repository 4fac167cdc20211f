"""Plain, slow Gimotar: one function per mechanism, written from the design's equations in 64-bit, whole sequences,
token by token where the design is a recurrence. It shares no code with the package (only the tensor names and the keys
of config.json, which are the design's own).

A model is (config dict, {tensor name: float64 tensor}). `forward(config, tensors, tokens)` returns the logits of every
position, and with `layers=True` also the residual stream after every layer.
"""
from __future__ import annotations
import math

import torch

F = torch.float64
DECAY_SHARPNESS = 8.0       # log a = -DECAY_SHARPNESS * r * softplus(lam)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def embedding(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """Scaled token rows plus (unscaled) hashed rows of (previous token, token); the first token takes the last row."""
    e = cfg["embedding"]
    b = e["bigram"]
    rows = []
    for i, t in enumerate(tokens):
        r = b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
        rows.append(w["embed"][t] * e["scale"] + w["bigram"][r])
    return torch.stack(rows)


def one_plus_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance from one."""
    return rms(x, eps) * (1.0 + g)


# ---- rotations
def angles(rot: dict, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, (n, dims / 2), scaled by wavelength if the rotation says so."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc is not None:
        def turn_dim(t):
            return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(turn_dim(sc["fast"])), 0)
        hi = min(math.ceil(turn_dim(sc["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    a = torch.arange(n, dtype=F)[:, None] * f[None, :]
    return torch.cos(a) * mag, torch.sin(a) * mag


def rotate_halves(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x: (T, heads, dim). Dimension i is paired with i + dims/2, the dimensions from `dims` on pass."""
    h = dims // 2
    u, v = x[..., :h], x[..., h:dims]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def rotate_neighbours(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x: (T, heads, dim). Dimension 2i is paired with 2i + 1, the dimensions from `dims` on pass."""
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- softmax attention under a mask
def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, visible,
                     sink: torch.Tensor | None = None) -> torch.Tensor:
    """q: (T, H, d), k: (T, H, d), v: (T, H, dv) (keys and values already given per query head). `visible(i, j)` says
    whether position i sees key j. sink (H,): one more term exp(sink_h) in the denominator, without a value."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for i in range(T):
        js = [j for j in range(T) if visible(i, j)]
        for h in range(H):
            s = torch.stack([(q[i, h] * k[j, h]).sum() * scale for j in js])
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = sum(e[n] * v[j, h] for n, j in enumerate(js)) / den
    return out


def masked_attention_fast(q, k, v, scale, mask, sink=None):
    """The same with the mask as a (T, T) boolean matrix, vectorised (for the longer sequences of the tests)."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], -math.inf)
    if sink is not None:
        s = torch.cat([s, sink[:, None, None].expand(-1, s.shape[1], 1)], -1)
    p = torch.softmax(s, -1)
    if sink is not None:
        p = p[..., :-1]
    return torch.einsum("hij,jhd->ihd", p, v)


def causal_mask(T: int) -> torch.Tensor:
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def chunk_mask(T: int, size: int) -> torch.Tensor:
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & (i[None, :] // size == i[:, None] // size)


# ---- mixers
def rglru_gates(w: dict, p: str, u: torch.Tensor, blocks: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Recurrence gate r and input gate i, each from block-diagonal matrices over `blocks` equal parts of u."""
    T, W = u.shape
    ub = u.view(T, blocks, W // blocks)
    r = sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
    i = sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
    return r, i


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x: (T, C); w: (C, taps), the last column multiplies the token's own input; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], 0)
    return torch.stack([(pad[t: t + taps].T * w).sum(-1) for t in range(T)]) + b


def rglru_recurrence(u, r, i, lam):
    a = torch.exp(-DECAY_SHARPNESS * r * softplus(lam))
    S = torch.zeros(u.shape[1], dtype=F)
    out = []
    for t in range(u.shape[0]):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out.append(S)
    return torch.stack(out)


def rglru(cfg: dict, w: dict, p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    r, i = rglru_gates(w, p, u, m["blocks"])
    S = rglru_recurrence(u, r, i, w[p + "lam"])
    return (S * y) @ w[p + "o"].T


def latent_attention(cfg: dict, w: dict, p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    eps = cfg["norm"]["eps"]
    cos, sin = angles(m["rot"], T)
    q = (h @ w[p + "q"].T).view(T, H, d + dr)
    q = torch.cat([q[..., :d], rotate_neighbours(q[..., d:], cos, sin, m["rot"]["dims"])], -1)
    dkv = h @ w[p + "dkv"].T
    c = rms(dkv[:, :rank], eps) * w[p + "dkv.norm"]
    kr = rotate_neighbours(dkv[:, None, rank:], cos, sin, m["rot"]["dims"])           # (T, 1, dr), shared by the heads
    k = torch.cat([(c @ w[p + "uk"].T).view(T, H, d), kr.expand(T, H, dr)], -1)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    o = masked_attention_fast(q, k, v, m["scale"], causal_mask(T), w[p + "sink"])
    o = o.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def attention(cfg: dict, w: dict, p: str, m: dict, h: torch.Tensor, v_first: torch.Tensor | None):
    """Returns (result, this layer's unmixed-or-mixed values for the caller to keep if it is the first mixing layer)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    eps = cfg["norm"]["eps"]
    q = rms((h @ w[p + "q"].T).view(T, H, d), eps) * w[p + "q.norm"]
    k = rms((h @ w[p + "k"].T).view(T, G, d), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).view(T, G, dv)
    if m.get("rot") is not None:
        cos, sin = angles(m["rot"], T)
        q = rotate_halves(q, cos, sin, m["rot"]["dims"])
        k = rotate_halves(k, cos, sin, m["rot"]["dims"])
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rep = H // G
    mask = chunk_mask(T, m["mask"]["size"]) if m.get("mask") is not None else causal_mask(T)
    o = masked_attention_fast(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), m["scale"], mask)
    return o.reshape(T, H * dv) @ w[p + "o"].T, v


# ---- feed-forward
def expert(w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(z: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The `top` largest logits of every row and the softmax over them alone."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def mixture(cfg: dict, w: dict, p: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    z = h @ w[p + "router"].T + w[p + "router.b"]
    idx, wt = route(z, mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for n in range(idx.shape[1]):
            out[t] += wt[t, n] * expert(w, f"{p}e{int(idx[t, n])}.", h[t: t + 1])[0]
    if mlp.get("shared") is not None:
        out = out + expert(w, p + "shared.", h)
    return out


def forward(cfg: dict, w: dict, tokens: list[int], layers: bool = False):
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = embedding(cfg, w, tokens)
    streams = []
    v_first = None
    for n, L in enumerate(cfg["layers"]):
        p = f"l{n}."
        h = one_plus_norm(x, w[p + "norm1"], eps)
        if L["type"] == "rglru":
            a = rglru(cfg, w, p + "mix.", L["mixer"], h)
        elif L["type"] == "latent_attention":
            a = latent_attention(cfg, w, p + "mix.", L["mixer"], h)
        elif L["type"] == "attention":
            a, v = attention(cfg, w, p + "mix.", L["mixer"], h, v_first)
            if L["mixer"].get("v_mix") and v_first is None:
                v_first = v
        else:
            raise NotImplementedError(L["type"])
        if L.get("mlp") is not None:
            a = a + mixture(cfg, w, p + "mlp.", L["mlp"], h)
        x = x + mult * a
        streams.append(x)
    logits = one_plus_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(streams)) if layers else logits
