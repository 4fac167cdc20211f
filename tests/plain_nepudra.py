"""Plain, slow Nepudra: one function per mechanism, written from the design's equations in 64-bit, whole sequences,
token by token where the design is a recurrence. It shares no code with the package (only the tensor names and the keys
of config.json, which are the design's own).

A model is (config dict, {tensor name: float64 tensor}). `forward(config, tensors, tokens)` returns the logits of every
position, and with `layers=True` also the residual stream after every layer.
"""
from __future__ import annotations
import math

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def embedding(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """Token rows plus hashed rows of (previous token, token) pairs; a sequence's first token takes the table's last row."""
    b = cfg["embedding"]["bigram"]
    rows = []
    for i, t in enumerate(tokens):
        r = b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
        rows.append(w["embed"][t] + w["bigram"][r])
    return torch.stack(rows)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * g


def feed_forward(w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def yarn_angles(rot: dict, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, (n, dims / 2), of the scaled rotation."""
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
    ang = torch.arange(n, dtype=F)[:, None] * f[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate_halves(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x: (n, heads, dim); dimension i < dims / 2 is paired with i + dims / 2; dimensions from `dims` on pass."""
    half = dims // 2
    a, b = x[..., :half], x[..., half:dims]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def keys_values(cfg: dict, w: dict, p: str, m: dict, h: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """What a layer with projections of its own puts into its cache: keys (normed and rotated where the mixer does
    that) and values, (n, kv heads, size)."""
    n = h.shape[0]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(n, m["kv_heads"], m["dim"])
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(n, m["kv_heads"], m["vdim"])
    if p + "k.norm" in w:
        k = rms(k, cfg["norm"]["eps"]) * w[p + "k.norm"]
    if "rot" in m:
        cos, sin = yarn_angles(m["rot"], n)
        k = rotate_halves(k, cos, sin, m["rot"]["dims"])
    return k, v


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
                      softcap: float = 0.0) -> torch.Tensor:
    """q: (n, H, dim), k: (n, G, dim), v: (n, G, vdim). Row i sees keys j <= i, and with a window only i - j < window."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F)
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        i = torch.arange(n)[:, None]
        j = torch.arange(n)[None, :]
        seen = j <= i
        if window:
            seen &= (i - j) < window
        s = s.masked_fill(~seen, -math.inf)
        out[:, hq] = torch.softmax(s, -1) @ v[:, g]
    return out


def attention(cfg: dict, w: dict, p: str, m: dict, h: torch.Tensor, kv: tuple) -> torch.Tensor:
    """Both attention mixers: what one has and the other lacks is switched by the keys of `m` and the tensors present."""
    n = h.shape[0]
    H = m["heads"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, m["dim"])
    if p + "q.norm" in w:
        q = rms(q, cfg["norm"]["eps"]) * w[p + "q.norm"]
    if "rot" in m:
        cos, sin = yarn_angles(m["rot"], n)
        q = rotate_halves(q, cos, sin, m["rot"]["dims"])
    if "q_temp" in m:
        q = q * query_temperature(m["q_temp"], torch.arange(n, dtype=F))[:, None, None]
    k, v = kv
    o = softmax_attention(q, k, v, m["scale"], m.get("mask", {}).get("size", 0), m.get("softcap", 0.0))
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    y = o.reshape(n, -1) @ w[p + "o"].T
    if p + "o.b" in w:
        y = y + w[p + "o.b"]
    return y


def delta_recurrence(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d: torch.Tensor, a: torch.Tensor,
                     S: torch.Tensor | None = None, unit_eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """r, k, d, a: (n, H, dk); v: (n, H, dv); S: (H, dk, dv) or None for zeros. Per token and head, with the unit key u:
    S <- diag(d) S - (a u)(u^T S) + k v^T, both products from the state before the token; o = S^T r. Returns (o, S)."""
    n, H, dk = k.shape
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    S = torch.zeros(H, dk, v.shape[2], dtype=F) if S is None else S
    o = torch.zeros(n, H, v.shape[2], dtype=F)
    for t in range(n):
        back = torch.einsum("hi,hij->hj", u[t], S)
        S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * back[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hij,hi->hj", S, r[t])
    return o, S


def decay_of(z: torch.Tensor) -> torch.Tensor:
    """The decay of a key channel from its input: exp(-exp(-1/2) * sigmoid(z))."""
    return torch.exp(-math.exp(-0.5) * sigmoid(z))


def general_delta(cfg: dict, w: dict, p: str, m: dict, h: torch.Tensor, state: torch.Tensor | None = None) -> torch.Tensor:
    """The generalized delta rule mixer: projections, decays and removal rates, the recurrence, head norm, gate, output."""
    n = h.shape[0]
    H, dim = m["heads"], m["dim"]
    r = (h @ w[p + "r"].T).view(n, H, dim)
    k = (h @ w[p + "k"].T).view(n, H, dim)
    v = (h @ w[p + "v"].T).view(n, H, dim)
    d = decay_of(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]).view(n, H, dim)
    a = sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(n, H, dim)
    o, _ = delta_recurrence(r, k, v, d, a, state)
    o = rms(o, cfg["norm"]["eps"]).reshape(n, -1) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def depth_average(streams: list, c: torch.Tensor) -> torch.Tensor:
    """sum_j c[j] * streams[j] over all streams so far (the embedding output first)."""
    return sum(c[j] * streams[j] for j in range(len(streams)))


def query_temperature(q_temp: dict, positions: torch.Tensor) -> torch.Tensor:
    """The factor of the queries at each position: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    return 1.0 + q_temp["coef"] * torch.log(torch.floor((positions + 1) / q_temp["every"]) + 1.0)


def forward(cfg: dict, w: dict, tokens: list[int], layers: bool = False):
    eps = cfg["norm"]["eps"]
    x = embedding(cfg, w, tokens)
    streams = [x]
    after = []
    caches: dict[int, tuple] = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        h = scalar_norm(x, w[p + "norm1"], eps)
        if L["type"] == "general_delta":
            y = general_delta(cfg, w, p + "mix.", m, h)
        else:
            if "kv_from" in m:
                kv = caches[m["kv_from"]]
            else:
                kv = caches[i] = keys_values(cfg, w, p + "mix.", m, h)
            y = attention(cfg, w, p + "mix.", m, h, kv)
        x = x + y
        if L.get("mlp") is not None:
            x = x + feed_forward(w, p + "mlp.", scalar_norm(x, w[p + "norm2"], eps))
        streams.append(x)
        x = depth_average(streams, w[p + "dwa"])
        after.append(x)
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if layers else logits
