"""Attention over a cached latent: per token the cache holds one vector c (the normed first `latent_dim` outputs of the
down projection) and one rotated key part k_r (its last `rope_dim` outputs) that all heads share.

Per head h, with q_h = [q_n (nope_dim, not rotated) | q_r (rope_dim, rotated)], key j has the unrotated key
`W_uk,h c_j` and the value `W_uv,h c_j`; the score is `(q_n . W_uk,h c_j + q_r . k_r,j) * scale`, softmax over the
causal keys, output `W_o` on the concatenated heads. Neither keys nor values are ever built: since
`q_n . (W_uk,h c) = (W_uk,h^T q_n) . c` and `sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j)`, the step computes

    qa[n, h] = [W_uk,h^T q_n | rot(q_r)]                 (latent_dim + rope_dim)      one product per head
    ol[n, h] = sum_j softmax_j(qa[n, h] . [c_j | k_r,j] * scale) c_j                  attention with ONE shared key head
    o[n, h]  = W_uv,h ol[n, h]                                                         one product per head

so a step reads only the cache (latent_dim + rope_dim values per token, whatever the number of heads), for prompt
portions and decoded tokens alike. The rotation turns the first `rotated` dimensions of the rope part (pairs i,
i + rotated/2) by the token's position; the rest pass unchanged. A mixer built with `own_latent=False` has no down
projection: its schedule entry reads the cache slot another layer wrote earlier in the same step. Scores, softmax, the
latent's norm and the rotation are 32-bit in both dtypes.

Options: `pairing` "neighbours" pairs dimension 2i with 2i + 1 in the rotation instead of i with i + rotated/2; `sink`:
the softmax's denominator also holds `exp(sink_h)`, a learned number per head without key or value, not scaled, counted
once; `out_gate`: the concatenated heads are multiplied element by element by `sigmoid(W_gate h)` (of the mixer's own
input) before the output product; the sigmoid and the product are 32-bit.
"""
from __future__ import annotations
import torch

from ..cache import LatentNeed
from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer
from .retention import PAIRINGS

_NAMES = {"q": "q_proj", "down": "kv_down", "down_norm": "kv_norm", "up_k": "k_up", "up_v": "v_up", "out": "o_proj",
          "sink": "sinks", "gate": "g_proj"}


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, nope_dim: int, rope_dim: int, value_dim: int, latent_dim: int,
                 scale: float, rotated: int | None = None, eps: float = 1e-6, position: str = "rope",
                 own_latent: bool = True, window: int = 0, names: dict | None = None, pairing: str = "halves",
                 sink: bool = False, out_gate: bool = False):
        self.D, self.H, self.dn, self.dr, self.dv, self.r = hidden_size, num_heads, nope_dim, rope_dim, value_dim, latent_dim
        self.scale, self.eps, self.position, self.own, self.window = float(scale), float(eps), position, bool(own_latent), int(window)
        self.rotated = rope_dim if rotated is None else int(rotated)
        if self.rotated % 2 or not 0 <= self.rotated <= rope_dim:
            raise ValueError(f"{self.rotated} rotated dimensions must be even and at most rope_dim {rope_dim}")
        if pairing not in PAIRINGS:
            raise ValueError(f"pairing {pairing!r} is not one of {sorted(PAIRINGS)}")
        self.pairing, self.has_sink, self.out_gate = pairing, bool(sink), bool(out_gate)
        self.names = {**_NAMES, **(names or {})}
        self.wq = self.wd = self.norm_w = self.wuk_t = self.wuv = self.wo = self.sink = None

    def tensors(self) -> dict[str, ParamSpec]:
        n, H = self.names, self.H
        out = {n["q"]: ParamSpec((H * (self.dn + self.dr), self.D)), n["up_k"]: ParamSpec((H * self.dn, self.r)),
               n["up_v"]: ParamSpec((H * self.dv, self.r)), n["out"]: ParamSpec((self.D, H * self.dv))}
        if self.own:
            out[n["down"]] = ParamSpec((self.r + self.dr, self.D))
            out[n["down_norm"]] = ParamSpec((self.r,), role="vector", init="ones")
        if self.has_sink:
            out[n["sink"]] = ParamSpec((H,), role="vector")
        if self.out_gate:
            out[n["gate"]] = ParamSpec((H * self.dv, self.D))
        return out

    def bind(self, tensors, ops) -> None:
        n, H = self.names, self.H
        self.wq, self.wo = tensors[n["q"]], tensors[n["out"]]
        self.q_width = H * (self.dn + self.dr)
        if self.out_gate:      # one product for everything that reads h in float32: columns [q | gate]
            self.wq = torch.cat([self.wq, tensors[n["gate"]]], 0).contiguous()
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None
        # W_uk per head transposed once, (H, latent, nope): the per-head product W_uk,h^T q_n then reads rows like any other
        self.wuk_t = tensors[n["up_k"]].view(H, self.dn, self.r).transpose(1, 2).contiguous()
        self.wuv = tensors[n["up_v"]].view(H, self.dv, self.r).contiguous()
        if self.own:
            self.wd, self.norm_w = tensors[n["down"]], tensors[n["down_norm"]]
        ops.check_latent_attention(H, self.r + self.dr, self.r)

    def cache_need(self) -> LatentNeed:
        return LatentNeed(self.r + self.dr, self.window)

    def position_name(self) -> str | None:
        return self.position

    def step_needs(self) -> tuple[str, ...]:
        return ("latent_attention",)

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        H, dn, dr, dv, r = self.H, self.dn, self.dr, self.dv, self.r
        pos = ctx.positions[self.position]
        if cache.write != self.own:
            raise ValueError("a latent-attention layer writes the cache exactly when it has a down projection of its own")
        if self.own:
            dkv = ws.get("latent_down", (n, r + dr), torch.float32)
            ops.linear(h, self.wd, None, dkv)
            if self.pairing == "halves":
                ops.latent_cache_write(dkv, self.norm_w, self.eps, pos.cos, pos.sin, self.rotated, ctx.meta, cache)
            else:
                ops.latent_cache_write(dkv, self.norm_w, self.eps, pos.cos, pos.sin, self.rotated, ctx.meta, cache,
                                       pairing=PAIRINGS[self.pairing])
        q = ws.get("latent_q", (n, H, dn + dr), ops.dtype)
        gate = None
        if self.out_gate:
            qg = ws.get("latent_qg", (n, self.q_width + H * dv), torch.float32)
            ops.linear(h, self.wq, None, qg)
            ops.activate(qg, 0, "identity", q.view(n, self.q_width))                    # q rounded once, the gate stays 32-bit
            gate = (qg, self.q_width)
        else:
            ops.linear(h, self.wq, None, q.view(n, H * (dn + dr)))
        qa = ws.get("latent_qa", (n, H, r + dr), ops.dtype)
        if self.pairing == "halves":
            ops.rotate_heads(q, dn, pos.cos, pos.sin, self.rotated, ctx.meta, qa, r)   # qa[..., r:] = rot(q[..., dn:])
        else:
            ops.rotate_heads(q, dn, pos.cos, pos.sin, self.rotated, ctx.meta, qa, r, pairing=PAIRINGS[self.pairing])
        ops.linear_heads(q, 0, dn, self.wuk_t, qa, 0)                                   # qa[..., :r] = W_uk,h^T q_n
        ol = ws.get("latent_out", (n, H, r), ops.dtype)
        if self.has_sink:
            ops.latent_attention(qa, cache, ctx.meta, ol, r, self.scale, self.window, sink=self.sink)
        else:
            ops.latent_attention(qa, cache, ctx.meta, ol, r, self.scale, self.window)
        o = ws.get("attn_out", (n, H, dv), ops.dtype)
        ops.linear_heads(ol, 0, r, self.wuv, o, 0)                                      # o[:, h] = W_uv,h ol[:, h]
        if gate is not None:
            ops.gate_multiply(o.view(n, H * dv), gate[0], gate[1], "sigmoid", o.view(n, H * dv))
        delta = ws.get("delta", (n, self.D), torch.float32)
        ops.linear(o.view(n, H * dv), self.wo, None, delta)
        return delta
