"""Grouped-query attention over a sliding window that keeps the first tokens, with a sink in the softmax.

Row i (position p_i of its request) sees key j if `j <= i and (i - j < window or j < keep_first)` (window 0: every
earlier key). Kept tokens keep their true positions. Query head h reads kv head `h // (heads / kv_heads)`; keys have
`key_dim` and values `value_dim` dimensions. The score is `(q . k) * scale`; with `sink` the softmax's denominator
also holds `exp(sink_h)`, a learned number per head that has no key and no value and is not scaled:

    o = sum_j exp(s_j - m) v_j / (sum_j exp(s_j - m) + exp(sink_h - m)),      m = max(max_j s_j, sink_h)

q and k are rotated by position on their first `rotated` dimensions (`pairing` "neighbours": 2i with 2i+1; "halves":
i with i + rotated/2), v is not. One product with the rows [q; k; v] leaves float32; the rotation, scores, softmax and
the value sum are 32-bit in both dtypes; keys and values are rounded once into the paged cache. The cache group of this
mixer gives back pages that lie wholly between the kept first tokens and the window.

Options, all off by default: `bias` names the products that have one (of "q", "k", "v", "out"; tensor `<name><bias_suffix>`);
`qk_norm`: every q and k head is divided by its root mean square (`norm_eps` inside the root) and multiplied by a weight
of key_dim values shared by the heads (`<q><norm_suffix>`, `<k><norm_suffix>`), before the rotation; `query_temperature`
(coef, every): q at position p is multiplied by `1 + coef * ln(floor((p + 1) / every) + 1)`; `softcap` c > 0: the scaled
score s becomes `c * tanh(s / c)`; `head_gate`: head h's output is multiplied by `sigmoid(W_gate h)_h`, one number per
head, before the output product; `own_kv=False`: the layer has no key and value projections and reads, with queries of
its own, the cache that another layer's mixer wrote (its schedule entry names that cache slot); `cache_window`: the
window the cache must keep when other layers read it too (None: this mixer's own); `span` s > 0: a chunked causal mask,
row i sees key j <= i only if `floor(i / s) = floor(j / s)`, blocks counted from position 0 of the sequence (with a
window both must hold; the cache keeps every token); `value_mix`: "source" keeps this layer's values (the float32
product, before they are rounded into the cache) for the step under `value_mix_key`, "blend" replaces this layer's
values by `(1 - lam) v + lam v_source` of the same token before they are cached, with lam the layer's own number
(tensor `<value_mix>`, which a source layer may carry and never reads). The norms, the temperature, the cap, the gate
and the blend are 32-bit in both dtypes.
"""
from __future__ import annotations
import torch

from ..cache import KVNeed
from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer
from .retention import PAIRINGS

_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "sink": "sinks", "out": "o_proj", "gate": "g_proj",
          "value_mix": "v_mix"}


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 window: int = 0, keep_first: int = 0, sink: bool = True, rotated: int = 0, pairing: str = "neighbours",
                 position: str | None = None, names: dict | None = None, bias: tuple = (), bias_suffix: str = ".bias",
                 qk_norm: bool = False, norm_eps: float = 1e-6, norm_suffix: str = "_norm", query_temperature: tuple | None = None,
                 softcap: float = 0.0, head_gate: bool = False, own_kv: bool = True, cache_window: int | None = None,
                 span: int = 0, value_mix: str | None = None, value_mix_key: str = "first_values"):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        if pairing not in PAIRINGS:
            raise ValueError(f"pairing {pairing!r} is not one of {sorted(PAIRINGS)}")
        if rotated % 2 or not 0 <= rotated <= key_dim:
            raise ValueError(f"{rotated} rotated dimensions must be even and at most key_dim {key_dim}")
        self.D, self.Hq, self.Hkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, key_dim, value_dim
        self.scale, self.window, self.keep_first, self.has_sink = float(scale), int(window), int(keep_first), bool(sink)
        self.rotated, self.pairing, self.position = int(rotated), pairing, (position if rotated else None)
        self.names = {**_NAMES, **(names or {})}
        if not set(bias) <= {"q", "k", "v", "out"}:
            raise ValueError(f"bias {bias!r} names something else than the q, k, v and out products")
        if query_temperature is not None and int(query_temperature[1]) <= 0:
            raise ValueError(f"query temperature {query_temperature!r}: the period must be positive")
        self.bias, self.bias_suffix = tuple(bias), bias_suffix
        self.qk_norm, self.norm_eps, self.norm_suffix = bool(qk_norm), float(norm_eps), norm_suffix
        self.q_temp = (float(query_temperature[0]), int(query_temperature[1])) if query_temperature is not None else None
        self.softcap, self.head_gate, self.own_kv = float(softcap), bool(head_gate), bool(own_kv)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window and (not self.window or self.cache_window < self.window):
            raise ValueError(f"a cache that keeps {self.cache_window} tokens cannot serve a window of {self.window or 'all'}")
        self.span = int(span)
        if self.span < 0 or (self.span and self.keep_first):
            raise ValueError(f"a chunked mask of {span} positions: the size must be positive, and no first tokens are kept")
        if value_mix not in (None, "source", "blend") or (value_mix and not own_kv):
            raise ValueError(f"value_mix {value_mix!r} is not one of None, 'source', 'blend', or the layer has no values of its own")
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.wqkv = self.bqkv = self.wo = self.bo = self.sink = self.q_norm_w = self.k_norm_w = self.mix_w = None

    def tensors(self) -> dict[str, ParamSpec]:
        n = self.names
        rows = {"q": self.Hq * self.dk, "k": self.Hkv * self.dk, "v": self.Hkv * self.dv, "out": self.D}
        out = {n["q"]: ParamSpec((rows["q"], self.D))}      # (declaration order is the order in which random weights are drawn)
        if self.own_kv:
            out[n["k"]] = ParamSpec((rows["k"], self.D))
            out[n["v"]] = ParamSpec((rows["v"], self.D))
        out[n["out"]] = ParamSpec((self.D, self.Hq * self.dv))
        for x in self.bias:
            if self.own_kv or x not in ("k", "v"):
                out[n[x] + self.bias_suffix] = ParamSpec((rows[x],), role="vector")
        if self.qk_norm:
            out[n["q"] + self.norm_suffix] = ParamSpec((self.dk,), role="vector", init="ones")
            if self.own_kv:
                out[n["k"] + self.norm_suffix] = ParamSpec((self.dk,), role="vector", init="ones")
        if self.head_gate:
            out[n["gate"]] = ParamSpec((self.Hq, self.D))
        if self.has_sink:
            out[n["sink"]] = ParamSpec((self.Hq,), role="vector")
        if self.value_mix is not None:
            out[n["value_mix"]] = ParamSpec((), role="vector", ignore=self.value_mix == "source")
        return out

    def bind(self, tensors, ops) -> None:
        n = self.names
        # one product for everything that reads h: columns [q | k | v | gate] (k and v only with projections of its own)
        parts = ["q"] + (["k", "v"] if self.own_kv else []) + (["gate"] if self.head_gate else [])
        self.wqkv = torch.cat([tensors[n[x]] for x in parts], 0).contiguous()
        self.bqkv = None
        if set(self.bias) & set(parts):
            self.bqkv = torch.cat([tensors[n[x] + self.bias_suffix].float() if x in self.bias else
                                   torch.zeros(tensors[n[x]].shape[0], dtype=torch.float32, device=self.wqkv.device)
                                   for x in parts], 0).contiguous()
        self.width = self.wqkv.shape[0]
        self.off_gate = self.width - self.Hq
        self.wo = tensors[n["out"]]
        self.bo = tensors[n["out"] + self.bias_suffix].float().contiguous() if "out" in self.bias else None
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None
        if self.qk_norm:
            self.q_norm_w = tensors[n["q"] + self.norm_suffix].float().contiguous()
            self.k_norm_w = tensors[n["k"] + self.norm_suffix].float().contiguous() if self.own_kv else None
        if self.value_mix == "blend":
            self.mix_w = tensors[n["value_mix"]].float().reshape(1).contiguous()
        ops.check_sink_attention(self.Hq, self.Hkv, self.dk, self.dv)

    def cache_need(self) -> KVNeed:
        return KVNeed(self.Hkv, self.dk, self.cache_window, value_dim=self.dv,
                      keep_first=self.keep_first if self.cache_window else 0)

    def position_name(self) -> str | None:
        return self.position

    def step_needs(self) -> tuple[str, ...]:
        return ("portions",)      # its kernels tile the rows of portions: the longest portion is part of a step's shape

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        Hq, Hkv, dk, dv = self.Hq, self.Hkv, self.dk, self.dv
        if cache.write != self.own_kv:
            raise ValueError("a mixer with key and value projections of its own writes its cache slot, one without reads "
                             "another layer's: the schedule entry says otherwise")
        # (a source of values for later layers keeps its product in a buffer that no other layer writes)
        qkv = ws.get("sink_qkv" if self.value_mix != "source" else "sink_qkv:" + self.value_mix_key, (n, self.width), torch.float32)
        ops.linear(h, self.wqkv, self.bqkv, qkv)
        if self.value_mix is not None:
            off_v = (Hq + Hkv) * dk
            if self.value_mix == "source":
                ctx.shared[self.value_mix_key] = (qkv, off_v, Hkv * dv)
            else:
                if self.value_mix_key not in ctx.shared:
                    raise ValueError(f"no earlier layer of this step left its values under {self.value_mix_key!r}")
                src, src_off, src_w = ctx.shared[self.value_mix_key]
                if src_w != Hkv * dv or src.shape[0] != n:
                    raise ValueError(f"the values to blend with have another shape: {src_w} against {Hkv * dv} per row")
                ops.blend_columns(qkv, off_v, src, src_off, Hkv * dv, self.mix_w)
        q = ws.get("sink_q", (n, Hq * dk), ops.dtype)
        pos = ctx.positions[self.position] if self.position is not None else None
        plain = not (self.qk_norm or self.q_temp or self.head_gate) and self.own_kv
        if plain:
            ops.rotate_kv_write(qkv, pos.cos if pos else None, pos.sin if pos else None, self.rotated, PAIRINGS[self.pairing],
                                ctx.meta, cache, q, Hq, Hkv, dk, dv)
        else:
            ops.rotate_kv_write(qkv, pos.cos if pos else None, pos.sin if pos else None, self.rotated, PAIRINGS[self.pairing],
                                ctx.meta, cache, q, Hq, Hkv, dk, dv, q_norm=self.q_norm_w, k_norm=self.k_norm_w,
                                norm_eps=self.norm_eps, query_temperature=self.q_temp)
        o = ws.get("sink_out", (n, Hq * dv), ops.dtype)
        if self.span:
            ops.sink_attention(q, cache, ctx.meta, o, Hq, Hkv, dk, dv, self.scale, self.window, self.keep_first, self.sink,
                               softcap=self.softcap, gate=(qkv, self.off_gate) if self.head_gate else None, span=self.span)
        elif self.softcap or self.head_gate:
            ops.sink_attention(q, cache, ctx.meta, o, Hq, Hkv, dk, dv, self.scale, self.window, self.keep_first, self.sink,
                               softcap=self.softcap, gate=(qkv, self.off_gate) if self.head_gate else None)
        else:
            ops.sink_attention(q, cache, ctx.meta, o, Hq, Hkv, dk, dv, self.scale, self.window, self.keep_first, self.sink)
        delta = ws.get("sink_delta", (n, self.D), torch.float32)
        ops.linear(o, self.wo, self.bo, delta)
        return delta
