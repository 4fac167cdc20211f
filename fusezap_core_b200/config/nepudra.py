"""Typed configuration of the Nepudra decoder, read from its own config.json keys, and its model description.

config.json: `architecture` "Nepudra"; `vocab`, `width`; `norm.eps`; `embedding.bigram` (`buckets`, `mul_prev`,
`mul_cur`); `layers`: a list whose entries give `type` (the mixer kind: "attention", "attention_2" or "general_delta"),
`mixer` (its sizes and constants) and `mlp` (`kind` "dense" with `ff`, or null for none). Tensor names: `embed`,
`bigram`, `final.norm`, `head`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.dwa`.

What the design is made of (every piece is a part of this package that another design can name with other constants):

  embedding      the token's row plus a row of a second table chosen by a hash of (previous token, token)
                 (embedding extra `hashed_pair`; the previous token is request state)
  layer          block `depth_average` around `pre_norm`: x <- x + mixer(norm1(x)); x <- x + ff(norm2(x)); the result
                 X_(i+1) is kept, and what the next layer reads is sum_j c_i[j] X_j over j = 0 .. i+1 (X_0: the
                 embedding's output, c_i: the layer's tensor `dwa`)
  norm           `rmsnorm` with `scalar`: one learned number for all coordinates
  attention      mixer `sink_attention` without sink or rotation: biases on q, k, v and the output product, q times
                 1 + coef ln(floor((p + 1) / every) + 1) at position p, scores capped by cap tanh(s / cap), all earlier
                 keys, a sigmoid gate per head; a layer with `kv_from` j reads layer j's cache with queries of its own
  attention_2    the same mixer with biases on q, k, v, per-head RMS norms of q and k with a weight, rotated halves with
                 YaRN-scaled frequencies (`rope` kind "yarn") on the first `rot.dims` dimensions, a sliding window and
                 the gate per head
  general_delta  mixer `general_delta`: S <- diag(d) S - (a u)(u^T S) + k v^T per head, o = S^T r, with d =
                 exp(-rate sigmoid(W_w2 tanh(W_w1 h) + w0)), a = sigmoid(W_a h + b), u the unit key; o divided by its
                 root mean square per head, times a weight and a sigmoid gate; S is request state in 32-bit
  feed-forward   `swiglu` with the tanh form of gelu as its activation
  output         the model's scalar norm, then the output matrix `head`
"""
from __future__ import annotations
import math
from dataclasses import dataclass
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_KINDS = ("attention", "attention_2", "general_delta")
DECAY_RATE = math.exp(-0.5)     # the factor in the exponent of the delta rule's decay: fixed by the design
UNIT_EPS = 1e-6                 # inside the root of the unit key's norm: fixed by the design
YARN_MAGNITUDE = 0.1            # cos and sin are multiplied by YARN_MAGNITUDE * ln(factor) + 1: fixed by the design


def _need(m: dict, keys: tuple, where: str) -> None:
    missing = [k for k in keys if k not in m]
    if missing:
        raise ValueError(f"config.json: {where} lacks {missing}")


@dataclass(frozen=True)
class YarnRotation:
    base: float
    dims: int
    scaling: tuple | None = None        # (factor, original, fast, slow) or None

    @staticmethod
    def from_json(r: dict, dim: int, where: str) -> "YarnRotation":
        _need(r, ("base", "dims"), where + ".rot")
        sc = r.get("scaling")
        if sc is not None:
            _need(sc, ("factor", "original", "fast", "slow"), where + ".rot.scaling")
            sc = (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
            if sc[0] <= 0 or sc[1] <= 0 or sc[2] <= 0 or sc[3] <= 0:
                raise ValueError(f"config.json: {where}.rot.scaling: factor, original, fast and slow must be positive")
        out = YarnRotation(float(r["base"]), int(r["dims"]), sc)
        if out.dims % 2 or not 0 < out.dims <= dim:
            raise ValueError(f"config.json: {where}.rot.dims {out.dims} must be even, positive and at most dim {dim}")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return out

    def name(self) -> str:
        return f"yarn{self.dims}@{self.base!r}" + (f"~{self.scaling!r}" if self.scaling else "")

    def spec(self) -> PartSpec:
        p: dict[str, Any] = {"head_dim": self.dims, "theta": self.base, "precise": True}
        if self.scaling is not None:
            f, orig, fast, slow = self.scaling
            p.update(kind="yarn", factor=f, original_max_position_embeddings=orig, turns_fast=fast, turns_slow=slow,
                     magnitude=YARN_MAGNITUDE * math.log(f) + 1.0)
        return PartSpec("rope", p)


@dataclass(frozen=True)
class AttentionConfig:
    """Both attention kinds; what a kind does not have is None / 0 / False."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                      # 0: every earlier key
    softcap: float = 0.0                 # 0: scores are not capped
    q_temp: tuple | None = None          # (coef, every)
    rot: YarnRotation | None = None
    qk_norm: bool = False
    out_bias: bool = False
    kv_from: int | None = None

    @staticmethod
    def from_json(kind: str, m: dict, where: str) -> "AttentionConfig":
        _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
        qt = m.get("q_temp")
        if qt is not None:
            _need(qt, ("coef", "every"), where + ".q_temp")
            qt = (float(qt["coef"]), int(qt["every"]))
            if qt[1] <= 0:
                raise ValueError(f"config.json: {where}.q_temp.every must be positive")
        mask = m.get("mask")
        if mask is not None:
            _need(mask, ("size",), where + ".mask")
        rot = YarnRotation.from_json(m["rot"], int(m["dim"]), where) if m.get("rot") is not None else None
        second = kind == "attention_2"
        out = AttentionConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                              int(mask["size"]) if mask is not None else 0, float(m.get("softcap") or 0.0), qt, rot,
                              qk_norm=second, out_bias=not second,
                              kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else None)
        if min(out.heads, out.kv_heads, out.dim, out.vdim) <= 0 or out.heads % out.kv_heads:
            raise ValueError(f"config.json: {where}: heads must be a positive multiple of kv_heads, dim and vdim positive")
        if out.window < 0 or (mask is not None and out.window == 0):
            raise ValueError(f"config.json: {where}.mask.size must be positive")
        if out.softcap < 0:
            raise ValueError(f"config.json: {where}.softcap must be positive")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                               "vdim": self.vdim}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        if self.window:
            out["mask"] = {"size": self.window}
        if self.q_temp is not None:
            out["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        if self.softcap:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class GeneralDeltaConfig:
    heads: int
    dim: int

    @staticmethod
    def from_json(m: dict, where: str) -> "GeneralDeltaConfig":
        _need(m, ("heads", "dim"), where)
        out = GeneralDeltaConfig(int(m["heads"]), int(m["dim"]))
        if min(out.heads, out.dim) <= 0:
            raise ValueError(f"config.json: {where}: heads and dim must be positive")
        return out

    def to_json(self) -> dict:
        return {"dim": self.dim, "heads": self.heads}


@dataclass(frozen=True)
class NepudraLayer:
    type: str
    mixer: Any                     # AttentionConfig | GeneralDeltaConfig
    ff: int                        # 0: the layer has no feed-forward


@dataclass(frozen=True)
class NepudraConfig:
    vocab: int
    width: int
    norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: tuple
    max_position: int = 1 << 17      # positions are not bounded by the design; the engine sizes its tables itself

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("config: vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError(f"config: norm.eps must be positive, got {self.norm_eps!r}")
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("config: embedding.bigram needs positive buckets and multipliers that are not negative")
        for i, L in enumerate(self.layers):
            j = getattr(L.mixer, "kv_from", None)
            if j is None:
                continue
            if not 0 <= j < i or self.layers[j].type == "general_delta" or self.layers[j].mixer.kv_from is not None:
                raise ValueError(f"config: layers[{i}].mixer.kv_from {j} must name an earlier attention layer with "
                                 f"projections of its own")
            a, b = L.mixer, self.layers[j].mixer
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ValueError(f"config: layers[{i}] reads the keys and values of layers[{j}], whose sizes differ")

    @staticmethod
    def from_json(c: dict) -> "NepudraConfig":
        _need(c, ("vocab", "width", "layers", "norm", "embedding"), "the top level")
        _need(c["norm"], ("eps",), "norm")
        _need(c["embedding"], ("bigram",), "embedding")
        b = c["embedding"]["bigram"]
        _need(b, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
        layers = []
        for i, L in enumerate(c["layers"]):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise NotImplementedError(f"config.json: {where}.type {kind!r} is not supported (have {list(MIXER_KINDS)})")
            _need(L, ("mixer",), where)
            if kind == "general_delta":
                mixer: Any = GeneralDeltaConfig.from_json(L["mixer"], where + ".mixer")
            else:
                mixer = AttentionConfig.from_json(kind, L["mixer"], where + ".mixer")
            mlp = L.get("mlp")
            ff = 0
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise NotImplementedError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not supported (have ['dense'])")
                _need(mlp, ("ff",), where + ".mlp")
                ff = int(mlp["ff"])
                if ff <= 0:
                    raise ValueError(f"config.json: {where}.mlp.ff must be positive")
            layers.append(NepudraLayer(kind, mixer, ff))
        return NepudraConfig(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), int(b["buckets"]),
                             int(b["mul_prev"]), int(b["mul_cur"]), tuple(layers), int(c.get("max_position", 1 << 17)))

    def to_json(self) -> dict:
        return {"architecture": "Nepudra",
                "embedding": {"bigram": {"buckets": self.buckets, "mul_cur": self.mul_cur, "mul_prev": self.mul_prev}},
                "layers": [{"mixer": L.mixer.to_json(), "mlp": {"ff": L.ff, "kind": "dense"} if L.ff else None, "type": L.type}
                           for L in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def random_optional_groups(self, expected: dict) -> set:
        return {"lm_head"}

    # ---- the model description
    def _cache_window(self, owner: int) -> int:
        """The window the cache of layer `owner` must keep: the widest among the layers that read it (0: everything)."""
        widths = [L.mixer.window for i, L in enumerate(self.layers)
                  if L.type != "general_delta" and (i == owner or L.mixer.kv_from == owner)]
        return 0 if 0 in widths else max(widths)

    def _attention(self, i: int, a: AttentionConfig, positions: dict) -> PartSpec:
        if a.rot is not None:
            positions.setdefault(a.rot.name(), a.rot.spec())
        owner = i if a.kv_from is None else a.kv_from
        return PartSpec("sink_attention", {
            "hidden_size": self.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "key_dim": a.dim,
            "value_dim": a.vdim, "scale": a.scale, "window": a.window, "keep_first": 0, "sink": False,
            "rotated": a.rot.dims if a.rot is not None else 0, "pairing": "halves",
            "position": a.rot.name() if a.rot is not None else None,
            "bias": ("q", "k", "v", "out") if a.out_bias else ("q", "k", "v"), "bias_suffix": ".b",
            "qk_norm": a.qk_norm, "norm_eps": self.norm_eps, "norm_suffix": ".norm", "query_temperature": a.q_temp,
            "softcap": a.softcap, "head_gate": True, "own_kv": a.kv_from is None, "cache_window": self._cache_window(owner),
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}})

    def _general_delta(self, d: GeneralDeltaConfig) -> PartSpec:
        return PartSpec("general_delta", {
            "hidden_size": self.width, "num_heads": d.heads, "key_dim": d.dim, "value_dim": d.dim,
            "decay_rate": DECAY_RATE, "unit_eps": UNIT_EPS, "eps": self.norm_eps,
            "names": {"r": "r", "k": "k", "v": "v", "gate": "g", "remove": "a", "remove_bias": "a.b", "decay_in": "w1",
                      "decay_out": "w2", "decay_bias": "w0", "norm": "norm", "out": "o"}})

    def spec(self) -> ModelSpec:
        D = self.width
        def norm() -> PartSpec:
            return PartSpec("rmsnorm", {"size": D, "eps": self.norm_eps, "name": "", "scalar": True})
        positions: dict[str, PartSpec] = {}
        layers, schedule = [], []
        n_layers = len(self.layers)
        for i, L in enumerate(self.layers):
            mixer = self._general_delta(L.mixer) if L.type == "general_delta" else self._attention(i, L.mixer, positions)
            ffn = None
            if L.ff:
                ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": L.ff, "names": ("gate", "up", "down"),
                                          "suffix": "", "activation": "gelu_tanh"})
            inner = PartSpec("pre_norm", {"names": ("norm1", "mix", "norm2", "mlp"), "norms": (norm(), norm())})
            block = PartSpec("depth_average", {"inner": inner, "depth": i, "depths": n_layers, "hidden_size": D, "name": "dwa"})
            layers.append(LayerSpec(f"l{i}.", block, mixer, ffn))
            kv_from = getattr(L.mixer, "kv_from", None)
            schedule.append(ScheduleEntry(i, i if kv_from is None else kv_from, write_cache=kv_from is None))
        final = PartSpec("rmsnorm", {"size": D, "eps": self.norm_eps, "name": "norm", "scalar": True})
        extra = PartSpec("hashed_pair", {"hidden_size": D, "buckets": self.buckets, "mul_prev": self.mul_prev,
                                         "mul_cur": self.mul_cur, "name": "bigram"})
        return ModelSpec(
            architecture="Nepudra", hidden_size=D, vocab_size=self.vocab, embed_name="embed", lm_head_name="head",
            tie_embeddings=False, final_norm=final, final_norm_name="final.norm", layers=tuple(layers),
            schedule=tuple(schedule), positions=positions, max_position=self.max_position, embed_extras=(extra,))
