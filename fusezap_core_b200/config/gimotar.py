"""Typed configuration of the Gimotar decoder, read from its own config.json keys, and its model description.

config.json: `architecture` "Gimotar"; `vocab`, `width`; `norm.eps`; `residual_mult`; `embedding.scale` and
`embedding.bigram` (`buckets`, `mul_prev`, `mul_cur`); `layers`: a list whose entries give `type` (the mixer kind:
"rglru", "latent_attention" or "attention"), `mixer` (its sizes and constants) and `mlp` (`kind` "moe" with `expert.ff`,
`router.experts`, `router.top` and optionally `shared.ff`, or null for none). Tensor names: `embed`, `bigram`,
`final.norm`, and per layer i `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`. The output matrix is the embedding table.

What the design is made of (every piece is a part of this package that another design can name with other constants):

  embedding         the token's row times `embedding.scale`, plus a row of a second table chosen by a hash of (previous
                    token, token) (embedding extra `hashed_pair`; the previous token is request state)
  layer             block `parallel_shared`: h = norm1(x); x <- x + m (mixer(h) + ff(h)), m = `residual_mult`
  norm              `rmsnorm` with `offset` 1: the stored weight is the distance from one
  rglru             mixer `rglru`: two branches of `width` channels, y = gelu_tanh(W_y h + b) and u = conv(W_x h + b) (a
                    short causal convolution with a bias); gates r, i = sigmoid of block-diagonal products of u; a =
                    exp(-c r softplus(lam)), S <- a S + sqrt(1 - a^2) i u in 32-bit request state; W_o (S y)
  latent_attention  mixer `latent_attention`: a cached latent and one rotated key part shared by the heads, neighbouring
                    dimensions paired in the rotation, YaRN-scaled frequencies, a sink in the softmax and an output gate
                    sigmoid(W_g h) on the concatenated heads
  attention         mixer `sink_attention` without a sink: per-head RMS norms of q and k, rotated halves on the first
                    `rot.dims` dimensions, a chunked causal mask (`span`), and the values blended with those of the
                    first such layer (`value_mix`)
  feed-forward      `routed_moe`: router logits with a bias, the `top` largest, softmax over the chosen, a shared expert
  output            the model's norm, then the embedding table (without its scale) as output matrix
"""
from __future__ import annotations
import math
from dataclasses import dataclass
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_KINDS = ("rglru", "latent_attention", "attention")
DECAY_SHARPNESS = 8.0           # log a = -DECAY_SHARPNESS * r * softplus(lam): fixed by the design
YARN_MAGNITUDE = 0.1            # cos and sin are multiplied by YARN_MAGNITUDE * ln(factor) + 1: fixed by the design
VALUE_MIX_KEY = "first_values"  # under which a step keeps the first mixing layer's values for the later ones


def _need(m: dict, keys: tuple, where: str) -> None:
    missing = [k for k in keys if k not in m]
    if missing:
        raise ValueError(f"config.json: {where} lacks {missing}")


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: tuple | None = None        # (factor, original, fast, slow) or None

    @staticmethod
    def from_json(r: dict, dim: int, where: str) -> "Rotation":
        _need(r, ("base", "dims"), where + ".rot")
        sc = r.get("scaling")
        if sc is not None:
            _need(sc, ("factor", "original", "fast", "slow"), where + ".rot.scaling")
            sc = (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
            if min(sc) <= 0:
                raise ValueError(f"config.json: {where}.rot.scaling: factor, original, fast and slow must be positive")
        out = Rotation(float(r["base"]), int(r["dims"]), sc)
        if out.dims % 2 or not 0 < out.dims <= dim:
            raise ValueError(f"config.json: {where}.rot.dims {out.dims} must be even, positive and at most {dim}")
        if not out.base > 0 or out.base == 1.0:
            raise ValueError(f"config.json: {where}.rot.base must be positive and not 1")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return out

    def name(self) -> str:
        return f"rot{self.dims}@{self.base!r}" + (f"~{self.scaling!r}" if self.scaling else "")

    def spec(self) -> PartSpec:
        p: dict[str, Any] = {"head_dim": self.dims, "theta": self.base, "precise": True}
        if self.scaling is not None:
            f, orig, fast, slow = self.scaling
            p.update(kind="yarn", factor=f, original_max_position_embeddings=orig, turns_fast=fast, turns_slow=slow,
                     magnitude=YARN_MAGNITUDE * math.log(f) + 1.0)
        return PartSpec("rope", p)


@dataclass(frozen=True)
class RglruConfig:
    width: int
    blocks: int
    conv: int

    @staticmethod
    def from_json(m: dict, where: str) -> "RglruConfig":
        _need(m, ("width", "blocks", "conv"), where)
        out = RglruConfig(int(m["width"]), int(m["blocks"]), int(m["conv"]))
        if out.width <= 0 or out.blocks <= 0 or out.width % out.blocks or out.conv < 1:
            raise ValueError(f"config.json: {where}: width must be a positive multiple of blocks, conv at least 1")
        return out

    def to_json(self) -> dict:
        return {"blocks": self.blocks, "conv": self.conv, "width": self.width}


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotation

    @staticmethod
    def from_json(m: dict, where: str) -> "LatentConfig":
        _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), where)
        out = LatentConfig(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]),
                           float(m["scale"]), Rotation.from_json(m["rot"], int(m["rot_dim"]), where))
        if min(out.heads, out.dim, out.rot_dim, out.vdim, out.kv_rank) <= 0:
            raise ValueError(f"config.json: {where}: heads, dim, rot_dim, vdim and kv_rank must be positive")
        return out

    def to_json(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot": self.rot.to_json(),
                "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    span: int = 0                        # 0: every earlier key; else a position sees its own block of `span` positions
    rot: Rotation | None = None
    v_mix: bool = False

    @staticmethod
    def from_json(m: dict, where: str) -> "AttentionConfig":
        _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
        mask = m.get("mask")
        if mask is not None:
            _need(mask, ("size",), where + ".mask")
        rot = Rotation.from_json(m["rot"], int(m["dim"]), where) if m.get("rot") is not None else None
        out = AttentionConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                              int(mask["size"]) if mask is not None else 0, rot, bool(m.get("v_mix", False)))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) <= 0 or out.heads % out.kv_heads:
            raise ValueError(f"config.json: {where}: heads must be a positive multiple of kv_heads, dim and vdim positive")
        if out.span < 0 or (mask is not None and out.span == 0):
            raise ValueError(f"config.json: {where}.mask.size must be positive")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                               "vdim": self.vdim}
        if self.span:
            out["mask"] = {"size": self.span}
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        if self.v_mix:
            out["v_mix"] = True
        return out


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int = 0                   # 0: no shared expert

    @staticmethod
    def from_json(m: dict, where: str) -> "MoEConfig":
        if m.get("kind") != "moe":
            raise NotImplementedError(f"config.json: {where}.kind {m.get('kind')!r} is not supported (have ['moe'])")
        _need(m, ("expert", "router"), where)
        _need(m["expert"], ("ff",), where + ".expert")
        _need(m["router"], ("experts", "top"), where + ".router")
        shared = m.get("shared")
        if shared is not None:
            _need(shared, ("ff",), where + ".shared")
        out = MoEConfig(int(m["router"]["experts"]), int(m["router"]["top"]), int(m["expert"]["ff"]),
                        int(shared["ff"]) if shared is not None else 0)
        if out.ff <= 0 or out.shared_ff < 0 or not 0 < out.top <= out.experts:
            raise ValueError(f"config.json: {where}: ff must be positive and top lie in 1..experts")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class GimotarLayer:
    type: str
    mixer: Any                     # RglruConfig | LatentConfig | AttentionConfig
    mlp: MoEConfig | None


@dataclass(frozen=True)
class GimotarConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embed_scale: float
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
        mixing = [L.mixer for L in self.layers if L.type == "attention" and L.mixer.v_mix]
        if any((a.kv_heads, a.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for a in mixing):
            raise ValueError("config: the layers that mix their values with the first one's need values of one shape")

    @staticmethod
    def from_json(c: dict) -> "GimotarConfig":
        _need(c, ("vocab", "width", "layers", "norm", "embedding", "residual_mult"), "the top level")
        _need(c["norm"], ("eps",), "norm")
        _need(c["embedding"], ("bigram", "scale"), "embedding")
        b = c["embedding"]["bigram"]
        _need(b, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
        layers = []
        for i, L in enumerate(c["layers"]):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise NotImplementedError(f"config.json: {where}.type {kind!r} is not supported (have {list(MIXER_KINDS)})")
            _need(L, ("mixer",), where)
            make = {"rglru": RglruConfig, "latent_attention": LatentConfig, "attention": AttentionConfig}[kind]
            mixer = make.from_json(L["mixer"], where + ".mixer")
            mlp = MoEConfig.from_json(L["mlp"], where + ".mlp") if L.get("mlp") is not None else None
            layers.append(GimotarLayer(kind, mixer, mlp))
        return GimotarConfig(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), float(c["residual_mult"]),
                             float(c["embedding"]["scale"]), int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"]),
                             tuple(layers), int(c.get("max_position", 1 << 17)))

    def to_json(self) -> dict:
        return {"architecture": "Gimotar",
                "embedding": {"bigram": {"buckets": self.buckets, "mul_cur": self.mul_cur, "mul_prev": self.mul_prev},
                              "scale": self.embed_scale},
                "layers": [{"mixer": L.mixer.to_json(), "mlp": L.mlp.to_json() if L.mlp is not None else None, "type": L.type}
                           for L in self.layers],
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    def random_optional_groups(self, expected: dict) -> set:
        return set()

    # ---- the model description
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name, "offset": 1.0})

    def _rglru(self, r: RglruConfig) -> PartSpec:
        return PartSpec("rglru", {
            "hidden_size": self.width, "width": r.width, "blocks": r.blocks, "taps": r.conv, "sharpness": DECAY_SHARPNESS,
            "names": {"gate_branch": "y", "in": "x", "conv": "conv", "recur_gate": "ra", "input_gate": "ri", "decay": "lam",
                      "out": "o", "bias": "b"}})

    def _latent(self, a: LatentConfig, positions: dict) -> PartSpec:
        positions.setdefault(a.rot.name(), a.rot.spec())
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": a.heads, "nope_dim": a.dim, "rope_dim": a.rot_dim, "value_dim": a.vdim,
            "latent_dim": a.kv_rank, "scale": a.scale, "rotated": a.rot.dims, "eps": self.norm_eps,
            "position": a.rot.name(), "pairing": "neighbours", "sink": True, "out_gate": True,
            "names": {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "out": "o",
                      "sink": "sink", "gate": "g"}})

    def _attention(self, a: AttentionConfig, positions: dict, mix: str | None) -> PartSpec:
        if a.rot is not None:
            positions.setdefault(a.rot.name(), a.rot.spec())
        return PartSpec("sink_attention", {
            "hidden_size": self.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "key_dim": a.dim,
            "value_dim": a.vdim, "scale": a.scale, "window": 0, "keep_first": 0, "sink": False, "span": a.span,
            "rotated": a.rot.dims if a.rot is not None else 0, "pairing": "halves",
            "position": a.rot.name() if a.rot is not None else None,
            "qk_norm": True, "norm_eps": self.norm_eps, "norm_suffix": ".norm",
            "value_mix": mix, "value_mix_key": VALUE_MIX_KEY,
            "names": {"q": "q", "k": "k", "v": "v", "out": "o", "value_mix": "vmix"}})

    def _moe(self, m: MoEConfig) -> PartSpec:
        return PartSpec("routed_moe", {
            "hidden_size": self.width, "intermediate_size": m.ff, "num_experts": m.experts, "top": m.top,
            "shared_size": m.shared_ff, "renormalize": True, "router_bias": True, "shared_gate": False,
            "names": {"router": "router", "router_bias": "router.b", "expert": "e{}", "gate": "gate", "up": "up",
                      "down": "down", "shared": "shared"}})

    def spec(self) -> ModelSpec:
        positions: dict[str, PartSpec] = {}
        layers, schedule = [], []
        seen_mix = False
        for i, L in enumerate(self.layers):
            if L.type == "rglru":
                mixer = self._rglru(L.mixer)
            elif L.type == "latent_attention":
                mixer = self._latent(L.mixer, positions)
            else:
                mix = None
                if L.mixer.v_mix:
                    mix = "blend" if seen_mix else "source"
                    seen_mix = True
                mixer = self._attention(L.mixer, positions, mix)
            block = PartSpec("parallel_shared", {"hidden_size": self.width, "residual_mult": self.residual_mult,
                                                 "norm": self._norm(""), "names": ("norm1", "mix", "mlp")})
            layers.append(LayerSpec(f"l{i}.", block, mixer, self._moe(L.mlp) if L.mlp is not None else None))
            schedule.append(ScheduleEntry(i, i))
        extra = PartSpec("hashed_pair", {"hidden_size": self.width, "buckets": self.buckets, "mul_prev": self.mul_prev,
                                         "mul_cur": self.mul_cur, "name": "bigram"})
        return ModelSpec(
            architecture="Gimotar", hidden_size=self.width, vocab_size=self.vocab, embed_name="embed", lm_head_name=None,
            tie_embeddings=True, final_norm=self._norm("norm"), final_norm_name="final.norm", layers=tuple(layers),
            schedule=tuple(schedule), positions=positions, max_position=self.max_position, embed_scale=self.embed_scale,
            embed_extras=(extra,))
