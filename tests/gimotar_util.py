"""Small Gimotar configurations shared by the CPU and GPU tests of that design.

They differ from one another in every size and constant and keep apart what a model could make equal: key, rotated and
value sizes unequal, the latent no multiple of 32, grouped and ungrouped heads, chunks shorter and longer than a page,
heads rotated in part and in whole, with and without scaled frequencies, one and several parts of the recurrence's
gates, two to five taps, every order of the three layer types, layers without feed-forward and without a shared expert,
one, two and three layers that blend their values."""
from __future__ import annotations
import copy
import os

import numpy as np
import torch


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def rglru(width, blocks, conv):
    return "rglru", {"width": width, "blocks": blocks, "conv": conv}


def latent(heads, dim, rot_dim, vdim, rank, scale, r):
    return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": r}


def att(heads, kv, dim, vdim, scale, size=None, r=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if r:
        m["rot"] = r
    if v_mix:
        m["v_mix"] = True
    return "attention", m


def moe(experts, top, ff, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def model(vocab, width, eps, mult, scale, bigram, layers):
    return {"architecture": "Gimotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": scale, "bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}, "layers": layers}


GIM_MIX = model(173, 64, 1e-5, 0.4, 6.0, (97, 7, 3), [      # attention first; the recurrence in the middle; two blending layers
    layer(att(4, 2, 16, 8, 0.3, 9, rot(5000.0, 8), v_mix=True), moe(5, 2, 24, 16)),
    layer(rglru(48, 3, 4), moe(4, 1, 16)),
    layer(latent(3, 8, 4, 12, 20, 0.4, rot(100.0, 4, (4.0, 16, 4.0, 0.5))), moe(6, 6, 8, 24)),
    layer(att(2, 2, 24, 8, 0.25, 5, rot(300.0, 24), v_mix=True)),
])
GIM_ODD = model(89, 96, 1e-6, 1.0, 1.0, (211, 1, 13), [     # the recurrence first; no scale, no multiplier; a chunk longer than the sequence
    layer(rglru(40, 1, 2), moe(3, 2, 20, 12)),
    layer(latent(5, 12, 6, 10, 36, 0.2, rot(10000.0, 6)), None),
    layer(att(6, 2, 12, 20, 0.35, 300, None, v_mix=True), moe(7, 3, 12)),
    layer(att(3, 3, 8, 24, 0.2, 7, rot(50.0, 2), v_mix=False), moe(2, 1, 8, 8)),
    layer(att(4, 2, 20, 20, 0.3, None, rot(250000.0, 10), v_mix=True), None),
    layer(rglru(56, 7, 5), None),
    layer(att(2, 2, 16, 20, 0.3, 16, rot(20.0, 16), v_mix=True), moe(4, 2, 8, 4)),
])
GIM_ONE = model(61, 32, 1e-4, 0.3, 2.5, (30, 5, 1), [        # single heads; one layer of each kind; one blending layer alone
    layer(latent(1, 16, 8, 16, 8, 0.25, rot(20.0, 8, (8.0, 64, 2.0, 1.0))), moe(1, 1, 40)),
    layer(att(1, 1, 32, 16, 0.25, 33, rot(1000.0, 32), v_mix=True), moe(3, 1, 16, 16)),
    layer(rglru(32, 32, 3), moe(2, 2, 24, 8)),
])
CONFIGS = {"mix": (GIM_MIX, 3), "odd": (GIM_ODD, 5), "one": (GIM_ONE, 9)}
STD_SCALE = 5.0


def drawn_config(seed: int, small: bool = True) -> dict:
    """A configuration drawn from a seed: the three layer types in any order, odd and even sizes (the tensor-core
    kernels' 64 and 128 among them), with and without feed-forward, shared expert, chunks, rotation and blending."""
    rng = np.random.default_rng((1000 if small else 5000) + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers = []
    kv_mix = (int(pick(1, 2)), int(pick(8, 24) if small else pick(32, 64, 128)))
    kinds = ["rglru", "latent_attention", "attention"] + [pick("rglru", "latent_attention", "attention", "attention")
                                                          for _ in range(int(rng.integers(0, 4)))]
    rng.shuffle(kinds)
    for kind in kinds:
        mlp = None
        if rng.random() < 0.75:
            e = int(pick(1, 3, 8))
            mlp = moe(e, int(pick(1, min(2, e), e)), int(pick(8, 20, 32) if small else pick(64, 96, 200)), int(pick(0, 16, 40) if small else pick(0, 128)))
        if kind == "rglru":
            b = int(pick(1, 2, 4))
            layers.append(layer(rglru(b * int(pick(6, 8, 20) if small else pick(40, 64, 96)), b, int(pick(2, 3, 4, 5))), mlp))
        elif kind == "latent_attention":
            dr = int(pick(2, 8, 12) if small else pick(16, 32, 64))
            sc = pick(None, (4.0, 16, 4.0, 0.5), (2.0, 2048, 32.0, 1.0))
            layers.append(layer(latent(int(pick(1, 2, 5)), int(pick(8, 12, 16) if small else pick(32, 64, 128)), dr,
                                       int(pick(8, 12, 24) if small else pick(48, 64, 128)), int(pick(12, 16, 40) if small else pick(64, 96, 256)),
                                       float(pick(0.1, 0.3)), rot(float(pick(50.0, 10000.0)), int(pick(2, dr)), sc)), mlp))
        else:
            mixing = rng.random() < 0.6
            kv, dv = (kv_mix if mixing else (int(pick(1, 3)), int(pick(8, 12, 40) if small else pick(48, 64, 128))))
            dk = int(pick(8, 12, 16, 40) if small else pick(48, 64, 96, 128))
            if not small and dk in (64, 128) and rng.random() < 0.5 and not mixing:
                dv = dk
            r = pick(None, rot(float(pick(50.0, 250000.0)), int(pick(2, dk, dk // 4 * 2 or 2))))
            layers.append(layer(att(kv * int(pick(1, 2, 4)), kv, dk, dv, float(pick(0.1, 0.3)),
                                    pick(None, 1, 3, 7, 16, 33) if small else pick(None, 17, 64, 96, 200), r, mixing), mlp))
    return model(int(pick(37, 64, 150) if small else pick(300, 512, 777)), int(pick(24, 40, 56, 72) if small else pick(192, 200, 256, 384)),
                 float(pick(1e-6, 1e-5)), float(pick(0.25, 0.5, 1.0)), float(pick(1.0, 3.0, 11.0)),
                 (int(pick(1, 31, 1021)), int(pick(0, 1, 31)), int(pick(1, 17))), layers)


def make_dir(name: str, tmp, cfg: dict | None = None, seed: int | None = None, change=None, dtype: str = "float32") -> tuple[str, dict, dict]:
    """Writes configuration `name` with seeded random weights; `change(tensors)` may edit them before they are written.
    Returns (folder, config, weights by name)."""
    from fusezap_core_b200.weights import write_random_model
    from fusezap_core_b200.weights.safetensors_io import read_model_dir, write_file
    base, s = CONFIGS.get(name, (cfg, seed))
    cfg = copy.deepcopy(cfg if cfg is not None else base)
    d = os.path.join(str(tmp), f"gimotar-{name}")
    write_random_model(cfg, d, seed if seed is not None else s, dtype, norm_noise=True, std_scale=STD_SCALE)
    w = read_model_dir(d)
    if change is not None:
        w = {k: v.clone() for k, v in w.items()}
        change(w)
        write_file(os.path.join(d, "model.safetensors"), w)
    return d, cfg, w


def tokens_for(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], n).tolist() for n in lengths]


def plain_logits(cfg: dict, w: dict, toks) -> np.ndarray:
    import plain_gimotar
    w = {k: v.double() for k, v in w.items()}
    for n, L in enumerate(cfg["layers"]):      # a source layer's own blend weight is never read: the oracle may lack it
        w.setdefault(f"l{n}.mix.vmix", torch.zeros((), dtype=torch.float64))
    return plain_gimotar.forward(cfg, w, list(toks)).numpy()


def rounded(w: dict) -> dict:
    """The weights as a bfloat16 engine holds them: matrices rounded once, vectors stored in 32-bit as they are."""
    return {k: v.to(torch.bfloat16).to(torch.float32) if v.dim() >= 2 else v for k, v in w.items()}
