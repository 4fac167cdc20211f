"""Small Nepudra configurations shared by the CPU and GPU tests of that design.

They differ from one another in every size and constant and keep apart what a model could make equal: key and value
sizes unequal, heads rotated in part and in whole, grouped and ungrouped heads, windows shorter and longer than a page,
temperature periods of a few tokens, caps near the scores' size, every order of the three layer types, layers without
feed-forward, a cache read by one and by two later layers, with and without frequency scaling."""
from __future__ import annotations
import copy
import os

import numpy as np
import torch


def _att(heads, kv, dim, vdim, scale, coef, every, cap, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "q_temp": {"coef": coef, "every": every},
         "softcap": cap}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _att2(heads, kv, dim, vdim, scale, size, base, dims, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}, "rot": rot}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


NEP_MIX = {       # window first; a cache read by a later layer; the recurrence in the middle; partly rotated heads
    "architecture": "Nepudra", "vocab": 173, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 7, "mul_cur": 3}},
    "layers": [
        _layer("attention_2", _att2(4, 2, 16, 8, 0.3, 9, 5000.0, 8, (4.0, 16, 4.0, 0.5)), 48),
        _layer("attention", _att(4, 1, 8, 24, 0.4, 0.7, 5, 2.5), 40),
        _layer("general_delta", {"heads": 2, "dim": 12}, 0),
        _layer("attention", _att(4, 1, 8, 24, 0.25, 0.3, 3, 4.0, kv_from=1), 24),
    ]}
NEP_ODD = {       # the recurrence first; sizes that are no multiples of 16; ungrouped heads; a window shorter than a page;
                  # unscaled frequencies on whole heads; two readers of one cache; an attention layer without feed-forward
    "architecture": "Nepudra", "vocab": 89, "width": 96, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 211, "mul_prev": 1, "mul_cur": 13}},
    "layers": [
        _layer("general_delta", {"heads": 3, "dim": 20}, 56),
        _layer("attention", _att(3, 3, 24, 40, 0.2, 1.5, 7, 1.0), 0),
        _layer("attention_2", _att2(2, 2, 12, 20, 0.35, 5, 300.0, 12), 24),
        _layer("attention", _att(3, 3, 24, 40, 0.15, 0.1, 2, 30.0, kv_from=1), 32),
        _layer("attention", _att(3, 3, 24, 40, 0.3, 0.9, 11, 0.75, kv_from=1), 0),
    ]}
NEP_ONE = {       # a single head everywhere; a long window; one layer of each kind
    "architecture": "Nepudra", "vocab": 61, "width": 32, "norm": {"eps": 1e-4},
    "embedding": {"bigram": {"buckets": 30, "mul_prev": 5, "mul_cur": 1}},
    "layers": [
        _layer("attention", _att(1, 1, 32, 16, 0.25, 0.4, 4, 6.0), 40),
        _layer("attention_2", _att2(6, 1, 8, 8, 0.35, 33, 20.0, 2, (8.0, 64, 2.0, 1.0)), 0),
        _layer("general_delta", {"heads": 1, "dim": 40}, 16),
    ]}
CONFIGS = {"mix": (NEP_MIX, 3), "odd": (NEP_ODD, 5), "one": (NEP_ONE, 9)}
STD_SCALE = 5.0


def drawn_config(seed: int) -> dict:
    """A configuration drawn from a seed: odd and even sizes, the three layer types in any order, grouped and ungrouped
    heads, key and value sizes equal and unequal (the sizes 64 and 128 among them), heads rotated in part and in whole
    with and without scaled frequencies, windows from a few tokens to longer than the sequence, temperature periods of
    one token and more, caps below and above the scores, caches read by later layers, layers without feed-forward."""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers, owners = [], []
    for i in range(int(rng.integers(2, 7))):
        ff = int(pick(0, 16, 36, 64))
        kind = pick("attention", "attention", "attention_2", "general_delta")
        if kind == "general_delta":
            layers.append(_layer(kind, {"heads": int(pick(1, 2, 3)), "dim": int(pick(8, 12, 20, 48, 64))}, ff))
        elif kind == "attention_2":
            kv, dk = int(pick(1, 2, 3)), int(pick(8, 12, 16, 40, 64, 128))
            dims = int(pick(2, dk, dk // 2 // 2 * 2 or 2))
            scaling = pick(None, (4.0, 16, 4.0, 0.5), (8.0, 64, 32.0, 1.0), (2.0, 2048, 32.0, 1.0))
            layers.append(_layer(kind, _att2(kv * int(pick(1, 2, 3)), kv, dk, dk if dk >= 64 else int(pick(4, 8, 12, 40)), float(pick(0.2, 0.35)),
                                             int(pick(1, 3, 7, 16, 64, 200)), float(pick(50.0, 10000.0, 250000.0)), dims, scaling), ff))
        elif owners and rng.random() < 0.4:
            j = int(pick(*owners))
            m = dict(layers[j]["mixer"], scale=float(pick(0.15, 0.3)), softcap=float(pick(0.75, 5.0, 30.0)),
                     q_temp={"coef": float(pick(0.1, 0.5, 1.5)), "every": int(pick(1, 2, 5, 256))}, kv_from=j)
            layers.append(_layer(kind, m, ff))
        else:
            kv, dk = int(pick(1, 2, 3)), int(pick(8, 16, 24, 64, 96, 128))
            owners.append(i)
            layers.append(_layer(kind, _att(kv * int(pick(1, 2, 4)), kv, dk, dk if dk >= 64 else int(pick(8, 24, 40)), float(pick(0.1, 0.25)),
                                            float(pick(0.1, 0.5, 1.5)), int(pick(1, 3, 16, 256)), float(pick(0.75, 5.0, 30.0))), ff))
    return {"architecture": "Nepudra", "vocab": int(pick(37, 64, 150)), "width": int(pick(24, 40, 56, 72, 100)),
            "norm": {"eps": float(pick(1e-6, 1e-5))},
            "embedding": {"bigram": {"buckets": int(pick(1, 31, 1021)), "mul_prev": int(pick(0, 1, 31)), "mul_cur": int(pick(1, 17))}},
            "layers": layers}


def drawn_model_config(seed: int) -> dict:
    """A configuration of a small model's size drawn from a seed: widths of a few hundred that are and are not multiples
    of 64, head sizes from 32 to 128 (equal and unequal for keys and values, the tensor-core kernels' 64 and 128 among
    them), groups of 1 to 6 query heads, windows of tens to hundreds of tokens, every layer type at least once."""
    rng = np.random.default_rng(5000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    kinds = ["attention", "attention_2", "general_delta"] + [pick("attention", "attention_2", "general_delta")
                                                             for _ in range(int(rng.integers(1, 4)))]
    rng.shuffle(kinds)
    layers, owners = [], []
    for i, kind in enumerate(kinds):
        ff = int(pick(0, 128, 200, 384))
        if kind == "general_delta":
            layers.append(_layer(kind, {"heads": int(pick(1, 2, 5, 8)), "dim": int(pick(16, 32, 64, 80, 128))}, ff))
        elif kind == "attention_2":
            kv, dk = int(pick(1, 2, 3)), int(pick(32, 48, 64, 80, 112, 128))
            scaling = pick(None, (8.0, 1024, 16.0, 2.0), (2.0, 128, 8.0, 0.5), (16.0, 4096, 32.0, 1.0))
            layers.append(_layer(kind, _att2(kv * int(pick(1, 2, 3)), kv, dk, int(pick(dk, dk, 32, 64, 128)), float(pick(dk ** -0.5, 0.08)),
                                             int(pick(17, 64, 100, 128, 200)), float(pick(10000.0, 1e6)), int(pick(dk, dk // 2, 16)), scaling), ff))
        elif owners and rng.random() < 0.7:
            j = int(pick(*owners))
            layers.append(_layer(kind, dict(layers[j]["mixer"], scale=float(pick(0.08, 0.12)), softcap=float(pick(5.0, 30.0)),
                                            q_temp={"coef": float(pick(0.1, 1.0)), "every": int(pick(64, 100))}, kv_from=j), ff))
        else:
            kv, dk = int(pick(1, 2, 4)), int(pick(32, 48, 64, 80, 112, 128))
            owners.append(i)
            layers.append(_layer(kind, _att(kv * int(pick(1, 2, 6)), kv, dk, int(pick(dk, dk, 32, 64, 128)), float(pick(dk ** -0.5, 0.08)),
                                            float(pick(0.1, 1.0)), int(pick(64, 100, 512)), float(pick(5.0, 30.0, 50.0))), ff))
    return {"architecture": "Nepudra", "vocab": int(pick(300, 512, 777)), "width": int(pick(192, 200, 256, 264, 384)),
            "norm": {"eps": float(pick(1e-6, 1e-5))},
            "embedding": {"bigram": {"buckets": int(pick(509, 4093)), "mul_prev": int(pick(37, 1000003)), "mul_cur": int(pick(13, 999983))}},
            "layers": layers}


def make_dir(name: str, tmp, cfg: dict | None = None, seed: int | None = None, change=None) -> tuple[str, dict, dict]:
    """Writes configuration `name` with seeded random weights (float32); `change(tensors)` may edit them before they
    are written. Returns (folder, config, weights by name)."""
    from fusezap_core_b200.weights import write_random_model
    from fusezap_core_b200.weights.safetensors_io import read_model_dir, write_file
    base, s = CONFIGS.get(name, (cfg, seed))
    cfg = copy.deepcopy(cfg if cfg is not None else base)
    d = os.path.join(str(tmp), f"nepudra-{name}")
    write_random_model(cfg, d, seed if seed is not None else s, "float32", norm_noise=True, std_scale=STD_SCALE)
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
    import plain_nepudra
    return plain_nepudra.forward(cfg, {k: v.double() for k, v in w.items()}, list(toks)).numpy()


def rounded(w: dict) -> dict:
    """The weights as a bfloat16 engine holds them: matrices rounded once, vectors stored in 32-bit as they are."""
    return {k: v.to(torch.bfloat16).to(torch.float32) if v.dim() >= 2 else v for k, v in w.items()}
