"""Gimotar through the trace replay program on the GPU: a `bin/trace_run` process replays the same requests whole, with
their last 32 tokens one by one, in portions down to two tokens, and four at a time in a pool so small that pages and
state slots are used again; every position is compared with the plain model's logits of the whole request, and in
float32 the cuttings must agree with each other bit for bit (every sum's order is a function of the row alone).

The small configurations are those of `gimotar_util`; the larger one has layer sizes of a few hundred that reach the
tensor-core products and both tensor-core attention kernels, a bfloat16 checkpoint and requests of up to 1,300 tokens,
many chunks long, replayed by a small scheduler in a pool that does not hold all requests."""
import copy

import numpy as np
import pytest
import torch

from gimotar_util import CONFIGS, att, latent, layer, model, moe, plain_logits, rglru, rot, rounded, tokens_for
from test_gimotar_gpu import agrees
from test_replay_gpu import LENGTHS, POOL_TOKENS, build_trace
from util import TraceBuilder, run_trace

pytestmark = pytest.mark.gpu


def _write(cfg: dict, path: str, seed: int, dtype: str) -> dict:
    from fusezap_core_b200.weights import write_random_model
    from fusezap_core_b200.weights.safetensors_io import read_model_dir
    write_random_model(copy.deepcopy(cfg), path, seed, dtype, norm_noise=True, std_scale=5.0)
    return read_model_dir(path)


def _oracle(cfg, w, ids, dtype):
    w = {k: v.float() if v.dtype.is_floating_point else v for k, v in w.items()}
    return plain_logits(cfg, rounded(w) if dtype == "bfloat16" else w, ids)


def _compare(got: dict, ref_of, refs, dtype: str, what: str) -> None:
    for rid, rows in sorted(got.items()):
        ref = refs[ref_of(rid)]
        assert sorted(rows) == list(range(len(ref))), f"{what} {rid}: positions {sorted(rows)[:5]}..."
        agrees(np.stack([rows[p] for p in range(len(ref))]), ref, dtype, (what, rid))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_replay_all_cuttings(name, dtype, tmp_path):
    cfg, seed = CONFIGS[name]
    w = _write(cfg, str(tmp_path / "m"), seed, "float32")
    P = tokens_for(cfg, LENGTHS, seed=3)
    refs = [_oracle(cfg, w, ids, dtype) for ids in P]
    tb = build_trace(P)
    assert tb.most_live == 4 and max(len(s["entries"]) for s in tb.steps) == 4
    outs = run_trace(str(tmp_path / "m"), dtype, str(tmp_path / "out"), max_tokens=POOL_TOKENS, steps=tb.steps)
    got = tb.collect(outs, cfg["vocab"])
    assert {r[0] for r in got} == {"w", "d", "p", "m"}
    if dtype == "float32":
        for rid, rows in sorted(got.items()):
            if rid[0] == "w":
                continue
            whole = got["w" + rid[1:]]
            for p, row in rows.items():
                assert np.array_equal(row, whole[p]), (f"{name}: request {rid} position {p} differs from the whole "
                                                       f"request's row by {np.abs(row - whole[p]).max():.3e}")
    _compare(got, lambda rid: int(rid[1:]), refs, dtype, name)


LARGER = model(512, 384, 1e-5, 0.35, 19.6, (2039, 29, 13), [
    layer(att(12, 3, 64, 64, 0.125, 100, rot(250000.0, 32), v_mix=True), moe(8, 2, 128, 256)),
    layer(rglru(320, 4, 4), moe(6, 3, 96)),
    layer(latent(6, 64, 32, 64, 128, 0.1, rot(10000.0, 32, (8.0, 256, 16.0, 1.0))), moe(4, 1, 200, 64)),
    layer(att(6, 3, 128, 64, 0.09, 64, rot(5000.0, 128), v_mix=True), None),
    layer(att(4, 4, 128, 128, 0.09, 200, rot(300.0, 16)), moe(5, 5, 64)),
    layer(rglru(256, 1, 3), moe(3, 1, 64, 128)),
])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_a_larger_model_with_long_requests_in_a_small_pool(dtype, tmp_path):
    cfg = LARGER
    w = _write(cfg, str(tmp_path / "m"), 11, "bfloat16")
    assert w["embed"].dtype == torch.bfloat16
    lengths = (1300, 260, 1, 23, 333, 97)
    P = dict(zip("abcdef", tokens_for(cfg, lengths, seed=5)))
    refs = {r: _oracle(cfg, w, ids, dtype) for r, ids in P.items()}
    # a little scheduler: up to four live; portions of changing size, then each request's last tokens one by one
    rng = np.random.default_rng(8)
    tb, waiting, live, peak = TraceBuilder(), list(P), {}, 0
    single = {r: max(0, len(P[r]) - int(rng.integers(8, 140))) for r in P}
    while waiting or live:
        while waiting and len(live) < 4 and (not live or rng.random() < 0.7):
            live[waiting.pop(0)] = 0
        peak = max(peak, sum(-(-len(P[r]) // 64) * 64 for r in live))
        entries, ends = [], []
        for r in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue
            at = live[r]
            n = 1 if at >= single[r] else min(int(rng.choice([2, 3, 5, 16, 17, 64, 100, 200])), single[r] - at)
            entries.append((r, P[r][at: at + n], "all"))
            live[r] = at + n
            if live[r] == len(P[r]):
                ends.append(r)
                del live[r]
        if entries:
            tb.step(entries, end=ends)
    assert max(len(s["entries"]) for s in tb.steps) == 4 and peak < sum(-(-n // 64) * 64 for n in lengths)
    outs = run_trace(str(tmp_path / "m"), dtype, str(tmp_path / "out"), max_tokens=peak, steps=tb.steps)
    _compare(tb.collect(outs, cfg["vocab"]), lambda rid: rid, refs, dtype, "larger")
