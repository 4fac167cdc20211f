"""Nepudra on the GPU: the whole model through the engine's step function, cache manager and kernels against the plain
implementation (`plain_nepudra.py`, 64-bit, whole sequences), in float32 and bfloat16."""
import numpy as np
import pytest
import torch

from nepudra_util import CONFIGS, _att, _att2, _layer, make_dir, plain_logits, rounded, tokens_for
from pepilix_util import run_cut, run_mixed
from fusezap_core_b200.cache import CacheManager
from fusezap_core_b200.engine import StepRunner, load_model

pytestmark = pytest.mark.gpu
# float32: sequential 32-bit sums against a 64-bit oracle. The head norm of the delta rule divides small recurrent
# outputs by their root mean square, which carries the rounding of a nearly empty state into a sequence's first tokens,
# so the bound is asked of 19 rows in 20 and no row may be off by more than ten times the bound.
LIMIT = {"float32": 2e-5, "bfloat16": 3e-2}


def row_errors(got, ref):
    """Per row: the root-mean-square difference (row mean removed), relative to the rms of the reference's logits."""
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    scale = float(np.sqrt(((ref - ref.mean(-1, keepdims=True)) ** 2).mean()))
    return np.sqrt((d ** 2).mean(-1)) / scale


def agrees(got, ref, dtype, what=None):
    e = row_errors(got, ref)
    assert np.quantile(e, 0.95) < LIMIT[dtype] and e.max() < 10 * LIMIT[dtype], (what, float(np.quantile(e, 0.95)), float(e.max()))


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("nepudra")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, dtype, page=4, pages=48, slots=3, max_len=192):
    model = load_model(d, dtype, "cuda:0", max_len=max_len)
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, model.ops.dtype, "cuda:0")
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


def oracle(cfg, w, toks, dtype):
    return plain_logits(cfg, w if dtype == "float32" else rounded(w), toks)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size_against_the_whole_sequence(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype)
    toks = tokens_for(cfg, (75,), seed=11)[0]
    ref = oracle(cfg, w, toks, dtype)
    for cuts in ((75,), (1,), (2,), (5, 3, 1, 7, 2, 19), (40, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1)):
        got = run_cut(runner, cache, "r", toks, cuts)
        model.ops.check_errors()
        agrees(got, ref, dtype, (name, cuts))
        cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype, page=4, pages=40, slots=3, max_len=96)
    reqs = dict(zip("abcde", tokens_for(cfg, (61, 9, 33, 2, 47), seed=5)))
    plan = [[("a", 17), ("b", 2)], [("a", 1), ("b", 7), ("c", 30)], [("a", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 2)],
            [("a", 22), ("c", 1), ("e", 5)], [("e", 1)], [("e", 40)], [("e", 1)]]
    got = run_mixed(runner, cache, reqs, plan)
    model.ops.check_errors()
    for r, toks in reqs.items():
        agrees(got[r], oracle(cfg, w, toks, dtype), dtype, (name, r))
    cache.check()
    assert cache.states.num_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_windows_temperature_periods_and_page_borders(dirs, dtype):
    d, cfg, w = dirs["mix"]
    model, cache, runner = engine_parts(d, dtype, page=8, pages=48, slots=2, max_len=384)
    toks = tokens_for(cfg, (340,), seed=23)[0]
    ref = oracle(cfg, w, toks, dtype)
    got = run_cut(runner, cache, "long", toks, (21,) + (1,) * 319)
    model.ops.check_errors()
    agrees(got, ref, dtype)
