"""Gimotar on the CPU: the package's host side (configuration, model description, weights, state slots for the recurrence,
the convolution and the previous token, values handed from the first blending layer to the later ones, step packing,
scheduler, entry point) with the plain operation table, against the plain implementation on whole sequences."""
import copy

import numpy as np
import pytest
import torch

from gimotar_util import CONFIGS, GIM_MIX, GIM_ODD, drawn_config, make_dir, plain_logits, tokens_for
from pepilix_util import rel_rms, run_cut, run_mixed
from plain_ops import PlainOpsGated
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import CacheManager, KVNeed, LatentNeed
from fusezap_core_b200.config import describe
from fusezap_core_b200.config.gimotar import GimotarConfig
from fusezap_core_b200.engine import Portion, StepRunner, load_model


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gimotar")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, page=4, pages=48, slots=3, max_len=160):
    model = load_model(d, "float32", "cpu", max_len=max_len, ops=PlainOpsGated(torch.float32))
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, torch.float32, "cpu")
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


def test_config_reads_every_size_and_round_trips():
    for cfg in (GIM_MIX, GIM_ODD):
        typed = GimotarConfig.from_json(cfg)
        back = typed.to_json()
        assert GimotarConfig.from_json(back) == typed
        for a, b in zip(cfg["layers"], back["layers"]):
            assert a["type"] == b["type"] and a["mixer"] == b["mixer"] and a["mlp"] == b["mlp"]
        assert (back["vocab"], back["width"], back["residual_mult"], back["embedding"]) == \
               (cfg["vocab"], cfg["width"], cfg["residual_mult"], cfg["embedding"])
    typed, spec = describe(GIM_MIX)
    assert spec.tie_embeddings and spec.embed_scale == 6.0 and spec.lm_head_name is None
    kinds = [L.mixer.kind for L in spec.layers]
    assert kinds == ["sink_attention", "rglru", "latent_attention", "sink_attention"]
    assert [L.mixer.params.get("value_mix") for L in spec.layers] == ["source", None, None, "blend"]
    assert spec.layers[0].mixer.params["span"] == 9 and spec.layers[3].ffn is None
    assert spec.layers[2].mixer.params["pairing"] == "neighbours" and spec.layers[1].mixer.params["sharpness"] == 8.0


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not supported"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(blocks=5), "multiple of blocks"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "values of one shape"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c.pop("residual_mult"), "lacks"),
    (lambda c: c["embedding"].pop("scale"), "lacks"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "lacks"),
])
def test_config_refusals(change, message):
    cfg = copy.deepcopy(GIM_MIX)
    change(cfg)
    with pytest.raises((ValueError, NotImplementedError), match=message):
        describe(cfg)


def test_random_weights_name_every_tensor(dirs):
    d, cfg, w = dirs["mix"]
    names = set(w)
    assert {"embed", "bigram", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.q.norm", "l0.mix.k.norm",
            "l0.mix.o", "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e4.gate", "l0.mlp.e0.down", "l0.mlp.shared.up",
            "l1.mix.y", "l1.mix.y.b", "l1.mix.x", "l1.mix.x.b", "l1.mix.conv", "l1.mix.conv.b", "l1.mix.ra", "l1.mix.ra.b",
            "l1.mix.ri", "l1.mix.ri.b", "l1.mix.lam", "l1.mix.o", "l2.mix.q", "l2.mix.dkv", "l2.mix.dkv.norm", "l2.mix.uk",
            "l2.mix.uv", "l2.mix.sink", "l2.mix.g", "l2.mix.o", "l3.mix.vmix"} <= names
    assert "head" not in names and "l1.mlp.shared.up" not in names and not any(k.startswith("l3.mlp") for k in names)
    assert w["bigram"].shape == (98, 64) and w["l1.mix.ra"].shape == (3, 16, 16) and w["l1.mix.conv"].shape == (48, 4)
    assert w["l2.mix.dkv"].shape == (24, 64) and w["l2.mix.uk"].shape == (24, 20) and w["l3.mix.vmix"].shape == ()
    assert w["l2.mix.g"].shape == (36, 64) and w["l0.mlp.router.b"].shape == (5,)


def test_state_and_caches_are_declared_per_layer(dirs):
    d, cfg, w = dirs["mix"]
    model, cache, runner = engine_parts(d, slots=2)
    needs = model.state_needs()
    assert sorted(needs) == [(-1, "bigram.prev"), (1, "S"), (1, "conv")]
    assert needs[(1, "S")] == (48,) and needs[(1, "conv")] == (3, 48)
    caches = model.cache_needs()
    assert caches[0] == KVNeed(2, 16, 0, value_dim=8) and caches[2] == LatentNeed(24, 0) and caches[3] == KVNeed(2, 24, 0, value_dim=8)
    assert model.graph_safe()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size_against_the_whole_sequence(dirs, name):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d)
    toks = tokens_for(cfg, (50,), seed=11)[0]
    ref = plain_logits(cfg, w, toks)
    for cuts in ((50,), (1,), (2,), (5, 3, 1, 7, 2, 19)):
        assert rel_rms(run_cut(runner, cache, "r", toks, cuts), ref) < 2e-5, (name, cuts)
        cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dirs, name):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, page=4, pages=30, slots=3, max_len=64)
    reqs = dict(zip("abcde", tokens_for(cfg, (41, 9, 23, 2, 30), seed=5)))
    plan = [[("a", 17), ("b", 2)], [("a", 1), ("b", 7), ("c", 20)], [("a", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 2)],
            [("a", 2), ("c", 1), ("e", 5)], [("e", 1)], [("e", 24)]]
    got = run_mixed(runner, cache, reqs, plan)
    cache.check()
    assert cache.live_requests() == [] and cache.states.num_free == 3
    for r, toks in reqs.items():
        assert rel_rms(got[r], plain_logits(cfg, w, toks)) < 2e-5, (name, r)


def test_a_requests_state_survives_steps_of_other_requests(dirs):
    """A request left out of steps in which another one takes its place in the batch goes on from its own recurrent
    state, convolution inputs and previous token."""
    d, cfg, w = dirs["one"]
    model, cache, runner = engine_parts(d, slots=2)
    a, b = tokens_for(cfg, (9, 7), seed=3)
    runner.run([Portion("a", a[:4], [])])
    runner.run([Portion("b", b[:6], [])])
    got_a = runner.run([Portion("a", a[4:], list(range(5)))]).numpy().copy()
    got_b = runner.run([Portion("b", b[6:], [0])]).numpy()
    assert rel_rms(got_a, plain_logits(cfg, w, a)[4:]) < 2e-5 and rel_rms(got_b, plain_logits(cfg, w, b)[6:]) < 2e-5


def test_the_first_blending_layers_own_weight_is_not_read(dirs, tmp_path):
    d, cfg, w = make_dir("mix", tmp_path, change=lambda t: t.update({"l0.mix.vmix": torch.tensor(0.9)}))
    model, cache, runner = engine_parts(d)
    toks = tokens_for(cfg, (20,), seed=1)[0]
    assert rel_rms(run_cut(runner, cache, "r", toks, (20,)), plain_logits(cfg, dirs["mix"][2], toks)) < 2e-5


def test_a_strong_blend_of_values_shows_in_the_logits(tmp_path):
    d, cfg, w = make_dir("mix", tmp_path, change=lambda t: t.update({"l3.mix.vmix": torch.tensor(0.8)}))
    model, cache, runner = engine_parts(d)
    toks = tokens_for(cfg, (40,), seed=4)[0]
    ref = plain_logits(cfg, w, toks)
    for cuts in ((40,), (1,), (7, 2, 1)):
        assert rel_rms(run_cut(runner, cache, "r", toks, cuts), ref) < 2e-5, cuts
    assert rel_rms(plain_logits(cfg, {**w, "l3.mix.vmix": torch.tensor(0.0)}, toks), ref) > 1e-3


def test_greedy_generation_through_the_entry_point(dirs):
    """Through `LLMEngine` and its scheduler: portions of prompts beside decoding requests, more requests than state
    slots, a pool that does not hold all of them at once."""
    d, cfg, w = dirs["odd"]
    eng = LLMEngine.from_pretrained(d, dtype="float32", device="cpu", ops=PlainOpsGated(torch.float32), max_model_len=64,
                                    num_blocks=14, block_size=8, max_num_seqs=2, max_prefill_tokens=8, cuda_graphs=False)
    P = tokens_for(cfg, (7, 19, 2, 30), seed=2)
    out = eng.generate(P, SamplingParams(max_tokens=5, ignore_eos=True))
    for prompt, new in zip(P, out):
        lg = plain_logits(cfg, w, list(prompt) + new)
        for i, t in enumerate(new):
            row = lg[len(prompt) - 1 + i]
            assert int(row.argmax()) == t or row.max() - row[t] < 1e-3


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(seed, tmp_path):
    """The host side reads every size and constant from the configuration: drawn ones (the GPU tests' own) against the
    plain model, whole, in portions and token by token."""
    cfg = drawn_config(seed)
    d, cfg, w = make_dir(f"drawn{seed}", tmp_path, cfg, seed)
    model, cache, runner = engine_parts(d, page=4, pages=30, slots=2, max_len=64)
    toks = tokens_for(cfg, (40,), seed=seed)[0]
    ref = plain_logits(cfg, w, toks)
    for cuts in ((40,), (1,), (6, 2, 1, 17)):
        assert rel_rms(run_cut(runner, cache, "r", toks, cuts), ref) < 2e-5, (seed, cuts)
