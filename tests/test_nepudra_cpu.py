"""Nepudra on the CPU: the package's host side (configuration, model description, weights, borrowed caches, windows,
state slots for the recurrence and the previous token, step packing, scheduler, entry point) with the plain operation
table, against the plain implementation on whole sequences."""
import copy
import json

import numpy as np
import pytest
import torch

from nepudra_util import CONFIGS, NEP_MIX, NEP_ODD, drawn_config, make_dir, plain_logits, tokens_for
from pepilix_util import rel_rms, run_cut, run_mixed
from plain_ops import PlainOpsDeep
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import CacheManager, KVNeed
from fusezap_core_b200.config import describe
from fusezap_core_b200.config.nepudra import NepudraConfig
from fusezap_core_b200.engine import Portion, StepRunner, load_model


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("nepudra")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, page=4, pages=48, slots=3, max_len=160):
    model = load_model(d, "float32", "cpu", max_len=max_len, ops=PlainOpsDeep(torch.float32))
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, torch.float32, "cpu")
    return model, cache, StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=slots)


def test_config_reads_every_size_and_round_trips():
    typed, spec = describe(copy.deepcopy(NEP_MIX))
    assert isinstance(typed, NepudraConfig) and typed.to_json() == json.loads(json.dumps(NEP_MIX))
    assert [L.mixer.kind for L in spec.layers] == ["sink_attention", "sink_attention", "general_delta", "sink_attention"]
    assert [L.block.kind for L in spec.layers] == ["depth_average"] * 4 and spec.layers[2].ffn is None
    first, owner, reader = (spec.layers[i].mixer.params for i in (0, 1, 3))
    assert (first["window"], first["rotated"], first["qk_norm"], first["softcap"], first["query_temperature"]) == (9, 8, True, 0.0, None)
    assert first["bias"] == ("q", "k", "v") and owner["bias"] == ("q", "k", "v", "out")
    assert (owner["query_temperature"], owner["softcap"], owner["window"], owner["value_dim"]) == ((0.7, 5), 2.5, 0, 24)
    assert reader["own_kv"] is False and owner["own_kv"] is True
    assert [(e.layer, e.cache, e.write_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]
    assert spec.layers[0].ffn.params["activation"] == "gelu_tanh"
    assert spec.embed_extras[0].params["buckets"] == 97 and len(spec.positions) == 1


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="other"), "not supported"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "sizes differ"),
    (lambda c: c["layers"][0]["mlp"].update(kind="other"), "not supported"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.pop("norm"), "lacks"),
])
def test_config_refusals(change, message):
    c = copy.deepcopy(NEP_MIX)
    change(c)
    with pytest.raises((ValueError, NotImplementedError), match=message):
        describe(c)


def test_random_weights_name_every_tensor(dirs):
    d, cfg, w = dirs["mix"]
    assert {"embed", "bigram", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b",
            "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.down", "l0.dwa", "l1.mix.o.b",
            "l2.mix.r", "l2.mix.a", "l2.mix.a.b", "l2.mix.w1", "l2.mix.w2", "l2.mix.w0", "l2.mix.norm", "l2.dwa",
            "l3.mix.q", "l3.mix.q.b", "l3.mix.g", "l3.mix.o.b", "l3.dwa"} <= set(w)
    assert not {"l0.mix.o.b", "l1.mix.q.norm", "l2.norm2", "l3.mix.k", "l3.mix.v", "l3.mix.k.b"} & set(w)
    assert w["final.norm"].shape == () and w["l1.norm2"].shape == () and tuple(w["bigram"].shape) == (98, 64)
    assert [tuple(w[f"l{i}.dwa"].shape) for i in range(4)] == [(2,), (3,), (4,), (5,)]
    assert tuple(w["l1.mix.v"].shape) == (24, 64) and tuple(w["l1.mix.g"].shape) == (4, 64) and tuple(w["l2.mix.norm"].shape) == (24,)
    assert w["l2.mix.w2"].shape[1] == w["l2.mix.w1"].shape[0]


def test_inner_size_of_the_decay_projection_comes_from_the_checkpoint(tmp_path):
    def other_rank(w):
        g = torch.Generator().manual_seed(0)
        w["l2.mix.w1"], w["l2.mix.w2"] = torch.randn(5, 64, generator=g) * 0.1, torch.randn(24, 5, generator=g) * 0.1
    d, cfg, w = make_dir("rank", tmp_path, NEP_MIX, 4, change=other_rank)
    model, cache, runner = engine_parts(d)
    toks = tokens_for(cfg, (20,), seed=1)[0]
    assert rel_rms(run_cut(runner, cache, "r", toks, (20,)), plain_logits(cfg, w, toks)) < 2e-5


def test_a_cache_keeps_the_widest_window_of_its_readers():
    c = copy.deepcopy(NEP_ODD)
    needs = describe(c)[1]
    from fusezap_core_b200.engine.model import DecoderModel
    model = DecoderModel(needs)
    got = model.cache_needs()
    assert sorted(got) == [1, 2] and got[1] == KVNeed(3, 24, 0, value_dim=40) and got[2] == KVNeed(2, 12, 5, value_dim=20)


def test_state_is_declared_per_layer_and_for_the_embedding(dirs):
    d, cfg, w = dirs["mix"]
    model, cache, runner = engine_parts(d, slots=2)
    needs = model.state_needs()
    assert sorted(needs) == [(-1, "bigram.prev"), (2, "S")]
    assert needs[(-1, "bigram.prev")] == ((1,), torch.int32)
    assert cache.states.tensors[(-1, "bigram.prev")].dtype == torch.int32
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


def test_the_previous_token_of_a_request_survives_steps_of_other_requests(dirs):
    """A request left out of steps in which another one takes its place in the batch still hashes with its own last token."""
    d, cfg, w = dirs["one"]
    model, cache, runner = engine_parts(d, slots=2)
    a, b = tokens_for(cfg, (9, 7), seed=3)
    runner.run([Portion("a", a[:4], [])])
    runner.run([Portion("b", b[:6], [])])
    got_a = runner.run([Portion("a", a[4:], list(range(5)))]).numpy().copy()      # (the logits live in a buffer the next step reuses)
    got_b = runner.run([Portion("b", b[6:], [0])]).numpy()
    assert rel_rms(got_a, plain_logits(cfg, w, a)[4:]) < 2e-5 and rel_rms(got_b, plain_logits(cfg, w, b)[6:]) < 2e-5


def test_greedy_generation_through_the_entry_point(dirs):
    """Through `LLMEngine` and its scheduler: portions of prompts beside decoding requests, more requests than state
    slots, a pool that does not hold all of them at once."""
    d, cfg, w = dirs["odd"]
    eng = LLMEngine.from_pretrained(d, dtype="float32", device="cpu", ops=PlainOpsDeep(torch.float32), max_model_len=64,
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
