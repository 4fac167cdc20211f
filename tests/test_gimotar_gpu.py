"""Gimotar on the GPU: every new or extended kernel alone against its plain function, then the model in both dtypes (portions
down to two tokens, unequal batches with pages and slots used again, long decoding across chunk borders, generation
through the entry point and the command line, drawn configurations)."""
import json
import math

import numpy as np
import pytest
import torch

import plain_gimotar as plain
from gimotar_util import CONFIGS, drawn_config, make_dir, plain_logits, rounded, tokens_for
from pepilix_util import run_cut, run_mixed
from fusezap_core_b200 import LLMEngine, SamplingParams
from fusezap_core_b200.cache import CacheManager, KVNeed
from fusezap_core_b200.engine import StepRunner, load_model
from fusezap_core_b200.kernels import cuda_ops
from fusezap_core_b200.parts import LayerCache

pytestmark = pytest.mark.gpu
LIMIT = {"float32": 2e-5, "bfloat16": 3e-2}
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


def row_errors(got, ref):
    """Per row: the root-mean-square difference (row mean removed), relative to the rms of the reference's logits."""
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    scale = float(np.sqrt(((ref - ref.mean(-1, keepdims=True)) ** 2).mean()))
    return np.sqrt((d ** 2).mean(-1)) / scale


def agrees(got, ref, dtype, what=None):
    """float32: the bound for 19 rows in 20, ten times it for all. bfloat16: where two experts' router logits nearly
    tie, rounding picks the other one and that row differs by much more (the oracle does not round), so the bound is
    asked of the median row, twice it of nine rows in ten, and no row may be off by the scale of the logits itself."""
    e = row_errors(got, ref)
    if dtype == "float32":
        assert np.quantile(e, 0.95) < LIMIT[dtype] and e.max() < 10 * LIMIT[dtype], (what, float(np.quantile(e, 0.95)), float(e.max()))
    else:
        assert np.median(e) < LIMIT[dtype] and np.quantile(e, 0.9) < 2 * LIMIT[dtype] and e.max() < 1.0, \
            (what, float(np.median(e)), float(np.quantile(e, 0.9)), float(e.max()))


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gimotar")
    return {name: make_dir(name, tmp) for name in CONFIGS}


def engine_parts(d, dtype, page=4, pages=48, slots=3, max_len=192):
    model = load_model(d, dtype, DEV, max_len=max_len)
    cache = CacheManager(model.cache_needs(), model.state_needs(), page, pages, slots, max_len, model.ops.dtype, DEV)
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
    first = None
    for cuts in ((75,), (1,), (2,), (5, 3, 1, 7, 2, 19), (40, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1)):
        got = run_cut(runner, cache, "r", toks, cuts)
        model.ops.check_errors()
        agrees(got, ref, dtype, (name, cuts))
        cache.check()
        if dtype == "float32":      # every sum's order is a function of the row alone: the cuttings agree bit for bit
            first = got if first is None else first
            assert np.array_equal(got, first), (name, cuts)


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
    cache.check()
    assert cache.live_requests() == [] and cache.states.num_free == 3
    for r, toks in reqs.items():
        agrees(got[r], oracle(cfg, w, toks, dtype), dtype, (name, r))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "one"])
def test_long_decoding_across_chunk_and_page_borders(dirs, name, dtype):
    d, cfg, w = dirs[name]
    model, cache, runner = engine_parts(d, dtype, page=8, pages=48, slots=2, max_len=384)
    toks = tokens_for(cfg, (340,), seed=23)[0]
    ref = oracle(cfg, w, toks, dtype)
    got = run_cut(runner, cache, "long", toks, (21,) + (1,) * 319)
    model.ops.check_errors()
    agrees(got, ref, dtype)


# ---------------------------------------------------------------------------------------- each mechanism alone
from test_gizulorn_gpu import Meta, close, paged, scan_portions, shuffled_tables


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,B", [(48, 3), (176, 2), (7, 7), (130, 1), (1024, 4)])
def test_recurrent_unit_carries_its_state_across_portions(dtype, W, B):
    """Two sequences cut into portions down to one token and interleaved, a slot nobody uses, a row of padding: the scan
    with its coefficients computed in a launch of their own (long portions) and inside the scan (short ones) leave the
    same bits, and both follow the plain recurrence."""
    ops, g, T, dt = cuda_ops(dtype), torch.Generator().manual_seed(W), 70, DT[dtype]
    bw = W // B
    u = [(torch.randn(T, W, generator=g)).to(dt) for _ in range(2)]
    y = [(torch.randn(T, W, generator=g)).to(dt) for _ in range(2)]
    gates = [torch.randn(T, B, 2 * bw, generator=g) * 2 for _ in range(2)]
    bias = torch.randn(B, 2 * bw, generator=g)
    lam = torch.randn(W, generator=g) * 3
    lam[0] = -30.0        # a channel that hardly forgets: 1 - a^2 keeps its digits
    refs = []
    for r in range(2):
        gb = gates[r].to(F) + bias.to(F)
        rr, ii = plain.sigmoid(gb[..., :bw]).reshape(T, W), plain.sigmoid(gb[..., bw:]).reshape(T, W)
        refs.append(plain.rglru_recurrence(u[r].to(F), rr, ii, lam.to(F)) * y[r].to(F))
    outs = {}
    for cook_rows in (0, 1 << 30):
        import fusezap_core_b200.kernels.table as table
        old, table.RGLRU_COOK_ROWS = table.RGLRU_COOK_ROWS, cook_rows
        try:
            state = torch.zeros(4, W, device=DEV)
            state[2] = 3.0
            got = [torch.zeros(T, W, dtype=dt) for _ in range(2)]
            for step in scan_portions(T, seed=W + B):
                meta = Meta([(n, at, (1, 3)[r]) for r, at, n in step], pad=1)
                meta.max_portion = max(n for _, _, n in step)
                rows = lambda xs: torch.cat([xs[r][at: at + n] for r, at, n in step] + [torch.zeros(1, *xs[0].shape[1:], dtype=xs[0].dtype)]).to(DEV)
                out = torch.full((meta.n_rows, W), 7.0, dtype=dt, device=DEV)
                ops.rglru_scan(rows(u), rows(gates), bias.to(DEV), lam.to(DEV), rows(y), 8.0, state, meta, out)
                k = 0
                for r, at, n in step:
                    got[r][at: at + n] = out[k: k + n].cpu()
                    k += n
            assert float(state[2].min()) == 3.0 and float(state[0].abs().max()) == 0.0
            outs[cook_rows] = got
            for r in range(2):
                close(got[r], refs[r], dtype, f"request {r}")
        finally:
            table.RGLRU_COOK_ROWS = old
    for r in range(2):
        assert torch.equal(outs[0][r], outs[1 << 30][r])


def test_recurrent_unit_is_the_plain_recurrence_of_the_design():
    """`plain.rglru_recurrence` against the equations written out token by token for one channel."""
    u, r, i, lam = (torch.tensor(x, dtype=F) for x in ([[0.5], [-1.0], [2.0]], [[0.2], [0.9], [0.5]], [[0.7], [0.1], [1.0]], [0.3]))
    S, want = 0.0, []
    for t in range(3):
        a = math.exp(-8.0 * float(r[t]) * math.log1p(math.exp(0.3)))
        S = a * S + math.sqrt(1 - a * a) * float(i[t]) * float(u[t])
        want.append(S)
    assert torch.allclose(plain.rglru_recurrence(u, r, i, lam)[:, 0], torch.tensor(want, dtype=F), atol=1e-14)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,taps", [(48, 4), (40, 2), (7, 5), (256, 3), (33, 1)])
def test_convolution_with_a_bias_across_portions(dtype, C, taps):
    ops, g, T, dt = cuda_ops(dtype), torch.Generator().manual_seed(C), 40, DT[dtype]
    x = [torch.randn(T, C, generator=g).to(dt) for _ in range(2)]
    w = torch.randn(C, taps, generator=g).to(dt)
    b = torch.randn(C, generator=g)
    state = torch.zeros(3, max(taps - 1, 1), C, device=DEV)[:, : taps - 1] if taps > 1 else None
    got = [torch.zeros(T, C, dtype=dt) for _ in range(2)]
    for step in scan_portions(T, seed=taps):
        meta = Meta([(n, at, (2, 0)[r]) for r, at, n in step], pad=1)
        rows = torch.cat([x[r][at: at + n] for r, at, n in step] + [torch.zeros(1, C, dtype=dt)]).to(DEV)
        out = torch.empty_like(rows)
        ops.short_conv(rows, w.to(DEV), state.contiguous() if state is not None else None, meta, out, False, None, bias=b.to(DEV)) \
            if state is None else ops.short_conv(rows, w.to(DEV), state, meta, out, False, None, bias=b.to(DEV))
        k = 0
        for r, at, n in step:
            got[r][at: at + n] = out[k: k + n].cpu()
            k += n
    for r in range(2):
        close(got[r], plain.causal_conv(x[r].to(F), w.to(F), b.to(F)), dtype, f"request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("L,R,dims,H,dn", [(40, 8, 8, 3, 12), (48, 24, 24, 6, 40), (20, 6, 4, 5, 8), (36, 12, 2, 1, 16)])
def test_neighbouring_dimensions_are_paired_in_the_latent_rotation(dtype, L, R, dims, H, dn):
    """The cache entry's rotated key part and the queries' rotated part, with scaled frequencies and a magnitude."""
    from fusezap_core_b200.parts.rope import RotaryEncoding
    from test_pepilix_gpu import _pool
    ops, g, page, dt = cuda_ops(dtype), torch.Generator().manual_seed(L), 4, DT[dtype]
    rot = {"base": 300.0, "dims": dims, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 0.5}}
    pos = RotaryEncoding(dims, 300.0, kind="yarn", factor=4.0, original_max_position_embeddings=16, turns_fast=4.0,
                         turns_slow=0.5, precise=True, magnitude=0.1 * math.log(4.0) + 1.0)
    pos.prepare(64, torch.device(DEV))
    cos, sin = plain.angles(rot, 64)
    assert (pos.cos.cpu().to(F) - cos).abs().max() < 1e-6 and (pos.sin.cpu().to(F) - sin).abs().max() < 1e-6
    tables = torch.tensor([[5, 2, 7, 0, -1, -1], [1, 6, 3, -1, -1, -1]], dtype=torch.int32)
    meta = Meta([(9, 3, -1), (2, 7, -1)], tables, pad=2)
    down = torch.randn(13, L + R, generator=g)
    w = torch.rand(L, generator=g) + 0.5
    pool = _pool(8, page, L + R, dtype)
    ops.latent_cache_write(down.to(DEV), w.to(DEV), 1e-5, pos.cos, pos.sin, dims, meta, LayerCache(keys=pool, group=0, page_size=page), pairing=1)
    q = torch.randn(13, H, dn + R, generator=g).to(dt)
    qa = torch.zeros(13, H, L + R, dtype=dt, device=DEV)
    ops.rotate_heads(q.to(DEV), dn, pos.cos, pos.sin, dims, meta, qa, L, pairing=1)
    ops.check_errors()
    tol = 3e-6 if dtype == "float32" else 2.0 ** -8
    seen = torch.zeros(8, page, dtype=torch.bool)
    for i in range(11):
        s, p = int(meta.seq_row[i]), int(meta.pos[i])
        c = down[i, :L].to(F)
        c = c / torch.sqrt((c * c).mean() + 1e-5) * w.to(F)
        kr = plain.rotate_neighbours(down[i: i + 1, None, L:].to(F), cos[p: p + 1], sin[p: p + 1], dims)[0, 0]
        ref = torch.cat([c, kr])
        pg = int(tables[s, p // page])
        assert ((pool[pg, p % page].cpu().to(F) - ref).abs() <= tol * (1 + ref.abs())).all(), f"row {i}"
        seen[pg, p % page] = True
        qr = plain.rotate_neighbours(q[i: i + 1, :, dn:].to(F), cos[p: p + 1], sin[p: p + 1], dims)[0]
        assert ((qa[i, :, L:].cpu().to(F) - qr).abs() <= tol * (1 + qr.abs())).all(), f"query row {i}"
    assert float(pool.float().abs().sum(-1).cpu()[~seen].max()) == 0.0
    assert float(qa[11:].float().abs().max()) == 0.0


def _latent_reference(q, ent, Wv, scale, p, sink):
    """q: (H, W); ent: (T, W); the softmax over keys 0 .. p with one more term exp(sink_h) in the denominator."""
    s = (q.to(F) @ ent[: p + 1].to(F).T) * scale
    s = torch.cat([s, sink.to(F)[:, None]], -1)
    return torch.softmax(s, -1)[:, :-1] @ ent[: p + 1, :Wv].to(F)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,W,Wv,page", [(4, 96, 72, 16), (40, 22, 16, 4), (1, 104, 72, 8), (16, 576, 512, 16), (5, 64, 32, 8), (7, 48, 40, 64)])
def test_latent_attention_with_a_sink(dtype, H, W, Wv, page):
    """A long portion behind a prefix, single tokens and a padding row, sinks from far below to far above the scores;
    in bfloat16 the tensor-core kernel, the same without its cut along the keys, and the general kernel."""
    from test_pepilix_gpu import _pool
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(H * W), DT[dtype]
    T = [300, 75]
    ent = [(torch.randn(t, W, generator=g)).to(dt) for t in T]
    sink = torch.linspace(-6.0, 9.0, H) if H > 1 else torch.tensor([2.0])
    n_pages = sum(-(-t // page) for t in T) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    pool = _pool(n_pages, page, W, dtype)
    tables = torch.full((2, 80), -1, dtype=torch.int32)
    for i, t in enumerate(T):
        for k in range(-(-t // page)):
            tables[i, k] = pg = perm.pop()
            chunk = ent[i][k * page: (k + 1) * page]
            pool[pg, : chunk.shape[0]] = chunk.to(DEV)
    cache = LayerCache(keys=pool, group=0, page_size=page)
    tol = 2e-5 if dtype == "float32" else 2.0 ** -6
    for meta in (Meta([(45, 255, -1), (1, 74, -1)], tables, pad=1), Meta([(1, 299, -1), (1, 0, -1)], tables, pad=1)):
        n = meta.n_rows
        q = (torch.randn(n, H, W, generator=g) * 0.5).to(dt)
        outs = []
        for knob in (None, "latent_key_cuts", "latent_tensor_cores"):
            if knob and dtype == "float32":
                continue
            if knob:
                setattr(ops, knob, False)
            try:
                out = torch.empty(n, H, Wv, dtype=dt, device=DEV)
                ops.latent_attention(q.to(DEV), cache, meta, out, Wv, 0.3, 0, sink=sink.to(DEV))
                ops.check_errors()
            finally:
                if knob:
                    setattr(ops, knob, True)
            outs.append(out)
            for i in range(n - 1):
                s, p = int(meta.seq_row[i]), int(meta.pos[i])
                ref = _latent_reference(q[i], ent[s], Wv, 0.3, p, sink)
                assert ((out[i].cpu().to(F) - ref).abs() <= tol * (1 + ref.abs())).all(), (knob, f"row {i}")
            assert float(out[n - 1].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sink_takes_its_share_once_and_a_far_key_is_still_found(dtype):
    """Among 1,000 keys one matches the query. With a sink far below the scores the output is that key's values; with a
    sink equal to the key's score it is half of them (the sink counts once, unscaled, and has no value), for a row of a
    portion and for a single token whose keys are cut into ranges."""
    from test_pepilix_gpu import _pool
    ops, dt = cuda_ops(dtype), DT[dtype]
    H, W, Wv, page, T = 2, 48, 32, 16, 1000
    for far in (0, 15, 16, 511, 900):
        g = torch.Generator().manual_seed(far)
        ent = (torch.randn(T, W, generator=g) * 0.1).to(dt)
        q = torch.zeros(20, H, W)
        q[:, :, Wv + 3] = 4.0
        ent[far] = 0
        ent[far, Wv + 3] = 8.0
        ent[far, :Wv] = torch.randn(Wv, generator=g).to(dt)
        score = 4.0 * 8.0 * 0.5                         # the loud key's score at scale 0.5
        pool = _pool(64, page, W, dtype)
        pool.view(-1, W)[:T] = ent.to(DEV)
        tables = torch.arange(64, dtype=torch.int32).view(1, 64)
        cache = LayerCache(keys=pool, group=0, page_size=page)
        for meta in (Meta([(20, T - 20, -1)], tables), Meta([(1, T - 1, -1)], tables)):
            n = meta.n_rows
            for sink, share in ((-30.0, 1.0), (score, 0.5), (score + math.log(3.0), 0.25)):
                out = torch.empty(n, H, Wv, dtype=dt, device=DEV)
                ops.latent_attention(q[:n].to(dt).to(DEV).contiguous(), cache, meta, out, Wv, 0.5, 0,
                                     sink=torch.tensor([sink, sink], device=DEV))
                want = ent[far, :Wv].float() * share
                assert (out.cpu().float() - want).abs().max() < (1e-3 if dtype == "float32" else 2e-2), (far, sink)


def chunked_rows(dtype, Hq, Hkv, dk, dv, span, T, portions, page, seed, loud=None, scale=0.3):
    """One sequence of T tokens in shuffled pages; `portions` ((rows, first position) each) are asked for in one step.
    loud: (key position, factor): that key and every query point one way, so that its score stands out."""
    ops, g, dt = cuda_ops(dtype), torch.Generator().manual_seed(seed), DT[dtype]
    q = torch.randn(T, Hq, dk, generator=g).to(dt)
    k = torch.randn(T, Hkv, dk, generator=g).to(dt)
    v = torch.randn(T, Hkv, dv, generator=g).to(dt)
    if loud is not None:
        j, factor = loud
        way = torch.nn.functional.normalize(torch.randn(dk, generator=g), dim=0)
        k[j] = (way * factor).to(dt)
        q = (q.float() * 0.1 + way * factor).to(dt)
    pages = -(-T // page)
    table = shuffled_tables(1, pages, pages + 5, seed)
    cache = paged(KVNeed(Hkv, dk, 0, value_dim=dv), page, pages + 5, dtype)
    qkv = torch.cat([q.view(T, -1), k.view(T, -1), v.view(T, -1)], 1).float()
    ops.rotate_kv_write(qkv.to(DEV), None, None, 0, 0, Meta([(T, 0, 0)], table), cache, torch.empty(T, Hq * dk, dtype=dt, device=DEV), Hq, Hkv, dk, dv)
    meta = Meta([(n, p0, 0) for n, p0 in portions], table.repeat(len(portions), 1), pad=1)
    meta.max_portion = max(n for n, _ in portions)
    rows = [p for n, p0 in portions for p in range(p0, p0 + n)]
    qs = torch.cat([q[rows].view(len(rows), -1), torch.zeros(1, Hq * dk, dtype=dt)]).to(DEV)
    out = torch.empty(len(rows) + 1, Hq * dv, dtype=dt, device=DEV)
    ops.sink_attention(qs, cache, meta, out, Hq, Hkv, dk, dv, scale, 0, 0, None, span=span)
    ops.check_errors()
    assert float(out[-1].abs().max()) == 0.0
    rep = Hq // Hkv
    ref = plain.masked_attention_fast(q.to(F), k.to(F).repeat_interleave(rep, 1), v.to(F).repeat_interleave(rep, 1), scale,
                                      plain.chunk_mask(T, span))
    return out[:-1].view(len(rows), Hq, dv), ref[rows], v


def test_the_two_plain_attentions_agree():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(23, 2, 6, generator=g, dtype=F) for _ in range(3))
    sink = torch.tensor([0.5, -2.0], dtype=F)
    slow = plain.masked_attention(q, k, v, 0.4, lambda i, j: j <= i and i // 5 == j // 5, sink)
    assert (slow - plain.masked_attention_fast(q, k, v, 0.4, plain.chunk_mask(23, 5), sink)).abs().max() < 1e-12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,dk,dv,span", [(4, 2, 16, 8, 9), (3, 3, 24, 40, 300), (8, 2, 80, 48, 88), (6, 3, 64, 64, 33),
                                               (4, 4, 128, 128, 70), (2, 1, 128, 128, 64), (1, 1, 32, 16, 1), (6, 1, 64, 64, 100)])
def test_attention_under_a_chunked_mask(dtype, Hq, Hkv, dk, dv, span):
    """Rows of long and short portions and single tokens, at the start of the sequence and far into it (in bfloat16 the
    sizes 64 and 128 run their long portions on tensor cores)."""
    got, ref, _ = chunked_rows(dtype, Hq, Hkv, dk, dv, span, T=200, page=4, seed=Hq * dk + span,
                               portions=[(70, 0), (2, 80), (1, 97), (1, 199), (1, 5), (90, 100)])
    if dtype == "bfloat16" and dk == dv and dk in (64, 128):
        err, ref = (got.detach().cpu().to(F) - ref).abs(), ref.to(F)
        assert not (err > 2.0 ** -7 * (ref.abs() + 4 * ref.abs().mean() + 1e-3)).any(), float(err.max())
    else:
        close(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("as_portion", [True, False])
@pytest.mark.parametrize("dk,dv,span", [(16, 8, 12), (64, 64, 96), (80, 48, 88), (128, 128, 70), (64, 64, 64)])
def test_a_loud_key_is_seen_exactly_inside_its_own_chunk(dtype, as_portion, dk, dv, span):
    """One key's score exceeds all others by far, so a row's output is that key's value if the row sees the key: keys at
    a chunk's first and last place, at page borders, for the rows just before and after the next chunk begins, in prompt
    portions (70 rows: the tensor-core kernel where the sizes allow) and for single tokens."""
    page, T = 8, 400
    for j in (0, span - 1, span, 2 * span + 3, 3 * span - 1, (T - 1) // span * span):
        if j >= T:
            continue
        end = (j // span + 1) * span                   # the first position of the next chunk
        rows = sorted({p for p in (j, j + 1, end - 2, end - 1, end, end + 1, T - 1) if j <= p < T})
        portions = [(r - max(0, r - 69) + 1, max(0, r - 69)) for r in rows] if as_portion else [(1, p) for p in rows]
        got, ref, v = chunked_rows(dtype, 2, 1, dk, dv, span, T, portions, page, seed=j, loud=(j, 12.0))
        close(got, ref, dtype, f"key {j}")
        at = 0
        for n, p0 in portions:
            for p in range(p0, p0 + n):
                sees = j <= p and p // span == j // span
                same = bool((got[at].float().cpu() - v[j].float()).abs().max() < 0.05)
                if p >= j:
                    assert same == sees, (j, p, sees)
                at += 1


def test_small_row_operations():
    """The blend of two layers' values, the gate on the concatenated heads, the copy that rounds once."""
    g = torch.Generator().manual_seed(0)
    for dtype in ("float32", "bfloat16"):
        ops, dt = cuda_ops(dtype), DT[dtype]
        dst, src = torch.randn(9, 50, generator=g), torch.randn(9, 70, generator=g)
        want = dst.clone()
        want[:, 13: 13 + 24] = (1 - 0.3) * dst[:, 13: 37] + 0.3 * src[:, 40: 64]
        d = dst.to(DEV)
        ops.blend_columns(d, 13, src.to(DEV), 40, 24, torch.tensor([0.3], device=DEV))
        assert (d.cpu() - want).abs().max() < 1e-6
        x, gate = torch.randn(9, 24, generator=g).to(dt), torch.randn(9, 70, generator=g) * 3
        out = torch.empty(9, 24, dtype=dt, device=DEV)
        ops.gate_multiply(x.to(DEV), gate.to(DEV), 40, "sigmoid", out)
        close(out, x.to(F) * plain.sigmoid(gate[:, 40: 64].to(F)), dtype)
        ops.activate(gate.to(DEV), 5, "identity", out)
        close(out, gate[:, 5: 29].to(F), dtype)
        ops.activate(gate.to(DEV), 5, "gelu_tanh", out)
        close(out, plain.gelu_tanh(gate[:, 5: 29].to(F)), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,I,shared,n", [(5, 2, 24, 16, 40), (1, 1, 40, 0, 7), (6, 6, 8, 24, 300), (10, 3, 80, 112, 1), (3, 1, 64, 64, 130)])
def test_experts_with_a_router_bias_an_ungated_shared_expert_and_the_blocks_other_term(dtype, E, top, I, shared, n):
    from fusezap_core_b200.parts.routed_moe import RoutedMoE
    from fusezap_core_b200.engine.step import StepContext, Workspace
    ops, g, dt, D = cuda_ops(dtype), torch.Generator().manual_seed(E * I), DT[dtype], 64
    names = {"router": "router", "router_bias": "router.b", "expert": "e{}", "gate": "gate", "up": "up", "down": "down", "shared": "shared"}
    ff = RoutedMoE(D, I, E, top, shared_size=shared, renormalize=True, router_bias=True, shared_gate=False, names=names)
    w = {k: (torch.randn(p.shape, generator=g) * (1.0 if p.role == "vector" else 0.2)) for k, p in ff.tensors().items()}
    w = {k: v.to(dt).float() if v.dim() >= 2 else v for k, v in w.items()}
    ff.bind({k: (v.to(dt) if v.dim() >= 2 else v).to(DEV) for k, v in w.items()}, ops)
    h = torch.randn(n + 1, D, generator=g).to(dt)
    add = torch.randn(n + 1, D, generator=g)
    meta = Meta([(n, 0, -1)], pad=1)
    ctx = StepContext(ops, Workspace(torch.device(DEV), n + 1), meta, {}, None)
    out = ff.forward(ctx, h.to(DEV), add=add.to(DEV), scale=0.3)
    ops.check_errors()
    mlp = {"router": {"top": top}, "shared": {"ff": shared} if shared else None}
    ref = 0.3 * (add[:n].to(F) + plain.mixture({}, {k: v.to(F) for k, v in w.items()}, "", mlp, h[:n].to(F)))
    err = (out[:n].cpu().to(F) - ref).abs().max(-1).values / ref.abs().max()
    # (a row whose chosen logits nearly tie with the next one may choose otherwise in bfloat16)
    assert float(err.median()) < (1e-5 if dtype == "float32" else 2e-2) and float((err > 0.1).float().mean()) < 0.1
    assert float(out[n].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [64, 200, 1030])
def test_a_norm_whose_weight_is_stored_around_zero(dtype, D):
    """The part adds one to the stored weight in float32; the pending term joins the stream in the same pass; selected rows."""
    from fusezap_core_b200.parts.norm import RMSNorm
    from fusezap_core_b200.engine.step import StepContext, Workspace
    ops, g = cuda_ops(dtype), torch.Generator().manual_seed(D)
    norm = RMSNorm(D, 1e-5, name="w", offset=1.0)
    w = torch.randn(D, generator=g) * 0.3
    norm.bind({"w": w.to(DEV)}, ops)
    x, delta = torch.randn(9, D, generator=g), torch.randn(9, D, generator=g)
    ctx = StepContext(ops, Workspace(torch.device(DEV), 9), Meta([(9, 0, -1)]), {}, None)
    xd = x.to(DEV)
    h = norm.forward(ctx, xd, delta.to(DEV))
    close(h, plain.one_plus_norm((x + delta).to(F), w.to(F), 1e-5), dtype)
    assert (xd.cpu() - (x + delta)).abs().max() < 1e-6
    rows = torch.tensor([7, -1, 0], dtype=torch.int32, device=DEV)
    h = norm.forward(ctx, xd, None, rows=rows)
    ref = plain.one_plus_norm((x + delta)[[7, 0]].to(F), w.to(F), 1e-5)
    close(h[[0, 2]], ref, dtype)
    assert float(h[1].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_strong_blend_of_values_shows_in_the_logits(dtype, tmp_path):
    """Blend weights of 0.8 and -0.5 in the later layers (and a first layer's own weight that must not matter): the model
    follows the plain one, whole, in portions and token by token, and differs from itself without the blend."""
    def strong(t):
        t.update({"l0.mix.vmix": torch.tensor(0.9), "l3.mix.vmix": torch.tensor(0.8)})
    d, cfg, w = make_dir("mix", tmp_path, change=strong)
    model, cache, runner = engine_parts(d, dtype)
    toks = tokens_for(cfg, (60,), seed=4)[0]
    ref = oracle(cfg, w, toks, dtype)
    for cuts in ((60,), (1,), (7, 2, 1)):
        agrees(run_cut(runner, cache, "r", toks, cuts), ref, dtype, cuts)
    plainer = oracle(cfg, {**w, "l3.mix.vmix": torch.tensor(0.0)}, toks, dtype)
    assert row_errors(plainer, ref).max() > 0.1


# ------------------------------------------------------------------------------------------------ the model, further
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dirs, dtype):
    """Through `LLMEngine` and its scheduler (portions of prompts beside decoding requests, more requests than state
    slots, a pool that does not hold all requests at once): every generated token is the plain model's choice, or
    within rounding of it."""
    d, cfg, w = dirs["odd"]
    eng = LLMEngine.from_pretrained(d, dtype=dtype, device=DEV, max_model_len=96, num_blocks=20, block_size=8,
                                    max_num_seqs=3, max_prefill_tokens=16)
    P = tokens_for(cfg, (7, 23, 2, 41, 12), seed=2)
    out = eng.generate(P, SamplingParams(max_tokens=9, ignore_eos=True))
    margin = 1e-3 if dtype == "float32" else 0.15
    for prompt, new in zip(P, out):
        lg = oracle(cfg, w, list(prompt) + new, dtype)
        for i, t in enumerate(new):
            row = lg[len(prompt) - 1 + i]
            assert int(row.argmax()) == t or row.max() - row[t] < margin, (dtype, i, t)


def test_command_line_generates_from_a_preset_with_random_weights(capsys):
    from fusezap_core_b200.cli import main
    assert main(["generate", "--random", "tiny-gimotar", "--prompt-lens", "5,40,1", "--max-tokens", "6", "--ignore-eos",
                 "--max-model-len", "128", "--num-blocks", "32", "--max-num-seqs", "2"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    assert [o["num_prompt_tokens"] for o in lines] == [5, 40, 1]
    assert all(len(o["token_ids"]) == 6 and o["finish_reason"] == "length" for o in lines)


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Every size and constant comes from the configuration: drawn ones in float32 against the plain model (whole, in
    portions, token by token), and in bfloat16; a long prompt first, so that prompt portions reach every kernel."""
    cfg = drawn_config(seed)
    d, cfg, w = make_dir(f"drawn{seed}", tmp_path, cfg, seed)
    toks = tokens_for(cfg, (150,), seed=seed)[0]
    for dtype in ("float32", "bfloat16"):
        model, cache, runner = engine_parts(d, dtype, page=16, pages=12, slots=2, max_len=160)
        ref = oracle(cfg, w, toks, dtype)
        for cuts in ((150,), (130, 1), (70, 2, 1, 17)):
            got = run_cut(runner, cache, "r", toks, cuts)
            model.ops.check_errors()
            agrees(got, ref, dtype, (seed, dtype, cuts, json.dumps(cfg)[:600]))


@pytest.mark.parametrize("seed", range(4))
def test_configurations_of_a_small_models_size(seed, tmp_path):
    """Widths of a few hundred, head sizes up to 128, prompts of hundreds of tokens in a pool that holds the live requests
    only: whole, with a decoded tail, in portions down to two tokens, and beside other requests, in both dtypes."""
    cfg = drawn_config(seed, small=False)
    d, cfg, w = make_dir(f"model{seed}", tmp_path, cfg, seed)
    L = (421, 700, 333, 1000)[seed]
    toks, *others = tokens_for(cfg, (L, 1, 23, 97), seed=seed)
    for dtype in ("float32", "bfloat16"):
        need = sum(-(-len(t) // 64) * 64 for t in [toks] + others)
        model, cache, runner = engine_parts(d, dtype, page=16, pages=need // 16, slots=4, max_len=1024)
        refs = [oracle(cfg, w, t, dtype) for t in [toks] + others]
        what = (seed, dtype, json.dumps(cfg)[:600])
        for cuts in ((L,), (L - 40,) + (1,) * 40, (5, 64, 2, 33, 128, 7, 1, 1, 100, 2, 16, 17)):
            got = run_cut(runner, cache, "r", toks, cuts)
            model.ops.check_errors()
            agrees(got, refs[0], dtype, (*what, cuts))
        reqs = dict(zip("abcd", [toks] + others))
        plan = [[("a", 100), ("b", 1)], [("a", 2), ("c", 23)], [("a", 64), ("d", 50)], [("a", 1), ("d", 2)]] + \
               [[("a", 200), ("d", 1)]] * 50
        got = run_mixed(runner, cache, reqs, plan)
        model.ops.check_errors()
        for r, ref in zip("abcd", refs):
            agrees(got[r], ref, dtype, (*what, "mixed", r))
