"""Nepudra on the GPU: the whole model through the engine's step function, cache manager and kernels against the plain
implementation (`plain_nepudra.py`, 64-bit, whole sequences), in float32 and bfloat16."""
import numpy as np
import pytest
import torch

from nepudra_util import CONFIGS, drawn_config, drawn_model_config, make_dir, plain_logits, rounded, tokens_for
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


# ---------------------------------------------------------------------------------------- each mechanism alone
import plain_nepudra as plain
from fusezap_core_b200.cache import KVNeed
from fusezap_core_b200.kernels import cuda_ops
from fusezap_core_b200.parts import LayerCache
from test_gizulorn_gpu import DEV, DT, F, Meta, close, paged, scan_portions, shuffled_tables


@pytest.mark.parametrize("H,dk,dv", [(2, 16, 16), (3, 20, 12), (1, 48, 48), (4, 8, 40), (2, 64, 64), (1, 128, 128), (5, 12, 7),
                                     (1, 136, 24)])
def test_general_delta_scan_carries_its_state_across_portions(H, dk, dv):
    """Two requests in interleaved portions down to one token, in slots 3 and 1 of four: every output against the plain
    recurrence over the whole sequence, the other slots untouched."""
    ops, g, T = cuda_ops("float32"), torch.Generator().manual_seed(dk + dv), 70
    off_a = 2 * H * dk + H * dv + 3                     # (some columns lie between v and the removal inputs)
    ld = off_a + H * dk + 2
    proj = [torch.randn(T, ld, generator=g) for _ in range(2)]
    din = [torch.randn(T, H * dk, generator=g) * 2 for _ in range(2)]
    dbias, abias = torch.randn(H * dk, generator=g), torch.randn(H * dk, generator=g)
    rate, unit_eps = 0.6, 1e-6
    state = torch.zeros(4, *ops.recurrent_state_shape(H, dk, dv), device=DEV)
    state[2] = 3.0
    slots, got = (3, 1), [torch.zeros(T, H * dv), torch.zeros(T, H * dv)]
    for step in scan_portions(T, seed=dk):
        meta = Meta([(n, p0, slots[r]) for r, p0, n in step], pad=1)
        cat = lambda xs, w: torch.cat([xs[r][p0: p0 + n] for r, p0, n in step] + [torch.zeros(1, w)]).to(DEV)
        out = torch.full((meta.n_rows, H * dv), 9.0, device=DEV)
        ops.general_delta_scan(cat(proj, ld), H, dk, dv, off_a, cat(din, H * dk), dbias.to(DEV), abias.to(DEV), rate, unit_eps,
                               state, meta, out)
        at = 0
        for r, p0, n in step:
            got[r][p0: p0 + n] = out[at: at + n].cpu()
            at += n
    ops.check_errors()
    for r in (0, 1):
        x = proj[r].to(F)
        rr, k = x[:, :H * dk].view(T, H, dk), x[:, H * dk: 2 * H * dk].view(T, H, dk)
        v = x[:, 2 * H * dk: 2 * H * dk + H * dv].view(T, H, dv)
        d = torch.exp(-rate * plain.sigmoid(din[r].to(F) + dbias.to(F))).view(T, H, dk)
        a = plain.sigmoid(x[:, off_a: off_a + H * dk] + abias.to(F)).view(T, H, dk)
        ref, _ = plain.delta_recurrence(rr, k, v, d, a, None, unit_eps)
        close(got[r].view(T, H, dv), ref, "float32", f"request {r}")
    assert (state[2] == 3.0).all() and float(state[0].abs().max()) == 0.0


def test_a_written_pair_is_read_back_until_its_key_is_removed():
    """Inputs made so that a fault shows: token 0 writes k0 v0^T; with decay 1 and no removal a query along k0 reads v0
    back after any number of tokens whose keys are orthogonal to k0; with removal rate 1 a later token whose key is k0
    again erases exactly that row before it writes its own."""
    ops, H, dk, dv, T = cuda_ops("float32"), 1, 16, 8, 40
    k = torch.zeros(T, dk)
    k[0, 0] = 2.0
    for t in range(1, T):
        k[t, 1 + t % (dk - 1)] = 1.0
    k[30] = k[0]
    v = torch.randn(T, dv, generator=torch.Generator().manual_seed(1))
    r = torch.zeros(T, dk)
    r[:, 0] = 0.5                                        # every query reads row 0 of the state: 0.5 * 2 * v0 = v0
    proj = torch.cat([r, k, v, torch.full((T, dk), 30.0)], 1)     # removal inputs: sigmoid(30) = 1
    proj[:30, 2 * dk + dv:] = -30.0                                # ... but none before token 30
    din = torch.full((T, dk), -40.0)                               # sigmoid -> 0: decay exp(0) = 1
    state = torch.zeros(1, *ops.recurrent_state_shape(H, dk, dv), device=DEV)
    outs = []
    for p0, n in ((0, 1), (1, 9), (10, 1), (11, 19), (30, 1), (31, 9)):
        out = torch.empty(n, dv, device=DEV)
        ops.general_delta_scan(proj[p0: p0 + n].to(DEV), H, dk, dv, 2 * dk + dv, din[p0: p0 + n].to(DEV), torch.zeros(dk, device=DEV),
                               torch.zeros(dk, device=DEV), 1.0, 0.0, state, Meta([(n, p0, 0)]), out)
        outs.append(out.cpu())
    o = torch.cat(outs)
    assert float((o[:30] - v[0]).abs().max()) < 1e-5
    assert float((o[30:] - v[30]).abs().max()) < 1e-5 and float((v[30] - v[0]).abs().max()) > 0.1


def test_hashed_pair_rows_first_tokens_and_the_token_before_a_portion():
    """Rows of two requests in portions down to one token, multipliers whose products leave 32 bits, a padding row; the
    first token of a request takes the last row whatever its slot held before."""
    from fusezap_core_b200.parts import EMBED_EXTRAS, build
    from fusezap_core_b200.config import PartSpec
    ops, D, buckets, mp, mc, V = cuda_ops("float32"), 24, 97, 2_000_000_011, 1_999_999_973, 50_000
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    g = torch.Generator().manual_seed(4)
    table = torch.randn(buckets + 1, D, generator=g)
    toks = [torch.randint(0, V, (n,), generator=g).tolist() for n in (23, 9)]
    w = {"embed": torch.zeros(V, D, dtype=F), "bigram": table.to(F)}
    ref = [plain.embedding(cfg, w, t) for t in toks]
    state = torch.full((3, 1), 12345, dtype=torch.int32, device=DEV)      # (slots hold what an earlier request left)
    steps = [[(0, 0, 1), (1, 0, 4)], [(0, 1, 1)], [(0, 2, 7), (1, 4, 1)], [(1, 5, 4)], [(0, 9, 14)]]
    slots = (2, 0)
    for step in steps:
        meta = Meta([(n, p0, slots[r]) for r, p0, n in step], pad=1)
        ids = torch.tensor([t for r, p0, n in step for t in toks[r][p0: p0 + n]] + [0], dtype=torch.int32, device=DEV)
        x = torch.ones(meta.n_rows, D, device=DEV)
        ops.hashed_pair_embed(table.to(DEV), ids, meta, state, buckets, mp, mc, x)
        ops.check_errors()
        at = 0
        for r, p0, n in step:
            assert torch.equal(x[at: at + n].cpu() - 1.0, (ref[r][p0: p0 + n].float() + 1.0) - 1.0), (r, p0)
            at += n
        assert float((x[at:] - 1.0).abs().max()) == 0.0
    assert state.view(-1).tolist() == [toks[1][-1], 12345, toks[0][-1]]


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,L", [(64, 3), (320, 6), (100, 1), (2050, 4)])
def test_depth_average_keeps_every_stream_and_feeds_the_norm(dtype, D, L, fused):
    """Layer by layer: the kept streams, the averaged stream and the norm of it (of all rows, and of chosen rows at the
    last depth), with the sum folded into the norm's pass and without."""
    ops, g, n = cuda_ops(dtype), torch.Generator().manual_seed(D), 11
    ops.fuse_depth_norm = fused
    streams = torch.zeros(n, L + 1, D, device=DEV)
    x0 = torch.randn(n, D, generator=g)
    x = x0.clone().to(DEV)
    ops.depth_average(streams, -1, None, x, None)
    kept, cur = [x0.to(F)], x0.to(F)
    wn = (1 + 0.1 * torch.randn(D, generator=g)).float()
    for depth in range(L):
        delta, coef = torch.randn(n, D, generator=g), torch.randn(depth + 2, generator=g)
        kept.append(cur + delta.to(F))
        cur = plain.depth_average(kept, coef.to(F))
        href = plain.rms(cur, 1e-5) * wn.to(F)
        h = torch.empty(n, D, dtype=DT[dtype], device=DEV)
        if depth == L - 1:            # chosen rows only: nothing but h is written
            rows = torch.tensor([n - 1, -1, 0, 3], dtype=torch.int32, device=DEV)
            hr = torch.empty(4, D, dtype=DT[dtype], device=DEV)
            before = (streams.clone(), x.clone())
            if ops.depth_average_rmsnorm(streams, depth, coef.to(DEV), x, delta.to(DEV), wn.to(DEV), 1e-5, hr, rows):
                assert fused and torch.equal(streams, before[0]) and torch.equal(x, before[1])
                close(hr[[0, 2, 3]], href[[n - 1, 0, 3]], dtype, "chosen rows")
                assert float(hr[1].abs().max()) == 0.0
            else:
                assert not fused
        if not ops.depth_average_rmsnorm(streams, depth, coef.to(DEV), x, delta.to(DEV), wn.to(DEV), 1e-5, h):
            assert not fused
            ops.depth_average(streams, depth, coef.to(DEV), x, delta.to(DEV))
            ops.add_rmsnorm(x, None, wn.to(DEV), 1e-5, h)
        ops.check_errors()
        close(streams[:, depth + 1], kept[-1], "float32", f"kept {depth}")
        close(x, cur, "float32", f"average {depth}")
        close(h, href, dtype, f"norm {depth}")
    ops.fuse_depth_norm = True


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,dk,dv,dims,scaling,normed,temp", [
    (4, 2, 16, 8, 8, (4.0, 16, 4.0, 0.5), True, None), (3, 3, 24, 40, 24, None, True, (0.7, 3)), (2, 1, 96, 96, 96, (4.0, 64, 8.0, 1.0), True, None),
    (6, 1, 8, 8, 0, None, False, (1.5, 1)), (2, 2, 64, 64, 32, (8.0, 32, 2.0, 1.0), False, (0.2, 7)), (8, 2, 128, 128, 2, (2.0, 8, 3.0, 0.1), True, (0.5, 256))])
def test_rotation_with_head_norms_scaled_frequencies_and_query_temperature(dtype, Hq, Hkv, dk, dv, dims, scaling, normed, temp):
    """Two portions (one past several temperature periods) and a padding row on shuffled pages: q as the attention
    reads it, k and v as the cache holds them, against the plain functions."""
    from fusezap_core_b200.parts.rope import RotaryEncoding
    ops, g, page, eps = cuda_ops(dtype), torch.Generator().manual_seed(dk + dv), 4, 1e-5
    rot = {"base": 300.0, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    portions = [(7, 250, 0), (1, 0, 1), (3, 1, 2)]
    tables = shuffled_tables(3, 70, 300, seed=dk)
    meta = Meta(portions, tables, pad=1)
    n = meta.n_rows
    qkv = torch.randn(n, (Hq + Hkv) * dk + Hkv * dv, generator=g)
    qn, kn = ((1 + 0.2 * torch.randn(dk, generator=g)).float(), (1 + 0.2 * torch.randn(dk, generator=g)).float()) if normed else (None, None)
    cache = paged(KVNeed(Hkv, dk, 0, value_dim=dv), page, 300, dtype)
    cos = sin = None
    if dims:
        kw = dict(kind="yarn", factor=scaling[0], original_max_position_embeddings=scaling[1], turns_fast=scaling[2],
                  turns_slow=scaling[3], magnitude=0.1 * np.log(scaling[0]) + 1.0) if scaling else {}
        enc = RotaryEncoding(dims, 300.0, precise=True, **kw)
        enc.prepare(280, torch.device(DEV))
        cos, sin = enc.cos, enc.sin
    q_out = torch.empty(n, Hq * dk, dtype=DT[dtype], device=DEV)
    ops.rotate_kv_write(qkv.to(DEV), cos, sin, dims, 0, meta, cache, q_out, Hq, Hkv, dk, dv,
                        q_norm=qn.to(DEV) if normed else None, k_norm=kn.to(DEV) if normed else None, norm_eps=eps, query_temperature=temp)
    ops.check_errors()
    at = 0
    for s, (cnt, p0, _) in enumerate(portions):
        x = qkv[at: at + cnt].to(F)
        q = x[:, :Hq * dk].view(cnt, Hq, dk)
        k = x[:, Hq * dk:(Hq + Hkv) * dk].view(cnt, Hkv, dk)
        if normed:
            q, k = plain.rms(q, eps) * qn.to(F), plain.rms(k, eps) * kn.to(F)
        if dims:
            c, sn = plain.yarn_angles(rot, p0 + cnt)
            q, k = plain.rotate_halves(q, c[p0:], sn[p0:], dims), plain.rotate_halves(k, c[p0:], sn[p0:], dims)
        if temp:
            q = q * plain.query_temperature({"coef": temp[0], "every": temp[1]}, torch.arange(p0, p0 + cnt, dtype=F))[:, None, None]
        close(q_out[at: at + cnt].view(cnt, Hq, dk), q, dtype, "q")
        for i in range(cnt):
            pg, off = int(tables[s, (p0 + i) // page]), (p0 + i) % page
            close(cache.keys[pg, :, off], k[i], dtype, "k")
            close(cache.values[pg, :, off], x[i, (Hq + Hkv) * dk:].view(Hkv, dv), dtype, "v")
        at += cnt
    assert float(q_out[at:].abs().max()) == 0.0


def attention_rows(dtype, Hq, Hkv, dk, dv, window, cap, gated, T, portions, page, seed, loud=None, scale=0.3):
    """One sequence of T tokens in shuffled pages; `portions` ((rows, first position) each) are asked for in one step,
    each through a block table of its own. loud: (key position, factor): that key and every query point one way, so
    that its score stands out. Returns (outputs of the rows, the plain result for them, the values)."""
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
    cache = paged(KVNeed(Hkv, dk, window, value_dim=dv), page, pages + 5, dtype)
    qkv = torch.cat([q.view(T, -1), k.view(T, -1), v.view(T, -1)], 1).float()
    ops.rotate_kv_write(qkv.to(DEV), None, None, 0, 0, Meta([(T, 0, 0)], table), cache, torch.empty(T, Hq * dk, dtype=dt, device=DEV), Hq, Hkv, dk, dv)
    meta = Meta([(n, p0, 0) for n, p0 in portions], table.repeat(len(portions), 1), pad=1)
    meta.max_portion = max(n for n, _ in portions)      # (a step of single tokens takes the kernels that cut a row's keys into runs)
    rows = [p for n, p0 in portions for p in range(p0, p0 + n)]
    qs = torch.cat([q[rows].view(len(rows), -1), torch.zeros(1, Hq * dk, dtype=dt)]).to(DEV)
    gl = torch.randn(T, Hq + 3, generator=g) * 2
    gate = (torch.cat([gl[rows], torch.zeros(1, Hq + 3)]).to(DEV), 2) if gated else None
    out = torch.empty(len(rows) + 1, Hq * dv, dtype=dt, device=DEV)
    ops.sink_attention(qs, cache, meta, out, Hq, Hkv, dk, dv, scale, window, 0, None, softcap=cap, gate=gate)
    ops.check_errors()
    assert float(out[-1].abs().max()) == 0.0
    ref = plain.softmax_attention(q.to(F), k.to(F), v.to(F), scale, window, cap)
    if gated:
        ref = ref * plain.sigmoid(gl[:, 2: 2 + Hq].to(F))[:, :, None]
    return out[:-1].view(len(rows), Hq, dv), ref[rows], v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,dk,dv,window,cap,gated", [
    (4, 2, 16, 8, 9, 2.5, True), (3, 3, 24, 40, 0, 1.0, True), (8, 2, 96, 96, 0, 20.0, True), (6, 3, 96, 96, 33, 0.0, True),
    (8, 2, 64, 64, 0, 3.0, True), (4, 4, 128, 128, 70, 0.0, True), (2, 1, 128, 128, 0, 0.75, False), (6, 1, 64, 64, 65, 30.0, False),
    (1, 1, 32, 16, 5, 0.0, False)])      # (in bfloat16 the sizes 64 and 128 run their long portions on tensor cores)
def test_attention_with_capped_scores_windows_and_head_gates(dtype, Hq, Hkv, dk, dv, window, cap, gated):
    """Rows of long and short portions and single tokens, at the start of the sequence and far into it."""
    got, ref, _ = attention_rows(dtype, Hq, Hkv, dk, dv, window, cap, gated, T=200, page=4, seed=Hq * dk + window,
                                 portions=[(70, 0), (2, 80), (1, 97), (1, 199), (1, 5), (90, 100)])
    if dtype == "bfloat16" and dk == dv and dk in (64, 128):
        # the tensor-core kernel rounds the softmax weights to bfloat16 for the value product: besides the rounding of
        # the result, each of up to 200 terms is off by up to 2^-9 of itself, which shows where the terms cancel
        err, ref = (got.detach().cpu().to(F) - ref).abs(), ref.to(F)
        assert not (err > 2.0 ** -7 * (ref.abs() + 4 * ref.abs().mean() + 1e-3)).any(), float(err.max())
    else:
        close(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("as_portion", [True, False])
@pytest.mark.parametrize("dk,dv,window,cap", [(16, 8, 12, 0.0), (64, 64, 12, 0.0), (96, 96, 0, 50.0), (64, 64, 0, 50.0), (128, 128, 70, 60.0)])
def test_a_loud_key_is_seen_exactly_where_the_mask_says(dtype, as_portion, dk, dv, window, cap):
    """One key's score exceeds all others by far (also under the cap, which is chosen above it), so a row's output is
    that key's value if the row sees the key: the first key, keys at page borders and far back, just inside and just
    outside the window, for rows of prompt portions (64 rows and more: the tensor-core kernel where the sizes allow)
    and for single tokens."""
    page, T = 8, 700
    far = window or 500
    for j in (0, 7, 8, 300 if window else 15, T - 1 - far, T - far, T - 2):
        rows = sorted({p for p in (j, j + 1, j + far - 1, j + far, j + far + 1, T - 1) if j <= p < T})
        if as_portion:
            portions, p = [], None
            for r in rows:                       # portions of 70 rows that end at the rows of interest
                lo = max(0, r - 69)
                portions.append((r - lo + 1, lo))
        else:
            portions = [(1, p) for p in rows]
        got, ref, v = attention_rows(dtype, 2, 1, dk, dv, window, cap, False, T, portions, page, seed=j, loud=(j, 12.0), scale=0.3)
        close(got, ref, dtype, f"key {j}")
        at = 0
        for n, p0 in portions:
            for p in range(p0, p0 + n):
                sees = j <= p and (not window or p - j < window)
                same = bool((got[at].float().cpu() - v[j].float()).abs().max() < 0.05)
                if p >= j:
                    assert same == sees, (j, p, sees)
                at += 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,dk,dv,window", [(4, 2, 64, 64, 0), (6, 3, 32, 96, 37), (2, 1, 128, 128, 0), (4, 1, 24, 40, 20)])
def test_wide_and_narrow_loads_of_the_cache_give_the_same_bits(dtype, Hq, Hkv, dk, dv, window):
    """The attention kernels read keys and values 16 bytes at a time where sizes, strides and addresses allow it and
    element by element otherwise. The same pages in a pool whose first element lies at an odd address take the narrow
    path: portions and single tokens leave the same bits on both."""
    ops, g, page, B, T = cuda_ops(dtype), torch.Generator().manual_seed(dk + dv), 8, 3, 150
    per = -(-T // page)
    need = KVNeed(Hkv, dk, 0, value_dim=dv)
    shape = need.pool_shape(1, B * per + 2, page)
    count = 1
    for x in shape:
        count *= x
    even = torch.randn(count, generator=g).to(DT[dtype]).to(DEV)
    shifted = torch.zeros(count + 8, dtype=DT[dtype], device=DEV)
    shifted[1: 1 + count] = even
    caches = []
    for flat in (even, shifted[1: 1 + count]):
        keys, values = need.views(flat.view(shape)[0])
        caches.append(LayerCache(keys, values, 0, page, True, {}))
    assert caches[0].keys.data_ptr() % 16 == 0 and caches[1].keys.data_ptr() % 16 != 0
    tables = shuffled_tables(B, per, B * per + 2, 5)
    for portions in ([(40, T - 40, 0), (1, T - 1, 1), (17, 60, 2)], [(1, T - 1, 0), (1, 77, 1), (1, 8, 2)]):
        meta = Meta(portions, tables, pad=1)
        meta.max_portion = max(n for n, _, _ in portions)
        n = meta.n_rows
        q = torch.randn(n, Hq * dk, generator=g).to(DT[dtype]).to(DEV)
        gate = torch.randn(n, Hq, generator=g).to(DEV)
        outs = []
        for cache in caches:
            out = torch.empty(n, Hq * dv, dtype=DT[dtype], device=DEV)
            before, ops.sink_tensor_cores = ops.sink_tensor_cores, False     # (the tensor-core kernel takes aligned pools only)
            try:
                ops.sink_attention(q, cache, meta, out, Hq, Hkv, dk, dv, 0.2, window, 0, None, softcap=9.0, gate=(gate, 0))
            finally:
                ops.sink_tensor_cores = before
            ops.check_errors()
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), portions


# ------------------------------------------------------------------------------------------------ the model, further
from fusezap_core_b200 import LLMEngine, SamplingParams


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
    import json
    from fusezap_core_b200.cli import main
    assert main(["generate", "--random", "tiny-nepudra", "--prompt-lens", "5,40,1", "--max-tokens", "6", "--ignore-eos",
                 "--max-model-len", "128", "--num-blocks", "32", "--max-num-seqs", "2"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    assert [o["num_prompt_tokens"] for o in lines] == [5, 40, 1]
    assert all(len(o["token_ids"]) == 6 and o["finish_reason"] == "length" for o in lines)


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Every size and constant comes from the configuration: drawn ones in float32 against the plain model (whole, in
    portions, token by token), and in bfloat16; a long prompt first, so that prompt portions reach every kernel."""
    import json
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
    import json
    cfg = drawn_model_config(seed)
    d, cfg, w = make_dir(f"model{seed}", tmp_path, cfg, seed)
    L = (421, 700, 333, 1000)[seed]
    toks, *others = tokens_for(cfg, (L, 1, 23, 97), seed=seed)
    for dtype in ("float32", "bfloat16"):
        need = sum(-(-len(t) // 64) * 64 for t in [toks] + others)
        model, cache, runner = engine_parts(d, dtype, page=16, pages=need // 16, slots=4, max_len=1024)
        refs = [oracle(cfg, w, t, dtype) for t in [toks] + others]
        what = (seed, dtype, json.dumps(cfg)[:600])
        for cuts in ((L,), (L - 40,) + (1,) * 40, (5, 64, 2, 33, 128, 7, 1, 1, 100, 2, 16, 17)):
            agrees(run_cut(runner, cache, "r", toks, cuts), refs[0], dtype, what + (cuts[:3],))
            model.ops.check_errors()
        plan = [[("a", 200), ("b", 1)], [("a", 3), ("c", 20)], [("a", 1), ("c", 1), ("d", 50)], [("a", 64), ("c", 2), ("d", 2)],
                [("a", 1), ("d", 45)]] + [[("a", 1)]] * 6 + [[("a", 2000)]]
        got = run_mixed(runner, cache, dict(zip("abcd", [toks] + others)), plan)
        model.ops.check_errors()
        for r, ref in zip("acd", (refs[0], refs[2], refs[3])):
            agrees(got[r], ref, dtype, what + (r,))
