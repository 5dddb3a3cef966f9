"""Pesanex on the device against its plain statement (tests/plain_pesanex.py, float64, whole sequences).

Whole models: every way of cutting the work (whole prompts, a tail decoded token by token, portions down to two
tokens and one, mixed batches with four state slots that are used again), bit for bit against one another in 32-bit;
long decoding; long portions cut into segments; greedy generation through the scheduler.  Mechanisms alone: the
centred norm and the norm of a branch, rotation with unit-norm heads and value heads of their own size, attention
with sinks (a far key made to stand out, contexts at the edges of pages and of the kernels' tiles and chunks), the
decayed-state recurrence with its state carried from call to call.
"""
import math

import pytest
import torch

import plain_pesanex as plain
import traces
from helpers import folder_weights, max_diff
from pesanex_configs import CONFIGS, write_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runner_for(folder, dtype, page_size, pages, slots=4, poison=True):
    from wllm_b200.config import EngineConfig
    from wllm_b200.engine import build_model, build_runner
    eng = EngineConfig(dtype=dtype, block_size=page_size, max_num_seqs=slots)
    return build_runner(build_model(folder, eng.dtype, eng.device), eng, num_pages=pages, poison_pages=poison)


def plain_rows(folder, name, reqs):
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    return {(rid, p): row.float() for rid, toks in reqs.items() for p, row in enumerate(plain.forward(toks, w, CONFIGS[name]))}


def close_enough(rows, ref, dtype, what=""):
    """32-bit: every logit within 2e-4 of the scale.  bfloat16: by rows.  A head of the recurrence is divided by its
    own root mean square, so where q . k of a sequence's first tokens nearly cancels, rounding q and k to bfloat16 can
    turn the whole head round (the plain statement does the same with its inputs rounded): single rows may be far off
    in any implementation.  So the typical row must be close and few rows may be far."""
    assert set(rows) == set(ref)
    scale = max(1.0, max(float(r.abs().max()) for r in ref.values()))
    if dtype == torch.float32:
        assert max_diff(rows, ref) < 2e-4 * scale, what
        return
    rel = sorted(float((rows[k].double() - ref[k].double()).pow(2).mean().sqrt() / ref[k].double().pow(2).mean().sqrt()) for k in ref)
    assert rel[len(rel) // 2] < 0.03 and rel[int(len(rel) * 0.9)] < 0.1, (what, rel[len(rel) // 2], rel[int(len(rel) * 0.9)], rel[-1])


def requests_of(name, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in CONFIGS:
        folder = write_folder(str(tmp_path_factory.mktemp("pesanex") / name), name)
        reqs = requests_of(name, (5, 64, 31, 90, 2, 47, 70, 25, 1, 113, 17), seed=3)
        out[name] = (folder, reqs, plain_rows(folder, name, reqs))
    return out


CUTS = (("whole", traces.whole), ("tail", lambda r: traces.tail_singly(r, 16)), ("portions", traces.portions),
        ("mixed", lambda r: traces.mixed(r, seed=5)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_matches_the_plain_statement(setups, name, dtype):
    folder, reqs, ref = setups[name]
    first = None
    for cut, make in CUTS:
        steps = make(reqs)
        pages = -(-traces.peak_tokens(steps) // 16)
        runner = runner_for(folder, dtype, 16, pages)
        rows = traces.run_in_process(runner, steps)
        close_enough(rows, ref, dtype, cut)
        assert all(f == pages for f in runner.cache.free_pages()) and runner.cache.slots.num_free == 4
        if cut == "mixed":      # pages and state slots were used again
            assert all(g.pool.takes > pages for g in runner.cache.groups) and len(reqs) > 4
        if dtype == torch.float32:      # no portion is long enough to be cut into segments: every cut gives the same bits
            if first is None:
                first = rows
            else:
                bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                assert not bad, f"{cut}: first differing (request, position) {bad[0]}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_keeps_the_state(setups, dtype):
    folder = setups["mix"][0]
    reqs = requests_of("mix", (190,), seed=8)
    ref = plain_rows(folder, "mix", reqs)
    steps = traces.tail_singly(reqs, 150)
    runner = runner_for(folder, dtype, 16, -(-traces.peak_tokens(steps) // 16))
    close_enough(traces.run_in_process(runner, steps), ref, dtype)


def test_decoding_from_captured_graphs_advances_the_state_once_a_step(setups):
    """The run that warms a capture up must leave no trace in the state slots; rows under graphs are the eager rows."""
    folder, reqs, ref = setups["plain"]
    some = {k: reqs[k] for k in ("r1", "r2", "r5")}
    steps = traces.tail_singly(some, 24)
    rows = {}
    for graphs in (False, True):
        runner = runner_for(folder, torch.float32, 16, -(-traces.peak_tokens(steps) // 16), poison=False)
        assert runner.model.graph_safe
        if graphs:
            runner.enable_graphs()
        rows[graphs] = traces.run_in_process(runner, steps)
        assert (runner.graph_launches > 0) == graphs
        close_enough(rows[graphs], {k: v for k, v in ref.items() if k[0] in some}, torch.float32)
    bad = sorted(k for k in rows[False] if not torch.equal(rows[False][k], rows[True][k]))
    assert not bad, f"first differing (request, position) {bad[0]}"


@pytest.mark.parametrize("name", ["mix", "plain"])
def test_long_portions_cut_into_segments(setups, name, monkeypatch):
    """The recurrence over a long portion runs as segments side by side (local end states, chained, walked again);
    here already from 24 tokens in segments of 8, beside short requests and decoded tokens in the same batch."""
    from wllm_b200.kernels import ops
    monkeypatch.setattr(ops, "LINATTN_SEGMENT_FROM", 24)
    monkeypatch.setattr(ops, "LINATTN_MIN_SEGMENT", 8)
    assert ops.linattn_segment_plan(150, 1, 2, 24)[1] > 2
    folder = setups[name][0]
    reqs = requests_of(name, (150, 61, 9, 230), seed=21)
    ref = plain_rows(folder, name, reqs)
    for cut, make in (("whole", traces.whole), ("portions", lambda r: traces.portions(r, sizes=(50, 71, 2, 30, 29, 100))),
                      ("mixed", lambda r: traces.mixed(r, seed=2, max_portion=60))):
        steps = make(reqs)
        runner = runner_for(folder, torch.float32, 16, -(-traces.peak_tokens(steps) // 16))
        close_enough(traces.run_in_process(runner, steps), ref, torch.float32, cut)


def test_greedy_generation_through_the_scheduler(setups):
    from wllm_b200 import LLM, SamplingParams
    folder, reqs, _ = setups["mix"]
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    prompts = [reqs["r0"], reqs["r2"], reqs["r3"][:40], reqs["r8"]]
    llm = LLM(folder, dtype="float32", block_size=16, num_blocks=12, chunked_prefill_tokens=24, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        for _ in range(10):
            toks.append(int(plain.forward(toks, w, CONFIGS["mix"])[-1].argmax()))
        assert o.token_ids == toks[len(prompt):]
    assert llm.runner.cache.slots.num_free == 3 and all(f == 12 for f in llm.runner.cache.free_pages())
    bf = LLM(folder, dtype="bfloat16", block_size=16, num_blocks=12, chunked_prefill_tokens=24, max_num_seqs=3, cuda_graphs=True)
    assert [len(o.token_ids) for o in bf.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))] == [10] * 4


# ------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H", [96, 320, 1000, 4099])
def test_centred_norm_and_norm_of_a_branch(H):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(H)
    n = 7
    x = torch.randn(n, H, generator=g) * 3 + 1.5
    d = torch.randn(3, n, H, generator=g)
    w = torch.randn(H, generator=g)
    want = plain.layer_norm((x + d.sum(0)).double(), w.double(), 1e-5)
    resid, out = x.to(DEV), torch.empty(n, H, device=DEV)
    ops.rmsnorm(resid, d.to(DEV), w.to(DEV), 1e-5, 0.0, out, delta_splits=3, center=True)
    assert (out.cpu().double() - want).abs().max() < 1e-5 and (resid.cpu() - (x + d[0] + d[1] + d[2])).abs().max() < 1e-6
    rows = torch.tensor([5, 0, 2], dtype=torch.int32, device=DEV)
    some = torch.empty(3, H, device=DEV)
    ops.rmsnorm(resid, None, w.to(DEV), 1e-5, 0.0, some, rows=rows, center=True)
    assert (some.cpu().double() - want[[5, 0, 2]]).abs().max() < 1e-5
    # a branch alone (centred), and the mean of two branches (root mean square), one of them still in parts, one bfloat16
    a, b = torch.randn(n, H, generator=g) * 2, (torch.randn(n, H, generator=g) + 0.5).bfloat16()
    wb = w.bfloat16()
    y = ops.branch_norm((a.to(DEV), 0), w.to(DEV), torch.empty(n, H, device=DEV), 1e-5, center=True)
    assert (y.cpu().double() - plain.layer_norm(a.double(), w.double(), 1e-5)).abs().max() < 1e-5
    y = ops.branch_norm((d.to(DEV), 3), wb.to(DEV), torch.empty(n, H, device=DEV), 1e-6, factor=0.5, b=(b.to(DEV), 0),
                        weight_b=wb.flip(0).contiguous().to(DEV))
    want = 0.5 * (plain.unit_rms(d.sum(0).double(), 1e-6) * wb.double() + plain.unit_rms(b.double(), 1e-6) * wb.flip(0).double())
    assert (y.cpu().double() - want).abs().max() < 1e-5


@pytest.mark.parametrize("H", [96, 1000, 4099])
@pytest.mark.parametrize("two", [False, True])
def test_the_norm_behind_a_sublayer_inside_the_next_norm(H, two):
    """One kernel: the branch (or the mean of two normed branches) through its own layer norm, added to the residual,
    and the residual's next norm; also at selected rows, where the residual stays as it is."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(H + two)
    n = 6
    x, a, b = torch.randn(n, H, generator=g) * 2, torch.randn(2, n, H, generator=g), (torch.randn(n, H, generator=g) * 3).bfloat16()
    wa, wb, wp, w = (torch.randn(H, generator=g) for _ in range(4))
    u = a.sum(0).double()
    if two:
        u = 0.5 * (plain.unit_rms(u, 1e-6) * wa.double() + plain.unit_rms(b.double(), 1e-6) * wb.double())
    r = x.double() + plain.layer_norm(u, wp.double(), 1e-5)
    want = plain.layer_norm(r, w.double(), 1e-5)
    more = dict(gain_a=wa.to(DEV), b=(b.to(DEV), 0), gain_b=wb.to(DEV), inner_eps=1e-6, factor=0.5) if two else {}
    resid, out = x.to(DEV), torch.empty(n, H, device=DEV)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    some = ops.sandwich_norm(resid, (a.to(DEV), 2), torch.empty(2, H, device=DEV), wp.to(DEV), True, 1e-5, w.to(DEV), 0.0, True,
                             1e-5, rows=rows, **more)
    assert torch.equal(resid.cpu(), x) and (some.cpu().double() - want[[4, 1]]).abs().max() < 2e-5
    ops.sandwich_norm(resid, (a.to(DEV), 2), out, wp.to(DEV), True, 1e-5, w.to(DEV), 0.0, True, 1e-5, **more)
    assert (out.cpu().double() - want).abs().max() < 2e-5 and (resid.cpu().double() - r).abs().max() < 1e-5


def paged(dense, page_size, perm):
    """dense [T, heads, d] -> pool [pages, heads, page_size, d] with token t in page perm[t // page_size]."""
    T, heads, d = dense.shape
    pool = torch.full((len(perm), heads, page_size, d), float("nan"), dtype=dense.dtype)
    for t in range(T):
        pool[perm[t // page_size], :, t % page_size] = dense[t]
    return pool


@pytest.mark.parametrize("in_parts", [0, 3])
def test_rotation_with_unit_norm_heads_and_value_heads_of_their_own_size(in_parts):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    n, nq, nkv, hd, vd, rot, ps, eps = 37, 4, 2, 24, 40, 16, 16, 1e-5
    width = (nq + nkv) * hd + nkv * vd
    fused = torch.randn(max(1, in_parts), n, width + 10, generator=g)        # the row is wider than q|k|v: a fused product
    total = fused.sum(0)
    positions = torch.arange(100, 100 + n)
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)])
    perm = [2, 0, 1]
    slots = torch.tensor([perm[t // ps] * ps + t % ps for t in range(n)], dtype=torch.int32)
    k_pages = torch.zeros(3, nkv, ps, hd, device=DEV)
    v_pages = torch.zeros(3, nkv, ps, vd, device=DEV)
    q_out = torch.empty(n, nq * hd, device=DEV)
    src = fused.to(DEV) if in_parts else fused[0].to(DEV)
    ops.rope_kv_write(src[..., :width], q_out, positions.int().to(DEV), slots.to(DEV), inv_freq.to(DEV), k_pages, v_pages,
                      nq, nkv, hd, rot, ps, in_splits=in_parts, vd=vd, unit_norm_eps=eps)
    t64 = total.double()
    q = plain.unit_rms(plain.rotate_half(t64[:, :nq * hd].view(n, nq, hd), positions, rot, 50.0), eps)
    k = plain.unit_rms(plain.rotate_half(t64[:, nq * hd:(nq + nkv) * hd].view(n, nkv, hd), positions, rot, 50.0), eps)
    v = t64[:, (nq + nkv) * hd:width].view(n, nkv, vd)
    assert (q_out.cpu().double().view(n, nq, hd) - q).abs().max() < 2e-5
    got_k = torch.stack([k_pages.cpu()[perm[t // ps], :, t % ps] for t in range(n)])
    got_v = torch.stack([v_pages.cpu()[perm[t // ps], :, t % ps] for t in range(n)])
    assert (got_k.double() - k).abs().max() < 2e-5 and (got_v.double() - v).abs().max() < 1e-6


@pytest.mark.parametrize("hd,vd,rot", [(64, 64, 32), (256, 256, 128), (128, 48, 128), (24, 8, 16), (80, 16, 0)])
def test_rotation_with_unit_norm_heads_over_a_prompt_in_bfloat16(hd, vd, rot):
    """Prompts in bfloat16 take a kernel of their own (16-byte loads, a warp every fourth head); it agrees with the plain
    statement, and a portion of few tokens (the head-a-warp kernel) gives the same rows up to the last bit's rounding."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(hd + vd)
    n, nq, nkv, ps, eps = 300, 5, 2, 16, 1e-6
    width = (nq + nkv) * hd + nkv * vd
    fused = torch.randn(n, width + 8, generator=g).bfloat16()
    positions = torch.arange(7, 7 + n)
    inv_freq = torch.tensor([300.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)])
    pages = -(-n // ps)
    slots = torch.arange(n, dtype=torch.int32)
    outs = []
    for rows in (slice(0, n), slice(0, 40)):
        m = rows.stop
        k_pages = torch.zeros(pages, nkv, ps, hd, dtype=torch.bfloat16, device=DEV)
        v_pages = torch.zeros(pages, nkv, ps, vd, dtype=torch.bfloat16, device=DEV)
        q_out = torch.empty(m, nq * hd, dtype=torch.bfloat16, device=DEV)
        ops.rope_kv_write(fused.to(DEV)[:m, :width], q_out, positions[:m].int().to(DEV), slots[:m].to(DEV), inv_freq.to(DEV), k_pages,
                          v_pages, nq, nkv, hd, rot, ps, vd=vd, unit_norm_eps=eps)
        outs.append((q_out.cpu().float(), k_pages.cpu().float(), v_pages.cpu().float()))
    t64 = fused.double()
    q = plain.unit_rms(plain.rotate_half(t64[:, :nq * hd].view(n, nq, hd), positions, rot, 300.0), eps)
    k = plain.unit_rms(plain.rotate_half(t64[:, nq * hd:(nq + nkv) * hd].view(n, nkv, hd), positions, rot, 300.0), eps)
    v = t64[:, (nq + nkv) * hd:width].view(n, nkv, vd)
    got_q, got_k, got_v = outs[0]
    assert (got_q.double().view(n, nq, hd) - q).abs().max() < 0.03
    pk = got_k.view(pages, nkv, ps, hd).permute(0, 2, 1, 3).reshape(pages * ps, nkv, hd)[:n]
    pv = got_v.view(pages, nkv, ps, vd).permute(0, 2, 1, 3).reshape(pages * ps, nkv, vd)[:n]
    assert (pk.double() - k).abs().max() < 0.03 and torch.equal(pv.double(), v)
    assert (outs[1][0] - got_q[:40]).abs().max() < 0.02          # the two kernels round a head's sum in another order


def sink_attention_plain(q, k, v, sinks, scale, rep):
    """q [Tq, nq, hd] are the last Tq positions of k, v [T, nkv, .]; float64."""
    T, Tq = k.shape[0], q.shape[0]
    out = torch.zeros(Tq, q.shape[1], v.shape[-1], dtype=torch.float64)
    for i in range(Tq):
        last = T - Tq + i
        for h in range(q.shape[1]):
            s = (k[: last + 1, h // rep] @ q[i, h]) * scale
            top = max(float(s.max()), float(sinks[h]))
            e = torch.exp(s - top)
            out[i, h] = (e[:, None] * v[: last + 1, h // rep]).sum(0) / (e.sum() + math.exp(float(sinks[h]) - top))
    return out


def standing_out(T, nq, nkv, hd, vd, seed):
    """Keys and values in which one key far back (position 3, or the first) carries a score well above the rest for every
    query, with a value of its own size: dropping it, or the sink, changes the result by much."""
    g = torch.Generator().manual_seed(seed)
    k, v = torch.randn(T, nkv, hd, generator=g), torch.randn(T, nkv, vd, generator=g)
    far = min(3, T - 1)
    direction = torch.randn(hd, generator=g)
    direction /= direction.norm()
    k[far] = 6.0 * direction
    v[far] = 5.0
    return k, v, direction


@pytest.mark.parametrize("T", [1, 16, 17, 63, 64, 65, 129, 700])
@pytest.mark.parametrize("hd,vd", [(32, 16), (64, 64), (24, 80)])
def test_attention_with_sinks_in_32_bit(T, hd, vd):
    """The three 32-bit kernels (a warp a row, a warp a chunk of a row, tiles of rows) on contexts that end on, just
    before and just behind the edges of pages (16), tiles (32) and chunks (64), with grouped heads."""
    from wllm_b200.kernels import ops
    nq, nkv, ps, scale = 6, 2, 16, 0.3
    k, v, direction = standing_out(T, nq, nkv, hd, vd, seed=T)
    g = torch.Generator().manual_seed(T + 1)
    Tq = min(T, 37)
    q = torch.randn(Tq, nq, hd, generator=g) + 4.0 * direction
    sinks = torch.tensor([-3.0, 0.0, 2.0, 5.0, 9.0, 14.0])
    want = sink_attention_plain(q.double(), k.double(), v.double(), sinks.double(), scale, nq // nkv)
    pages_n = -(-T // ps)
    perm = list(reversed(range(pages_n)))
    kp, vp = paged(k, ps, perm).to(DEV), paged(v, ps, perm).to(DEV)
    table = torch.tensor([[0] * pages_n, perm], dtype=torch.int32, device=DEV)        # the request is row 1 of the table
    qd = q.reshape(Tq, nq * hd).to(DEV)
    positions = torch.arange(T - Tq, T, dtype=torch.int32, device=DEV)
    token_req = torch.ones(Tq, dtype=torch.int32, device=DEV)
    outs = {}
    outs["walk"] = ops.paged_attention_simt(qd, torch.empty(Tq, nq * vd, device=DEV), kp, vp, token_req, positions, table, nq,
                                            nkv, hd, ps, 0, scale, vd=vd, sinks=sinks.to(DEV))
    chunks = ops.simt_chunks(T, 0)
    scratch = torch.empty(Tq * nq * chunks * (vd + 2), device=DEV)
    outs["split"] = ops.paged_attention_simt(qd, torch.empty(Tq, nq * vd, device=DEV), kp, vp, token_req, positions, table,
                                             nq, nkv, hd, ps, 0, scale, scratch, chunks, vd=vd, sinks=sinks.to(DEV))
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    starts, lens, ctxs = z.clone(), z.clone(), z.clone()
    lens[1], ctxs[1] = Tq, T
    outs["tiled"] = ops.paged_attention_simt_tiled(qd, torch.empty(Tq, nq * vd, device=DEV), kp, vp, starts, lens, ctxs, table,
                                                   Tq, nq, nkv, hd, ps, 0, scale, vd=vd, sinks=sinks.to(DEV))
    for name, got in outs.items():
        assert (got.cpu().double().view(Tq, nq, vd) - want).abs().max() < 2e-5, name
        assert torch.equal(got, outs["walk"]), name
    # without the sink the rows come out differently by much: the test would see a sink that is left out
    plain_out = ops.paged_attention_simt(qd, torch.empty(Tq, nq * vd, device=DEV), kp, vp, token_req, positions, table, nq,
                                         nkv, hd, ps, 0, scale, vd=vd)
    assert (plain_out.cpu().double().view(Tq, nq, vd) - want).abs().max() > 0.1


@pytest.mark.parametrize("T", [1, 31, 64, 65, 129, 700, 2100])
@pytest.mark.parametrize("hd", [32, 64, 128])
def test_attention_with_sinks_on_the_tensor_core_kernels(T, hd):
    """bfloat16, keys and values of one size: the decode kernel (its splits and their merge) and the prefill kernels
    take the sink into their last normalisation."""
    from wllm_b200.kernels import ops
    nq, nkv, ps, scale = 4, 2, 16, 0.25
    k, v, direction = standing_out(T, nq, nkv, hd, hd, seed=T)
    k, v = k.bfloat16(), v.bfloat16()
    g = torch.Generator().manual_seed(T + 1)
    sinks = torch.tensor([-3.0, 1.0, 6.0, 12.0])
    pages_n = -(-T // ps)
    perm = list(reversed(range(pages_n)))
    kp, vp = paged(k, ps, perm).to(DEV), paged(v, ps, perm).to(DEV)
    kp, vp = torch.nan_to_num(kp), torch.nan_to_num(vp)
    table = torch.tensor([perm], dtype=torch.int32, device=DEV)
    one = torch.ones(1, dtype=torch.int32, device=DEV)
    for Tq in sorted({1, min(T, 150)}):
        q = (torch.randn(Tq, nq, hd, generator=g) + 3.0 * direction).bfloat16()
        want = sink_attention_plain(q.double(), k.double(), v.double(), sinks.double(), scale, nq // nkv)
        qd, out = q.reshape(Tq, nq * hd).to(DEV), torch.zeros(Tq, nq * hd, dtype=torch.bfloat16, device=DEV)
        starts, lens, ctxs = one * 0, one * Tq, one * T
        if Tq == 1:
            split_keys, max_splits = ops.decode_split_plan(nkv, -(-T // 512) * 512, 32 if hd % 64 == 0 else 64)
            scratch = torch.empty(ops.attention_mma_scratch_floats(1, nq, hd, max_splits), device=DEV)
            ops.attention_mma_decode(qd, out, kp, vp, starts, lens, ctxs, table, nq, nkv, hd, ps, 0, scale, split_keys,
                                     max_splits, scratch, sinks=sinks.to(DEV))
        else:
            ops.attention_mma_prefill(qd, out, kp, vp, starts, lens, ctxs, table, Tq, nq, nkv, hd, ps, 0, scale,
                                      skip_single=False, sinks=sinks.to(DEV))
        torch.cuda.synchronize()
        assert ops.tc_gemm_status(DEV) == 0
        err = (out.cpu().double().view(Tq, nq, hd) - want).abs().max()
        assert err < 0.06, (Tq, float(err))


@pytest.mark.parametrize("per_channel", [True, False])
@pytest.mark.parametrize("H,D,V", [(2, 24, 40), (3, 16, 8), (1, 130, 33), (4, 64, 64), (2, 32, 33), (2, 48, 100), (1, 256, 68)])
def test_the_recurrence_with_its_state_carried_from_call_to_call(per_channel, H, D, V):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(H * D + V)
    lens_by_call = [[5, 1, 40], [1, 1, 3], [17, 2, 1]]       # three requests, three steps
    slots = [2, 0, 3]
    state = torch.zeros(5, H, D, V, device=DEV)
    ref_state = [None, None, None]
    rank, tau, rot = 6, 3.0, (8 if not per_channel else 0)
    W = 2 * H * D + 2 * H * V + (rank if per_channel else 0) + 5
    w2, b2 = torch.randn(H * D, rank, generator=g), torch.rand(H * D, generator=g) * 6 - 2
    head_decay = torch.tensor([0.7, 0.9, 0.99, 1.0][:H])
    norm_w = torch.randn(V, generator=g)
    inv_freq = torch.tensor([100.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)])
    pos0 = [0, 0, 0]
    for lens in lens_by_call:
        n = sum(lens)
        fused = torch.randn(2, n, W, generator=g)
        total = fused.sum(0).double()
        positions = torch.cat([torch.arange(p, p + m) for p, m in zip(pos0, lens)])
        bufs = [torch.empty(n, H * D, device=DEV), torch.empty(n, H * D, device=DEV), torch.empty(n, H * V, device=DEV)]
        decay = torch.empty(n, H * D, device=DEV) if per_channel else None
        ops.linattn_prepare(fused.to(DEV)[..., 3:], 2, 0, H * D, 2 * H * D, H, D, V, positions.int().to(DEV), *bufs,
                            q_scale=0.5, k_scale=2.0, inv_freq=inv_freq.to(DEV) if rot else None, rot_dim=rot,
                            low_off=2 * H * D + 2 * H * V if per_channel else -1, w2=w2.to(DEV) if per_channel else None,
                            b2=b2.to(DEV) if per_channel else None, tau=tau, decay=decay)
        o = torch.empty(n, H * V, device=DEV)
        starts = torch.tensor([sum(lens[:i]) for i in range(3)], dtype=torch.int32, device=DEV)
        ops.linattn_scan(bufs[0], bufs[1], bufs[2], decay, None if per_channel else head_decay.to(DEV), state, o, starts,
                         torch.tensor(lens, dtype=torch.int32, device=DEV), torch.tensor(slots, dtype=torch.int32, device=DEV),
                         H, D, V)
        gated = torch.empty(n, H * V, device=DEV)
        ops.head_gate_norm(o, fused.to(DEV)[..., 3:], 2, 2 * H * D + H * V, norm_w.to(DEV) if per_channel else None, 1e-5,
                           gated, H, V)
        total = total[:, 3:]
        for i, m in enumerate(lens):
            rows = slice(int(starts[i]), int(starts[i]) + m)
            p = positions[rows]
            q = plain.rotate_half(total[rows, :H * D].view(m, H, D), p, rot, 100.0) * 0.5
            k = plain.rotate_half(total[rows, H * D:2 * H * D].view(m, H, D), p, rot, 100.0) * 2.0
            v = total[rows, 2 * H * D:2 * H * D + H * V].view(m, H, V)
            if per_channel:
                z = total[rows, 2 * H * D + 2 * H * V:2 * H * D + 2 * H * V + rank] @ w2.double().T + b2.double()
                a = (torch.sigmoid(z) ** (1.0 / tau)).view(m, H, D)
            else:
                a = head_decay.double()[None, :, None].expand(m, H, D)
            want_o, ref_state[i] = plain.decayed_outer_scan(q, k, v, a, ref_state[i])
            assert (o.cpu().double()[rows].view(m, H, V) - want_o).abs().max() < 1e-4 * max(1.0, float(want_o.abs().max()))
            gate = total[rows, 2 * H * D + H * V:2 * H * D + 2 * H * V].view(m, H, V)
            want_g = plain.unit_rms(want_o, 1e-5) * (norm_w.double() if per_channel else 1.0) * plain.silu(gate)
            assert (gated.cpu().double()[rows].view(m, H, V) - want_g).abs().max() < 2e-4
            assert (state[slots[i]].cpu().double() - ref_state[i]).abs().max() < 1e-4 * max(1.0, float(ref_state[i].abs().max()))
            pos0[i] += m
    assert float(state[1].abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0       # slots of nobody stay untouched


def test_segments_give_the_walk_up_to_rounding():
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    H, D, V, lens = 2, 40, 72, [100, 1, 33, 64]
    n = sum(lens)
    q, k, v = (torch.randn(n, H * x, generator=g).to(DEV) for x in (D, D, V))
    decay = (torch.rand(n, H * D, generator=g) * 0.5 + 0.5).to(DEV)
    starts = torch.tensor([sum(lens[:i]) for i in range(4)], dtype=torch.int32, device=DEV)
    ql, slots = torch.tensor(lens, dtype=torch.int32, device=DEV), torch.tensor([1, 3, 0, 2], dtype=torch.int32, device=DEV)
    start_state = torch.randn(4, H, D, V, generator=g).to(DEV)
    results = []
    for seg_len in (0, 8, 32, 48):
        state, o = start_state.clone(), torch.empty(n, H * V, device=DEV)
        max_seg = -(-max(lens) // seg_len) if seg_len else 1
        ops.linattn_scan(q, k, v, decay, None, state, o, starts, ql, slots, H, D, V, seg_len, max_seg,
                         torch.empty(4 * max_seg * H * D * V, device=DEV), torch.empty(4 * max_seg * H * D, device=DEV))
        results.append((o, state))
    for o, state in results[1:]:
        assert (o - results[0][0]).abs().max() < 2e-4 and (state - results[0][1]).abs().max() < 2e-4
