"""Taritar on the device against its plain statement (tests/plain_taritar.py, float64, whole sequences).

Whole models: every way of cutting the work (whole prompts, a tail decoded token by token, portions down to two tokens
and one, mixed batches whose pages and slots are used again), bit for bit against one another in 32-bit; long decoding
past every window; decoding from captured graphs; greedy generation through the scheduler.  Mechanisms alone: the
streams' update and norm, the embedding with position rows, the clamped gated unit and the tanh cap, attention with a
score cap and kept first keys (one key made to stand out just inside and just outside every edge, pages in scrambled
order, all three kernels), the router's choice by groups, the experts' grouped products.
"""
import math

import pytest
import torch

import plain_taritar as plain
import traces
from helpers import folder_weights, max_diff
from taritar_configs import CONFIGS, write_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runner_for(folder, dtype, page_size, pages, slots=4, poison=True):
    from wllm_b200.config import EngineConfig
    from wllm_b200.engine import build_model, build_runner
    eng = EngineConfig(dtype=dtype, block_size=page_size, max_num_seqs=slots)
    return build_runner(build_model(folder, eng.dtype, eng.device), eng, num_pages=pages, poison_pages=poison)


def plain_rows(folder, name, reqs):
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    return {(rid, p): row.float() for rid, toks in reqs.items() for p, row in enumerate(plain.forward(CONFIGS[name], w, toks))}


def close_enough(rows, ref, dtype, what=""):
    """32-bit: every logit within 2e-4 of the logits' scale.  bfloat16: by rows.  The router sees the norm's output rounded
    to bfloat16, and with random weights some token's two best experts (or groups) lie closer together than that rounding,
    so its choice, and with it the whole row, may differ from the plain statement's in any implementation: the typical
    row must be within 1.5 % of the rows' scale (observed 0.5 %), nine in ten within 4 %."""
    assert set(rows) == set(ref)
    scale = max(1.0, max(float(r.abs().max()) for r in ref.values()))
    if dtype == torch.float32:
        assert max_diff(rows, ref) < 2e-4 * scale, what
        return
    rms = math.sqrt(sum(float(r.double().pow(2).mean()) for r in ref.values()) / len(ref))
    rel = sorted(float((rows[k].double() - ref[k].double()).pow(2).mean().sqrt()) / rms for k in ref)
    assert rel[len(rel) // 2] < 0.015 and rel[int(len(rel) * 0.9)] < 0.04, (what, rel[len(rel) // 2], rel[int(len(rel) * 0.9)], rel[-1])


def requests_of(name, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in CONFIGS:
        folder = write_folder(str(tmp_path_factory.mktemp("taritar") / name), name)
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
        if cut == "mixed":      # pages and slots were used again
            assert all(g.pool.takes > pages for g in runner.cache.groups if g.spec.window is None) and len(reqs) > 4
        if dtype == torch.float32:
            if first is None:
                first = rows
            else:
                bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                assert not bad, f"{cut}: first differing (request, position) {bad[0]}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["wide", "one"])
def test_long_decoding_passes_every_window_and_gives_pages_back(setups, name, dtype):
    folder = setups[name][0]
    reqs = requests_of(name, (230,), seed=8)
    ref = plain_rows(folder, name, reqs)
    steps = traces.tail_singly(reqs, 200)
    runner = runner_for(folder, dtype, 16, 15)          # 15 pages hold 240 tokens
    held = []
    rows = {}
    from wllm_b200.engine import StepEntry
    rc = runner.cache.open("r0")
    pos = 0
    for s in steps:
        e = s["entries"][0]
        logits = runner.step([StepEntry(rc, e["tokens"], e["want"])]).float().cpu()
        for w, row in zip(e["want"], logits):
            rows[("r0", pos + w)] = row
        pos += len(e["tokens"])
        held.append([sum(1 for p in t if p >= 0) for t in rc.tables])
    close_enough(rows, ref, dtype)
    for g, spec in enumerate(runner.model.group_specs):
        if spec.window is not None:      # a window group holds the window's pages and those of the kept first keys, no more
            most = -(-spec.window // 16) + 1 + -(-spec.keep_first // 16)
            assert held[-1][g] <= most < 15, (spec, held[-1])
    runner.cache.close(rc)


def test_long_portions_behind_released_pages_on_the_tensor_memory_attention(setups):
    """Heads of 128 elements: a portion of more than 64 tokens runs on pairs of CTAs (tcgen05).  The second portion comes when
    the window has passed pages that were given back (and hold NaN): it walks the kept keys' tile, then the window's."""
    from wllm_b200.engine import StepEntry
    folder = setups["heads128"][0]
    reqs = requests_of("heads128", (260,), seed=12)
    ref = plain_rows(folder, "heads128", reqs)
    runner = runner_for(folder, torch.bfloat16, 16, 17)
    rc = runner.cache.open("r0")
    rows, pos = {}, 0
    for n in (100, 130, 1, 29):
        toks = reqs["r0"][pos:pos + n]
        logits = runner.step([StepEntry(rc, toks, list(range(n)))]).float().cpu()
        rows.update({("r0", pos + i): row for i, row in enumerate(logits)})
        pos += n
        if pos == 100:
            assert rc.tables[0][0] >= 0 and rc.tables[0][1] >= 0 and rc.tables[0][2] == -1     # kept keys stay, the window passed a page
    close_enough(rows, ref, torch.bfloat16)
    from wllm_b200.kernels import ops
    assert ops.tc_gemm_status(DEV) == 0


def test_decoding_from_captured_graphs_gives_the_eager_rows(setups):
    folder, reqs, ref = setups["wide"]
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


def test_greedy_generation_through_the_scheduler(setups):
    from wllm_b200 import LLM, SamplingParams
    folder, reqs, _ = setups["wide"]
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    prompts = [reqs["r0"], reqs["r2"], reqs["r3"][:40], reqs["r8"]]
    llm = LLM(folder, dtype="float32", block_size=16, num_blocks=12, chunked_prefill_tokens=24, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        for _ in range(10):
            toks.append(int(plain.forward(CONFIGS["wide"], w, toks)[-1].argmax()))
        assert o.token_ids == toks[len(prompt):]
    assert llm.runner.cache.slots.num_free == 3 and all(f == 12 for f in llm.runner.cache.free_pages())
    bf = LLM(folder, dtype="bfloat16", block_size=16, num_blocks=12, chunked_prefill_tokens=24, max_num_seqs=3, cuda_graphs=True)
    assert [len(o.token_ids) for o in bf.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))] == [10] * 4


def test_a_sequence_longer_than_the_position_table_is_refused(setups):
    from wllm_b200.engine import StepEntry
    folder = setups["plain"][0]
    runner = runner_for(folder, torch.float32, 16, 20)
    rc = runner.cache.open("x")
    with pytest.raises(ValueError, match="positions"):
        runner.step([StepEntry(rc, [1] * (CONFIGS["plain"]["max_positions"] + 1), [0])])


# ------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("H", [40, 256, 1000, 4100])
def test_streams_update_and_norm(S, H):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(S * 1000 + H)
    n, eps = 5, 1e-5
    x = torch.randn(S, n, H, generator=g) * 2
    y = torch.randn(3, n, H, generator=g)
    mix, w_out, w_in = torch.eye(S) + 0.4 * torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    gain = 1 + 0.3 * torch.randn(H, generator=g)
    new = torch.einsum("st,snw->tnw", mix.double(), x.double()) + w_out.double()[:, None, None] * y.sum(0).double()[None]
    want = plain.rms_norm(torch.einsum("s,snw->nw", w_in.double(), new), gain.double(), eps)
    streams, out = x.to(DEV), torch.empty(n, H, device=DEV)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    some = ops.hyper_norm(streams, streams, S, (y.to(DEV), 3), mix.to(DEV), w_out.to(DEV), w_in.to(DEV), gain.to(DEV), eps,
                          torch.empty(2, H, device=DEV), rows)
    assert torch.equal(streams.cpu(), x)                                  # at selected rows the streams stay as they are
    ops.hyper_norm(streams, streams, S, (y.to(DEV), 3), mix.to(DEV), w_out.to(DEV), w_in.to(DEV), gain.to(DEV), eps, out)
    tol = 2e-5 * float(want.abs().max())
    assert (out.cpu().double() - want).abs().max() < tol and (streams.cpu().double() - new).abs().max() < 1e-5
    assert torch.equal(some.cpu(), out.cpu()[[4, 1]])
    # one pending tensor in bfloat16, bfloat16 out; then the plain sum of the streams without anything pending
    yb = y[0].bfloat16()
    s2, ob = x.to(DEV), torch.empty(n, H, dtype=torch.bfloat16, device=DEV)
    ops.hyper_norm(s2, s2, S, (yb.to(DEV), 0), mix.to(DEV), w_out.to(DEV), w_in.to(DEV), gain.to(DEV), eps, ob)
    new2 = torch.einsum("st,snw->tnw", mix.double(), x.double()) + w_out.double()[:, None, None] * yb.double()[None]
    want2 = plain.rms_norm(torch.einsum("s,snw->nw", w_in.double(), new2), gain.double(), eps)
    assert (ob.cpu().double() - want2).abs().max() < 0.01 * float(want2.abs().max())
    total = ops.hyper_norm(s2, s2, S, None, None, None, None, gain.to(DEV), eps, torch.empty(n, H, device=DEV))
    assert (total.cpu().double() - plain.rms_norm(new2.sum(0), gain.double(), eps)).abs().max() < 1e-4 * float(want2.abs().max()) + 1e-4
    # the first norm of a model: every stream starts as the same rows
    e = torch.randn(n, H, generator=g)
    spread = torch.full((S, n, H), float("nan"), device=DEV)
    first = ops.hyper_norm(e.to(DEV), spread, S, None, None, None, w_in.to(DEV), gain.to(DEV), eps, torch.empty(n, H, device=DEV))
    assert torch.equal(spread.cpu(), e[None].expand(S, n, H))
    assert (first.cpu().double() - plain.rms_norm(w_in.double().sum() * e.double(), gain.double(), eps)).abs().max() < 1e-4


def test_embedding_adds_the_position_row_unscaled():
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    table, pos = torch.randn(30, 72, generator=g).bfloat16(), torch.randn(50, 72, generator=g).bfloat16()
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    at = torch.tensor([0, 49, 7, 8], dtype=torch.int32)
    out = ops.embed_gather(ids.to(DEV), table.to(DEV), 0.37, torch.empty(4, 72, device=DEV), pos.to(DEV), at.to(DEV))
    want = table.double()[ids.long()] * 0.37 + pos.double()[at.long()]
    assert (out.cpu().double() - want).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gated_unit_and_tanh_cap(dtype):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(9, 2 * 40, generator=g) * 3).to(dtype)
    limit, slope = 1.3, 1.702
    out = ops.gated_act(gu.to(DEV), torch.empty(9, 40, dtype=dtype, device=DEV), "capped_swish", limit, slope)
    a, b = gu.double()[:, :40].clamp(max=limit), gu.double()[:, 40:].clamp(-limit, limit)
    want = a * torch.sigmoid(slope * a) * (b + 1)
    assert (out.cpu().double() - want).abs().max() < (1e-6 if dtype == torch.float32 else 0.02)
    assert float(want.min()) < -0.2 and float((gu.double()[:, :40] > limit).float().mean()) > 0.1      # both clamps bite
    x = torch.randn(7, 33, generator=g) * 40
    capped = ops.tanh_cap(x.to(DEV).clone(), 11.0)
    assert (capped.cpu().double() - 11.0 * torch.tanh(x.double() / 11.0)).abs().max() < 1e-5


def paged(keys, values, page_size, order_seed):
    """Keys [L, G, d] and values [L, G, dv] of one sequence on pages in scrambled order: pools and the block table."""
    L, G, d = keys.shape
    pages = -(-L // page_size)
    perm = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(order_seed))[:pages]
    kp = torch.full((pages + 3, G, page_size, d), float("nan"), dtype=keys.dtype)
    vp = torch.full((pages + 3, G, page_size, values.shape[-1]), float("nan"), dtype=keys.dtype)
    for j in range(L):
        kp[perm[j // page_size], :, j % page_size] = keys[j]
        vp[perm[j // page_size], :, j % page_size] = values[j]
    return kp.to(DEV), vp.to(DEV), perm.to(torch.int32)[None].contiguous().to(DEV)


def plain_attention_rows(q, k, v, positions, scale, cap, size, keep):
    """q [n, H, d] at `positions` over keys k [L, G, d], values v: the plain statement's scores, mask and softmax."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for r, p in enumerate(positions):
        j = torch.arange(k.shape[0])
        seen = (j <= p) & ((p - j < size) | (j < keep)) if size else (j <= p)
        heads = []
        for a in range(H):
            s = (k[:, a // (H // G)].double() @ q[r, a].double()) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~seen, float("-inf"))
            heads.append(torch.softmax(s, 0) @ v[:, a // (H // G)].double())
        out.append(torch.cat(heads))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("size,keep,cap", [(40, 5, 6.0), (90, 33, 0.0), (16, 16, 18.0), (8, 70, 4.0), (64, 0, 2.5), (130, 1, 0.0)])
def test_attention_with_a_cap_and_kept_first_keys_at_every_edge(size, keep, cap, dtype):
    """One key at a time is made to stand out (a key along the query, long enough to take all the weight when it is seen)
    just inside and just outside the window and the kept keys, for rows in a prompt's portion and for a single decoded
    row, on pages in scrambled order, through all three kernels, whose results are one, bit for bit."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(size * 7 + keep)
    H, G, d, dv, ps, L = 4, 2, 16, 24, 16, 300
    scale = 0.4
    k = torch.randn(L, G, d, generator=g).to(dtype)
    v = torch.randn(L, G, dv, generator=g).to(dtype)
    kp, vp, table = paged(k.float().to(dtype), v, ps, 5)
    n0 = 236                                          # the rows: positions n0 .. L-1, one portion of a prompt
    positions = list(range(n0, L))
    q = torch.randn(len(positions), H, d, generator=g).to(dtype)
    edges = sorted({e for e in (keep - 1, keep, keep + 1, 0, n0 - size, n0 - size + 1, L - 1 - size, L - size, L - 1 - size + 1, 63, 64, 31, 32)
                    if 0 <= e < L})
    for edge in edges:
        k2 = k.clone()
        k2[edge] = (q[0, 0::2] * 6).to(dtype)         # along the queries of row n0 (heads 0 and 2: one per key/value head)
        kp2, _, _ = paged(k2, v, ps, 5)
        want = plain_attention_rows(q, k2, v, positions, scale, cap, size, keep)
        pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
        req = torch.zeros(len(positions), dtype=torch.int32, device=DEV)
        qd = q.reshape(len(positions), H * d).to(DEV)
        outs = []
        for kind in ("walk", "split", "tiled"):
            out = torch.empty(len(positions), H * dv, dtype=dtype, device=DEV)
            if kind == "tiled":
                one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
                ops.paged_attention_simt_tiled(qd, out, kp2, vp, one(0), one(len(positions)), one(L), table, len(positions), H, G, d,
                                               ps, size, scale, vd=dv, cap=cap, keep=keep)
            else:
                chunks = ops.simt_chunks(L, size, keep)
                scratch = torch.empty(len(positions) * H * chunks * (dv + 2), device=DEV) if kind == "split" else None
                ops.paged_attention_simt(qd, out, kp2, vp, req, pos_t, table, H, G, d, ps, size, scale, scratch, chunks, vd=dv,
                                         cap=cap, keep=keep)
            outs.append(out.cpu())
            err = (out.cpu().double() - want).abs().max()
            assert err < (2e-5 if dtype == torch.float32 else 0.03), (kind, edge, float(err))
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), edge
        # the last row alone, as a decoded token
        last = torch.empty(1, H * dv, dtype=dtype, device=DEV)
        ops.paged_attention_simt(qd[-1:], last, kp2, vp, req[:1], pos_t[-1:], table, H, G, d, ps, size, scale, vd=dv, cap=cap, keep=keep)
        assert torch.equal(last.cpu(), outs[0][-1:])
    # the standing-out key changes the first row's output when and only when the mask lets it be seen
    base = plain_attention_rows(q[:1], k, v, positions[:1], scale, cap, size, keep)
    for edge in (n0 - size, n0 - size + 1):
        if edge < 0 or edge < keep:
            continue
        k2 = k.clone()
        k2[edge] = (q[0, 0::2] * 6).to(dtype)
        moved = (plain_attention_rows(q[:1], k2, v, positions[:1], scale, cap, size, keep) - base).abs().max()
        assert (moved > 0.05) == (edge == n0 - size + 1)


@pytest.mark.parametrize("E,top,groups,kept", [(8, 2, 4, 2), (15, 4, 5, 3), (6, 3, 2, 1), (5, 1, 1, 1), (64, 6, 8, 3), (7, 7, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_router_chooses_by_groups(E, top, groups, kept, dtype):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    n, H = 37, 72
    x = torch.randn(n, H, generator=g).to(dtype)
    wr, wg = torch.randn(E, H, generator=g).bfloat16().float() * 0.5, torch.randn(H, generator=g).bfloat16().float() * 0.3
    chosen = torch.empty(n, top, dtype=torch.int32, device=DEV)
    weights, gate = torch.empty(n, top, device=DEV), torch.empty(n, device=DEV)
    ops.moe_route(x.to(DEV), wr.to(DEV), wg.to(DEV), chosen, weights, gate, groups, kept)
    scores = torch.softmax(x.double() @ wr.double().T, -1)
    want = plain.route(scores, top, groups, kept)
    assert torch.equal(chosen.cpu().long(), want)
    assert (weights.cpu().double() - scores.gather(1, want)).abs().max() < 1e-6
    assert (gate.cpu().double() - torch.sigmoid(x.double() @ wg.double())).abs().max() < 1e-6
    if kept < groups and top > kept:       # the limit bites: somewhere an expert of a dropped group would have been among the best
        assert not torch.equal(want.sort(1).values, scores.topk(top, -1).indices.sort(1).values)
    # the pairs sorted by expert, stably
    count, offset = torch.empty(E, dtype=torch.int32, device=DEV), torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order, place = torch.empty(n * top, dtype=torch.int32, device=DEV), torch.empty(n * top, dtype=torch.int32, device=DEV)
    ops.moe_plan(chosen, count, offset, order, place)
    flat = want.reshape(-1)
    stable = torch.sort(flat, stable=True).indices
    assert torch.equal(order.cpu().long(), stable) and torch.equal(place.cpu().long()[stable], torch.arange(n * top))
    assert torch.equal(count.cpu().long(), torch.bincount(flat, minlength=E)) and int(offset[-1]) == n * top


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,top,H,I", [(1, 5, 1, 40, 8), (50, 6, 3, 72, 24), (200, 4, 2, 64, 100)])
def test_experts_as_grouped_products(n, E, top, H, I, dtype):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(n + E)
    x = torch.randn(n, H, generator=g).to(dtype)
    w = {f"e{j}.{k}": (torch.randn(s, generator=g) * 0.2).to(dtype).double()
         for j in range(E) for k, s in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
    chosen = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    weights = torch.rand(n, top, generator=g)
    shared, gate = torch.randn(2, n, H, generator=g), torch.rand(n, generator=g)
    limit, slope = 0.9, 1.702
    want = torch.zeros(n, H, dtype=torch.float64)
    for t in range(n):
        for k in range(top):
            want[t] += weights[t, k].double() * plain.capped_glu(w, f"e{int(chosen[t, k])}.", x[t:t + 1].double(), limit)[0]
    want += gate.double()[:, None] * shared.sum(0).double()
    w_gu = torch.stack([torch.cat([w[f"e{j}.gate"], w[f"e{j}.up"]]) for j in range(E)]).to(dtype).to(DEV)
    w_d = torch.stack([w[f"e{j}.down"] for j in range(E)]).to(dtype).to(DEV)
    count, offset = torch.empty(E, dtype=torch.int32, device=DEV), torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order, place = torch.empty(n * top, dtype=torch.int32, device=DEV), torch.empty(n * top, dtype=torch.int32, device=DEV)
    ops.moe_plan(chosen.to(DEV), count, offset, order, place)
    act = ops.moe_grouped(x.to(DEV), w_gu, torch.empty(n * top, I, dtype=dtype, device=DEV), offset, order, top, True, limit, slope)
    y = ops.moe_grouped(act, w_d, torch.empty(n * top, H, device=DEV), offset, order, top, False)
    out = ops.moe_combine(y, place, weights.to(DEV), (shared.to(DEV), 2), gate.to(DEV), torch.empty(n, H, device=DEV))
    assert (out.cpu().double() - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.03)
    # a token's output does not depend on what else is in the batch: the first rows alone give the same bits
    m = min(n, 3)
    ops.moe_plan(chosen[:m].contiguous().to(DEV), count, offset, order[:m * top], place[:m * top])
    act = ops.moe_grouped(x[:m].to(DEV), w_gu, torch.empty(m * top, I, dtype=dtype, device=DEV), offset, order[:m * top], top, True, limit, slope)
    y = ops.moe_grouped(act, w_d, torch.empty(m * top, H, device=DEV), offset, order[:m * top], top, False)
    few = ops.moe_combine(y, place[:m * top], weights[:m].contiguous().to(DEV), (shared[:, :m].contiguous().to(DEV), 2),
                          gate[:m].contiguous().to(DEV), torch.empty(m, H, device=DEV))
    assert torch.equal(few.cpu(), out.cpu()[:m])


@pytest.mark.parametrize("hd,n0", [(32, 236), (48, 236), (64, 236), (64, 150), (128, 236), (128, 90)])
@pytest.mark.parametrize("size,keep,cap", [(40, 5, 6.0), (90, 33, 0.0), (16, 16, 18.0), (8, 70, 4.0), (64, 0, 2.5), (130, 1, 0.0), (100, 64, 3.0)])
def test_tensor_core_attention_with_a_cap_and_kept_first_keys(size, keep, cap, hd, n0):
    """The bfloat16 kernels (mma.sync and tcgen05) that walk a list of key tiles (the kept keys' tiles, then the window's): a
    prompt's portion and decoded rows, with one key standing out at every edge, pages in scrambled order, page sizes 16 and 64, keys
    cut into several splits."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(size * 7 + keep + hd)
    H, G, L, dtype = 4, 2, 300, torch.bfloat16
    scale = 0.4 * (16 / hd) ** 0.5
    k = torch.randn(L, G, hd, generator=g).to(dtype)
    v = torch.randn(L, G, hd, generator=g).to(dtype)
    # head sizes 32 and 48: mma.sync; 64 and 128: the tensor-memory kernel of one CTA a tile of 128 rows (n0 = 236: one tile, 150:
    # three); 128 with more than 128 rows (n0 = 90): pairs of CTAs
    positions = list(range(n0, L))
    q = torch.randn(len(positions), H, hd, generator=g).to(dtype)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    edges = sorted({e for e in (keep - 1, keep, 0, n0 - size, n0 - size + 1, L - 1 - size, L - size, 63, 64, 127, 128) if 0 <= e < L})
    for ps in (16, 64):
        for edge in edges:
            k2 = k.clone()
            k2[edge] = (q[0, 0::2] * 6).to(dtype)
            kp, vp, table = paged(k2, v, ps, 5 + ps)
            want = plain_attention_rows(q, k2, v, positions, scale, cap, size, keep)
            qd = q.reshape(len(positions), H * hd).to(DEV)
            out = torch.empty(len(positions), H * hd, dtype=dtype, device=DEV)
            ops.attention_mma_prefill(qd, out, kp, vp, one(0), one(len(positions)), one(L), table, len(positions), H, G, hd, ps, size,
                                      scale, skip_single=False, cap=cap, keep=keep)
            err = (out.cpu().double() - want).abs().max()
            assert err < 0.03, ("prefill", ps, edge, float(err))
            # the last three rows as decoded tokens of three requests of different lengths on the same pages
            R = 3
            tables = table.expand(R, -1).contiguous()
            starts = torch.arange(R, dtype=torch.int32, device=DEV)
            lens = torch.ones(R, dtype=torch.int32, device=DEV)
            ctxs = torch.tensor([L - 2, L - 1, L], dtype=torch.int32, device=DEV)
            for split_keys, max_splits in ((512, 1), (128, 3), (64, 5)):
                scratch = torch.empty(ops.attention_mma_scratch_floats(R, H, hd, max_splits), device=DEV)
                od = torch.empty(R, H * hd, dtype=dtype, device=DEV)
                ops.attention_mma_decode(qd[-3:].contiguous(), od, kp, vp, starts, lens, ctxs, tables, H, G, hd, ps, size, scale,
                                         split_keys, max_splits, scratch, cap=cap, keep=keep)
                err = (od.cpu().double() - want[-3:]).abs().max()
                assert err < 0.03, ("decode", ps, edge, split_keys, float(err))
    assert ops.tc_gemm_status(DEV) == 0


@pytest.mark.parametrize("M", [3, 70, 300])
def test_the_clamped_unit_in_the_products_epilogue(M):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(M)
    K, I, limit, slope = 96, 160, 0.7, 1.702
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, generator=g) * 0.15).bfloat16()
    out = ops.gated_linear(a.to(DEV), w.to(DEV), "capped_swish", torch.empty(M, I, dtype=torch.bfloat16, device=DEV),
                           lambda shape, dtype: torch.empty(shape, dtype=dtype, device=DEV), limit, slope)
    gate, up = (a.double() @ w.double()[:I].T).clamp(max=limit), (a.double() @ w.double()[I:].T).clamp(-limit, limit)
    want = gate * torch.sigmoid(slope * gate) * (up + 1)
    assert (out.cpu().double() - want).abs().max() < 0.02 and float((a.double() @ w.double()[:I].T > limit).float().mean()) > 0.1
    assert ops.tc_gemm_status(DEV) == 0


@pytest.mark.parametrize("hd,rot", [(80, 80), (128, 64), (32, 16)])
def test_interleaved_rotation_of_many_rows_is_that_of_few(hd, rot):
    """A prompt of many bfloat16 rows takes a kernel of its own (a CTA a token, 16-byte loads); its bits are those of the
    kernel that serves few rows, and both match the plain rotation of the pairs (2i, 2i + 1)."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(hd)
    n, nq, nkv, ps = 300, 3, 2, 16
    qkv = torch.randn(n, (nq + 2 * nkv) * hd, generator=g).bfloat16()
    pos = torch.randint(0, 5000, (n,), generator=g).to(torch.int32)
    slots = torch.randperm(20 * ps, generator=g)[:n].to(torch.int32)
    inv = (500.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float()
    outs = []
    for pieces in (1, 3):
        q = torch.zeros(n, nq * hd, dtype=torch.bfloat16, device=DEV)
        kp, vp = (torch.zeros(20, nkv, ps, hd, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        step = n // pieces
        for i in range(0, n, step):
            ops.rope_kv_write(qkv[i:i + step].to(DEV), q[i:i + step], pos[i:i + step].to(DEV), slots[i:i + step].to(DEV), inv.to(DEV),
                              kp, vp, nq, nkv, hd, rot, ps, pairing="interleaved")
        outs.append((q.cpu(), kp.cpu(), vp.cpu()))
    assert all(torch.equal(a, b) for a, b in zip(*outs))
    want = plain.rotate_interleaved(qkv[:, :nq * hd].double().view(n, nq, hd), pos.long(), rot, 500.0).reshape(n, -1)
    assert (outs[0][0].double() - want).abs().max() < 0.03
    krow = outs[0][1][slots[7] // ps, 1, slots[7] % ps].double()
    kwant = plain.rotate_interleaved(qkv[7:8, (nq + 1) * hd:(nq + 2) * hd].double().view(1, 1, hd), pos[7:8].long(), rot, 500.0).reshape(-1)
    assert (krow - kwant).abs().max() < 0.03
    assert torch.equal(outs[0][2][slots[7] // ps, 0, slots[7] % ps], qkv[7, (nq + nkv) * hd:(nq + nkv + 1) * hd])
    # queries alone, as a layer rotates them that reads another layer's keys and values
    q2 = torch.zeros(n, nq * hd, dtype=torch.bfloat16, device=DEV)
    ops.rope_kv_write(qkv[:, :nq * hd].contiguous().to(DEV), q2, pos.to(DEV), None, inv.to(DEV), None, None, nq, 0, hd, rot, ps,
                      pairing="interleaved")
    assert torch.equal(q2.cpu(), outs[0][0])


@pytest.mark.parametrize("n,E,top,H,I", [(300, 6, 4, 72, 24), (700, 5, 4, 64, 104), (130, 40, 8, 128, 264)])
def test_experts_on_the_tensor_memory_product(n, E, top, H, I):
    """Many rows: the tokens' rows copied into sorted order, row tiles of 128 rows of one expert each from the table that the
    plan leaves on the device (experts with no row, with a few and with more than a tile), both products on tcgen05."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(n + E)
    dtype = torch.bfloat16
    x = torch.randn(n, H, generator=g).to(dtype)
    w = {f"e{j}.{k}": (torch.randn(s, generator=g) * 0.2).to(dtype).double()
         for j in range(E) for k, s in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
    usable = E - 1                      # the last expert gets no row
    chosen = torch.stack([torch.randperm(usable, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    chosen[: n // 2, 0] = 0             # one expert with more than a tile of rows
    for t in range(n // 2):             # (no expert twice for a token)
        for k in range(1, top):
            if chosen[t, k] == 0:
                chosen[t, k] = usable - 1 if (usable - 1) not in chosen[t].tolist() else [e for e in range(usable) if e not in chosen[t].tolist()][0]
    weights = torch.rand(n, top, generator=g)
    limit, slope = 0.9, 1.702
    want = torch.zeros(n, H, dtype=torch.float64)
    for t in range(n):
        for k in range(top):
            want[t] += weights[t, k].double() * plain.capped_glu(w, f"e{int(chosen[t, k])}.", x[t:t + 1].double(), limit)[0]
    w_gu = torch.stack([torch.cat([w[f"e{j}.gate"], w[f"e{j}.up"]]) for j in range(E)]).to(dtype).to(DEV)
    w_d = torch.stack([w[f"e{j}.down"] for j in range(E)]).to(dtype).to(DEV)
    pairs = n * top
    count, offset = torch.empty(E, dtype=torch.int32, device=DEV), torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order, place = torch.empty(pairs, dtype=torch.int32, device=DEV), torch.empty(pairs, dtype=torch.int32, device=DEV)
    tiles = torch.full((1 + 3 * ops.moe_row_tiles(pairs, E),), -7, dtype=torch.int32, device=DEV)
    ops.moe_plan(chosen.to(DEV), count, offset, order, place)
    one_warp = [t.clone() for t in (count, offset, order, place)]
    scratch = torch.empty(ops.MOE_PLAN_SEGMENTS * E, dtype=torch.int32, device=DEV) if n == 700 else None     # 2,800 pairs: in segments
    ops.moe_plan(chosen.to(DEV), count, offset, order, place, tiles, scratch)
    assert all(torch.equal(a, b) for a, b in zip(one_warp, (count, offset, order, place)))
    table = tiles.cpu().tolist()
    counts = torch.bincount(chosen.reshape(-1).long(), minlength=E).tolist()
    assert table[0] == sum(-(-c // 128) for c in counts) and counts[-1] == 0 and (max(counts) > 128) == (n >= 300)
    seen = []
    for i in range(table[0]):
        e, row0, rows = table[1 + 3 * i: 4 + 3 * i]
        seen.extend(range(row0, row0 + rows))
        assert 0 < rows <= 128 and int(offset[e]) <= row0 and row0 + rows <= int(offset[e + 1])
    assert seen == list(range(pairs))
    rows = ops.moe_gather(x.to(DEV), order, top, torch.empty(pairs, H, dtype=dtype, device=DEV))
    assert torch.equal(rows.cpu(), x[(order.cpu().long() // top)])
    act = ops.gemm_bf16_tc_grouped(rows, w_gu, torch.empty(pairs, I, dtype=dtype, device=DEV), tiles, True, limit, slope)
    y = ops.gemm_bf16_tc_grouped(act, w_d, torch.empty(pairs, H, device=DEV), tiles, False)
    out = ops.moe_combine(y, place, weights.to(DEV), None, None, torch.empty(n, H, device=DEV))
    assert ops.tc_gemm_status(DEV) == 0
    assert (out.cpu().double() - want).abs().max() < 0.03 * max(1.0, float(want.abs().max()))


def test_a_model_whose_experts_run_on_the_tensor_memory_product(setups, monkeypatch):
    from wllm_b200.parts.experts import RoutedExperts
    monkeypatch.setattr(RoutedExperts, "TC_FROM_PAIRS", 64)
    folder, reqs, ref = setups["wide"]
    steps = traces.whole(reqs)
    runner = runner_for(folder, torch.bfloat16, 16, -(-traces.peak_tokens(steps) // 16))
    close_enough(traces.run_in_process(runner, steps), ref, torch.bfloat16, "whole, experts on tcgen05")
