"""The Podizen decoder on the GPU: every new kernel and every new option of an older one against the plain PyTorch
statement of its operator (tests/torch_ops.py), attention inputs made so that one key stands out at the edges of
windows, pooled blocks and pages, and the engine -- whole prompts, decoding, portions, mixed batches, captured steps,
generation, the trace runner -- against tests/plain_podizen.py."""
import json
import random
import subprocess
from types import SimpleNamespace

import pytest
import torch

import plain_podizen as plain
import traces
from conftest import ROOT, random_tokens
from torch_ops import TorchOps

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL32 = 2e-4


@pytest.fixture(scope="module")
def ops():
    from pytriton_llama_b200.ops.cuda import CudaOps
    return CudaOps(torch.device("cuda:0"))


def _ctx(q_lens, starts, slots, device):
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    return SimpleNamespace(num_requests=len(q_lens), num_tokens=q_start[-1], q_start=t(q_start), state_slot=t(slots), max_q_len=max(q_lens),
                           max_ctx_len=max(s + n for s, n in zip(starts, q_lens)), work={},
                           tok_req=t([r for r, n in enumerate(q_lens) for _ in range(n)]),
                           positions=t([s + i for s, n in zip(starts, q_lens) for i in range(n)]))


def _close(got, ref, dtype, what, scale=None, tol=None):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all(), what
    scale = scale or max(1.0, float(ref.abs().max()))
    tol = tol or (2e-5 if dtype == "float32" else 1.2e-2)
    assert (got - ref).abs().max() <= tol * scale, f"{what}: {(got - ref).abs().max():.3e} of {scale:.2f}"


def _rand(gen, *shape, scale=1.0):
    return torch.randn(*shape, generator=gen) * scale


# ---------------------------------------------------------------------------- norm after a sub-layer, sum over depth
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 256, 200, 1030, 33, 2048, 4096, 8200])
def test_post_norm_residual_depth_sum_and_next_norm(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    dt, T, ref = DTYPES[dtype], 13, TorchOps()
    a, b = _rand(g, T, width).to(dt), _rand(g, T, width, scale=3.0).to(dt)
    wa, wb, post, nxt = (1 + 0.2 * _rand(g, width) for _ in range(4))
    res = _rand(g, T, width)
    results = _rand(g, 6, T, width)
    coeffs = _rand(g, 5)
    dev = lambda t: None if t is None else t.cuda()
    cases = {
        "one output": dict(outs=[a], weights=None),
        "a float32 output": dict(outs=[a.float() * 1.001], weights=None),
        "mean of two normed members": dict(outs=[a, b], weights=[wa, wb]),
        "one normed member": dict(outs=[b], weights=[wb]),
    }
    for what, c in cases.items():
        for depth in (None, 0, 4):
            for with_next in (True, False):
                ra, rb = res.clone().cuda(), res.clone()
                ha, hb = results.clone().cuda(), results.clone()
                kw_a = dict(results=ha, index=depth, coeffs=coeffs.cuda()) if depth is not None else {}
                kw_b = dict(results=hb, index=depth, coeffs=coeffs) if depth is not None else {}
                ya, ra2 = ops.post_norm_add([dev(o) for o in c["outs"]], None if c["weights"] is None else [dev(w) for w in c["weights"]],
                                            post.cuda(), 1e-5, ra, dtype=dt, next_weight=nxt.cuda() if with_next else None, **kw_a)
                yb, _ = ref.post_norm_add(c["outs"], c["weights"], post, 1e-5, rb, dtype=dt, next_weight=nxt if with_next else None, **kw_b)
                assert ra2 is ra and (ya is None) == (not with_next)
                tol = 2e-5 if dtype == "float32" or c["outs"][0].dtype == torch.float32 else None
                _close(ra, rb, "float32", f"{what}, depth {depth}: stream", tol=3e-6)
                if depth is not None:
                    _close(ha[depth], hb[depth], "float32", f"{what}, depth {depth}: the layer's result", tol=3e-6)
                    assert torch.equal(ha[depth + 1:].cpu(), results[depth + 1:]) and torch.equal(ha[:depth].cpu(), results[:depth])
                if with_next:
                    _close(ya, yb, dtype, f"{what}, depth {depth}: next norm")
    got = ops.mean_of_normed([(a.cuda(), wa.cuda()), (b.cuda(), wb.cuda())], 1e-5, dt)
    _close(got, ref.mean_of_normed([(a, wa), (b, wb)], 1e-5, dt), dtype, "the mean alone")


# ---------------------------------------------------------------------------- per-head norm, rotation of halves, cache write
def _paged(gen, q_lens, starts, page, pages=64, width=24):
    """Block tables over shuffled pages and the slots of the step's tokens."""
    perm = torch.randperm(pages, generator=gen).tolist()
    bt = torch.full((len(q_lens), width), -1, dtype=torch.int32)
    slots, k = [], 0
    for r, (n, s) in enumerate(zip(q_lens, starts)):
        for b in range(-(-(s + n) // page)):
            bt[r, b] = perm[k]
            k += 1
        slots += [int(bt[r, p // page]) * page + p % page for p in range(s, s + n)]
    return bt, torch.tensor(slots, dtype=torch.int32)


def _summary_tables(gen, q_lens, starts, page, block, width):
    """Block tables of the pages of block means and, per token, the slot of the block it completes (-1: none)."""
    ends = [s + n for s, n in zip(starts, q_lens)]
    need = [-(-(e // block) // page) for e in ends]
    perm = torch.randperm(sum(need) + 2, generator=gen).tolist()
    bt = torch.full((len(q_lens), max(width, max(need) + 1)), -1, dtype=torch.int32)
    k, slots = 0, []
    for r, n in enumerate(need):
        for b in range(n):
            bt[r, b] = perm[k]
            k += 1
    for r, (n, s) in enumerate(zip(q_lens, starts)):
        for p in range(s, s + n):
            b = (p + 1) // block - 1
            slots.append(int(bt[r, b // page]) * page + b % page if (p + 1) % block == 0 else -1)
    return bt, torch.tensor(slots, dtype=torch.int32), sum(need) + 2


HEAD_SHAPES = [   # H, G, d, dv, page, rotated, normed
    (4, 2, 64, 64, 16, 32, True), (6, 3, 48, 80, 8, 48, True), (2, 1, 24, 40, 4, 0, False), (8, 2, 128, 128, 16, 64, True),
    (3, 3, 16, 16, 4, 2, True), (5, 1, 72, 8, 32, 72, False), (1, 1, 200, 24, 8, 100, True), (2, 2, 8, 264, 4, 4, True),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,page,rot,normed", HEAD_SHAPES)
def test_head_norm_rotation_of_halves_and_cache_write(ops, dtype, H, G, d, dv, page, rot, normed):
    g = torch.Generator().manual_seed(H * 100 + d)
    dt, ref = DTYPES[dtype], TorchOps()
    q_lens, starts = [70, 1, 7, 1], [0, 900, 21, 3]
    cd, cc = _ctx(q_lens, starts, [0, 1, 2, 3], "cuda:0"), _ctx(q_lens, starts, [0, 1, 2, 3], "cpu")
    T = sum(q_lens)
    pages = sum(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 3
    bt, slots = _paged(g, q_lens, starts, page, pages, width=-(-901 // page) + 2)
    extra = 24          # columns after q, k, v (a gate) that stay as they are
    proj = _rand(g, T, H * d + G * (d + dv) + extra).to(dt)
    cache = _rand(g, pages, G * page * (d + dv), scale=0.5).to(dt)
    qn, kn = 1 + 0.3 * _rand(g, d), 1 + 0.3 * _rand(g, d)
    freq = 30.0 ** (-torch.arange(max(rot // 2, 1), dtype=torch.float32) * 2 / max(rot, 1))
    eps = 1e-5 if normed else 0.0
    pa, ca, pb, cb = proj.clone().cuda(), cache.clone().cuda(), proj.clone(), cache.clone()
    ops.head_norm_rotate_store(pa, H, G, d, dv, qn.cuda(), kn.cuda(), eps, cd.positions, freq.cuda() if rot else None, rot, slots.cuda(), ca, page)
    ref.head_norm_rotate_store(pb, H, G, d, dv, qn, kn, eps, cc.positions, freq if rot else None, rot, slots, cb, page)
    # (the device works the angles out in 64 bits: at position 900 a float32 product would be off by up to 900 * 2^-24)
    _close(pa, pb, dtype, "q and k in place")
    _close(ca, cb, dtype, "cache")
    assert torch.equal(pa[:, -extra:].cpu(), proj[:, -extra:])
    # heads that are only turned (the two halves of a retention's projection), nothing stored
    pq = proj.clone().cuda()
    ops.head_norm_rotate_store(pq, H + G, 0, d, dv, None, None, 0.0, cd.positions, freq.cuda() if rot else None, rot, None, None, 1)
    pr = proj.clone()
    ref.head_norm_rotate_store(pr, H + G, 0, d, dv, None, None, 0.0, cc.positions, freq if rot else None, rot, None, None, 1)
    _close(pq, pr, dtype, "turned alone")
    # a table in 64 bits gives the same as its float32 rounding up to that rounding
    if rot:
        p64 = proj.clone().cuda()
        ops.head_norm_rotate_store(p64, H + G, 0, d, dv, None, None, 0.0, cd.positions, freq.double().cuda(), rot, None, None, 1)
        _close(p64, pr, dtype, "table in 64 bits")
    assert torch.equal(pq[:, (H + G) * d:].cpu(), proj[:, (H + G) * d:])


# ---------------------------------------------------------------------------- block means and the attention over them
POOL_SHAPES = [   # H, G, d, dv, page, window, block, bias, gate
    (4, 2, 64, 64, 16, 20, 6, 0.0, False), (6, 3, 48, 80, 8, 9, 12, 0.0, False), (2, 1, 24, 40, 4, 5, 1, 0.0, True),
    (8, 2, 128, 128, 16, 40, 16, 8.0, True), (3, 3, 16, 16, 4, 1, 3, 0.0, False), (5, 1, 72, 8, 32, 33, 7, 8.0, False),
    (8, 2, 64, 40, 16, 100, 0, 8.0, True), (4, 4, 32, 32, 8, 0, 0, 5.0, True), (6, 2, 64, 128, 16, 50, 10, 0.0, False),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,page,window,block,bias,gate", POOL_SHAPES)
def test_block_means_and_attention_with_bias_gate_and_pooled_blocks(ops, dtype, H, G, d, dv, page, window, block, bias, gate):
    # a prompt that passes many blocks, single tokens, portions
    _pooled_attention_case(ops, dtype, H, G, d, dv, page, window, block, bias, gate, [300, 1, 37, 1, 2], [0, 190, 61, 3, 254])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,window,block", [(4, 2, 64, 30, 4), (2, 1, 128, 17, 3), (4, 4, 64, 200, 2)])
def test_hundreds_of_block_means_fill_several_key_tiles(ops, dtype, H, G, d, window, block):
    """More block means than one key tile of the prompt kernels holds, in a whole prompt and in a portion that follows
    700 cached positions (whose means earlier steps made), beside a single token far out."""
    _pooled_attention_case(ops, dtype, H, G, d, d, 16, window, block, 8.0, True, [900, 150, 1], [0, 700, 820])


def _pooled_attention_case(ops, dtype, H, G, d, dv, page, window, block, bias, gate, q_lens, starts):
    g = torch.Generator().manual_seed(H * 100 + d + block)
    dt, ref = DTYPES[dtype], TorchOps()
    R = len(q_lens)
    cd, cc = _ctx(q_lens, starts, list(range(R)), "cuda:0"), _ctx(q_lens, starts, list(range(R)), "cpu")
    T = sum(q_lens)
    pages = sum(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 3
    bt, slots = _paged(g, q_lens, starts, page, pages, width=max(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 2)
    gate_col = H * d + G * (d + dv)
    proj = _rand(g, T, gate_col + H * dv).to(dt)
    cache = _rand(g, pages, G * page * (d + dv), scale=0.5).to(dt)
    # this step's keys and values go to the cache first
    for t in range(T):
        pg, off = divmod(int(slots[t]), page)
        kp, vp = TorchOps._page_views(cache, pg, G, page, d, dv)
        kp[:, off] = proj[t, H * d:(H + G) * d].view(G, d)
        vp[:, off] = proj[t, (H + G) * d:(H + G) * d + G * dv].view(G, dv)
    kw_a, kw_b = {}, {}
    if block:
        sbt, sslots, spages = _summary_tables(g, q_lens, starts, page, block, 4)
        summary = _rand(g, spages, G * page * (d + dv), scale=0.5).to(dt)       # means of blocks that earlier steps completed: noise
        sa, sb = summary.clone().cuda(), summary.clone()
        ops.pool_blocks(cache.cuda(), bt.cuda(), cd.tok_req, cd.positions, sslots.cuda(), sa, G, d, dv, page, block)
        ref.pool_blocks(cache, bt, cc.tok_req, cc.positions, sslots, sb, G, d, dv, page, block)
        _close(sa, sb, dtype, "block means")
        kw_a, kw_b = dict(pool=block, summary=sb.clone().cuda(), summary_table=sbt.cuda()), dict(pool=block, summary=sb, summary_table=sbt)
    if bias:
        kw_a["distance_bias"] = kw_b["distance_bias"] = bias
    if gate:
        kw_a["gate_column"] = kw_b["gate_column"] = gate_col
    want = ref.window_attention(proj, cache, bt, cc.tok_req, cc.positions, H, G, d, dv, page, 0.2, window, 0, **kw_b)
    hints = ops.hints_for(q_lens, [s + n for s, n in zip(starts, q_lens)])
    out = ops.window_attention(proj.cuda(), cache.cuda(), bt.cuda(), cd.tok_req, cd.positions, H, G, d, dv, page, 0.2, window, 0,
                               hints=hints, **kw_a)
    _close(out, want, dtype, "as the engine calls it", tol=2e-5 if dtype == "float32" else 2e-2)
    pooled = (block, kw_a["summary"].data_ptr(), kw_a["summary_table"].data_ptr(), kw_a["summary_table"].shape[1], kw_a["summary"].shape[0]) \
        if block else (0, None, None, 0, 0)
    for splits in (1, 3):
        out = torch.empty((T, H * dv), dtype=dt, device="cuda:0")
        ops._window_attention_simt(out, proj.cuda(), cache.cuda(), bt.cuda(), cd.tok_req, cd.positions, H, G, d, dv, page, 0.2, window, 0,
                                   splits, None, (0, 0, 0.0, 1, bias, gate_col if gate else -1, *pooled))
        _close(out, want, dtype, f"{splits} parts", tol=2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [4, 16])
@pytest.mark.parametrize("q_len", [1, 5, 140])
def test_a_key_that_stands_out_is_seen_where_window_and_blocks_say(ops, dtype, page, q_len):
    """One key (position ``spike``) with a score far above the others and a value of its own: the result is that value
    where the query sees the key as a token, a block's share of it where it sees the key's block, nothing of it where
    the key has left the window and its block is not yet whole behind it."""
    H, G, d, dv, window, block, spike, n = 2, 1, 32, 32, 24, 10, 33, 140
    dt, ref = DTYPES[dtype], TorchOps()
    g = torch.Generator().manual_seed(page + q_len)
    start = n - q_len
    cd, cc = _ctx([q_len], [start], [0], "cuda:0"), _ctx([q_len], [start], [0], "cpu")
    bt, _ = _paged(g, [n], [0], page, -(-n // page) + 2, width=-(-n // page) + 1)
    keys, values = _rand(g, n, d, scale=0.05), _rand(g, n, dv, scale=0.1)
    keys[spike, 0] = 6.0
    values[spike] = 50.0
    cache = torch.zeros(-(-n // page) + 2, G * page * (d + dv)).to(dt)
    for p in range(n):
        kp, vp = TorchOps._page_views(cache, int(bt[0, p // page]), G, page, d, dv)
        kp[0, p % page], vp[0, p % page] = keys[p].to(dt), values[p].to(dt)
    sbt, _, spages = _summary_tables(g, [n], [0], page, block, 4)
    summary = torch.zeros(spages, G * page * (d + dv)).to(dt)
    all_pos = _ctx([n], [0], [0], "cpu")
    every = torch.tensor([int(sbt[0, ((p + 1) // block - 1) // page]) * page + ((p + 1) // block - 1) % page if (p + 1) % block == 0 else -1
                          for p in range(n)], dtype=torch.int32)
    ref.pool_blocks(cache, bt, all_pos.tok_req, all_pos.positions, every, summary, G, d, dv, page, block)
    q = torch.zeros(q_len, H * d + G * (d + dv))
    q[:, 0] = 4.0
    q[:, d] = 4.0
    q = q.to(dt)
    want = ref.window_attention(q, cache, bt, cc.tok_req, cc.positions, H, G, d, dv, page, 1.0, window, 0, pool=block, summary=summary,
                                summary_table=sbt)
    got = ops.window_attention(q.cuda(), cache.cuda(), bt.cuda(), cd.tok_req, cd.positions, H, G, d, dv, page, 1.0, window, 0,
                               hints=ops.hints_for([q_len], [n]), pool=block, summary=summary.cuda(), summary_table=sbt.cuda())
    _close(got, want, dtype, "spiked key", tol=1e-4 if dtype == "float32" else 2e-2)
    for i in range(q_len):
        p = start + i
        seen_as_token = 0 <= p - spike < window
        block_seen = (spike // block) * block + block - 1 <= p - window
        level = float(want[i, 0])
        if seen_as_token:
            assert level > 45, (p, level)
        elif block_seen:
            assert 0.5 < level < 45, (p, level)
        else:
            assert abs(level) < 0.3, (p, level)


# ---------------------------------------------------------------------------- retention
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,dv", [(3, 48, 64), (2, 20, 40), (1, 128, 128), (2, 200, 24), (4, 8, 8), (1, 64, 33), (4, 32, 32)])
def test_retention_walk_and_its_state(ops, dtype, H, d, dv):
    g = torch.Generator().manual_seed(H * 10 + d)
    dt, ref = DTYPES[dtype], TorchOps()
    q_lens, starts, slots = [70, 1, 9, 1], [0, 40, 17, 0], [2, 0, 3, 1]
    cd, cc = _ctx(q_lens, starts, slots, "cuda:0"), _ctx(q_lens, starts, slots, "cpu")
    T = sum(q_lens)
    proj = _rand(g, T, 2 * H * d + 2 * H * dv, scale=0.7).to(dt)
    decay = torch.tensor([1.0, 0.0, 0.97, 0.9995][:H] + [0.9] * max(0, H - 4))
    state = _rand(g, 5, H, d, dv, scale=0.3)
    sa, sb = state.clone().cuda(), state.clone()
    a = ops.gla_scan(proj.cuda(), None, None, 1.0, sa, cd, H, d, dv, 1.0, head_decay=decay.cuda(), k_scale=d ** -0.5)
    b = ref.gla_scan(proj, None, None, 1.0, sb, cc, H, d, dv, 1.0, head_decay=decay, k_scale=d ** -0.5)
    _close(a, b, "float32", "read-outs", tol=2e-5)
    _close(sa, sb, "float32", "states", tol=2e-5)
    assert torch.equal(sa[4].cpu(), state[4])                     # a slot of no request in the step


def test_a_far_token_survives_a_decay_of_one_and_dies_under_a_strong_one(ops):
    H, d, dv, n = 2, 16, 16, 700
    proj = torch.zeros(n, 2 * H * d + 2 * H * dv)
    proj[0, H * d:2 * H * d] = 1.0            # the first token's key
    proj[0, 2 * H * d:2 * H * d + H * dv] = 3.0
    proj[:, :H * d] = 1.0                      # every query reads it
    cd = _ctx([n], [0], [0], "cuda:0")
    state = torch.zeros(1, H, d, dv, device="cuda:0")
    out = ops.gla_scan(proj.cuda(), None, None, 1.0, state, cd, H, d, dv, 1.0, head_decay=torch.tensor([1.0, 0.9]).cuda(), k_scale=0.25)
    assert torch.allclose(out[-1, :dv].cpu(), torch.full((dv,), 3.0 * d * 0.25), rtol=1e-6)
    assert float(out[-1, dv:].abs().max()) < 1e-20 and float(out[5, dv]) == pytest.approx(3.0 * d * 0.25 * 0.9 ** 5, rel=1e-5)


# ---------------------------------------------------------------------------- experts with grouped softmax routing
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,W,ff,E,top,groups,keep,shared", [(45, 64, 32, 8, 4, 4, 3, True), (3, 96, 64, 16, 1, 16, 1, False),
                                                             (200, 48, 24, 6, 2, 1, 1, True), (17, 40, 16, 9, 3, 3, 2, False),
                                                             (64, 128, 96, 64, 6, 8, 3, True), (5, 32, 8, 1, 1, 1, 1, True),
                                                             (33, 72, 40, 12, 12, 4, 4, False), (9, 64, 16, 130, 5, 10, 2, False)])
def test_routed_experts_softmax_groups_renormalised(ops, dtype, T, W, ff, E, top, groups, keep, shared):
    g = torch.Generator().manual_seed(T + E)
    dt, ref = DTYPES[dtype], TorchOps()
    x = _rand(g, T, W).to(dt)
    logits = _rand(g, T, E, scale=2.0)
    w_gu, w_d = _rand(g, E, 2 * ff, W, scale=W ** -0.5).to(dt), _rand(g, E, W, ff, scale=ff ** -0.5).to(dt)
    sh = _rand(g, T, W).to(dt) if shared else None
    opts = dict(score="softmax", groups=groups, keep_groups=keep, renormalise=True)
    a = ops.routed_experts(x.cuda(), logits.cuda(), w_gu.cuda(), w_d.cuda(), top, False, sh.cuda() if shared else None, **opts)
    b = ref.routed_experts(x, logits, w_gu, w_d, top, False, sh, **opts)
    _close(a, b, dtype, "experts", tol=2e-5 if dtype == "float32" else 2e-2)


def test_routing_takes_the_best_groups_and_weights_sum_to_one(ops):
    """Logits made so that the best single expert sits in a group that is not kept only if groups are ignored, and ties
    go to the lower number: the chosen experts are read off a down projection that writes the expert's own number."""
    E, W, ff = 8, 16, 8
    logits = torch.tensor([[0.0, 3.0, 2.9, 2.8, -1.0, 2.95, 0.5, 0.4],       # groups of 2: best scores 3.0, 2.9, 2.95, 0.5
                           [1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0]])
    x = torch.ones(2, W)
    w_gu = torch.zeros(E, 2 * ff, W)
    w_gu[:, :ff, 0] = 20.0                      # silu(gate) * up = 20 * 1 in every inner entry
    w_gu[:, ff:, 0] = 1.0
    w_d = torch.zeros(E, W, ff)
    for e in range(E):
        w_d[e, e, 0] = 1.0 / 20.0               # expert e writes 1 to entry e of the output
    out = ops.routed_experts(x.cuda(), logits.cuda(), w_gu.cuda(), w_d.cuda(), 2, False, None, score="softmax", groups=4, keep_groups=2,
                             renormalise=True).cpu()
    assert sorted(torch.nonzero(out[0] > 1e-6).flatten().tolist()) == [1, 5]     # groups 0 and 2 are kept: experts 1 and 5, not 2
    assert out[0].sum().item() == pytest.approx(1.0, rel=1e-5) and out[0, 1] > out[0, 5]
    assert sorted(torch.nonzero(out[1] > 1e-6).flatten().tolist()) == [0, 1]     # all equal: the lowest group, the lowest experts
    assert out[1, 0].item() == pytest.approx(0.5, rel=1e-5)


# ---------------------------------------------------------------------------- the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, dtype, cfg=None, seed=5):
        if (name, dtype) not in made:
            folder = tmp_path_factory.mktemp(f"podizen_{name}_{dtype}")
            plain.write_model(folder, cfg or plain.TINY[name], seed, DTYPES[dtype])
            made[(name, dtype)] = folder
        return made[(name, dtype)]
    return get


def _engine(folder, dtype, page, pages, max_seq_len=512, slots=4, **extra):
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine
    return Engine(folder, EngineConfig(dtype=dtype, page_size=page, max_gpu_num_blocks=pages, max_seq_len=max_seq_len,
                                       max_num_seqs=slots, **extra), device="cuda:0")


def _reference(folder, seqs):
    from pytriton_llama_b200.weights import read_folder
    cfg = json.loads((folder / "config.json").read_text())
    W = read_folder(folder)
    return {r: plain.forward(cfg, W, s) for r, s in seqs.items()}


def _assert_logits(got, ref, dtype, what):
    diff = (got.double().cpu() - ref).abs()
    if dtype == "float32":
        assert diff.max() < TOL32 * max(1.0, float(ref.abs().max())), f"{what}: {diff.max():.3e}"
    else:
        centred = (got.double().cpu() - ref) - (got.double().cpu() - ref).mean(-1, keepdim=True)
        rms = centred.pow(2).mean(-1).sqrt() / ref.std()
        # Rounding alone: 0.04 to 0.09 of the logits' spread in the typical row of these models (every sub-layer's output
        # is normed to unit size before it is added, so a rounding error of a small output counts like one of a large
        # one).  A row where a router's scores lie
        # within rounding of each other may take another expert than the float64 computation does, and the rows after it
        # feel that through the mixers: such rows are allowed, as long as they are few.  A fault of a mechanism shows in
        # float32, where the bound is 2e-4.
        off = int((rms > 0.4).sum())
        assert rms.median() < 0.1 + 0.06 * (rms.numel() < 4) and off <= max(1, rms.numel() // 10), \
            f"{what}: median row {rms.median():.3f} of the logits' spread, {off} of {rms.numel()} rows beyond 0.4"


# Heads of 64 and 128, widths that are multiples of 64, windows and blocks that prompts pass.
WIDE = plain.config(300, 128, [
    plain.layer("attention", plain.gated_attention(4, 2, 64, 64, 0.125, size=40), plain.moe(64, 8, 2, groups=4, keep=2, shared=64)),
    plain.layer("parallel", plain.parallel(plain.pooled_attention(4, 2, 64, 128, 0.125, size=24, pool=8, rot=plain.rotation(32, 10000.0)),
                                           plain.retention(2, 64, 64, (0.96875, 0.998), rot=plain.rotation(64, 1.0e5))), plain.moe(32, 4, 1)),
    plain.layer("parallel", plain.parallel(plain.pooled_attention(2, 1, 128, 64, 0.09, size=33, pool=16, rot=plain.rotation(128, 500.0)),
                                           plain.retention(4, 32, 32, (0.9, 0.99, 0.999, 1.0))), None),
    plain.layer("attention", plain.gated_attention(8, 1, 32, 48, 0.17, size=70), plain.moe(48, 6, 3, groups=2, keep=1, shared=16)),
])


def _config(name):
    return WIDE if name == "WIDE" else plain.TINY[name]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("C", 16), ("WIDE", 16)])
def test_every_cut_gives_the_whole_sequence_logits(folders, dtype, name, page):
    folder = folders(name, dtype, _config(name))
    vocab = _config(name)["vocab"]
    seqs = {f"r{i}": random_tokens(n, vocab, 700 + i) for i, n in enumerate([1, 9, 33, 150, 12, 27, 64])}
    ref = _reference(folder, seqs)
    for family in (traces.whole, traces.prefill_then_decode, traces.portions, traces.mixed):
        steps = family(seqs)
        pages = -(-traces.max_live_tokens(steps, 16) // page)
        eng = _engine(folder, dtype, page, pages)
        got = traces.replay(eng, steps)
        for r in seqs:
            _assert_logits(got[r], ref[r][traces.wanted_positions(steps, r)], dtype, f"{family.__name__} {r}")
        eng.check_device_status()
        eng.cache.check_invariants()
        assert eng.cache.free_slots() == 4 and all(eng.cache.free_pages(g) == eng.cache.groups[g].pool.num_pages for g in eng._paged_groups())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_from_captured_graphs(folders, dtype):
    folder = folders("WIDE", dtype, WIDE)
    seqs = {f"g{i}": random_tokens(n, 300, 300 + i) for i, n in enumerate([80, 7, 55, 21, 33])}
    ref = _reference(folder, seqs)
    eng = _engine(folder, dtype, 16, 40, compiled_model=True)
    for turn in range(3):           # the same steps again: shapes seen twice are captured, then replayed
        for family in (traces.prefill_then_decode, traces.mixed):
            steps = family(seqs)
            got = traces.replay(eng, steps)
            for r in seqs:
                _assert_logits(got[r], ref[r][traces.wanted_positions(steps, r)], dtype, f"turn {turn} {family.__name__} {r}")
    assert any(not isinstance(k, tuple) for k in eng._graphs)             # decode steps were captured
    eng.check_device_status()


def _random_config(seed):
    """Sizes drawn freely: head sizes that are no power of two, one to three kv heads, windows of 1 to 60 positions, blocks
    of 1 to 20, part of a head or all of it rotated, layers in any order, with and without feed-forwards and shared
    experts, groups of one to four experts."""
    rng = random.Random(seed)
    width = rng.choice([48, 56, 64, 72, 88, 100])
    layers = []
    for i in range(rng.randint(2, 5)):
        mlp = None
        if rng.random() > 0.2:
            groups = rng.choice([1, 2, 3, 4])
            per = rng.randint(1, 4)
            keep = rng.randint(1, groups)
            mlp = plain.moe(rng.choice([8, 24, 40]), groups * per, rng.randint(1, keep * per), groups=groups if rng.random() < 0.8 else 0,
                            keep=keep, shared=rng.choice([0, 16, 40]))
            if not mlp["router"].get("groups"):
                mlp["router"]["top"] = rng.randint(1, groups * per)
        G, d = rng.randint(1, 3), rng.choice([8, 16, 24, 40, 64])
        if rng.random() < 0.45:
            m = plain.gated_attention(G * rng.choice([1, 2, 4]), G, d, rng.choice([8, 16, 24, 40, 64]), rng.uniform(0.1, 0.4),
                                      rng.choice([0, rng.randint(1, 60)]))
            layers.append(plain.layer("attention", m, mlp))
            continue
        size = rng.choice([0, rng.randint(1, 60)])
        rot = None if rng.random() < 0.2 else plain.rotation(rng.choice([2, d // 2 // 2 * 2, d]), rng.choice([30.0, 10000.0]))
        left = plain.pooled_attention(G * rng.choice([1, 2, 4]), G, d, rng.choice([8, 16, 24, 40, 64]), rng.uniform(0.1, 0.4), size,
                                      rng.choice([0, rng.randint(1, 20)]) if size else 0, rot)
        Hr, dr = rng.randint(1, 4), rng.choice([8, 12, 20, 36, 64])
        right = plain.retention(Hr, dr, rng.choice([8, 24, 40, 64]), [rng.choice([0.5, 0.9, 0.99, 0.9995, 1.0]) for _ in range(Hr)],
                                None if rng.random() < 0.2 else plain.rotation(rng.choice([2, dr // 2 // 2 * 2, dr]), rng.choice([30.0, 1.0e6])))
        layers.append(plain.layer("parallel", plain.parallel(left, right), mlp))
    return plain.config(rng.randint(50, 300), width, layers, eps=rng.choice([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configurations(tmp_path, dtype, seed):
    cfg = _random_config(seed)
    plain.write_model(tmp_path, cfg, seed, DTYPES[dtype])
    seqs = {f"r{i}": random_tokens(n, cfg["vocab"], 40 * seed + i) for i, n in enumerate([90, 1, 33, 14])}
    ref = _reference(tmp_path, seqs)
    page = random.Random(seed).choice([4, 8, 16, 32])
    for family in (traces.whole, traces.mixed):
        steps = family(seqs)
        eng = _engine(tmp_path, dtype, page, -(-traces.max_live_tokens(steps, 32) // page) + 1)
        got = traces.replay(eng, steps)
        for r in seqs:
            _assert_logits(got[r], ref[r][traces.wanted_positions(steps, r)], dtype, f"seed {seed} {family.__name__} {r}")
        eng.check_device_status()


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_traces_in_float32(folders, seed):
    folder = folders("A", "float32")
    rng = random.Random(seed)
    seqs = {f"t{i}": random_tokens(rng.randint(1, 200), 97, 900 + 10 * seed + i) for i in range(7)}
    ref = _reference(folder, seqs)
    steps = traces.random_trace(seqs, rng)
    for graphs in (False, True):
        eng = _engine(folder, "float32", 4, -(-traces.max_live_tokens(steps, 4) // 4), compiled_model=graphs)
        got = traces.replay(eng, steps)
        for r in got:
            _assert_logits(got[r], ref[r][traces.wanted_positions(steps, r)], "float32", f"trace {seed} {r}")
        eng.cache.check_invariants()


def test_batch_does_not_change_a_request(folders):
    from pytriton_llama_b200.engine.engine import StepEntry
    folder = folders("WIDE", "float32", WIDE)
    seqs = {"a": random_tokens(137, 300, 1), "b": random_tokens(8, 300, 2), "c": random_tokens(61, 300, 3)}
    eng = _engine(folder, "float32", 16, 40)
    together = eng.step([StepEntry(r, s, list(range(len(s)))) for r, s in seqs.items()]).logits
    eng.finish_all()
    at = 0
    for r, s in seqs.items():
        alone = eng.step([StepEntry(r, s, list(range(len(s))))]).logits
        eng.finish(r)
        assert torch.allclose(together[at:at + len(s)], alone, atol=2e-5, rtol=1e-5), r
        at += len(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    from pytriton_llama_b200.engine.engine import StepEntry
    folder = folders("WIDE", dtype, WIDE)
    toks = random_tokens(400, 300, 21)
    ref = _reference(folder, {"a": toks})["a"]
    eng = _engine(folder, dtype, 16, 9)           # 9 pages for 400 tokens: pages the windows have passed come back
    rows = [eng.step([StepEntry("a", toks[:3], [0, 1, 2])]).logits] + [eng.step([StepEntry("a", [t], [0])]).logits for t in toks[3:]]
    _assert_logits(torch.cat(rows), ref, dtype, "400 tokens, one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(folders, dtype):
    from pytriton_llama_b200 import LLM, EngineConfig, SamplingParams
    folder = folders("A", dtype)
    prompts = [random_tokens(n, 97, 40 + i) for i, n in enumerate([5, 23, 2, 14, 9, 31])]
    cfg = EngineConfig(dtype=dtype, page_size=4, max_gpu_num_blocks=60, max_seq_len=64, max_num_seqs=3, max_batched_tokens=16)
    outs = LLM(folder, cfg).generate(prompts, SamplingParams(temperature=0.0, max_gen_len=8))
    near, far = 0, []
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        logits = _reference(folder, {"x": p + o})["x"]
        slack = 1e-3 if dtype == "float32" else 0.05 * float(logits.std())
        for i, tok in enumerate(o):
            row = logits[len(p) + i - 1]
            if row[tok] >= row.max() - slack:
                near += 1
            else:
                far.append((i, tok, int(row.argmax())))
    # in 16 bits a router's close call may send a token to another expert than the float64 computation does, and what is
    # generated after it differs: a few such tokens are allowed; in float32 none
    assert not far if dtype == "float32" else len(far) <= 4, far


def test_trace_runner_and_command_line(folders, tmp_path):
    folder = folders("WIDE", "bfloat16", WIDE)
    seqs = {"a": random_tokens(90, 300, 1), "b": random_tokens(13, 300, 2)}
    steps = traces.mixed(seqs)
    lines = "\n".join(json.dumps(s) for s in steps) + "\n"
    for dtype in ("bfloat16", "float32"):
        out = tmp_path / dtype
        proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                               "--max-tokens", str(traces.max_live_tokens(steps))], input=lines, text=True, capture_output=True,
                              timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
        ref = _reference(folder, seqs)
        fed = {r: 0 for r in seqs}
        got, want = [], []
        for s in steps:
            rows = torch.frombuffer(bytearray((out / f"{s['step']}.f32").read_bytes()), dtype=torch.float32).view(-1, 300)
            at = 0
            for e in s["entries"]:
                for w in e["want"]:
                    got.append(rows[at])
                    want.append(ref[e["id"]][fed[e["id"]] + w])
                    at += 1
                fed[e["id"]] += len(e["tokens"])
        _assert_logits(torch.stack(got), torch.stack(want), dtype, f"{dtype} replay")
    import sys
    proc = subprocess.run([sys.executable, str(ROOT / "cli.py"), "--checkpoints_dir", str(folder), "--temperature", "0",
                           "--max_gen_len", "5", "--max_seq_len", "64", "--page_size", "16", "--prompt_ids", "3", "1", "4", "1", "5"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert len(proc.stdout.split()) == 5
