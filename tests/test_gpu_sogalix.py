"""The Sogalix decoder on the GPU: every new kernel against the plain PyTorch statement of its operator
(tests/torch_ops.py), inputs made so that one key, the sink term or a far token shows, and the engine -- whole
prompts, decoding, portions, mixed batches, captured steps, generation -- against tests/plain_sogalix.py."""
import json
import math
import random
import subprocess
from types import SimpleNamespace

import pytest
import torch

import plain_sogalix as plain
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
                           max_ctx_len=max(s + n for s, n in zip(starts, q_lens)), work={}, attn_splits=1,
                           tok_req=t([r for r, n in enumerate(q_lens) for _ in range(n)]),
                           positions=t([s + i for s, n in zip(starts, q_lens) for i in range(n)]))


def _close(got, ref, dtype, what, scale=None, tol=None):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), (what, "not finite at", (~torch.isfinite(got)).nonzero()[:6].tolist(), int((~torch.isfinite(got)).sum()))
    scale = scale or max(1.0, float(ref.abs().max()))
    tol = tol or (2e-5 if dtype == "float32" else 1.2e-2)
    assert (got - ref).abs().max() <= tol * scale, f"{what}: {(got - ref).abs().max():.3e} of {scale:.2f}"


def _rand(gen, *shape, scale=1.0):
    return torch.randn(*shape, generator=gen) * scale


def _paged(gen, q_lens, starts, page, pages, width):
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


# ---------------------------------------------------------------------------- layer norm and activation
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [32, 48, 257, 1024, 5000])
def test_layer_norm_with_the_residual_add(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    dt, T, ref = DTYPES[dtype], 21, TorchOps()
    x, res = _rand(g, T, width).to(dt), _rand(g, T, width, scale=3.0) + 50.0        # a mean far from zero: the variance must not cancel
    w, b, extra = 1 + 0.2 * _rand(g, width), 0.3 * _rand(g, width), _rand(g, width)
    ya, ra = ops.add_layernorm(x.cuda(), res.clone().cuda(), w.cuda(), b.cuda(), 1e-5)
    yb, rb = ref.add_layernorm(x, res.clone(), w, b, 1e-5)
    _close(ya, yb, dtype, "normed sum")
    assert torch.equal(ra.cpu(), rb)
    ya, ra = ops.add_layernorm(x.cuda(), res.clone().cuda(), w.cuda(), b.cuda(), 1e-5, add_bias=extra.cuda())
    yb, rb = ref.add_layernorm(x, res.clone(), w, b, 1e-5, add_bias=extra)
    _close(ya, yb, dtype, "with a projection's bias")
    _close(ra, rb, "float32", "sum with a projection's bias")
    rows = torch.tensor([T - 1, 0, 5], dtype=torch.int32)
    before = res.clone().cuda()
    ya, none = ops.add_layernorm(x.cuda(), before, w.cuda(), b.cuda(), 1e-5, rows=rows.cuda())
    yb, _ = ref.add_layernorm(x, res.clone(), w, b, 1e-5, rows=rows)
    _close(ya, yb, dtype, "chosen rows")
    assert none is None and torch.equal(before.cpu(), res)
    ya, ra = ops.add_layernorm(x.cuda(), None, w.cuda(), b.cuda(), 1e-5, dtype=torch.float32, keep_sum=False)   # the start of a stream
    yb, _ = ref.add_layernorm(x, None, w, b, 1e-5, dtype=torch.float32, keep_sum=False)
    assert ra is None and ya.dtype == torch.float32
    _close(ya, yb, "float32", "float32 result from the compute type")
    ya, _ = ops.add_layernorm(None, res.clone().cuda(), w.cuda(), b.cuda(), 1e-5, dtype=dt)                   # a norm without an add
    yb, _ = ref.add_layernorm(None, res.clone(), w, b, 1e-5, dtype=dt)
    _close(ya, yb, dtype, "no add")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_xielu(ops, dtype):
    x = (torch.linspace(-12, 12, 1001)[None, :] * torch.tensor([[1.0], [0.01]])).to(DTYPES[dtype])
    for ap, aq in ((0.7, 1.2), (0.05, 0.5), (2.0, 3.0)):
        _close(ops.xielu(x.cuda(), ap, aq), TorchOps().xielu(x, ap, aq), dtype, "xielu", tol=None if dtype == "float32" else 6e-3)


# ---------------------------------------------------------------------------- generalized delta rule
def _delta_inputs(g, T, H, d, dt, rank=5):
    n = H * d
    proj = _rand(g, T, 4 * n).to(dt)
    aw = _rand(g, T, n + rank, scale=1.5)
    return proj, aw, _rand(g, n), _rand(g, n, rank), 2 * torch.rand(n, generator=g) - 1


@pytest.mark.parametrize("T,n,rank,extra", [(1, 7, 3, 0), (16, 128, 32, 5), (17, 129, 33, 4), (70, 300, 70, 1), (5, 1000, 64, 8)])
def test_decay_argument_tiles_and_single_rows(ops, T, n, rank, extra):
    g = torch.Generator().manual_seed(T + n + rank)
    aw, w2 = _rand(g, T, extra + rank, scale=1.5), _rand(g, n, rank)
    za = ops.lowrank_tanh_linear(aw.cuda(), extra, w2.cuda())
    _close(za, TorchOps().lowrank_tanh_linear(aw, extra, w2), "float32", "decay argument")
    # a row alone has the bits it has inside a tile
    t = T // 2
    alone = ops.lowrank_tanh_linear(aw[t:t + 1].contiguous().cuda(), extra, w2.cuda())
    assert torch.equal(alone[0], za[t])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d", [(3, 32), (2, 20), (1, 128), (2, 200), (4, 4), (1, 64), (5, 8), (1, 40)])
def test_delta_walk_and_its_state(ops, dtype, H, d):
    g = torch.Generator().manual_seed(H * 1000 + d)
    dt, ref = DTYPES[dtype], TorchOps()
    step = ([37, 1, 5, 2], [0, 9, 3, 0], [2, 0, 3, 1])       # a fresh portion, a single token, a running request, a fresh one over noise
    T, n = sum(step[0]), H * d
    proj, aw, a_b, w2, w_b = _delta_inputs(g, T, H, d, dt)
    za, zb = ops.lowrank_tanh_linear(aw.cuda(), n, w2.cuda()), ref.lowrank_tanh_linear(aw, n, w2)
    _close(za, zb, "float32", "decay argument")
    S0 = _rand(g, 4, H, d, d, scale=0.3)
    Sa, Sb = S0.clone().cuda(), S0.clone()
    limit = math.exp(-0.5)
    oa = ops.general_delta_scan(proj.cuda(), aw.cuda(), a_b.cuda(), zb.cuda(), w_b.cuda(), limit, Sa, _ctx(*step, "cuda:0"), H, d, 1e-6)
    ob = ref.general_delta_scan(proj, aw, a_b, zb, w_b, limit, Sb, _ctx(*step, "cpu"), H, d, 1e-6)
    _close(oa, ob, "float32", "read-outs")
    _close(Sa, Sb, "float32", "states")
    # the same tokens in portions of 20, 2, 1 and 14 give the same read-outs and state
    Sc = S0.clone().cuda()
    outs = []
    for lo, hi in ((0, 20), (20, 22), (22, 23), (23, 37)):
        outs.append(ops.general_delta_scan(proj[lo:hi].contiguous().cuda(), aw[lo:hi].contiguous().cuda(), a_b.cuda(), zb[lo:hi].contiguous().cuda(),
                                           w_b.cuda(), limit, Sc, _ctx([hi - lo], [lo], [2], "cuda:0"), H, d, 1e-6))
    _close(torch.cat(outs), ob[:37], "float32", "read-outs in portions")
    _close(Sc[2], Sb[2], "float32", "state after four portions")
    # rows of a padded shape (state slot -1) are skipped and touch no state
    Sd = S0.clone().cuda()
    ops.general_delta_scan(proj[:5].contiguous().cuda(), aw[:5].contiguous().cuda(), a_b.cuda(), zb[:5].contiguous().cuda(), w_b.cuda(), limit, Sd,
                           _ctx([3, 2], [4, 0], [1, -1], "cuda:0"), H, d, 1e-6)
    assert torch.equal(Sd[[0, 2, 3]].cpu(), S0[[0, 2, 3]]) and not torch.equal(Sd[1].cpu(), S0[1])


def test_a_far_token_survives_hundreds_of_decays_and_a_removed_one_is_gone(ops):
    """Decay close to one and no removal: the value written at token 0 is read 600 tokens later, smaller by the decays
    alone.  Then a second key along the same direction with removal rate one wipes it: only the new value is read."""
    H, d, T = 1, 16, 600
    n = H * d
    limit = math.exp(-0.5)
    proj = torch.zeros(T, 4 * n)
    proj[0, n] = 1.0                                       # k_0 = e_0
    proj[0, 2 * n + 3] = 5.0                               # v_0 = 5 e_3
    proj[:, 0] = 4.0                                       # every r reads key channel 0
    aw = torch.full((T, n), -40.0)                         # removal rate 0
    z = torch.full((T, n), -9.0)                           # decay exp(-limit * sigmoid(-9)), close to one
    bias = torch.zeros(n)
    S = torch.zeros(1, H, d, d).cuda()
    out = ops.general_delta_scan(proj.cuda(), aw.cuda(), bias.cuda(), z.cuda(), bias.cuda(), limit, S, _ctx([T], [0], [0], "cuda:0"), H, d, 1e-6)
    w = math.exp(-limit / (1 + math.exp(9.0)))
    want = 4.0 * 5.0 * w ** torch.arange(T, dtype=torch.float64)
    assert torch.allclose(out[:, 3].double().cpu(), want, rtol=3e-5, atol=0)
    proj2 = torch.zeros(1, 4 * n)
    proj2[0, 0], proj2[0, n], proj2[0, 2 * n + 7] = 4.0, 2.0, 1.0          # k = 2 e_0, v = e_7
    one = torch.full((1, n), 40.0)                                       # removal rate 1
    out2 = ops.general_delta_scan(proj2.cuda(), one.cuda(), bias.cuda(), z[:1].cuda(), bias.cuda(), limit, S, _ctx([1], [T], [0], "cuda:0"), H, d, 0.0 + 1e-12)
    row = out2[0].double().cpu()
    assert abs(row[7] - 8.0) < 1e-4                                      # r . k v = 4 * 2 * 1
    assert abs(row[3] - 4.0 * 5.0 * w ** (T - 1) * (w - 1.0)) < 1e-4     # what the decay kept minus all of it: (w - 1) S, next to nothing


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d", [(3, 8), (2, 40), (1, 128)])
def test_head_norm_with_a_sigmoid_gate_and_a_weight_per_head(ops, dtype, H, d):
    g = torch.Generator().manual_seed(H + d)
    dt, T, n = DTYPES[dtype], 9, H * d
    o, w, gate = _rand(g, T, n, scale=3.0), 1 + 0.3 * _rand(g, n), _rand(g, T, 4 * n).to(dt)
    a, b = torch.zeros(T, n, dtype=dt).cuda(), torch.zeros(T, n, dtype=dt)
    ops.gated_head_norm(o.cuda(), w.cuda(), 1e-5, gate.cuda(), 3 * n, H, d, a, 0, 1.0, gate_kind="sigmoid", weight_per_head=True)
    TorchOps().gated_head_norm(o, w, 1e-5, gate, 3 * n, H, d, b, 0, 1.0, gate_kind="sigmoid", weight_per_head=True)
    _close(a, b, dtype, "normed, gated heads")


# ---------------------------------------------------------------------------- attention with a sink term and a query temperature
SINK_SHAPES = [   # H, G, d, dv, page, coef, every
    (6, 1, 48, 48, 16, 0.3, 7), (4, 2, 64, 64, 16, 0.0, 1), (4, 1, 64, 64, 16, 0.7, 9), (3, 3, 16, 24, 4, 1.0, 1), (8, 2, 128, 128, 8, 0.5, 64), (2, 1, 24, 8, 32, 0.2, 3),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,page,coef,every", SINK_SHAPES)
def test_attention_with_sink_and_temperature(ops, dtype, H, G, d, dv, page, coef, every):
    g = torch.Generator().manual_seed(H * 100 + d)
    dt, ref = DTYPES[dtype], TorchOps()
    q_lens, starts = [150, 1, 7, 1, 2], [0, 90, 21, 0, 130]      # a prompt, single tokens (one at position 0), portions
    cd, cc = _ctx(q_lens, starts, [0] * 5, "cuda:0"), _ctx(q_lens, starts, [0] * 5, "cpu")
    T = sum(q_lens)
    pages = sum(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 3
    bt, _ = _paged(g, q_lens, starts, page, pages, width=-(-150 // page) + 2)
    q = _rand(g, T, H * d).to(dt)
    cache = _rand(g, pages, G * page * (d + dv), scale=0.7).to(dt)
    for sink in (True, False):
        want = ref.window_attention(q, cache, bt, cc.tok_req, cc.positions, H, G, d, dv, page, 0.2, sink=sink, temp_coef=coef, temp_every=every)
        hints = ops.hints_for(q_lens, [s + n for s, n in zip(starts, q_lens)])
        got = ops.window_attention(q.cuda(), cache.cuda(), bt.cuda(), cd.tok_req, cd.positions, H, G, d, dv, page, 0.2, hints=hints, sink=sink,
                                   temp_coef=coef, temp_every=every)
        _close(got, want, dtype, f"sink {sink}", tol=2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share(ops, dtype):
    """One key with score 0 beside the sink: weight 1/2.  All scores far below zero: the output vanishes; without the
    sink it would be the value.  Scores far above zero: the sink is nothing."""
    dt, H, d, page = DTYPES[dtype], 2, 16, 4
    bt = torch.tensor([[1, 0]], dtype=torch.int32)
    cache = torch.zeros(2, page * 2 * d)
    cache[1].view(2, page, d)[1, 0, :] = 3.0                 # the value of position 0
    c = _ctx([1], [0], [0], "cuda:0")
    for key0, want in ((0.0, 1.5), (-40.0, 0.0), (40.0, 3.0)):
        cache[1].view(2, page, d)[0, 0, 0] = key0
        q = torch.zeros(1, H * d)
        q[0, 0::d] = 1.0
        out = ops.window_attention(q.to(dt).cuda(), cache.to(dt).cuda(), bt.cuda(), c.tok_req, c.positions, H, 1, d, d, page, 1.0, sink=True)
        assert torch.allclose(out.float().cpu(), torch.full((1, H * d), want), atol=1e-3), (key0, out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,page,shared", [(48, 16, False), (32, 4, False), (128, 8, False), (40, 16, True), (96, 8, True)])
@pytest.mark.parametrize("q_len", [1, 2, 140])
def test_a_key_that_stands_out_is_seen_wherever_it_lies(ops, dtype, d, page, shared, q_len):
    """One key gets a large score with every query; its value is a one-hot.  It lies at the first position, at page
    borders, far back among hundreds, at the query's own position -- and one position after the last query but one,
    which that query must not see.  ``shared``: the value is the first entries of the key itself (the latent form)."""
    H, G = (4, 1) if shared else (4, 2)
    dv = d - 8 if shared else d
    dt, ref = DTYPES[dtype], TorchOps()
    total = 300
    start = total - q_len
    g = torch.Generator().manual_seed(d + q_len)
    pages = -(-total // page) + 2
    bt, _ = _paged(g, [q_len], [start], page, pages, width=-(-total // page) + 1)
    last = total - 1
    for loud in (0, 1, page - 1, page, 2 * page - 1, 150, last - last % page - 1, last - last % page, last - 1, last):
        per_page = G * page * (d if shared else d + dv)
        cache = _rand(g, pages, per_page, scale=0.05).to(dt)
        q = _rand(g, q_len, H * d, scale=0.05)
        q[:, d - 1::d] = 6.0                               # the last entry of every head
        pg, off = int(bt[0, loud // page]), loud % page
        flat = cache[pg].view(-1)
        for kv in range(G):
            kbase = (kv * page + off) * d
            vbase = kbase if shared else G * page * d + (kv * page + off) * dv
            flat[vbase:vbase + dv] = 0
            flat[vbase + 1] = 8.0                                                        # value: one-hot at entry 1
            flat[kbase + d - 1] = 6.0                                                    # key: its last entry (not a value entry)
        q = q.to(dt)
        c, cc = _ctx([q_len], [start], [0], "cuda:0"), _ctx([q_len], [start], [0], "cpu")
        hints = ops.hints_for([q_len], [total])
        out = ops.window_attention(q.cuda(), cache.cuda(), bt.cuda(), c.tok_req, c.positions, H, G, d, dv, page, 1.0, hints=hints, sink=not shared,
                                   shared_values=shared)
        got = out[-1].float().cpu().view(H, dv)[:, 1]
        assert bool((got > 4.0).all()), (loud, got)
        if q_len > 1 and loud == last:                     # the query before the last does not see the last position
            assert bool((out[-2].float().cpu().view(H, dv)[:, 1] < 1.0).all())
        _close(out, ref.window_attention(q, cache, bt, cc.tok_req, cc.positions, H, G, d, dv, page, 1.0, sink=not shared, shared_values=shared),
               dtype, f"loud key at {loud}", tol=2e-5 if dtype == "float32" else 2e-2)


# ---------------------------------------------------------------------------- the latents
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Q,R,n,dims,extra,page", [(28, 20, 8, 8, 3, 4), (96, 64, 32, 32, 4, 16), (10, 12, 24, 24, 1, 8), (300, 512, 64, 64, 16, 16),
                                                  (14, 6, 4, 2, 2, 4), (9, 7, 5, 4, 0, 8)])
def test_latent_norms_rotation_and_cache_write(ops, dtype, Q, R, n, dims, extra, page):
    g = torch.Generator().manual_seed(Q + R)
    dt, ref = DTYPES[dtype], TorchOps()
    q_lens, starts = [40, 1, 6], [0, 77, 13]
    cd, cc = _ctx(q_lens, starts, [0, 1, 2], "cuda:0"), _ctx(q_lens, starts, [0, 1, 2], "cpu")
    T = sum(q_lens)
    pages = sum(-(-(s + k) // page) for s, k in zip(starts, q_lens)) + 2
    bt, slots = _paged(g, q_lens, starts, page, pages, width=-(-78 // page) + 1)
    slots[5] = -1                                          # a row of a padded shape: nothing is stored for it
    proj = _rand(g, T, Q + R + n + extra, scale=2.0).to(dt)
    cache = _rand(g, pages, page * (R + n)).to(dt)
    wq, wkv, freq = 1 + 0.2 * _rand(g, Q), 1 + 0.2 * _rand(g, R), torch.rand(max(dims // 2, 1), generator=g)
    ca, cb = cache.clone().cuda(), cache.clone()
    qa = ops.latent_norm_store(proj.cuda(), Q, wq.cuda(), R, wkv.cuda(), n, 1e-5, cd.positions, freq.cuda(), dims, slots.cuda(), ca, page)
    qb = ref.latent_norm_store(proj, Q, wq, R, wkv, n, 1e-5, cc.positions, freq, dims, slots, cb, page)
    _close(qa, qb, dtype, "normed query latent")
    _close(ca, cb, dtype, "cache")
    # a layer that reads another's latent: only the query latent, whatever follows it in the row
    cu = cache.clone().cuda()
    qa = ops.latent_norm_store(proj.cuda(), Q, wq.cuda(), 0, None, 0, 1e-5, cd.positions, None, 0, None, None, page)
    _close(qa, qb, dtype, "query latent alone")
    assert torch.equal(cu.cpu(), cache)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,R,n,page", [(4, 64, 16, 16), (2, 128, 64, 8), (3, 20, 8, 4), (16, 512, 64, 16), (1, 33, 2, 16)])
def test_attention_over_the_latents_portions_as_products_and_single_tokens(ops, dtype, H, R, n, page):
    """Prompts from position 0, portions after a cached prefix (one crossing the query chunk), single tokens and a
    portion of two, in one step: in bfloat16 the portions go through the gathered rows and two products."""
    g = torch.Generator().manual_seed(H + R)
    dt, ref, d = DTYPES[dtype], TorchOps(), R + n
    q_lens, starts = [150, 1, 70, 1, 2, 600], [0, 90, 121, 0, 130, 37]
    cd, cc = _ctx(q_lens, starts, [0] * 6, "cuda:0"), _ctx(q_lens, starts, [0] * 6, "cpu")
    T = sum(q_lens)
    pages = sum(-(-(s + k) // page) for s, k in zip(starts, q_lens)) + 3
    bt, _ = _paged(g, q_lens, starts, page, pages, width=-(-640 // page) + 2)
    q = _rand(g, T, H * d, scale=1.5).to(dt)
    cache = _rand(g, pages, page * d, scale=0.7).to(dt)
    hints = ops.hints_for(q_lens, [s + k for s, k in zip(starts, q_lens)])
    hints.tok_req, hints.positions, hints.attn_splits = cd.tok_req, cd.positions, 1
    got = ops.latent_attention(q.cuda(), cache.cuda(), bt.cuda(), hints, H, R, n, page, d ** -0.5)
    want = ref.latent_attention(q, cache, bt, cc, H, R, n, page, d ** -0.5)
    _close(got, want, dtype, "weighted latents", tol=2e-5 if dtype == "float32" else 2e-2)
    old = ops.LATENT_QUERY_CHUNK
    try:            # chunks of 64 tokens: the cut falls inside every longer portion
        ops.LATENT_QUERY_CHUNK = 64
        got = ops.latent_attention(q.cuda(), cache.cuda(), bt.cuda(), hints, H, R, n, page, d ** -0.5)
    finally:
        ops.LATENT_QUERY_CHUNK = old
    _close(got, want, dtype, "chunks of 64", tol=2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,n,R,dims", [(3, 16, 8, 20, 8), (4, 64, 32, 64, 32), (1, 8, 24, 12, 24), (5, 6, 4, 6, 2), (2, 128, 64, 512, 64)])
def test_rotation_of_one_part_of_every_head(ops, dtype, H, d, n, R, dims):
    g = torch.Generator().manual_seed(H + d + n)
    dt, T = DTYPES[dtype], 23
    x = _rand(g, T, H * (d + n)).to(dt)
    pos = torch.randint(0, 5000, (T,), generator=g, dtype=torch.int32)
    freq = 1000.0 ** (-torch.arange(dims // 2, dtype=torch.float64) * 2 / dims)
    a, b = torch.zeros(T, H * (R + n), dtype=dt).cuda(), torch.zeros(T, H * (R + n), dtype=dt)
    ops.rotate_head_part(x.cuda(), d + n, d, a, R + n, R, H, n, pos.cuda(), freq.float().cuda(), dims)
    TorchOps().rotate_head_part(x, d + n, d, b, R + n, R, H, n, pos, freq.float(), dims)
    _close(a, b, dtype, "rotated parts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 7, 13, 40, 150])
@pytest.mark.parametrize("H,n_in,n_out,x_ld,out_ld", [(3, 16, 20, 24, 28), (4, 64, 64, 96, 96), (1, 8, 12, 32, 36), (5, 6, 6, 10, 10),
                                                     (2, 128, 512, 192, 576), (2, 512, 128, 512, 128), (6, 20, 24, 20, 24)])
def test_products_per_head_with_and_without_the_gate(ops, dtype, T, H, n_in, n_out, x_ld, out_ld):
    g = torch.Generator().manual_seed(T + H + n_in)
    dt, ref = DTYPES[dtype], TorchOps()
    x, w = _rand(g, T, H * x_ld).to(dt), _rand(g, H, n_out, n_in, scale=n_in ** -0.5).to(dt)
    gate = _rand(g, T, 11 + H).to(dt)
    for use_gate in (False, True):
        a, b = torch.zeros(T, H * out_ld, dtype=dt).cuda(), torch.zeros(T, H * out_ld, dtype=dt)
        kw = {"gate_column": 11} if use_gate else {}
        ops.head_linear(x.cuda(), x_ld, x_ld - n_in, w.cuda(), a, out_ld, 0, H, gate=gate.cuda() if use_gate else None, **kw)
        ref.head_linear(x, x_ld, x_ld - n_in, w, b, out_ld, 0, H, gate=gate if use_gate else None, **kw)
        _close(a, b, dtype, f"gate {use_gate}")


# ---------------------------------------------------------------------------- the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, dtype, cfg=None, seed=5):
        if (name, dtype) not in made:
            folder = tmp_path_factory.mktemp(f"sogalix_{name}_{dtype}")
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
    else:       # rounding alone: about 0.01 of the logits' spread in a row
        centred = (got.double().cpu() - ref) - (got.double().cpu() - ref).mean(-1, keepdim=True)
        rms = centred.pow(2).mean(-1).sqrt() / ref.std()
        assert rms.max() < 0.12 and rms.median() < 0.04 + 0.06 * (rms.numel() < 4), \
            f"{what}: median row {rms.median():.3f}, worst {rms.max():.3f} of the logits' spread"


# Wide enough for the tensor-core paths: attention heads of 64 and of 128 with the sink and a temperature that steps
# inside the prompts, latents of 64 and 128 entries (read by a second layer), delta heads of 64 channels.
WIDE = plain.config(300, 128, [
    plain.layer("latent_attention", plain.latent(4, 32, 16, 32, 64, 96, 0.14, 10000.0), plain.dense(192)),
    plain.layer("general_delta", plain.delta(2, 64), None),
    plain.layer("attention", plain.attention(4, 2, 64, 64, 0.125, q_temp=(0.5, 48)), plain.dense(64)),
    plain.layer("latent_attention", plain.latent(2, 64, 16, 64, 64, 48, 0.11, 10000.0, kv_from=0), None),
    plain.layer("attention", plain.attention(2, 1, 128, 128, 0.09), None),
    plain.layer("latent_attention", plain.latent(2, 64, 32, 48, 128, 80, 0.1, 500.0), plain.dense(96)),
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
        assert eng.cache.free_slots() == 4 and all(eng.cache.free_pages(g) == pages for g in eng._paged_groups())


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


def _random_config(seed, least_rank=1):
    """Sizes drawn freely: head sizes that are no power of two, one to three kv heads, ranks from 1 up, rotated parts of
    2 to 12 entries, temperatures that step every 1 to 40 positions, any order of layers, readers of earlier latents.
    (A latent of one entry is, after its unit norm, the sign of its input, which rounding to bfloat16 can turn over:
    the bfloat16 runs ask for ``least_rank`` 5.)"""
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72])
    layers, latents = [], []
    for i in range(rng.randint(2, 6)):
        kind = rng.choice(["general_delta", "attention", "latent_attention"])
        mlp = plain.dense(rng.choice([16, 40, 56])) if rng.random() < 0.6 else None
        if kind == "general_delta":
            mixer = plain.delta(rng.randint(1, 4), rng.choice([4, 6, 16, 20, 36]))
        elif kind == "attention":
            G = rng.randint(1, 3)
            mixer = plain.attention(G * rng.randint(1, 3), G, rng.choice([6, 12, 16, 40]), rng.choice([4, 12, 16, 24]), rng.uniform(0.15, 0.5),
                                    q_temp=(rng.uniform(0.1, 1.0), rng.randint(1, 40)) if rng.random() < 0.7 else None)
        else:
            heads, dim, vdim, q_rank = rng.randint(1, 4), rng.choice([4, 10, 16]), rng.choice([6, 8, 20]), max(least_rank, rng.choice([1, 9, 24]))
            if latents and rng.random() < 0.5:
                src = rng.choice(latents)
                m = layers[src]["mixer"]
                mixer = plain.latent(heads, dim, m["rot_dim"], vdim, m["kv_rank"], q_rank, rng.uniform(0.2, 0.5), m["rot"]["base"], kv_from=src)
            else:
                mixer = plain.latent(heads, dim, rng.choice([2, 4, 12]), vdim, max(least_rank, rng.choice([1, 5, 16, 33])), q_rank, rng.uniform(0.2, 0.5),
                                     rng.choice([10.0, 1000.0, 1e6]))
                latents.append(i)
        layers.append(plain.layer(kind, mixer, mlp))
    return plain.config(rng.choice([33, 101, 260]), width, layers, eps=rng.choice([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configurations(tmp_path, dtype, seed):
    cfg = _random_config(seed, least_rank=5 if dtype == "bfloat16" else 1)
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
    eng = _engine(folder, dtype, 16, 26)
    rows = [eng.step([StepEntry("a", toks[:3], [0, 1, 2])]).logits] + [eng.step([StepEntry("a", [t], [0])]).logits for t in toks[3:]]
    _assert_logits(torch.cat(rows), ref, dtype, "400 tokens, one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(folders, dtype):
    from pytriton_llama_b200 import LLM, EngineConfig, SamplingParams
    folder = folders("A", dtype)
    prompts = [random_tokens(n, 97, 40 + i) for i, n in enumerate([5, 23, 2, 14, 9, 31])]
    cfg = EngineConfig(dtype=dtype, page_size=4, max_gpu_num_blocks=60, max_seq_len=64, max_num_seqs=3, max_batched_tokens=16)
    outs = LLM(folder, cfg).generate(prompts, SamplingParams(temperature=0.0, max_gen_len=8))
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        logits = _reference(folder, {"x": p + o})["x"]
        slack = 1e-3 if dtype == "float32" else 0.05 * float(logits.std())
        for i, tok in enumerate(o):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - slack, (i, tok, int(row.argmax()))


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
