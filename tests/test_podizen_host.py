"""The Podizen decoder through the engine's host side, without a GPU: configuration, registry, weight names, the
cache's pages of block means, and -- with the plain PyTorch operator set of tests/torch_ops.py in place of the CUDA
kernels -- every way of cutting requests into steps against the whole-sequence plain implementation of
tests/plain_podizen.py."""
import copy
import json

import pytest
import torch

import plain_podizen as plain
import traces
from conftest import random_tokens
from torch_ops import TorchOps
from pytriton_llama_b200.cache.manager import CacheManager
from pytriton_llama_b200.config import ConfigError, EngineConfig, PodizenConfig, resolve_architecture
from pytriton_llama_b200.engine.engine import Engine, StepEntry
from pytriton_llama_b200.parts.base import CacheNeed

TOL = 2e-4      # float32 operators against float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg=None, seed=5, weights=None):
        if name not in made:
            folder = tmp_path_factory.mktemp(f"podizen_{name}")
            plain.write_model(folder, cfg or plain.TINY[name], seed, weights=weights)
            made[name] = folder
        return made[name]
    return get


def _engine(folder, page, pages, max_seq_len=256, slots=4):
    cfg = EngineConfig(dtype="float32", page_size=page, max_gpu_num_blocks=pages, max_seq_len=max_seq_len, max_num_seqs=slots)
    return Engine(folder, cfg, device="cpu", ops=TorchOps())


def _reference(folder, seqs):
    from pytriton_llama_b200.weights import read_folder
    cfg = json.loads((folder / "config.json").read_text())
    W = read_folder(folder)
    return {r: plain.forward(cfg, W, s) for r, s in seqs.items()}


def _seqs(lengths, vocab, seed):
    return {f"r{i}": random_tokens(n, vocab, seed * 100 + i) for i, n in enumerate(lengths)}


def _close(got, want, tol=TOL):
    err = (got.double() - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), err


# ---------------------------------------------------------------------------- configuration and names
def test_config_reads_every_key_and_round_trips():
    cfg = PodizenConfig.from_dict(plain.TINY_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (97, 48, 1e-5)
    assert [L.type for L in cfg.layers] == ["parallel", "attention", "parallel", "attention"] and cfg.layers[2].mlp is None
    left, right = cfg.layers[0].mixer.left, cfg.layers[0].mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.window, left.pool) == (4, 2, 16, 24, 0.3, 11, 5)
    assert (left.rot.dims, left.rot.base, right.rot.dims, right.decay) == (8, 1000.0, 8, (0.9, 0.97, 0.995))
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window) == (4, 1, 16, 8, 9)
    m = cfg.layers[0].mlp
    assert (m.ff, m.experts, m.top, m.groups, m.keep, m.shared_ff) == (24, 6, 2, 2, 1, 16)
    assert (cfg.layers[1].mlp.groups, cfg.layers[1].mlp.keep, cfg.layers[1].mlp.shared_ff) == (1, 1, 0)
    assert PodizenConfig.from_dict(cfg.to_dict()) == cfg
    for other in (plain.TINY_B, plain.TINY_C):
        c = PodizenConfig.from_dict(other)
        assert PodizenConfig.from_dict(c.to_dict()) == c
    assert PodizenConfig.from_dict(plain.TINY_C).layers[1].mixer.window == 0
    assert resolve_architecture(plain.TINY_A).name == "Podizen"


@pytest.mark.parametrize("change", [
    lambda c: c.pop("vocab"), lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][3]["mixer"].update(heads=5),
    lambda c: c["layers"][0]["mlp"].update(kind="dense"), lambda c: c["norm"].update(eps=0), lambda c: c.update(layers=[]),
    lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 1.5, 0.5]),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=5), lambda c: c["layers"][0]["mlp"]["router"].update(top=4),
    lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=3),
    lambda c: c["layers"][0]["mixer"].pop("right"),
])
def test_config_names_what_is_wrong(change):
    bad = copy.deepcopy(plain.TINY_A)
    change(bad)
    with pytest.raises(ConfigError):
        PodizenConfig.from_dict(bad)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_model_expects_the_checkpoint_names_and_shapes(name):
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY[name])
    model = DecoderModel(arch.spec_from_config(arch.config_from_dict(plain.TINY[name])), Runtime(torch.device("cpu"), torch.float32, None))
    assert {k: tuple(v.shape) for k, v in model.expected_tensors().items()} == plain.tensor_shapes(plain.TINY[name])


def test_cache_needs_of_the_layers():
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY_A)
    needs = DecoderModel(arch.spec_from_config(arch.config_from_dict(plain.TINY_A)), Runtime(torch.device("cpu"), torch.float32, None)).cache_entries()
    assert (needs[0].kind, needs[0].window, needs[0].pool_block, needs[0].v_dim, needs[0].kv_heads) == ("window", 11, 5, 24, 2)
    assert needs[0].states == (("right.S", (3, 8, 12)),)
    assert (needs[1].kind, needs[1].window, needs[1].pool_block, needs[1].states) == ("window", 9, 0, ())
    assert (needs[2].window, needs[2].pool_block) == (7, 7)        # blocks longer than the window: their keys are held until they are whole
    arch = resolve_architecture(plain.TINY_C)
    needs = DecoderModel(arch.spec_from_config(arch.config_from_dict(plain.TINY_C)), Runtime(torch.device("cpu"), torch.float32, None)).cache_entries()
    assert (needs[0].kind, needs[0].pool_block, needs[1].kind, needs[2].kind) == ("window", 0, "full", "full")


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from pytriton_llama_b200.weights import read_folder, write_random_model
    folder = write_random_model(tmp_path / "m", plain.TINY_A, seed=3, dtype=torch.float32, std=0.2)
    cfg = json.loads((folder / "config.json").read_text())
    W = read_folder(folder)
    toks = random_tokens(30, 97, 2)
    got = traces.replay(_engine(folder, 8, 24), traces.portions({"x": toks}))["x"]
    _close(got, plain.forward(cfg, W, toks))


# ---------------------------------------------------------------------------- the cache: pages of block means
def test_pages_of_block_means_grow_with_whole_blocks_and_come_back_at_the_end():
    need = CacheNeed(kind="window", kv_heads=1, head_dim=8, window=10, pool_block=3)
    cm = CacheManager({0: need}, page_size=4, num_pages=12, max_requests=2, max_seq_len=200, device="cpu", dtype=torch.float32)
    assert [g.need.kind for g in cm.groups] == ["window", "summary"] and cm.entry_summary_group == {0: 1}
    summary_pages = cm.groups[1].pool.num_pages
    cm.admit("a")
    slots = cm.append("a", 14)
    # positions 2, 5, 8, 11 complete blocks 0..3: the first page of means, entries 0..3
    page0 = cm.block_table("a", 1)[0]
    assert slots[1] == [page0 * 4 + (p + 1) // 3 - 1 if p % 3 == 2 else -1 for p in range(14)]
    assert len(cm.block_table("a", 1)) == 1
    assert cm.append("a", 1)[1] == [cm.block_table("a", 1)[1] * 4]          # position 14 completes block 4: a second page
    for _ in range(40):
        cm.append("a", 1)
        cm.check_invariants()
    assert all(p >= 0 for p in cm.block_table("a", 1)) and len(cm.block_table("a", 1)) == -(-(55 // 3) // 4)
    assert sum(p >= 0 for p in cm.block_table("a", 0)) <= 4                 # the window's pages went back meanwhile
    assert cm.pages_needed("a", 2) == {0: 1, 1: 1 if (57 // 3) > 4 * len(cm.block_table("a", 1)) else 0}
    cm.release("a")
    assert cm.free_pages(0) == 12 and cm.free_pages(1) == summary_pages
    cm.check_invariants()


def test_a_request_that_does_not_fit_the_pages_of_block_means_is_refused_whole():
    need = CacheNeed(kind="window", kv_heads=1, head_dim=8, window=4, pool_block=2)
    cm = CacheManager({0: need}, page_size=2, num_pages=4, max_requests=1, max_seq_len=64, device="cpu", dtype=torch.float32)
    pages = cm.groups[1].pool.num_pages
    assert pages == 3                                   # 4 pages of tokens over blocks of 2, one more for the request
    assert cm.can_append([(None, 4 * pages)]) is False or cm.groups[0].pool.num_pages * 2 < 4 * pages
    cm.admit("a")
    cm.append("a", 8)
    for _ in range(4):                                  # 12 tokens: 6 means, 3 pages
        cm.append("a", 1)
    assert cm.free_pages(1) == 0
    assert not cm.can_append([("a", 2)])
    cm.release("a")
    assert cm.free_pages(1) == pages


# ---------------------------------------------------------------------------- every cut equals the whole sequence
@pytest.mark.parametrize("name,page", [("A", 4), ("A", 16), ("B", 8), ("C", 4)])
def test_every_cut_of_the_requests_matches_the_plain_implementation(folders, name, page):
    folder = folders(name)
    vocab = plain.TINY[name]["vocab"]
    seqs = _seqs([41, 1, 23, 58, 9], vocab, 21)
    want = _reference(folder, seqs)
    for steps in (traces.whole(seqs), traces.prefill_then_decode(seqs, 12), traces.portions(seqs), traces.mixed(seqs)):
        eng = _engine(folder, page, max(40, traces.max_live_tokens(steps, page) // page + 8))
        got = traces.replay(eng, steps)
        for rid in seqs:
            _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])


def test_six_requests_through_three_slots_and_few_pages_reuse_what_was_freed(folders):
    folder = folders("A")
    seqs = _seqs([30, 17, 44, 5, 26, 38], 97, 4)
    want = _reference(folder, seqs)
    steps = traces.mixed(seqs, live=3)
    pages = traces.max_live_tokens(steps, 4) // 4 + 2
    eng = _engine(folder, 4, pages, slots=3)
    got = traces.replay(eng, steps)
    for rid in seqs:
        _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])
    assert eng.cache.free_slots() == 3
    assert all(eng.cache.free_pages(g) == grp.pool.num_pages for g, grp in enumerate(eng.cache.groups) if grp.paged)


def test_an_unequal_batch_equals_each_request_alone(folders):
    folder = folders("B")
    seqs = _seqs([33, 2, 14], 70, 8)
    eng = _engine(folder, 8, 40)
    together = eng.step([StepEntry(r, s, list(range(len(s)))) for r, s in seqs.items()]).logits
    eng.finish_all()
    at = 0
    for r, s in seqs.items():
        alone = eng.step([StepEntry(r, s, list(range(len(s))))]).logits
        eng.finish(r)
        assert torch.allclose(together[at:at + len(s)], alone, atol=1e-5, rtol=1e-5)
        at += len(s)


def test_long_decoding_token_by_token_past_windows_and_blocks(folders):
    folder = folders("A")
    toks = random_tokens(150, 97, 13)
    want = _reference(folder, {"x": toks})["x"]
    eng = _engine(folder, 4, 60)
    rows = [eng.step([StepEntry("x", [t], [0])]).logits[0] for t in toks]
    _close(torch.stack(rows), want)


# ---------------------------------------------------------------------------- each mechanism alone
def _one_layer(kind, mixer, mlp, width=32):
    return plain.config(41, width, [plain.layer(kind, mixer, mlp)])


_RET = plain.retention(1, 8, 8, (0.9,))
_ATT = plain.gated_attention(2, 1, 8, 8, 0.4, size=6)
ALONE = {
    "bias_gate_window": _one_layer("attention", plain.gated_attention(4, 2, 8, 12, 0.4, size=6), None),
    "bias_gate_everything": _one_layer("attention", plain.gated_attention(3, 3, 12, 8, 0.3), None),
    "window_one": _one_layer("attention", plain.gated_attention(2, 1, 8, 8, 0.4, size=1), None),
    "pooled": _one_layer("parallel", plain.parallel(plain.pooled_attention(2, 1, 8, 12, 0.4, size=5, pool=3, rot=plain.rotation(4, 20.0)), _RET), None),
    "pooled_long_blocks": _one_layer("parallel", plain.parallel(plain.pooled_attention(2, 2, 8, 8, 0.4, size=3, pool=9), _RET), None),
    "pooled_window_one": _one_layer("parallel", plain.parallel(plain.pooled_attention(1, 1, 8, 8, 0.4, size=1, pool=2, rot=plain.rotation(8, 5.0)), _RET), None),
    "retention": _one_layer("parallel", plain.parallel(plain.pooled_attention(1, 1, 8, 8, 0.4, size=4),
                                                       plain.retention(3, 12, 20, (0.5, 0.95, 1.0), rot=plain.rotation(6, 30.0))), None),
    "moe_top1_groups": _one_layer("attention", _ATT, plain.moe(12, 8, 1, groups=4, keep=1)),
    "moe_top3_groups_shared": _one_layer("attention", _ATT, plain.moe(12, 9, 3, groups=3, keep=2, shared=20)),
    "moe_no_groups": _one_layer("attention", _ATT, plain.moe(12, 5, 2)),
    "moe_all_chosen": _one_layer("attention", _ATT, plain.moe(12, 4, 4, groups=2, keep=2, shared=4)),
    "odd_width": _one_layer("attention", _ATT, plain.moe(10, 3, 2), width=27),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_in_a_one_layer_model(folders, name):
    folder = folders("alone_" + name, ALONE[name], seed=3)
    seqs = _seqs([27, 12], 41, 6)
    want = _reference(folder, seqs)
    for steps in (traces.whole(seqs), traces.portions(seqs, sizes=(3, 2, 9, 2))):
        got = traces.replay(_engine(folder, 4, 30), steps)
        for rid in seqs:
            _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])


def test_depth_coefficients_weigh_every_earlier_result(folders):
    """Three layers whose coefficients single out one earlier result each: a result that is dropped or taken from the
    wrong layer changes the logits by far more than the tolerance."""
    cfg = plain.config(41, 32, [plain.layer("attention", _ATT, None), plain.layer("attention", _ATT, plain.moe(8, 2, 1)),
                                plain.layer("attention", _ATT, None)])
    W = plain.random_weights(cfg, 9)
    W["l0.dwa"] = torch.tensor([0.0, 1.0])
    W["l1.dwa"] = torch.tensor([1.5, -0.5, 0.25])
    W["l2.dwa"] = torch.tensor([0.0, 2.0, 0.0, 0.5])
    folder = folders("depth", cfg, weights=W)
    toks = random_tokens(19, 41, 3)
    want = plain.forward(cfg, W, toks)
    dropped = dict(W)
    dropped["l2.dwa"] = torch.tensor([0.0, 0.0, 0.0, 0.5])
    assert (plain.forward(cfg, dropped, toks) - want).abs().max() > 0.1
    got = traces.replay(_engine(folder, 4, 20), traces.portions({"x": toks}, sizes=(4, 2, 6)))["x"]
    _close(got, want)


# ---------------------------------------------------------------------------- edges that random weights would hide
def _spiked(cfg, seed, prefix, normed=False):
    """Weights such that the key of token 1 dominates the scores of every query that sees it, in the softmax mixer
    whose tensors start with ``prefix``.  Token 1's embedding lies along stream entry 0 alone; every other token has
    0.8 there and 1.0 at entry 1.  Queries and keys read entry 0 into entry 4 of every head (outside what the tests
    rotate) and nothing else, so a score is the product of the two tokens' entries 0.  Where heads are normed
    (``normed``) keys also read entry 1 into entry 5: a key's size is lost in the norm, its direction is not, and
    only token 1 has nothing at entry 1."""
    W = plain.random_weights(cfg, seed)
    m = cfg["layers"][0]["mixer"]
    m = m["left"] if "left" in m else m
    d = m["dim"]
    W["embed"][:, 0] = 0.8
    W["embed"][:, 1] = 1.0
    W["embed"][1] = 0.0
    W["embed"][1, 0] = 6.0
    W["l0.norm1"] = torch.ones_like(W["l0.norm1"])
    for name, heads in (("q", m["heads"]), ("k", m["kv_heads"])):
        w = torch.zeros_like(W[prefix + name])
        for h in range(heads):
            w[h * d + 4, 0] = 2.0
            if normed and name == "k":
                w[h * d + 5, 1] = 4.0
        W[prefix + name] = w
    if normed:
        W[prefix + "q.norm"] = torch.full((d,), 3.0)
        W[prefix + "k.norm"] = torch.full((d,), 3.0)
    return W


def _edge_tokens(n, spike):
    toks = [2 + (7 * i) % 30 for i in range(n)]
    toks[spike] = 1
    return toks


@pytest.mark.parametrize("window", [5, 8])
def test_a_key_just_inside_and_just_outside_the_window_in_prompt_and_decoding(folders, window):
    cfg = _one_layer("attention", plain.gated_attention(2, 1, 8, 8, 1.0, size=window), None)
    spike = 9
    W = _spiked(cfg, 4, "l0.mix.")
    toks = _edge_tokens(30, spike)
    want = plain.forward(cfg, W, toks)
    # the logits at the last position that sees the spike and at the first that does not differ by far more than the
    # tolerance from what they would be with a window one longer or one shorter
    for delta in (-1, 1):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["mask"]["size"] = window + delta
        moved = plain.forward(other, W, toks)
        edge = spike + window - 1 + (1 if delta > 0 else 0)
        assert (moved[edge] - want[edge]).abs().max() > 50 * TOL * want.abs().max(), (delta, (moved[edge] - want[edge]).abs().max())
    folder = folders(f"edge_window_{window}", cfg, weights=W)
    for steps in (traces.whole({"x": toks}), traces.prefill_then_decode({"x": toks}, 30 - spike - 2),
                  traces.portions({"x": toks}, sizes=(2, 3, 2, 5))):
        got = traces.replay(_engine(folder, 4, 20), steps)["x"]
        _close(got, want[traces.wanted_positions(steps, "x")])


@pytest.mark.parametrize("window,pool", [(4, 3), (3, 5), (6, 2)])
def test_a_block_just_seen_and_not_yet_seen_in_prompt_and_decoding(folders, window, pool):
    left = plain.pooled_attention(2, 1, 8, 8, 1.0, size=window, pool=pool)
    cfg = _one_layer("parallel", plain.parallel(left, _RET), None)
    spike = 2 * pool + 1                      # inside the third block
    W = _spiked(cfg, 6, "l0.mix.left.", normed=True)
    n = 3 * pool + window + 8
    toks = _edge_tokens(n, spike)
    want = plain.forward(cfg, W, toks)
    first_seen = 3 * pool - 1 + window        # the first query that sees the third block's mean
    for changed in ({"pool": pool + 1}, {"size": window + 1}, {"size": window - 1} if window > 1 else {"pool": pool - 1}):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"].update(changed)
        moved = plain.forward(other, W, toks)
        assert (moved[first_seen - 1:first_seen + 1] - want[first_seen - 1:first_seen + 1]).abs().max() > 20 * TOL * want.abs().max(), changed
    folder = folders(f"edge_pool_{window}_{pool}", cfg, weights=W)
    for page in (4, 16):
        for steps in (traces.whole({"x": toks}), traces.prefill_then_decode({"x": toks}, n - spike - 2),
                      traces.portions({"x": toks}, sizes=(2, 3, 2, 5))):
            got = traces.replay(_engine(folder, page, 20), steps)["x"]
            _close(got, want[traces.wanted_positions(steps, "x")])


def test_the_first_tokens_and_a_far_key_among_hundreds(folders):
    """A retention head that never forgets carries the first token to position 400; the pooled blocks carry a spiked
    key from the start of the sequence into a window that left it long ago."""
    left = plain.pooled_attention(2, 1, 8, 8, 1.0, size=16, pool=4, rot=plain.rotation(4, 100.0))
    cfg = _one_layer("parallel", plain.parallel(left, plain.retention(2, 8, 8, (1.0, 0.99))), None)
    W = _spiked(cfg, 8, "l0.mix.left.", normed=True)
    toks = _edge_tokens(400, 5)
    want = plain.forward(cfg, W, toks)
    without = list(toks)
    without[5] = 3
    assert (plain.forward(cfg, W, without)[-1] - want[-1]).abs().max() > 50 * TOL * want.abs().max()
    folder = folders("far", cfg, weights=W)
    steps = traces.portions({"x": toks[:360]}, sizes=(32, 17, 64, 2))
    steps[-1]["end"] = []
    steps += [{"step": len(steps) + i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks[360:])]
    eng = _engine(folder, 16, 12, max_seq_len=512)          # 12 pages of 16: the window's pages must come back on the way
    got = traces.replay(eng, steps)["x"]
    _close(got, want[traces.wanted_positions(steps, "x")])


def test_the_plain_router_keeps_the_best_groups():
    s = torch.tensor([0.05, 0.30, 0.10, 0.04, 0.26, 0.25], dtype=torch.float64)
    chosen, w = plain.route(s, 2, 3, 1)            # groups {0,1}, {2,3}, {4,5}: the first has the largest score
    assert sorted(chosen.tolist()) == [0, 1] and torch.allclose(w.sum(), torch.tensor(1.0, dtype=torch.float64))
    chosen, _ = plain.route(s, 2, 3, 2)            # two groups kept: experts 1 and 4
    assert sorted(chosen.tolist()) == [1, 4]
    chosen, _ = plain.route(s, 2, 1, 1)
    assert sorted(chosen.tolist()) == [1, 4]


# ---------------------------------------------------------------------------- generation through the public entry point
def test_greedy_generation_through_the_scheduler_matches_the_plain_argmax(folders):
    from pytriton_llama_b200 import LLM, SamplingParams
    folder = folders("B")
    from pytriton_llama_b200.weights import read_folder
    W = read_folder(folder)
    prompts = list(_seqs([9, 21, 3], 70, 17).values())
    llm = LLM(folder, EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=40, max_seq_len=64, max_num_seqs=2,
                                   max_batched_tokens=8, compiled_model=False), device="cpu", ops=TorchOps())
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_gen_len=7))
    for p, out in zip(prompts, got):
        logits = plain.forward(plain.TINY_B, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 1e-4, (i, tok, int(row.argmax()))
