"""The Sogalix decoder through the engine's host side, without a GPU: configuration, registry, weight names, cache
entries that several layers read, and -- with the plain PyTorch operator set of tests/torch_ops.py in place of the
CUDA kernels -- every way of cutting requests into steps against the whole-sequence plain implementation of
tests/plain_sogalix.py."""
import copy
import json

import pytest
import torch

import plain_sogalix as plain
import traces
from conftest import random_tokens
from torch_ops import TorchOps
from pytriton_llama_b200.config import ConfigError, EngineConfig, SogalixConfig, resolve_architecture
from pytriton_llama_b200.engine.engine import Engine, StepEntry

TOL = 2e-4      # float32 operators against float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg=None, seed=5, weights=None):
        if name not in made:
            folder = tmp_path_factory.mktemp(f"sogalix_{name}")
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
    cfg = SogalixConfig.from_dict(plain.TINY_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (97, 48, 1e-5)
    assert [L.type for L in cfg.layers] == ["latent_attention", "general_delta", "attention", "latent_attention"]
    assert cfg.layers[2].mlp is None and cfg.layers[0].mlp.ff == 40
    lat, att, dl = cfg.layers[3].mixer, cfg.layers[2].mixer, cfg.layers[1].mixer
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.q_rank, lat.scale, lat.kv_from) == (3, 16, 8, 24, 20, 28, 0.25, 0)
    assert (lat.rot.dims, lat.rot.base) == (8, 1000.0) and cfg.layers[0].mixer.kv_from is None
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.scale, att.q_temp.coef, att.q_temp.every) == (4, 2, 16, 24, 0.3, 0.4, 5)
    assert (dl.heads, dl.dim) == (3, 8)
    assert SogalixConfig.from_dict(cfg.to_dict()) == cfg
    assert SogalixConfig.from_dict(plain.TINY_B).layers[1].mixer.q_temp is None
    assert resolve_architecture(plain.TINY_A).name == "Sogalix"


@pytest.mark.parametrize("change", [
    lambda c: c.pop("vocab"), lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][2]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mlp"].update(kind="moe"), lambda c: c["norm"].update(eps=0), lambda c: c.update(layers=[]),
    lambda c: c["layers"][3]["mixer"].update(kv_from=1), lambda c: c["layers"][3]["mixer"].update(kv_from=3),
    lambda c: c["layers"][3]["mixer"].update(kv_rank=24), lambda c: c["layers"][3]["mixer"]["rot"].update(base=7.0),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), lambda c: c["layers"][2]["mixer"]["q_temp"].update(every=0),
    lambda c: c["layers"][1]["mixer"].pop("dim"), lambda c: c["layers"][0]["mixer"].pop("scale"),
])
def test_config_names_what_is_wrong(change):
    bad = copy.deepcopy(plain.TINY_A)
    change(bad)
    with pytest.raises(ConfigError):
        SogalixConfig.from_dict(bad)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_model_expects_the_checkpoint_names_and_shapes(name):
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY[name])
    model = DecoderModel(arch.spec_from_config(arch.config_from_dict(plain.TINY[name])), Runtime(torch.device("cpu"), torch.float32, None))
    want = plain.tensor_shapes(plain.TINY[name])
    got = {k: tuple(v.shape) for k, v in model.expected_tensors().items()}
    assert set(got) == set(want)
    for k, shape in got.items():        # (a negative size is one that only the checkpoint fixes)
        assert len(shape) == len(want[k]) and all(a < 0 or a == b for a, b in zip(shape, want[k])), k


def test_readers_of_a_latent_share_its_cache_entry_and_the_delta_rule_keeps_a_state():
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY_C)
    spec = arch.spec_from_config(arch.config_from_dict(plain.TINY_C))
    assert [(e.layer, e.cache, e.write) for e in spec.run_order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False), (4, 1, False)]
    needs = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32, None)).cache_entries()
    assert sorted(needs) == [0, 1, 2]
    assert (needs[0].kind, needs[0].kv_heads, needs[0].head_dim, needs[0].v_dim, needs[0].shared_values) == ("full", 1, 24, 8, False)
    # a position of the latent layers holds the latent and the rotated key part once, and no values
    assert (needs[1].kind, needs[1].kv_heads, needs[1].head_dim, needs[1].stored_v_dim, needs[1].v_dim) == ("full", 1, 6 + 4, 0, 6)
    assert needs[2].kind == "none" and needs[2].states == (("S", (4, 4, 4)),)


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from pytriton_llama_b200.weights import read_folder, write_random_model
    folder = write_random_model(tmp_path / "m", plain.TINY_A, seed=3, dtype=torch.float32, std=0.2)
    cfg = json.loads((folder / "config.json").read_text())
    W = read_folder(folder)
    toks = random_tokens(30, 97, 2)
    eng = _engine(folder, 8, 24)
    got = traces.replay(eng, traces.portions({"x": toks}))["x"]
    _close(got, plain.forward(cfg, W, toks))


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


def test_portions_of_two_tokens_and_single_tokens_from_the_first_position_on(folders):
    folder = folders("C")
    seqs = _seqs([21, 16], 50, 3)
    want = _reference(folder, seqs)
    for sizes in ((2,), (1, 2), (2, 1, 1, 3)):
        steps = traces.portions(seqs, sizes=sizes)
        got = traces.replay(_engine(folder, 4, 30), steps)
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
    assert eng.cache.free_slots() == 3 and all(eng.cache.free_pages(g) == pages for g, grp in enumerate(eng.cache.groups) if grp.paged)


def test_a_freed_state_slot_starts_from_zero_for_the_next_request(folders):
    folder = folders("B")
    seqs = _seqs([35, 12], 70, 9)
    want = _reference(folder, seqs)
    eng = _engine(folder, 8, 20, slots=1)             # one slot: the second request walks over what the first left in it
    for rid, toks in seqs.items():
        head = eng.step([StepEntry(rid, toks[:5], list(range(5)))]).logits
        tail = eng.step([StepEntry(rid, toks[5:], list(range(len(toks) - 5)))]).logits
        eng.finish(rid)
        _close(torch.cat([head, tail]), want[rid])


def test_an_unequal_batch_equals_each_request_alone(folders):
    folder = folders("C")
    seqs = _seqs([33, 2, 14], 50, 8)
    eng = _engine(folder, 8, 40)
    together = eng.step([StepEntry(r, s, list(range(len(s)))) for r, s in seqs.items()]).logits
    eng.finish_all()
    at = 0
    for r, s in seqs.items():
        alone = eng.step([StepEntry(r, s, list(range(len(s))))]).logits
        eng.finish(r)
        assert torch.allclose(together[at:at + len(s)], alone, atol=1e-5, rtol=1e-5)
        at += len(s)


def test_long_decoding_token_by_token(folders):
    folder = folders("A")
    toks = random_tokens(150, 97, 13)
    want = _reference(folder, {"x": toks})["x"]
    eng = _engine(folder, 4, 60)
    rows = [eng.step([StepEntry("x", [t], [0])]).logits[0] for t in toks]
    _close(torch.stack(rows), want)


# ---------------------------------------------------------------------------- each mechanism alone
def _one_layer(kind, mixer, mlp, width=32, eps=1e-5):
    return plain.config(41, width, [plain.layer(kind, mixer, mlp)], eps=eps)


def _two_latent_layers(first, second):
    return plain.config(41, 32, [plain.layer("latent_attention", first, None), plain.layer("latent_attention", second, None)])


ALONE = {
    "delta": _one_layer("general_delta", plain.delta(2, 12), None),
    "delta_one_channel_heads": _one_layer("general_delta", plain.delta(5, 1), None),
    "delta_wide": _one_layer("general_delta", plain.delta(1, 72), None, eps=1e-3),
    "sink": _one_layer("attention", plain.attention(2, 1, 8, 8, 0.4), None),
    "sink_value_sizes": _one_layer("attention", plain.attention(4, 4, 6, 10, 0.5), None),
    "temperature": _one_layer("attention", plain.attention(2, 2, 8, 4, 0.4, q_temp=(0.8, 7)), None),
    "temperature_every_1": _one_layer("attention", plain.attention(3, 1, 8, 8, 0.3, q_temp=(0.25, 1)), None),
    "latent": _one_layer("latent_attention", plain.latent(2, 8, 4, 6, 10, 12, 0.35, 100.0), None),
    "latent_one_head_rank_1": _one_layer("latent_attention", plain.latent(1, 4, 2, 4, 1, 1, 0.5, 10.0), None),
    "latent_reader": _two_latent_layers(plain.latent(2, 8, 4, 6, 10, 12, 0.35, 100.0), plain.latent(3, 6, 4, 8, 10, 7, 0.5, 100.0, kv_from=0)),
    "dense": _one_layer("general_delta", plain.delta(1, 8), plain.dense(24)),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_in_a_one_layer_model(folders, name):
    folder = folders("alone_" + name, ALONE[name], seed=3)
    seqs = _seqs([27, 12], 41, 6)
    want = _reference(folder, seqs)
    for steps in (traces.whole(seqs), traces.portions(seqs, sizes=(3, 2, 9, 2)), traces.prefill_then_decode(seqs, 9)):
        got = traces.replay(_engine(folder, 4, 30), steps)
        for rid in seqs:
            _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])


# ---------------------------------------------------------------------------- weights made so that a fault would show
def _loud(folder_factory, name, cfg, change, seed=11):
    """A model folder whose random weights ``change`` has edited (a dictionary name -> float32 tensor)."""
    W = plain.random_weights(cfg, seed)
    change(W)
    return folder_factory(name, cfg, seed, weights=W)


def test_the_temperature_steps_where_it_should(folders):
    cfg = _one_layer("attention", plain.attention(2, 2, 8, 4, 0.4, q_temp=(1.5, 6)), None)

    def sharpen(W):
        W["l0.mix.q"] *= 6.0            # scores large enough that the factor at the step moves the logits
    folder = _loud(folders, "loud_temp", cfg, sharpen)
    toks = random_tokens(20, 41, 5)
    want = _reference(folder, {"x": toks})["x"]
    # the plain implementation with the step one position late differs where the step lies (p + 1 = 6 -> p = 5)
    late = copy.deepcopy(cfg)
    late["layers"][0]["mixer"]["q_temp"]["every"] = 7
    wrong = plain.forward(late, _weights(folder), toks)
    assert (wrong[5] - want[5]).abs().max() > 100 * TOL and (wrong[4] - want[4]).abs().max() < 1e-9
    for steps in (traces.whole({"x": toks}), traces.prefill_then_decode({"x": toks}, 17), traces.portions({"x": toks}, sizes=(5, 2, 1))):
        got = traces.replay(_engine(folder, 4, 12), steps)["x"]
        _close(got, want[traces.wanted_positions(steps, "x")])


def _weights(folder):
    from pytriton_llama_b200.weights import read_folder
    return read_folder(folder)


def test_the_sink_takes_its_share_at_every_position(folders):
    cfg = _one_layer("attention", plain.attention(2, 1, 8, 8, 0.4), None)

    def quiet(W):
        W["l0.mix.q"] *= 0.0            # every score is 0: n keys and the sink share 1 / (n + 1) each
        W["l0.mix.v"] = W["l0.mix.v"] * 0 + 1.0 / 32
    folder = _loud(folders, "loud_sink", cfg, quiet)
    toks = random_tokens(40, 41, 8)
    want = _reference(folder, {"x": toks})["x"]
    for steps in (traces.whole({"x": toks}), traces.prefill_then_decode({"x": toks}, 30)):
        got = traces.replay(_engine(folder, 8, 12), steps)["x"]
        _close(got, want[traces.wanted_positions(steps, "x")], tol=2e-5)


def test_a_key_far_back_is_found_by_attention_and_by_the_delta_state(folders):
    cfg = plain.config(41, 32, [plain.layer("attention", plain.attention(2, 1, 8, 8, 1.0), None),
                                plain.layer("general_delta", plain.delta(2, 8), None),
                                plain.layer("latent_attention", plain.latent(2, 8, 4, 6, 10, 12, 1.0, 100.0), None)])

    def loud(W):
        for name in ("l0.mix.q", "l0.mix.k", "l2.mix.uq", "l2.mix.uk"):
            W[name] *= 3.0              # softmaxes with a few keys that stand out, wherever they lie
        W["l1.mix.w0"] -= 6.0           # slow decay: what was written long ago is still in the state
    folder = _loud(folders, "loud_far", cfg, loud)
    toks = random_tokens(230, 41, 2)
    want = _reference(folder, {"x": toks})["x"]
    for page, steps in ((16, traces.prefill_then_decode({"x": toks}, 40)), (4, traces.portions({"x": toks}, sizes=(63, 2, 64, 1, 33)))):
        got = traces.replay(_engine(folder, page, 300 // page, max_seq_len=256), steps)["x"]
        _close(got, want[traces.wanted_positions(steps, "x")], tol=5e-4)


def test_a_reader_sees_the_other_layers_rotated_key_part(folders):
    cfg = _two_latent_layers(plain.latent(2, 2, 8, 6, 4, 12, 0.6, 30.0), plain.latent(3, 2, 8, 8, 4, 7, 0.6, 30.0, kv_from=0))

    def loud(W):
        W["l0.mix.dkv"][4:] *= 4.0      # the rotated key part dominates the scores of both layers
        W["l1.mix.uq"] *= 2.0
    folder = _loud(folders, "loud_reader", cfg, loud)
    seqs = _seqs([37, 20], 41, 4)
    want = _reference(folder, seqs)
    for steps in (traces.whole(seqs), traces.mixed(seqs, live=2)):
        got = traces.replay(_engine(folder, 4, 24), steps)
        for rid in seqs:
            _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])


# ---------------------------------------------------------------------------- generation through the public entry point
def test_greedy_generation_through_the_scheduler_matches_the_plain_argmax(folders):
    from pytriton_llama_b200 import LLM, SamplingParams
    folder = folders("B")
    W = _weights(folder)
    prompts = list(_seqs([9, 21, 3], 70, 17).values())
    llm = LLM(folder, EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=40, max_seq_len=64, max_num_seqs=2,
                                   max_batched_tokens=8, compiled_model=False), device="cpu", ops=TorchOps())
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_gen_len=7))
    for p, out in zip(prompts, got):
        logits = plain.forward(plain.TINY_B, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 1e-4, (i, tok, int(row.argmax()))
