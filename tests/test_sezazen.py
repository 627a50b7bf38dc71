"""Sezazen on the host: configuration, run order, weight binding, and the engine's logic (cache per pass, portions,
mixed batches, pages and slots used again) with the plain torch stand-in kernels, against the plain implementation."""
from __future__ import annotations

import copy
import json

import pytest
import torch

import helpers as H
import plain_sezazen as plain
import sezazen_helpers as S
from reference_kernels import TorchReferenceKernels
from spite_b200.config import (ConfigError, JunctionCall, LayerCall, SezazenConfig, config_from_dict, load_config)
from spite_b200.engine import Engine
from spite_b200.engine.model import Model
from spite_b200.weights import WeightError, bind_tensors, random_checkpoint_tensors


def test_the_architecture_is_found_by_its_name():
    cfg = config_from_dict(S.CONFIG_P)
    assert isinstance(cfg, SezazenConfig)
    assert cfg.to_dict() == S.CONFIG_P                      # nothing is lost or invented on the way
    assert config_from_dict(dict(S.CONFIG_P, architectures=["Sezazen"])).width == 64


@pytest.mark.parametrize("name", list(S.CONFIGS))
def test_run_order_and_caches(name):
    raw = S.CONFIGS[name][0]
    plan = SezazenConfig.from_dict(raw).plan()
    layers = [c for c in plan.order if isinstance(c, LayerCall)]
    assert [c.layer for c in layers] == [i for i, _, _ in plain.layer_order(raw)]
    assert [c.cache for c in layers] == list(range(len(layers)))       # every run of a layer has its own cache
    # a junction stands before the first layer of every pass, with the pass number
    want, got = [], []
    for i, t, first in plain.layer_order(raw):
        if first:
            want.append(t)
    for k, c in enumerate(plan.order):
        if isinstance(c, JunctionCall):
            got.append(c.step)
            nxt = plan.order[k + 1]
            assert isinstance(nxt, LayerCall) and nxt.layer == raw["loop"]["start"]
    assert got == want
    assert plan.tie_word_embeddings and plan.position_table == raw["max_positions"]
    assert plan.embedding_scale == raw["embedding"]["scale"]


def test_every_constant_of_the_file_reaches_the_plan():
    raw = copy.deepcopy(S.CONFIG_P)
    raw["layers"][1]["mixer"].update(scale=0.77, vdim=20)
    raw["layers"][1]["mlp"]["router"]["top"] = 3
    raw["norm"]["eps"] = 3e-3
    plan = SezazenConfig.from_dict(raw).plan()
    mixer = plan.blocks[1].mixer.params
    assert mixer["softmax_scale"] == 0.77 and mixer["value_dim"] == 20 and mixer["head_dim"] == 32
    assert mixer["sink_logit"] == 0.0 and mixer["window"] == ("full", 0)
    assert plan.blocks[1].ffn.params["top_k"] == 3 and plan.blocks[1].ffn.params["activation"] == "relu2"
    assert plan.final_norm.params["eps"] == 3e-3
    assert "ffn" not in plan.blocks[2].parts                # mlp: null


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="recurrent"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda d: d["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_are_named(change, word):
    raw = copy.deepcopy(S.CONFIG_P)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        SezazenConfig.from_dict(raw)


def test_experts_stored_one_by_one_are_stacked_and_a_missing_one_is_listed():
    cfg = SezazenConfig.from_dict(S.CONFIG_P)
    tensors = random_checkpoint_tensors(cfg, seed=3, std=0.1)
    bound = bind_tensors(cfg, tensors)
    up = bound["layers.1.ffn.experts_up"]
    assert tuple(up.shape) == (6, 40, 64)
    for e in range(6):
        assert torch.equal(up[e], tensors[f"l1.mlp.e{e}.up"])
    assert torch.equal(bound["layers.3.ffn.experts_down"][4], tensors["l3.mlp.e4.down"])
    assert "layers.2.ffn_norm.weight" not in bound and "layers.3.ffn.shared_up_proj" not in bound
    tensors["l2.norm2"] = torch.ones(64)                  # the norm of a feed-forward the layer does not have: passed over
    assert set(bind_tensors(cfg, tensors)) == set(bound)
    del tensors["l1.mlp.e4.down"]
    tensors["l3.mlp.e1.up"] = tensors["l3.mlp.e1.up"][:, :10]
    tensors["l9.norm1"] = torch.ones(64)
    with pytest.raises(WeightError) as e:
        bind_tensors(cfg, tensors)
    assert [n for n, _ in e.value.missing] == ["l1.mlp.e4.down"]
    assert [n for n, _, _ in e.value.wrong_shape] == ["l3.mlp.e1.up"]
    assert e.value.unexpected == ["l9.norm1"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: S.write_model(tmp_path_factory.mktemp(f"sezazen_{n}"), n) for n in S.CONFIGS}


def host_engine(folder, tokens, page_size=16, max_requests=4):
    k = TorchReferenceKernels(torch.float32, "cpu")
    model = Model.from_folder(folder, dtype="float32", device="cpu", kernels=k)
    return Engine(model, cache_tokens=tokens, page_size=page_size, max_requests=max_requests)


def requests_for(folder, lens, seed):
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("name", list(S.CONFIGS))
def test_folder_round_trip_and_whole_prompts(folders, name):
    folder = folders[name]
    assert load_config(folder).to_dict() == S.CONFIGS[name][0]
    reqs = requests_for(folder, (37, 1, 20), 10)
    eng = host_engine(folder, 64)
    S.compare_with_plain(H.run_steps(eng, H.steps_whole(reqs)), folder, reqs, 2e-5)
    assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups


@pytest.mark.parametrize("name", ["P", "Q"])
def test_the_residual_stream_after_every_layer_run(folders, name):
    folder = folders[name]
    toks = requests_for(folder, (19,), 20)["r0"]
    cfg, tensors = S.folder_contents(str(folder))
    _, layers = plain.forward(cfg, tensors, toks, return_layers=True)
    eng = host_engine(folder, 64)
    seen = []
    eng.model.layer_tap = lambda i, h: seen.append((i, h.clone()))
    H.run_steps(eng, H.steps_whole({"a": toks}))
    assert [i for i, _ in seen] == list(range(layers.shape[0]))
    for i, h in seen:
        assert float((h - layers[i]).abs().max()) <= 2e-5 * float(layers[i].abs().max()), f"layer run {i}"


@pytest.mark.parametrize("name", list(S.CONFIGS))
def test_portions_decoding_and_mixed_batches_on_the_host(folders, name):
    """Token by token after a prompt, portions down to two tokens, and up to four live requests in a pool that
    forces pages and slots to be used again: the logits are those of the whole sequence."""
    folder = folders[name]
    reqs = requests_for(folder, (45, 9, 30, 3, 26, 17), 30)
    cuts = {"decoded": H.steps_last_decoded(reqs, 12), "portions": H.steps_portions(reqs, seed=2),
            "mixed": H.steps_mixed(reqs, {r: max(1, len(t) - 6) for r, t in reqs.items()}, seed=3)}
    for what, steps in cuts.items():
        eng = host_engine(folder, H.max_tokens_of(steps) if what == "mixed" else 64, page_size=16)
        S.compare_with_plain(H.run_steps(eng, steps), folder, reqs, 2e-5)
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what


def test_a_pass_of_the_loop_does_not_read_another_pass_cache(folders):
    """Every run of a looped layer keeps keys of its own: after a prompt, the caches of the passes differ."""
    folder = folders["P"]
    eng = host_engine(folder, 64)
    toks = requests_for(folder, (20,), 40)["r0"]
    H.run_steps(eng, [{"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": []}])
    first, second = eng.storage.layer_cache(1, True), eng.storage.layer_cache(3, True)     # layer 1 in pass 0 and in pass 1
    assert first.group == second.group and first.kv.data_ptr() != second.kv.data_ptr()
    assert not torch.equal(first.kv, second.kv)


def test_the_command_line_writes_a_random_model_folder(tmp_path):
    """`spite random` with a Sezazen configuration: experts one tensor each, as the design's files have them."""
    from spite_b200 import cli
    from spite_b200.weights import load_bound_tensors
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(S.CONFIG_Q))
    out = tmp_path / "model"
    assert cli.main(["random", "--config", str(cfg_file), "--out", str(out), "--seed", "4", "--std", "0.05"]) == 0
    config = load_config(out)
    assert isinstance(config, SezazenConfig) and config.loop.times == 3
    _, tensors = plain.load_folder(out)
    assert sorted(n for n in tensors if n.startswith("l0.mlp.e")) == sorted(f"l0.mlp.e{e}.{w}" for e in range(4) for w in ("up", "down"))
    assert tuple(tensors["loop.step"].shape) == (3, 128) and tuple(tensors["pos"].shape) == (1024, 128)
    bound = load_bound_tensors(out, config)
    assert tuple(bound["layers.0.ffn.experts_up"].shape) == (4, 64, 128)
    assert tuple(bound["junctions.0.in_proj"].shape) == (128, 256)
