"""Mibezen on the host: configuration, weight binding, the plain implementation's mechanisms against loops written
here, and the engine's logic (latent cache of one plane, chunks, blended values kept for later layers, portions,
mixed batches, pages and slots used again) with the plain torch stand-in kernels against the plain implementation."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import helpers as H
import mibezen_helpers as Z
import plain_mibezen as plain
from reference_kernels import TorchReferenceKernels
from spite_b200.config import ConfigError, MibezenConfig, config_from_dict, load_config
from spite_b200.engine import Engine
from spite_b200.engine.model import Model
from spite_b200.parts.position import yarn_frequencies
from spite_b200.weights import WeightError, bind_tensors, random_checkpoint_tensors


# ---------------------------------------------------------------------------- configuration
def test_the_architecture_is_found_by_its_name():
    cfg = config_from_dict(Z.CONFIG_U)
    assert isinstance(cfg, MibezenConfig)
    assert cfg.to_dict() == Z.CONFIG_U                      # nothing is lost or invented on the way
    assert config_from_dict(dict(Z.CONFIG_W, architectures=["Mibezen"])).width == 100
    assert MibezenConfig.from_dict(Z.CONFIG_W).to_dict() == Z.CONFIG_W and "logit_softcap" not in Z.CONFIG_W


def test_every_constant_of_the_file_reaches_the_plan():
    raw = copy.deepcopy(Z.CONFIG_U)
    raw["layers"][0]["mixer"].update(scale=0.77, vdim=20, kv_rank=36)
    raw["layers"][0]["mixer"]["rot"]["scaling"]["factor"] = 5.0
    raw["layers"][1]["mixer"]["mask"]["size"] = 31
    raw["layers"][3]["mlp"]["router"]["top"] = 4
    raw["norm"]["eps"] = 3e-3
    raw["logit_softcap"] = 11.0
    plan = MibezenConfig.from_dict(raw).plan()
    lat = plan.blocks[0].mixer.params
    assert (lat["softmax_scale"], lat["value_dim"], lat["kv_rank"], lat["q_rank"], lat["head_dim"], lat["rotary_dim"]) == \
        (0.77, 20, 36, 40, 16, 8)
    assert lat["norm_eps"] == 3e-3 and lat["position"].params["scaling"]["factor"] == 5.0 and lat["position"].params["theta"] == 10000.0
    att = plan.blocks[1].mixer.params
    assert att["window"] == ("chunk", 31) and att["value_mix"] == "source" and att["head_sinks"] and att["head_gate"]
    assert att["distance_slopes"] == tuple(2.0 ** (-8.0 * (h + 1) / 6) for h in range(6))
    assert plan.blocks[2].mixer.params["window"] == ("full", 0) and plan.blocks[2].mixer.params["value_mix"] is None
    assert plan.blocks[3].mixer.params["value_mix"] == "blend"
    assert plan.blocks[3].ffn.params["top_k"] == 4 and "ffn" not in plan.blocks[2].parts
    assert plan.blocks[4].mixer.params["position"].params["scaling"] is None
    assert plan.final_norm.params == {"size": 64, "eps": 3e-3, "gain_offset": 1.0}
    assert plan.logit_softcap == 11.0 and not plan.tie_word_embeddings
    assert [c.cache for c in plan.order] == [0, 1, 2, 3, 4]


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="recurrent"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"].update(rot_dim=7), "rot"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=4), "dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda d: d["layers"][1]["mixer"].update(heads=5), "kv_heads"),
    (lambda d: d["layers"][3]["mixer"].update(vdim=8), "v_mix"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d.update(logit_softcap=-1.0), "softcap"),
])
def test_bad_configurations_are_named(change, word):
    raw = copy.deepcopy(Z.CONFIG_U)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        MibezenConfig.from_dict(raw)


def test_tensor_names_stacked_experts_and_the_error_lists():
    cfg = MibezenConfig.from_dict(Z.CONFIG_U)
    tensors = random_checkpoint_tensors(cfg, seed=3, std=0.1)
    assert tuple(tensors["l1.mix.vmix"].shape) == () and tuple(tensors["l1.mix.sink"].shape) == (6,)
    assert tuple(tensors["l0.mix.dkv"].shape) == (48, 64) and tuple(tensors["l0.mix.dkv.norm"].shape) == (40,)
    assert tuple(tensors["l0.mix.uq"].shape) == (3 * 24, 40) and tuple(tensors["head"].shape) == (300, 64)
    bound = bind_tensors(cfg, tensors)
    gate = bound["layers.0.ffn.experts_gate"]
    assert tuple(gate.shape) == (5, 40, 64)
    for e in range(5):
        assert torch.equal(gate[e], tensors[f"l0.mlp.e{e}.gate"])
    assert "layers.2.ffn_norm.weight" not in bound and "layers.2.mixer.value_mix" not in bound
    tensors["l2.norm2"] = torch.ones(64)                  # of a feed-forward the layer does not have: passed over
    tensors["l2.mix.vmix"] = torch.tensor(0.5)            # of a layer that does not blend: passed over
    assert set(bind_tensors(cfg, tensors)) == set(bound)
    del tensors["l3.mlp.e4.down"]
    tensors["l0.mix.uk"] = tensors["l0.mix.uk"][:, :10]
    tensors["l9.norm1"] = torch.ones(64)
    with pytest.raises(WeightError) as e:
        bind_tensors(cfg, tensors)
    assert [n for n, _ in e.value.missing] == ["l3.mlp.e4.down"]
    assert [n for n, _, _ in e.value.wrong_shape] == ["l0.mix.uk"]
    assert e.value.unexpected == ["l9.norm1"]


# ---------------------------------------------------------------------------- mechanisms, each against loops
def test_stretched_frequencies_against_the_rule_written_out():
    for dims, base, (factor, orig, fast, slow) in [(8, 10000.0, (8.0, 64, 4.0, 0.5)), (32, 20000.0, (4.0, 128, 16.0, 2.0)),
                                                   (6, 100.0, (3.0, 16, 2.0, 1.0)), (16, 3000.0, (2.0, 32, 8.0, 1.0)),
                                                   (4, 50.0, (2.0, 8, 1.0, 1.0))]:       # the last: an empty band
        f, amp = yarn_frequencies(dims, base, {"factor": factor, "original": orig, "fast": fast, "slow": slow})
        where = lambda t: dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))
        lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
        for i in range(dims // 2):
            plain_f = base ** (-2.0 * i / dims)
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            assert f[i] == pytest.approx(plain_f / factor * ramp + plain_f * (1 - ramp), rel=1e-12)
        assert amp == pytest.approx(0.1 * math.log(factor) + 1.0)
        cos, sin = plain.yarn_table({"dims": dims, "base": base, "scaling": {"factor": factor, "original": orig, "fast": fast, "slow": slow}},
                                    9, torch.float64)
        for i in range(dims // 2):
            assert float(cos[7, i]) == pytest.approx(math.cos(7 * f[i]) * amp, abs=1e-12)
            assert float(sin[7, i]) == pytest.approx(math.sin(7 * f[i]) * amp, abs=1e-12)
    assert yarn_frequencies(8, 100.0, None) == ([100.0 ** (-2.0 * i / 8) for i in range(4)], 1.0)


def test_plain_chunk_attention_against_loops():
    """Scores, bias, chunk, sink, blending and gate written out element by element in float64."""
    g = torch.Generator().manual_seed(1)
    T, d, H, G, dk, dv, size = 23, 20, 4, 2, 6, 4, 5
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 0.4, "mask": {"size": size}}
    W = {n: torch.randn(s, generator=g, dtype=torch.float64) * 0.5 for n, s in
         {"q": (H * dk, d), "k": (G * dk, d), "v": (G * dv, d), "g": (H, d), "o": (d, H * dv), "sink": (H,)}.items()}
    h = torch.randn((T, d), generator=g, dtype=torch.float64)
    v_first = torch.randn((T, G, dv), generator=g, dtype=torch.float64)
    lam = torch.tensor(0.3, dtype=torch.float64)
    got, v_used = plain.chunk_attention(h, W, m, v_first, lam)
    want = torch.zeros((T, d), dtype=torch.float64)
    for i in range(T):
        heads = []
        for a in range(H):
            kv = a // (H // G)
            q = W["q"][a * dk:(a + 1) * dk] @ h[i]
            slope = 2.0 ** (-8.0 * (a + 1) / H)
            sc, vals = [], []
            for j in range(i + 1):
                if j // size != i // size:
                    continue
                k = W["k"][kv * dk:(kv + 1) * dk] @ h[j]
                v = 0.7 * (W["v"][kv * dv:(kv + 1) * dv] @ h[j]) + 0.3 * v_first[j, kv]
                sc.append(float(q @ k) * 0.4 - slope * (i - j))
                vals.append(v)
            den = sum(math.exp(s) for s in sc) + math.exp(float(W["sink"][a]))
            o = sum(math.exp(s) / den * v for s, v in zip(sc, vals))
            heads.append(o / (1.0 + math.exp(-float(W["g"][a] @ h[i]))))
        want[i] = W["o"] @ torch.cat(heads)
    assert float((got - want).abs().max()) < 1e-10
    assert float((v_used - (0.7 * (h @ W["v"].T).reshape(T, G, dv) + 0.3 * v_first)).abs().max()) < 1e-12


def test_plain_latent_attention_against_loops():
    g = torch.Generator().manual_seed(2)
    T, d, H, dn, dr, dv, rq, rkv = 11, 18, 3, 4, 6, 5, 7, 9
    rot = {"base": 50.0, "dims": dr, "scaling": {"factor": 3.0, "original": 8, "fast": 1.0, "slow": 0.25}}
    m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": dv, "q_rank": rq, "kv_rank": rkv, "scale": 0.3, "rot": rot}
    shapes = {"dq": (rq, d), "dq.norm": (rq,), "uq": (H * (dn + dr), rq), "dkv": (rkv + dr, d), "dkv.norm": (rkv,),
              "uk": (H * dn, rkv), "uv": (H * dv, rkv), "g": (H, d), "o": (d, H * dv)}
    W = {n: torch.randn(s, generator=g, dtype=torch.float64) * 0.6 for n, s in shapes.items()}
    h = torch.randn((T, d), generator=g, dtype=torch.float64)
    eps = 1e-3
    got = plain.latent_attention(h, W, m, eps)
    f, amp = yarn_frequencies(dr, 50.0, rot["scaling"])

    def turn(v, p):
        out = v.clone()
        for i in range(dr // 2):
            c, s = math.cos(p * f[i]) * amp, math.sin(p * f[i]) * amp
            out[2 * i], out[2 * i + 1] = v[2 * i] * c - v[2 * i + 1] * s, v[2 * i + 1] * c + v[2 * i] * s
        return out

    def norm(v, w):
        return v / math.sqrt(float((v * v).mean()) + eps) * w
    want = torch.zeros((T, d), dtype=torch.float64)
    lat = [norm((W["dkv"] @ h[j])[:rkv], W["dkv.norm"]) for j in range(T)]
    shared = [turn((W["dkv"] @ h[j])[rkv:], j) for j in range(T)]
    for i in range(T):
        q = W["uq"] @ norm(W["dq"] @ h[i], W["dq.norm"])
        heads = []
        for a in range(H):
            qa = q[a * (dn + dr):(a + 1) * (dn + dr)]
            qn, qr = qa[:dn], turn(qa[dn:], i)
            sc = [float(qn @ (W["uk"][a * dn:(a + 1) * dn] @ lat[j]) + qr @ shared[j]) * 0.3 for j in range(i + 1)]
            den = sum(math.exp(s) for s in sc)
            o = sum(math.exp(s) / den * (W["uv"][a * dv:(a + 1) * dv] @ lat[j]) for j, s in enumerate(sc))
            heads.append(o / (1.0 + math.exp(-float(W["g"][a] @ h[i]))))
        want[i] = W["o"] @ torch.cat(heads)
    assert float((got - want).abs().max()) < 1e-10


def test_plain_router_and_experts_against_loops():
    g = torch.Generator().manual_seed(3)
    T, d, E, top, f = 7, 12, 5, 3, 6
    W = {"router": torch.randn((E, d), generator=g, dtype=torch.float64)}
    for e in range(E):
        W[f"e{e}.gate"] = torch.randn((f, d), generator=g, dtype=torch.float64) * 0.5
        W[f"e{e}.up"] = torch.randn((f, d), generator=g, dtype=torch.float64) * 0.5
        W[f"e{e}.down"] = torch.randn((d, f), generator=g, dtype=torch.float64) * 0.5
    h = torch.randn((T, d), generator=g, dtype=torch.float64)
    got = plain.moe_ff(h, W, {"router": {"experts": E, "top": top}})
    for t in range(T):
        z = [float(W["router"][e] @ h[t]) for e in range(E)]
        s = [math.exp(x) / sum(math.exp(y) for y in z) for x in z]
        chosen = sorted(range(E), key=lambda e: -s[e])[:top]
        total = sum(s[e] for e in chosen) + 1e-20
        want = torch.zeros(d, dtype=torch.float64)
        for e in chosen:
            a, u = W[f"e{e}.gate"] @ h[t], W[f"e{e}.up"] @ h[t]
            want += s[e] / total * (W[f"e{e}.down"] @ (a / (1 + torch.exp(-a)) * u))
        assert float((got[t] - want).abs().max()) < 1e-5       # (the plain router runs in float32)
    hh = torch.randn((3, d), generator=g, dtype=torch.float64)
    assert float((plain.dense_ff(hh, {"up": W["e0.up"], "down": W["e0.down"]}) -
                  (torch.clamp(hh @ W["e0.up"].T, min=0) ** 2) @ W["e0.down"].T).abs().max()) < 1e-12
    x = torch.randn((4, d), generator=g, dtype=torch.float64)
    w = torch.randn(d, generator=g, dtype=torch.float64) * 0.2
    assert float((plain.norm_around_zero(x, w, 1e-2) - x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-2) * (1 + w)).abs().max()) < 1e-12


# ---------------------------------------------------------------------------- the engine on the host
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: Z.write_model(tmp_path_factory.mktemp(f"mibezen_{n}"), n) for n in Z.CONFIGS}


def host_engine(folder, tokens, page_size=16, max_requests=4):
    k = TorchReferenceKernels(torch.float32, "cpu")
    model = Model.from_folder(folder, dtype="float32", device="cpu", kernels=k)
    return Engine(model, cache_tokens=tokens, page_size=page_size, max_requests=max_requests)


def requests_for(folder, lens, seed):
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("name", list(Z.CONFIGS))
def test_folder_round_trip_and_whole_prompts(folders, name):
    folder = folders[name]
    assert load_config(folder).to_dict() == Z.CONFIGS[name][0]
    reqs = requests_for(folder, (53, 1, 20), 10)
    eng = host_engine(folder, 64)
    Z.compare_with_plain(H.run_steps(eng, H.steps_whole(reqs)), folder, reqs, 2e-5)
    assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups


def test_caches_latent_rows_of_one_plane_and_one_group_per_window(folders):
    eng = host_engine(folders["U"], 64)
    keys = eng.storage.group_keys
    lat = [k for k in keys if k.planes == 1]
    assert sorted((k.head_dim, k.num_kv_heads) for k in lat) == [(32, 1), (48, 1)]        # kv_rank + rot_dim, one kv head
    assert all(k.window.kind == "full" for k in lat)
    assert sorted((k.window.kind, k.window.size) for k in keys if k.planes == 2) == [("chunk", 24), ("chunk", 40), ("full", 0)]
    for g, k in enumerate(keys):
        assert eng.storage.kv[g].shape[1] == k.planes


def test_the_residual_stream_after_every_layer(folders):
    folder = folders["U"]
    toks = requests_for(folder, (29,), 20)["r0"]
    cfg, tensors = Z.folder_contents(str(folder))
    layers = []
    plain.forward(cfg, tensors, toks, tap=lambda i, x: layers.append(x.clone()))
    eng = host_engine(folder, 64)
    seen = []
    eng.model.layer_tap = lambda i, h: seen.append((i, h.clone()))
    H.run_steps(eng, H.steps_whole({"a": toks}))
    assert [i for i, _ in seen] == list(range(len(layers)))
    for i, h in seen:
        assert float((h - layers[i]).abs().max()) <= 2e-5 * float(layers[i].abs().max()), f"layer {i}"


@pytest.mark.parametrize("name", list(Z.CONFIGS))
def test_portions_decoding_and_mixed_batches_on_the_host(folders, name):
    """Token by token after a prompt, portions down to two tokens, and up to four live requests in a pool that
    forces pages and slots to be used again: the logits are those of the whole sequence.  The prompts are longer than
    every chunk, so portions start and end inside chunks and decoded tokens cross their borders."""
    folder = folders[name]
    reqs = requests_for(folder, (61, 9, 30, 3, 47, 17), 30)
    cuts = {"decoded": H.steps_last_decoded(reqs, 30), "portions": H.steps_portions(reqs, seed=2),
            "mixed": H.steps_mixed(reqs, {r: max(1, len(t) - 6) for r, t in reqs.items()}, seed=3)}
    for what, steps in cuts.items():
        eng = host_engine(folder, H.max_tokens_of(steps) if what == "mixed" else 64, page_size=16)
        Z.compare_with_plain(H.run_steps(eng, steps), folder, reqs, 2e-5)
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what


def test_pages_behind_a_chunk_go_back_while_the_latent_pages_stay(folders):
    eng = host_engine(folders["U"], 128, page_size=8)
    toks = requests_for(folders["U"], (100,), 40)["r0"]
    H.run_steps(eng, [{"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [99]}], "end": []}])
    for g, key in enumerate(eng.storage.group_keys):
        held = [p for p in eng.cache.block_table("a", g) if p >= 0]
        if key.window.kind == "chunk":
            first = (100 // key.window.size) * key.window.size
            assert len(held) == -(-100 // 8) - first // 8, key
        else:
            assert len(held) == -(-100 // 8), key


def test_the_command_line_writes_a_random_model_folder(tmp_path):
    from spite_b200 import cli
    from spite_b200.weights import load_bound_tensors
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(Z.CONFIG_V))
    out = tmp_path / "model"
    assert cli.main(["random", "--config", str(cfg_file), "--out", str(out), "--seed", "4", "--std", "0.05"]) == 0
    config = load_config(out)
    assert isinstance(config, MibezenConfig) and config.layers[1].mixer.kv_rank == 96
    _, tensors = plain.load_folder(out)
    assert sorted(n for n in tensors if n.startswith("l0.mlp.e1.")) == ["l0.mlp.e1.down", "l0.mlp.e1.gate", "l0.mlp.e1.up"]
    bound = load_bound_tensors(out, config)
    assert tuple(bound["layers.3.mixer.k_up"].shape) == (8 * 16, 48) and tuple(bound["head.weight"].shape) == (520, 128)
