"""Random Sezazen configurations on the GPU: sizes, head counts, layer order, loop and constants are drawn per
seed (head sizes that are no multiple of 16, value heads larger and smaller than key heads, widths and expert
sizes that are no multiple of 8, more query heads per kv head than the tensor-core kernels take, as many
experts a token as there are experts), then the engine runs whole prompts, portions and a mixed schedule in
float32 (bit-identical between the cuts) and in bfloat16 against the plain implementation."""
import json
import random

import pytest
import torch

import helpers as H
import plain_sezazen as plain
import sezazen_helpers as S
from spite_b200.config import SezazenConfig
from spite_b200.weights import save_file, write_random_model

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([48, 64, 72, 100, 128, 192, 256])
    layers = []
    for _ in range(rng.randint(2, 5)):
        heads = rng.choice([1, 2, 3, 4, 6, 8, 12, 20])
        kv = rng.choice([k for k in range(1, heads + 1) if heads % k == 0])
        mixer = {"heads": heads, "kv_heads": kv, "dim": rng.choice([8, 16, 24, 32, 40, 64, 80, 96, 128]),
                 "vdim": rng.choice([8, 10, 16, 24, 32, 48, 56, 64, 96, 128]), "scale": round(rng.uniform(0.05, 0.4), 3)}
        kind = rng.choice(["none", "dense", "moe", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = {"kind": "dense", "ff": rng.choice([32, 60, 96, 200])}
        else:
            E = rng.choice([2, 3, 5, 8, 16])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([16, 24, 44, 64, 128])},
                   "router": {"experts": E, "top": rng.randint(1, min(4, E))}}
            if rng.random() < 0.6:
                mlp["shared"] = {"ff": rng.choice([20, 64, 128])}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Sezazen", "vocab": rng.choice([101, 256, 517, 1000]), "width": width, "max_positions": 512,
           "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "embedding": {"scale": round(rng.uniform(0.5, 12.0), 2)},
           "layers": layers}
    if rng.random() < 0.75:
        a = rng.randrange(len(layers))
        cfg["loop"] = {"start": a, "stop": rng.randint(a + 1, len(layers)), "times": rng.randint(1, 4)}
    return cfg


@pytest.fixture(scope="module", params=range(10))
def model_folder(request, tmp_path_factory):
    seed = request.param
    cfg = random_config(seed)
    folder = tmp_path_factory.mktemp(f"sezazen_random_{seed}")
    write_random_model(folder, SezazenConfig.from_dict(cfg), seed=seed, std=0.06)
    _, tensors = plain.load_folder(folder)
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():                          # norm gains away from one
        if t.dim() == 1:
            tensors[name] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
    save_file(tensors, folder / "model.safetensors")
    return folder, cfg, seed


def _run(model, steps, page):
    from spite_b200.engine import Engine
    eng = Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page, max_requests=4)
    out = H.run_steps(eng, steps)
    eng.check()
    return out


def test_float32_every_cut(model_folder):
    from spite_b200.engine import Model
    folder, cfg, seed = model_folder
    model = Model.from_folder(folder, dtype="float32", device=DEV)
    reqs = {r: H.random_tokens(cfg["vocab"], n, seed * 10 + i) for i, (r, n) in enumerate({"a": 140, "b": 33, "c": 1, "d": 58}.items())}
    n_prompt = {r: max(1, len(t) - 7) for r, t in reqs.items()}
    cuts = {"whole": _run(model, H.steps_whole(reqs), 64), "portions": _run(model, H.steps_portions(reqs, seed=seed), 16),
            "decoded": _run(model, H.steps_last_decoded(reqs, 20), 64),
            "mixed": _run(model, H.steps_mixed(reqs, n_prompt, seed=seed), 16)}
    for res in cuts.values():
        S.compare_with_plain(res, folder, reqs, 2e-5)
    H.assert_cuts_identical(cuts)


def test_bfloat16_every_cut(model_folder):
    from spite_b200.engine import Model
    folder, cfg, seed = model_folder
    model = Model.from_folder(folder, dtype="bfloat16", device=DEV)
    reqs = {r: S.decisive_tokens(folder, n, seed * 10 + i, 0.04) for i, (r, n) in enumerate({"a": 140, "b": 33, "c": 1}.items())}
    n_prompt = {r: max(1, len(t) - 7) for r, t in reqs.items()}
    for steps, page in ((H.steps_whole(reqs), 64), (H.steps_portions(reqs, seed=seed), 16), (H.steps_last_decoded(reqs, 20), 64),
                        (H.steps_mixed(reqs, n_prompt, seed=seed), 64)):
        S.compare_with_plain(_run(model, steps, page), folder, reqs, 2.5e-2)


def test_the_drawn_configurations_differ(tmp_path):
    kinds = [json.dumps(random_config(s), sort_keys=True) for s in range(10)]
    assert len(set(kinds)) == 10
    assert any("loop" not in json.loads(k) for k in kinds) and any(json.loads(k).get("loop", {}).get("start") == 0 for k in kinds)


def test_bfloat16_long_prompt(model_folder):
    """A prompt of several hundred tokens (several 128-row tiles of the prompt kernels, keys hundreds of positions
    back, key splits in decoding) in bfloat16: whole, its last 40 tokens decoded, and in portions."""
    from spite_b200.engine import Model
    folder, cfg, seed = model_folder
    if seed not in (0, 8):
        pytest.skip("long prompts for two of the configurations")
    model = Model.from_folder(folder, dtype="bfloat16", device=DEV)
    reqs = {"long": S.decisive_tokens(folder, 300, seed + 100, 0.04)}
    for steps, page in ((H.steps_whole(reqs), 64), (H.steps_last_decoded(reqs, 40), 64),
                        (H.steps_portions(reqs, seed=seed, sizes=(2, 17, 64, 150)), 64)):
        S.compare_with_plain(_run(model, steps, page), folder, reqs, 2.5e-2)
