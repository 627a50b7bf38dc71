"""Small Sezazen configurations for the tests (none has the sizes of a published model), model folders with
random weights, and the comparison with the plain implementation (`plain_sezazen`)."""
from __future__ import annotations

import functools
import random
from pathlib import Path

import torch

import plain_sezazen as plain
from helpers import note_error
from spite_b200.config import SezazenConfig
from spite_b200.weights import write_random_model


def _attn(heads, kv, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}


def _moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


# layers that differ in every size; value heads larger and smaller than key heads; two experts a token and one;
# a layer without a feed-forward; a loop over the middle layers
CONFIG_P = {
    "architecture": "Sezazen", "vocab": 300, "width": 64, "max_positions": 512, "norm": {"eps": 1e-6},
    "embedding": {"scale": 3.5},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.3), "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention", "mixer": _attn(6, 3, 32, 16, 0.2), "mlp": _moe(6, 2, 40, 56)},
        {"type": "attention", "mixer": _attn(2, 2, 48, 48, 0.15), "mlp": None},
        {"type": "attention", "mixer": _attn(8, 1, 16, 8, 0.25), "mlp": _moe(5, 1, 24)},
    ],
    "loop": {"start": 1, "stop": 3, "times": 2}}

# sizes that reach the tcgen05 and TMA kernels (cache rows of 64 elements, widths that are multiples of 64); the
# loop starts at the first layer and covers every layer; three experts a token
CONFIG_Q = {
    "architecture": "Sezazen", "vocab": 520, "width": 128, "max_positions": 1024, "norm": {"eps": 1e-5},
    "embedding": {"scale": 8.0},
    "layers": [
        {"type": "attention", "mixer": _attn(6, 2, 64, 64, 0.125), "mlp": _moe(4, 3, 64, 128)},
        {"type": "attention", "mixer": _attn(4, 4, 64, 40, 0.1), "mlp": {"kind": "dense", "ff": 192}},
    ],
    "loop": {"start": 0, "stop": 2, "times": 3}}

# awkward sizes and no loop: a width that is no multiple of 8, seven heads on one kv head, odd vocabulary
CONFIG_R = {
    "architecture": "Sezazen", "vocab": 301, "width": 100, "max_positions": 256, "norm": {"eps": 1e-4},
    "embedding": {"scale": 1.0},
    "layers": [
        {"type": "attention", "mixer": _attn(7, 1, 24, 10, 0.2), "mlp": _moe(3, 1, 44, 20)},
        {"type": "attention", "mixer": _attn(3, 3, 12, 30, 0.3), "mlp": {"kind": "dense", "ff": 60}},
    ]}

# a loop that runs once, over the last layer alone
CONFIG_S = dict(CONFIG_R, loop={"start": 1, "stop": 2, "times": 1})

CONFIGS = {"P": (CONFIG_P, 0.08, 5), "Q": (CONFIG_Q, 0.05, 6), "R": (CONFIG_R, 0.07, 7), "S": (CONFIG_S, 0.07, 8)}


def write_model(folder, name: str, dtype=torch.bfloat16, norm_gains=True) -> Path:
    """A model folder with random weights; norm gains are drawn around one so that a lost gain shows."""
    cfg, std, seed = CONFIGS[name]
    config = SezazenConfig.from_dict(cfg)
    folder = write_random_model(folder, config, seed=seed, std=std, dtype=dtype)
    if norm_gains:
        from spite_b200.weights import save_file
        _, tensors = plain.load_folder(folder)
        g = torch.Generator().manual_seed(seed)
        for name_, t in tensors.items():
            if t.dim() == 1:
                tensors[name_] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        save_file(tensors, Path(folder) / "model.safetensors")
    return Path(folder)


@functools.lru_cache(maxsize=None)
def folder_contents(folder: str):
    return plain.load_folder(folder)


_plain_cache: dict = {}


def plain_logits(folder, tokens) -> torch.Tensor:
    key = (str(folder), tuple(tokens))
    if key not in _plain_cache:
        cfg, tensors = folder_contents(str(folder))
        _plain_cache[key] = plain.forward(cfg, tensors, list(tokens))
    return _plain_cache[key]


def decisive_tokens(folder, n: int, seed: int, min_margin: float) -> list[int]:
    """A token sequence in which every routing decision of the plain implementation is clear (the last chosen
    expert's logit exceeds the best one left out by `min_margin` at every routed layer run and position): in
    bfloat16, where rounding decides which expert runs, two correct implementations differ by an expert's output."""
    cfg, tensors = folder_contents(str(folder))
    rng = random.Random(seed)
    toks: list[int] = []
    while len(toks) < n:
        for _ in range(300):
            cand = toks + [rng.randrange(cfg["vocab"])]
            info = {}
            plain.forward(cfg, tensors, cand, collect=info)
            m = info["router_margins"]
            if m.numel() == 0 or float(m[:, -1].min()) >= min_margin:
                toks = cand
                break
        else:
            raise RuntimeError("no token with clear routing found")
    return toks


def compare_with_plain(results: dict, folder, requests: dict, tol: float):
    """Every logits row against the plain implementation, as a fraction of the largest logit of the sequence;
    names the first position beyond `tol`."""
    worst = 0.0
    for r, toks in requests.items():
        ref = plain_logits(folder, toks)
        scale = float(ref.abs().max())
        for p in range(len(toks)):
            if (r, p) not in results:
                continue
            err = float((results[(r, p)] - ref[p]).abs().max()) / scale
            worst = max(worst, err)
            assert err <= tol, (f"request {r!r}, position {p} (first wrong one): error {err:.3e} of the "
                                f"logit scale exceeds {tol:.1e} (worst before it: {worst:.3e})")
    note_error(worst, tol)
    return worst
