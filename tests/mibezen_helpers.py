"""Small Mibezen configurations for the tests (none has the sizes of a published model), model folders with
random weights, and the comparison with the plain implementation (`plain_mibezen`)."""
from __future__ import annotations

import functools
import random
from pathlib import Path

import torch

import plain_mibezen as plain
from helpers import note_error
from spite_b200.config import MibezenConfig
from spite_b200.weights import save_file, write_random_model


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": rot}


def attn(heads, kv, dim, vdim, scale, chunk=None, v_mix=False):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if chunk:
        d["mask"] = {"size": chunk}
    return d


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


# Layers that differ in every size.  The first blending layer is not the first layer; the second one has another key
# size than its source; one attention layer neither blends nor has a chunk; one layer has no feed-forward; one latent
# layer rotates with plain frequencies, the other with a stretch whose ramp lies inside the pairs.
CONFIG_U = {
    "architecture": "Mibezen", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
    "layers": [
        {"type": "latent_attention", "mixer": latent(3, 16, 8, 24, 40, 40, 0.21, 10000.0, (8.0, 64, 4.0, 0.5)), "mlp": moe(5, 2, 40)},
        {"type": "attention", "mixer": attn(6, 3, 16, 16, 0.25, chunk=24, v_mix=True), "mlp": dense(96)},
        {"type": "attention", "mixer": attn(2, 2, 24, 8, 0.3), "mlp": None},
        {"type": "attention", "mixer": attn(6, 3, 32, 16, 0.18, chunk=40, v_mix=True), "mlp": moe(6, 1, 24)},
        {"type": "latent_attention", "mixer": latent(2, 24, 4, 16, 24, 28, 0.15, 500.0), "mlp": dense(72)},
    ]}

# Sizes that reach the tensor-core and TMA kernels in bfloat16: cache rows of 64 and 128 elements (attention heads of
# 64; latent rows of 48 + 16 and 96 + 32), chunks that are multiples of a page and not, widths that are multiples of 64.
CONFIG_V = {
    "architecture": "Mibezen", "vocab": 520, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": attn(8, 2, 64, 64, 0.125, chunk=128, v_mix=True), "mlp": moe(4, 3, 64)},
        {"type": "latent_attention", "mixer": latent(4, 32, 32, 32, 64, 96, 0.12, 20000.0, (4.0, 128, 16.0, 2.0)), "mlp": dense(192)},
        {"type": "attention", "mixer": attn(4, 2, 64, 64, 0.1, chunk=100, v_mix=True), "mlp": dense(128)},
        {"type": "latent_attention", "mixer": latent(8, 16, 16, 48, 48, 48, 0.2, 3000.0, (2.0, 32, 8.0, 1.0)), "mlp": moe(8, 2, 32)},
    ]}

# Awkward sizes: a width that is no multiple of 8, seven heads on one kv head, a chunk shorter than a page, odd ranks,
# every expert chosen, an odd vocabulary, no cap on the logits.
CONFIG_W = {
    "architecture": "Mibezen", "vocab": 301, "width": 100, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "attention", "mixer": attn(7, 1, 10, 6, 0.3, chunk=7), "mlp": moe(3, 3, 44)},
        {"type": "latent_attention", "mixer": latent(5, 12, 6, 10, 22, 30, 0.2, 100.0, (3.0, 16, 2.0, 1.0)), "mlp": moe(3, 1, 20)},
        {"type": "attention", "mixer": attn(3, 3, 12, 30, 0.3, v_mix=True), "mlp": dense(60)},
    ]}

CONFIGS = {"U": (CONFIG_U, 0.09, 5), "V": (CONFIG_V, 0.06, 6), "W": (CONFIG_W, 0.08, 7)}


def write_model(folder, name: str, dtype=torch.bfloat16) -> Path:
    """A model folder with random weights.  What a lost or misread tensor must show in is drawn away from its neutral
    value: norm gains around zero with a spread, latent gains around one, sinks of order one, blending weights well
    inside (0, 1), gate rows large enough for gates far from one half."""
    cfg, std, seed = CONFIGS[name]
    config = MibezenConfig.from_dict(cfg)
    folder = write_random_model(folder, config, seed=seed, std=std, dtype=dtype)
    _, tensors = plain.load_folder(folder)
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if n.endswith((".norm1", ".norm2")) or n == "final.norm":
            tensors[n] = (0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith((".dq.norm", ".dkv.norm")):
            tensors[n] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(".sink"):
            tensors[n] = (1.5 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(".vmix"):
            tensors[n] = (0.25 + 0.5 * torch.rand((), generator=g)).to(t.dtype)
        elif n.endswith(".mix.g"):
            tensors[n] = (t.float() * 6.0).to(t.dtype)
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
    expert's logit exceeds the best one left out by `min_margin` at every routed layer and position): in
    bfloat16, where rounding decides which expert runs, two correct implementations differ by an expert's output."""
    cfg, tensors = folder_contents(str(folder))
    rng = random.Random(seed)
    toks: list[int] = []
    while len(toks) < n:
        for _ in range(300):
            cand = toks + [rng.randrange(cfg["vocab"])]
            margins = []
            plain.forward(cfg, tensors, cand, margins=margins)
            if all(float(m[-1]) >= min_margin for m in margins):
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


def generate_greedy(cfg, tensors, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        row = plain.forward(cfg, tensors, toks)[-1]
        toks.append(int(torch.argmax(row)))
    return toks[len(prompt):]
