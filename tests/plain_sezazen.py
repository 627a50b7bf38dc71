"""Plain, slow implementation of the Sezazen decoder: whole sequences, no cache, float32 (or float64)
on the CPU, one function per mechanism, written from the design's equations.  It shares no code with
the package: it has its own safetensors reader and takes the parsed config.json as a dict.

Notation: x is the residual stream [T, d] of one sequence, h a mixer's or feed-forward's input.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---------------------------------------------------------------------------------- files
def read_safetensors(path) -> dict:
    """8-byte little-endian header length, JSON header (name -> dtype, shape, data_offsets), data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = memoryview(raw)[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t
    return out


def load_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ---------------------------------------------------------------------------------- mechanisms
def rms_norm(x, w, eps):
    """y = x * w / sqrt(mean(x^2) + eps): the epsilon joins the mean square before the square root is taken."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def embedding(tokens, embed, pos, scale):
    """x_p = scale * embed[token_p] + pos[p], p = 0, 1, ...: the factor applies to the token's row only."""
    T = len(tokens)
    x = embed[torch.tensor(tokens, dtype=torch.long)] * scale
    if pos is not None:
        x = x + pos[:T]
    return x


def sink_attention(h, wq, wk, wv, wo, heads, kv_heads, dim, vdim, scale):
    """Causal grouped-query attention, no rotation of q and k.  Weights
    p_ij = exp(s_ij) / (1 + sum_{j' <= i} exp(s_ij')): the 1 is exp(0), the share of a sink that contributes nothing
    to the output, so the weights of a row sum to less than one."""
    T = h.shape[0]
    q = (h @ wq.T).reshape(T, heads, dim)
    k = (h @ wk.T).reshape(T, kv_heads, dim)
    v = (h @ wv.T).reshape(T, kv_heads, vdim)
    rep = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    for a in range(heads):
        g = a // rep
        s = ((q[:, a] @ k[:, g].T) * scale).masked_fill(future, -math.inf)      # [T, T], row i sees j <= i
        m = s.max(-1, keepdim=True).values.clamp_min(0.0)       # stabilised; the sink's score is 0
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + torch.exp(-m)
        out[:, a] = (e / den) @ v[:, g]
    return out.reshape(T, heads * vdim) @ wo.T


def dense_ff(h, w_gate, w_up, w_down):
    g = h @ w_gate.T
    return ((g * torch.sigmoid(g)) * (h @ w_up.T)) @ w_down.T


def relu2_expert(h, w_up, w_down):
    z = torch.relu(h @ w_up.T)
    return (z * z) @ w_down.T


def moe_ff(h, w_router, experts, top, shared, margins=None):
    """s = sigmoid(router logits); the experts with the `top` largest s run, expert e on s_e * h (the raw
    score scales what goes into the expert; the chosen scores are not made to sum to one); a shared expert runs on h.
    `margins`, a list, receives per token the gap between the last chosen logit and the best one left out."""
    z = h.to(torch.float32) @ w_router.to(torch.float32).T
    s = torch.sigmoid(z).to(h.dtype)
    if margins is not None and z.shape[1] > top:
        zs = torch.sort(z, dim=-1, descending=True).values
        margins.append(zs[:, top - 1] - zs[:, top])
    out = torch.zeros_like(h)
    order = torch.argsort(-s, dim=-1, stable=True)[:, :top]
    for t in range(h.shape[0]):
        for e in order[t].tolist():
            up, down = experts[e]
            out[t] += relu2_expert(s[t, e] * h[t:t + 1], up, down)[0]
    if shared is not None:
        out = out + relu2_expert(h, shared[0], shared[1])
    return out


def loop_entry(x, x0, w_in, step_vec):
    """x <- W_in [x; x0] + step[t]."""
    return torch.cat([x, x0], -1) @ w_in.T + step_vec


# ---------------------------------------------------------------------------------- the model
def layer_order(cfg):
    """[(layer index, pass number or None, first of its pass)] in run order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    order += [(i, None, False) for i in range(b, n)]
    return order


def forward(cfg, w, tokens, dtype=torch.float32, return_layers=False, collect=None):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run).
    `collect`, a dict, receives "router_margins" [routed layer runs, T]."""
    margins = [] if collect is not None else None
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = embedding(tokens, W["embed"], W.get("pos"), float(cfg["embedding"]["scale"]))
    x0 = x.clone()
    after = []
    for i, t, first in layer_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = loop_entry(x, x0, W["loop.in"], W["loop.step"][t])
        mx = L["mixer"]
        if L["type"] != "attention":
            raise ValueError(f"unknown layer type {L['type']!r}")
        x = x + sink_attention(rms_norm(x, W[p + "norm1"], eps), W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"],
                               W[p + "mix.o"], int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"]),
                               float(mx["scale"]))
        mlp = L.get("mlp")
        if mlp:
            h = rms_norm(x, W[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_ff(h, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
            elif mlp["kind"] == "moe":
                E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                experts = [(W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"]) for e in range(E)]
                shared = (W[p + "mlp.shared.up"], W[p + "mlp.shared.down"]) if mlp.get("shared") else None
                x = x + moe_ff(h, W[p + "mlp.router"], experts, top, shared, margins)
            else:
                raise ValueError(f"unknown mlp kind {mlp['kind']!r}")
        after.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    if collect is not None:
        collect["router_margins"] = torch.stack(margins) if margins else torch.zeros((0, len(tokens)))
    return (logits, torch.stack(after)) if return_layers else logits


def generate_greedy(cfg, w, prompt, n_new, dtype=torch.float32):
    """`n_new` tokens by argmax (ties to the highest index), recomputing the whole sequence every time."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        row = forward(cfg, w, toks, dtype=dtype)[-1]
        best = int((row == row.max()).nonzero().max())
        out.append(best)
        toks.append(best)
    return out
