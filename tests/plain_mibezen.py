"""Plain, slow implementation of the Mibezen decoder: whole sequences, no cache, float32 (or float64) on the
CPU, one function per mechanism, written from the design's equations.  It shares no code with the package:
it has its own safetensors reader and takes the parsed config.json as a dict.

Notation: x is the residual stream [T, d] of one sequence, h a mixer's or feed-forward's input, positions
count from 0.
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
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
    return out


def load_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ---------------------------------------------------------------------------------- mechanisms
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps): the epsilon joins the mean square under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The layer norms and the final norm: the gain is stored as its distance from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    """The norms of the latents: the gain is stored as it is."""
    return rms(x, eps) * w


def yarn_table(rot: dict, T: int, dtype):
    """cos and sin [T, dims/2] of the rotation with stretched wavelengths.

    f_i = base^(-2i/dims).  A pair whose wavelength is short against the original context keeps f_i, one whose
    wavelength is long gets f_i / factor, with a linear ramp over the pair index between the two borders
    lo = floor(dim(fast)), hi = ceil(dim(slow)), dim(t) = dims ln(original / (2 pi t)) / (2 ln base).  Both
    tables are multiplied by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(ang) * amp).to(dtype), (torch.sin(ang) * amp).to(dtype)


def rotate_neighbours(v, cos, sin):
    """v [T, ..., dims]: elements (2i, 2i+1) turn by the angle of pair i at the row's position."""
    T = v.shape[0]
    shape = [T] + [1] * (v.dim() - 2) + [cos.shape[-1]]
    c, s = cos.reshape(shape), sin.reshape(shape)
    a, b = v[..., 0::2], v[..., 1::2]
    out = torch.empty_like(v)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = b * c + a * s
    return out


def head_gate(h, wg):
    """sigmoid(W_g h): one factor per token and head, from the mixer's own input."""
    return torch.sigmoid(h @ wg.T)


def latent_attention(h, W, m, eps):
    """Attention whose queries, keys and values pass through low-rank latents; a part of every query and one key
    part shared by all heads carry the rotation.  Written in the expanded form: keys and values of every head
    are made from the latent of every position."""
    T = h.shape[0]
    H, dn, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = norm_plain(h @ W["dq"].T, W["dq.norm"], eps)
    q = (cq @ W["uq"].T).reshape(T, H, dn + dr)
    down = h @ W["dkv"].T
    c = norm_plain(down[:, :r], W["dkv.norm"], eps)
    k_rot = down[:, r:]                                           # [T, dr], one for all heads, not normed
    cos, sin = yarn_table(m["rot"], T, h.dtype)
    assert int(m["rot"]["dims"]) == dr
    q_rot = rotate_neighbours(q[..., dn:], cos, sin)
    k_rot = rotate_neighbours(k_rot, cos, sin)
    k_n = (c @ W["uk"].T).reshape(T, H, dn)
    v = (c @ W["uv"].T).reshape(T, H, dv)
    future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a, :dn] @ k_n[:, a].T + q_rot[:, a] @ k_rot.T) * float(m["scale"])
        s = s.masked_fill(future, -math.inf)
        out[:, a] = torch.softmax(s, -1) @ v[:, a]
    out = out * head_gate(h, W["g"])[:, :, None]
    return out.reshape(T, H * dv) @ W["o"].T


def chunk_attention(h, W, m, v_first, lam):
    """Grouped-query attention without rotation: a bias that grows with distance, sight limited to the query's
    own chunk (if the layer has a mask), a learned sink per head in the softmax's denominator, values mixed with those of the first such
    layer.  Returns (output, the values this layer used)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    size = int(m["mask"]["size"]) if m.get("mask") else T         # without a mask the whole sequence is one chunk
    q = (h @ W["q"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, G, d)
    v = (h @ W["v"].T).reshape(T, G, dv)
    if v_first is not None:
        v = (1.0 - lam) * v + lam * v_first
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)              # i - j
    hidden = (pos[None, :] > pos[:, None]) | ((pos[:, None] // size) != (pos[None, :] // size))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"]) - slope * dist
        s = s.masked_fill(hidden, -math.inf)
        sink = W["sink"][a].to(h.dtype)
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        out[:, a] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))) @ v[:, g]
    out = out * head_gate(h, W["g"])[:, :, None]
    return out.reshape(T, H * dv) @ W["o"].T, v


def dense_ff(h, W):
    """down(relu(up h)^2)"""
    return torch.relu(h @ W["up"].T) ** 2 @ W["down"].T


def moe_ff(h, W, f):
    """Softmax over all experts, the `top` largest chosen, their scores renormalised to sum one, gated experts."""
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    scores = torch.softmax((h @ W["router"].T).float(), -1).to(h.dtype)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(E), key=lambda e: (-float(scores[t, e]), e))[:top]
        total = sum(scores[t, e] for e in chosen) + 1e-20
        for e in chosen:
            g = W[f"e{e}.gate"] @ h[t]
            y = W[f"e{e}.down"] @ ((g * torch.sigmoid(g)) * (W[f"e{e}.up"] @ h[t]))
            out[t] += scores[t, e] / total * y
    return out


def router_margins(h, W, f):
    """Per token: the gap between the last chosen and the first rejected router logit."""
    top = int(f["router"]["top"])
    z = (h @ W["router"].T).sort(-1, descending=True).values
    return z[:, top - 1] - z[:, top] if z.shape[1] > top else torch.full((h.shape[0],), math.inf)


# ---------------------------------------------------------------------------------- the model
def sub(tensors, prefix, dtype):
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, dtype=torch.float32, tap=None, margins=None):
    """Logits [T, vocab] of one sequence.  `tap(i, x)` receives the residual stream after every layer;
    `margins`, a list, collects the router margins of every mixture-of-experts layer."""
    eps = float(config["norm"]["eps"])
    x = tensors["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, L in enumerate(config["layers"]):
        W = sub(tensors, f"l{i}.mix.", dtype)
        h = norm_around_zero(x, tensors[f"l{i}.norm1"].to(dtype), eps)
        if L["type"] == "latent_attention":
            x = x + latent_attention(h, W, L["mixer"], eps)
        elif L["type"] == "attention":
            mixes = bool(L["mixer"].get("v_mix"))
            y, v = chunk_attention(h, W, L["mixer"], v_first if mixes else None, W["vmix"] if mixes else None)
            if mixes and v_first is None:
                v_first = v
            x = x + y
        else:
            raise ValueError(L["type"])
        f = L.get("mlp")
        if f is not None:
            F = sub(tensors, f"l{i}.mlp.", dtype)
            h = norm_around_zero(x, tensors[f"l{i}.norm2"].to(dtype), eps)
            if f["kind"] == "dense":
                x = x + dense_ff(h, F)
            else:
                if margins is not None:
                    margins.append(router_margins(h, F, f))
                x = x + moe_ff(h, F, f)
        if tap is not None:
            tap(i, x)
    x = norm_around_zero(x, tensors["final.norm"].to(dtype), eps)
    logits = x @ tensors["head"].to(dtype).T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
