"""Sezazen on the GPU.  First every new mechanism alone against a plain computation written here from its
equation (the sink in every attention kernel, value heads of another size than key heads, squared-ReLU
products, learned positions, the loop's junction); then the engine in float32 and bfloat16 against the plain
implementation in every cut (whole, token by token, portions down to two tokens, mixed batches in a pool whose
pages and slots are used again, free pages poisoned), and greedy generation through `LLM.generate`."""
import json
import math

import pytest
import torch

import helpers as H
import plain_sezazen as plain
import sezazen_helpers as S
from spite_b200.cache import LayerCache, Window
from test_gpu_kernels import close, fill_cache, make_batch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
KTOL = {torch.float32: 1e-5, torch.bfloat16: 1.2e-2}
MARGIN = 0.03           # router logit margin that bfloat16 rounding cannot flip at these sizes


def kernels(dtype):
    from spite_b200.kernels.cuda import CudaKernels
    return CudaKernels(dtype, DEV)


# ---------------------------------------------------------------------------- the sink, kernel by kernel
def sink_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, sink):
    """p_j = exp(s_j) / (exp(sink) + sum_j' exp(s_j')) over the keys j <= position, float64, with loops."""
    out = torch.zeros(q.shape, dtype=torch.float64)
    group, off = nq // nkv, 0
    for s, (start, n) in enumerate(specs):
        for t in range(n):
            pos = start + t
            for h in range(nq):
                sc = (k_all[s][:pos + 1, h // group].double() @ q[off + t, h].double()) * scale
                m = max(float(sc.max()), sink)
                e = torch.exp(sc - m)
                den = e.sum() + math.exp(sink - m)
                out[off + t, h] = (e / den) @ v_all[s][:pos + 1, h // group].double()
        off += n
    return out


# (kernel library that must serve the call, dtype, query heads, kv heads, row size, page size, segments)
SINK_CASES = [
    ("attention", torch.float32, 5, 1, 24, 16, [(0, 1), (0, 40), (130, 1), (61, 7)]),
    ("attention", torch.bfloat16, 6, 3, 24, 16, [(0, 1), (0, 40), (130, 1), (61, 7)]),
    ("attention_mma", torch.bfloat16, 4, 2, 48, 16, [(0, 1), (200, 1), (31, 2), (1500, 1)]),
    ("attention_rows", torch.bfloat16, 6, 2, 32, 32, [(0, 33), (100, 20), (0, 12)]),
    ("attention_decode", torch.bfloat16, 8, 2, 64, 64, [(0, 1), (63, 1), (64, 1), (3000, 1), (517, 2)]),
    ("attention_tc", torch.bfloat16, 6, 2, 64, 64, [(0, 300), (200, 130), (0, 70)]),
    ("attention_tc", torch.bfloat16, 4, 1, 128, 64, [(0, 140), (900, 64)]),
]


@pytest.mark.parametrize("sink", [0.0, 1.5, -3.0])
@pytest.mark.parametrize("case", range(len(SINK_CASES)))
def test_the_sink_in_every_attention_kernel(case, sink):
    """Small scores, so that the sink holds a large share of every softmax (half of the first token's), and one
    row whose query is aligned with a far key, which then outweighs the sink: a sink that is left out, counted
    twice (once per key split) or given the wrong score shows in every row."""
    library, dtype, nq, nkv, hd, P, specs = SINK_CASES[case]
    ks = kernels(dtype)
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 3
    batch, tables = make_batch(specs, P, n_pages, 60 + case, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(61 + case)
    k_all = [torch.randn((s + n, nkv, hd), generator=g).to(dtype) for s, n in specs]
    v_all = [torch.randn((s + n, nkv, hd), generator=g).to(dtype) for s, n in specs]
    q = torch.randn((M, nq, hd), generator=g) * 0.3
    last = M - 1                                             # the last row looks far back, at key 1 of its request
    q[last, 0] = k_all[-1][min(1, specs[-1][0]), 0].float() * (12.0 / math.sqrt(hd))
    q = q.to(dtype)
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=dtype)
    fill_cache(kv, tables, [(s + n, 0) for s, n in specs], k_all, v_all, P)
    out = torch.empty((M, nq * hd), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks.paged_attention(q.reshape(M, nq * hd).to(DEV), out, batch, LayerCache(0, kv.to(DEV), None, P, False),
                       num_heads=nq, window=Window("full", 0), softmax_scale=scale, sink_logit=sink)
    torch.cuda.synchronize()
    assert not ks.errors()
    assert ks.launches_by_library[library] > 0, dict(ks.launches_by_library)
    ref = sink_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, sink)
    close(out.view(M, nq, hd), ref, KTOL[dtype], f"attention with a sink of {sink} ({library})")
    # the sink matters: without it the first token of a request would return its own value unchanged
    first = sum(n for _, n in specs[:[s for s, _ in specs].index(0)])
    plain_first = v_all[[s for s, _ in specs].index(0)][0, 0].double()
    assert float((ref[first, 0] - plain_first).abs().max()) > 0.05


def test_key_splits_count_the_sink_once():
    """One decoded token over 20,000 keys: the decode kernel splits the keys among blocks and merges; all scores are
    small, so the sink's share is 1 / (n + 1) and a sink per split would show."""
    ks = kernels(torch.bfloat16)
    nq, nkv, hd, P, C = 4, 1, 64, 64, 20000
    for use_decode, library in ((True, "attention_decode"), (False, "attention_mma")):
        ks.use_decode_attention = use_decode
        n_pages = C // P + 2
        batch, tables = make_batch([(C - 1, 1)], P, n_pages, 70, DEV)
        g = torch.Generator(device=DEV).manual_seed(71)
        kv = torch.randn((2, n_pages, nkv, P, hd), generator=g, device=DEV) * 0.5
        kv[1] += 1.0                                         # values with a mean, so that the output is of order one
        kv = kv.to(torch.bfloat16)
        q = (torch.randn((1, nq, hd), generator=g, device=DEV) * 0.05).to(torch.bfloat16)
        out = torch.empty((1, nq * hd), dtype=torch.bfloat16, device=DEV)
        sink = 9.0                                           # exp(9) is about 8,100: two fifths of the key count
        ks.paged_attention(q.reshape(1, nq * hd), out, batch, LayerCache(0, kv, None, P, False), num_heads=nq,
                           window=Window("full", 0), softmax_scale=0.125, sink_logit=sink)
        assert ks.launches_by_library[library] > 0
        tbl = torch.tensor(tables[0], device=DEV)
        K = kv[0][tbl].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[0, :C].double()
        V = kv[1][tbl].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[0, :C].double()
        for h in range(nq):
            sc = (K @ q[0, h].double()) * 0.125
            e = torch.exp(sc)
            ref = (e / (e.sum() + math.exp(sink))) @ V
            no_sink = (e / e.sum()) @ V
            got = out.view(nq, hd)[h].double()
            assert float((got - ref).abs().max()) <= 0.02 * float(no_sink.abs().max()), library
            assert float((no_sink - ref).abs().max()) > 0.2 * float(no_sink.abs().max())     # the sink is visible


# ---------------------------------------------------------------------------- value heads of another size
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kd,vd", [(16, 24), (32, 8), (64, 40), (24, 24), (10, 6)])
def test_attention_part_with_value_heads_of_another_size(dtype, kd, vd):
    """The attention part alone, in an engine of one layer without a feed-forward: keys of size kd, values of
    size vd, a sink, its own score scale; against the plain mixer, whole and token by token."""
    from spite_b200.config import BlockSpec, LayerCall, ModelPlan, PartSpec
    from spite_b200.engine import Engine
    from spite_b200.engine.model import Model
    d, nq, nkv, V = 48, 6, 2, 50
    norm = PartSpec("rms_norm", {"size": d, "eps": 1e-5})
    mixer = PartSpec("paged_attention", {"hidden_size": d, "num_heads": nq, "num_kv_heads": nkv, "head_dim": kd,
                                         "value_dim": vd, "position": PartSpec("no_position", {}), "softmax_scale": 0.21,
                                         "sink_logit": 0.0})
    plan = ModelPlan(hidden_size=d, vocab_size=V, blocks=(BlockSpec("prenorm_residual", {"mixer_norm": norm, "mixer": mixer}),),
                     order=(LayerCall(0, 0, True),), final_norm=norm, tie_word_embeddings=True, max_positions=256)
    model = Model(plan, dtype=dtype, device=DEV)
    from spite_b200.kernels import build
    build.ensure_built(model.kernel_libraries())
    g = torch.Generator().manual_seed(kd * 100 + vd)
    params = {n: (torch.ones(s.shape) if s.init == "ones" else torch.randn(s.shape, generator=g) * 0.25).to(torch.bfloat16)
              for n, s in model.param_specs().items()}
    model.load_params(params)
    toks = H.random_tokens(V, 70, 5)
    P = {n: t.float() for n, t in params.items()}
    x = P["embed.weight"][torch.tensor(toks)]
    x = x + plain.sink_attention(plain.rms_norm(x, P["layers.0.mixer_norm.weight"], 1e-5), P["layers.0.mixer.q_proj"],
                                 P["layers.0.mixer.k_proj"], P["layers.0.mixer.v_proj"], P["layers.0.mixer.o_proj"],
                                 nq, nkv, kd, vd, 0.21)
    ref = plain.rms_norm(x, P["final_norm.weight"], 1e-5) @ P["embed.weight"].T
    reqs = {"a": toks}
    for steps in (H.steps_whole(reqs), H.steps_last_decoded(reqs, 20), H.steps_portions(reqs, seed=1)):
        eng = Engine(model, cache_tokens=128, page_size=16, max_requests=2)
        got = H.run_steps(eng, steps)
        worst = max(float((got[("a", p)] - ref[p]).abs().max()) for p in range(len(toks))) / float(ref.abs().max())
        assert worst <= TOL[dtype], f"kd {kd}, vd {vd}: {worst:.3e}"


# ---------------------------------------------------------------------------- squared-ReLU products
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 40, 48), (5, 200, 64), (13, 128, 192), (40, 72, 200), (64, 64, 64), (300, 136, 320),
                                   (700, 520, 128)])
def test_linear_with_squared_relu(dtype, M, N, K):
    """relu(s y)^2 in the epilogue of every product kernel a one-group product can reach (CUDA cores, weight
    streaming, mma.sync, tcgen05 on one block and on pairs), with and without a row scale."""
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn((M, K), generator=g).to(dtype)
    w = (torch.randn((N, K), generator=g) / math.sqrt(K)).to(dtype)
    s = torch.rand((M,), generator=g) + 0.25
    for scale in (None, s):
        out = torch.empty((M, N), dtype=dtype, device=DEV)
        ks.linear(x.to(DEV), w.to(DEV), out, activation="relu2", row_scale=None if scale is None else scale.to(DEV))
        y = x.double() @ w.double().T
        if scale is not None:
            y = y * scale.double()[:, None]
        close(out, torch.relu(y) ** 2, KTOL[dtype], f"relu2 product {M}x{N}x{K}")
    assert not ks.errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,E,F,K", [(1, 3, 24, 48), (9, 5, 40, 64), (150, 7, 72, 64), (64, 16, 48, 128), (900, 6, 136, 192),
                                     (2100, 3, 64, 64)])
def test_grouped_squared_relu_experts(dtype, M, E, F, K):
    """An expert's first product without a gate, grouped by expert: act(s_token * (x_token W_e^T)) in sorted order;
    some experts get no token."""
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(M + E)
    x = torch.randn((M, K), generator=g).to(dtype)
    w = (torch.randn((E, F, K), generator=g) / math.sqrt(K)).to(dtype)
    ids = torch.randint(0, E, (M,), generator=g)
    if E > 2:
        ids[ids == 1] = 0                                    # expert 1 stays empty
    scale = torch.rand((M,), generator=g) + 0.25
    order = torch.sort(ids, stable=True)
    rows = order.indices.to(torch.int32)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(torch.bincount(ids, minlength=E), 0)
    out = torch.empty((M, F), dtype=dtype, device=DEV)
    ks.grouped_linear_act(x.to(DEV), w.to(DEV), rows.to(DEV), offsets.to(DEV), scale.to(DEV), out, activation="relu2")
    ref = torch.empty((M, F), dtype=torch.float64)
    for i in range(M):
        t = int(rows[i])
        ref[i] = torch.relu(scale[t].double() * (w[int(ids[t])].double() @ x[t].double())) ** 2
    close(out, ref, KTOL[dtype], f"grouped relu2 product {M}x{E}x{F}x{K}")
    assert not ks.errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,d,E,top,f,fs", [(1, 64, 4, 2, 40, 0), (23, 96, 6, 3, 32, 48), (300, 128, 5, 1, 64, 128), (40, 100, 3, 3, 20, 12)])
def test_the_mixture_of_experts_without_gates_alone(dtype, M, d, E, top, f, fs):
    """The feed-forward part by itself: sigmoid scores, the `top` largest chosen, expert e fed with s_e * h (raw
    scores), relu(.)^2 between up and down, a shared expert of its own size."""
    from spite_b200.config import PartSpec
    from spite_b200.kernels import build
    from spite_b200.parts import BuildContext, build_part
    build.ensure_built(["elementwise", "gemm_simt", "gemm_stream", "gemm_skinny", "gemm_tc", "gemm_tc_pair", "gemm_tc_experts", "moe"])
    ks = kernels(dtype)
    part = build_part("feed_forward", PartSpec("moe_sigmoid_prescaled", {
        "hidden_size": d, "num_experts": E, "top_k": top, "expert_size": f, "shared_size": fs, "activation": "relu2"}),
        BuildContext(ks, dtype, torch.device(DEV)))
    g = torch.Generator().manual_seed(M + E)
    params = {n: (torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1])).to(torch.bfloat16) for n, s in part.param_specs().items()}
    params["router"] = (params["router"].float() * 6).to(torch.bfloat16)          # scores well apart from one half
    assert "experts_gate_up" not in params and "shared_gate_proj" not in params
    part.bind({n: t.to(DEV) for n, t in params.items()})
    x = torch.randn((M, d), generator=g).to(dtype)
    if dtype == torch.bfloat16:                              # keep tokens whose choice of experts rounding cannot change
        z = torch.sort(x.float() @ params["router"].float().T, descending=True).values
        if E > top:
            x = x[(z[:, top - 1] - z[:, top]) > 0.05]
    h = torch.zeros((x.shape[0], d), dtype=torch.float32, device=DEV)
    part.forward(x.to(DEV), h, None)
    torch.cuda.synchronize()
    P = {n: t.double() for n, t in params.items()}
    experts = [(P["experts_up"][e], P["experts_down"][e]) for e in range(E)]
    shared = (P["shared_up_proj"], P["shared_down_proj"]) if fs else None
    ref = plain.moe_ff(x.double(), P["router"], experts, top, shared)
    close(h, ref, 2e-2 if dtype == torch.bfloat16 else 1e-5, "mixture of experts without gates")


# ---------------------------------------------------------------------------- positions and the junction
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_learned_positions(dtype):
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(1)
    table = torch.randn((37, 100), generator=g).to(dtype)
    pos_table = torch.randn((64, 100), generator=g).to(dtype)
    toks = torch.randint(0, 37, (21,), generator=g).to(torch.int32)
    pos = torch.randint(0, 64, (21,), generator=g).to(torch.int32)
    h = torch.empty((21, 100), dtype=torch.float32, device=DEV)
    ks.embed(table.to(DEV), toks.to(DEV), h, scale=2.5, position_table=pos_table.to(DEV), positions=pos.to(DEV))
    ref = table[toks.long()].double() * 2.5 + pos_table[pos.long()].double()        # the factor applies to the token's row only
    close(h, ref, 1e-6, "embedding with positions")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,d", [(1, 64), (19, 100), (300, 128)])
def test_the_junction_of_a_loop(dtype, M, d):
    """h <- W [h; h0] + step[t] for every step vector, against the plain computation."""
    from spite_b200.parts import BuildContext, build_part
    from spite_b200.config import PartSpec
    from spite_b200.kernels import build
    build.ensure_built(["elementwise", "gemm_simt", "gemm_stream", "gemm_skinny", "gemm_tc", "gemm_tc_pair"])
    ks = kernels(dtype)
    part = build_part("junction", PartSpec("reinject_linear", {"hidden_size": d, "steps": 3}), BuildContext(ks, dtype, torch.device(DEV)))
    g = torch.Generator().manual_seed(M + d)
    w = (torch.randn((d, 2 * d), generator=g) / math.sqrt(2 * d)).to(torch.bfloat16)
    step = torch.randn((3, d), generator=g).to(torch.bfloat16)
    part.bind({"in_proj": w.to(DEV), "step": step.to(DEV)})
    h = torch.randn((M, d), generator=g)
    h0 = torch.randn((M, d), generator=g)
    for t in range(3):
        hd = h.clone().to(DEV)
        part.forward(hd, h0.to(DEV), None, t)
        a, b = (h.to(dtype), h0.to(dtype)) if dtype == torch.bfloat16 else (h, h0)       # the product's inputs are rounded
        ref = plain.loop_entry(a.double(), b.double(), w.double(), step[t].double())
        close(hd, ref, KTOL[dtype] if dtype == torch.bfloat16 else 1e-5, f"junction, step {t}")


# ---------------------------------------------------------------------------- the engine
@pytest.fixture(scope="module", params=list(S.CONFIGS))
def folder(request, tmp_path_factory):
    return S.write_model(tmp_path_factory.mktemp(f"sezazen_{request.param}"), request.param), request.param


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, folder):
    from spite_b200.engine import Model
    path, name = folder
    dtype = request.param
    model = Model.from_folder(path, dtype=dtype, device=DEV)
    vocab = model.plan.vocab_size
    lengths = {"a": 150 if name == "Q" else 83, "b": 40, "c": 37, "d": 66, "e": 1, "f": 21}
    if dtype == "float32":
        requests = {r: H.random_tokens(vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    else:
        requests = {r: S.decisive_tokens(path, n, i, MARGIN) for i, (r, n) in enumerate(lengths.items())}
    return path, model, requests, TOL[dtype], dtype


def _engine(model, steps, page_size):
    from spite_b200.engine import Engine
    return Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page_size, max_requests=4)


def poison_free_pages(engine):
    """Whatever a free page held last is not finite: a kernel that reads a masked key of a reused page shows it."""
    for g, pool in enumerate(engine.cache.pools):
        if pool._free:
            engine.storage.kv[g][:, :, torch.tensor(pool._free, device=DEV)] = float("nan")


def test_every_cut_gives_the_logits_of_the_whole_sequence(setup):
    path, model, requests, tol, dtype = setup
    n_prompt = {r: max(1, len(t) - 9) for r, t in requests.items()}
    cuts = {"whole": (H.steps_whole(requests), 64), "whole, small pages": (H.steps_whole(requests), 16),
            "last 32 decoded": (H.steps_last_decoded(requests, 32), 64),
            "portions": (H.steps_portions(requests, seed=4), 64),
            "portions of 2 and 3": (H.steps_portions(requests, seed=5, sizes=(2, 3)), 16),
            "mixed": (H.steps_mixed(requests, n_prompt, seed=6), 64),
            "mixed, small pages": (H.steps_mixed(requests, n_prompt, seed=7, sizes=(2, 5, 17, 40)), 16)}
    results = {}
    for what, (steps, page) in cuts.items():
        eng = _engine(model, steps, page)
        results[what] = H.run_steps(eng, steps, before_step=poison_free_pages)
        S.compare_with_plain(results[what], path, requests, tol)
        eng.check()
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what
    if dtype == "float32":
        H.assert_cuts_identical(results)


def test_the_residual_stream_layer_run_by_layer_run(setup):
    path, model, requests, tol, dtype = setup
    cfg, tensors = S.folder_contents(str(path))
    toks = requests["c"]
    _, layers = plain.forward(cfg, tensors, toks, return_layers=True)
    seen = []
    model.layer_tap = lambda i, h: seen.append(h.float().cpu())
    try:
        steps = H.steps_whole({"c": toks})
        H.run_steps(_engine(model, steps, 64), steps)
    finally:
        model.layer_tap = None
    assert len(seen) == layers.shape[0]
    for i, h in enumerate(seen):
        err = float((h - layers[i]).abs().max()) / float(layers[i].abs().max())
        assert err <= (2e-5 if dtype == "float32" else 3e-2), f"layer run {i}: {err:.3e}"


def test_long_decoding_after_a_short_prompt(setup):
    """Three prompt tokens, then 128 tokens one by one (decode steps replayed from CUDA graphs, pages taken one
    after the other)."""
    path, model, requests, tol, dtype = setup
    vocab = model.plan.vocab_size
    toks = H.random_tokens(vocab, 131, 77) if dtype == "float32" else S.decisive_tokens(path, 131, 77, MARGIN)
    reqs = {"long": toks}
    steps = H.steps_last_decoded(reqs, 128)
    S.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), path, reqs, tol)


def test_greedy_generation_through_the_entry_point(setup):
    """`LLM.generate` (scheduler, sampler, engine): the tokens are the plain implementation's argmax at every
    step where its best two logits are not within rounding of each other."""
    from spite_b200 import LLM
    path, model, requests, tol, dtype = setup
    cfg, tensors = S.folder_contents(str(path))
    prompts = [requests["b"][:30], requests["c"][:7], requests["f"][:2], requests["d"][:50]]
    llm = LLM(model, cache_tokens=4 * 128, page_size=16, max_requests=3, max_batch_tokens=24)
    outs = llm.generate(prompts, max_tokens=12, temperature=0.0)
    compared = 0
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        toks = list(prompt)
        for tok in out:
            row = plain.forward(cfg, tensors, toks)[-1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 2 * tol * float(row.abs().max()):
                assert tok == int(torch.argmax(row)), f"after {len(toks)} tokens"
                compared += 1
            toks.append(tok)                                 # follow the engine's own sequence
    assert compared >= 12


def test_trace_replay_program(folder, tmp_path):
    """`bin/trace_run` as a program: a mixed schedule in, logits files out, equal to the plain implementation."""
    import os, subprocess, sys
    import numpy as np
    from pathlib import Path
    path, name = folder
    vocab = json.loads((path / "config.json").read_text())["vocab"]
    requests = {r: H.random_tokens(vocab, n, 90 + i) for i, (r, n) in enumerate({"a": 70, "b": 33, "c": 5}.items())}
    steps = H.steps_mixed(requests, {r: len(t) - 4 for r, t in requests.items()}, seed=9)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(path), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(H.max_tokens_of(steps))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    pos, got = {}, {}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        i = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(rows[i].copy())
                i += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert i == rows.shape[0]
    S.compare_with_plain(got, path, requests, 2e-5)


def test_the_command_line_runs_a_sezazen_folder(tmp_path):
    """`spite random`, `spite run` (greedy, float32: the plain implementation's tokens) and `spite bench`."""
    import subprocess, sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spite = lambda *a: subprocess.run([sys.executable, str(root / "bin" / "spite")] + [str(x) for x in a],
                                      capture_output=True, text=True, timeout=900)
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(S.CONFIG_P))
    model = tmp_path / "model"
    assert spite("random", "--config", cfg_file, "--out", model, "--seed", 3, "--std", 0.08).returncode == 0
    cfg, W = plain.load_folder(model)
    prompt = H.random_tokens(300, 17, 2)
    proc = spite("run", "-m", model, "-p", " ".join(map(str, prompt)), "--max-tokens", 6, "--temperature", 0,
                 "--dtype", "fp32", "--page-size", 16, "--num-pages", 8)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == plain.generate_greedy(cfg, W, prompt, 6)
    proc = spite("bench", "-m", model, "--n-prompt", 40, "--n-tokens", 12, "--n-runs", 2, "--json", "--dtype", "bf16")
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads(proc.stdout)
    assert report["decode_tps"] > 0 and report["prefill_tps"] > 0
