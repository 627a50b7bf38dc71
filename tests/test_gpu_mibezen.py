"""Mibezen on the GPU.  First every new mechanism alone against a plain computation written here from its equation
(distance bias, per-head sinks and head gates in every attention kernel; caches of one plane; blended values and
gate columns in the prepare kernel; the latent kernels; products per head; the softmax router with weighted
outputs; the mixers as parts); then the engine in float32 and bfloat16 against the plain implementation in every
cut (whole, token by token, portions down to two tokens, mixed batches in a pool whose pages and slots are used
again, free pages poisoned), long decoding, greedy generation through `LLM.generate`, and `bin/trace_run`."""
import json
import math

import pytest
import torch

import helpers as H
import mibezen_helpers as Z
import plain_mibezen as plain
from spite_b200.cache import LayerCache, Window
from spite_b200.parts import Rotation
from test_gpu_kernels import close, fill_cache, make_batch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
KTOL = {torch.float32: 1e-5, torch.bfloat16: 1.2e-2}
MARGIN = 0.03           # router logit margin that bfloat16 rounding cannot flip at these sizes


def kernels(dtype):
    from spite_b200.kernels.cuda import CudaKernels
    return CudaKernels(dtype, DEV)


# ---------------------------------------------------------------------------- bias, sinks and gates, kernel by kernel
def biased_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, sinks, slopes, gates):
    """p_j = exp(s_j - slope_h (i - j)) / (exp(sink_h) + sum over the visible j'), times the gate; float64 loops."""
    out = torch.zeros(q.shape[:2] + (v_all[0].shape[-1],), dtype=torch.float64)
    group, off = nq // nkv, 0
    for s, (start, n) in enumerate(specs):
        for t in range(n):
            pos = start + t
            lo = window.lowest_visible(pos)
            js = torch.arange(lo, pos + 1)
            for h in range(nq):
                sc = (k_all[s][lo:pos + 1, h // group].double() @ q[off + t, h].double()) * scale
                if slopes is not None:
                    sc = sc - float(slopes[h]) * (pos - js).double()
                m = float(sc.max()) if sinks is None else max(float(sc.max()), float(sinks[h]))
                e = torch.exp(sc - m)
                den = e.sum() + (0.0 if sinks is None else math.exp(float(sinks[h]) - m))
                o = (e / den) @ v_all[s][lo:pos + 1, h // group].double()
                out[off + t, h] = o * (1.0 if gates is None else float(gates[off + t, h]))
        off += n
    return out


# (kernel library that must serve the call, dtype, query heads, kv heads, row size, page size, window, segments)
BIAS_CASES = [
    ("attention", torch.float32, 5, 1, 24, 16, ("chunk", 50), [(0, 1), (0, 60), (130, 1), (99, 3)]),
    ("attention", torch.bfloat16, 6, 3, 24, 16, ("full", 0), [(0, 1), (0, 40), (130, 1), (61, 7)]),
    ("attention", torch.float32, 3, 3, 300, 16, ("full", 0), [(0, 9), (40, 1)]),                 # a row of more than 256 elements
    ("attention_mma", torch.bfloat16, 4, 2, 48, 16, ("chunk", 200), [(0, 1), (199, 1), (200, 1), (398, 3), (1500, 1)]),
    ("attention_rows", torch.bfloat16, 6, 2, 32, 32, ("chunk", 40), [(0, 45), (100, 30), (0, 12), (78, 4)]),
    ("attention_decode", torch.bfloat16, 8, 2, 64, 64, ("full", 0), [(0, 1), (63, 1), (64, 1), (3000, 1), (517, 2)]),
    ("attention_decode", torch.bfloat16, 8, 4, 128, 64, ("chunk", 100), [(99, 1), (100, 1), (299, 1), (250, 1)]),
    ("attention_tc", torch.bfloat16, 6, 2, 64, 64, ("chunk", 200), [(0, 300), (150, 130), (0, 70)]),
    ("attention_tc", torch.bfloat16, 4, 1, 128, 64, ("full", 0), [(0, 140), (900, 64)]),
]


@pytest.mark.parametrize("case", range(len(BIAS_CASES)))
def test_bias_sinks_and_gates_in_every_attention_kernel(case):
    """Slopes from strong to weak, sinks of both signs and gates between 0 and 1; small scores, so that bias and sink
    shape every softmax, and one row whose query is aligned with the first key it may see (far away, or just inside its
    chunk): a bias with the wrong sign or distance, a sink left out or counted per key split, a gate on the wrong head
    and a chunk border one token off all show."""
    library, dtype, nq, nkv, hd, P, win, specs = BIAS_CASES[case]
    ks = kernels(dtype)
    window = Window(*win)
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 3
    batch, tables = make_batch(specs, P, n_pages, 60 + case, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(61 + case)
    k_all = [torch.randn((s + n, nkv, hd), generator=g).to(dtype) for s, n in specs]
    v_all = [torch.randn((s + n, nkv, hd), generator=g).to(dtype) for s, n in specs]
    q = torch.randn((M, nq, hd), generator=g) * 0.3
    last_pos = specs[-1][0] + specs[-1][1] - 1
    first_seen = window.lowest_visible(last_pos)
    q[M - 1, nq - 1] = k_all[-1][first_seen, nkv - 1].float() * (12.0 / math.sqrt(hd))       # the weakest slope looks far back
    q = q.to(dtype)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq)])
    sinks = torch.randn(nq, generator=g) * 1.5
    gates = torch.rand((M, nq), generator=g)
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=dtype)
    fill_cache(kv, tables, [(s + n, 0) for s, n in specs], k_all, v_all, P)
    out = torch.empty((M, nq * hd), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks.paged_attention(q.reshape(M, nq * hd).to(DEV), out, batch, LayerCache(0, kv.to(DEV), None, P, False),
                       num_heads=nq, window=window, softmax_scale=scale, head_sinks=sinks.to(DEV),
                       head_slopes=slopes.to(DEV), head_gates=gates.to(DEV))
    torch.cuda.synchronize()
    assert not ks.errors()
    assert ks.launches_by_library[library] > 0, dict(ks.launches_by_library)
    ref = biased_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, sinks, slopes, gates)
    close(out.view(M, nq, hd), ref, KTOL[dtype], f"attention with bias, sinks and gates ({library})")
    # each of the three matters in the reference itself
    for what, other in (("slopes", biased_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, sinks, None, gates)),
                        ("sinks", biased_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, None, slopes, gates))):
        assert float((other - ref).abs().max()) > 0.05, what
    if first_seen > 0:                                       # the key just outside the window is not seen
        wider = Window("full", 0) if win[0] == "full" else Window("chunk", 10 ** 6)
        assert float((biased_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, wider, sinks, slopes, gates) - ref).abs().max()) > 1e-3


def test_key_splits_count_a_head_sink_once_and_carry_the_bias():
    """One decoded token over 20,000 keys: the decode kernels split the keys among blocks and merge.  Scores are small,
    so the sink's share is large and a sink per split would show; the slope of the last head is so weak that keys
    thousands of positions back still count."""
    ks = kernels(torch.bfloat16)
    nq, nkv, hd, P, C = 4, 1, 64, 64, 20000
    slopes = torch.tensor([0.02, 0.005, 0.001, 0.0002], device=DEV)
    sinks = torch.tensor([3.0, 5.0, 6.5, 8.0], device=DEV)
    for use_decode, library in ((True, "attention_decode"), (False, "attention_mma")):
        ks.use_decode_attention = use_decode
        n_pages = C // P + 2
        batch, tables = make_batch([(C - 1, 1)], P, n_pages, 70, DEV)
        g = torch.Generator(device=DEV).manual_seed(71)
        kv = torch.randn((2, n_pages, nkv, P, hd), generator=g, device=DEV) * 0.5
        kv[1] += 1.0
        kv = kv.to(torch.bfloat16)
        q = (torch.randn((1, nq, hd), generator=g, device=DEV) * 0.05).to(torch.bfloat16)
        out = torch.empty((1, nq * hd), dtype=torch.bfloat16, device=DEV)
        ks.paged_attention(q.reshape(1, nq * hd), out, batch, LayerCache(0, kv, None, P, False), num_heads=nq,
                           window=Window("full", 0), softmax_scale=0.125, head_sinks=sinks, head_slopes=slopes)
        assert ks.launches_by_library[library] > 0
        tbl = torch.tensor(tables[0], device=DEV)
        K = kv[0][tbl].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[0, :C].double()
        V = kv[1][tbl].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[0, :C].double()
        dist = (C - 1 - torch.arange(C, device=DEV)).double()
        for h in range(nq):
            e = torch.exp((K @ q[0, h].double()) * 0.125 - float(slopes[h]) * dist)
            ref = (e / (e.sum() + math.exp(float(sinks[h])))) @ V
            no_sink = (e / e.sum()) @ V
            got = out.view(nq, hd)[h].double()
            assert float((got - ref).abs().max()) <= 0.02 * float(no_sink.abs().max()), (library, h)
            assert float((no_sink - ref).abs().max()) > 0.1 * float(no_sink.abs().max())


# (library, dtype, heads, row size, page size, segments): one kv head whose key rows are also the values
ONE_PLANE_CASES = [
    ("attention", torch.float32, 5, 36, 16, [(0, 20), (77, 1)]),
    ("attention", torch.float32, 3, 520, 16, [(0, 6), (30, 1)]),
    ("attention_mma", torch.bfloat16, 4, 112, 16, [(0, 1), (300, 1), (31, 2)]),
    ("attention_rows", torch.bfloat16, 4, 48, 32, [(0, 40), (100, 24)]),
    ("attention_decode", torch.bfloat16, 8, 128, 64, [(0, 1), (1000, 1), (64, 1)]),
    ("attention_tc", torch.bfloat16, 8, 64, 64, [(0, 200), (130, 64)]),
    ("attention_tc", torch.bfloat16, 16, 128, 64, [(0, 150)]),
]


@pytest.mark.parametrize("case", range(len(ONE_PLANE_CASES)))
def test_a_cache_of_one_plane_serves_keys_and_values(case):
    library, dtype, nq, hd, P, specs = ONE_PLANE_CASES[case]
    ks = kernels(dtype)
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 2
    batch, tables = make_batch(specs, P, n_pages, 80 + case, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(81 + case)
    k_all = [torch.randn((s + n, 1, hd), generator=g).to(dtype) for s, n in specs]
    q = (torch.randn((M, nq, hd), generator=g) * 0.5).to(dtype)
    gates = torch.rand((M, nq), generator=g)
    two = torch.zeros((2, n_pages, 1, P, hd), dtype=dtype)
    fill_cache(two, tables, [(s + n, 0) for s, n in specs], k_all, k_all, P)
    out = torch.empty((M, nq * hd), dtype=dtype, device=DEV)
    ks.paged_attention(q.reshape(M, nq * hd).to(DEV), out, batch, LayerCache(0, two[:1].contiguous().to(DEV), None, P, False),
                       num_heads=nq, window=Window("full", 0), softmax_scale=0.2, head_gates=gates.to(DEV))
    torch.cuda.synchronize()
    assert ks.launches_by_library[library] > 0, dict(ks.launches_by_library)
    ref = biased_attention_reference(q, k_all, k_all, specs, nq, 1, 0.2, Window("full", 0), None, None, gates)
    close(out.view(M, nq, hd), ref, KTOL[dtype], f"keys as values ({library})")
    # the same result laid out head by head
    by_head = torch.empty((nq * M, hd), dtype=dtype, device=DEV)
    ks.paged_attention(q.reshape(M, nq * hd).to(DEV), by_head, batch, LayerCache(0, two[:1].contiguous().to(DEV), None, P, False),
                       num_heads=nq, window=Window("full", 0), softmax_scale=0.2, head_gates=gates.to(DEV), out_by_head=True)
    torch.cuda.synchronize()
    assert torch.equal(by_head.view(nq, M, hd).transpose(0, 1).contiguous().view(M, nq * hd), out)


# ---------------------------------------------------------------------------- the prepare kernel's additions
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,vd,other_hd", [(6, 3, 16, 16, 16), (4, 2, 32, 20, 24), (7, 1, 10, 6, 10)])
def test_prepare_blends_values_and_makes_gates(dtype, nq, nkv, hd, vd, other_hd):
    ks = kernels(dtype)
    P, n_pages = 16, 10
    specs = [(0, 19), (30, 1), (15, 3)]
    batch, tables = make_batch(specs, P, n_pages, 20, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(nq * 10 + hd)
    cols = (nq + 2 * nkv) * hd
    width = cols + nq + (-nq % 8)
    qkv = torch.randn((M, width), generator=g).to(dtype)
    other_cols = 5 * other_hd + nkv * other_hd + 3           # the other layer's row: something before, its values, something after
    other = torch.randn((M, other_cols), generator=g).to(dtype)
    lam = 0.37
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=dtype, device=DEV)
    q_out = torch.empty((M, nq * hd), dtype=dtype, device=DEV)
    gates = torch.empty((M, nq), dtype=torch.float32, device=DEV)
    ks.qk_prepare(qkv.to(DEV), q_out, batch, LayerCache(0, kv, None, P, True), num_heads=nq, rotation=None, qk_norm=None,
                  temperature=None, value_mix=(other.to(DEV), 5 * other_hd, other_hd, vd, lam), gates_out=gates)
    torch.cuda.synchronize()
    close(gates, torch.sigmoid(qkv[:, cols:cols + nq].double()), 1e-6, "gates")
    assert torch.equal(q_out.cpu(), qkv[:, :nq * hd])
    t = 0
    for s, (start, n) in enumerate(specs):
        for i in range(n):
            pos = start + i
            page = tables[s][pos // P]
            for kvh in range(nkv):
                k_row = kv[0, page, kvh, pos % P].cpu()
                v_row = kv[1, page, kvh, pos % P].cpu().double()
                assert torch.equal(k_row, qkv[t, (nq + kvh) * hd:(nq + kvh + 1) * hd])
                v = qkv[t, (nq + nkv + kvh) * hd:(nq + nkv + kvh + 1) * hd].double()
                o = other[t, 5 * other_hd + kvh * other_hd: 5 * other_hd + kvh * other_hd + vd].double()
                want = v.clone()
                want[:vd] = (1 - lam) * v[:vd] + lam * o
                assert float((v_row - want).abs().max()) <= (1e-6 if dtype == torch.float32 else 2e-2), (t, kvh)
            t += 1


# ---------------------------------------------------------------------------- the latent kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,dn,dr,rq,rkv,row", [(3, 16, 8, 40, 40, 48), (5, 12, 6, 22, 30, 36), (8, 32, 32, 64, 96, 128), (2, 8, 64, 16, 200, 264)])
def test_latent_prepare_and_queries(dtype, nq, dn, dr, rq, rkv, row):
    ks = kernels(dtype)
    P, n_pages = 16, 16
    specs = [(0, 19), (130, 1), (15, 3)]
    batch, tables = make_batch(specs, P, n_pages, 30, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(nq + row)
    inv_freq = (torch.rand(dr // 2, generator=g) * 0.9 + 0.01).to(torch.float32)
    rot = Rotation(inv_freq.to(DEV), "neighbours", dr, 1.23)
    cols = rq + rkv + dr + nq
    down = torch.randn((M, cols + 3), generator=g)
    qg, kg = torch.randn(rq, generator=g), torch.randn(rkv, generator=g)
    kv = torch.full((1, n_pages, 1, P, row), 7.0, dtype=dtype, device=DEV)
    cq = torch.empty((M, rq), dtype=dtype, device=DEV)
    gates = torch.empty((M, nq), dtype=torch.float32, device=DEV)
    ks.latent_prepare(down.to(DEV), cq, batch, LayerCache(0, kv, None, P, True), q_rank=rq, kv_rank=rkv, rotation=rot,
                      q_gain=qg.to(DEV), kv_gain=kg.to(DEV), eps=1e-3, num_gates=nq, gates_out=gates)
    q = torch.randn((M, nq * (dn + dr)), generator=g).to(dtype)
    qa = torch.full((M, nq * row), 5.0, dtype=dtype, device=DEV)
    rows = torch.empty(nq * M, dtype=torch.int32, device=DEV)
    offs = torch.empty(nq + 1, dtype=torch.int32, device=DEV)
    qs = torch.empty((nq * M, dn), dtype=dtype, device=DEV)
    ks.latent_queries(q.to(DEV), qa, batch, num_heads=nq, head_dim=dn, kv_rank=rkv, rotation=rot, rows_out=rows, offsets_out=offs,
                      sorted_out=qs)
    torch.cuda.synchronize()
    assert torch.equal(qs.cpu().view(nq, M, dn), q.view(M, nq, dn + dr)[:, :, :dn].transpose(0, 1))
    tol = 1e-5 if dtype == torch.float32 else 1.2e-2
    d64 = down.double()

    def norm(x, w):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3) * w.double()

    def turn(v, pos):
        out = v.clone()
        for i in range(dr // 2):
            a = float(torch.tensor(pos, dtype=torch.float32) * inv_freq[i])      # the angle is a float32 product
            c, s = math.cos(a) * 1.23, math.sin(a) * 1.23
            out[..., 2 * i] = v[..., 2 * i] * c - v[..., 2 * i + 1] * s
            out[..., 2 * i + 1] = v[..., 2 * i + 1] * c + v[..., 2 * i] * s
        return out
    close(cq, norm(d64[:, :rq], qg), tol, "query latent")
    close(gates, torch.sigmoid(d64[:, rq + rkv + dr:rq + rkv + dr + nq]), 1e-6, "gates")
    assert rows.view(nq, M).cpu().tolist() == [[m * nq + h for m in range(M)] for h in range(nq)]
    assert offs.cpu().tolist() == [h * M for h in range(nq + 1)]
    t = 0
    qav = qa.view(M, nq, row).cpu().double()
    for s, (start, n) in enumerate(specs):
        for i in range(n):
            pos = start + i
            got = kv[0, tables[s][pos // P], 0, pos % P].cpu().double()
            want = torch.zeros(row, dtype=torch.float64)
            want[:rkv] = norm(d64[t, rq:rq + rkv], kg)
            want[rkv:rkv + dr] = turn(d64[t, rq + rkv:rq + rkv + dr], pos)
            assert float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), f"cache row of token {t}"
            qw = turn(q[t].double().view(nq, dn + dr)[:, dn:], pos)
            assert float((qav[t, :, rkv:rkv + dr] - qw).abs().max()) <= tol * max(1.0, float(qw.abs().max()))
            assert float(qav[t, :, rkv + dr:].abs().max()) == 0.0 if row > rkv + dr else True
            assert float((qav[t, :, :rkv] - 5.0).abs().max()) == 0.0               # left for the product that follows
            t += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,G,K,N,lda,ldc", [(1, 4, 32, 96, 48, 112), (7, 3, 16, 40, 24, 48), (40, 8, 64, 128, 96, 160), (300, 4, 96, 32, 128, 32),
                                              (700, 2, 128, 64, 192, 64), (5, 5, 12, 30, 18, 36), (16, 16, 64, 64, 64, 128)])
def test_products_per_head(dtype, M, G, K, N, lda, ldc):
    """out[m, g, :N] = a[m, g, :K] @ w[g]^T over (token, head) rows listed head by head; what lies beyond K and N stays."""
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(M + G + K)
    a = (torch.randn((M * G, lda), generator=g) * 0.5).to(dtype)
    w = (torch.randn((G, N, K), generator=g) / math.sqrt(K)).to(dtype)
    out = torch.full((M * G, ldc), 3.0, dtype=dtype, device=DEV)
    rows = torch.tensor([m * G + h for h in range(G) for m in range(M)], dtype=torch.int32, device=DEV)
    offs = torch.tensor([h * M for h in range(G + 1)], dtype=torch.int32, device=DEV)
    ks.grouped_linear_rows(a.to(DEV), w.to(DEV), rows, offs, out)
    torch.cuda.synchronize()
    assert not ks.errors()
    ref = torch.einsum("mgk,gnk->mgn", a.double().view(M, G, lda)[:, :, :K], w.double())
    close(out.view(M, G, ldc)[:, :, :N], ref, KTOL[dtype], "product per head")
    if ldc > N:
        assert float((out.view(M, G, ldc)[:, :, N:].float() - 3.0).abs().max()) == 0.0
    # the same with the rows of `a` laid out head by head already
    out2 = torch.full((M * G, ldc), 3.0, dtype=dtype, device=DEV)
    a_sorted = a.view(M, G, lda).transpose(0, 1).reshape(G * M, lda).contiguous()
    ks.grouped_linear_rows(a_sorted.to(DEV), w.to(DEV), rows, offs, out2, a_sorted=True)
    torch.cuda.synchronize()
    close(out2.view(M, G, ldc)[:, :, :N], ref, KTOL[dtype], "product per head, rows in place")


# ---------------------------------------------------------------------------- router and experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,d,E,top,f", [(1, 64, 4, 2, 40), (23, 96, 6, 3, 32), (300, 128, 16, 3, 64), (40, 100, 3, 3, 20), (700, 64, 5, 1, 48)])
def test_the_softmax_router_with_weighted_outputs_alone(dtype, M, d, E, top, f):
    from spite_b200.config import PartSpec
    from spite_b200.kernels import build
    from spite_b200.parts import BuildContext, build_part
    build.ensure_built(["elementwise", "gemm_simt", "gemm_stream", "gemm_skinny", "gemm_tc", "gemm_tc_pair", "gemm_tc_experts", "moe"])
    ks = kernels(dtype)
    part = build_part("feed_forward", PartSpec("moe_softmax_topk", {"hidden_size": d, "num_experts": E, "top_k": top, "expert_size": f}),
                      BuildContext(ks, dtype, torch.device(DEV)))
    g = torch.Generator().manual_seed(M + E)
    params = {n: (torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1])).to(torch.bfloat16) for n, s in part.param_specs().items()}
    params["router"] = (params["router"].float() * 6).to(torch.bfloat16)          # shares far from uniform
    part.bind({n: t.to(DEV) for n, t in params.items()})
    x = torch.randn((M, d), generator=g).to(dtype)
    if dtype == torch.bfloat16 and E > top:                  # keep tokens whose choice of experts rounding cannot change
        z = torch.sort(x.float() @ params["router"].float().T, descending=True).values
        x = x[(z[:, top - 1] - z[:, top]) > 0.05]
    h = torch.zeros((x.shape[0], d), dtype=torch.float32, device=DEV)
    part.keep_router_logits = True
    part.forward(x.to(DEV), h, None)
    torch.cuda.synchronize()
    W = {"router": params["router"].double()}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = (params[n][e].double() for n in ("experts_gate", "experts_up", "experts_down"))
    ref = plain.moe_ff(x.double(), W, {"router": {"experts": E, "top": top}})
    close(h, ref, 2e-2 if dtype == torch.bfloat16 else 1e-5, "softmax router, weighted outputs")
    r = part.last_routing
    assert float((r.weights.sum(0) - 1.0).abs().max()) < 1e-5                   # the chosen shares are renormalised
    for s in range(top):
        assert torch.equal(r.sorted_weights[s], r.weights[s][r.sorted_rows[s].long()])


# ---------------------------------------------------------------------------- the mixers as parts
def one_layer_model(mixer_spec, d, V, dtype, seed, tune=None, std=0.25):
    from spite_b200.config import BlockSpec, LayerCall, ModelPlan, PartSpec
    from spite_b200.engine.model import Model
    from spite_b200.kernels import build
    norm = PartSpec("rms_norm", {"size": d, "eps": 1e-5})
    plan = ModelPlan(hidden_size=d, vocab_size=V, blocks=(BlockSpec("prenorm_residual", {"mixer_norm": norm, "mixer": mixer_spec}),),
                     order=(LayerCall(0, 0, True),), final_norm=norm, tie_word_embeddings=True, max_positions=1024)
    model = Model(plan, dtype=dtype, device=DEV)
    build.ensure_built(model.kernel_libraries())
    g = torch.Generator().manual_seed(seed)
    params = {n: (torch.ones(s.shape) if s.init == "ones" else torch.randn(s.shape, generator=g) * std).to(torch.bfloat16)
              for n, s in model.param_specs().items()}
    if tune:
        tune(params, g)
    model.load_params(params)
    return model, {n: t.float() for n, t in params.items()}


def run_cuts(model, toks, ref, tol, what, single=1.0):
    """Every position's logits in three cuts.  `single` > 1 lets single positions reach `single * tol` while the median
    stays under a quarter of `tol` (a model of one layer with a tied head has positions where one rounded key moves the
    result several times as far as usual, in every order of the roundings)."""
    from spite_b200.engine import Engine
    reqs = {"a": toks}
    for steps in (H.steps_whole(reqs), H.steps_last_decoded(reqs, 20), H.steps_portions(reqs, seed=1, sizes=(2, 3, 5, 17))):
        eng = Engine(model, cache_tokens=192, page_size=16, max_requests=2)
        got = H.run_steps(eng, steps)
        eng.check()
        errs = torch.tensor([float((got[("a", p)] - ref[p]).abs().max()) for p in range(len(toks))]) / float(ref.abs().max())
        assert float(errs.max()) <= tol * single, f"{what}: {float(errs.max()):.3e} at position {int(errs.argmax())}"
        assert single == 1.0 or float(errs.median()) <= tol / 4, f"{what}: median {float(errs.median()):.3e}"


def plain_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,dn,dr,dv,rq,rkv,scaling", [(3, 16, 8, 24, 40, 40, (8.0, 64, 4.0, 0.5)), (4, 32, 32, 32, 64, 96, None),
                                                       (5, 12, 6, 10, 22, 30, (3.0, 16, 2.0, 1.0)), (2, 8, 16, 8, 24, 280, None),
                                                       (20, 8, 8, 8, 32, 24, (2.0, 32, 4.0, 1.0))])
def test_latent_attention_part_alone(dtype, nq, dn, dr, dv, rq, rkv, scaling):
    """The latent mixer in an engine of one layer: against the expanded form (keys and values of every head made from
    every position's latent), whole, token by token and in portions."""
    from spite_b200.config import PartSpec
    d, V = 48, 50
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    spec = PartSpec("latent_attention", {
        "hidden_size": d, "num_heads": nq, "head_dim": dn, "rotary_dim": dr, "value_dim": dv, "q_rank": rq, "kv_rank": rkv,
        "softmax_scale": 0.3, "norm_eps": 1e-5, "head_gate": True,
        "position": PartSpec("rotary_yarn", {"rotary_dim": dr, "theta": 300.0, "scaling": sc})})

    def tune(p, g):
        for n in ("layers.0.mixer.q_latent_norm", "layers.0.mixer.kv_latent_norm"):
            p[n] = (1.0 + 0.3 * torch.randn(p[n].shape, generator=g)).to(torch.bfloat16)
        p["layers.0.mixer.gate_proj"] = (p["layers.0.mixer.gate_proj"].float() * 4).to(torch.bfloat16)
    # (moderate weights: with scores of tens, one bfloat16 rounding of a key moves a softmax by several per cent in
    # every implementation)
    model, P = one_layer_model(spec, d, V, dtype, nq * 100 + rkv, tune, std=0.17)
    toks = H.random_tokens(V, 90, 5)
    x = P["embed.weight"][torch.tensor(toks)]
    m = {"heads": nq, "dim": dn, "rot_dim": dr, "vdim": dv, "kv_rank": rkv, "scale": 0.3, "rot": {"base": 300.0, "dims": dr, "scaling": sc}}
    W = {"dq": "q_down", "dq.norm": "q_latent_norm", "uq": "q_up", "dkv": "kv_down", "dkv.norm": "kv_latent_norm", "uk": "k_up",
         "uv": "v_up", "g": "gate_proj", "o": "o_proj"}
    W = {k: P["layers.0.mixer." + v] for k, v in W.items()}
    x = x + plain.latent_attention(plain_norm(x, P["layers.0.mixer_norm.weight"], 1e-5), W, m, 1e-5)
    ref = plain_norm(x, P["final_norm.weight"], 1e-5) @ P["embed.weight"].T
    run_cuts(model, toks, ref, TOL[dtype], f"latent attention {nq} heads, row {rkv}+{dr}", single=2.0 if dtype == "bfloat16" else 1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,kd,vd,chunk", [(6, 3, 16, 16, 24), (8, 2, 64, 64, 64), (7, 1, 10, 6, 7), (4, 4, 32, 48, 0), (4, 2, 128, 128, 50), (5, 5, 9, 7, 11)])
def test_attention_part_with_bias_sinks_gate_and_chunk_alone(dtype, nq, nkv, kd, vd, chunk):
    from spite_b200.config import PartSpec
    d, V = 48, 50
    slopes = tuple(2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq))
    spec = PartSpec("paged_attention", {"hidden_size": d, "num_heads": nq, "num_kv_heads": nkv, "head_dim": kd, "value_dim": vd,
                                        "position": PartSpec("no_position", {}), "softmax_scale": 0.21,
                                        "window": ("chunk", chunk) if chunk else ("full", 0), "head_sinks": True,
                                        "distance_slopes": slopes, "head_gate": True})

    def tune(p, g):
        p["layers.0.mixer.sinks"] = (torch.randn(nq, generator=g) * 1.5).to(torch.bfloat16)
        p["layers.0.mixer.gate_proj"] = (p["layers.0.mixer.gate_proj"].float() * 4).to(torch.bfloat16)
    model, P = one_layer_model(spec, d, V, dtype, nq * 100 + kd, tune)
    toks = H.random_tokens(V, 90, 6)
    x = P["embed.weight"][torch.tensor(toks)]
    m = {"heads": nq, "kv_heads": nkv, "dim": kd, "vdim": vd, "scale": 0.21}
    if chunk:
        m["mask"] = {"size": chunk}
    W = {k: P["layers.0.mixer." + v] for k, v in {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "gate_proj", "o": "o_proj", "sink": "sinks"}.items()}
    y, _ = plain.chunk_attention(plain_norm(x, P["layers.0.mixer_norm.weight"], 1e-5), W, m, None, None)
    ref = plain_norm(x + y, P["final_norm.weight"], 1e-5) @ P["embed.weight"].T
    run_cuts(model, toks, ref, TOL[dtype], f"attention {nq}/{nkv} heads of {kd}/{vd}, chunk {chunk}")


# ---------------------------------------------------------------------------- the engine
@pytest.fixture(scope="module", params=list(Z.CONFIGS))
def folder(request, tmp_path_factory):
    return Z.write_model(tmp_path_factory.mktemp(f"mibezen_{request.param}"), request.param), request.param


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, folder):
    from spite_b200.engine import Model
    path, name = folder
    dtype = request.param
    model = Model.from_folder(path, dtype=dtype, device=DEV)
    vocab = model.plan.vocab_size
    lengths = {"a": 210 if name == "V" else 97, "b": 40, "c": 37, "d": 66, "e": 1, "f": 21}
    if dtype == "float32":
        requests = {r: H.random_tokens(vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    else:
        requests = {r: Z.decisive_tokens(path, n, i, MARGIN) for i, (r, n) in enumerate(lengths.items())}
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
        Z.compare_with_plain(results[what], path, requests, tol)
        eng.check()
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what
    if dtype == "float32":
        H.assert_cuts_identical(results)


def test_the_residual_stream_layer_by_layer(setup):
    path, model, requests, tol, dtype = setup
    cfg, tensors = Z.folder_contents(str(path))
    toks = requests["c"]
    layers = []
    plain.forward(cfg, tensors, toks, tap=lambda i, x: layers.append(x.clone()))
    seen = []
    model.layer_tap = lambda i, h: seen.append(h.float().cpu())
    try:
        steps = H.steps_whole({"c": toks})
        H.run_steps(_engine(model, steps, 64), steps)
    finally:
        model.layer_tap = None
    assert len(seen) == len(layers)
    for i, h in enumerate(seen):
        err = float((h - layers[i]).abs().max()) / float(layers[i].abs().max())
        assert err <= (2e-5 if dtype == "float32" else 3e-2), f"layer {i}: {err:.3e}"


def test_long_decoding_after_a_short_prompt(setup):
    """Three prompt tokens, then 160 tokens one by one (decode steps replayed from CUDA graphs, pages taken one after
    the other, every chunk of the configuration crossed while decoding)."""
    path, model, requests, tol, dtype = setup
    vocab = model.plan.vocab_size
    toks = H.random_tokens(vocab, 163, 77) if dtype == "float32" else Z.decisive_tokens(path, 163, 77, MARGIN)
    reqs = {"long": toks}
    steps = H.steps_last_decoded(reqs, 160)
    eng = _engine(model, steps, 16)
    Z.compare_with_plain(H.run_steps(eng, steps), path, reqs, tol)
    assert eng.graph_replays > 100


def test_greedy_generation_through_the_entry_point(setup):
    """`LLM.generate` (scheduler, sampler, engine): the tokens are the plain implementation's argmax at every
    step where its best two logits are not within rounding of each other."""
    from spite_b200 import LLM
    path, model, requests, tol, dtype = setup
    cfg, tensors = Z.folder_contents(str(path))
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
    import subprocess, sys
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
    Z.compare_with_plain(got, path, requests, 2e-5)


def test_the_command_line_runs_a_mibezen_folder(tmp_path):
    """`spite random`, `spite run` (greedy, float32: the plain implementation's tokens) and `spite bench`."""
    import subprocess, sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spite = lambda *a: subprocess.run([sys.executable, str(root / "bin" / "spite")] + [str(x) for x in a],
                                      capture_output=True, text=True, timeout=900)
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(Z.CONFIG_U))
    model = tmp_path / "model"
    assert spite("random", "--config", cfg_file, "--out", model, "--seed", 3, "--std", 0.08).returncode == 0
    cfg, W = plain.load_folder(model)
    prompt = H.random_tokens(300, 17, 2)
    proc = spite("run", "-m", model, "-p", " ".join(map(str, prompt)), "--max-tokens", 6, "--temperature", 0,
                 "--dtype", "fp32", "--page-size", 16, "--num-pages", 8)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == Z.generate_greedy(cfg, W, prompt, 6)
    proc = spite("bench", "-m", model, "--n-prompt", 40, "--n-tokens", 12, "--n-runs", 2, "--json", "--dtype", "bf16")
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads(proc.stdout)
    assert report["decode_tps"] > 0 and report["prefill_tps"] > 0
