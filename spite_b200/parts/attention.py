"""Grouped-query attention over the paged cache.

One part serves every attention layer: the window rule (all keys, the keys of
the query's chunk, the last W keys), the position encoding, the per-head norm of
q and k (after or before the rotation, with gains or without), the
temperature factor, a value size that differs from the key size, and a sink in
the softmax (an extra term exp(sink) in the sum, with nothing behind it) are constructor parameters.

Formulas: crates/spite-models/src/llama/llama4.rs:126-207 (projections, rotation
then norm, temperature factor on layers without rotation, append to the cache,
attention, output projection added to the residual stream) and
crates/spite-compute/src/flash_attn.rs:111-156 (scores, mask, softmax, values).
"""
from __future__ import annotations

import math

import torch

from ..cache import PagedKV, Window
from ..config.specs import ConfigError, PartSpec
from .base import Mixer, ParamSpec, QkNorm, build_part, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    graph_safe = True
    kernel_libraries = ("gemm_simt", "attention", "attention_mma", "attention_rows", "attention_tc", "attention_decode")

    def __init__(self, ctx, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window=("full", 0), qk_norm_eps=None, qk_norm_gain=False,
                 qk_norm_before_rotation=False, temperature_tuning=None, softmax_scale=None,
                 value_dim=None, sink_logit=None):
        """`head_dim` is the size of a query and a key head, `value_dim` that of a value head (default: the
        same).  `sink_logit`, if given, is the score of a sink: a term exp(sink) in every softmax's sum that adds
        nothing to the output, p_j = exp(s_j) / (exp(sink) + sum exp(s_j'))."""
        super().__init__(ctx)
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads evenly")
        if head_dim % 2 or head_dim > 256:
            raise ConfigError(f"head_dim {head_dim} must be even and at most 256")
        self.d, self.nq, self.nkv = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.kd = int(head_dim)
        self.vd = int(value_dim) if value_dim else self.kd
        if self.vd < 1 or self.vd > 256:
            raise ConfigError(f"value_dim {self.vd} must lie in 1..256")
        self.sink_logit = None if sink_logit is None else float(sink_logit)
        self.window = window if isinstance(window, Window) else Window(window[0], int(window[1]))
        self.position = build_part("position", position, ctx)
        # Keys and values share the cache's pages and the attention kernels' tiles, which have one row size.  Where
        # the two sizes differ it is the larger one, in bfloat16 rounded up to the tensor-core kernels' step of 16.  The projection
        # matrices get zero rows (and the output projection zero columns) for the padding, so the padded
        # elements are exact zeros: they add nothing to a score and come out of the attention as zeros.
        # A rotation or a per-head norm would have to know which elements of a row are padding: a layer
        # with either keeps its rows as they are.
        may_pad = qk_norm_eps is None and self.position.rotation() is None
        hd = max(self.kd, self.vd)
        step = 16 if self.vd != self.kd and ctx.dtype == torch.bfloat16 and hd <= 128 else 2
        self.hd = -(-hd // step) * step
        if self.hd != self.kd and not may_pad:
            raise ConfigError(f"a value size {self.vd} other than the key size {self.kd} cannot be combined "
                              f"with a rotation or a per-head norm of q and k")
        # only the attention kernels that these sizes can reach are compiled for the model
        libs = ["gemm_simt", "attention"]
        if ctx.dtype == torch.bfloat16 and self.hd % 16 == 0 and self.hd <= 128 and self.nq // self.nkv <= 16:
            libs += ["attention_mma", "attention_rows"]
            if self.hd in (64, 128):
                libs += ["attention_tc", "attention_decode"]
        self.kernel_libraries = tuple(libs)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.qk_norm_gain = bool(qk_norm_gain) and self.qk_norm_eps is not None
        self.qk_norm_before_rotation = bool(qk_norm_before_rotation)
        self.qk_norm = None if self.qk_norm_eps is None else QkNorm(self.qk_norm_eps, self.qk_norm_before_rotation)
        if temperature_tuning is not None:
            floor, scale = temperature_tuning
            if float(floor) != int(floor) or int(floor) < 1:
                raise ConfigError(f"temperature floor_scale {floor} must be a positive integer")
            temperature_tuning = (int(floor), float(scale))
        self.temperature = temperature_tuning
        self.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.kd)
        self.wqkv = self.wo = None

    def param_specs(self):
        d, nq, nkv, kd, vd = self.d, self.nq, self.nkv, self.kd, self.vd
        specs = {"q_proj": ParamSpec((nq * kd, d)), "k_proj": ParamSpec((nkv * kd, d)),
                 "v_proj": ParamSpec((nkv * vd, d)), "o_proj": ParamSpec((d, nq * vd))}
        if self.qk_norm_gain:
            specs.update({"q_norm": ParamSpec((kd,), "ones"), "k_norm": ParamSpec((kd,), "ones")})
        return specs

    def _pad_heads(self, w, heads, size):
        """[heads * size, d] -> [heads * hd, d]: every head's rows followed by zero rows up to the cache's row size."""
        if size == self.hd:
            return w
        out = torch.zeros((heads, self.hd, w.shape[1]), dtype=w.dtype, device=w.device)
        out[:, :size] = w.view(heads, size, w.shape[1])
        return out.view(heads * self.hd, w.shape[1])

    def bind(self, params):
        dt = self.ctx.dtype
        # q, k and v rows in one matrix: one product per layer instead of three
        self.wqkv = torch.cat([self._pad_heads(params["q_proj"].to(dt), self.nq, self.kd),
                               self._pad_heads(params["k_proj"].to(dt), self.nkv, self.kd),
                               self._pad_heads(params["v_proj"].to(dt), self.nkv, self.vd)], 0).contiguous()
        # the output projection's columns, head by head, with zero columns for the padding
        self.wo = self._pad_heads(params["o_proj"].to(dt).t().contiguous(), self.nq, self.vd).t().contiguous()
        if self.qk_norm_gain:
            self.qk_norm = QkNorm(self.qk_norm_eps, self.qk_norm_before_rotation,
                                  params["q_norm"].to(torch.float32).contiguous(),
                                  params["k_norm"].to(torch.float32).contiguous())

    def weight_bytes(self):
        return (self.wqkv.numel() + self.wo.numel()) * self.wqkv.element_size()

    def cache_request(self):
        return PagedKV(self.window, self.nkv, self.hd), None

    def forward(self, x, h, batch, cache):
        M = x.shape[0]
        k = self.k
        qkv = torch.empty((M, (self.nq + 2 * self.nkv) * self.hd), dtype=x.dtype, device=x.device)
        k.linear(x, self.wqkv, qkv)
        q = torch.empty((M, self.nq * self.hd), dtype=x.dtype, device=x.device)
        k.qk_prepare(qkv, q, batch, cache, num_heads=self.nq, rotation=self.position.rotation(),
                     qk_norm=self.qk_norm, temperature=self.temperature)
        o = torch.empty_like(q)
        # keys and values of earlier positions were cached by earlier steps; this step's own were written by
        # the prepare kernel just before, which is what the attention kernel waits for
        k.paged_attention(q, o, batch, cache, num_heads=self.nq, window=self.window,
                          softmax_scale=self.softmax_scale, cache_settled=True, sink_logit=self.sink_logit)
        k.linear(o, self.wo, h, accumulate=True)
