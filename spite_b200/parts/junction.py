"""Junctions: what happens to the residual stream between two layers of the run order.

`reinject_linear`: h <- W [h; h0] + b[step].  The stream is mixed with the embedding's output h0 through
one matrix [d, 2d] (the columns that multiply h first), and a learned vector of the pass is added.  A
model that applies a range of its layers repeatedly puts this before every pass.
The product runs in the activation type with float32 sums; the vector and the sum are float32.
"""
from __future__ import annotations

import torch

from ..config.specs import ConfigError
from .base import Junction, ParamSpec, register_junction


@register_junction("reinject_linear")
class ReinjectLinear(Junction):
    graph_safe = True
    kernel_libraries = ("elementwise", "gemm_simt")

    def __init__(self, ctx, hidden_size: int, steps: int):
        super().__init__(ctx)
        if steps < 1:
            raise ConfigError("a junction needs at least one step vector")
        self.d, self.steps = int(hidden_size), int(steps)
        self.w = self.bias = None

    def param_specs(self):
        return {"in_proj": ParamSpec((self.d, 2 * self.d)), "step": ParamSpec((self.steps, self.d))}

    def bind(self, params):
        self.w = params["in_proj"].to(self.ctx.dtype).contiguous()
        self.bias = params["step"].to(torch.float32).contiguous()       # added in float32; a bfloat16 vector converts exactly

    def weight_bytes(self):
        return self.w.numel() * self.w.element_size() + self.bias.numel() * 4

    def forward(self, h, h0, batch, step: int):
        if not 0 <= step < self.steps:
            raise ConfigError(f"junction step {step} outside its {self.steps} vectors")
        x = torch.empty((h.shape[0], 2 * self.d), dtype=self.ctx.dtype, device=h.device)
        # x = [h; h0] in the activation type, and h becomes the pass's vector in every row: the product is then
        # added to it like every other product that ends in the residual stream
        self.k.pack_pair(h, h0, x, refill=self.bias[step])
        self.k.linear(x, self.w, h, accumulate=True)
