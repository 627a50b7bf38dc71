"""RMS norm with a gain vector (crates/spite-models/src/dense.rs:175-181).  `gain_offset` serves checkpoints that
store the gain as its distance from a constant (around zero for a gain around one): the gain applied is
`gain_offset + weight`."""
from __future__ import annotations

import torch

from .base import Norm, ParamSpec, register_norm


@register_norm("rms_norm")
class RmsNorm(Norm):
    graph_safe = True
    kernel_libraries = ("elementwise",)

    def __init__(self, ctx, size: int, eps: float, gain_offset: float = 0.0):
        super().__init__(ctx)
        self.size, self.eps, self.gain_offset = int(size), float(eps), float(gain_offset)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), "normal" if self.gain_offset else "ones")}

    def bind(self, params):
        # the gain is applied in float32; a bfloat16 gain converts exactly
        self.weight = params["weight"].to(torch.float32).contiguous()
        if self.gain_offset:
            self.weight = (self.weight + self.gain_offset).contiguous()     # one float32 sum, as the formula has it

    def weight_bytes(self):
        return self.weight.numel() * 4

    def forward(self, h, out, rows=None):
        self.k.rms_norm(h, self.weight, self.eps, out, rows)
        return out
