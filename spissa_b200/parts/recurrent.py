"""Mixers that carry a fixed-size state instead of keys and values (not in the reference).

Retention: linear attention with one fixed decay per head and neither softmax nor denominator.
    q, k [heads·dim], v, g [heads·vdim] = projections of x (no bias);  per head, with S₀ = 0 [dim, vdim]:
    S_t = γ_h · S_{t-1} + (k_t / √dim) v_tᵀ,   o_t = S_tᵀ q_t,   ô_t = o_t / sqrt(mean(o_t²) + eps);
    y_t = Wo · ( concat_h(ô_t) ⊙ silu(g_t) ).

minGRU: a gated recurrence whose gates read the current token only.
    z_t = sigmoid(Wz x_t + bz),  u_t = Wx x_t + bx,  c_t = u_t + ½ where u_t ≥ 0 and sigmoid(u_t) where u_t < 0;
    S_t = (1 − z_t) ⊙ S_{t-1} + z_t ⊙ c_t  (S₀ = 0),   y_t = Wo · ( S_t ⊙ silu(Wg x_t) ).

Both states are 32-bit and belong to the sequence's slot; the recurrences run in 32-bit on the unrounded
projections, which are one matrix product over the stacked weights.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Mixer, StateRequest, WeightSpec
from .linear import Linear
from .registry import register_part
from ..phases import phase


@register_part("mixer", "retention")
class Retention(Mixer):
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay, eps: float, prefix: str = "",
                 names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.dim, self.vdim = int(hidden_size), int(num_heads), int(dim), int(vdim)
        self.decay_values = [float(g) for g in decay]
        if len(self.decay_values) != self.num_heads:
            raise ValueError(f"{prefix}: {len(self.decay_values)} decays for {self.num_heads} heads")
        self.eps = float(eps)
        n = dict(q="q", k="k", v="v", g="g", o="o")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.proj = self.o = self.decay = None

    def weight_specs(self):
        H, nh, d, vd = self.hidden_size, self.num_heads, self.dim, self.vdim
        return [WeightSpec(self.names["q"], (nh * d, H)), WeightSpec(self.names["k"], (nh * d, H)),
                WeightSpec(self.names["v"], (nh * vd, H)), WeightSpec(self.names["g"], (nh * vd, H)),
                WeightSpec(self.names["o"], (H, nh * vd))]

    def cache_request(self):
        return StateRequest((self.num_heads, self.dim, self.vdim), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(torch.cat([tensors[self.names[k]] for k in ("q", "k", "v", "g")], dim=0))
        self.o = Linear(tensors[self.names["o"]])
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)

    def forward(self, x, step, cache, residual):
        with phase("mixer_projection_ms"):
            p = self.proj(x, out_dtype=torch.float32)
        with phase("retention_ms"):
            y = torch.empty(x.shape[0], self.num_heads * self.vdim, dtype=self.rt.act_dtype, device=x.device)
            K.retention(p, cache.state, self.decay, y, step, self.num_heads, self.dim, self.vdim, self.eps)
        with phase("o_projection+mixer_residual_ms"):
            self.o(y, out=residual, accumulate=True)


@register_part("mixer", "mingru")
class MinGRU(Mixer):
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, hidden_size: int, width: int, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.width = int(hidden_size), int(width)
        n = dict(z="z", zb="z.b", x="x", xb="x.b", g="g", o="o")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.proj = self.o = self.zb = self.xb = None

    def weight_specs(self):
        H, W = self.hidden_size, self.width
        return [WeightSpec(self.names["z"], (W, H)), WeightSpec(self.names["zb"], (W,)),
                WeightSpec(self.names["x"], (W, H)), WeightSpec(self.names["xb"], (W,)),
                WeightSpec(self.names["g"], (W, H)), WeightSpec(self.names["o"], (H, W))]

    def cache_request(self):
        return StateRequest((self.width,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(torch.cat([tensors[self.names[k]] for k in ("z", "x", "g")], dim=0))
        self.o = Linear(tensors[self.names["o"]])
        self.zb = tensors[self.names["zb"]].contiguous()
        self.xb = tensors[self.names["xb"]].contiguous()

    def forward(self, x, step, cache, residual):
        with phase("mixer_projection_ms"):
            p = self.proj(x, out_dtype=torch.float32)
        with phase("mingru_ms"):
            y = torch.empty(x.shape[0], self.width, dtype=self.rt.act_dtype, device=x.device)
            K.mingru(p, self.zb, self.xb, cache.state, y, step, self.width)
        with phase("o_projection+mixer_residual_ms"):
            self.o(y, out=residual, accumulate=True)
