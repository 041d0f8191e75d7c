"""Mixers that carry a fixed-size state instead of keys and values (not in the reference).

Retention: linear attention with one fixed decay per head and neither softmax nor denominator.
    q, k [heads·dim], v, g [heads·vdim] = projections of x (no bias);  per head, with S₀ = 0 [dim, vdim]:
    S_t = γ_h · S_{t-1} + (k_t / √dim) v_tᵀ,   o_t = S_tᵀ q_t,   ô_t = o_t / sqrt(mean(o_t²) + eps);
    y_t = Wo · ( concat_h(ô_t) ⊙ silu(g_t) ).

minGRU: a gated recurrence whose gates read the current token only.
    z_t = sigmoid(Wz x_t + bz),  u_t = Wx x_t + bx,  c_t = u_t + ½ where u_t ≥ 0 and sigmoid(u_t) where u_t < 0;
    S_t = (1 − z_t) ⊙ S_{t-1} + z_t ⊙ c_t  (S₀ = 0),   y_t = Wo · ( S_t ⊙ silu(Wg x_t) ).

Gated linear attention: linear attention whose state decays per key channel by a gate that reads the token.
    q, k [heads·dim], v, g [heads·vdim] = projections of x (no bias), q times dim^(−1/2);
    z = Wa2 (Wa1 x) + b [heads·dim] through a low rank,  α_t = sigmoid(z_t)^(1/τ);  per head, with S₀ = 0 [dim, vdim]:
    S_t = diag(α_t) S_{t-1} + k_t v_tᵀ,   o_t = S_tᵀ q_t,   ô_t = o_t / sqrt(mean(o_t²) + eps) ⊙ w  (w [vdim], shared by heads);
    y_t = Wo · ( concat_h(ô_t) ⊙ silu(g_t) ) · out_scale.

All states are 32-bit and belong to the sequence's slot; the recurrences run in 32-bit on the unrounded
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


@register_part("mixer", "gla")
class GatedLinearAttention(Mixer):
    """``rank`` is the size of the low-rank input of the decays; None: the checkpoint's tensors say it (random weights
    then take 16)."""
    graph_safe = True
    kernel_modules = ("hybrid",)

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, tau: float, eps: float,
                 rank: int | None = None, out_scale: float = 1.0, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.dim, self.vdim = int(hidden_size), int(num_heads), int(dim), int(vdim)
        self.tau, self.eps, self.out_scale = float(tau), float(eps), float(out_scale)
        if not self.tau > 0:
            raise ValueError(f"{prefix}: tau must be positive")
        self.rank = int(rank) if rank else None
        n = dict(q="q", k="k", v="v", g="g", o="o", a1="a1", a2="a2", a2b="a2.b", norm="norm")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.proj = self.o = self.a2 = self.a2b = self.norm = None

    def weight_specs(self):
        H, nh, d, vd, r = self.hidden_size, self.num_heads, self.dim, self.vdim, self.rank or -16
        return [WeightSpec(self.names["q"], (nh * d, H)), WeightSpec(self.names["k"], (nh * d, H)),
                WeightSpec(self.names["v"], (nh * vd, H)), WeightSpec(self.names["g"], (nh * vd, H)),
                WeightSpec(self.names["o"], (H, nh * vd)), WeightSpec(self.names["a1"], (r, H)),
                WeightSpec(self.names["a2"], (nh * d, r)), WeightSpec(self.names["a2b"], (nh * d,)),
                WeightSpec(self.names["norm"], (vd,), init="ones")]

    def cache_request(self):
        return StateRequest((self.num_heads, self.dim, self.vdim), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        a1, a2 = tensors[self.names["a1"]], tensors[self.names["a2"]]
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{self.prefix}: the two halves of the decay projection disagree on the rank "
                             f"({a1.shape[0]} and {a2.shape[1]})")
        self.rank = int(a1.shape[0])
        self.proj = Linear(torch.cat([tensors[self.names[k]] for k in ("q", "k", "v", "g", "a1")], dim=0))
        self.o = Linear(tensors[self.names["o"]])
        self.a2 = a2.contiguous()
        self.a2b = tensors[self.names["a2b"]].contiguous()
        self.norm = tensors[self.names["norm"]].contiguous()

    def forward(self, x, step, cache, residual):
        with phase("mixer_projection_ms"):
            p = self.proj(x, out_dtype=torch.float32)              # the recurrence reads unrounded products
        with phase("gla_ms"):
            y = torch.empty(x.shape[0], self.num_heads * self.vdim, dtype=self.rt.act_dtype, device=x.device)
            K.gla(p, cache.state, self.a2, self.a2b, self.norm, y, step, self.num_heads, self.dim, self.vdim, self.rank,
                  self.tau, self.eps, self.out_scale)
        with phase("o_projection+mixer_residual_ms"):
            self.o(y, out=residual, accumulate=True)
