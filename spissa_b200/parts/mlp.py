"""Feed-forwards.

PolyNorm feed-forward: down( a·N(z) + b·N(z²) + c·N(z³) + e ) with z = x·Wupᵀ, powers element by element and
N(v) = v / sqrt(mean(v²) + eps) over a token's row; (a, b, c, e) is a learned tensor of four numbers (not in the
reference). The activation runs in 32-bit on the unrounded product.

SwiGLU feed-forward: down( silu(x·Wgᵀ) ⊙ (x·Wuᵀ) ), silu(z) = z / (1 + e^{-z}).

crates/spissa-runtime/src/models/llama/generate.rs:590-637 (gate, up), :642-763 (down);
crates/spissa-runtime/src/ops.rs:192-194 (silu). Gate and up run as one matrix product
over the stacked weight [Wg; Wu]; the down projection adds into the residual stream.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import FeedForward, WeightSpec
from .linear import GatedLinear, Linear
from .registry import register_part
from ..phases import phase


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.gate_up = self.down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["gate"], (I, H)), WeightSpec(self.names["up"], (I, H)),
                WeightSpec(self.names["down"], (H, I))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        if g.dtype != u.dtype:
            raise ValueError(f"{self.prefix}: gate and up projections must share a storage type")
        self.gate_up = GatedLinear(g, u)
        self.down = Linear(tensors[self.names["down"]])

    def fused_fields(self):
        gu = self.gate_up
        if gu is None or not gu.block or gu.weight.dtype != torch.bfloat16 or self.down.weight.dtype != torch.bfloat16:
            return None
        return dict(kind="swiglu", gate_up=gu.weight, pair=gu.block, down=self.down.weight,
                    hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    def forward(self, x, step, residual):
        with phase("gate_projection+up_projection+activation_multiply_ms"):
            act = self.gate_up(x, self.rt.act_dtype)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)


@register_part("ffn", "polynorm")
class PolyNormMLP(FeedForward):
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size, self.eps = int(hidden_size), int(intermediate_size), float(eps)
        n = dict(up="up", down="down", act="act")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.up = self.down = self.coef = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["up"], (I, H)), WeightSpec(self.names["down"], (H, I)),
                WeightSpec(self.names["act"], (4,), init="const:0.5")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.up = Linear(tensors[self.names["up"]])
        self.down = Linear(tensors[self.names["down"]])
        self.coef = tensors[self.names["act"]].contiguous()

    def forward(self, x, step, residual):
        with phase("up_projection_ms"):
            z = self.up(x, out_dtype=torch.float32)                # the activation's statistics read unrounded products
        with phase("activation_ms"):
            act = torch.empty(x.shape[0], self.intermediate_size, dtype=self.rt.act_dtype, device=x.device)
            K.polynorm(z, self.coef, act, self.eps)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)
