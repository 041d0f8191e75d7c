"""Differential attention over the paged cache, as a mixer (not in the reference).

Every query head carries two maps: q [heads · 2 · dim] and k [kv_heads · 2 · dim] are laid out head by head as
[map 1 | map 2]; query head h reads kv head h // (heads / kv_heads). Each map is a softmax attention of its own
over the SAME values v [kv_heads · vdim]:

    s = (q_m · k_m) · scale;   s ← cap · tanh(s / cap)  (cap None: no capping);   a_m = softmax(s) · v
    o = a_1 − λ · a_2,   λ = exp(Σ lq1 ⊙ lk1) − exp(Σ lq2 ⊙ lk2) + diff      (one number per layer)
    ô = o / sqrt(mean(o²) + eps) · (1 − diff)                                  (per head, no weight)
    y = Wo · concat_h(ô) + bo

Positions: the position part's frequencies turn neighbouring pairs (2i, 2i+1) over the first ``rotary_dim`` dims of
each map of each head of q and k. Visibility: a query at position p sees key j ≤ p when p − j < window (``window``
None: always) or j < keep_first; the kept first keys keep their true positions. q, k, v and the output may have
biases. Scores, weights, λ and the per-head norm are 32-bit in every mode.
"""
from __future__ import annotations

import math

import torch

from ..csrc import lib as K
from .base import KVCacheRequest, Mixer, WeightSpec
from .linear import Linear
from .registry import build_part, register_part
from ..phases import phase


@register_part("mixer", "diff_attention")
class DiffAttention(Mixer):
    graph_safe = True
    kernel_modules = ("seqmix",)
    kernel_modules_bf16 = ("diff_flash",)          # the tensor-core kernel of prompt steps

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, diff: float,
                 scale: float, eps: float, softcap=None, window=None, keep_first: int = 0, position=None,
                 bias: bool = True, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim = int(dim), int(vdim)
        self.diff, self.scale, self.eps = float(diff), float(scale), float(eps)
        self.softcap = float(softcap) if softcap else None
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.bias = bool(bias)
        n = dict(q="q", k="k", v="v", o="o", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2", bias_suffix=".b")
        n.update(names or {})
        self.bias_suffix = n.pop("bias_suffix")
        self.names = {k: prefix + v for k, v in n.items()}
        self.position = build_part("position", position) if position is not None else None
        if self.position is not None and getattr(self.position, "pairing", "half") != "interleaved":
            raise ValueError(f"{prefix}: this mixer's kernel rotates neighbouring pairs (pairing 'interleaved')")
        self.qkv = self.o = self.qkv_bias = self.o_bias = None
        self.lam = None

    def children(self):
        return [self.position] if self.position is not None else []

    def weight_specs(self):
        H, nh, g, d, vd = self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim
        shapes = dict(q=(nh * 2 * d, H), k=(g * 2 * d, H), v=(g * vd, H), o=(H, nh * vd))
        specs = [WeightSpec(self.names[k], s) for k, s in shapes.items()]
        if self.bias:
            specs += [WeightSpec(self.names[k] + self.bias_suffix, (s[0],)) for k, s in shapes.items()]
        return specs + [WeightSpec(self.names[k], (d,)) for k in ("lq1", "lk1", "lq2", "lk2")]

    def cache_request(self):
        return KVCacheRequest(self.num_kv_heads, 2 * self.dim, self.window, v_head_dim=self.vdim,
                              keep_first=self.keep_first)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        q, k, v = (tensors[self.names[n]] for n in ("q", "k", "v"))
        self.qkv = Linear(torch.cat([q, k, v], dim=0))
        self.o = Linear(tensors[self.names["o"]])
        if self.bias:
            self.qkv_bias = torch.cat([tensors[self.names[n] + self.bias_suffix] for n in ("q", "k", "v")]).contiguous()
            self.o_bias = tensors[self.names["o"] + self.bias_suffix].contiguous()
        l = {n: tensors[self.names[n]].float().cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        # one number per layer, in 32-bit like everything that weighs the maps
        self.lam = float(torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum())
                         + torch.tensor(self.diff, dtype=torch.float32))

    def forward(self, x, step, cache, residual):
        nh, g, d, vd = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        T = x.shape[0]
        inv_freq, rd = self.position.rotary() if self.position is not None else (None, 0)
        with phase("qkv_projection_ms"):
            qkv = self.qkv(x, out_dtype=torch.float32)             # bias and rotation read unrounded products
        with phase("rotary+kv_append_ms"):
            q = torch.empty(T, nh * 2 * d, dtype=self.rt.act_dtype, device=x.device)
            # the output bias enters the stream here, ahead of the output projection that accumulates into it
            K.diff_qkv_store(qkv, self.qkv_bias, q, cache.k_pool, cache.v_pool, cache, inv_freq, 2 * nh, 2 * g, g, d, vd, rd,
                             residual if self.o_bias is not None else None, self.o_bias)
        with phase("attention_ms"):
            ctx = torch.empty(T, nh * vd, dtype=self.rt.act_dtype, device=x.device)
            args = (nh, g, d, vd, self.window, self.keep_first, self.scale, self.softcap, self.lam, self.eps, 1.0 - self.diff)
            if (not step.all_single and q.dtype == torch.bfloat16 and cache.k_pool.dtype == torch.bfloat16
                    and K.diff_flash_supported(d, vd, nh, g, cache.page_size)):
                # a prompt step: 64 queries per CTA on the tensor cores, both maps over one fetch of the values
                tiles = K.query_tiles(step.host["new_counts"], K.diff_flash_query_tile())
                K.diff_flash_prefill(q, cache.k_pool, cache.v_pool, ctx, cache, step.seq_start, step.n_seqs, tiles, *args)
            else:
                K.diff_attention(q, cache.k_pool, cache.v_pool, ctx, cache, *args)
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)
