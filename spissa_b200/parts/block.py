"""The pre-norm arrangement of a layer: h += mixer(norm(h)); h += ffn(norm(h)).

crates/spissa-runtime/src/models/llama/generate.rs:190-199 (norm before attention),
:459 (first residual sum), :465-471 (norm before the feed-forward), :773 (second sum).
The residual stream ``h`` is 32-bit in every mode; mixer and feed-forward add into it.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Block, CacheBundle, StateRequest, WeightSpec
from .registry import build_part, register_part
from ..phases import phase


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, mixer, ffn, norms: dict, prefix: str = ""):
        super().__init__(prefix)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn)
        self.mixer_norm = build_part("norm", norms["mixer"])
        self.ffn_norm = build_part("norm", norms["ffn"])

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_request(self):
        return self.mixer.cache_request()

    def fused_fields(self):
        f = dict(kind="prenorm", mixer_norm=self.mixer_norm.fused_fields(), mixer=self.mixer.fused_fields(),
                 ffn_norm=self.ffn_norm.fused_fields(), ffn=self.ffn.fused_fields())
        return None if any(v is None for v in f.values()) else f

    def forward(self, h, step, cache):
        with phase("attention_norm_ms"):
            x = self.mixer_norm.forward(h)
        self.mixer.forward(x, step, cache, h)
        with phase("mlp_norm_ms"):
            x = self.ffn_norm.forward(h)
        self.ffn.forward(x, step, h)


@register_part("block", "prenorm_shift")
class ShiftedPreNormBlock(Block):
    """The pre-norm arrangement with a token shift in front of the mixer:

        a_t = norm(h_t);  x_t = a_t + (a_{t-1} − a_t) ⊙ mu;  h += mixer(x);  h += ffn(norm(h))

    with a_{-1} = 0 and ``mu`` a learned vector (``shift_name``). The last a of a sequence is state: the block asks
    the cache for one row of the stream's width per run beside whatever its mixer asks for, and hands the mixer the
    view named "mixer". The feed-forward sees no shift and may be absent (``ffn`` None). When the norm describes itself
    as dynamic tanh, norm and shift run as one kernel on the 32-bit stream."""
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, mixer, ffn, norms: dict, hidden_size: int, shift_name: str, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.shift_name = shift_name
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.mixer_norm = build_part("norm", norms["mixer"])
        self.ffn_norm = build_part("norm", norms["ffn"]) if ffn is not None else None
        self.mu = None

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def weight_specs(self):
        return [WeightSpec(self.shift_name, (self.hidden_size,))]

    def cache_request(self):
        return CacheBundle.of(mixer=self.mixer.cache_request(), shift=StateRequest((self.hidden_size,), torch.float32))

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.mu = tensors[self.shift_name].contiguous()

    def forward(self, h, step, cache):
        state = cache["shift"].state
        x = torch.empty(h.shape[0], self.hidden_size, dtype=self.rt.act_dtype, device=h.device)
        with phase("mixer_norm+shift_ms"):
            f = self.mixer_norm.fused_fields()
            if f is not None and f.get("kind") == "dyt":
                K.token_shift(h, self.mu, state, x, step, dyt=(f["weight"], f["bias"], f["alpha"]))
            else:
                K.token_shift(self.mixer_norm.forward(h), self.mu, state, x, step)
        self.mixer.forward(x, step, cache.get("mixer"), h)
        if self.ffn is not None:
            with phase("mlp_norm_ms"):
                x = self.ffn_norm.forward(h)
            self.ffn.forward(x, step, h)
