"""Two mixers side by side that read the same input; their outputs add up (not in the reference).

    y += left(x) + right(x)

Each side is a mixer of its own kind with its own tensors (prefix ``left.`` / ``right.``) and its own cache or
state; a side's weight in the sum is that side's own ``out_scale`` parameter, so it costs no pass of its own.
"""
from __future__ import annotations

from .base import CacheBundle, Mixer
from .registry import build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    def __init__(self, left, right, prefix: str = ""):
        super().__init__(prefix)
        self.left = build_part("mixer", left)
        self.right = build_part("mixer", right)

    @property
    def graph_safe(self):
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def children(self):
        return [self.left, self.right]

    def cache_request(self):
        return CacheBundle.of(left=self.left.cache_request(), right=self.right.cache_request())

    def forward(self, x, step, cache, residual):
        self.left.forward(x, step, cache.get("left"), residual)
        self.right.forward(x, step, cache.get("right"), residual)
