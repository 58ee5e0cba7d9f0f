"""Two mixers side by side on the same input: out = left_scale * left(h) + right_scale * right(h).

Both sides end in a plain output projection, so the sum is one product: each side writes what its projection
would read, already times its scale, into its own columns of one buffer, and the two projection matrices lie
side by side as one matrix. The layer's cache is that of both: the pages of the side that has keys, and the
states of both under the names "left.*" and "right.*".
"""
from __future__ import annotations

import torch

from .base import CacheNeed, Mixer, build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    """params: hidden, left (PartSpec of a mixer), right (PartSpec), left_scale, right_scale."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.left = build_part("mixer", p["left"], runtime)
        self.right = build_part("mixer", p["right"], runtime)
        self.left_scale, self.right_scale = float(p["left_scale"]), float(p["right_scale"])
        for side in (self.left, self.right):
            if side.mixed_size is None:
                raise ValueError(f"mixer {side.spec.kind!r} does not offer its output projection apart; it cannot stand in a parallel pair")
        self.mixed_size = self.left.mixed_size + self.right.mixed_size
        self.w_o = None

    def tensor_decls(self):
        return self.left.tensor_decls() + self.right.tensor_decls()

    def ignorable_tensors(self):
        return self.left.ignorable_tensors() + self.right.ignorable_tensors()

    def load(self, tensors):
        self.left.load(tensors)
        self.right.load(tensors)
        self.w_o = torch.cat([self.left.output_weight(), self.right.output_weight()], dim=1).contiguous()

    def cache_need(self):
        return CacheNeed.merged([("left.", self.left.cache_need()), ("right.", self.right.cache_need())])

    def output_weight(self):
        return self.w_o

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        n = self.left.mixed_size
        self.left.mix_into(h, ctx, cache.sub("left."), out[:, :n], scale * self.left_scale)
        self.right.mix_into(h, ctx, cache.sub("right."), out[:, n:], scale * self.right_scale)

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.linear(mixed, self.w_o, out)
        return out
