"""A short causal convolution over time, one filter per channel, with the tail of its input as per-request state.

out[t] = act( bias + sum_j w[:, j] * x[t - taps + 1 + j]  (+ x[t]) ), zeros before the start of the sequence; the
last column of ``w`` is the current token's. With ``residual`` the input itself is added, which is the form that
stands in front of a sub-layer (the sub-layer then reads x + conv(x)); with an activation and a bias it is the form
inside state-space and delta-rule mixers. The last taps - 1 inputs of every request are kept, as float, in a state
of shape (taps - 1, channels), so a portion continues where the one before stopped, wherever the prompt was cut.
"""
from __future__ import annotations

from .base import CacheNeed, SequenceFilter, TensorDecl, register_part


@register_part("filter", "short_conv")
class ShortConv(SequenceFilter):
    """params: channels, taps, weight_name, bias_name (None: no bias), activation ("none" | "silu"), residual (bool),
    state_name (the name of its state among the layer's states; default "tail"); segments: instead of one weight,
    a list of (tensor name, channels) whose filters lie side by side (several convolutions run as one)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.channels = int(p["channels"])
        self.taps = int(p["taps"])
        if not (1 <= self.taps <= 16):
            raise ValueError(f"a short convolution has 1 to 16 taps, not {self.taps}")
        self.segments = [(self.prefix + n, int(c)) for n, c in p["segments"]] if p.get("segments") else \
            [(self.prefix + p.get("weight_name", "weight"), self.channels)]
        if sum(c for _, c in self.segments) != self.channels:
            raise ValueError("the segments of a short convolution must add up to its channels")
        self.bias_name = self.prefix + p["bias_name"] if p.get("bias_name") else None
        self.activation = p.get("activation", "none")
        if self.activation not in ("none", "silu"):
            raise ValueError(f"activation {self.activation!r} is not known (none, silu)")
        self.residual = bool(p.get("residual", False))
        self.state_name = p.get("state_name", "tail")
        self.weight = self.bias = None

    def tensor_decls(self):
        decls = [TensorDecl(n, (c, self.taps)) for n, c in self.segments]
        if self.bias_name:
            decls.append(TensorDecl(self.bias_name, (self.channels,)))
        return decls

    def load(self, tensors):
        import torch

        self.weight = torch.cat([tensors[n] for n, _ in self.segments], dim=0).contiguous()
        self.bias = tensors[self.bias_name].contiguous() if self.bias_name else None

    def cache_need(self):
        if self.taps == 1:
            return None
        return CacheNeed(states=((self.state_name, (self.taps - 1, self.channels)),))

    def forward(self, x, ctx, cache, out=None, prefix: str = ""):
        if out is None:
            out = self.rt.empty_act((x.shape[0], self.channels))
        state = cache.states[prefix + self.state_name] if self.taps > 1 else None
        self.rt.kernels.causal_conv(x, self.weight, self.bias, state, ctx, out, self.activation, self.residual)
        return out
