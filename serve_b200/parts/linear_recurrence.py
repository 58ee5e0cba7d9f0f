"""Mixers that carry a matrix state per head from token to token instead of a cache of keys.

All three keep S [dk, dv] per (request, head) in float and differ in how a token changes it:

  "lightning"    S <- decay_h S + k v^T,  o = S^T q          q, k, v = silu of their projections; decay_h fixed per head
  "mamba2"       S <- exp(-exp(A_h) dt) S + dt B x^T,  y = S^T C + D_h x      dt = softplus(dt' + bias_h); x, B, C pass a
                 short convolution and silu first; heads share B and C in groups
  "gated_delta"  S <- g . S (a decay per row of S);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                 q, k, v pass a short convolution and silu, q and k become unit vectors, q times dk^-1/2

The read-out goes through a root-mean-square norm with a gate (parts/gated_norm.py) and an output projection.
One kernel walks the tokens of every request of the step in order (csrc/sequence_ops.cu), so a prompt cut into
portions, or decoded token by token, runs the same arithmetic in the same order as the whole prompt at once.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PartSpec
from .base import CacheNeed, Mixer, TensorDecl, build_part, register_part


class RecurrentMixer(Mixer):
    """What the three share: input projections fused into one product, a float read-out, norm and gate, output projection."""

    def _common(self, p):
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.eps = float(p["eps"])
        self.names = dict(p.get("names", {}))

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def output_weight(self):
        return self.w_o

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.linear(mixed, self.w_o, out)
        return out

    def _readout(self, t):
        return torch.empty((t, self.mixed_size), dtype=torch.float32, device=self.rt.device)


@register_part("mixer", "lightning")
class LightningMixer(RecurrentMixer):
    """params: hidden, heads, dim, vdim, decay (one per head), eps."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.decay_values = [float(d) for d in p["decay"]]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.heads} heads")
        self.mixed_size = self.heads * self.vdim
        self.norm = build_part("norm", PartSpec("gated_group_rms", {"channels": self.mixed_size, "groups": 1, "eps": self.eps,
                                                                    "weight_name": self.names.get("norm", "norm"), "gate": "sigmoid"},
                                                self.prefix), runtime)
        self.decay = None

    def tensor_decls(self):
        hk, hv = self.heads * self.dim, self.heads * self.vdim
        return [TensorDecl(self._name("q"), (hk, self.hidden)), TensorDecl(self._name("k"), (hk, self.hidden)),
                TensorDecl(self._name("v"), (hv, self.hidden)), TensorDecl(self._name("g"), (hv, self.hidden)),
                TensorDecl(self._name("o"), (self.hidden, hv))] + self.norm.tensor_decls()

    def load(self, tensors):
        self.w_in = torch.cat([tensors[self._name(n)] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = tensors[self._name("o")].contiguous()
        self.norm.load(tensors)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def cache_need(self):
        return CacheNeed(states=(("state", (self.heads, self.dim, self.vdim)),))

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, hk, hv = h.shape[0], self.heads * self.dim, self.heads * self.vdim
        proj = self.rt.empty_act((t, 2 * hk + 2 * hv))
        k.linear(h, self.w_in, proj)
        y = self._readout(t)
        k.linear_recurrence("decay", proj[:, :hk], proj[:, hk: 2 * hk], proj[:, 2 * hk: 2 * hk + hv], cache.states["state"], ctx, y,
                            self.heads, self.heads, self.dim, self.vdim, decay=self.decay)
        self.norm.forward(y, proj[:, 2 * hk + hv:], out, scale)


@register_part("mixer", "mamba2")
class Mamba2Mixer(RecurrentMixer):
    """params: hidden, heads, vdim, state, groups, norm_groups, taps, eps."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.vdim, self.n, self.groups = int(p["vdim"]), int(p["state"]), int(p["groups"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads do not split into {self.groups} groups")
        self.inner = self.mixed_size = self.heads * self.vdim
        self.conv_channels = self.inner + 2 * self.groups * self.n
        self.conv = build_part("filter", PartSpec("short_conv", {
            "channels": self.conv_channels, "taps": int(p["taps"]), "weight_name": self.names.get("conv", "conv"),
            "bias_name": self.names.get("conv_bias", "conv.b"), "activation": "silu", "state_name": "conv_tail"}, self.prefix), runtime)
        self.norm = build_part("norm", PartSpec("gated_group_rms", {
            "channels": self.inner, "groups": int(p["norm_groups"]), "eps": self.eps, "weight_name": self.names.get("norm", "norm"),
            "gate": "silu", "gate_first": True}, self.prefix), runtime)

    def tensor_decls(self):
        vec = lambda n: TensorDecl(self._name(n), (self.heads,), role="vector", init="norm")
        return ([TensorDecl(self._name("in"), (2 * self.inner + 2 * self.groups * self.n + self.heads, self.hidden)),
                 TensorDecl(self._name("o"), (self.hidden, self.inner)), vec("dt_bias"), vec("A_log"), vec("D")]
                + self.conv.tensor_decls() + self.norm.tensor_decls())

    def load(self, tensors):
        self.w_in = tensors[self._name("in")].contiguous()
        self.w_o = tensors[self._name("o")].contiguous()
        self.dt_bias, self.a_log, self.d_skip = (tensors[self._name(n)].contiguous() for n in ("dt_bias", "A_log", "D"))
        self.conv.load(tensors)
        self.norm.load(tensors)

    def cache_need(self):
        return CacheNeed.merged([("", CacheNeed(states=(("state", (self.heads, self.n, self.vdim)),))), ("", self.conv.cache_need())])

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, inner, gn = h.shape[0], self.inner, self.groups * self.n
        proj = self.rt.empty_act((t, 2 * inner + 2 * gn + self.heads))
        k.linear(h, self.w_in, proj)
        xbc = self.conv.forward(proj[:, inner: 2 * inner + 2 * gn], ctx, cache)
        y = self._readout(t)
        k.linear_recurrence("ssm", xbc[:, inner + gn:], xbc[:, inner: inner + gn], xbc[:, :inner], cache.states["state"], ctx, y,
                            self.heads, self.groups, self.n, self.vdim, aux=proj[:, 2 * inner + 2 * gn:], a_log=self.a_log,
                            dt_bias=self.dt_bias, d_skip=self.d_skip)
        self.norm.forward(y, proj[:, :inner], out, scale)


@register_part("mixer", "gated_delta")
class GatedDeltaMixer(RecurrentMixer):
    """params: hidden, heads, kv_heads, dim, vdim, taps, eps, rank (width of the two-step projections of the decay rate
    and of the gate; None: whatever the weight file has)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.kv_heads, self.dim, self.vdim = int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.rank = int(p["rank"]) if p.get("rank") else -1
        self.qk, self.mixed_size = self.kv_heads * self.dim, self.heads * self.vdim
        seg = lambda n, c: (self.names.get(n + "_conv", n + ".conv"), c)
        self.conv = build_part("filter", PartSpec("short_conv", {
            "channels": 2 * self.qk + self.mixed_size, "taps": int(p["taps"]), "activation": "silu", "state_name": "conv_tail",
            "segments": [seg("q", self.qk), seg("k", self.qk), seg("v", self.mixed_size)]}, self.prefix), runtime)
        self.norm = build_part("norm", PartSpec("gated_group_rms", {
            "channels": self.mixed_size, "groups": self.heads, "eps": self.eps, "weight_size": self.vdim,
            "weight_name": self.names.get("norm", "norm"), "gate": "sigmoid"}, self.prefix), runtime)

    def tensor_decls(self):
        hid, r = self.hidden, self.rank
        return ([TensorDecl(self._name("q"), (self.qk, hid)), TensorDecl(self._name("k"), (self.qk, hid)),
                 TensorDecl(self._name("v"), (self.mixed_size, hid)), TensorDecl(self._name("b"), (self.heads, hid)),
                 TensorDecl(self._name("a1"), (r, hid)), TensorDecl(self._name("a2"), (self.heads * self.dim, r)),
                 TensorDecl(self._name("g1"), (r, hid)), TensorDecl(self._name("g2"), (self.mixed_size, r)),
                 TensorDecl(self._name("o"), (hid, self.mixed_size)),
                 TensorDecl(self._name("A_log"), (self.heads,), role="vector", init="norm"),
                 TensorDecl(self._name("dt_bias"), (self.heads * self.dim,), role="vector", init="norm")]
                + self.conv.tensor_decls() + self.norm.tensor_decls())

    def load(self, tensors):
        t = lambda n: tensors[self._name(n)]
        if t("a1").shape[0] != t("a2").shape[1] or t("g1").shape[0] != t("g2").shape[1]:
            raise ValueError(f"{self.prefix}: the two steps of a low-rank projection do not fit each other")
        self.rank_a, self.rank_g = t("a1").shape[0], t("g1").shape[0]
        self.w_in = torch.cat([t(n) for n in ("q", "k", "v", "b", "a1", "g1")], dim=0).contiguous()
        self.w_a2, self.w_g2, self.w_o = t("a2").contiguous(), t("g2").contiguous(), t("o").contiguous()
        self.a_log, self.dt_bias = t("A_log").contiguous(), t("dt_bias").contiguous()
        self.conv.load(tensors)
        self.norm.load(tensors)

    def cache_need(self):
        return CacheNeed.merged([("", CacheNeed(states=(("state", (self.heads, self.dim, self.vdim)),))), ("", self.conv.cache_need())])

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, qk, hv, hd = h.shape[0], self.qk, self.mixed_size, self.heads
        n_conv = 2 * qk + hv
        proj = self.rt.empty_act((t, n_conv + hd + self.rank_a + self.rank_g))
        k.linear(h, self.w_in, proj)
        qkv = self.conv.forward(proj[:, :n_conv], ctx, cache)
        at = n_conv + hd
        rate = self.rt.empty_act((t, hd * self.dim))
        k.linear(proj[:, at: at + self.rank_a], self.w_a2, rate)
        gate = self.rt.empty_act((t, hv))
        k.linear(proj[:, at + self.rank_a:], self.w_g2, gate)
        y = self._readout(t)
        k.linear_recurrence("delta", qkv[:, :qk], qkv[:, qk: 2 * qk], qkv[:, 2 * qk:], cache.states["state"], ctx, y, hd, self.kv_heads,
                            self.dim, self.vdim, aux=proj[:, n_conv: n_conv + hd], rate=rate, a_log=self.a_log, dt_bias=self.dt_bias,
                            q_scale=1.0 / math.sqrt(self.dim))
        self.norm.forward(y, gate, out, scale)
