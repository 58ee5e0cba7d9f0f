"""Grouped-query softmax attention without rotation: normalised queries and keys, capped scores, a sink.

q = W_q h, k = W_k h, v = W_v h. With ``qk_norm_eps`` the whole query projection of a token (all heads at once) is
divided by its root mean square and multiplied by a weight of that size ("q.norm"), and the key projection likewise
("k.norm"). With ``q_temp`` = {coef, every} the query at position p is then multiplied by
1 + coef * ln(floor((p + 1) / every) + 1). score = (q . k) * scale; with ``softcap`` c the score becomes
c * tanh(score / c). Causal. With ``sink`` the softmax's denominator also holds exp(sink_h), a learned number per head
that has no key and no value. Positions enter through the temperature and the mask only. Query/key size and value
size may differ: the cache pages and the kernels have one head size, the larger of the two rounded up to a multiple
of 16; projection matrices and norm weights are padded with zeros at load, which changes no score and no output (the
mean of squares is taken over the true size).
"""
from __future__ import annotations

import math

import torch

from .base import CacheNeed, Mixer, TensorDecl, register_part
from .biased_attention import _pad_heads


@register_part("mixer", "capped_sink_attention")
class CappedSinkAttention(Mixer):
    """params: hidden, heads, kv_heads, dim, vdim, scale, softcap (None: none), sink (bool), qk_norm_eps (None: no norm),
    q_temp ({coef, every} or None), window (None), names."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim)
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.sink = bool(p.get("sink", False))
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        t = p.get("q_temp")
        self.temp_coef, self.temp_every = (float(t["coef"]), int(t["every"])) if t else (0.0, 1)
        self.window = int(p["window"]) if p.get("window") else None
        self.names = dict(p.get("names", {}))
        self.head_dim = 16 * -(-max(self.dim, self.vdim) // 16)
        self.mixed_size = self.heads * self.head_dim
        runtime.kernels.check_attention_shape(self.heads, self.kv_heads, self.head_dim)

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def kernel_needs(self):
        return {"attention_head_dims": [self.head_dim], "libraries": ["prep"]}

    def tensor_decls(self):
        decls = [TensorDecl(self._name("q"), (self.heads * self.dim, self.hidden)),
                 TensorDecl(self._name("k"), (self.kv_heads * self.dim, self.hidden)),
                 TensorDecl(self._name("v"), (self.kv_heads * self.vdim, self.hidden)),
                 TensorDecl(self._name("o"), (self.hidden, self.heads * self.vdim))]
        if self.qk_norm_eps is not None:
            decls += [TensorDecl(self._name("q.norm"), (self.heads * self.dim,), role="vector", init="norm"),
                      TensorDecl(self._name("k.norm"), (self.kv_heads * self.dim,), role="vector", init="norm")]
        if self.sink:
            decls.append(TensorDecl(self._name("sink"), (self.heads,), role="vector", init="normal"))
        return decls

    def load(self, tensors):
        d = self.head_dim
        self.w_in = torch.cat([_pad_heads(tensors[self._name("q")], self.heads, self.dim, d),
                               _pad_heads(tensors[self._name("k")], self.kv_heads, self.dim, d),
                               _pad_heads(tensors[self._name("v")], self.kv_heads, self.vdim, d)], dim=0).contiguous()
        w_o = tensors[self._name("o")]
        if self.vdim != d:
            padded = w_o.new_zeros((self.hidden, self.heads, d))
            padded[:, :, : self.vdim] = w_o.view(self.hidden, self.heads, self.vdim)
            w_o = padded.view(self.hidden, self.heads * d)
        self.w_o = w_o.contiguous()
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            # norm weights as float vectors laid out like the padded projection
            self.q_norm = _pad_heads(tensors[self._name("q.norm")].float().view(-1, 1), self.heads, self.dim, d).view(-1).contiguous()
            self.k_norm = _pad_heads(tensors[self._name("k.norm")].float().view(-1, 1), self.kv_heads, self.dim, d).view(-1).contiguous()
        self.sinks = tensors[self._name("sink")].float().contiguous() if self.sink else None

    def cache_need(self):
        return CacheNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def output_weight(self):
        return self.w_o

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        if scale != 1.0 or not out.is_contiguous():
            raise ValueError("capped_sink_attention writes its heads unscaled into a contiguous buffer")
        k = self.rt.kernels
        t, d = h.shape[0], self.head_dim
        proj = self.rt.empty_act((t, (self.heads + 2 * self.kv_heads) * d))
        k.linear(h, self.w_in, proj)
        table = ctx.block_tables[cache.group]
        k.normed_qk_cache_write(proj, ctx.positions, ctx.token_row, self.heads, self.kv_heads, d, self.dim, self.q_norm, self.k_norm,
                                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, self.temp_coef, self.temp_every,
                                cache.k, cache.v, table, cache.page_size, cache.writes)
        k.attention(proj, cache.k, cache.v, table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions, self.heads, self.kv_heads, d,
                    cache.page_size, self.scale, self.window or 0, out, ctx.shape, softcap=self.softcap, sinks=self.sinks)

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.linear(mixed, self.w_o, out)
        return out
