"""Grouped-query softmax attention without rotation, where position enters through the scores.

score(i, j) = (q_i . k_j) * scale - slope_h * (i - j), slope_h = 2^(-slope_power (h + 1) / heads) for head h; a query at
position i sees the keys j <= i of its own block of ``chunk`` positions (floor(i / chunk) == floor(j / chunk), counted
from the start of the sequence) or all of them without a chunk. Options: every value head divided by its root mean
square before it is cached; one sigmoid gate per head on the output, from a projection of the layer's input. Query/key
size and value size may differ: the cache pages and the kernels have one head size, the larger of the two rounded up
to a multiple of 16, and the projection matrices are padded with zero rows (zero columns for the output projection)
at load, which changes no score and no output.
"""
from __future__ import annotations

import math

import torch

from .base import CacheNeed, Mixer, TensorDecl, register_part


def _pad_heads(w: torch.Tensor, n_heads: int, size: int, padded: int) -> torch.Tensor:
    """[n_heads * size, K] -> [n_heads * padded, K] with zero rows after each head's own."""
    if size == padded:
        return w
    out = w.new_zeros((n_heads, padded, w.shape[1]))
    out[:, :size] = w.view(n_heads, size, -1)
    return out.view(n_heads * padded, -1)


@register_part("mixer", "distance_bias_attention")
class DistanceBiasAttention(Mixer):
    """params: hidden, heads, kv_heads, dim, vdim, scale, chunk (None: all keys), slope_power (None: no bias),
    value_norm_eps (None: values as projected), head_gate (bool), window (None)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim)
        self.chunk = int(p["chunk"]) if p.get("chunk") else None
        self.window = int(p["window"]) if p.get("window") else None
        self.slope_power = float(p["slope_power"]) if p.get("slope_power") is not None else None
        self.value_norm_eps = float(p["value_norm_eps"]) if p.get("value_norm_eps") is not None else None
        self.head_gate = bool(p.get("head_gate", False))
        self.names = dict(p.get("names", {}))
        self.head_dim = 16 * -(-max(self.dim, self.vdim) // 16)
        self.gate_cols = 8 * -(-self.heads // 8) if self.head_gate else 0        # keeps the rows of the product 16-byte multiples
        self.mixed_size = self.heads * self.head_dim
        runtime.kernels.check_attention_shape(self.heads, self.kv_heads, self.head_dim)

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def tensor_decls(self):
        decls = [TensorDecl(self._name("q"), (self.heads * self.dim, self.hidden)),
                 TensorDecl(self._name("k"), (self.kv_heads * self.dim, self.hidden)),
                 TensorDecl(self._name("v"), (self.kv_heads * self.vdim, self.hidden)),
                 TensorDecl(self._name("o"), (self.hidden, self.heads * self.vdim))]
        if self.head_gate:
            decls.append(TensorDecl(self._name("g"), (self.heads, self.hidden)))
        return decls

    def load(self, tensors):
        d = self.head_dim
        parts = [_pad_heads(tensors[self._name("q")], self.heads, self.dim, d), _pad_heads(tensors[self._name("k")], self.kv_heads, self.dim, d),
                 _pad_heads(tensors[self._name("v")], self.kv_heads, self.vdim, d)]
        if self.head_gate:
            parts.append(_pad_heads(tensors[self._name("g")], 1, self.heads, self.gate_cols))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        w_o = tensors[self._name("o")]
        if self.vdim != d:
            padded = w_o.new_zeros((self.hidden, self.heads, d))
            padded[:, :, : self.vdim] = w_o.view(self.hidden, self.heads, self.vdim)
            w_o = padded.view(self.hidden, self.heads * d)
        self.w_o = w_o.contiguous()
        self.slopes = None
        if self.slope_power is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_power * (h + 1) / self.heads) for h in range(self.heads)],
                                       dtype=torch.float32, device=self.w_o.device)

    def cache_need(self):
        return CacheNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window, chunk=self.chunk)

    def output_weight(self):
        return self.w_o

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, d = h.shape[0], self.head_dim
        n_qkv = (self.heads + 2 * self.kv_heads) * d
        proj = self.rt.empty_act((t, n_qkv + self.gate_cols))
        k.linear(h, self.w_in, proj)
        table = ctx.block_tables[cache.group]
        if cache.writes:
            k.kv_norm_cache_write(proj, ctx.positions, ctx.token_row, self.heads, self.kv_heads, d,
                                  self.vdim if self.value_norm_eps is not None else 0, self.value_norm_eps or 0.0, cache.k, cache.v, table,
                                  cache.page_size)
        if not self.head_gate and scale == 1.0 and out.is_contiguous():
            attn = out
        else:
            attn = self.rt.empty_act((t, self.heads * d))
        k.attention(proj, cache.k, cache.v, table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions, self.heads, self.kv_heads, d,
                    cache.page_size, self.scale, self.window or 0, attn, ctx.shape, slopes=self.slopes, chunk=self.chunk or 0)
        if attn is not out:
            gate = proj[:, n_qkv: n_qkv + self.heads] if self.head_gate else None
            k.gated_norm(attn, out, groups=0, gate=gate, gate_act="sigmoid", scale=scale)

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.linear(mixed, self.w_o, out)
        return out
