"""The Bapavik decoder, whole sequences at a time, in plain torch on the CPU: one function per mechanism.

A slow restatement of the design's equations that shares no code with the engine; the tests compare the engine
with it. Every function takes one sequence ([T, ...] tensors, position 0 first) and works in the dtype of its
inputs (the tests use float64 or float32). Notation: T tokens, W width, H query heads, G key/value heads.

The design: x = embed[token] * s; pre-norm layers with a layer norm that has a weight and no bias; two mixers,
softmax attention whose queries and keys are normalised over the whole projection, with a query temperature that grows
with the logarithm of the position, capped scores and a sink in the denominator, and latent attention whose keys and
values are read out of one small vector per token plus one rotated key part shared by the heads; feed-forwards that are
dense (clamped gated activation), a mixture of small experts chosen by a table over token ids, or absent; a run of
layers may repeat with the same weights; final layer norm and an untied head.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch


# ---- small pieces -------------------------------------------------------------------------------------------
def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight over the last axis, var = mean of squared deviations; no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotate_interleaved(x, base: float, dims: int):
    """x [T, ..., D]: the first ``dims`` elements of the last axis as pairs (2i, 2i+1), each turned by position * base^(-2i/dims)."""
    t = x.shape[0]
    out = x.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ang = torch.arange(t, dtype=x.dtype) * f
        c, s = torch.cos(ang), torch.sin(ang)
        shape = (t,) + (1,) * (x.dim() - 2)
        c, s = c.view(shape), s.view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def query_temperature(t: int, coef: float, every: int, dtype):
    """1 + coef * ln(floor((p + 1) / every) + 1) for p = 0 .. t-1."""
    p = torch.arange(t)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


# ---- mixers ---------------------------------------------------------------------------------------------------
def sink_attention(h, w, p, m, eps):
    """Grouped-query causal attention without rotation. p: tensor-name prefix, m: the mixer's sizes and constants."""
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps)             # over all heads' rows at once
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(t, kvh, vdim)
    q = q * query_temperature(t, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None]
    q, k = q.view(t, heads, dim), k.view(t, kvh, dim)
    cap = m["softcap"]
    out = h.new_zeros(t, heads, vdim)
    rep = heads // kvh
    causal = torch.arange(t)[None, :] > torch.arange(t)[:, None]
    for hd in range(heads):
        g = hd // rep
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = cap * torch.tanh(s / cap)
        s = s.masked_fill(causal, float("-inf"))
        sink = w[p + "sink"][hd]
        top = torch.maximum(s.max(-1).values, sink)
        e = torch.exp(s - top[:, None])
        out[:, hd] = (e @ v[:, g]) / (e.sum(-1) + torch.exp(sink - top))[:, None]
    return out.reshape(t, heads * vdim) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Keys and values read out of a latent vector per token, plus one rotated key part that all heads share."""
    heads, dim, rd, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    t = h.shape[0]
    q = (h @ w[p + "q"].T).view(t, heads, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate_interleaved(q[..., dim:], m["rot"]["base"], m["rot"]["dims"])
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, rank:], m["rot"]["base"], m["rot"]["dims"])          # [T, rd], one for all heads
    k_plain = (c @ w[p + "uk"].T).view(t, heads, dim)
    v = (c @ w[p + "uv"].T).view(t, heads, vdim)
    causal = torch.arange(t)[None, :] > torch.arange(t)[:, None]
    out = h.new_zeros(t, heads, vdim)
    for hd in range(heads):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = torch.softmax(s.masked_fill(causal, float("-inf")), -1) @ v[:, hd]
    return out.reshape(t, heads * vdim) @ w[p + "o"].T


MIXERS = {"attention": sink_attention, "latent_attention": latent_attention}


# ---- feed-forwards --------------------------------------------------------------------------------------------
def dense_feed_forward(h, w, p, f):
    g = torch.clamp(h @ w[p + "gate"].T, max=f["limit"])
    u = torch.clamp(h @ w[p + "up"].T, -f["limit"], f["limit"])
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def table_experts(h, tokens, w, p, f):
    """Each token's experts come from a table over token ids; every chosen expert weighs 1 / top."""
    top = f["router"]["top"]
    table = w[p + "table"].long()
    out = torch.zeros_like(h)
    for i, tok in enumerate(tokens):
        for e in table[tok].tolist():
            a = torch.relu(h[i] @ w[f"{p}e{e}.up"].T) ** 2
            out[i] = out[i] + (a @ w[f"{p}e{e}.down"].T) / top
    return out


def feed_forward(h, tokens, w, p, f):
    return dense_feed_forward(h, w, p, f) if f["kind"] == "dense" else table_experts(h, tokens, w, p, f)


# ---- the model ------------------------------------------------------------------------------------------------
def layer_order(cfg: dict) -> List[int]:
    """Indices of the layers in running order: layers start .. stop-1 run ``times`` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(w: Dict[str, torch.Tensor], cfg: dict, tokens, streams=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        x = x + MIXERS[layer["type"]](layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(layer_norm(x, w[p + "norm2"], eps), tokens, w, p + "mlp.", layer["mlp"])
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a weight file of this design."""
    width, vocab = cfg["width"], cfg["vocab"]
    s = {"embed": (vocab, width), "final.norm": (width,), "head": (vocab, width)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = (width,)
        if layer["type"] == "attention":
            s[p + "mix.q"] = (m["heads"] * m["dim"], width)
            s[p + "mix.k"] = (m["kv_heads"] * m["dim"], width)
            s[p + "mix.v"] = (m["kv_heads"] * m["vdim"], width)
            s[p + "mix.q.norm"] = (m["heads"] * m["dim"],)
            s[p + "mix.k.norm"] = (m["kv_heads"] * m["dim"],)
            s[p + "mix.sink"] = (m["heads"],)
        else:
            s[p + "mix.q"] = (m["heads"] * (m["dim"] + m["rot_dim"]), width)
            s[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], width)
            s[p + "mix.dkv.norm"] = (m["kv_rank"],)
            s[p + "mix.uk"] = (m["heads"] * m["dim"], m["kv_rank"])
            s[p + "mix.uv"] = (m["heads"] * m["vdim"], m["kv_rank"])
        s[p + "mix.o"] = (width, m["heads"] * m["vdim"])
        f = layer.get("mlp")
        if f is None:
            continue
        s[p + "norm2"] = (width,)
        if f["kind"] == "dense":
            s[p + "mlp.gate"] = s[p + "mlp.up"] = (f["ff"], width)
            s[p + "mlp.down"] = (width, f["ff"])
        else:
            for e in range(f["router"]["experts"]):
                s[f"{p}mlp.e{e}.up"] = (f["expert"]["ff"], width)
                s[f"{p}mlp.e{e}.down"] = (width, f["expert"]["ff"])
            s[p + "mlp.table"] = (vocab, f["router"]["top"])
    return s
