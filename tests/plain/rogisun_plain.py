"""The Rogisun decoder, whole sequences at a time, in plain torch on the CPU: one function per mechanism.

A slow restatement of the design's equations that shares no code with the engine; the GPU tests compare the
engine with it. Every function takes one sequence ([T, ...] tensors, position 0 first) and works in the dtype
of its inputs (the tests use float64 or float32). Notation: T tokens, W width, H heads.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.nn.functional as F


# ---- small pieces -------------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (weight None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def causal_conv(h, w, bias=None):
    """Per channel over time: out[t] = sum_j w[:, j] * h[t - taps + 1 + j], zeros before the start. h [T, C], w [C, taps]."""
    t, taps = h.shape[0], w.shape[1]
    padded = torch.cat([h.new_zeros(taps - 1, h.shape[1]), h], 0)
    out = torch.zeros_like(h)
    for j in range(taps):
        out = out + padded[j: j + t] * w[:, j]
    return out if bias is None else out + bias


def input_conv(h, w):
    """What a sub-layer reads: h + conv(h)."""
    return h + causal_conv(h, w)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


# ---- recurrent mixers ---------------------------------------------------------------------------------------
def lightning_mixer(h, w, p, m, eps):
    """Linear attention with a fixed decay per head. p: tensor-name prefix, m: the mixer's sizes."""
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = F.silu(h @ w[p + "q"].T).view(t, heads, dim)
    k = F.silu(h @ w[p + "k"].T).view(t, heads, dim)
    v = F.silu(h @ w[p + "v"].T).view(t, heads, vdim)
    out = h.new_zeros(t, heads, vdim)
    for hd in range(heads):
        s = h.new_zeros(dim, vdim)
        for i in range(t):
            s = m["decay"][hd] * s + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s.T @ q[i, hd]
    y = rms_norm(out.reshape(t, heads * vdim), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def mamba2_mixer(h, w, p, m, eps):
    """Selective state space layer with a scalar decay per head and token."""
    heads, vdim, n, groups, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = heads * vdim
    t = h.shape[0]
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    xbc = F.silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(t, heads, vdim)
    b = xbc[:, inner: inner + groups * n].view(t, groups, n)
    c = xbc[:, inner + groups * n:].view(t, groups, n)
    dt = softplus(dt + w[p + "dt_bias"])
    a = torch.exp(-torch.exp(w[p + "A_log"]) * dt)                    # [T, heads]
    y = h.new_zeros(t, heads, vdim)
    for hd in range(heads):
        g = hd // (heads // groups)
        s = h.new_zeros(n, vdim)
        for i in range(t):
            s = a[i, hd] * s + dt[i, hd] * torch.outer(b[i, g], x[i, hd])
            y[i, hd] = s.T @ c[i, g] + w[p + "D"][hd] * x[i, hd]
    y = y.reshape(t, inner) * F.silu(z)
    y = rms_norm(y.view(t, ng, inner // ng), None, eps).reshape(t, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def gated_delta_mixer(h, w, p, m, eps):
    """Delta rule with a decay per head and key channel."""
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]

    def conv_silu(name):
        return F.silu(causal_conv(h @ w[p + name].T, w[p + name + ".conv"]))

    q = conv_silu("q").view(t, kvh, dim)
    k = conv_silu("k").view(t, kvh, dim)
    v = conv_silu("v").view(t, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                            # [T, heads]
    rate = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(t, heads, dim)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * rate)   # [T, heads, dim]
    out = h.new_zeros(t, heads, vdim)
    for hd in range(heads):
        kh = hd // (heads // kvh)
        s = h.new_zeros(dim, vdim)
        for i in range(t):
            s = g[i, hd][:, None] * s
            u = beta[i, hd] * (v[i, hd] - s.T @ k[i, kh])
            s = s + torch.outer(k[i, kh], u)
            out[i, hd] = s.T @ q[i, kh]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(t, heads, vdim)
    y = rms_norm(out, w[p + "norm"], eps) * gate
    return y.reshape(t, heads * vdim) @ w[p + "o"].T


# ---- attention ----------------------------------------------------------------------------------------------
def chunked_bias_attention(h, w, p, m, eps):
    """Grouped-query softmax attention without rotation: normalised values, a linear distance penalty per head,
    keys visible only inside the query's own block of mask.size positions, one output gate per head."""
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, scale = m["mask"]["size"], m["scale"]
    t = h.shape[0]
    q = (h @ w[p + "q"].T).view(t, heads, dim)
    k = (h @ w[p + "k"].T).view(t, kvh, dim)
    v = rms_norm((h @ w[p + "v"].T).view(t, kvh, vdim), None, eps)
    gate = torch.sigmoid(h @ w[p + "g"].T)                             # [T, heads]
    pos = torch.arange(t)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[:, None] // size) == (pos[None, :] // size))
    out = h.new_zeros(t, heads, vdim)
    for hd in range(heads):
        kh = hd // (heads // kvh)
        slope = 2.0 ** (-8.0 * (hd + 1) / heads)
        s = (q[:, hd] @ k[:, kh].T) * scale - slope * dist
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, kh]
    out = out * gate[:, :, None]
    return out.reshape(t, heads * vdim) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * chunked_bias_attention(h, w, p + "left.", m["left"], eps)
            + m["right_scale"] * gated_delta_mixer(h, w, p + "right.", m["right"], eps))


MIXERS = {"lightning": lightning_mixer, "mamba2": mamba2_mixer, "parallel": parallel_mixer}


# ---- feed-forward -------------------------------------------------------------------------------------------
def expert(x, w, p, limit):
    g = torch.clamp(x @ w[p + "gate"].T, max=limit)
    u = torch.clamp(x @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def routed_experts(h, w, p, f, margins: list = None):
    """Sigmoid router; each token's input is scaled by the score of each of its `top` experts. ``margins``, if a list,
    receives the smallest gap between a chosen and a rejected expert's logit (how close the closest call was)."""
    n, top, limit = f["router"]["experts"], f["router"]["top"], f["expert"]["limit"]
    z = h @ w[p + "router"].T
    scores = torch.sigmoid(z)
    best = torch.topk(z, top, dim=-1).indices          # the largest scores are the largest logits (sigmoid rounds big ones to ties)
    if margins is not None and top < n:
        ranked = torch.sort(z, dim=-1, descending=True).values
        margins.append(float((ranked[:, top - 1] - ranked[:, top]).min()))
    out = torch.zeros_like(h)
    for e in range(n):
        for slot in range(top):
            rows = (best[:, slot] == e).nonzero().flatten()
            if len(rows):
                out[rows] += expert(scores[rows, e][:, None] * h[rows], w, f"{p}e{e}.", limit)
    return out


# ---- the model ----------------------------------------------------------------------------------------------
def forward(w: Dict[str, torch.Tensor], cfg: dict, tokens: List[int], residuals: list = None, margins: list = None):
    """Logits [T, vocab] of one sequence; ``residuals``, if a list, receives the stream after every layer, and
    ``margins`` the closest call of every router."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = input_conv(rms_norm(x, w[p + "norm1"], eps), w[p + "canon1"])
        x = x + MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            h = input_conv(rms_norm(x, w[p + "norm2"], eps), w[p + "canon2"])
            x = x + routed_experts(h, w, p + "mlp.", layer["mlp"], margins)
        if residuals is not None:
            residuals.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, from its configuration."""
    width, taps = cfg["width"], cfg["canon"]["taps"]
    s = {"embed": (cfg["vocab"], width), "final.norm": (width,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        s[p + "norm1"] = (width,)
        s[p + "canon1"] = (width, taps)
        if kind == "lightning":
            for n, rows in (("q", m["dim"]), ("k", m["dim"]), ("v", m["vdim"]), ("g", m["vdim"])):
                s[p + "mix." + n] = (m["heads"] * rows, width)
            s[p + "mix.o"] = (width, m["heads"] * m["vdim"])
            s[p + "mix.norm"] = (m["heads"] * m["vdim"],)
        elif kind == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            s[p + "mix.in"] = (2 * inner + 2 * gn + m["heads"], width)
            s[p + "mix.conv"] = (inner + 2 * gn, m["conv"])
            s[p + "mix.conv.b"] = (inner + 2 * gn,)
            for n in ("dt_bias", "A_log", "D"):
                s[p + "mix." + n] = (m["heads"],)
            s[p + "mix.norm"] = (inner,)
            s[p + "mix.o"] = (width, inner)
        elif kind == "parallel":
            a, d = m["left"], m["right"]
            q = p + "mix.left."
            s[q + "q"] = (a["heads"] * a["dim"], width)
            s[q + "k"] = (a["kv_heads"] * a["dim"], width)
            s[q + "v"] = (a["kv_heads"] * a["vdim"], width)
            s[q + "g"] = (a["heads"], width)
            s[q + "o"] = (width, a["heads"] * a["vdim"])
            q = p + "mix.right."
            for n, rows in (("q", d["kv_heads"] * d["dim"]), ("k", d["kv_heads"] * d["dim"]), ("v", d["heads"] * d["vdim"])):
                s[q + n] = (rows, width)
                s[q + n + ".conv"] = (rows, d["conv"])
            s[q + "b"] = (d["heads"], width)
            s[q + "A_log"] = (d["heads"],)
            s[q + "norm"] = (d["vdim"],)
            rank = d["rank"]                 # width of the two-step projections (a file gives it by its shapes)
            s[q + "a1"], s[q + "a2"] = (rank, width), (d["heads"] * d["dim"], rank)
            s[q + "dt_bias"] = (d["heads"] * d["dim"],)
            s[q + "g1"], s[q + "g2"] = (rank, width), (d["heads"] * d["vdim"], rank)
            s[q + "o"] = (width, d["heads"] * d["vdim"])
        else:
            raise ValueError(kind)
        f = layer.get("mlp")
        if f is not None:
            s[p + "norm2"] = (width,)
            s[p + "canon2"] = (width, taps)
            s[p + "mlp.router"] = (f["router"]["experts"], width)
            for e in range(f["router"]["experts"]):
                s[f"{p}mlp.e{e}.gate"] = (f["expert"]["ff"], width)
                s[f"{p}mlp.e{e}.up"] = (f["expert"]["ff"], width)
                s[f"{p}mlp.e{e}.down"] = (width, f["expert"]["ff"])
    return s
