"""Shared by the Bapavik tests: small configurations of their own, seeded weights, engines on either backend.

Two backends: "emu" runs the engine's own parts, cache manager and step function on the CPU over the torch stand-ins of
tests/emu_kernels.py (no GPU needed, float32); "cuda" runs the real kernels. The oracle is tests/plain/bapavik_plain.py
in float64.
"""
from __future__ import annotations

import json
import os

import pytest
import torch

from tests.plain import bapavik_plain as P

ATT = lambda heads, kv, dim, vdim, scale, cap, coef, every: {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                                                             "softcap": cap, "q_temp": {"coef": coef, "every": every}}
LAT = lambda heads, dim, rot, vdim, rank, scale, base: {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
                                                        "scale": scale, "rot": {"base": base, "dims": rot}}
DENSE = lambda ff, limit: {"kind": "dense", "ff": ff, "limit": limit}
MOE = lambda experts, top, ff: {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}

# Sizes differ between layers and from each other wherever the design allows: value heads smaller and larger than the
# query/key heads; one key/value head per query head and one for all; a temperature step of one position and of many;
# a low cap that really bends the scores; latent rows (rank + rotated part) that are no multiple of 16; experts with one
# choice per token and with all of them; every kind of feed-forward behind every kind of mixer, and none; loops over the
# first layers, over inner layers, over one layer, and no loop at all.
CONFIGS = {
    "a": {"architecture": "Bapavik", "width": 64, "vocab": 150, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
          "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
        {"type": "attention", "mixer": ATT(4, 2, 24, 16, 0.2, 30.0, 0.3, 16), "mlp": DENSE(96, 1.5)},
        {"type": "latent_attention", "mixer": LAT(4, 16, 8, 24, 40, 0.2, 10000.0), "mlp": MOE(6, 2, 32)},
        {"type": "attention", "mixer": ATT(2, 2, 16, 32, 0.25, 4.0, 0.5, 1), "mlp": MOE(4, 1, 48)},
        {"type": "latent_attention", "mixer": LAT(2, 24, 4, 16, 20, 0.19, 500.0), "mlp": None},
    ]},
    # sizes that are multiples of nothing: no vector load, no tensor-core tile and no padded head fits them exactly
    "o": {"architecture": "Bapavik", "width": 100, "vocab": 131, "norm": {"eps": 3e-5}, "embedding": {"scale": 5.5},
          "loop": {"start": 1, "stop": 2, "times": 3}, "layers": [
        {"type": "latent_attention", "mixer": LAT(5, 12, 6, 10, 30, 0.22, 3000.0), "mlp": DENSE(70, 0.9)},
        {"type": "attention", "mixer": ATT(6, 1, 20, 12, 0.2, 8.0, 0.2, 7), "mlp": MOE(5, 3, 22)},
        {"type": "attention", "mixer": ATT(3, 3, 12, 20, 0.3, 50.0, 0.7, 33), "mlp": None},
        {"type": "latent_attention", "mixer": LAT(3, 20, 10, 28, 70, 0.18, 20000.0), "mlp": MOE(3, 3, 30)},
    ]},
    "q": {"architecture": "Bapavik", "width": 48, "vocab": 97, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
        {"type": "latent_attention", "mixer": LAT(3, 8, 8, 16, 24, 0.25, 100.0), "mlp": MOE(7, 2, 16)},
        {"type": "attention", "mixer": ATT(6, 3, 8, 8, 0.35, 15.0, 1.0, 5), "mlp": DENSE(64, 2.5)},
    ]},
}

# Layers as wide as a real model's: heads of 128 (attention) and latent rows of 192 + 64, experts and dense widths that are
# multiples of 64, so the bfloat16 products run on the tensor-core tiles and the attention on its widest head sizes.
CONFIGS["wide"] = {"architecture": "Bapavik", "width": 512, "vocab": 300, "norm": {"eps": 1e-5}, "embedding": {"scale": 12.0}, "layers": [
    {"type": "attention", "mixer": ATT(8, 2, 128, 64, 0.088, 50.0, 0.3, 128), "mlp": MOE(8, 2, 128)},
    {"type": "latent_attention", "mixer": LAT(8, 64, 64, 64, 192, 0.088, 10000.0), "mlp": DENSE(1024, 1.5)},
]}


def make_weights(cfg: dict, seed: int, expert_gain: float = 1.0):
    """float32 weights by name (tables int32), sized so that every layer's output matters."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in P.tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "table":
            t = torch.rand((shape[0], cfg["layers"][int(name[1:].split(".")[0])]["mlp"]["router"]["experts"]), generator=g).argsort(1)
            w[name] = t[:, : shape[1]].to(torch.int32).contiguous()
            continue
        if leaf in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        else:
            t = torch.randn(shape, generator=g) * 1.5 / shape[-1] ** 0.5
        if leaf == "down" and ".e" in name:
            t = t * expert_gain
        w[name] = t.bfloat16().float()          # values that a bfloat16 file holds exactly
    return w


def plain_logits(w, cfg, tokens, streams=None):
    w64 = {k: (v.double() if v.dtype.is_floating_point else v) for k, v in w.items()}
    with torch.no_grad():
        return P.forward(w64, cfg, tokens, streams).float()


def write_model(path: str, cfg: dict, w, dtype=torch.float32) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: (v.to(dtype) if v.dtype.is_floating_point else v).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))
    return path


BACKENDS = [pytest.param(("emu", "float32"), id="emu"),
            pytest.param(("cuda", "float32"), id="cuda-f32", marks=pytest.mark.gpu),
            pytest.param(("cuda", "bfloat16"), id="cuda-bf16", marks=pytest.mark.gpu)]


def runtime_for(backend):
    from tests.rogisun_cases import runtime_for as make

    return make(backend)


def make_engine(folder, backend, page, num_pages, max_slots=4, graphs=False, budget=512, context=None):
    from tests.rogisun_cases import make_engine as make

    return make(folder, backend, page, num_pages, max_slots, graphs, budget, context)


def tolerance(backend, plain) -> float:
    scale = max(float(p.abs().max()) for p in plain.values())
    return scale * (2e-4 if backend[1] == "float32" else 2.0 ** -5)


def compare_rows(got, plain, backend) -> float:
    """Every collected row against the plain logits. float32: every element within ``tolerance``. bfloat16: a row's error is
    the root mean square of its difference (means taken off) over that of the plain row; activations are rounded to 8 bits
    several times a layer, which gives a few percent; every value must be finite."""
    from tests import helpers

    if backend[1] == "float32":
        return helpers.compare_with_plain(got, plain, atol=tolerance(backend, plain))
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = plain[rid][pos]
        assert bool(torch.isfinite(row).all()), f"request {rid!r} position {pos}: not finite"
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt())
        worst = max(worst, e)
        assert e <= 0.08, f"request {rid!r} position {pos}: relative error {e:.3f}"
    return worst
