"""Shared by the Rogisun tests: small configurations of their own, seeded weights, engines on either backend.

Two backends: "emu" runs the engine's own parts, cache and step function on the CPU over the torch stand-ins of
tests/emu_kernels.py (no GPU needed, float32); "cuda" runs the real kernels. The oracle is tests/plain/rogisun_plain.py
in float64.
"""
from __future__ import annotations

import copy
import json
import os

import pytest
import torch

from tests.plain import rogisun_plain as P

MOE = lambda experts, top, ff, limit: {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}

# Sizes differ between layers and from each other wherever the design allows: two experts per token and one; groups
# of heads that share keys on either side of the parallel pair; query/key size below and above the value size (the
# second needs padding to a head size of 32); blocks of positions that are no multiple of a cache page; a layer
# without a feed-forward; convolutions of 2, 3 and 4 taps.
CONFIGS = {
    "p": {"architecture": "Rogisun", "width": 64, "vocab": 160, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "layers": [
        {"type": "lightning", "mixer": {"heads": 2, "dim": 16, "vdim": 24, "decay": [0.9, 0.985]}, "mlp": MOE(4, 2, 24, 1.5)},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3, "mask": {"size": 24}},
            "right": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 2, "rank": 8},
            "left_scale": 0.7, "right_scale": 1.3}, "mlp": None},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 8, "state": 12, "groups": 2, "norm_groups": 2, "conv": 3}, "mlp": MOE(3, 1, 16, 0.8)},
    ]},
    # sizes that are multiples of nothing: no vector load, no tensor-core tile and no padded head fits them exactly
    "o": {"architecture": "Rogisun", "width": 100, "vocab": 131, "norm": {"eps": 3e-5}, "canon": {"taps": 5}, "layers": [
        {"type": "mamba2", "mixer": {"heads": 5, "vdim": 6, "state": 10, "groups": 5, "norm_groups": 3, "conv": 3}, "mlp": MOE(7, 2, 22, 1.1)},
        {"type": "lightning", "mixer": {"heads": 5, "dim": 12, "vdim": 20, "decay": [0.7, 0.8, 0.9, 0.95, 0.99]}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 12, "scale": 0.2, "mask": {"size": 17}},
            "right": {"heads": 3, "kv_heads": 3, "dim": 12, "vdim": 10, "conv": 5, "rank": 7},
            "left_scale": 0.9, "right_scale": 0.8}, "mlp": MOE(3, 3, 30, 0.9)},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 40, "scale": 0.15, "mask": {"size": 64}},
            "right": {"heads": 4, "kv_heads": 1, "dim": 20, "vdim": 6, "conv": 2, "rank": 3},
            "left_scale": 0.4, "right_scale": 1.1}, "mlp": MOE(4, 1, 18, 3.0)},
    ]},
    "q": {"architecture": "Rogisun", "width": 48, "vocab": 97, "norm": {"eps": 1e-6}, "canon": {"taps": 2}, "layers": [
        {"type": "parallel", "mixer": {
            "left": {"heads": 3, "kv_heads": 3, "dim": 24, "vdim": 16, "scale": 0.25, "mask": {"size": 10}},
            "right": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 16, "conv": 4, "rank": 6},
            "left_scale": 1.0, "right_scale": 0.5}, "mlp": MOE(5, 3, 8, 2.0)},
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 16, "state": 20, "groups": 1, "norm_groups": 1, "conv": 2}, "mlp": None},
        {"type": "lightning", "mixer": {"heads": 3, "dim": 8, "vdim": 16, "decay": [0.5, 0.93, 0.999]}, "mlp": MOE(2, 1, 32, 1.0)},
    ]},
}


# Layers as wide as a real model's: heads of 128, states of 128 rows, norm groups of 768 values, blocks of 256 positions, experts
# whose widths are multiples of 32. The tiny configurations never reach the kernels' paths for these sizes (sixteen rows of a
# state per thread with eight lanes a column, 16-byte convolution loads, a block per norm group, tensor-core tiles).
CONFIGS["wide"] = {"architecture": "Rogisun", "width": 512, "vocab": 300, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "layers": [
    {"type": "lightning", "mixer": {"heads": 6, "dim": 128, "vdim": 128, "decay": [0.9, 0.95, 0.97, 0.99, 0.995, 0.999]}, "mlp": MOE(8, 2, 128, 2.0)},
    {"type": "mamba2", "mixer": {"heads": 12, "vdim": 64, "state": 128, "groups": 2, "norm_groups": 1, "conv": 4}, "mlp": MOE(8, 2, 128, 2.0)},
    {"type": "parallel", "mixer": {
        "left": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 256}},
        "right": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 4, "rank": 32},
        "left_scale": 0.5, "right_scale": 0.5}, "mlp": MOE(8, 2, 128, 2.0)},
]}


def make_weights(cfg: dict, seed: int, router_gain: float = 6.0, expert_gain: float = 1.0):
    """float32 weights by name, sized so that every layer's output matters; routers with a wide spread of logits.
    ``expert_gain`` scales the experts' last matrices (see settled_weights)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in P.tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith(("canon1", "canon2", ".conv")):
            t = torch.randn(shape, generator=g) * 0.4
        elif leaf in ("norm", "norm1", "norm2", "D"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.rand(shape, generator=g) * 1.5 - 1.0
        elif leaf in ("dt_bias", "b"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf == "router":
            t = torch.randn(shape, generator=g) * router_gain / shape[-1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) * 1.5 / shape[-1] ** 0.5
        if leaf == "down":
            t = t * expert_gain
        w[name] = t.bfloat16().float()          # values that a bfloat16 file holds exactly
    return w


def plain_logits(w, cfg, tokens, margins=None):
    w64 = {k: v.double() for k, v in w.items()}
    with torch.no_grad():
        return P.forward(w64, cfg, tokens, margins=margins).float()


def settled_weights(cfg: dict, requests, min_margin: float = 0.05, expert_gain: float = 1.0):
    """Weights (by trying seeds) with which no router decision on the given requests is a close call in float32. In
    bfloat16 the router's input carries rounding of a few parts in a thousand, and with random routers about one
    decision in a hundred is closer than that: whole-model tests in bfloat16 therefore use ``expert_gain`` 0.1, which
    keeps every kernel on its path but makes the turn of one near-tie a small change of the stream instead of a new
    sequence (the experts themselves are tested at full strength alone, on inputs without close calls, and in float32)."""
    for seed in range(100, 140):
        w = make_weights(cfg, seed, expert_gain=expert_gain)
        margins = []
        plain = {rid: plain_logits(w, cfg, toks, margins) for rid, toks in requests.items()}
        if not margins or min(margins) >= min_margin:
            return w, plain
    raise AssertionError("no seed gives clear router decisions; widen the routers' spread")


def write_model(path: str, cfg: dict, w, dtype=torch.float32) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))
    return path


BACKENDS = [pytest.param(("emu", "float32"), id="emu"),
            pytest.param(("cuda", "float32"), id="cuda-f32", marks=pytest.mark.gpu),
            pytest.param(("cuda", "bfloat16"), id="cuda-bf16", marks=pytest.mark.gpu)]


def runtime_for(backend):
    """(Runtime, device) of a backend, for tests that build single parts."""
    from serve_b200.engine.runtime import Runtime

    kind, dtype = backend
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    if kind == "emu":
        from tests.emu_kernels import EmuKernels

        return Runtime(EmuKernels("cpu", torch.float64), "cpu", dt), "cpu"
    from serve_b200.kernels import load_kernels

    return Runtime(load_kernels("cuda:0"), "cuda:0", dt), "cuda:0"


def make_engine(folder, backend, page, num_pages, max_slots=4, graphs=False, budget=512, context=None):
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine

    kind, dtype = backend
    ec = EngineConfig(dtype=dtype, page_size=page, num_pages=num_pages, max_slots=max_slots, max_tokens_per_step=budget,
                      max_context=context or num_pages * page, use_cuda_graphs=graphs and kind == "cuda",
                      device="cpu" if kind == "emu" else "cuda:0")
    if kind == "emu":
        from tests.emu_kernels import EmuKernels

        return Engine.from_folder(folder, ec, kernels=EmuKernels("cpu"))
    return Engine.from_folder(folder, ec)


def tolerance(backend, plain) -> float:
    """float32: rounding of float sums. bfloat16: activations are rounded to 8 bits several times a layer; the bound is
    2^-5 of the largest logit (these models have convolutions and recurrences between the roundings)."""
    scale = max(float(p.abs().max()) for p in plain.values())
    return scale * (2e-4 if backend[1] == "float32" else 2.0 ** -5)


def compare_rows(got, plain, backend) -> float:
    """Every collected row against the plain logits. float32: every element within ``tolerance``. bfloat16: a row's
    error is the root mean square of its difference (means taken off) over that of the plain row; rounding to 8 bits
    several times a layer gives a few percent. A router may also turn a near-tie the other way in bfloat16, which
    changes that token's row and, through the states, fades into the rows after it; so at most 3 % of the rows (or two) may
    exceed the bound, none may be 10 times over it, and every value must be finite. (The float32 run of the same kernels
    is the sharp test of every mask, edge and state; bfloat16 differs from it only in the type the kernels load and store.)"""
    from tests import helpers

    if backend[1] == "float32":
        return helpers.compare_with_plain(got, plain, atol=tolerance(backend, plain))
    bound, over, worst = 0.12, [], 0.0
    for (rid, pos), row in got.items():
        ref = plain[rid][pos]
        assert bool(torch.isfinite(row).all()), f"request {rid!r} position {pos}: not finite"
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt())
        worst = max(worst, e)
        if e > bound:
            over.append((rid, pos, round(e, 3)))
    assert len(over) <= max(2, 0.03 * len(got)) and worst <= 10 * bound, f"{len(over)} of {len(got)} rows over the bound: {sorted(over)[:8]}"
    return worst
