"""The Bapavik decoder as a layer description.

x = embed[token] * scale; pre-norm layers whose norm is a layer norm with a weight and no bias; the mixer of a layer
is softmax attention without rotation (queries and keys normalised over the whole projection, a query temperature
that grows with the logarithm of the position, capped scores, a sink in the softmax's denominator) or latent
attention (keys and values read out of one small cached vector per token, plus one rotated key part shared by all
heads); the feed-forward is dense with a clamped gated activation, a set of small experts that a table over token
ids picks, or absent. A run of layers may repeat with the same weights, each pass with a cache of its own. Final
layer norm and an untied head. Tensor names: "embed", "final.norm", "head", and under "l<i>." the layer's "norm1",
"mix.*", "norm2", "mlp.*".
"""
from __future__ import annotations

from ..config.bapavik import BapavikConfig
from ..config.base import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the dense feed-forward's activation: g * sigmoid(1.702 g) * (u + 1) on clamped g and u
SWISH_ALPHA = 1.702


def _mixer_spec(kind: str, m: dict, width: int, eps: float, prefix: str) -> PartSpec:
    if kind == "attention":
        return PartSpec("capped_sink_attention", {
            "hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
            "softcap": m.get("softcap"), "sink": True, "qk_norm_eps": eps, "q_temp": m.get("q_temp")}, prefix)
    return PartSpec("latent_attention", {
        "hidden": width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
        "scale": m["scale"], "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"], "eps": eps}, prefix)


def _feed_forward_spec(f: dict, width: int, vocab: int, prefix: str) -> PartSpec:
    if f["kind"] == "dense":
        return PartSpec("gated_dense", {"hidden": width, "intermediate": f["ff"], "activation": "clamped_swish", "limit": f["limit"],
                                        "alpha": SWISH_ALPHA, "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix)
    return PartSpec("table_experts", {"hidden": width, "experts": f["router"]["experts"], "top": f["router"]["top"],
                                      "ff": f["expert"]["ff"], "vocab": vocab, "activation": "relu_squared"}, prefix)


def bapavik_spec(cfg: BapavikConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.eps
    norm = lambda name, prefix: PartSpec("layer_norm", {"size": width, "eps": eps, "weight_name": name}, prefix)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": norm("norm1", p), "mixer": _mixer_spec(layer["type"], layer["mixer"], width, eps, p + "mix.")}
        if layer["mlp"] is not None:
            parts["feed_forward_norm"] = norm("norm2", p)
            parts["feed_forward"] = _feed_forward_spec(layer["mlp"], width, cfg.vocab, p + "mlp.")
        layers.append(LayerSpec(PartSpec("pre_norm_filtered"), parts))
    spec = ModelSpec(
        architecture=BapavikConfig.architecture, hidden_size=width, vocab_size=cfg.vocab,
        embedding=PartSpec("table", {"vocab": cfg.vocab, "hidden": width, "name": "embed", "scale": cfg.embedding_scale}),
        layers=layers, schedule=[ScheduleEntry(i) for i in cfg.layer_order()],
        final_norm=norm("final.norm", ""),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": width, "name": "head", "tied_to": None}),
        max_position=cfg.max_position)
    spec.validate()
    return spec


register_architecture(BapavikConfig.architecture, BapavikConfig, bapavik_spec)
