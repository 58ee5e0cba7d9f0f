"""The Rogisun decoder as a layer description.

A stack of pre-norm layers, each reading its sub-layers' inputs through a short residual convolution over time,
with one of three mixers (fixed-decay linear attention; a selective state space layer; softmax attention with a
distance penalty inside blocks of positions, side by side with a gated delta rule) and a feed-forward of routed
experts, or none. The head is the embedding table. Tensor names: "embed", "final.norm", and under "l<i>." the
layer's "norm1", "canon1", "mix.*", "norm2", "canon2", "mlp.*".
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.rogisun import RogisunConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the distance penalty of head h of H is 2^(-8 (h + 1) / H) per position
SLOPE_POWER = 8.0
# the experts' activation: g * sigmoid(1.702 g) * (u + 1) on clamped g and u
SWISH_ALPHA = 1.702


def _mixer_spec(kind: str, m: dict, width: int, eps: float, prefix: str) -> PartSpec:
    if kind == "lightning":
        return PartSpec("lightning", {"hidden": width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                      "decay": list(m["decay"]), "eps": eps}, prefix)
    if kind == "mamba2":
        return PartSpec("mamba2", {"hidden": width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
                                   "norm_groups": m["norm_groups"], "taps": m["conv"], "eps": eps}, prefix)
    a, d = m["left"], m["right"]
    left = PartSpec("distance_bias_attention", {
        "hidden": width, "heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"], "vdim": a["vdim"], "scale": a["scale"],
        "chunk": a["mask"]["size"], "slope_power": SLOPE_POWER, "value_norm_eps": eps, "head_gate": True}, prefix + "left.")
    right = PartSpec("gated_delta", {"hidden": width, "heads": d["heads"], "kv_heads": d["kv_heads"], "dim": d["dim"], "vdim": d["vdim"],
                                     "taps": d["conv"], "eps": eps, "rank": d.get("rank")}, prefix + "right.")
    return PartSpec("parallel", {"hidden": width, "left": left, "right": right, "left_scale": m["left_scale"],
                                 "right_scale": m["right_scale"]}, prefix)


def rogisun_spec(cfg: RogisunConfig) -> ModelSpec:
    width, eps, taps = cfg.width, cfg.eps, cfg.canon_taps
    norm = lambda name, prefix: PartSpec("rms", {"size": width, "eps": eps, "weight_name": name}, prefix)
    canon = lambda name, prefix: PartSpec("short_conv", {"channels": width, "taps": taps, "weight_name": name, "residual": True}, prefix)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": norm("norm1", p), "mixer_filter": canon("canon1", p),
                 "mixer": _mixer_spec(layer["type"], layer["mixer"], width, eps, p + "mix.")}
        f = layer["mlp"]
        if f is not None:
            parts["feed_forward_norm"] = norm("norm2", p)
            parts["feed_forward_filter"] = canon("canon2", p)
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden": width, "experts": f["router"]["experts"], "top": f["router"]["top"], "ff": f["expert"]["ff"],
                "score": "sigmoid", "renormalise": False, "scale_input": True, "activation": "clamped_swish",
                "limit": f["expert"]["limit"], "alpha": SWISH_ALPHA}, p + "mlp.")
        layers.append(LayerSpec(PartSpec("pre_norm_filtered"), parts))
    spec = ModelSpec(
        architecture=RogisunConfig.architecture, hidden_size=width, vocab_size=cfg.vocab,
        embedding=PartSpec("table", {"vocab": cfg.vocab, "hidden": width, "name": "embed"}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("final.norm", ""),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": width, "name": "head", "tied_to": "embed"}),
        max_position=cfg.max_position)
    spec.validate()
    return spec


register_architecture(RogisunConfig.architecture, RogisunConfig, rogisun_spec)
