"""What follows the read-out of a recurrent mixer: a root-mean-square norm over groups of channels and a gate.

out = scale * [gate] * rms_groups([gate] * y) * weight, computed in float from the float read-out y:
``groups`` equal parts of a row are each divided by their own root mean square (eps inside the root); the weight
has one entry per channel, or fewer that repeat (one vector shared by all heads); the gate, sigmoid or silu of a
projection of the layer's input, multiplies either before the norm or after it.
"""
from __future__ import annotations

from .base import Part, TensorDecl, register_part


@register_part("norm", "gated_group_rms")
class GatedGroupRMS(Part):
    """params: channels, groups, eps, weight_size (default channels), weight_name, gate ("sigmoid" | "silu" | None),
    gate_first (bool)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.channels = int(p["channels"])
        self.groups = int(p["groups"])
        self.eps = float(p["eps"])
        self.weight_size = int(p.get("weight_size", self.channels))
        if self.groups <= 0 or self.channels % self.groups or self.channels % self.weight_size:
            raise ValueError(f"{self.channels} channels do not split into {self.groups} groups / weights of {self.weight_size}")
        self.weight_name = self.prefix + p.get("weight_name", "weight")
        self.gate = p.get("gate")
        self.gate_first = bool(p.get("gate_first", False))
        self.weight = None

    def tensor_decls(self):
        return [TensorDecl(self.weight_name, (self.weight_size,), role="vector", init="norm")]

    def load(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, y, gate, out, scale: float = 1.0):
        self.rt.kernels.gated_norm(y, out, groups=self.groups, eps=self.eps, weight=self.weight,
                                   gate=gate if self.gate else None, gate_act=self.gate or "sigmoid",
                                   gate_first=self.gate_first, scale=scale)
        return out
