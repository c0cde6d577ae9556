"""Junctions: what a run order may place between two layers, acting on the residual itself.

"concat_linear"  x <- W [x ; x0]: the residual and the embedding output side by side (x first) through one matrix
                 W [width, 2 width].  params: hidden_size, weight (tensor name).  The operand row is formed in the
                 activation dtype; the product accumulates in float32 and writes the float32 residual.
"""
from __future__ import annotations

from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from .base import Junction, register_junction
from .linear import project


@register_junction("concat_linear")
class ConcatLinear(Junction):
    graph_safe = True
    needs_embedding_output = True

    def __init__(self, spec, prefix="", workspace=None):
        super().__init__(spec, prefix)
        self.hidden = int(spec["hidden_size"])
        self.weight_name = prefix + spec["weight"]
        self.ws, self.weight = workspace, None

    def requirements(self):
        return [TensorReq(self.weight_name, (self.hidden, 2 * self.hidden))]

    def load(self, source, device):
        self.weight = source.get(self.weight_name, device).contiguous()

    def run(self, x, x0, batch) -> None:
        cat = self.ws.get("junction_cat", (x.shape[0], 2 * self.hidden), batch.dtype)
        with phase("junction"):
            K.concat_rows(x, x0, cat)
            project(cat, self.weight, x)
