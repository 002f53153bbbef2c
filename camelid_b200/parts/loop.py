"""The input of a pass over a stretch of layers that runs several times with the same weights:
from the second pass on the embedding output is added to the residual stream, and before
every pass a vector of that pass (row ``number`` of a [passes, hidden] tensor)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, TensorSpec, register_part


@register_part("pass_input", "loop_step")
class LoopStep(Part):
    graph_safe = True
    graph_safe_any_step = True
    needs_base = True              # the engine keeps the embedding output for it

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.passes = int(params["passes"])
        self.tensor = params.get("tensor") or self.prefix + "weight"
        self.steps = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.passes, self.hidden_size), "low_rank")}

    def load(self, tensors, device, dtype):
        self.steps = tensors[self.tensor].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, h, base, number: int):
        ops.add_rows_vec(h, base if number > 0 else None, self.steps[number])
