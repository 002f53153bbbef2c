"""Several mixers side by side: all read the same rows, and the layer adds the mean of their
outputs, each first RMS-normed over the model width with a weight of its own
(``<prefix><branch>.out``):

    y = (1 / B) * sum over branches b of rmsnorm(mixer_b(x)) * out_b.

A branch is any registered mixer that offers ``branch_output(ctx, x, name)``; each keeps its
own cache or state (the entry's cache needs are the branches' together).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import ConfigError
from .base import Part, TensorSpec, build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixers(Part):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.names = [name for name, _ in params["branches"]]
        self.branches = [build_part("mixer", spec) for _, spec in params["branches"]]
        if not 1 <= len(self.branches) <= 4:
            raise ConfigError("branches", f"1 to 4 mixers can stand side by side, got {len(self.branches)}")
        for name, b in zip(self.names, self.branches):
            if not hasattr(b, "branch_output"):
                raise ConfigError("branches", f"the mixer {b.kind!r} of branch {name!r} cannot stand beside others")
        self.out_w = None

    @property
    def graph_safe(self):
        return all(b.graph_safe for b in self.branches)

    @property
    def graph_safe_any_step(self):
        return all(b.graph_safe_any_step for b in self.branches)

    def tensor_specs(self):
        specs = {}
        for name, b in zip(self.names, self.branches):
            specs.update(b.tensor_specs())
            specs[f"{self.prefix}{name}.out"] = TensorSpec((self.hidden_size,), "norm")
        return specs

    def load(self, tensors, device, dtype):
        for b in self.branches:
            b.load(tensors, device, dtype)
        self.out_w = [tensors[f"{self.prefix}{name}.out"].to(device=device, dtype=torch.float32).contiguous()
                      for name in self.names]
        # Branches that read the same rows through one stacked input matrix each (``w_in``): all of them stacked
        # once more, so that one product serves every branch; each keeps its rows of it as a view.
        self.w_in = None
        self.in_cols = []
        if len(self.branches) > 1 and all(getattr(b, "w_in", None) is not None for b in self.branches):
            stacked = torch.cat([b.w_in for b in self.branches], dim=0).contiguous()
            at = 0
            for b in self.branches:
                n = b.w_in.shape[0]
                b.w_in = stacked[at:at + n]
                self.in_cols.append((at, n))
                at += n
            self.w_in = stacked

    def cache_spec(self):
        return [b.cache_spec() for b in self.branches]

    def query_tile_sizes(self):
        return [r for b in self.branches for r in b.query_tile_sizes()]

    def forward(self, ctx, x, residual):
        if self.w_in is not None:
            from . import linear
            proj = linear.product_rows_f32(ctx, x, self.w_in, "branches_proj")
            ys = [b.branch_output(ctx, x, f"branch{i}_out", proj[:, at:at + n])
                  for i, (b, (at, n)) in enumerate(zip(self.branches, self.in_cols))]
        else:
            ys = [b.branch_output(ctx, x, f"branch{i}_out") for i, b in enumerate(self.branches)]
        ops.norm_combine(list(zip(ys, self.out_w)), residual, self.eps, 1.0 / len(self.branches))
