"""Token shift: what a mixer reads is its input mixed, channel by channel, with the input of
the token before: x'_t = x_t + (x_(t-1) - x_t) * mix, zeros before a sequence's first token.
The last row of a step is kept per sequence (float32) for the first row of the next."""
from __future__ import annotations

import torch

from ..cache.book import StateSpec
from ..csrc import ops
from .base import Part, TensorSpec, register_part


@register_part("shift", "token_shift")
class TokenShift(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.tensor = params.get("tensor") or self.prefix + "weight"
        self.mix = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.hidden_size,), "fraction")}

    def load(self, tensors, device, dtype):
        self.mix = tensors[self.tensor].to(device=device, dtype=torch.float32).contiguous()

    def cache_spec(self):
        return StateSpec((1, self.hidden_size), "float32", "shift")

    def forward(self, ctx, x):
        state = ctx.state("shift")                                # [slots, 1, hidden]
        out = ctx.buffer("shifted", tuple(x.shape), x.dtype)
        ops.token_shift(x, self.mix, state, ctx.row_seq, ctx.row_pos, ctx.seq_row0, ctx.seq_slot, out)
        ops.keep_last_rows(x, 0, self.hidden_size, state, ctx.seq_row0, ctx.seq_new, ctx.seq_start, ctx.seq_slot, ctx.n_seqs)
        return out
