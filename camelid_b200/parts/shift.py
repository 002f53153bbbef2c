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

    def norm_and_shift(self, ctx, h, norm):
        """One-token steps after an RMS norm of the library: norm, shift and the kept row in one launch (the
        same arithmetic as the parts one after the other). None where that does not apply."""
        if not (ctx.decode and getattr(norm, "kind", "") == "rmsnorm" and ctx.deferred is None
                and self.hidden_size * 4 <= 48 * 1024):
            return None
        pending, ctx.pending = ctx.pending, None
        out = ctx.buffer("shifted", (ctx.n_rows, self.hidden_size))
        ops.rmsnorm_shift(h, norm.weight, norm.eps, self.mix, ctx.state("shift"), ctx.row_seq, ctx.row_pos, ctx.seq_slot, out,
                          pending)
        return out

    def forward(self, ctx, x):
        state = ctx.state("shift")                                # [slots, 1, hidden]
        out = ctx.buffer("shifted", tuple(x.shape), x.dtype)
        ops.token_shift(x, self.mix, state, ctx.row_seq, ctx.row_pos, ctx.seq_row0, ctx.seq_slot, out)
        ops.keep_last_rows(x, 0, self.hidden_size, state, ctx.seq_row0, ctx.seq_new, ctx.seq_start, ctx.seq_slot, ctx.n_seqs)
        return out
