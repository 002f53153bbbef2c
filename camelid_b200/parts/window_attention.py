"""Softmax attention over a sliding window without rotation, as a mixer: grouped queries, keys
and values of different sizes, optional per-head RMS norm of q and k (one weight per channel,
shared by the heads), an optional penalty on distance

    score(i, j) = (q_i . k_j) * scale - r1[head] * ln(1 + r2[head] * (i - j)),    0 <= i - j < window,

and an optional output gate: the concatenated heads times sigmoid(x Wg^T) before the output
projection. Tensors under the prefix: ``q``, ``k``, ``v``, ``o`` (and ``g``, ``q.norm``,
``k.norm``, ``r1``, ``r2`` where the options ask for them), linear weights [out, in].

Scores, softmax weights and the norms are float32; keys and values lie in the paged cache in
the compute type, and a windowed group gives back the pages no later query can see.
"""
from __future__ import annotations

import torch

from ..cache.book import KVSpec
from ..csrc import ops
from ..errors import ConfigError
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("mixer", "window_attention")
class WindowAttention(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.window = int(params["window"]) if params.get("window") else None
        self.scale = float(params["scale"]) if params.get("scale") is not None else self.head_dim ** -0.5
        self.qk_norm = bool(params.get("qk_norm", False))
        self.penalty = params.get("distance_penalty")
        self.output_gate = bool(params.get("output_gate", False))
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ConfigError("num_kv_heads", f"{self.num_kv_heads} kv heads do not divide {self.num_heads} heads")
        if self.penalty not in (None, "log"):
            raise ConfigError("distance_penalty", f"unknown penalty {self.penalty!r}; known: log")
        if self.value_dim > 256:
            raise ConfigError("value_dim", f"the window attention kernel takes values of up to 256 channels, got {self.value_dim}")
        if self.window is not None and self.window <= 0:
            raise ConfigError("window", f"must be greater than zero, got {self.window}")
        self.q_width = self.num_heads * self.head_dim
        self.k_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_kv_heads * self.value_dim
        self.o_width = self.num_heads * self.value_dim
        self.gate_col = self.q_width + self.k_width + self.v_width
        self.w_in = self.w_o = self.q_w = self.k_w = self.r1 = self.r2 = None

    def tensor_specs(self):
        p, hid = self.prefix, self.hidden_size
        specs = {p + "q": TensorSpec((self.q_width, hid)), p + "k": TensorSpec((self.k_width, hid)),
                 p + "v": TensorSpec((self.v_width, hid)), p + "o": TensorSpec((hid, self.o_width))}
        if self.output_gate:
            specs[p + "g"] = TensorSpec((self.o_width, hid))
        if self.qk_norm:
            specs[p + "q.norm"] = TensorSpec((self.head_dim,), "norm")
            specs[p + "k.norm"] = TensorSpec((self.head_dim,), "norm")
        if self.penalty:
            specs[p + "r1"] = TensorSpec((self.num_heads,), "fraction")
            specs[p + "r2"] = TensorSpec((self.num_heads,), "fraction")
        return specs

    def load(self, tensors, device, dtype):
        p = self.prefix
        names = ["q", "k", "v"] + (["g"] if self.output_gate else [])
        self.w_in = torch.cat([to_device(tensors[p + n], device, dtype) for n in names], dim=0).contiguous()
        self.w_o = to_device(tensors[p + "o"], device, dtype)
        f32 = lambda n: tensors[p + n].to(device=device, dtype=torch.float32).contiguous()      # noqa: E731
        if self.qk_norm:
            self.q_w, self.k_w = f32("q.norm"), f32("k.norm")
        if self.penalty:
            self.r1, self.r2 = f32("r1"), f32("r2")

    def cache_spec(self):
        return KVSpec(self.num_kv_heads, self.head_dim, self.window,
                      self.value_dim if self.value_dim != self.head_dim else None)

    def query_tile_sizes(self):
        if self.value_dim == self.head_dim and self.head_dim in (64, 128):
            return [ops.attn_tc_tiling(self.num_heads, self.num_kv_heads)[0]]
        return []

    def attend(self, ctx, x, proj=None):
        """The gated heads [rows, heads * value_dim] in the compute type: the input of the output projection.
        ``proj``: x @ w_in^T in float32 where a caller has made it already (as columns of a wider product)."""
        n = ctx.n_rows
        group, k_pages, v_pages = ctx.kv()
        table = ctx.block_table(group)
        if proj is None:
            proj = linear.product_rows_f32(ctx, x, self.w_in, "wa_proj")
        q = ctx.buffer("wa_q", (n, self.q_width))
        ops.qk_norm_kv_write(proj, self.q_w, self.k_w, self.eps, ctx.row_seq, ctx.row_pos, table, q, k_pages, v_pages,
                             self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim)
        out = ctx.buffer("wa_out", (n, self.o_width))
        # prompts in bfloat16 with keys and values of 64 or 128 channels: the tcgen05 kernel of the library's
        # attention (scores and softmax in float there too), then the gate; everything else on the kernel below
        if not ctx.decode and self.value_dim == self.head_dim and ops.attn_tc_usable(q, out, self.head_dim):
            rows, hpc, chunks = ops.attn_tc_tiling(self.num_heads, self.num_kv_heads)
            tile_seq, tile_q0, n_tiles = ctx.query_tiles(rows)
            ops.attn_prefill_tc(q, out, k_pages, v_pages, table, tile_seq, tile_q0, n_tiles, ctx.seq_row0, ctx.seq_start,
                                ctx.seq_new, self.num_heads, self.num_kv_heads, self.head_dim, rows, hpc, chunks,
                                self.window or 0, self.scale, linear._err_word(q.device), self.r1, self.r2)
            if self.output_gate:
                ops.gate_rows_(out, proj, self.gate_col)
            return out
        ops.window_attention(q, k_pages, v_pages, table, ctx.row_seq, ctx.row_pos, self.r1, self.r2,
                             proj if self.output_gate else None, self.gate_col, out, self.num_heads, self.num_kv_heads,
                             self.head_dim, self.value_dim, self.window or 0, self.scale)
        return out

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self.attend(ctx, x), self.w_o, residual, "o_partial")

    def branch_output(self, ctx, x, name: str, proj=None):
        """The mixer's output as float32 [rows, hidden] or split sums [splits, rows, hidden], in a buffer of its own."""
        return linear.product_f32(ctx, self.attend(ctx, x, proj), self.w_o, name)
