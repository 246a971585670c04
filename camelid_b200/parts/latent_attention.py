"""Softmax attention whose keys and values of all heads are linear maps of one *latent* row per position.

With h the mixer's input, H heads, per head ``head_dim`` unturned and ``rot_dim`` turned query/key channels, values of
``value_dim`` channels and a latent of ``rank`` channels:

    q = Wq h                         head by head [a_h (head_dim), b_h (rot_dim)]
    d = Wdkv h                       rank + rot_dim rows: c = rmsnorm(d[:rank]) * w, t = turned(d[rank:])
    k_h = [Uk_h c, t],  v_h = Uv_h c
    score_h(i, j) = (a_h(i) . Uk_h c_j + turned(b_h(i)) . t_j) * scale,   j <= i
    out_h = softmax over j (with exp(sink_h) as one more term of the denominator) of v_h, times sigmoid(Wg h)_h

The cache keeps [c_j, t_j] only: one row of rank + rot_dim channels per position for all heads, whose first rank
channels are the values as well (``KVSpec.values_in_keys``). The maps are moved to the query's side, for prompts and
single tokens alike: a' = Uk_h^T a_h (a product per head), attention of [a', turned b] over the rows [c, t] with values
c, then Uv_h on the result (a product per head); a head's gate, being one number, is applied before that map. Prompts
in bfloat16 whose sizes allow it take a tensor-core kernel of their own (all heads of a tile of tokens against a page of
keys that is fetched once), everything else the library's general attention kernel.

Options: ``sink``, ``output_gate`` ("head" or none), ``position`` (a rotary part of ``rot_dim`` channels; pairs of
neighbours or of halves; its ``amplitude`` multiplies sines and cosines), ``scale``.
Tensors under the prefix: ``q``, ``dkv``, ``dkv.norm``, ``uk`` [H * head_dim, rank], ``uv`` [H * value_dim, rank], ``o``
(and ``g``, ``sink``). Scores, softmax, the latent's norm and the rotation are float32.
"""
from __future__ import annotations

import torch

from ..cache.book import KVSpec
from ..config.plan import PartSpec
from ..csrc import ops
from ..errors import ConfigError
from . import linear
from .base import Part, TensorSpec, build_part, register_part, to_device


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.num_heads = int(params["num_heads"])
        self.head_dim = int(params["head_dim"])
        self.rot_dim = int(params["rot_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.rank = int(params["rank"])
        self.scale = float(params["scale"]) if params.get("scale") is not None else (self.head_dim + self.rot_dim) ** -0.5
        self.sink = bool(params.get("sink", False))
        self.output_gate = {False: None, None: None, True: "head"}.get(params.get("output_gate", False), params.get("output_gate"))
        self.position = build_part("position", params.get("position") or PartSpec("none"))
        if self.output_gate not in (None, "head"):
            raise ConfigError("output_gate", f"unknown output gate {self.output_gate!r}; known: head")
        if self.position.rotary_dim != self.rot_dim:
            raise ConfigError("rot_dim", f"the turned part has {self.rot_dim} channels, the position encoding turns {self.position.rotary_dim}")
        if self.rot_dim % 2 or self.rot_dim > 256:
            raise ConfigError("rot_dim", f"must be even and at most 256, got {self.rot_dim}")
        if not 1 <= self.rank <= 512:
            raise ConfigError("rank", f"the attention kernel takes latents of 1..512 channels, got {self.rank}")
        if min(self.num_heads, self.head_dim, self.value_dim) < 1:
            raise ConfigError("num_heads", "heads, head_dim and value_dim must be greater than zero")
        self.q_width = self.num_heads * (self.head_dim + self.rot_dim)
        self.key_dim = self.rank + self.rot_dim                    # channels of a cached row, and of an absorbed query head
        self.gate_width = self.num_heads if self.output_gate else 0
        self.w_in = self.w_o = self.w_uk_t = self.w_uv = self.c_w = self.sink_w = None

    def tensor_specs(self):
        p, hid = self.prefix, self.hidden_size
        specs = {p + "q": TensorSpec((self.q_width, hid)), p + "dkv": TensorSpec((self.key_dim, hid)),
                 p + "dkv.norm": TensorSpec((self.rank,), "norm"), p + "uk": TensorSpec((self.num_heads * self.head_dim, self.rank)),
                 p + "uv": TensorSpec((self.num_heads * self.value_dim, self.rank)),
                 p + "o": TensorSpec((hid, self.num_heads * self.value_dim))}
        if self.output_gate:
            specs[p + "g"] = TensorSpec((self.gate_width, hid))
        if self.sink:
            specs[p + "sink"] = TensorSpec((self.num_heads,), "input_bias")
        return specs

    def load(self, tensors, device, dtype):
        p, H = self.prefix, self.num_heads
        names = ["q", "dkv"] + (["g"] if self.output_gate else [])
        self.w_in = torch.cat([to_device(tensors[p + n], device, dtype) for n in names], dim=0).contiguous()
        self.w_o = to_device(tensors[p + "o"], device, dtype)
        # per head [outputs, inputs]: Uk_h^T takes head_dim channels to rank, Uv_h takes rank channels to value_dim
        self.w_uk_t = to_device(tensors[p + "uk"], device, dtype).view(H, self.head_dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = to_device(tensors[p + "uv"], device, dtype).view(H, self.value_dim, self.rank).contiguous()
        self.c_w = tensors[p + "dkv.norm"].to(device=device, dtype=torch.float32).contiguous()
        if self.sink:
            self.sink_w = tensors[p + "sink"].to(device=device, dtype=torch.float32).contiguous()
        self.position.load(tensors, device, dtype)

    def cache_spec(self):
        return KVSpec(1, self.key_dim, None, self.rank, None, 0, True)

    def query_tile_sizes(self):
        return [ops.latent_prompt_tokens(self.num_heads)]

    def attend(self, ctx, x):
        """The gated heads [rows, heads * value_dim] in the compute type: the input of the output projection."""
        n, H, pos = ctx.n_rows, self.num_heads, self.position
        group, k_pages, v_pages = ctx.kv()
        table = ctx.block_table(group)
        sums = linear.product_f32(ctx, x, self.w_in, "la_proj")           # split sums where the step is small: added below
        q_plain = ctx.buffer("la_q_plain", (n, H * self.head_dim))
        q_full = ctx.buffer("la_q", (n, H * self.key_dim))
        gate = ctx.buffer("la_gate", (n, self.gate_width), torch.float32) if self.output_gate else None
        ops.latent_prepare(sums, self.c_w, self.eps, pos.inv_freq, pos.pairing == "interleaved", pos.amplitude, ctx.row_seq,
                           ctx.row_pos, table, q_plain, q_full, k_pages, H, self.head_dim, self.rot_dim, self.rank, gate)
        ops.head_product(q_plain, self.head_dim, self.w_uk_t, q_full, self.key_dim)
        mixed = ctx.buffer("la_mixed", (n, H * self.rank))               # per head: the weighted latents, gated
        if ops.latent_prompt_usable(q_full, self.rank, self.rot_dim):
            # bfloat16: pages of keys against tiles of (token, head) rows on the tensor cores. Single tokens: a tile is one
            # token's heads, and the pages of a long context are dealt to several blocks (how many follows from the block
            # table's width alone, which a captured step is keyed by), at least two pages each
            tile_seq, tile_q0, n_tiles = ctx.query_tiles(ops.latent_prompt_tokens(H))
            partial, per = None, 0
            if ctx.decode and table.shape[1] >= 4:
                splits = min(32, table.shape[1] // 2)
                per = (table.shape[1] + splits - 1) // splits
                partial = ctx.buffer("la_partial", (splits, n, H, self.rank + 2), torch.float32)
            ops.latent_prompt(q_full, k_pages, mixed, table, tile_seq, tile_q0, n_tiles, ctx.seq_row0, ctx.seq_start, ctx.seq_new,
                              H, self.rank, self.rot_dim, self.scale, self.sink_w, gate, 0, partial, per)
        else:
            ops.window_attention(q_full, k_pages, v_pages, table, ctx.row_seq, ctx.row_pos, None, None, gate, 0, mixed, H, 1,
                                 self.key_dim, self.rank, 0, self.scale, 0, self.sink_w, True, values_in_keys=True)
        out = ctx.buffer("la_out", (n, H * self.value_dim))
        ops.head_product(mixed, self.rank, self.w_uv, out, self.value_dim)
        return out

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self.attend(ctx, x), self.w_o, residual, "o_partial")

    def branch_output(self, ctx, x, name: str, proj=None):
        """The mixer's output as float32 [rows, hidden] or split sums [splits, rows, hidden], in a buffer of its own."""
        return linear.product_f32(ctx, self.attend(ctx, x), self.w_o, name)
