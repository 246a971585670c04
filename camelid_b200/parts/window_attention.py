"""Softmax attention over a limited stretch of keys, as a mixer: grouped queries, keys and values of
different sizes, and a set of options that designs combine:

* ``window``: a query sees the last ``window`` keys; ``chunk``: it sees the keys of its own block of
  ``chunk`` positions (blocks counted from position 0 of the sequence); neither: all keys before it.
* ``qk_norm``: RMS norm of q and k, ``"head"`` (or True) per head with one weight per channel shared by
  the heads, ``"full"`` over the whole projection (all heads at once) with a weight per column.
* ``position``: a rotary encoding (``parts/position.py``) applied to q and k after the norm, pairs of
  neighbouring channels or of the two halves; absent: no rotation.
* ``distance_penalty`` ``"log"``:

      score(i, j) = (q_i . k_j) * scale - r1[head] * ln(1 + r2[head] * (i - j)).

* ``sink``: one learned number per head whose exponential is one more term of the softmax denominator
  (no key, no value, not scaled).
* ``output_gate``: the heads times sigmoid(x Wg^T) before the output projection, ``"channel"`` (or True)
  a number per channel of every head, ``"head"`` one number per head.
* ``keep_first`` n (with ``window``): the first n keys of a sequence stay visible to every later query beside the
  window's (they keep their own positions); the cache holds on to their pages.
* ``bias``: q, k and v have biases (``q.b``, ``k.b``, ``v.b``), added in the projection, before the norms.
* ``softcap`` c: the scaled score becomes c tanh(score / c) before the softmax.
* ``difference`` d (differential attention): every head has two score maps. q holds, head by head, [map 1, map 2] of
  ``head_dim`` channels each, and so does k; each map is a softmax attention of its own over the same values (the q/k
  norm runs per head and map); with L = exp(lq1 . lk1) - exp(lq2 . lk2) + d (four vectors of ``head_dim`` numbers, one
  L for the layer) the head's output is (a1 - L a2) / rms(a1 - L a2) * (1 - d), the root mean square over the head's
  value channels. The cache keeps a key head's two maps as one row of 2 * ``head_dim`` channels.

Tensors under the prefix: ``q``, ``k``, ``v``, ``o`` (and ``g``, ``q.norm``, ``k.norm``, ``r1``, ``r2``,
``sink``, ``lq1``, ``lk1``, ``lq2``, ``lk2`` where the options ask for them), linear weights [out, in].

Scores, softmax weights and the norms are float32; keys and values lie in the paged cache in
the compute type, and a windowed group gives back the pages no later query can see.
"""
from __future__ import annotations

import torch

from ..cache.book import KVSpec
from ..config.plan import PartSpec
from ..csrc import ops
from ..errors import ConfigError
from . import linear
from .base import Part, TensorSpec, build_part, register_part, to_device


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
        self.qk_norm = {False: None, None: None, True: "head"}.get(params.get("qk_norm", False), params.get("qk_norm"))
        self.penalty = params.get("distance_penalty")
        self.output_gate = {False: None, None: None, True: "channel"}.get(params.get("output_gate", False), params.get("output_gate"))
        self.chunk = int(params["chunk"]) if params.get("chunk") else None
        self.keep_first = int(params.get("keep_first") or 0)
        self.bias = bool(params.get("bias", False))
        self.sink = bool(params.get("sink", False))
        self.softcap = float(params["softcap"]) if params.get("softcap") else 0.0
        self.difference = float(params["difference"]) if params.get("difference") is not None else None
        self.maps = 2 if self.difference is not None else 1
        self.position = build_part("position", params.get("position") or PartSpec("none"))
        if self.qk_norm not in (None, "head", "full"):
            raise ConfigError("qk_norm", f"unknown q/k norm {self.qk_norm!r}; known: head, full")
        if self.output_gate not in (None, "channel", "head"):
            raise ConfigError("output_gate", f"unknown output gate {self.output_gate!r}; known: channel, head")
        if self.chunk is not None and self.chunk <= 0:
            raise ConfigError("chunk", f"must be greater than zero, got {self.chunk}")
        if self.position.rotary_dim > self.head_dim:
            raise ConfigError("rotary_dim", f"{self.position.rotary_dim} exceeds the head size {self.head_dim}")
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ConfigError("num_kv_heads", f"{self.num_kv_heads} kv heads do not divide {self.num_heads} heads")
        if self.penalty not in (None, "log"):
            raise ConfigError("distance_penalty", f"unknown penalty {self.penalty!r}; known: log")
        if self.softcap < 0:
            raise ConfigError("softcap", f"must be greater than zero, got {self.softcap}")
        if self.maps == 2 and (self.qk_norm == "full" or self.position.rotary_dim > 0):
            raise ConfigError("difference", "differential attention runs with a per-head q/k norm or none and without rotation")
        if self.value_dim > 256:
            raise ConfigError("value_dim", f"the window attention kernel takes values of up to 256 channels, got {self.value_dim}")
        if self.window is not None and self.window <= 0:
            raise ConfigError("window", f"must be greater than zero, got {self.window}")
        if self.keep_first < 0 or (self.keep_first and (self.window is None or self.chunk is not None or self.maps == 2)):
            raise ConfigError("keep_first", "kept first keys go with a window (and one score map, no blocks of positions)")
        self.q_width = self.num_heads * self.maps * self.head_dim
        self.k_width = self.num_kv_heads * self.maps * self.head_dim
        self.v_width = self.num_kv_heads * self.value_dim
        self.o_width = self.num_heads * self.value_dim
        self.gate_width = {None: 0, "channel": self.o_width, "head": self.num_heads}[self.output_gate]
        # q and k that are rotated, or normed over all heads at once, go through the preparing kernel that does both
        self.prepare = self.position.rotary_dim > 0 or self.qk_norm == "full" or self.bias
        if self.bias and self.maps == 2:
            raise ConfigError("bias", "projection biases are not built for two score maps")
        self.gate_col = self.q_width + self.k_width + self.v_width
        self.w_in = self.w_o = self.q_w = self.k_w = self.r1 = self.r2 = self.sink_w = self.b_in = None
        self.lam = 0.0                  # the factor of the second map, known once the weights are

    def tensor_specs(self):
        p, hid = self.prefix, self.hidden_size
        specs = {p + "q": TensorSpec((self.q_width, hid)), p + "k": TensorSpec((self.k_width, hid)),
                 p + "v": TensorSpec((self.v_width, hid)), p + "o": TensorSpec((hid, self.o_width))}
        if self.output_gate:
            specs[p + "g"] = TensorSpec((self.gate_width, hid))
        if self.qk_norm:
            full = self.qk_norm == "full"
            specs[p + "q.norm"] = TensorSpec((self.q_width if full else self.head_dim,), "norm")
            specs[p + "k.norm"] = TensorSpec((self.k_width if full else self.head_dim,), "norm")
        if self.sink:
            specs[p + "sink"] = TensorSpec((self.num_heads,), "input_bias")
        if self.bias:
            for n, width in (("q.b", self.q_width), ("k.b", self.k_width), ("v.b", self.v_width)):
                specs[p + n] = TensorSpec((width,), "input_bias")
        if self.penalty:
            specs[p + "r1"] = TensorSpec((self.num_heads,), "fraction")
            specs[p + "r2"] = TensorSpec((self.num_heads,), "fraction")
        if self.maps == 2:
            for n in ("lq1", "lk1", "lq2", "lk2"):
                specs[p + n] = TensorSpec((self.head_dim,), "input_bias")
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
        if self.sink:
            self.sink_w = f32("sink")
        if self.bias:                   # one float32 row for the stacked product's columns (nothing for the gate's)
            self.b_in = torch.cat([f32("q.b"), f32("k.b"), f32("v.b"),
                                   torch.zeros(self.gate_width, dtype=torch.float32, device=device)]).contiguous()
        if self.maps == 2:              # one number for the layer, in float32 like the scores it weighs
            l1 = torch.exp(torch.sum(f32("lq1") * f32("lk1")))
            l2 = torch.exp(torch.sum(f32("lq2") * f32("lk2")))
            self.lam = float((l1 - l2 + torch.tensor(self.difference, dtype=torch.float32, device=l1.device)).item())
        self.position.load(tensors, device, dtype)

    def cache_spec(self):
        key_dim = self.maps * self.head_dim
        return KVSpec(self.num_kv_heads, key_dim, self.window, self.value_dim if self.value_dim != key_dim else None, self.chunk,
                      self.keep_first)

    @property
    def _tc_prompts(self) -> bool:
        """Whether prompts can run on the tcgen05 kernel of the library's attention (bfloat16 and the sizes permitting)."""
        # (two score maps with one gate number per head: no design has both; they stay on the general kernel)
        return self.head_dim in (64, 128) and self.value_dim in (64, 128) and not (self.maps == 2 and self.output_gate == "head")

    def query_tile_sizes(self):
        if self._tc_prompts:
            return [ops.attn_tc_tiling(self.num_heads, self.num_kv_heads)[0]]
        return []

    def attend(self, ctx, x, proj=None):
        """The gated heads [rows, heads * value_dim] in the compute type: the input of the output projection.
        ``proj``: x @ w_in^T in float32 where a caller has made it already (as columns of a wider product)."""
        n = ctx.n_rows
        group, k_pages, v_pages = ctx.kv()
        table = ctx.block_table(group)
        q = ctx.buffer("wa_q", (n, self.q_width))
        if self.prepare:
            # the product's split sums (few rows) are added by the preparing kernel, which also hands the gate's logits on
            pos = self.position
            sums = proj if proj is not None else linear.product_f32(ctx, x, self.w_in, "wa_proj")
            proj = ctx.buffer("wa_gate", (n, self.gate_width), torch.float32) if self.output_gate else None
            ops.qkv_prepare(sums, self.q_w, self.k_w, {None: 0, "head": 1, "full": 2}[self.qk_norm], self.eps, pos.inv_freq,
                            pos.rotary_dim, pos.pairing == "interleaved", ctx.row_seq, ctx.row_pos, table, q, k_pages, v_pages,
                            self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, proj, self.b_in, pos.amplitude)
            gate_col = 0
        else:
            gate_col = self.gate_col
            if proj is None:
                proj = linear.product_rows_f32(ctx, x, self.w_in, "wa_proj")
            ops.qk_norm_kv_write(proj, self.q_w, self.k_w, self.eps, ctx.row_seq, ctx.row_pos, table, q, k_pages, v_pages,
                                 self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.maps)
        out = ctx.buffer("wa_out", (n, self.o_width))
        # prompts in bfloat16 with keys (of one score map) and values of 64 or 128 channels: the tcgen05 kernel of the library's
        # attention (scores and softmax in float there too), then the gate; everything else on the kernel below
        if not ctx.decode and self._tc_prompts and ops.attn_tc_usable(q, out, self.head_dim, self.value_dim):
            rows, hpc, chunks = ops.attn_tc_tiling(self.num_heads, self.num_kv_heads)
            tile_seq, tile_q0, n_tiles = ctx.query_tiles(rows)
            # two score maps: each is an attention of its own there (float32 rows), and a second kernel takes their difference
            heads_out = out if self.maps == 1 else ctx.buffer("wa_maps", (n, self.maps * self.o_width), torch.float32)
            ops.attn_prefill_tc(q, heads_out, k_pages, v_pages, table, tile_seq, tile_q0, n_tiles, ctx.seq_row0, ctx.seq_start,
                                ctx.seq_new, self.num_heads, self.num_kv_heads, self.head_dim, rows, hpc, chunks,
                                self.window or 0, self.scale, linear._err_word(q.device), self.r1, self.r2, self.chunk or 0,
                                self.sink_w, proj if self.output_gate == "head" else None, gate_col,
                                self.maps, self.softcap, self.value_dim, self.keep_first)
            if self.maps == 2:
                ops.maps_difference(heads_out, self.lam, self.eps, 1.0 - self.difference, out, self.num_heads, self.value_dim)
            if self.output_gate == "channel":
                ops.gate_rows_(out, proj, gate_col)
            return out
        ops.window_attention(q, k_pages, v_pages, table, ctx.row_seq, ctx.row_pos, self.r1, self.r2,
                             proj if self.output_gate else None, gate_col, out, self.num_heads, self.num_kv_heads,
                             self.head_dim, self.value_dim, self.window or 0, self.scale, self.chunk or 0, self.sink_w,
                             self.output_gate == "head", self.softcap,
                             (self.lam, self.eps, 1.0 - self.difference) if self.maps == 2 else None, self.keep_first)
        return out

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self.attend(ctx, x), self.w_o, residual, "o_partial")

    def branch_output(self, ctx, x, name: str, proj=None):
        """The mixer's output as float32 [rows, hidden] or split sums [splits, rows, hidden], in a buffer of its own."""
        return linear.product_f32(ctx, self.attend(ctx, x, proj), self.w_o, name)
