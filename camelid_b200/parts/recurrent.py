"""Mixers that keep a matrix state S [key_dim, value_dim] per head and sequence instead of keys
and values. The state is float32, starts at zero and is carried from token to token; gates,
decays, unit norms and the read-out norm are float32 as well.

``matrix_memory``: per head, with q = x Wq^T / sqrt(key_dim), k, v and capped log gates
i = cap tanh((x Wi^T + bi) / cap), f = logsigmoid(cap tanh((x Wf^T + bf) / cap)):

    m' = max(f + m, i)          (m starts at 0)
    S' = e^(f + m - m') S + e^(i - m') k v^T,   n' likewise with k alone
    o  = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)

then o / rms(o) per head, times ``norm`` (all heads' size), times sigmoid(x Wg^T), then Wo.
Tensors: ``q k v g o i i.b f f.b norm``.

``channel_delta``: the gated delta rule with a decay per head and key channel. q, k
(``num_qk_heads`` heads, shared by groups of value heads) and v pass a short causal
convolution per channel (``<name>.conv`` [channels, taps], the last tap the current token's)
and SiLU; q and k become unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times
1 / sqrt(key_dim); beta = sigmoid(x Wb^T); g = exp(-exp(A_log[head]) softplus(Wa2 (Wa1 x) + dt_bias)):

    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

then o / rms(o) per head times ``norm`` (value_dim, shared), times sigmoid(Wg2 (Wg1 x)), then
Wo. The last taps - 1 inputs of the convolution are state too. Tensors:
``q q.conv k k.conv v v.conv b A_log dt_bias a1 a2 g1 g2 norm o``; the width of the two
low-rank pairs is the stored tensors' own.

``gated_delta``: the same rule with one decay per head, g = exp(-exp(A_log[head]) softplus(Wa x + dt_bias[head])) (S <- g S),
the decay's and the gate's inputs straight from the mixer's input (``a`` [heads, hidden], ``g`` [heads x value_dim, hidden])
and a SiLU gate on the read-out. Both are one part with three options: ``decay`` "channel" | "head", ``low_rank`` (the
pairs a1/a2, g1/g2 or the plain matrices a, g) and ``gate`` "sigmoid" | "silu".
"""
from __future__ import annotations

import torch

from ..cache.book import StateSpec
from ..config.plan import PartSpec
from ..csrc import ops
from ..errors import ConfigError, WeightsError
from . import linear
from .base import Part, TensorSpec, build_part, register_part, to_device


def _check_dims(key_dim: int, value_dim: int):
    if not 1 <= key_dim <= 256:
        raise ConfigError("key_dim", f"the scan kernels take key sizes 1..256, got {key_dim}")
    if value_dim < 1:
        raise ConfigError("value_dim", f"must be greater than zero, got {value_dim}")


@register_part("mixer", "matrix_memory")
class MatrixMemory(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.num_heads = int(params["num_heads"])
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        self.gate_cap = float(params["gate_cap"])
        _check_dims(self.key_dim, self.value_dim)
        self.qk_width = self.num_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        # columns of the stacked input projection: q, k, v, output gate, input gate, forget gate
        self.cols = (0, self.qk_width, 2 * self.qk_width, 2 * self.qk_width + 2 * self.v_width,
                     2 * self.qk_width + 2 * self.v_width + self.num_heads)
        self.gate_col = 2 * self.qk_width + self.v_width
        self.w_in = self.w_o = self.i_bias = self.f_bias = self.norm_w = None

    def tensor_specs(self):
        p, hid, h = self.prefix, self.hidden_size, self.num_heads
        return {p + "q": TensorSpec((self.qk_width, hid)), p + "k": TensorSpec((self.qk_width, hid)),
                p + "v": TensorSpec((self.v_width, hid)), p + "g": TensorSpec((self.v_width, hid)),
                p + "o": TensorSpec((hid, self.v_width)), p + "norm": TensorSpec((self.v_width,), "norm"),
                p + "i": TensorSpec((h, hid)), p + "i.b": TensorSpec((h,), "input_bias"),
                p + "f": TensorSpec((h, hid)), p + "f.b": TensorSpec((h,), "forget_bias")}

    def load(self, tensors, device, dtype):
        p = self.prefix
        self.w_in = torch.cat([to_device(tensors[p + n], device, dtype) for n in ("q", "k", "v", "g", "i", "f")], 0).contiguous()
        self.w_o = to_device(tensors[p + "o"], device, dtype)
        f32 = lambda n: tensors[p + n].to(device=device, dtype=torch.float32).contiguous()      # noqa: E731
        self.i_bias, self.f_bias, self.norm_w = f32("i.b"), f32("f.b"), f32("norm")

    def cache_spec(self):
        # S column by column with n as one more column; the running maximum, one copy per column
        return [StateSpec((self.num_heads, self.value_dim + 1, self.key_dim), "float32", "memory"),
                StateSpec((self.num_heads, self.value_dim + 1), "float32", "maximum")]

    def read_out(self, ctx, x, proj=None):
        n = ctx.n_rows
        if proj is None:
            proj = linear.product_rows_f32(ctx, x, self.w_in, "mm_proj")
        raw = ctx.buffer("mm_raw", (n, self.num_heads, self.value_dim + 2), torch.float32)
        ops.memory_scan(proj, self.cols, self.i_bias, self.f_bias, self.gate_cap, self.key_dim ** -0.5, ctx.state("memory"),
                        ctx.state("maximum"), ctx.seq_row0, ctx.seq_new, ctx.seq_start, ctx.seq_slot, raw, ctx.n_seqs, self.num_heads,
                        self.key_dim, self.value_dim)
        out = ctx.buffer("mm_out", (n, self.v_width))
        ops.head_norm_gate(raw, True, self.norm_w, True, proj, self.gate_col, out, self.num_heads, self.value_dim, self.eps)
        return out

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self.read_out(ctx, x), self.w_o, residual, "o_partial")

    def branch_output(self, ctx, x, name: str, proj=None):
        return linear.product_f32(ctx, self.read_out(ctx, x, proj), self.w_o, name)


@register_part("mixer", "channel_delta")
class ChannelDelta(Part):
    graph_safe = True
    graph_safe_any_step = True
    default_decay, default_gate, default_low_rank = "channel", "sigmoid", True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.num_heads = int(params["num_heads"])
        self.num_qk_heads = int(params.get("num_qk_heads") or self.num_heads)
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        self.taps = int(params["conv_taps"])
        _check_dims(self.key_dim, self.value_dim)
        if self.num_qk_heads <= 0 or self.num_heads % self.num_qk_heads:
            raise ConfigError("num_qk_heads", f"{self.num_qk_heads} q/k heads do not divide {self.num_heads} heads")
        if self.taps < 1:
            raise ConfigError("conv_taps", f"must be at least 1, got {self.taps}")
        self.decay = params.get("decay") or self.default_decay
        self.gate = params.get("gate") or self.default_gate
        self.low_rank = bool(params["low_rank"]) if params.get("low_rank") is not None else self.default_low_rank
        if self.decay not in ("channel", "head"):
            raise ConfigError("decay", f"one decay per key 'channel' or per 'head', got {self.decay!r}")
        if self.gate not in ("sigmoid", "silu"):
            raise ConfigError("gate", f"unknown read-out gate {self.gate!r}; known: sigmoid, silu")
        # the low-rank width is the stored tensors' own; this one is for random weights
        self.rank = int(params.get("rank") or max(8, self.hidden_size // 8 // 8 * 8))
        self.qk_width = self.num_qk_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        self.decay_width = self.num_heads * (self.key_dim if self.decay == "channel" else 1)
        self.channels = 2 * self.qk_width + self.v_width
        self.w_in = self.w_low = self.w_high = self.w_o = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def tensor_specs(self):
        p, hid, r = self.prefix, self.hidden_size, self.rank
        specs = {p + "q": TensorSpec((self.qk_width, hid)), p + "q.conv": TensorSpec((self.qk_width, self.taps), "conv"),
                 p + "k": TensorSpec((self.qk_width, hid)), p + "k.conv": TensorSpec((self.qk_width, self.taps), "conv"),
                 p + "v": TensorSpec((self.v_width, hid)), p + "v.conv": TensorSpec((self.v_width, self.taps), "conv"),
                 p + "b": TensorSpec((self.num_heads, hid)), p + "A_log": TensorSpec((self.num_heads,), "log_rate"),
                 p + "dt_bias": TensorSpec((self.decay_width,), "log_rate"), p + "norm": TensorSpec((self.value_dim,), "norm"),
                 p + "o": TensorSpec((hid, self.v_width))}
        if self.low_rank:
            specs.update({p + "a1": TensorSpec((r, hid), "linear", (0,)), p + "a2": TensorSpec((self.decay_width, r), "low_rank", (1,)),
                          p + "g1": TensorSpec((r, hid), "linear", (0,)), p + "g2": TensorSpec((self.v_width, r), "low_rank", (1,))})
        else:
            specs.update({p + "a": TensorSpec((self.decay_width, hid)), p + "g": TensorSpec((self.v_width, hid))})
        return specs

    def load(self, tensors, device, dtype):
        p = self.prefix
        dev = lambda n: to_device(tensors[p + n], device, dtype)                                  # noqa: E731
        f32 = lambda n: tensors[p + n].to(device=device, dtype=torch.float32).contiguous()      # noqa: E731
        self.w_o = dev("o")
        self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], 0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")
        if not self.low_rank:           # the decays' and the gate's inputs are columns of the one input product
            self.w_in = torch.cat([dev(n) for n in ("q", "k", "v", "b", "a", "g")], 0).contiguous()
            return
        self.w_in = torch.cat([dev(n) for n in ("q", "k", "v", "b")], 0).contiguous()
        a1, a2, g1, g2 = dev("a1"), dev("a2"), dev("g1"), dev("g2")
        wrong = [(p + n, exp, tuple(t.shape)) for n, t, exp in (("a2", a2, (self.decay_width, a1.shape[0])),
                                                                ("g2", g2, (self.v_width, g1.shape[0]))) if tuple(t.shape) != exp]
        if wrong:
            raise WeightsError(wrong_shape=wrong)
        ra, rg = a1.shape[0], g1.shape[0]
        # both low-rank pairs as two products: [a1; g1] x, then a block-diagonal [a2 0; 0 g2]; the inner
        # width is padded with zeros to a multiple of 8 (what the tensor-core product takes)
        inner = (ra + rg + 7) // 8 * 8
        self.w_low = torch.zeros((inner, self.hidden_size), dtype=a1.dtype, device=a1.device)
        self.w_low[:ra], self.w_low[ra:ra + rg] = a1, g1
        self.w_high = torch.zeros((self.decay_width + self.v_width, inner), dtype=a1.dtype, device=a1.device)
        self.w_high[:self.decay_width, :ra] = a2
        self.w_high[self.decay_width:, ra:ra + rg] = g2

    def cache_spec(self):
        return [StateSpec((self.num_heads, self.value_dim, self.key_dim), "float32", "memory"),
                StateSpec((max(self.taps - 1, 1), self.channels), "float32", "conv")]

    def read_out(self, ctx, x):
        n = ctx.n_rows
        proj = linear.product_rows_f32(ctx, x, self.w_in, "cd_proj")
        if self.low_rank:
            low = ctx.buffer("cd_low", (n, self.w_low.shape[0]))
            linear.product_act(ctx, x, self.w_low, low, "cd_low_partial", gelu=False)
            high = linear.product_rows_f32(ctx, low, self.w_high, "cd_high")      # decay inputs, then gate inputs
        else:
            high = proj[:, self.channels + self.num_heads:]                        # the same two, behind q, k, v and beta
        conv_state = ctx.state("conv")
        qkv = ctx.buffer("cd_qkv", (n, self.channels), torch.float32)
        decays = ctx.buffer("cd_decay", (n, self.decay_width), torch.float32)
        ops.conv_unit(proj, self.conv_w, conv_state, ctx.row_seq, ctx.row_pos, ctx.seq_row0, ctx.seq_slot, qkv,
                      self.num_qk_heads, self.num_heads, self.key_dim, self.value_dim, self.key_dim ** -0.5,
                      update_state=ctx.decode, decay=(high[:, :self.decay_width], self.a_log, self.dt_bias, decays))
        if self.taps > 1 and not ctx.decode:
            ops.keep_last_rows(proj, 0, self.channels, conv_state, ctx.seq_row0, ctx.seq_new, ctx.seq_start, ctx.seq_slot,
                               ctx.n_seqs)
        raw = ctx.buffer("cd_raw", (n, self.v_width), torch.float32)
        ops.delta_scan(qkv, proj, self.channels, decays, self.a_log, self.dt_bias, ctx.state("memory"),
                       ctx.seq_row0, ctx.seq_new, ctx.seq_start, ctx.seq_slot, raw, ctx.n_seqs, self.num_heads,
                       self.num_qk_heads, self.key_dim, self.value_dim, decay_ready=True)
        out = ctx.buffer("cd_out", (n, self.v_width))
        ops.head_norm_gate(raw, False, self.norm_w, False, high, self.decay_width, out, self.num_heads, self.value_dim, self.eps,
                           gate_silu=self.gate == "silu")
        return out

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self.read_out(ctx, x), self.w_o, residual, "o_partial")

    def branch_output(self, ctx, x, name: str, proj=None):
        return linear.product_f32(ctx, self.read_out(ctx, x), self.w_o, name)


@register_part("mixer", "gated_delta")
class GatedDelta(ChannelDelta):
    """The gated delta rule with one decay per head, plain matrices for the decay's and the gate's inputs and a SiLU
    gate on the read-out (each still an option of its own)."""
    default_decay, default_gate, default_low_rank = "head", "silu", False


@register_part("mixer", "retention")
class Retention(Part):
    """Linear attention with a fixed decay per head and no softmax or denominator. q, k (``num_heads`` x ``key_dim``) and v
    (``num_heads`` x ``value_dim``) are plain projections; the first channels of every q and k head are turned by the
    position (``position``: a rotary part), k is then multiplied by key_dim^-1/2;

        S_t = decay[head] S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t

    o is divided by its root mean square per head (no weight), the heads side by side are multiplied by silu(Wg x) (a
    number per channel) and projected by Wo. S is float32 per sequence and head, zero at the start; rotation, scaling,
    the scan and the norm are float32. ``decay``: one number per head. Tensors ``q k v g o``."""
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.num_heads = int(params["num_heads"])
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        _check_dims(self.key_dim, self.value_dim)
        self.decay = tuple(float(d) for d in params["decay"])
        if len(self.decay) != self.num_heads:
            raise ConfigError("decay", f"one decay per head: {self.num_heads} heads, {len(self.decay)} decays")
        self.position = build_part("position", params.get("position") or PartSpec("none"))
        if self.position.rotary_dim > self.key_dim:
            raise ConfigError("rotary_dim", f"{self.position.rotary_dim} exceeds the head size {self.key_dim}")
        self.qk_width = self.num_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        self.cols = (0, self.qk_width, 2 * self.qk_width)            # q, k, v in the stacked product; the gate behind them
        self.gate_col = 2 * self.qk_width + self.v_width
        self.w_in = self.w_o = self.decay_w = None

    def tensor_specs(self):
        p, hid = self.prefix, self.hidden_size
        return {p + "q": TensorSpec((self.qk_width, hid)), p + "k": TensorSpec((self.qk_width, hid)),
                p + "v": TensorSpec((self.v_width, hid)), p + "g": TensorSpec((self.v_width, hid)),
                p + "o": TensorSpec((hid, self.v_width))}

    def load(self, tensors, device, dtype):
        p = self.prefix
        self.w_in = torch.cat([to_device(tensors[p + n], device, dtype) for n in ("q", "k", "v", "g")], 0).contiguous()
        self.w_o = to_device(tensors[p + "o"], device, dtype)
        self.decay_w = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)
        self.position.load(tensors, device, dtype)

    def cache_spec(self):
        return StateSpec((self.num_heads, self.value_dim, self.key_dim), "float32", "retention")

    def read_out(self, ctx, x):
        n, pos = ctx.n_rows, self.position
        proj = linear.product_rows_f32(ctx, x, self.w_in, "rt_proj")
        # q and k heads stand side by side: one pass turns both and scales the k heads
        ops.rotate_rows_(proj, 0, 2 * self.num_heads, self.key_dim, pos.rotary_dim, pos.pairing == "interleaved", pos.inv_freq,
                         pos.amplitude, ctx.row_pos, self.num_heads, self.key_dim ** -0.5)
        raw = ctx.buffer("rt_raw", (n, self.v_width), torch.float32)
        ops.retention_scan(proj, self.cols, self.decay_w, ctx.state("retention"), ctx.seq_row0, ctx.seq_new, ctx.seq_start,
                           ctx.seq_slot, raw, ctx.n_seqs, self.num_heads, self.key_dim, self.value_dim)
        out = ctx.buffer("rt_out", (n, self.v_width))
        ops.head_norm_gate(raw, False, None, False, proj, self.gate_col, out, self.num_heads, self.value_dim, self.eps, gate_silu=True)
        return out

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self.read_out(ctx, x), self.w_o, residual, "o_partial")

    def branch_output(self, ctx, x, name: str, proj=None):
        return linear.product_f32(ctx, self.read_out(ctx, x), self.w_o, name)
