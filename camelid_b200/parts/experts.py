"""A routed feed-forward (mixture of experts): every row goes through the ``top`` of ``experts`` small
gated feed-forwards that a linear router picks for it, and, where the layer has one, through a shared
expert that every row uses.

    z = x Wr^T (float32)            s = sigmoid(z)   or   softmax(z) over the experts   (``scoring``)
    chosen: the ``top`` experts with the largest s;  weights w = s of the chosen (``renormalize``: / their sum)
    expert_e(u) = Wd_e (silu(Wg_e u) * (Wu_e u))
    y = sum over the chosen of expert_e(w x)          (``weight_on`` "input")
      = sum over the chosen of w expert_e(x)          (``weight_on`` "output")
    y += shared(x)

Options that designs combine: ``identity`` n: the router has n more outputs behind the experts', *identity experts* whose
output is the row itself (times the weight) and that have no tensors; ``correction``: a tensor ``correction`` [experts +
identity] is added to the scores for the choice alone (the weights use the scores without it); ``groups`` (count, keep):
the experts (identity ones included) form ``count`` equal groups of neighbours, a group's score is its largest choice
score, and only experts of the ``keep`` best groups can be chosen; ``route_scale`` multiplies the weights; ``gate_act``
and ``shared_gate_act`` (alpha, limit, shift): the experts' gated activation min(g, limit) sigmoid(alpha min(g, limit))
(clamp(u, +-limit) + shift) instead of silu(g) u.

Tensors under the prefix: ``router`` [experts, hidden]; per expert ``e<i>.gate``, ``e<i>.up`` [ff, hidden] and
``e<i>.down`` [hidden, ff]; the shared expert's under ``shared.`` with the same three names. The experts'
matrices are stacked into three tensors at load time. Router logits, scores and weights are float32; the
row order of the grouped products is made on the device (``csrc/experts.cu``), so the part runs inside
captured graphs.
"""
from __future__ import annotations

import torch

from ..config.plan import PartSpec
from ..csrc import ops
from ..errors import ConfigError
from . import linear
from .base import Part, TensorSpec, build_part, register_part, to_device


@register_part("ffn", "routed_experts")
class RoutedExperts(Part):
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True
    takes_stream = True             # ``output`` takes the float32 stream (``stream=``) for the identity experts' rows

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.identity = int(params.get("identity") or 0)
        self.routed = self.experts + self.identity          # outputs of the router
        self.correction = bool(params.get("correction", False))
        self.groups, self.keep_groups = (int(v) for v in (params.get("groups") or (1, 1)))
        self.route_scale = float(params["route_scale"]) if params.get("route_scale") is not None else 1.0
        self.act = ops.GateAct(*params["gate_act"]) if params.get("gate_act") else None
        self.top = int(params["top"])
        self.ff = int(params["expert_size"])
        self.scoring = params.get("scoring") or "sigmoid"
        self.renormalize = bool(params.get("renormalize", False))
        self.weight_on = params.get("weight_on") or "output"
        if not 1 <= self.top <= self.routed:
            raise ConfigError("top", f"each row picks 1..{self.routed} experts, got {self.top}")
        if self.routed > 1024:
            raise ConfigError("experts", f"the routing kernel takes up to 1,024 experts, got {self.routed}")
        if self.identity < 0:
            raise ConfigError("identity", f"must not be negative, got {self.identity}")
        if self.groups < 1 or self.routed % self.groups or not 1 <= self.keep_groups <= self.groups:
            raise ConfigError("groups", f"{self.groups} groups (of which {self.keep_groups} stay open) do not divide "
                              f"{self.routed} experts into equal groups")
        if self.top > self.keep_groups * (self.routed // self.groups):
            raise ConfigError("top", f"{self.top} choices do not fit into {self.keep_groups} groups of {self.routed // self.groups}")
        if self.scoring not in ("sigmoid", "softmax"):
            raise ConfigError("scoring", f"unknown scoring {self.scoring!r}; known: sigmoid, softmax")
        if self.weight_on not in ("input", "output"):
            raise ConfigError("weight_on", f"the weight multiplies the expert's 'input' or 'output', got {self.weight_on!r}")
        self.shared = None
        if params.get("shared_size"):
            self.shared = build_part("ffn", PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                                                "intermediate_size": int(params["shared_size"]),
                                                                "names": ("gate", "up", "down"),
                                                                "gate_act": params.get("shared_gate_act")}, prefix + "shared."))
        self.w_router = self.w_gate = self.w_up = self.w_down = self.w_correction = None

    def tensor_specs(self):
        p, hid = self.prefix, self.hidden_size
        specs = {p + "router": TensorSpec((self.routed, hid))}
        if self.correction:
            specs[p + "correction"] = TensorSpec((self.routed,), "choice_bias")
        for e in range(self.experts):
            specs[f"{p}e{e}.gate"] = TensorSpec((self.ff, hid))
            specs[f"{p}e{e}.up"] = TensorSpec((self.ff, hid))
            specs[f"{p}e{e}.down"] = TensorSpec((hid, self.ff))
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
        return specs

    def load(self, tensors, device, dtype):
        p = self.prefix
        self.w_router = to_device(tensors[p + "router"], device, dtype)
        if self.correction:
            self.w_correction = tensors[p + "correction"].to(device=device, dtype=torch.float32).contiguous()
        stack = lambda n: torch.stack([to_device(tensors[f"{p}e{e}.{n}"], device, dtype)       # noqa: E731
                                       for e in range(self.experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        # bfloat16 with sizes the tensor-core kernel takes: gate and up packed per expert as the dense SwiGLU has them
        self.w_gate_up = None
        if dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.ff % 16 == 0 and str(device) != "cpu":
            self.w_gate_up = torch.stack([linear.pack_gate_up(self.w_gate[e], self.w_up[e], 16) for e in range(self.experts)]).contiguous()
            self.w_gate = self.w_up = None
        if self.shared is not None:
            self.shared.load(tensors, device, dtype)

    def output(self, ctx, x, name: str, stream=None):
        """(y, None): float32 [rows, hidden] in the step's buffer ``name``. ``stream``: the rows of ``x`` in float32
        where the caller has them (what an identity expert hands back); else ``x`` itself."""
        rows, top, E = x.shape[0], self.top, self.routed
        pairs = rows * top
        i32 = lambda n, k: ctx.buffer(f"{name}_{n}", (k,), torch.int32)        # noqa: E731
        logits = linear.product_f32(ctx, x, self.w_router, name + "_router")          # split sums where the step has few rows
        ids, wts = i32("ids", pairs), ctx.buffer(name + "_wts", (pairs,), torch.float32)
        ops.route_topk(logits, top, self.scoring == "softmax", self.renormalize, ids, wts, self.w_correction, self.groups,
                       self.keep_groups, self.route_scale)
        rank, counts, offsets, tile_first = i32("rank", pairs), i32("counts", E), i32("offsets", E + 1), i32("tiles", E + 1)
        tc = self.w_gate_up is not None
        ops.expert_plan(ids, E, rank, counts, offsets, tile_first, ops.EXPERT_TILE_ROWS_TC if tc else ops.EXPERT_TILE_ROWS)
        xs, place = ctx.buffer(name + "_xs", (pairs, self.hidden_size)), i32("place", pairs)
        ops.expert_gather(x, ids, wts, rank, offsets, top, self.weight_on == "input", xs, place, self.experts)
        act = ctx.buffer(name + "_eact", (pairs, self.ff))
        ys = ctx.buffer(name + "_ys", (pairs, self.hidden_size), torch.float32)
        if tc:          # the grouped products on the tensor cores; float32 and odd sizes on the CUDA cores
            err = linear._err_word(x.device)
            ops.gemm_tc_grouped(xs, self.w_gate_up, act, ops.TC_SWIGLU, offsets, tile_first, err, self.act)
            ops.gemm_tc_grouped(act, self.w_down, ys, ops.TC_STORE_F32, offsets, tile_first, err)
        else:
            ops.expert_gemm(xs, self.w_gate, self.w_up, act, offsets, tile_first, self.act)
            ops.expert_gemm(act, self.w_down, None, ys, offsets, tile_first)
        shared = self.shared.output(ctx, x, name + "_shared")[0] if self.shared is not None else None
        out = ctx.buffer(name, (rows, self.hidden_size), torch.float32)
        same = (ids, self.experts, stream if stream is not None else x) if self.identity else None
        ops.expert_combine(ys, place, wts, top, self.weight_on == "output", shared, out, same)
        return out, None

    def forward(self, ctx, x, residual):
        y, _ = self.output(ctx, x, "experts_out")
        ctx.settle(residual)
        ops.add_partials(residual, y.unsqueeze(0))
