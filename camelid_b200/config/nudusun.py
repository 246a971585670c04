"""The Nudusun decoder's config.json as a typed configuration, and its plan.

Nudusun norms *after* each residual sum: x <- N1(a x + mixer(x)), x <- N2(a x + ff(x)), a one number of the model, the
sublayers reading x as it is. The stream starts as c * E[token] + P[position] (a multiplier and a table of learned
position rows). A layer's mixer is ``delta`` (a gated delta rule with one decay and one write strength per head, short
causal convolutions with SiLU on q, k, v, unit q and k, a SiLU gate on the per-head normed read-out) or ``attention``
(differential attention: two score maps per head over the same values, RMS-normed q and k per map, a tanh cap on the
scores, a sliding window, no rotation; the second map is subtracted with a learned factor and the difference normed per
head). The feed-forward is a routed one: a softmax router over the experts and a few identity experts, the choice made on
scores plus a correction within the best groups of neighbouring experts, weights scaled and not renormalised, experts
with a clamped gated activation, and a shared expert. At its end a layer takes a per-layer token input from its own
columns of a second embedding table.

Keys read (all sizes and constants come from here): ``architecture``, ``vocab``, ``width``, ``max_positions``,
``norm.eps``, ``postln_alpha``, ``embedding.scale``, ``token_side.dim``, ``layers[i].type`` ("attention" | "delta"),
``layers[i].mixer.{dim, vdim, heads, kv_heads}`` and, for attention, ``{scale, softcap, diff, mask.size}``, for delta
``conv``; ``layers[i].mlp`` null or ``{kind: "moe", expert.{ff, limit}, router.{experts, top, identity, scale,
groups.{count, keep}}, shared.{ff, limit}}``. Missing ``mask``: all earlier keys; missing ``softcap``: none; missing
``token_side``: no token input; missing ``shared``, ``identity``, ``groups``, ``limit``: none of it.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError
from .fomatar import _get, _positive
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

GATE_ALPHA = 1.702          # the experts' activation is g * sigmoid(1.702 g) * (u + 1) on clamped g and u
GATE_SHIFT = 1.0


def _heads(m, where):
    out = {"dim": _positive(m, "dim", where), "heads": _positive(m, "heads", where), "kv_heads": _positive(m, "kv_heads", where)}
    out["vdim"] = _positive(m, "vdim", where, out["dim"])
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(where + ".kv_heads", f"{out['kv_heads']} does not divide {out['heads']} heads")
    return out


def _limit(d, where):
    v = _get(d, "limit", where, float, None)
    if v is not None and v <= 0:
        raise ConfigError(where + ".limit", f"must be greater than zero, got {v}")
    return v


@dataclass(frozen=True)
class NudusunConfig:
    raw: dict
    vocab: int
    width: int
    eps: float
    alpha: float
    embed_scale: float
    max_positions: int
    side_dim: Optional[int]
    layers: tuple                   # dicts: type, mixer, mlp (validated)

    @classmethod
    def from_dict(cls, d: dict) -> "NudusunConfig":
        vocab = _positive(d, "vocab", "")
        width = _positive(d, "width", "")
        eps = _get(_get(d, "norm", ""), "eps", "norm", float)
        alpha = _get(d, "postln_alpha", "", float, 1.0)
        scale = _get(_get(d, "embedding", "", None, {}), "scale", "embedding", float, 1.0)
        max_positions = _positive(d, "max_positions", "")
        side = _get(d, "token_side", "", None, None)
        side_dim = _positive(side, "dim", "token_side") if side is not None else None
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers", "must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"layers[{i}]"
            kind = _get(L, "type", w)
            m, wm = _get(L, "mixer", w), w + ".mixer"
            if kind == "attention":
                mixer = _heads(m, wm)
                mixer["scale"] = _get(m, "scale", wm, float)
                mixer["diff"] = _get(m, "diff", wm, float)
                mixer["softcap"] = _get(m, "softcap", wm, float, None)
                if mixer["softcap"] is not None and mixer["softcap"] <= 0:
                    raise ConfigError(wm + ".softcap", f"must be greater than zero, got {mixer['softcap']}")
                mask = _get(m, "mask", wm, None, None)
                mixer["window"] = _positive(mask, "size", wm + ".mask") if mask is not None else None
            elif kind == "delta":
                mixer = _heads(m, wm)
                mixer["conv"] = _positive(m, "conv", wm)
            else:
                raise ConfigError(w + ".type", f"unknown layer type {kind!r}; known: attention, delta")
            mlp = L.get("mlp")
            if mlp is not None:
                wf = w + ".mlp"
                mk = _get(mlp, "kind", wf)
                if mk != "moe":
                    raise ConfigError(wf + ".kind", f"unknown feed-forward {mk!r}; known: moe")
                router, expert = _get(mlp, "router", wf), _get(mlp, "expert", wf)
                shared = _get(mlp, "shared", wf, None, None)
                groups = _get(router, "groups", wf + ".router", None, None)
                mlp = {"kind": mk, "ff": _positive(expert, "ff", wf + ".expert"), "limit": _limit(expert, wf + ".expert"),
                       "experts": _positive(router, "experts", wf + ".router"), "top": _positive(router, "top", wf + ".router"),
                       "identity": _get(router, "identity", wf + ".router", int, 0),
                       "scale": _get(router, "scale", wf + ".router", float, 1.0),
                       "groups": (_positive(groups, "count", wf + ".router.groups"), _positive(groups, "keep", wf + ".router.groups"))
                       if groups is not None else None,
                       "shared_ff": _positive(shared, "ff", wf + ".shared") if shared is not None else None,
                       "shared_limit": _limit(shared, wf + ".shared") if shared is not None else None}
                total = mlp["experts"] + mlp["identity"]
                if mlp["identity"] < 0:
                    raise ConfigError(wf + ".router.identity", f"must not be negative, got {mlp['identity']}")
                if mlp["top"] > total:
                    raise ConfigError(wf + ".router.top", f"{mlp['top']} choices among {total} experts")
                if mlp["groups"] is not None:
                    count, keep = mlp["groups"]
                    if total % count or keep > count:
                        raise ConfigError(wf + ".router.groups", f"{count} groups (keeping {keep}) do not divide {total} experts")
                    if mlp["top"] > keep * (total // count):
                        raise ConfigError(wf + ".router.top", f"{mlp['top']} choices do not fit into {keep} groups of {total // count}")
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        return cls(copy.deepcopy(d), vocab, width, eps, alpha, scale, max_positions, side_dim, tuple(layers))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    @property
    def stop_token_ids(self) -> tuple:
        return ()


def _gate_act(limit):
    return (GATE_ALPHA, limit if limit is not None else float("inf"), GATE_SHIFT)


def nudusun_plan(cfg: NudusunConfig) -> ModelPlan:
    """Parts per layer (tensor names ``l<i>.…``); every layer runs once, in order."""
    norm = {"hidden_size": cfg.width, "eps": cfg.eps}
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m, f = f"l{i}.", L["mixer"], L["mlp"]
        if L["type"] == "attention":
            mixer = PartSpec("window_attention", {
                "hidden_size": cfg.width, "eps": cfg.eps, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                "head_dim": m["dim"], "value_dim": m["vdim"], "window": m["window"], "scale": m["scale"], "qk_norm": "head",
                "softcap": m["softcap"], "difference": m["diff"]}, p + "mix.")
        else:
            mixer = PartSpec("gated_delta", {
                "hidden_size": cfg.width, "eps": cfg.eps, "num_heads": m["heads"], "num_qk_heads": m["kv_heads"],
                "key_dim": m["dim"], "value_dim": m["vdim"], "conv_taps": m["conv"], "decay": "head", "gate": "silu",
                "low_rank": False}, p + "mix.")
        ffn = None
        if f is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": cfg.width, "experts": f["experts"], "top": f["top"], "expert_size": f["ff"],
                "shared_size": f["shared_ff"], "scoring": "softmax", "renormalize": False, "weight_on": "output",
                "identity": f["identity"], "correction": True, "groups": f["groups"], "route_scale": f["scale"],
                "gate_act": _gate_act(f["limit"]), "shared_gate_act": _gate_act(f["shared_limit"])}, p + "mlp.")
        after = None
        if cfg.side_dim is not None:
            after = PartSpec("token_side", {"hidden_size": cfg.width, "vocab_size": cfg.vocab, "dim": cfg.side_dim, "layer": i,
                                            "layers": len(cfg.layers), "eps": cfg.eps, "table": "side.embed"}, p + "side.")
        layers.append(LayerSpec(
            arrangement="postnorm",
            norm1=PartSpec("rmsnorm", {**norm, "tensor": p + "norm1"}),
            mixer=mixer,
            norm2=PartSpec("rmsnorm", {**norm, "tensor": p + "norm2"}) if ffn is not None else None,
            ffn=ffn,
            residual_scale=cfg.alpha,
            after=after,
        ))
    return ModelPlan(
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "embed",
                                         "scale": cfg.embed_scale, "position_tensor": "pos", "positions": cfg.max_positions}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {**norm, "tensor": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "tensor": "head"}),
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_position=cfg.max_positions,
        stop_token_ids=(),
    )
