"""The Kizezen decoder's config.json as a typed configuration, and its plan.

Kizezen is a pre-norm decoder, x += mixer(norm1(x)) and x += ff(norm2(x)) with RMS norms, whose layers take one of
three mixers in the order ``layers`` gives:

* ``attention``: grouped queries with biases on q, k and v, an RMS norm of q and of k over their whole projections, a
  rotation of the first ``rot.dims`` channels of every head (pairs of the two halves; frequencies stretched band by
  band), a window of ``mask.size`` keys beside which the first ``mask.keep_first`` keys of the sequence stay visible,
  one more term exp(sink[head]) in the softmax denominator and a sigmoid gate per head computed from the mixer's input;
* ``latent_attention``: all heads' keys and values are maps of one normed latent row of ``kv_rank`` channels per position
  plus one turned key part of ``rot_dim`` channels shared by the heads (pairs of neighbouring channels; frequencies
  blended along a ramp, sines and cosines scaled); every earlier key is seen; sink and gate as above;
* ``retention``: S <- decay[head] S + k v^T, o = S^T q, with q and k turned (pairs of halves) and k / sqrt(dim); o normed
  per head without weight, times silu of a gate per channel.

The feed-forward is dense with the exact GELU, or absent. Rows start as embed[token] * ``embedding.scale``; the logits
are head(final norm(x)) * ``logit_scale``.

Keys read (all sizes and constants come from here): ``architecture``, ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``logit_scale``, ``layers[i].type``, ``layers[i].mlp`` null or ``{kind: "dense", ff}``, and of
``layers[i].mixer``: attention ``{dim, vdim, heads, kv_heads, scale, mask.{size, keep_first}, rot}``; latent_attention
``{dim, rot_dim, vdim, heads, kv_rank, scale, rot}``; retention ``{dim, vdim, heads, decay[heads], rot}``.
``rot`` = ``{dims, base, scaling}``; ``scaling`` may be missing (plain frequencies), ``{factor, low, high, original}`` (bands)
or ``{factor, fast, slow, original}`` (ramp). Missing: ``mask`` (all earlier keys), ``mask.keep_first`` (0), ``rot`` (no
rotation; not for latent attention), ``vdim`` (``dim``), ``kv_heads`` (``heads``), ``embedding.scale`` and
``logit_scale`` (1).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import ConfigError
from .fomatar import NO_POSITION_LIMIT, _get, _positive
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("attention", "latent_attention", "retention")


def _rot(m: dict, where: str, limit: int, required: bool = False):
    """The ``rot`` entry of a mixer as the parameters of a rotary position part (None: no rotation)."""
    rot = _get(m, "rot", where, None, ... if required else None)
    if rot is None:
        return None
    w = where + ".rot"
    dims, base = _get(rot, "dims", w, int), _get(rot, "base", w, float)
    if dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(w + ".dims", f"must be even and at most {limit}, got {dims}")
    if base <= 0:
        raise ConfigError(w + ".base", f"must be greater than zero, got {base}")
    if dims == 0:
        return None
    sc = _get(rot, "scaling", w, None, None)
    scaling = None
    if sc is not None:
        ws = w + ".scaling"
        factor, original = _get(sc, "factor", ws, float), _get(sc, "original", ws, float)
        if factor <= 0 or original <= 0:
            raise ConfigError(ws, "factor and original must be greater than zero")
        if "fast" in sc or "slow" in sc:
            fast, slow = _get(sc, "fast", ws, float), _get(sc, "slow", ws, float)
            if fast <= 0 or slow <= 0 or base == 1.0:
                raise ConfigError(ws, "fast and slow must be greater than zero (and the base not 1)")
            scaling = {"rope_type": "ramp", "factor": factor, "original": original, "fast": fast, "slow": slow}
        else:
            low, high = _get(sc, "low", ws, float), _get(sc, "high", ws, float)
            if high == low:
                raise ConfigError(ws + ".high", "must differ from low")
            scaling = {"rope_type": "llama3", "factor": factor, "low_freq_factor": low, "high_freq_factor": high,
                       "original_max_position_embeddings": original}
    return {"rotary_dim": dims, "theta": base, "scaling": scaling}


def _mixer(kind: str, m: dict, w: str) -> dict:
    out = {"heads": _positive(m, "heads", w), "dim": _positive(m, "dim", w)}
    out["vdim"] = _positive(m, "vdim", w, out["dim"])
    if kind == "attention":
        out["kv_heads"] = _positive(m, "kv_heads", w, out["heads"])
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(w + ".kv_heads", f"{out['kv_heads']} does not divide {out['heads']} heads")
        out["scale"] = _get(m, "scale", w, float)
        mask = _get(m, "mask", w, None, None)
        out["window"] = _positive(mask, "size", w + ".mask") if mask is not None else None
        out["keep_first"] = _get(mask, "keep_first", w + ".mask", int, 0) if mask is not None else 0
        if out["keep_first"] < 0:
            raise ConfigError(w + ".mask.keep_first", f"must not be negative, got {out['keep_first']}")
        out["rot"] = _rot(m, w, out["dim"])
    elif kind == "latent_attention":
        out["rot_dim"] = _positive(m, "rot_dim", w)
        out["kv_rank"] = _positive(m, "kv_rank", w)
        out["scale"] = _get(m, "scale", w, float)
        out["rot"] = _rot(m, w, out["rot_dim"], required=True)
        if out["rot"] is None or out["rot"]["rotary_dim"] != out["rot_dim"]:
            raise ConfigError(w + ".rot.dims", f"must equal rot_dim ({out['rot_dim']})")
    else:
        decay = _get(m, "decay", w)
        if not isinstance(decay, list) or len(decay) != out["heads"] or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(w + ".decay", f"must be a list of {out['heads']} numbers (one per head)")
        out["decay"] = tuple(float(d) for d in decay)
        out["rot"] = _rot(m, w, out["dim"])
    return out


@dataclass(frozen=True)
class KizezenConfig:
    raw: dict
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple                   # dicts: type, mixer (validated), mlp

    @classmethod
    def from_dict(cls, d: dict) -> "KizezenConfig":
        vocab = _positive(d, "vocab", "")
        width = _positive(d, "width", "")
        eps = _get(_get(d, "norm", ""), "eps", "norm", float)
        emb_scale = _get(_get(d, "embedding", "", None, None) or {}, "scale", "embedding", float, 1.0)
        logit_scale = _get(d, "logit_scale", "", float, 1.0)
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers", "must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"layers[{i}]"
            kind = _get(L, "type", w)
            if kind not in MIXERS:
                raise ConfigError(w + ".type", f"unknown layer type {kind!r}; known: {', '.join(MIXERS)}")
            mixer = _mixer(kind, _get(L, "mixer", w), w + ".mixer")
            mlp = L.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", w + ".mlp")
                if mk != "dense":
                    raise ConfigError(w + ".mlp.kind", f"unknown feed-forward {mk!r}; known: dense")
                mlp = {"kind": mk, "ff": _positive(mlp, "ff", w + ".mlp")}
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        return cls(copy.deepcopy(d), vocab, width, eps, emb_scale, logit_scale, tuple(layers))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    @property
    def stop_token_ids(self) -> tuple:
        return ()


def _position(rot, pairing: str):
    return PartSpec("rope", {**rot, "pairing": pairing}) if rot is not None else None


def kizezen_plan(cfg: KizezenConfig) -> ModelPlan:
    """Parts per layer (tensor names ``l<i>.…``); every layer runs once, in order."""
    norm = {"hidden_size": cfg.width, "eps": cfg.eps}
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m, f = f"l{i}.", L["mixer"], L["mlp"]
        common = {"hidden_size": cfg.width, "eps": cfg.eps, "num_heads": m["heads"]}
        if L["type"] == "attention":
            mixer = PartSpec("window_attention", {
                **common, "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"], "window": m["window"],
                "keep_first": m["keep_first"] if m["window"] else 0, "scale": m["scale"], "qk_norm": "full", "bias": True,
                "sink": True, "output_gate": "head", "position": _position(m["rot"], "split")}, p + "mix.")
        elif L["type"] == "latent_attention":
            mixer = PartSpec("latent_attention", {
                **common, "head_dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"], "rank": m["kv_rank"],
                "scale": m["scale"], "sink": True, "output_gate": "head", "position": _position(m["rot"], "interleaved")}, p + "mix.")
        else:
            mixer = PartSpec("retention", {**common, "key_dim": m["dim"], "value_dim": m["vdim"], "decay": m["decay"],
                                           "position": _position(m["rot"], "split")}, p + "mix.")
        ffn = PartSpec("dense", {"hidden_size": cfg.width, "intermediate_size": f["ff"], "activation": "gelu_erf",
                                 "bias": False}, p + "mlp.") if f is not None else None
        layers.append(LayerSpec(
            arrangement="prenorm",
            norm1=PartSpec("rmsnorm", {**norm, "tensor": p + "norm1"}),
            mixer=mixer,
            norm2=PartSpec("rmsnorm", {**norm, "tensor": p + "norm2"}) if ffn is not None else None,
            ffn=ffn,
        ))
    return ModelPlan(
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "embed",
                                         "scale": cfg.embedding_scale}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {**norm, "tensor": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "tensor": "head",
                                  "scale": cfg.logit_scale}),
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_position=NO_POSITION_LIMIT,
        stop_token_ids=(),
    )
