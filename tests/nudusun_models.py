"""Small Nudusun configurations and random weights for the tests, made here by the tensor naming rule itself (not from
the library's tensor lists), stored in bfloat16 as a model folder."""
import json
import os

import torch


def attn(dim, vdim, heads, kv_heads, window, scale, diff, softcap=None):
    m = {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "diff": diff}
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    return m


def delta(dim, vdim, heads, kv_heads, conv):
    return {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "conv": conv}


def moe(experts, top, ff, limit, identity=0, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, alpha=1.8, scale=4.0, side=None, positions=512, eps=1e-5):
    c = {"architecture": "Nudusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
         "embedding": {"scale": scale}, "max_positions": positions, "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    return c


# every size differs from every other: a delta layer first, two value heads per q/k head, three taps; an attention with
# three query heads per kv head, a window of 9 and a cap; an attention without feed-forward whose window of 70 straddles
# pages of 64, values wider than both maps together; a delta layer with one tap and all three experts chosen
MIXED = config(64, 97, [
    layer("delta", delta(16, 24, 4, 2, 3), moe(5, 2, 24, 1.5, identity=1, groups=(3, 2), scale=1.7, shared=(40, 3.0))),
    layer("attention", attn(8, 12, 6, 2, 9, 0.4, 0.25, softcap=5.0), moe(4, 3, 16, 0.8, identity=2, groups=(3, 2), scale=2.2, shared=(8, 1.0))),
    layer("attention", attn(16, 40, 3, 3, 70, 0.3, 0.4)),
    layer("delta", delta(24, 8, 2, 1, 1), moe(3, 3, 32, 2.5)),
], alpha=1.5, side=8)
# a width that no tensor-core product takes, head sizes that are no multiples of 8, a token input of 6 channels, one kv head,
# one group kept of three
ODD = config(44, 61, [
    layer("attention", attn(12, 20, 3, 1, 33, 0.29, 0.1, softcap=30.0), moe(7, 2, 20, 1.2, identity=2, groups=(3, 1), scale=0.9, shared=(12, 2.0))),
    layer("delta", delta(20, 12, 3, 3, 5), moe(3, 1, 28, 4.0, identity=1)),
], alpha=1.0, scale=1.0, side=6, eps=1e-6)
# sizes of the tensor-core products; windows of 130 and 200 over pages of 64; four of fifteen experts in two of five groups
WIDE = config(128, 83, [
    layer("attention", attn(64, 64, 4, 2, 130, 0.125, 0.3, softcap=40.0), moe(13, 4, 64, 2.0, identity=2, groups=(5, 2), scale=2.0, shared=(64, 2.0))),
    layer("delta", delta(64, 64, 4, 2, 4), moe(8, 2, 32, 1.0, shared=(96, 7.0))),
    layer("attention", attn(32, 128, 2, 1, 200, 0.17, 0.6), moe(6, 2, 48, 3.0, identity=2, groups=(2, 1))),
], alpha=2.5, scale=8.0, side=16)
# no window (every earlier key is seen), no token input, no cap, no shared expert, alpha left to its default
OPEN = config(48, 50, [
    layer("attention", attn(16, 24, 2, 1, None, 0.25, 0.2), moe(4, 2, 16, 1.5, identity=2, groups=(3, 2))),
    layer("delta", delta(8, 16, 3, 3, 2)),
    layer("attention", attn(8, 8, 4, 2, 40, 0.3, 0.35), moe(2, 1, 24, 2.0)),
])
del OPEN["postln_alpha"]
# every row goes through all experts of its routed layers (identity ones included), so no choice can fall the other way
# under rounding: bfloat16 is held to the bound on every row here; sizes of the tensor-core kernels
ALL_EXPERTS = config(192, 73, [
    layer("delta", delta(32, 64, 6, 3, 4), moe(3, 4, 80, 2.0, identity=1, groups=(2, 2), scale=1.5, shared=(48, 2.0))),
    layer("attention", attn(64, 32, 6, 2, 100, 0.125, 0.3, softcap=20.0), moe(3, 3, 32, 1.0)),
    layer("delta", delta(128, 32, 2, 2, 2)),
], alpha=1.2, side=8)
# maps and values of 64 and 128 channels, unlike each other (the tensor-core prompt attention in its mixed sizes): maps of
# 64 under values of 128 with a cap and a window of 100, maps of 128 over values of 64 without a window; all experts chosen
PAIRED = config(128, 89, [
    layer("attention", attn(64, 128, 4, 2, 100, 0.11, 0.25, softcap=25.0), moe(2, 3, 48, 2.0, identity=1, shared=(32, 2.0))),
    layer("delta", delta(32, 64, 4, 2, 3)),
    layer("attention", attn(128, 64, 2, 1, None, 0.08, 0.45), moe(3, 3, 32, 1.5)),
], alpha=2.5, scale=8.0, side=8)
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "open": OPEN, "all_experts": ALL_EXPERTS, "paired": PAIRED}


def tensor_shapes(cfg):
    """name -> (shape, kind of values) by the naming rule."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, W), "embed"), "pos": ((cfg["max_positions"], W), "pos"), "final.norm": ((W,), "norm"), "head": ((V, W), "head")}
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        out["side.embed"] = ((V, len(cfg["layers"]) * side), "embed")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = ((W,), "norm")
        q = p + "mix."
        if L["type"] == "attention":
            out[q + "q"], out[q + "k"], out[q + "v"] = ((H * 2 * D, W), "linear"), ((G * 2 * D, W), "linear"), ((G * Dv, W), "linear")
            out[q + "q.norm"], out[q + "k.norm"] = ((D,), "norm"), ((D,), "norm")
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[q + n] = ((D,), "lambda")
            out[q + "o"] = ((W, H * Dv), "linear")
        else:
            T = m["conv"]
            out[q + "q"], out[q + "k"], out[q + "v"] = ((G * D, W), "linear"), ((G * D, W), "linear"), ((H * Dv, W), "linear")
            out[q + "q.conv"], out[q + "k.conv"], out[q + "v.conv"] = ((G * D, T), "conv"), ((G * D, T), "conv"), ((H * Dv, T), "conv")
            out[q + "b"], out[q + "a"], out[q + "g"] = ((H, W), "gate"), ((H, W), "gate"), ((H * Dv, W), "gate")
            out[q + "A_log"], out[q + "dt_bias"], out[q + "norm"] = ((H,), "rate"), ((H,), "bias"), ((Dv,), "norm")
            out[q + "o"] = ((W, H * Dv), "linear")
        f = L.get("mlp")
        if f is not None:
            out[p + "norm2"] = ((W,), "norm")
            q = p + "mlp."
            names = [f"e{e}" for e in range(f["router"]["experts"])] + (["shared"] if f.get("shared") else [])
            for n in names:
                ff = f["shared"]["ff"] if n == "shared" else f["expert"]["ff"]
                out[f"{q}{n}.gate"], out[f"{q}{n}.up"], out[f"{q}{n}.down"] = ((ff, W), "expert"), ((ff, W), "expert"), ((W, ff), "linear")
            routed = f["router"]["experts"] + f["router"].get("identity", 0)
            out[q + "router"], out[q + "correction"] = ((routed, W), "router"), ((routed,), "correction")
        if side:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = ((side, W), "gate"), ((W, side), "linear"), ((W,), "norm")
    return out


def random_weights(cfg, seed):
    """name -> bfloat16 tensor, of the order a trained model has, so that every mechanism moves the logits: experts that
    reach their clamps, routers with clear choices, corrections that change some of them, decays well below one."""
    gen = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=gen)
        t = {"linear": lambda: r * (1.0 / shape[-1] ** 0.5), "expert": lambda: r * (2.5 / shape[-1] ** 0.5),
             "gate": lambda: r * (2.0 / shape[-1] ** 0.5), "router": lambda: r * (5.0 / shape[-1] ** 0.5),
             "embed": lambda: r * 0.8, "pos": lambda: r * 0.5, "head": lambda: r * (4.0 / W ** 0.5), "norm": lambda: 1.0 + 0.3 * r,
             "bias": lambda: 0.3 * r, "rate": lambda: -1.0 + 0.5 * r, "conv": lambda: 0.25 + 0.3 * r, "lambda": lambda: 0.3 * r,
             "correction": lambda: 0.05 * r}[kind]()
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, weights=None):
    from camelid_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    weights = weights if weights is not None else random_weights(cfg, seed)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return weights


def as_float64(weights):
    return {n: t.to(torch.float64).numpy() for n, t in weights.items()}
