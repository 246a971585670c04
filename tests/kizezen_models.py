"""Small Kizezen configurations and random weights for the tests, made here by the tensor naming rule itself (not from
the library's tensor lists), stored in bfloat16 as a model folder."""
import json
import os

import torch


def rot(dims, base, **scaling):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling
    return r


def attn(dim, vdim, heads, kv_heads, window, kept, r, scale):
    m = {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "scale": scale}
    if window:
        m["mask"] = {"size": window, "keep_first": kept}
    if r is not None:
        m["rot"] = r
    return {"type": "attention", "mixer": m}


def latent(dim, rot_dim, vdim, heads, rank, r, scale):
    return {"type": "latent_attention", "mixer": {"dim": dim, "rot_dim": rot_dim, "vdim": vdim, "heads": heads, "kv_rank": rank,
                                                   "rot": r, "scale": scale}}


def retention(dim, vdim, decay, r):
    m = {"dim": dim, "vdim": vdim, "heads": len(decay), "decay": list(decay)}
    if r is not None:
        m["rot"] = r
    return {"type": "retention", "mixer": m}


def layer(mixer, ff=None):
    return {**mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(width, vocab, layers, emb=1.0, logit=1.0, eps=1e-5):
    return {"architecture": "Kizezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb},
            "logit_scale": logit, "layers": layers}


# every size differs from every other: three query heads to a kv head, values wider than keys, a window of 9 with 3
# kept keys, part of each head turned, bands over an original length of 32; a latent narrower than a head's keys and
# values together; a layer without feed-forward; an attention that sees everything and turns nothing
MIXED = config(64, 97, [
    layer(retention(24, 40, (0.9, 0.99, 0.999), rot(16, 100.0)), 104),
    layer(attn(24, 40, 6, 2, 9, 3, rot(8, 100.0, factor=4.0, low=1.0, high=4.0, original=32), 0.3), 72),
    layer(latent(16, 8, 12, 3, 40, rot(8, 50.0, factor=4.0, fast=8.0, slow=1.0, original=16), 0.25)),
    layer(attn(8, 12, 4, 4, None, 0, None, 0.35), 48),
    layer(retention(16, 8, (0.5, 1.0), None), 56),
], emb=3.0, logit=0.7)
# a width that no tensor-core product takes, head sizes that are no multiples of 8, one kv head; 65 kept keys (more than
# a page) beside a window of 70 over pages of 64; more kept keys than the window is long; one head
ODD = config(44, 61, [
    layer(attn(12, 20, 3, 1, 70, 65, rot(6, 500.0), 0.29), 36),
    layer(latent(10, 6, 7, 2, 18, rot(6, 1000.0, factor=2.0, fast=4.0, slow=0.5, original=8), 0.3), 20),
    layer(retention(20, 4, (0.97,), rot(20, 37.0, factor=8.0, low=1.0, high=2.0, original=64))),
    layer(attn(20, 4, 2, 2, 5, 12, rot(20, 10000.0), 0.22), 52),
], emb=1.0, logit=1.0, eps=1e-6)
# sizes of the tensor-core kernels: heads of 64 and of 128 channels for keys and values, windows of 130 and 200 with 70
# and 10 kept keys over pages of 64; a latent of 96 channels; a retention with keys of 128 channels
WIDE = config(128, 83, [
    layer(attn(64, 64, 4, 2, 130, 70, rot(32, 10000.0, factor=8.0, low=1.0, high=4.0, original=128), 0.125), 256),
    layer(latent(64, 32, 64, 4, 96, rot(32, 10000.0, factor=8.0, fast=32.0, slow=1.0, original=64), 0.1), 136),
    layer(attn(128, 128, 2, 1, 200, 10, rot(64, 1000.0), 0.09), 256),
    layer(retention(128, 64, (0.98, 0.999), rot(128, 10000.0)), 192),
    layer(attn(128, 64, 2, 2, 64, 0, rot(128, 1000.0), 0.09)),
], emb=2.0, logit=0.4)
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE}


def tensor_shapes(cfg):
    """name -> (shape, kind of values) by the naming rule."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, W), "embed"), "final.norm": ((W,), "norm"), "head": ((V, W), "head")}
    for i, L in enumerate(cfg["layers"]):
        p, q, m = f"l{i}.", f"l{i}.mix.", L["mixer"]
        H, D = m["heads"], m["dim"]
        Dv = m.get("vdim", D)
        out[p + "norm1"] = ((W,), "norm")
        if L["type"] == "attention":
            G = m.get("kv_heads", H)
            out[q + "q"], out[q + "k"], out[q + "v"] = ((H * D, W), "linear"), ((G * D, W), "linear"), ((G * Dv, W), "linear")
            out[q + "q.b"], out[q + "k.b"], out[q + "v.b"] = ((H * D,), "bias"), ((G * D,), "bias"), ((G * Dv,), "bias")
            out[q + "q.norm"], out[q + "k.norm"] = ((H * D,), "norm"), ((G * D,), "norm")
            out[q + "sink"], out[q + "g"], out[q + "o"] = ((H,), "sink"), ((H, W), "gate"), ((W, H * Dv), "linear")
        elif L["type"] == "latent_attention":
            R, C = m["rot_dim"], m["kv_rank"]
            out[q + "q"], out[q + "dkv"], out[q + "dkv.norm"] = ((H * (D + R), W), "linear"), ((C + R, W), "linear"), ((C,), "norm")
            out[q + "uk"], out[q + "uv"] = ((H * D, C), "linear"), ((H * Dv, C), "linear")
            out[q + "sink"], out[q + "g"], out[q + "o"] = ((H,), "sink"), ((H, W), "gate"), ((W, H * Dv), "linear")
        else:
            out[q + "q"], out[q + "k"], out[q + "v"] = ((H * D, W), "linear"), ((H * D, W), "linear"), ((H * Dv, W), "linear")
            out[q + "g"], out[q + "o"] = ((H * Dv, W), "gate"), ((W, H * Dv), "linear")
        if L.get("mlp"):
            out[p + "norm2"] = ((W,), "norm")
            out[p + "mlp.up"], out[p + "mlp.down"] = ((L["mlp"]["ff"], W), "linear"), ((W, L["mlp"]["ff"]), "linear")
    return out


def random_weights(cfg, seed):
    """name -> bfloat16 tensor, of the order a trained model has, so that every mechanism moves the logits: sinks that
    take a visible share of the softmax, gates away from one half, biases."""
    gen = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=gen)
        t = {"linear": lambda: r * (1.0 / shape[-1] ** 0.5), "gate": lambda: r * (2.0 / shape[-1] ** 0.5),
             "embed": lambda: r * 0.8, "head": lambda: r * (4.0 / W ** 0.5), "norm": lambda: 1.0 + 0.3 * r,
             "sink": lambda: 0.5 + r, "bias": lambda: 0.3 * r}[kind]()
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
    return {k: v.to(torch.float64).numpy() for k, v in weights.items()}


def random_config(seed, tensor_cores=False):
    """A configuration drawn from a seed: sizes, head counts, order and number of layers, windows, kept keys, turned
    channels, scaling laws and their numbers all vary; small enough for the plain implementation. ``tensor_cores``:
    head and latent sizes that the bfloat16 prompt kernels on the tensor cores take."""
    import random
    rng = random.Random(seed if not tensor_cores else 1000 + seed)
    even = lambda lo, hi: 2 * rng.randint(lo // 2, hi // 2)      # noqa: E731

    def a_rot(limit, law):
        dims = even(2, limit)
        kind = rng.choice(["none", law, law])
        base = rng.choice([37.0, 1000.0, 250000.0])
        if kind == "none":
            return rot(dims, base)
        if kind == "bands":
            low = rng.choice([0.5, 1.0])
            return rot(dims, base, factor=rng.choice([2.0, 8.0]), low=low, high=low * rng.choice([2.0, 4.0]), original=rng.choice([16, 64, 2048]))
        return rot(dims, base, factor=rng.choice([2.0, 8.0, 40.0]), fast=rng.choice([4.0, 32.0]), slow=rng.choice([0.5, 1.0]),
                   original=rng.choice([8, 64, 2048]))

    layers = []
    for i in range(rng.randint(3, 5)):
        kind = ["attention", "latent_attention", "retention"][i] if i < 3 else rng.choice(["attention", "latent_attention", "retention"])
        ff = rng.choice([None, 24, 52, 88, 120])
        if kind == "attention":
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 3])
            dim = rng.choice([64, 128]) if tensor_cores else even(4, 32)
            window = rng.choice([None, 3, 17, 64, 100])
            layers.append(layer(attn(dim, rng.choice([64, 128]) if tensor_cores else rng.randint(3, 40), heads, kv, window, rng.choice([0, 1, 5, 70]) if window else 0,
                                     a_rot(dim, "bands") if rng.random() < 0.8 else None, rng.uniform(0.1, 0.4)), ff))
        elif kind == "latent_attention":
            rd = rng.choice([16, 32]) if tensor_cores else even(2, 16)
            r = a_rot(rd, "ramp")
            r["dims"] = rd
            layers.append(layer(latent(rng.randint(3, 24), rd, rng.randint(3, 24), rng.randint(1, 4),
                                       rng.choice([32, 64, 96, 128]) if tensor_cores else rng.choice([8, 20, 32, 64]), r,
                                       rng.uniform(0.1, 0.4)), ff))
        else:
            dim = even(4, 40)
            decay = tuple(rng.uniform(0.5, 1.0) for _ in range(rng.randint(1, 4)))
            layers.append(layer(retention(dim, rng.randint(3, 40), decay, a_rot(dim, "bands") if rng.random() < 0.7 else None), ff))
    rng.shuffle(layers)
    return config(rng.choice([64, 128]) if tensor_cores else rng.choice([40, 48, 72, 96]), rng.randint(50, 120), layers, emb=rng.choice([1.0, 0.5, 12.0]),
                  logit=rng.choice([1.0, 0.5, 2.0]), eps=rng.choice([1e-5, 1e-6]))
