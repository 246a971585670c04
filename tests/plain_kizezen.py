"""The Kizezen decoder, plainly: float64 numpy, whole sequences, no cache or state, one function per
mechanism. It shares no code with the library; the GPU tests compare the library with it.

A layer is  x += mixer(norm1(x))  and then  x += ff(norm2(x))  (RMS norms with a weight; a layer may have no
feed-forward). Three mixers:

* attention: grouped queries with biases on q, k, v; q and k RMS-normed over their whole projections; the first
  channels of every head turned by the position (pairs (i, i + dims / 2), frequencies stretched band by band);
  query i sees key j <= i when i - j < window or j < kept; the softmax denominator holds exp(sink[head]) as well;
  every head's output times sigmoid of one gate logit per head.
* latent attention: keys and values of all heads are made from one normed latent row per position plus one turned
  key part shared by the heads (pairs (2i, 2i + 1), frequencies blended by a ramp, sines and cosines scaled);
  all earlier keys are seen; sink and gate as above.
* retention: S_t = d_head S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k turned by the position and k / sqrt(dim);
  o divided by its root mean square per head, times silu of a gate per channel.
"""
from __future__ import annotations

import math

import numpy as np


def rms_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float64)
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * np.asarray(w, dtype=np.float64)


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# ---- frequencies -----------------------------------------------------------------------------------------------
def base_frequencies(dims, base):
    return np.float64(base) ** (-2.0 * np.arange(dims // 2) / dims)


def banded_frequencies(dims, base, sc):
    """Short waves stay, long waves are slowed by the factor, the band between is blended."""
    out = []
    for f in base_frequencies(dims, base):
        wave = 2.0 * math.pi / f
        if wave < sc["original"] / sc["high"]:
            out.append(f)
        elif wave > sc["original"] / sc["low"]:
            out.append(f / sc["factor"])
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * f / sc["factor"] + s * f)
    return np.array(out)


def ramped_frequencies(dims, base, sc):
    """(frequencies, amplitude): every frequency a blend of itself and itself / factor along a ramp over the pair
    index, whose ends are the pairs that turn `fast` and `slow` times within the original length."""
    def where(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), dims - 1)
    f = base_frequencies(dims, base)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def frequencies(rot):
    """(frequencies, amplitude) of a `rot` entry of the configuration."""
    sc = rot.get("scaling")
    if not sc:
        return base_frequencies(rot["dims"], rot["base"]), 1.0
    if "fast" in sc:
        return ramped_frequencies(rot["dims"], rot["base"], sc)
    return banded_frequencies(rot["dims"], rot["base"], sc), 1.0


def turn(x, positions, freq, amp, dims, layout):
    """x [tokens, heads, dim]: the first `dims` channels of every head turned by position * freq; `layout` "half"
    pairs channel i with i + dims / 2, "pairs" pairs 2i with 2i + 1."""
    out = np.array(x, dtype=np.float64)
    if not dims:
        return out
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = amp * np.cos(ang)[:, None, :], amp * np.sin(ang)[:, None, :]
    if layout == "half":
        a, b = slice(0, dims // 2), slice(dims // 2, dims)
    else:
        a, b = slice(0, dims, 2), slice(1, dims, 2)
    u, v = out[..., a].copy(), out[..., b].copy()
    out[..., a] = u * c - v * s
    out[..., b] = v * c + u * s
    return out


# ---- softmax attention -----------------------------------------------------------------------------------------
def visible(n, window=None, kept=0):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    m = j <= i
    if window:
        m &= (i - j < window) | (j < kept)
    return m


def sink_softmax(scores, mask, sink):
    s = np.where(mask, scores, -np.inf)
    top = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.where(mask, np.exp(s - top), 0.0)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - top))


def attention_core(q, k, v, gate, sink, m, positions=None):
    """[n, H * Dv] from q [n, H * D] and k [n, G * D] (normed already), v [n, G * Dv], gate logits [n, H]: rotation, the
    window with its kept first keys, the sink and the gate."""
    n = q.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    pos = np.arange(n) if positions is None else positions
    q, k, v = q.reshape(n, H, D), k.reshape(n, G, D), v.reshape(n, G, Dv)
    rot = m.get("rot")
    if rot:
        f, amp = frequencies(rot)
        q, k = turn(q, pos, f, amp, rot["dims"], "half"), turn(k, pos, f, amp, rot["dims"], "half")
    mask = m.get("mask") or {}
    see = visible(n, mask.get("size"), mask.get("keep_first", 0))
    out = np.zeros((n, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        w = sink_softmax((q[:, hd] @ k[:, g].T) * m["scale"], see, float(sink[hd]))
        out[:, hd] = (w @ v[:, g]) * sigmoid(gate[:, hd:hd + 1])
    return out.reshape(n, H * Dv)


def attention_mixer(h, t, m, eps, positions=None):
    q = rms_norm(h @ t["q"].T + t["q.b"], t["q.norm"], eps)
    k = rms_norm(h @ t["k"].T + t["k.b"], t["k.norm"], eps)
    return attention_core(q, k, h @ t["v"].T + t["v.b"], h @ t["g"].T, t["sink"], m, positions) @ t["o"].T


def latent_core(q, down, gate, t, m, eps, positions=None):
    """[n, H * Dv] from the query rows [n, H * (D + R)], the down projection's rows [n, C + R] and gate logits [n, H]."""
    n = q.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m.get("vdim", m["dim"]), m["kv_rank"]
    pos = np.arange(n) if positions is None else positions
    q = q.reshape(n, H, D + R)
    latent = rms_norm(down[:, :C], t["dkv.norm"], eps)
    f, amp = frequencies(m["rot"])
    k_turned = turn(down[:, None, C:], pos, f, amp, R, "pairs")[:, 0]                  # [n, R], one for all heads
    q_turned = turn(q[:, :, D:], pos, f, amp, R, "pairs")
    k_plain = (latent @ t["uk"].T).reshape(n, H, D)
    v = (latent @ t["uv"].T).reshape(n, H, Dv)
    see = visible(n)
    out = np.zeros((n, H, Dv))
    for hd in range(H):
        s = (q[:, hd, :D] @ k_plain[:, hd].T + q_turned[:, hd] @ k_turned.T) * m["scale"]
        out[:, hd] = (sink_softmax(s, see, float(t["sink"][hd])) @ v[:, hd]) * sigmoid(gate[:, hd:hd + 1])
    return out.reshape(n, H * Dv)


def latent_attention_mixer(h, t, m, eps, positions=None):
    return latent_core(h @ t["q"].T, h @ t["dkv"].T, h @ t["g"].T, t, m, eps, positions) @ t["o"].T


# ---- retention -------------------------------------------------------------------------------------------------
def retention_core(q, k, v, m, positions=None, conditioning=None):
    """[n, H, Dv]: the read-outs S_t^T q_t before the norm, token by token from S = 0. `conditioning` (a list) gets, per
    row, the smallest ratio over the heads of |o_t| to the root sum of squares of its terms' sizes
    d^(t - j) |q_t| |k_j| |v_j|: where it is tiny the read-out is what cancellation left, and the norm behind it, which
    keeps only the direction, magnifies whatever rounding the terms carry (a first token whose q and k are nearly
    orthogonal, say)."""
    n = q.shape[0]
    H, D, Dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    pos = np.arange(n) if positions is None else positions
    q, k, v = q.reshape(n, H, D), k.reshape(n, H, D), v.reshape(n, H, Dv)
    rot = m.get("rot")
    if rot:
        f, amp = frequencies(rot)
        q, k = turn(q, pos, f, amp, rot["dims"], "half"), turn(k, pos, f, amp, rot["dims"], "half")
    k = k * D ** -0.5
    out = np.zeros((n, H, Dv))
    for hd in range(H):
        S = np.zeros((D, Dv))
        for i in range(n):
            S = m["decay"][hd] * S + np.outer(k[i, hd], v[i, hd])
            out[i, hd] = S.T @ q[i, hd]
    if conditioning is not None:
        ratios = []
        i, j = np.arange(n)[:, None], np.arange(n)[None, :]
        for hd in range(H):
            size = np.where(j <= i, np.float64(m["decay"][hd]) ** np.maximum(i - j, 0), 0.0) * (
                np.linalg.norm(q[:, hd], axis=1)[:, None] * (np.linalg.norm(k[:, hd], axis=1) * np.linalg.norm(v[:, hd], axis=1))[None, :])
            ratios.append(np.linalg.norm(out[:, hd], axis=1) / np.maximum(np.sqrt((size * size).sum(axis=1)), 1e-300))
        conditioning.append(np.min(np.stack(ratios), axis=0))
    return out


def retention_mixer(h, t, m, eps, positions=None, conditioning=None):
    n = h.shape[0]
    out = rms_norm(retention_core(h @ t["q"].T, h @ t["k"].T, h @ t["v"].T, m, positions, conditioning), None, eps)
    return (out.reshape(n, -1) * silu(h @ t["g"].T)) @ t["o"].T


def dense_ff(h, t):
    return gelu_erf(h @ t["up"].T) @ t["down"].T


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer, "retention": retention_mixer}


def part(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, layers_out=None, conditioning=None):
    """Logits [tokens, vocab] of one sequence; `layers_out` (a list) gets the stream after every layer, `conditioning`
    (a list) one array per retention layer (see `retention_core`)."""
    eps = cfg["norm"]["eps"]
    T = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    x = T["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        more = {"conditioning": conditioning} if L["type"] == "retention" and conditioning is not None else {}
        x = x + MIXERS[L["type"]](rms_norm(x, T[p + "norm1"], eps), part(T, p + "mix."), L["mixer"], eps, **more)
        if L.get("mlp"):
            x = x + dense_ff(rms_norm(x, T[p + "norm2"], eps), part(T, p + "mlp."))
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, T["final.norm"], eps) @ T["head"].T * cfg["logit_scale"]
