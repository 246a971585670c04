"""The Nudusun decoder, plainly: float64 numpy, whole sequences, no cache, one function per mechanism.
It shares no code with the library; the GPU tests compare the library with it.

The stream starts as  x_t = c * E[token_t] + P[t]  (c one number of the model, P a table of learned position
rows). A layer norms *after* each sum:  x <- N1(a x + mixer(x)),  x <- N2(a x + ff(x))  (a one number of the
model; the sublayers read x as it is), then takes a per-layer token input: with e_t the layer's own columns of
a second embedding table,  y = Wp (gelu(Wg x) * e_t),  x <- x + y / rms(y) * w.

The mixer is a scalar-gated delta rule (short causal convolutions with SiLU on q, k, v; unit q and k; one decay
and one write strength per head and token; read-out normed per head and gated by SiLU) or a differential
attention (two score maps per head over the same values, each with RMS-normed q and k, a tanh cap on the scores
and a sliding window; the second map's output is subtracted with a learned factor, the difference normed per
head). The feed-forward is a routed one: softmax router over the real experts and a few *identity* experts
(whose output is the input itself), the choice made on scores plus a correction and only within the best
groups of neighbouring experts, weights from the uncorrected scores; clamped gated experts; a shared expert.
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def embed(tokens, table, positions, scale, first=0):
    """Rows c * E[token] + P[position]; the positions count from `first`."""
    tokens = np.asarray(tokens)
    return scale * table[tokens] + positions[first + np.arange(len(tokens))]


def causal_conv(x, taps):
    """x [n, channels], taps [channels, T]: y_t = sum_j taps[:, T - 1 - j] * x_(t - j), zeros before the start."""
    n, T = x.shape[0], taps.shape[1]
    y = np.zeros_like(x)
    for j in range(T):
        if j < n:
            y[j:] += taps[:, T - 1 - j] * x[:n - j]
    return y


def unit(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def delta_rule(q, k, v, beta, decay):
    """q, k [n, H, D], v [n, H, Dv], beta and decay [n, H] -> o [n, H, Dv]. Per head, token by token:
    S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  (the read-out sees the token's own write)."""
    n, H, D = q.shape
    out = np.zeros_like(v)
    for h in range(H):
        S = np.zeros((D, v.shape[2]))
        for t in range(n):
            S = decay[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            out[t, h] = S.T @ q[t, h]
    return out


def same(x):
    return x


def delta_mixer(h, t, cfg, eps, r=same):
    """h [n, width]: the mixer's input rows; t: the mixer's tensors by short name; cfg: its sizes. `r` (here and below)
    stands where a 16-bit engine stores a sublayer's input and its inner rows: the identity, or a rounding."""
    n, h = h.shape[0], r(h)
    H, G, D, Dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = silu(causal_conv(h @ t["q"].T, t["q.conv"])).reshape(n, G, D)
    k = silu(causal_conv(h @ t["k"].T, t["k.conv"])).reshape(n, G, D)
    v = silu(causal_conv(h @ t["v"].T, t["v.conv"])).reshape(n, H, Dv)
    q, k = unit(q) * D ** -0.5, unit(k)
    share = H // G
    q, k = np.repeat(q, share, axis=1), np.repeat(k, share, axis=1)          # head h reads q/k head h // share
    beta = 1.0 / (1.0 + np.exp(-(h @ t["b"].T)))
    decay = np.exp(-np.exp(t["A_log"]) * softplus(h @ t["a"].T + t["dt_bias"]))
    o = delta_rule(q, k, v, beta, decay)
    o = rms(o, eps) * t["norm"] * silu(h @ t["g"].T).reshape(n, H, Dv)
    return r(o.reshape(n, H * Dv)) @ t["o"].T


def window_mask(n, window):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    m = j <= i
    if window:
        m &= (i - j) < window
    return m


def capped_softmax(scores, mask, cap):
    if cap:
        scores = cap * np.tanh(scores / cap)
    s = np.where(mask, scores, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def difference_factor(t, diff):
    return math.exp(float(np.sum(t["lq1"] * t["lk1"]))) - math.exp(float(np.sum(t["lq2"] * t["lk2"]))) + diff


def differential_attention(h, t, cfg, eps, r=same):
    n, h = h.shape[0], r(h)
    H, G, D, Dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = r(rms((h @ t["q"].T).reshape(n, H, 2, D), eps) * t["q.norm"])       # head by head, [map 1, map 2]
    k = r(rms((h @ t["k"].T).reshape(n, G, 2, D), eps) * t["k.norm"])
    v = r((h @ t["v"].T).reshape(n, G, Dv))
    mask = window_mask(n, (cfg.get("mask") or {}).get("size"))
    lam, diff = difference_factor(t, cfg["diff"]), cfg["diff"]
    out = np.zeros((n, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        a = [capped_softmax((q[:, hd, m] @ k[:, g, m].T) * cfg["scale"], mask, cfg.get("softcap")) @ v[:, g] for m in (0, 1)]
        out[:, hd] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    return r(out.reshape(n, H * Dv)) @ t["o"].T


def clamped_expert(h, t, name, limit, r=same):
    g = np.minimum(h @ t[name + ".gate"].T, limit)
    u = np.clip(h @ t[name + ".up"].T, -limit, limit)
    return r(g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ t[name + ".down"].T


def route(h, t, cfg, margins=None):
    """(chosen [n, top] expert numbers, weights [n, top]). Experts `experts .. experts + identity` are the identity
    ones. `margins` (a list) receives per row the smallest gap of the choice: between the last chosen choice score and
    the best one left out, and between the last group kept and the best one closed."""
    r = cfg["router"]
    E, top = r["experts"] + r.get("identity", 0), r["top"]
    z = h @ t["router"].T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    choice = s + t["correction"] if "correction" in t else s.copy()
    groups = r.get("groups")
    gap = np.full(h.shape[0], np.inf)
    if groups:
        per = E // groups["count"]
        best = choice.reshape(-1, groups["count"], per).max(axis=-1)
        if groups["keep"] < groups["count"]:
            ranked = -np.sort(-best, axis=-1)
            gap = ranked[:, groups["keep"] - 1] - ranked[:, groups["keep"]]
        for row in range(h.shape[0]):
            kept = np.argsort(-best[row], kind="stable")[:groups["keep"]]
            closed = np.ones(groups["count"], dtype=bool)
            closed[kept] = False
            choice[row, np.repeat(closed, per)] = -np.inf
    order = np.argsort(-choice, axis=-1, kind="stable")
    chosen = order[:, :top]
    if margins is not None:
        ranked = np.take_along_axis(choice, order, axis=-1)
        margins.append(np.minimum(gap, ranked[:, top - 1] - ranked[:, top]) if top < E else gap)
    return chosen, np.take_along_axis(s, chosen, axis=-1) * r.get("scale", 1.0)


def routed_ff(h, t, cfg, margins=None, r=same):
    real = cfg["router"]["experts"]
    exact, h = h, r(h)
    chosen, weights = route(h, t, cfg, margins)
    out = np.zeros_like(h)
    for row in range(h.shape[0]):
        for e, w in zip(chosen[row], weights[row]):
            # an identity expert hands back the row of the stream itself
            y = exact[row] if e >= real else clamped_expert(h[row:row + 1], t, f"e{e}", cfg["expert"]["limit"], r)[0]
            out[row] += w * y
    if cfg.get("shared"):
        out += clamped_expert(h, t, "shared", cfg["shared"]["limit"], r)
    return out


def token_input(x, tokens, table, i, t, dim, eps, r=same):
    """What layer i adds from its own columns of the second table."""
    e = table[np.asarray(tokens), i * dim:(i + 1) * dim]
    y = r(gelu_tanh(r(x) @ t["gate"].T) * e) @ t["proj"].T
    return rms(y, eps) * t["norm"]


def sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, probe=None, margins=None, r=same):
    """Logits [tokens, vocab] of one sequence; `probe(i, x)` sees the stream after every layer. With a rounding `r`
    the result shows how far 16-bit storage between the steps moves each row: a measure of the row's sensitivity."""
    f64 = lambda n: np.asarray(tensors[n], dtype=np.float64)          # noqa: E731
    eps, a = config["norm"]["eps"], config.get("postln_alpha", 1.0)
    x = embed(tokens, f64("embed"), f64("pos"), config["embedding"]["scale"])
    side = config.get("token_side")
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        mixer = delta_mixer if L["type"] == "delta" else differential_attention
        x = rms(a * x + mixer(x, sub(tensors, p + "mix."), L["mixer"], eps, r), eps) * f64(p + "norm1")
        if L.get("mlp") is not None:
            x = rms(a * x + routed_ff(x, sub(tensors, p + "mlp."), L["mlp"], margins, r), eps) * f64(p + "norm2")
        if side:
            x = x + token_input(x, tokens, f64("side.embed"), i, sub(tensors, p + "side."), side["dim"], eps, r)
        if probe is not None:
            probe(i, x)
    return r(rms(x, eps) * f64("final.norm")) @ f64("head").T
