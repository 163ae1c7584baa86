"""A plain, slow implementation of the Fapenex design in float64 numpy: one function per mechanism, whole sequences at a
time, no cache, no batching.  The tests hold the engine against it.  It shares no code with the package.

A model is (cfg, w): cfg the contents of config.json, w a dict name -> float64 array.

    embedding        x_t = embed[token_t] + pos[t]
    layer            x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))); norms are x / rms(x) * (1 + weight)
    latent_attention queries through a normed latent, keys and values from one normed latent per position, no rotation,
                     a sliding window, ordinary softmax
    delta            gated delta rule behind short convolutions with silu, unit q and k, one decay and one write strength
                     per head, a norm per head and a silu gate on the way out
    attention        grouped heads with biases, a norm per head of q and k ahead of a partial rotate-half rotation with
                     stretched frequencies, keys of the query's own chunk only, softmax with one more in the denominator
    feed-forward     router logits with a bias, the top few, softmax over the chosen; clamped gated units; a shared unit
                     times a sigmoid gate per token
    loop             layers start .. stop-1 run `times` times; before each pass x += step[pass]
    output           final norm, the embedding table as output matrix, a scale, c tanh(. / c)
"""
from __future__ import annotations

import math

import numpy as np


def operand(a):
    """Every operand of a matrix product passes here.  The identity; a test that wants to know what 16-bit operands alone do
    to a model's logits replaces it by a rounding."""
    return a


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_plain(x, weight, eps):
    return rms_unit(x, eps) * weight


def norm_one_plus(x, weight, eps):
    return rms_unit(x, eps) * (1.0 + weight)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rotary_frequencies(rot):
    """(frequency of each pair, factor of cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, rot):
    """x [T, heads, dim]: element i < dims/2 of a head pairs with element i + dims/2."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_frequencies(rot)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = (np.cos(a) * mag)[:, None, :], (np.sin(a) * mag)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# ---- masks -------------------------------------------------------------------------------------------------------------
def sees_window(i, j, size):
    return 0 <= i - j < size


def sees_chunk(i, j, size):
    return j <= i and i // size == j // size


def visibility(positions, rule, size):
    p = np.asarray(positions)
    return np.array([[rule(int(i), int(j), size) for j in p] for i in p], dtype=bool)


def masked_softmax_attention(q, k, v, scale, see, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  `sink`: one more term exp(0) in the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[-1]))
    for hd in range(H):
        g = hd // (H // G)
        s = np.where(see, (q[:, hd] @ k[:, g].T) * scale, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        if sink:
            m = np.maximum(m, 0.0)
        p = np.exp(s - m)
        den = p.sum(axis=-1, keepdims=True) + (np.exp(-m) if sink else 0.0)
        out[:, hd] = (p / den) @ v[:, g]
    return out


# ---- mixers ------------------------------------------------------------------------------------------------------------
def latent_attention(h, m, w, p, eps, positions=None):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    positions = np.arange(T) if positions is None else np.asarray(positions)
    cq = operand(norm_plain(h @ w[p + "dq"].T, w[p + "dq.norm"], eps))
    q = operand((cq @ w[p + "uq"].T).reshape(T, H, d))
    c = operand(norm_plain(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps))
    k = operand((c @ w[p + "uk"].T).reshape(T, H, d))
    v = operand((c @ w[p + "uv"].T).reshape(T, H, dv))
    see = visibility(positions, sees_window, int(m["mask"]["size"]))
    out = masked_softmax_attention(q, k, v, float(m["scale"]), see, sink=False)
    return operand(out.reshape(T, H * dv)) @ w[p + "o"].T


def chunk_attention(h, m, w, p, eps, positions=None):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q, k = norm_plain(q, w[p + "q.norm"], eps), norm_plain(k, w[p + "k.norm"], eps)
    if m.get("rot") and int(m["rot"].get("dims") or 0):
        q, k = rotate_half(q, positions, m["rot"]), rotate_half(k, positions, m["rot"])
    see = visibility(positions, sees_chunk, int(m["mask"]["size"]))
    out = masked_softmax_attention(operand(q), operand(k), operand(v), float(m["scale"]), see, sink=True)
    return operand(out.reshape(T, H * dv)) @ w[p + "o"].T


def short_conv(u, taps, before=None):
    """u [T, C], taps [C, J] (last column: the current row); `before` [J - 1, C]: the rows ahead of the first (zeros)."""
    T, C = u.shape
    J = taps.shape[1]
    pad = np.zeros((J - 1, C)) if before is None else before
    full = np.concatenate([pad, u], axis=0)
    out = np.zeros((T, C))
    for j in range(J):
        out += full[j: j + T] * taps[:, j]
    return out


def unit_vector(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def delta_recurrence(q, k, v, g, beta, state=None):
    """q, k [T, H, dk], v [T, H, dv], g, beta [T, H] -> (o [T, H, dv], S [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = np.zeros((H, dk, dv)) if state is None else state.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            S[hd] = g[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, hd])
            S[hd] = S[hd] + np.outer(k[t, hd], u)
            o[t, hd] = S[hd].T @ q[t, hd]
    return o, S


def delta_mixer(h, m, w, p, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q, k = unit_vector(q) * d ** -0.5, unit_vector(k)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    beta = sigmoid(h @ w[p + "b"].T)
    g = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o, _ = delta_recurrence(q, k, v, g, beta)
    o = rms_unit(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).reshape(T, H, dv)
    return operand(o.reshape(T, H * dv)) @ w[p + "o"].T


# ---- feed-forward ------------------------------------------------------------------------------------------------------
def clamped_unit(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return operand(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def router_logits(h, w, p):
    return h @ w[p + "router"].T + w[p + "router.b"]


def route(h, w, p, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen only."""
    z = router_logits(h, w, p)
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return chosen, e / e.sum(axis=-1, keepdims=True)


def router_margin(h, w, p, top):
    """Per row: the gap between the last chosen logit and the first one left out."""
    z = np.sort(router_logits(h, w, p), axis=-1)[:, ::-1]
    return z[:, top - 1] - z[:, top] if z.shape[1] > top else np.full(z.shape[0], np.inf)


def experts_ff(h, mlp, w, p, margins=None):
    top = int(mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    chosen, weight = route(h, w, p, top)
    if margins is not None:
        margins.append(router_margin(h, w, p, top))
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], weight[t]):
            out[t] += s * clamped_unit(h[t: t + 1], w, f"{p}e{int(e)}.", limit)[0]
    if mlp.get("shared"):
        gate = sigmoid(h @ w[p + "shared.sg"].T)          # [T, 1]
        out += gate * clamped_unit(h, w, p + "shared.", float(mlp["shared"]["limit"]))
    return out


# ---- the model ---------------------------------------------------------------------------------------------------------
MIXERS = {"latent_attention": latent_attention, "delta": delta_mixer, "attention": chunk_attention}


def layer(x, spec, w, p, eps, margins=None):
    h = operand(norm_one_plus(x, w[p + "norm1"], eps))
    x = x + norm_one_plus(MIXERS[spec["type"]](h, spec["mixer"], w, p + "mix.", eps), w[p + "norm1b"], eps)
    if spec.get("mlp") is not None:
        h = operand(norm_one_plus(x, w[p + "norm2"], eps))
        x = x + norm_one_plus(experts_ff(h, spec["mlp"], w, p + "mlp.", margins), w[p + "norm2b"], eps)
    return x


def run_order(cfg):
    """(layer, pass number if the pass starts here else None) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(cfg, w, tokens, streams=None, margins=None):
    """Logits [T, vocab] of one whole sequence.  `streams`: a list that receives the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    tokens = np.asarray(tokens)
    x = w["embed"][tokens] + w["pos"][: len(tokens)]
    for i, opens in run_order(cfg):
        if opens is not None:
            x = x + w["loop.step"][opens]
        x = layer(x, cfg["layers"][i], w, f"l{i}.", eps, margins)
        if streams is not None:
            streams.append(x.copy())
    logits = operand(norm_one_plus(x, w["final.norm"], eps)) @ w["embed"].T * float(cfg.get("logit_scale") or 1.0)
    cap = cfg.get("logit_softcap")
    return float(cap) * np.tanh(logits / float(cap)) if cap else logits
