"""A plain, slow implementation of the Vipovik design in float64 numpy: one function per mechanism, whole sequences at a
time, no cache, no batching.  The tests hold the engine against it.  It shares no code with the package.

A model is (cfg, w): cfg the contents of config.json, w a dict name -> float64 array.

    layer            x += mixer(rms(x) * norm1); x += ff(rms(x) * norm2)
    mixer 'parallel' left_scale * window_attention(h) + right_scale * time_mix(h)
    window attention rotate-half rotation of the leading rot.dims elements with stretched frequencies, unit RMS norm of q and
                     k per head, capped scores c tanh(s / c), a sliding window that also keeps the first tokens
    time mix         token shift with one mixing vector per projection, a decay exp(-exp(.)) per key channel, a bonus for the
                     current token, a unit RMS norm per head times a weight, a silu gate
    feed-forward     dense: down(gelu(up h)); experts: softmax router, the top few renormalised, clamped gated units
    loop             layers start .. stop-1 run `times` times; before each pass x <- W [x | x0] + step[pass]
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_erf(z):
    erf = np.vectorize(math.erf)
    return 0.5 * z * (1.0 + erf(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


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


def visible(i, j, mask):
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if mask is None:
        return True
    size = mask.get("size")
    return (size is None or i - j < int(size)) or j < int(mask.get("keep_first") or 0)


def visibility(positions, mask):
    """[T, T] of ``visible`` for every pair of positions."""
    p = np.asarray(positions)
    i, j = p[:, None], p[None, :]
    see = j <= i
    if mask is not None and mask.get("size") is not None:
        see &= (i - j < int(mask["size"])) | (j < int(mask.get("keep_first") or 0))
    return see


def window_attention(h, m, w, prefix, eps, positions=None):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ w[prefix + "q"].T).reshape(T, H, d)
    k = (h @ w[prefix + "k"].T).reshape(T, G, d)
    v = (h @ w[prefix + "v"].T).reshape(T, G, dv)
    if m.get("rot"):
        q, k = rotate_half(q, positions, m["rot"]), rotate_half(k, positions, m["rot"])
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    out = capped_attention(q, k, v, float(m["scale"]), m.get("softcap"), m.get("mask"), positions)
    return out.reshape(T, H * dv) @ w[prefix + "o"].T


def capped_attention(q, k, v, scale, cap, mask, positions):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]: capped scores, softmax over the visible keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[-1]))
    see = visibility(positions, mask)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        if cap:
            s = float(cap) * np.tanh(s / float(cap))
        s = np.where(see, s, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, hd] = (p / p.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out


def time_mix(h, m, w, prefix, eps, state=None, last=None):
    """Returns (output, state, last input).  ``state`` [heads, dim, dim] and ``last`` [width] continue a sequence."""
    T, width = h.shape
    H, d = int(m["heads"]), int(m["dim"])
    mix = {s: shifted(h, w[prefix + "mu." + s], last) for s in "rkvgw"}
    r = (mix["r"] @ w[prefix + "r"].T).reshape(T, H, d)
    k = (mix["k"] @ w[prefix + "k"].T).reshape(T, H, d)
    v = (mix["v"] @ w[prefix + "v"].T).reshape(T, H, d)
    gate = silu(mix["g"] @ w[prefix + "g"].T)
    decay = np.exp(-np.exp(np.tanh(mix["w"] @ w[prefix + "w1"].T) @ w[prefix + "w2"].T + w[prefix + "w0"])).reshape(T, H, d)
    o, S = bonus_recurrence(r, k, v, decay, w[prefix + "u"].reshape(H, d), state)
    o = rms_unit(o, eps).reshape(T, H * d) * w[prefix + "norm"] * gate
    return o @ w[prefix + "o"].T, S, h[-1].copy()


def shifted(h, mu, last=None):
    """h_t + (h_(t-1) - h_t) * mu; the row before the first is ``last`` (zeros at the start of a sequence)."""
    prev = np.vstack([np.zeros((1, h.shape[1])) if last is None else last[None, :], h[:-1]])
    return h + (prev - h) * mu


def bonus_recurrence(r, k, v, decay, u, state=None):
    """Per head: o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(decay_t) S + k_t v_t^T.  r, k, decay [T, H, d], v
    [T, H, dv], u [H, d]; returns (o [T, H, dv], S [H, d, dv])."""
    T, H, d = k.shape
    S = np.zeros((H, d, v.shape[-1])) if state is None else state.copy()
    o = np.zeros((T, H, v.shape[-1]))
    for t in range(T):
        for hd in range(H):
            kv = np.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S[hd] + u[hd][:, None] * kv).T @ r[t, hd]
            S[hd] = decay[t, hd][:, None] * S[hd] + kv
    return o, S


def parallel_mixer(h, m, w, prefix, eps):
    left = window_attention(h, m["left"], w, prefix + "left.", eps)
    right, _, _ = time_mix(h, m["right"], w, prefix + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def dense_ff(h, w, prefix):
    return gelu_erf(h @ w[prefix + "up"].T) @ w[prefix + "down"].T


def expert_unit(h, w, prefix, limit):
    g = np.minimum(h @ w[prefix + "gate"].T, limit)
    u = np.clip(h @ w[prefix + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def route(h, w, prefix, top):
    """(chosen experts [T, top], their weights [T, top])."""
    z = h @ w[prefix + "router"].T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, axis=-1)
    return chosen, picked / (picked.sum(axis=-1, keepdims=True) + 1e-20)


def router_margin(h, w, prefix, top):
    """Per row: how far (in the router's output) the last chosen expert lies above the first one left out."""
    z = np.sort(h @ w[prefix + "router"].T, axis=-1)[:, ::-1]
    return z[:, top - 1] - z[:, top] if z.shape[1] > top else np.full(h.shape[0], np.inf)


def experts_ff(h, mlp, w, prefix, margins=None):
    chosen, weights = route(h, w, prefix, int(mlp["router"]["top"]))
    if margins is not None:
        margins.append(router_margin(h, w, prefix, int(mlp["router"]["top"])))
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], weights[t]):
            out[t] += s * expert_unit(h[t:t + 1], w, f"{prefix}e{int(e)}.", float(mlp["expert"]["limit"]))[0]
    return out


def feed_forward(h, mlp, w, prefix, margins=None):
    return dense_ff(h, w, prefix) if mlp["kind"] == "dense" else experts_ff(h, mlp, w, prefix, margins)


def layer(x, spec, w, prefix, eps, margins=None):
    if spec["type"] != "parallel":
        raise ValueError(spec["type"])
    x = x + parallel_mixer(rms_norm(x, w[prefix + "norm1"], eps), spec["mixer"], w, prefix + "mix.", eps)
    if spec.get("mlp") is not None:
        x = x + feed_forward(rms_norm(x, w[prefix + "norm2"], eps), spec["mlp"], w, prefix + "mlp.", margins)
    return x


def run_order(cfg):
    """(layer, pass number or None, whether a pass starts here) for every layer run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, n)]


def forward(cfg, w, tokens, streams=None, margins=None):
    """Logits [T, vocab] of a whole sequence; ``streams`` (a list) receives the stream after every layer run, ``margins`` the
    router margins [T] of every run of a routed feed-forward."""
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    x = x0
    for i, t, opens in run_order(cfg):
        if opens:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(x, cfg["layers"][i], w, f"l{i}.", eps, margins)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
