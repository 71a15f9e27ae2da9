"""Plain, slow Dozazen decoder: whole sequences, no cache, one function per mechanism.

The oracle of the Dozazen tests.  It shares no code with the product package: it takes the
dict of a config.json and a dict of float64 NumPy arrays keyed by tensor name, and recomputes
every position of a sequence from scratch.  Notation: x is the hidden state [T, width], h a
normalised copy of it, p a position counted from 0.

`rnd` is a rounding hook: the identity gives the exact model; `round_bf16` rounds where a
bfloat16 engine does (the inputs and outputs of matrix products and activations), which is how
the tests size the tolerance of the bfloat16 engine.  Norms, the hidden state, angles, scores
and softmax weights are never rounded: the design computes them in 32-bit.
"""
from __future__ import annotations

import math

import numpy as np


def identity(x):
    return x


def round_bf16(x):
    f = np.asarray(x, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


# ----------------------------------------------------------------------------- mechanisms


def embedding(tokens, table, scale):
    """x[t] = table[token[t]] * scale"""
    return table[np.asarray(tokens, dtype=np.int64)] * scale


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w, eps inside the root"""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """f_i = base^(-2i/dims), then rescaled by wavelength l = 2 pi / f: kept where l < original/high, divided by
    `factor` where l > original/low, blended in between."""
    dims = rot["dims"]
    freqs = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            wavelength = 2.0 * math.pi / f
            if wavelength < sc["original"] / sc["high"]:
                pass
            elif wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        freqs.append(f)
    return np.array(freqs, dtype=np.float64)


def rotate_interleaved(t, positions, rot):
    """t [T, heads, d]: the pair (t[2i], t[2i+1]), i < dims/2, turns by the angle p * f_i; the rest passes."""
    if rot is None:
        return t
    dims = rot["dims"]
    angle = np.asarray(positions, dtype=np.float64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    out = t.copy()
    u, v = t[..., 0:dims:2], t[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(positions_q, positions_k, chunk):
    """[Tq, Tk] bool: key j is seen from query i if j <= i and (with chunks) both lie in the same chunk."""
    i = np.asarray(positions_q)[:, None]
    j = np.asarray(positions_k)[None, :]
    ok = j <= i
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    return ok


def capped(scores, cap):
    return cap * np.tanh(scores / cap) if cap else scores


def sink_softmax(scores, ok):
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)) over the visible keys: a sink of score 0 that has no value."""
    m = np.maximum(np.max(np.where(ok, scores, -np.inf), axis=-1, keepdims=True), 0.0)
    e = np.where(ok, np.exp(scores - m), 0.0)
    return e / (np.exp(-m) + e.sum(-1, keepdims=True))


def attend(q, k, v, positions_q, positions_k, scale, cap, chunk):
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, vd] -> [Tq, H, vd]; query head h uses key/value head h // (H/G)."""
    H, G = q.shape[1], k.shape[1]
    ok = visible(positions_q, positions_k, chunk)
    out = np.zeros((q.shape[0], H, v.shape[2]), dtype=np.float64)
    for h in range(H):
        g = h // (H // G)
        p = sink_softmax(capped(q[:, h] @ k[:, g].T * scale, cap), ok)
        out[:, h] = p @ v[:, g]
    return out


def attention_mixer(h, w, prefix, m, rnd=identity):
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m.get("vdim") or m["dim"]
    h = rnd(h)
    q = rnd(h @ w[prefix + "q"].T + w[prefix + "q.b"]).reshape(T, H, d)
    k = rnd(h @ w[prefix + "k"].T + w[prefix + "k.b"]).reshape(T, G, d)
    v = rnd(h @ w[prefix + "v"].T + w[prefix + "v.b"]).reshape(T, G, vd)
    pos = np.arange(T)
    q, k = rnd(rotate_interleaved(q, pos, m.get("rot"))), rnd(rotate_interleaved(k, pos, m.get("rot")))
    chunk = m["mask"]["size"] if m.get("mask") else None
    o = rnd(attend(q, k, v, pos, pos, m["scale"], m.get("softcap"), chunk))
    return rnd(o.reshape(T, H * vd) @ w[prefix + "o"].T)


def gated_mlp(h, w, prefix, rnd=identity):
    h = rnd(h)
    return rnd(rnd(rnd(gelu_tanh(rnd(h @ w[prefix + "gate"].T))) * rnd(h @ w[prefix + "up"].T)) @ w[prefix + "down"].T)


def mix_in(x, x0, w, rnd=identity):
    """x <- W [x; x0]"""
    return rnd(np.concatenate([x, x0], axis=-1)) @ w.T


def layer(x, w, i, spec, eps, rnd=identity):
    p = f"l{i}."
    x = x + rms_norm(attention_mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], rnd), w[p + "norm1b"], eps)
    if spec.get("mlp"):
        x = x + rms_norm(gated_mlp(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", rnd), w[p + "norm2b"], eps)
    return x


def run_order(cfg):
    """[(layer, whether a pass starts here)]"""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, rnd=identity, states=None):
    """Logits [T, vocab] of every position; `states` (a list) receives the hidden state after every layer run."""
    eps = cfg["norm"]["eps"]
    x = embedding(tokens, w["embed"], (cfg.get("embedding") or {}).get("scale", 1.0))
    x0 = x
    for i, starts in run_order(cfg):
        if starts:
            x = mix_in(x, x0, w["loop.in"], rnd)
        x = layer(x, w, i, cfg["layers"][i], eps, rnd)
        if states is not None:
            states.append(x)
    z = rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T * cfg.get("logit_scale", 1.0)
    return capped(z, cfg.get("logit_softcap"))


def generate_greedy(cfg, w, prompt, n_new):
    tokens, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
        tokens.append(out[-1])
    return out
