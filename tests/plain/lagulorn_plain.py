"""Plain float64 restatement of the Lagulorn decoder: whole sequences, no cache, no batching, one function
per mechanism, NumPy only.  It shares no code with the package and is the oracle of its tests.

Notation: x [T, width] a sequence's hidden rows; W matrices stored [out, in] and applied as x @ W.T;
`cfg` is the dict of a config.json, `w` a dict name -> float64 array.  `rnd` (default: the identity) is applied
to what a 16-bit implementation may round: the input and the output of every matrix product.  The tests take
the deviation it causes as the scale of their bfloat16 tolerance.
"""
from __future__ import annotations

import math

import numpy as np


def same(x):
    return x


def round_bf16(x):
    """Round to the nearest bfloat16 (ties to even), as float64."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, weight, eps):
    """A norm whose stored weight lies around zero: unit rms, times (1 + weight)."""
    return rms_unit(x, eps) * (1.0 + weight)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def embedding(table, ids, scale):
    return table[np.asarray(ids)] * scale


# ---------------------------------------------------------------- mixers
def lightning_mixer(h, w, p, m, eps, rnd=same):
    """Linear attention with a per-head decay: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; the heads side by
    side get unit rms together, a weight, a sigmoid gate, and the output projection."""
    T = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    q = silu(rnd(h @ w[p + "q"].T)).reshape(T, H, d)
    k = silu(rnd(h @ w[p + "k"].T)).reshape(T, H, d)
    v = silu(rnd(h @ w[p + "v"].T)).reshape(T, H, vd)
    out = np.zeros((T, H, vd))
    for head in range(H):
        state = np.zeros((d, vd))
        for t in range(T):
            state = m["decay"][head] * state + np.outer(k[t, head], v[t, head])
            out[t, head] = state.T @ q[t, head]
    flat = rms_unit(out.reshape(T, H * vd), eps) * w[p + "norm"]
    return rnd(rnd(flat * sigmoid(rnd(h @ w[p + "g"].T))) @ w[p + "o"].T)


def window_softmax_attention(q, k, v, scale, window):
    """q [T, d], k [T, d], v [T, vd]: position i reads j with 0 <= i - j < window (None: every j <= i)."""
    T = q.shape[0]
    out = np.zeros((T, v.shape[1]))
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        s = (k[lo:i + 1] @ q[i]) * scale
        p = np.exp(s - s.max())
        out[i] = (p / p.sum()) @ v[lo:i + 1]
    return out


def differential_mixer(h, w, p, m, eps, rnd=same):
    """Two softmax maps per head over the same values, o = a1 - lambda a2, unit rms per head, times (1 - diff)."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window = m["mask"]["size"] if m.get("mask") else None
    q = rnd(h @ w[p + "q"].T).reshape(T, H, 2, d)
    k = rnd(h @ w[p + "k"].T).reshape(T, G, 2, d)
    v = rnd(h @ w[p + "v"].T).reshape(T, G, vd)
    q = rnd(rms_unit(q, eps) * w[p + "q.norm"])
    k = rnd(rms_unit(k, eps) * w[p + "k.norm"])
    lam = (math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"])))
           + m["diff"])
    heads = []
    for head in range(H):
        g = head // (H // G)
        a1 = window_softmax_attention(q[:, head, 0], k[:, g, 0], v[:, g], m["scale"], window)
        a2 = window_softmax_attention(q[:, head, 1], k[:, g, 1], v[:, g], m["scale"], window)
        heads.append(rms_unit(a1 - lam * a2, eps) * (1.0 - m["diff"]))
    return rnd(rnd(np.concatenate(heads, axis=1)) @ w[p + "o"].T)


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p, rnd=same):
    return rnd(rnd(gelu_erf(rnd(h @ w[p + "up"].T))) @ w[p + "down"].T)


def route(z, correction, top, groups_count, groups_keep):
    """z [n] router logits of one token -> (chosen indices, their weights).  Scores are the softmax over all
    outputs; the choice is made on score + correction, restricted to the best groups; weights are plain scores."""
    s = np.exp(z - z.max())
    s = s / s.sum()
    choice = s + correction
    n = z.shape[0]
    if groups_count and groups_count > 1:
        size = n // groups_count
        best = np.array([choice[g * size:(g + 1) * size].max() for g in range(groups_count)])
        kept = np.argsort(-best, kind="stable")[:groups_keep]
        mask = np.full(n, -np.inf)
        for g in kept:
            mask[g * size:(g + 1) * size] = 0.0
        choice = choice + mask
    chosen = np.argsort(-choice, kind="stable")[:top]
    return chosen, s[chosen]


def expert(h, gate, up, down, limit, rnd=same):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return rnd(g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe_ff(h, w, p, mlp, rnd=same):
    r = mlp["router"]
    n_real, n_id = r["experts"], r.get("identity", 0) or 0
    groups = r.get("groups") or {}
    z = h @ w[p + "router"].T
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], w[p + "correction"], r["top"], groups.get("count", 1), groups.get("keep", 1))
        for e, weight in zip(chosen, weights):
            if e >= n_real:
                out[t] += weight * h[t]
            else:
                q = f"{p}e{e}."
                out[t] += weight * expert(h[t], w[q + "gate"], w[q + "up"], w[q + "down"], mlp["expert"]["limit"], rnd)
    assert n_real + n_id == z.shape[1]
    return rnd(out)


# ---------------------------------------------------------------- a layer and the model
def hyper_step(xs, hc, m, sublayer):
    """xs [s, T, width]; hc = (into [s], out [s], mix [s, s] indexed [from, to]).  The sublayer reads the weighted
    sum of the streams; every new stream is a mix of the old ones plus its share of the sublayer's output."""
    into, out, mix = hc
    y = sublayer(np.tensordot(into, xs, axes=(0, 0)))
    return np.einsum("st,sij->tij", mix, xs) + m * out[:, None, None] * y[None]


def forward(cfg, w, tokens, want_layers=False, rnd=same):
    """Logits [T, vocab] of one sequence (and, if asked, the sum of the streams after every layer run)."""
    eps = cfg["norm"]["eps"]
    m = cfg.get("residual_mult", 1.0)
    s = cfg.get("streams")
    x = embedding(w["embed"], tokens, (cfg.get("embedding") or {}).get("scale", 1.0))
    xs = np.stack([x] * (s or 1))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        owner = layer.get("weights_of", i)
        p = f"l{owner}."
        mixer = {"lightning": lightning_mixer, "attention": differential_mixer}[layer["type"]]
        subs = [(1, lambda u: mixer(rnd(norm_one_plus(u, w[p + "norm1"], eps)), w, p + "mix.", layer["mixer"], eps, rnd))]
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = (lambda u: dense_ff(u, w, p + "mlp.", rnd)) if mlp["kind"] == "dense" else (lambda u: moe_ff(u, w, p + "mlp.", mlp, rnd))
            subs.append((2, lambda u: ff(rnd(norm_one_plus(u, w[p + "norm2"], eps)))))
        for number, sub in subs:
            if s is None:
                xs = xs + m * sub(xs[0])[None]
            else:
                xs = hyper_step(xs, (w[f"{p}hc{number}.in"], w[f"{p}hc{number}.out"], w[f"{p}hc{number}.mix"]), m, sub)
        after.append(xs.sum(axis=0))
    logits = rnd(norm_one_plus(xs.sum(axis=0), w["final.norm"], eps)) @ w["head"].T
    return (logits, np.stack(after)) if want_layers else logits


def generate_greedy(cfg, w, prompt, n_new):
    """The tokens that greedy choice appends to `prompt` (the whole sequence is recomputed for every token)."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
