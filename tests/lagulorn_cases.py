"""Shared by the Lagulorn tests: small configurations that differ in every size and option, and model folders
with weights lively enough that attention is peaked, routers decide clearly and the streams really mix; stored in
bfloat16 so that the plain implementation reads the same values."""
import copy
import os

import numpy as np


def attention(heads, kv, dim, vdim, scale, diff, mask=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "attention", "mixer": m}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def moe(ff, limit, experts, top, identity=None, groups=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp, weights_of=None):
    out = dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


# Three streams; a lightning layer first, with a decay of exactly 1 and experts without identity or groups; an attention layer
# with two key/value heads, values narrower than keys and a window that is no multiple of a page, run twice with the same
# weights; a layer without feed-forward; an attention layer without a window, as many key/value heads as heads, identity
# experts and four groups of which two are kept; the first layer once more at the end.
_A0 = layer(lightning(3, 16, 24, [0.9, 0.5, 1.0]), moe(40, 2.0, 6, 2))
_A1 = layer(attention(4, 2, 16, 8, 0.3, 0.2, 70), dense(96))
L_A = {
    "architecture": "Lagulorn", "vocab": 211, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "residual_mult": 0.7, "streams": 3,
    "layers": [_A0, _A1, dict(_A1, weights_of=1), layer(lightning(2, 8, 8, [0.97, 0.8]), None),
               layer(attention(2, 2, 24, 40, 0.25, 0.5), moe(24, 0.5, 5, 3, identity=3, groups=(4, 2))), dict(_A0, weights_of=0)],
}
# No streams (a plain residual sum), no residual multiplier, no embedding scale; a window of exactly one page; one expert
# chosen among five groups of one; a single lightning head whose values are wider than its keys.
L_B = {
    "architecture": "Lagulorn", "vocab": 128, "width": 96, "norm": {"eps": 1e-5},
    "layers": [layer(attention(2, 1, 32, 32, 0.18, 0.1, 64), moe(48, 1.5, 4, 1, identity=1, groups=(5, 1))),
               layer(lightning(1, 64, 128, [0.999]), dense(128))],
}
# One stream that still has its connection tensors; head sizes the tensor cores like; a window of several pages; a state
# of 256 x 256 that only the token-by-token form takes; eight experts in two groups, both kept.
L_C = {
    "architecture": "Lagulorn", "vocab": 320, "width": 128, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-5},
    "residual_mult": 1.5, "streams": 1,
    "layers": [layer(lightning(2, 128, 128, [0.99, 0.95]), moe(64, 1.0, 8, 4, groups=(2, 2))),
               layer(attention(8, 2, 64, 64, 0.125, 0.3, 200), dense(256)),
               layer(lightning(1, 256, 256, [0.9]), None),
               layer(attention(8, 2, 64, 64, 0.125, 0.3, 200), dense(256), weights_of=1)],
}
# Sizes that rule out every vector path: a width that is no multiple of 4, odd head sizes and vocabulary; windows of one
# position (a token sees itself only) and of seven; a decay of zero (the state is the last token's alone); every expert
# chosen (top = experts + identity).
L_D = {
    "architecture": "Lagulorn", "vocab": 97, "width": 50, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
    "residual_mult": 0.5, "streams": 2,
    "layers": [layer(attention(2, 1, 11, 7, 0.3, 0.4, 7), moe(30, 1.0, 3, 5, identity=2)),
               layer(lightning(3, 5, 9, [0.0, 0.7, 0.95]), dense(21)),
               layer(attention(3, 3, 6, 9, 0.4, 0.25, 1), None)],
}
CASES = {"A": L_A, "B": L_B, "C": L_C, "D": L_D}


def case(name, **changes):
    cfg = copy.deepcopy(CASES[name])
    cfg.update(changes)
    return cfg


def lively_weights(specs, seed):
    """{name: bfloat16 tensor}: matrices N(0, 1/fan_in) (routers four times that, so that choices are clear), the
    embedding table N(0, 1), norm weights around 0 or 1 as the part stores them, lambda vectors and corrections small,
    connection tensors near a plain residual sum (in near 1/s, out near 1, mix near the identity) with enough noise
    that every entry matters."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        spec = specs[name]
        draw = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        tail = name.rsplit(".", 1)[-1]
        if ".hc" in name:
            s = spec.shape[0]
            draw = {"in": 1.0 / s + 0.3 * draw, "out": 1.0 + 0.3 * draw}.get(tail, torch.eye(s) + 0.2 * draw) if tail != "mix" \
                else torch.eye(s) + 0.2 * draw
        elif spec.role == "norm":
            draw = 1.0 + 0.2 * draw
        elif tail in ("lq1", "lk1", "lq2", "lk2"):
            draw = 0.3 * draw
        elif tail == "correction":
            draw = 0.1 * draw
        elif spec.role == "bias":                      # norm weights stored around zero
            draw = 0.2 * draw
        elif tail == "router":
            draw = 4.0 * draw / (spec.shape[-1] ** 0.5)
        elif name != "embed":
            draw = draw / (spec.shape[-1] ** 0.5)
        out[name] = draw.to(torch.bfloat16)
    return out


def make_folder(tmp_path, cfg, seed, name="model", tensors=None, decided=False):
    """Write a model folder; returns (folder, weights as float64 NumPy arrays by name).  `decided`: the routers'
    corrections lie 2 apart (scores lie in [0, 1]), so the SET of chosen experts is the same for every token and no
    rounding can change it, while the weights still follow the token: what a comparison in bfloat16 needs, where a
    close call between two experts would otherwise be decided differently by a rounded input."""
    import torch
    import qwen3_b200 as q
    config = q.config_from_dict(cfg)
    if tensors is None:
        tensors = lively_weights(q.build_model(config.plan()).weight_specs(), seed)
    if decided:
        gen = torch.Generator().manual_seed(seed + 1)
        for key in tensors:
            if key.endswith(".correction"):
                n = tensors[key].numel()
                tensors[key] = (2.0 * torch.randperm(n, generator=gen).float() - n).to(torch.bfloat16)
    folder = os.path.join(str(tmp_path), name)
    q.write_model_folder(folder, config, tensors)
    return folder, {k: v.to(torch.float64).numpy() for k, v in tensors.items()}


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]
