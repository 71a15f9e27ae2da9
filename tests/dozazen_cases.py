"""Shared by the Dozazen tests: small configurations that differ in every size and option, and model
folders with weights lively enough that attention is not uniform (matrices of unit gain, biases,
norm weights around 1), stored in bfloat16 so that the plain implementation reads the same values."""
import copy
import os

import numpy as np


def _mixer(heads, kv, dim, vdim, scale, rot=None, softcap=None, mask=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    if mask is not None:
        m["mask"] = {"size": mask}
    return m


# A stretch in the middle that runs three times; value heads of another size than key heads; a rotation over
# part of the head with all three cases of the frequency rescaling; chunks that are no multiple of a page; a
# layer without feed-forward; a layer without chunks and one without rotation; head sizes that are no multiple
# of 16; a feed-forward width that is no multiple of 8; an odd vocabulary.
Z_A = {
    "architecture": "Dozazen", "vocab": 211, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6},
    "logit_scale": 1.5, "logit_softcap": 9.0, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": _mixer(4, 2, 32, 16, 0.2, {"base": 10000.0, "dims": 16,
                                             "scaling": {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 64}}, 6.0, 40)},
        {"type": "attention", "mlp": None,
         "mixer": _mixer(2, 2, 16, 32, 0.3, {"base": 500.0, "dims": 16}, None, 70)},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 50},
         "mixer": _mixer(6, 1, 24, 24, 0.25, {"base": 1000.0, "dims": 8,
                                              "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}}, 30.0, None)},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 64}, "mixer": _mixer(3, 3, 32, 20, 0.18, None, 12.0, 64)},
    ],
}
# No stretch that repeats in one, a single pass in the other; chunks of one and of two pages; the whole head rotated;
# as many key/value heads as query heads; no scale on the embedding, no cap on the logits.
Z_B = {
    "architecture": "Dozazen", "vocab": 128, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 128},
         "mixer": _mixer(4, 4, 64, 64, 0.125, {"base": 50000.0, "dims": 64}, 50.0, 128)},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 128},
         "mixer": _mixer(2, 1, 64, 64, 0.125, {"base": 50000.0, "dims": 32,
                                               "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 128}}, 50.0, 64)},
    ],
}
Z_B1 = dict(copy.deepcopy(Z_B), loop={"start": 0, "stop": 1, "times": 1})
Z_B1["layers"][1]["mixer"].update(heads=34, kv_heads=1)      # more query heads per key/value head than a tensor-core tile has rows
# Sizes that the tensor-core kernels take (head sizes in steps of 16, widths in steps of 8), every layer twice.
Z_C = {
    "architecture": "Dozazen", "vocab": 320, "width": 128, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-5},
    "logit_scale": 2.5, "logit_softcap": 11.0, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 256},
         "mixer": _mixer(8, 2, 64, 32, 0.125, {"base": 100000.0, "dims": 32,
                                               "scaling": {"factor": 6.0, "low": 1.5, "high": 5.0, "original": 256}}, 17.0, 200)},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 256},
         "mixer": _mixer(4, 1, 32, 64, 0.2, {"base": 100000.0, "dims": 32}, 25.0, 104)},
    ],
}
# Sizes that rule out every vector path: a width that is no multiple of 4, odd head sizes and vocabulary, chunks of one
# position (a token sees itself and the sink) and of seven.
Z_D = {
    "architecture": "Dozazen", "vocab": 97, "width": 50, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
    "logit_scale": 3.0, "logit_softcap": 4.0, "loop": {"start": 1, "stop": 2, "times": 2},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 30},
         "mixer": _mixer(2, 1, 11, 7, 0.3, {"base": 50.0, "dims": 6}, 3.0, 7)},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 21}, "mixer": _mixer(5, 5, 6, 9, 0.4, {"base": 50.0, "dims": 6}, None, 1)},
    ],
}
CASES = {"A": Z_A, "B": Z_B, "B1": Z_B1, "C": Z_C, "D": Z_D}


def case(name, **changes):
    cfg = copy.deepcopy(CASES[name])
    cfg.update(changes)
    return cfg


def lively_weights(specs, seed):
    """{name: bfloat16 tensor}: matrices N(0, 1/fan_in), biases N(0, 0.5), norm weights 1 + N(0, 0.2), the
    embedding table N(0, 1)."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        spec = specs[name]
        draw = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        if spec.role == "norm":
            draw = 1.0 + 0.2 * draw
        elif spec.role == "bias":
            draw = 0.5 * draw
        elif name != "embed":
            draw = draw / (spec.shape[-1] ** 0.5)
        out[name] = draw.to(torch.bfloat16)
    return out


def make_folder(tmp_path, cfg, seed, name="model"):
    """Write a model folder; returns (folder, weights as float64 NumPy arrays by name)."""
    import torch
    import qwen3_b200 as q
    config = q.config_from_dict(cfg)
    tensors = lively_weights(q.build_model(config.plan()).weight_specs(), seed)
    folder = os.path.join(str(tmp_path), name)
    q.write_model_folder(folder, config, tensors)
    return folder, {k: v.to(torch.float64).numpy() for k, v in tensors.items()}


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]
