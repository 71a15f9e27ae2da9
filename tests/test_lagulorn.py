"""Lagulorn without a GPU: the configuration, the plan it makes, and the plain implementation against itself."""
import copy

import numpy as np
import pytest

from lagulorn_cases import CASES, case
from plain import lagulorn_plain as plain


@pytest.mark.parametrize("name", sorted(CASES))
def test_configuration_round_trip_and_plan(name):
    import qwen3_b200 as q
    cfg = case(name)
    config = q.config_from_dict(cfg)
    assert isinstance(config, q.LagulornConfig)
    assert q.config_from_dict(config.to_dict()) == config
    plan = config.plan()
    owners = [i for i, layer in enumerate(cfg["layers"]) if layer.get("weights_of") is None]
    assert len(plan.layers) == len(owners) and len(plan.order) == len(cfg["layers"])
    assert plan.streams == (cfg.get("streams") or 1) and plan.residual_dtype == "float32"
    # a layer with borrowed weights runs its owner's parts on a cache of its own
    for run, layer in enumerate(cfg["layers"]):
        owner = layer.get("weights_of")
        assert plan.order[run] == owners.index(run if owner is None else owner)
        assert (plan.caches[run] >= len(owners)) == (owner is not None)
    assert len(set(plan.caches)) == len(plan.caches)
    model = q.build_model(plan)
    names = set(model.weight_specs())
    assert {f"l{i}.norm1" for i in owners} <= names and "embed" in names and "final.norm" in names and "head" in names
    assert not any(n.startswith(f"l{i}.") for n in names for i in range(len(cfg["layers"])) if i not in owners)
    assert (f"l{owners[0]}.hc1.mix" in names) == ("streams" in cfg)
    # a layer without feed-forward reads no second norm; a file that holds one all the same still loads
    for i in owners:
        assert (f"l{i}.norm2" in model.ignorable_names()) == (cfg["layers"][i].get("mlp") is None)
        assert (f"l{i}.norm2" in names) == (cfg["layers"][i].get("mlp") is not None)
    needs = model.cache_needs()
    for run, layer in enumerate(cfg["layers"]):
        need, m = needs[plan.caches[run]], layer["mixer"]
        if layer["type"] == "lightning":
            assert need.kind == "none" and need.state_shape == (m["heads"], m["dim"], m["vdim"])
        else:
            assert need.kind == ("window" if m.get("mask") else "full") and need.window == (m.get("mask") or {}).get("size")
            assert need.num_kv_heads == 2 * m["kv_heads"] and need.value_heads in (None, m["kv_heads"])


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][4]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][4]["mlp"]["router"]["groups"].update(keep=1), "groups"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=0), "weights_of"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "kind"),
])
def test_configuration_faults_are_named(change, message):
    import qwen3_b200 as q
    cfg = case("A")
    change(cfg)
    with pytest.raises(q.ConfigError, match=message):
        q.config_from_dict(cfg)


def test_router_of_the_plain_implementation():
    # scores 0.4, 0.3, 0.2, 0.1 in two groups; the correction makes the second group win although its scores are smaller
    z = np.log(np.array([0.4, 0.3, 0.2, 0.1]))
    chosen, weights = plain.route(z, np.array([0.0, 0.0, 0.3, 0.0]), 2, 2, 1)
    assert list(chosen) == [2, 3] and np.allclose(weights, [0.2, 0.1])
    # negative choice scores: an expert outside the kept groups never wins, even against negative candidates
    chosen, _ = plain.route(z, np.array([-1.0, -2.0, -0.5, -0.95]), 2, 2, 1)
    assert list(chosen) == [2, 3]
    chosen, weights = plain.route(z, np.zeros(4), 3, 1, 1)
    assert list(chosen) == [0, 1, 2] and np.isclose(weights.sum(), 0.9)


def test_lightning_recurrence_equals_its_sum_form():
    """o_t = sum_(j <= t) decay^(t - j) (q_t . k_j) v_j: the recurrence of the plain implementation against the sum."""
    rng = np.random.default_rng(0)
    T, H, d, vd, width = 40, 2, 6, 5, 16
    m = {"heads": H, "dim": d, "vdim": vd, "decay": [0.8, 1.0]}
    w = {"q": rng.standard_normal((H * d, width)), "k": rng.standard_normal((H * d, width)), "v": rng.standard_normal((H * vd, width)),
         "g": rng.standard_normal((H * vd, width)), "o": np.eye(H * vd), "norm": np.ones(H * vd)}
    h = rng.standard_normal((T, width)) * 0.3
    got = plain.lightning_mixer(h, w, "", m, 1e-6)
    q, k, v = (plain.silu(h @ w[n].T) for n in "qkv")
    o = np.zeros((T, H * vd))
    for head in range(H):
        for t in range(T):
            for j in range(t + 1):
                o[t, head * vd:(head + 1) * vd] += m["decay"][head] ** (t - j) * (q[t, head * d:(head + 1) * d] @ k[j, head * d:(head + 1) * d]) \
                    * v[j, head * vd:(head + 1) * vd]
    want = plain.rms_unit(o, 1e-6) * plain.sigmoid(h @ w["g"].T)
    assert np.allclose(got, want, atol=1e-10)


def test_one_stream_with_unit_connections_is_the_plain_residual_sum():
    import qwen3_b200 as q
    from lagulorn_cases import lively_weights
    cfg = case("B")
    specs = q.build_model(q.config_from_dict(cfg).plan()).weight_specs()
    w = {k: v.double().numpy() for k, v in lively_weights(specs, 3).items()}
    toks = list(range(30))
    plain_sum = plain.forward(cfg, w, toks)
    one = dict(copy.deepcopy(cfg), streams=1, residual_mult=1.0)
    for i in range(len(cfg["layers"])):
        for c in ("hc1", "hc2"):
            w[f"l{i}.{c}.in"], w[f"l{i}.{c}.out"], w[f"l{i}.{c}.mix"] = np.ones(1), np.ones(1), np.ones((1, 1))
    assert np.allclose(plain.forward(one, w, toks), plain_sum, atol=1e-12)
