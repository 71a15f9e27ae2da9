"""Dozazen without a GPU: the configuration and its plan, the rotation's frequencies, the order of a head's
values for the kernels, and the cache book's chunk groups."""
import copy
import json

import numpy as np
import pytest

from dozazen_cases import CASES, case
from plain import dozazen_plain as plain


def test_config_round_trip_and_registry():
    import qwen3_b200 as q
    for name, cfg in CASES.items():
        config = q.config_from_dict(cfg)
        assert type(config).__name__ == "DozazenConfig"
        assert q.config_from_dict(json.loads(json.dumps(config.to_dict()))) == config
    assert "Dozazen" in q.known_architectures() and "Qwen3ForCausalLM" in q.known_architectures()


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "heads"),
    (lambda c: c["layers"][0]["mixer"].update(dim=258), "dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 9, "times": 2}), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].update(scale="big"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
])
def test_config_rejections(change, word):
    import qwen3_b200 as q
    cfg = case("A")
    change(cfg)
    with pytest.raises(q.ConfigError) as e:
        q.config_from_dict(cfg)
    assert word in str(e.value)


def test_plan_orders_runs_caches_and_steps():
    import qwen3_b200 as q
    plan = q.config_from_dict(case("A")).plan()
    assert plan.order == [0, 1, 2, 1, 2, 1, 2, 3]
    assert plan.caches == [0, 1, 2, 4, 5, 6, 7, 3]                      # every pass of the stretch has caches of its own
    assert [s.before_run for s in plan.stream_steps] == [1, 3, 5] and {s.name for s in plan.stream_steps} == {"loop.in"}
    assert plan.cache_owners() == [0, 1, 2, 3, 1, 2, 1, 2]
    assert [plan.order[run] for run in range(len(plan.order))] == [i for i, _ in plain.run_order(case("A"))]
    assert plan.layers[1].feed_forward is None and plan.residual_dtype == "float32" and plan.stop_token_ids == []
    plain_b = q.config_from_dict(case("B")).plan()
    assert plain_b.order == [0, 1] and plain_b.stream_steps == [] and plain_b.caches in (None, [0, 1])
    once = q.config_from_dict(case("B1")).plan()
    assert once.order == [0, 1] and [s.before_run for s in once.stream_steps] == [0]
    model = q.build_model(plan)
    needs = model.cache_needs()
    assert [(n.kind, n.window, n.num_kv_heads, n.head_dim, n.value_dim) for n in needs[:4]] == [
        ("chunk", 40, 2, 32, 16), ("chunk", 70, 2, 16, 32), ("full", None, 1, 24, None), ("chunk", 64, 3, 32, 20)]
    assert needs[4] == needs[1] and needs[5] == needs[2] and len(needs) == 8
    specs = model.weight_specs()
    assert specs["loop.in"].shape == (64, 128) and specs["l0.mix.q.b"].shape == (128,) and specs["l0.mix.v"].shape == (32, 64)
    assert specs["l2.mix.o"].shape == (64, 6 * 24) and "l1.mlp.gate" not in specs and "l1.norm2" not in specs
    assert specs["embed"].shape == (211, 64) and specs["head"].shape == (211, 64) and specs["final.norm"].shape == (64,)


def test_a_plan_refuses_caches_that_belong_to_another_layer():
    import dataclasses
    import qwen3_b200 as q
    plan = q.config_from_dict(case("A")).plan()
    with pytest.raises(ValueError):
        dataclasses.replace(plan, caches=[0, 1, 2, 2, 5, 6, 7, 3])
    with pytest.raises(ValueError):
        dataclasses.replace(plan, caches=[0, 1])


def test_rotary_frequencies_with_rescaling_and_the_kernel_order():
    from qwen3_b200.parts.position import RotaryEmbedding
    seen = set()
    for cfg in CASES.values():
        for layer in cfg["layers"]:
            rot = layer["mixer"].get("rot")
            if rot is None:
                continue
            part = RotaryEmbedding(layer["mixer"]["dim"], rot["base"], 1 << 20, rot["dims"], interleaved=True,
                                   scaling=rot.get("scaling"))
            want = plain.rotary_frequencies(rot)
            assert np.allclose(part.frequencies(), want, rtol=1e-12, atol=0)
            if rot.get("scaling"):
                plain_f = plain.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
                ratio = want / plain_f
                seen |= {"kept" if r == 1.0 else "divided" if abs(r - 1 / rot["scaling"]["factor"]) < 1e-12 else "blended" for r in ratio}
            order = part.kernel_order()
            d, r = layer["mixer"]["dim"], rot["dims"]
            assert sorted(order) == list(range(d)) and order[:r // 2] == list(range(0, r, 2)) and order[r:] == list(range(r, d))
    assert seen == {"kept", "divided", "blended"}
    assert RotaryEmbedding(16, 10000.0, 64).kernel_order() is None


def test_interleaved_rotation_equals_the_half_split_one_on_reordered_values():
    import torch
    from qwen3_b200.parts.position import RotaryEmbedding
    rot = {"base": 300.0, "dims": 12, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 20}}
    part = RotaryEmbedding(20, rot["base"], 512, rot["dims"], interleaved=True, scaling=rot["scaling"])
    part.prepare(300, "cpu")
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((7, 3, 20)), rng.standard_normal((7, 2, 20))
    pos = np.array([0, 1, 2, 63, 64, 200, 299])
    want_q, want_k = plain.rotate_interleaved(q, pos, rot), plain.rotate_interleaved(k, pos, rot)
    tq, tk = torch.tensor(q, dtype=torch.float32), torch.tensor(k, dtype=torch.float32)
    part.apply_(tq, tk, torch.tensor(pos))
    assert np.allclose(tq.numpy(), want_q, atol=2e-5) and np.allclose(tk.numpy(), want_k, atol=2e-5)
    order = part.kernel_order()
    rq, rk = torch.tensor(q[..., order], dtype=torch.float32), torch.tensor(k[..., order], dtype=torch.float32)
    part.apply_(rq, rk, torch.tensor(pos), kernel_order=True)
    assert np.allclose(rq.numpy(), want_q[..., order], atol=2e-5)
    # the dot products, which are all that attention reads, are those of the interleaved form
    assert np.allclose(np.einsum("thd,sgd->tshg", rq.numpy(), rk.numpy()), np.einsum("thd,sgd->tshg", want_q, want_k), atol=1e-4)


def test_chunk_groups_return_the_pages_of_finished_chunks():
    from qwen3_b200.cache import CacheBook, CacheNeed
    book = CacheBook([CacheNeed("chunk", 1, 16, window=80), CacheNeed("full", 1, 16), CacheNeed("chunk", 2, 16, window=64, value_dim=8)],
                     max_tokens=64 * 12, max_seq_len=64 * 8)
    assert len(book.groups) == 3
    s = book.alloc_slot()

    def held(g):
        return sum(1 for p in book.groups[g].table[s] if p >= 0)

    def step(n):
        book.reserve([(s, n)])
        book.commit([(s, n)])

    step(79)                    # positions 0..78: the first chunk of 80 is still open
    assert (held(0), held(1), held(2)) == (2, 2, 1)          # the chunks of 64: page 0 is finished
    step(1)                     # length 80: the next query opens chunk [80, 160), which starts inside page 1
    assert (held(0), held(1), held(2)) == (1, 2, 1)
    step(81)                    # length 161: chunk [160, 240) starts inside page 2
    assert (held(0), held(1), held(2)) == (1, 3, 1)
    step(200)                   # length 361: chunk [320, 400) starts at page 5; a portion that crossed chunks held all its pages
    assert (held(0), held(1), held(2)) == (1, 6, 1)
    other = book.alloc_slot()
    book.reserve([(other, 130)])                               # pages given back are handed out again
    book.commit([(other, 130)])
    assert book.groups[0].n_free == 12 - 1 - 2
    book.free_slot(s)
    book.free_slot(other)
    assert all(g.n_free == 12 for g in book.groups) and book.pages_held() == 0
