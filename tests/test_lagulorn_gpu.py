"""Lagulorn on the GPU against the plain implementation (tests/plain/lagulorn_plain.py): every mechanism alone,
then the engine under every way of cutting requests into steps, in 32-bit and in bfloat16."""
import os

import numpy as np
import pytest

import schedules
from lagulorn_cases import CASES, case, lively_weights, make_folder, random_tokens
from plain import lagulorn_plain as plain
from test_engine_gpu import run_steps

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
FP32_TOL = 3e-4


def torch_dtype(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def dev(a, dtype):
    import torch
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


# ============================================================================ mechanisms, one at a time
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams,hidden", [(1, 64), (2, 50), (3, 384), (8, 1024), (4, 4100), (16, 72)])
def test_streams_settle_sum_and_norm_in_one_pass(dtype, streams, hidden):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(streams * hidden)
    T, N = torch_dtype(dtype), 6
    x = rng.standard_normal((N, streams, hidden)) * 2
    y = dev(rng.standard_normal((N, hidden)), T)
    mix, out_c, in_c = rng.standard_normal((streams, streams)), rng.standard_normal(streams), rng.standard_normal(streams)
    w = dev(1 + 0.3 * rng.standard_normal(hidden), torch.float32)
    f32 = lambda a: dev(a, torch.float32)
    xd = f32(x).double().cpu().numpy()
    yd, wd = y.double().cpu().numpy(), w.double().cpu().numpy()
    mixd, outd, ind = (f32(a).double().cpu().numpy() for a in (mix, out_c, in_c))
    settled = np.einsum("ft,nfh->nth", mixd, xd) + outd[None, :, None] * yd[:, None, :]
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    # a norm of the weighted sum alone: the streams stay as they are
    s = f32(x).view(N, streams * hidden)
    got = torch.empty((N, hidden), dtype=T, device="cuda")
    ops.hyper_norm(s, streams, None, None, None, f32(in_c), w, 1e-5, got)
    u = np.tensordot(xd, ind, axes=(1, 0))
    assert np.allclose(got.double().cpu().numpy(), plain.rms_unit(u, 1e-5) * wd, **tol)
    assert np.array_equal(s.double().cpu().numpy().reshape(xd.shape), xd)
    # settle and read in one pass
    ops.hyper_norm(s, streams, y, f32(mix), f32(out_c), f32(in_c), w, 1e-5, got)
    assert np.allclose(s.double().cpu().numpy().reshape(xd.shape), settled, rtol=1e-5, atol=1e-5)
    u = np.tensordot(settled, ind, axes=(1, 0))
    assert np.allclose(got.double().cpu().numpy(), plain.rms_unit(u, 1e-5) * wd, **tol)
    # settle alone
    s2 = f32(x).view(N, streams * hidden)
    ops.hyper_norm(s2, streams, y, f32(mix), f32(out_c), None, None, 0.0, None)
    assert np.allclose(s2.double().cpu().numpy().reshape(xd.shape), settled, rtol=1e-5, atol=1e-5)
    # the tail: chosen rows, the plain sum of the streams, nothing written back; and the sum itself in 32-bit
    s3 = f32(x).view(N, streams * hidden)
    rows = torch.tensor([4, 0, 5], dtype=torch.int32, device="cuda")
    tail = torch.empty((3, hidden), dtype=T, device="cuda")
    ops.hyper_norm(s3, streams, y, f32(mix), f32(out_c), None, w, 1e-6, tail, rows=rows)
    total = settled.sum(axis=1)[[4, 0, 5]]
    assert np.allclose(tail.double().cpu().numpy(), plain.rms_unit(total, 1e-6) * wd, **tol)
    assert np.array_equal(s3.double().cpu().numpy().reshape(xd.shape), xd)
    sums = torch.empty((3, hidden), dtype=torch.float32, device="cuda")
    ops.hyper_norm(s3, streams, y, f32(mix), f32(out_c), None, None, 0.0, sums, rows=rows, normalize=False)
    assert np.allclose(sums.double().cpu().numpy(), total, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_fills_every_stream(dtype):
    import torch
    from qwen3_b200.csrc import ops
    table = dev(np.random.default_rng(1).standard_normal((37, 50)), torch_dtype(dtype))
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device="cuda")
    out = torch.empty((5, 3 * 50), dtype=torch.float32, device="cuda")
    ops.embedding_streams(ids, table, out, 2.5, 3)
    want = plain.embedding(table.double().cpu().numpy(), ids.cpu().numpy(), 2.5)
    assert np.allclose(out.cpu().numpy().reshape(5, 3, 50), want[:, None, :], rtol=1e-6, atol=0)


def plain_lightning(q, k, v, decay, state):
    """o [T, vd] and the state after the tokens, from silu-ed q, k [T, d], v [T, vd] and a state [d, vd] before them."""
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        state = decay * state + np.outer(k[t], v[t])
        out[t] = state.T @ q[t]
    return out, state


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,d,vd", [(3, 5, 9), (2, 16, 24), (1, 64, 128), (2, 128, 128), (1, 256, 64), (1, 256, 256), (2, 48, 96)])
def test_lightning_recurrence_token_by_token_and_in_chunks(dtype, heads, d, vd):
    """Both forms against the recurrence, over sequences of unequal length in slots in no particular order, continued in
    a second step from the state the first left: decays of 0, 1, nearly 1 and small; lengths around the chunk size."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(d * vd + heads)
    T = torch_dtype(dtype)
    decay = ([0.0, 1.0, 0.999, 0.3] * 2)[:heads] if heads > 1 else [0.97]
    first, second = [1, 31, 32, 33, 100, 64], [70, 1, 2, 40, 0, 33]
    slots = [4, 0, 5, 2, 7, 1]
    cols = 2 * heads * (d + vd)
    chunked_ok = ops.lightning_chunks_fit(d, vd)
    forms = [(False, False)] + ([(True, False)] if chunked_ok else [])
    if dtype == "bfloat16" and ops.lightning_chunks_tc_fit(d, vd):
        forms.append((True, True))                                # the chunks' products on the tensor cores
    for chunked, tensor_cores in forms:
        ops.lightning_tensor_cores = tensor_cores
        state = torch.zeros((9, heads, d, vd), dtype=torch.float32, device="cuda")
        state[3] = 7.0                                            # a slot no sequence uses
        want_state = {s: np.zeros((heads, d, vd)) for s in slots}
        for lengths in (first, second):
            live = [(s, n) for s, n in zip(slots, lengths) if n > 0]
            N = sum(n for _, n in live)
            proj = dev(rng.standard_normal((N, cols)) * 0.7, T)
            pd = proj.double().cpu().numpy()
            start = np.concatenate([[0], np.cumsum([n for _, n in live])]).astype(np.int32)
            out = torch.full((N, heads * vd), 9.0, dtype=torch.float32, device="cuda")
            ops.lightning_attention(proj, state, dev(decay, torch.float32), dev(start, torch.int32),
                                    dev([s for s, _ in live], torch.int32), out, len(live), heads, d, vd, chunked)
            got = out.double().cpu().numpy()
            for i, (slot, n) in enumerate(live):
                rows = pd[start[i]:start[i + 1]]
                for h in range(heads):
                    q = plain.silu(rows[:, h * d:(h + 1) * d])
                    k = plain.silu(rows[:, (heads + h) * d:(heads + h + 1) * d])
                    v = plain.silu(rows[:, 2 * heads * d + h * vd:2 * heads * d + (h + 1) * vd])
                    o, want_state[slot][h] = plain_lightning(q, k, v, decay[h], want_state[slot][h])
                    scale = max(1.0, float(np.abs(o).max()))
                    err = float(np.abs(got[start[i]:start[i + 1], h * vd:(h + 1) * vd] - o).max())
                    assert err <= 3e-5 * scale, (chunked, tensor_cores, slot, h, err, scale)
        final = state.double().cpu().numpy()
        for slot in slots:
            assert np.allclose(final[slot], want_state[slot], rtol=3e-5, atol=3e-5 * max(1.0, np.abs(want_state[slot]).max()))
        assert float((state[3] - 7.0).abs().max()) == 0.0 and float(state[6].abs().max()) == 0.0 and float(state[8].abs().max()) == 0.0
    ops.lightning_tensor_cores = True


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_unit_rms_over_all_heads(dtype):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(2)
    T, N, size = torch_dtype(dtype), 5, 72
    o = dev(rng.standard_normal((N, size)) * 30, torch.float32)
    proj = dev(rng.standard_normal((N, 200)), T)
    w = dev(1 + 0.2 * rng.standard_normal(size), torch.float32)
    out = torch.empty((N, size), dtype=T, device="cuda")
    ops.gated_norm(o, proj[:, 128:], w, 1e-5, out)
    want = plain.rms_unit(o.double().cpu().numpy(), 1e-5) * w.double().cpu().numpy() * plain.sigmoid(proj[:, 128:].double().cpu().numpy())
    assert np.allclose(out.double().cpu().numpy(), want, atol=1e-5 if dtype == "float32" else 2e-2)


class Paged:
    """Keys and values of a few sequences written into pages in no particular order through qkv_prepare."""

    def __init__(self, rng, lengths, nq, nkv, nv, d, vd, T, rows):
        import torch
        from qwen3_b200.csrc import ops
        self.lengths = lengths
        per_seq = max(-(-n // 64) for n in lengths)
        n_pages = per_seq * len(lengths) + 1
        self.table = dev(rng.permutation(n_pages - 1)[:per_seq * len(lengths)].reshape(len(lengths), per_seq), torch.int32)
        self.k_pages = torch.zeros((n_pages, nkv, 64, d), dtype=T, device="cuda")
        self.v_pages = torch.zeros((n_pages, nv, 64, vd), dtype=T, device="cuda")
        seq = np.concatenate([np.full(n, s) for s, n in enumerate(lengths)])
        pos = np.concatenate([np.arange(n) for n in lengths])
        q = torch.empty((len(seq), nq * d), dtype=T, device="cuda")
        ops.qkv_prepare(rows, q, self.k_pages, self.v_pages, None, None, None, None, dev(seq, torch.int32), dev(pos, torch.int32),
                        self.table, len(seq), nq, nkv, d, 0.0, value_dim=vd, value_heads=nv)
        self.q, self.seq, self.pos = q, seq, pos


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,nv,d,vd,window", [(8, 2, 1, 16, 8, 70), (4, 4, 2, 24, 40, 64), (6, 2, 2, 32, 32, 0), (4, 2, 1, 48, 80, 120),
                                                   (2, 2, 1, 11, 7, 1), (16, 4, 2, 64, 128, 200), (8, 2, 1, 16, 16, 70), (4, 4, 4, 32, 16, 1),
                                                   (2, 2, 2, 64, 64, 64)])
def test_windowed_attention_with_shared_values_and_keys_that_stand_out(dtype, nq, nkv, nv, d, vd, window):
    """Every query is made to point at ONE earlier key whose score then dominates: keys just inside and just outside the
    window, at page borders, the first tokens, and far back.  Inside, the output is that key's value; outside, it is not.
    Several key heads share a value head (`value_heads`); the output stays in 32-bit."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(nq * d + window)
    T = torch_dtype(dtype)
    lengths = [300, 65, 1, 200]
    N = sum(lengths)
    width = (nq + nkv) * d + nv * vd
    rows = rng.standard_normal((N, width)) * 0.3
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(lengths)])
    pos = np.concatenate([np.arange(n) for n in lengths])
    start = np.concatenate([[0], np.cumsum(lengths)])
    # query at position i of sequence 0 and 3 looks for the key at i - back(i)
    backs = [0, 1, 62, 63, 64, 65, 127, 128, 129, 190, 250]
    if window:
        backs += [window - 2, window - 1, window, window + 1]
    target = {}
    for s in (0, 3):
        for i in range(lengths[s]):
            back = backs[(i * 7 + s) % len(backs)]
            if back <= i:
                target[(s, i)] = i - back
    big = 6.0
    for (s, i), j in target.items():
        u = rng.standard_normal(d)
        u /= np.linalg.norm(u)
        for kh in range(nkv):
            rows[start[s] + j, (nq + kh) * d:(nq + kh + 1) * d] += big * u * (1 + 0.1 * kh)
        rows[start[s] + i, :nq * d] += np.tile(big * u, nq)
    rows_t = dev(rows, T)
    paged = Paged(rng, lengths, nq, nkv, nv, d, vd, T, rows_t)
    out = torch.full((N, nq * vd), 5.0, dtype=torch.float32, device="cuda")
    scale = 0.9
    ops.attention_generic(paged.q, paged.k_pages, paged.v_pages, out, dev(seq, torch.int32), dev(pos, torch.int32), paged.table, N,
                          nq, nkv, d, scale, window or None, value_dim=vd, value_heads=nv)
    got = out.double().cpu().numpy().reshape(N, nq, vd)
    rd = rows_t.double().cpu().numpy()
    worst = 0.0
    for s, n in enumerate(lengths):
        block = rd[start[s]:start[s + 1]]
        for h in range(nq):
            kh = h // (nq // nkv)
            vh = kh // (nkv // nv)
            want = plain.window_softmax_attention(block[:, h * d:(h + 1) * d], block[:, (nq + kh) * d:(nq + kh + 1) * d],
                                                  block[:, (nq + nkv) * d + vh * vd:(nq + nkv) * d + (vh + 1) * vd], scale, window or None)
            worst = max(worst, float(np.abs(got[start[s]:start[s + 1], h] - want).max()))
    assert worst <= (2e-5 if dtype == "float32" else 3e-2), worst
    wants = {}
    for s_, n in enumerate(lengths):
        block = rd[start[s_]:start[s_ + 1]]
        for h in range(nq):
            kh = h // (nq // nkv)
            vh = kh // (nkv // nv)
            wants[s_, h] = plain.window_softmax_attention(block[:, h * d:(h + 1) * d], block[:, (nq + kh) * d:(nq + kh + 1) * d],
                                                          block[:, (nq + nkv) * d + vh * vd:(nq + nkv) * d + (vh + 1) * vd], scale, window or None)
    if dtype == "bfloat16" and ops.attention_capped_fits(d, vd, window, nq // nkv):
        # the tiled tensor-core kernels: whole prompts, prompts continued from a cached prefix, and single tokens
        seq_start = dev(start, torch.int32)
        zeros = dev(np.zeros(len(lengths)), torch.int32)
        tiled = torch.full((N, nq * vd), 5.0, dtype=torch.float32, device="cuda")
        ops.attention_capped_prefill(paged.q, paged.k_pages, paged.v_pages, tiled, seq_start, zeros, paged.table, len(lengths),
                                     max(lengths), nq, nkv, d, vd, scale, window=window or None, value_heads=nv)
        got_t = tiled.double().cpu().numpy().reshape(N, nq, vd)
        for (s_, h), want in wants.items():
            assert float(np.abs(got_t[start[s_]:start[s_ + 1], h] - want).max()) <= 3e-2, ("prompt", s_, h)
        cut = [170, 64, 0, 1]                                   # tokens cached before the step
        keep = np.concatenate([np.arange(start[i] + cut[i], start[i + 1]) for i in range(len(lengths))])
        new_start = np.concatenate([[0], np.cumsum([lengths[i] - cut[i] for i in range(len(lengths))])])
        part = torch.full((len(keep), nq * vd), 5.0, dtype=torch.bfloat16, device="cuda")
        ops.attention_capped_prefill(paged.q[dev(keep, torch.int64)].contiguous(), paged.k_pages, paged.v_pages, part,
                                     dev(new_start, torch.int32), dev(cut, torch.int32), paged.table, len(lengths),
                                     max(lengths[i] - cut[i] for i in range(len(lengths))), nq, nkv, d, vd, scale,
                                     window=window or None, value_heads=nv)
        got_p = part.double().cpu().numpy().reshape(len(keep), nq, vd)
        assert float(np.abs(got_p - got_t[keep]).max()) <= 2e-2
        picks = [(0, p) for p in (0, 1, 63, 64, 65, 127, 128, 200, 299)] + [(1, 64), (2, 0), (3, 199), (3, 119), (3, 120), (3, 121)]
        if window > 1:
            picks += [(0, window - 1), (0, window), (0, window + 1)]
        rows_at = np.array([start[s_] + p for s_, p in picks])
        for splits in (1, 3, 16):
            one = torch.full((len(picks), nq * vd), 5.0, dtype=torch.float32, device="cuda")
            scratch = torch.full((len(picks) * nq * splits * (vd + 2),), float("nan"), dtype=torch.float32, device="cuda")
            ops.attention_capped_decode(paged.q[dev(rows_at, torch.int64)].contiguous(), paged.k_pages, paged.v_pages, one, scratch,
                                        dev([s_ for s_, _ in picks], torch.int32), dev([p for _, p in picks], torch.int32), paged.table,
                                        len(picks), nq, nkv, d, vd, scale, 0.0, None, False, splits, window=window or None, value_heads=nv)
            got_d = one.double().cpu().numpy().reshape(len(picks), nq, vd)
            for i, (s_, p) in enumerate(picks):
                for h in range(nq):
                    assert float(np.abs(got_d[i, h] - wants[s_, h][p]).max()) <= 3e-2, ("decode", splits, s_, p, h)
    # the test has teeth: with the window off by one in either direction the plain result moves by far more than that
    if window > 1:
        block = rd[:lengths[0]]
        exact = plain.window_softmax_attention(block[:, :d], block[:, nq * d:(nq + 1) * d], block[:, (nq + nkv) * d:(nq + nkv) * d + vd], scale, window)
        for other in (window - 1, window + 1):
            off = plain.window_softmax_attention(block[:, :d], block[:, nq * d:(nq + 1) * d], block[:, (nq + nkv) * d:(nq + nkv) * d + vd], scale, other)
            assert float(np.abs(off - exact).max()) > 0.2


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_maps_become_one_head(dtype):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(4)
    N, H, G, vd, lam, eps, diff = 7, 6, 2, 40, 0.83, 1e-5, 0.3
    r = H // G
    a = rng.standard_normal((N, G, 2, r, vd))
    out = torch.empty((N, H * vd), dtype=torch_dtype(dtype), device="cuda")
    ops.diff_combine(dev(a, torch.float32), out, N, H, r, vd, lam, eps, 1.0 - diff)
    ad = dev(a, torch.float32).double().cpu().numpy()
    want = plain.rms_unit(ad[:, :, 0] - lam * ad[:, :, 1], eps).reshape(N, H * vd) * (1.0 - diff)
    assert np.allclose(out.double().cpu().numpy(), want, atol=1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_plain_activations(dtype):
    import torch
    from qwen3_b200.csrc import ops
    x = dev(np.linspace(-6, 6, 1001), torch_dtype(dtype))
    xd = x.double().cpu().numpy()
    out = torch.empty_like(x)
    for kind, fn in (("gelu", plain.gelu_erf), ("silu", plain.silu)):
        ops.activation(x, out, kind)
        assert np.allclose(out.double().cpu().numpy(), fn(xd), atol=1e-6 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("outputs,real,top,groups,keep", [(12, 9, 2, 3, 1), (8, 5, 3, 4, 2), (6, 6, 2, 1, 1), (5, 4, 1, 5, 1), (5, 3, 5, 1, 1),
                                                          (64, 60, 8, 8, 3)])
def test_router_scores_groups_choice_and_weights(outputs, real, top, groups, keep):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(outputs * top)
    N, hidden = 50, 40
    h = dev(rng.standard_normal((N, hidden)), torch.float32)
    w = dev(rng.standard_normal((outputs, hidden)) * 0.5, torch.float32)
    corr = dev(rng.standard_normal(outputs) * 0.2 - 0.3, torch.float32)            # mostly negative choice scores
    ids = torch.empty(N * top, dtype=torch.int32, device="cuda")
    tw = torch.empty(N * top, dtype=torch.float32, device="cuda")
    idw = torch.empty(N, dtype=torch.float32, device="cuda")
    ops.moe_route(h, w, corr, ids, tw, idw, real, top, groups, keep)
    z = h.double().cpu().numpy() @ w.double().cpu().numpy().T
    ids, tw, idw = ids.cpu().numpy().reshape(N, top), tw.cpu().numpy().reshape(N, top), idw.cpu().numpy()
    for t in range(N):
        chosen, weights = plain.route(z[t], corr.double().cpu().numpy(), top, groups, keep)
        assert list(ids[t]) == list(chosen), (t, ids[t], chosen)
        assert np.allclose(tw[t], weights, rtol=1e-5, atol=1e-7)
        assert np.isclose(idw[t], sum(w_ for e, w_ in zip(chosen, weights) if e >= real), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,ff", [(72, 40), (96, 64)])
@pytest.mark.parametrize("N", [1, 7, 33, 300])
def test_routed_experts_against_the_plain_feed_forward(dtype, N, hidden, ff):
    """The whole part: few tokens (the small tiles of a decode step) and many (large tiles, experts with several tiles
    and experts with none), identity experts, groups; a width and an expert size that are no multiples of the tiles."""
    import torch
    from qwen3_b200.parts.moe import RoutedExperts
    from qwen3_b200.engine.context import Scratch
    rng = np.random.default_rng(N)
    T = torch_dtype(dtype)
    mlp = {"expert": {"ff": ff, "limit": 0.8}, "router": {"experts": 6, "identity": 2, "top": 3, "groups": {"count": 4, "keep": 3}}}
    part = RoutedExperts(hidden, ff, 6, 3, 0.8, identity=2, group_count=4, group_keep=3, prefix="mlp.")
    tensors = lively_weights(part.weight_specs(""), 5)
    part.bind({k: v.to(device="cuda", dtype=T if v.dim() == 2 else torch.float32) for k, v in tensors.items()}, "", T, "cuda")
    x = dev(rng.standard_normal((N, hidden)), T)

    class Ctx:
        n_tokens, dtype, scratch = N, T, Scratch("cuda")
    out = part.forward(x, Ctx)
    w = {k: v.double().numpy() for k, v in tensors.items()}
    want = plain.moe_ff(x.double().cpu().numpy(), w, "mlp.", mlp)
    err = np.abs(out.double().cpu().numpy() - want).max(axis=1)
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert float(np.mean(err > tol)) <= (0.0 if dtype == "float32" else 0.02), float(err.max())


# ============================================================================ the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("lagulorn")
    out = {}
    for i, name in enumerate(sorted(CASES)):
        out[name, "float32"] = make_folder(base, case(name), seed=23 + i, name=name)
        # bfloat16 runs use routers whose set of chosen experts no rounding can change (see make_folder)
        out[name, "bfloat16"] = make_folder(base, case(name), seed=23 + i, name=name + "_decided", decided=True)
    return out


def engine_for(folder, dtype, max_tokens, **kw):
    from qwen3_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def make_requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lengths)}


_exact = {}


def oracle(name, weights, toks):
    key = (name, id(weights), tuple(toks))
    if key not in _exact:
        cfg = case(name)
        exact = plain.forward(cfg, weights, toks)
        rounded = plain.forward(cfg, weights, toks, rnd=plain.round_bf16)
        scale = float(np.abs(exact).max())
        _exact[key] = (exact, 4.0 * float(np.max(np.abs(rounded - exact))) + 1e-6, scale)
    return _exact[key]


def check(got, requests, name, weights, dtype, label):
    for rid, toks in requests.items():
        exact, bf16_tol, scale = oracle(name, weights, toks)
        tol = FP32_TOL * max(1.0, scale) if dtype == "float32" else bf16_tol
        for p in range(len(toks)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            assert np.all(np.isfinite(row)), f"{label}: request {rid} position {p}: non-finite logits"
            err = float(np.max(np.abs(row - exact[p])))
            assert err <= tol, f"{label} [{dtype}] case {name}: request {rid} position {p} of {len(toks)}: {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name", sorted(CASES))
def test_sum_of_the_streams_after_every_layer_run(folders, name):
    """32-bit: the sum of the streams after each run of a layer (a layer with borrowed weights counts too)."""
    import torch
    from qwen3_b200 import StepEntry
    folder, weights = folders[name, "float32"]
    cfg = case(name)
    toks = random_tokens(np.random.default_rng(0), 150, cfg["vocab"])
    engine = engine_for(folder, "float32", 192)
    seen = []

    def after_run(run, residual, pending, ctx):
        x = residual.view(ctx.n_tokens, engine.plan.streams, -1).double()
        if pending is not None:
            x = torch.einsum("ft,nfh->nth", pending.mix.double(), x) + pending.out_coef.double()[None, :, None] * pending.branch.double()[:, None, :]
        seen.append(x.sum(1).cpu().numpy())
    engine.model.after_run = after_run
    slot = engine.new_sequence()
    engine.step([StepEntry(slot, toks, [0])])
    _, states = plain.forward(cfg, weights, toks, want_layers=True)
    assert len(seen) == len(states) == len(cfg["layers"])
    for run, (got, want) in enumerate(zip(seen, states)):
        err = float(np.max(np.abs(got - want)))
        assert err <= 2e-4 * max(1.0, float(np.max(np.abs(want)))), f"case {name}: after run {run}: {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [1, 2, 15, 16, 17, 69, 70, 71, 141, 300]), ("B", [63, 64, 65, 129, 260]),
                                          ("C", [31, 199, 201, 450]), ("D", [1, 8, 70, 150])])
def test_whole_requests(folders, name, lengths, dtype):
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=1)
    steps, rows = schedules.whole(requests)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, name, weights, dtype, "whole")
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,tail", [("A", [30, 100, 215], 160), ("B", [70, 200], 140), ("C", [230, 420], 210), ("D", [20, 90], 40)])
def test_prompt_then_token_by_token_across_window_edges(folders, name, lengths, tail, dtype):
    """The last `tail` tokens one a step, more than a window of them: the window passes over decoded tokens, the
    recurrent state is carried through a long decode (a request shorter than the tail goes token by token from its
    first token)."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=2)
    steps, rows = schedules.tail_one_by_one(requests, tail)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "tail one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,length,cuts", [
    ("A", 260, [2, 4, 31, 33, 69, 71, 80, 82, 120, 190, 258]), ("A", 150, list(range(2, 150, 2))),
    ("B", 200, [63, 65, 128, 130]), ("C", 420, [16, 199, 201, 203, 400]), ("D", 100, [3, 10, 12, 50])])
def test_prompts_fed_in_portions(folders, name, length, cuts, dtype):
    """Portions of many sizes, down to two tokens, that start and end at, before and after window, chunk and page edges."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), [length], seed=3)
    steps, rows = schedules.chunked(requests, {"r0": cuts})
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == length
    check(got, requests, name, weights, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,prompts,batch", [
    ("A", [13, 130, 9, 90, 66, 45, 128, 3], [5, 100, 1, 64, 65, 40, 39, 3], 3),
    ("B", [140, 70, 200, 66], [130, 1, 64, 63], 2),
    ("C", [300, 110, 9, 260, 210], [199, 104, 1, 201, 103], 3),
    ("D", [30, 7, 50], [8, 7, 1], 3),
])
def test_unequal_batches_one_after_another(folders, name, lengths, prompts, batch, dtype):
    """Requests of different lengths start together and are decoded together; the shorter ones end earlier; the next
    batch takes over their slots, pages and state rows.  Every row must be what the request gives alone."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=4)
    steps, rows = schedules.batched(requests, dict(zip(requests, prompts)), batch, want_all_prompt=True)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "batches")
    assert engine.cache.pages_held() == 0 and engine.cache.slots.n_free == engine.cache.n_slots
    again = run_steps(engine, steps, rows)                       # the same once more: other slots and pages, same rows
    worst = max(float(np.max(np.abs(got[k] - again[k]))) for k in got)
    assert worst <= (1e-5 if dtype == "float32" else 0.05) * max(1.0, oracle(name, weights, requests["r0"])[2]), worst


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_steps_of_portions_and_single_tokens(folders, dtype):
    folder, weights = folders["A", dtype]
    requests = make_requests(case("A"), [150, 90, 200], seed=5)
    steps, rows = schedules.mixed(requests, {"r0": 38, "r1": 41, "r2": 1}, {"r0": 1, "r1": 7, "r2": 33})
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name="A", weights=weights, dtype=dtype, label="mixed")


def test_window_groups_free_pages_while_decoding_and_a_reused_slot_starts_from_nothing(folders):
    """A long decode in a cache that holds the window only: the windowed layers give back the pages that fell out of
    the window, and a slot that is used again starts with a zero state."""
    from qwen3_b200 import StepEntry
    folder, weights = folders["B", "float32"]
    toks = random_tokens(np.random.default_rng(6), 330, 128)
    exact, _, scale = oracle("B", weights, toks)
    engine = engine_for(folder, "float32", 384, n_slots=1)
    for round_ in range(2):
        slot = engine.new_sequence()
        rows = [engine.step([StepEntry(slot, toks[:100], [99])])[0].cpu().numpy()]
        for p in range(100, 330):
            rows.append(engine.step([StepEntry(slot, [toks[p]], [0])])[0].cpu().numpy())
        assert max(len(g.held_pages(slot)) for g in engine.cache.groups) <= 2          # a window of 64 keys: two pages at most
        engine.release(slot)
        err = max(float(np.max(np.abs(r - exact[99 + i]))) for i, r in enumerate(rows))
        assert err <= FP32_TOL * max(1.0, scale), (round_, err)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(folders, name):
    import qwen3_b200 as q
    folder, weights = folders[name, "float32"]
    cfg = case(name)
    rng = np.random.default_rng(7)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 38, 1, 70)]
    engine = engine_for(folder, "float32", 64 * 8)
    got = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=12))
    for p, r in zip(prompts, got):
        assert r.token_ids == plain.generate_greedy(cfg, weights, p, 12) and r.stop_reason == q.MAX_NEW_TOKENS
    assert engine.cache.pages_held() == 0
    small = engine_for(folder, "float32", 64 * 4, n_slots=2)      # fewer slots than requests: one batch after another
    again = q.generate_token_ids(small, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=12))
    assert [r.token_ids for r in again] == [r.token_ids for r in got]


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_from_the_command_line(tmp_path, folders, dtype, monkeypatch):
    from test_trace_run_gpu import replay
    unpadded = schedules.peak_tokens
    monkeypatch.setattr(schedules, "peak_tokens", lambda steps, page=64: unpadded(steps, 1))
    folder, weights = folders["A", dtype]
    cfg = case("A")
    requests = make_requests(cfg, [75, 1, 130], seed=8)
    w_steps, w_rows = schedules.whole(requests)
    b_steps, b_rows = schedules.batched(requests, {"r0": 40, "r1": 1, "r2": 81}, 3)
    steps, rows = [], []
    for part_steps, part_rows in ((w_steps, w_rows), (b_steps, b_rows)):
        for s, r in zip(part_steps, part_rows):
            steps.append(dict(s, step=len(steps)))
            rows.append([(f"{len(steps)}:{rid}", rid, p) for rid, p in r])
    got = replay(folder, dtype, steps, [[(tag, p) for tag, _, p in r] for r in rows], str(tmp_path / "out"), cfg["vocab"])
    for r in rows:
        for tag, rid, p in r:
            exact, bf16_tol, scale = oracle("A", weights, requests[rid])
            err = float(np.max(np.abs(got[(tag, p)] - exact[p])))
            assert err <= (FP32_TOL * max(1.0, scale) if dtype == "float32" else bf16_tol), (tag, p, err)
