"""Dozazen on the GPU against the plain implementation (tests/plain/dozazen_plain.py): every mechanism alone,
then the engine under every way of cutting requests into steps, in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import schedules
from dozazen_cases import case, make_folder, random_tokens
from plain import dozazen_plain as plain
from test_engine_gpu import run_steps

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
FP32_TOL = 3e-4


def torch_dtype(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


# ============================================================================ mechanisms, one at a time
@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding(dtype):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(1)
    table = torch.tensor(rng.standard_normal((37, 50)), dtype=torch_dtype(dtype), device="cuda")
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device="cuda")
    out = torch.empty((5, 50), dtype=torch.float32, device="cuda")
    ops.embedding_scaled(ids, table, out, 2.5)
    want = plain.embedding(ids.cpu().numpy(), table.double().cpu().numpy(), 2.5)
    assert np.allclose(out.cpu().numpy(), want, rtol=1e-6, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [8, 50, 64, 1000, 1024, 4100, 8192, 9000])
def test_sandwich_norm_all_three_forms(dtype, size):
    """A norm of the stream; a branch normalised and added; both in one pass.  Sizes that take the register
    forms (1, 2, 4, 8 groups a thread) and the walking form (odd sizes, long rows)."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(size)
    rows, T = 5, torch_dtype(dtype)
    x = rng.standard_normal((rows, size)) * 3
    y = torch.tensor(rng.standard_normal((rows, size)) * 0.1, dtype=T, device="cuda")
    w1, w2 = 1 + 0.3 * rng.standard_normal(size), 1 + 0.3 * rng.standard_normal(size)
    w1t, w2t = (torch.tensor(w, dtype=torch.float32, device="cuda") for w in (w1, w2))
    w1, w2 = w1t.double().cpu().numpy(), w2t.double().cpu().numpy()
    yd = y.double().cpu().numpy()
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    # norm alone
    stream = torch.tensor(x, dtype=torch.float32, device="cuda")
    xd = stream.double().cpu().numpy()
    out = torch.empty((rows, size), dtype=T, device="cuda")
    ops.sandwich_norm(stream, None, None, 0.0, w2t, 1e-5, out)
    assert np.allclose(out.double().cpu().numpy(), plain.rms_norm(xd, w2, 1e-5), **tol)
    assert np.array_equal(stream.double().cpu().numpy(), xd)
    # sum alone
    ops.sandwich_norm(stream, y, w1t, 1e-6, None, 0.0, None)
    summed = xd + plain.rms_norm(yd, w1, 1e-6)
    assert np.allclose(stream.double().cpu().numpy(), summed, rtol=2e-6, atol=2e-6)
    # both
    stream = torch.tensor(x, dtype=torch.float32, device="cuda")
    ops.sandwich_norm(stream, y, w1t, 1e-6, w2t, 1e-5, out)
    assert np.allclose(stream.double().cpu().numpy(), summed, rtol=2e-6, atol=2e-6)
    assert np.allclose(out.double().cpu().numpy(), plain.rms_norm(summed, w2, 1e-5), **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_concat_cast_gathered_norm_and_capped_logits(dtype):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(3)
    T = torch_dtype(dtype)
    a = torch.tensor(rng.standard_normal((6, 20)), dtype=torch.float32, device="cuda")
    b = torch.tensor(rng.standard_normal((6, 20)), dtype=torch.float32, device="cuda")
    both = torch.empty((6, 40), dtype=T, device="cuda")
    ops.concat_cast(a, b, both)
    assert torch.equal(both, torch.cat([a, b], dim=1).to(T))
    w = torch.tensor(1 + 0.2 * rng.standard_normal(20), dtype=torch.float32, device="cuda")
    idx = torch.tensor([5, 0, 3], dtype=torch.int32, device="cuda")
    rows = torch.empty((3, 20), dtype=T, device="cuda")
    ops.gather_rows_norm(a, idx, w, 1e-5, rows)
    want = plain.rms_norm(a.double().cpu().numpy()[[5, 0, 3]], w.double().cpu().numpy(), 1e-5)
    assert np.allclose(rows.double().cpu().numpy(), want, atol=2e-5 if dtype == "float32" else 2e-2)
    z = torch.tensor(rng.standard_normal((4, 33)) * 20, dtype=torch.float32, device="cuda")
    zd = z.double().cpu().numpy()
    ops.scale_softcap(z, 1.5, 7.0)
    assert np.allclose(z.cpu().numpy(), plain.capped(zd * 1.5, 7.0), atol=1e-5)
    z2 = torch.tensor(zd, dtype=torch.float32, device="cuda")
    ops.scale_softcap(z2, 0.25, 0.0)
    assert np.allclose(z2.cpu().numpy(), zd * 0.25, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
def test_gelu_gating(dtype, interleaved):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(4)
    T = torch_dtype(dtype)
    g = torch.tensor(rng.standard_normal((7, 24)) * 3, dtype=T, device="cuda")
    u = torch.tensor(rng.standard_normal((7, 24)), dtype=T, device="cuda")
    if interleaved:
        gate_up = torch.stack([g.view(7, 3, 8), u.view(7, 3, 8)], dim=2).reshape(7, 48).contiguous()
    else:
        gate_up = torch.cat([g, u], dim=1).contiguous()
    out = torch.empty((7, 24), dtype=T, device="cuda")
    ops.silu_mul(gate_up, out, interleaved, "gelu_tanh")
    want = plain.gelu_tanh(g.double().cpu().numpy()) * u.double().cpu().numpy()
    assert np.allclose(out.double().cpu().numpy(), want, atol=1e-5 if dtype == "float32" else 3e-2, rtol=1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("rows", [3, 40, 300])
def test_gelu_gating_in_the_products_epilogues(rows):
    """The gate/up product with the activation in its epilogue, in its three forms (few rows, weights first, pairs of
    SMs), against the plain product: both sums rounded to bfloat16, then round(gelu(g)) * u."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(rows)
    K, inter = 128, 256
    x = torch.tensor(rng.standard_normal((rows, K)), dtype=torch.bfloat16, device="cuda")
    gate = torch.tensor(rng.standard_normal((inter, K)) / 8, dtype=torch.bfloat16, device="cuda")
    up = torch.tensor(rng.standard_normal((inter, K)) / 8, dtype=torch.bfloat16, device="cuda")
    w = ops.interleave_gate_up(gate, up)
    xd = x.double().cpu().numpy()
    g = plain.round_bf16(xd @ gate.double().cpu().numpy().T)
    u = plain.round_bf16(xd @ up.double().cpu().numpy().T)
    want = plain.round_bf16(plain.gelu_tanh(g)) * u
    out = torch.empty((rows, inter), dtype=torch.bfloat16, device="cuda")
    if rows <= 8:
        ops.gemm_skinny_gated(x, w, out, "gelu_tanh")
    elif rows <= 128:
        ops.gemm_tcgen05_mid_gated(x, w, out, activation="gelu_tanh")
    else:
        ops.gemm_tcgen05_pair(x, w, out, gated=True, activation="gelu_tanh")
    err = np.abs(out.double().cpu().numpy() - want)
    assert float(err.max()) <= 0.03 + 0.02 * float(np.abs(want).max()), float(err.max())
    silu = torch.empty_like(out)                                   # the default stays SiLU
    if rows <= 8:
        ops.gemm_skinny_gated(x, w, silu)
    elif rows <= 128:
        ops.gemm_tcgen05_mid_gated(x, w, silu)
    else:
        ops.gemm_tcgen05_pair(x, w, silu, gated=True)
    want_silu = plain.round_bf16(g / (1 + np.exp(-g))) * u
    assert float(np.abs(silu.double().cpu().numpy() - want_silu).max()) <= 0.03 + 0.02 * float(np.abs(want_silu).max())


# ---------------------------------------------------------------------------- attention over pages
class Paged:
    """Keys and values of a few sequences in pages that lie in no particular order, as the kernels read them."""

    def __init__(self, lengths, nkv, d, vd, dtype, seed, spikes=(), n_spare=3):
        import torch
        rng = np.random.default_rng(seed)
        self.lengths, self.nkv, self.d, self.vd = lengths, nkv, d, vd
        T = torch_dtype(dtype)
        pages_per_seq = max(-(-n // 64) for n in lengths)
        n_pages = sum(-(-n // 64) for n in lengths) + n_spare
        order = rng.permutation(n_pages)
        self.table = np.full((len(lengths), pages_per_seq), -1, dtype=np.int32)
        self.k, self.v = [], []
        k_pages = torch.zeros((n_pages, nkv, 64, d), dtype=T)
        v_pages = torch.zeros((n_pages, nkv, 64, vd), dtype=T)
        # what lies in unused cells must never be read: make it loud
        k_pages += 50.0
        v_pages += 1000.0
        at = 0
        self.direction = rng.standard_normal(d)
        self.direction /= np.linalg.norm(self.direction)
        for s, n in enumerate(lengths):
            k = rng.standard_normal((n, nkv, d)) * 0.5
            v = rng.standard_normal((n, nkv, vd))
            for j in spikes:
                if 0 <= j < n:
                    k[j] = self.direction * 12.0           # a key that every query looks at, if it may
            k = torch.tensor(k, dtype=T)
            v = torch.tensor(v, dtype=T)
            self.k.append(k.double().numpy())
            self.v.append(v.double().numpy())
            for pg in range(-(-n // 64)):
                page = int(order[at]); at += 1
                self.table[s, pg] = page
                lo, hi = pg * 64, min(n, pg * 64 + 64)
                k_pages[page, :, :hi - lo] = k[lo:hi].transpose(0, 1)
                v_pages[page, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        self.k_pages, self.v_pages = k_pages.cuda(), v_pages.cuda()

    def queries(self, tokens, nq, dtype, seed):
        """Queries for (sequence, position) pairs: the spike direction plus noise."""
        import torch
        rng = np.random.default_rng(seed)
        q = rng.standard_normal((len(tokens), nq, self.d)) * 0.3 + self.direction * 2.0
        return torch.tensor(q, dtype=torch_dtype(dtype))


def attention_cases():
    # (query heads, kv heads, d, vd, scale, softcap, chunk, sink)
    return [(4, 2, 32, 16, 0.3, 8.0, 40, True), (6, 1, 24, 20, 0.25, 0.0, 90, True), (2, 2, 64, 64, 0.125, 30.0, 64, True),
            (8, 2, 64, 32, 0.2, 15.0, 200, True), (3, 3, 16, 48, 0.5, 5.0, 0, True), (4, 1, 128, 128, 0.09, 20.0, 128, False),
            (4, 2, 128, 128, 0.09, 25.0, 100, True), (2, 1, 64, 64, 0.125, 0.0, 0, True), (2, 2, 64, 64, 0.125, 10.0, 72, False),
            (2, 1, 64, 64, 0.125, 5.0, 1, True), (3, 1, 11, 7, 0.3, 3.0, 7, True), (5, 5, 80, 48, 0.11, 12.0, 50, True),
            (12, 1, 32, 32, 0.18, 7.0, 130, True)]


def edge_positions(n, chunk):
    """Positions of a sequence where a fault would sit: the first tokens, both sides of every chunk and page edge, the end."""
    edges = {0, 1, 2, n - 1, n - 2}
    for step in (64, chunk or 64):
        for e in range(step, n + 1, step):
            edges |= {e - 2, e - 1, e, e + 1}
    return sorted(p for p in edges if 0 <= p < n)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,vd,scale,cap,chunk,sink", attention_cases())
def test_attention_over_pages_at_every_edge(dtype, nq, nkv, d, vd, scale, cap, chunk, sink):
    """Every query of three sequences at once (a prompt step), then single queries at the edges (decode steps), with
    keys that stand out placed just inside and just outside the chunks, at page borders, at the very start and far
    back: a key that is wrongly seen or wrongly missed moves the output by its whole value."""
    import torch
    from qwen3_b200.csrc import ops
    lengths = [300, 131, 64]
    c = chunk or 10 ** 9
    spikes = sorted({0, 1, 63, 64, 65, 127, 128, 129} | {e + o for e in range(0, 300, chunk or 64) for o in (-1, 0, 1)})
    paged = Paged(lengths, nkv, d, vd, dtype, seed=nq * 1000 + d, spikes=spikes)
    table = torch.tensor(paged.table, device="cuda")
    tol = 2e-5 if dtype == "float32" else 3e-2

    def run(tokens, seed):
        q = paged.queries(tokens, nq, dtype, seed)
        seq = torch.tensor([s for s, _ in tokens], dtype=torch.int32, device="cuda")
        pos = torch.tensor([p for _, p in tokens], dtype=torch.int32, device="cuda")
        out = torch.empty((len(tokens), nq * vd), dtype=torch_dtype(dtype), device="cuda")
        ops.attention_generic(q.cuda().view(len(tokens), nq * d).contiguous(), paged.k_pages, paged.v_pages, out, seq, pos, table,
                              len(tokens), nq, nkv, d, scale, None, value_dim=vd, softcap=cap, chunk=chunk or None, sink=sink)
        got = out.double().cpu().numpy().reshape(len(tokens), nq, vd)
        qd = q.double().numpy()
        for i, (s, p) in enumerate(tokens):
            n = p + 1
            if sink:
                want = plain.attend(qd[i:i + 1], paged.k[s][:n], paged.v[s][:n], [p], np.arange(n), scale, cap, chunk or None)[0]
            else:
                ok = plain.visible([p], np.arange(n), chunk or None)
                want = np.zeros((nq, vd))
                for h in range(nq):
                    sc = plain.capped(qd[i, h] @ paged.k[s][:n, h // (nq // nkv)].T * scale, cap)
                    e = np.where(ok[0], np.exp(sc - sc[ok[0]].max()), 0.0)
                    want[h] = (e / e.sum()) @ paged.v[s][:n, h // (nq // nkv)]
            assert np.allclose(got[i], want, atol=tol, rtol=tol), (s, p, float(np.abs(got[i] - want).max()))

    run([(s, p) for s, n in enumerate(lengths) for p in range(n)], seed=1)
    for s, n in enumerate(lengths):
        for p in edge_positions(n, chunk):
            run([(s, p)], seed=p)
    run([(s, p) for s, n in enumerate(lengths) for p in edge_positions(n, chunk)[-3:]], seed=9)       # unequal sequences, one token each


def plain_rows(paged, qd, tokens, nq, nkv, scale, cap, chunk, sink):
    out = []
    for i, (s, p) in enumerate(tokens):
        n = p + 1
        if sink:
            out.append(plain.attend(qd[i:i + 1], paged.k[s][:n], paged.v[s][:n], [p], np.arange(n), scale, cap, chunk or None)[0])
            continue
        ok = plain.visible([p], np.arange(n), chunk or None)
        want = np.zeros((nq, paged.vd))
        for h in range(nq):
            sc = plain.capped(qd[i, h] @ paged.k[s][:n, h // (nq // nkv)].T * scale, cap)
            e = np.where(ok[0], np.exp(sc - sc[ok[0]].max()), 0.0)
            want[h] = (e / e.sum()) @ paged.v[s][:n, h // (nq // nkv)]
        out.append(want)
    return np.stack(out)


@pytest.mark.parametrize("nq,nkv,d,vd,scale,cap,chunk,sink", [c for c in attention_cases() if c[2] % 16 == 0 and c[3] % 16 == 0])
def test_tensor_core_attention_over_pages_at_every_edge(nq, nkv, d, vd, scale, cap, chunk, sink):
    """The bfloat16 tensor-core kernels on the same data: prompts whole and continued from every kind of place,
    single tokens at the edges with one, three and sixteen key ranges."""
    import torch
    from qwen3_b200.csrc import ops
    lengths = [300, 131, 64]
    spikes = sorted({0, 1, 63, 64, 65, 127, 128, 129} | {e + o for e in range(0, 300, chunk or 64) for o in (-1, 0, 1)})
    paged = Paged(lengths, nkv, d, vd, "bfloat16", seed=nq * 1000 + d + 1, spikes=spikes)
    table = torch.tensor(paged.table, device="cuda")
    tol = 4e-2

    def compare(got, q, tokens, label):
        want = plain_rows(paged, q.double().numpy(), tokens, nq, nkv, scale, cap, chunk, sink)
        got = got.double().cpu().numpy().reshape(len(tokens), nq, vd)
        for i, key in enumerate(tokens):
            assert np.allclose(got[i], want[i], atol=tol, rtol=tol), (label, key, float(np.abs(got[i] - want[i]).max()))

    def prompt(starts):
        starts = [min(a, n - 1) for a, n in zip(starts, lengths)]
        tokens = [(s, p) for s, n in enumerate(lengths) for p in range(starts[s], n)]
        q = paged.queries(tokens, nq, "bfloat16", seed=sum(starts) + 1)
        counts = [n - a for n, a in zip(lengths, starts)]
        seq_start = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device="cuda")
        pos0 = torch.tensor(starts, dtype=torch.int32, device="cuda")
        out = torch.full((len(tokens), nq * vd), 7.0, dtype=torch.bfloat16, device="cuda")
        ops.attention_capped_prefill(q.cuda().view(len(tokens), nq * d).contiguous(), paged.k_pages, paged.v_pages, out, seq_start,
                                     pos0, table, len(lengths), max(counts), nq, nkv, d, vd, scale, cap, chunk or None, sink)
        compare(out, q, tokens, f"prompt from {starts}")
        if ops.attention_capped_prefill_tc_fits(d, vd, None):          # the same on tcgen05
            out.fill_(7.0)
            ops.attention_capped_prefill_tc(q.cuda().view(len(tokens), nq * d).contiguous(), paged.k_pages, paged.v_pages, out,
                                            seq_start, pos0, table, len(lengths), max(counts), len(tokens), nq, nkv, d, scale, cap,
                                            chunk or None, sink)
            assert ops.tcgen05_status(out.device) == 0
            compare(out, q, tokens, f"tcgen05 prompt from {starts}")

    prompt([0, 0, 0])
    c = chunk or 64
    prompt([c - 1, c + 1, 63])                # portions that start right before and right after an edge, and a single last token
    prompt([2 * c, 64, 1])
    prompt([130, 129, 62])

    def decode(tokens, splits):
        q = paged.queries(tokens, nq, "bfloat16", seed=len(tokens) * 7 + splits)
        seq = torch.tensor([s for s, _ in tokens], dtype=torch.int32, device="cuda")
        pos = torch.tensor([p for _, p in tokens], dtype=torch.int32, device="cuda")
        out = torch.full((len(tokens), nq * vd), 7.0, dtype=torch.bfloat16, device="cuda")
        scratch = torch.full((len(tokens) * nq * splits * (vd + 2),), float("nan"), dtype=torch.float32, device="cuda")
        ops.attention_capped_decode(q.cuda().view(len(tokens), nq * d).contiguous(), paged.k_pages, paged.v_pages, out, scratch, seq,
                                    pos, table, len(tokens), nq, nkv, d, vd, scale, cap, chunk or None, sink, splits)
        compare(out, q, tokens, f"decode with {splits} ranges")

    everything = [(s, p) for s, n in enumerate(lengths) for p in edge_positions(n, chunk)]
    for splits in (1, 3, 16):
        decode(everything, splits)
    decode([(0, 299)], 2)
    decode([(2, 0), (1, 130), (0, 64)], 5)


@pytest.mark.parametrize("nq,nkv,d,vd,rot,chunk", [(8, 2, 64, 32, 32, 200), (4, 4, 16, 48, 16, 40), (6, 1, 128, 128, 64, 0)])
def test_decode_attention_that_prepares_its_own_rows(nq, nkv, d, vd, rot, chunk):
    """The decode attention in its fused form (bias, rotation and cache write inside) against the same step done by
    qkv_prepare and the unfused kernel: the same outputs and the same cache, at positions on both sides of chunk and
    page edges, first tokens included."""
    import torch
    from qwen3_b200.csrc import ops
    from qwen3_b200.parts.position import RotaryEmbedding
    rng = np.random.default_rng(d + vd)
    part = RotaryEmbedding(d, 10000.0, 1024, rot)
    part.prepare(512, "cuda")
    lengths = [0, 1, 63, 64, 65, (chunk or 100) - 1, chunk or 100, (chunk or 100) + 1, 300, 191, 192]     # tokens cached before the step
    n = len(lengths)
    pages_per_seq = 5
    n_pages = n * pages_per_seq + 1
    table = torch.tensor(rng.permutation(n_pages - 1)[:n * pages_per_seq].reshape(n, pages_per_seq), dtype=torch.int32, device="cuda")
    base_k = torch.tensor(rng.standard_normal((n_pages, nkv, 64, d)) * 0.5, dtype=torch.bfloat16, device="cuda")
    base_v = torch.tensor(rng.standard_normal((n_pages, nkv, 64, vd)), dtype=torch.bfloat16, device="cuda")
    width = (nq + nkv) * d + nkv * vd
    qkv = torch.tensor(rng.standard_normal((n, width)), dtype=torch.bfloat16, device="cuda")
    bias = torch.tensor(rng.standard_normal(width) * 0.5, dtype=torch.float32, device="cuda")
    seq = torch.arange(n, dtype=torch.int32, device="cuda")
    pos = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    # unfused: prepare, then attend
    k1, v1 = base_k.clone(), base_v.clone()
    q = torch.empty((n, nq * d), dtype=torch.bfloat16, device="cuda")
    ops.qkv_prepare(qkv, q, k1, v1, None, None, part.cos, part.sin, seq, pos, table, n, nq, nkv, d, 0.0, bias=bias, value_dim=vd)
    want = torch.empty((n, nq * vd), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(n * nq * 16 * (vd + 2), dtype=torch.float32, device="cuda")
    ops.attention_capped_decode(q, k1, v1, want, scratch, seq, pos, table, n, nq, nkv, d, vd, 0.2, 9.0, chunk or None, True, 3)
    for splits in (1, 3, 16):
        k2, v2 = base_k.clone(), base_v.clone()
        got = torch.full((n, nq * vd), 7.0, dtype=torch.bfloat16, device="cuda")
        scratch.fill_(float("nan"))
        ops.attention_capped_decode_fused(qkv, k2, v2, got, scratch, bias, part.cos, part.sin, seq, pos, table, n, nq, nkv, d, vd,
                                          0.2, 9.0, chunk or None, True, splits)
        assert torch.equal(k1, k2) and torch.equal(v1, v2), splits
        err = float((got.float() - want.float()).abs().max())
        assert err <= 2e-2, (splits, err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_projection_rows_get_bias_rotation_and_their_place_in_the_pages(dtype):
    """qkv_prepare with a bias, values of another size than keys and a rotation over part of the head."""
    import torch
    from qwen3_b200.csrc import ops
    from qwen3_b200.parts.position import RotaryEmbedding
    rng = np.random.default_rng(5)
    T = torch_dtype(dtype)
    nq, nkv, d, vd, n = 3, 2, 24, 40, 70
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 3.0, "low": 1.0, "high": 2.0, "original": 16}}
    part = RotaryEmbedding(d, rot["base"], 256, rot["dims"], interleaved=True, scaling=rot["scaling"])
    part.prepare(128, "cuda")
    order = part.kernel_order()
    width = (nq + nkv) * d + nkv * vd
    rows = torch.tensor(rng.standard_normal((n, width)), dtype=T)
    bias = torch.tensor(rng.standard_normal(width) * 0.5, dtype=T).float()
    # the kernel sees heads whose values are already in its own order
    perm = np.concatenate([h * d + np.array(order) for h in range(nq + nkv)] + [np.arange((nq + nkv) * d, width)])
    q_out = torch.empty((n, nq * d), dtype=T, device="cuda")
    k_pages = torch.zeros((3, nkv, 64, d), dtype=T, device="cuda")
    v_pages = torch.zeros((3, nkv, 64, vd), dtype=T, device="cuda")
    table = torch.tensor([[2, 0]], dtype=torch.int32, device="cuda")
    pos0 = 50                                                 # the rows continue a sequence and cross a page border
    seq = torch.zeros(n, dtype=torch.int32, device="cuda")
    pos = torch.arange(pos0, pos0 + n, dtype=torch.int32, device="cuda")
    ops.qkv_prepare(rows[:, perm].contiguous().cuda(), q_out, k_pages, v_pages, None, None, part.cos, part.sin, seq, pos, table,
                    n, nq, nkv, d, 0.0, bias=bias[perm].contiguous().cuda(), value_dim=vd)
    full = rows.double().numpy() + bias.double().numpy()
    if dtype == "bfloat16":
        full = plain.round_bf16(full)
    positions = np.arange(pos0, pos0 + n)
    want_q = plain.rotate_interleaved(full[:, :nq * d].reshape(n, nq, d), positions, rot)[..., order]
    want_k = plain.rotate_interleaved(full[:, nq * d:(nq + nkv) * d].reshape(n, nkv, d), positions, rot)[..., order]
    want_v = full[:, (nq + nkv) * d:].reshape(n, nkv, vd)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert np.allclose(q_out.double().cpu().numpy().reshape(n, nq, d), want_q, atol=tol)
    k_got = torch.cat([k_pages[2, :, 50:], k_pages[0, :, :pos0 + n - 64]], dim=1).transpose(0, 1).double().cpu().numpy()
    v_got = torch.cat([v_pages[2, :, 50:], v_pages[0, :, :pos0 + n - 64]], dim=1).transpose(0, 1).double().cpu().numpy()
    assert np.allclose(k_got, want_k, atol=tol) and np.allclose(v_got, want_v, atol=tol)
    assert float(k_pages[1].abs().max()) == 0.0 and float(k_pages[2, :, :50].abs().max()) == 0.0     # nothing else was written


# ============================================================================ the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("dozazen")
    return {name: make_folder(base, case(name), seed=17 + i, name=name) for i, name in enumerate(["A", "B", "B1", "C", "D"])}


def engine_for(folder, dtype, max_tokens, **kw):
    from qwen3_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def make_requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lengths)}


_exact = {}


def oracle(name, weights, toks):
    key = (name, tuple(toks))
    if key not in _exact:
        cfg = case(name)
        exact = plain.forward(cfg, weights, toks)
        rounded = plain.forward(cfg, weights, toks, rnd=plain.round_bf16)
        _exact[key] = (exact, 4.0 * float(np.max(np.abs(rounded - exact))) + 1e-6)
    return _exact[key]


def check(got, requests, name, weights, dtype, label):
    for rid, toks in requests.items():
        exact, bf16_tol = oracle(name, weights, toks)
        tol = FP32_TOL if dtype == "float32" else bf16_tol
        for p in range(len(toks)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            assert np.all(np.isfinite(row)), f"{label}: request {rid} position {p}: non-finite logits"
            err = float(np.max(np.abs(row - exact[p])))
            assert err <= tol, f"{label} [{dtype}] case {name}: request {rid} position {p} of {len(toks)}: {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name", ["A", "B", "B1", "C", "D"])
def test_hidden_state_after_every_layer_run(folders, name):
    """32-bit: the stream after each run of a layer (a repeated layer counts each time) against the plain model."""
    import torch
    from qwen3_b200 import StepEntry
    from qwen3_b200.parts.block import settle
    folder, weights = folders[name]
    cfg = case(name)
    toks = random_tokens(np.random.default_rng(0), 150, cfg["vocab"])
    engine = engine_for(folder, "float32", 192)
    seen = []
    for block in engine.model.blocks:
        def forward(residual, delta, ctx, cache, inner=block.forward):
            residual, delta = inner(residual, delta, ctx, cache)
            settle(residual, delta)
            seen.append(residual.clone())
            return residual, None
        block.forward = forward
    slot = engine.new_sequence()
    engine.step([StepEntry(slot, toks, [0])])
    states = []
    plain.forward(cfg, weights, toks, states=states)
    assert len(seen) == len(states) == len(plain.run_order(cfg))
    for run, (got, want) in enumerate(zip(seen, states)):
        err = float(np.max(np.abs(got.double().cpu().numpy() - want)))
        assert err <= 2e-4 * max(1.0, float(np.max(np.abs(want)))), f"case {name}: after run {run}: {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [1, 2, 39, 40, 41, 141, 300]), ("B", [63, 64, 65, 129, 260]),
                                          ("B1", [5, 200]), ("C", [104, 105, 201, 450]), ("D", [1, 8, 70, 150])])
def test_whole_requests(folders, name, lengths, dtype):
    folder, weights = folders[name]
    requests = make_requests(case(name), lengths, seed=1)
    steps, rows = schedules.whole(requests)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, name, weights, dtype, "whole")
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,tail", [("A", [30, 100, 215], 90), ("B", [70, 200], 70), ("C", [230, 420], 100), ("D", [20, 90], 40)])
def test_prompt_then_token_by_token_across_chunk_edges(folders, name, lengths, tail, dtype):
    """The last `tail` tokens one a step: decoding passes over chunk and page edges (a request shorter than the
    tail goes token by token from its first token)."""
    folder, weights = folders[name]
    requests = make_requests(case(name), lengths, seed=2)
    steps, rows = schedules.tail_one_by_one(requests, tail)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "tail one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,length,cuts", [
    ("A", 260, [2, 4, 39, 41, 80, 82, 120, 190, 258]), ("A", 150, list(range(2, 150, 2))),
    ("B", 200, [63, 65, 128, 130]), ("C", 420, [103, 105, 199, 201, 203, 400])])
def test_prompts_fed_in_portions(folders, name, length, cuts, dtype):
    """Portions of many sizes, down to two tokens, that start and end at, before and after chunk and page edges."""
    folder, weights = folders[name]
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
])
def test_unequal_batches_one_after_another(folders, name, lengths, prompts, batch, dtype):
    """Requests of different lengths start together and are decoded together; the shorter ones end earlier; the
    next batch takes over their slots and pages.  Every row must be what the request gives alone."""
    folder, weights = folders[name]
    requests = make_requests(case(name), lengths, seed=4)
    steps, rows = schedules.batched(requests, dict(zip(requests, prompts)), batch, want_all_prompt=True)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "batches")
    assert engine.cache.pages_held() == 0 and engine.cache.slots.n_free == engine.cache.n_slots
    again = run_steps(engine, steps, rows)                       # the same once more: other slots and pages, same rows
    worst = max(float(np.max(np.abs(got[k] - again[k]))) for k in got)
    assert worst <= (1e-5 if dtype == "float32" else 0.05), worst


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_steps_of_portions_and_single_tokens(folders, dtype):
    folder, weights = folders["A"]
    requests = make_requests(case("A"), [150, 90, 200], seed=5)
    steps, rows = schedules.mixed(requests, {"r0": 38, "r1": 41, "r2": 1}, {"r0": 1, "r1": 7, "r2": 33})
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name="A", weights=weights, dtype=dtype, label="mixed")


def test_chunk_groups_free_pages_while_decoding_and_results_do_not_depend_on_the_pages(folders):
    """A long decode in a cache too small to hold the whole sequence in every group: the chunked layers give the
    pages of finished chunks back, so a cache sized for the layer without chunks is enough, and a slot that is
    used again starts from nothing."""
    from qwen3_b200 import StepEntry
    folder, weights = folders["B"]
    toks = random_tokens(np.random.default_rng(6), 330, 128)
    exact, _ = oracle("B", weights, toks)
    engine = engine_for(folder, "float32", 384)
    for round_ in range(2):
        slot = engine.new_sequence()
        rows = [engine.step([StepEntry(slot, toks[:100], [99])])[0].cpu().numpy()]
        for p in range(100, 330):
            rows.append(engine.step([StepEntry(slot, [toks[p]], [0])])[0].cpu().numpy())
        held = {g.need.window: len(g.held_pages(slot)) for g in engine.cache.groups}
        assert held == {128: 2, 64: 1}, held                 # length 330: chunk [256, 384) holds pages 4 and 5, chunk [320, 384) page 5
        engine.release(slot)
        err = max(float(np.max(np.abs(r - exact[99 + i]))) for i, r in enumerate(rows))
        assert err <= FP32_TOL, (round_, err)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(folders, name):
    import qwen3_b200 as q
    folder, weights = folders[name]
    cfg = case(name)
    rng = np.random.default_rng(7)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 38, 1, 70)]
    engine = engine_for(folder, "float32", 64 * 8)
    got = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=12))
    for p, r in zip(prompts, got):
        assert r.token_ids == plain.generate_greedy(cfg, weights, p, 12) and r.stop_reason == q.MAX_NEW_TOKENS
    assert engine.cache.pages_held() == 0
    # fewer slots than requests: one batch after another
    small = engine_for(folder, "float32", 64 * 4, n_slots=2)
    again = q.generate_token_ids(small, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=12))
    assert [r.token_ids for r in again] == [r.token_ids for r in got]


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_from_the_command_line(tmp_path, folders, dtype, monkeypatch):
    from test_trace_run_gpu import replay
    # --max-tokens counts the tokens of the live requests without the padding of their last pages
    unpadded = schedules.peak_tokens
    monkeypatch.setattr(schedules, "peak_tokens", lambda steps, page=64: unpadded(steps, 1))
    folder, weights = folders["A"]
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
            exact, bf16_tol = oracle("A", weights, requests[rid])
            err = float(np.max(np.abs(got[(tag, p)] - exact[p])))
            assert err <= (FP32_TOL if dtype == "float32" else bf16_tol), (tag, p, err)


def test_the_command_line_generates_from_token_ids(folders):
    """bin/qwen3_chat on a Dozazen folder: the model class comes from config.json, the design has no stop tokens of its own."""
    folder, weights = folders["A"]
    cfg = case("A")
    prompts = [[7, 8, 9], [100, 3]]
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_chat"), folder, "--greedy", "--dtype", "float32",
                          "--max-new-tokens", "6", "--max-context", "64", "--tokens", "7,8,9", "--tokens", "100 3"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.strip().splitlines() if l and l[0].isdigit()]
    assert len(lines) == 2
    for p, line in zip(prompts, lines):
        assert [int(t) for t in line.split("#")[0].strip().split(",")] == plain.generate_greedy(cfg, weights, p, 6)
