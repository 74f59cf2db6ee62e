"""Parity of the tcgen05 forward kernel and the tcgen05 projection with the oracle."""

import math

import pytest
import torch

import oracle
import probjax_b200 as pj
from _gpu_util import assert_close, cases, dev, load_golden, oracle_fwd, randn

pytestmark = pytest.mark.gpu
TC = "b200:tcgen05"


def _run(q, k, v, impl=TC, **kw):
    d = dev()
    args = {n: (t.to(d) if isinstance(t, torch.Tensor) else t) for n, t in kw.items()}
    out, lse = pj.attention_forward(q.to(d), k.to(d), v.to(d), return_lse=True, impl=impl, **args)
    pj.check_status(d)  # a timed-out wait inside the kernel raises here
    return out, lse


def test_one_tile_identity_values():
    """Smallest case: one 128x128 tile, V = identity-like, so O = P and every row of
    O sums to 1; catches descriptor / layout mistakes before the real cases."""
    q, k = randn((1, 128, 1, 128), torch.bfloat16, 1), randn((1, 128, 1, 128), torch.bfloat16, 2)
    v = torch.eye(128, dtype=torch.bfloat16).reshape(1, 128, 1, 128)
    sc = 1 / math.sqrt(128)
    out, lse = _run(q, k, v, sm_scale=sc)
    want, want_lse = oracle_fwd(q, k, v, sm_scale=sc)
    assert_close(out, lse, want, want_lse, torch.bfloat16, "identity V")
    assert torch.allclose(out.float().sum(-1).cpu(), torch.ones(1, 128, 1), atol=2e-2)


@pytest.mark.parametrize("name", ["c2_small", "c2_small_causal", "c3_small"])
def test_golden(name):
    inp = cases.make_inputs(name)
    kw = {n: inp[n] for n in ("causal", "sm_scale", "kv_lengths", "bias") if n in inp}
    out, lse = _run(inp["q"], inp["k"], inp["v"], **kw)
    want, want_lse = load_golden(name)
    assert_close(out, lse, want, want_lse, inp["q"].dtype, name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize(
    "b,lq,lkv,hq,hkv,d,dv,causal",
    [
        (1, 256, 256, 1, 1, 128, 128, False),
        (2, 512, 512, 4, 2, 128, 128, True),
        (1, 200, 333, 2, 1, 128, 128, False),   # ragged: tails on both axes
        (1, 333, 200, 2, 2, 128, 128, True),    # more queries than keys, causal
        (2, 100, 1000, 4, 4, 64, 64, False),
        (1, 640, 640, 2, 1, 64, 64, True),
        (1, 1, 300, 2, 2, 128, 128, False),     # a single query row
        (1, 300, 300, 2, 2, 192, 128, True),    # latent-attention head shape
        (1, 130, 70, 3, 1, 192, 128, False),
    ],
)
def test_shapes(dtype, b, lq, lkv, hq, hkv, d, dv, causal):
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, dv), dtype, 3)
    sc = 1 / math.sqrt(d)
    out, lse = _run(q, k, v, causal=causal, sm_scale=sc)
    want, want_lse = oracle_fwd(q, k, v, causal=causal, sm_scale=sc)
    assert_close(out, lse, want, want_lse, dtype, f"{(b, lq, lkv, hq, hkv, d, dv, causal)}")


@pytest.mark.parametrize("bshape", [(1, 4), (2, 4), (1, 1)])
@pytest.mark.parametrize("lkv", [384, 331])  # 331: the bias rows are not 16-byte aligned
def test_key_lengths_and_bias(bshape, lkv):
    b, lq, h, d = 2, 300, 4, 64
    q, k, v = randn((b, lq, h, d), torch.bfloat16, 4), randn((b, lkv, h, d), torch.bfloat16, 5), randn((b, lkv, h, d), torch.bfloat16, 6)
    bias = randn((*bshape, lq, lkv), torch.float32, 7)
    lens = torch.tensor([77, lkv], dtype=torch.int32)
    for causal in (False, True):
        out, lse = _run(q, k, v, causal=causal, kv_lengths=lens, bias=bias, sm_scale=0.125)
        want, want_lse = oracle_fwd(q, k, v, causal=causal, kv_lengths=lens, bias=bias, sm_scale=0.125)
        assert_close(out, lse, want, want_lse, torch.bfloat16, f"bias{bshape} lkv={lkv} causal={causal}")


def test_zero_length_batch_rows():
    q, k, v = randn((3, 140, 2, 128), torch.bfloat16, 1), randn((3, 256, 2, 128), torch.bfloat16, 2), randn((3, 256, 2, 128), torch.bfloat16, 3)
    lens = torch.tensor([0, 256, 5], dtype=torch.int32)
    out, lse = _run(q, k, v, kv_lengths=lens, sm_scale=0.1)
    assert (out[0] == 0).all() and torch.isinf(lse[0]).all() and (lse[0] > 0).all()
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=0.1)
    assert_close(out, lse, want, want_lse, torch.bfloat16, "zero length")


def test_large_scores_do_not_overflow():
    # scores spread over hundreds of units: the running maximum must keep up
    q, k, v = randn((1, 256, 1, 128), torch.bfloat16, 1) * 6, randn((1, 512, 1, 128), torch.bfloat16, 2) * 6, randn((1, 512, 1, 128), torch.bfloat16, 3)
    out, lse = _run(q, k, v, sm_scale=1.0)
    want, want_lse = oracle_fwd(q, k, v, sm_scale=1.0)
    assert_close(out, None, want, None, torch.bfloat16, "large scores")
    assert float(((lse.cpu() - want_lse) / want_lse.abs().clamp_min(1)).abs().max()) < 1e-3


def test_repeatable_bit_for_bit_and_equal_to_generic():
    q, k, v = randn((2, 512, 4, 128), torch.bfloat16, 1), randn((2, 512, 2, 128), torch.bfloat16, 2), randn((2, 512, 2, 128), torch.bfloat16, 3)
    a, la = _run(q, k, v, causal=True, sm_scale=0.09)
    b, lb = _run(q, k, v, causal=True, sm_scale=0.09)
    assert torch.equal(a, b) and torch.equal(la, lb)
    g, lg = _run(q, k, v, impl="b200:generic", causal=True, sm_scale=0.09)
    assert float((a.float() - g.float()).abs().max()) <= 2e-2
    assert float((la - lg).abs().max()) <= 1e-3


def test_auto_dispatch_picks_the_kernel_by_shape():
    from probjax_b200 import _lib

    d = dev()
    q = randn((1, 128, 2, 128), torch.bfloat16, 1).to(d)
    n0 = _lib.launch_count()
    pj.attention_forward(q, q, q, sm_scale=0.1)
    assert _lib.launch_count() == n0 + 1
    with pytest.raises(NotImplementedError, match="tcgen05"):
        pj.attention_forward(q.float(), q.float(), q.float(), impl=TC)
    q24 = randn((1, 50, 2, 24), torch.bfloat16, 1).to(d)
    with pytest.raises(NotImplementedError, match="head dims"):
        pj.attention_forward(q24, q24, q24, impl=TC)
    out = pj.attention_forward(q24, q24, q24, sm_scale=0.2)  # auto falls to the generic kernel
    want, _ = oracle_fwd(q24, q24, q24, sm_scale=0.2)
    assert_close(out, None, want, None, torch.bfloat16, "auto generic")


@pytest.mark.parametrize("impl", [TC, "b200:generic", None])
def test_latent_attention_golden(impl):
    inp = cases.make_inputs("c5_small")
    d = dev()
    out, lse = pj.mla(inp["q"].to(d), inp["cache"].to(d), inp["wk"].to(d), inp["wv"].to(d),
                      mask=pj.CausalMask(), sm_scale=inp["sm_scale"], return_lse=True, implementation=impl)
    pj.check_status(d)
    want, want_lse = load_golden("c5_small")
    assert_close(out, lse, want, want_lse, torch.bfloat16, f"c5_small {impl}")


@pytest.mark.parametrize("impl", [TC, "b200:generic"])
@pytest.mark.parametrize("s_len,dh,r", [(128, 128, 64), (300, 64, 136), (64, 128, 8), (700, 192, 576)])
def test_projection_product(impl, s_len, dh, r):
    """The up-projection K = C.W_K^T, V = C.W_V^T (ragged tile tails on every axis),
    checked through the whole latent-attention call against the oracle."""
    d = dev()
    dv = 128 if dh == 192 else dh
    cache = randn((1, s_len, r), torch.bfloat16, 1)
    std = 1.0 / math.sqrt(r)  # keeps the projected keys and values O(1), where the 2e-2 bound is meaningful
    wk, wv = (randn((2, dh, r), torch.float32, 2) * std).bfloat16(), (randn((2, dv, r), torch.float32, 3) * std).bfloat16()
    q = randn((1, 40, 2, dh), torch.bfloat16, 4)
    if impl == TC and r < 64:  # the tensor-map path needs at least one full 64-wide K slice
        with pytest.raises(NotImplementedError, match="projection"):
            pj.mla(q.to(d), cache.to(d), wk.to(d), wv.to(d), sm_scale=0.05, implementation=impl)
        return
    got = pj.mla(q.to(d), cache.to(d), wk.to(d), wv.to(d), sm_scale=0.05, implementation=impl)
    pj.check_status(d)
    want = oracle.mla_reference(q, cache, wk, wv, sm_scale=0.05, factorisation="materialized")
    assert_close(got, None, want, None, torch.bfloat16, f"projection {(s_len, dh, r)}")


def test_host_buffer_call_matches_device_call():
    inp = cases.make_inputs("c2_small_causal")
    q, k, v = (inp[n].pin_memory() for n in ("q", "k", "v"))
    out, lse = pj.attention_forward(q, k, v, causal=True, sm_scale=inp["sm_scale"], return_lse=True)
    assert not out.is_cuda and out.is_pinned()
    want, want_lse = load_golden("c2_small_causal")
    assert_close(out, lse, want, want_lse, torch.bfloat16, "host buffers")
    out2 = pj.attention_forward(q.numpy() if q.dtype != torch.bfloat16 else q, k, v, causal=True, sm_scale=inp["sm_scale"])
    assert torch.equal(out, out2)


def test_seeded_random_shape_sweep():
    """Twenty seeded random problems on the tcgen05 kernel: ragged lengths on both
    axes, every head shape it is built for, GQA ratios, masks and biases."""
    import numpy as np

    rng = np.random.default_rng(7)
    shapes = [(64, 64), (128, 128), (192, 128)]
    for case in range(20):
        d, dv = shapes[case % 3]
        hkv = int(rng.integers(1, 3))
        hq = hkv * int(rng.integers(1, 5))
        b, lq, lkv = int(rng.integers(1, 3)), int(rng.integers(1, 700)), int(rng.integers(1, 900))
        dtype = torch.bfloat16 if case % 2 else torch.float16
        q, k, v = randn((b, lq, hq, d), dtype, 5 * case), randn((b, lkv, hkv, d), dtype, 5 * case + 1), randn((b, lkv, hkv, dv), dtype, 5 * case + 2)
        kw = dict(causal=bool(rng.integers(0, 2)), sm_scale=1 / math.sqrt(d))
        if rng.integers(0, 2):
            kw["kv_lengths"] = torch.from_numpy(rng.integers(0, lkv + 1, size=b).astype(np.int32))
        if rng.integers(0, 3) == 0:
            kw["bias"] = randn((1, hq, lq, lkv), torch.float32, 2000 + case)
        out, lse = _run(q, k, v, **kw)
        want, want_lse = oracle_fwd(q, k, v, **kw)
        assert_close(out, lse, want, want_lse, dtype, f"case {case}: {(b, lq, lkv, hq, hkv, d, dv)} {sorted(kw)}")


@pytest.mark.parametrize("causal", [False, True])
def test_host_buffer_call_with_query_row_chunks(causal):
    """Long query sequences without an LSE result go through the host pipeline in blocks of query
    rows (mask band shifted per block); the result must not depend on that."""
    b, lq, lkv, hq, hkv, d = 2, 2304, 2048, 4, 2, 128
    q, k, v = randn((b, lq, hq, d), torch.bfloat16, 1), randn((b, lkv, hkv, d), torch.bfloat16, 2), randn((b, lkv, hkv, d), torch.bfloat16, 3)
    lens = torch.tensor([lkv, 777], dtype=torch.int32)
    sc = 1 / math.sqrt(d)
    out_host = pj.attention_forward(q.pin_memory(), k.pin_memory(), v.pin_memory(), causal=causal, kv_lengths=lens, sm_scale=sc)
    assert not out_host.is_cuda
    out_dev = pj.attention_forward(q.to(dev()), k.to(dev()), v.to(dev()), causal=causal, kv_lengths=lens, sm_scale=sc)
    assert torch.equal(out_host, out_dev.cpu())


@pytest.mark.parametrize("d,dv", [(128, 128), (64, 64), (192, 128)])
def test_rows_past_the_valid_length_may_hold_anything(d, dv):
    """K / V rows between kv_lengths[b] and Lkv (a cache tail that was never written) must not
    reach the result: NaN and inf there give the same bits as zeros."""
    b, lq, lkv, hq, hkv = 2, 300, 700, 4, 2
    q, k, v = randn((b, lq, hq, d), torch.bfloat16, 1), randn((b, lkv, hkv, d), torch.bfloat16, 2), randn((b, lkv, hkv, dv), torch.bfloat16, 3)
    lens = torch.tensor([517, 130], dtype=torch.int32)
    clean_k, clean_v = k.clone(), v.clone()
    for i in range(b):
        clean_k[i, lens[i]:] = 0
        clean_v[i, lens[i]:] = 0
        k[i, lens[i]:] = float("nan")
        v[i, lens[i]:] = float("nan")
        v[i, lens[i] + 1] = float("inf")
    sc = 1 / math.sqrt(d)
    for causal in (False, True):
        got, lse = pj.attention_forward(q.to(dev()), k.to(dev()), v.to(dev()), causal=causal, kv_lengths=lens, sm_scale=sc,
                                        return_lse=True, impl="b200:tcgen05")
        ref, lse_ref = pj.attention_forward(q.to(dev()), clean_k.to(dev()), clean_v.to(dev()), causal=causal, kv_lengths=lens,
                                            sm_scale=sc, return_lse=True, impl="b200:tcgen05")
        assert torch.isfinite(got).all()
        assert torch.equal(got, ref) and torch.equal(lse, lse_ref)


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float16, 64)])
@pytest.mark.parametrize("b,h,lq,lkv", [(1, 3, 600, 1100), (2, 80, 512, 1024), (1, 2, 256, 4096)])
def test_last_wave_cut_into_kv_halves(dtype, d, b, h, lq, lkv):
    """Unmasked problems whose last wave of work items fills at most half of the SMs run those items as
    two CTAs each (KV halves, fp32 partials, a merge kernel): 6, 320 = 2 x 148 + 24 and 2 work items here.
    Output and log-sum-exp against the oracle, and bit-repeatable."""
    q = randn((b, lq, h, d), dtype, 1)
    k = randn((b, lkv, max(h // 2, 1), d), dtype, 2) if h % 2 == 0 else randn((b, lkv, h, d), dtype, 2)
    v = randn(tuple(k.shape), dtype, 3)
    sc = 1 / math.sqrt(d)
    out, lse = _run(q, k, v, sm_scale=sc)
    want, want_lse = oracle_fwd(q[:, :, : min(h, 6)], k[:, :, : max(min(h, 6) // (2 if h % 2 == 0 else 1), 1)],
                                v[:, :, : max(min(h, 6) // (2 if h % 2 == 0 else 1), 1)], sm_scale=sc)
    assert_close(out[:, :, : min(h, 6)], lse[:, : min(h, 6)], want, want_lse, dtype, f"kv halves b{b} h{h} lq{lq} lkv{lkv}")
    if h > 6:  # the last heads too (their work items are the ones cut in two)
        hk = k.shape[2]
        g = h // hk
        want, want_lse = oracle_fwd(q[:, :, -g:], k[:, :, -1:], v[:, :, -1:], sm_scale=sc)
        assert_close(out[:, :, -g:], lse[:, -g:], want, want_lse, dtype, "kv halves, last heads")
    again, lse2 = _run(q, k, v, sm_scale=sc)
    assert torch.equal(out, again) and torch.equal(lse, lse2)
