"""Parity of the generic (CUDA-core, exact fp32) forward kernel with the CPU oracle."""

import math

import pytest
import torch

import probjax_b200 as pj
from _gpu_util import assert_close, cases, dev, load_golden, oracle_fwd, randn

pytestmark = pytest.mark.gpu
GEN = "b200:generic"


def _run(q, k, v, **kw):
    d = dev()
    args = {n: (t.to(d) if isinstance(t, torch.Tensor) else t) for n, t in kw.items()}
    out, lse = pj.attention_forward(q.to(d), k.to(d), v.to(d), return_lse=True, impl=GEN, **args)
    pj.check_status(d)
    return out, lse


@pytest.mark.parametrize("name", ["c1_small", "c1_full", "ragged_bias", "c2_small", "c2_small_causal", "c3_small"])
def test_golden(name):
    inp = cases.make_inputs(name)
    kw = {n: inp[n] for n in ("causal", "sm_scale", "kv_lengths", "bias") if n in inp}
    out, lse = _run(inp["q"], inp["k"], inp["v"], **kw)
    want, want_lse = load_golden(name)
    assert_close(out, lse, want, want_lse, inp["q"].dtype, name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize(
    "b,lq,lkv,hq,hkv,d,dv,causal",
    [
        (2, 40, 40, 4, 2, 16, 16, True),      # tests/test_attention_gqa_splitkv.py:83-97
        (2, 40, 40, 4, 1, 16, 16, False),
        (1, 1, 300, 8, 2, 32, 32, False),     # decode shapes, :235-243
        (1, 4, 1000, 8, 2, 32, 32, False),
        (1, 50, 50, 2, 2, 24, 24, True),      # tests/test_attention_xla.py:424-431
        (1, 133, 97, 3, 3, 30, 30, False),    # odd everything (tests/test_attention.py:480-543 uses D30, D100)
        (1, 70, 130, 2, 1, 100, 100, True),
        (1, 65, 64, 2, 2, 256, 256, False),   # largest head width
        (2, 33, 47, 4, 2, 48, 20, False),     # value width differs from key width
        (1, 200, 10, 2, 2, 64, 64, True),     # more queries than keys under a causal mask
    ],
)
def test_shapes(dtype, b, lq, lkv, hq, hkv, d, dv, causal):
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, dv), dtype, 3)
    sc = 1 / math.sqrt(d)
    out, lse = _run(q, k, v, causal=causal, sm_scale=sc)
    want, want_lse = oracle_fwd(q, k, v, causal=causal, sm_scale=sc)
    assert_close(out, lse, want, want_lse, dtype, f"{(b, lq, lkv, hq, hkv, d, dv, causal)}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bshape", [(2, 4), (1, 1), (1, 4), (2, 1)])
def test_bias_broadcast_and_key_lengths(dtype, bshape):
    b, lq, lkv, h, d = 2, 70, 90, 4, 32
    q, k, v = randn((b, lq, h, d), dtype, 4), randn((b, lkv, h, d), dtype, 5), randn((b, lkv, h, d), dtype, 6)
    bias = randn((*bshape, lq, lkv), torch.float32, 7)
    lens = torch.tensor([33, 90], dtype=torch.int32)
    out, lse = _run(q, k, v, causal=True, kv_lengths=lens, bias=bias, sm_scale=0.25)
    want, want_lse = oracle_fwd(q, k, v, causal=True, kv_lengths=lens, bias=bias, sm_scale=0.25)
    assert_close(out, lse, want, want_lse, dtype, f"bias{bshape}")


def test_rows_without_keys_are_zero_with_infinite_lse():
    # tests/test_attention_device_defaults.py:317-328, tests/test_attention_xla.py:241-249
    q, k, v = randn((3, 9, 2, 16), torch.float32, 8), randn((3, 20, 2, 16), torch.float32, 9), randn((3, 20, 2, 16), torch.float32, 10)
    lens = torch.tensor([0, 20, 7], dtype=torch.int32)
    out, lse = _run(q, k, v, kv_lengths=lens, sm_scale=1.0)
    assert (out[0] == 0).all() and torch.isinf(lse[0]).all() and (lse[0] > 0).all()
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=1.0)
    assert_close(out, lse, want, want_lse, torch.float32, "empty rows")


def test_lengths_beyond_capacity_are_clamped():
    q, k, v = randn((2, 5, 2, 16), torch.float32, 11), randn((2, 12, 2, 16), torch.float32, 12), randn((2, 12, 2, 16), torch.float32, 13)
    out, lse = _run(q, k, v, kv_lengths=torch.tensor([99, -3], dtype=torch.int32), sm_scale=0.5)
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=torch.tensor([12, 0]), sm_scale=0.5)
    assert_close(out, lse, want, want_lse, torch.float32, "clamped")


def test_empty_batch_and_single_row():
    d = dev()
    q = torch.zeros(0, 4, 2, 16, device=d)
    assert pj.attention_forward(q, q, q, impl=GEN).shape == (0, 4, 2, 16)
    q, k, v = randn((1, 1, 1, 8), torch.float32, 1), randn((1, 1, 1, 8), torch.float32, 2), randn((1, 1, 1, 8), torch.float32, 3)
    out, lse = _run(q, k, v, sm_scale=1.0)
    assert torch.allclose(out.cpu(), v, atol=1e-6)  # one key: the output is its value
    assert torch.allclose(lse.cpu().reshape(()), (q * k).sum(), atol=1e-5)


def test_seeded_random_shape_sweep():
    """Thirty seeded random problems (ragged lengths, odd head widths, GQA ratios,
    masks and biases in every combination) against the oracle."""
    import numpy as np

    rng = np.random.default_rng(2024)
    for case in range(30):
        hkv = int(rng.integers(1, 4))
        hq = hkv * int(rng.integers(1, 4))
        b, lq, lkv = int(rng.integers(1, 4)), int(rng.integers(1, 150)), int(rng.integers(1, 200))
        d, dv = int(rng.integers(1, 80)), int(rng.integers(1, 80))
        dtype = [torch.float32, torch.bfloat16, torch.float16][case % 3]
        causal = bool(rng.integers(0, 2))
        q, k, v = randn((b, lq, hq, d), dtype, 3 * case), randn((b, lkv, hkv, d), dtype, 3 * case + 1), randn((b, lkv, hkv, dv), dtype, 3 * case + 2)
        kw = dict(causal=causal, sm_scale=float(rng.uniform(0.05, 0.5)))
        if rng.integers(0, 2):
            kw["kv_lengths"] = torch.from_numpy(rng.integers(0, lkv + 1, size=b).astype(np.int32))
        if rng.integers(0, 2):
            kw["bias"] = randn((1 if rng.integers(0, 2) else b, 1 if rng.integers(0, 2) else hq, lq, lkv), torch.float32, 1000 + case)
        out, lse = _run(q, k, v, **kw)
        want, want_lse = oracle_fwd(q, k, v, **kw)
        assert_close(out, lse, want, want_lse, dtype, f"case {case}: {(b, lq, lkv, hq, hkv, d, dv)} {sorted(kw)}")
