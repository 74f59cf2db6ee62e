"""Index-band masks (local windows, bottom-right causal) through the forward and backward
kernels, against the CPU oracle evaluated with the mask's dense boolean form -- the reference
tests its window masks the same way (tests/test_attention_masks.py: kernel vs dense reference
built from ``mask.dense``)."""

import math

import pytest
import torch

import probjax_b200 as pj
from _gpu_util import assert_close, dev, oracle_fwd, randn

pytestmark = pytest.mark.gpu


def _mask_cases(lq, lkv):
    return [
        pj.LocalWindowMask(5, 3),
        pj.LocalWindowMask(200, 0),
        pj.LocalWindowMask(130, 140),
        pj.CausalLocalWindowMask(17),
        pj.CausalLocalWindowMask(300),
        pj.CausalFromBottomRightMask(lq, lkv),
        pj.CausalMask() & pj.LocalWindowMask(64, 64),
    ]


@pytest.mark.parametrize("impl,dtype,d,dv", [
    ("b200:generic", torch.float32, 40, 24),
    ("b200:tcgen05", torch.bfloat16, 128, 128),
    ("b200:tcgen05", torch.float16, 64, 64),
    ("b200:tcgen05", torch.bfloat16, 192, 128),
])
@pytest.mark.parametrize("lq,lkv", [(300, 300), (257, 700), (520, 391)])
def test_band_forward_matches_oracle(impl, dtype, d, dv, lq, lkv):
    b, hq, hkv = 2, 4, 2
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, dv), dtype, 3)
    sc = 1 / math.sqrt(d)
    lens = torch.tensor([lkv, max(1, lkv // 2)], dtype=torch.int32)
    for i, mask in enumerate(_mask_cases(lq, lkv)):
        with_len = i % 2 == 1
        m = (mask & pj.KVLenMask(lens)) if with_len else mask
        out, lse = pj.mha(q.to(dev()), k.to(dev()), v.to(dev()), mask=m, sm_scale=sc, return_lse=True,
                          implementation=impl)
        keep = mask.dense(lq, lkv, batch_size=b)
        want, want_lse = oracle_fwd(q, k, v, sm_scale=sc, keep=keep, kv_lengths=lens if with_len else None)
        assert_close(out, lse, want, want_lse, dtype, f"{impl} {mask} lens={with_len}")


def test_rows_without_visible_keys_are_zero():
    # a band entirely to the left of the first rows: those rows see nothing
    b, lq, lkv, h, d = 1, 200, 200, 2, 64
    q, k, v = (randn((b, lq, h, d), torch.bfloat16, s).to(dev()) for s in (1, 2, 3))
    out, lse = pj.attention_forward(q, k, v, band=(-40, -10), sm_scale=0.125, return_lse=True)
    assert (out[:, :10] == 0).all() and torch.isinf(lse[:, :, :10]).all() and (lse[:, :, :10] > 0).all()
    idx = torch.arange(lq)
    dqk = idx[:, None] - idx[None, :]
    keep = ((dqk >= 10) & (dqk <= 40))[None, None]
    want, want_lse = oracle_fwd(q, k, v, sm_scale=0.125, keep=keep)
    assert_close(out, lse, want, want_lse, torch.bfloat16, "left band")


def _dense64(q, k, v, keep, sc):
    rep = q.shape[2] // k.shape[2]
    kk, vv = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * sc
    s = s.masked_fill(~keep, -math.inf)
    m = s.amax(-1, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    return torch.einsum("bhqk,bkhd->bqhd", e / torch.where(den > 0, den, torch.ones_like(den)), vv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_band_gradients(dtype):
    b, lq, lkv, hq, hkv, d = 2, 150, 170, 4, 2, 32
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, d), dtype, 3)
    g = randn((b, lq, hq, d), dtype, 4)
    sc = 1 / math.sqrt(d)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for mask in (pj.LocalWindowMask(20, 9), pj.CausalLocalWindowMask(40), pj.CausalFromBottomRightMask(lq, lkv)):
        qd, kd, vd = (x.to(dev()).requires_grad_(True) for x in (q, k, v))
        out = pj.flex_attention(qd, kd, vd, mask=mask, sm_scale=sc, enable_gqa=True)
        out.backward(g.to(dev()))
        q64, k64, v64 = (x.double().requires_grad_(True) for x in (q, k, v))
        keep = mask.dense(lq, lkv, batch_size=b)
        ref = _dense64(q64, k64, v64, keep, sc)
        ref.backward(g.double())
        for name, a, r in (("dq", qd.grad, q64.grad), ("dk", kd.grad, k64.grad), ("dv", vd.grad, v64.grad)):
            rel = float((a.double().cpu() - r).norm() / r.norm())
            assert rel < tol, (str(mask), name, rel)


def test_masks_and_biases_without_a_native_form_run_through_the_dense_lowering():
    """Segment / prefix masks and ALiBi-style biases reach the kernels as one additive tensor
    (-inf where masked), while the causal part of the expression stays native."""
    b, lq, h, d = 2, 200, 4, 64
    dtype = torch.bfloat16
    q, k, v = (randn((b, lq, h, d), dtype, s) for s in (1, 2, 3))
    seg = torch.stack([torch.arange(lq) // 50, torch.arange(lq) // 70])
    sc = 1 / math.sqrt(d)
    cases = [
        (pj.CausalMask() & pj.SameSegmentMask(seg), None),
        (pj.PrefixLMMask(torch.tensor([30, 120])), pj.CausalAlibiBias()),
        (pj.SeqLenMask(torch.tensor([200, 77])), pj.SumBias(pj.ConstantBias(0.5), pj.DistanceDecayBias(0.01))),
        (None, pj.SymmetricAlibiBias()),
    ]
    for mask, bias in cases:
        out, lse = pj.flex_attention(q.to(dev()), k.to(dev()), v.to(dev()), mask=mask, bias=bias, sm_scale=sc,
                                     return_lse=True)
        keep = None if mask is None else mask.dense(lq, lq, batch_size=b)
        bt = None if bias is None else bias.dense(lq, lq, batch_size=b, num_heads=h)
        want, want_lse = oracle_fwd(q, k, v, sm_scale=sc, keep=keep, bias=bt)
        assert_close(out, lse, want, want_lse, dtype, f"{type(mask).__name__} + {type(bias).__name__}")
