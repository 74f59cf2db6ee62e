"""Gradients of the attention forward (pjx_attn_bwd through torch autograd) against
float64 autograd of the dense softmax formula -- the way the reference checks its
backward kernels (tests/test_attention_gqa_splitkv.py:83-97, 304-319: gradients of the
kernel path vs jax.grad of the dense reference, fp32 rel < 1e-5 on CPU, bf16 rel < 1e-2)."""

import math

import pytest
import torch

import probjax_b200 as pj
from _gpu_util import dev, randn

pytestmark = pytest.mark.gpu


def _dense(q, k, v, causal, kv_lengths, bias, sc):
    """Differentiable float64 dense attention with repeat GQA semantics."""
    rep = q.shape[2] // k.shape[2]
    kk, vv = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * sc
    if bias is not None:
        s = s + bias
    lq, lk = s.shape[-2:]
    keep = torch.ones(1, 1, lq, lk, dtype=torch.bool)
    if causal:
        keep = keep & torch.tril(torch.ones(lq, lk, dtype=torch.bool))[None, None]
    if kv_lengths is not None:
        keep = keep & (torch.arange(lk)[None, :] < kv_lengths[:, None])[:, None, None, :]
    s = s.masked_fill(~keep, -math.inf)
    m = s.amax(-1, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    p = e / torch.where(den > 0, den, torch.ones_like(den))
    return torch.einsum("bhqk,bkhd->bqhd", p, vv)


def _rel(a, b):
    return float((a.double().cpu() - b).norm() / b.norm().clamp_min(1e-30))


@pytest.mark.parametrize(
    "dtype,b,lq,lkv,hq,hkv,d,dv,causal,lengths,bias",
    [
        (torch.float32, 2, 40, 40, 4, 2, 16, 16, True, False, False),     # GQA, causal
        (torch.float32, 2, 40, 40, 4, 1, 16, 16, False, False, False),    # MQA
        (torch.float32, 1, 50, 77, 2, 2, 24, 40, True, True, True),       # ragged, Dv != D, lengths + bias
        (torch.float32, 2, 33, 65, 3, 3, 100, 100, False, True, False),   # odd head width
        (torch.bfloat16, 1, 200, 333, 4, 2, 128, 128, True, True, True),
        (torch.bfloat16, 2, 130, 130, 8, 2, 64, 64, False, False, False),
        (torch.float16, 1, 96, 160, 2, 2, 192, 128, True, False, False),
    ],
)
def test_gradients_match_dense_autograd(dtype, b, lq, lkv, hq, hkv, d, dv, causal, lengths, bias):
    dvc = dev()
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, dv), dtype, 3)
    g = randn((b, lq, hq, dv), dtype, 4)
    lens = torch.tensor([lkv, max(1, lkv // 3)][:b], dtype=torch.int32) if lengths else None
    bt = randn((1, hq, lq, lkv), torch.float32, 5) if bias else None
    sc = 1 / math.sqrt(d)
    mask = None
    if causal:
        mask = pj.CausalMask()
    if lens is not None:
        mask = pj.KVLenMask(lens) if mask is None else (mask & pj.KVLenMask(lens))
    qd, kd, vd = (x.to(dvc).requires_grad_(True) for x in (q, k, v))
    out = pj.flex_attention(qd, kd, vd, mask=mask, bias=None if bt is None else pj.DenseBias(bt), sm_scale=sc,
                            enable_gqa=True)
    out.backward(g.to(dvc))
    q64, k64, v64 = (x.double().requires_grad_(True) for x in (q, k, v))
    ref = _dense(q64, k64, v64, causal, lens, None if bt is None else bt.double(), sc)
    ref.backward(g.double())
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert _rel(out.detach(), ref.detach()) < tol
    assert _rel(qd.grad, q64.grad) < tol, "dq"
    assert _rel(kd.grad, k64.grad) < tol, "dk"
    assert _rel(vd.grad, v64.grad) < tol, "dv"
    if lens is not None:  # keys past the valid length get exactly zero gradient
        short = int(lens[-1])
        assert (kd.grad[-1, short:] == 0).all() and (vd.grad[-1, short:] == 0).all()


def test_zero_length_rows_and_no_grad_paths():
    dvc = dev()
    q, k, v = (randn((2, 9, 2, 16), torch.float32, s) for s in (1, 2, 3))
    lens = torch.tensor([0, 9], dtype=torch.int32)
    qd, kd, vd = (x.to(dvc).requires_grad_(True) for x in (q, k, v))
    out = pj.flex_attention(qd, kd, vd, mask=pj.KVLenMask(lens), sm_scale=0.25)
    out.sum().backward()
    assert (qd.grad[0] == 0).all() and (kd.grad[0] == 0).all() and (vd.grad[0] == 0).all()
    assert torch.isfinite(qd.grad).all() and torch.isfinite(kd.grad).all() and torch.isfinite(vd.grad).all()
    # under no_grad the plain forward runs (no residuals are kept)
    with torch.no_grad():
        out2 = pj.flex_attention(qd, kd, vd, mask=pj.KVLenMask(lens), sm_scale=0.25)
    assert not out2.requires_grad and torch.equal(out2, out.detach())
    with pytest.raises(NotImplementedError, match="DenseBias"):
        bias = torch.zeros(1, 2, 9, 9, device=dvc, requires_grad=True)
        pj.flex_attention(qd, kd, vd, bias=pj.DenseBias(bias), sm_scale=0.25)
