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


@pytest.mark.parametrize("bshape", [(1, 4, 40, 56), (2, 1, 40, 56), (2, 4, 40, 56), (1, 1, 40, 56)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gradient_of_a_learnable_dense_bias(bshape, dtype):
    """d(loss)/d(bias) = dS, summed over the axes the bias broadcasts (configuration 3 of the
    benchmark set has a learnable fp32 bias [H, Sq, Skv])."""
    dvc = dev()
    b, hq, hkv, lq, lkv, d = 2, 4, 2, 40, 56, 32
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, d), dtype, 3)
    g = randn((b, lq, hq, d), dtype, 4)
    bias = randn(bshape, torch.float32, 5)
    lens = torch.tensor([lkv, 30], dtype=torch.int32)
    sc = 1 / math.sqrt(d)
    qd, kd, vd = (x.to(dvc).requires_grad_(True) for x in (q, k, v))
    bd = bias.to(dvc).requires_grad_(True)
    out = pj.flex_attention(qd, kd, vd, mask=pj.CausalMask() & pj.KVLenMask(lens), bias=pj.DenseBias(bd), sm_scale=sc,
                            enable_gqa=True)
    out.backward(g.to(dvc))
    q64, k64, v64, b64 = (x.double().requires_grad_(True) for x in (q, k, v, bias))
    ref = _dense(q64, k64, v64, True, lens, b64, sc)
    ref.backward(g.double())
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert bd.grad is not None and bd.grad.shape == bias.shape
    assert _rel(bd.grad, b64.grad) < tol, _rel(bd.grad, b64.grad)
    assert _rel(qd.grad, q64.grad) < tol and _rel(kd.grad, k64.grad) < tol and _rel(vd.grad, v64.grad) < tol
    # only the bias asks for a gradient
    bd2 = bias.to(dvc).requires_grad_(True)
    pj.flex_attention(q.to(dvc), k.to(dvc), v.to(dvc), bias=pj.DenseBias(bd2), sm_scale=sc, enable_gqa=True).sum().backward()
    assert bd2.grad is not None and torch.isfinite(bd2.grad).all()


def _grads64(q, k, v, g, keep, sc):
    q64, k64, v64 = (x.double().requires_grad_(True) for x in (q, k, v))
    rep = q.shape[2] // k.shape[2]
    kk, vv = k64.repeat_interleave(rep, dim=2), v64.repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q64, kk) * sc
    s = s.masked_fill(~keep, -math.inf)
    m = s.amax(-1, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    out = torch.einsum("bhqk,bkhd->bqhd", e / torch.where(den > 0, den, torch.ones_like(den)), vv)
    out.backward(g.double())
    return q64.grad, k64.grad, v64.grad


@pytest.mark.parametrize(
    "dtype,b,lq,lkv,hq,hkv,d,band,lengths",
    [
        (torch.bfloat16, 1, 128, 128, 1, 1, 128, (None, None), False),   # one tile, no mask
        (torch.bfloat16, 2, 256, 384, 4, 2, 128, (None, None), False),   # GQA, several tiles
        (torch.bfloat16, 2, 300, 300, 4, 1, 128, (None, 0), False),      # causal, ragged tails, MQA
        (torch.float16, 2, 200, 333, 2, 2, 64, (None, 0), True),         # key lengths
        (torch.bfloat16, 1, 520, 391, 2, 2, 64, (-100, 30), True),       # window band
        (torch.bfloat16, 2, 257, 700, 6, 3, 128, (None, 443), False),    # bottom-right causal
        (torch.float16, 3, 130, 260, 2, 2, 128, (-64, 0), True),         # a sequence without keys
    ],
)
def test_tcgen05_backward_matches_dense_autograd_and_generic(dtype, b, lq, lkv, hq, hkv, d, band, lengths):
    dvc = dev()
    q, k, v = randn((b, lq, hq, d), dtype, 11), randn((b, lkv, hkv, d), dtype, 12), randn((b, lkv, hkv, d), dtype, 13)
    g = randn((b, lq, hq, d), dtype, 14)
    sc = 1 / math.sqrt(d)
    lens = None
    if lengths:
        lens = torch.tensor([lkv, max(1, lkv // 3), 0][:b], dtype=torch.int32)
    i, j = torch.arange(lq)[:, None], torch.arange(lkv)[None, :]
    keep = torch.ones(lq, lkv, dtype=torch.bool)
    if band[0] is not None:
        keep &= j >= i + band[0]
    if band[1] is not None:
        keep &= j <= i + band[1]
    keep = keep[None, None].expand(b, 1, lq, lkv).clone()
    if lens is not None:
        keep &= (torch.arange(lkv)[None, :] < lens[:, None])[:, None, None, :]
    qd, kd, vd, gd = (x.to(dvc) for x in (q, k, v, g))
    o, lse = pj.attention_forward(qd, kd, vd, band=band, kv_lengths=lens, sm_scale=sc, return_lse=True)
    got = pj.attention_backward(qd, kd, vd, o, lse, gd, band=band, kv_lengths=lens, sm_scale=sc, impl="b200:tcgen05")
    gen = pj.attention_backward(qd, kd, vd, o, lse, gd, band=band, kv_lengths=lens, sm_scale=sc, impl="b200:generic")
    pj.check_status()
    want = _grads64(q, k, v, g, keep, sc)
    for name, a, c, w in zip(("dq", "dk", "dv"), got, gen, want):
        assert torch.isfinite(a).all(), name
        assert _rel(a, w) < 2e-2, (name, _rel(a, w))
        assert _rel(a, c.double().cpu()) < 2e-2, (name, "vs generic", _rel(a, c.double().cpu()))
    if lens is not None and b == 3:  # the sequence without keys has zero gradients everywhere
        assert all((x[2] == 0).all() for x in got)


def test_tcgen05_backward_refuses_what_it_does_not_compute():
    dvc = dev()
    q = randn((1, 64, 2, 96), torch.bfloat16, 1).to(dvc)
    o, lse = pj.attention_forward(q, q, q, sm_scale=0.1, return_lse=True)
    with pytest.raises(NotImplementedError, match="head dims"):
        pj.attention_backward(q, q, q, o, lse, q, sm_scale=0.1, impl="b200:tcgen05")
    # auto falls back to the CUDA-core kernels
    dq, dk, dv = pj.attention_backward(q, q, q, o, lse, q, sm_scale=0.1)
    assert torch.isfinite(dq).all()


@pytest.mark.parametrize(
    "dtype,b,lq,lkv,hq,hkv,d,dv,mask_kind",
    [
        (torch.float32, 2, 45, 70, 4, 2, 24, 40, "causal_len"),
        (torch.float32, 1, 64, 64, 2, 2, 100, 100, "window"),
        (torch.bfloat16, 2, 130, 200, 4, 1, 128, 128, "none"),
        (torch.float16, 1, 96, 96, 2, 2, 64, 64, "causal_len"),
    ],
)
def test_forward_mode_tangent_matches_dense_jvp(dtype, b, lq, lkv, hq, hkv, d, dv, mask_kind):
    """pjx_attn_jvp_band through torch forward-mode AD against torch.func.jvp of the float64 dense
    formula (the reference tests diff_mode="forward" against jax.jvp of its dense path)."""
    import torch.autograd.forward_ad as fwd_ad

    dvc = dev()
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, dv), dtype, 3)
    tq, tk, tv = randn((b, lq, hq, d), dtype, 4), randn((b, lkv, hkv, d), dtype, 5), randn((b, lkv, hkv, dv), dtype, 6)
    sc = 1 / math.sqrt(d)
    lens = torch.tensor([lkv, max(1, lkv // 3)][:b], dtype=torch.int32)
    if mask_kind == "causal_len":
        mask = pj.CausalMask() & pj.KVLenMask(lens)
    elif mask_kind == "window":
        mask = pj.LocalWindowMask(9, 4)
    else:
        mask = None
    keep = torch.ones(b, 1, lq, lkv, dtype=torch.bool) if mask is None else mask.dense(lq, lkv, batch_size=b)

    def dense(q_, k_, v_):
        rep = hq // hkv
        kk, vv = k_.repeat_interleave(rep, dim=2), v_.repeat_interleave(rep, dim=2)
        s = torch.einsum("bqhd,bkhd->bhqk", q_, kk) * sc
        s = s.masked_fill(~keep, -math.inf)
        return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), vv)

    _, want = torch.func.jvp(dense, (q.double(), k.double(), v.double()), (tq.double(), tk.double(), tv.double()))
    with fwd_ad.dual_level():
        qd, kd, vd = (fwd_ad.make_dual(x.to(dvc), t.to(dvc)) for x, t in ((q, tq), (k, tk), (v, tv)))
        out = pj.flex_attention(qd, kd, vd, mask=mask, sm_scale=sc, enable_gqa=True)
        primal, tangent = fwd_ad.unpack_dual(out)
    assert tangent is not None
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert _rel(tangent, want) < tol, _rel(tangent, want)
    # a missing tangent is a zero tangent
    got_q_only = pj.attention_jvp(q.to(dvc), k.to(dvc), v.to(dvc),
                                  pj.attention_forward(q.to(dvc), k.to(dvc), v.to(dvc), band=pj.masks.lower_mask(mask, b, lq, lkv).band,
                                                       kv_lengths=pj.masks.lower_mask(mask, b, lq, lkv).kv_lengths, sm_scale=sc,
                                                       return_lse=True)[1],
                                  tq.to(dvc), None, None, band=pj.masks.lower_mask(mask, b, lq, lkv).band,
                                  kv_lengths=pj.masks.lower_mask(mask, b, lq, lkv).kv_lengths, sm_scale=sc)
    _, want_q = torch.func.jvp(lambda q_: dense(q_, k.double(), v.double()), (q.double(),), (tq.double(),))
    assert _rel(got_q_only, want_q) < tol


@pytest.mark.parametrize("absorbed", [False, True])
def test_latent_attention_gradients(absorbed):
    """mla differentiates through the materialized K, V and the attention kernels
    (latent_attention.py:554-585); reference: float64 autograd of the same composition."""
    dvc = dev()
    dtype = torch.bfloat16
    b, lq, s_len, h, r = 2, 70, 90, 4, 64
    dqk, dv_ = (r, r) if absorbed else (48, 32)
    q, cache = randn((b, lq, h, dqk), dtype, 1), randn((b, s_len, r), dtype, 2)
    wk = None if absorbed else (randn((h, dqk, r), dtype, 3) / math.sqrt(r)).to(dtype)
    wv = None if absorbed else (randn((h, dv_, r), dtype, 4) / math.sqrt(r)).to(dtype)
    g = randn((b, lq, h, dv_), dtype, 5)
    sc = 1 / math.sqrt(dqk)
    leaves = [x.to(dvc).requires_grad_(True) for x in (q, cache) + (() if absorbed else (wk, wv))]
    out = pj.mla(leaves[0], leaves[1], *(leaves[2:] if not absorbed else (None, None)), mask=pj.CausalMask(), sm_scale=sc)
    out.backward(g.to(dvc))
    ref = [x.double().requires_grad_(True) for x in (q, cache) + (() if absorbed else (wk, wv))]
    if absorbed:
        k64 = v64 = ref[1][:, :, None, :].expand(b, s_len, h, r)
    else:
        k64 = torch.einsum("bsr,hdr->bshd", ref[1], ref[2])
        v64 = torch.einsum("bsr,hdr->bshd", ref[1], ref[3])
    sco = torch.einsum("bqhd,bkhd->bhqk", ref[0], k64) * sc
    sco = sco.masked_fill(~torch.tril(torch.ones(lq, s_len, dtype=torch.bool))[None, None], -math.inf)
    o64 = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sco, -1), v64)
    o64.backward(g.double())
    assert _rel(out.detach(), o64.detach()) < 2e-2
    for name, a, w in zip(("dq", "dcache", "dwk", "dwv"), leaves, ref):
        assert _rel(a.grad, w.grad) < 3e-2, (name, _rel(a.grad, w.grad))


def test_backward_ignores_rows_past_the_valid_length():
    """K / V rows between kv_lengths[b] and Lkv may hold anything (NaN here): the gradients equal
    those of zero-filled tails bit for bit, and the tails themselves get zero gradients."""
    dvc = dev()
    b, lq, lkv, hq, hkv, d = 2, 300, 700, 4, 2, 128
    q, k, v = randn((b, lq, hq, d), torch.bfloat16, 1), randn((b, lkv, hkv, d), torch.bfloat16, 2), randn((b, lkv, hkv, d), torch.bfloat16, 3)
    g = randn((b, lq, hq, d), torch.bfloat16, 4)
    lens = torch.tensor([517, 130], dtype=torch.int32)
    clean_k, clean_v = k.clone(), v.clone()
    for i in range(b):
        clean_k[i, lens[i]:] = 0
        clean_v[i, lens[i]:] = 0
        k[i, lens[i]:] = float("nan")
        v[i, lens[i]:] = float("nan")
    sc = 1 / math.sqrt(d)
    res = []
    for kk, vv in ((k, v), (clean_k, clean_v)):
        qd, kd, vd, gd = (x.to(dvc) for x in (q, kk, vv, g))
        o, lse = pj.attention_forward(qd, kd, vd, causal=True, kv_lengths=lens, sm_scale=sc, return_lse=True)
        res.append(pj.attention_backward(qd, kd, vd, o, lse, gd, causal=True, kv_lengths=lens, sm_scale=sc, impl="b200:tcgen05"))
    for a, c in zip(*res):
        assert torch.isfinite(a).all() and torch.equal(a, c)
    for i in range(b):
        assert (res[0][1][i, lens[i]:] == 0).all() and (res[0][2][i, lens[i]:] == 0).all()
