"""Seeded random shapes through every kernel family, each against the CPU oracle.

The fixed cases of the other files are the reference's test shapes and the benchmark configurations;
this file walks the space between them: odd lengths, every supported head width, GQA group sizes,
ragged key lengths with empty sequences, bands, dense biases, the in-kernel score modifiers, split
lengths of the decode, paged caches and the absorbed latent decode on both of its kernels.  The draws
are fixed by the seeds, so a failure names a reproducible case.
"""

import math
import random

import pytest
import torch

import oracle
import probjax_b200 as pj
from probjax_b200 import masks as M
from _gpu_util import assert_close, dev, randn

pytestmark = pytest.mark.gpu


def _draw_forward(rng):
    dtype = rng.choice([torch.bfloat16, torch.float16, torch.float32])
    hkv = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 4])
    d = rng.choice([16, 32, 64, 128] if dtype != torch.float32 else [8, 16, 40, 64])
    dv = d if rng.random() < 0.8 else rng.choice([16, 32, 64])
    return dict(dtype=dtype, B=rng.randint(1, 3), Lq=rng.randint(1, 300), Lkv=rng.randint(1, 400), hkv=hkv,
                hq=hkv * group, d=d, dv=dv, mask=rng.choice(["none", "causal", "window", "bottom_right", "lengths", "segments"]),
                bias=rng.choice(["none", "none", "dense", "alibi", "softcap"]))


@pytest.mark.parametrize("seed", range(24))
def test_forward_random_shape(seed):
    rng = random.Random(1000 + seed)
    c = _draw_forward(rng)
    dt, B, Lq, Lkv = c["dtype"], c["B"], c["Lq"], c["Lkv"]
    if c["mask"] in ("causal", "window", "segments"):
        Lkv = Lq  # these masks are defined on square problems here
    q = randn((B, Lq, c["hq"], c["d"]), dt, seed * 7 + 1)
    k = randn((B, Lkv, c["hkv"], c["d"]), dt, seed * 7 + 2)
    v = randn((B, Lkv, c["hkv"], c["dv"]), dt, seed * 7 + 3)
    sc = 1 / math.sqrt(c["d"])
    g = torch.Generator().manual_seed(seed)
    mask, keep = None, None
    if c["mask"] == "causal":
        mask = M.CausalMask()
    elif c["mask"] == "window":
        mask = M.LocalWindowMask(rng.randint(1, 40), rng.randint(0, 40))
    elif c["mask"] == "bottom_right":
        mask = M.CausalFromBottomRightMask(Lq, Lkv)
    elif c["mask"] == "lengths":
        lens = torch.randint(0, Lkv + 1, (B,), generator=g)
        mask = M.KVLenMask(lens)
    elif c["mask"] == "segments":
        seg = torch.sort(torch.randint(0, 4, (B, Lq), generator=g), dim=1).values.to(torch.int32)
        mask = M.BlockDiagonalCausalMask(seg)
    if mask is not None:
        keep = mask.dense(Lq, Lkv, batch_size=B, num_heads=1)
    bias, dense, score_fn = None, None, None
    if c["bias"] == "dense":
        dense = torch.randn((rng.choice([1, B]), rng.choice([1, c["hq"]]), Lq, Lkv), generator=g)
        bias = M.DenseBias(dense)
    elif c["bias"] == "alibi":
        bias = M.SymmetricAlibiBias()
        dense = bias.dense(Lq, Lkv, num_heads=c["hq"])
    elif c["bias"] == "softcap":
        bias = M.SoftCappingBias(3.0)
        score_fn = lambda s, qi, ki: 3.0 * torch.tanh(s / 3.0)  # noqa: E731
    want, want_lse = oracle.xla_attention(q, k, v, keep=keep, bias=dense, sm_scale=sc, return_lse=True, score_fn=score_fn)
    d = dev()
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=mask, bias=bias, sm_scale=sc, return_lse=True, split_kv=False)
    pj.check_status(d)
    assert_close(got, lse, want, want_lse, dt, f"seed {seed}: {c}")


@pytest.mark.parametrize("seed", range(12))
def test_decode_random_shape(seed):
    """Split-KV decode, contiguous and paged, arbitrary split lengths, ragged lengths with empty sequences."""
    rng = random.Random(2000 + seed)
    dt = rng.choice([torch.bfloat16, torch.float16])
    B, hkv, group = rng.randint(1, 5), rng.choice([1, 2, 4]), rng.choice([1, 2, 4, 8])
    d_ = rng.choice([64, 128])
    lq = rng.choice([1, 1, 2, 4]) if group <= 4 else 1
    pages, page = rng.randint(1, 12), 64 * rng.randint(1, 3)
    S = pages * page
    q = randn((B, lq, hkv * group, d_), dt, seed + 11)
    k = randn((B, S, hkv, d_), dt, seed + 12)
    v = randn((B, S, hkv, d_), dt, seed + 13)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(0, S + 1, (B,), generator=g).to(torch.int32)
    sc = 1 / math.sqrt(d_)
    want, want_lse = oracle.xla_attention(q, k, v, kv_lengths=lens, sm_scale=sc, return_lse=True)
    d = dev()
    for split_len in (0, 64, 64 * rng.randint(2, 9)):
        got, lse = pj.decode_forward(q.to(d), k.to(d), v.to(d), kv_lengths=lens.to(d), sm_scale=sc, split_len=split_len,
                                     return_lse=True)
        assert_close(got, lse, want, want_lse, dt, f"seed {seed}: decode split_len {split_len}")
    perm = torch.stack([torch.randperm(pages, generator=g) + i * pages for i in range(B)])
    kp = torch.empty((B * pages, page, hkv, d_), dtype=dt)
    vp = torch.empty_like(kp)
    for i in range(B):
        for pg in range(pages):
            kp[perm[i, pg]] = k[i, pg * page:(pg + 1) * page]
            vp[perm[i, pg]] = v[i, pg * page:(pg + 1) * page]
    got, lse = pj.decode_paged(q.to(d), kp.to(d), vp.to(d), perm.to(torch.int32), lens, sm_scale=sc, return_lse=True)
    assert_close(got, lse, want, want_lse, dt, f"seed {seed}: paged decode")


@pytest.mark.parametrize("seed", range(8))
def test_latent_decode_random_shape(seed):
    """Absorbed latent decode on both kernels: widths 128 .. 576, head counts that need several row
    groups, several query tokens, ragged lengths, NaN beyond the lengths."""
    rng = random.Random(3000 + seed)
    dt = rng.choice([torch.bfloat16, torch.float16])
    R = rng.choice([128, 256, 512, 576])
    lq = rng.choice([1, 1, 2, 3])
    H = rng.choice([1, 4, 7, 16, 24, 40])
    B, S = rng.randint(1, 4), rng.randint(1, 1200)
    q = randn((B, lq, H, R), dt, seed + 21)
    cache = (randn((B, S, R), torch.float32, seed + 22) * 0.5).to(dt)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(0, S + 1, (B,), generator=g).to(torch.int32)
    sc = 1 / math.sqrt(R)
    shared = cache[:, :, None, :]
    want, want_lse = oracle.xla_attention(q, shared, shared, kv_lengths=lens, sm_scale=sc, return_lse=True)
    poisoned = cache.clone()
    for b in range(B):
        poisoned[b, int(lens[b]):] = float("nan")
    d = dev()
    for impl in ("b200:tcgen05", "b200:generic"):
        for split_len in (0, 128, 64 * rng.randint(1, 12)):
            got, lse = pj.mla_decode(q.to(d), poisoned.to(d), kv_lengths=lens.to(d), sm_scale=sc, split_len=split_len,
                                     return_lse=True, impl=impl)
            pj.check_status(d)
            assert_close(got, lse, want, want_lse, dt, f"seed {seed}: {impl} R={R} H={H} Lq={lq} S={S} split_len {split_len}")


@pytest.mark.parametrize("seed", range(8))
def test_backward_random_shape(seed):
    """dQ, dK, dV at random shapes (tcgen05 kernels for 16-bit D in {64, 128}, exact kernels otherwise)
    against float64 autograd of the dense formula."""
    rng = random.Random(4000 + seed)
    dt = rng.choice([torch.bfloat16, torch.float32, torch.float16])
    hkv, group = rng.choice([1, 2]), rng.choice([1, 2, 4])
    d_ = rng.choice([64, 128]) if dt != torch.float32 else rng.choice([16, 32, 64])
    B, Lq = rng.randint(1, 2), rng.randint(1, 260)
    causal = rng.random() < 0.5
    Lkv = Lq if causal else rng.randint(1, 300)
    q = randn((B, Lq, hkv * group, d_), dt, seed + 31)
    k = randn((B, Lkv, hkv, d_), dt, seed + 32)
    v = randn((B, Lkv, hkv, d_), dt, seed + 33)
    go = randn((B, Lq, hkv * group, d_), dt, seed + 34)
    sc = 1 / math.sqrt(d_)
    d = dev()
    qd, kd, vd = (x.to(d).requires_grad_(True) for x in (q, k, v))
    out = pj.mha(qd, kd, vd, mask=M.CausalMask() if causal else None, sm_scale=sc)
    out.backward(go.to(d))
    pj.check_status(d)
    q64, k64, v64 = (x.double().requires_grad_(True) for x in (q, k, v))
    s = torch.einsum("bqhd,bkhd->bhqk", q64, k64.repeat_interleave(group, 2)) * sc
    if causal:
        s = s.masked_fill(~torch.tril(torch.ones(Lq, Lkv, dtype=torch.bool)), -math.inf)
    o64 = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v64.repeat_interleave(group, 2))
    o64.backward(go.double())
    tol = 1e-4 if dt == torch.float32 else 3e-2
    for name, a, w in (("dq", qd.grad, q64.grad), ("dk", kd.grad, k64.grad), ("dv", vd.grad, v64.grad)):
        rel = float((a.double().cpu() - w).norm() / w.norm().clamp_min(1e-30))
        assert rel <= tol, f"seed {seed} {dt} B{B} Lq{Lq} Lkv{Lkv} H{hkv}x{group} D{d_} causal={causal}: {name} rel {rel:.3e}"
