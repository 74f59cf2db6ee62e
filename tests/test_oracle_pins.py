"""Pins the CPU oracle against the known-answer formulas of the reference's own
tests (the reference needs jax and cannot run offline; see oracle/__init__.py).

Each test names the reference test it restates.  Inputs are seeded normals of the
reference test's shapes; the expected value is an independent float64 formula.
"""

import math
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from oracle.attention_oracle import LOG2E

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402


def _inputs(b, lq, lkv, hq, hkv, d, seed=0, dtype=torch.float32, dv=None):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, lq, hq, d, generator=g).to(dtype)
    k = torch.randn(b, lkv, hkv, d, generator=g).to(dtype)
    v = torch.randn(b, lkv, hkv, dv or d, generator=g).to(dtype)
    return q, k, v


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _tril(lq, lk):
    return torch.tril(torch.ones(lq, lk, dtype=torch.bool))[None, None]


# tests/test_attention_gqa_splitkv.py:83-97 -- flex GQA vs the dense repeat formula
@pytest.mark.parametrize("hkv", [1, 2])
@pytest.mark.parametrize("causal", [False, True])
def test_gqa_matches_dense_formula(hkv, causal):
    q, k, v = _inputs(2, 40, 40, 4, hkv, 16, seed=hkv)
    got = oracle.xla_attention(q, k, v, causal=causal, sm_scale=1 / math.sqrt(16))
    want, _ = oracle.dense_formula(q, k, v, sm_scale=1 / math.sqrt(16), keep=_tril(40, 40) if causal else None)
    assert _rel(got, want) < 1e-5


# tests/test_attention_gqa_splitkv.py:175-201 -- split-KV output and natural-log LSE
@pytest.mark.parametrize(
    "b,lq,lkv,hq,hkv,d,splits",
    [(1, 1, 200, 4, 4, 16, 4), (2, 3, 130, 4, 2, 16, 3), (1, 4, 96, 8, 1, 32, 2), (1, 2, 50, 2, 1, 24, 1)],
)
def test_splitkv_output_and_lse(b, lq, lkv, hq, hkv, d, splits):
    q, k, v = _inputs(b, lq, lkv, hq, hkv, d, seed=lkv)
    out, lse, _, _ = oracle.splitkv_reference(q, k, v, sm_scale=1 / math.sqrt(d), num_splits=splits)
    want, want_lse = oracle.dense_formula(q, k, v, sm_scale=1 / math.sqrt(d))
    assert out.shape == q.shape
    assert _rel(out, want) < 1e-5
    # logsumexp of the scaled scores, natural log, [B, Hq, Lq]
    kr = torch.repeat_interleave(k, hq // hkv, dim=2).double()
    s = torch.einsum("bqhd,bkhd->bhqk", q.double(), kr) / math.sqrt(d)
    np.testing.assert_allclose(lse.numpy(), torch.logsumexp(s, -1).numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(want_lse.numpy(), torch.logsumexp(s, -1).numpy(), rtol=1e-10, atol=1e-10)


# tests/test_attention_gqa_splitkv.py:235-243 -- decode shapes on the CPU path
@pytest.mark.parametrize("lq", [1, 4])
@pytest.mark.parametrize("lkv", [300, 1000])
def test_decode_shapes(lq, lkv):
    q, k, v = _inputs(1, lq, lkv, 8, 2, 32, seed=lq * lkv)
    got = oracle.xla_attention(q, k, v, sm_scale=1 / math.sqrt(32))
    want, _ = oracle.dense_formula(q, k, v, sm_scale=1 / math.sqrt(32))
    assert _rel(got, want) < 1e-5


# tests/test_attention_xla.py:91-147 -- kvlen and kvlen & causal masks, B2 T32 H2 D16, scale 0.25
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("strategy", ["dense", "tiled"])
def test_kvlen_masks(causal, strategy):
    q, k, v = _inputs(2, 32, 32, 2, 2, 16, seed=3)
    lengths = torch.tensor([20, 32])
    keep = (torch.arange(32)[None, :] < lengths[:, None])[:, None, None, :]
    if causal:
        keep = keep & _tril(32, 32)
    got = oracle.xla_attention(q, k, v, causal=causal, kv_lengths=lengths, sm_scale=0.25, strategy=strategy,
                               block_q=16, block_k=16)
    want, _ = oracle.dense_formula(q, k, v, sm_scale=0.25, keep=keep)
    assert _rel(got, want) < 1e-5


# tests/test_attention_xla.py:108-179, 208-223 -- dense bias [B,H,T,T] and broadcast [1,1,T,T], Lq40 Lkv24
@pytest.mark.parametrize("bshape", [(2, 2), (1, 1), (1, 2)])
def test_dense_bias_is_added_after_scaling(bshape):
    q, k, v = _inputs(2, 40, 24, 2, 2, 16, seed=5)
    bias = torch.randn(*bshape, 40, 24, generator=torch.Generator().manual_seed(9))
    got = oracle.xla_attention(q, k, v, bias=bias, sm_scale=0.25)
    want, _ = oracle.dense_formula(q, k, v, sm_scale=0.25, bias=bias)
    assert _rel(got, want) < 1e-5
    # the bias is not scaled: doubling sm_scale must not equal doubling the bias
    other = oracle.xla_attention(q, k, v, bias=2 * bias, sm_scale=0.25)
    assert _rel(other, want) > 1e-3


# tests/test_attention_xla.py:241-249, tests/test_attention_device_defaults.py:317-328 -- rows without keys
def test_fully_masked_rows_are_zero_and_finite():
    q, k, v = _inputs(2, 8, 16, 2, 2, 8, seed=1)
    lengths = torch.tensor([0, 16])
    for strategy in ("dense", "tiled"):
        out, lse = oracle.xla_attention(q, k, v, kv_lengths=lengths, sm_scale=1.0, strategy=strategy,
                                        block_q=4, block_k=4, return_lse=True)
        assert torch.isfinite(out).all()
        assert (out[0] == 0).all()
        assert torch.isinf(lse[0]).all() and (lse[0] > 0).all()
        assert torch.isfinite(lse[1]).all()


# tests/test_attention_xla.py:408-421 -- bf16 vs fp32 within 2e-2 relative
def test_bf16_close_to_fp32():
    q, k, v = _inputs(2, 64, 64, 4, 4, 32, seed=11)
    ref = oracle.xla_attention(q, k, v, sm_scale=1 / math.sqrt(32))
    got = oracle.xla_attention(q.bfloat16(), k.bfloat16(), v.bfloat16(), sm_scale=1 / math.sqrt(32))
    assert got.dtype == torch.bfloat16
    assert _rel(got.float(), ref) < 2e-2


# tests/test_attention_xla.py:424-431 -- unaligned S50 D24 causal + dense bias through the tiled strategy
def test_unaligned_tiled():
    q, k, v = _inputs(1, 50, 50, 2, 2, 24, seed=13)
    bias = torch.randn(1, 2, 50, 50, generator=torch.Generator().manual_seed(2))
    got = oracle.xla_attention(q, k, v, causal=True, bias=bias, sm_scale=0.2, strategy="tiled", block_q=16, block_k=16)
    want, _ = oracle.dense_formula(q, k, v, sm_scale=0.2, keep=_tril(50, 50), bias=bias)
    assert _rel(got, want) < 1e-5


def test_strategy_thresholds():
    # attention_xla.py:63-69, 586-592
    assert oracle.auto_strategy(256, 256) == ("dense", None, None)
    assert oracle.auto_strategy(257, 256) == ("tiled", 257, 256)
    assert oracle.auto_strategy(512, 512) == ("tiled", 512, 512)
    assert oracle.auto_strategy(1024, 513) == ("tiled", 256, 256)


def test_tiled_equals_dense_above_threshold():
    q, k, v = _inputs(1, 600, 600, 2, 1, 16, seed=17)
    a = oracle.xla_attention(q, k, v, causal=True, sm_scale=0.25)  # auto -> 256-tiles (balanced to 200)
    b, _ = oracle.dense_formula(q, k, v, sm_scale=0.25, keep=_tril(600, 600))
    assert _rel(a, b) < 1e-5


def test_gqa_head_count_error():
    # tests/test_attention_gqa_splitkv.py:145-148 -- message mentions "multiple"
    q, k, v = _inputs(1, 4, 4, 3, 2, 8)
    with pytest.raises(ValueError, match="multiple"):
        oracle.xla_attention(q, k, v)


# tests/test_latent_attention.py:64-68, 234-258, 300-327 -- materialized and absorbed vs dense softmax
@pytest.mark.parametrize("causal", [False, True])
def test_mla_matches_dense_over_materialized_kv(causal):
    g = torch.Generator().manual_seed(21)
    b, s, h, d, r, dv = 2, 32, 4, 16, 8, 12
    q = torch.randn(b, s, h, d, generator=g)
    cache = torch.randn(b, s, r, generator=g)
    wk = torch.randn(h, d, r, generator=g) * 0.3
    wv = torch.randn(h, dv, r, generator=g) * 0.3
    key, value = oracle.materialize_kv(cache, wk, wv, h)
    want, _ = oracle.dense_formula(q, key, value, sm_scale=1 / math.sqrt(d), keep=_tril(s, s) if causal else None)
    for fact in ("materialized", "absorbed", "auto"):
        got = oracle.mla_reference(q, cache, wk, wv, causal=causal, factorisation=fact)
        assert got.shape == (b, s, h, dv)
        assert float((got.double() - want).abs().max()) < 1e-5
    # absorbed call form: K = V = latent, one shared head
    q2 = torch.randn(b, s, h, r, generator=g)
    got = oracle.mla_reference(q2, cache, causal=causal)
    shared = cache[:, :, None, :]
    want, _ = oracle.dense_formula(q2, shared, shared, sm_scale=1 / math.sqrt(r), keep=_tril(s, s) if causal else None)
    assert float((got.double() - want).abs().max()) < 1e-5


# tests/test_attention_xla.py:458-498 -- CPU MLA path with KVLenMask([20, 32]), q_len in {32, 4}
@pytest.mark.parametrize("q_len", [32, 4])
def test_mla_kvlen(q_len):
    g = torch.Generator().manual_seed(q_len)
    b, s, h, d, r, dv = 2, 32, 2, 16, 8, 16
    q = torch.randn(b, q_len, h, d, generator=g)
    cache = torch.randn(b, s, r, generator=g)
    wk, wv = torch.randn(h, d, r, generator=g), torch.randn(h, dv, r, generator=g)
    lengths = torch.tensor([20, 32])
    keep = (torch.arange(s)[None, :] < lengths[:, None])[:, None, None, :]
    key, value = oracle.materialize_kv(cache, wk, wv, h)
    want, _ = oracle.dense_formula(q, key, value, sm_scale=1 / math.sqrt(d), keep=keep)
    got = oracle.mla_reference(q, cache, wk, wv, kv_lengths=lengths)
    assert float((got.double() - want).abs().max()) < 2e-5


def test_combine_matches_unsplit():
    # attention_splitkv.py:236-250: combining per-split partials reproduces the whole
    q, k, v = _inputs(2, 2, 300, 4, 2, 16, seed=31)
    lengths = torch.tensor([37, 300])
    out, lse, o_part, lse_part = oracle.splitkv_reference(q, k, v, sm_scale=0.25, num_splits=5, kv_lengths=lengths)
    keep = (torch.arange(300)[None, :] < lengths[:, None])[:, None, None, :]
    want, want_lse = oracle.dense_formula(q, k, v, sm_scale=0.25, keep=keep)
    assert _rel(out, want) < 1e-5
    np.testing.assert_allclose(lse.numpy(), want_lse.numpy(), rtol=1e-5, atol=1e-5)
    # splits past a sequence's length are empty: base-2 LSE at the reference's NEG_INF
    assert (lse_part[0, :, 1:] <= -1e15).all()


def test_rope_interleaved_pairs():
    # layers/encoding.py:171-211: pair (x[2i], x[2i+1]) rotated by pos * base^(-2i/D)
    x = torch.randn(1, 5, 2, 8, generator=torch.Generator().manual_seed(0))
    y = oracle.rope_interleaved(x)
    for t in range(5):
        for i in range(4):
            ang = t * (10000.0 ** (-2 * i / 8))
            e, o = x[0, t, 1, 2 * i].item(), x[0, t, 1, 2 * i + 1].item()
            assert abs(y[0, t, 1, 2 * i].item() - (e * math.cos(ang) - o * math.sin(ang))) < 1e-5
            assert abs(y[0, t, 1, 2 * i + 1].item() - (o * math.cos(ang) + e * math.sin(ang))) < 1e-5
    np.testing.assert_allclose(y.norm().item(), x.norm().item(), rtol=1e-5)


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_golden_fixtures_match_oracle(name):
    """The committed fixtures are what the oracle produces today, from the same inputs."""
    fx = np.load(os.path.join(os.path.dirname(__file__), "golden", f"{name}.npz"))
    inp = cases.make_inputs(name)
    sums = cases.input_checksums(inp)
    for key, val in zip(fx["checksum_keys"], fx["checksum_vals"]):
        assert sums[str(key)] == pytest.approx(float(val), rel=1e-12, abs=1e-9)
    out, lse = cases.oracle_outputs(name, inp)
    tol = 1e-6 if cases.CASES[name]["dtype"] == "f32" else 2e-3
    np.testing.assert_allclose(out.numpy(), fx["out"].astype(np.float32), atol=tol, rtol=tol)
    np.testing.assert_allclose(lse.numpy(), fx["lse"], atol=1e-5, rtol=1e-5)


def test_config_generator_shapes():
    c = oracle.make_config(2, B=1, S=128)
    assert c["q"].shape == (1, 128, 32, 128) and c["k"].shape == (1, 128, 8, 128) and c["q"].dtype == torch.bfloat16
    c = oracle.make_config(4, B=2, cap=512)
    assert c["k"].shape == (2, 512, 8, 128) and int(c["kv_lengths"].max()) <= 512
    c = oracle.make_config(5, B=1, S=64, d_model=128)
    assert c["q"].shape == (1, 64, 16, 192) and c["cache"].shape == (1, 64, 576)
    assert c["wk"].shape == (16, 192, 576) and c["wv"].shape == (16, 128, 576)
    assert LOG2E == pytest.approx(1 / math.log(2))


def _hash_u32(seed, b, h, q, k):
    """`_dropout_mask_counter` (kernels/attention.py:116-148) in Python integers, one element."""
    m = 0xFFFFFFFF
    x = seed & m
    x ^= (b * 0x85EBCA6B) & m
    x ^= (h * 0xC2B2AE35) & m
    x ^= (q * 0x27D4EB2F) & m
    x ^= (k * 0x165667B1) & m
    x ^= x >> 16
    x = (x * 0x7FEB352D) & m
    x ^= x >> 15
    x = (x * 0x846CA68B) & m
    x ^= x >> 16
    return x


# tests/test_attention_xla.py:226-237 -- counter dropout: the same mask on every strategy
def test_counter_dropout_hash_and_seed_folding():
    seed = oracle.rng_seed_from_key([0, 11])  # the two words of jax.random.key(11) under threefry
    assert seed == (11 * 0x9E3779B9) & 0xFFFFFFFF
    assert oracle.rng_seed_from_key(5) == 5
    assert oracle.rng_seed_from_key([1, 2, 3, 4]) == (
        1 ^ ((2 * 0x9E3779B9) & 0xFFFFFFFF) ^ ((3 * (0x85EBCA6B + 2)) & 0xFFFFFFFF) ^ ((4 * (0x85EBCA6B + 3)) & 0xFFFFFFFF))
    rate = 0.3
    scale = oracle.counter_dropout_scale(seed, 2, 3, torch.arange(5, 45), torch.arange(64), rate)
    assert scale.shape == (2, 3, 40, 64) and scale.dtype == torch.float32
    for b, h, qi, kj in [(0, 0, 0, 0), (1, 2, 39, 63), (1, 0, 7, 31), (0, 1, 20, 5)]:
        u = np.float32(_hash_u32(seed, b, h, 5 + qi, kj)) * np.float32(2.0 ** -32)
        want = 0.0 if u < np.float32(rate) else np.float32(1.0 / (1.0 - rate))
        assert float(scale[b, h, qi, kj]) == float(want)
    dropped = float((scale == 0).float().mean())
    assert abs(dropped - rate) < 0.02, dropped
    # every (batch, head) plane differs
    assert not torch.equal(scale[0, 0], scale[0, 1]) and not torch.equal(scale[0, 0], scale[1, 0])


@pytest.mark.parametrize("causal", [False, True])
def test_counter_dropout_tiled_equals_dense(causal):
    q, k, v = _inputs(2, 40, 56, 4, 2, 16, seed=21)
    seed, rate = 1234567, 0.3
    kw = dict(causal=causal, sm_scale=0.25, dropout=(seed, rate), return_lse=True)
    a, la = oracle.xla_attention(q, k, v, strategy="dense", **kw)
    b, lb = oracle.xla_attention(q, k, v, strategy="tiled", block_q=16, block_k=16, **kw)
    assert _rel(a, b) < 1e-5 and torch.allclose(la, lb, atol=1e-5)
    plain, lp = oracle.xla_attention(q, k, v, causal=causal, sm_scale=0.25, return_lse=True)
    assert torch.allclose(la, lp, atol=1e-6)  # the normaliser ignores dropout
    assert _rel(a, plain) > 1e-2
    # E[dropout(p)] = p: averaged over many seeds the output approaches the undropped one
    acc = sum(oracle.xla_attention(q, k, v, causal=causal, sm_scale=0.25, dropout=(s, rate)) for s in range(200)) / 200
    assert _rel(acc, plain) < 0.12
