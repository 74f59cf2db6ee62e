"""The reference call signatures end to end on the GPU, and size-independent
properties at the benchmark's full sizes."""

import math

import pytest
import torch

import oracle
import probjax_b200 as pj
from _gpu_util import assert_close, dev, oracle_fwd, randn

pytestmark = pytest.mark.gpu


def test_flex_attention_masks_and_bias_objects():
    d = dev()
    b, t, h, dd = 2, 32, 2, 16  # tests/test_attention_xla.py:91-147 (B2 T32 H2 D16, scale 0.25)
    q, k, v = (randn((b, t, h, dd), torch.float32, s) for s in (1, 2, 3))
    lens = torch.tensor([20, 32], dtype=torch.int32)
    bias = randn((b, h, t, t), torch.float32, 4)
    for mask, kw in [
        (None, {}),
        (pj.NoMask(), {}),
        (pj.CausalMask(), dict(causal=True)),
        (pj.KVLenMask(lens), dict(kv_lengths=lens)),
        (pj.KVLenMask(lens) & pj.CausalMask(), dict(kv_lengths=lens, causal=True)),
    ]:
        for bobj, bkw in [(None, {}), (pj.DenseBias(bias), dict(bias=bias)), (pj.DenseBias(bias[:1, :1]), dict(bias=bias[:1, :1]))]:
            got, lse = pj.flex_attention(q.to(d), k.to(d), v.to(d), mask=mask, bias=bobj, sm_scale=0.25, return_lse=True)
            want, want_lse = oracle_fwd(q, k, v, sm_scale=0.25, **kw, **bkw)
            assert_close(got, lse, want, want_lse, torch.float32, f"{type(mask).__name__} {bool(bobj)}")


def test_default_scale_rank3_and_extra_batch_dims():
    d = dev()
    q, k, v = (randn((40, 4, 16), torch.float32, s) for s in (1, 2, 3))
    got = pj.flex_attention(q.to(d), k.to(d), v.to(d), mask=pj.CausalMask())
    want, _ = oracle_fwd(q[None], k[None], v[None], causal=True, sm_scale=1 / 4.0)  # layers/attention.py:1524-1525
    assert got.shape == (40, 4, 16)
    assert_close(got[None], None, want, None, torch.float32, "rank 3")
    q5 = randn((2, 3, 20, 4, 16), torch.float32, 5)
    got = pj.dot_product_attention(q5.to(d), q5.to(d)[..., :2, :], q5.to(d)[..., :2, :])  # GQA like Flax
    want, _ = oracle_fwd(q5.reshape(6, 20, 4, 16), q5.reshape(6, 20, 4, 16)[..., :2, :], q5.reshape(6, 20, 4, 16)[..., :2, :], sm_scale=0.25)
    assert got.shape == q5.shape
    assert_close(got.reshape(6, 20, 4, 16), None, want, None, torch.float32, "rank 5")


def test_dot_product_attention_takes_dense_mask_and_bias_arrays():
    """The Flax-style call (layers/attention.py:1293-1319): boolean mask and additive bias given as
    arrays broadcastable to [*batch, H, Q, K], with extra batch dimensions and fewer K/V heads."""
    d = dev()
    q = randn((2, 3, 24, 4, 16), torch.float32, 1)
    k, v = randn((2, 3, 30, 2, 16), torch.float32, 2), randn((2, 3, 30, 2, 16), torch.float32, 3)
    g = torch.Generator().manual_seed(4)
    keep = torch.rand((2, 3, 1, 24, 30), generator=g) > 0.3   # per batch element, shared by the heads
    keep[..., 0] = True                                      # every row keeps at least one key
    bias = randn((4, 24, 30), torch.float32, 5)               # per head, shared by the batch
    got = pj.dot_product_attention(q.to(d), k.to(d), v.to(d), mask=keep.to(d), bias=bias.to(d))
    want, _ = oracle_fwd(q.reshape(6, 24, 4, 16), k.reshape(6, 30, 2, 16), v.reshape(6, 30, 2, 16),
                         keep=keep.reshape(6, 1, 24, 30), bias=bias[None], sm_scale=0.25)
    assert got.shape == q.shape
    assert_close(got.reshape(6, 24, 4, 16), None, want, None, torch.float32, "dense arrays")
    # an array bias together with a mask object
    got = pj.dot_product_attention(q[0].to(d), k[0].to(d), v[0].to(d), mask=pj.CausalMask(), bias=bias.to(d))
    want, _ = oracle_fwd(q[0], k[0], v[0], causal=True, bias=bias[None], sm_scale=0.25)
    assert_close(got, None, want, None, torch.float32, "array bias with a mask object")


def test_mha_defaults_and_padding_mask():
    d = dev()
    q, k, v = (randn((1, 50, 2, 24), torch.float32, s) for s in (1, 2, 3))
    got = pj.mha(q.to(d), k.to(d), v.to(d))  # default sm_scale = 1.0 (kernels/attention.py:2699)
    want, _ = oracle_fwd(q, k, v, sm_scale=1.0)
    assert_close(got, None, want, None, torch.float32, "mha default scale")
    # QKVLengthMask: rows past q_length see nothing, keys past kv_length are masked
    m = pj.QKVLengthMask(q_length=30, kv_length=41)
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=m, sm_scale=0.2, return_lse=True)
    keep = m.dense(50, 50)
    want, want_lse = oracle_fwd(q, k, v, keep=keep, sm_scale=0.2)
    assert_close(got, lse, want, want_lse, torch.float32, "QKVLengthMask")
    with pytest.raises(NotImplementedError):  # only the counter-hash dropout is a kernel path
        pj.mha(q.to(d), k.to(d), v.to(d), rng=1, dropout_rate=0.1, dropout_impl="materialize")


def test_mha_flash_signature():
    # flash_attention3.py:344-397: KVLenMask or none, causal flag, no bias / other masks
    d = dev()
    q, k = randn((2, 200, 4, 128), torch.bfloat16, 1), randn((2, 200, 2, 128), torch.bfloat16, 2)
    lens = torch.tensor([200, 77], dtype=torch.int32)
    got, lse = pj.mha_flash(q.to(d), k.to(d), k.to(d), mask=pj.KVLenMask(lens), causal=True, enable_gqa=True,
                            save_residuals=True)
    want, want_lse = oracle_fwd(q, k, k, causal=True, kv_lengths=lens, sm_scale=1 / math.sqrt(128))
    assert_close(got, lse, want, want_lse, torch.bfloat16, "mha_flash")
    with pytest.raises(NotImplementedError, match="causal=True"):
        pj.mha_flash(q.to(d), k.to(d), k.to(d), mask=pj.CausalMask(), enable_gqa=True)
    with pytest.raises(NotImplementedError, match="bias"):
        pj.mha_flash(q.to(d), k.to(d), k.to(d), bias=pj.DenseBias(torch.zeros(1, 1, 200, 200)), enable_gqa=True)


def test_dispatch_route():
    d = dev()
    assert pj.device_attention_defaults(d)["route"] == "b200"
    q, k = randn((2, 64, 4, 64), torch.bfloat16, 1), randn((2, 64, 2, 64), torch.bfloat16, 2)
    got = pj.b200_attention_or_none(q.to(d), k.to(d), k.to(d), mask=pj.CausalMask(), sm_scale=0.125)
    want, _ = oracle_fwd(q, k, k, causal=True, sm_scale=0.125)
    assert_close(got, None, want, None, torch.bfloat16, "route")
    # a mask the kernels do not implement: "not mine", or ValueError when forced
    kp = pj.KeyPaddingMask(torch.tensor([3, 9]))
    assert pj.b200_attention_or_none(q.to(d), k.to(d), k.to(d), mask=kp, sm_scale=1.0) is None
    with pytest.raises(ValueError, match="cannot compute"):
        pj.b200_attention_or_none(q.to(d), k.to(d), k.to(d), mask=kp, sm_scale=1.0, force=True)
    assert pj.b200_attention_or_none(q.to(d), k.to(d), k.to(d), dropout_rate=0.1, sm_scale=1.0) is None


def test_split_kv_routing_rule():
    # kernels/attention.py:2649-2689: Lq <= 64 and Lkv >= 1024 picks split-KV; KVLenMask keeps it
    from probjax_b200 import _lib

    d = dev()
    q = randn((2, 1, 8, 128), torch.bfloat16, 1).to(d)
    k = randn((2, 1100, 2, 128), torch.bfloat16, 2).to(d)
    assert pj.use_splitkv(q, k) and not pj.use_splitkv(q, k[:, :1000]) and pj.use_splitkv(q, k[:, :1000], split_kv=True)
    assert not pj.use_splitkv(q, k, causal=True) and not pj.use_splitkv(q, k, split_kv=False)
    lens = torch.tensor([1100, 300], dtype=torch.int32)
    n0 = _lib.launch_count()
    got, lse = pj.flex_attention(q, k, k, mask=pj.KVLenMask(lens), enable_gqa=True, return_lse=True)
    assert _lib.launch_count() == n0 + 2  # split kernel + combine
    want, want_lse = oracle_fwd(q, k, k, kv_lengths=lens, sm_scale=1 / math.sqrt(128))
    assert_close(got, lse, want, want_lse, torch.bfloat16, "split-KV route")
    # decode step as MultiHeadAttention issues it: KeyPaddingMask with one query row (layers/attention.py:658-673)
    got = pj.flex_attention(q, k, k, mask=pj.KeyPaddingMask(lens), enable_gqa=True)
    assert_close(got, None, want, None, torch.bfloat16, "KeyPaddingMask decode")


def test_mla_absorbed_and_small_shapes():
    d = dev()
    g = torch.Generator().manual_seed(21)  # tests/test_latent_attention.py:234-258 (b2 s32 h4 d16 r8 dv12)
    b, s, h, dd, r, dv = 2, 32, 4, 16, 8, 12
    q, cache = torch.randn(b, s, h, dd, generator=g), torch.randn(b, s, r, generator=g)
    wk, wv = torch.randn(h, dd, r, generator=g) * 0.3, torch.randn(h, dv, r, generator=g) * 0.3
    for mask, kw in [(None, {}), (pj.CausalMask(), dict(causal=True)), (pj.KVLenMask(torch.tensor([20, 32])), dict(kv_lengths=torch.tensor([20, 32])))]:
        got = pj.mla(q.to(d), cache.to(d), wk.to(d), wv.to(d), mask=mask)
        want = oracle.mla_reference(q, cache, wk, wv, **kw)
        assert got.shape == (b, s, h, dv)
        assert float((got.cpu() - want).abs().max()) < 1e-4
    q2 = torch.randn(b, s, h, r, generator=g)
    got = pj.mla(q2.to(d), cache.to(d), mask=pj.CausalMask())
    want = oracle.mla_reference(q2, cache, causal=True)
    assert float((got.cpu() - want).abs().max()) < 1e-4


def _row_sample_check(q, k, v, out, lse, rows, causal, sc, kv_lengths=None, bias=None):
    """Oracle comparison on a sample of query rows of a large problem."""
    qs = q[:, rows].cpu()
    lkv = k.shape[1]
    keep = torch.ones(1, 1, len(rows), lkv, dtype=torch.bool)
    if causal:
        keep = keep & (torch.arange(lkv)[None, :] <= torch.tensor(rows)[:, None])[None, None]
    if kv_lengths is not None:
        keep = keep & (torch.arange(lkv)[None, :] < kv_lengths.cpu()[:, None])[:, None, None, :]
    b = None if bias is None else bias[:, :, rows].cpu()
    want, want_lse = oracle.dense_formula(qs, k.cpu(), v.cpu(), sm_scale=sc, keep=keep, bias=b)
    assert_close(out[:, rows], lse[:, :, rows], want.float(), want_lse.float(), q.dtype, "row sample")


@pytest.mark.parametrize("causal", [False, True])
def test_full_size_gqa_prefill_properties(causal):
    """Configuration 2 at full size (B4 Hq32 Hkv8 S4096 D128): normalisation
    (V = 1 gives exactly 1), linearity in V, and oracle parity on sampled rows."""
    d = dev()
    c = oracle.make_config(2, causal=causal)
    q, k, v = c["q"].to(d), c["k"].to(d), c["v"].to(d)
    out, lse = pj.attention_forward(q, k, v, causal=causal, sm_scale=c["sm_scale"], return_lse=True)
    pj.check_status(d)
    ones = pj.attention_forward(q, k, torch.ones_like(v), causal=causal, sm_scale=c["sm_scale"])
    assert float((ones.float() - 1).abs().max()) <= 8e-3  # bf16 rounding of P and of the output
    twice = pj.attention_forward(q, k, v * 2, causal=causal, sm_scale=c["sm_scale"])
    assert torch.equal(twice, out * 2)  # scaling V by a power of two is exact
    rows = [0, 1, 127, 128, 129, 255, 256, 1000, 2047, 2048, 3000, 4095]
    _row_sample_check(q[:1], k[:1], v[:1], out[:1], lse[:1], rows, causal, c["sm_scale"])
    _row_sample_check(q[3:], k[3:], v[3:], out[3:], lse[3:], rows, causal, c["sm_scale"])


def test_full_size_masked_biased_attention():
    """Configuration 3 at full size (B8 H16 S1024 D64, key lengths + fp32 bias)."""
    d = dev()
    c = oracle.make_config(3)
    q, k, v = c["q"].to(d), c["k"].to(d), c["v"].to(d)
    out, lse = pj.flex_attention(q, k, v, mask=pj.KVLenMask(c["kv_lengths"]), bias=pj.DenseBias(c["bias"]),
                                 sm_scale=c["sm_scale"], return_lse=True)
    pj.check_status(d)
    rows = [0, 63, 64, 500, 1023]
    _row_sample_check(q, k, v, out, lse, rows, False, c["sm_scale"], kv_lengths=c["kv_lengths"], bias=c["bias"])


def test_full_size_decode():
    """Configuration 4 at full size (B16 Hq32 Hkv8 D128, capacity 32768, ragged):
    oracle parity for every row (one query row per sequence keeps the oracle cheap)."""
    d = dev()
    c = oracle.make_config(4)
    q, k, v = c["q"].to(d), c["k"].to(d), c["v"].to(d)
    out, lse = pj.flex_attention(q, k, v, mask=pj.KVLenMask(c["kv_lengths"]), enable_gqa=True, return_lse=True)
    want, want_lse = oracle_fwd(c["q"], c["k"], c["v"], kv_lengths=c["kv_lengths"], sm_scale=c["sm_scale"])
    assert_close(out, lse, want, want_lse, torch.bfloat16, "config 4")


def test_full_size_latent_attention():
    """Configuration 5 at full size (B8 H16 S2048, rank 512 + rotary 64): sampled rows
    against the dense formula over the materialised keys and values of one batch row."""
    d = dev()
    c = oracle.make_config(5)
    out, lse = pj.mla(c["q"].to(d), c["cache"].to(d), c["wk"].to(d), c["wv"].to(d), mask=pj.CausalMask(),
                      sm_scale=c["sm_scale"], return_lse=True)
    pj.check_status(d)
    key, value = oracle.materialize_kv(c["cache"][:1], c["wk"], c["wv"], 16)
    rows = [0, 1, 127, 128, 700, 2047]
    _row_sample_check(c["q"][:1], key, value, out[:1], lse[:1], rows, True, c["sm_scale"])


@pytest.mark.parametrize("dtype,shape,rot", [
    (torch.float32, (2, 300, 3, 64), None),
    (torch.bfloat16, (1, 2048, 1, 64), None),      # the decoupled rotary key of the latent configuration
    (torch.float16, (2, 100, 4, 128), 64),         # partial rotary width: the tail is copied
])
def test_rope_interleaved_matches_the_oracle(dtype, shape, rot):
    """pjx_rope_interleaved against the oracle's restatement of layers/encoding.py:171-211."""
    x = randn(shape, dtype, 7)
    got = pj.rope_interleaved(x.to(dev()), rotary_dim=rot)
    want = x.clone().float()
    r = shape[-1] if rot is None else rot
    want[..., :r] = oracle.rope_interleaved(x[..., :r].float())
    # fp32 angles of a few thousand radians: the device's sin / cos arguments differ from the host's in the last bits
    tol = 2e-3 if dtype == torch.float32 else 3e-2
    assert float((got.float().cpu() - want).abs().max()) <= tol
    if rot is not None:
        assert torch.equal(got[..., r:].cpu(), x[..., r:])
    # explicit positions and an offset agree with each other
    pos = torch.arange(shape[1], dtype=torch.float32) + 5.0
    a = pj.rope_interleaved(x.to(dev()), positions=pos, rotary_dim=rot)
    b = pj.rope_interleaved(x.to(dev()), offset=5.0, rotary_dim=rot)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,m,n,k", [(torch.bfloat16, 300, 520, 192), (torch.float16, 1000, 256, 64), (torch.float32, 70, 33, 20)])
def test_linear_projection(dtype, m, n, k):
    """pjx_linear (the projections around the attention call) against a float64 product."""
    x, w = randn((2, m // 2, k), dtype, 1), (randn((n, k), dtype, 2) / math.sqrt(k)).to(dtype)
    got = pj.linear(x.to(dev()), w.to(dev()))
    pj.check_status()
    want = x.double() @ w.double().t()
    assert got.shape == (2, m // 2, n)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got.double().cpu() - want).abs().max()) <= tol


def _layer_reference(layer, x_q, x_kv, *, causal):
    """float64 restatement of the layer's forward (layers/latent_attention.py:424-481, 640-709) on the
    layer's own (rounded) weights."""
    f = lambda t: None if t is None else t.detach().double().cpu()
    wkv_a, wq, wk, wv, wo = f(layer.wkv_a), f(layer.wq), f(layer.wk), f(layer.wv), f(layer.wo)
    x_q, x_kv = x_q.double(), x_kv.double()
    latent = x_kv @ wkv_a.t()
    if layer.latent_norm_scale is not None:
        latent = latent * torch.rsqrt((latent ** 2).mean(-1, keepdim=True) + layer.eps) * f(layer.latent_norm_scale)
    h, dqk = layer.num_heads, layer.qk_head_dim
    q = (x_q @ wq.t()).reshape(x_q.shape[0], x_q.shape[1], h, dqk)
    if layer.mode == "materialized":
        key = torch.einsum("bsr,hdr->bshd", latent, wk)
        val = torch.einsum("bsr,hdr->bshd", latent, wv)
    else:
        key = val = latent[:, :, None, :].expand(-1, -1, h, -1)
    s = torch.einsum("bqhd,bkhd->bhqk", q, key) / math.sqrt(dqk)
    if causal:
        s = s.masked_fill(~torch.tril(torch.ones(s.shape[-2], s.shape[-1], dtype=torch.bool)), -math.inf)
    attn = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), val)
    if layer.mode == "absorbed" and wv is not None:
        attn = torch.einsum("bqhr,hdr->bqhd", attn, wv)
    return attn.reshape(attn.shape[0], attn.shape[1], -1) @ wo.t()


@pytest.mark.parametrize("mode,kw", [("materialized", dict(qk_head_dim=128, v_head_dim=128)),
                                     ("absorbed", dict(v_head_dim=64)),
                                     ("absorbed", dict(value_projection=False))])
def test_latent_attention_layer_steps(mode, kw):
    """The layer around the latent kernel: encoder + RMS norm, query projection, attention, the value
    projection folded onto the absorbed output, output projection -- every step a kernel of the library."""
    from probjax_b200.latent_layer import MultiHeadLatentAttention

    d = dev()
    layer = MultiHeadLatentAttention(4, 256, kv_lora_rank=128, mode=mode, out_features=192, device=d, seed=3, **kw)
    x = randn((2, 200, 256), torch.bfloat16, 9)
    n0 = pj._lib.launch_count()
    got = layer(x.to(d), mask=pj.CausalMask())
    assert pj._lib.launch_count() - n0 >= 5  # encoder, norm, query projection, attention, output projection
    pj.check_status(d)
    want = _layer_reference(layer, x, x, causal=True)
    rel = float((got.double().cpu() - want).norm() / want.norm())
    assert got.shape == (2, 200, 192) and rel <= 2e-2, f"{mode} {kw}: relative error {rel:.3e}"


def test_latent_attention_layer_dropout():
    """Dropout through the layer: off under `deterministic=True`, reproducible for a given key, different
    from call to call on the kept stream."""
    from probjax_b200.latent_layer import MultiHeadLatentAttention

    d = dev()
    kw = dict(kv_lora_rank=128, mode="absorbed", v_head_dim=64, out_features=192, device=d, seed=3)
    plain = MultiHeadLatentAttention(4, 256, **kw)
    layer = MultiHeadLatentAttention(4, 256, dropout_rate=0.2, **kw)
    x = randn((2, 200, 256), torch.bfloat16, 9).to(d)
    base = plain(x, mask=pj.CausalMask())
    assert torch.equal(layer(x, mask=pj.CausalMask(), deterministic=True), base)
    a = layer(x, mask=pj.CausalMask(), deterministic=False, rng=[3, 4])
    b = layer(x, mask=pj.CausalMask(), deterministic=False, rng=[3, 4])
    c = layer(x, mask=pj.CausalMask(), deterministic=False)
    e = layer(x, mask=pj.CausalMask(), deterministic=False)
    pj.check_status(d)
    assert torch.equal(a, b) and not torch.equal(a, base) and not torch.equal(c, e)
    assert bool(torch.isfinite(a).all())
    # dropout is unbiased: the difference to the deterministic output averages out
    assert abs(float((a.float() - base.float()).mean())) < 0.05 * float(base.float().abs().mean())


def test_rms_norm_and_per_head_linear():
    from probjax_b200.latent_layer import per_head_linear, rms_norm

    d = dev()
    for dtype, width, tol in ((torch.float32, 100, 1e-5), (torch.bfloat16, 512, 1e-2), (torch.float16, 576, 2e-3)):
        x = randn((7, 33, width), dtype, 1)
        scale = torch.rand(width, generator=torch.Generator().manual_seed(2)) + 0.5
        got = rms_norm(x.to(d), scale.to(d), eps=1e-6)
        want = x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6) * scale.double()
        assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
        assert torch.equal(rms_norm(x.to(d)), rms_norm(x.to(d), torch.ones(width)))
    for dtype, (h, n, k), tol in ((torch.bfloat16, (3, 128, 512), 2e-2), (torch.float32, (2, 24, 40), 1e-5),
                                  (torch.float16, (4, 72, 64), 5e-3)):
        x, w = randn((5, 31, h, k), dtype, 3), (randn((h, n, k), dtype, 4).float() / math.sqrt(k)).to(dtype)
        got = per_head_linear(x.to(d), w.to(d))
        want = torch.einsum("bqhk,hnk->bqhn", x.double(), w.double())
        rel = float((got.double().cpu() - want).norm() / want.norm())
        assert got.shape == (5, 31, h, n) and rel <= tol, (dtype, rel)
