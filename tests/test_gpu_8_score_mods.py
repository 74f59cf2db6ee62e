"""Structured masks and score modifiers evaluated inside the kernels (``pjx_score_mod``).

The matrix is the reference's own: every mask and every bias its kernels support, singly and
in the combinations of tests/test_latent_attention.py:357-444 (B2 S32 H4 D16), against the oracle
fed with the classes' dense definitions.  Both forward kernels run (exact fp32 and tcgen05), the
backward and the forward-mode derivative are checked against float64 autograd of the same dense
formula, and a larger case asserts that no ``[Q, K]`` tensor is allocated on the device.
"""

import math

import pytest
import torch

import oracle
import probjax_b200 as pj
from probjax_b200 import masks as M
from _gpu_util import assert_close, dev, randn

pytestmark = pytest.mark.gpu

B, S, H, D = 2, 32, 4, 16


def _masks(b=B, s=S):
    g = torch.Generator().manual_seed(11)
    seg = torch.sort(torch.randint(0, 3, (b, s), generator=g), dim=1).values.to(torch.int32)
    keep_tok = torch.rand((b, s), generator=g) > 0.3
    return {
        "no_mask": M.NoMask(),
        "causal": M.CausalMask(),
        "local_window": M.LocalWindowMask(8, 8),
        "causal_local_window": M.CausalLocalWindowMask(8),
        "causal_from_bottom_right": M.CausalFromBottomRightMask(s, s),
        "prefix_lm": M.PrefixLMMask(torch.tensor([8, 3][:b])),
        "block_diagonal": M.BlockDiagonalMask(seg),
        "block_diagonal_causal": M.BlockDiagonalCausalMask(seg),
        "qkv_length": M.QKVLengthMask(s - 5, s - 3),
        "key_padding": M.KeyPaddingMask(torch.randint(1, s + 1, (s,), generator=g)),
        "seq_len": M.SeqLenMask(torch.tensor([s, 20][:b])),
        "kv_len": M.KVLenMask(torch.tensor([s, 20][:b])),
        "same_segment": M.SameSegmentMask(seg, seg.flip(1)),
        "marginalization": M.MarginalizationMask(keep_tok),
    }


def _biases(h=H, s=S):
    g = torch.Generator().manual_seed(12)
    return {
        "identity": M.IdentityBias(),
        "constant": M.ConstantBias(0.3),
        "dense": M.DenseBias(torch.randn((1, 1, s, s), generator=g)),
        "causal_alibi": M.CausalAlibiBias(),
        "symmetric_alibi": M.SymmetricAlibiBias(),
        "distance_decay": M.DistanceDecayBias(0.7),
        "soft_capping": M.SoftCappingBias(2.0),
        "per_head_scale": M.PerHeadScaleBias(torch.rand((h,), generator=g) + 0.5),
        "t5": M.T5RelativePositionBias(torch.randn((h, 8), generator=g), num_buckets=8, max_distance=16),
        "learned_relative": M.LearnedRelativePositionBias(torch.randn((1, 11), generator=g), max_distance=5),
        "alibi_plus_t5_plus_cap": M.SumBias(M.SumBias(M.CausalAlibiBias(), M.SoftCappingBias(3.0)),
                                            M.T5RelativePositionBias(torch.randn((h, 6), generator=g), num_buckets=6,
                                                                     max_distance=12, bidirectional=False)),
    }


def _dense_keep(mask, b, s):
    """The mask's dense definition, with KeyPaddingMask's per-query-row lengths spelled out."""
    if isinstance(mask, M.KeyPaddingMask):
        return (torch.arange(s)[None, :] < mask.lengths.reshape(-1)[:, None])[None, None]
    return mask.dense(s, s, batch_size=b, num_heads=1)


def _score_fn(bias, heads):
    """Non-dense part of a bias expression as a function of the scaled scores, restating the classes'
    ``__call__`` (attention_mask_bias.py:553-579 sums deltas; 2564-2582 soft cap; 2606-2636 head scale)."""
    terms = M._bias_terms(bias)

    def fn(s, q_idx, k_idx):
        out = s
        for t in terms:
            if isinstance(t, M.SoftCappingBias):
                out = out + (t.softcap * torch.tanh(s / t.softcap) - s)
            elif isinstance(t, M.PerHeadScaleBias):
                out = out + (s * t.scales.expand(heads)[None, :, None, None] - s)
            elif not isinstance(t, (M.DenseBias, M.IdentityBias)):
                full = t.dense(int(q_idx.max()) + 1, int(k_idx.max()) + 1, batch_size=1, num_heads=heads)
                out = out + full[:, :, q_idx][:, :, :, k_idx]
        return out

    return fn


def _dense_part(bias):
    dense = [t.bias for t in M._bias_terms(bias) if isinstance(t, M.DenseBias)]
    return sum(dense[1:], dense[0]) if dense else None


def _want(q, k, v, mask, bias, sm_scale, heads):
    b, s = q.shape[0], q.shape[1]
    keep = None if mask is None else _dense_keep(mask, b, s)
    return oracle.xla_attention(q, k, v, keep=keep, bias=_dense_part(bias), sm_scale=sm_scale, return_lse=True,
                                score_fn=None if bias is None else _score_fn(bias, heads))


@pytest.mark.parametrize("name", list(_masks()))
def test_every_mask_fp32_and_tcgen05(name):
    d = dev()
    mask = _masks()[name]
    sc = 1 / math.sqrt(D)
    q, k, v = (randn((B, S, H, D), torch.float32, s) for s in (1, 2, 3))
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=mask, sm_scale=sc, return_lse=True)
    want, want_lse = _want(q, k, v, mask, None, sc, H)
    assert_close(got, lse, want, want_lse, torch.float32, f"fp32 {name}")
    # tensor-core kernel: bf16, D = 64, two KV heads, a length that is not a tile multiple
    s2, h2, d2 = 200, 4, 64
    mask2 = _masks(B, s2)[name]
    q2, k2, v2 = randn((B, s2, h2, d2), torch.bfloat16, 4), randn((B, s2, 2, d2), torch.bfloat16, 5), randn((B, s2, 2, d2), torch.bfloat16, 6)
    got, lse = pj.mha(q2.to(d), k2.to(d), v2.to(d), mask=mask2, sm_scale=0.125, return_lse=True, implementation="b200:tcgen05")
    pj.check_status(d)
    want, want_lse = _want(q2, k2, v2, mask2, None, 0.125, h2)
    assert_close(got, lse, want, want_lse, torch.bfloat16, f"tcgen05 {name}")


@pytest.mark.parametrize("name", ["block_diagonal", "block_diagonal_causal", "same_segment", "marginalization", "seq_len",
                                  "unsorted_ids", "many_segments_with_lengths"])
def test_segment_masks_skip_key_tiles(name):
    """Segment masks over several KV tiles on the tensor-core kernel, where the KV loop of a query tile is cut
    to the keys whose ids can match: sorted ids (block diagonal), ids in reverse order on the key side, ids
    that give dropped tokens a segment of their own, ids in random order that differ per sequence, and 16
    short segments under key lengths.  Keys outside the ranges hold NaN where that is well defined."""
    d = dev()
    b, s, h, hk, dd = 2, 1000, 4, 2, 64
    g = torch.Generator().manual_seed(77)
    lens = None
    if name == "unsorted_ids":
        mask = M.SameSegmentMask(torch.randint(0, 5, (b, s), generator=g).to(torch.int32))
    elif name == "many_segments_with_lengths":
        seg = (torch.arange(s) // 64).to(torch.int32)[None].expand(b, s).contiguous()
        lens = torch.tensor([s, 391], dtype=torch.int32)
        mask = M.ComposeMask("and", M.BlockDiagonalCausalMask(seg), M.KVLenMask(lens))
    else:
        mask = _masks(b, s)[name]
    q, k, v = randn((b, s, h, dd), torch.bfloat16, 4), randn((b, s, hk, dd), torch.bfloat16, 5), randn((b, s, hk, dd), torch.bfloat16, 6)
    want, want_lse = _want(q, k, v, mask, None, 0.125, h)
    kd, vd = k.clone(), v.clone()
    if lens is not None:
        for i in range(b):
            kd[i, int(lens[i]):] = float("nan")
            vd[i, int(lens[i]):] = float("nan")
    got, lse = pj.mha(q.to(d), kd.to(d), vd.to(d), mask=mask, sm_scale=0.125, return_lse=True, implementation="b200:tcgen05")
    pj.check_status(d)
    assert_close(got, lse, want, want_lse, torch.bfloat16, f"tcgen05 {name} over several KV tiles")
    if name in ("block_diagonal_causal", "same_segment"):  # with a bias expression on top
        bias = M.SumBias(M.CausalAlibiBias(), M.SoftCappingBias(3.0))
        got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=mask, bias=bias, sm_scale=0.125, return_lse=True,
                          implementation="b200:tcgen05")
        want, want_lse = _want(q, k, v, mask, bias, 0.125, h)
        assert_close(got, lse, want, want_lse, torch.bfloat16, f"tcgen05 {name} + bias over several KV tiles")


@pytest.mark.parametrize("lq,lkv,causal", [(700, 700, False), (500, 900, False), (640, 640, True), (130, 1000, False)])
def test_relative_table_over_several_kv_tiles(lq, lkv, causal):
    """A relative-position bias alone on the tensor-core kernel over many KV tiles (the kernel stages the
    window of the table that a tile pair uses in shared memory, two buffers in turn), rectangular problems
    included: table entries from -(Lq - 1) to Lkv - 1."""
    d = dev()
    b, h, hk, dd = 2, 4, 2, 64
    g = torch.Generator().manual_seed(5)
    bias = M.T5RelativePositionBias(torch.randn((h, 16), generator=g), num_buckets=16, max_distance=64)
    mask = M.CausalMask() if causal else None
    q, k, v = randn((b, lq, h, dd), torch.bfloat16, 7), randn((b, lkv, hk, dd), torch.bfloat16, 8), randn((b, lkv, hk, dd), torch.bfloat16, 9)
    dense = bias.dense(lq, lkv, batch_size=1, num_heads=h)
    keep = None if mask is None else mask.dense(lq, lkv, batch_size=b, num_heads=1)
    want, want_lse = oracle.xla_attention(q, k, v, keep=keep, bias=dense, sm_scale=0.125, return_lse=True)
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=mask, bias=bias, sm_scale=0.125, return_lse=True, implementation="b200:tcgen05")
    pj.check_status(d)
    assert_close(got, lse, want, want_lse, torch.bfloat16, f"tcgen05 T5 table Lq={lq} Lkv={lkv} causal={causal}")


@pytest.mark.parametrize("name", list(_biases()))
def test_every_bias_fp32_and_tcgen05(name):
    d = dev()
    bias = _biases()[name]
    sc = 1 / math.sqrt(D)
    q, k, v = (randn((B, S, H, D), torch.float32, s) for s in (1, 2, 3))
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), bias=bias, sm_scale=sc, return_lse=True)
    want, want_lse = _want(q, k, v, None, bias, sc, H)
    assert_close(got, lse, want, want_lse, torch.float32, f"fp32 {name}")
    s2, h2, d2 = 200, 4, 128
    bias2 = _biases(h2, s2)[name]
    q2, k2, v2 = randn((B, s2, h2, d2), torch.bfloat16, 4), randn((B, s2, 1, d2), torch.bfloat16, 5), randn((B, s2, 1, d2), torch.bfloat16, 6)
    got, lse = pj.mha(q2.to(d), k2.to(d), v2.to(d), mask=M.CausalMask(), bias=bias2, sm_scale=0.09, return_lse=True,
                      implementation="b200:tcgen05")
    pj.check_status(d)
    want, want_lse = _want(q2, k2, v2, M.CausalMask(), bias2, 0.09, h2)
    assert_close(got, lse, want, want_lse, torch.bfloat16, f"tcgen05 {name}")


@pytest.mark.parametrize("mask_name,bias_name", [("causal", "dense"), ("kv_len", "causal_alibi"), ("local_window", "identity"),
                                                 ("same_segment", "constant"), ("prefix_lm", "soft_capping"),
                                                 ("marginalization", "t5"), ("seq_len", "per_head_scale")])
def test_mask_and_bias_together_through_mha_flex_and_mla(mask_name, bias_name):
    """tests/test_latent_attention.py:425-444: mask and bias together; ``mla`` equals ``mha`` over the
    materialized K / V for the same mask and bias objects."""
    d = dev()
    mask, bias = _masks()[mask_name], _biases()[bias_name]
    sc = 1 / math.sqrt(D)
    q, k, v = (randn((B, S, H, D), torch.float32, s) for s in (1, 2, 3))
    want, want_lse = _want(q, k, v, mask, bias, sc, H)
    got, lse = pj.flex_attention(q.to(d), k.to(d), v.to(d), mask=mask, bias=bias, return_lse=True)
    assert_close(got, lse, want, want_lse, torch.float32, f"flex {mask_name} + {bias_name}")
    r = 8
    cache, wk, wv = randn((B, S, r), torch.float32, 7), randn((H, D, r), torch.float32, 8), randn((H, D, r), torch.float32, 9)
    got = pj.mla(q.to(d), cache.to(d), wk.to(d), wv.to(d), mask=mask, bias=bias, sm_scale=sc)
    key, value = oracle.materialize_kv(cache, wk, wv, H)
    want, _ = _want(q, key, value, mask, bias, sc, H)
    assert_close(got, None, want, None, torch.float32, f"mla {mask_name} + {bias_name}")


@pytest.mark.parametrize("mask_name,bias_name", [("same_segment", "soft_capping"), ("prefix_lm", "per_head_scale"),
                                                 ("marginalization", "causal_alibi"), ("key_padding", "t5")])
def test_backward_and_forward_mode_with_modifiers(mask_name, bias_name):
    """Gradients through the modifiers: reverse mode (dq, dk, dv) and a forward-mode tangent against
    float64 autograd of the dense formula with the same modifiers."""
    d = dev()
    mask, bias = _masks()[mask_name], _biases()[bias_name]
    sc = 1 / math.sqrt(D)
    q, k, v = (randn((B, S, H, D), torch.float32, s) for s in (1, 2, 3))
    g_o = randn((B, S, H, D), torch.float32, 10)
    qd, kd, vd = (x.to(d).requires_grad_(True) for x in (q, k, v))
    out = pj.mha(qd, kd, vd, mask=mask, bias=bias, sm_scale=sc)
    out.backward(g_o.to(d))
    # float64 reference
    q64, k64, v64 = (x.double().requires_grad_(True) for x in (q, k, v))
    s64 = torch.einsum("bqhd,bkhd->bhqk", q64, k64) * sc
    s64 = _score_fn(bias, H)(s64, torch.arange(S), torch.arange(S))
    dense = _dense_part(bias)
    if dense is not None:
        s64 = s64 + dense.double()
    keep = _dense_keep(mask, B, S)
    s64 = s64.masked_fill(~keep, -math.inf)
    rowmax = s64.amax(-1, keepdim=True)
    rowmax = torch.where(torch.isfinite(rowmax), rowmax, torch.zeros_like(rowmax))
    p64 = torch.exp(s64 - rowmax)
    den = p64.sum(-1, keepdim=True)
    p64 = p64 / torch.where(den > 0, den, torch.ones_like(den))
    o64 = torch.einsum("bhqk,bkhd->bqhd", p64, v64)
    assert float((out.detach().cpu().double() - o64.detach()).abs().max()) <= 1e-4
    o64.backward(g_o.double())
    for name, a, w in (("dq", qd.grad, q64.grad), ("dk", kd.grad, k64.grad), ("dv", vd.grad, v64.grad)):
        rel = float((a.double().cpu() - w).norm() / w.norm())
        assert rel <= 1e-4, f"{mask_name} + {bias_name}: {name} relative error {rel:.3e}"
    # forward mode: tangent of o along a random direction of q and k
    import torch.autograd.forward_ad as fwd_ad

    tq, tk = randn((B, S, H, D), torch.float32, 21), randn((B, S, H, D), torch.float32, 22)
    with fwd_ad.dual_level():
        dual_o = pj.mha(fwd_ad.make_dual(q.to(d), tq.to(d)), fwd_ad.make_dual(k.to(d), tk.to(d)), v.to(d), mask=mask,
                        bias=bias, sm_scale=sc, diff_mode="forward")
        t_o = fwd_ad.unpack_dual(dual_o).tangent
    q64b, k64b = q.double().requires_grad_(True), k.double().requires_grad_(True)

    def f(qq, kk):
        ss = torch.einsum("bqhd,bkhd->bhqk", qq, kk) * sc
        ss = _score_fn(bias, H)(ss, torch.arange(S), torch.arange(S))
        if dense is not None:
            ss = ss + dense.double()
        ss = ss.masked_fill(~keep, -math.inf)
        mm = ss.amax(-1, keepdim=True)
        mm = torch.where(torch.isfinite(mm), mm, torch.zeros_like(mm))
        pp = torch.exp(ss - mm)
        dd = pp.sum(-1, keepdim=True)
        pp = pp / torch.where(dd > 0, dd, torch.ones_like(dd))
        return torch.einsum("bhqk,bkhd->bqhd", pp, v.double())

    _, want_t = torch.func.jvp(f, (q64b.detach(), k64b.detach()), (tq.double(), tk.double()))
    rel = float((t_o.double().cpu() - want_t).norm() / want_t.norm())
    assert rel <= 1e-4, f"{mask_name} + {bias_name}: forward-mode relative error {rel:.3e}"


def test_low_rank_bias_is_folded_into_q_and_k():
    """layers/attention.py:1602-1639: ``LowRankBias`` terms become extra q / k columns (no [Q, K] tensor)."""
    d = dev()
    q, k, v = randn((B, S, H, D), torch.float32, 1), randn((B, S, 2, D), torch.float32, 2), randn((B, S, 2, D), torch.float32, 3)
    qf, kf = randn((H, S + 4, 3), torch.float32, 4), randn((H, S + 4, 3), torch.float32, 5)
    bias = M.SumBias(M.LowRankBias(qf, kf, scale=0.5), M.CausalAlibiBias())
    got = pj.flex_attention(q.to(d), k.to(d), v.to(d), mask=M.CausalMask(), bias=bias, enable_gqa=True)
    dense = bias.dense(S, S, batch_size=B, num_heads=H)
    want = oracle.xla_attention(q, k, v, causal=True, bias=dense, sm_scale=1 / math.sqrt(D))
    assert_close(got, None, want, None, torch.float32, "low-rank folding")


def test_no_score_sized_tensor_is_allocated():
    """A segment mask with ALiBi at S = 4096: the device memory the call takes beyond its inputs and
    its output stays far below one [Q, K] plane (64 MB in float32), let alone [H, Q, K]."""
    d = dev()
    b, s, h, dd = 1, 4096, 8, 128
    q, k, v = (randn((b, s, h, dd), torch.bfloat16, i).to(d) for i in (1, 2, 3))
    seg = (torch.arange(s) // 1000).to(torch.int32)[None]
    mask, bias = M.SameSegmentMask(seg) & M.CausalMask(), M.CausalAlibiBias()
    pj.mha(q, k, v, mask=mask, bias=bias, sm_scale=0.09)  # warm-up: module load, cached scratch
    torch.cuda.synchronize(d)
    torch.cuda.reset_peak_memory_stats(d)
    base = torch.cuda.memory_allocated(d)
    out = pj.mha(q, k, v, mask=mask, bias=bias, sm_scale=0.09)
    torch.cuda.synchronize(d)
    extra = torch.cuda.max_memory_allocated(d) - base
    assert extra <= out.numel() * out.element_size() + (4 << 20), f"{extra} bytes allocated"
    # and it is right: rows of the last segment against the oracle on that segment alone (block diagonal)
    lo = 4000
    want = oracle.xla_attention(q[:, lo:].cpu(), k[:, lo:].cpu(), v[:, lo:].cpu(), causal=True, sm_scale=0.09,
                                bias=M.CausalAlibiBias().dense(s - lo, s - lo, num_heads=h))
    assert_close(out[:, lo:], None, want, None, torch.bfloat16, "segment + alibi at S=4096")


def _dense_dropout_reference(q, k, v, keep, bias_fn, dense, sc, drop):
    """float64 restatement with the counter-hash dropout: probabilities are normalised over all kept
    keys, then dropped / rescaled by ``drop`` (kernels/attention.py:497-505)."""
    ss = torch.einsum("bqhd,bkhd->bhqk", q, k) * sc
    if bias_fn is not None:
        ss = bias_fn(ss, _IDX, _IDX)
    if dense is not None:
        ss = ss + dense.double()
    if keep is not None:
        ss = ss.masked_fill(~keep, -math.inf)
    mm = ss.amax(-1, keepdim=True)
    mm = torch.where(torch.isfinite(mm), mm, torch.zeros_like(mm))
    pp = torch.exp(ss - mm)
    dd = pp.sum(-1, keepdim=True)
    pp = pp / torch.where(dd > 0, dd, torch.ones_like(dd))
    return torch.einsum("bhqk,bkhd->bqhd", pp * drop, v)


_IDX = torch.arange(S)


@pytest.mark.parametrize("rate", [0.1, 0.5])
def test_counter_dropout_forward_fp32_and_tcgen05(rate):
    """Attention dropout with the reference's counter hash: the kernels regenerate the oracle's mask
    from (seed, batch, head, row, key); the log-sum-exp is the undropped one."""
    d = dev()
    key = [0x1234ABCD, 0x0BADF00D]
    seed = oracle.rng_seed_from_key(key)
    sc = 1 / math.sqrt(D)
    q, k, v = (randn((B, S, H, D), torch.float32, s) for s in (1, 2, 3))
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=M.CausalMask(), bias=M.CausalAlibiBias(), rng=key, sm_scale=sc,
                      dropout_rate=rate, return_lse=True)
    want, want_lse = oracle.xla_attention(q, k, v, causal=True, sm_scale=sc, return_lse=True, dropout=(seed, rate),
                                          score_fn=_score_fn(M.CausalAlibiBias(), H))
    assert_close(got, lse, want, want_lse, torch.float32, f"fp32 dropout {rate}")
    plain = pj.mha(q.to(d), k.to(d), v.to(d), mask=M.CausalMask(), bias=M.CausalAlibiBias(), sm_scale=sc)
    assert float((plain - got).abs().max()) > 1e-3, "dropout changed nothing"
    # tensor-core kernel, GQA, ragged length, dropout alone (no other modifier) and through flex_attention
    s2, h2, d2 = 200, 4, 64
    q2, k2, v2 = randn((B, s2, h2, d2), torch.bfloat16, 4), randn((B, s2, 2, d2), torch.bfloat16, 5), randn((B, s2, 2, d2), torch.bfloat16, 6)
    got, lse = pj.flex_attention(q2.to(d), k2.to(d), v2.to(d), dropout_rng=torch.tensor(key), dropout_rate=rate,
                                 deterministic=False, sm_scale=0.125, enable_gqa=True, return_lse=True,
                                 implementation="b200:tcgen05")
    pj.check_status(d)
    want, want_lse = oracle.xla_attention(q2, k2, v2, sm_scale=0.125, return_lse=True, dropout=(seed, rate))
    assert_close(got, lse, want, want_lse, torch.bfloat16, f"tcgen05 dropout {rate}")
    # deterministic=True switches it off
    off = pj.flex_attention(q2.to(d), k2.to(d), v2.to(d), dropout_rng=key, dropout_rate=rate, deterministic=True,
                            sm_scale=0.125, enable_gqa=True)
    want_off = oracle.xla_attention(q2, k2, v2, sm_scale=0.125)
    assert_close(off, None, want_off, None, torch.bfloat16, "deterministic")


def test_counter_dropout_backward_forward_mode_and_latent():
    """Both derivatives regenerate the mask of the forward (kernels/attention.py:1038-1039) and ``mla``
    takes the same arguments."""
    d = dev()
    key, rate = 77, 0.25
    seed = oracle.rng_seed_from_key(key)
    mask, bias = _masks()["same_segment"], _biases()["soft_capping"]
    keep = _dense_keep(mask, B, S)
    drop = oracle.counter_dropout_scale(seed, B, H, _IDX, _IDX, rate).double()
    sc = 1 / math.sqrt(D)
    q, k, v = (randn((B, S, H, D), torch.float32, s) for s in (1, 2, 3))
    g_o = randn((B, S, H, D), torch.float32, 10)
    qd, kd, vd = (x.to(d).requires_grad_(True) for x in (q, k, v))
    out = pj.mha(qd, kd, vd, mask=mask, bias=bias, rng=key, sm_scale=sc, dropout_rate=rate)
    out.backward(g_o.to(d))
    q64, k64, v64 = (x.double().requires_grad_(True) for x in (q, k, v))
    o64 = _dense_dropout_reference(q64, k64, v64, keep, _score_fn(bias, H), None, sc, drop)
    assert float((out.detach().cpu().double() - o64.detach()).abs().max()) <= 1e-4
    o64.backward(g_o.double())
    for name, a, w in (("dq", qd.grad, q64.grad), ("dk", kd.grad, k64.grad), ("dv", vd.grad, v64.grad)):
        rel = float((a.double().cpu() - w).norm() / w.norm())
        assert rel <= 1e-4, f"dropout: {name} relative error {rel:.3e}"
    # tensor-core backward kernels do not take modifiers: 16-bit inputs go through the exact kernels too
    qh, kh, vh = (x.to(torch.bfloat16).to(d).requires_grad_(True) for x in (q, k, v))
    pj.mha(qh, kh, vh, rng=key, sm_scale=sc, dropout_rate=rate).backward(g_o.to(torch.bfloat16).to(d))
    q64b, k64b, v64b = (x.to(torch.bfloat16).double().requires_grad_(True) for x in (q, k, v))
    _dense_dropout_reference(q64b, k64b, v64b, None, None, None, sc, drop).backward(g_o.to(torch.bfloat16).double())
    for name, a, w in (("dq", qh.grad, q64b.grad), ("dk", kh.grad, k64b.grad), ("dv", vh.grad, v64b.grad)):
        rel = float((a.double().cpu() - w).norm() / w.norm())
        assert rel <= 2e-2, f"bf16 dropout: {name} relative error {rel:.3e}"
    # forward mode
    import torch.autograd.forward_ad as fwd_ad

    tq, tk, tv = (randn((B, S, H, D), torch.float32, s) for s in (21, 22, 23))
    with fwd_ad.dual_level():
        dual_o = pj.mha(fwd_ad.make_dual(q.to(d), tq.to(d)), fwd_ad.make_dual(k.to(d), tk.to(d)),
                        fwd_ad.make_dual(v.to(d), tv.to(d)), mask=mask, bias=bias, rng=key, sm_scale=sc,
                        dropout_rate=rate, diff_mode="forward")
        t_o = fwd_ad.unpack_dual(dual_o).tangent
    _, want_t = torch.func.jvp(lambda a, b_, c: _dense_dropout_reference(a, b_, c, keep, _score_fn(bias, H), None, sc, drop),
                               (q.double(), k.double(), v.double()), (tq.double(), tk.double(), tv.double()))
    rel = float((t_o.double().cpu() - want_t).norm() / want_t.norm())
    assert rel <= 1e-4, f"dropout: forward-mode relative error {rel:.3e}"
    # latent attention: materialized K / V with the same dropout arguments
    r = 8
    cache, wk, wv = randn((B, S, r), torch.float32, 7), randn((H, D, r), torch.float32, 8), randn((H, D, r), torch.float32, 9)
    got = pj.mla(q.to(d), cache.to(d), wk.to(d), wv.to(d), mask=mask, rng=key, dropout_rate=rate, sm_scale=sc)
    kk, vv = oracle.materialize_kv(cache, wk, wv, H)
    want = oracle.xla_attention(q, kk, vv, keep=keep, sm_scale=sc, dropout=(seed, rate))
    assert_close(got, None, want, None, torch.float32, "mla dropout")


def test_dropout_argument_checks():
    """attention_xla.py:637-641: a rate without a key is an error; the materialized-mask variant
    (a [B, H, Q, K] tensor of jax.random draws) is not built."""
    d = dev()
    q, k, v = (randn((1, 16, 2, 16), torch.float32, s).to(d) for s in (1, 2, 3))
    with pytest.raises(ValueError, match="prng_key must be provided"):
        pj.mha(q, k, v, dropout_rate=0.1)
    with pytest.raises(NotImplementedError, match="counter-hash"):
        pj.mha(q, k, v, rng=3, dropout_rate=0.1, dropout_impl="materialize")
    with pytest.raises(ValueError, match=r"\[0, 1\)"):
        pj.mha(q, k, v, rng=3, dropout_rate=1.0)


def test_batched_low_rank_and_learned_alibi():
    """Per-example factors (attention_mask_bias.py:2028-2192) ride on extra q / k columns; caller-owned
    ALiBi slopes (2258-2351) are a relative-position table in the kernels, or -- when they require a
    gradient -- two folded columns through which the gradient reaches them."""
    d = dev()
    sc = 1 / math.sqrt(D)
    q, k, v = randn((B, S, H, D), torch.float32, 1), randn((B, S, 2, D), torch.float32, 2), randn((B, S, 2, D), torch.float32, 3)
    log_m = randn((B, S), torch.float32, 4)
    bias = M.SumBias(M.BatchedLowRankBias.from_key_bias(log_m), M.CausalAlibiBias())
    got = pj.flex_attention(q.to(d), k.to(d), v.to(d), mask=M.CausalMask(), bias=bias, enable_gqa=True)
    dense = log_m[:, None, None, :] + M.CausalAlibiBias().dense(S, S, num_heads=H)
    want = oracle.xla_attention(q, k, v, causal=True, bias=dense, sm_scale=sc)
    assert_close(got, None, want, None, torch.float32, "per-example key bias")
    # caller-owned slopes, no gradient: in-kernel table (fp32 and tensor-core kernels)
    slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625])
    la = M.LearnedAlibiBias(slopes, query_offset=2, key_offset=0)
    dense = la.dense(S, S, num_heads=H)
    got, lse = pj.mha(q.to(d), k.to(d), v.to(d), mask=M.CausalMask(), bias=la, sm_scale=sc, return_lse=True)
    want, want_lse = oracle.xla_attention(q, k, v, causal=True, bias=dense, sm_scale=sc, return_lse=True)
    assert_close(got, lse, want, want_lse, torch.float32, "learned alibi table")
    qh, kh, vh = randn((B, 200, H, 64), torch.bfloat16, 5), randn((B, 200, 2, 64), torch.bfloat16, 6), randn((B, 200, 2, 64), torch.bfloat16, 7)
    got = pj.mha(qh.to(d), kh.to(d), vh.to(d), mask=M.CausalMask(), bias=la, sm_scale=0.125, implementation="b200:tcgen05")
    want = oracle.xla_attention(qh, kh, vh, causal=True, bias=la.dense(200, 200, num_heads=H), sm_scale=0.125)
    assert_close(got, None, want, None, torch.bfloat16, "learned alibi table, tcgen05")
    # slopes that require a gradient: folded, d loss / d slopes against float64 autograd
    sl = slopes.clone().to(d).requires_grad_(True)
    g_o = randn((B, S, H, D), torch.float32, 8)
    out = pj.mha(q.to(d), k.to(d), v.to(d), mask=M.CausalMask(), bias=M.LearnedAlibiBias(sl), sm_scale=sc)
    out.backward(g_o.to(d))
    sl64 = slopes.double().requires_grad_(True)
    pos = torch.arange(S, dtype=torch.float64)
    s64 = torch.einsum("bqhd,bkhd->bhqk", q.double(), k.double().repeat_interleave(2, 2)) * sc
    s64 = s64 - sl64[None, :, None, None] * (pos[:, None] - pos[None, :])
    s64 = s64.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool)), -math.inf)
    o64 = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s64, -1), v.double().repeat_interleave(2, 2))
    assert float((out.detach().cpu().double() - o64.detach()).abs().max()) <= 1e-4
    o64.backward(g_o.double())
    rel = float((sl.grad.double().cpu() - sl64.grad).norm() / sl64.grad.norm())
    assert rel <= 1e-3, f"slope gradient relative error {rel:.3e}"
