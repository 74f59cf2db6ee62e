"""Parity of the split-KV decode kernel, its combine and the sharded decode."""

import math

import pytest
import torch

import oracle
import probjax_b200 as pj
from probjax_b200 import dist as pjd
from _gpu_util import assert_close, cases, dev, load_golden, oracle_fwd, randn

pytestmark = pytest.mark.gpu


def _decode(q, k, v, lens, sc, **kw):
    d = dev()
    out, lse = pj.decode_forward(q.to(d), k.to(d), v.to(d), kv_lengths=None if lens is None else lens.to(d),
                                 sm_scale=sc, return_lse=True, **kw)
    torch.cuda.synchronize()
    return out, lse


def test_golden():
    inp = cases.make_inputs("c4_small")
    out, lse = _decode(inp["q"], inp["k"], inp["v"], inp["kv_lengths"], inp["sm_scale"])
    want, want_lse = load_golden("c4_small")
    assert_close(out, lse, want, want_lse, torch.bfloat16, "c4_small")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize(
    "b,lq,lkv,hq,hkv,d,split_len",
    [
        (1, 1, 200, 4, 4, 64, 0),       # tests/test_attention_gqa_splitkv.py:175-183 shapes, widened to a kernel head dim
        (2, 3, 130, 4, 2, 64, 64),
        (1, 4, 96, 8, 2, 128, 0),
        (1, 2, 50, 2, 1, 64, 0),
        (3, 1, 2100, 32, 8, 128, 256),  # the benchmark's head geometry
        (2, 1, 1, 8, 2, 128, 0),        # a single key
        (2, 2, 777, 16, 2, 128, 128),   # 16 packed rows: the most the kernel takes
    ],
)
def test_shapes(dtype, b, lq, lkv, hq, hkv, d, split_len):
    q, k, v = randn((b, lq, hq, d), dtype, 1), randn((b, lkv, hkv, d), dtype, 2), randn((b, lkv, hkv, d), dtype, 3)
    lens = torch.randint(1, lkv + 1, (b,), generator=torch.Generator().manual_seed(lkv), dtype=torch.int32)
    lens[0] = lkv
    sc = 1 / math.sqrt(d)
    out, lse = _decode(q, k, v, lens, sc, split_len=split_len)
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=sc)
    assert_close(out, lse, want, want_lse, dtype, f"{(b, lq, lkv, hq, hkv, d, split_len)}")
    # without lengths the whole cache counts
    out, lse = _decode(q, k, v, None, sc, split_len=split_len)
    want, want_lse = oracle_fwd(q, k, v, sm_scale=sc)
    assert_close(out, lse, want, want_lse, dtype, "full cache")


def test_garbage_past_the_valid_length_is_never_read():
    b, cap, hq, hkv, d = 2, 700, 8, 2, 128
    q, k, v = randn((b, 1, hq, d), torch.bfloat16, 1), randn((b, cap, hkv, d), torch.bfloat16, 2), randn((b, cap, hkv, d), torch.bfloat16, 3)
    lens = torch.tensor([130, 401], dtype=torch.int32)
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=0.1)
    for i in range(b):
        k[i, int(lens[i]):] = float("nan")
        v[i, int(lens[i]):] = float("inf")
    out, lse = _decode(q, k, v, lens, 0.1, split_len=64)
    assert_close(out, lse, want, want_lse, torch.bfloat16, "poisoned tail")


def test_zero_length_sequences():
    q, k, v = randn((3, 1, 8, 128), torch.bfloat16, 1), randn((3, 300, 2, 128), torch.bfloat16, 2), randn((3, 300, 2, 128), torch.bfloat16, 3)
    lens = torch.tensor([0, 300, 0], dtype=torch.int32)
    out, lse = _decode(q, k, v, lens, 0.2)
    assert (out[0] == 0).all() and (out[2] == 0).all()
    assert torch.isinf(lse[0]).all() and (lse[0] > 0).all()
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=0.2)
    assert_close(out, lse, want, want_lse, torch.bfloat16, "zero lengths")


def test_shapes_outside_the_streaming_kernel_use_the_generic_forward():
    # D = 32 and fp32 are not streaming-kernel cases (tests/test_attention_gqa_splitkv.py:235-243 shapes)
    for dtype, d, lq, lkv in [(torch.float32, 32, 1, 300), (torch.bfloat16, 32, 4, 1000), (torch.float32, 128, 1, 500)]:
        q, k, v = randn((1, lq, 8, d), dtype, 1), randn((1, lkv, 2, d), dtype, 2), randn((1, lkv, 2, d), dtype, 3)
        lens = torch.tensor([lkv - 17], dtype=torch.int32)
        out, lse = _decode(q, k, v, lens, 0.3)
        want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=0.3)
        assert_close(out, lse, want, want_lse, dtype, f"fallback {dtype} {d}")


def test_splitkv_forward_signature():
    # attention_splitkv.py:137-149: num_splits fixes the split count; LSE is natural log [B, Hq, Lq]
    d = dev()
    q, k, v = randn((2, 3, 4, 64), torch.bfloat16, 1), randn((2, 130, 2, 64), torch.bfloat16, 2), randn((2, 130, 2, 64), torch.bfloat16, 3)
    out, lse = pj.splitkv_forward(q.to(d), k.to(d), v.to(d), sm_scale=0.125, num_splits=3, return_lse=True)
    want, want_lse, _, _ = oracle.splitkv_reference(q, k, v, sm_scale=0.125, num_splits=3)
    assert lse.shape == (2, 4, 3)
    assert_close(out, lse, want, want_lse, torch.bfloat16, "splitkv_forward")
    with pytest.raises(ValueError, match="multiple"):
        pj.splitkv_forward(q.to(d)[:, :, :3], k.to(d), v.to(d), sm_scale=1.0)


def test_combine_entry_point():
    g = torch.Generator().manual_seed(0)
    P, N, Dv = 5, 37, 128
    o_parts = torch.randn(P, N, Dv, generator=g)
    lse_parts = torch.randn(P, N, generator=g) * 3
    lse_parts[2] = float("inf")          # a part without keys
    lse_parts[:, 5] = float("inf")       # a row no part has keys for
    o, lse = pj.combine_partials(o_parts.to(dev()), lse_parts.to(dev()))
    neg = torch.where(torch.isinf(lse_parts), torch.tensor(-float("inf")), lse_parts)
    w = torch.softmax(neg.double(), dim=0)
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    want = (w[..., None] * o_parts.double()).sum(0)
    want_lse = torch.logsumexp(neg.double(), 0)
    assert float((o.cpu().double() - want).abs().max()) < 1e-5
    assert (o.cpu()[5] == 0).all() and torch.isinf(lse.cpu()[5]) and lse.cpu()[5] > 0
    fin = torch.isfinite(want_lse)
    assert float((lse.cpu().double()[fin] - want_lse[fin]).abs().max()) < 1e-5


@pytest.mark.parametrize("world,page", [(2, 64), (4, 256), (8, 128)])
def test_sharded_decode_emulated_on_one_gpu(world, page):
    """Every rank's shard is run in turn on this GPU and the partials are combined
    with the same kernel the multi-GPU path uses: the result must equal the
    unsharded decode and the oracle."""
    d = dev()
    b, cap, hq, hkv, dd = 4, 3000, 32, 8, 128
    q, k, v = randn((b, 1, hq, dd), torch.bfloat16, 1), randn((b, cap, hkv, dd), torch.bfloat16, 2), randn((b, cap, hkv, dd), torch.bfloat16, 3)
    lens = torch.tensor([3000, 17, 1500, 640], dtype=torch.int32)
    sc = 1 / math.sqrt(dd)
    recs_o, recs_l = [], []
    for r in range(world):
        kl, vl = pjd.shard_cache(k, r, world, page).to(d), pjd.shard_cache(v, r, world, page).to(d)
        ll = pjd.local_lengths(lens, r, world, page).to(d)
        o, lse = pj.decode_forward(q.to(d), kl, vl, kv_lengths=ll, sm_scale=sc, return_lse=True, partial_f32=True)
        assert o.dtype == torch.float32
        recs_o.append(o.reshape(-1, dd))
        recs_l.append(lse.permute(0, 2, 1).reshape(-1))
    o, lse = pj.combine_partials(torch.stack(recs_o), torch.stack(recs_l), out_dtype=torch.bfloat16)
    o, lse = o.reshape(b, 1, hq, dd), lse.reshape(b, 1, hq).permute(0, 2, 1)
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=sc)
    assert_close(o, lse, want, want_lse, torch.bfloat16, f"sharded x{world}")
    # world size 1 through the public function (no process group)
    o1, lse1 = pjd.decode_sharded(q.to(d), k.to(d), v.to(d), lens, page=page, sm_scale=sc, return_lse=True)
    assert_close(o1, lse1, want, want_lse, torch.bfloat16, "decode_sharded world=1")


@pytest.mark.parametrize("use_graph", [False, True])
def test_sharded_decoder_object_single_rank(use_graph):
    """The preallocated decoder (optionally replaying one CUDA graph per step)
    gives the same answer as the oracle, also after the lengths change."""
    d = dev()
    b, cap, hq, hkv, dd = 3, 2000, 32, 8, 128
    q, k, v = randn((b, 1, hq, dd), torch.bfloat16, 1), randn((b, cap, hkv, dd), torch.bfloat16, 2), randn((b, cap, hkv, dd), torch.bfloat16, 3)
    lens = torch.tensor([2000, 900, 33], dtype=torch.int32)
    sc = 1 / math.sqrt(dd)
    dec = pjd.ShardedDecoder(q.to(d), k.to(d), v.to(d), lens, page=128, sm_scale=sc, use_graph=use_graph)
    o, lse = dec(return_lse=True)
    torch.cuda.synchronize()
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=sc)
    assert_close(o, lse, want, want_lse, torch.bfloat16, "ShardedDecoder")
    lens2 = torch.tensor([5, 2000, 1000], dtype=torch.int32)
    dec.set_lengths(lens2)
    o, lse = dec(return_lse=True)
    torch.cuda.synchronize()
    want, want_lse = oracle_fwd(q, k, v, kv_lengths=lens2, sm_scale=sc)
    assert_close(o, lse, want, want_lse, torch.bfloat16, "ShardedDecoder after set_lengths")


def test_missing_peer_is_reported_not_waited_for_forever():
    """Failure detection of the fused sharded decode: rank 0 of a two-rank exchange
    whose peer never publishes.  The wait on the peer's flag is bounded: the kernel
    gives up after about two seconds, the status word reads DEVICE_TIMEOUT, and the
    device stays usable."""
    import ctypes

    from probjax_b200 import _lib

    L = _lib.lib()
    d = dev()
    b, cap, hq, hkv, dd = 1, 256, 8, 2, 128
    q, k, v = randn((b, 1, hq, dd), torch.bfloat16, 1).to(d), randn((b, cap, hkv, dd), torch.bfloat16, 2).to(d), randn((b, cap, hkv, dd), torch.bfloat16, 3).to(d)
    nbytes = L.pjx_attn_decode_sharded_buffer_bytes(b, 1, hq, dd, 2)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=d)
    absent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=d)  # nobody ever raises rank 1's flag
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), absent_peer.data_ptr())
    ws = torch.empty(L.pjx_attn_decode_workspace_bytes(b, 1, hq, hkv, dd, cap, 0), dtype=torch.uint8, device=d)
    o = torch.empty(b, 1, hq, dd, dtype=torch.bfloat16, device=d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    stream = torch.cuda.current_stream(d).cuda_stream
    rc = L.pjx_attn_decode_sharded(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, o.data_ptr(), None, b, 1, hq, hkv, dd, dd,
                                   cap, _lib.PJX_BF16, 0.1, 0, ws.data_ptr(), ws.numel(), 0, 2, ptrs, 1, 0, status.data_ptr(), stream)
    assert rc == 0
    assert L.pjx_read_status(status.data_ptr(), stream) == _lib.PJX_ERR_DEVICE_TIMEOUT
    with pytest.raises(_lib.KernelTimeout):
        _lib.check(_lib.PJX_ERR_DEVICE_TIMEOUT)
    # the context is intact: the same call as a one-rank exchange completes and is correct
    status.zero_()
    mine.zero_()
    one = (ctypes.c_void_p * 1)(mine.data_ptr())
    rc = L.pjx_attn_decode_sharded(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, o.data_ptr(), None, b, 1, hq, hkv, dd, dd,
                                   cap, _lib.PJX_BF16, 0.1, 0, ws.data_ptr(), ws.numel(), 0, 1, one, 1, 0, status.data_ptr(), stream)
    assert rc == 0 and L.pjx_read_status(status.data_ptr(), stream) == 0
    want, _ = oracle_fwd(q, k, v, sm_scale=0.1)
    assert_close(o, None, want, None, torch.bfloat16, "after a timed-out exchange")


def test_sharded_decode_rank0_of_two_with_the_peer_record_prefilled():
    """The two-rank exchange on one GPU, without one launch waiting for another: rank 1's partial
    (its own split-KV decode over its shard) and its flags are written into rank 0's exchange
    buffer by the test, then rank 0 runs its sharded step; the result must equal the oracle over
    the whole cache.  Covers both exchange forms: the one-kernel form (small grid) and the
    three-kernel form (a grid larger than one wave of CTAs), on two steps of opposite parity."""
    import ctypes

    import oracle
    from probjax_b200 import _lib, decode_forward
    from probjax_b200 import dist as pjd

    L = _lib.lib()
    d = dev()
    for (B, cap, page, split_len) in ((3, 2048, 128, 0), (5, 4096, 256, 64)):
        c = oracle.make_config(4, B=B, cap=cap)
        c["kv_lengths"][0] = 7  # rank 1 holds nothing of this sequence
        Hq, Hkv, D = c["q"].shape[2], c["k"].shape[2], c["q"].shape[3]
        want, want_lse = oracle.xla_attention(c["q"], c["k"], c["v"], kv_lengths=c["kv_lengths"], sm_scale=c["sm_scale"],
                                              return_lse=True)
        q = c["q"].to(d)
        shards = [(pjd.shard_cache(c["k"], r, 2, page).to(d), pjd.shard_cache(c["v"], r, 2, page).to(d),
                   pjd.local_lengths(c["kv_lengths"], r, 2, page).to(d)) for r in range(2)]
        o1, lse1 = decode_forward(q, shards[1][0], shards[1][1], kv_lengths=shards[1][2], sm_scale=c["sm_scale"],
                                  return_lse=True, partial_f32=True)
        lay = pjd.exchange_layout(B, 1, Hq, D, 2)
        assert lay["bytes"] <= L.pjx_attn_decode_sharded_buffer_bytes(B, 1, Hq, D, 2)
        mine = torch.zeros(L.pjx_attn_decode_sharded_buffer_bytes(B, 1, Hq, D, 2), dtype=torch.uint8, device=d)
        peer = torch.zeros_like(mine)  # rank 0's stores to rank 1 land here and are not looked at
        f32, u32 = mine.view(torch.float32), mine.view(torch.int32)
        k0, v0, l0 = shards[0]
        ws = torch.empty(L.pjx_attn_decode_workspace_bytes(B, 1, Hq, Hkv, D, k0.shape[1], split_len), dtype=torch.uint8, device=d)
        o = torch.empty(B, 1, Hq, D, dtype=torch.bfloat16, device=d)
        lse = torch.empty(B, Hq, 1, dtype=torch.float32, device=d)
        status = torch.zeros(1, dtype=torch.int32, device=d)
        ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
        stream = torch.cuda.current_stream(d).cuda_stream
        N = lay["N"]
        for step in (1, 2):
            par = step & 1
            f32[lay["o"](par, 1): lay["o"](par, 1) + N * D] = o1.reshape(-1)
            f32[lay["lse"](par, 1): lay["lse"](par, 1) + N] = lse1.permute(0, 2, 1).reshape(-1)  # rows in [B, Lq, Hq] order
            u32[lay["rank_flags"] + 1] = step
            rec = pjd.ll_records(o1.reshape(N, D), lse1.permute(0, 2, 1).reshape(-1), step)
            u32[lay["ll"](par, 1) * 4: (lay["ll"](par, 1) + N * lay["lines"]) * 4] = rec.reshape(-1)
            o.zero_()
            rc = L.pjx_attn_decode_sharded(q.data_ptr(), k0.data_ptr(), v0.data_ptr(), l0.data_ptr(), o.data_ptr(),
                                           lse.data_ptr(), B, 1, Hq, Hkv, D, D, k0.shape[1], _lib.PJX_BF16, c["sm_scale"],
                                           split_len, ws.data_ptr(), ws.numel(), 0, 2, ptrs, step, 0, status.data_ptr(), stream)
            assert rc == 0, _lib.last_error()
            assert L.pjx_read_status(status.data_ptr(), stream) == 0
            assert_close(o, lse, want, want_lse, torch.bfloat16, f"sharded rank 0 of 2, B={B} step {step}")
        # rank 0 stored its own partial into the peer's buffer as well, under the step number
        pu32 = peer.view(torch.int32)
        sent = pu32[lay["ll"](0, 0) * 4: (lay["ll"](0, 0) + N * lay["lines"]) * 4].view(N, lay["lines"], 4)
        assert int(pu32[lay["rank_flags"]]) == 2 or bool((sent[:, :, 1] == 2).all() and (sent[:, :, 3] == 2).all())


def test_sharded_decode_over_a_paged_local_cache():
    """The sharded step with this rank's share held in shuffled pool pages (one rank, exchange with
    itself): bit-identical to the same step over the contiguous local cache, right against the oracle."""
    c = oracle.make_config(4, B=4, cap=2048)
    c["kv_lengths"][1] = 100
    d = dev()
    q, k, v = c["q"].to(d), c["k"].to(d), c["v"].to(d)
    page = 128
    B, cap = k.shape[0], k.shape[1]
    mp = cap // page
    perm = torch.randperm(B * mp, generator=torch.Generator().manual_seed(3)).view(B, mp).to(torch.int32)
    kp = torch.empty((B * mp, page) + tuple(k.shape[2:]), dtype=k.dtype, device=d)
    vp = torch.empty_like(kp)
    kp[perm.view(-1).long().to(d)] = k.view(B * mp, page, *k.shape[2:])
    vp[perm.view(-1).long().to(d)] = v.view(B * mp, page, *v.shape[2:])
    dense = pjd.FusedShardedDecoder(q, k, v, c["kv_lengths"], page=page, sm_scale=c["sm_scale"])
    paged = pjd.FusedShardedDecoder(q, kp, vp, c["kv_lengths"], page=page, sm_scale=c["sm_scale"], block_table=perm)
    # steps that may start while the previous step's kernel is still finishing (programmatic dependent launch)
    chained = pjd.FusedShardedDecoder(q, k, v, c["kv_lengths"], page=page, sm_scale=c["sm_scale"], overlap_steps=True)
    for _ in range(2):
        o1, l1 = dense(return_lse=True)
        o2, l2 = paged(return_lse=True)
    for _ in range(20):
        o3, l3 = chained(return_lse=True)
    dense.check_status()
    paged.check_status()
    chained.check_status()
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    assert torch.equal(o1, o3) and torch.equal(l1, l3)
    want, want_lse = oracle_fwd(c["q"], c["k"], c["v"], kv_lengths=c["kv_lengths"], sm_scale=c["sm_scale"])
    assert_close(o2, l2, want, want_lse, torch.bfloat16, "paged sharded decode")


def test_decode_cache_steps_match_causal_attention():
    """A ragged batch decoded token by token through DecodeCache (append kernel + split-KV
    decode) equals attention over each sequence's prefix (the reference's decode branch,
    layers/attention.py:603-675, checks its cache the same way in tests/test_attention.py)."""
    import oracle

    b, hq, hkv, d, cap = 3, 8, 2, 64, 256
    dtype = torch.bfloat16
    start = torch.tensor([0, 17, 100], dtype=torch.int32)
    steps = 5
    k_all, v_all = randn((b, cap, hkv, d), dtype, 1), randn((b, cap, hkv, d), dtype, 2)
    q_all = randn((b, steps, hq, d), dtype, 3)
    cache = pj.DecodeCache(b, cap, hkv, d, dtype=dtype, device=dev())
    # prefill each sequence's prefix in one append of the longest length, then fix the positions
    cache.update(k_all[:, :100].to(dev()), v_all[:, :100].to(dev()), advance=False)
    cache.reset(start)
    for t in range(steps):
        pos = start + t
        kn = torch.stack([k_all[i, pos[i]] for i in range(b)])[:, None].to(dev())
        vn = torch.stack([v_all[i, pos[i]] for i in range(b)])[:, None].to(dev())
        out = cache.step(q_all[:, t : t + 1].to(dev()), kn, vn)
        assert cache.cache_index.tolist() == (pos + 1).tolist()
        want = oracle.xla_attention(q_all[:, t : t + 1], k_all, v_all, kv_lengths=pos + 1, sm_scale=1 / math.sqrt(d))
        assert float((out.float().cpu() - want.float()).abs().max()) <= 2e-2
    assert not cache.overflowed()
    # running past the capacity is reported, not written
    cache.reset(torch.tensor([cap, 0, 0]))
    cache.update(k_all[:, :1].to(dev()), v_all[:, :1].to(dev()))
    assert cache.overflowed() and cache.cache_index.tolist() == [cap, 1, 1]


def test_decode_step_replays_as_a_cuda_graph():
    """Append + decode is two launches without a host round trip, so a step can be captured once
    and replayed: positions advance on the device between replays."""
    import oracle

    b, hq, hkv, d, cap = 2, 8, 2, 128, 512
    dtype = torch.bfloat16
    k_all, v_all = randn((b, cap, hkv, d), dtype, 1), randn((b, cap, hkv, d), dtype, 2)
    q_all = randn((b, 8, hq, d), dtype, 3)
    start = torch.tensor([300, 5], dtype=torch.int32)
    cache = pj.DecodeCache(b, cap, hkv, d, dtype=dtype, device=dev())
    cache.update(k_all[:, :300].to(dev()), v_all[:, :300].to(dev()), advance=False)
    cache.reset(start)
    q_in = torch.empty((b, 1, hq, d), dtype=dtype, device=dev())
    k_in, v_in = (torch.empty((b, 1, hkv, d), dtype=dtype, device=dev()) for _ in range(2))

    def feed(t):
        pos = start + t
        q_in.copy_(q_all[:, t : t + 1])
        k_in.copy_(torch.stack([k_all[i, pos[i]] for i in range(b)])[:, None])
        v_in.copy_(torch.stack([v_all[i, pos[i]] for i in range(b)])[:, None])

    side = torch.cuda.Stream()
    feed(0)
    with torch.cuda.stream(side):  # warm-up outside the capture (workspaces, status word)
        cache.step(q_in, k_in, v_in)
    side.synchronize()
    cache.reset(start)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        out = cache.step(q_in, k_in, v_in)
    cache.reset(start)  # the capture itself does not run the kernels
    for t in range(4):
        feed(t)
        graph.replay()
        torch.cuda.synchronize()
        assert cache.cache_index.tolist() == (start + t + 1).tolist()
        want = oracle.xla_attention(q_all[:, t : t + 1], k_all, v_all, kv_lengths=start + t + 1, sm_scale=1 / math.sqrt(d))
        assert float((out.float().cpu() - want.float()).abs().max()) <= 2e-2


@pytest.mark.parametrize("dtype,d,page", [(torch.bfloat16, 128, 256), (torch.float16, 64, 64)])
def test_paged_cache_decode_equals_contiguous_decode(dtype, d, page):
    """The same keys scattered over shuffled pages of a pool give the bits of the contiguous
    decode (same tiles, same order), which is checked against the oracle elsewhere."""
    b, hq, hkv, cap = 3, 8, 2, 1024
    lens = torch.tensor([1024, 333, 65], dtype=torch.int32)
    q = randn((b, 1, hq, d), dtype, 1)
    k, v = randn((b, cap, hkv, d), dtype, 2), randn((b, cap, hkv, d), dtype, 3)
    max_pages = cap // page
    n_pages = b * max_pages + 5
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(0))[: b * max_pages].view(b, max_pages)
    k_pool = torch.full((n_pages, page, hkv, d), float("nan"), dtype=dtype)
    v_pool = torch.full((n_pages, page, hkv, d), float("nan"), dtype=dtype)
    for i in range(b):
        for pg in range(max_pages):
            k_pool[perm[i, pg]] = k[i, pg * page : (pg + 1) * page]
            v_pool[perm[i, pg]] = v[i, pg * page : (pg + 1) * page]
    sc = 1 / math.sqrt(d)
    got, lse = pj.decode_paged(q.to(dev()), k_pool.to(dev()), v_pool.to(dev()), perm.to(torch.int32), lens, sm_scale=sc,
                               return_lse=True)
    want, want_lse = pj.decode_forward(q.to(dev()), k.to(dev()), v.to(dev()), kv_lengths=lens, sm_scale=sc, return_lse=True)
    assert torch.isfinite(got).all()
    assert torch.equal(got, want) and torch.equal(lse, want_lse)
    ref, ref_lse = oracle_fwd(q, k, v, kv_lengths=lens, sm_scale=sc)
    assert_close(got, lse, ref, ref_lse, dtype, "paged decode")
    with pytest.raises(ValueError, match="multiple of 64"):
        pj.decode_paged(q.to(dev()), k_pool[:, :48].contiguous().to(dev()), v_pool[:, :48].contiguous().to(dev()),
                        perm.to(torch.int32), lens, sm_scale=sc)


@pytest.mark.parametrize("R,H,dtype", [(576, 16, torch.bfloat16), (512, 32, torch.float16), (576, 6, torch.bfloat16)])
@pytest.mark.parametrize("mask", ["none", "causal", "bottom_right", "causal+lengths"])
def test_absorbed_latent_attention_over_many_tokens(R, H, dtype, mask):
    """Absorbed latent attention (K = V = latent, latent_attention.py:604-607) at the wide latents with
    hundreds of query tokens: every token runs as a one-token sequence of the latent decode kernels.
    Output and LSE against the oracle on the shared cache; keys past the valid lengths hold NaN."""
    d = dev()
    B, S = 3, 700
    Lq = 333 if mask == "bottom_right" else S
    q = randn((B, Lq, H, R), dtype, 5)
    cache = (randn((B, S, R), torch.float32, 6) * 0.5).to(dtype)
    sc = 1 / math.sqrt(R)
    lens, m = None, None
    keep = None
    if mask == "causal":
        m = pj.CausalMask()
        keep = m.dense(Lq, S, batch_size=B, num_heads=1)
    elif mask == "bottom_right":
        m = pj.CausalFromBottomRightMask(Lq, S)
        keep = m.dense(Lq, S, batch_size=B, num_heads=1)
    elif mask == "causal+lengths":
        lens = torch.tensor([700, 0, 129], dtype=torch.int32)
        m = pj.ComposeMask("and", pj.CausalMask(), pj.KVLenMask(lens))
        keep = pj.CausalMask().dense(Lq, S, batch_size=B, num_heads=1)
    shared = cache[:, :, None, :]
    want, want_lse = oracle.xla_attention(q, shared, shared, keep=keep, kv_lengths=lens, sm_scale=sc, return_lse=True)
    poisoned = cache.clone()
    if lens is not None:
        for b in range(B):
            poisoned[b, int(lens[b]):] = float("nan")
    for impl in (None, "b200:tcgen05", "b200:generic"):
        got, lse = pj.mla(q.to(d), poisoned.to(d), mask=m, sm_scale=sc, return_lse=True, implementation=impl)
        pj.check_status(d)
        assert_close(got, lse, want, want_lse, dtype, f"absorbed latent attention R={R} H={H} {mask} impl={impl}")


@pytest.mark.parametrize("R,H,Lq,dtype", [(576, 16, 1, torch.bfloat16), (512, 16, 1, torch.float16), (576, 8, 2, torch.bfloat16),
                                          (256, 5, 3, torch.bfloat16), (128, 32, 1, torch.bfloat16), (576, 6, 4, torch.float16)])
def test_absorbed_latent_decode(R, H, Lq, dtype):
    """Decode step of absorbed latent attention (K = V = latent) at real latent widths, ragged
    lengths and a cache tail full of NaN: every row against the oracle's absorbed form
    (latent_attention.py:604-607), through ``mla`` (routing) and the raw call (several split lengths)."""
    d = dev()
    B, S = 5, 1500
    q = randn((B, Lq, H, R), dtype, 1)
    cache = (randn((B, S, R), torch.float32, 2) * 0.5).to(dtype)
    lens = torch.tensor([1500, 1, 777, 64, 0], dtype=torch.int32)
    sc = 1 / math.sqrt(R)
    shared = cache[:, :, None, :]
    want, want_lse = oracle.xla_attention(q, shared, shared, kv_lengths=lens, sm_scale=sc, return_lse=True)
    poisoned = cache.clone()
    for b in range(B):
        poisoned[b, int(lens[b]):] = float("nan")
    got, lse = pj.mla(q.to(d), poisoned.to(d), mask=pj.KVLenMask(lens), sm_scale=sc, return_lse=True)
    assert_close(got, lse, want, want_lse, dtype, f"absorbed latent decode R={R} H={H} Lq={Lq}")
    pj.check_status(d)
    for impl in ("b200:tcgen05", "b200:generic"):  # TMA + tcgen05 kernel (the default) and the mma.sync kernel
        for split_len in (64, 256, 1536):
            got2, lse2 = pj.mla_decode(q.to(d), poisoned.to(d), kv_lengths=lens.to(d), sm_scale=sc, split_len=split_len,
                                       return_lse=True, impl=impl)
            pj.check_status(d)
            assert_close(got2, lse2, want, want_lse, dtype, f"{impl} split_len {split_len}")
    # no lengths: the whole cache
    got3 = pj.mla_decode(q.to(d), cache.to(d), sm_scale=sc)
    want3 = oracle.xla_attention(q, shared, shared, sm_scale=sc)
    assert_close(got3, None, want3, None, dtype, "whole cache")
    again = pj.mla_decode(q.to(d), cache.to(d), sm_scale=sc)
    assert torch.equal(got3, again)  # bit-repeatable
