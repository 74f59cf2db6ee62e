"""Host-side logic that needs no GPU: the C-ABI library loads and exports every
declared symbol, argument validation mirrors the reference's errors, mask
lowering, the dispatch seam, and the partition arithmetic of the sharded decode
(including a two-rank gloo run of the exchange)."""

import ctypes
import os
import re
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "pjx_attention.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pjx_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    from probjax_b200 import _lib

    handle = ctypes.CDLL(os.fspath(built_lib))
    names = _header_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    # the ctypes table binds exactly the declared functions
    assert sorted(_lib.SIGNATURES) == names
    L = _lib.lib()
    assert L.pjx_version() >= 100
    assert L.pjx_status_string(0) == b"ok"


def test_abi_validation_without_a_gpu(built_lib):
    """Argument errors are reported before anything touches the device."""
    from probjax_b200 import _lib

    L = _lib.lib()
    # Hq not a multiple of Hkv -> bad argument mentioning "multiple"
    rc = L.pjx_attn_fwd(None, None, None, None, None, None, None, 0, 0, 1, 4, 4, 3, 2, 8, 8, 0, 0, 1.0, 0, None, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "multiple" in _lib.last_error()
    with pytest.raises(ValueError, match="multiple"):
        _lib.check(rc)
    # unknown dtype
    assert L.pjx_attn_fwd(None, None, None, None, None, None, None, 0, 0, 1, 4, 4, 2, 2, 8, 8, 7, 0, 1.0, 0, None, None) == _lib.PJX_ERR_BAD_ARG
    # empty batch is a no-op
    assert L.pjx_attn_fwd(None, None, None, None, None, None, None, 0, 0, 0, 4, 4, 2, 2, 8, 8, 1, 0, 1.0, 0, None, None) == 0
    # mla: one projection without the other
    rc = L.pjx_mla_fwd(1, 1, 1, None, 1, None, None, None, 0, 0, 1, 4, 4, 2, 8, 8, 8, 1, 0, 1.0, 0, None, 0, None, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "both wk and wv" in _lib.last_error()
    # absorbed form needs Dqk == R
    rc = L.pjx_mla_fwd(1, 1, None, None, 1, None, None, None, 0, 0, 1, 4, 4, 2, 16, 8, 8, 1, 0, 1.0, 0, None, 0, None, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "qk_head_dim == kv_lora_rank" in _lib.last_error()
    # absorbed form at the wide latents: partials of the latent decode kernels live in the workspace
    assert L.pjx_mla_workspace_bytes(8, 2048, 16, 128, 128, 128, 1, 0) == 0
    need = L.pjx_mla_workspace_bytes(8, 2048, 16, 576, 576, 576, 1, 0)
    assert need >= 2048 * 16 * 577 * 4
    rc = L.pjx_mla_fwd(16, 16, None, None, 16, None, None, None, 0, 0, 8, 2048, 2048, 16, 576, 576, 576, 1, 1, 1.0, 0,
                       None, 0, None, None)
    assert rc == _lib.PJX_ERR_WORKSPACE and "mla workspace" in _lib.last_error()
    # decode workspace query and split-length rule
    assert L.pjx_attn_decode_default_split_len(16, 8, 32768) % 64 == 0
    need = L.pjx_attn_decode_workspace_bytes(16, 1, 32, 8, 128, 32768, 1024)
    assert need >= 16 * 8 * 32 * 4 * 129 * 4
    rc = L.pjx_attn_decode_splitkv(16, 16, 16, None, 16, None, 1, 1, 8, 2, 128, 128, 4096, 1, 1.0, 100, 0, None, 0, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "multiple of 64" in _lib.last_error()
    rc = L.pjx_attn_decode_splitkv(16, 16, 16, None, 16, None, 1, 1, 8, 2, 128, 128, 4096, 1, 1.0, 256, 0, None, 0, None)
    assert rc == _lib.PJX_ERR_WORKSPACE
    # backward / forward-mode / band entry points validate the same way
    rc = L.pjx_attn_bwd_band(1, 1, 1, 1, 1, 1, 1, 1, 1, None, None, 0, 0, None, 1, 4, 4, 3, 2, 8, 8, 1, -5, 0, 1.0, 0,
                             None, 0, None, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "multiple" in _lib.last_error()
    rc = L.pjx_attn_bwd_band(1, 1, 1, 1, 1, 1, 1, 1, 1, None, None, 0, 0, None, 1, 4, 4, 2, 2, 8, 8, 1, -5, 0, 1.0, 0,
                             None, 0, None, None)
    assert rc == _lib.PJX_ERR_WORKSPACE
    assert L.pjx_attn_bwd_workspace_bytes(2, 130, 4) == 2 * 2 * 4 * 256 * 4  # two padded float arrays
    rc = L.pjx_attn_jvp_band(1, 1, 1, None, None, None, 1, 1, None, None, 0, 0, 1, 4, 4, 3, 2, 8, 8, 1, 0, 0, 1.0, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "multiple" in _lib.last_error()
    assert L.pjx_attn_fwd_band(None, None, None, None, None, None, None, 0, 0, 1, 4, 4, 2, 2, 8, 8, 7, 0, 0, 1.0, 0, None, None) \
        == _lib.PJX_ERR_BAD_ARG
    # projections, rotary embedding, cache update
    assert L.pjx_linear(1, 1, 1, 4, 4, 0, 1, 0, None, None) == _lib.PJX_ERR_BAD_ARG
    assert L.pjx_linear(None, None, None, 0, 4, 8, 1, 0, None, None) == 0
    rc = L.pjx_rope_interleaved(1, 1, None, 0.0, 1, 4, 2, 64, 7, 10000.0, 1, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "rotary_dim" in _lib.last_error()
    rc = L.pjx_kv_cache_append(None, None, None, None, None, 2, 16, 1, 2, 64, 64, 1, 1, None, None)
    assert rc == _lib.PJX_ERR_BAD_ARG and "null" in _lib.last_error()
    assert L.pjx_launch_count() == 0


def test_python_api_validation_errors():
    import probjax_b200 as pj

    q = torch.zeros(2, 8, 4, 16)
    k = torch.zeros(2, 8, 2, 16)
    # layers/attention.py:1503-1508: heads differ without enable_gqa
    with pytest.raises(ValueError, match="enable_gqa=True"):
        pj.flex_attention(q, k, k)
    # layers/attention.py:1490-1495: dtypes differ
    with pytest.raises(ValueError, match="same dtype"):
        pj.flex_attention(q, k.half(), k, enable_gqa=True)
    # kernels/attention.py:2113-2120
    with pytest.raises(ValueError, match="multiple"):
        pj.mha(torch.zeros(1, 4, 3, 8), torch.zeros(1, 4, 2, 8), torch.zeros(1, 4, 2, 8))
    with pytest.raises(ValueError, match="implementation"):
        pj.flex_attention(q, q, q, implementation="cudnn")
    # latent_attention.py:668-696
    with pytest.raises(ValueError, match="rank 4"):
        pj.mla(torch.zeros(8, 4, 16), torch.zeros(8, 4, 16))
    with pytest.raises(ValueError, match="rank 3"):
        pj.mla(torch.zeros(1, 8, 4, 16), torch.zeros(1, 8, 4, 16))
    with pytest.raises(ValueError, match="batch mismatch"):
        pj.mla(torch.zeros(1, 8, 4, 16), torch.zeros(2, 8, 16))
    with pytest.raises(ValueError, match="both wk and wv"):
        pj.mla(torch.zeros(1, 8, 4, 16), torch.zeros(1, 8, 16), wk=torch.zeros(4, 16, 16))
    with pytest.raises(ValueError, match="qk_head_dim == kv_lora_rank"):
        pj.mla(torch.zeros(1, 8, 4, 16), torch.zeros(1, 8, 8))
    with pytest.raises(ValueError, match="wk must be"):
        pj.mla(torch.zeros(1, 8, 4, 16), torch.zeros(1, 8, 8), wk=torch.zeros(4, 8, 8), wv=torch.zeros(4, 8, 8))


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback():
    """Without a GPU every compute call raises; nothing is computed on the host."""
    import probjax_b200 as pj

    q = torch.zeros(1, 8, 2, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pj.flex_attention(q, q, q)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pj.mla(torch.zeros(1, 8, 2, 16), torch.zeros(1, 8, 16))
    assert pj.device_attention_defaults() is None
    assert pj.b200_attention_or_none(q, q, q, sm_scale=1.0) is None
    with pytest.raises(ValueError, match="cannot compute"):
        pj.b200_attention_or_none(q, q, q, sm_scale=1.0, force=True)


def test_mask_truth_tables():
    """tests/test_attention_mask_bias.py:62-67, 130-135, 152-162, 182-188 restated."""
    from probjax_b200 import CausalMask, KeyPaddingMask, KVLenMask, NoMask, QKVLengthMask

    def idx(n):
        return torch.arange(n, dtype=torch.int32)

    assert NoMask()(idx(5), idx(7)).shape == (5, 7) and NoMask()(idx(5), idx(7)).all()
    got = CausalMask()(idx(6), idx(6))
    assert torch.equal(got, idx(6)[:, None] >= idx(6)[None, :])
    got = QKVLengthMask(q_length=4, kv_length=6)(idx(7), idx(9))
    assert torch.equal(got, (idx(7)[:, None] < 4) & (idx(9)[None, :] < 6))
    lengths = torch.tensor([2, 4, 6], dtype=torch.int32)
    dense = KVLenMask(lengths).dense(5, 6, batch_size=3, num_heads=2)
    want = (idx(6)[None, :] < lengths[:, None])[:, None, None, :].expand(3, 2, 5, 6)
    assert torch.equal(dense, want)
    with pytest.raises(ValueError, match="does not match"):
        KVLenMask(lengths).dense(5, 6, batch_size=2)
    seg_q = torch.tensor([1, 3, 5, 6], dtype=torch.int32)
    got = KeyPaddingMask(torch.tensor([6]))(idx(4), idx(6), seg_q=seg_q)
    assert torch.equal(got, idx(6)[None, :] < seg_q[:, None])
    both = (CausalMask() & KVLenMask(lengths)).dense(6, 6, batch_size=3)
    assert torch.equal(both, CausalMask().dense(6, 6, batch_size=3) & KVLenMask(lengths).dense(6, 6, batch_size=3))


def test_mask_lowering():
    from probjax_b200 import CausalMask, ComposeMask, DenseBias, KeyPaddingMask, KVLenMask, NoMask, QKVLengthMask
    from probjax_b200.masks import lower_bias, lower_mask

    assert lower_mask(None, 2, 8, 8).causal is False
    assert lower_mask(NoMask(), 2, 8, 8).kv_lengths is None
    assert lower_mask(CausalMask(), 2, 8, 8).causal is True
    lm = lower_mask(CausalMask() & KVLenMask([3, 8]), 2, 8, 8)
    assert lm.causal and lm.kv_lengths.tolist() == [3, 8]
    lm = lower_mask(KVLenMask([3, 8]) & QKVLengthMask(q_length=5, kv_length=6), 2, 8, 8)
    assert lm.kv_lengths.tolist() == [3, 6] and lm.q_limit == 5
    assert lower_mask(KeyPaddingMask(torch.tensor([4, 7])), 2, 1, 8).kv_lengths.tolist() == [4, 7]
    with pytest.raises(NotImplementedError):
        lower_mask(KeyPaddingMask(torch.tensor([4, 7])), 2, 4, 8)
    with pytest.raises(NotImplementedError):
        lower_mask(ComposeMask("or", CausalMask(), NoMask()), 2, 8, 8)
    with pytest.raises(ValueError):
        lower_mask(KVLenMask([1, 2, 3]), 2, 8, 8)
    with pytest.raises(ValueError):  # attention_mask_bias.py:1815-1823
        DenseBias(torch.zeros(8, 8))
    b = DenseBias(torch.zeros(1, 4, 8, 8))
    assert lower_bias(b, 2, 4, 8, 8).shape == (1, 4, 8, 8)
    with pytest.raises(ValueError, match="shape mismatch"):
        lower_bias(b, 2, 4, 8, 9)
    with pytest.raises(ValueError, match="head dim"):
        lower_bias(b, 2, 2, 8, 8)


def test_block_cyclic_partition():
    from probjax_b200.dist import local_capacity, local_lengths, shard_cache

    rng = np.random.default_rng(0)
    for world in (1, 2, 4, 8):
        for page in (1, 16, 256):
            lens = torch.from_numpy(rng.integers(0, 5000, size=32))
            per_rank = torch.stack([local_lengths(lens, r, world, page) for r in range(world)])
            assert torch.equal(per_rank.sum(0).to(torch.int64), lens)  # every token lives on exactly one rank
            # brute force
            for b in range(4):
                t = torch.arange(int(lens[b]))
                for r in range(world):
                    assert int(per_rank[r, b]) == int((((t // page) % world) == r).sum())
            assert int((per_rank.max(0).values - per_rank.min(0).values).max()) <= page
    cache = torch.arange(2 * 40 * 1 * 1).reshape(2, 40, 1, 1)
    parts = [shard_cache(cache, r, 4, 8) for r in range(4)]
    assert [p.shape[1] for p in parts] == [16, 8, 8, 8]
    assert [local_capacity(40, r, 4, 8) for r in range(4)] == [16, 8, 8, 8]
    assert parts[1][0, :, 0, 0].tolist() == list(range(8, 16))
    # the first local_lengths rows of a shard are exactly the valid tokens of that rank
    lens = torch.tensor([19, 40])
    for r in range(4):
        ll = local_lengths(lens, r, 4, 8)
        valid = parts[r][0, : int(ll[0]), 0, 0]
        assert (valid < 19).all() and int(ll.sum()) > 0 or int(ll[0]) == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _sharded_worker(rank, world, port, page, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    import oracle
    from probjax_b200.dist import decode_sharded, shard_cache

    c = oracle.make_config(4, B=3, Hq=8, Hkv=2, D=32, cap=700, dtype="f32")
    q, k, v, lens = c["q"], c["k"], c["v"], c["kv_lengths"]
    lens[0] = 5  # shorter than one page: most ranks hold nothing of this sequence
    k_loc, v_loc = shard_cache(k, rank, world, page), shard_cache(v, rank, world, page)

    def local_fn(q_, k_, v_, l_):  # CPU stand-in for the decode kernel
        o, lse = oracle.xla_attention(q_, k_, v_, kv_lengths=l_, sm_scale=c["sm_scale"], return_lse=True)
        return o.float(), lse

    def combine_fn(o_parts, lse_parts):  # CPU stand-in for pjx_attn_combine (natural log, +inf = empty)
        neg = torch.where(torch.isinf(lse_parts) & (lse_parts > 0), torch.tensor(-float("inf")), lse_parts)
        m = neg.max(0).values
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        w = torch.exp(neg - m)
        den = w.sum(0)
        o = (w[..., None] * o_parts).sum(0) / torch.where(den > 0, den, torch.ones_like(den))[..., None]
        return o, torch.where(den > 0, m + torch.log(den), torch.tensor(float("inf")))

    o, lse = decode_sharded(q, k_loc, v_loc, lens, page=page, sm_scale=c["sm_scale"], return_lse=True,
                            _local_fn=local_fn, _combine_fn=combine_fn)
    want, want_lse = oracle.xla_attention(q, k, v, kv_lengths=lens, sm_scale=c["sm_scale"], return_lse=True)
    err = float((o - want).abs().max())
    err_lse = float((lse - want_lse).abs().max())
    torch.save({"err": err, "err_lse": err_lse}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_decode_two_ranks_gloo(tmp_path):
    """World size 2 on CPU: partition, all-gather and combine reproduce the unsharded answer."""
    world, page = 2, 64
    mp.spawn(_sharded_worker, args=(world, _free_port(), page, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        assert res["err"] < 1e-5 and res["err_lse"] < 1e-5


def test_window_masks_lower_to_bands_and_compose():
    import torch
    from probjax_b200.masks import (CausalFromBottomRightMask, CausalLocalWindowMask, CausalMask, KVLenMask,
                                    LocalWindowMask, lower_mask)

    lm = lower_mask(LocalWindowMask(7, 3), 2, 16, 16)
    assert (lm.band_lo, lm.band_hi, lm.causal, lm.banded) == (-7, 3, False, True)
    assert lower_mask(LocalWindowMask(7), 2, 16, 16).band == (-7, 0)
    assert lower_mask(CausalLocalWindowMask(5), 2, 16, 16).band == (-5, 0)
    assert lower_mask(CausalFromBottomRightMask(4, 10), 2, 4, 10).band == (None, 6)
    assert lower_mask(CausalMask(), 2, 16, 16).causal
    both = lower_mask(CausalMask() & LocalWindowMask(9, 9) & KVLenMask(torch.tensor([3, 16])), 2, 16, 16)
    assert both.band == (-9, 0) and both.kv_lengths.tolist() == [3, 16] and not both.causal
    # dense forms follow the reference's predicates (attention_mask_bias.py:651-782)
    i, j = torch.arange(6)[:, None], torch.arange(8)[None, :]
    assert torch.equal(LocalWindowMask(2, 1).dense(6, 8)[0, 0], (i - j >= -1) & (i - j <= 2))
    assert torch.equal(CausalLocalWindowMask(2).dense(6, 8)[0, 0], (i - j >= 0) & (i - j <= 2))
    assert torch.equal(CausalFromBottomRightMask(6, 8).dense(6, 8)[0, 0], i + 2 >= j)


def test_dense_lowered_masks_and_biases_follow_the_reference_predicates():
    """Classes without a native kernel form: dense semantics of attention_mask_bias.py and the
    split of an AND-expression into a native part and a dense residual."""
    import math

    import torch
    from probjax_b200 import masks as M

    i, j = torch.arange(6)[:, None], torch.arange(7)[None, :]
    ids_q, ids_k = torch.tensor([0, 0, 1, 1, 2, 2]), torch.tensor([0, 0, 0, 1, 1, 2, 2])
    assert torch.equal(M.PrefixLMMask(torch.tensor([3, 1])).dense(6, 7, batch_size=2)[1, 0], (j < 1) | (i >= j))
    assert torch.equal(M.BlockDiagonalMask(ids_q, ids_k).dense(6, 7)[0, 0], ids_q[:, None] == ids_k[None, :])
    assert torch.equal(M.BlockDiagonalCausalMask(ids_q, ids_k).dense(6, 7)[0, 0],
                       (ids_q[:, None] == ids_k[None, :]) & (i >= j))
    assert torch.equal(M.SameSegmentMask(torch.stack([ids_q, ids_q + 1])).dense(6, 6, batch_size=2)[1, 0],
                       ids_q[:, None] == ids_q[None, :])
    sl = M.SeqLenMask(torch.tensor([4, 6])).dense(6, 7, batch_size=2)
    assert torch.equal(sl[0, 0], ((i < 4) & (j < 4)) | (i == j))
    keep = torch.tensor([True, False, True, True, False, True, True])
    assert torch.equal(M.MarginalizationMask(keep).dense(6, 7)[0, 0], (keep[:6, None] & keep[None, :]) | (i == j))
    assert torch.equal(M.NotMask(M.CausalMask()).dense(6, 7)[0, 0], ~(i >= j))
    assert torch.equal((M.ComposeMask("or", M.CausalMask(), M.LocalWindowMask(0, 2))).dense(6, 7)[0, 0],
                       (i >= j) | ((i - j >= -2) & (i - j <= 0)))
    # biases
    slopes = torch.exp2(-(torch.arange(4.0) + 1))
    assert torch.allclose(M.CausalAlibiBias().dense(6, 7, num_heads=4)[0], -slopes[:, None, None] * (i - j).clamp_min(0))
    assert torch.allclose(M.SymmetricAlibiBias().dense(6, 7, num_heads=4)[0], -slopes[:, None, None] * (i - j).abs())
    assert torch.allclose(M.DistanceDecayBias(0.5).dense(6, 7)[0, 0], -0.5 * (i - j).abs().float())
    qf, kf = torch.randn(2, 8, 3), torch.randn(2, 9, 3)
    assert torch.allclose(M.LowRankBias(qf, kf, scale=2.0).dense(6, 7, num_heads=2)[0],
                          2.0 * torch.einsum("hqr,hkr->hqk", qf[:, :6], kf[:, :7]))
    both = M.SumBias(M.ConstantBias(1.5), M.DistanceDecayBias(1.0)).dense(6, 7)
    assert torch.allclose(both[0, 0], 1.5 - (i - j).abs().float())
    # an AND-expression keeps its native part native
    lm, residual = M.split_mask(M.CausalMask() & M.NotMask(M.SameSegmentMask(ids_q)) & M.KVLenMask(torch.tensor([5])), 1, 6, 6)
    assert lm.causal and lm.kv_lengths.tolist() == [5] and isinstance(residual, M.NotMask)
    add = M.lower_dense(residual, M.ConstantBias(2.0), 1, 2, 6, 6)
    want = torch.where(ids_q[:, None] != ids_q[None, :], torch.tensor(2.0), torch.tensor(-math.inf))
    assert torch.equal(add[0, 0], want)


def test_structured_lowering_of_masks_and_biases():
    """Masks and biases the kernels evaluate per element lower to O(B T) / O(H T) data whose meaning
    equals the classes' dense definitions (attention_mask_bias.py)."""
    import torch
    from probjax_b200 import masks as M

    b, t = 2, 9
    i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]

    def keep_of(lm):  # the kernels' rule, evaluated densely
        band = torch.ones(t, t, dtype=torch.bool)
        if lm.band_lo is not None:
            band &= j >= i + lm.band_lo
        if lm.band_hi is not None:
            band &= j <= i + lm.band_hi
        out = band[None].expand(b, t, t).clone()
        if lm.prefix_len is not None:
            out |= j[None] < lm.prefix_len[:, None, None]
        if lm.seg_q is not None:
            out &= lm.seg_q.expand(b, t)[:, :, None] == lm.seg_k.expand(b, t)[:, None, :]
        if lm.row_kv_limit is not None:
            out &= j[None] < lm.row_kv_limit.expand(b, t)[:, :, None]
        if lm.kv_lengths is not None:
            out &= j[None] < lm.kv_lengths[:, None, None]
        return out

    g = torch.Generator().manual_seed(3)
    seg = torch.randint(0, 3, (b, t), generator=g)
    tok = torch.rand((b, t), generator=g) > 0.4
    for mask in (M.SameSegmentMask(seg, seg.flip(1)), M.BlockDiagonalMask(seg[0]), M.BlockDiagonalCausalMask(seg),
                 M.SeqLenMask(torch.tensor([9, 4])), M.MarginalizationMask(tok), M.PrefixLMMask(torch.tensor([3, 0])),
                 M.PrefixLMMask(torch.tensor([2, 5])) & M.KVLenMask(torch.tensor([7, 9])),
                 M.SameSegmentMask(seg) & M.CausalLocalWindowMask(3)):
        lm, residual = M.split_mask(mask, b, t, t)
        assert residual is None and lm.structured, type(mask).__name__
        assert torch.equal(keep_of(lm), mask.dense(t, t, batch_size=b)[:, 0]), type(mask).__name__
    rows = torch.randint(1, t + 1, (t,), generator=g)
    lm = M.lower_mask(M.KeyPaddingMask(rows), b, t, t)
    assert torch.equal(keep_of(lm)[1], j < rows[:, None])
    # a prefix cannot be merged with a band from another mask: that part goes dense
    lm, residual = M.split_mask(M.PrefixLMMask(torch.tensor([3, 5])) & M.LocalWindowMask(2, 2), b, t, t)
    assert lm.prefix_len is not None and isinstance(residual, M.LocalWindowMask)
    # two segment masks: one native, one dense
    lm, residual = M.split_mask(M.SameSegmentMask(seg) & M.MarginalizationMask(tok), b, t, t)
    assert lm.seg_q is not None and isinstance(residual, M.MarginalizationMask)

    heads = 4
    rel = (j - i)
    t5 = M.T5RelativePositionBias(torch.randn(heads, 8, generator=g), num_buckets=8, max_distance=16)
    lr = M.LearnedRelativePositionBias(torch.randn(1, 7, generator=g), max_distance=3)
    assert torch.equal(lr.dense(t, t)[0, 0], lr.tab[0][rel.clamp(-3, 3) + 3])
    for bias in (t5, lr, M.ConstantBias(0.25), M.SumBias(M.CausalAlibiBias(), M.SymmetricAlibiBias()),
                 M.SumBias(M.DistanceDecayBias(0.5), M.SumBias(t5, M.ConstantBias(-1.0)))):
        lb = M.lower_bias_structured(bias, b, heads, t, t)
        assert lb.dense is None and lb.structured
        total = torch.zeros(heads, t, t)
        if lb.rel_bias is not None:
            assert lb.rel_bias.shape[1] == 2 * t - 1
            total = total + lb.rel_bias.expand(heads, -1)[:, (rel + t - 1).reshape(-1)].reshape(heads, t, t)
        if lb.alibi_slopes is not None:
            dist = (i - j).clamp_min(0) if lb.alibi_mode == 1 else (i - j).abs()
            total = total - lb.alibi_slopes[:, None, None] * dist
        want = bias.dense(t, t, batch_size=1, num_heads=heads)[0].expand(heads, t, t)
        assert torch.allclose(total, want, atol=1e-6), type(bias).__name__
    lb = M.lower_bias_structured(M.SumBias(M.SoftCappingBias(5.0), M.PerHeadScaleBias(torch.tensor([2.0]))), b, heads, t, t)
    assert lb.softcap == 5.0 and lb.head_scale.tolist() == [2.0] * heads
    # T5 buckets (attention_mask_bias.py:2417-2449), 8 buckets, bidirectional: 4 per sign, distances 0 and 1
    # exact, then 2 + floor(2 ln(d / 2) / ln 8) capped at 3; keys after the query use buckets 4..7
    bk = M._t5_bucket(torch.tensor([0, -1, -3, -4, -100, 1, 3, 100]), num_buckets=8, max_distance=16, bidirectional=True)
    assert bk.tolist() == [0, 1, 2, 2, 3, 5, 6, 7]
    lm2, res2 = M.split_mask(M.CausalMask(), 1, 6, 6)
    assert res2 is None and lm2.causal


def test_raw_wrappers_reject_mismatched_tensors_before_the_library_call():
    """The C ABI takes every size from q, k and v; the host wrapper must refuse tensors that
    disagree with them (the reference raises a shape error at trace time for the same calls)."""
    import torch
    from probjax_b200 import attention as A

    q = torch.zeros(2, 8, 4, 16)
    k = torch.zeros(2, 12, 2, 16)
    v = torch.zeros(2, 12, 2, 24)
    assert A._check_call(q, k, v) == (2, 8, 12, 4, 2, 16, 24)
    bad = [
        dict(k=torch.zeros(2, 12, 2, 8)),                    # head width differs from q
        dict(k=torch.zeros(3, 12, 2, 16)),                   # batch differs
        dict(v=torch.zeros(2, 10, 2, 24)),                   # v shorter than k
        dict(v=torch.zeros(2, 12, 1, 24)),                   # v head count differs from k
        dict(k=torch.zeros(2, 12, 3, 16), v=torch.zeros(2, 12, 3, 24)),  # 4 query heads over 3 kv heads
        dict(k=k.half()),                                    # dtype differs
        dict(bias=torch.zeros(1, 4, 8, 11)),                 # bias key axis
        dict(bias=torch.zeros(3, 4, 8, 12)),                 # bias batch axis neither 1 nor B
        dict(bias=torch.zeros(4, 8, 12)),                    # bias rank
        dict(kv_lengths=torch.zeros(1, dtype=torch.int32)),  # fewer lengths than batch rows
        dict(o=torch.zeros(2, 8, 4, 16)),                    # o must carry v's width
        dict(d_o=torch.zeros(2, 8, 2, 24)),
        dict(lse=torch.zeros(2, 8, 4)),                      # lse is [B, Hq, Lq]
        dict(q=torch.zeros(8, 4, 16)),                       # rank 3
    ]
    for kw in bad:
        args = dict(q=q, k=k, v=v)
        args.update(kw)
        qq, kk, vv = args.pop("q"), args.pop("k"), args.pop("v")
        with pytest.raises(ValueError):
            A._check_call(qq, kk, vv, **args)
    # every raw wrapper goes through the validator before it touches the library
    import inspect

    for fn in (A.attention_forward, A.attention_backward, A.attention_jvp, A.decode_forward):
        assert "_check_call(" in inspect.getsource(fn), fn.__name__


def test_ffi_shim_is_consistent_and_compiles_without_jaxlib(tmp_path):
    """The XLA FFI shim cannot run here (no jaxlib), but its gate must hold: the file compiles to an
    object that only says why it is empty, every handler symbol it defines is one the Python side
    registers, and every C function it forwards to is declared in the header."""
    import re
    import shutil
    import subprocess

    from probjax_b200 import build as B
    from probjax_b200 import jax_ffi

    src = (B.CSRC / "ffi_shim.cc").read_text()
    defined = re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\(\s*(\w+)", src)
    assert sorted(defined) == sorted(jax_ffi.TARGETS)
    header = (B.INCLUDE / "pjx_attention.h").read_text()
    for fn in set(re.findall(r"\b(pjx_[a-z0-9_]+)\(", src)) - {"pjx_ffi_unavailable"}:
        assert re.search(r"\b" + fn + r"\(", header), f"{fn} is not declared in pjx_attention.h"
    assert not jax_ffi.available() or B.jax_include_dir()
    if B.jax_include_dir() is None:
        assert B.build_ffi() is None
        obj = tmp_path / "ffi_shim.o"
        gxx = shutil.which("g++")
        res = subprocess.run([gxx, "-std=c++17", "-c", "-fPIC", "-I", str(B.INCLUDE), str(B.CSRC / "ffi_shim.cc"),
                              "-o", str(obj)], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
        syms = subprocess.run(["nm", "-g", str(obj)], capture_output=True, text=True).stdout
        assert "pjx_ffi_unavailable" in syms


def test_low_rank_family_factors_and_dense_forms():
    """attention_mask_bias.py:2028-2192 (per-example factors), 2258-2351 (caller-owned ALiBi slopes):
    ``dense`` equals ``scale * qf @ kf^T`` / ``-slope ((q + qo) - (k + ko))`` and the factor layouts are
    the ones ``flex_attention`` concatenates onto q and k."""
    from probjax_b200 import masks as M

    g = torch.Generator().manual_seed(5)
    log_m = torch.randn((3, 10), generator=g)
    kb = M.BatchedLowRankBias.from_key_bias(log_m)
    qf, kf = kb.factors(7, 10, 4)
    assert tuple(qf.shape) == (3, 7, 1, 1) and tuple(kf.shape) == (3, 10, 1, 1) and kb.rank == 1
    d = kb.dense(7, 10, batch_size=3, num_heads=4)
    assert torch.allclose(d.expand(3, 4, 7, 10), log_m[:, None, None, :].expand(3, 4, 7, 10))
    with pytest.raises(ValueError, match="exceeds maximum"):
        kb.factors(7, 11, 4)
    with pytest.raises(ValueError, match=r"\[B, length, rank\]"):
        M.BatchedLowRankBias(torch.zeros(3, 4), torch.zeros(3, 4))
    with pytest.raises(ValueError, match="same batch size"):
        M.BatchedLowRankBias(torch.zeros(2, 4, 1), torch.zeros(3, 4, 1))
    lb = M.lower_bias_structured(kb, 3, 4, 7, 10)
    assert lb.low_rank == (kb,) and lb.dense is None and not lb.structured
    with pytest.raises(ValueError, match="Cannot broadcast factors of batch"):
        M.lower_bias_structured(kb, 2, 4, 7, 10)

    slopes = torch.tensor([0.5, 0.25])
    la = M.LearnedAlibiBias(slopes, query_offset=3, key_offset=1)
    want = -slopes[:, None, None] * ((torch.arange(6)[:, None] + 3) - (torch.arange(9)[None, :] + 1))
    assert torch.allclose(la.dense(6, 9, num_heads=2)[0], want.float())
    qf, kf = la.factors(6, 9, 2)
    assert tuple(qf.shape) == (1, 6, 2, 2) and tuple(kf.shape) == (1, 9, 2, 2)
    assert torch.allclose(torch.einsum("bqhr,bkhr->bhqk", qf, kf)[0], want)
    lb = M.lower_bias_structured(la, 1, 2, 6, 9)  # no gradient asked for: a relative-position table
    assert lb.low_rank == () and tuple(lb.rel_bias.shape) == (2, 14)
    assert torch.allclose(lb.rel_bias[:, (torch.arange(9)[None, :] - torch.arange(6)[:, None]) + 5], want.float())
    lg = M.LearnedAlibiBias(slopes.clone().requires_grad_(True))
    assert M.lower_bias_structured(lg, 1, 2, 6, 9).low_rank == (lg,)  # folded: the gradient reaches the slopes
    with pytest.raises(ValueError, match="cannot broadcast"):
        M.lower_bias_structured(M.LearnedAlibiBias(torch.ones(3)), 1, 2, 6, 9)


def test_latent_layer_dropout_resolution():
    """tests/test_latent_attention.py:589-630 -- a rate needs an explicit `deterministic`; a kept stream
    or a per-call key supplies the randomness; rates outside [0, 1) are rejected."""
    from probjax_b200.latent_layer import MultiHeadLatentAttention

    def layer(**kw):
        return MultiHeadLatentAttention(2, 32, kv_lora_rank=16, dtype=torch.float32, device="cpu", **kw)

    for rate in (-0.1, 1.0, 1.5):
        with pytest.raises(ValueError, match="dropout_rate"):
            layer(dropout_rate=rate)
    plain = layer()
    assert plain._resolve_dropout(None, None) == (0.0, None)  # no rate: `deterministic` is not needed
    lay = layer(dropout_rate=0.1)
    with pytest.raises(ValueError, match="No `deterministic` argument"):
        lay._resolve_dropout(None, 7)  # a key alone must not switch dropout on
    assert lay._resolve_dropout(True, 7) == (0.0, None)
    assert lay._resolve_dropout(False, 7) == (0.1, 7)
    lay = layer(dropout_rate=0.1, deterministic=False, seed=5)
    a, b = lay._resolve_dropout(None, None), lay._resolve_dropout(None, None)
    assert a[0] == b[0] == 0.1 and a[1] != b[1] and a[1][0] == 5  # the kept stream advances per call
    lay = layer(dropout_rate=0.1, deterministic=False, keep_rngs=False)
    with pytest.raises(ValueError, match="keep_rngs=True"):
        lay._resolve_dropout(None, None)
    assert lay._resolve_dropout(None, [1, 2]) == (0.1, [1, 2])
