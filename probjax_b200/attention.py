"""probjax.nn's attention call signatures on top of the sm_100a CUDA library.

``dot_product_attention`` / ``flex_attention`` (probjax/nn/layers/attention.py:
1205-1319, 1426-1759), ``mha`` (probjax/nn/pallas_kernels/kernels/attention.py:
2692-2984), ``splitkv_forward`` (.../attention_splitkv.py:137-250) and ``mla``
(.../latent_attention.py:636-766) with the same argument names, defaults, layouts
(``[..., T, H, D]``) and errors.  Arrays are torch tensors: CUDA tensors are used in
place; CPU tensors and NumPy arrays go through the library's host-buffer call
(copy in, compute on the GPU, copy out).  There is no CPU computation here: every
function ends in a call into ``libpjx_attention.so`` and raises when that library
or a GPU is missing.
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from . import _lib
from .masks import (AttentionBias, AttentionMask, LoweredBias, LoweredMask, NoMask, lower_bias, lower_bias_structured,
                    lower_dense, lower_mask, split_mask)

_DTYPES = {torch.float32: _lib.PJX_F32, torch.bfloat16: _lib.PJX_BF16, torch.float16: _lib.PJX_F16}
_IMPL = {None: _lib.IMPL_AUTO, "b200": _lib.IMPL_AUTO, "b200:generic": _lib.IMPL_GENERIC,
         "b200:tcgen05": _lib.IMPL_SM100}

# kernels/attention.py:2649-2650
_SPLITKV_MAX_Q_LEN = 64
_SPLITKV_MIN_KV_LEN = 1024

_status_words: dict = {}
_scratch: dict = {}


def _ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _status_word(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel on ``device`` reported a timed-out wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(device)
    rc = _lib.lib().pjx_read_status(_ptr(word), _stream(device))
    if rc:
        word.zero_()
    _lib.check(rc)


def _scratch_bytes(device, tag: str, nbytes: int) -> torch.Tensor:
    """A cached, growing device byte buffer (decode partials, projections, staging), one per
    (device, CUDA stream, purpose): calls issued on different streams never share scratch, and a
    buffer that is outgrown is only dropped by the stream that owns it, whose earlier kernels
    are ordered before anything that reuses the memory."""
    device = torch.device(device)
    key = (device.index or 0, _stream(device), tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _check_call(q, k, v, *, bias=None, kv_lengths=None, o=None, lse=None, d_o=None, what="attention"):
    """Shape, dtype and device agreement of the tensors of one kernel call.  The C ABI takes
    sizes from q, k and v and indexes every other buffer with them, so a mismatch here would
    read or write past an allocation; the reference raises at trace time for the same mistakes."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dim() != 4:
            raise ValueError(f"{what}: {name} must be rank 4 [B, T, H, D], got shape {tuple(t.shape)}")
    if q.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {q.dtype}; expected float32, bfloat16 or float16")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"{what}: q, k and v must share a dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    if k.device != q.device or v.device != q.device:
        raise ValueError(f"{what}: q, k and v must live on one device, got {q.device}, {k.device}, {v.device}")
    B, Lq, Hq, D = q.shape
    Lkv, Hkv = k.shape[1], k.shape[2]
    if tuple(k.shape) != (B, Lkv, Hkv, D):
        raise ValueError(f"{what}: k must be [B={B}, Lkv, Hkv, D={D}], got {tuple(k.shape)}")
    if tuple(v.shape[:3]) != (B, Lkv, Hkv):
        raise ValueError(f"{what}: v must be [B={B}, Lkv={Lkv}, Hkv={Hkv}, Dv], got {tuple(v.shape)}")
    _gqa_group(Hq, Hkv)
    Dv = v.shape[3]
    if bias is not None:
        if bias.dim() != 4 or tuple(bias.shape[-2:]) != (Lq, Lkv) or bias.shape[0] not in (1, B) \
                or bias.shape[1] not in (1, Hq):
            raise ValueError(f"{what}: bias must be [B|1, H|1, Lq={Lq}, Lkv={Lkv}], got {tuple(bias.shape)}")
    if kv_lengths is not None and kv_lengths.numel() != B:
        raise ValueError(f"{what}: kv_lengths must hold B={B} entries, got {kv_lengths.numel()}")
    for name, t, shape in (("o", o, (B, Lq, Hq, Dv)), ("d_o", d_o, (B, Lq, Hq, Dv)), ("lse", lse, (B, Hq, Lq))):
        if t is not None and tuple(t.shape) != shape:
            raise ValueError(f"{what}: {name} must be {shape}, got {tuple(t.shape)}")
    return B, Lq, Lkv, Hq, Hkv, D, Dv


def _as_tensor(x):
    if isinstance(x, torch.Tensor):
        return x
    if isinstance(x, np.ndarray):
        return torch.from_numpy(np.ascontiguousarray(x))
    raise TypeError(f"expected a torch.Tensor or numpy.ndarray, got {type(x).__name__}")


def _result(given, shape, dtype, device, pin=False):
    """The caller's result tensor if it fits (contiguous, right shape / dtype / side), else a new one."""
    if given is not None:
        if tuple(given.shape) != tuple(shape) or given.dtype != dtype or given.device.type != torch.device(device).type \
                or not given.is_contiguous():
            raise ValueError(f"result tensor must be contiguous {tuple(shape)} {dtype} on {device}")
        return given
    if torch.device(device).type == "cpu":
        return torch.empty(shape, dtype=dtype, pin_memory=pin)
    return torch.empty(shape, dtype=dtype, device=device)


def _require_gpu():
    _lib.lib()  # raises when the library is not built
    if not torch.cuda.is_available():
        raise RuntimeError("probjax_b200 needs a CUDA device (sm_100a); there is no CPU path")


def _gqa_group(hq: int, hkv: int) -> int:
    # kernels/attention.py:2113-2120
    if hq % hkv != 0:
        raise ValueError(f"query heads ({hq}) must be a multiple of key/value heads ({hkv})")
    return hq // hkv


_constant_copies: dict = {}  # (id of a library constant, device, dtype) -> (the constant, its device copy)


class ScoreMods:
    """The ``pjx_score_mod`` argument of one call: the structured part of a lowered mask and bias
    (segment ids, per-row key limits, prefix lengths, relative-position table, ALiBi slopes, per-head
    scale, soft cap) as device tensors plus the C struct that points at them.  Keeps the tensors
    alive for as long as the object lives."""

    def __init__(self, lm: LoweredMask | None = None, lb: LoweredBias | None = None, device=None,
                 dropout_rate: float = 0.0, dropout_seed: int = 0):
        import ctypes

        self.device = torch.device(device)
        self._keep = []
        st = _lib.ScoreMod()

        def put(t, dtype):
            if getattr(t, "_pjx_constant", False):
                # a constant of the library (ALiBi slopes): one device copy per device, not one pageable
                # upload -- which waits for the stream -- per call
                key = (id(t), self.device.index or 0, dtype)
                hit = _constant_copies.get(key)
                if hit is None:
                    hit = _constant_copies[key] = (t, t.to(device=self.device, dtype=dtype).contiguous())
                t = hit[1]
            else:
                t = torch.as_tensor(t).to(device=self.device, dtype=dtype).contiguous()
            self._keep.append(t)
            return t

        if lm is not None:
            if lm.seg_q is not None:
                sq, sk = put(lm.seg_q, torch.int32), put(lm.seg_k, torch.int32)
                st.seg_q, st.seg_k = sq.data_ptr(), sk.data_ptr()
                st.seg_q_batch_stride = 0 if sq.shape[0] == 1 else sq.stride(0)
                st.seg_k_batch_stride = 0 if sk.shape[0] == 1 else sk.stride(0)
            if lm.row_kv_limit is not None:
                rl = put(lm.row_kv_limit, torch.int32)
                st.row_kv_limit = rl.data_ptr()
                st.row_kv_limit_batch_stride = 0 if rl.shape[0] == 1 else rl.stride(0)
            if lm.prefix_len is not None:
                st.prefix_len = put(lm.prefix_len, torch.int32).data_ptr()
        if lb is not None:
            if lb.rel_bias is not None:
                rb = put(lb.rel_bias, torch.float32)
                st.rel_bias = rb.data_ptr()
                st.rel_bias_head_stride = 0 if rb.shape[0] == 1 else rb.stride(0)
            if lb.alibi_slopes is not None:
                st.alibi_slopes = put(lb.alibi_slopes, torch.float32).data_ptr()
                st.alibi_mode = int(lb.alibi_mode)
            if lb.head_scale is not None:
                st.head_scale = put(lb.head_scale, torch.float32).data_ptr()
            st.softcap = float(lb.softcap)
        if not 0.0 <= dropout_rate < 1.0:
            raise ValueError(f"dropout_rate must be in [0, 1), got {dropout_rate}")
        st.dropout_rate = float(dropout_rate)
        st.dropout_seed = int(dropout_seed) & 0xFFFFFFFF
        self.struct = st
        self.active = bool(self._keep) or st.softcap > 0 or st.dropout_rate > 0
        self.nbytes = sum(t.numel() * t.element_size() for t in self._keep)
        self._ref = ctypes.byref(st)

    @staticmethod
    def arg(mods):
        """The pointer to pass for ``mods`` (``None`` = a null pointer)."""
        return None if mods is None or not mods.active else mods._ref


# ---------------------------------------------------------------------------
# Raw calls (rank-4 tensors, structural mask)
# ---------------------------------------------------------------------------


_BAND_NO_LOWER, _BAND_NO_UPPER = -(1 << 30), 1 << 30


def _band_args(causal, band):
    """(band_lo, band_hi) C arguments from the ``causal`` flag and an optional
    ``(lo, hi)`` pair (``None`` = open side): key ``j`` is visible to query ``i`` iff
    ``i + lo <= j <= i + hi``."""
    lo, hi = (None, None) if band is None else band
    if causal:
        hi = 0 if hi is None else min(int(hi), 0)
    lo = _BAND_NO_LOWER if lo is None else max(int(lo), _BAND_NO_LOWER)
    hi = _BAND_NO_UPPER if hi is None else min(int(hi), _BAND_NO_UPPER)
    return lo, hi


def attention_forward(q, k, v, *, causal=False, band=None, kv_lengths=None, bias=None, sm_scale=1.0,
                      return_lse=False, impl=None, out=None, lse_out=None, mods: ScoreMods | None = None):
    """One ``pjx_attn_fwd_mod`` call. ``q [B,Lq,Hq,D]``, ``k [B,Lkv,Hkv,D]``,
    ``v [B,Lkv,Hkv,Dv]``; CUDA tensors stay on the device, host tensors use the
    host-buffer entry point.  ``band = (lo, hi)`` limits query ``i`` to keys
    ``i + lo .. i + hi`` (``None`` leaves a side open; ``causal`` is ``(None, 0)``).
    ``out`` / ``lse_out`` are optional preallocated result tensors (same side as the
    inputs).  Returns ``o`` or ``(o, lse)``."""
    _require_gpu()
    band_lo, band_hi = _band_args(causal, band)
    q, k, v = _as_tensor(q), _as_tensor(k), _as_tensor(v)
    if q.is_cuda != k.is_cuda or q.is_cuda != v.is_cuda:
        raise ValueError("q, k and v must live on the same side (all CUDA or all host)")
    B, Lq, Lkv, Hq, Hkv, D, Dv = _check_call(
        q, k, v, bias=None if bias is None else _as_tensor(bias),
        kv_lengths=None if kv_lengths is None else _as_tensor(kv_lengths), what="attention_forward")
    if impl not in _IMPL:
        raise ValueError(f"implementation must be one of {sorted(x for x in _IMPL if x)} or None, got {impl!r}")
    on_device = q.is_cuda
    if k.is_cuda != on_device or v.is_cuda != on_device:
        raise ValueError("q, k and v must live on the same side (all CUDA or all host)")
    L = _lib.lib()
    if on_device:
        dev = q.device
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = _result(out, (B, Lq, Hq, Dv), q.dtype, dev)
        lse = _result(lse_out, (B, Hq, Lq), torch.float32, dev) if return_lse else None
        kvl = None if kv_lengths is None else _as_tensor(kv_lengths).to(device=dev, dtype=torch.int32).contiguous()
        bs = hs = 0
        bt = None
        if bias is not None:
            bt = _as_tensor(bias).to(device=dev, dtype=torch.float32).contiguous()
            bs = 0 if bt.shape[0] == 1 else bt.stride(0)
            hs = 0 if bt.shape[1] == 1 else bt.stride(1)
        with torch.cuda.device(dev):
            rc = L.pjx_attn_fwd_mod(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(kvl), _ptr(bt), bs, hs,
                                    B, Lq, Lkv, Hq, Hkv, D, Dv, _DTYPES[q.dtype], band_lo, band_hi,
                                    float(sm_scale), ScoreMods.arg(mods), _IMPL[impl], _ptr(_status_word(dev)),
                                    _stream(dev))
        _lib.check(rc)
        return (o, lse) if return_lse else o
    # host buffers
    if ScoreMods.arg(mods) is not None:
        raise NotImplementedError("the host-buffer entry point takes no structured masks or score modifiers")
    is_causal = band_lo == _BAND_NO_LOWER and band_hi == 0
    if not is_causal and (band_lo != _BAND_NO_LOWER or band_hi != _BAND_NO_UPPER):
        raise NotImplementedError("the host-buffer entry point takes no mask band other than the causal one")
    dev = torch.device("cuda", torch.cuda.current_device())
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    pin = q.is_pinned()
    o = _result(out, (B, Lq, Hq, Dv), q.dtype, torch.device("cpu"), pin)
    lse = _result(lse_out, (B, Hq, Lq), torch.float32, torch.device("cpu"), pin) if return_lse else None
    kvl = None if kv_lengths is None else _as_tensor(kv_lengths).to(device="cpu", dtype=torch.int32).contiguous()
    bt = None if bias is None else _as_tensor(bias).to(device="cpu", dtype=torch.float32).contiguous()
    bb, bh = (bt.shape[0], bt.shape[1]) if bt is not None else (0, 0)
    need = L.pjx_attn_fwd_host_staging_bytes(bb, bh, int(return_lse), B, Lq, Lkv, Hq, Hkv, D, Dv, _DTYPES[q.dtype])
    staging = _scratch_bytes(dev, "staging", need)
    with torch.cuda.device(dev):
        rc = L.pjx_attn_fwd_host(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(kvl), _ptr(bt), bb, bh,
                                 B, Lq, Lkv, Hq, Hkv, D, Dv, _DTYPES[q.dtype], int(is_causal), float(sm_scale),
                                 _IMPL[impl], _ptr(staging), staging.numel(), _stream(dev))
    _lib.check(rc)
    return (o, lse) if return_lse else o


def attention_backward(q, k, v, o, lse, d_o, *, causal=False, band=None, kv_lengths=None, bias=None,
                       sm_scale=1.0, impl=None, bias_grad=False, mods: ScoreMods | None = None):
    """One ``pjx_attn_bwd_mod`` call on CUDA tensors: ``(dq, dk, dv)`` for the forward
    that produced ``o`` and ``lse`` from the same arguments; with ``bias_grad`` also the
    gradient of the dense bias (float32, the bias' shape)."""
    _require_gpu()
    band_lo, band_hi = _band_args(causal, band)
    dev = q.device
    B, Lq, Lkv, Hq, Hkv, D, Dv = _check_call(
        q, k, v, bias=None if bias is None else _as_tensor(bias),
        kv_lengths=None if kv_lengths is None else _as_tensor(kv_lengths), o=o, lse=lse, d_o=d_o,
        what="attention_backward")
    if o.dtype != q.dtype or d_o.dtype != q.dtype or o.device != dev or d_o.device != dev or lse.device != dev:
        raise ValueError("attention_backward: o and d_o must have q's dtype, and o, d_o, lse its device")
    q, k, v, o, d_o = (x.contiguous() for x in (q, k, v, o, d_o))
    lse = lse.contiguous().float()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    kvl = None if kv_lengths is None else _as_tensor(kv_lengths).to(device=dev, dtype=torch.int32).contiguous()
    bs = hs = 0
    bt = None
    if bias is not None:
        bt = _as_tensor(bias).to(device=dev, dtype=torch.float32).contiguous()
        bs = 0 if bt.shape[0] == 1 else bt.stride(0)
        hs = 0 if bt.shape[1] == 1 else bt.stride(1)
    dbias = None
    if bias_grad:
        if bt is None:
            raise ValueError("bias_grad needs a bias")
        dbias = torch.empty_like(bt)
    L = _lib.lib()
    ws = _scratch_bytes(dev, "bwd", L.pjx_attn_bwd_workspace_bytes(B, Lq, Hq))
    with torch.cuda.device(dev):
        rc = L.pjx_attn_bwd_mod(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(d_o), _ptr(dq), _ptr(dk),
                                _ptr(dv), _ptr(kvl), _ptr(bt), bs, hs, _ptr(dbias), B, Lq, Lkv, Hq, Hkv, D, Dv,
                                _DTYPES[q.dtype], band_lo, band_hi, float(sm_scale), ScoreMods.arg(mods), _IMPL[impl],
                                _ptr(ws), ws.numel(), _ptr(_status_word(dev)), _stream(dev))
    _lib.check(rc)
    return (dq, dk, dv, dbias) if bias_grad else (dq, dk, dv)


def attention_jvp(q, k, v, lse, tq=None, tk=None, tv=None, *, causal=False, band=None, kv_lengths=None, bias=None,
                  sm_scale=1.0, mods: ScoreMods | None = None):
    """One ``pjx_attn_jvp_mod`` call on CUDA tensors: the tangent of ``o`` for tangents
    ``tq, tk, tv`` (``None`` = zero) of the forward that produced ``lse``."""
    _require_gpu()
    band_lo, band_hi = _band_args(causal, band)
    dev = q.device
    B, Lq, Lkv, Hq, Hkv, D, Dv = _check_call(
        q, k, v, bias=None if bias is None else _as_tensor(bias),
        kv_lengths=None if kv_lengths is None else _as_tensor(kv_lengths), lse=lse, what="attention_jvp")
    for name, t, like in (("tq", tq, q), ("tk", tk, k), ("tv", tv, v)):
        if t is not None and (tuple(t.shape) != tuple(like.shape) or t.device != dev):
            raise ValueError(f"attention_jvp: {name} must match its primal's shape {tuple(like.shape)} and device")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    tq, tk, tv = (None if t is None else t.to(q.dtype).contiguous() for t in (tq, tk, tv))
    lse = lse.contiguous().float()
    t_o = torch.empty((B, Lq, Hq, Dv), dtype=q.dtype, device=dev)
    kvl = None if kv_lengths is None else _as_tensor(kv_lengths).to(device=dev, dtype=torch.int32).contiguous()
    bs = hs = 0
    bt = None
    if bias is not None:
        bt = _as_tensor(bias).to(device=dev, dtype=torch.float32).contiguous()
        bs = 0 if bt.shape[0] == 1 else bt.stride(0)
        hs = 0 if bt.shape[1] == 1 else bt.stride(1)
    with torch.cuda.device(dev):
        rc = _lib.lib().pjx_attn_jvp_mod(_ptr(q), _ptr(k), _ptr(v), _ptr(tq), _ptr(tk), _ptr(tv), _ptr(lse), _ptr(t_o),
                                         _ptr(kvl), _ptr(bt), bs, hs, B, Lq, Lkv, Hq, Hkv, D, Dv, _DTYPES[q.dtype],
                                         band_lo, band_hi, float(sm_scale), ScoreMods.arg(mods), _stream(dev))
    _lib.check(rc)
    return t_o


class _AttentionFunction(torch.autograd.Function):
    """Differentiable forward: the regular forward kernels with the LSE kept as the
    residual, and ``pjx_attn_bwd`` for the gradients of q, k and v (the reference wires
    its kernels the same way, kernels/attention.py:3156-3270)."""

    @staticmethod
    def forward(ctx, q, k, v, band, kv_lengths, bias, sm_scale, impl, mods=None):
        o, lse = attention_forward(q, k, v, band=band, kv_lengths=kv_lengths, bias=bias, sm_scale=sm_scale,
                                   return_lse=True, impl=impl, mods=mods)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.save_for_forward(q, k, v, lse)
        ctx.args = (band, kv_lengths, bias, sm_scale, impl, mods)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def jvp(ctx, tq, tk, tv, *_):
        # forward-mode: the reference's diff_mode="forward" path (kernels/attention.py:3303-3330)
        q, k, v, lse = ctx.saved_tensors
        band, kv_lengths, bias, sm_scale, _impl, mods = ctx.args
        t_o = attention_jvp(q, k, v, lse, tq, tk, tv, band=band, kv_lengths=kv_lengths, bias=bias, sm_scale=sm_scale,
                            mods=mods)
        return t_o, None

    @staticmethod
    def backward(ctx, d_o, _d_lse):
        q, k, v, o, lse = ctx.saved_tensors
        band, kv_lengths, bias, sm_scale, impl, mods = ctx.args
        want_dbias = bias is not None and ctx.needs_input_grad[5]
        # a forced tensor-core forward does not force the tensor-core backward, which takes fewer shapes
        grads = attention_backward(q, k, v, o, lse, d_o, band=band, kv_lengths=kv_lengths, bias=bias, sm_scale=sm_scale,
                                   impl=impl if impl == "b200:generic" else None, bias_grad=want_dbias, mods=mods)
        dbias = grads[3].to(bias.dtype) if want_dbias else None
        return grads[0], grads[1], grads[2], None, None, dbias, None, None, None


def _wants_grad(*tensors) -> bool:
    """Reverse-mode (requires_grad) or forward-mode (a dual tensor) differentiation is active."""
    import torch.autograd.forward_ad as fwd_ad

    for t in tensors:
        if not isinstance(t, torch.Tensor):
            continue
        if torch.is_grad_enabled() and t.requires_grad:
            return True
        if fwd_ad.unpack_dual(t).tangent is not None:
            return True
    return False


def decode_forward(q, k_cache, v_cache, *, kv_lengths=None, sm_scale, split_len=0, return_lse=False,
                   partial_f32=False):
    """One ``pjx_attn_decode_splitkv`` call on CUDA tensors (split-KV kernel +
    combine).  ``partial_f32`` returns ``o`` in float32 (a rank's partial of a
    sequence-sharded decode)."""
    _require_gpu()
    if not q.is_cuda:
        raise ValueError("decode_forward takes CUDA tensors")
    dev = q.device
    B, Lq, cap, Hq, Hkv, D, Dv = _check_call(
        q, k_cache, v_cache, kv_lengths=None if kv_lengths is None else _as_tensor(kv_lengths), what="decode_forward")
    q, k_cache, v_cache = q.contiguous(), k_cache.contiguous(), v_cache.contiguous()
    L = _lib.lib()
    o = torch.empty((B, Lq, Hq, Dv), dtype=torch.float32 if partial_f32 else q.dtype, device=dev)
    lse = torch.empty((B, Hq, Lq), dtype=torch.float32, device=dev) if return_lse else None
    kvl = None if kv_lengths is None else _as_tensor(kv_lengths).to(device=dev, dtype=torch.int32).contiguous()
    need = L.pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, cap, int(split_len))
    ws = _scratch_bytes(dev, "decode", need)
    with torch.cuda.device(dev):
        rc = L.pjx_attn_decode_splitkv(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(kvl), _ptr(o), _ptr(lse),
                                       B, Lq, Hq, Hkv, D, Dv, cap, _DTYPES[q.dtype], float(sm_scale),
                                       int(split_len), int(partial_f32), _ptr(ws), ws.numel(), _stream(dev))
    _lib.check(rc)
    return (o, lse) if return_lse else o


def mla_decode(q, cache, *, kv_lengths=None, sm_scale=None, split_len=0, return_lse=False, impl=None):
    """One ``pjx_mla_decode_absorbed_impl`` call on CUDA tensors: the decode step of absorbed latent
    attention, ``q [B, Lq, H, R]`` over ``cache [B, S, R]`` with ``K = V = cache`` (``Lq <= 16``,
    latent width 128 / 256 / 512 / 576, bf16 or fp16).  ``impl``: ``None`` (the tcgen05 kernel),
    ``"b200:generic"`` (the mma.sync kernel) or ``"b200:tcgen05"``."""
    if impl not in _IMPL:
        raise ValueError(f"impl must be None or one of {sorted(k for k in _IMPL if k)}")
    _require_gpu()
    if not q.is_cuda or q.dim() != 4 or cache.dim() != 3:
        raise ValueError("mla_decode takes CUDA tensors q [B, Lq, H, R] and cache [B, S, R]")
    if cache.dtype != q.dtype or cache.device != q.device or cache.shape[0] != q.shape[0] or cache.shape[2] != q.shape[3]:
        raise ValueError(f"mla_decode: cache {tuple(cache.shape)} {cache.dtype} does not match q {tuple(q.shape)} {q.dtype}")
    if q.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {q.dtype}; expected float32, bfloat16 or float16")
    dev = q.device
    q, cache = q.contiguous(), cache.contiguous()
    B, Lq, H, R = q.shape
    S = cache.shape[1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(R)
    kvl = None if kv_lengths is None else _as_tensor(kv_lengths).to(device=dev, dtype=torch.int32).contiguous()
    if kvl is not None and kvl.numel() != B:
        raise ValueError(f"mla_decode: kv_lengths must hold B={B} entries, got {kvl.numel()}")
    L = _lib.lib()
    o = torch.empty((B, Lq, H, R), dtype=q.dtype, device=dev)
    lse = torch.empty((B, H, Lq), dtype=torch.float32, device=dev) if return_lse else None
    ws = _scratch_bytes(dev, "mla_decode", L.pjx_mla_decode_workspace_bytes(B, Lq, H, R, S, int(split_len)))
    with torch.cuda.device(dev):
        rc = L.pjx_mla_decode_absorbed_impl(_ptr(q), _ptr(cache), _ptr(kvl), _ptr(o), _ptr(lse), B, Lq, H, R, S,
                                            _DTYPES[q.dtype], float(sm_scale), int(split_len), _IMPL[impl], _ptr(ws),
                                            ws.numel(), _ptr(_status_word(dev)), _stream(dev))
    _lib.check(rc)
    return (o, lse) if return_lse else o


def _latent_decode_applies(q, cache, wk, lm, bt, mods) -> bool:
    """Absorbed call that is a decode step the latent kernel takes: few query tokens, no mask but
    key lengths, no bias; always for latents wider than the regular kernels' head widths."""
    if wk is not None or bt is not None or mods is not None or lm.banded or lm.q_limit is not None:
        return False
    if q.dtype not in (torch.bfloat16, torch.float16) or cache.shape[2] not in (128, 256, 512, 576):
        return False
    Lq, H = q.shape[1], q.shape[2]
    if Lq > 16 or not any(H % g == 0 for g in range(1, 16 // Lq + 1)):
        return False
    return cache.shape[2] > 256 or cache.shape[1] >= _SPLITKV_MIN_KV_LEN


def combine_partials(o_parts, lse_parts, *, out_dtype=None):
    """``pjx_attn_combine``: ``o_parts [P, N, Dv]`` fp32, ``lse_parts [P, N]`` natural
    log (``+inf`` = no keys) -> ``(o [N, Dv], lse [N])``."""
    _require_gpu()
    o_parts, lse_parts = o_parts.contiguous().float(), lse_parts.contiguous().float()
    P, N, Dv = o_parts.shape
    out_dtype = out_dtype or torch.float32
    o = torch.empty((N, Dv), dtype=out_dtype, device=o_parts.device)
    lse = torch.empty((N,), dtype=torch.float32, device=o_parts.device)
    with torch.cuda.device(o_parts.device):
        rc = _lib.lib().pjx_attn_combine(_ptr(o_parts), _ptr(lse_parts), P, N, Dv, _ptr(o), _ptr(lse),
                                         _DTYPES[out_dtype], _stream(o_parts.device))
    _lib.check(rc)
    return o, lse


# ---------------------------------------------------------------------------
# Reference call signatures
# ---------------------------------------------------------------------------


def _validate_qkv(query, key, value, enable_gqa):
    # layers/attention.py:1490-1516
    if (query.dtype != key.dtype) or (query.dtype != value.dtype):
        raise ValueError(
            "Expected query, key, and value to have the same dtype, "
            f"but got query.dtype: {query.dtype}, key.dtype: {key.dtype}, "
            f"and value.dtype: {value.dtype} instead."
        )
    if (query.dim() < 3) or (key.dim() < 3) or (value.dim() < 3):
        raise ValueError(
            "Expected query, key, and value to all be at least 3 dimensional, but got query.ndim: "
            f"{query.dim()}, key.ndim: {key.dim()}, and value.ndim: {value.dim()} instead."
        )
    if (not enable_gqa) and query.shape[-2] != key.shape[-2]:
        raise ValueError(
            "Expect query and key/value to have the same number of heads "
            f"but got Hq={query.shape[-2]} and Hkv={key.shape[-2]}. "
            "Try setting enable_gqa=True for GQA."
        )
    if enable_gqa and query.shape[-2] % key.shape[-2] != 0:
        raise ValueError(
            "Expect number of query heads to be a multiple of kv heads for GQA "
            f"but got Hq={query.shape[-2]} and Hkv={key.shape[-2]}."
        )


def use_splitkv(q, k, *, causal=False, bias=None, q_limit=None, dropout_rate=0.0, split_kv=None) -> bool:
    """Whether the split-KV decode kernel runs (kernels/attention.py:2653-2689).
    Unlike the reference's kernel this one takes per-batch key lengths, so a
    ``KVLenMask`` does not disable it."""
    if split_kv is False or causal or bias is not None or q_limit is not None or dropout_rate > 0:
        return False
    if q.dim() != 4 or not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    hq, hkv = q.shape[2], k.shape[2]
    if q.shape[-1] != k.shape[-1] or q.shape[-1] not in (64, 128) or (hq // hkv) * q.shape[1] > 16:
        return False
    if split_kv:
        return True
    return q.shape[1] <= _SPLITKV_MAX_Q_LEN and k.shape[1] >= _SPLITKV_MIN_KV_LEN


def _apply_q_limit(out, lse, q_limit):
    if q_limit is not None:
        out[:, q_limit:] = 0
        if lse is not None:
            lse[:, :, q_limit:] = float("inf")
    return out, lse


def rng_seed_from_key(rng) -> int:
    """The 32-bit dropout seed from ``rng``: an int, or the words of a PRNG key (a sequence, array or
    tensor of integers) folded as the reference folds them (kernels/attention.py:151-159)."""
    if isinstance(rng, torch.Tensor):
        rng = rng.reshape(-1).tolist()
    elif isinstance(rng, np.ndarray):
        rng = rng.reshape(-1).tolist()
    words = [int(w) & 0xFFFFFFFF for w in (rng if isinstance(rng, (list, tuple)) else [rng])]
    if not words:
        raise ValueError("empty PRNG key")
    seed = words[0]
    if len(words) > 1:
        seed ^= (words[1] * 0x9E3779B9) & 0xFFFFFFFF
        for i in range(2, len(words)):
            seed ^= (words[i] * ((0x85EBCA6B + i) & 0xFFFFFFFF)) & 0xFFFFFFFF
    return seed & 0xFFFFFFFF


def _dropout_args(rng, dropout_rate, dropout_impl):
    """(rate, seed) of an attention call, with the reference's checks (attention_xla.py:637-641)."""
    if not dropout_rate > 0:
        return 0.0, 0
    if not dropout_rate < 1:
        raise ValueError(f"dropout_rate must be in [0, 1), got {dropout_rate}")
    if rng is None:
        raise ValueError("prng_key must be provided when dropout_rate>0")
    if dropout_impl != "counter":
        raise NotImplementedError(f"dropout_impl={dropout_impl!r}: only the counter-hash dropout runs in the kernels")
    return float(dropout_rate), rng_seed_from_key(rng)


def masks_DenseBias(t):
    from .masks import DenseBias

    return DenseBias(t)


def _fold_low_rank(q, k, v, terms, sm_scale: float):
    """``LowRankBias`` terms as extra feature columns of q and k: ``sm_scale (q' . k') = sm_scale q.k +
    scale qf.kf`` with both factors multiplied by ``sqrt(scale / sm_scale)`` and cast to the input dtype,
    as the reference folds them (layers/attention.py:1602-1639).  The factors are per query head, so
    K / V heads are repeated to the query head count first."""
    if sm_scale <= 0:
        raise ValueError("LowRankBias requires a positive sm_scale")
    B, Lq, Hq, _ = q.shape
    Lkv, Hkv = k.shape[1], k.shape[2]
    if Hkv != Hq:
        k, v = k.repeat_interleave(Hq // Hkv, dim=2), v.repeat_interleave(Hq // Hkv, dim=2)
    q_extra, k_extra = [], []
    for t in terms:  # LowRankBias, BatchedLowRankBias, LearnedAlibiBias: factors [B|1, length, H|1, rank]
        qf, kf = t.factors(Lq, Lkv, Hq)
        f = math.sqrt(t.scale / sm_scale)
        qf = (qf.to(q.device).float() * f).to(q.dtype)
        kf = (kf.to(q.device).float() * f).to(q.dtype)
        q_extra.append(qf.expand(B, Lq, Hq, qf.shape[-1]))
        k_extra.append(kf.expand(B, Lkv, Hq, kf.shape[-1]))
    return torch.cat([q, *q_extra], dim=-1), torch.cat([k, *k_extra], dim=-1), v


def mha(q, k, v, mask: AttentionMask | None = None, bias: AttentionBias | None = None, rng=None,
        sm_scale: float = 1.0, block_sizes=None, backward_pass_impl: str = "auto", num_warps=None,
        num_stages: int = 2, grid=None, interpret: bool = False, debug: bool = False,
        dropout_rate: float = 0.0, dropout_impl: str = "counter", diff_mode: str = "reverse",
        split_kv: bool | None = None, *, return_lse: bool = False, implementation: str | None = None):
    """``mha`` (kernels/attention.py:2692-2711): rank-4 ``[B, T, H, D]`` inputs,
    default ``sm_scale=1.0``.  Tile-size / warp / stage arguments are accepted for
    signature compatibility and ignored (the kernels pick their own tiling)."""
    if diff_mode not in ("reverse", "forward"):
        raise ValueError(f"diff_mode must be 'reverse' or 'forward', got {diff_mode!r}.")
    q, k, v = _as_tensor(q), _as_tensor(k), _as_tensor(v)
    _gqa_group(q.shape[-2], k.shape[-2])
    if v.shape[-2] != k.shape[-2]:
        raise ValueError(f"key and value need the same number of heads, got {k.shape[-2]} and {v.shape[-2]}.")
    drop_rate, drop_seed = _dropout_args(rng, dropout_rate, dropout_impl)
    if interpret:
        raise NotImplementedError("interpret mode belongs to the Pallas kernels; this library runs CUDA only")
    B, Lq = q.shape[0], q.shape[1]
    # What the kernels take natively: a band, key lengths, a query limit, and -- evaluated per element
    # from O(B T) / O(H T) data -- segment ids, per-row key limits, a prefix, relative-position tables,
    # ALiBi slopes, a per-head scale and a soft cap.  Only what is left (or / xor / not compositions)
    # is densified into the additive bias.
    lm, residual = split_mask(mask, B, Lq, k.shape[1])
    lb = lower_bias_structured(bias, B, q.shape[2], Lq, k.shape[1])
    if lb.low_rank:
        q, k, v = _fold_low_rank(q, k, v, lb.low_rank, float(sm_scale))
    bt = lb.dense
    if residual is not None:  # mask classes without a native form: their dense -inf tensor rides on the bias
        bt = lower_dense(residual, None if bt is None else masks_DenseBias(bt), B, q.shape[2], Lq, k.shape[1])
    wants_mods = lm.structured or lb.structured or drop_rate > 0
    mods = ScoreMods(lm, lb, q.device, drop_rate, drop_seed) if wants_mods and q.is_cuda else None
    if wants_mods and not q.is_cuda:
        raise NotImplementedError("structured masks, score modifiers and dropout take CUDA tensors")
    if _wants_grad(q, k, v, bt):
        # differentiation always runs the regular kernels (attention_splitkv.py:253-272)
        if not q.is_cuda:
            raise NotImplementedError("differentiable attention takes CUDA tensors")
        if lm.q_limit is not None:
            raise NotImplementedError("gradients under a query-length mask are not implemented")
        out, lse = _AttentionFunction.apply(q, k, v, lm.band, lm.kv_lengths, bt, float(sm_scale), implementation, mods)
        res = (out, lse) if return_lse else out
    elif mods is None and use_splitkv(q, k, causal=lm.banded, bias=bt, q_limit=lm.q_limit, dropout_rate=dropout_rate,
                                      split_kv=split_kv):
        res = decode_forward(q, k, v, kv_lengths=lm.kv_lengths, sm_scale=sm_scale, return_lse=return_lse)
    else:
        res = attention_forward(q, k, v, band=lm.band, kv_lengths=lm.kv_lengths, bias=bt, sm_scale=sm_scale,
                                return_lse=return_lse, impl=implementation, mods=mods)
    out, lse = res if return_lse else (res, None)
    out, lse = _apply_q_limit(out, lse, lm.q_limit)
    return (out, lse) if return_lse else out


def flex_attention(query, key, value, mask: AttentionMask | None = None, bias: AttentionBias | None = None,
                   dropout_rng=None, dropout_rate: float = 0.0, broadcast_dropout: bool = False,
                   deterministic=True, dtype=None, precision=None, module=None,
                   sm_scale: Optional[float] = None, enable_gqa: bool = False, block_q: int = 128,
                   block_k: int = 128, block_q_dkv: int = 64, block_kv_dkv: int = 64, block_q_dq: int = 64,
                   block_kv_dq: int = 64, backward_pass_impl: str = "auto", num_warps=None, num_stages: int = 2,
                   grid=None, interpret: bool = False, debug: bool = False, dropout_impl: str = "counter",
                   diff_mode: str = "reverse", split_kv: bool | None = None, implementation: str | None = None,
                   *, return_lse: bool = False):
    """``flex_attention`` (layers/attention.py:1426-1457): ``[..., T, H, D]`` inputs,
    default ``sm_scale = 1/sqrt(D)``; ``implementation`` is ``None`` or ``"b200"``."""
    query, key, value = _as_tensor(query), _as_tensor(key), _as_tensor(value)
    if dtype is not None:
        query, key, value = query.to(dtype), key.to(dtype), value.to(dtype)
    _validate_qkv(query, key, value, enable_gqa)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(query.shape[-1])
    if implementation not in _IMPL:
        raise ValueError(
            f"implementation must be None or one of {sorted(x for x in _IMPL if x)}, got {implementation!r}"
        )
    active_dropout = dropout_rate if not deterministic and dropout_rate > 0 else 0.0
    squeeze = query.dim() == 3
    if squeeze:
        query, key, value = query[None], key[None], value[None]
    batch_shape = query.shape[:-3]
    if key.shape[:-3] != batch_shape or value.shape[:-3] != batch_shape:
        raise ValueError(f"batch dimensions differ: {tuple(query.shape)}, {tuple(key.shape)}, {tuple(value.shape)}")
    q4, k4, v4 = (x.reshape((-1,) + tuple(x.shape[-3:])) for x in (query, key, value))
    res = mha(q4, k4, v4, mask=mask, bias=bias, rng=dropout_rng, sm_scale=sm_scale, dropout_rate=active_dropout,
              dropout_impl=dropout_impl, interpret=interpret, diff_mode=diff_mode, split_kv=split_kv,
              return_lse=return_lse, implementation=implementation)
    out, lse = res if return_lse else (res, None)
    out = out.reshape(tuple(batch_shape) + tuple(out.shape[-3:]))
    if squeeze:
        out = out[0]
    if return_lse:
        lse = lse.reshape(tuple(batch_shape) + tuple(lse.shape[-2:]))
        return out, (lse[0] if squeeze else lse)
    return out


def _dense_arrays_as_bias(mask, bias, batch_shape, heads, q_len, kv_len):
    """Dense ``mask`` (boolean, True = keep) / ``bias`` arrays broadcastable to
    ``[*batch, H, Q, K]`` (the Flax convention, layers/attention.py:1293-1319) as one
    ``DenseBias`` ``[B|1, H|1, Q, K]`` with ``-inf`` where masked."""
    from .masks import DenseBias

    nb = len(batch_shape)
    total = None
    for arr, is_mask in ((mask, True), (bias, False)):
        if arr is None:
            continue
        t = _as_tensor(arr)
        if t.dim() > nb + 3:
            raise ValueError(f"mask / bias rank {t.dim()} exceeds [*batch, H, Q, K] (rank {nb + 3})")
        t = t.reshape((1,) * (nb + 3 - t.dim()) + tuple(t.shape))
        lead = tuple(t.shape[:nb])
        if any(d != 1 for d in lead):
            t = t.expand(tuple(batch_shape) + tuple(t.shape[nb:]))
        t = t.reshape((-1,) + tuple(t.shape[nb:]))  # [B|1, H|1, Q|1, K|1]
        if t.shape[1] not in (1, heads):
            raise ValueError(f"cannot broadcast mask / bias head dim {t.shape[1]} to {heads}")
        t = t.expand(t.shape[0], t.shape[1], q_len, kv_len)
        if is_mask:
            t = torch.zeros(t.shape, dtype=torch.float32, device=t.device).masked_fill_(~t.bool(), float("-inf"))
        else:
            t = t.float()
        total = t if total is None else total + t.to(total.device)
    return None if total is None else DenseBias(total.contiguous())


def dot_product_attention(query, key, value, mask=None, bias=None, dropout_rng=None, dropout_rate: float = 0.0,
                          broadcast_dropout: bool = False, deterministic=True, dtype=None, precision=None,
                          module=None, sm_scale: Optional[float] = None, enable_gqa: bool = False,
                          implementation: str | None = None):
    """``dot_product_attention`` (layers/attention.py:1205-1221): the default
    ``attention_fn`` of ``MultiHeadAttention``.  Like Flax, K/V may carry fewer
    heads than Q.  ``mask`` / ``bias`` are mask / bias objects of
    :mod:`probjax_b200.masks` or, as on the reference's Flax path (1293-1319), dense arrays
    broadcastable to ``[*batch, H, Q, K]`` (boolean keep-mask, additive bias); arrays become one
    dense additive tensor for the kernels.  Rows whose keys are all masked come out as zeros
    (the kernel convention), where the Flax einsum would average the values."""
    if module is not None or precision is not None:
        raise NotImplementedError("sowing (module=) and explicit precision belong to the Flax einsum path")
    arrays = (mask is not None and not isinstance(mask, AttentionMask)) or \
             (bias is not None and not isinstance(bias, AttentionBias))
    if arrays:
        query, key = _as_tensor(query), _as_tensor(key)
        if query.dim() < 3:
            raise ValueError("dense mask / bias arrays need query of rank >= 3 [..., T, H, D]")
        arr_mask = None if isinstance(mask, AttentionMask) else mask
        arr_bias = None if isinstance(bias, AttentionBias) else bias
        dense = _dense_arrays_as_bias(arr_mask, arr_bias, tuple(query.shape[:-3]), query.shape[-2], query.shape[-3],
                                      key.shape[-3])
        if isinstance(bias, AttentionBias):
            from .masks import SumBias

            dense = SumBias(bias, dense)
        mask = mask if isinstance(mask, AttentionMask) else None
        bias = dense
    return flex_attention(query, key, value, mask=mask, bias=bias, dropout_rng=dropout_rng,
                          dropout_rate=dropout_rate, deterministic=deterministic, dtype=dtype,
                          sm_scale=sm_scale, enable_gqa=True, implementation=implementation)


def mha_flash(query, key, value, mask=None, bias=None, dropout_rng=None, dropout_rate: float = 0.0,
              broadcast_dropout: bool = True, deterministic: bool = True, dtype=None, precision=None, module=None,
              sm_scale: Optional[float] = None, enable_gqa: bool = False, block_q=None, block_k=None, block_kv=None,
              max_concurrent_steps: int = 2, use_schedule_barrier: bool = True, causal: bool = False,
              compute_wgs_bwd=None, block_q_dkv=None, block_kv_dkv=None, block_q_dq=None, block_kv_dq=None,
              save_residuals: bool = False, use_pipeline_emitter: bool = False):
    """``mha_flash`` (probjax/nn/pallas_kernels/kernels/flash_attention3.py:344-372), the
    reference's warp-specialised Hopper kernel, with the same restrictions so call
    sites behave alike: ``mask`` is ``None`` / ``NoMask`` / ``KVLenMask``, causal
    attention is asked for with ``causal=True``, no bias, no dropout.  With
    ``save_residuals`` it also returns the natural-log LSE ``[B, Hq, Lq]`` (the
    reference returns its base-2 residual; multiply by ``log2(e)`` to compare)."""
    from .masks import CausalMask, KVLenMask

    if mask is not None and type(mask) is not NoMask and type(mask) is not KVLenMask:
        raise NotImplementedError(
            "mha_flash supports mask=None, NoMask or KVLenMask (use causal=True for "
            f"causal attention), got {type(mask).__name__}."
        )
    if bias is not None:
        raise NotImplementedError("mha_flash does not support additive attention bias.")
    if not deterministic and dropout_rate != 0.0:
        raise NotImplementedError("mha_flash does not support dropout.")
    full = mask
    if causal:
        full = CausalMask() if not isinstance(mask, KVLenMask) else (mask & CausalMask())
    return flex_attention(query, key, value, mask=full, dtype=dtype, sm_scale=sm_scale, enable_gqa=enable_gqa,
                          split_kv=False, return_lse=save_residuals)


def splitkv_forward(q, k, v, *, sm_scale: float, num_splits: int | None = None, block_k: int | None = None,
                    num_warps: int = 4, num_stages: int = 2, interpret: bool = False, return_lse: bool = False,
                    kv_lengths=None):
    """``splitkv_forward`` (attention_splitkv.py:137-149).  Returns
    ``[B, Lq, Hq, Dv]`` in ``q.dtype`` and, with ``return_lse``, the natural-log LSE
    ``[B, Hq, Lq]``.  ``num_splits`` fixes the number of KV splits (rounded so a
    split is a multiple of 64 keys); ``kv_lengths [B]`` (an extension) gives
    per-sequence valid lengths of the cache."""
    if interpret:
        raise NotImplementedError("interpret mode belongs to the Pallas kernels; this library runs CUDA only")
    q, k, v = _as_tensor(q), _as_tensor(k), _as_tensor(v)
    hq, hkv = q.shape[2], k.shape[2]
    if hq % hkv:
        raise ValueError(f"Hq={hq} must be a multiple of Hkv={hkv}.")
    split_len = 0
    if num_splits is not None:
        if num_splits < 1:
            raise ValueError("num_splits must be positive")
        per_split = -(-k.shape[1] // num_splits)
        split_len = max(64, -(-per_split // 64) * 64)
    return decode_forward(q, k, v, kv_lengths=kv_lengths, sm_scale=sm_scale, split_len=split_len,
                          return_lse=return_lse)


def mla(q, cache, wk=None, wv=None, *, mask=None, bias=None, rng=None, sm_scale: float | None = None,
        block_sizes=None, backward_pass_impl: str = "auto", num_warps=None, num_stages: int = 2,
        interpret: bool = False, debug: bool = False, dropout_rate: float = 0.0, dropout_impl: str = "counter",
        return_lse: bool = False, implementation: str | None = None):
    """``mla`` (latent_attention.py:636-654): ``q [B,Q,H,Dqk]`` over a shared latent
    ``cache [B,S,R]`` with per-head up-projections ``wk [H,Dqk,R]``, ``wv [H,Dv,R]``
    (materialized) or none (absorbed, ``K = V = cache``)."""
    q, cache = _as_tensor(q), _as_tensor(cache)
    wk = None if wk is None else _as_tensor(wk)
    wv = None if wv is None else _as_tensor(wv)
    # latent_attention.py:668-696
    if q.dim() != 4:
        raise ValueError(f"q must be rank 4 [B,Q,H,D], got shape {tuple(q.shape)}")
    if cache.dim() != 3:
        raise ValueError(f"cache must be rank 3 [B,S,R], got shape {tuple(cache.shape)}")
    if q.shape[0] != cache.shape[0]:
        raise ValueError(f"batch mismatch: q has {q.shape[0]}, cache has {cache.shape[0]}")
    H, Dqk, R = q.shape[-2], q.shape[-1], cache.shape[-1]
    if (wk is None) != (wv is None):
        raise ValueError(
            "provide both wk and wv (materialized) or neither (absorbed); mixing the two is not supported"
        )
    if wk is None and Dqk != R:
        raise ValueError(f"absorbed mode (wk=None) requires qk_head_dim == kv_lora_rank ({Dqk} != {R})")
    if wk is not None and tuple(wk.shape) != (H, Dqk, R):
        raise ValueError(f"wk must be {(H, Dqk, R)}, got {tuple(wk.shape)}")
    if wv is not None and (wv.shape[0] != H or wv.shape[2] != R):
        raise ValueError(f"wv must be [heads, v_head_dim, {R}], got {tuple(wv.shape)}")
    drop_rate, drop_seed = _dropout_args(rng, dropout_rate, dropout_impl)
    if interpret:
        raise NotImplementedError("interpret mode belongs to the Pallas kernels; this library runs CUDA only")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(Dqk)  # latent_attention.py:698-701
    _require_gpu()
    if not q.is_cuda:
        raise NotImplementedError("mla takes CUDA tensors")
    if implementation not in _IMPL:
        raise ValueError(f"implementation must be None or one of {sorted(x for x in _IMPL if x)}")
    dev = q.device
    B, Lq, S = q.shape[0], q.shape[1], cache.shape[1]
    Dv = R if wv is None else wv.shape[1]
    # the same masks and biases as mha (latent_attention.py:636-766 shares its mask / bias machinery)
    lm, residual = split_mask(mask, B, Lq, S)
    lb = lower_bias_structured(bias, B, H, Lq, S)
    if lb.low_rank:
        raise NotImplementedError("mla does not fold LowRankBias terms (the latent has no per-head key columns)")
    bt = lb.dense
    if residual is not None:
        bt = lower_dense(residual, None if bt is None else masks_DenseBias(bt), B, H, Lq, S)
    mods = ScoreMods(lm, lb, dev, drop_rate, drop_seed) if (lm.structured or lb.structured or drop_rate > 0) else None
    q, cache = q.contiguous(), cache.contiguous()
    wk = None if wk is None else wk.to(dev).contiguous()
    wv = None if wv is None else wv.to(dev).contiguous()
    if wk is not None and (wk.dtype != q.dtype or wv.dtype != q.dtype or cache.dtype != q.dtype):
        raise ValueError("q, cache, wk and wv must share a dtype")
    if _wants_grad(q, cache, wk, wv):
        # Differentiation goes through the materialized K and V and the regular attention kernels, as
        # in the reference (latent_attention.py:554-585); the up-projections and their gradients run
        # on the projection kernel (pjx_linear) as well.
        if lm.q_limit is not None:
            raise NotImplementedError("gradients under a query-length mask are not implemented")
        if wk is not None:
            from .cache import linear_autograd

            kmat = linear_autograd(cache, wk.reshape(H * Dqk, R)).view(B, S, H, Dqk)
            vmat = linear_autograd(cache, wv.reshape(H * Dv, R)).view(B, S, H, Dv)
        else:
            kmat = vmat = cache[:, :, None, :]  # one shared KV head
        out, lse = _AttentionFunction.apply(q, kmat, vmat, lm.band, lm.kv_lengths, bt, float(sm_scale), implementation,
                                            mods)
        return (out, lse) if return_lse else out
    if _latent_decode_applies(q, cache, wk, lm, bt, mods):
        return mla_decode(q, cache, kv_lengths=lm.kv_lengths, sm_scale=sm_scale, return_lse=return_lse)
    o = torch.empty((B, Lq, H, Dv), dtype=q.dtype, device=dev)
    lse = torch.empty((B, H, Lq), dtype=torch.float32, device=dev) if return_lse else None
    kvl = None if lm.kv_lengths is None else lm.kv_lengths.to(device=dev, dtype=torch.int32).contiguous()
    bs = hs = 0
    if bt is not None:
        bt = bt.to(device=dev, dtype=torch.float32).contiguous()
        bs = 0 if bt.shape[0] == 1 else bt.stride(0)
        hs = 0 if bt.shape[1] == 1 else bt.stride(1)
    L = _lib.lib()
    need = L.pjx_mla_workspace_bytes(B, S, H, Dqk, Dv, R, _DTYPES[q.dtype], int(wk is not None))
    ws = _scratch_bytes(dev, "mla", need)
    band_lo, band_hi = _band_args(False, lm.band)
    with torch.cuda.device(dev):
        rc = L.pjx_mla_fwd_mod(_ptr(q), _ptr(cache), _ptr(wk), _ptr(wv), _ptr(o), _ptr(lse), _ptr(kvl), _ptr(bt), bs, hs,
                               B, Lq, S, H, Dqk, Dv, R, _DTYPES[q.dtype], band_lo, band_hi, float(sm_scale),
                               ScoreMods.arg(mods), _IMPL[implementation], _ptr(ws), ws.numel(),
                               _ptr(_status_word(dev)), _stream(dev))
    _lib.check(rc)
    o, lse = _apply_q_limit(o, lse, lm.q_limit)
    return (o, lse) if return_lse else o
