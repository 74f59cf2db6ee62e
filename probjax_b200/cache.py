"""Autoregressive KV cache for decode steps.

Host-side mirror of the cache the reference's attention layer keeps
(probjax/nn/layers/attention.py: ``init_cache`` 727-757, decode branch 603-675):
``cached_key`` / ``cached_value`` ``[B, capacity, Hkv, D]`` and a write position.  The
reference shares one ``cache_index`` across the batch and masks with
``KeyPaddingMask(cur_index + 1)``; here every sequence has its own position (a ragged
batch), the update is one kernel launch (``pjx_kv_cache_append``) that also advances the
positions on the device, and attention over the filled prefix is the split-KV decode
kernel with ``kv_lengths = positions``.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from .attention import _DTYPES, _IMPL, _ptr, _require_gpu, _scratch_bytes, _status_word, _stream, mha
from .masks import CausalFromBottomRightMask, KVLenMask


class DecodeCache:
    def __init__(self, batch: int, capacity: int, num_kv_heads: int, head_dim: int, v_head_dim: int | None = None,
                 dtype=torch.bfloat16, device=None):
        _require_gpu()
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self.batch, self.capacity = int(batch), int(capacity)
        self.cached_key = torch.zeros((batch, capacity, num_kv_heads, head_dim), dtype=dtype, device=device)
        self.cached_value = torch.zeros((batch, capacity, num_kv_heads, v_head_dim), dtype=dtype, device=device)
        # [0, B): positions; [B, 2B): scratch counters of the append kernel (zero between launches)
        self._positions = torch.zeros((2 * batch,), dtype=torch.int32, device=device)
        self._overflow = torch.zeros((1,), dtype=torch.int32, device=device)

    @property
    def cache_index(self) -> torch.Tensor:
        """``int32 [B]``: number of valid tokens per sequence (a view, updated on the device)."""
        return self._positions[: self.batch]

    def reset(self, lengths=None):
        self._positions.zero_()
        self._overflow.zero_()
        if lengths is not None:
            self._positions[: self.batch] = torch.as_tensor(lengths, dtype=torch.int32, device=self._positions.device)

    def overflowed(self) -> bool:
        """Whether an update ran past the capacity (synchronises)."""
        return bool(self._overflow.item())

    def update(self, key: torch.Tensor, value: torch.Tensor, advance: bool = True):
        """Append ``key [B, n, Hkv, D]`` / ``value [B, n, Hkv, Dv]`` at each sequence's position."""
        ck, cv = self.cached_key, self.cached_value
        if key.shape[0] != self.batch or key.shape[2:] != ck.shape[2:] or value.shape[2:] != cv.shape[2:] \
                or value.shape[:2] != key.shape[:2]:
            raise ValueError(
                f"Autoregressive cache shape error, expected key [B={self.batch}, n, {ck.shape[2]}, {ck.shape[3]}] and "
                f"value [B, n, {cv.shape[2]}, {cv.shape[3]}], got {tuple(key.shape)} and {tuple(value.shape)}."
            )
        if key.dtype != ck.dtype or value.dtype != cv.dtype:
            raise ValueError("key / value dtype differs from the cache dtype")
        key, value = key.contiguous(), value.contiguous()
        dev = ck.device
        with torch.cuda.device(dev):
            rc = _lib.lib().pjx_kv_cache_append(_ptr(ck), _ptr(cv), _ptr(key), _ptr(value), _ptr(self._positions),
                                                self.batch, self.capacity, key.shape[1], ck.shape[2], ck.shape[3],
                                                cv.shape[3], _DTYPES[ck.dtype], int(advance), _ptr(self._overflow),
                                                _stream(dev))
        _lib.check(rc)

    def attend(self, query: torch.Tensor, *, sm_scale: float | None = None, return_lse: bool = False,
               prefix_length: int | None = None):
        """Attention of ``query [B, n, Hq, D]`` over the filled prefix.  One query token per
        sequence is a decode step (split-KV kernel, ragged positions).  Several query tokens
        (a prefill chunk just appended) need ``prefix_length``: the common number of valid
        tokens after the append, for the bottom-right causal mask."""
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(query.shape[-1])
        mask = KVLenMask(self.cache_index)
        if query.shape[1] > 1:
            if prefix_length is None:
                raise ValueError("attend with several query tokens needs prefix_length (tokens valid after the append)")
            mask = mask & CausalFromBottomRightMask(query.shape[1], int(prefix_length))
        return mha(query, self.cached_key, self.cached_value, mask=mask, sm_scale=sm_scale, return_lse=return_lse)

    def step(self, query, key, value, *, sm_scale: float | None = None):
        """One decode step: append the token's key / value, then attend over the prefix."""
        self.update(key, value)
        return self.attend(query, sm_scale=sm_scale)


def rope_interleaved(x: torch.Tensor, positions=None, *, base: float = 10_000.0, rotary_dim: int | None = None,
                     offset: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Interleaved rotary embedding of ``x [..., T, H, D]`` on the device (``pjx_rope_interleaved``):
    the reference's rotary layer (layers/encoding.py:171-211) with its ``rotary_dim`` / ``offset``
    options; ``positions`` is ``[T]`` or ``None`` (= ``arange(T) + offset``)."""
    _require_gpu()
    if not x.is_cuda or x.dim() < 3:
        raise ValueError("rope_interleaved takes a CUDA tensor [..., T, H, D]")
    x = x.contiguous()
    T, H, D = x.shape[-3:]
    outer = x.numel() // max(T * H * D, 1)
    rotary_dim = D if rotary_dim is None else int(rotary_dim)
    y = torch.empty_like(x) if out is None else out
    pos = None if positions is None else torch.as_tensor(positions).to(device=x.device, dtype=torch.float32).contiguous()
    if pos is not None and pos.numel() != T:
        raise ValueError(f"positions must have {T} entries, got {pos.numel()}")
    with torch.cuda.device(x.device):
        rc = _lib.lib().pjx_rope_interleaved(_ptr(x), _ptr(y), _ptr(pos), float(offset), outer, T, H, D, rotary_dim,
                                             float(base), _DTYPES[x.dtype], _stream(x.device))
    _lib.check(rc)
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, *, implementation: str | None = None) -> torch.Tensor:
    """``x [..., K] @ weight[N, K]^T`` on the device (``pjx_linear``): the bias-free query / key /
    value / output projections around the attention call (layers/attention.py:591-594).  A fused
    QKV projection is one call with the three weights concatenated along ``N``."""
    _require_gpu()
    if not x.is_cuda or x.dtype != weight.dtype or x.shape[-1] != weight.shape[-1] or weight.dim() != 2:
        raise ValueError("linear takes CUDA tensors x [..., K] and weight [N, K] of one dtype")
    if implementation not in _IMPL:
        raise ValueError(f"implementation must be None or one of {sorted(k for k in _IMPL if k)}")
    x2 = x.contiguous().view(-1, x.shape[-1])
    w = weight.to(x.device).contiguous()
    y = torch.empty((x2.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().pjx_linear(_ptr(x2), _ptr(w), _ptr(y), x2.shape[0], w.shape[0], w.shape[1], _DTYPES[x.dtype],
                                   _IMPL[implementation], _ptr(_status_word(x.device)), _stream(x.device))
    _lib.check(rc)
    return y.view(*x.shape[:-1], w.shape[0])


class _LinearFunction(torch.autograd.Function):
    """``linear`` with its gradients computed by the same kernel: ``dx = dy . w`` and ``dw = dy^T . x`` are
    again products of the ``A . B^T`` form once the second operand is transposed (a copy)."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return linear(x, weight)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dx = dw = None
        dy2 = dy.reshape(-1, dy.shape[-1]).to(x.dtype)
        if ctx.needs_input_grad[0]:
            dx = linear(dy2, weight.t().contiguous()).reshape(x.shape)          # [M, N] . [K, N]^T
        if ctx.needs_input_grad[1]:
            x2 = x.reshape(-1, x.shape[-1])
            dw = linear(dy2.t().contiguous(), x2.t().contiguous())              # [N, M] . [K, M]^T
        return dx, dw


def linear_autograd(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """:func:`linear` that records itself for reverse-mode differentiation (both gradients on ``pjx_linear``)."""
    return _LinearFunction.apply(x, weight)


def decode_paged(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, kv_lengths,
                 *, sm_scale: float | None = None, split_len: int = 0, return_lse: bool = False):
    """Split-KV decode over a paged cache (``pjx_attn_decode_paged``): ``k_pool`` / ``v_pool``
    ``[num_pages, page_size, Hkv, D]``, ``block_table int32 [B, max_pages]`` (page of every logical
    block of a sequence), ``kv_lengths [B]``.  ``page_size`` must be a multiple of 64."""
    _require_gpu()
    if not q.is_cuda:
        raise ValueError("decode_paged takes CUDA tensors")
    dev = q.device
    if q.dim() != 4 or k_pool.dim() != 4 or v_pool.dim() != 4:
        raise ValueError("decode_paged: q must be [B, Lq, Hq, D] and the pools [num_pages, page_size, Hkv, D]")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or k_pool.device != dev or v_pool.device != dev:
        raise ValueError("decode_paged: q and the page pools must share a dtype and a device")
    q, k_pool, v_pool = q.contiguous(), k_pool.contiguous(), v_pool.contiguous()
    B, Lq, Hq, D = q.shape
    page_size, Hkv, Dv = k_pool.shape[1], k_pool.shape[2], v_pool.shape[3]
    if k_pool.shape[3] != D or tuple(v_pool.shape[:3]) != tuple(k_pool.shape[:3]):
        raise ValueError(f"decode_paged: pools must be [P, page, Hkv, D={D}] / [P, page, Hkv, Dv], got "
                         f"{tuple(k_pool.shape)} and {tuple(v_pool.shape)}")
    if Hq % Hkv != 0:
        raise ValueError(f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    bt = torch.as_tensor(block_table).to(device=dev, dtype=torch.int32).contiguous()
    if bt.dim() != 2 or bt.shape[0] != B:
        raise ValueError(f"block_table must be [B={B}, max_pages], got {tuple(bt.shape)}")
    max_pages = bt.shape[1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    kvl = torch.as_tensor(kv_lengths).to(device=dev, dtype=torch.int32).contiguous()
    if kvl.numel() != B:
        raise ValueError(f"decode_paged: kv_lengths must hold B={B} entries, got {kvl.numel()}")
    L = _lib.lib()
    o = torch.empty((B, Lq, Hq, Dv), dtype=q.dtype, device=dev)
    lse = torch.empty((B, Hq, Lq), dtype=torch.float32, device=dev) if return_lse else None
    need = L.pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, max_pages * page_size, int(split_len))
    ws = _scratch_bytes(dev, "decode", need)
    with torch.cuda.device(dev):
        rc = L.pjx_attn_decode_paged(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(bt), _ptr(kvl), _ptr(o), _ptr(lse), B, Lq, Hq,
                                     Hkv, D, Dv, page_size, max_pages, _DTYPES[q.dtype], float(sm_scale), int(split_len),
                                     _ptr(ws), ws.numel(), _stream(dev))
    _lib.check(rc)
    return (o, lse) if return_lse else o
