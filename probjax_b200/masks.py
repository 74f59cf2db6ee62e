"""Mask and bias objects of the attention call signatures.

Host-side mirror of the part of the reference's object model the kernels take
(probjax/nn/pallas_kernels/attention_mask_bias.py): ``NoMask`` (585),
``CausalMask`` (617), ``LocalWindowMask`` (651), ``CausalLocalWindowMask`` (707),
``CausalFromBottomRightMask`` (753), ``QKVLengthMask`` (1079), ``KeyPaddingMask``
(1132), ``KVLenMask`` (1401), ``ComposeMask`` (326) and ``DenseBias`` (1808).  A mask is a
callable ``mask(q_idx, k_idx, seg_q=None, seg_k=None) -> [Q, K] bool`` and can be
materialised with ``dense``; masks combine with ``&``.

The kernels do not evaluate these callables.  :func:`lower_mask` reduces a mask
expression to the three things the kernels implement natively -- a band of visible
keys around each query row (``i + lo <= j <= i + hi``; the causal mask is the band
``(-inf, 0)``), per-batch key lengths and a query-row limit -- and raises
``NotImplementedError`` for anything else, which the dispatcher reports as "not mine".
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch


def _idx(n, device=None):
    return torch.arange(n, dtype=torch.int32, device=device)


class AttentionMask:
    """Base class (attention_mask_bias.py:36-230)."""

    stateful: bool = False
    query_independent: bool = False

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        raise NotImplementedError

    def dense(self, q_len: int, kv_len: int, *, batch_size: int = 1, num_heads: int = 1,
              seg_q=None, seg_k=None) -> torch.Tensor:
        """Boolean ``[B, H, Q, K]`` (attention_mask_bias.py:65-105)."""
        q_idx, k_idx = _idx(q_len), _idx(kv_len)
        rows = []
        for b in range(batch_size):
            def take(d):
                if d is None:
                    return None
                d = torch.as_tensor(d)
                if d.dim() >= 2 or (d.dim() == 1 and d.shape[0] == batch_size):
                    return d[b]
                return d
            mk = self(q_idx, k_idx, take(seg_q), take(seg_k))
            rows.append(mk.expand(num_heads, q_len, kv_len))
        return torch.stack(rows)

    def __and__(self, other):
        if not isinstance(other, AttentionMask):
            return NotImplemented
        return ComposeMask("and", self, other)


@dataclass(frozen=True)
class NoMask(AttentionMask):
    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        return torch.ones((q_idx.shape[0], k_idx.shape[0]), dtype=torch.bool)


@dataclass(frozen=True)
class CausalMask(AttentionMask):
    """Key ``j`` is visible to query ``i`` iff ``i >= j`` (attention_mask_bias.py:627-629)."""

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        return q_idx[:, None] >= k_idx[None, :]


@dataclass(frozen=True)
class LocalWindowMask(AttentionMask):
    """``-right_window <= i - j <= left_window`` (attention_mask_bias.py:651-704);
    ``right_window=None`` means 0."""

    left_window: int
    right_window: Optional[int] = None

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        dqk = q_idx[:, None].to(torch.int64) - k_idx[None, :].to(torch.int64)
        rw = 0 if self.right_window is None else int(self.right_window)
        return (dqk >= -rw) & (dqk <= int(self.left_window))


@dataclass(frozen=True)
class CausalLocalWindowMask(AttentionMask):
    """Query ``i`` sees keys ``[i - left_window, i]`` (attention_mask_bias.py:707-750)."""

    left_window: int

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        dqk = q_idx[:, None].to(torch.int64) - k_idx[None, :].to(torch.int64)
        return (dqk >= 0) & (dqk <= int(self.left_window))


@dataclass(frozen=True)
class CausalFromBottomRightMask(AttentionMask):
    """Causal mask aligned to the last key: ``i + (kv_length - q_length) >= j``
    (attention_mask_bias.py:753-782)."""

    q_length: int
    kv_length: int

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        shift = int(self.kv_length) - int(self.q_length)
        return (q_idx[:, None].to(torch.int64) + shift) >= k_idx[None, :].to(torch.int64)


@dataclass(frozen=True)
class QKVLengthMask(AttentionMask):
    """``i < q_length and j < kv_length`` (attention_mask_bias.py:1087-1099)."""

    q_length: int
    kv_length: int
    block_sparse: bool = True

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        return (q_idx[:, None] < self.q_length) & (k_idx[None, :] < self.kv_length)


class KVLenMask(AttentionMask):
    """Per-batch key length: batch ``b`` sees keys ``[0, kv_lengths[b])``
    (attention_mask_bias.py:1401-1532)."""

    stateful = True
    query_independent = True

    def __init__(self, kv_lengths):
        self.kv_lengths = torch.as_tensor(kv_lengths)

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        length = seg_q if seg_q is not None else seg_k
        if length is None:
            raise ValueError("KVLenMask needs the batch element's length (use dense())")
        length = torch.as_tensor(length).reshape(-1)[0]
        return (k_idx[None, :] < length).expand(q_idx.shape[0], k_idx.shape[0])

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1, seg_q=None, seg_k=None):
        lengths = self.kv_lengths.reshape(-1).cpu()
        if batch_size != lengths.shape[0]:
            raise ValueError(
                f"KVLenMask.dense batch_size={batch_size} does not match stored lengths {lengths.shape[0]}"
            )
        valid = _idx(kv_len)[None, :] < lengths[:, None]
        return valid[:, None, None, :].expand(batch_size, num_heads, q_len, kv_len)


class KeyPaddingMask(AttentionMask):
    """Key lengths given per *query row*: ``j < seg_q[i]``
    (attention_mask_bias.py:1132-1234; the 1-D form is windowed by the query
    slice, which is why the reference documents it as not being a per-batch
    mask).  With one query row per sequence and ``lengths [B]`` it coincides with
    :class:`KVLenMask`, which is how the decode path of ``MultiHeadAttention``
    uses it (probjax/nn/layers/attention.py:658-673)."""

    stateful = True

    def __init__(self, lengths):
        self.lengths = torch.as_tensor(lengths)

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        rows = self.lengths if seg_q is None else torch.as_tensor(seg_q)
        rows = rows.reshape(-1)
        if rows.shape[0] == 1:
            rows = rows.expand(q_idx.shape[0])
        return k_idx[None, :] < rows[:, None]


class ComposeMask(AttentionMask):
    """Logical combination of two masks (attention_mask_bias.py:326-525); only
    ``and`` lowers to the kernels."""

    def __init__(self, op: str, lhs: AttentionMask, rhs: AttentionMask):
        if op not in ("and", "or", "xor"):
            raise ValueError(f"unknown mask op {op!r}")
        self.op, self.lhs, self.rhs = op, lhs, rhs
        self.stateful = lhs.stateful or rhs.stateful

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1, seg_q=None, seg_k=None):
        a = self.lhs.dense(q_len, kv_len, batch_size=batch_size, num_heads=num_heads)
        b = self.rhs.dense(q_len, kv_len, batch_size=batch_size, num_heads=num_heads)
        return {"and": a & b, "or": a | b, "xor": a ^ b}[self.op]

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        a, b = self.lhs(q_idx, k_idx, seg_q, seg_k), self.rhs(q_idx, k_idx, seg_q, seg_k)
        return {"and": a & b, "or": a | b, "xor": a ^ b}[self.op]


class AttentionBias:
    """Base class (attention_mask_bias.py:233-318): ``bias(scores, h, q_idx, k_idx, data)``."""

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        raise NotImplementedError


class DenseBias(AttentionBias):
    """Additive ``[B|1, H|1, Q, K]`` tensor, added after scaling and not scaled
    (attention_mask_bias.py:1808-1922)."""

    def __init__(self, bias):
        bias = torch.as_tensor(bias)
        if bias.dim() != 4:
            raise ValueError("bias must have shape [B|1, H|1, Q, K]")
        self.bias = bias

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        b = self.bias
        if tuple(b.shape[-2:]) != (q_len, kv_len):
            raise ValueError(
                f"DenseBias shape mismatch: bias[...,Q,K]={tuple(b.shape[-2:])} vs ({q_len},{kv_len})"
            )
        if b.shape[0] not in (1, batch_size):
            raise ValueError(f"Cannot broadcast bias batch dim {b.shape[0]} to {batch_size}")
        if b.shape[1] not in (1, num_heads):
            raise ValueError(f"Cannot broadcast bias head dim {b.shape[1]} to {num_heads}")
        return b.expand(batch_size, num_heads, q_len, kv_len)


@dataclass
class LoweredMask:
    band_lo: Optional[int] = None     # key j visible to query i iff i + band_lo <= j (None: no bound)
    band_hi: Optional[int] = None     # ... and j <= i + band_hi (None: no bound)
    kv_lengths: Optional[Any] = None  # int32 tensor [B] or None
    q_limit: Optional[int] = None     # query rows >= q_limit see no key

    @property
    def causal(self) -> bool:
        """The band is exactly the causal mask."""
        return self.band_hi == 0 and self.band_lo is None

    @property
    def band(self):
        return (self.band_lo, self.band_hi)

    @property
    def banded(self) -> bool:
        return self.band_lo is not None or self.band_hi is not None


def lower_mask(mask, batch: int, q_len: int, kv_len: int) -> LoweredMask:
    """Reduce a mask expression to (causal, kv_lengths, q_limit) or raise
    ``NotImplementedError`` when the kernels do not implement it."""
    if mask is None or isinstance(mask, NoMask):
        return LoweredMask()
    if isinstance(mask, CausalMask):
        return LoweredMask(band_hi=0)
    if isinstance(mask, LocalWindowMask):
        rw = 0 if mask.right_window is None else int(mask.right_window)
        return LoweredMask(band_lo=-int(mask.left_window), band_hi=rw)
    if isinstance(mask, CausalLocalWindowMask):
        return LoweredMask(band_lo=-int(mask.left_window), band_hi=0)
    if isinstance(mask, CausalFromBottomRightMask):
        return LoweredMask(band_hi=int(mask.kv_length) - int(mask.q_length))
    if isinstance(mask, KVLenMask):
        lengths = mask.kv_lengths.reshape(-1)
        if lengths.shape[0] != batch:
            raise ValueError(f"KVLenMask holds {lengths.shape[0]} lengths for a batch of {batch}")
        return LoweredMask(kv_lengths=lengths.to(torch.int32))
    if isinstance(mask, QKVLengthMask):
        out = LoweredMask()
        if mask.kv_length < kv_len:
            out.kv_lengths = torch.full((batch,), max(int(mask.kv_length), 0), dtype=torch.int32)
        if mask.q_length < q_len:
            out.q_limit = max(int(mask.q_length), 0)
        return out
    if isinstance(mask, KeyPaddingMask):
        lengths = mask.lengths.reshape(-1)
        if q_len == 1 and lengths.shape[0] == batch:
            return LoweredMask(kv_lengths=lengths.to(torch.int32))
        raise NotImplementedError(
            "KeyPaddingMask gives key lengths per query row; only the one-query-row decode form "
            "lowers to the kernels (use KVLenMask for per-batch key lengths)"
        )
    if isinstance(mask, ComposeMask) and mask.op == "and":
        a = lower_mask(mask.lhs, batch, q_len, kv_len)
        b = lower_mask(mask.rhs, batch, q_len, kv_len)
        out = LoweredMask()
        los = [x for x in (a.band_lo, b.band_lo) if x is not None]
        his = [x for x in (a.band_hi, b.band_hi) if x is not None]
        out.band_lo = max(los) if los else None
        out.band_hi = min(his) if his else None
        if a.kv_lengths is not None and b.kv_lengths is not None:
            out.kv_lengths = torch.minimum(a.kv_lengths.cpu(), b.kv_lengths.cpu()) \
                if a.kv_lengths.device != b.kv_lengths.device else torch.minimum(a.kv_lengths, b.kv_lengths)
        else:
            out.kv_lengths = a.kv_lengths if a.kv_lengths is not None else b.kv_lengths
        limits = [x for x in (a.q_limit, b.q_limit) if x is not None]
        out.q_limit = min(limits) if limits else None
        return out
    raise NotImplementedError(f"mask {type(mask).__name__} is not implemented by the sm_100a kernels")


def lower_bias(bias, batch: int, heads: int, q_len: int, kv_len: int):
    """``DenseBias`` -> float32 ``[Bb, Hb, Q, K]`` tensor, or None."""
    if bias is None:
        return None
    if isinstance(bias, DenseBias):
        bias.dense(q_len, kv_len, batch_size=batch, num_heads=heads)  # shape validation
        return bias.bias
    raise NotImplementedError(f"bias {type(bias).__name__} is not implemented by the sm_100a kernels")
