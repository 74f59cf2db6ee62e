"""Mask and bias objects of the attention call signatures.

Host-side mirror of the part of the reference's object model the kernels take
(probjax/nn/pallas_kernels/attention_mask_bias.py): ``NoMask`` (585),
``CausalMask`` (617), ``LocalWindowMask`` (651), ``CausalLocalWindowMask`` (707),
``CausalFromBottomRightMask`` (753), ``QKVLengthMask`` (1079), ``KeyPaddingMask``
(1132), ``KVLenMask`` (1401), ``ComposeMask`` (326) and ``DenseBias`` (1808).  A mask is a
callable ``mask(q_idx, k_idx, seg_q=None, seg_k=None) -> [Q, K] bool`` and can be
materialised with ``dense``; masks combine with ``&``.

Further classes are carried with their dense definition only -- ``NotMask`` (530),
``PrefixLMMask`` (785), ``BlockDiagonalMask`` (871), ``BlockDiagonalCausalMask`` (984),
``SeqLenMask`` (1239), ``SameSegmentMask`` (1537), ``MarginalizationMask`` (1671), ``or`` /
``xor`` compositions, and the additive biases ``ConstantBias`` (1781), ``SumBias`` (553),
``CausalAlibiBias`` (2230), ``SymmetricAlibiBias`` (2355), ``DistanceDecayBias`` (2387),
``LowRankBias`` (1926): :func:`lower_dense` turns them into one additive float32 tensor
(``-inf`` where masked) that the kernels take as a dense bias.  That costs ``O(H Q K)``
memory; it widens what runs on the kernels, it is not a fused implementation.

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


class NotMask(AttentionMask):
    """Logical complement (attention_mask_bias.py:530-548)."""

    def __init__(self, inner: AttentionMask):
        self.inner = inner
        self.stateful = inner.stateful

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        return ~self.inner(q_idx, k_idx, seg_q, seg_k)

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1, seg_q=None, seg_k=None):
        return ~self.inner.dense(q_len, kv_len, batch_size=batch_size, num_heads=num_heads)


class _PerBatchMask(AttentionMask):
    """Masks whose data is per batch element: ``dense`` evaluates ``pair(b)`` -> ``[Q, K]`` bool."""

    stateful = True

    def _pair(self, b, q_len, kv_len):
        raise NotImplementedError

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1, seg_q=None, seg_k=None):
        rows = [self._pair(b, q_len, kv_len).expand(num_heads, q_len, kv_len) for b in range(batch_size)]
        return torch.stack(rows)


def _row(data, b):
    """Batch element ``b`` of ``[B, T]`` data, or shared ``[T]`` data."""
    data = torch.as_tensor(data)
    return data[b] if data.dim() >= 2 else data


class PrefixLMMask(_PerBatchMask):
    """Keys in ``[0, prefix_length)`` visible to all queries, causal elsewhere
    (attention_mask_bias.py:785-866); ``prefix_lengths`` scalar or ``[B]``."""

    def __init__(self, prefix_lengths):
        self.prefix_lengths = torch.as_tensor(prefix_lengths)

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        p = self.prefix_lengths if seg_q is None else torch.as_tensor(seg_q)
        p = p.reshape(-1)[0]
        return (k_idx[None, :] < p) | (q_idx[:, None] >= k_idx[None, :])

    def _pair(self, b, q_len, kv_len):
        p = self.prefix_lengths.reshape(-1)
        return self(_idx(q_len), _idx(kv_len), p[b if p.shape[0] > 1 else 0])


class BlockDiagonalMask(_PerBatchMask):
    """Same block id (attention_mask_bias.py:871-980); ids ``[T]`` or ``[B, T]``."""

    def __init__(self, query_block_ids, key_block_ids=None):
        self.query_block_ids = torch.as_tensor(query_block_ids)
        self.key_block_ids = None if key_block_ids is None else torch.as_tensor(key_block_ids)

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        qids = self.query_block_ids if seg_q is None else torch.as_tensor(seg_q)
        kids = torch.as_tensor(seg_k) if seg_k is not None else (self.key_block_ids if self.key_block_ids is not None else qids)
        return qids[..., :, None] == kids[..., None, :]

    def _pair(self, b, q_len, kv_len):
        qids = _row(self.query_block_ids, b)[:q_len]
        kids = _row(self.key_block_ids if self.key_block_ids is not None else self.query_block_ids, b)[:kv_len]
        return qids[:, None] == kids[None, :]


class BlockDiagonalCausalMask(BlockDiagonalMask):
    """Causal inside each block id (attention_mask_bias.py:984-1075)."""

    def __call__(self, q_idx, k_idx, seg_q=None, seg_k=None):
        return super().__call__(q_idx, k_idx, seg_q, seg_k) & (q_idx[:, None] >= k_idx[None, :])

    def _pair(self, b, q_len, kv_len):
        return super()._pair(b, q_len, kv_len) & (_idx(q_len)[:, None] >= _idx(kv_len)[None, :])


class SameSegmentMask(BlockDiagonalMask):
    """Same segment id (attention_mask_bias.py:1537-1667)."""

    def __init__(self, query_segment_ids, key_segment_ids=None):
        super().__init__(query_segment_ids, key_segment_ids)


class SeqLenMask(_PerBatchMask):
    """Per-batch sequence length ``L``: full attention inside ``[0, L)`` on both axes, only the
    diagonal outside (attention_mask_bias.py:1239-1396)."""

    def __init__(self, seq_lengths):
        self.seq_lengths = torch.as_tensor(seq_lengths)

    def _pair(self, b, q_len, kv_len):
        length = self.seq_lengths.reshape(-1)[b]
        q_idx, k_idx = _idx(q_len), _idx(kv_len)
        rect = (q_idx[:, None] < length) & (k_idx[None, :] < length)
        return rect | (q_idx[:, None] == k_idx[None, :])

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1, seg_q=None, seg_k=None):
        if batch_size != self.seq_lengths.reshape(-1).shape[0]:
            raise ValueError(
                f"SeqLenMask.dense batch_size={batch_size} does not match stored lengths "
                f"{self.seq_lengths.reshape(-1).shape[0]}"
            )
        return super().dense(q_len, kv_len, batch_size=batch_size, num_heads=num_heads)


class MarginalizationMask(_PerBatchMask):
    """Keep-mask on tokens with the diagonal always kept (attention_mask_bias.py:1671-1777)."""

    def __init__(self, mask):
        self.mask = torch.as_tensor(mask).bool()

    def _pair(self, b, q_len, kv_len):
        m = _row(self.mask, b)
        return (m[:q_len, None] & m[None, :kv_len]) | (_idx(q_len)[:, None] == _idx(kv_len)[None, :])


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


class ConstantBias(AttentionBias):
    """``scores + value`` (attention_mask_bias.py:1781-1804)."""

    def __init__(self, value: float):
        self.value = float(value)

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        return torch.full((1, 1, q_len, kv_len), self.value, dtype=torch.float32)


class SumBias(AttentionBias):
    """Sum of two additive biases (attention_mask_bias.py:553-579)."""

    def __init__(self, lhs: AttentionBias, rhs: AttentionBias):
        self.lhs, self.rhs = lhs, rhs

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        a = self.lhs.dense(q_len, kv_len, batch_size=batch_size, num_heads=num_heads)
        b = self.rhs.dense(q_len, kv_len, batch_size=batch_size, num_heads=num_heads)
        return a.float().cpu() + b.float().cpu() if a.device != b.device else a.float() + b.float()


def _alibi_slopes(num_heads):
    # attention_mask_bias.py:2223-2227: slope(h) = 2^-(h+1)
    return torch.exp2(-(torch.arange(num_heads, dtype=torch.float32) + 1.0))


class CausalAlibiBias(AttentionBias):
    """``-slope(h) * relu(i - j)`` (attention_mask_bias.py:2230-2254)."""

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        dist = (_idx(q_len)[:, None] - _idx(kv_len)[None, :]).clamp_min(0).float()
        return -(_alibi_slopes(num_heads)[None, :, None, None] * dist[None, None])


class SymmetricAlibiBias(AttentionBias):
    """``-slope(h) * |i - j|`` (attention_mask_bias.py:2355-2379)."""

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        dist = (_idx(q_len)[:, None] - _idx(kv_len)[None, :]).abs().float()
        return -(_alibi_slopes(num_heads)[None, :, None, None] * dist[None, None])


class DistanceDecayBias(AttentionBias):
    """``-alpha * |i - j|`` (attention_mask_bias.py:2387-2414)."""

    def __init__(self, alpha: float = 1.0):
        self.alpha = float(alpha)

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        dist = (_idx(q_len)[:, None] - _idx(kv_len)[None, :]).abs().float()
        return (-self.alpha * dist)[None, None]


class LowRankBias(AttentionBias):
    """``scale * query_factors @ key_factors^T`` with factors ``[H|1, max_length, rank]``
    (attention_mask_bias.py:1926-2024).  Lowered densely here; the reference folds the factors
    into Q and K instead."""

    def __init__(self, query_factors, key_factors, *, scale: float = 1.0):
        qf, kf = torch.as_tensor(query_factors), torch.as_tensor(key_factors)
        qf = qf[None] if qf.dim() == 2 else qf
        kf = kf[None] if kf.dim() == 2 else kf
        if qf.dim() != 3 or kf.dim() != 3:
            raise ValueError("factors must have shape [H|1, length, rank]")
        if qf.shape[-1] != kf.shape[-1]:
            raise ValueError("query and key factors must have the same rank")
        if qf.shape[0] != kf.shape[0]:
            raise ValueError("query and key factors must have the same head count")
        if scale < 0:
            raise ValueError("scale must be non-negative")
        self.query_factors, self.key_factors, self.scale = qf, kf, float(scale)

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        if q_len > self.query_factors.shape[1]:
            raise ValueError(f"q_len={q_len} exceeds maximum {self.query_factors.shape[1]}")
        if kv_len > self.key_factors.shape[1]:
            raise ValueError(f"kv_len={kv_len} exceeds maximum {self.key_factors.shape[1]}")
        if self.query_factors.shape[0] not in (1, num_heads):
            raise ValueError(f"Cannot broadcast factor head dim {self.query_factors.shape[0]} to {num_heads}")
        qf, kf = self.query_factors[:, :q_len].float(), self.key_factors[:, :kv_len].float()
        return (self.scale * torch.einsum("hqr,hkr->hqk", qf, kf))[None]


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


def _merge_lowered(a: LoweredMask, b: LoweredMask) -> LoweredMask:
    """AND of two lowered masks: the tighter band, the shorter key lengths, the lower query limit."""
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


def split_mask(mask, batch: int, q_len: int, kv_len: int):
    """``(LoweredMask, residual)``: the part of an AND-expression the kernels implement natively,
    and the rest (``None`` if nothing is left) for :func:`lower_dense`."""
    try:
        return lower_mask(mask, batch, q_len, kv_len), None
    except NotImplementedError:
        pass
    if isinstance(mask, ComposeMask) and mask.op == "and":
        la, ra = split_mask(mask.lhs, batch, q_len, kv_len)
        lb, rb = split_mask(mask.rhs, batch, q_len, kv_len)
        residual = ra if rb is None else (rb if ra is None else ComposeMask("and", ra, rb))
        return _merge_lowered(la, lb), residual
    return LoweredMask(), mask


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
        return _merge_lowered(lower_mask(mask.lhs, batch, q_len, kv_len), lower_mask(mask.rhs, batch, q_len, kv_len))
    raise NotImplementedError(f"mask {type(mask).__name__} is not implemented by the sm_100a kernels")


def lower_bias(bias, batch: int, heads: int, q_len: int, kv_len: int):
    """Additive bias -> float32 ``[Bb, Hb, Q, K]`` tensor, or None.  ``DenseBias`` passes
    through; the other additive classes are evaluated densely."""
    if bias is None:
        return None
    if isinstance(bias, DenseBias):
        bias.dense(q_len, kv_len, batch_size=batch, num_heads=heads)  # shape validation
        return bias.bias
    if isinstance(bias, (ConstantBias, SumBias, CausalAlibiBias, SymmetricAlibiBias, DistanceDecayBias, LowRankBias)):
        return bias.dense(q_len, kv_len, batch_size=batch, num_heads=heads).float()
    raise NotImplementedError(f"bias {type(bias).__name__} is not implemented by the sm_100a kernels")


_DENSE_LEAVES = ()  # filled below, once the classes exist


def _dense_lowerable(mask) -> bool:
    """Mask expressions whose ``dense`` form is defined for a whole batch here (``KeyPaddingMask``
    with per-query-row data, for one, is not)."""
    if isinstance(mask, ComposeMask):
        return _dense_lowerable(mask.lhs) and _dense_lowerable(mask.rhs)
    if isinstance(mask, NotMask):
        return _dense_lowerable(mask.inner)
    return isinstance(mask, _DENSE_LEAVES)


def lower_dense(mask, bias, batch: int, heads: int, q_len: int, kv_len: int):
    """Fallback lowering for masks :func:`lower_mask` refuses: the mask's dense boolean form
    becomes ``-inf`` entries of one additive float32 ``[B|1, H|1, Q, K]`` tensor, summed with
    the bias.  Rows without a visible key come out as zeros, as with the structural masks."""
    if not _dense_lowerable(mask):
        raise NotImplementedError(f"mask {type(mask).__name__} is not implemented by the sm_100a kernels")
    keep = mask.dense(q_len, kv_len, batch_size=batch, num_heads=1)
    add = torch.zeros(keep.shape, dtype=torch.float32).masked_fill_(~keep.cpu(), float("-inf"))
    bt = lower_bias(bias, batch, heads, q_len, kv_len)
    if bt is not None:
        add = add.to(bt.device) + bt.float()
    return add


_DENSE_LEAVES = (NoMask, CausalMask, LocalWindowMask, CausalLocalWindowMask, CausalFromBottomRightMask, QKVLengthMask,
                 KVLenMask, PrefixLMMask, BlockDiagonalMask, BlockDiagonalCausalMask, SameSegmentMask, SeqLenMask,
                 MarginalizationMask)
