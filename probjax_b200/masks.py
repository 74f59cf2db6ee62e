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

import functools
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


def _library_constant(t):
    """Marks a tensor the library computed from Python scalars alone: its device copy may be cached
    (nobody else holds it, so nobody can change it)."""
    t._pjx_constant = True
    return t


@functools.lru_cache(maxsize=64)
def _alibi_slopes(num_heads):
    # attention_mask_bias.py:2223-2227: slope(h) = 2^-(h+1)
    return _library_constant(torch.exp2(-(torch.arange(num_heads, dtype=torch.float32) + 1.0)))


@functools.lru_cache(maxsize=64)
def _constant_slopes(num_heads, value):
    return _library_constant(torch.full((num_heads,), value, dtype=torch.float32))


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

    @property
    def rank(self) -> int:
        return self.query_factors.shape[-1]

    def factors(self, q_len, kv_len, num_heads):
        """Factors in attention layout ``[1, length, H|1, rank]`` (attention_mask_bias.py:1974-2000)."""
        if q_len > self.query_factors.shape[1]:
            raise ValueError(f"q_len={q_len} exceeds maximum {self.query_factors.shape[1]}")
        if kv_len > self.key_factors.shape[1]:
            raise ValueError(f"kv_len={kv_len} exceeds maximum {self.key_factors.shape[1]}")
        if self.query_factors.shape[0] not in (1, num_heads):
            raise ValueError(f"Cannot broadcast factor head dim {self.query_factors.shape[0]} to {num_heads}")
        return self.query_factors[:, :q_len].permute(1, 0, 2)[None], self.key_factors[:, :kv_len].permute(1, 0, 2)[None]

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        qf, kf = self.factors(q_len, kv_len, num_heads)
        return self.scale * torch.einsum("bqhr,bkhr->bhqk", qf.float(), kf.float())


class BatchedLowRankBias(AttentionBias):
    """Per-example factored bias ``scale * query_factors[b] @ key_factors[b]^T`` with factors
    ``[B, length, rank]`` shared by the heads (attention_mask_bias.py:2028-2192).  Folded into extra
    q / k columns like :class:`LowRankBias`; a query factor of length 1 broadcasts over the rows."""

    def __init__(self, query_factors, key_factors, *, scale: float = 1.0):
        qf, kf = torch.as_tensor(query_factors), torch.as_tensor(key_factors)
        if qf.dim() != 3 or kf.dim() != 3:
            raise ValueError("factors must have shape [B, length, rank]")
        if qf.shape[-1] != kf.shape[-1]:
            raise ValueError("query and key factors must have the same rank")
        if qf.shape[0] != kf.shape[0]:
            raise ValueError("query and key factors must have the same batch size")
        if scale < 0:
            raise ValueError("scale must be non-negative")
        self.query_factors, self.key_factors, self.scale = qf, kf, float(scale)

    @classmethod
    def from_key_bias(cls, key_bias, q_len: int = 1) -> "BatchedLowRankBias":
        """Rank-1 bias that adds ``key_bias[b, j]`` to every score of key ``j`` (2069-2083)."""
        kb = torch.as_tensor(key_bias)
        if kb.dim() != 2:
            raise ValueError("key_bias must have shape [B, kv_len]")
        return cls(torch.ones((kb.shape[0], q_len, 1), dtype=kb.dtype, device=kb.device), kb[..., None])

    @property
    def rank(self) -> int:
        return self.query_factors.shape[-1]

    def factors(self, q_len, kv_len, num_heads):
        """``[B, length, 1, rank]`` (2089-2127): broadcast over the heads by the caller."""
        if self.query_factors.shape[1] == 1:
            qf = self.query_factors.expand(-1, q_len, -1)
        elif q_len <= self.query_factors.shape[1]:
            qf = self.query_factors[:, :q_len]
        else:
            raise ValueError(f"q_len={q_len} exceeds maximum {self.query_factors.shape[1]}")
        if kv_len > self.key_factors.shape[1]:
            raise ValueError(f"kv_len={kv_len} exceeds maximum {self.key_factors.shape[1]}")
        return qf[:, :, None, :], self.key_factors[:, :kv_len, None, :]

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        qf, kf = self.factors(q_len, kv_len, num_heads)
        return self.scale * torch.einsum("bqhr,bkhr->bhqk", qf.float(), kf.float())


class LearnedAlibiBias(AttentionBias):
    """``scores - slope[h] * ((q + query_offset) - (k + key_offset))`` with caller-owned slopes
    ``[H|1]`` (attention_mask_bias.py:2258-2351; meant for use under a causal mask).  When the slopes
    require a gradient it is folded into two extra q / k columns as in the reference, so the gradient
    reaches them through dq / dk; otherwise the kernels read it from a float32 table indexed by the
    head and ``k - q``."""

    scale = 1.0
    rank = 2

    def __init__(self, slopes, *, query_offset: int = 0, key_offset: int = 0):
        s = torch.as_tensor(slopes)
        s = s[None] if s.dim() == 0 else s
        if s.dim() != 1:
            raise ValueError("slopes must have shape [H|1]")
        self.slopes, self.query_offset, self.key_offset = s, int(query_offset), int(key_offset)

    def _head_slopes(self, num_heads):
        if self.slopes.shape[0] not in (1, num_heads):
            raise ValueError(f"slope head count {self.slopes.shape[0]} cannot broadcast to {num_heads}")
        return self.slopes.expand(num_heads)

    def factors(self, q_len, kv_len, num_heads):
        """``q' = (-slope * q_pos, 1)``, ``k' = (1, slope * k_pos)``: ``[1, length, H, 2]`` (2296-2321)."""
        sl = self._head_slopes(num_heads)
        q_pos = torch.arange(q_len, dtype=sl.dtype, device=sl.device) + self.query_offset
        k_pos = torch.arange(kv_len, dtype=sl.dtype, device=sl.device) + self.key_offset
        qf = torch.stack((-sl[:, None] * q_pos[None], torch.ones((num_heads, q_len), dtype=sl.dtype, device=sl.device)), -1)
        kf = torch.stack((torch.ones((num_heads, kv_len), dtype=sl.dtype, device=sl.device), sl[:, None] * k_pos[None]), -1)
        return qf.transpose(0, 1)[None], kf.transpose(0, 1)[None]

    def relative_table(self, q_len, kv_len, num_heads):
        """``[H, q_len + kv_len - 1]`` float32: entry ``(j - i) + q_len - 1`` is the bias of ``(i, j)``."""
        rel = torch.arange(-(q_len - 1), kv_len, dtype=torch.float32)  # j - i
        sl = self._head_slopes(num_heads).detach().float().cpu()
        return sl[:, None] * (rel[None, :] - float(self.query_offset - self.key_offset))

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        tab = self.relative_table(q_len, kv_len, num_heads)
        idx = (_idx(kv_len)[None, :] - _idx(q_len)[:, None] + (q_len - 1)).to(torch.int64)
        return tab[:, idx][None]


class IdentityBias(AttentionBias):
    """Leaves the scores as they are (attention_mask_bias.py, ``IdentityBias``)."""

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        return torch.zeros((1, 1, q_len, kv_len), dtype=torch.float32)


def _t5_bucket(relative_position, *, num_buckets: int, max_distance: int, bidirectional: bool):
    """T5 log-bucketing of ``k - q`` (attention_mask_bias.py:2417-2449)."""
    import math

    rp = -relative_position.to(torch.int64)
    if bidirectional:
        half = num_buckets // 2
        sign_bucket = (rp < 0).to(torch.int64) * half
        rp = rp.abs()
        nb = half
    else:
        sign_bucket = torch.zeros_like(rp)
        rp = rp.clamp_min(0)
        nb = num_buckets
    max_exact = nb // 2
    is_small = rp < max_exact
    rp_f = rp.to(torch.float32)
    val_large = max_exact + (torch.log(rp_f.clamp_min(1.0) / max_exact) / math.log(max_distance / max_exact)
                             * (nb - max_exact))
    val_large = val_large.to(torch.int64).clamp_max(nb - 1)
    return torch.where(is_small, rp, val_large) + sign_bucket


class _RelativeBias(AttentionBias):
    """Biases that depend on the head and on ``k - q`` only: ``table(rel) -> [H|1, len(rel)]``."""

    def table(self, rel):
        raise NotImplementedError

    def relative_table(self, q_len, kv_len):
        """``[H|1, q_len + kv_len - 1]`` float32: entry ``(j - i) + q_len - 1`` is the bias of ``(i, j)``."""
        rel = torch.arange(-(q_len - 1), kv_len, dtype=torch.int64)
        return self.table(rel).float()

    def dense(self, q_len, kv_len, *, batch_size=1, num_heads=1):
        rel = _idx(kv_len)[None, :].to(torch.int64) - _idx(q_len)[:, None].to(torch.int64)
        return self.table(rel.reshape(-1)).float().reshape(-1, q_len, kv_len)[None]


class T5RelativePositionBias(_RelativeBias):
    """``table[h, bucket(k - q)]`` with T5's bucketing (attention_mask_bias.py:2453-2517)."""

    def __init__(self, bias_table, *, num_buckets: int, max_distance: int = 128, bidirectional: bool = True):
        bt = torch.as_tensor(bias_table)
        bt = bt[None] if bt.dim() == 1 else bt
        if bt.dim() != 2:
            raise ValueError("bias_table must have shape [H|1, num_buckets]")
        if bt.shape[-1] != int(num_buckets):
            raise ValueError("bias_table last dim must equal num_buckets")
        self.bias_table, self.num_buckets = bt, int(num_buckets)
        self.max_distance, self.bidirectional = int(max_distance), bool(bidirectional)

    def table(self, rel):
        buckets = _t5_bucket(rel, num_buckets=self.num_buckets, max_distance=self.max_distance,
                             bidirectional=self.bidirectional)
        return self.bias_table.cpu()[:, buckets]


class LearnedRelativePositionBias(_RelativeBias):
    """``table[h, clip(k - q, -M, M) + M]`` (attention_mask_bias.py:2521-2560)."""

    def __init__(self, table, *, max_distance: int):
        t = torch.as_tensor(table)
        t = t[None] if t.dim() == 1 else t
        if t.dim() != 2:
            raise ValueError("table must have shape [H|1, 2*max_distance+1]")
        if t.shape[-1] != 2 * int(max_distance) + 1:
            raise ValueError("table last dim must be 2*max_distance+1")
        self.tab, self.max_distance = t, int(max_distance)

    def table(self, rel):
        return self.tab.cpu()[:, rel.clamp(-self.max_distance, self.max_distance) + self.max_distance]


class SoftCappingBias(AttentionBias):
    """``softcap * tanh(scores / softcap)`` (attention_mask_bias.py:2564-2601).  Not additive: it has
    no dense form; the kernels evaluate it (and its derivative ``1 - tanh^2``) on the scores."""

    def __init__(self, softcap: float = 20.0):
        if softcap <= 0:
            raise ValueError("softcap must be > 0")
        self.softcap = float(softcap)


class PerHeadScaleBias(AttentionBias):
    """``scores * scale[h]`` (attention_mask_bias.py:2606-2650).  Not additive, no dense form."""

    def __init__(self, scales):
        s = torch.as_tensor(scales, dtype=torch.float32)
        s = s[None] if s.dim() == 0 else s
        if s.dim() != 1:
            raise ValueError("scales must be shape [H|1]")
        self.scales = s


@dataclass
class LoweredMask:
    band_lo: Optional[int] = None     # key j visible to query i iff i + band_lo <= j (None: no bound)
    band_hi: Optional[int] = None     # ... and j <= i + band_hi (None: no bound)
    kv_lengths: Optional[Any] = None  # int32 tensor [B] or None
    q_limit: Optional[int] = None     # query rows >= q_limit see no key
    # evaluated inside the kernels from O(B T) data (pjx_score_mod):
    seg_q: Optional[Any] = None         # int32 [Bs, Lq]: key j visible iff seg_q[b, i] == seg_k[b, j]
    seg_k: Optional[Any] = None         # int32 [Bs, Lkv]
    row_kv_limit: Optional[Any] = None  # int32 [Bs, Lq]: key j visible iff j < row_kv_limit[b, i]
    prefix_len: Optional[Any] = None    # int32 [B]: keys j < prefix_len[b] visible to every row (OR with the band)

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

    @property
    def structured(self) -> bool:
        """Carries data the kernels evaluate per element (segments, row limits, prefix)."""
        return self.seg_q is not None or self.row_kv_limit is not None or self.prefix_len is not None


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
    # one pair of segment ids, one set of row limits, one prefix; the prefix is OR-ed with the band, so
    # it cannot be merged with a band that comes from another mask: (A | P) & C != (A & C) | P
    for name in ("seg_q", "seg_k", "row_kv_limit", "prefix_len"):
        x, y = getattr(a, name), getattr(b, name)
        if x is not None and y is not None:
            raise _MergeConflict(f"two masks with {name} data")
        setattr(out, name, x if x is not None else y)
    if (a.prefix_len is not None and b.banded) or (b.prefix_len is not None and a.banded):
        raise _MergeConflict("a prefix mask cannot be AND-ed with another band natively")
    return out


class _MergeConflict(NotImplementedError):
    """Two natively lowered masks whose AND has no native form."""


def _token_ids(keep, length):
    """Segment ids for masks of the form ``(a_i & a_j) | i == j``: 0 where ``a``, else a negative id of
    the token's own, so that equality of ids is the mask."""
    t = torch.arange(length, dtype=torch.int32)
    return torch.where(keep[..., :length], torch.zeros((), dtype=torch.int32), -(t + 1))


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
        try:
            merged = _merge_lowered(la, lb)
        except _MergeConflict:  # keep the left side native, the whole right side goes dense
            merged, rb = la, mask.rhs
        residual = ra if rb is None else (rb if ra is None else ComposeMask("and", ra, rb))
        return merged, residual
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
        lengths = mask.lengths
        if q_len == 1 and lengths.dim() == 1 and lengths.shape[0] == batch:
            return LoweredMask(kv_lengths=lengths.to(torch.int32))
        # per query row (the reference lays 1-D data out as (1, T, 1, 1), attention_mask_bias.py:1175-1204)
        if lengths.dim() == 1 and lengths.shape[0] in (1, q_len):
            return LoweredMask(row_kv_limit=lengths.to(torch.int32).expand(q_len).reshape(1, q_len).contiguous())
        if lengths.dim() == 2 and lengths.shape[0] in (1, batch) and lengths.shape[1] == q_len:
            return LoweredMask(row_kv_limit=lengths.to(torch.int32).contiguous())
        raise NotImplementedError(
            "KeyPaddingMask gives key lengths per query row: pass [Lq] or [B, Lq] lengths "
            "(use KVLenMask for per-batch key lengths)"
        )
    if isinstance(mask, BlockDiagonalMask):  # also BlockDiagonalCausalMask, SameSegmentMask
        qids = mask.query_block_ids
        kids = mask.key_block_ids if mask.key_block_ids is not None else qids
        qids = (qids if qids.dim() == 2 else qids[None])[:, :q_len].to(torch.int32).contiguous()
        kids = (kids if kids.dim() == 2 else kids[None])[:, :kv_len].to(torch.int32).contiguous()
        if qids.shape[1] != q_len or kids.shape[1] != kv_len or qids.shape[0] not in (1, batch) \
                or kids.shape[0] not in (1, batch):
            raise ValueError(f"segment ids {tuple(qids.shape)} / {tuple(kids.shape)} do not cover "
                             f"[B|1, {q_len}] / [B|1, {kv_len}]")
        return LoweredMask(seg_q=qids, seg_k=kids, band_hi=0 if isinstance(mask, BlockDiagonalCausalMask) else None)
    if isinstance(mask, SeqLenMask):
        lengths = mask.seq_lengths.reshape(-1).cpu()
        if lengths.shape[0] != batch:
            raise ValueError(f"SeqLenMask holds {lengths.shape[0]} lengths for a batch of {batch}")
        n = max(q_len, kv_len)
        ids = _token_ids(torch.arange(n)[None, :] < lengths[:, None], n)
        return LoweredMask(seg_q=ids[:, :q_len].contiguous(), seg_k=ids[:, :kv_len].contiguous())
    if isinstance(mask, MarginalizationMask):
        keep = mask.mask.cpu()
        keep = keep if keep.dim() == 2 else keep[None]
        n = max(q_len, kv_len)
        if keep.shape[1] < n or keep.shape[0] not in (1, batch):
            raise ValueError(f"MarginalizationMask data {tuple(keep.shape)} does not cover [B|1, {n}]")
        ids = _token_ids(keep, n)
        return LoweredMask(seg_q=ids[:, :q_len].contiguous(), seg_k=ids[:, :kv_len].contiguous())
    if isinstance(mask, PrefixLMMask):
        pl = mask.prefix_lengths.reshape(-1).to(torch.int32)
        if pl.shape[0] not in (1, batch):
            raise ValueError(f"PrefixLMMask holds {pl.shape[0]} lengths for a batch of {batch}")
        return LoweredMask(band_hi=0, prefix_len=pl.expand(batch).contiguous())
    if isinstance(mask, ComposeMask) and mask.op == "and":
        return _merge_lowered(lower_mask(mask.lhs, batch, q_len, kv_len), lower_mask(mask.rhs, batch, q_len, kv_len))
    raise NotImplementedError(f"mask {type(mask).__name__} is not implemented by the sm_100a kernels")


@dataclass
class LoweredBias:
    """A bias expression as the kernels take it: one dense tensor (or none) plus the modifiers
    evaluated per element from O(H T) data."""

    dense: Optional[Any] = None         # float32 [B|1, H|1, Q, K]
    rel_bias: Optional[Any] = None      # float32 [H|1, Q + K - 1]
    alibi_slopes: Optional[Any] = None  # float32 [H]
    alibi_mode: int = 0                 # 1: -slope * relu(i - j), 2: -slope * |i - j|
    head_scale: Optional[Any] = None    # float32 [H]
    softcap: float = 0.0
    low_rank: tuple = ()                # LowRankBias terms, for the caller to fold into Q / K

    @property
    def structured(self) -> bool:
        return (self.rel_bias is not None or self.alibi_slopes is not None or self.head_scale is not None
                or self.softcap > 0)


def _bias_terms(bias):
    if bias is None:
        return []
    if isinstance(bias, SumBias):
        return _bias_terms(bias.lhs) + _bias_terms(bias.rhs)
    return [bias]


def lower_bias_structured(bias, batch: int, heads: int, q_len: int, kv_len: int) -> LoweredBias:
    """A (sum of) bias objects as a :class:`LoweredBias`: nothing of size ``Q x K`` is built except for
    ``DenseBias`` terms, which already are that tensor."""
    out = LoweredBias()
    low_rank = []
    for term in _bias_terms(bias):
        if isinstance(term, IdentityBias):
            continue
        if isinstance(term, DenseBias):
            term.dense(q_len, kv_len, batch_size=batch, num_heads=heads)  # shape validation
            d = term.bias.float()
            out.dense = d if out.dense is None else out.dense + d.to(out.dense.device)
            continue
        if isinstance(term, (LowRankBias, BatchedLowRankBias)) or (
                isinstance(term, LearnedAlibiBias) and term.slopes.requires_grad):
            if isinstance(term, BatchedLowRankBias) and term.query_factors.shape[0] not in (1, batch):
                raise ValueError(f"Cannot broadcast factors of batch {term.query_factors.shape[0]} to {batch}")
            low_rank.append(term)
            continue
        if isinstance(term, SoftCappingBias):
            if out.softcap > 0:
                raise NotImplementedError("two soft-capping terms in one bias sum")
            out.softcap = term.softcap
            continue
        if isinstance(term, PerHeadScaleBias):
            if out.head_scale is not None:
                raise NotImplementedError("two per-head scale terms in one bias sum")
            if term.scales.shape[0] not in (1, heads):
                raise ValueError(f"Cannot broadcast {term.scales.shape[0]} head scales to {heads} heads")
            out.head_scale = term.scales.float().expand(heads).contiguous()
            continue
        slopes = mode = None
        if isinstance(term, CausalAlibiBias):
            slopes, mode = _alibi_slopes(heads), 1
        elif isinstance(term, SymmetricAlibiBias):
            slopes, mode = _alibi_slopes(heads), 2
        elif isinstance(term, DistanceDecayBias):
            slopes, mode = _constant_slopes(heads, float(term.alpha)), 2
        if slopes is not None and out.alibi_slopes is None:
            out.alibi_slopes, out.alibi_mode = slopes, mode
            continue
        # everything else that depends on (head, j - i) only goes into the relative-position table
        if slopes is not None:
            rel = torch.arange(-(q_len - 1), kv_len, dtype=torch.float32)
            dist = (-rel).clamp_min(0) if mode == 1 else rel.abs()
            tab = -(slopes[:, None] * dist[None, :])
        elif isinstance(term, ConstantBias):
            tab = torch.full((1, q_len + kv_len - 1), term.value, dtype=torch.float32)
        elif isinstance(term, LearnedAlibiBias):
            tab = term.relative_table(q_len, kv_len, heads)
        elif isinstance(term, _RelativeBias):
            tab = term.relative_table(q_len, kv_len)
            if tab.shape[0] not in (1, heads):
                raise ValueError(f"Cannot broadcast a bias table of {tab.shape[0]} heads to {heads}")
        else:
            raise NotImplementedError(f"bias {type(term).__name__} is not implemented by the sm_100a kernels")
        if out.rel_bias is None:
            out.rel_bias = tab
        else:  # [1, n] + [H, n] broadcasts
            out.rel_bias = out.rel_bias + tab
    out.low_rank = tuple(low_rank)
    if out.rel_bias is not None:
        out.rel_bias = out.rel_bias.contiguous()
    return out


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
