"""CPU restatement of the reference's XLA attention path (test infrastructure).

Every function names the reference file:line it follows (paths are relative to
the probjax project root).  Arithmetic is torch on CPU: fp32 scores and
accumulation on the dtype-rounded inputs, exactly as the reference's
``einsum(..., preferred_element_type=float32)`` does.

This module is a checker.  The shipped package never imports it.
"""

from __future__ import annotations

import math

import numpy as np
import torch

# probjax/nn/pallas_kernels/kernels/attention_xla.py:63-69
DENSE_MAX_SCORES = 256 * 256
SINGLE_TILE_MAX_SCORES = 512 * 512
DEFAULT_BLOCK_Q = 256
DEFAULT_BLOCK_K = 256

LOG2E = 1.4426950408889634
# probjax/nn/pallas_kernels/kernel_utils/common.py:17
NEG_INF = -1e15


def auto_strategy(q_len: int, kv_len: int):
    """attention_xla.py:586-592 -- (strategy, block_q, block_k) by score count."""
    if q_len * kv_len <= DENSE_MAX_SCORES:
        return "dense", None, None
    if q_len * kv_len <= SINGLE_TILE_MAX_SCORES:
        return "tiled", q_len, kv_len
    return "tiled", DEFAULT_BLOCK_Q, DEFAULT_BLOCK_K


def _balanced_block(length: int, target: int) -> int:
    """attention_xla.py:595-598."""
    n = max(1, math.ceil(length / target))
    return math.ceil(length / n)


def _as_t(x, dtype=None):
    if x is None:
        return None
    t = x if isinstance(x, torch.Tensor) else torch.as_tensor(np.asarray(x))
    t = t.detach().cpu()
    return t if dtype is None else t.to(dtype)


# ---------------------------------------------------------------------------
# Independent dense formula (what the reference's tests compare against)
# ---------------------------------------------------------------------------


def dense_formula(q, k, v, *, sm_scale, keep=None, bias=None):
    """float64 dense softmax attention with ``repeat`` GQA semantics.

    Restates the test oracle of the reference,
    tests/test_attention_gqa_splitkv.py:41-53 (output) and :198-201
    (``logsumexp`` of the scaled scores, natural log).  ``keep`` is a boolean
    ``[B|1, H|1, Q, K]`` array, ``bias`` an additive ``[B|1, H|1, Q, K]`` array
    added after scaling (attention_xla.py:12, 227-274).  Rows with no valid
    key give 0 and ``lse = +inf`` (attention_xla.py:358-361, 417-420).
    Returns ``(out [B,Lq,Hq,Dv] float64, lse [B,Hq,Lq] float64)``.
    """
    q, k, v = (_as_t(x, torch.float64) for x in (q, k, v))
    rep = q.shape[2] // k.shape[2]
    k = torch.repeat_interleave(k, rep, dim=2)
    v = torch.repeat_interleave(v, rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * float(sm_scale)
    if bias is not None:
        s = s + _as_t(bias, torch.float64)
    if keep is not None:
        s = torch.where(_as_t(keep, torch.bool), s, torch.tensor(-math.inf, dtype=torch.float64))
    m = s.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    p = torch.exp(s - m)
    l_ = p.sum(dim=-1, keepdim=True)
    nonempty = l_ > 0
    p = p / torch.where(nonempty, l_, torch.ones_like(l_))
    out = torch.einsum("bhqk,bkhd->bqhd", p, v)
    lse = torch.where(
        nonempty, m + torch.log(torch.where(nonempty, l_, torch.ones_like(l_))),
        torch.tensor(math.inf, dtype=torch.float64),
    )[..., 0]
    return out, lse


# ---------------------------------------------------------------------------
# Restatement of xla_attention
# ---------------------------------------------------------------------------


def rng_seed_from_key(key) -> int:
    """The 32-bit seed the kernels take, folded from the words of a PRNG key as
    ``_rng_seed_from_key`` does (probjax/nn/pallas_kernels/kernels/attention.py:151-159)."""
    words = [int(w) & 0xFFFFFFFF for w in (key if hasattr(key, "__iter__") else [key])]
    seed = words[0]
    if len(words) > 1:
        seed ^= (words[1] * 0x9E3779B9) & 0xFFFFFFFF
        for i in range(2, len(words)):
            seed ^= (words[i] * ((0x85EBCA6B + i) & 0xFFFFFFFF)) & 0xFFFFFFFF
    return seed & 0xFFFFFFFF


def counter_dropout_scale(seed: int, batch: int, heads: int, q_idx, k_idx, rate: float):
    """Multiplier ``0`` (dropped) or ``1 / (1 - rate)`` of every probability ``[B, H, q, k]``:
    restatement of ``_dropout_mask_counter`` (kernels/attention.py:116-148) in uint32 arithmetic,
    and of ``drop_scale`` on the XLA path (attention_xla.py:280-305)."""
    import numpy as np

    with np.errstate(over="ignore"):
        b = np.arange(batch, dtype=np.uint32)[:, None, None, None]
        h = np.arange(heads, dtype=np.uint32)[None, :, None, None]
        q = np.asarray(q_idx, dtype=np.uint32)[None, None, :, None]
        k = np.asarray(k_idx, dtype=np.uint32)[None, None, None, :]
        x = np.uint32(seed) ^ (b * np.uint32(0x85EBCA6B))
        x = x ^ (h * np.uint32(0xC2B2AE35))
        x = x ^ (q * np.uint32(0x27D4EB2F))
        x = x ^ (k * np.uint32(0x165667B1))
        x = x ^ (x >> np.uint32(16))
        x = x * np.uint32(0x7FEB352D)
        x = x ^ (x >> np.uint32(15))
        x = x * np.uint32(0x846CA68B)
        x = x ^ (x >> np.uint32(16))
    u = x.astype(np.float32) * np.float32(1.0 / float(2 ** 32))
    dropped = u < np.float32(rate)
    return torch.from_numpy(np.where(dropped, np.float32(0.0), np.float32(1.0 / (1.0 - rate))).astype(np.float32))


class _Mods:
    """Score modifiers on a ``[B, Hq, bq, kc]`` tile (attention_xla.py:171-279).

    Order: the scaled scores get the bias added, then masked entries are set to
    ``-inf`` (:236-246 bias, :247-273 mask, :269-271 padded keys).
    """

    def __init__(self, *, causal, kv_lengths, keep, bias, q_len, kv_len, kv_pad, score_fn=None, dropout=None):
        self.score_fn = score_fn
        self.dropout = dropout  # (seed, rate) of the counter-hash dropout, or None
        self.causal = bool(causal)
        self.kv_lengths = None if kv_lengths is None else _as_t(kv_lengths, torch.int64).reshape(-1)
        self.keep = None if keep is None else _as_t(keep, torch.bool)
        self.bias = None if bias is None else _as_t(bias, torch.float32)
        self.q_len, self.kv_len = q_len, kv_len
        self.kv_padded = kv_pad != kv_len

    @property
    def any(self):
        return (
            self.causal
            or self.kv_lengths is not None
            or self.keep is not None
            or self.bias is not None
            or self.kv_padded
            or self.score_fn is not None
        )

    @staticmethod
    def _window(x, q0, bq, k0, kc):
        """Tile window of a ``[.., Q, K]`` array, zero padded past its end."""
        q1, k1 = min(q0 + bq, x.shape[-2]), min(k0 + kc, x.shape[-1])
        w = x[..., q0:q1, k0:k1]
        if w.shape[-2] != bq or w.shape[-1] != kc:
            w = torch.nn.functional.pad(w, (0, kc - w.shape[-1], 0, bq - w.shape[-2]))
        return w

    def apply(self, s, q0, bq, k0, kc):
        if not self.any:
            return s
        if self.score_fn is not None:
            # a bias object is a function of the scaled scores, the head and the absolute indices
            # (attention_xla.py:236-246 calls ``self.bias(s_bh, h, span_q, span_k, data=chunk)``)
            s = self.score_fn(s, q0 + torch.arange(bq), k0 + torch.arange(kc))
        if self.bias is not None:
            s = s + self._window(self.bias, q0, bq, k0, kc)
        keep = None
        qi = q0 + torch.arange(bq)
        ki = k0 + torch.arange(kc)
        if self.causal:  # attention_mask_bias.py:617-646 (q_idx >= k_idx)
            keep = (qi[:, None] >= ki[None, :])[None, None]
        if self.kv_lengths is not None:  # attention_mask_bias.py:1401-1532
            kl = (ki[None, :] < self.kv_lengths[:, None])[:, None, None, :]
            keep = kl if keep is None else keep & kl
        if self.keep is not None:
            kw = self._window(self.keep, q0, bq, k0, kc)
            keep = kw if keep is None else keep & kw
        if self.kv_padded:
            valid = (ki < self.kv_len)[None, None, None, :]
            keep = valid if keep is None else keep & valid
        if keep is not None:
            s = torch.where(keep, s, torch.tensor(-math.inf))
        return s

    def drop_scale(self, shape, q0, bq, k0, kc):
        """attention_xla.py:280-305: per-probability multiplier of a tile, or None."""
        if self.dropout is None:
            return None
        seed, rate = self.dropout
        return counter_dropout_scale(seed, shape[0], shape[1], q0 + torch.arange(bq), k0 + torch.arange(kc), rate)

    def tile_is_dead(self, q0, bq, k0):
        """Static tile skipping of the tiled strategy (attention_xla.py:318-331,
        373-377): a causal tile whose first key lies past its last query."""
        return self.causal and k0 > q0 + bq - 1


def _scores(q5, kc, sm_scale):
    """attention_xla.py:339-344 -- fp32 scores, scale skipped when exactly 1."""
    s = torch.einsum("bhgqd,bhkd->bhgqk", q5.float(), kc.float())
    if sm_scale != 1.0:
        s = s * float(sm_scale)
    b, hkv, g, q, k = s.shape
    return s.reshape(b, hkv * g, q, k)


def _pv(p, vc, hkv):
    """attention_xla.py:347-350 -- P is rounded to V's dtype before the product."""
    b, hq, q, k = p.shape
    p5 = p.reshape(b, hkv, hq // hkv, q, k).to(vc.dtype).float()
    return torch.einsum("bhgqk,bhkd->bhgqd", p5, vc.float())


def _dense_forward(q5, k, v, mods, sm_scale):
    """attention_xla.py:353-366 (plus the LSE, which the tiled path defines)."""
    hkv = k.shape[1]
    q_len, kv_len = q5.shape[3], k.shape[2]
    s = mods.apply(_scores(q5, k, sm_scale), 0, q_len, 0, kv_len)
    m = s.max(dim=-1).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    p = torch.exp(s - m[..., None])
    l_ = p.sum(dim=-1)
    nonempty = l_ > 0
    l_safe = torch.where(nonempty, l_, torch.ones_like(l_))
    p = p / l_safe[..., None]
    lse = torch.where(nonempty, m + torch.log(l_safe), torch.tensor(math.inf))
    drop = mods.drop_scale(p.shape, 0, q_len, 0, kv_len)  # after the normaliser (attention_xla.py:14-15)
    if drop is not None:
        p = p * drop
    return _pv(p, v, hkv), lse


def _tiled_forward(q5, k, v, mods, sm_scale, bq, kc):
    """attention_xla.py:380-429 -- online softmax over ``bq x kc`` tiles."""
    b, hkv, g, q_total, _ = q5.shape
    dv = v.shape[-1]
    hq = hkv * g
    nq, nk = q_total // bq, k.shape[2] // kc
    o_all = torch.empty(b, hkv, g, q_total, dv, dtype=torch.float32)
    lse_all = torch.empty(b, hq, q_total, dtype=torch.float32)
    for i in range(nq):
        q0 = i * bq
        qi = q5[:, :, :, q0 : q0 + bq]
        o = torch.zeros(b, hkv, g, bq, dv, dtype=torch.float32)
        m = torch.full((b, hq, bq), -math.inf, dtype=torch.float32)
        l_ = torch.zeros(b, hq, bq, dtype=torch.float32)
        for j in range(nk):
            k0 = j * kc
            if mods.tile_is_dead(q0, bq, k0):
                continue
            kj, vj = k[:, :, k0 : k0 + kc], v[:, :, k0 : k0 + kc]
            s = mods.apply(_scores(qi, kj, sm_scale), q0, bq, k0, kc)
            m_new = torch.maximum(m, s.max(dim=-1).values)
            m_safe = torch.where(torch.isfinite(m_new), m_new, torch.zeros_like(m_new))
            corr = torch.exp(m - m_safe)
            p = torch.exp(s - m_safe[..., None])
            l_ = l_ * corr + p.sum(dim=-1)
            drop = mods.drop_scale(p.shape, q0, bq, k0, kc)
            if drop is not None:
                p = p * drop
            o = o * corr.reshape(b, hkv, g, bq)[..., None] + _pv(p, vj, hkv)
            m = m_new
        nonempty = l_ > 0
        l_safe = torch.where(nonempty, l_, torch.ones_like(l_))
        o_all[:, :, :, q0 : q0 + bq] = o / l_safe.reshape(b, hkv, g, bq)[..., None]
        lse_all[:, :, q0 : q0 + bq] = torch.where(
            nonempty, m + torch.log(l_safe), torch.tensor(math.inf)
        )
    return o_all, lse_all


def xla_attention(
    q,
    k,
    v,
    *,
    causal: bool = False,
    kv_lengths=None,
    keep=None,
    bias=None,
    sm_scale: float = 1.0,
    strategy: str = "auto",
    block_q: int | None = None,
    block_k: int | None = None,
    return_lse: bool = False,
    score_fn=None,
    dropout=None,
):
    """Restatement of ``xla_attention`` (attention_xla.py:601-721), forward only.

    ``q [B,Lq,Hq,D]``, ``k [B,Lkv,Hkv,D]``, ``v [B,Lkv,Hkv,Dv]``.  The mask is
    given structurally (``causal``: ``CausalMask``; ``kv_lengths [B]``:
    ``KVLenMask``) and/or as a dense boolean ``keep [B|1,H|1,Q,K]``; ``bias`` is
    a dense additive ``[B|1,H|1,Q,K]`` array (``DenseBias``); ``score_fn(s, q_idx, k_idx)``
    stands for a non-dense bias object: it maps the scaled scores ``s [B,Hq,q,k]`` of the
    rows ``q_idx`` and keys ``k_idx`` to modified scores (:236-246); ``dropout = (seed, rate)``
    is the counter-hash dropout (:14-15, 280-305).  Output has
    ``q``'s dtype; the optional LSE is natural log ``[B,Hq,Lq]`` fp32 with
    ``+inf`` for rows without a valid key (:417-420).
    """
    q, k, v = _as_t(q), _as_t(k), _as_t(v)
    batch, q_len, hq, _ = q.shape
    kv_len, hkv = k.shape[1], k.shape[2]
    if hq % hkv != 0:  # :630-631
        raise ValueError(f"query heads {hq} must be a multiple of kv heads {hkv}")
    if v.shape[:3] != k.shape[:3]:  # :632-633
        raise ValueError(f"k {tuple(k.shape)} and v {tuple(v.shape)} must agree on [B, T, H]")
    g = hq // hkv
    out_dtype = q.dtype

    if strategy == "auto":  # :653-655
        strategy, auto_bq, auto_bk = auto_strategy(q_len, kv_len)
        block_q, block_k = block_q or auto_bq, block_k or auto_bk
    if strategy == "dense":
        bq, kc = q_len, kv_len
    elif strategy == "tiled":
        bq = _balanced_block(q_len, block_q or DEFAULT_BLOCK_Q)
        kc = _balanced_block(kv_len, block_k or DEFAULT_BLOCK_K)
    else:
        raise ValueError(f"unknown strategy {strategy!r}")
    q_pad = math.ceil(q_len / bq) * bq
    kv_pad = math.ceil(kv_len / kc) * kc

    def to_bhtd(x, total):  # :668-672
        x = x.permute(0, 2, 1, 3)
        if x.shape[2] != total:
            x = torch.nn.functional.pad(x, (0, 0, 0, total - x.shape[2]))
        return x

    q5 = to_bhtd(q, q_pad).reshape(batch, hkv, g, q_pad, q.shape[-1])
    kt, vt = to_bhtd(k, kv_pad), to_bhtd(v, kv_pad)
    mods = _Mods(
        causal=causal, kv_lengths=kv_lengths, keep=keep, bias=bias,
        q_len=q_len, kv_len=kv_len, kv_pad=kv_pad, score_fn=score_fn, dropout=dropout,
    )
    if strategy == "dense":
        o5, lse = _dense_forward(q5, kt, vt, mods, sm_scale)
    else:
        o5, lse = _tiled_forward(q5, kt, vt, mods, sm_scale, bq, kc)
    o = o5.reshape(batch, hq, q_pad, v.shape[-1])[:, :, :q_len]  # :677-679
    out = o.permute(0, 2, 1, 3).to(out_dtype).contiguous()
    if return_lse:
        return out, lse[:, :, :q_len].contiguous()
    return out


# ---------------------------------------------------------------------------
# Split-KV decode: partials + exact combine
# ---------------------------------------------------------------------------


def combine_partials(o_part, lse_part_base2):
    """Exact combine of per-split partials (attention_splitkv.py:236-250).

    ``o_part [..., S, R, Dv]`` (each normalised by its own sum) and base-2
    ``lse_part [..., S, R]`` (``-1e15`` or ``-inf`` for an empty split).
    Returns ``(out [..., R, Dv] fp32, natural-log lse [..., R] fp32)``; a row
    whose every split is empty gives 0 and ``+inf``.
    """
    o_part = _as_t(o_part, torch.float32)
    lse = _as_t(lse_part_base2, torch.float32)
    lse = torch.where(lse <= NEG_INF, torch.tensor(-math.inf), lse)
    m = lse.max(dim=-2, keepdim=True).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w = torch.exp2(lse - m)
    denom = w.sum(dim=-2)
    out = torch.einsum("...sr,...srd->...rd", w, o_part) / torch.where(
        denom == 0, torch.ones_like(denom), denom
    )[..., None]
    nat = torch.where(
        denom > 0, (m[..., 0, :] + torch.log2(torch.where(denom > 0, denom, torch.ones_like(denom)))) / LOG2E,
        torch.tensor(math.inf),
    )
    return out, nat


def splitkv_reference(q, k, v, *, sm_scale, num_splits, kv_lengths=None):
    """Split-KV forward on CPU (attention_splitkv.py:43-103 kernel math,
    :121-134 GQA row packing ``g * Lq + t``, :184 split length, :236-250
    combine).  ``kv_lengths [B]`` extends the reference (whose split kernel has
    no mask) with per-sequence valid lengths; the expected answer is then the
    one ``flex_attention(..., mask=KVLenMask(lengths))`` gives.

    Returns ``(out [B,Lq,Hq,Dv] in q.dtype, lse [B,Hq,Lq] fp32 natural log,
    o_part, lse_part)``.
    """
    q, k, v = _as_t(q), _as_t(k), _as_t(v)
    b, lq, hq, d = q.shape
    lkv, hkv = k.shape[1], k.shape[2]
    dv = v.shape[-1]
    if hq % hkv:
        raise ValueError(f"Hq={hq} must be a multiple of Hkv={hkv}.")
    g = hq // hkv
    rows = g * lq
    split_len = math.ceil(lkv / num_splits)
    num_splits = math.ceil(lkv / split_len)
    qp = q.reshape(b, lq, hkv, g, d).permute(0, 2, 3, 1, 4).reshape(b, hkv, rows, d).float()
    kt, vt = k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)
    lens = (
        torch.full((b,), lkv, dtype=torch.int64)
        if kv_lengths is None
        else _as_t(kv_lengths, torch.int64).reshape(-1)
    )
    o_part = torch.zeros(b, hkv, num_splits, rows, dv)
    lse_part = torch.full((b, hkv, num_splits, rows), NEG_INF)
    qk_scale = float(sm_scale) * LOG2E
    for s_ in range(num_splits):
        k0, k1 = s_ * split_len, min((s_ + 1) * split_len, lkv)
        sc = torch.einsum("bhrd,bhkd->bhrk", qp, kt[:, :, k0:k1].float()) * qk_scale
        valid = (torch.arange(k0, k1)[None, :] < lens[:, None])[:, None, None, :]
        sc = torch.where(valid, sc, torch.tensor(-math.inf))
        m = sc.max(dim=-1).values
        m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        p = torch.exp2(sc - m_safe[..., None])
        l_ = p.sum(dim=-1)
        o = torch.einsum("bhrk,bhkd->bhrd", p.to(v.dtype).float(), vt[:, :, k0:k1].float())
        safe = torch.where(l_ == 0, torch.ones_like(l_), l_)
        o_part[:, :, s_] = o / safe[..., None]
        lse_part[:, :, s_] = torch.where(l_ == 0, torch.tensor(NEG_INF), m_safe + torch.log2(safe))
    out, nat = combine_partials(o_part, lse_part)
    out = out.reshape(b, hkv, g, lq, dv).permute(0, 3, 1, 2, 4).reshape(b, lq, hq, dv).to(q.dtype)
    nat = nat.reshape(b, hkv, g, lq).reshape(b, hq, lq)
    return out.contiguous(), nat.contiguous(), o_part, lse_part


# ---------------------------------------------------------------------------
# Latent attention
# ---------------------------------------------------------------------------


def materialize_kv(cache, wk, wv, num_heads):
    """latent_attention.py:396-410 -- ``K_h = C W_K[h]^T``, ``V_h = C W_V[h]^T``
    in the input dtype; a missing projection means the latent itself."""
    cache = _as_t(cache)

    def up(w):
        if w is None:
            return cache[..., None, :].expand(*cache.shape[:-1], num_heads, cache.shape[-1])
        w = _as_t(w)
        return torch.einsum("bsr,hdr->bshd", cache.float(), w.float()).to(cache.dtype)

    return up(wk), up(wv)


def mla_reference(q, cache, wk=None, wv=None, *, sm_scale=None, factorisation="auto", **mask_kw):
    """CPU path of ``mla`` (latent_attention.py:591-625 ``_xla_mla``; default
    scale :698-701).  ``factorisation`` "auto" applies the reference's FLOP-count
    rule (:616-625); "materialized"/"absorbed" force one.  ``mask_kw`` goes to
    :func:`xla_attention` (``causal``, ``kv_lengths``, ``keep``, ``bias``,
    ``return_lse``).
    """
    q, cache = _as_t(q), _as_t(cache)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    shared = cache[:, :, None, :]
    if wk is None:
        return xla_attention(q, shared, shared, sm_scale=sm_scale, **mask_kw)
    wk, wv = _as_t(wk), _as_t(wv)
    q_len, kv_len, rank = q.shape[1], cache.shape[1], cache.shape[-1]
    dk, dv = wk.shape[1], wv.shape[1]
    materialized_cost = kv_len * rank * (dk + dv) + q_len * kv_len * (dk + dv)
    absorbed_cost = q_len * rank * (dk + dv) + 2 * q_len * kv_len * rank
    use_absorbed = absorbed_cost < materialized_cost if factorisation == "auto" else factorisation == "absorbed"
    if use_absorbed:
        q_lat = torch.einsum("bqhd,hdr->bqhr", q.float(), wk.float()).to(q.dtype)
        res = xla_attention(q_lat, shared, shared, sm_scale=sm_scale, **mask_kw)
        o_lat, rest = (res[0], res[1:]) if isinstance(res, tuple) else (res, ())
        out = torch.einsum("bqhr,hdr->bqhd", o_lat.float(), wv.float()).to(q.dtype)
        return (out, *rest) if rest else out
    key, value = materialize_kv(cache, wk, wv, q.shape[-2])
    return xla_attention(q, key, value, sm_scale=sm_scale, **mask_kw)


def rope_interleaved(x, positions=None, base: float = 10_000.0):
    """Interleaved (even/odd pair) rotary embedding over the last axis;
    ``x [..., T, H, D]`` or ``[..., T, D]`` with tokens on axis ``-3``/``-2``.
    Follows layers/encoding.py:171-211 (inverse frequencies
    ``base ** (-2i/D)``, pairs ``(x[2i], x[2i+1])`` rotated by ``pos * f_i``).
    """
    x = _as_t(x)
    d = x.shape[-1]
    tok_axis = -3 if x.dim() >= 4 else -2
    t = x.shape[tok_axis]
    pos = torch.arange(t, dtype=torch.float32) if positions is None else _as_t(positions, torch.float32)
    inv = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    if tok_axis == -3:
        cos, sin = cos[:, None, :], sin[:, None, :]
    xf = x.float()
    even, odd = xf[..., ::2], xf[..., 1::2]
    re = even * cos - odd * sin
    ro = odd * cos + even * sin
    return torch.stack((re, ro), dim=-1).reshape(x.shape).to(x.dtype)
