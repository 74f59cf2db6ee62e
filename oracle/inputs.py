"""Seeded synthetic inputs for the five benchmark configurations (test infrastructure).

The reference's own benchmarks draw iid normal tensors from a seed
(docs/scripts/benchmark_kernel_attn_ext.py); no dataset is involved.  Values are
drawn in fp32 with ``numpy.random.Generator(PCG64)`` and rounded to the
configuration's dtype *before* either the kernels or the oracle see them.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .attention_oracle import rope_interleaved

_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def _normal(rng, shape, dtype, std=1.0):
    x = rng.standard_normal(size=shape, dtype=np.float32)
    if std != 1.0:
        x *= np.float32(std)
    return torch.from_numpy(x).to(dtype)


def make_config(index: int, **over):
    """Inputs of configuration ``index`` (1-5); keyword overrides shrink a case
    (e.g. ``B=1, S=512``) without changing how the values are drawn.

    Returns a dict of torch CPU tensors plus the call's scalars.
    """
    ss = np.random.SeedSequence(20240 + index)
    r = [np.random.Generator(np.random.PCG64(s)) for s in ss.spawn(8)]
    if index == 1:  # causal MHA fp32
        B, H, S, D = (over.get(n, d) for n, d in (("B", 2), ("H", 4), ("S", 256), ("D", 64)))
        dt = _DT[over.get("dtype", "f32")]
        q, k, v = (_normal(r[i], (B, S, H, D), dt) for i in range(3))
        return dict(q=q, k=k, v=v, causal=True, sm_scale=1.0 / math.sqrt(D))
    if index == 2:  # GQA prefill bf16
        B, Hq, Hkv, S, D = (
            over.get(n, d) for n, d in (("B", 4), ("Hq", 32), ("Hkv", 8), ("S", 4096), ("D", 128))
        )
        dt = _DT[over.get("dtype", "bf16")]
        q = _normal(r[0], (B, S, Hq, D), dt)
        k = _normal(r[1], (B, S, Hkv, D), dt)
        v = _normal(r[2], (B, S, Hkv, D), dt)
        return dict(q=q, k=k, v=v, causal=bool(over.get("causal", False)), sm_scale=1.0 / math.sqrt(D))
    if index == 3:  # key-length mask + dense bias
        B, H, S, D = (over.get(n, d) for n, d in (("B", 8), ("H", 16), ("S", 1024), ("D", 64)))
        dt = _DT[over.get("dtype", "bf16")]
        q, k, v = (_normal(r[i], (B, S, H, D), dt) for i in range(3))
        lo = max(1, S // 4)
        kv_lengths = torch.from_numpy(r[3].integers(lo, S + 1, size=B).astype(np.int32))
        bias = _normal(r[4], (1, H, S, S), torch.float32)
        return dict(q=q, k=k, v=v, kv_lengths=kv_lengths, bias=bias, causal=False,
                    sm_scale=1.0 / math.sqrt(D))
    if index == 4:  # GQA split-KV decode over a ragged cache
        B, Hq, Hkv, D, cap = (
            over.get(n, d) for n, d in (("B", 16), ("Hq", 32), ("Hkv", 8), ("D", 128), ("cap", 32768))
        )
        dt = _DT[over.get("dtype", "bf16")]
        q = _normal(r[0], (B, 1, Hq, D), dt)
        k = _normal(r[1], (B, cap, Hkv, D), dt)
        v = _normal(r[2], (B, cap, Hkv, D), dt)
        if over.get("full", False):
            kv_lengths = torch.full((B,), cap, dtype=torch.int32)
        else:
            lo = max(1, cap // 32)
            kv_lengths = torch.from_numpy(r[3].integers(lo, cap + 1, size=B).astype(np.int32))
        return dict(q=q, k=k, v=v, kv_lengths=kv_lengths, sm_scale=1.0 / math.sqrt(D))
    if index == 5:  # latent attention with a decoupled rotary key
        B, H, S, R, dr, dn, dv, dm = (
            over.get(n, d)
            for n, d in (("B", 8), ("H", 16), ("S", 2048), ("R", 512), ("d_rope", 64),
                         ("d_nope", 128), ("d_v", 128), ("d_model", 2048))
        )
        dt = _DT[over.get("dtype", "bf16")]
        hidden = _normal(r[0], (B, S, dm), dt)
        w_dkv = _normal(r[1], (dm, R + dr), dt, 0.02)
        w_q = _normal(r[2], (dm, H * (dn + dr)), dt, 0.02)
        w_uk = _normal(r[3], (H, dn, R), dt, 0.02)
        w_uv = _normal(r[4], (H, dv, R), dt, 0.02)
        hf = hidden.float()
        ckr = hf @ w_dkv.float()
        c_kv, k_rope = ckr[..., :R], ckr[..., R:]
        # RMSNorm with unit scale on the latent (layers/latent_attention.py:313-319, 435-438)
        c_kv = c_kv * torch.rsqrt(c_kv.pow(2).mean(-1, keepdim=True) + 1e-6)
        qf = (hf @ w_q.float()).reshape(B, S, H, dn + dr)
        q_nope, q_rope = qf[..., :dn], qf[..., dn:]
        k_rope = rope_interleaved(k_rope)
        q_rope = rope_interleaved(q_rope)
        cache = torch.cat([c_kv, k_rope], dim=-1).to(dt)  # [B,S,R+dr]
        q = torch.cat([q_nope, q_rope], dim=-1).to(dt)  # [B,S,H,dn+dr]
        wk = torch.zeros(H, dn + dr, R + dr, dtype=dt)
        wk[:, :dn, :R] = w_uk
        wk[:, dn:, R:] = torch.eye(dr, dtype=dt)
        wv = torch.zeros(H, dv, R + dr, dtype=dt)
        wv[:, :, :R] = w_uv
        return dict(q=q, cache=cache, wk=wk, wv=wv, causal=True, sm_scale=1.0 / math.sqrt(dn + dr))
    raise ValueError(f"no configuration {index}")
