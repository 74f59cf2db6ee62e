"""JAX side of the drop-in: registers the XLA FFI handlers of ``libpjx_ffi.so`` (built from
``csrc/ffi_shim.cc``) and provides the ``impl`` functions a probjax maintainer hands to
``make_kernel_primitive`` (probjax/core/custom_primitives/sharded_primitive.py:382-483) in place
of the Pallas launchers.  The KernelSpecs -- and with them sharding over batch / heads, vmap and
abstract evaluation -- stay the reference's own.

Importing this module needs ``jax`` (>= 0.4.31 for ``jax.ffi``; the reference pins >= 0.9) and the
shim library; without them :func:`available` is False and everything else raises.  Nothing in the
torch-side package imports it.

Conventions of the handlers (see ``ffi_shim.cc``): an absent optional operand is a zero-element
array, scratch memory is an extra uint8 result sized by the matching ``pjx_*_workspace_bytes``.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

from . import _lib

_PKG = Path(__file__).resolve().parent
FFI_LIB_PATH = Path(os.environ.get("PJX_FFI_LIB", _PKG / "libpjx_ffi.so"))

TARGETS = (
    "pjx_ffi_mha_fwd", "pjx_ffi_mha_bwd", "pjx_ffi_mha_jvp", "pjx_ffi_decode_splitkv",
    "pjx_ffi_decode_splitkv_static", "pjx_ffi_decode_paged", "pjx_ffi_combine", "pjx_ffi_mla_fwd",
    "pjx_ffi_linear", "pjx_ffi_rope", "pjx_ffi_kv_cache_append",
)

BAND_NO_LOWER, BAND_NO_UPPER = -(1 << 30), 1 << 30
_registered = False


def available() -> bool:
    try:
        import jax.ffi  # noqa: F401
    except Exception:
        return False
    return FFI_LIB_PATH.exists()


def register() -> None:
    """``jax.ffi.register_ffi_target`` for every handler, platform CUDA (idempotent)."""
    global _registered
    if _registered:
        return
    import jax

    if not FFI_LIB_PATH.exists():
        raise RuntimeError(f"{FFI_LIB_PATH} is missing: build it with `python -m probjax_b200.build --ffi`")
    _lib.lib()  # the handlers resolve their symbols against libpjx_attention.so
    handle = ctypes.CDLL(os.fspath(FFI_LIB_PATH))
    for name in TARGETS:
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(handle, name)), platform="CUDA")
    _registered = True


def _absent(dtype):
    import jax.numpy as jnp

    return jnp.zeros((0,), dtype)


def _band(static) -> tuple[int, int]:
    """(band_lo, band_hi) from the statics the reference's specs carry: ``causal`` or a window."""
    if "band" in static:
        lo, hi = static["band"]
        return (BAND_NO_LOWER if lo is None else int(lo)), (BAND_NO_UPPER if hi is None else int(hi))
    return BAND_NO_LOWER, (0 if static.get("causal") else BAND_NO_UPPER)


def mha_fwd_impl(q, k, v, rng_seed=None, b_data=None, q_id=None, k_id=None, dropout_mask=None, index_offset=None,
                 index_offset_size=None, *, kv_lengths=None, return_residuals=True, **static):
    """``impl`` for the ``mha_fwd`` / ``mha_fwd_res`` (+ ``_gqa``) specs (kernels/attention.py:2456-2565).
    ``b_data`` is the ``DenseBias`` operand ``[B|1, H|1, Q, K]``; ``kv_lengths`` the ``KVLenMask`` data as
    ``int32[B]``.  Dropout and block-sparse offsets have no B200 kernel: those calls keep the Pallas impl."""
    import jax
    import jax.numpy as jnp

    register()
    if dropout_mask is not None or index_offset is not None or static.get("dropout_rate", 0.0) > 0:
        raise NotImplementedError("dropout / block-sparse iteration: not a B200 kernel call")
    B, Lq, Hq, _ = q.shape
    Dv = v.shape[-1]
    lo, hi = _band(static)
    out_types = (jax.ShapeDtypeStruct((B, Lq, Hq, Dv), q.dtype),
                 jax.ShapeDtypeStruct((B, Hq, Lq) if return_residuals else (0,), jnp.float32),
                 jax.ShapeDtypeStruct((0,), jnp.int32))
    o, lse, _ = jax.ffi.ffi_call("pjx_ffi_mha_fwd", out_types)(
        q, k, v,
        _absent(jnp.int32) if kv_lengths is None else kv_lengths.astype(jnp.int32).reshape(-1),
        _absent(jnp.float32) if b_data is None else b_data.astype(jnp.float32),
        sm_scale=float(static.get("sm_scale", 1.0)), band_lo=lo, band_hi=hi)
    return (o, lse) if return_residuals else o


def mha_bwd_impl(q, k, v, o, lse, d_o, b_data=None, *, kv_lengths=None, bias_grad=False, **static):
    """``impl`` for the ``mha_bwd`` spec (kernels/attention.py:2509-2534).  ``lse`` is the natural-log
    residual of :func:`mha_fwd_impl`, not the base-2 residual of the Triton kernels."""
    import jax
    import jax.numpy as jnp

    register()
    B, Lq, Hq, _ = q.shape
    lo, hi = _band(static)
    ws = int(_lib.lib().pjx_attn_bwd_workspace_bytes(B, Lq, Hq))
    out_types = (jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct(k.shape, k.dtype),
                 jax.ShapeDtypeStruct(v.shape, v.dtype),
                 jax.ShapeDtypeStruct(b_data.shape if (bias_grad and b_data is not None) else (0,), jnp.float32),
                 jax.ShapeDtypeStruct((ws,), jnp.uint8), jax.ShapeDtypeStruct((0,), jnp.int32))
    dq, dk, dv, dbias, _, _ = jax.ffi.ffi_call("pjx_ffi_mha_bwd", out_types)(
        q, k, v, o, lse, d_o,
        _absent(jnp.int32) if kv_lengths is None else kv_lengths.astype(jnp.int32).reshape(-1),
        _absent(jnp.float32) if b_data is None else b_data.astype(jnp.float32),
        sm_scale=float(static.get("sm_scale", 1.0)), band_lo=lo, band_hi=hi)
    return (dq, dk, dv, dbias) if bias_grad else (dq, dk, dv)


def mha_jvp_impl(q, k, v, tq, tk, tv, lse, b_data=None, *, kv_lengths=None, **static):
    """Forward-mode rule (``mha_jvp_from_lse_kernel``, kernels/attention.py:536-660)."""
    import jax
    import jax.numpy as jnp

    register()
    B, Lq, Hq, _ = q.shape
    lo, hi = _band(static)
    z = _absent(q.dtype)
    (t_o,) = jax.ffi.ffi_call("pjx_ffi_mha_jvp", (jax.ShapeDtypeStruct((B, Lq, Hq, v.shape[-1]), q.dtype),))(
        q, k, v, z if tq is None else tq, z if tk is None else tk, z if tv is None else tv, lse,
        _absent(jnp.int32) if kv_lengths is None else kv_lengths.astype(jnp.int32).reshape(-1),
        _absent(jnp.float32) if b_data is None else b_data.astype(jnp.float32),
        sm_scale=float(static.get("sm_scale", 1.0)), band_lo=lo, band_hi=hi)
    return t_o


def splitkv_forward_impl(q, k, v, *, sm_scale, kv_lengths=None, return_lse=False, split_len=0, static_scratch=False):
    """Stands where ``splitkv_forward`` calls ``pl.pallas_call`` (attention_splitkv.py:204-234).
    ``static_scratch`` uses the entry point that needs no workspace result."""
    import jax
    import jax.numpy as jnp

    register()
    B, Lq, Hq, _ = q.shape
    cap, Hkv, Dv = k.shape[1], k.shape[2], v.shape[3]
    lens = _absent(jnp.int32) if kv_lengths is None else kv_lengths.astype(jnp.int32).reshape(-1)
    outs = [jax.ShapeDtypeStruct((B, Lq, Hq, Dv), q.dtype),
            jax.ShapeDtypeStruct((B, Hq, Lq) if return_lse else (0,), jnp.float32)]
    if static_scratch:
        res = jax.ffi.ffi_call("pjx_ffi_decode_splitkv_static", tuple(outs))(
            q, k, v, lens, sm_scale=float(sm_scale), split_len=int(split_len))
    else:
        ws = int(_lib.lib().pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, cap, int(split_len)))
        outs.append(jax.ShapeDtypeStruct((max(ws, 256),), jnp.uint8))
        res = jax.ffi.ffi_call("pjx_ffi_decode_splitkv", tuple(outs))(
            q, k, v, lens, sm_scale=float(sm_scale), split_len=int(split_len))
    return (res[0], res[1]) if return_lse else res[0]


def mla_fwd_impl(q, cache, wk=None, wv=None, rng_seed=None, b_data=None, q_id=None, k_id=None, dropout_mask=None, *,
                 kv_lengths=None, return_residuals=False, **static):
    """``impl`` for the ``mla_fwd`` / ``mla_fwd_absorbed`` specs (kernels/latent_attention.py:204-244)."""
    import jax
    import jax.numpy as jnp

    register()
    B, Lq, H, Dqk = q.shape
    S, R = cache.shape[1], cache.shape[2]
    Dv = R if wv is None else wv.shape[1]
    code = {jnp.dtype("float32"): 0, jnp.dtype("bfloat16"): 1, jnp.dtype("float16"): 2}[jnp.dtype(q.dtype)]
    ws = int(_lib.lib().pjx_mla_workspace_bytes(B, S, H, Dqk, Dv, R, code, int(wk is not None)))
    z = _absent(q.dtype)
    out_types = (jax.ShapeDtypeStruct((B, Lq, H, Dv), q.dtype),
                 jax.ShapeDtypeStruct((B, H, Lq) if return_residuals else (0,), jnp.float32),
                 jax.ShapeDtypeStruct((ws,), jnp.uint8), jax.ShapeDtypeStruct((0,), jnp.int32))
    o, lse, _, _ = jax.ffi.ffi_call("pjx_ffi_mla_fwd", out_types)(
        q, cache, z if wk is None else wk, z if wv is None else wv,
        _absent(jnp.int32) if kv_lengths is None else kv_lengths.astype(jnp.int32).reshape(-1),
        _absent(jnp.float32) if b_data is None else b_data.astype(jnp.float32),
        sm_scale=float(static.get("sm_scale", Dqk ** -0.5)), causal=bool(static.get("causal", False)))
    return (o, lse) if return_residuals else o


def kv_cache_append(k_cache, v_cache, k_new, v_new, positions, *, advance=True):
    """The decode branch's cache update (layers/attention.py:631-643) as one custom call; caches and
    positions are donated and updated in place (``input_output_aliases``)."""
    import jax

    register()
    out_types = (jax.ShapeDtypeStruct(k_cache.shape, k_cache.dtype), jax.ShapeDtypeStruct(v_cache.shape, v_cache.dtype),
                 jax.ShapeDtypeStruct(positions.shape, positions.dtype))
    return jax.ffi.ffi_call("pjx_ffi_kv_cache_append", out_types, input_output_aliases={0: 0, 1: 1, 4: 2})(
        k_cache, v_cache, k_new, v_new, positions, advance=bool(advance))
