"""ctypes binding of ``libpjx_attention.so`` (the C ABI in ``include/pjx_attention.h``).

There is no fallback: if the shared library is missing or fails to load,
:func:`lib` raises, and every attention call in this package raises with it.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# PJX_ATTENTION_LIB points at another build of the same library (e.g. a debug build).
LIB_PATH = Path(os.environ.get("PJX_ATTENTION_LIB", _PKG / "libpjx_attention.so"))

PJX_OK, PJX_ERR_BAD_ARG, PJX_ERR_UNSUPPORTED, PJX_ERR_WORKSPACE, PJX_ERR_DEVICE_TIMEOUT, PJX_ERR_CUDA = range(6)
PJX_F32, PJX_BF16, PJX_F16 = 0, 1, 2
IMPL_AUTO, IMPL_GENERIC, IMPL_SM100 = 0, 1, 2

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

class ScoreMod(C.Structure):
    """``pjx_score_mod`` of the header, field by field."""

    _fields_ = [
        ("seg_q", _vp), ("seg_k", _vp), ("seg_q_batch_stride", _i64), ("seg_k_batch_stride", _i64),
        ("row_kv_limit", _vp), ("row_kv_limit_batch_stride", _i64),
        ("prefix_len", _vp),
        ("rel_bias", _vp), ("rel_bias_head_stride", _i64),
        ("alibi_slopes", _vp), ("alibi_mode", C.c_int32),
        ("head_scale", _vp),
        ("softcap", _f),
        ("dropout_rate", _f),
        ("dropout_seed", C.c_uint32),
    ]


_modp = C.POINTER(ScoreMod)

# name -> (restype, argtypes); mirrors include/pjx_attention.h declaration by declaration.
SIGNATURES = {
    "pjx_version": (_i, []),
    "pjx_status_string": (C.c_char_p, [_i]),
    "pjx_last_error": (C.c_char_p, []),
    "pjx_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                          _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp]),
    "pjx_attn_fwd_band": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                               _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp]),
    "pjx_attn_fwd_mod": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                              _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _modp, _i, _vp, _vp]),
    "pjx_attn_bwd_mod": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp,
                              _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _modp, _i, _vp, _sz, _vp, _vp]),
    "pjx_attn_jvp_mod": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                              _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _modp, _vp]),
    "pjx_mla_fwd_mod": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                             _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _modp, _i, _vp, _sz, _vp, _vp]),
    "pjx_attn_bwd_band": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp,
                               _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp, _vp]),
    "pjx_attn_jvp_band": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                               _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "pjx_attn_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                          _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "pjx_attn_bwd_workspace_bytes": (_sz, [_i, _i, _i]),
    "pjx_attn_decode_splitkv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f,
                                     _i, _i, _vp, _sz, _vp]),
    "pjx_attn_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i]),
    "pjx_attn_decode_default_split_len": (_i, [_i, _i, _i]),
    "pjx_attn_decode_splitkv_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp]),
    "pjx_attn_decode_static_scratch_bytes": (_sz, []),
    "pjx_attn_decode_sharded": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _sz,
                                     _i, _i, _vp, C.c_uint32, _i, _vp, _vp]),
    "pjx_attn_decode_sharded_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i,
                                           _vp, _sz, _i, _i, _vp, C.c_uint32, _i, _vp, _vp]),
    "pjx_attn_decode_sharded_buffer_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "pjx_linear": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp]),
    "pjx_linear_strided": (_i, [_vp, _i64, _vp, _vp, _i64, _i64, _i, _i, _i, _i, _vp, _vp]),
    "pjx_rms_norm": (_i, [_vp, _vp, _vp, _i64, _i, _f, _i, _vp]),
    "pjx_rope_interleaved": (_i, [_vp, _vp, _vp, _f, _i64, _i, _i, _i, _i, _f, _i, _vp]),
    "pjx_attn_decode_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i,
                                   _vp, _sz, _vp]),
    "pjx_kv_cache_append": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "pjx_attn_combine": (_i, [_vp, _vp, _i, _i64, _i, _vp, _vp, _i, _vp]),
    "pjx_mla_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                         _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp, _vp]),
    "pjx_mla_decode_absorbed": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "pjx_mla_decode_absorbed_impl": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _sz, _vp, _vp]),
    "pjx_mla_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "pjx_mla_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i, _i]),
    "pjx_attn_fwd_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                               _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "pjx_attn_fwd_host_staging_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i]),
    "pjx_read_status": (_i, [_vp, _vp]),
    "pjx_launch_count": (_i64, []),
}

_lib = None


class KernelTimeout(RuntimeError):
    """A bounded wait inside a kernel expired (the device stays usable)."""


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m probjax_b200.build` "
                "(nvcc, sm_100a). This package has no other execution path."
            )
        handle = C.CDLL(os.fspath(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().pjx_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Turn a pjx_status into the exception the reference raises for that case."""
    if rc == PJX_OK:
        return
    msg = last_error() or lib().pjx_status_string(rc).decode()
    if rc == PJX_ERR_BAD_ARG:
        raise ValueError(msg)
    if rc == PJX_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    if rc == PJX_ERR_DEVICE_TIMEOUT:
        raise KernelTimeout(msg)
    raise RuntimeError(f"pjx status {rc}: {msg}")


def launch_count() -> int:
    return int(lib().pjx_launch_count())
