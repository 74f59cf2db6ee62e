"""GPU dispatch seam: the per-compute-capability routing table and the route
function for Blackwell.

The reference keeps a table of defaults keyed by CUDA compute-capability major
(probjax/nn/layers/attention_device.py:38-64; only key 9 exists there) and walks
route functions ``route(q, k, v, *, mask, bias, dropout_rate, sm_scale, force)``
that return the output or ``None`` for "not mine, fall through"
(probjax/nn/layers/attention.py:1254-1263, 1564-1570); ``force=True`` turns a
``None`` into a ``ValueError`` (1537-1550).  This module adds the entry for major
10 and the route that runs the sm_100a kernels.
"""

from __future__ import annotations

import os

import torch

from . import attention as _att

# attention_device.py:23-25 style switch: PROBJAX_ATTENTION_B200=0 opts out.
_ENV = "PROBJAX_ATTENTION_B200"

# attention_device.py:55-64 has only a `9:` entry; this is the `10:` one.
DEVICE_DEFAULTS = {
    10: {
        "route": "b200",
        "dtypes": ("float32", "bfloat16", "float16"),
        "max_head_dim": 256,
        "tcgen05_head_dims": ((64, 64), (128, 128), (192, 128)),
        "splitkv_max_q_len": _att._SPLITKV_MAX_Q_LEN,
        "splitkv_min_kv_len": _att._SPLITKV_MIN_KV_LEN,
    }
}


def _compute_capability_major(device=None) -> int | None:
    if not torch.cuda.is_available():
        return None
    return torch.cuda.get_device_capability(device)[0]


def device_attention_defaults(device=None):
    """The table entry of the current device, or None (attention_device.py:84-89)."""
    if os.environ.get(_ENV, "1") == "0":
        return None
    return DEVICE_DEFAULTS.get(_compute_capability_major(device))


def b200_attention_or_none(q, k, v, *, mask=None, bias=None, dropout_rate: float = 0.0, sm_scale: float,
                           force: bool = False):
    """Route for compute capability 10: rank-4 ``[B, T, H, D]`` inputs.

    Returns the attention output when the sm_100a kernels compute this call
    exactly, else ``None`` -- or raises ``ValueError`` when ``force`` is set
    (the reference's ``implementation="cudnn"`` / ``"mosaic"`` behaviour).
    """
    reason = None
    if device_attention_defaults(q.device if isinstance(q, torch.Tensor) and q.is_cuda else None) is None:
        reason = "no sm_100 device (or disabled by PROBJAX_ATTENTION_B200=0)"
    elif dropout_rate > 0:
        reason = "active dropout"
    elif q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        reason = "inputs must be rank 4"
    elif q.shape[-1] > 256 or v.shape[-1] > 256:
        reason = "head dim above 256"
    elif q.shape[2] % k.shape[2] != 0:
        reason = "query heads not a multiple of kv heads"
    if reason is None:
        try:
            return _att.mha(q, k, v, mask=mask, bias=bias, sm_scale=sm_scale)
        except NotImplementedError as e:  # mask / bias the kernels do not implement
            reason = str(e)
    if force:
        raise ValueError(f"implementation='b200' cannot compute this call: {reason}")
    return None
