"""The latent-attention layer's steps around the attention call, on the device kernels.

Host-side mirror of ``MultiHeadLatentAttention`` (probjax/nn/layers/latent_attention.py:112-709)
for inference: the latent encoder ``wkv_a`` followed by an RMS norm (encode_latent, 424-438), the
query projection (455-457), attention over the shared latent -- ``K = V = C`` in ``absorbed`` mode,
per-head up-projections ``wk`` / ``wv`` in ``materialized`` mode -- the value projection folded onto
the absorbed output (``einsum("...qhr,hdr->...qhd")``, 468-474) and the output projection.

Every step is a kernel of ``libpjx_attention.so``: ``pjx_linear`` (projections), ``pjx_rms_norm``,
``pjx_mla_fwd_mod`` (attention, with the same mask / bias objects as ``mha``) and one
``pjx_linear_strided`` call per head for the value fold, which reads the ``[.., H, R]`` attention
output in place.  Weights are torch tensors in the ``[out, in]`` layout of ``pjx_linear``; the
module's attention dropout follows the reference's resolution rules (``dropout_rate`` /
``deterministic`` / ``keep_rngs`` at construction, ``deterministic`` / ``rng`` per call, 600-632) with a
counter of its own standing in for the kept ``nnx`` dropout stream; there is no parameter
initialisation policy beyond a seeded normal draw for tests.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from .attention import _DTYPES, _IMPL, _ptr, _require_gpu, _status_word, _stream, mla
from .cache import linear

MODES = ("absorbed", "materialized")


def rms_norm(x: torch.Tensor, scale: torch.Tensor | None = None, *, eps: float = 1e-6, out: torch.Tensor | None = None):
    """``x * rsqrt(mean(x^2, -1) + eps) * scale`` on the device (``pjx_rms_norm``), float32 arithmetic,
    result in ``x.dtype``: the ``nnx.RMSNorm`` the layer applies to the encoded latent."""
    _require_gpu()
    if not x.is_cuda or x.dtype not in _DTYPES:
        raise ValueError("rms_norm takes a CUDA tensor of dtype float32, bfloat16 or float16")
    x = x.contiguous()
    width = x.shape[-1]
    rows = x.numel() // max(width, 1)
    y = torch.empty_like(x) if out is None else out
    if tuple(y.shape) != tuple(x.shape) or y.dtype != x.dtype or not y.is_contiguous():
        raise ValueError("rms_norm: out must match x")
    sc = None
    if scale is not None:
        sc = scale.to(device=x.device, dtype=torch.float32).contiguous()
        if sc.numel() != width:
            raise ValueError(f"rms_norm: scale must hold {width} entries, got {sc.numel()}")
    with torch.cuda.device(x.device):
        rc = _lib.lib().pjx_rms_norm(_ptr(x), _ptr(sc), _ptr(y), rows, width, float(eps), _DTYPES[x.dtype], _stream(x.device))
    _lib.check(rc)
    return y


def per_head_linear(x: torch.Tensor, weight: torch.Tensor, *, implementation: str | None = None) -> torch.Tensor:
    """``einsum("...hk,hnk->...hn")``: head ``h`` of ``x [..., H, K]`` times ``weight[h] [N, K]^T``, one
    ``pjx_linear_strided`` call per head on the tensor in place (no gather, no transpose)."""
    _require_gpu()
    if not x.is_cuda or x.dtype != weight.dtype or weight.dim() != 3 or x.shape[-2:] != (weight.shape[0], weight.shape[2]):
        raise ValueError("per_head_linear takes x [..., H, K] and weight [H, N, K] of one dtype on the GPU")
    if implementation not in _IMPL:
        raise ValueError(f"implementation must be None or one of {sorted(k for k in _IMPL if k)}")
    x = x.contiguous()
    w = weight.to(x.device).contiguous()
    H, N, K = w.shape
    M = x.numel() // (H * K)
    y = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=x.dtype, device=x.device)
    es = x.element_size()
    L = _lib.lib()
    with torch.cuda.device(x.device):
        for h in range(H):
            rc = L.pjx_linear_strided(x.data_ptr() + h * K * es, H * K, w.data_ptr() + h * N * K * es,
                                      y.data_ptr() + h * N * es, H * N, M, N, K, _DTYPES[x.dtype],
                                      _IMPL[implementation], _ptr(_status_word(x.device)), _stream(x.device))
            _lib.check(rc)
    return y


class MultiHeadLatentAttention:
    """Inference-time ``MultiHeadLatentAttention`` (layers/latent_attention.py:112-395 for the
    arguments and their checks).  ``__call__(inputs_q, inputs_kv=None, *, mask=None, bias=None)``
    returns ``[..., Q, out_features]``; ``encode_latent`` gives the cache entry ``[..., S, R]``."""

    def __init__(self, num_heads: int, in_features: int, *, kv_lora_rank: int, mode: str = "absorbed",
                 out_features: int | None = None, in_kv_features: int | None = None, qk_head_dim: int | None = None,
                 v_head_dim: int | None = None, latent_norm: bool = True, kv_encoder: bool = True,
                 value_projection: bool = True, eps: float = 1e-6, dtype=torch.bfloat16, device=None, seed: int = 0,
                 dropout_rate: float = 0.0, deterministic: bool | None = None, keep_rngs: bool = True):
        if mode not in MODES:
            raise ValueError(f"mode must be one of {MODES}, got {mode!r}")
        if num_heads <= 0 or kv_lora_rank <= 0:
            raise ValueError("num_heads and kv_lora_rank must be positive")
        if not 0.0 <= dropout_rate < 1.0:
            raise ValueError(f"dropout_rate must be in [0, 1), got {dropout_rate}; "
                             "a rate of 1 or more zeroes the output and a negative rate "
                             "biases it")
        self.dropout_rate, self.deterministic = float(dropout_rate), deterministic
        # the kept dropout stream: (seed, call counter) words folded into the kernels' 32-bit seed
        self._kept_stream = [int(seed) & 0xFFFFFFFF, 0] if keep_rngs and self.dropout_rate > 0.0 else None
        if not value_projection and mode != "absorbed":
            raise ValueError("value_projection=False is only supported in absorbed mode "
                             "(K = V = C); materialized mode needs wv to form values")
        self.num_heads, self.in_features = int(num_heads), int(in_features)
        self.in_kv_features = int(in_kv_features or in_features)
        self.kv_lora_rank, self.mode = int(kv_lora_rank), mode
        self.out_features = int(out_features or in_features)
        self.kv_encoder, self.value_projection, self.eps = bool(kv_encoder), bool(value_projection), float(eps)
        if mode == "materialized":
            self.qk_head_dim = int(qk_head_dim or self.in_features // num_heads)
        else:
            if qk_head_dim is not None and int(qk_head_dim) != self.kv_lora_rank:
                raise ValueError(
                    "absorbed mode (K = V = C) requires qk_head_dim == "
                    f"kv_lora_rank, got qk_head_dim={qk_head_dim} and kv_lora_rank={self.kv_lora_rank}; use "
                    "mode='materialized' to learn a per-head K/V projection, or set qk_head_dim=kv_lora_rank")
            self.qk_head_dim = self.kv_lora_rank
        self.v_head_dim = int(v_head_dim if v_head_dim is not None
                              else (self.qk_head_dim if mode == "materialized" else self.kv_lora_rank))
        if not self.value_projection and self.v_head_dim != self.kv_lora_rank:
            raise ValueError(
                "value_projection=False leaves the attention output at "
                f"kv_lora_rank={self.kv_lora_rank}, so v_head_dim must equal it; got v_head_dim={self.v_head_dim}.  "
                "Keep the value projection to use a different v_head_dim")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        g = torch.Generator().manual_seed(seed)

        def init(*shape, fan_in):
            return (torch.randn(*shape, generator=g) / math.sqrt(fan_in)).to(dtype).to(dev)

        H, R = self.num_heads, self.kv_lora_rank
        self.wkv_a = init(R, self.in_kv_features, fan_in=self.in_kv_features) if self.kv_encoder else None
        self.latent_norm_scale = torch.ones(R, dtype=torch.float32, device=dev) if (self.kv_encoder and latent_norm) else None
        self.wq = init(H * self.qk_head_dim, self.in_features, fan_in=self.in_features)
        self.wk = init(H, self.qk_head_dim, R, fan_in=R) if mode == "materialized" else None
        has_wv = mode == "materialized" or self.value_projection
        self.wv = init(H, self.v_head_dim, R, fan_in=R) if has_wv else None
        self.wo = init(self.out_features, H * self.v_head_dim, fan_in=H * self.v_head_dim)

    def encode_latent(self, inputs_kv: torch.Tensor) -> torch.Tensor:
        """``H -> C``: the single entry written to the cache, ``[..., S, R]`` (424-438)."""
        if self.wkv_a is None:
            raise RuntimeError("encode_latent is unavailable when kv_encoder=False; this layer "
                               "expects a precomputed bank passed as its `inputs_kv` argument.")
        latent = linear(inputs_kv, self.wkv_a)
        if self.latent_norm_scale is not None:
            latent = rms_norm(latent, self.latent_norm_scale, eps=self.eps, out=latent)
        return latent

    def _resolve_dropout(self, deterministic, rng):
        """(rate, rng) of one call (latent_attention.py:604-632)."""
        if self.dropout_rate == 0.0:
            return 0.0, None
        deterministic = deterministic if deterministic is not None else self.deterministic
        if deterministic is None:
            raise ValueError("No `deterministic` argument was provided to "
                             "MultiHeadLatentAttention as either a __call__ argument, "
                             "class attribute, or nnx.flag.")
        if deterministic:
            return 0.0, None
        if rng is not None:
            return self.dropout_rate, rng
        if self._kept_stream is not None:
            self._kept_stream[1] += 1
            return self.dropout_rate, list(self._kept_stream)
        raise ValueError("'rng'/'rngs' must be provided to __call__, or the layer "
                         "built with keep_rngs=True, when dropout is enabled")

    def __call__(self, inputs_q: torch.Tensor, inputs_kv: torch.Tensor | None = None, *, mask=None, bias=None,
                 sm_scale: float | None = None, deterministic: bool | None = None, rng=None) -> torch.Tensor:
        drop_rate, drop_rng = self._resolve_dropout(deterministic, rng)
        inputs_kv = inputs_q if inputs_kv is None else inputs_kv
        latent = self.encode_latent(inputs_kv) if self.kv_encoder else inputs_kv
        lead = inputs_q.shape[:-2]
        q = linear(inputs_q, self.wq).reshape(-1, inputs_q.shape[-2], self.num_heads, self.qk_head_dim)
        lat3 = latent.reshape(-1, latent.shape[-2], self.kv_lora_rank)
        scale = 1.0 / math.sqrt(self.qk_head_dim) if sm_scale is None else float(sm_scale)
        if self.mode == "materialized":
            attn = mla(q, lat3, self.wk, self.wv, mask=mask, bias=bias, sm_scale=scale, rng=drop_rng,
                       dropout_rate=drop_rate)
        else:
            attn = mla(q, lat3, mask=mask, bias=bias, sm_scale=scale, rng=drop_rng, dropout_rate=drop_rate)  # [B, Q, H, R]
            if self.wv is not None:  # fold W_V in, then the shared output projection (468-474)
                attn = per_head_linear(attn, self.wv)
        out = linear(attn.reshape(attn.shape[0], attn.shape[1], self.num_heads * self.v_head_dim), self.wo)
        return out.reshape(tuple(lead) + (inputs_q.shape[-2], self.out_features))
