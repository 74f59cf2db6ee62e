"""B200-native (sm_100a) implementation of probjax.nn's attention forward path.

Public names mirror the reference: ``dot_product_attention``, ``flex_attention``,
``mha``, ``splitkv_forward``, ``mla``, the mask / bias objects and the GPU dispatch
route.  All computation happens in ``libpjx_attention.so`` (hand-written CUDA);
build it with ``python -m probjax_b200.build``.
"""

from .attention import (  # noqa: F401
    attention_backward,
    attention_forward,
    attention_jvp,
    check_status,
    combine_partials,
    decode_forward,
    dot_product_attention,
    flex_attention,
    mha,
    mha_flash,
    mla,
    mla_decode,
    rng_seed_from_key,
    splitkv_forward,
    use_splitkv,
)
from .cache import DecodeCache, decode_paged, linear, rope_interleaved  # noqa: F401
from .latent_layer import MultiHeadLatentAttention, per_head_linear, rms_norm  # noqa: F401
from .dispatch import b200_attention_or_none, device_attention_defaults  # noqa: F401
from .masks import (  # noqa: F401
    AttentionBias,
    AttentionMask,
    BatchedLowRankBias,
    BlockDiagonalCausalMask,
    BlockDiagonalMask,
    CausalAlibiBias,
    CausalFromBottomRightMask,
    CausalLocalWindowMask,
    CausalMask,
    ComposeMask,
    ConstantBias,
    DenseBias,
    DistanceDecayBias,
    IdentityBias,
    KeyPaddingMask,
    KVLenMask,
    LearnedAlibiBias,
    LearnedRelativePositionBias,
    LocalWindowMask,
    LowRankBias,
    MarginalizationMask,
    NoMask,
    NotMask,
    PerHeadScaleBias,
    PrefixLMMask,
    QKVLengthMask,
    SameSegmentMask,
    SeqLenMask,
    SoftCappingBias,
    SumBias,
    SymmetricAlibiBias,
    T5RelativePositionBias,
)

__version__ = "0.1.0"
