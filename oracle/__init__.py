"""CPU restatement of probjax's XLA (CPU) attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this directory: it exists so that the
CUDA kernels can be checked against the reference's arithmetic and so that the
benchmark can time a CPU baseline next to them.  Only the test-suite, the
repository's smoke check and the benchmark's CPU leg use it.

Pinning status: the reference itself needs jax/flax, which are not available
offline, so it cannot be executed to produce vectors.  The restatement is
instead pinned against the known-answer *formulas* the reference's own tests
use for this path (dense fp32 softmax with ``repeat`` GQA semantics, natural-log
``logsumexp``, the mask truth tables, zero output for rows without a valid key;
see ``tests/test_oracle_pins.py`` for the file:line of each).
"""

from .attention_oracle import (  # noqa: F401
    dense_formula,
    xla_attention,
    splitkv_reference,
    combine_partials,
    mla_reference,
    materialize_kv,
    rope_interleaved,
    auto_strategy,
    counter_dropout_scale,
    rng_seed_from_key,
)
from .inputs import make_config  # noqa: F401
