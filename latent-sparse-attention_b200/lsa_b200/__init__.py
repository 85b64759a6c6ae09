"""lsa_b200 - Latent Sparse Attention's selection-plus-attention path on B200 (sm_100a).

`lsa_b200.core` keeps the operator API of the reference's `lsa.core` (latent key/query map, pooling, bucketing,
flat and tree search, sparse attend); `lsa_b200.ops` are the tensor-level kernel wrappers underneath;
`lsa_b200.layer` strings them into one attention layer's prefill and decode. Everything runs in the hand-written
CUDA kernels of `liblsa_b200.so`; there is no CPU or library fallback.
"""

from lsa_b200.budget import EarlyBudget, budget_at  # noqa: F401

__version__ = "0.1.0"
