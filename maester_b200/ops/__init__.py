"""Hot ops: native sm_100a kernels for bf16 CUDA tensors, plain-PyTorch definitions elsewhere."""
from maester_b200.ops.functional import (  # noqa: F401
    attention_block,
    embedding,
    glu,
    glu_mlp,
    kv_block_lower_bounds,
    linear,
    linear_cross_entropy,
    loss_backward_scale,
    rmsnorm,
    rmsnorm_fork,
    rope_table,
    use_native,
)
