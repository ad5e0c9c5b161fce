"""B200-native (sm_100a) fused linear-cross-entropy: a drop-in for the reference's
``tritium.linear_cross_entropy`` / ``tritium.linear_cross_entropy_backward``.

Importing this package needs no GPU; calling an op needs libhelion_lce.so (built in-tree by
``helion_b200.build``) and an sm_100 device. There is no CPU or torch fallback.
"""

from .ce_ops import cross_entropy, cross_entropy_backward
from .decode_ops import greedy_head, sample_head, topk_head
from .install import install, uninstall
from .matmul_ops import matmul, matmul_vec
from .norm_ops import residual_rmsnorm, rmsnorm, rmsnorm_backward
from .optim_ops import adamw_step, clip_grad_norm, grad_sumsq
from .ops import linear_cross_entropy, linear_cross_entropy_backward

__all__ = [
    "adamw_step",
    "clip_grad_norm",
    "cross_entropy",
    "cross_entropy_backward",
    "grad_sumsq",
    "greedy_head",
    "install",
    "linear_cross_entropy",
    "linear_cross_entropy_backward",
    "matmul",
    "matmul_vec",
    "residual_rmsnorm",
    "rmsnorm",
    "rmsnorm_backward",
    "sample_head",
    "topk_head",
    "uninstall",
]
