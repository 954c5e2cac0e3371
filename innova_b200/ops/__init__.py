"""Operators. CUDA tensors run the hand-written sm_100a kernels; CPU tensors run plain PyTorch."""
from .gemm import gemm, linear, mlp_gelu, EPI_NONE, EPI_GELU, EPI_DGELU, EPI_ADD, EPI_ATOMIC, EPI_GELU_DG, EPI_MUL  # noqa: F401
from .functional import (layer_norm, rms_norm, norm_residual, embedding, gelu, swiglu, rope_tables, rope_qk, cross_entropy,  # noqa: F401
                         lm_head_cross_entropy)
from .attention import flash_attention, attention_reference  # noqa: F401
from .mea import MEAConfig, MemoryEfficientAttention  # noqa: F401
from .runtime import check_status, status_tensor  # noqa: F401
