"""B200-native grouped dual-NVFP4 GEMM behind the nvfp4_gemm surface.

Same public names as the reference package (python/nvfp4_gemm/__init__.py:41-49).
``import nvfp4_gemm`` resolves to this package through the thin alias package of
that name at the repository root.
"""
__version__ = "0.1.0"

from . import _C, layout
from ._C import get_num_sms, m_grouped_bf16_dual_nvfp4_gemm_contiguous, set_num_sms
from ._C import m_grouped_bf16_dual_nvfp4_gemm_masked
from .layout import dequantize_weight_nvfp4, load_checkpoint_weights_nvfp4, make_m_indices, quantize_weight_nvfp4

__all__ = [
    "m_grouped_bf16_dual_nvfp4_gemm_contiguous",
    "m_grouped_bf16_dual_nvfp4_gemm_masked",
    "quantize_weight_nvfp4",
    "load_checkpoint_weights_nvfp4",
    "dequantize_weight_nvfp4",
    "make_m_indices",
    "layout",
    "get_num_sms",
    "set_num_sms",
]
