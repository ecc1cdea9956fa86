"""Splash (block-sparse flash) attention for NVIDIA B200 in hand-written sm_100a CUDA.

Same import surface as the reference package (`splash_attention_mgpu/__init__.py:4-21`).
"""

from .config import DEFAULT_MASK_VALUE, BlockSizes, SegmentIds
from .mask_info import GpuMaskInfo, process_mask
from .splash_attention import (
    SplashAttentionKernel,
    attention_reference,
    check_device_status,
    make_splash_mha,
    make_splash_mqa,
)
from .splash_attention_mask import (
    CausalMask,
    ChunkedCausalMask,
    FullMask,
    LocalMask,
    Mask,
    MultiHeadMask,
    NumpyMask,
)

__all__ = [
    "BlockSizes", "CausalMask", "ChunkedCausalMask", "DEFAULT_MASK_VALUE",
    "FullMask", "GpuMaskInfo", "LocalMask", "Mask", "MultiHeadMask",
    "NumpyMask", "SegmentIds", "SplashAttentionKernel", "attention_reference",
    "check_device_status", "make_splash_mha", "make_splash_mqa", "process_mask",
]
