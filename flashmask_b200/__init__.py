"""flashmask_b200 — FlashMask attention for NVIDIA B200 (sm_100a).

Hand-written CUDA kernels behind a C ABI (``libflashmask_b200.so``); this
package is the thin PyTorch host that mirrors the reference operator surface.
"""
from .interface import FlashMaskFunc, flashmask_attention, sliding_window_indices  # noqa: F401
from .ops import (FlashMaskInfo, _flash_attn_bwd, _flash_attn_fwd, bwd_tile_shape,  # noqa: F401
                  count_visible, fwd_tile_shape, prepare_mask)

__version__ = "0.1.0"
