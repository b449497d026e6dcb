"""B200-native RG-LRU hot path (hand-written sm_100a CUDA kernels behind a C ABI).

Public surface mirrors the reference's modules for this path:
``RG_LRU``, ``RecurrentBlock``, ``BlockDiagonalLinear``, ``RecurrentBlockCache``
plus the operator-level entry points in :mod:`griffin_b200.ops`.
"""

from .modules import BlockDiagonalLinear, RG_LRU, RecurrentBlock, RecurrentBlockCache, token_flags
from .ops import causal_conv, decode_conv, decode_step, linear_scan, rglru, rglru_grouped, rglru_merged
from ._lib import check_device
from .selfcheck import cuda_scan_is_usable

__all__ = [
    "BlockDiagonalLinear", "RG_LRU", "RecurrentBlock", "RecurrentBlockCache", "token_flags",
    "causal_conv", "decode_conv", "decode_step", "linear_scan", "rglru", "rglru_grouped", "rglru_merged",
    "cuda_scan_is_usable", "check_device",
]
