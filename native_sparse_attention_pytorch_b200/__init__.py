"""B200-native Native Sparse Attention hot path (sm_100a CUDA kernels behind a C ABI)."""
from . import ops
from .native_sparse_attention import SparseAttention
from .norm import RMSNorm, rms_norm
from .ops import (
    native_sparse_attend,
    block_diagonal_attend,
    compressed_attend,
    select_blocks,
    sliding_window_attend,
    gated_combine,
)

__all__ = ['SparseAttention', 'RMSNorm', 'rms_norm', 'native_sparse_attend', 'block_diagonal_attend', 'compressed_attend',
           'select_blocks', 'sliding_window_attend', 'gated_combine']
