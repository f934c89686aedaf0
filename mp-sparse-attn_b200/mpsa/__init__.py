"""B200-native kernels for diagonal-tiled mixed-precision (MXFP) attention.

`mpsa.ops` holds the tensor-level operations (torch tensors in, torch tensors out, CUDA work
done by libmpsa.so through its C-ABI); the `ours` package beside this one mirrors the
reference project's module and function names on top of them.
"""
from . import _lib  # noqa: F401
from . import kvstore  # noqa: F401
from .ops import (  # noqa: F401
    TILE_SKIP, TILE_FP8, TILE_FP4, QuantizedOperand, QuantizedV, quantize_mx, column_mean, quantize_v_seq, quantize_nvfp4, quantize_nvfp4_bh, quantize_qk, quantize_int8, prepare_vt,
    precision_map_band, router_statistic, precision_map_online, prepare_kv, attention_forward, attention_forward_quantized, attention_forward_routed, attention_forward_host, attention_merge, diagonal_tiled_attention, gemm_block_scaled, gemm_block_scaled_batched, check_status,
)
