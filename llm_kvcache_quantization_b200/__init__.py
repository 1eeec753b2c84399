"""B200-native quantized KV-cache decode path.

Public surface (names follow the reference project):
  kernels:  decode_attn_int8, decode_attn_int4 (+ decode_attn_fp16, decode_attn_int4_asym,
            decode_attn_int4_outlier)
  caches:   INT8KVCache, INT4KVCache, FP16KVCache
  quant:    quantize_symmetric_int8[_with_scale], quantize_symmetric_int4[_with_scale],
            quantize_asymmetric_groupwise, pack_int4, unpack_int4, dequantize_*

All compute runs in libkvq.so (CUDA, sm_100a).  There is no CPU fallback: the
entry points raise if the library is missing or a tensor is not on a CUDA device.
"""
import os as _os

# The sequence-sharded exchange kernel moves data with plain peer stores; torch's symmetric-memory buffers must not
# be bound to an NVLink multicast object.  Set before anything touches symmetric memory.
_os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"

from .cache import FP16KVCache, INT4KVCache, INT8KVCache  # noqa: E402
from .kivi import KIVIStyleKVCache, RoleAwareAsymKVCache
from .kernels import (decode_attn_fp16, decode_attn_int4, decode_attn_int4_asym,
                      decode_attn_int4_outlier, decode_attn_int8)
from .quant import (dequantize_asymmetric_groupwise, dequantize_symmetric_int4,
                    dequantize_symmetric_int8, pack_int4, quantize_asymmetric_groupwise,
                    quantize_symmetric_int4, quantize_symmetric_int4_with_scale,
                    quantize_symmetric_int8, quantize_symmetric_int8_with_scale, unpack_int4)

__all__ = [
    "FP16KVCache", "INT4KVCache", "INT8KVCache", "KIVIStyleKVCache", "RoleAwareAsymKVCache",
    "decode_attn_fp16", "decode_attn_int4", "decode_attn_int4_asym", "decode_attn_int4_outlier",
    "decode_attn_int8",
    "dequantize_asymmetric_groupwise", "dequantize_symmetric_int4", "dequantize_symmetric_int8",
    "pack_int4", "quantize_asymmetric_groupwise", "quantize_symmetric_int4",
    "quantize_symmetric_int4_with_scale", "quantize_symmetric_int8",
    "quantize_symmetric_int8_with_scale", "unpack_int4",
]
