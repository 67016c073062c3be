"""Int4 storage format and the min-max quantiser used to build W4A16 layers."""
from .packing import pack_int4, unpack_int4
from .awq import _per_group_minmax_quantize, quantize_awq

__all__ = ["pack_int4", "unpack_int4", "_per_group_minmax_quantize", "quantize_awq"]
