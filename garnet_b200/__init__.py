"""B200 (sm_100a) implementation of Garnet's quantized-matmul hot path.

The product is `lib/libgarnet_b200.so` (C ABI in include/garnet_b200.h); this
package is the thin host-side mirror of the reference's operator interface
used by tests and benchmarks."""
from ._lib import GarnetB200Error, lib  # noqa: F401
from .linear import GlueList, HostBatch, LinearList, W4A16Linear, forward_group, pack_host, packed_bytes, quantize_int4  # noqa: F401
from .moe import GptOssMoe, MoeOptions, mxfp4_decode  # noqa: F401

__all__ = ["GarnetB200Error", "lib", "W4A16Linear", "pack_host", "packed_bytes", "quantize_int4", "forward_group", "HostBatch", "LinearList", "GlueList", "GptOssMoe",
           "MoeOptions", "mxfp4_decode"]
