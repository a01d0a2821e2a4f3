"""B200-native paged GQA decode attention over packed INT2/INT4 KV caches.

Drop-in for the decode path of FOSCAR's Python API: `QuantKVLayout.create/allocate/bind`,
`QuantKVCache.append/append_quantized/dequantize/recount_v_max`, `get_capabilities`,
`is_supported`, `PagedDecodeWrapper(workspace).plan/run` (eager and CUDA-graph mode) and
`graph_workspace_bytes`. All compute is hand-written sm_100a CUDA behind a C ABI
(include/foscar_b200.h); there is no CPU or PyTorch fallback.
"""
from .device import get_capabilities, is_supported
from .kv_cache import QuantKVCache, QuantKVLayout
from .wrapper import PagedDecodeWrapper, graph_workspace_bytes

__version__ = "0.1.0"

__all__ = ["PagedDecodeWrapper", "QuantKVCache", "QuantKVLayout", "get_capabilities",
           "is_supported", "graph_workspace_bytes", "__version__"]
