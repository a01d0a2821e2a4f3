"""Import alias: `import foscar` resolves to the B200-native implementation, so code written
against FOSCAR's public names runs unchanged."""
from foscar_b200 import (PagedDecodeWrapper, QuantKVCache, QuantKVLayout, __version__,  # noqa
                         get_capabilities, graph_workspace_bytes, is_supported)

__all__ = ["PagedDecodeWrapper", "QuantKVCache", "QuantKVLayout", "get_capabilities",
           "is_supported", "graph_workspace_bytes", "__version__"]
