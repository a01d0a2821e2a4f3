"""Device queries: architecture whitelist, capability descriptor, current-device helpers.

Mirrors the reference's device layer for this path (src/foscar/_utils.py:58-179), narrowed to
the one architecture this library is built for: B200, compute capability 10.0 ("sm100").
"""
from __future__ import annotations

import contextlib
import functools
from typing import Optional

import torch

from .pool_format import HEAD_DIMS, PAGE_SIZE, QUANT_BITS

#: Compute capabilities a decode kernel exists for, by the architecture name every API reports.
ARCH_OF_CC = {(10, 0): "sm100"}


@functools.cache
def _cc(index: int) -> tuple:
    return tuple(torch.cuda.get_device_capability(index))


def cuda_index(device=None) -> int:
    """The CUDA ordinal of `device`; None or an index-less CUDA device is the current device."""
    spec = None if device is None else torch.device(device)
    if spec is not None and spec.type != "cuda":
        raise ValueError(f"{spec} is not a CUDA device")
    if spec is None or spec.index is None:
        return torch.cuda.current_device()
    return spec.index


def device_arch(device=None) -> Optional[str]:
    return ARCH_OF_CC.get(_cc(cuda_index(device)))


def require_arch(device=None) -> str:
    """The architecture name of `device`; RuntimeError for a device without a decode kernel."""
    arch = device_arch(device)
    if arch is None:
        major, minor = _cc(cuda_index(device))
        raise RuntimeError(
            f"foscar_b200 has no kernel for compute capability {major}.{minor}; it runs on "
            f"sm100 (compute capability 10.0, B200)")
    return arch


def sm_count(device=None) -> int:
    return torch.cuda.get_device_properties(cuda_index(device)).multi_processor_count


def on_device(device):
    """Context making `device` current (launches bind the current device's stream)."""
    wanted = cuda_index(device)
    already = torch.cuda.current_device() == wanted
    return contextlib.nullcontext() if already else torch.cuda.device(wanted)


def current_stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(cuda_index(device)).cuda_stream


def is_supported(device=None) -> bool:
    if not torch.cuda.is_available():
        return False
    return device_arch(device) is not None


def get_capabilities(device=None) -> dict:
    """Static capability descriptor; every key is always present
    (src/foscar/_utils.py:133-179)."""
    ok = is_supported(device)
    return {
        "arch": "sm100" if ok else "unsupported",
        "paged": ok,
        "dtypes": ["float8_e4m3fn"] if ok else [],
        "head_dims": ",".join(str(d) for d in HEAD_DIMS) if ok else "",
        "page_sizes": [PAGE_SIZE] if ok else [],
        "reductions": ["none", "kernel"] if ok else [],
        "speculative": False,
        "atomic_reduction": False,
        "skip_softmax": False,
        "kv_layouts": ["QuantKVLayout"] if ok else [],
        "quantized_bits": list(QUANT_BITS) if ok else [],
        "quantized_validated": ok,
        "quantized_page_sizes": [PAGE_SIZE] if ok else [],
    }
