"""`QuantKVLayout` and `QuantKVCache`: one layer's quantized KV-cache layout and pools.

Host-side mirror of the reference's cache objects (src/foscar/kv_cache.py:258-877): the same
names, fields, argument meaning, pool geometry (byte-identical, region-major) and refusals.
Every operation on the pools launches a kernel of the C-ABI library on the current stream;
nothing here computes on the host.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Optional

import torch

from . import _lib, device as _dev
from .pool_format import (HEAD_DIMS, PAGE_SIZE, QUANT_BITS, VMAX_BINS, envelope_refusal,
                          normalize_pair, scale_block_sections)

#: Most tokens one `append` takes (32-bit token counters, with slack).
MAX_APPEND_TOKENS = 2**31 - 512
#: Most requests one `dequantize` takes.
MAX_DEQUANT_REQUESTS = 2**31 - 512
SCALE_DTYPES = (torch.float32, torch.bfloat16)
V_PAGE_MAX_DTYPE = torch.uint32
READER = "IntDecodeSm100"


def clip_index(ratio, head_dim: int) -> int:
    """Order-statistic index of `append`'s per-row clip, -1 for none: a ratio r in (0, 1] clamps a
    row to +-(its |x| sorted ascending)[min(int(r*D), D-1)] (src/foscar/kv_cache.py:104-118)."""
    if ratio is not None:
        numeric = isinstance(ratio, (int, float)) and not isinstance(ratio, bool)
        if not numeric or ratio <= 0.0 or ratio > 1.0:
            raise ValueError(f"a clip ratio is a number in (0, 1], or None for no clip; got "
                             f"{ratio!r}")
        return min(head_dim - 1, int(ratio * head_dim))
    return -1


def _positive_int(name, value):
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ValueError(f"{name} must be a positive int; got {value!r}")


def _resolve(arch, bits, head_dim, num_kv_heads, k_quant, v_quant, scale_dtype):
    """Every field of a layout, validated (src/foscar/kv_cache.py:136-225)."""
    if arch != "sm100":
        raise ValueError(f"arch must be 'sm100'; got {arch!r}")
    if isinstance(bits, bool) or not isinstance(bits, int) or bits not in QUANT_BITS:
        raise ValueError(f"bits must be one of {QUANT_BITS}; got {bits!r}")
    _positive_int("head_dim", head_dim)
    _positive_int("num_kv_heads", num_kv_heads)
    if head_dim not in HEAD_DIMS:
        raise ValueError(f"head_dim {head_dim} is not accepted on {arch}; the decode accepts "
                         f"{list(HEAD_DIMS)} there")
    k_quant = normalize_pair(k_quant, head_dim, "k_quant")
    v_quant = normalize_pair(v_quant, head_dim, "v_quant")
    k_sub_token = k_quant[0] == "token" and k_quant[1] < head_dim
    if scale_dtype is None:
        scale_dtype = torch.bfloat16 if k_sub_token else torch.float32
    if scale_dtype not in SCALE_DTYPES:
        raise ValueError(f"scale_dtype must be one of {SCALE_DTYPES}; got {scale_dtype!r}")
    why = envelope_refusal(k_quant, v_quant, head_dim)
    if why is not None:
        raise ValueError(f"k_quant={k_quant} v_quant={v_quant} is outside the decode's "
                         f"envelope: {why}")
    if k_sub_token and scale_dtype != torch.bfloat16:
        raise ValueError(f"k_quant={k_quant} needs a bfloat16 scale pool on Blackwell; got "
                         f"{scale_dtype}")
    return dict(arch=arch, bits=bits, head_dim=head_dim, num_kv_heads=num_kv_heads,
                k_quant=k_quant, v_quant=v_quant, scale_dtype=scale_dtype, reader=READER,
                code_pool_order=None, k_pool_permuted=True, v_pool_permuted=True)


@dataclasses.dataclass(frozen=True)
class QuantKVLayout:
    """One layer's cache layout: stored width, head dimension, KV heads, K and V granularity,
    scale dtype, and the pool orders the decode reads. Build it with `QuantKVLayout.create`;
    a hand-built instance whose fields disagree with what `create` resolves is refused."""
    arch: str
    bits: int
    head_dim: int
    num_kv_heads: int
    k_quant: tuple
    v_quant: tuple
    scale_dtype: torch.dtype
    reader: str
    code_pool_order: Optional[str]
    k_pool_permuted: Optional[bool]
    v_pool_permuted: Optional[bool]

    def __post_init__(self):
        want = _resolve(self.arch, self.bits, self.head_dim, self.num_kv_heads, self.k_quant,
                        self.v_quant, self.scale_dtype)
        mine = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        if mine != want:
            diff = {k: (mine[k], want[k]) for k in want if mine[k] != want[k]}
            raise ValueError(f"a QuantKVLayout is built by QuantKVLayout.create(); these fields "
                             f"disagree with what the reader resolves: {diff}")

    @classmethod
    def create(cls, *, bits, head_dim, num_kv_heads, k_quant=None, v_quant=None,
               scale_dtype=None, device=None) -> "QuantKVLayout":
        """The production layout for `device` (default: the current CUDA device)."""
        return cls._create(_dev.require_arch(device), bits=bits, head_dim=head_dim,
                           num_kv_heads=num_kv_heads, k_quant=k_quant, v_quant=v_quant,
                           scale_dtype=scale_dtype)

    @classmethod
    def _create(cls, arch, *, bits, head_dim, num_kv_heads, k_quant=None, v_quant=None,
                scale_dtype=None, kernel_kwargs=None) -> "QuantKVLayout":
        """`create()` for a named architecture; needs no GPU."""
        if kernel_kwargs:
            raise TypeError("kernel_kwargs is retired: this library has one build per layout")
        return cls(**_resolve(arch, bits, head_dim, num_kv_heads, k_quant, v_quant, scale_dtype))

    # -- geometry ---------------------------------------------------------------------------
    def _sections(self) -> dict:
        return scale_block_sections(self.k_quant, self.v_quant, self.head_dim)

    def _blocks(self) -> dict:
        sec = self._sections()
        row = (PAGE_SIZE, self.head_dim * self.bits // 8)
        return {"k_codes": row, "v_codes": row,
                "scales": (PAGE_SIZE, 4) if sec["legacy"] else (sec["block_tot"],),
                "v_page_max": () if self.has_v_page_max else None}

    @property
    def has_v_page_max(self) -> bool:
        """Whether the cache keeps `v_page_max` and `v_max_hist`: token-wise V."""
        return self.v_quant[0] == "token"

    @property
    def is_token_wise(self) -> bool:
        return self.k_quant[0] == "token" and self.v_quant[0] == "token"

    @property
    def is_page_channel_k(self) -> bool:
        """K per channel over the 64 tokens of a page, V per token over the whole head: the
        channel-wise layout this build writes (by whole pages), reads back and decodes."""
        return self.k_quant == ("channel", PAGE_SIZE) and self.v_quant == ("token", self.head_dim)

    def pool_dtypes(self) -> dict:
        return {"k_codes": torch.uint8, "v_codes": torch.uint8, "scales": self.scale_dtype,
                "v_page_max": V_PAGE_MAX_DTYPE if self.has_v_page_max else None}

    def pool_shapes(self, num_pages: int) -> dict:
        _positive_int("num_pages", num_pages)
        return {name: None if block is None else (num_pages, self.num_kv_heads, *block)
                for name, block in self._blocks().items()}

    def _page_bytes(self) -> dict:
        sizes, dtypes = {}, self.pool_dtypes()
        for name, block in self._blocks().items():
            if block is None:
                continue
            n = self.num_kv_heads
            for extent in block:
                n *= extent
            sizes[name] = n * dtypes[name].itemsize
        return sizes

    def bytes_per_page(self) -> int:
        """Bytes one page takes across K, V, scales and page maxima, all KV heads."""
        return sum(self._page_bytes().values())

    # -- caches -----------------------------------------------------------------------------
    def allocate(self, num_pages: int, *, device=None) -> "QuantKVCache":
        """A fresh `num_pages`-page cache on `device`, laid out and initialised as `bind` does."""
        _positive_int("num_pages", num_pages)
        index = _dev.cuda_index(device)
        buffer = torch.empty(num_pages * self.bytes_per_page(), dtype=torch.uint8,
                             device=torch.device("cuda", index))
        return self.bind(buffer, num_pages)

    def bind(self, buffer: torch.Tensor, num_pages: int) -> "QuantKVCache":
        """A cache over an engine-owned uint8 buffer, region-major `[K | V | scales | page
        maxima]`; zeroes only the page maxima (src/foscar/kv_cache.py:405-455)."""
        _positive_int("num_pages", num_pages)
        if not isinstance(buffer, torch.Tensor):
            raise TypeError(f"bind() takes a torch.Tensor; got {type(buffer).__name__}")
        need = num_pages * self.bytes_per_page()
        problems = (
            (buffer.dtype != torch.uint8, f"bind() takes a uint8 buffer; got {buffer.dtype}"),
            (not buffer.is_contiguous(), "bind() takes a C-contiguous buffer"),
            (buffer.numel() < need, f"a {num_pages}-page cache of this layout needs {need} "
                                    f"bytes; the buffer holds {buffer.numel()}"),
            (buffer.data_ptr() % 16 != 0, "bind() takes a buffer whose start is 16-byte aligned"),
        )
        for wrong, message in problems:
            if wrong:
                raise ValueError(message)
        _require_device(self, buffer.device)
        # one region per pool, in the order of _page_bytes(), each as long as its pages
        raw = buffer.reshape(-1)
        shapes, dtypes = self.pool_shapes(num_pages), self.pool_dtypes()
        views, offset = {}, 0
        for pool, per_page in self._page_bytes().items():
            length = num_pages * per_page
            chunk = raw.narrow(0, offset, length)
            offset += length
            if pool == "v_page_max":
                chunk.zero_()
            typed = chunk if dtypes[pool] == torch.uint8 else chunk.view(dtypes[pool])
            views[pool] = typed.view(shapes[pool])
        hist = None
        if "v_page_max" in views:
            hist = torch.zeros(VMAX_BINS, dtype=torch.int32, device=buffer.device)
            hist = hist.view(V_PAGE_MAX_DTYPE)
        return QuantKVCache._build(self, views["k_codes"], views["v_codes"], views["scales"],
                                   views.get("v_page_max"), hist)


def _require_device(layout, device):
    arch = _dev.require_arch(device)
    if arch != layout.arch:
        raise ValueError(f"this layout was resolved for {layout.arch}, and {device} is {arch}; "
                         f"create the layout for the device the cache lives on")


class QuantKVCache:
    """One layer's pools in global memory: `k_codes`, `v_codes`, `scales`, and with token-wise V
    `v_page_max` (uint32 [NP, HKV]) and `v_max_hist` (uint32 [256]). Built only by
    `QuantKVLayout.allocate` / `bind`. The pools are views into the engine's buffer.

    Engine contracts (src/foscar/kv_cache.py:492-510): every use of a page begins with a write at
    position 0; no decode of a layer runs concurrently with an append to it; after a raw copy
    into the buffer call `recount_v_max()`; bind once per buffer.

    Device-side faults set bits of `status` (int32 [1] on the device) instead of trapping;
    `last_status()` reads it (it waits for the device)."""

    __slots__ = ("layout", "num_pages", "device", "k_codes", "v_codes", "scales", "v_page_max",
                 "v_max_hist", "status", "_c_pools")

    def __init__(self, *args, **kwargs):
        raise TypeError("a QuantKVCache is built by QuantKVLayout.allocate() or "
                        "QuantKVLayout.bind()")

    @classmethod
    def _build(cls, layout, k_codes, v_codes, scales, v_page_max, v_max_hist) -> "QuantKVCache":
        cache = object.__new__(cls)
        fields = dict(layout=layout, num_pages=int(k_codes.shape[0]), device=k_codes.device,
                      k_codes=k_codes, v_codes=v_codes, scales=scales, v_page_max=v_page_max,
                      v_max_hist=v_max_hist,
                      status=torch.zeros(1, dtype=torch.int32, device=k_codes.device))
        for name, value in fields.items():
            setattr(cache, name, value)
        k_axis, k_group = layout.k_quant

        def address(t):
            return None if t is None else t.data_ptr()
        cache._c_pools = _lib.Pools(
            bits=layout.bits, head_dim=layout.head_dim, num_kv_heads=layout.num_kv_heads,
            k_groups=layout.head_dim // k_group if k_axis == "token" else 1,
            scale_bf16=int(layout.scale_dtype == torch.bfloat16), num_pages=cache.num_pages,
            k_channel_group=k_group if k_axis == "channel" else 0,
            k_codes=address(k_codes), v_codes=address(v_codes), scales=address(scales),
            v_page_max=address(v_page_max), v_max_hist=address(v_max_hist))
        return cache

    def last_status(self) -> int:
        """The device status word (0 = no fault). Waits for the device."""
        return int(self.status.item())

    def _refuse_channel_wise(self, method):
        lay = self.layout
        if not lay.is_token_wise:
            raise NotImplementedError(
                f"{method}() writes token-wise layouts only; k_quant={lay.k_quant} "
                f"v_quant={lay.v_quant} has a channel-wise tensor"
                + (" (write it by whole pages with append_page_groups() or "
                   "append_quantized_page_groups())"
                   if lay.is_page_channel_k else ""))

    def _check_slots(self, slot_mapping, num_tokens):
        ok = (isinstance(slot_mapping, torch.Tensor) and slot_mapping.dtype == torch.int64
              and slot_mapping.dim() == 1 and slot_mapping.shape[0] == num_tokens
              and slot_mapping.is_contiguous())
        if not ok:
            raise ValueError(f"slot_mapping must be a contiguous int64 [{num_tokens}] tensor")
        self._same_device("slot_mapping", slot_mapping)

    def _same_device(self, name, x):
        if x.device != self.device:
            raise ValueError(f"{name} is on {x.device}; the cache is on {self.device}")

    def recount_v_max(self) -> None:
        """Clear every page maximum's sign bit and rebuild `v_max_hist` from the cells, on the
        current stream; no host wait, capturable (src/foscar/kv_cache.py:595-616)."""
        if self.v_page_max is None:
            return
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_recount_vmax(ctypes.byref(self._c_pools),
                                                   _dev.current_stream_ptr(self.device)),
                       "recount_v_max")

    def _check_token_rows(self, name, x, rows=None):
        """bf16 [T, HKV, D] input rows (T = `rows` when given): each token's [HKV, D] block
        contiguous, token stride free, rows 16-byte aligned."""
        H, D = self.layout.num_kv_heads, self.layout.head_dim
        good = isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and x.dim() == 3 \
            and (x.shape[1], x.shape[2]) == (H, D) and (rows is None or x.shape[0] == rows)
        if not good:
            lead = "T" if rows is None else rows
            extra = " (64 rows per page)" if rows is not None else ""
            raise ValueError(f"{name} must be a bfloat16 [{lead}, {H}, {D}] tensor{extra}; got "
                             f"{getattr(x, 'dtype', None)} {tuple(getattr(x, 'shape', ()))}")
        self._same_device(name, x)
        token, head, channel = x.stride()
        if (head, channel) != (D, 1):
            raise ValueError(f"{name} must have a contiguous [num_kv_heads, head_dim] row per "
                             f"token (strides (*, {D}, 1)); got {tuple(x.stride())}")
        if x.data_ptr() % 16 != 0 or (token * x.element_size()) % 16 != 0:
            raise ValueError(f"every token row of {name} must start 16-byte aligned")

    def append(self, k: torch.Tensor, v: torch.Tensor, slot_mapping: torch.Tensor, *,
               k_clip=None, v_clip=None) -> None:
        """Quantize and write tokens: k, v bfloat16 [T, HKV, D] (head dimension contiguous, free
        token stride, 16-byte aligned rows); slot_mapping int64 [T], token t to page slot // 64,
        position slot % 64; a negative slot is skipped (src/foscar/kv_cache.py:618-687). A slot at
        or past num_pages * 64 is skipped and sets a status bit (the reference traps)."""
        lay = self.layout
        self._refuse_channel_wise("append")
        self._check_token_rows("k", k)
        self._check_token_rows("v", v)
        tokens = k.shape[0]
        if v.shape[0] != tokens:
            raise ValueError(f"k has {tokens} tokens and v has {v.shape[0]}")
        if tokens > MAX_APPEND_TOKENS:
            raise ValueError(f"one append takes at most {MAX_APPEND_TOKENS} tokens; got "
                             f"{tokens}: split it into several appends")
        self._check_slots(slot_mapping, k.shape[0])
        kc, vc = clip_index(k_clip, lay.head_dim), clip_index(v_clip, lay.head_dim)
        if k.shape[0] == 0:
            return
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_append(
                ctypes.byref(self._c_pools), k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0),
                slot_mapping.data_ptr(), k.shape[0], kc, vc, self.status.data_ptr(),
                _dev.current_stream_ptr(self.device)), "append")

    def append_page_groups(self, k: torch.Tensor, v: torch.Tensor, page_indices: torch.Tensor,
                           valid_tokens: Optional[torch.Tensor] = None) -> None:
        """Quantize and write whole pages of a cache whose K is quantized per channel over the
        64 tokens of a page (`k_quant=("channel", 64)`, V per token). The reference's decode
        reads this layout (src/foscar/_sm100/int_fold_decode.py:5012-5036) but its `append`
        refuses it (src/foscar/kv_cache.py:643-644); this is the writer it lacks.

        k, v: bfloat16 [P * 64, HKV, D] (same layout rules as `append`), page i's tokens being
        rows [64 i, 64 i + valid_tokens[i]); page_indices int32 [P]; valid_tokens int32 [P] or
        None (every page full). A channel's (s, z) come from the page's valid tokens only, so a
        page that gains tokens (the last page of a growing context) is written again with all of
        them; an engine keeps those few tokens in bf16 until then."""
        lay = self.layout
        if not lay.is_page_channel_k:
            raise NotImplementedError(
                f"append_page_groups() writes k_quant=('channel', {PAGE_SIZE}) with token-wise V; "
                f"this cache has k_quant={lay.k_quant} v_quant={lay.v_quant}")
        groups = self._check_page_groups(page_indices, valid_tokens)
        self._check_token_rows("k", k, rows=groups * PAGE_SIZE)
        self._check_token_rows("v", v, rows=groups * PAGE_SIZE)
        if groups == 0:
            return
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_append_page_groups(
                ctypes.byref(self._c_pools), k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0),
                page_indices.data_ptr(),
                None if valid_tokens is None else valid_tokens.data_ptr(), groups,
                self.status.data_ptr(), _dev.current_stream_ptr(self.device)),
                "append_page_groups")

    def _check_page_groups(self, page_indices, valid_tokens) -> int:
        if (not isinstance(page_indices, torch.Tensor) or page_indices.dtype != torch.int32
                or page_indices.dim() != 1 or not page_indices.is_contiguous()
                or page_indices.device != self.device):
            raise ValueError(f"page_indices must be a contiguous int32 [P] tensor on {self.device}")
        groups = page_indices.numel()
        if valid_tokens is not None and (
                not isinstance(valid_tokens, torch.Tensor) or valid_tokens.dtype != torch.int32
                or tuple(valid_tokens.shape) != (groups,) or not valid_tokens.is_contiguous()
                or valid_tokens.device != self.device):
            raise ValueError(f"valid_tokens must be a contiguous int32 [{groups}] tensor on "
                             f"{self.device}")
        return groups

    def append_quantized_page_groups(self, k_codes, k_scale, k_zero, v_codes, v_scale, v_zero,
                                     page_indices: torch.Tensor,
                                     valid_tokens: Optional[torch.Tensor] = None) -> None:
        """Layout-only write of whole pages an engine quantized itself, for a cache whose K is
        quantized per channel over the 64 tokens of a page: what `append_quantized` is to
        `append`, for `append_page_groups` (the reference's `append_quantized` refuses these
        layouts, src/foscar/kv_cache.py:769-774).

        k_codes, v_codes: uint8 [P * 64, HKV, D], one value per byte, page i's tokens being rows
        [64 i, 64 i + valid_tokens[i]); k_scale, k_zero: f32 [P, HKV, D] (per page and channel);
        v_scale, v_zero: f32 [P * 64, HKV]. Codes are masked to the stored width and records
        saturated to the quantizing writer's ranges."""
        lay = self.layout
        if not lay.is_page_channel_k:
            raise NotImplementedError(
                f"append_quantized_page_groups() writes k_quant=('channel', {PAGE_SIZE}) with "
                f"token-wise V; this cache has k_quant={lay.k_quant} v_quant={lay.v_quant}")
        groups = self._check_page_groups(page_indices, valid_tokens)
        H, D, T = lay.num_kv_heads, lay.head_dim, groups * PAGE_SIZE
        wanted = {"k_codes": (k_codes, torch.uint8, (T, H, D)),
                  "k_scale": (k_scale, torch.float32, (groups, H, D)),
                  "k_zero": (k_zero, torch.float32, (groups, H, D)),
                  "v_codes": (v_codes, torch.uint8, (T, H, D)),
                  "v_scale": (v_scale, torch.float32, (T, H)),
                  "v_zero": (v_zero, torch.float32, (T, H))}
        for name, (x, dtype, shape) in wanted.items():
            if not (isinstance(x, torch.Tensor) and x.dtype == dtype
                    and tuple(x.shape) == shape):
                raise ValueError(f"{name} must be a {dtype} {list(shape)} tensor; got "
                                 f"{getattr(x, 'dtype', None)} {tuple(getattr(x, 'shape', ()))}")
            if not x.is_contiguous():
                raise ValueError(f"{name} must be C-contiguous")
            self._same_device(name, x)
            if dtype == torch.uint8 and x.data_ptr() % 16 != 0:
                raise ValueError(f"{name} must start 16-byte aligned")
        if T > MAX_APPEND_TOKENS:
            raise ValueError(f"one append takes at most {MAX_APPEND_TOKENS} tokens; got {T}: "
                             f"split it into several appends")
        if groups == 0:
            return
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_append_quantized_page_groups(
                ctypes.byref(self._c_pools), k_codes.data_ptr(), k_scale.data_ptr(),
                k_zero.data_ptr(), v_codes.data_ptr(), v_scale.data_ptr(), v_zero.data_ptr(),
                page_indices.data_ptr(),
                None if valid_tokens is None else valid_tokens.data_ptr(), groups,
                self.status.data_ptr(), _dev.current_stream_ptr(self.device)),
                "append_quantized_page_groups")

    def append_quantized(self, k_codes, k_scale, k_zero, v_codes, v_scale, v_zero,
                         slot_mapping) -> None:
        """Layout-only write of engine-quantized tokens (src/foscar/kv_cache.py:689-767): codes
        uint8 [T, HKV, D] one value per byte; f32 scales and zero points [T, HKV] ([T, HKV, g] for
        K over head_dim // g); records saturated to the quantizing writer's ranges."""
        lay = self.layout
        self._refuse_channel_wise("append_quantized")
        H, D = lay.num_kv_heads, lay.head_dim
        T = k_codes.shape[0] if isinstance(k_codes, torch.Tensor) and k_codes.dim() else None
        groups = D // lay.k_quant[1]
        k_group = (T, H, groups) if groups > 1 else (T, H)
        wanted = {"k_codes": (k_codes, torch.uint8, (T, H, D)),
                  "k_scale": (k_scale, torch.float32, k_group),
                  "k_zero": (k_zero, torch.float32, k_group),
                  "v_codes": (v_codes, torch.uint8, (T, H, D)),
                  "v_scale": (v_scale, torch.float32, (T, H)),
                  "v_zero": (v_zero, torch.float32, (T, H))}
        for name, (x, dtype, shape) in wanted.items():
            matches = isinstance(x, torch.Tensor) and x.dtype == dtype \
                and tuple(x.shape) == shape
            if not matches:
                spelled = ["T" if extent is None else extent for extent in shape]
                raise ValueError(f"{name} must be a {dtype} {spelled} tensor; got "
                                 f"{getattr(x, 'dtype', None)} {tuple(getattr(x, 'shape', ()))}")
            if not x.is_contiguous():
                raise ValueError(f"{name} must be C-contiguous")
            self._same_device(name, x)
            if dtype == torch.uint8 and x.data_ptr() % 16 != 0:
                raise ValueError(f"{name} must start 16-byte aligned")
        if T > MAX_APPEND_TOKENS:
            raise ValueError(f"one append takes at most {MAX_APPEND_TOKENS} tokens; got {T}: "
                             f"split it into several appends")
        self._check_slots(slot_mapping, T)
        if T == 0:
            return
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_append_quantized(
                ctypes.byref(self._c_pools), k_codes.data_ptr(), k_scale.data_ptr(),
                k_zero.data_ptr(), v_codes.data_ptr(), v_scale.data_ptr(), v_zero.data_ptr(),
                slot_mapping.data_ptr(), T, self.status.data_ptr(),
                _dev.current_stream_ptr(self.device)), "append_quantized")

    def _check_rows_out(self, name, x):
        """A bf16 [N, HKV, D] destination whose token rows are whole, apart and 16-byte aligned."""
        H, D = self.layout.num_kv_heads, self.layout.head_dim
        typed = isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and x.dim() == 3
        if not typed or (x.shape[1], x.shape[2]) != (H, D):
            raise ValueError(f"{name} must be a bfloat16 [N, {H}, {D}] tensor; got "
                             f"{getattr(x, 'dtype', None)} {tuple(getattr(x, 'shape', ()))}")
        self._same_device(name, x)
        token, head, channel = x.stride()
        overlapping = x.shape[0] > 1 and token < H * D
        if channel != 1 or head != D or overlapping:
            raise ValueError(f"{name} must hold each token's [num_kv_heads, head_dim] row "
                             f"contiguously, rows not overlapping (strides (>= {H * D}, {D}, 1)); "
                             f"got {tuple(x.stride())}")
        if x.data_ptr() % 16 != 0 or (token * x.element_size()) % 16 != 0:
            raise ValueError(f"every token row of {name} must start 16-byte aligned")

    def dequantize(self, k_out, v_out, page_indptr, page_indices, seq_lens, out_indptr) -> None:
        """Read K and V of a batch back into bf16 rows: `k_out[out_indptr[b] + t] =
        bf16(fma(s_k, q, z_k))` for t < seq_lens[b], V likewise
        (src/foscar/kv_cache.py:792-877). No host wait, no allocation, capturable. Out-of-range
        page ids, rows or lengths are skipped and set a status bit (the reference traps)."""
        lay = self.layout
        if not lay.is_token_wise and not lay.is_page_channel_k:
            raise NotImplementedError(
                f"dequantize() reads token-wise layouts only, the layouts append() writes (and "
                f"K per channel over a page, which append_page_groups() writes); "
                f"k_quant={lay.k_quant} v_quant={lay.v_quant} has a channel-wise tensor")
        H, D = lay.num_kv_heads, lay.head_dim
        self._check_rows_out("k_out", k_out)
        self._check_rows_out("v_out", v_out)
        if k_out.shape[0] != v_out.shape[0]:
            raise ValueError(f"k_out has {k_out.shape[0]} rows and v_out has {v_out.shape[0]}")
        for name, x, allowed in (("page_indptr", page_indptr, (torch.int32,)),
                                 ("page_indices", page_indices, (torch.int32,)),
                                 ("seq_lens", seq_lens, (torch.int32,)),
                                 ("out_indptr", out_indptr, (torch.int32, torch.int64))):
            flat = (isinstance(x, torch.Tensor) and x.dtype in allowed and x.dim() == 1
                    and x.is_contiguous())
            if not flat:
                kinds = " or ".join(str(t) for t in allowed)
                raise ValueError(f"{name} must be a contiguous one-dimensional {kinds} tensor; "
                                 f"got {getattr(x, 'dtype', None)} "
                                 f"{tuple(getattr(x, 'shape', ()))}")
            self._same_device(name, x)
        batch = seq_lens.shape[0]
        if page_indptr.shape[0] != batch + 1 or out_indptr.shape[0] != batch:
            raise ValueError(f"seq_lens has {batch} requests, so page_indptr must have "
                             f"{batch + 1} entries and out_indptr {batch}; got "
                             f"{page_indptr.shape[0]} and {out_indptr.shape[0]}")
        if batch > MAX_DEQUANT_REQUESTS:
            raise ValueError(f"one dequantize takes at most {MAX_DEQUANT_REQUESTS} requests; got "
                             f"{batch}: split it into several calls")
        if page_indices.shape[0] * H > 2**31 - 1:
            raise ValueError(f"one dequantize launches a CTA per page entry and KV head, at most "
                             f"2^31 - 1; got {page_indices.shape[0]} entries and {H} KV heads: "
                             f"split it into several calls")
        if batch == 0:
            return
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_dequantize(
                ctypes.byref(self._c_pools), k_out.data_ptr(), v_out.data_ptr(), k_out.stride(0),
                v_out.stride(0), k_out.shape[0], page_indptr.data_ptr(), page_indices.data_ptr(),
                page_indices.shape[0], seq_lens.data_ptr(), out_indptr.data_ptr(),
                int(out_indptr.dtype == torch.int64), batch, self.status.data_ptr(),
                _dev.current_stream_ptr(self.device)), "dequantize")
