"""`PagedDecodeWrapper`: plan/run of paged GQA decode over a `QuantKVCache`, eager and
CUDA-graph mode.

Host-side mirror of the reference wrapper for the Blackwell arm (src/foscar/wrapper.py:569-1350
eager, :1353-1676 graph mode): same call forms, argument meaning, properties and refusals.
Planning differs by design. A plan is a list of pieces (request, KV head, head tile, range of
sequence tiles) sized from the step's lengths and the SM count so that every CTA streams the
same number of tiles; the reference picks one uniform split count from the longest request.
When the lengths may not be read on the host (`max_kv_len=` given with device `seq_lens`) the
plan is a uniform split count resolved on the device.
"""
from __future__ import annotations

import ctypes
import functools
from typing import Optional

import numpy as np
import torch

from . import _lib, device as _dev
from .kv_cache import QuantKVCache, QuantKVLayout
from .pool_format import PAGE_SIZE

_OUT_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
_OUT_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_Q_DTYPE = torch.float8_e4m3fn
_RETIRED_PLAN_ARGS = ("num_kv_heads", "head_dim", "page_size", "bits", "k_quant", "v_quant")
_RETIRED_RUN_ARGS = ("k_cache", "v_cache", "scale_pool", "pscale_lp", "k_pool_order")
#: Most pieces one unit may be cut into (the leading extent of the partial buffers).
MAX_SPLITS = 64
_GRAPH_HOST_BUFFERS = 4
_GRAPH_MAX_KV_LEN = 2**31 - 64


def _head_tiles(num_qo_heads, num_kv_heads):
    return (num_qo_heads // num_kv_heads + 7) // 8


def _check_num_qo_heads(num_qo_heads, num_kv_heads):
    if (isinstance(num_qo_heads, bool) or not isinstance(num_qo_heads, int)
            or num_qo_heads <= 0 or num_qo_heads % num_kv_heads != 0):
        raise ValueError(f"num_qo_heads ({num_qo_heads!r}) must be a positive multiple of the "
                         f"layout's num_kv_heads ({num_kv_heads})")


def _resolve_io_dtypes(layout, q_data_type, o_data_type):
    if q_data_type is None:
        q_data_type = _Q_DTYPE
    if q_data_type != _Q_DTYPE:
        raise ValueError(f"the {layout.reader} decode reads a {_Q_DTYPE} query; got "
                         f"q_data_type={q_data_type}")
    if o_data_type is None:
        o_data_type = torch.bfloat16
    if o_data_type not in _OUT_DTYPES:
        raise ValueError(f"the {layout.reader} decode writes a {list(_OUT_DTYPES)} output; got "
                         f"o_data_type={o_data_type}")
    return q_data_type, o_data_type


def _refuse_retired(where, positional, keywords, retired, replacement):
    if "kernel_kwargs" in keywords:
        raise TypeError(f"{where}: kernel_kwargs is retired from the public API; the layout "
                        f"carries every configuration a plan needs (QuantKVLayout.create)")
    named = sorted(set(keywords) & set(retired))
    if named or positional:
        what = f"{named}" if named else f"{len(positional)} extra positional argument(s)"
        raise TypeError(f"{where}: {what} belong to the retired call form; {replacement}")
    if keywords:
        raise TypeError(f"{where}: unexpected keyword argument(s) {sorted(keywords)}")


def _fail_closed_plan(method):
    """A failed plan leaves the wrapper unplanned."""
    @functools.wraps(method)
    def wrapped(self, *args, **kwargs):
        self._invalidate_plan()
        try:
            return method(self, *args, **kwargs)
        except Exception:
            self._invalidate_plan()
            raise
    return wrapped


def _carve_partials(workspace, splits, batch, hq, d):
    """(o_partial [S,B,1,HQ,D], l_partial [S,B,1,HQ], m_partial [S,B,1,HQ]) f32 views, in that
    order, from the front of the workspace (src/foscar/wrapper.py:134-173)."""
    ws = workspace.view(-1).view(torch.uint8)
    ws = ws[: ws.numel() // 4 * 4].view(torch.float32)
    n_o, n_r = splits * batch * hq * d, splits * batch * hq
    need = n_o + 2 * n_r
    if ws.numel() < need:
        raise RuntimeError(
            f"kernel reduction with kv_splits={splits} batch_size={batch} q_len_per_req=1 "
            f"num_qo_heads={hq} head_dim={d} requires {need * 4} byte workspace which exceeds "
            f"provided workspace of {ws.numel() * 4} bytes")
    return (ws[:n_o].view(splits, batch, 1, hq, d), ws[n_o:n_o + n_r].view(splits, batch, 1, hq),
            ws[n_o + n_r:need].view(splits, batch, 1, hq))


def _fit_splits(workspace, batch, hq, d, cap=MAX_SPLITS):
    """The most partial slots (<= cap) the workspace holds."""
    floats = workspace.numel() * workspace.element_size() // 4
    return int(max(1, min(cap, floats // (batch * hq * (d + 2)))))


def graph_workspace_bytes(max_batch: int, num_qo_heads: int, layout: QuantKVLayout, *,
                          max_kv_len: int, device=None) -> int:
    """Workspace bytes that serve graph-mode wrappers of every batch size up to `max_batch`
    (src/foscar/wrapper.py:395-419): the partial buffers at the most pieces a unit can get."""
    if isinstance(max_batch, bool) or not isinstance(max_batch, int) or max_batch < 1:
        raise ValueError(f"max_batch must be a positive int; got {max_batch!r}")
    dev = torch.device("cuda", _dev.cuda_index(device))
    arch = _dev.require_arch(dev)
    if layout.arch != arch:
        raise ValueError(f"the layout was resolved for {layout.arch} and {dev} is {arch}")
    _check_num_qo_heads(num_qo_heads, layout.num_kv_heads)
    sms = _dev.sm_count(dev) * _lib.ctas_per_sm(layout.bits, layout.head_dim)
    tiles = -(-int(max_kv_len) // _lib.tile_tokens(layout.bits, layout.head_dim))
    ovh = _lib.piece_overhead(layout.bits, layout.head_dim)
    words = 0
    for batch in range(1, max_batch + 1):
        splits = _graph_split_cap(batch, layout.num_kv_heads,
                                  _head_tiles(num_qo_heads, layout.num_kv_heads), sms, tiles, ovh)
        words = max(words, splits * batch * num_qo_heads * (layout.head_dim + 2))
    return 4 * words


def _graph_split_cap(batch, hkv, head_tiles, sms, max_tiles, overhead):
    """The split cap a graph-mode bucket plans with (the leading extent of its partial buffers).

    The balanced planner never cuts a unit into more pieces than the cap it is given (it raises
    every CTA's share until the longest unit fits), so any cap is valid; this one is what the
    most skewed step of the bucket wants: one request at `max_tiles` tiles and every other at a
    single tile, which gives the smallest share per CTA against the longest unit."""
    per_request = hkv * head_tiles
    worst_total = (per_request * (max_tiles + overhead)
                   + (batch - 1) * per_request * (1 + overhead) + overhead * (sms - 1))
    share = max(overhead + 1, -(-worst_total // sms))
    wanted = -(-max_tiles // max(1, share - overhead)) + 2
    return int(max(1, min(MAX_SPLITS, max_tiles, sms, wanted)))


class PagedDecodeWrapper:
    """Paged GQA decode over a quantized KV cache on B200.

    `PagedDecodeWrapper(workspace)` is eager mode: `plan()` once per step, `run()` once per
    layer. `PagedDecodeWrapper(workspace, use_cuda_graph=True)` is graph mode: `plan()` once,
    capture `run()`, then `update(lengths)` + replay per step."""

    def __new__(cls, float_workspace_buffer: torch.Tensor = None, use_cuda_graph: bool = False):
        if use_cuda_graph and cls is PagedDecodeWrapper:
            cls = _GraphDecodeWrapper
        return super().__new__(cls)

    # Split units are merged inside the decode kernel by the piece that arrives last. False
    # restores the separate merge launch (fq_merge) after every decode.
    fused_merge = True

    # What fq_decode's argument block takes from the plan. The block is built once per plan and
    # reused by every run(); assigning any of these attributes drops it.
    _PLAN_STATE = frozenset((
        "_float_workspace_buffer", "_status", "_o_data_type", "_num_qo_heads", "_batch_size",
        "_kv_splits", "_seqlens", "_table_offsets", "_page_table", "_o_partial", "_l_partial",
        "_m_partial", "_max_splits", "_worklist", "_split_counts", "_unit_counters",
        "_work_rows", "_plan_ctas", "_merge", "_q_len"))

    def __setattr__(self, name, value):
        if name in self._PLAN_STATE:
            object.__setattr__(self, "_plan_args", None)
        object.__setattr__(self, name, value)

    def __init__(self, float_workspace_buffer: torch.Tensor, use_cuda_graph: bool = False):
        if not isinstance(float_workspace_buffer, torch.Tensor):
            raise TypeError("float_workspace_buffer must be a torch.Tensor")
        self._float_workspace_buffer = float_workspace_buffer
        self.device = float_workspace_buffer.device
        self._status = None
        #: kernels this wrapper has launched (decode and merge)
        self.launches = 0
        self._invalidate_plan()

    def _invalidate_plan(self):
        self._planned = False
        self._layout = None
        self._bits = None
        self._q_data_type = self._o_data_type = None
        self._num_qo_heads = self._num_kv_heads = self._head_dim = None
        self._q_len, self._cols = 1, None
        self._sm_scale = None
        self._batch_size = None
        self._max_kv_len = None
        self._kv_splits = None
        self._reduction = None
        self._seqlens = self._table_offsets = self._page_table = None
        self._o_partial = self._l_partial = self._m_partial = None
        self._max_splits = 1
        self._worklist = None          # device int32 list, explicit plans only
        self._split_counts = None      # device int32 [units], explicit plans only
        self._unit_counters = None     # device int32 [units]: in-kernel merge of split units
        self._work_rows = 0
        self._plan_ctas = 0
        self._merge = False

    # -- read-only view of what plan() decided ----------------------------------------------
    @property
    def kv_splits(self) -> int:
        """Most pieces any (request, KV head) is cut into by the current plan."""
        return self._kv_splits

    @property
    def reduction(self) -> str:
        """"none" when every unit is one piece, else "kernel"."""
        return self._reduction

    @property
    def bits(self) -> Optional[int]:
        return self._bits

    def last_status(self) -> int:
        """Device status word of this wrapper's launches (0 = no fault). Waits for the device.

        A launch that ended on a device wait that ran out (bit 0x10) may have left the arrival
        counters of split units non-zero; they are cleared here, on this stream, so that the next
        launch or graph replay merges correctly again."""
        if self._status is None:
            return 0
        word = int(self._status.item())
        if word & _lib.STATUS_TIMEOUT and self._unit_counters is not None:
            with _dev.on_device(self.device):
                self._unit_counters.zero_()
        return word

    def _status_ptr(self):
        if self._status is None:
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._status.data_ptr()

    # -- plan --------------------------------------------------------------------------------
    @_fail_closed_plan
    def plan(self, indptr: torch.Tensor, indices: torch.Tensor, seq_lens: torch.Tensor,
             num_qo_heads: int, layout: QuantKVLayout = None, *retired_positional,
             q_data_type=None, o_data_type=None, sm_scale: Optional[float] = None,
             kv_splits: Optional[int] = None, reduction: str = "auto", q_len_per_req: int = 1,
             max_kv_len: Optional[int] = None, non_blocking: bool = True, **retired) -> None:
        """Plan one step's batch over caches of `layout` (src/foscar/wrapper.py:663-830).

        indptr int32 [B+1], indices int32 [pages], seq_lens int32/int64 [B]. `kv_splits=None`
        lets the planner choose: a balanced piece list when the lengths are readable on the
        host (CPU `seq_lens`, or no `max_kv_len`, which costs one device wait as in the
        reference), else a uniform count from `max_kv_len` with no wait. An explicit
        `kv_splits` is a uniform count. `reduction` is "auto", "none" (needs one piece per
        unit) or "kernel"."""
        if retired_positional or retired or not isinstance(layout, QuantKVLayout):
            _refuse_retired("PagedDecodeWrapper.plan", retired_positional, retired,
                            _RETIRED_PLAN_ARGS,
                            "build the cache layout with QuantKVLayout.create(bits=, head_dim=, "
                            "num_kv_heads=, k_quant=, v_quant=) and pass it as plan(indptr, "
                            "indices, seq_lens, num_qo_heads, layout)")
            raise TypeError(f"PagedDecodeWrapper.plan: layout must be a QuantKVLayout; got "
                            f"{type(layout).__name__}")
        arch = _dev.require_arch(self.device)
        if layout.arch != arch:
            raise ValueError(f"the layout was resolved for {layout.arch} and this wrapper's "
                             f"device {self.device} is {arch}; create the layout for the device "
                             f"that decodes it")
        q_len = self._check_q_len(q_len_per_req)
        _check_num_qo_heads(num_qo_heads, layout.num_kv_heads)
        if seq_lens.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"seq_lens must be int32 or int64; got {seq_lens.dtype}")
        batch = seq_lens.numel()
        if batch == 0:
            raise ValueError("plan() needs at least one request; seq_lens is empty")
        if indptr.numel() < batch:
            raise ValueError(f"indptr length ({indptr.numel()}) must be at least batch_size "
                             f"({batch})")
        q_data_type, o_data_type = _resolve_io_dtypes(layout, q_data_type, o_data_type)
        if reduction not in ("auto", "none", "kernel"):
            if reduction == "atomic":
                raise NotImplementedError("quantized decode has no atomic-reduction arm")
            raise ValueError(f'quantized reduction must be "none" or "kernel"; got {reduction!r}')
        self._set_common(layout, num_qo_heads, q_data_type, o_data_type, sm_scale, batch, q_len)

        host_lens = None
        if kv_splits is None or kv_splits <= 0:
            if seq_lens.device.type == "cpu" or max_kv_len is None:
                host_lens = seq_lens.detach().to("cpu", torch.int32).numpy()   # waits if on GPU
        if host_lens is not None and q_len > 1 and int(host_lens.min()) < q_len:
            raise ValueError(f"seq_lens counts the {q_len} query tokens of each request (they "
                             f"are appended before the decode); got a length of "
                             f"{int(host_lens.min())}")
        if max_kv_len is None:
            max_kv_len = int(host_lens.max()) if host_lens is not None else \
                int(seq_lens.max().item())
        self._max_kv_len = int(max_kv_len)

        def to_dev(t):
            return t.to(dtype=torch.int32, device=self.device, non_blocking=non_blocking)
        self._seqlens = to_dev(seq_lens).contiguous()
        self._page_table = to_dev(indices).contiguous()
        self._table_offsets = to_dev(indptr)[:batch].contiguous()

        with _dev.on_device(self.device):
            if host_lens is not None and reduction != "none":
                host_offsets = indptr.detach().to("cpu", torch.int32)[:batch].contiguous().numpy()
                self._plan_balanced(host_lens, host_offsets, non_blocking)
            else:
                self._plan_uniform(kv_splits, reduction)
            self._status_ptr()
        self._planned = True

    def _check_q_len(self, q_len_per_req):
        """Query tokens per request. The reference refuses anything but 1
        (src/foscar/wrapper.py:756-761); here the tokens of a request ride as further columns
        of their KV head's unit, token l attending to positions < seq_len - (q_len - 1 - l)."""
        if isinstance(q_len_per_req, bool) or not isinstance(q_len_per_req, int) \
                or not 1 <= q_len_per_req <= 64:
            raise ValueError(f"q_len_per_req must be an int in [1, 64]; got {q_len_per_req!r}")
        if q_len_per_req > 1 and not self.fused_merge:
            raise NotImplementedError("q_len_per_req > 1 needs the in-kernel merge of split "
                                      "units (fused_merge=True): the separate merge launch "
                                      "writes [batch, heads] rows only")
        return q_len_per_req

    def _set_common(self, layout, num_qo_heads, q_dtype, o_dtype, sm_scale, batch, q_len=1):
        if not layout.is_token_wise and not (layout.is_page_channel_k and layout.head_dim == 256):
            raise NotImplementedError(
                f"this build decodes token-wise layouts, and K per channel over a page "
                f"(k_quant=('channel', 64), token-wise V) at head_dim 256; k_quant="
                f"{layout.k_quant} v_quant={layout.v_quant} at head_dim {layout.head_dim} is "
                f"neither")
        if layout.head_dim == 256 and layout.is_token_wise \
                and layout.k_quant[1] < layout.head_dim:
            raise NotImplementedError(
                f"this build decodes whole-head K groups at head_dim 256; got "
                f"k_quant={layout.k_quant}")
        if layout.is_token_wise and layout.k_quant[1] < layout.head_dim and not (
                layout.head_dim == 128 and layout.k_quant[1] == 64):
            raise NotImplementedError(
                f"this build decodes K groups of 64 channels at head_dim 128 only; got "
                f"k_quant={layout.k_quant} at head_dim {layout.head_dim}")
        self._layout = layout
        self._bits = layout.bits
        self._q_data_type, self._o_data_type = q_dtype, o_dtype
        self._num_qo_heads, self._num_kv_heads = num_qo_heads, layout.num_kv_heads
        self._q_len = q_len
        # columns of the batch's units: a request's query tokens times its query heads
        self._cols = num_qo_heads * q_len
        self._head_dim = layout.head_dim
        self._sm_scale = layout.head_dim ** -0.5 if sm_scale is None else sm_scale
        self._batch_size = batch

    def _plan_uniform(self, kv_splits, reduction):
        lay = self._layout
        if kv_splits is None or kv_splits <= 0:
            kv_splits = _lib.load().fq_plan_splits(
                self._batch_size, lay.num_kv_heads, _head_tiles(self._cols, lay.num_kv_heads),
                self._max_kv_len, lay.bits, lay.head_dim,
                _dev.sm_count(self.device) * _lib.ctas_per_sm(lay.bits, lay.head_dim))
            if kv_splits < 1:
                _lib.check(kv_splits, "plan")
            if reduction == "none":
                kv_splits = 1
        if reduction == "none" and kv_splits != 1:
            raise ValueError(f'reduction="none" requires kv_splits == 1, got {kv_splits}')
        self._kv_splits = int(kv_splits)
        self._reduction = "none" if kv_splits == 1 and reduction != "kernel" else "kernel"
        self._merge = self._reduction == "kernel"
        self._max_splits = self._kv_splits
        if self._merge:
            self._o_partial, self._l_partial, self._m_partial = _carve_partials(
                self._float_workspace_buffer, self._kv_splits, self._batch_size,
                self._cols, self._head_dim)
            self._new_unit_counters()

    def _new_unit_counters(self):
        """Zeroed per-unit arrival counters: the decode kernel merges a split unit itself when
        its last piece arrives (and sets the counter back), so no merge launch follows."""
        if not self.fused_merge:
            self._unit_counters = None
            return
        units = self._batch_size * self._num_kv_heads * _head_tiles(self._cols,
                                                                     self._num_kv_heads)
        if self._unit_counters is None or self._unit_counters.numel() != units:
            self._unit_counters = torch.zeros(units, dtype=torch.int32, device=self.device)
        else:
            self._unit_counters.zero_()

    # Rows of a planned piece list carry their request's length and table offset, so the kernel
    # need not fetch them after the row (a dependent round trip less before a CTA's first tile).
    carry_requests = True

    def _plan_balanced(self, host_lens, host_offsets, non_blocking):
        lay, lib = self._layout, _lib.load()
        ht = _head_tiles(self._cols, lay.num_kv_heads)
        ctas = _dev.sm_count(self.device) * _lib.ctas_per_sm(lay.bits, lay.head_dim)
        units = self._batch_size * lay.num_kv_heads * ht
        words = int(lib.fq_worklist_words(self._batch_size, lay.num_kv_heads, ht, ctas))
        cap = _fit_splits(self._float_workspace_buffer, self._batch_size, self._cols,
                          self._head_dim)
        lens = np.ascontiguousarray(host_lens, dtype=np.int32)
        work = np.zeros(words, dtype=np.int32)
        counts = np.zeros(units, dtype=np.int32)
        pieces = lib.fq_plan_worklist(lens.ctypes.data, self._batch_size, lay.num_kv_heads, ht,
                                      ctas, cap, work.ctypes.data, words, counts.ctypes.data,
                                      lay.bits, lay.head_dim)
        if pieces == _lib.ERR_TOO_LARGE:
            # a unit would need more pieces than the workspace holds: plan uniformly instead
            self._plan_uniform(None, "auto")
            return
        if pieces < 0:
            _lib.check(pieces, "plan")
        if self.carry_requests:
            _lib.check(lib.fq_worklist_attach_requests(work.ctypes.data, words, lens.ctypes.data,
                                                       host_offsets.ctypes.data,
                                                       self._batch_size), "plan")
        most = int(counts.max())
        self._kv_splits = most
        self._reduction = "kernel" if most > 1 else "none"
        self._merge = most > 1
        self._max_splits = max(most, 1)
        if self._merge:
            self._o_partial, self._l_partial, self._m_partial = _carve_partials(
                self._float_workspace_buffer, most, self._batch_size, self._cols,
                self._head_dim)
            self._new_unit_counters()
        else:
            # the kernel still wants valid partial pointers for an explicit list
            self._o_partial = self._l_partial = self._m_partial = None
        both = torch.from_numpy(np.concatenate([work, counts]))
        dev = both.to(self.device, non_blocking=False)
        self._worklist, self._split_counts = dev[:words], dev[words:]
        self._work_rows = units + ctas
        self._plan_ctas = ctas

    # -- run ---------------------------------------------------------------------------------
    def _check_tensor(self, name, x, dtype):
        if x.dtype != dtype:
            raise ValueError(f"{name}.dtype={x.dtype} mismatches the planned {dtype}")
        if x.device != self.device:
            raise ValueError(f"{name} is on {x.device}; this wrapper plans for {self.device}")
        b, hq, d = self._batch_size, self._num_qo_heads, self._head_dim
        if self._q_len > 1:
            three_d = False
            if tuple(x.shape) != (b, self._q_len, hq, d):
                raise ValueError(f"{name} has shape {tuple(x.shape)}; the plan is for "
                                 f"[{b}, {self._q_len}, {hq}, {d}] (batch, query tokens, query "
                                 f"heads, head dimension)")
        elif tuple(x.shape) == (b, hq, d):
            three_d = True
        elif tuple(x.shape) == (b, 1, hq, d):
            three_d = False
        else:
            raise ValueError(f"{name} has shape {tuple(x.shape)}; the plan is for [{b}, {hq}, "
                             f"{d}] or [{b}, 1, {hq}, {d}] (batch, query heads, head dimension)")
        if not x.is_contiguous():
            raise ValueError(f"{name} must be C-contiguous; got strides {tuple(x.stride())}")
        if x.data_ptr() % 16:
            raise ValueError(f"{name} must start 16-byte aligned")
        return three_d

    def run(self, q: torch.Tensor, kv_cache: QuantKVCache = None, *retired_positional,
            out: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None,
            o_scale: Optional[float] = None, enable_pdl: bool = True,
            lse: Optional[torch.Tensor] = None, q_descale: Optional[torch.Tensor] = None,
            **retired) -> torch.Tensor:
        """Decode one layer (src/foscar/wrapper.py:1111-1233). q: fp8 e4m3 [B, HQ, D] or
        [B, 1, HQ, D]; `out=` bf16/f16/f32 of the same shape; `lse=` f32 [B, HQ] receives the
        natural-log log-sum-exp; `q_descale=` f32 [B, HQ] (any strides). With `out=` the call
        allocates nothing, reads no device value and does not wait, so it can be captured."""
        if retired_positional or retired or not isinstance(kv_cache, QuantKVCache):
            _refuse_retired("PagedDecodeWrapper.run", retired_positional, retired,
                            _RETIRED_RUN_ARGS,
                            "build the cache with layout.allocate() or layout.bind() and call "
                            "run(q, kv_cache, out=...)")
            raise TypeError(f"PagedDecodeWrapper.run: kv_cache must be a QuantKVCache; got "
                            f"{type(kv_cache).__name__}")
        if not self._planned:
            raise RuntimeError("Call plan() before run().")
        layout = kv_cache.layout
        if layout is not self._layout and layout != self._layout:
            raise ValueError(f"kv_cache was built for another layout than this plan's:\n"
                             f"  cache: {layout}\n  plan:  {self._layout}")
        if kv_cache.device != self.device:
            raise ValueError(f"kv_cache is on {kv_cache.device}; this wrapper plans for "
                             f"{self.device}")
        three_d = self._check_tensor("q", q, self._q_data_type)
        b, hq, d = self._batch_size, self._num_qo_heads, self._head_dim
        rows = (b, hq) if self._q_len == 1 else (b, self._q_len, hq)
        if lse is not None:
            if (lse.dtype != torch.float32 or lse.device != self.device
                    or tuple(lse.shape) != rows or not lse.is_contiguous()
                    or lse.data_ptr() % 16):
                raise ValueError(f"lse must be a C-contiguous, 16-byte aligned fp32 "
                                 f"{list(rows)} tensor on {self.device}; got {lse.dtype} "
                                 f"{tuple(lse.shape)}")
        if out is not None:
            self._check_tensor("out", out, self._o_data_type)
        if q_descale is not None:
            if (q_descale.dtype != torch.float32 or q_descale.device != self.device
                    or tuple(q_descale.shape) != rows):
                raise ValueError(f"q_descale must be an fp32 {list(rows)} tensor on "
                                 f"{self.device}; got {q_descale.dtype} "
                                 f"{tuple(q_descale.shape)} on {q_descale.device}")
            if self._q_len > 1 and q_descale.stride(0) != self._q_len * q_descale.stride(1):
                raise ValueError(f"q_descale's batch stride must be {self._q_len} token "
                                 f"strides; got strides {tuple(q_descale.stride())}")
        scale_s = self._sm_scale if sm_scale is None else sm_scale
        scale_o = 1.0 if o_scale is None else o_scale
        with _dev.on_device(self.device):
            return self._launch(q, kv_cache, out, scale_s, scale_o, three_d, q_descale, lse,
                                enable_pdl)

    def update(self, lengths) -> None:
        raise RuntimeError("update() is graph mode's per-step call: build the wrapper with "
                           "use_cuda_graph=True and plan() it first")

    def _build_plan_args(self):
        """fq_decode's argument block with everything the plan fixes filled in."""
        args = _lib.DecodeArgs()
        args.batch, args.num_qo_heads = self._batch_size, self._num_qo_heads
        args.q_len = self._q_len
        args.out_dtype = _OUT_CODE[self._o_data_type]
        args.kv_splits = 1 if self._worklist is not None else self._kv_splits
        args.max_splits = self._max_splits
        args.num_work = self._work_rows
        args.max_ctas = self._plan_ctas
        args.worklist = None if self._worklist is None else self._worklist.data_ptr()
        args.seq_lens = self._seqlens.data_ptr()
        args.page_table = self._page_table.data_ptr()
        args.table_offsets = self._table_offsets.data_ptr()
        args.table_len = self._page_table.numel()
        if self._o_partial is not None:
            args.o_partial = self._o_partial.data_ptr()
            args.l_partial = self._l_partial.data_ptr()
            args.m_partial = self._m_partial.data_ptr()
        elif self._worklist is not None:
            # an explicit list whose units are all single pieces never touches the partials
            ws = self._float_workspace_buffer.data_ptr()
            args.o_partial = args.l_partial = args.m_partial = ws
        args.status = self._status_ptr()
        if self._merge and self._unit_counters is not None:
            args.unit_counters = self._unit_counters.data_ptr()
            if self._split_counts is not None:
                args.split_counts = self._split_counts.data_ptr()
        return args

    def _launch(self, q, cache, out, scale_s, scale_o, three_d, q_descale, lse,
                enable_pdl=True):
        b, hq, d = self._batch_size, self._num_qo_heads, self._head_dim
        if out is None:
            out = torch.empty((b, hq, d) if three_d else (b, self._q_len, hq, d),
                              dtype=self._o_data_type, device=self.device)
        lib = _lib.load()
        stream = _dev.current_stream_ptr(self.device)
        args = self._plan_args
        if args is None:
            args = self._plan_args = self._build_plan_args()
        fused = self._merge and self._unit_counters is not None
        args.flags = 1 if enable_pdl else 0
        args.sm_scale, args.o_scale = scale_s, scale_o
        args.q = q.data_ptr()
        if q_descale is not None:
            args.q_descale = q_descale.data_ptr()
            # with several query tokens the kernel's "batch" stride is the token stride
            args.q_descale_stride_b, args.q_descale_stride_h = q_descale.stride()[-2:]
        else:
            args.q_descale = None
        args.out = out.data_ptr()
        # with a merge pass the decode's own final rows (one-piece units) still take the lse
        args.lse = None if lse is None else lse.data_ptr()
        _lib.check(lib.fq_decode(ctypes.byref(cache._c_pools), ctypes.byref(args), stream),
                   "decode")
        self.launches += 1
        if self._merge and not fused:
            self.launches += 1
            counts = None if self._split_counts is None else self._split_counts.data_ptr()
            _lib.check(lib.fq_merge(
                self._o_partial.data_ptr(), self._l_partial.data_ptr(),
                self._m_partial.data_ptr(), counts, self._kv_splits, self._max_splits, b, hq,
                self._num_kv_heads, d, scale_o, out.data_ptr(), _OUT_CODE[self._o_data_type],
                None if lse is None else lse.data_ptr(), stream), "merge")
        return out


def _graph_host_lengths(lengths, batch, max_kv_len):
    """The step's lengths as a checked int32 numpy array [B], each in [1, max_kv_len]."""
    if isinstance(lengths, torch.Tensor):
        if lengths.device.type != "cpu":
            raise ValueError("update() takes host lengths (a list, a numpy array or a CPU "
                             "tensor); a device tensor would force a wait")
        lengths = lengths.numpy()
    arr = np.asarray(lengths)
    if arr.shape != (batch,) or arr.dtype.kind not in "iu":
        raise ValueError(f"update() takes {batch} integer lengths, one per request of the "
                         f"bucket; got shape {arr.shape} dtype {arr.dtype}")
    if arr.min() < 1 or arr.max() > max_kv_len:
        raise ValueError(f"every length must be in [1, {max_kv_len}] (the bucket's max_kv_len); "
                         f"got [{int(arr.min())}, {int(arr.max())}]")
    return np.ascontiguousarray(arr, dtype=np.int32)


class _GraphDecodeWrapper(PagedDecodeWrapper):
    """CUDA-graph mode (src/foscar/wrapper.py:1353-1676). `plan()` once for one captured batch
    size; it allocates the bucket's device piece list and pinned host buffers. `update(lengths)`
    per step plans on the host and enqueues one asynchronous copy; the captured `run()` reads
    the list's header on the device, so one captured launch serves every step's plan."""

    def __init__(self, float_workspace_buffer: torch.Tensor, use_cuda_graph: bool = True):
        super().__init__(float_workspace_buffer, use_cuda_graph)
        self._graph = None

    def plan(self, indptr=None, indices=None, seq_lens=None, num_qo_heads=None, layout=None,
             *retired_positional, q_data_type=None, o_data_type=None, sm_scale=None,
             kv_splits=None, reduction="auto", q_len_per_req=1, max_kv_len=None,
             non_blocking=True, page_table=None, lse=False, q_descale=False, **retired) -> None:
        """Graph mode's plan: page_table int32 [B, max_pages] and seq_lens int32 [B] are the
        engine's own device buffers (addresses recorded, no value read); `max_kv_len` bounds
        every later `update`; `lse` / `q_descale` declare whether every `run` passes them."""
        if self._graph is not None:
            raise RuntimeError("a graph-mode wrapper plans once: a captured graph keeps the "
                               "addresses of its work list and scratch for the wrapper's life; "
                               "build one wrapper per captured batch size")
        with _dev.on_device(self.device):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("plan() runs once, before capture: it allocates and waits "
                                   "for the device, which a stream capture may not contain")
        if retired_positional or retired or not isinstance(layout, QuantKVLayout):
            _refuse_retired("PagedDecodeWrapper.plan", retired_positional, retired,
                            _RETIRED_PLAN_ARGS,
                            "graph mode plans with plan(page_table=, seq_lens=, num_qo_heads=, "
                            "layout=, max_kv_len=)")
            raise TypeError(f"PagedDecodeWrapper.plan: layout must be a QuantKVLayout; got "
                            f"{type(layout).__name__}")
        if indptr is not None or indices is not None:
            raise TypeError("graph mode's plan() takes the engine's page_table=, not indptr and "
                            "indices")
        if kv_splits is not None or reduction != "auto":
            raise TypeError("graph mode plans each step's splits in update(); kv_splits= and "
                            "reduction= are eager mode's")
        if non_blocking is not True:
            raise TypeError("non_blocking= is eager mode's; graph mode copies nothing at plan()")
        q_len = self._check_q_len(q_len_per_req)
        for name, flag in (("lse", lse), ("q_descale", q_descale)):
            if not isinstance(flag, bool):
                raise TypeError(f"graph mode's {name}= declares whether every run() passes "
                                f"{name}; it is a bool, got {flag!r}")
        arch = _dev.require_arch(self.device)
        if layout.arch != arch:
            raise ValueError(f"the layout was resolved for {layout.arch} and this wrapper's "
                             f"device {self.device} is {arch}")
        _check_num_qo_heads(num_qo_heads, layout.num_kv_heads)
        for name, t, rank in (("page_table", page_table, 2), ("seq_lens", seq_lens, 1)):
            if not isinstance(t, torch.Tensor) or t.dtype != torch.int32 or t.dim() != rank \
                    or t.device != self.device or not t.is_contiguous():
                raise ValueError(f"graph mode's {name} is the engine's contiguous int32 "
                                 f"{rank}-D buffer on {self.device}")
        batch, max_pages = page_table.shape
        if batch == 0 or tuple(seq_lens.shape) != (batch,):
            raise ValueError(f"page_table holds {batch} rows and seq_lens "
                             f"{tuple(seq_lens.shape)}; a bucket has one length per row, and at "
                             f"least one row")
        if batch * max_pages > 2**31 - 1:
            raise ValueError(f"the page table's {batch} x {max_pages} entries exceed int32 "
                             f"offsets")
        top = min(_GRAPH_MAX_KV_LEN, PAGE_SIZE * max_pages)
        if isinstance(max_kv_len, bool) or not isinstance(max_kv_len, int) \
                or not 1 <= max_kv_len <= top:
            raise ValueError(f"max_kv_len is the bucket's largest context, an int in [1, {top}]; "
                             f"got {max_kv_len!r}")
        q_data_type, o_data_type = _resolve_io_dtypes(layout, q_data_type, o_data_type)
        try:
            self._set_common(layout, num_qo_heads, q_data_type, o_data_type, sm_scale, batch,
                             q_len)
            self._max_kv_len = max_kv_len
            with _dev.on_device(self.device):
                self._graph = self._graph_setup(page_table, seq_lens, lse, q_descale)
                torch.cuda.synchronize(self.device)
        except Exception:
            self._invalidate_plan()
            self._graph = None
            raise
        self._planned = True

    def _graph_setup(self, page_table, seq_lens, lse, q_descale):
        lay, lib = self._layout, _lib.load()
        b, hq, d = self._batch_size, self._cols, self._head_dim
        ht = _head_tiles(hq, lay.num_kv_heads)
        ctas = _dev.sm_count(self.device) * _lib.ctas_per_sm(lay.bits, lay.head_dim)
        units = b * lay.num_kv_heads * ht
        words = int(lib.fq_worklist_words(b, lay.num_kv_heads, ht, ctas))
        tiles = -(-self._max_kv_len // _lib.tile_tokens(lay.bits, d))
        cap = _graph_split_cap(b, lay.num_kv_heads, ht, ctas, tiles,
                               _lib.piece_overhead(lay.bits, d))
        cap = min(cap, _fit_splits(self._float_workspace_buffer, b, hq, d))
        self._o_partial, self._l_partial, self._m_partial = _carve_partials(
            self._float_workspace_buffer, cap, b, hq, d)
        self._max_splits = cap
        self._kv_splits = cap
        self._reduction = "kernel"
        self._merge = True
        self._new_unit_counters()
        self._seqlens = seq_lens
        self._page_table = page_table.view(-1)
        self._table_offsets = (torch.arange(b, dtype=torch.int32, device=self.device)
                               * page_table.shape[1])
        total = words + units
        g = dict(words=words, units=units, ctas=ctas, ht=ht, cap=cap, lse=lse,
                 offsets=np.arange(b, dtype=np.int32) * int(page_table.shape[1]),
                 q_descale=q_descale, stream=None, next_host=0,
                 host=[torch.empty(total, dtype=torch.int32).pin_memory()
                       for _ in range(_GRAPH_HOST_BUFFERS)],
                 events=[torch.cuda.Event() for _ in range(_GRAPH_HOST_BUFFERS)],
                 recorded=[False] * _GRAPH_HOST_BUFFERS)
        # a valid plan at length 1 so that a warm-up or capture before the first update runs
        first = g["host"][0].numpy()
        self._plan_into(first, np.ones(b, dtype=np.int32), g)
        dev = g["host"][0].to(self.device)
        self._worklist, self._split_counts = dev[:words], dev[words:]
        g["device"] = dev
        self._work_rows = units + ctas
        self._plan_ctas = ctas
        self._status_ptr()
        return g

    def _plan_into(self, buf, lengths, g):
        lay, lib = self._layout, _lib.load()
        words = g["words"]
        pieces = lib.fq_plan_worklist(lengths.ctypes.data, self._batch_size, lay.num_kv_heads,
                                      g["ht"], g["ctas"], g["cap"], buf.ctypes.data, words,
                                      buf[words:].ctypes.data, lay.bits, lay.head_dim)
        if pieces < 0:
            _lib.check(pieces, "update")
        if self.carry_requests:
            _lib.check(lib.fq_worklist_attach_requests(buf.ctypes.data, words,
                                                       lengths.ctypes.data,
                                                       g["offsets"].ctypes.data,
                                                       self._batch_size), "update")

    def update(self, lengths) -> None:
        """Once per step, outside the graph and before its replay: plan the step from host
        `lengths` and enqueue one asynchronous copy of the piece list. Same stream every call;
        refused under capture. Waits only for the pinned buffer it is about to reuse."""
        g = self._graph
        if g is None:
            raise RuntimeError("update() follows the graph-mode wrapper's plan(); plan() it "
                               "first")
        with _dev.on_device(self.device):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("update() runs outside the graph, before each replay: under "
                                   "capture it would freeze one step's plan into every replay")
            lengths = _graph_host_lengths(lengths, self._batch_size, self._max_kv_len)
            stream = torch.cuda.current_stream()
            if g["stream"] is None:
                g["stream"] = stream
            elif stream != g["stream"]:
                raise RuntimeError(f"update() runs on the stream the graph replays on, the "
                                   f"stream of its first call ({g['stream']}); this call is on "
                                   f"{stream}")
            slot = g["next_host"]
            g["next_host"] = (slot + 1) % _GRAPH_HOST_BUFFERS
            if g["recorded"][slot]:
                g["events"][slot].synchronize()
            self._plan_into(g["host"][slot].numpy(), lengths, g)
            g["device"].copy_(g["host"][slot], non_blocking=True)
            g["events"][slot].record(stream)
            g["recorded"][slot] = True

    def _launch(self, q, cache, out, scale_s, scale_o, three_d, q_descale, lse,
                enable_pdl=True):
        g = self._graph
        if out is None:
            raise ValueError("graph mode's run() needs out=: a captured call writes a buffer the "
                             "engine owns, and allocates nothing")
        if (lse is not None) != g["lse"] or (q_descale is not None) != g["q_descale"]:
            raise ValueError(f"this bucket was planned with lse={g['lse']} and "
                             f"q_descale={g['q_descale']}; this call passes "
                             f"lse={'a tensor' if lse is not None else None} and "
                             f"q_descale={'a tensor' if q_descale is not None else None}")
        return super()._launch(q, cache, out, scale_s, scale_o, three_d, q_descale, lse,
                               enable_pdl)
