"""The three launch helpers of the reference's Blackwell arm, re-bound to this library's C ABI.

The reference reaches its compiled kernels through keyword-only launch helpers whose bodies
call a compiled function:
  - `launch_quant_append`  src/foscar/_sm100/quant_append.py:129-140
  - `launch_fold`          src/foscar/_sm100/fold_runtime.py:680-731
  - `launch_dequant`       src/foscar/_dequant_core.py:328-342
A maintainer who wants this engine under an unmodified `kv_cache.py` / `wrapper.py` replaces
those three bodies with the functions below (same names, same keywords, same tensors) and the
`compile_*` calls with `compile_fold` / `compile_quant_append` / `compile_dequant` here, which
only record what the compiled kernel used to fix at compile time. Everything goes through
`include/foscar_b200.h`; the module uses torch for nothing but `data_ptr()`, strides and the
current stream.

Differences from the reference helpers a caller can see: a launch that meets a bad page id or
length sets a bit in `compiled.status` (int32 [1]) instead of trapping; split units are merged
inside the decode launch when `compiled.unit_counters` is given (the reference launches its
reduction next, `launch_reduction`, src/foscar/_sm100/gqa_decode.py:377-456), otherwise
`launch_fold` issues `fq_merge` itself so that `o_bshd` is final when it returns to the stream.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Optional

import torch

from . import _lib
from . import device as _dev

_OUT_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


@dataclasses.dataclass
class Compiled:
    """What a compiled reference kernel fixed at compile time, as far as the C ABI needs it."""
    layout: object                       # a QuantKVLayout (bits, head_dim, num_kv_heads, ...)
    num_qo_heads: int = 0
    has_lse: bool = False
    has_q_descale: bool = False
    status: Optional[torch.Tensor] = None          # int32 [1], device
    unit_counters: Optional[torch.Tensor] = None   # int32 [B * HKV * head_tiles], zeroed


def _compiled(layout, device, **kw) -> Compiled:
    return Compiled(layout=layout, status=torch.zeros(1, dtype=torch.int32, device=device), **kw)


def compile_quant_append(layout, device="cuda") -> Compiled:
    return _compiled(layout, device)


def compile_dequant(layout, device="cuda") -> Compiled:
    return _compiled(layout, device)


def compile_fold(layout, *, num_qo_heads, has_lse=False, has_q_descale=False, batch_size=0,
                 fused_merge=True, device="cuda") -> Compiled:
    """`batch_size` > 0 with `fused_merge` allocates the per-unit arrival counters that let the
    decode launch merge its own split units; they must be zero before every launch and the
    launch leaves them zero unless it timed out (status bit 0x10)."""
    c = _compiled(layout, device, num_qo_heads=int(num_qo_heads), has_lse=bool(has_lse),
                  has_q_descale=bool(has_q_descale))
    if batch_size > 0 and fused_merge:
        tiles = (num_qo_heads // layout.num_kv_heads + 7) // 8
        c.unit_counters = torch.zeros(batch_size * layout.num_kv_heads * tiles,
                                      dtype=torch.int32, device=device)
    return c


def _pools(layout, k_codes, v_codes, scales, v_page_max=None, v_max_hist=None) -> _lib.Pools:
    p = _lib.Pools()
    p.bits, p.head_dim, p.num_kv_heads = layout.bits, layout.head_dim, layout.num_kv_heads
    channel_k = bool(getattr(layout, "is_page_channel_k", False))
    p.k_groups = 1 if channel_k else layout.head_dim // layout.k_quant[1]
    p.k_channel_group = 64 if channel_k else 0
    p.scale_bf16 = int(layout.scale_dtype == torch.bfloat16)
    p.num_pages = k_codes.shape[0]
    p.k_codes, p.v_codes, p.scales = k_codes.data_ptr(), v_codes.data_ptr(), scales.data_ptr()
    p.v_page_max = None if v_page_max is None else v_page_max.data_ptr()
    p.v_max_hist = None if v_max_hist is None else v_max_hist.data_ptr()
    return p


def _stream(t: torch.Tensor) -> int:
    return _dev.current_stream_ptr(t.device)


def launch_quant_append(compiled, *, inputs, slot_mapping, k_codes, v_codes, scales,
                        v_page_max=None, v_max_hist=None):
    """(k, v) bf16 [T, HKV, D] written at `slot_mapping` int64 [T]; a 6-tuple is the
    prequantized form (k codes, k scales, k zero points, v codes, v scales, v zero points)."""
    if v_page_max is None or v_max_hist is None:
        raise ValueError("the writer keeps v_page_max and v_max_hist for every layout it "
                         "writes; pass the cache's tensors")
    p = _pools(compiled.layout, k_codes, v_codes, scales, v_page_max, v_max_hist)
    lib = _lib.load()
    with _dev.on_device(k_codes.device):
        if len(inputs) == 2:
            k, v = inputs
            rc = lib.fq_append(ctypes.byref(p), k.data_ptr(), v.data_ptr(), k.stride(0),
                               v.stride(0), slot_mapping.data_ptr(), k.shape[0], -1, -1,
                               compiled.status.data_ptr(), _stream(k_codes))
        else:
            kq, ks, kz, vq, vs, vz = inputs
            rc = lib.fq_append_quantized(ctypes.byref(p), kq.data_ptr(), ks.data_ptr(),
                                         kz.data_ptr(), vq.data_ptr(), vs.data_ptr(),
                                         vz.data_ptr(), slot_mapping.data_ptr(), kq.shape[0],
                                         compiled.status.data_ptr(), _stream(k_codes))
    _lib.check(rc, "launch_quant_append")


def launch_fold(compiled, *, kv_splits, seqlens, table_offsets, page_table, q_bshd, o_bshd,
                o_partial=None, l_partial=None, m_partial=None, scale_s=1.0, scale_o=1.0,
                mKq=None, mVq=None, mScale=None, v_max_hist=None, q_descale=None, lse=None,
                dbg=None, enable_pdl=True):
    """One decode step on torch's current stream. q_bshd fp8 e4m3 [B, 1, HQ, D]; o_bshd
    [B, 1, HQ, D] bf16/f16/f32; seqlens, table_offsets ([B + 1]), page_table int32; the three
    partial tensors f32 ([kv_splits, B, 1, HQ, D] and [kv_splits, B, 1, HQ]) when
    kv_splits > 1; mKq, mVq, mScale the cache's pools; lse f32 [B, 1, HQ] exactly when
    compiled with has_lse, q_descale f32 [B, HQ] (any strides) exactly when compiled with
    has_q_descale. `dbg` is accepted and ignored."""
    if (lse is not None) != compiled.has_lse:
        raise TypeError("lse must be given exactly when the kernel was compiled with has_lse")
    if (q_descale is not None) != compiled.has_q_descale:
        raise TypeError("q_descale must be given exactly when the kernel was compiled with "
                        "has_q_descale")
    layout = compiled.layout
    batch, hq = q_bshd.shape[0], q_bshd.shape[-2]
    p = _pools(layout, mKq, mVq, mScale, None, v_max_hist)
    a = _lib.DecodeArgs()
    a.batch, a.num_qo_heads, a.out_dtype = batch, hq, _OUT_CODE[o_bshd.dtype]
    a.kv_splits = a.max_splits = int(kv_splits)
    a.flags = 1 if enable_pdl else 0
    a.sm_scale, a.o_scale = float(scale_s), float(scale_o)
    a.seq_lens, a.page_table = seqlens.data_ptr(), page_table.data_ptr()
    a.table_offsets, a.table_len = table_offsets.data_ptr(), page_table.numel()
    a.q, a.out = q_bshd.data_ptr(), o_bshd.data_ptr()
    if q_descale is not None:
        a.q_descale = q_descale.data_ptr()
        a.q_descale_stride_b, a.q_descale_stride_h = q_descale.stride()
    a.lse = None if lse is None else lse.data_ptr()
    a.status = compiled.status.data_ptr()
    split = kv_splits > 1
    if split:
        a.o_partial, a.l_partial = o_partial.data_ptr(), l_partial.data_ptr()
        a.m_partial = m_partial.data_ptr()
    fused = split and compiled.unit_counters is not None
    if fused:
        a.unit_counters = compiled.unit_counters.data_ptr()
    lib = _lib.load()
    stream = _stream(q_bshd)
    with _dev.on_device(q_bshd.device):
        _lib.check(lib.fq_decode(ctypes.byref(p), ctypes.byref(a), stream), "launch_fold")
        if split and not fused:
            _lib.check(lib.fq_merge(
                o_partial.data_ptr(), l_partial.data_ptr(), m_partial.data_ptr(), None,
                kv_splits, kv_splits, batch, hq, layout.num_kv_heads, layout.head_dim,
                float(scale_o), o_bshd.data_ptr(), _OUT_CODE[o_bshd.dtype],
                None if lse is None else lse.data_ptr(), stream), "launch_fold: merge")


def launch_dequant(compiled, *, threads=0, k_codes, v_codes, scales, k_out, v_out, page_indptr,
                   page_indices, seq_lens, out_indptr):
    """Read a batch back into bf16 rows [N, HKV, D]; `threads` is accepted and ignored."""
    batch = seq_lens.shape[0]
    if batch == 0:
        return
    p = _pools(compiled.layout, k_codes, v_codes, scales)
    with _dev.on_device(k_codes.device):
        _lib.check(_lib.load().fq_dequantize(
            ctypes.byref(p), k_out.data_ptr(), v_out.data_ptr(), k_out.stride(0), v_out.stride(0),
            k_out.shape[0], page_indptr.data_ptr(), page_indices.data_ptr(),
            page_indices.shape[0], seq_lens.data_ptr(), out_indptr.data_ptr(),
            int(out_indptr.dtype == torch.int64), batch, compiled.status.data_ptr(),
            _stream(k_codes)), "launch_dequant")
