"""Generate tests/golden/reference_host.json from the reference's own host-side functions.

Run once in the build container, where the reference checkout is importable:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

Only the reference's torch-free / CPU-runnable host layer is executed (its device kernels need a
GPU and its pinned DSL). The JSON is committed; the tests read the JSON, never the reference.
"""
import json
import os
import random
import struct
import sys

import torch


def main():
    from foscar._append_core import scale_range  # noqa: needs cutlass DSL importable
    from foscar._sm100.code_layout import code_field, code_row_index
    from foscar._sm100.fold_runtime import (pscale_lp_of_bucket, v_max_hist_of,
                                            v_page_max_for_pool, vmax_bucket)
    from foscar._sm100.scheduler import plan_splits_sm100
    from foscar.graph_plan import Bucket
    from foscar.kv_cache import QuantKVLayout, clip_index
    from foscar.quant_layout import quant_block_offsets

    out = {}
    out["code_field"] = {str(bits): [[code_field(bits, w, f) for f in range(32 // bits)]
                                     for w in range(256 * bits // 32)] for bits in (2, 4)}
    out["code_row_index"] = [[p, h, r, code_row_index(64, 8, p, h, r, wide=int)]
                             for p, h, r in ((0, 0, 0), (3, 5, 17), (70000, 7, 63))]
    pairs = []
    for d in (64, 128, 256):
        ks = [("token", g) for g in (64, 128, 256) if g <= d] + [("channel", g) for g in (64, 128, 256)]
        vs = [("token", d)] + [("channel", g) for g in (64, 128, 256)]
        for kq in ks:
            for vq in vs:
                pairs.append([d, list(kq), list(vq), quant_block_offsets(kq, vq, N=64, D=d)])
    out["quant_block_offsets"] = pairs

    rng = random.Random(0)
    pats = [0, 1, 0x80000000, 0x7F800000, 0x7FC00000, 0xFFFFFFFF, 0x0DA24260, 0x3F800000,
            0x3FE00000, 0x3FE00001, 0x43E00000, 0x43E00001, 0x00800000, 0x007FFFFF]
    pats += [rng.getrandbits(32) for _ in range(200)]
    for e in range(1, 255):
        for mant in (0, 0x600000, 0x600001, 0x7FFFFF):
            pats.append((e << 23) | mant)
    out["vmax_bucket"] = [[p, int(vmax_bucket(p))] for p in pats]
    out["pscale_lp_of_bucket"] = [[b, int(pscale_lp_of_bucket(b))] for b in (0, 27, 100, 127, 255)]

    g = torch.Generator().manual_seed(0)
    scales = torch.rand(6, 3, 64, 4, generator=g) * 4
    scales[1, 0, :, 2] = 0
    scales[2, 1, :, 2] = -1.0
    vpm = v_page_max_for_pool(scales)
    hist = v_max_hist_of(vpm)
    out["v_page_max_for_pool"] = {
        "sv_bits": scales[..., 2].contiguous().view(torch.int32).tolist(),
        "v_page_max": vpm.view(torch.int32).tolist(),
        "v_max_hist": hist.view(torch.int32).tolist()}

    out["scale_range"] = {str(q): [struct.unpack("<I", struct.pack("<f", x))[0]
                                   for x in scale_range(q)] for q in (3, 15)}
    out["clip_index"] = [[r, d, clip_index(r, d)] for r in (None, 1.0, 0.99, 0.5, 0.001)
                         for d in (64, 128, 256)]

    layouts = []
    for bits in (2, 4):
        for d, hkv, kq, vq, sd in ((128, 8, None, None, None), (64, 8, None, None, None),
                                   (256, 2, None, None, None), (128, 8, ("token", 64), None, None),
                                   (256, 2, ("channel", 64), None, None),
                                   (128, 4, None, None, torch.bfloat16),
                                   (128, 8, ("channel", 128), ("channel", 64), None)):
            lay = QuantKVLayout._create("sm100", bits=bits, head_dim=d, num_kv_heads=hkv,
                                        k_quant=kq, v_quant=vq, scale_dtype=sd)
            layouts.append(dict(
                bits=bits, head_dim=d, num_kv_heads=hkv,
                k_quant=None if kq is None else list(kq), v_quant=None if vq is None else list(vq),
                scale_dtype=None if sd is None else "bfloat16",
                resolved=dict(k_quant=list(lay.k_quant), v_quant=list(lay.v_quant),
                              scale_dtype=str(lay.scale_dtype).split(".")[-1], reader=lay.reader,
                              code_pool_order=lay.code_pool_order,
                              k_pool_permuted=lay.k_pool_permuted,
                              v_pool_permuted=lay.v_pool_permuted,
                              has_v_page_max=lay.has_v_page_max),
                bytes_per_page=lay.bytes_per_page(),
                pool_shapes={k: (None if v is None else list(v))
                             for k, v in lay.pool_shapes(5).items()}))
    out["layouts"] = layouts

    plans = []
    for bits in (2, 4):
        for b in (1, 2, 4, 8, 16, 32, 64, 128, 256):
            for hkv in (1, 2, 8):
                for kv in (128, 4096, 8192, 32768, 100352, 131072, 524288):
                    for tile, ht in ((256, 1), (128, 1), (256, 2)):
                        s, mode = plan_splits_sm100(b, hkv, kv, bits=bits, sm_count=148,
                                                    sequence_tile=tile, head_tiles=ht)
                        plans.append([bits, b, hkv, kv, tile, ht, s, mode])
    out["plan_splits_sm100"] = plans

    buckets = []
    for batch, hkv, tile, ht in ((1, 8, 256, 1), (4, 8, 256, 1), (16, 2, 256, 1), (3, 1, 128, 2),
                                 (32, 8, 256, 1)):
        bk = Bucket(batch, hkv, wave=148, tile=tile, max_kv_len=131072, head_tiles=ht)
        rec = dict(batch=batch, hkv=hkv, tile=tile, head_tiles=ht,
                   split_capable=bk.split_capable, s_tight=bk.s_tight, steps=[])
        if bk.split_capable:
            for _ in range(4):
                lengths = [rng.randint(1, 131072) for _ in range(batch)]
                rec["steps"].append(dict(lengths=lengths, chunks=bk.chunks(lengths).tolist()))
        buckets.append(rec)
    out["graph_buckets"] = buckets

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_host.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    sys.exit(main())
