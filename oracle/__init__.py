"""CPU restatement of the reference's quantized-KV path. TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs may import this
package, and only as the checker or the timed CPU baseline. The product (`foscar_b200`) never
imports it and has no CPU fallback.

Parity status: the writer/read-back arithmetic and the pool byte format are pinned against the
reference's own known-answer vectors and against its host functions imported in the build
container (tests/golden/make_golden.py). The decode output has no bit-level reference (the
reference's device kernels cannot run without its pinned DSL), so it is tolerance-checked
against `ref_attention` over the read-back values, as the reference's own GPU tests do.
Channel-wise K pools (`ref_channel`): parity unpinned (the reference ships no writer or fixture
for them; the quantizer is the token-wise one applied along a page's token axis).
"""
from .ref_quant import (  # noqa: F401
    code_channel, pack_rows, unpack_rows, quantize_rows, scale_range, saturate_given,
    CpuPools, ref_append, ref_append_quantized, ref_dequantize, ref_attention, ref_merge,
    ref_vmax_bucket, ref_v_max_hist, ref_pscale_lp, emulate_fold_decode,
)
from .ref_channel import (  # noqa: F401
    CpuChannelPools, ref_append_page_groups, ref_append_quantized_page_groups,
    ref_dequantize_channel,
)
