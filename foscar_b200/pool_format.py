"""Byte format of the quantized KV pools: where a code sits, how a scale block is sectioned,
and the exponent bin of a page maximum.

Torch-free integer arithmetic, shared by the host layer, the tests and (restated in C++) the
CUDA kernels, so the writer and the decode cannot disagree about a byte.

Follows the reference's format definitions:
  - code placement: src/foscar/_sm100/code_layout.py:24-43, docs/K_STORE_PERM.md:31-65
  - scale block sections: src/foscar/quant_layout.py:57-85
  - granularity envelope: src/foscar/quant_layout.py:137-166
  - page-maximum exponent bin: src/foscar/_sm100/fold_runtime.py:135-171
"""
from __future__ import annotations

PAGE_SIZE = 64
QUANT_BITS = (2, 4)
HEAD_DIMS = (64, 128, 256)
VMAX_BINS = 256
#: Bin of 1e-30: a table with no counted maximum resolves to this bin (lp = 108).
PSCALE_FLOOR_BUCKET = 27
GROUP_SIZES = (64, 128, 256)


def values_per_word(bits: int) -> int:
    if bits not in QUANT_BITS:
        raise ValueError(f"bits must be one of {QUANT_BITS}; got {bits!r}")
    return 32 // bits


def channel_of_field(bits: int, word: int, field: int) -> int:
    """Channel held by bit field `field` (bits [bits*f, bits*f+bits)) of 32-bit word `word` of a
    token row: even fields walk the word's first half of channels, odd fields its second."""
    w = values_per_word(bits)
    return w * word + (field >> 1) + (w >> 1) * (field & 1)


def field_of_channel(bits: int, channel: int):
    """Inverse of `channel_of_field`: (word, field, bit offset inside the row) of a channel."""
    w = values_per_word(bits)
    word, within = divmod(channel, w)
    half = w >> 1
    field = 2 * (within % half) + within // half
    return word, field, word * 32 + bits * field


def row_bytes(bits: int, head_dim: int) -> int:
    return head_dim * bits // 8


def normalize_pair(pair, head_dim: int, name: str):
    """An (axis, group) granularity as a plain (str, int) tuple; None means whole-head token-wise."""
    if pair is None:
        return ("token", head_dim)
    try:
        axis, group = pair
    except (TypeError, ValueError):
        raise ValueError(f"{name} must be an (axis, group) pair; got {pair!r}") from None
    return (str(axis), int(group))


def envelope_refusal(k_quant, v_quant, head_dim: int):
    """Why the decode refuses this granularity pair, or None when it reads it.

    K: token-wise over g in {64,128,256} with g <= D, or channel-wise over a token group in
    {64,128,256}. V: token-wise over the whole head, or channel-wise over such a token group."""
    (k_axis, k_group), (v_axis, v_group) = k_quant, v_quant
    if k_axis not in ("token", "channel"):
        return f"K axis must be 'token' or 'channel'; got {k_axis!r}"
    if v_axis not in ("token", "channel"):
        return f"V axis must be 'token' or 'channel'; got {v_axis!r}"
    if k_axis == "token":
        allowed = tuple(g for g in GROUP_SIZES if g <= head_dim)
        if k_group not in allowed:
            return (f"K token-wise group at head_dim={head_dim} must be in {allowed}; "
                    f"got {k_group}")
    elif k_group not in GROUP_SIZES:
        return f"K channel-wise token group must be in {GROUP_SIZES}; got {k_group}"
    if v_axis == "token":
        if v_group != head_dim:
            return f"V token-wise supports group == head_dim only; got {v_group}"
    elif v_group not in GROUP_SIZES:
        return f"V channel-wise token group must be in {GROUP_SIZES}; got {v_group}"
    return None


def scale_block_sections(k_quant, v_quant, head_dim: int, page: int = PAGE_SIZE) -> dict:
    """Element offsets of the per-(page, KV head) scale block.

    Keys: k_ring, v_ring, ring_tot, k_ch, v_ch, block_tot, legacy. Offsets count elements of the
    scale dtype; a section a tensor does not use is None. When K and V are both token-wise over
    the whole head the block is the interleaved [page, 4] = (s_k, z_k, s_v, z_v) form."""
    k_quant = (k_quant[0], int(k_quant[1]))
    v_quant = (v_quant[0], int(v_quant[1]))
    whole = ("token", head_dim)
    if k_quant == whole and v_quant == whole:
        return dict(k_ring=0, v_ring=0, ring_tot=4 * page, k_ch=None, v_ch=None,
                    block_tot=4 * page, legacy=True)

    def ring(q):
        return 0 if q[0] == "channel" else 2 * (head_dim // q[1]) * page

    def chan(q):
        return 2 * head_dim if q[0] == "channel" else 0

    kr, vr, kc, vc = ring(k_quant), ring(v_quant), chan(k_quant), chan(v_quant)
    return dict(k_ring=0 if kr else None, v_ring=kr if vr else None, ring_tot=kr + vr,
                k_ch=kr + vr if kc else None, v_ch=kr + vr + kc if vc else None,
                block_tot=kr + vr + kc + vc, legacy=False)


def vmax_bucket(bits: int) -> int:
    """Exponent bin in [0, 255] of a page maximum given as an f32 bit pattern: the sign is
    dropped, the pattern capped at +inf's, and 0x1FFFFF added so that a mantissa above 1.75
    carries into the exponent. lp = floor(log2(448 / x)) = 135 - bin for every normal x."""
    return (min(bits & 0x7FFFFFFF, 0x7F800000) + 0x1FFFFF) >> 23


def pscale_lp_of_bucket(bucket: int) -> int:
    return 135 - bucket


def pscale_lp_of_hist(hist) -> int:
    """The P-scale exponent a decode takes from a count table: 135 - max(top nonzero bin, 27)."""
    top = 0
    for b, n in enumerate(hist):
        if int(n) != 0:
            top = b
    return pscale_lp_of_bucket(max(top, PSCALE_FLOOR_BUCKET))


def q_head_tiling(num_qo_heads: int, num_kv_heads: int):
    """(heads per work item padded to the MMA's row count, head tiles per KV head).

    A work item carries up to eight query heads of one KV head; a larger GQA ratio is spread
    over ceil(ratio / 8) head tiles (src/foscar/_sm100/fold_runtime.py:71-74)."""
    ratio = num_qo_heads // num_kv_heads
    tiles = (ratio + 7) // 8
    per_tile = min(ratio, 8)
    padded = 4 if per_tile <= 4 else 8
    return padded, tiles
