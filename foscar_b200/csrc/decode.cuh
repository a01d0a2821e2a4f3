// Decode kernel parameters, work items and shared-memory plan (shared by decode.cu and the
// host-side launcher/planner in capi.cu).
#pragma once
#include "common.cuh"

namespace fq {

constexpr int TILE = 128;            // MMA rows: tensor-memory lanes, threads of a worker group
// Tokens per sequence tile. head_dim 128: one token per lane (two pages). head_dim 64: two tokens
// per lane, t and 128 + t of the tile (four pages): their 64-byte operand rows sit side by side
// in one 128-byte row, so a tile of 256 tokens costs what a 128-token tile of head_dim 128 costs.
// INT2 at head_dim 128 can be built the same way (-DFQ_INT2_TWO_TOKENS=1): two tokens per lane,
// each with a 128-byte operand row and a score chain of its own, in three worker groups instead
// of four (the V operand stage of 256 tokens is 32 KB a group), so that the per-tile waits,
// barriers, tensor-memory round trips and the O accumulation are paid once per 256 tokens. It
// passes the same tests and was measured no faster (long contexts +1 %, mixed batches +5 to
// +14 %), so the build with one token per lane is the default.
#ifndef FQ_INT2_TWO_TOKENS
#define FQ_INT2_TWO_TOKENS 0
#endif
__host__ __device__ constexpr bool two_token_build(int bits, int head_dim) {
  return FQ_INT2_TWO_TOKENS != 0 && bits == 2 && head_dim == 128;
}
__host__ __device__ constexpr int tile_tokens(int bits, int head_dim) {
  return head_dim == 64 || two_token_build(bits, head_dim) ? 256 : 128;
}
constexpr int WORK_WORDS = 8;        // int32 words per explicit work-list row
#ifndef FQ_WORKER_GROUPS
#define FQ_WORKER_GROUPS 4
#endif
constexpr int WORKER_GROUPS = FQ_WORKER_GROUPS;  // 128-thread groups, tile i -> group i % G
// Two CTAs of two worker groups each per SM instead of one CTA of four (-DFQ_INT2_TWO_CTAS=1,
// the INT2 builds): the CTAs' item epilogues and prologues overlap each other's tiles; each gets
// half the shared memory (the INT4 rings would be too shallow). Measured 16 to 31 % slower than
// one CTA of four groups on every workload tried, so it is off.
#ifndef FQ_INT2_TWO_CTAS
#define FQ_INT2_TWO_CTAS 0
#endif
__host__ __device__ constexpr int ctas_per_sm(int bits, int head_dim) {
  return FQ_INT2_TWO_CTAS != 0 && bits == 2 && head_dim <= 128 && !two_token_build(bits, head_dim)
             ? 2 : 1;
}
__host__ __device__ constexpr int worker_groups(int bits, int head_dim) {
  return two_token_build(bits, head_dim) ? 3 : (ctas_per_sm(bits, head_dim) == 2 ? 2 : WORKER_GROUPS);
}
// + 2 producers + 2 MMA issuers
__host__ __device__ constexpr int decode_threads(int bits, int head_dim) {
  return 32 * (4 * worker_groups(bits, head_dim) + 4);
}
constexpr int SMEM_LIMIT = 232448;   // 227 KiB opt-in limit per CTA on sm_100
// (two CTAs per SM: half of the SM's 228 KiB less the KiB the system keeps per CTA)
__host__ __device__ constexpr int smem_limit(int bits, int head_dim) {
  return ctas_per_sm(bits, head_dim) == 2 ? 115712 : SMEM_LIMIT;
}

struct DecodeParams {
  fq_pools p;
  fq_decode_args a;  // num_qo_heads here counts a unit's columns: q_len x the caller's heads
  int heads_per_kv;  // columns per KV head: q_len x the GQA ratio
  int head_tiles;    // ceil(heads_per_kv / 8)
  int q_len;         // query tokens per request (>= 1)
  int gqa;           // the caller's query heads per KV head
  int gqa_inv;       // ceil(2^16 / gqa)
  int hq;            // the caller's query heads
  int num_items;     // implicit: B*HKV*head_tiles*kv_splits; explicit: row capacity
  int ring_stages;
  int tile_tokens;   // tile_tokens(bits, head_dim)
  int item_slots;    // work items a CTA keeps decoded in shared memory
  long long wait_budget;   // cycle budget of one device wait
};

struct WorkItem {
  int b, kvh, ht, t0, t1, slot, len, table_off;
};

// Several query tokens per request (template flag MQ; the one-token builds carry none of it):
// column hl of KV head kvh is query token hl / gqa, head hl % gqa of the KV head's group. The
// quotient comes from a multiply and a shift (gqa_inv = ceil(2^16 / gqa), exact for hl < 512).
__device__ __forceinline__ int column_token(const DecodeParams& P, int hl) {
  return (hl * P.gqa_inv) >> 16;
}

// (token row, head) of column hl in the caller's q / out / lse / q_descale tensors
// [B * q_len, HQ]; at one query token (b, kvh * heads_per_kv + hl).
template <bool MQ>
__device__ __forceinline__ int2 caller_col(const DecodeParams& P, int b, int kvh, int hl) {
  if constexpr (!MQ) return make_int2(b, kvh * P.heads_per_kv + hl);
  const int l = column_token(P, hl);
  return make_int2(b * P.q_len + l, kvh * P.gqa + (hl - l * P.gqa));
}
template <bool MQ>
__device__ __forceinline__ long long caller_row(const DecodeParams& P, int b, int kvh, int hl) {
  if constexpr (!MQ)
    return static_cast<long long>(b) * P.a.num_qo_heads +
           (static_cast<long long>(kvh) * P.heads_per_kv + hl);
  const int2 c = caller_col<true>(P, b, kvh, hl);
  return static_cast<long long>(c.x) * P.hq + c.y;
}

// How many of the request's last positions column hl does not see: query token l of q_len
// attends to positions < len - (q_len - 1 - l).
__device__ __forceinline__ int column_lag(const DecodeParams& P, int hl) {
  return max(P.q_len - 1 - column_token(P, hl), 0);
}

// q_descale of column hl: element (token row, head).
template <bool MQ>
__device__ __forceinline__ float caller_descale(const DecodeParams& P, int b, int kvh, int hl) {
  if constexpr (!MQ) {
    const long long head = static_cast<long long>(kvh) * P.heads_per_kv + hl;
    return __ldg(P.a.q_descale + b * P.a.q_descale_stride_b + head * P.a.q_descale_stride_h);
  }
  const int2 c = caller_col<true>(P, b, kvh, hl);
  return __ldg(P.a.q_descale + c.x * P.a.q_descale_stride_b + c.y * P.a.q_descale_stride_h);
}

// Shared-memory plan for one (BITS, D) build. All offsets from a 1024-byte aligned base.
template <int BITS, int D>
struct SmemPlan {
  static constexpr int RB = D * BITS / 8;              // code row bytes
  static constexpr int CODE_PAGE = PAGE * RB;          // one page of K (or V) codes, one head
  static constexpr int SCALE_PAGE = PAGE * 16;         // f32 (s_k,z_k,s_v,z_v) records
  // Code rows in the ring are 16, 32 or 64 bytes; threads of a quarter-warp read the same
  // 16-byte chunk of eight consecutive rows, which at 32 and 64 bytes a row falls on two or
  // four bank groups only. The producers therefore store chunk c of row r at chunk
  // c ^ row_swizzle(r), which spreads those eight reads over all banks.
  static constexpr int CHUNKS = RB / 16;
  __host__ __device__ static constexpr int row_swizzle(int row) {
    return CHUNKS == 4 ? (row >> 1) & 3 : (CHUNKS == 2 ? (row >> 2) & 1 : 0);
  }
  static constexpr int TT = tile_tokens(BITS, D);      // tokens per tile
  static constexpr int G = worker_groups(BITS, D);     // worker groups of this build
  static constexpr bool PAIR = D == 64;                // two tokens per lane, rows side by side
  static constexpr bool TWO = TT == 2 * TILE && !PAIR; // two tokens per lane, a row each
  static constexpr int PPT = TT / PAGE;                // pages per tile
  static constexpr int K_OFF = 0;                      // a ring stage: K pages, V pages, records
  static constexpr int V_OFF = PPT * CODE_PAGE;
  static constexpr int S_OFF = 2 * PPT * CODE_PAGE;
  static constexpr int STAGE = 2 * PPT * CODE_PAGE + PPT * SCALE_PAGE;
  // Operand rows keep a 128-byte pitch (the swizzle atom) whatever D <= 128: head_dim 64 uses
  // the first half of each row.
  static constexpr int ROW = 128;
  static constexpr int VOP_STAGE = (TWO ? 2 : 1) * TILE * ROW;   // expanded V operand, one tile
  static constexpr int Q_BYTES = 16 * ROW;             // 16 MMA rows
  static constexpr int P_BYTES = TT * 16;              // 16 bytes (8 hi + 8 lo) per token, a
                                                       // plane of 128 rows per token of a lane
  static constexpr int VOP_OFF = 0;
  static constexpr int Q_OFF = VOP_OFF + G * VOP_STAGE;
  static constexpr int P_OFF = Q_OFF + 2 * Q_BYTES;
  // A group's state at the end of a work item (accumulators + (m,l,c), 4224 bytes) goes into the
  // group's own V operand stage: its last PV MMA is complete by then, every group has read the
  // states before the item's closing barrier, and V rows are next written after it.
  static constexpr int XCHG_BYTES = TILE * 8 * 4 + 128;
  static constexpr int XCHG_OFF = VOP_OFF;
  static constexpr int XCHG_STRIDE = VOP_STAGE;
  static_assert(XCHG_BYTES <= VOP_STAGE, "a group's state must fit its V stage");
  static constexpr int RED_OFF = P_OFF + G * P_BYTES;  // reductions
  // column maxima 256 B and sums 256 B per group; then 96 B of per-head constants per worker
  // warp (score scale, and score scale times the query sum of each K group); two 16-byte merge
  // notices; two items' per-head constants as the producer leaves them (2 x 96 B)
  static constexpr int HEADK_OFF = RED_OFF + 512 * G;
  static constexpr int INFO_OFF = HEADK_OFF + 96 * 4 * G;
  static constexpr int HEADC_OFF = INFO_OFF + 32;
  static constexpr int RED_BYTES = (HEADC_OFF + 192 - RED_OFF + 1023) / 1024 * 1024;
  static constexpr int BAR_OFF = RED_OFF + RED_BYTES;
  static constexpr int BAR_BYTES = 2048;   // barriers, then flags and diagnostics, then the
                                           // CTA's first work items as decoded at its start
  static constexpr int ITEM_OFF = BAR_OFF + 1280;
  static constexpr int ITEM_SLOTS = (BAR_BYTES - 1280) / 32;
  static constexpr int RING_OFF = (BAR_OFF + BAR_BYTES + 1023) / 1024 * 1024;
  static constexpr int max_ring_stages() {
    return (smem_limit(BITS, D) - 1024 /*alignment slack*/ - RING_OFF) / STAGE;
  }
};

// The items a launch runs, decoded the same way by every role of every CTA.
static __device__ __noinline__ WorkItem decode_item(const DecodeParams& P, int i) {
  WorkItem w;
  const fq_decode_args& a = P.a;
  int len = 0, table_off = 0;
  bool carried = false;   // the list's rows carry the request's length and table offset
  if (a.worklist != nullptr) {
    const int rows_off = __ldg(a.worklist + 3);   // header word 3: rows' word offset
    carried = __ldg(a.worklist + 4) != 0;         // header word 4: fq_worklist_attach_requests
    const int* rows = a.worklist + rows_off;
    const int4 r0 = __ldg(reinterpret_cast<const int4*>(rows) + 2 * i);
    const int4 r1 = __ldg(reinterpret_cast<const int4*>(rows) + 2 * i + 1);
    w.b = r0.x; w.kvh = r0.y; w.ht = r0.z; w.t0 = r0.w; w.t1 = r1.x; w.slot = r1.y;
    len = r1.z; table_off = r1.w;
    const bool ok = w.b >= 0 && w.b < a.batch && w.kvh >= 0 && w.kvh < P.p.num_kv_heads &&
                    w.ht >= 0 && w.ht < P.head_tiles && w.slot < a.max_splits;
    if (!ok) { w.b = 0; w.kvh = 0; w.ht = 0; w.t0 = w.t1 = 0; w.slot = -2; carried = false; }
  } else {
    const int S = a.kv_splits;
    w.slot = S > 1 ? i % S : -1;
    int rest = i / S;
    w.ht = rest % P.head_tiles; rest /= P.head_tiles;
    w.kvh = rest % P.p.num_kv_heads;
    w.b = rest / P.p.num_kv_heads;
    w.t0 = 0; w.t1 = 0x7FFFFFFF;
  }
  // Otherwise two more loads that depend on the row: with a cold L2 a further round trip
  // before the CTA's first page id can be requested.
  if (!carried) {
    len = __ldg(a.seq_lens + w.b);
    table_off = __ldg(a.table_offsets + w.b);
  }
  if (len < 0) len = 0;
  w.len = len;
  const int tiles = (len + P.tile_tokens - 1) / P.tile_tokens;
  if (a.worklist == nullptr) {
    const int S = a.kv_splits;
    const int per = (tiles + S - 1) / S;
    const int s = S > 1 ? w.slot : 0;
    w.t0 = min(s * per, tiles);
    w.t1 = min(w.t0 + per, tiles);
  } else {
    w.t0 = max(0, min(w.t0, tiles));
    w.t1 = max(w.t0, min(w.t1, tiles));
  }
  w.table_off = table_off;
  return w;
}

// The items one CTA runs: [begin, end) in steps of `step`. Implicit plans stride the grid over
// the item space. An explicit list carries a header {pieces, units, ctas, rows' word offset},
// then cta_start[ctas + 1], then the rows; CTA c runs rows [cta_start[c], cta_start[c+1]).
// The header is read on the device, so a captured launch follows a list rewritten between
// replays.
struct ItemRange {
  int begin, end, step;
};

// The CTA's k-th item (list index wi). The first items of a CTA (ITEM_SLOTS, plus as many as fit
// in the shared memory the ring leaves over: DecodeParams::item_slots in all) are decoded once,
// in parallel, when the CTA starts and kept in shared memory, so that no role pays the chain of
// dependent global loads at an item boundary; later ones are decoded on demand.
__device__ __forceinline__ WorkItem item_at(const DecodeParams& P, const WorkItem* cached,
                                            const WorkItem* more, int slots, int k, int wi) {
  if (k < slots) return cached[k];
  if (k < P.item_slots) return more[k - slots];   // shared memory the ring leaves over
  return decode_item(P, wi);
}
// Launch of the head_dim 256 build (decode_wide.cu), called by fq_decode with checked arguments.
int launch_decode_wide(DecodeParams& P, cudaStream_t stream);

__device__ inline ItemRange item_range(const DecodeParams& P) {
  if (P.a.worklist == nullptr)
    return ItemRange{static_cast<int>(blockIdx.x), P.num_items, static_cast<int>(gridDim.x)};
  const int pieces = min(__ldg(P.a.worklist), P.num_items);
  const int ctas = __ldg(P.a.worklist + 2);
  if (static_cast<int>(blockIdx.x) >= ctas) return ItemRange{0, 0, 1};
  const int b = __ldg(P.a.worklist + WORK_WORDS + blockIdx.x);
  const int e = __ldg(P.a.worklist + WORK_WORDS + blockIdx.x + 1);
  return ItemRange{max(0, min(b, pieces)), max(0, min(e, pieces)), 1};
}

// ---------------------------------------------------------------------------------------------
// Device helpers shared by the decode kernels
// ---------------------------------------------------------------------------------------------

__device__ inline float warp_max_f32(float x) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
  return r;
}
__device__ inline __half2 h2_exp2(__half2 x) {
  uint32_t r, a = *reinterpret_cast<uint32_t*>(&x);
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(a));
  return *reinterpret_cast<__half2*>(&r);
}
__device__ inline uint32_t f16x2_to_e4m3x2(__half2 x) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(*reinterpret_cast<uint32_t*>(&x)));
  return r;
}
__device__ inline __half2 e4m3x2_to_f16x2(uint32_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(static_cast<uint16_t>(v)));
  return *reinterpret_cast<__half2*>(&r);
}

// Load this thread's token row (RB bytes at `src`) as packed words.
template <int BITS, int D>
__device__ inline void load_row(uint32_t src, uint32_t (&w)[D * BITS / 32], int swz) {
#pragma unroll
  for (int v = 0; v < D * BITS / 128; ++v)
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w[4 * v]), "=r"(w[4 * v + 1]), "=r"(w[4 * v + 2]), "=r"(w[4 * v + 3])
                 : "r"(src + ((v ^ swz) << 4)));   // chunk v sits at chunk v ^ swz of the row
}
// Unpack packed words into exact operand bytes, one per code, in expansion order:
// out[(8/BITS) * wi + k] = (w[wi] >> (BITS * k)) & mask.
template <int BITS, int D>
__device__ inline void expand_words(const uint32_t (&w)[D * BITS / 32], uint32_t (&out)[D / 4]) {
  constexpr uint32_t MASK = BITS == 2 ? 0x03030303u : 0x0F0F0F0Fu;
  constexpr int PER = 8 / BITS;  // output words per input word
#pragma unroll
  for (int i = 0; i < D * BITS / 32; ++i)
#pragma unroll
    for (int k = 0; k < PER; ++k) out[PER * i + k] = (w[i] >> (BITS * k)) & MASK;
}
// The cheaper unpack for INT2 V rows: odd output words keep their codes two bits up, i.e. hold
// 4 * code, which is still an exact E4M3 byte (values up to 15 * 2^-9 are linear in the byte).
// Five instead of seven instructions per packed word; the channels at those positions
// (expanded position p with (p >> 2) & 1) come out of the PV MMA four times too large and are
// scaled back once per work item (v_position_scale).
template <int BITS, int D>
__device__ inline void expand_words_v(const uint32_t (&w)[D * BITS / 32], uint32_t (&out)[D / 4]) {
  if constexpr (BITS == 2) {
#pragma unroll
    for (int i = 0; i < D * BITS / 32; ++i) {
      const uint32_t hi = w[i] >> 4;
      out[4 * i + 0] = w[i] & 0x03030303u;
      out[4 * i + 1] = w[i] & 0x0C0C0C0Cu;
      out[4 * i + 2] = hi & 0x03030303u;
      out[4 * i + 3] = hi & 0x0C0C0C0Cu;
    }
  } else {
    expand_words<BITS, D>(w, out);
  }
}
template <int BITS>
__device__ inline float v_position_scale(int pos) {
  return BITS == 2 && ((pos >> 2) & 1) ? 0.25f : 1.f;
}

// Final value to the output tensor in its dtype.
__device__ __forceinline__ void store_value(void* out, int out_dtype, long long idx, float val) {
  if (out_dtype == 0) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(val);
  else if (out_dtype == 1) static_cast<__half*>(out)[idx] = __float2half_rn(val);
  else static_cast<float*>(out)[idx] = val;
}

// Merge of a split unit's partials: the arithmetic and slot order of merge_kernel. Heads h0,
// h0 + hstep, ... (< gp) of the unit's head tile, HU of them at a time with their loads going
// out together (the head_dim 256 kernel, where one group merges all eight heads of both channel
// halves, takes two: 130 against 136 us on its token-wise workload; four cost more in registers
// than they saved); the calling thread takes channel `ch`. Called
// by whole warps whose threads all work on the same heads: the slots' (m, l) pairs are fetched
// one per lane (the unit has at most 64 pieces) and handed round by shuffles, and the slots' o
// values eight at a time, so that a merge costs a few memory round trips whatever the piece
// count. Kept out of line: it runs a few times per launch.
template <bool MQ, int HU>
static __device__ __noinline__ void merge_unit_partials(const DecodeParams& P, int d, int gp, int ch,
                                                 bool writes_lse, int k, int b, int kvh, int ht,
                                                 int h0, int hstep) {
  constexpr float LN2 = 0.6931471805599453f;
  __threadfence();
  const long long rows = static_cast<long long>(P.a.batch) * P.a.num_qo_heads;
  const int lane = threadIdx.x & 31;
  if (k > 64) k = 64;
#pragma unroll 1
  for (int hb = h0; hb < gp; hb += hstep * HU) {
    int hl[HU];
    bool on[HU];
    long long row[HU];
#pragma unroll
    for (int u = 0; u < HU; ++u) {
      const int h = hb + u * hstep;
      hl[u] = ht * 8 + h;
      on[u] = h < gp && hl[u] < P.heads_per_kv;
      row[u] = static_cast<long long>(b) * P.a.num_qo_heads +
               (static_cast<long long>(kvh) * P.heads_per_kv + hl[u]);
    }
    // slot s: lane s % 32, word s / 32
    float ms[HU][2], ls[HU][2];
#pragma unroll
    for (int u = 0; u < HU; ++u)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int s = lane + 32 * j;
        const bool have = on[u] && s < k;
        ms[u][j] = have ? __ldcg(P.a.m_partial + s * rows + row[u]) : -INFINITY;
        ls[u][j] = have ? __ldcg(P.a.l_partial + s * rows + row[u]) : 0.f;
      }
    // With several heads at a time (the head_dim 256 kernel) the first eight slots' o values are
    // requested together with the (m, l) pairs: a unit of up to eight pieces then costs one
    // memory round trip, not two in sequence. In the head_dim 64/128 kernel the same order
    // measured 1 to 3 % slower on its many-item workload (register allocation of the kernel
    // around this out-of-line function), so there the fetch stays inside the loop.
    constexpr bool EARLY = HU > 1;
    float os[HU][8];
    auto fetch = [&](int s0) {
#pragma unroll
      for (int u = 0; u < HU; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i)
          os[u][i] = on[u] && s0 + i < k
                         ? __ldcg(P.a.o_partial + ((s0 + i) * rows + row[u]) * d + ch) : 0.f;
    };
    if constexpr (EARLY) fetch(0);
    float M[HU], wl[HU][2], den[HU], acc[HU];
#pragma unroll
    for (int u = 0; u < HU; ++u) {
      M[u] = fmaxf(ms[u][0], ms[u][1]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) M[u] = fmaxf(M[u], __shfl_xor_sync(0xFFFFFFFFu, M[u], o));
      // this lane's slots' weights (0 for a slot past k or without a maximum)
#pragma unroll
      for (int j = 0; j < 2; ++j)
        wl[u][j] = (M[u] > -INFINITY && lane + 32 * j < k) ? exp2f(ms[u][j] - M[u]) : 0.f;
      den[u] = acc[u] = 0.f;
    }
#pragma unroll 1
    for (int s0 = 0; s0 < k; s0 += 8) {
      if (!EARLY || s0 > 0) fetch(s0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int s = s0 + i;                     // (warp-uniform)
#pragma unroll
        for (int u = 0; u < HU; ++u) {
          const float wgt = __shfl_sync(0xFFFFFFFFu, s < 32 ? wl[u][0] : wl[u][1], s & 31);
          const float lv = __shfl_sync(0xFFFFFFFFu, s < 32 ? ls[u][0] : ls[u][1], s & 31);
          if (s < k) {
            den[u] += wgt * lv;
            acc[u] += wgt * os[u][i];
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < HU; ++u) {
      if (!on[u]) continue;
      const bool live = den[u] > 0.f;
      const long long orow = caller_row<MQ>(P, b, kvh, hl[u]);
      store_value(P.a.out, P.a.out_dtype, orow * d + ch,
                  live ? acc[u] / den[u] * P.a.o_scale : 0.f);
      if (writes_lse && P.a.lse != nullptr)
        P.a.lse[orow] = live ? (M[u] + log2f(den[u])) * LN2 : -INFINITY;
    }
  }
}

}  // namespace fq
