// Paged GQA decode attention over packed INT2/INT4 KV at head_dim 256, sm_100a.
//
// Same arithmetic as the head_dim 64/128 kernel (decode.cu; reference semantics
// src/foscar/wrapper.py:1153-1171, fold algebra src/foscar/_sm100/int_fold_decode.py:5-22,
// 378-434; the reference tiles head_dim 256 as two K/V boxes per page,
// src/foscar/_sm100/int_fold_decode.py:1509-1530, 3316-3413). A token's operand row is 256 bytes,
// two 128-byte rows of a tensor-memory lane (K) and two planes of the group's shared-memory stage
// (V, one per half of the channels), so the structure is laid out anew around that:
//
//   tiles         128 tokens = two pages = two ring stages of one page each; thread t of a worker
//                 group owns token t (stage t / 64, row t % 64)
//   S             one chain of eight K steps over the lane's two operand rows against a query
//                 stage of two 128-byte-swizzled atoms (channels 0-127, 128-255)
//   PV            two chains of four K steps, one per channel half, against the same P rows into
//                 two accumulators of 16 columns
//   O             accumulates in TENSOR MEMORY over the group's tiles of a work item (the PV MMA's
//                 accumulate flag); the group keeps (m, l, c) in registers and rescales O in
//                 place on the rare tile that raises its reference
//   work items    flow through the groups without a CTA-wide barrier: a group that has finished
//                 its last tile of an item leaves (m, warp sums of l and c) in the item's state
//                 slot, reports, and goes on; its next item accumulates into its other O buffer.
//                 The group with the item's last tile waits for the reports, reads every group's
//                 accumulator out of tensor memory (a warp reaches its lane quarter of any
//                 column), merges the groups in the fixed order of their last tiles and writes
//                 the output row, or the partials of a split piece (counted in on the unit's
//                 counter after the group's next tile; the piece that completes a unit merges it)
//
// Three worker groups (the expanded V operand of a tile is 32 KB), two producers, two MMA
// issuers: 16 warps, 128 registers a thread.
//
// K quantized per channel over the 64 tokens of a page (the reference's
// (("channel", 64), ("token", 256)) layout, src/foscar/_sm100/int_fold_decode.py:613-618,
// 5012-5133): the page's (s_d, z_d) fold into the query side, so the S MMA's B operand differs
// per page. Each group builds it per tile in its own stage: 48 rows = for each of the tile's two
// pages three E4M3 planes (p0 + p1/16 + p2/256) of s_d q_d 2^-m for up to 8 heads (the reference
// rounds Q' to one plane), S has 24 columns per page, and the bias sum_d z_d q_d is reduced per
// page over the group. Two worker groups in that build.
#include "decode.cuh"

namespace fq {
namespace wide {

#ifdef FQ_WAIT_PROFILE
// Diagnostic builds only: (start, end, SM id) of every CTA, times on the global timer,
// [gridDim.x][3]; and the cycles lane 0 of each role spent in each of its waits,
// [gridDim.x][6 roles][16 sites].
__device__ unsigned long long* g_cta_times = nullptr;
__device__ long long* g_wide_waits = nullptr;
#define WT_BEGIN() long long wt_[16] = {}
#define WT(site, ...)                          \
  do {                                         \
    const long long a_ = clock64();            \
    __VA_ARGS__;                               \
    wt_[site] += clock64() - a_;               \
  } while (0)
#define WT_MARK(var) const long long var = clock64()
#define WT_SINCE(site, var) wt_[site] += clock64() - (var)
#define WT_FLUSH(role)                                                           \
  do {                                                                           \
    if (g_wide_waits != nullptr)                                                 \
      for (int i_ = 0; i_ < 16; ++i_)                                            \
        g_wide_waits[(blockIdx.x * 6 + (role)) * 16 + i_] = wt_[i_];             \
  } while (0)
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#endif

#ifndef FQ_WAIT_PROFILE
#define WT_BEGIN() ((void)0)
#define WT(site, ...) do { __VA_ARGS__; } while (0)
#define WT_MARK(var) ((void)0)
#define WT_SINCE(site, var) ((void)0)
#define WT_FLUSH(role) ((void)0)
#endif

constexpr int D = 256;
constexpr int SPT = 2;                     // ring stages (pages) per tile
// worker groups: three; two when K is quantized per channel (the groups' own query stages and
// the larger scale blocks take the third group's shared memory)
__host__ __device__ constexpr int groups_of(bool kch) { return kch ? 2 : 3; }
__host__ __device__ constexpr int threads_of(bool kch) { return 32 * (4 * groups_of(kch) + 4); }

template <int BITS, bool KCH>
struct Plan {
  static constexpr int G = groups_of(KCH);
  static constexpr int RB = D * BITS / 8;            // code row bytes: 64 or 128
  static constexpr int CHUNKS = RB / 16;             // 4 or 8
  // chunk c of ring row r sits at chunk c ^ row_swizzle(r): eight consecutive rows read at the
  // same chunk index then fall on different banks
  __host__ __device__ static constexpr int row_swizzle(int row) {
    return CHUNKS == 8 ? (row & 7) : (row >> 1) & 3;
  }
  static constexpr int CODE_PAGE = PAGE * RB;
  // records of a page in a ring stage: 16 bytes a token, or (K per channel) the block of
  // [128 + 2 D] f32: V ring, then the channel rows s_d, z_d
  static constexpr int SCALE_PAGE = KCH ? (2 * PAGE + 2 * D) * 4 : PAGE * 16;
  static constexpr int K_OFF = 0, V_OFF = CODE_PAGE, S_OFF = 2 * CODE_PAGE;
  static constexpr int STAGE = 2 * CODE_PAGE + SCALE_PAGE;
  static constexpr int ROW = 128;
  static constexpr int VOP_PLANE = TILE * ROW;         // one channel half of a tile's V operand
  static constexpr int VOP_STAGE = 2 * VOP_PLANE;
  static constexpr int Q_ATOM = 16 * ROW;              // 16 query rows x 128 bytes
  static constexpr int Q_BYTES = 2 * Q_ATOM;
  // K per channel: the S MMA's B operand is built per tile by the group itself (QP: 48 rows,
  // 24 per page = three E4M3 planes of 8 heads, two atoms of 48 x 128 bytes); the producer
  // stages the raw query rows (QRAW)
  static constexpr int QP_ROWS = 48;
  static constexpr int QP_ATOM = QP_ROWS * ROW;
  static constexpr int QP_BYTES = 2 * QP_ATOM;
  static constexpr int QRAW_BYTES = 8 * D;
  static constexpr int P_BYTES = TILE * 16;
  static constexpr int VOP_OFF = 0;
  static constexpr int Q_OFF = VOP_OFF + G * VOP_STAGE;
  static constexpr int QRAW_OFF = Q_OFF + G * QP_BYTES;             // (K per channel)
  static constexpr int P_OFF = KCH ? QRAW_OFF + 2 * QRAW_BYTES : Q_OFF + 2 * Q_BYTES;
  static constexpr int RED_OFF = P_OFF + G * P_BYTES;              // column maxima [G][4][8]
  static constexpr int STATS_OFF = RED_OFF + 128 * G;              // page statistics [G][2][2][12]
  static constexpr int HEADK_OFF = STATS_OFF + (KCH ? 192 * G : 0);  // per-warp head constants
  static constexpr int HEADC_OFF = HEADK_OFF + 96 * 4 * G;         // producer's, two items
  static constexpr int META_WORDS = 72;                            // m[8], 4 x (l[8], c[8])
  static constexpr int STATE_OFF = HEADC_OFF + 192;
  static constexpr int STATE_BYTES = 2 * G * META_WORDS * 4;
  static constexpr int BAR_OFF = (STATE_OFF + STATE_BYTES + 7) / 8 * 8;
  static constexpr int MAX_STAGES = 20;
  static constexpr int BAR_WORDS = 2 * MAX_STAGES + 4 + 4 * G;
  static constexpr int FLAG_OFF = (BAR_OFF + 8 * BAR_WORDS + 15) / 16 * 16;
  static constexpr int ITEM_OFF = (FLAG_OFF + 96 + 31) / 32 * 32;
  static constexpr int ITEM_SLOTS = 16;
  static constexpr int RING_OFF = (ITEM_OFF + 32 * ITEM_SLOTS + 1023) / 1024 * 1024;
  static constexpr int max_ring_stages() { return (SMEM_LIMIT - 1024 - RING_OFF) / STAGE; }
  // tensor memory (f32 columns) per group: K operand 64, S 16 (K per channel: 24 per page, 64
  // reserved), two O accumulators of 32
  static constexpr int KOP_COLS = 64, S_COLS = KCH ? 64 : 16, O_COLS = 32;
  static constexpr int T_KOP = 0, T_S = G * KOP_COLS, T_O = T_S + G * S_COLS;
  static constexpr int T_USED = T_O + G * 2 * O_COLS;
  static_assert(T_USED <= 512, "tensor memory plan exceeds 512 columns");
};

struct Bars {
  uint32_t base;
  int ns;
  int G;
  __device__ uint32_t at(int i) const { return base + 8u * i; }
  __device__ uint32_t ring_full(int s) const { return at(s); }
  __device__ uint32_t ring_empty(int s) const { return at(ns + s); }
  __device__ uint32_t q_full(int s) const { return at(2 * ns + s); }
  __device__ uint32_t q_empty(int s) const { return at(2 * ns + 2 + s); }
  // per worker group; a group's n-th tile uses phase n & 1 (see decode.cu)
  __device__ uint32_t k_ready(int g) const { return at(2 * ns + 4 + g); }
  __device__ uint32_t s_done(int g) const { return at(2 * ns + 4 + G + g); }
  __device__ uint32_t pv_ready(int g) const { return at(2 * ns + 4 + 2 * G + g); }
  __device__ uint32_t pv_done(int g) const { return at(2 * ns + 4 + 3 * G + g); }
};

struct RingPos {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next(int ns) {
    if (++s == ns) { s = 0; ph ^= 1u; }
  }
  __device__ __forceinline__ void advance(int k, int ns) {
    s += k;
    while (s >= ns) { s -= ns; ph ^= 1u; }
  }
};

// A quarter of a token row (64 channels) as packed words; chunk v of the row sits at chunk
// v ^ swz. (The row is taken a quarter at a time in loops that are not unrolled: see the tile
// loop.)
template <int BITS>
__device__ inline void load_quarter_row(uint32_t row_addr, int quarter, int swz, uint32_t* w) {
  constexpr int QC = D * BITS / 8 / 64;   // 16-byte chunks per quarter row: 1 or 2
#pragma unroll
  for (int v = 0; v < QC; ++v)
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w[4 * v]), "=r"(w[4 * v + 1]), "=r"(w[4 * v + 2]), "=r"(w[4 * v + 3])
                 : "r"(row_addr + (((quarter * QC + v) ^ swz) << 4)));
}
// packed words of 64 channels -> 16 words of exact E4M3 operand bytes (expansion order)
template <int BITS>
__device__ inline void expand_quarter(const uint32_t* w, uint32_t* out, bool v_operand) {
  constexpr int NW = 64 * BITS / 32;
  if (BITS == 2 && v_operand) {
    // odd output words keep their codes two bits up (4 * code, still exact); see decode.cuh
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      const uint32_t hi = w[i] >> 4;
      out[4 * i + 0] = w[i] & 0x03030303u;
      out[4 * i + 1] = w[i] & 0x0C0C0C0Cu;
      out[4 * i + 2] = hi & 0x03030303u;
      out[4 * i + 3] = hi & 0x0C0C0C0Cu;
    }
  } else {
    constexpr uint32_t MASK = BITS == 2 ? 0x03030303u : 0x0F0F0F0Fu;
    constexpr int PER = 8 / BITS;
#pragma unroll
    for (int i = 0; i < NW; ++i)
#pragma unroll
      for (int k = 0; k < PER; ++k) out[PER * i + k] = (w[i] >> (BITS * k)) & MASK;
  }
}

// A split piece's count-in on its unit's counter, and the merge of the unit if the count is then
// complete. Called by all 128 threads of the group that wrote the piece's partials, some time
// after the stores: the barrier orders the group's stores before thread 0's release fence and
// atomic. Thread t merges channels t and 128 + t.
template <int BITS, bool MQ>
__device__ __noinline__ void count_in_piece(const DecodeParams& P, int gp, int wg, int t, int b,
                                            int kvh, int ht, volatile int* group_info) {
  named_barrier(1 + wg, 128);
  if (t == 0) {
    const int unit = (b * P.p.num_kv_heads + kvh) * P.head_tiles + ht;
    const int k = P.a.split_counts != nullptr ? __ldg(P.a.split_counts + unit) : P.a.kv_splits;
    __threadfence();
    const int seen = atomicAdd(P.a.unit_counters + unit, 1);
    if (seen == k - 1) P.a.unit_counters[unit] = 0;   // untouched until the next launch
    group_info[wg] = seen == k - 1 ? k : 0;
  }
  named_barrier(1 + wg, 128);
  const int k = group_info[wg];
  if (k > 0) {
    const int ch = channel_of_expanded_pos<BITS>(t);
    merge_unit_partials<MQ, 2>(P, D, gp, ch, t == 0, k, b, kvh, ht, 0, 1);
    merge_unit_partials<MQ, 2>(P, D, gp, 128 + ch, false, k, b, kvh, ht, 0, 1);
  }
}

// The request's last tile with several query tokens per request: column h sees positions below
// len - lag(h) only. Out of line, so that this rare path (and column_lag's division) costs the
// tile loop nothing. Returns, in `over`, the largest visible score (already relative to the
// column's reference).
template <int GP>
__device__ __noinline__ void mask_lagged_columns(const DecodeParams& P, int len, int ht, int pos,
                                                 float (&d)[GP], float& over) {
  float top = -INFINITY;
  for (int h = 0; h < GP; ++h) {
    if (pos >= len - column_lag(P, ht * 8 + h)) d[h] = -INFINITY;
    top = fmaxf(top, d[h]);
  }
  over = top;
}

template <int BITS, int GP, bool KCH, bool MQ>
__device__ __forceinline__ void worker_role(const DecodeParams& P, uint8_t* smem, uint32_t smem0,
                                            uint32_t tmem, const Bars& bars,
                                            volatile int* abort_flag, const ItemRange items) {
  using SP = Plan<BITS, KCH>;
  constexpr int G = SP::G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2, wq = warp & 3;
  const int t = threadIdx.x & 127;   // token row while unpacking and in softmax, channel in O
  const int NS = P.ring_stages;
  int* status = P.a.status;
  const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
  const uint32_t ring0 = smem0 + SP::RING_OFF;
  const uint32_t k_dst = tmem + lane_base + SP::T_KOP + wg * SP::KOP_COLS;
  const uint32_t s_src = tmem + lane_base + SP::T_S + wg * SP::S_COLS;
  const uint32_t o_lane = tmem + lane_base + SP::T_O;
  // this thread's V operand row with its swizzle phase folded in: chunk cc of the row sits at
  // v_row ^ (cc << 4)
  const uint32_t v_row = (smem0 + SP::VOP_OFF + wg * SP::VOP_STAGE + t * SP::ROW) |
                         static_cast<uint32_t>((t & 7) << 4);
  const uint32_t p_row = smem0 + SP::P_OFF + wg * SP::P_BYTES + t * 16;
  float* red_max = reinterpret_cast<float*>(smem + SP::RED_OFF);   // [wg][warp][8]
  float* head_k = reinterpret_cast<float*>(smem + SP::HEADK_OFF) + warp * 24;
  const volatile float* head_const =
      reinterpret_cast<const volatile float*>(smem + SP::HEADC_OFF);  // [2][24]
  volatile int* done_warps = reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF + 32);  // [2]
  volatile int* finished = reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF + 40);    // [2]
  volatile int* q_staged = reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF + 48);
  volatile int* group_info = reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF + 64);  // [G]
  constexpr float LN2 = 0.6931471805599453f;

  // pool-wide P-scale exponent from the count table: lp = 135 - max(top nonzero bin, 27)
  int lp;
  {
    int top = 0;
    if (P.p.v_max_hist != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int bin = lane * 8 + i;
        if (__ldg(P.p.v_max_hist + bin) != 0u) top = bin;
      }
    }
    top = __reduce_max_sync(0xFFFFFFFFu, top);
    lp = 135 - max(top, 27);
  }
  constexpr float MAX_LAG = 3.f;   // the group's reference may lag the true maximum by this much
  lp -= static_cast<int>(MAX_LAG);
  const float p2lp = exp2f(static_cast<float>(lp));
  const float o_mul = exp2f(static_cast<float>(9 - lp));

  WT_BEGIN();
  WT_MARK(role_t0);
  bool piece_pending = false;   // a split piece written but not yet counted in
  int piece_b = 0, piece_kvh = 0, piece_ht = 0;

  int qi = 0;       // non-empty items so far
  int it0 = 0;      // running index of the next item's first tile (every role counts alike)
  int mine = wg;    // running index of this group's next tile
  int n = 0;        // tiles this group has taken: the phase of its barriers
  RingPos rp;       // ring position of tile `mine`'s first stage
  rp.advance(SPT * wg, NS);
  const WorkItem* const item_cache = reinterpret_cast<const WorkItem*>(smem + SP::ITEM_OFF);
  const WorkItem* const item_more =
      reinterpret_cast<const WorkItem*>(smem + SP::RING_OFF + NS * SP::STAGE);
  const int su = t >> 6, srow = t & 63;   // this thread's ring stage of a tile and row in it
  for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
    const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
    const int nt = max(w.t1 - w.t0, 0);
    const int first = mine - it0;
    const int mytiles = first < nt ? (nt - 1 - first) / G + 1 : 0;
    // an item without tiles (an empty request) is finished by the group whose turn is next
    const bool closes_empty = nt == 0 && (it0 % G) == wg;
    const int qb = qi & 1;
    const int q_index = qi;
    const int item_t0 = it0;
    if (nt > 0) ++qi;
    it0 += nt;
    if (mytiles == 0 && !closes_empty) continue;
    // The groups that have tiles in the item, in the order of their last tiles: position p is
    // group (item_t0 + max(0, nt - G) + p) % G. The last of them finishes the item.
    const int parts = nt == 0 ? 1 : min(G, nt);
    const int pos = nt == 0 ? 0 : first + (mytiles - 1) * G - max(0, nt - G);
    const int par = ik & 1;   // which O accumulator and state slot the item uses
    const uint32_t o_src = o_lane + (wg * 2 + par) * SP::O_COLS;
    float* meta = reinterpret_cast<float*>(smem + SP::STATE_OFF) + (par * G + wg) * SP::META_WORDS;

    float m[GP], l[GP], c[GP];
#pragma unroll
    for (int h = 0; h < GP; ++h) { m[h] = -INFINITY; l[h] = 0.f; c[h] = 0.f; }
    // The item's per-head constants come from the first producer, which staged the query rows.
    // Only a group with a tile in the item waits for them, and on a count of staged items: a
    // group without tiles in the items before may be several stagings ahead of the producer,
    // where a phase-parity wait would take an older phase for the one it needs.
    __syncwarp();
    if (lane == 0 && mytiles > 0) {
      WT(0, count_wait(q_staged, q_index + 1, abort_flag, status));
      __threadfence_block();
    }
    __syncwarp();
    if (mytiles > 0 && lane < 24) head_k[lane] = head_const[qb * 24 + lane];
    __syncwarp();
    // K per channel: this thread builds four positions (4 * (t % 64) ...) of its page's half of
    // the S MMA's B operand; it keeps the item's query values at those positions
    float qf[KCH ? GP : 1][4];
    if constexpr (KCH) {
      if (mytiles > 0) {
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const uint32_t raw = *reinterpret_cast<const uint32_t*>(
              smem + SP::QRAW_OFF + qb * SP::QRAW_BYTES + h * D + 4 * srow);
          const float2 a = e4m3x2_to_f32x2(raw & 0xFFFF), b = e4m3x2_to_f32x2(raw >> 16);
          qf[h][0] = a.x; qf[h][1] = a.y; qf[h][2] = b.x; qf[h][3] = b.y;
        }
      }
    }

    bool pending = false;   // the group has a PV MMA of this item in flight or done
    for (int done = 0; done < mytiles; ++done, mine += G, rp.advance(SPT * G, NS), ++n) {
      const int tt = w.t0 + (mine - item_t0);
      RingPos rp1 = rp;
      rp1.next(NS);
      const uint32_t stage = ring0 + (su ? rp1.s : rp.s) * SP::STAGE;
      WT(1, mbar_wait(bars.ring_full(rp.s), rp.ph, abort_flag, status);
         mbar_wait(bars.ring_full(rp1.s), rp1.ph, abort_flag, status));
      // ---- K per channel: the page's (s_d, z_d) fold into the query side. Per page and head
      //   score = 2^m * (sum_d Q'_d c_d) + sum_d z_d q_d,   Q'_d = s_d q_d 2^-m as three E4M3 planes
      // p0 + p1/16 + p2/256 (the reference's Q' and bias, src/foscar/_sm100/int_fold_asm.py:21-63,
      // src/foscar/_sm100/int_fold_decode.py:5038-5133, round Q' to one plane; with outlier
      // channels two planes still left 1e-2 on a score, three leave 1e-3), m from
      // the bound max_d s_d * max_d |q_d| so that one number per page is reduced, not one per
      // head. The group builds the operand (48 rows: three planes of up to 8 heads for each of
      // the tile's two pages) in its own stage; its previous tile's S MMA, the stage's last reader,
      // is complete (the group read that S).
      float up[KCH ? GP : 1], ab[KCH ? GP : 1];   // per head: 2^m * 512 * A, and A * bias
      if constexpr (KCH) {
        const int pos0 = 4 * srow;                      // first of this thread's four positions
        const uint32_t rec = stage + SP::S_OFF;         // [V ring 128 | s_d 256 | z_d 256]
        float sd[4], zd[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ch = (pos0 & 128) + channel_of_expanded_pos<BITS>((pos0 & 127) + i);
          if (P.p.scale_bf16) {
            const uint16_t a = *reinterpret_cast<const uint16_t*>(
                smem + (rec - smem0) + (2 * PAGE + ch) * 2);
            const uint16_t b = *reinterpret_cast<const uint16_t*>(
                smem + (rec - smem0) + (2 * PAGE + D + ch) * 2);
            sd[i] = __uint_as_float(static_cast<uint32_t>(a) << 16);
            zd[i] = __uint_as_float(static_cast<uint32_t>(b) << 16);
          } else {
            sd[i] = *reinterpret_cast<const float*>(smem + (rec - smem0) + (2 * PAGE + ch) * 4);
            zd[i] = *reinterpret_cast<const float*>(smem + (rec - smem0) + (2 * PAGE + D + ch) * 4);
          }
        }
        float* stats = reinterpret_cast<float*>(smem + SP::STATS_OFF) + ((wg * 2 + su) * 2 + (wq & 1)) * 12;
        {
          const uint32_t smax_bits = __reduce_max_sync(
              0xFFFFFFFFu, __float_as_uint(fmaxf(fmaxf(sd[0], sd[1]), fmaxf(sd[2], sd[3]))));
          if (lane == 0) stats[0] = __uint_as_float(smax_bits);
#pragma unroll
          for (int h = 0; h < GP; ++h) {
            float bp = fmaf(zd[0], qf[h][0], fmaf(zd[1], qf[h][1],
                                                 fmaf(zd[2], qf[h][2], zd[3] * qf[h][3])));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) bp += __shfl_xor_sync(0xFFFFFFFFu, bp, o);
            if (lane == 0) stats[1 + h] = bp;
          }
        }
        named_barrier(1 + wg, 128);
        const float* st0 = reinterpret_cast<const float*>(smem + SP::STATS_OFF) + (wg * 2 + su) * 2 * 12;
        const float smax = fmaxf(st0[0], st0[12]);
        // rows 24 * page + 8 * plane + h of the group's operand stage; atom = channel half
        const uint32_t qp = smem0 + SP::Q_OFF + wg * SP::QP_BYTES + (pos0 >> 7) * SP::QP_ATOM +
                            (pos0 & 15);
        const int chunk = (pos0 & 127) >> 4;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          // m = floor(log2(smax * qamax)) - 7, so that |s_d q_d| 2^-m < 256
          const uint32_t eb = min(max((__float_as_uint(smax * head_k[8 + h]) >> 23) & 0xFFu, 40u),
                                  214u);
          const float dn = __uint_as_float((261u - eb) << 23);       // 2^-m = 2^(134 - e)
          const float upm = __uint_as_float((eb - 7u) << 23);        // 2^m  = 2^(e - 134)
          up[h] = upm * 512.f * head_k[h];
          ab[h] = head_k[h] * (st0[1 + h] + st0[13 + h]);
          float y[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) y[i] = sd[i] * qf[h][i] * dn;
          // y = p0 + p1 / 16 + p2 / 256, each plane the E4M3 rounding of what is left; this
          // thread's four positions of a plane go straight to the stage (the plane loop is not
          // unrolled: code size, see the K rows below)
#pragma unroll 1
          for (int k = 0; k < 3; ++k) {
            const uint32_t a = f32x2_to_e4m3x2(y[0], y[1]), b = f32x2_to_e4m3x2(y[2], y[3]);
            const int r = 24 * su + 8 * k + h;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(qp + r * 128 + ((chunk ^ (r & 7)) << 4)),
                         "r"(a | (b << 16)) : "memory");
            const float2 fa = e4m3x2_to_f32x2(a), fb = e4m3x2_to_f32x2(b);
            y[0] = (y[0] - fa.x) * 16.f; y[1] = (y[1] - fa.y) * 16.f;
            y[2] = (y[2] - fb.x) * 16.f; y[3] = (y[3] - fb.y) * 16.f;
          }
        }
        fence_proxy_async();
      }
      // ---- K row -> tensor memory, two 128-byte operand rows (the S MMA's A operand). The
      // columns are free: this group read the S of its previous tile, so that tile's MMA, their
      // last reader, is complete.
      tc_fence_after();
      // (a row goes a quarter at a time in a loop that is NOT unrolled, here and for V below: the
      // tile loop's code is large for the instruction cache with three or four warps a scheduler;
      // rolling these loops took 4 to 5 % off the launch)
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t wk[64 * BITS / 32], op[16];
        load_quarter_row<BITS>(stage + SP::K_OFF + srow * SP::RB, qd, SP::row_swizzle(srow), wk);
        expand_quarter<BITS>(wk, op, false);
        tmem_st16(k_dst + 16 * qd, op);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars.k_ready(wg));
      // the group's previous PV MMA must be complete before its V stage and P rows are rewritten
      if (pending) {
        WT(2, mbar_wait(bars.pv_done(wg), (n - 1) & 1, abort_flag, status));
        tc_fence_after();
      }
      // ---- V row -> the group's shared-memory stage, one 128-byte-swizzled plane per channel half
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t wv[64 * BITS / 32], op[16];
        load_quarter_row<BITS>(stage + SP::V_OFF + srow * SP::RB, qd, SP::row_swizzle(srow), wv);
        expand_quarter<BITS>(wv, op, true);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                           (v_row ^ static_cast<uint32_t>((4 * (qd & 1) + cc) << 4)) +
                           (qd >> 1) * SP::VOP_PLANE),
                       "r"(op[4 * cc]), "r"(op[4 * cc + 1]), "r"(op[4 * cc + 2]),
                       "r"(op[4 * cc + 3])
                       : "memory");
        }
      }
      // the token's record; then both ring stages go back to the producers
      float sk = 0.f, zk = 0.f, sv, zv;
      if constexpr (KCH) {   // V ring at the front of the page's block
        if (P.p.scale_bf16) {
          uint32_t vr;
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(vr) : "r"(stage + SP::S_OFF + srow * 4));
          sv = __uint_as_float(vr << 16); zv = __uint_as_float(vr & 0xFFFF0000u);
        } else {
          asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(sv), "=f"(zv)
                       : "r"(stage + SP::S_OFF + srow * 8));
        }
      } else if (P.p.scale_bf16) {   // (s, z) as bf16 pairs, 8 bytes a token
        uint32_t kr, vr;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(kr), "=r"(vr)
                     : "r"(stage + SP::S_OFF + srow * 8));
        sk = __uint_as_float(kr << 16); zk = __uint_as_float(kr & 0xFFFF0000u);
        sv = __uint_as_float(vr << 16); zv = __uint_as_float(vr & 0xFFFF0000u);
      } else {
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(sk), "=f"(zk), "=f"(sv), "=f"(zv)
                     : "r"(stage + SP::S_OFF + srow * 16));
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bars.ring_empty(rp.s));
        mbar_arrive(bars.ring_empty(rp1.s));
      }
      // positions past the request's length (its last tile only): score -inf, record neutral
      // (with several query tokens a column stops short of the request's last positions)
      const bool whole = (tt + 1) * TILE <= w.len - (MQ ? P.q_len - 1 : 0);
      const bool valid = whole || tt * TILE + t < w.len;
      const float ak = sk * 512.f;
      (void)ak; (void)zk;
      const float wsc = valid ? sv * p2lp : 0.f;
      if (!valid) zv = 0.f;
      // ---- raw scores; d = score - reference in one fused chain per head. The group's first
      // tile of an item has no reference yet: it takes the scores themselves and always goes
      // through the exact maximum. Otherwise the reference may lag by MAX_LAG, and only a tile
      // that exceeds it takes the exact column maximum and rescales l, c and O.
      WT(3, mbar_wait(bars.s_done(wg), n & 1, abort_flag, status));
      float d[GP];
      const bool fresh = !pending;
      {
        uint32_t raw[KCH ? 24 : 8];
        tc_fence_after();
        if constexpr (KCH) {   // the token's page's columns: three planes of eight heads
          tmem_ld8p(s_src + 24 * su, raw);
          tmem_ld8p(s_src + 24 * su + 8, raw + 8);
          tmem_ld8p(s_src + 24 * su + 16, raw + 16);
        } else {
          tmem_ld8p(s_src, raw);
        }
        tmem_ld_wait();
        tc_fence_before();
        float over = -INFINITY;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const float nm = fresh ? 0.f : -m[h];
          float dd;
          if constexpr (KCH)
            dd = fmaf(up[h],
                      fmaf(fmaf(__uint_as_float(raw[16 + h]), 0.0625f, __uint_as_float(raw[8 + h])),
                           0.0625f, __uint_as_float(raw[h])),
                      ab[h] + nm);
          else
            dd = fmaf(head_k[h] * ak, __uint_as_float(raw[h]), fmaf(head_k[8 + h], zk, nm));
          d[h] = valid ? dd : -INFINITY;
          over = fmaxf(over, d[h]);
        }
        if constexpr (MQ) {
          if (!whole) mask_lagged_columns<GP>(P, w.len, w.ht, tt * TILE + t, d, over);
        }
        if (fresh || named_barrier_or(1 + wg, 128, over > MAX_LAG)) {
          float* wmax = red_max + (wg * 4 + wq) * 8;
#pragma unroll
          for (int h = 0; h < GP; ++h) {
            const float wm = warp_max_f32(d[h]);
            if (lane == 0) wmax[h] = wm;
          }
          named_barrier(1 + wg, 128);
          const float* gm = red_max + wg * 4 * 8;
          float corr[GP];
#pragma unroll
          for (int h = 0; h < GP; ++h) {
            const float top = fmaxf(fmaxf(gm[h], gm[8 + h]), fmaxf(gm[16 + h], gm[24 + h]));
            const float shift = fresh ? top : fmaxf(top, 0.f);
            corr[h] = fresh ? 0.f : fast_exp2(-shift);
            l[h] *= corr[h];
            c[h] *= corr[h];
            m[h] = fresh ? shift : m[h] + shift;
            // (a column whose every score of the group's first tile is masked: only the
            // request's last tile, so the group has no further tile of this item)
            if constexpr (MQ) d[h] = shift == -INFINITY ? -INFINITY : d[h] - shift;
            else d[h] -= shift;
          }
          if (pending) {
            // every earlier tile's O of this item is complete in tensor memory: per channel half
            // columns h and 8 + h are head h's hi and lo sums
            tc_fence_after();
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              uint32_t o[16];
              tmem_ld16p(o_src + 16 * r, o);
              tmem_ld_wait();
#pragma unroll
              for (int h = 0; h < GP; ++h) {
                o[h] = __float_as_uint(__uint_as_float(o[h]) * corr[h]);
                o[8 + h] = __float_as_uint(__uint_as_float(o[8 + h]) * corr[h]);
              }
              tmem_st16(o_src + 16 * r, o);
            }
            tmem_st_wait();
            tc_fence_before();
          }
        }
      }
      // two heads per instruction in f16x2: p = 2^d, w = p * s_v 2^lp, E4M3 hi + lo/16
      uint32_t pw[4];
      {
        const __half2 wsc2 = __float2half2_rn(wsc);
        uint32_t hi[GP / 2], lo[GP / 2];
#pragma unroll
        for (int h = 0; h < GP; h += 2) {
          const __half2 e2 = h2_exp2(__floats2half2_rn(d[h], d[h + 1]));
          const float2 ef = __half22float2(e2);
          l[h] += ef.x;
          l[h + 1] += ef.y;
          c[h] = fmaf(ef.x, zv, c[h]);
          c[h + 1] = fmaf(ef.y, zv, c[h + 1]);
          const __half2 w2 = __hmul2(e2, wsc2);
          hi[h >> 1] = f16x2_to_e4m3x2(w2);
          const __half2 r2 =
              __hmul2(__hsub2(w2, e4m3x2_to_f16x2(hi[h >> 1])), __float2half2_rn(16.f));
          lo[h >> 1] = f16x2_to_e4m3x2(r2);
        }
        pw[0] = hi[0] | (hi[1] << 16);
        pw[2] = lo[0] | (lo[1] << 16);
        if constexpr (GP == 8) {
          pw[1] = hi[2] | (hi[3] << 16);
          pw[3] = lo[2] | (lo[3] << 16);
        } else {
          pw[1] = 0u;
          pw[3] = 0u;
        }
      }
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_row), "r"(pw[0]), "r"(pw[1]),
                   "r"(pw[2]), "r"(pw[3])
                   : "memory");
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        // The group's first PV MMA of the item starts its accumulator afresh: the item two
        // before this one, which used the same accumulator and state slot, must be finished.
        if (!pending) WT(4, count_wait(finished + par, ik >> 1, abort_flag, status));
        mbar_arrive(bars.pv_ready(wg));
      }
      pending = true;
      // a split piece finished before this tile is counted in now: its stores have drained
      if (piece_pending) {
        count_in_piece<BITS, MQ>(P, GP, wg, t, piece_b, piece_kvh, piece_ht, group_info);
        piece_pending = false;
      }
    }

    // ---- the group's part of the item is done
    if (pending) {
      WT(5, mbar_wait(bars.pv_done(wg), (n - 1) & 1, abort_flag, status));
      tc_fence_after();
    }
    if (mytiles == 0) {   // an item without tiles: its state slot must be free as well
      if (lane == 0) count_wait(finished + par, ik >> 1, abort_flag, status);
      __syncwarp();
    }
    {   // warp sums of l and c, and the group's reference, into the item's state slot
      float* wsum = meta + 8 + wq * 16;
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        float ls = l[h], cs = c[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          ls += __shfl_xor_sync(0xFFFFFFFFu, ls, o);
          cs += __shfl_xor_sync(0xFFFFFFFFu, cs, o);
        }
        if (lane == 0) { wsum[h] = ls; wsum[8 + h] = cs; }
        if (lane == 0 && wq == 0) meta[h] = m[h];
      }
    }
    const bool last = pos == parts - 1;
    if (!last) {
      // the group that holds the item's last tile reads this group's state and accumulator
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        atomicAdd(const_cast<int*>(done_warps) + par, 1);
      }
      continue;
    }
    // ---- this group holds the item's last tile: it finishes the item
    if (piece_pending) {   // (an item finished with no tile since the piece before it)
      count_in_piece<BITS, MQ>(P, GP, wg, t, piece_b, piece_kvh, piece_ht, group_info);
      piece_pending = false;
    }
    if (t == 0) {
      WT(7, count_wait(done_warps + par, 4 * (parts - 1), abort_flag, status));
      __threadfence_block();
    }
    WT_MARK(merge_t0);
    named_barrier(1 + wg, 128);
    tc_fence_after();
    // The groups' states meet in two steps. One thread per head takes the groups' references and
    // sums (in the fixed order of the groups' last tiles), fixes the item's reference and each
    // group's weight 2^(m_g - M) and leaves them in this group's own state slot; after a group
    // barrier every thread weighs the groups' accumulators of its two channels with them. (With
    // every thread redoing the per-head part, the four warps of the finishing group spent
    // 4.7 us per item here.)
    const int g_first = (item_t0 + max(0, nt - G)) % G;
    float* const fin = meta;   // this group's slot: [head][8] = weights of up to G groups, L, C, M
    if (t < GP) {
      const int h = t;
      float mg[G], lg[G], cg[G];
      float top = -INFINITY;
#pragma unroll
      for (int p = 0; p < G; ++p) {
        int g = g_first + p;
        if (g >= G) g -= G;
        if (nt == 0) g = wg;
        const float* gmeta =
            reinterpret_cast<const float*>(smem + SP::STATE_OFF) + (par * G + g) * SP::META_WORDS;
        const bool have = p < parts;
        mg[p] = have ? gmeta[h] : -INFINITY;
        lg[p] = have ? (gmeta[8 + h] + gmeta[24 + h]) + (gmeta[40 + h] + gmeta[56 + h]) : 0.f;
        cg[p] = have ? (gmeta[16 + h] + gmeta[32 + h]) + (gmeta[48 + h] + gmeta[64 + h]) : 0.f;
        top = fmaxf(top, mg[p]);
      }
      __syncwarp((1u << GP) - 1u);   // every head's thread has read this group's own slot
      float ls = 0.f, cs = 0.f;
#pragma unroll
      for (int p = 0; p < G; ++p) {
        const float wgt = mg[p] == -INFINITY ? 0.f : exp2f(mg[p] - top);
        ls = fmaf(wgt, lg[p], ls);
        cs = fmaf(wgt, cg[p], cs);
        fin[8 * h + p] = wgt;
      }
      fin[8 * h + 4] = ls;
      fin[8 * h + 5] = cs;
      fin[8 * h + 6] = top;
    }
    named_barrier(1 + wg, 128);
    float M[GP], L[GP], C[GP], O0[GP], O1[GP];   // O0 / O1: channels t and 128 + t
#pragma unroll
    for (int h = 0; h < GP; ++h) {
      O0[h] = O1[h] = 0.f;
      L[h] = fin[8 * h + 4];
      C[h] = fin[8 * h + 5];
      M[h] = fin[8 * h + 6];
    }
#pragma unroll 1
    for (int p = 0; p < parts; ++p) {
      int g = g_first + p;
      if (g >= G) g -= G;
      if (nt == 0) break;   // an empty request: no accumulator was written
      uint32_t r0[16], r1[16];
      tmem_ld16p(o_lane + (g * 2 + par) * SP::O_COLS, r0);
      tmem_ld16p(o_lane + (g * 2 + par) * SP::O_COLS + 16, r1);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        const float wgt = fin[8 * h + p];
        const float a0 = fmaf(__uint_as_float(r0[8 + h]), 0.0625f, __uint_as_float(r0[h]));
        const float a1 = fmaf(__uint_as_float(r1[8 + h]), 0.0625f, __uint_as_float(r1[h]));
        O0[h] = fmaf(wgt, a0, O0[h]);
        O1[h] = fmaf(wgt, a1, O1[h]);
      }
    }
    tc_fence_before();
    // The accumulators and the state slot are free for the item two further on. They are
    // released before the output goes to global memory.
    named_barrier(1 + wg, 128);
    if (t == 0) {
      done_warps[par] = 0;
      __threadfence_block();
      finished[par] = (ik >> 1) + 1;
    }
    if (w.slot != -2) {
      const int ch = channel_of_expanded_pos<BITS>(t);
      const float vps = o_mul * v_position_scale<BITS>(t);
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        const int hl = w.ht * 8 + h;
        if (hl >= P.heads_per_kv) continue;
        const float v0 = fmaf(O0[h], vps, C[h]), v1 = fmaf(O1[h], vps, C[h]);
        const long long head = static_cast<long long>(w.kvh) * P.heads_per_kv + hl;
        const long long row = static_cast<long long>(w.b) * P.a.num_qo_heads + head;
        if (w.slot < 0) {
          const long long orow = caller_row<MQ>(P, w.b, w.kvh, hl);
          const float inv = L[h] > 0.f ? P.a.o_scale / L[h] : 0.f;
          store_value(P.a.out, P.a.out_dtype, orow * D + ch, v0 * inv);
          store_value(P.a.out, P.a.out_dtype, orow * D + 128 + ch, v1 * inv);
          if (t == 0 && P.a.lse != nullptr)
            P.a.lse[orow] = L[h] > 0.f ? (M[h] + log2f(L[h])) * LN2 : -INFINITY;
        } else {
          const long long prow =
              static_cast<long long>(w.slot) * P.a.batch * P.a.num_qo_heads + row;
          P.a.o_partial[prow * D + ch] = v0;
          P.a.o_partial[prow * D + 128 + ch] = v1;
          if (t == 0) { P.a.l_partial[prow] = L[h]; P.a.m_partial[prow] = M[h]; }
        }
      }
      if (w.slot >= 0 && P.a.unit_counters != nullptr) {
        piece_pending = true;
        piece_b = w.b; piece_kvh = w.kvh; piece_ht = w.ht;
      }
    }
    WT_SINCE(9, merge_t0);
  }
  if (piece_pending)
    count_in_piece<BITS, MQ>(P, GP, wg, t, piece_b, piece_kvh, piece_ht, group_info);
  WT_SINCE(8, role_t0);
  if (t == 0) WT_FLUSH(wg);
}

template <int BITS, int GP, bool KCH, bool MQ>
__global__ void __launch_bounds__(threads_of(KCH), 1) decode_wide_kernel(const DecodeParams P) {
  using SP = Plan<BITS, KCH>;
  constexpr int G = SP::G;
  constexpr int W_PRODUCER = 4 * G, W_S = W_PRODUCER + 1, W_PV = W_PRODUCER + 2,
                W_PRODUCER2 = W_PRODUCER + 3;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem = smem_raw + (smem0 - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NS = P.ring_stages;
  Bars bars{smem0 + SP::BAR_OFF, NS, G};
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SP::FLAG_OFF + 24);
  int* status = P.a.status;
#ifdef FQ_WAIT_PROFILE
  if (threadIdx.x == 0 && g_cta_times != nullptr) {
    uint32_t smid;
    asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
    g_cta_times[3 * blockIdx.x] = global_ns();
    g_cta_times[3 * blockIdx.x + 2] = smid;
  }
#endif

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    set_wait_budget(abort_flag, P.wait_budget);
    volatile int* words = reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF + 32);
    // warps that have reported their part of an item [2], items finished [2], query stagings
    for (int i = 0; i < 5; ++i) words[i] = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(bars.ring_full(s), 32);  // one cp.async arrival per producer lane
      mbar_init(bars.ring_empty(s), 4);  // the four warps of the group that took the tile
    }
    for (int g = 0; g < G; ++g) {
      mbar_init(bars.k_ready(g), 4);
      mbar_init(bars.s_done(g), 1);
      mbar_init(bars.pv_ready(g), 4);
      mbar_init(bars.pv_done(g), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bars.q_full(s), 1);
      mbar_init(bars.q_empty(s), 1);
    }
    fence_barrier_init();
  }
  if (warp == W_S) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // see decode.cu: under a programmatic launch everything above may overlap the previous launch
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const ItemRange items = item_range(P);
  WorkItem* const item_cache = reinterpret_cast<WorkItem*>(smem + SP::ITEM_OFF);
  WorkItem* const item_more = reinterpret_cast<WorkItem*>(smem + SP::RING_OFF + NS * SP::STAGE);
  {
    const int k = threadIdx.x;
    const long long wi = items.begin + static_cast<long long>(k) * items.step;
    if (k < P.item_slots && wi < items.end) {
      const WorkItem w = decode_item(P, static_cast<int>(wi));
      if (k < SP::ITEM_SLOTS) item_cache[k] = w;
      else item_more[k - SP::ITEM_SLOTS] = w;
    }
  }
  __syncthreads();
  const uint32_t ring0 = smem0 + SP::RING_OFF;

  if (warp == W_PRODUCER || warp == W_PRODUCER2) {
    // ------------------------------------------------------------------ producers
    // Two warps take alternate ring stages; a stage is one page of one KV head (K codes, V
    // codes, scale records) as 16-byte cp.async copies from all lanes (see decode.cu). The first
    // producer also stages each item's query rows, in expansion order, as the S MMA's B operand.
    const int pi = warp == W_PRODUCER ? 0 : 1;
    const uint64_t stream_policy = l2_evict_first_policy();
    WT_BEGIN();
    WT_MARK(role_t0);
    int it = 0, qi = 0;
    RingPos rp;
    for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
      const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
      if (w.t1 <= w.t0) continue;
      const int npages = (w.len + PAGE - 1) / PAGE;
      const int first_page = SPT * w.t0, end_page = SPT * w.t1;
      const int pend = min(end_page, npages);
      auto fetch = [&](int pg0) {
        const int pg = pg0 + lane;
        int id = -1;
        if (pg < pend) {
          const long long e = static_cast<long long>(w.table_off) + pg;
          if (e >= 0 && e < P.a.table_len) id = __ldg(P.a.page_table + e);
          if (id < 0 || id >= P.p.num_pages) {
            id = -1;
            if (status) atomicOr(status, FQ_STATUS_BAD_PAGE);
          }
        }
        return id;
      };
      // (requested before the query rows are staged: the two global round trips overlap)
      int cur = fetch(first_page);
      if (pi == 0) {
        const int qb = qi & 1;
        WT(10, mbar_wait(bars.q_empty(qb), ((qi >> 1) & 1) ^ 1, abort_flag, status));
        // 16 rows of sixteen 16-byte chunks: a row's chunks sit in 16 neighbouring lanes
        // (K per channel: the 8 head rows only, unswizzled, for the workers to build the
        // operand from; the per-head constants are then the score scale and max |q|)
#pragma unroll
        for (int j = 0; j < (KCH ? 4 : 8); ++j) {
          const int chunk = lane + 32 * j;
          const int r = chunk >> 4, cc = chunk & 15;
          uint4 v = make_uint4(0, 0, 0, 0);
          const int hl = w.ht * 8 + r;
          const bool live = r < 8 && hl < P.heads_per_kv;
          const long long qrow = live ? caller_row<MQ>(P, w.b, w.kvh, hl) : 0;
          float qsum = 0.f;   // the row's sum of q (K per channel: its max |q|)
          if (live) {
            const uint4 in = __ldg(reinterpret_cast<const uint4*>(
                static_cast<const uint8_t*>(P.a.q) +
                qrow * D + 16 * cc));
            const uint32_t words[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 lo = e4m3x2_to_f32x2(words[i] & 0xFFFF);
              const float2 hi = e4m3x2_to_f32x2(words[i] >> 16);
              if constexpr (KCH)
                qsum = fmaxf(fmaxf(qsum, fmaxf(fabsf(lo.x), fabsf(lo.y))),
                             fmaxf(fabsf(hi.x), fabsf(hi.y)));
              else
                qsum += (lo.x + lo.y) + (hi.x + hi.y);
            }
            if (BITS == 2) {
              v.x = __byte_perm(in.x, in.y, 0x6420);
              v.y = __byte_perm(in.z, in.w, 0x6420);
              v.z = __byte_perm(in.x, in.y, 0x7531);
              v.w = __byte_perm(in.z, in.w, 0x7531);
            } else {
              v = in;
            }
          }
          if constexpr (KCH) {
            *reinterpret_cast<uint4*>(smem + SP::QRAW_OFF + qb * SP::QRAW_BYTES + r * D + 16 * cc) = v;
          } else {
            // atom cc / 8 holds channels [128 * (cc / 8), + 128); chunk cc % 8 of row r swizzled
            *reinterpret_cast<uint4*>(smem + SP::Q_OFF + qb * SP::Q_BYTES +
                                      (cc >> 3) * SP::Q_ATOM + r * 128 +
                                      (((cc & 7) ^ (r & 7)) << 4)) = v;
          }
          if (j < 4) {   // rows 0-7: per-head constants
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) {
              const float other = __shfl_xor_sync(0xFFFFFFFFu, qsum, o);
              qsum = KCH ? fmaxf(qsum, other) : qsum + other;
            }
            if (cc == 0) {
              float scale = 0.f;
              if (live) {
                scale = P.a.sm_scale * 1.4426950408889634f;
                if (P.a.q_descale != nullptr)
                  scale *= caller_descale<MQ>(P, w.b, w.kvh, hl);
              }
              float* hc = reinterpret_cast<float*>(smem + SP::HEADC_OFF) + qb * 24;
              hc[r] = scale;
              hc[8 + r] = KCH ? qsum : scale * qsum;
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          *reinterpret_cast<volatile int*>(smem + SP::FLAG_OFF + 48) = qi + 1;   // for the workers
          mbar_arrive(bars.q_full(qb));                                          // for the issuer
        }
      }
      ++qi;
      for (int base = first_page; base < end_page; base += 32) {
        const int nxt = base + 32 < end_page ? fetch(base + 32) : -1;
        for (int k = 0; k < 32 && base + k < end_page; ++k, ++it) {
          const int s = rp.s;
          const uint32_t eph = rp.ph ^ 1u;
          rp.next(NS);
          if ((it & 1) != pi) continue;
          const int id = __shfl_sync(0xFFFFFFFFu, cur, k);
          WT(11, mbar_wait(bars.ring_empty(s), eph, abort_flag, status));
          const uint32_t full = bars.ring_full(s);
          if (id >= 0) {
            const long long blk = static_cast<long long>(id) * P.p.num_kv_heads + w.kvh;
            const uint8_t* ks = P.p.k_codes + blk * SP::CODE_PAGE + 16 * lane;
            const uint8_t* vs = P.p.v_codes + blk * SP::CODE_PAGE + 16 * lane;
            const int scale_page = P.p.scale_bf16 ? SP::SCALE_PAGE / 2 : SP::SCALE_PAGE;   // bytes
            const uint8_t* ss = static_cast<const uint8_t*>(P.p.scales) + blk * scale_page +
                                16 * lane;
            const uint32_t dst0 = ring0 + s * SP::STAGE;
            // A lane's 16 bytes of each 512-byte step are chunk lane % CHUNKS of row
            // (step * 512 / RB + lane / CHUNKS): they go to that row's swizzled chunk.
#pragma unroll
            for (int c = 0; c < SP::CODE_PAGE; c += 512) {
              const int row = c / SP::RB + lane / SP::CHUNKS;
              const int chunk = (lane % SP::CHUNKS) ^ SP::row_swizzle(row);
              const uint32_t off = row * SP::RB + 16 * chunk;
              cp_async16_stream(dst0 + SP::K_OFF + off, ks + c, stream_policy);
              cp_async16_stream(dst0 + SP::V_OFF + off, vs + c, stream_policy);
            }
#pragma unroll
            for (int c = 0; c < SP::SCALE_PAGE; c += 512)
              if (c + 16 * lane < scale_page)
                cp_async16_stream(dst0 + SP::S_OFF + c + 16 * lane, ss + c, stream_policy);
          }
          cp_async_arrive(full);
        }
        cur = nxt;
      }
    }
    WT_SINCE(8, role_t0);
    if (lane == 0 && pi == 0) WT_FLUSH(3);
    // drain: every copy this warp issued has landed once its stage reports full
    for (int back = 0; back < NS && back < it; ++back) {
      if (--rp.s < 0) { rp.s = NS - 1; rp.ph ^= 1u; }
      mbar_wait_drain(bars.ring_full(rp.s), rp.ph, P.wait_budget / 16);
    }
  } else if (warp == W_S) {
    // ------------------------------------------------------------------ S issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc_e4m3(128, KCH ? SP::QP_ROWS : 16, 0, 0);
      constexpr uint32_t Q_HI = smem_desc_hi(1024, 2);
      constexpr int ATOM16 = (KCH ? SP::QP_ATOM : SP::Q_ATOM) >> 4;
      int qi = 0, g = 0;
      uint32_t gph = 0;
      WT_BEGIN();
      WT_MARK(role_t0);
      for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
        const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
        if (w.t1 <= w.t0) continue;
        const int qb = qi & 1;
        WT(13, mbar_wait(bars.q_full(qb), (qi >> 1) & 1, abort_flag, status));
        const uint32_t q_item = smem_desc_lo(smem0 + SP::Q_OFF + qb * SP::Q_BYTES, 16);
        for (int t = w.t0; t < w.t1; ++t) {
          WT(14, mbar_wait(bars.k_ready(g), gph, abort_flag, status));
          tc_fence_after();
          const uint32_t sd = tmem + SP::T_S + g * SP::S_COLS;
          const uint32_t ka = tmem + SP::T_KOP + g * SP::KOP_COLS;
          // the B operand: the item's query stage, or (K per channel) the operand the group
          // built for this tile
          const uint32_t q_lo =
              KCH ? smem_desc_lo(smem0 + SP::Q_OFF + g * SP::QP_BYTES, 16) : q_item;
          // eight K steps of 32 channels: the lane's two operand rows against the two atoms
          umma_ts_c<Q_HI, IDESC_S, false>(sd, ka, q_lo);
#pragma unroll
          for (int k = 1; k < 8; ++k)
            umma_ts_c<Q_HI, IDESC_S, true>(sd, ka + 8 * k,
                                           q_lo + (k >> 2) * ATOM16 + 2 * (k & 3));
          tc_commit(bars.s_done(g));
          if (t == w.t1 - 1) tc_commit(bars.q_empty(qb));
          if (++g == G) { g = 0; gph ^= 1u; }
        }
        ++qi;
      }
      WT_SINCE(8, role_t0);
      WT_FLUSH(4);
    }
    __syncwarp();
  } else if (warp == W_PV) {
    // ------------------------------------------------------------------ PV issuer
    // A group's O accumulates in tensor memory over the group's tiles of a work item: its first
    // tile of the item starts the accumulators afresh. One chain per channel half.
    if (lane == 0) {
      constexpr uint32_t IDESC_PV = make_idesc_e4m3(128, 16, 1, 1);
      constexpr uint32_t V_HI = smem_desc_hi(1024, 2), P_HI = smem_desc_hi(128, 0);
      const uint32_t v_lo0 = smem_desc_lo(smem0 + SP::VOP_OFF, 16);
      const uint32_t p_lo0 = smem_desc_lo(smem0 + SP::P_OFF, 128);
      int g = 0;
      uint32_t gph = 0;
      WT_BEGIN();
      WT_MARK(role_t0);
      for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
        const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
        for (int t = w.t0; t < w.t1; ++t) {
          const uint32_t acc = t - w.t0 >= G ? 1u : 0u;
          WT(15, mbar_wait(bars.pv_ready(g), gph, abort_flag, status));
          tc_fence_after();
          const uint32_t p_lo = p_lo0 + g * (SP::P_BYTES >> 4);
          const uint32_t od = tmem + SP::T_O + (g * 2 + (ik & 1)) * SP::O_COLS;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t vr = v_lo0 + g * (SP::VOP_STAGE >> 4) + r * (SP::VOP_PLANE >> 4);
            umma_ss_r<V_HI, P_HI, IDESC_PV>(od + 16 * r, vr, p_lo, acc);
#pragma unroll
            for (int k = 1; k < TILE / 32; ++k)
              umma_ss_c<V_HI, P_HI, IDESC_PV, true>(od + 16 * r, vr + k * (32 * SP::ROW >> 4),
                                                    p_lo + k * (32 * 16 >> 4));
          }
          tc_commit(bars.pv_done(g));
          if (++g == G) { g = 0; gph ^= 1u; }
        }
      }
      WT_SINCE(8, role_t0);
      WT_FLUSH(5);
    }
    __syncwarp();
  } else {
    worker_role<BITS, GP, KCH, MQ>(P, smem, smem0, tmem, bars, abort_flag, items);
  }

  tc_fence_before();
  __syncthreads();
#ifdef FQ_WAIT_PROFILE
  if (threadIdx.x == 0 && g_cta_times != nullptr) g_cta_times[3 * blockIdx.x + 1] = global_ns();
#endif
  if (warp == W_S) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace wide

#ifdef FQ_WAIT_PROFILE
extern "C" int fq_debug_set_cta_times(void* buffer) {
  return static_cast<int>(cudaMemcpyToSymbol(fq::wide::g_cta_times, &buffer, sizeof(buffer)));
}
extern "C" int fq_debug_set_wide_waits(void* buffer) {
  return static_cast<int>(cudaMemcpyToSymbol(fq::wide::g_wide_waits, &buffer, sizeof(buffer)));
}
#endif

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace wide {

template <int BITS, int GP, bool KCH, bool MQ>
static int launch(DecodeParams& P, cudaStream_t stream) {
  using SP = Plan<BITS, KCH>;
  constexpr int G = SP::G;
  constexpr int THREADS = threads_of(KCH);
  int stages = SP::max_ring_stages();
  if (stages > SP::MAX_STAGES) stages = SP::MAX_STAGES;
  if (const char* env = getenv("FOSCAR_B200_RING_STAGES")) {   // tuning knob for experiments
    const int want = atoi(env);
    if (want >= SPT * G && want < stages) stages = want;
  }
  stages &= ~1;   // each stage belongs to one of the two producers (see decode.cu)
  // a group runs at most one ring lap ahead of the S issuer's in-order walk over the tiles
  if (stages < SPT * G) return FQ_ERR_UNSUPPORTED;
  P.ring_stages = stages;
  P.tile_tokens = TILE;
  P.wait_budget = P.a.wait_budget_cycles > 0 ? P.a.wait_budget_cycles : WAIT_BUDGET_CYCLES;
  const int spare = SMEM_LIMIT - 1024 - SP::RING_OFF - stages * SP::STAGE;
  const int more = spare / 32 < THREADS - SP::ITEM_SLOTS ? (spare > 0 ? spare / 32 : 0)
                                                          : THREADS - SP::ITEM_SLOTS;
  P.item_slots = SP::ITEM_SLOTS + more;
  const int smem = SP::RING_OFF + stages * SP::STAGE + more * 32 + 1024;
  static bool configured[64] = {};
  auto kernel = decode_wide_kernel<BITS, GP, KCH, MQ>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_LIMIT);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  int ctas = P.a.max_ctas;
  if (ctas <= 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
      sms = 148;
    ctas = sms;
  }
  int grid = P.a.worklist ? ctas : (ctas < P.num_items ? ctas : P.num_items);
  if (grid < 1) grid = 1;
  if (P.a.flags & 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, P));
  }
  kernel<<<grid, THREADS, smem, stream>>>(P);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace wide

// Launch of the head_dim 256 build (called by fq_decode once the arguments are checked).
template <bool MQ>
static int launch_wide(DecodeParams& P, cudaStream_t stream) {
  const int gp = (P.heads_per_kv < 8 ? P.heads_per_kv : 8) <= 4 ? 4 : 8;
  if (P.p.k_channel_group != 0) {
    if (P.p.bits == 2)
      return gp == 4 ? wide::launch<2, 4, true, MQ>(P, stream)
                     : wide::launch<2, 8, true, MQ>(P, stream);
    return gp == 4 ? wide::launch<4, 4, true, MQ>(P, stream)
                   : wide::launch<4, 8, true, MQ>(P, stream);
  }
  if (P.p.bits == 2)
    return gp == 4 ? wide::launch<2, 4, false, MQ>(P, stream)
                   : wide::launch<2, 8, false, MQ>(P, stream);
  return gp == 4 ? wide::launch<4, 4, false, MQ>(P, stream)
                 : wide::launch<4, 8, false, MQ>(P, stream);
}

int launch_decode_wide(DecodeParams& P, cudaStream_t stream) {
  // (several query tokens per request: builds of their own, see decode.cuh)
  return P.q_len > 1 ? launch_wide<true>(P, stream) : launch_wide<false>(P, stream);
}

}  // namespace fq
