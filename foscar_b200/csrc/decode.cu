// Paged GQA decode attention over packed INT2/INT4 KV, sm_100a.
//
// What it computes follows the reference decode's semantics (src/foscar/wrapper.py:1153-1171;
// fold algebra src/foscar/_sm100/int_fold_decode.py:5-22, 378-434): codes are never
// dequantized. For token t and query head h
//     score = s_k[t] * (q_h . c_k[t]) + z_k[t] * sum(q_h)          (times sm_scale)
//     out_h = ( sum_t w[t,h] c_v[t]  +  sum_t p[t,h] z_v[t] ) / sum_t p[t,h]
// with w = p * s_v * 2^lp stored as two E4M3 planes (hi + lo/16).
// The structure is this library's own. One persistent CTA per SM, 20 warps, 128-token tiles:
//
//   warps 16, 19  producers on alternate tiles: page ids fetched 32 at a time a chunk ahead; a
//                 tile's two pages (K codes, V codes, scale records) as 16-byte cp.async copies
//                 from all lanes into a deep shared-memory ring, completion on an mbarrier. The
//                 first producer also stages each work item's query rows.
//   warps 0-15    four worker groups, tile i -> group i % 4. A group carries its tile through
//                 every stage: thread t unpacks token t's K row to exact E4M3 bytes
//                 (code * 2^-9) straight into TENSOR MEMORY as the S MMA's A operand, unpacks its
//                 V row into the group's 128-byte-swizzled shared-memory stage, folds the scales
//                 into S row t, joins the group's column max, writes its P row; one tile later
//                 thread d adds channel d of the tile's O to the group's accumulators. Each
//                 group keeps its own running (m, l, c, O); they are merged once per work item.
//   warp 17       S issuer (one thread):  S[128 tok x 16] = C_K . Q^T   (A from tensor memory)
//   warp 18       PV issuer (one thread): O^T[128 ch x 16] = C_V^T . [P_hi | P_lo]
//
// Why one group per tile rather than a role per stage: the kernel is bound by instruction issue
// and by hand-off latency, not by arithmetic. With separate unpack and softmax roles every tile
// crossed seven mbarrier hand-offs per warp and 28 warps walked the tile list; measured with all
// arithmetic removed, that skeleton alone took 70% of the launch time. Here a tile costs each of
// its four warps three waits (codes landed, S done, previous PV done) and three arrivals, the
// group's K stage, S, V stage, P rows and O need no barrier of their own (the group itself was
// their last reader), and a group's chain of dependent latencies (~1500-2000 cycles a tile)
// overlaps with the other three groups'.
// Every role walks the same list of work items, so the pipeline never drains inside an item.
// Byte-expansion yields channels in a fixed permuted order; Q is loaded in that order and O is
// stored through it, so no per-element fix-up exists anywhere.
//
// Variants of the same code (template parameters):
//   head_dim 64   a tile is 256 tokens, two per lane (t and 128 + t): their K rows side by side
//                 in the lane's 128-byte tensor-memory row, their V rows side by side in one
//                 shared-memory row; query rows 0-7 act on bytes 0-63 and rows 8-15 on bytes
//                 64-127, so one chain of S MMAs gives both tokens' scores (columns h, 8 + h);
//                 the PV MMA runs once per token set into its own 16 accumulator columns.
//   KG == 2       K quantized over two 64-channel groups (head_dim 128): the same split of the
//                 query rows puts each group's partial score in its own column.
//   KG == 3       whole-head K with bf16 record pairs (8 bytes a token) instead of f32 (16).
// Split units are merged inside this launch: a piece that wrote partials is counted in on its
// unit's counter one tile into the CTA's next item (or after its last), once every worker warp
// has reported its stores of the piece on a barrier, and the CTA that completes the count merges
// the unit (merge_unit_partials).
// The ring's stage count is kept even, so that each stage belongs to one of the two producers.
#include "decode.cuh"

#ifdef FQ_WAIT_PROFILE
#define FQ_STAMP_BEGIN() long long stamp_t = clock64()
#define FQ_STAMP(site)                                            \
  do {                                                            \
    const long long now_ = clock64();                             \
    wprof[site] += static_cast<int>(now_ - stamp_t);              \
    stamp_t = now_;                                               \
  } while (0)
#define FQ_ITEM_STAMP_BEGIN() long long item_t = clock64()
#define FQ_ITEM_STAMP(site)                                       \
  do {                                                            \
    const long long now_ = clock64();                             \
    wprof[site] += static_cast<int>(now_ - item_t);               \
    item_t = now_;                                                \
  } while (0)
#else
#define FQ_STAMP_BEGIN() ((void)0)
#define FQ_STAMP(site) ((void)0)
#define FQ_ITEM_STAMP_BEGIN() ((void)0)
#define FQ_ITEM_STAMP(site) ((void)0)
#endif

// Diagnostic builds only: a bit mask of roles whose arithmetic is skipped while every barrier
// arrival stays (1 softmax, 2 K unpack, 4 V unpack, 8 producers' copies; 16 / 32: one S / PV MMA
// per tile instead of four; 64 / 128: the INT2 K / V unpack at the instruction count of a 4-bit
// operand feed, i.e. two masks and a shift per packed word and half the operand words stored,
// at head_dim 128; 256 / 512: one of a row's eight V operand stores / four K operand stores
// only). The output is
// then meaningless; the launch time and instruction count show what each role costs.
#ifndef FQ_STUB_ROLES
#define FQ_STUB_ROLES 0
#endif

namespace fq {

#ifdef FQ_WAIT_PROFILE
// Diagnostic build only: per-CTA cycles (/16) each role spent blocked at each wait site.
__device__ int* g_wait_profile = nullptr;
#endif

namespace {

// barrier words: the ring's 2*ns first, then the fixed ones
template <int G>
struct Bars {
  uint32_t base;
  int ns;
  __device__ uint32_t at(int i) const { return base + 8u * i; }
  __device__ uint32_t ring_full(int s) const { return at(s); }
  __device__ uint32_t ring_empty(int s) const { return at(ns + s); }
  __device__ uint32_t q_full(int s) const { return at(2 * ns + s); }
  __device__ uint32_t q_empty(int s) const { return at(2 * ns + 2 + s); }
  // One barrier per worker group and event; a group's n-th tile uses phase n & 1:
  //   k_ready : the tile's K operand is in tensor memory (the group's 4 warps); the group has by
  //             then read the S of its previous tile
  //   s_done  : the tile's S MMA is complete (commit)
  //   pv_ready: the tile's V operand and P rows are in shared memory (4 warps); the group has by
  //             then read the O of its previous tile
  //   pv_done : the tile's PV MMA is complete (commit): O can be read, and the group's V stage
  //             and P rows are free
  __device__ uint32_t k_ready(int g) const { return at(2 * ns + 4 + g); }
  __device__ uint32_t s_done(int g) const { return at(2 * ns + 4 + G + g); }
  __device__ uint32_t pv_ready(int g) const { return at(2 * ns + 4 + 2 * G + g); }
  __device__ uint32_t pv_done(int g) const { return at(2 * ns + 4 + 3 * G + g); }
  // stored: every worker warp has issued its output or partial stores of the work item (one
  // phase per item): what orders a split piece's partials before its count-in
  __device__ uint32_t stored() const { return at(2 * ns + 4 + 4 * G); }
  // 2*ns + 5 + 4*G words of 8 bytes
};

// Position in the code ring: stage and phase, advanced without a division.
struct RingPos {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next(int ns) {
    if (++s == ns) { s = 0; ph ^= 1u; }
  }
  __device__ __forceinline__ void advance(int k, int ns) {  // k <= ns
    s += k;
    if (s >= ns) { s -= ns; ph ^= 1u; }
  }
};

// Tensor-memory column plan (f32 columns): per worker group one K operand stage (a 128-byte row
// per lane at head_dim 64, where a lane holds two tokens), one S buffer of 16 columns and one O
// buffer of 16 columns per token of a lane.
template <int BITS, int D>
struct TmemPlan {
  static constexpr int G = worker_groups(BITS, D);
  static constexpr bool PAIR = D == 64;
  static constexpr bool TWO = two_token_build(BITS, D);   // two 128-byte rows, two S buffers
  static constexpr int KOP_COLS = PAIR ? 32 : (TWO ? 2 : 1) * D / 4;
  static constexpr int S_COLS = TWO ? 32 : 16;
  static constexpr int O_COLS = PAIR ? 32 : 16;
  static constexpr int KOP = 0;
  static constexpr int S = G * KOP_COLS;
  static constexpr int O = S + G * S_COLS;
  static constexpr int USED = O + G * O_COLS;
  static constexpr int ALLOC = USED <= 128 ? 128 : (USED <= 256 ? 256 : 512);
  static_assert(USED <= 512, "tensor memory plan exceeds 512 columns");
};

// Worker role: one of four 128-thread groups. Group `wg` takes the tiles whose running index is
// `wg` modulo 4 and carries each of them through every stage itself: unpack K into tensor memory,
// unpack V into shared memory, fold the scales into the raw scores, softmax, write the P rows,
// and (one of its own tiles later) add the tile's O to its accumulators. The group keeps its own
// running (m, l, c, O); the four groups are merged once per work item.
// The request's last tile with several query tokens per request: column h sees positions below
// len - lag(h) only. Out of line, so that this rare path (and column_lag's division) costs the
// tile loop nothing: the scores pass through local memory here and nowhere else. `pos0` is the
// thread's first token position of the tile, `stride` the distance to its next one. Returns,
// in `over`, the largest excess of a visible score over its column's reference.
template <int NT, int GP>
__device__ __noinline__ void mask_lagged_columns(const DecodeParams& P, int len, int ht, int pos0,
                                                 int stride, float (&x)[NT][GP],
                                                 const float (&m)[GP], float& over) {
  float top = -INFINITY;
  for (int h = 0; h < GP; ++h) {
    const int lim = len - column_lag(P, ht * 8 + h);
    for (int u = 0; u < NT; ++u) {
      if (pos0 + u * stride >= lim) x[u][h] = -INFINITY;
      top = fmaxf(top, x[u][h] - m[h]);
    }
  }
  over = top;
}

template <int BITS, int D, int GP, int KG, bool MQ>
__device__ __forceinline__ void worker_role(const DecodeParams& P, uint8_t* smem, uint32_t smem0,
                                            uint32_t tmem, const Bars<SmemPlan<BITS, D>::G>& bars,
                                            volatile int* abort_flag, const ItemRange items,
                                            int* wprof) {
  using SP = SmemPlan<BITS, D>;
  using TP = TmemPlan<BITS, D>;
  constexpr int G = SP::G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2, wq = warp & 3;
  const int t = threadIdx.x & 127;  // token row while unpacking and in softmax, channel in O
  const int NS = P.ring_stages;
  int* status = P.a.status;
  const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
  const uint32_t ring0 = smem0 + SP::RING_OFF;
  const uint32_t k_dst = tmem + lane_base + TP::KOP + wg * TP::KOP_COLS;
  const uint32_t s_src = tmem + lane_base + TP::S + wg * TP::S_COLS;
  constexpr int NT = SP::TT / TILE;   // tokens per lane
  // a lane's O columns: at two tokens per lane, rows 0-63 (warps 0, 1) hold the first token
  // set's channels and take its P columns, rows 64-127 the second's
  const uint32_t o_src = tmem + lane_base + TP::O + wg * TP::O_COLS + (SP::PAIR && wq >= 2 ? 16 : 0);
  const uint32_t v_row = smem0 + SP::VOP_OFF + wg * SP::VOP_STAGE + t * SP::ROW;
  const uint32_t p_row = smem0 + SP::P_OFF + wg * SP::P_BYTES + t * 16;
#if FQ_STUB_ROLES & (64 | 128)
  {   // the operand words the short stubs never write: zero once
    uint32_t zero[8] = {};
    for (int v = 0; v < TP::KOP_COLS / 8; ++v) tmem_st8(k_dst + 8 * v, zero);
    tmem_st_wait();
    for (int cc = 0; cc < 8; ++cc)
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(v_row + (cc << 4)), "r"(0) : "memory");
  }
#endif
  float* red_max = reinterpret_cast<float*>(smem + SP::RED_OFF);              // [wg][buf][warp][8]
  float* red_sum = reinterpret_cast<float*>(smem + SP::RED_OFF + 256 * G);    // [wg][warp][16]
  // this warp's copy of the item's per-head constants: sm_scale*log2e*q_descale, and that times
  // the sum of the head's query values
  float* head_k = reinterpret_cast<float*>(smem + SP::HEADK_OFF) + warp * 24;
  // written per work item by thread 0 of group 0: {pieces, request, KV head, head tile} of the
  // unit this CTA must merge (pieces 0: none)
  volatile int* merge_info = reinterpret_cast<volatile int*>(smem + SP::INFO_OFF);
  const volatile float* head_const =
      reinterpret_cast<const volatile float*>(smem + SP::HEADC_OFF);  // [2][24]
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
  // w = p * s_v * 2^lp must stay inside E4M3 with p up to 2^MAX_LAG (see the softmax below)
  constexpr float MAX_LAG = 3.f;
  lp -= static_cast<int>(MAX_LAG);
  const float p2lp = exp2f(static_cast<float>(lp));
  const float o_mul = exp2f(static_cast<float>(9 - lp));

  auto merge_unit = [&](int k, int b, int kvh, int ht, int h0, int hstep) {
    if (t < D)
      merge_unit_partials<MQ, 1>(P, D, GP, channel_of_expanded_pos<BITS>(t), t == 0, k, b, kvh, ht, h0,
                          hstep);
  };
  // the split piece this CTA has written but not yet counted in (thread 0 of group 0 only)
  int pend_k = 0, pend_unit = 0, pend_b = 0, pend_kvh = 0, pend_ht = 0;
  uint32_t pend_phase = 0;   // phase of the `stored` barrier that covers the pending piece
  int seen = -1;        // the pending piece's count-in result; -1: not counted in yet
  int this_k = 0;       // pieces of the current item's unit (fetched at the item's start)

  int qi = 0;       // non-empty items so far: which query stage holds the item's rows
  int it0 = 0;      // running index of the current item's first tile (every role counts alike)
  int mine = wg;    // running index of this group's next tile
  int n = 0;        // tiles this group has taken: the phase of its barriers
  RingPos rp;       // ring position of tile `mine`
  rp.advance(wg, NS);
  FQ_ITEM_STAMP_BEGIN();
  const WorkItem* const item_cache = reinterpret_cast<const WorkItem*>(smem + SP::ITEM_OFF);
  const WorkItem* const item_more =
      reinterpret_cast<const WorkItem*>(smem + SP::RING_OFF + NS * SP::STAGE);
  for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
    const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
    const int nt = max(w.t1 - w.t0, 0);
    FQ_ITEM_STAMP(13);
    float m[GP], l[GP], c[GP], oacc[GP];
#pragma unroll
    for (int h = 0; h < GP; ++h) { m[h] = -INFINITY; l[h] = 0.f; c[h] = 0.f; oacc[h] = 0.f; }
    // The item's per-head constants (score scale, and score scale times the sum of the head's
    // query values) were computed by the first producer when it staged the query rows, well
    // ahead of the tiles; the warp keeps its own copy, read back from shared memory each tile
    // instead of living in 16 registers of every thread.
    __syncwarp();   // the warp's reads of the previous item's values are over
    if (nt > 0) {
      // Only a group with a tile in the item waits for the item's query stage: the stage cannot
      // be restaged before that group's K row has gone through the S MMA. A group without a tile
      // would have nothing holding the producer back, and a phase-parity wait that falls two
      // stagings behind never returns.
      if (mine < it0 + nt) {
        const int qb = qi & 1;
        mbar_wait(bars.q_full(qb), (qi >> 1) & 1, abort_flag, status, 14, wprof);
        if (lane < 24) head_k[lane] = head_const[qb * 24 + lane];
      }
      ++qi;
    }
    __syncwarp();
    bool pending = false;
    if (wg == 0 && t == 0 && w.slot >= 0 && P.a.unit_counters != nullptr) {
      const int unit = (w.b * P.p.num_kv_heads + w.kvh) * P.head_tiles + w.ht;
      this_k = P.a.split_counts != nullptr ? __ldg(P.a.split_counts + unit) : P.a.kv_splits;
    }
    FQ_ITEM_STAMP(16);

    // Add the group's previous tile's O (its PV MMA has had most of a tile's time to finish).
    // The wait also frees the group's V stage and P rows for the tile in hand.
    auto accumulate = [&]() {
      mbar_wait(bars.pv_done(wg), (n - 1) & 1, abort_flag, status, 15, wprof);
      tc_fence_after();
      uint32_t r[16];
      tmem_ld16(o_src, r);
      tmem_ld_wait();
      tc_fence_before();
#pragma unroll
      for (int h = 0; h < GP; ++h)
        oacc[h] += fmaf(__uint_as_float(r[8 + h]), 0.0625f, __uint_as_float(r[h]));
    };

    for (; mine < it0 + nt; mine += G, rp.advance(G, NS), ++n) {
      const int tt = w.t0 + (mine - it0);
      const uint32_t stage = ring0 + rp.s * SP::STAGE;
      mbar_wait(bars.ring_full(rp.s), rp.ph, abort_flag, status, 8, wprof);
      FQ_STAMP_BEGIN();
      // ---- K row(s) -> tensor memory (the S MMA's A operand). The stage is free: this group
      // read the S of its previous tile, so that tile's MMA, the stage's last reader, is
      // complete. With two tokens per lane (head_dim 64) the second token's 64 bytes follow the
      // first's in the lane's 128-byte row.
      {
        if constexpr (SP::PAIR) {
          // Two tokens per lane: one token's row (64 channels, 16 operand words) at a time, in a
          // loop that is NOT unrolled. This build's tile loop is the largest, and with the loop
          // rolled its code stays in the instruction cache better (INT4 838 -> 819 us on C5;
          // the same rolling at head_dim 128 cost 2 to 9 %).
          constexpr int QC = 64 * BITS / 128;   // 16-byte chunks of a token's row: 1 or 2
          tc_fence_after();
#pragma unroll 1
          for (int u = 0; u < 2; ++u) {
            uint32_t wk[64 * BITS / 32], op[16];
#if FQ_STUB_ROLES & 2
#pragma unroll
            for (int i = 0; i < 16; ++i) op[i] = n;
#else
            const uint32_t row = stage + SP::K_OFF + (u * TILE + t) * SP::RB;
#pragma unroll
            for (int v = 0; v < QC; ++v)
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(wk[4 * v]), "=r"(wk[4 * v + 1]), "=r"(wk[4 * v + 2]),
                             "=r"(wk[4 * v + 3])
                           : "r"(row + ((v ^ SP::row_swizzle(t)) << 4)));
            expand_words<BITS, 64>(wk, op);
#endif
            tmem_st16(k_dst + 16 * u, op);
          }
          FQ_STAMP(3);
        } else {
          uint32_t op[NT * D / 4];
#pragma unroll
          for (int u = 0; u < NT; ++u) {
            uint32_t wk[D * BITS / 32], part[D / 4];
#if FQ_STUB_ROLES & 2
#pragma unroll
            for (int i = 0; i < D / 4; ++i) part[i] = n;
#else
            load_row<BITS, D>(stage + SP::K_OFF + (u * TILE + t) * SP::RB, wk, SP::row_swizzle(t));
#if FQ_STUB_ROLES & 64
            if constexpr (BITS == 2) {
#pragma unroll
              for (int i = 0; i < D / 16; ++i) {
                part[2 * i] = wk[i] & 0x33333333u;
                part[2 * i + 1] = (wk[i] >> 2) & 0x33333333u;
              }
            } else
#endif
            expand_words<BITS, D>(wk, part);
#endif
#pragma unroll
            for (int i = 0; i < D / 4; ++i) op[u * (D / 4) + i] = part[i];
          }
          FQ_STAMP(3);
          tc_fence_after();
#pragma unroll
          for (int v = 0; v < NT * D / (((FQ_STUB_ROLES & 64) && BITS == 2) ? 64 : 32); ++v)
            if (!(FQ_STUB_ROLES & 512) || v == 0) tmem_st8(k_dst + 8 * v, op + 8 * v);
        }
        tmem_st_wait();
        FQ_STAMP(5);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars.k_ready(wg));
      }
      FQ_STAMP(17);
      if (pending) accumulate();
      FQ_STAMP(18);
      // ---- V row(s) -> the group's 128-byte-swizzled shared-memory stage (the PV MMA's A
      // operand), laid out like the K row
      if constexpr (SP::PAIR) {
        constexpr int QC = 64 * BITS / 128;
#pragma unroll 1
        for (int u = 0; u < 2; ++u) {
          uint32_t wv[64 * BITS / 32], op[16];
#if FQ_STUB_ROLES & 4
#pragma unroll
          for (int i = 0; i < 16; ++i) op[i] = n;
#else
          const uint32_t row = stage + SP::V_OFF + (u * TILE + t) * SP::RB;
#pragma unroll
          for (int v = 0; v < QC; ++v)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(wv[4 * v]), "=r"(wv[4 * v + 1]), "=r"(wv[4 * v + 2]),
                           "=r"(wv[4 * v + 3])
                         : "r"(row + ((v ^ SP::row_swizzle(t)) << 4)));
          expand_words_v<BITS, 64>(wv, op);
#endif
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                             v_row + (((4 * u + cc) ^ (t & 7)) << 4)),
                         "r"(op[4 * cc]), "r"(op[4 * cc + 1]), "r"(op[4 * cc + 2]),
                         "r"(op[4 * cc + 3])
                         : "memory");
          }
        }
        FQ_STAMP(6);
      } else {
        uint32_t op[NT * D / 4];
#pragma unroll
        for (int u = 0; u < NT; ++u) {
          uint32_t wv[D * BITS / 32], part[D / 4];
#if FQ_STUB_ROLES & 4
#pragma unroll
          for (int i = 0; i < D / 4; ++i) part[i] = n;
#else
          load_row<BITS, D>(stage + SP::V_OFF + (u * TILE + t) * SP::RB, wv, SP::row_swizzle(t));
#if FQ_STUB_ROLES & 128
          if constexpr (BITS == 2) {
#pragma unroll
            for (int i = 0; i < D / 16; ++i) {
              part[2 * i] = wv[i] & 0x33333333u;
              part[2 * i + 1] = (wv[i] >> 2) & 0x33333333u;
            }
          } else
#endif
          expand_words_v<BITS, D>(wv, part);
#endif
#pragma unroll
          for (int i = 0; i < D / 4; ++i) op[u * (D / 4) + i] = part[i];
        }
        FQ_STAMP(6);
#pragma unroll
        for (int u = 0; u < NT; ++u) {   // token 128 u + t is row 128 u + t of the stage
#pragma unroll
          for (int cc = 0; cc < D / (((FQ_STUB_ROLES & 128) && BITS == 2) ? 32 : 16); ++cc) {
            if ((FQ_STUB_ROLES & 256) && cc > 0) continue;
            const int oc = u * (D / 16) + cc;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                             v_row + u * TILE * SP::ROW + ((cc ^ (t & 7)) << 4)),
                         "r"(op[4 * oc]), "r"(op[4 * oc + 1]), "r"(op[4 * oc + 2]),
                         "r"(op[4 * oc + 3])
                         : "memory");
          }
        }
      }
      FQ_STAMP(9);
      // the tokens' records; then the ring stage goes back to the producers
      float sk[NT], zk[NT], sv[NT], zv[NT];
      float sk1[NT] = {}, zk1[NT] = {};   // the second K group's pair (KG == 2)
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        const int row = u * TILE + t;
        if constexpr (KG == 2) {   // K ring: (s, z) of both groups; V ring after the page's K ring
          uint32_t k0, k1, vr;
          const uint32_t slot = stage + SP::S_OFF + (row >> 6) * SP::SCALE_PAGE;
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(k0), "=r"(k1)
                       : "r"(slot + (row & 63) * 8));
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(vr) : "r"(slot + 8 * PAGE + (row & 63) * 4));
          sk[u] = __uint_as_float(k0 << 16); zk[u] = __uint_as_float(k0 & 0xFFFF0000u);
          sk1[u] = __uint_as_float(k1 << 16); zk1[u] = __uint_as_float(k1 & 0xFFFF0000u);
          sv[u] = __uint_as_float(vr << 16); zv[u] = __uint_as_float(vr & 0xFFFF0000u);
        } else if constexpr (KG != 3) {   // KG == 1: f32 records; KG == 3: bf16 pairs
          asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                       : "=f"(sk[u]), "=f"(zk[u]), "=f"(sv[u]), "=f"(zv[u])
                       : "r"(stage + SP::S_OFF + row * 16));
        } else {   // (s, z) as bf16 pairs, 8 bytes a token, each page at its f32-sized slot
          uint32_t kr, vr;
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];"
                       : "=r"(kr), "=r"(vr)
                       : "r"(stage + SP::S_OFF + (row >> 6) * SP::SCALE_PAGE + (row & 63) * 8));
          sk[u] = __uint_as_float(kr << 16); zk[u] = __uint_as_float(kr & 0xFFFF0000u);
          sv[u] = __uint_as_float(vr << 16); zv[u] = __uint_as_float(vr & 0xFFFF0000u);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars.ring_empty(rp.s));
      FQ_STAMP(19);
      // ---- raw scores: columns [0, GP) for the lane's first token, [8, 8 + GP) for its second
      mbar_wait(bars.s_done(wg), n & 1, abort_flag, status, 12, wprof);
      tc_fence_after();
      // (two tokens with a 128-byte row each: a 16-column S buffer per token, RS apart in raw)
      constexpr int RS = SP::TWO ? (KG == 2 ? 16 : 8) : 8;
      uint32_t raw[SP::TWO ? 2 * RS : ((NT == 2 || KG == 2) ? 16 : GP)];
      if constexpr (SP::TWO) {
        if constexpr (KG == 2) {
          tmem_ld16p(s_src, raw);
          tmem_ld16p(s_src + 16, raw + 16);
        } else {
          tmem_ld8p(s_src, raw);
          tmem_ld8p(s_src + 16, raw + 8);
        }
      } else if constexpr (NT == 2 || KG == 2) tmem_ld16(s_src, raw);
      else if constexpr (GP == 4) tmem_ld4(s_src, raw);
      else tmem_ld8(s_src, raw);
      tmem_ld_wait();
      tc_fence_before();
      FQ_STAMP(20);
      FQ_STAMP(10);   // the cost of one stamp itself
      uint32_t pw[NT][4];
#if FQ_STUB_ROLES & 1
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        pw[u][0] = __float_as_uint(sk[u] + zk[u]) & 1u; pw[u][1] = raw[0] & 1u;
        pw[u][2] = __float_as_uint(sv[u] + zv[u]) & 1u; pw[u][3] = 0u;
      }
#else
      // Only a request's last tile has positions past its length: their scores become -inf and
      // their records are neutralised, so stale shared memory can never reach the output.
      // Scores against the group's running reference m, which may lag the true maximum by up to
      // MAX_LAG (p <= 2^MAX_LAG; the P scale leaves that headroom below the E4M3 range). Only
      // when some score of the tile exceeds that does the group take the exact column maximum
      // and rescale; the common tile costs one reducing barrier instead of an exchange through
      // shared memory.
      float x[NT][GP], wsc[NT];
      float over = -INFINITY;
      // with several query tokens a column stops short of the request's last positions
      const bool whole = (tt + 1) * SP::TT <= w.len - (MQ ? P.q_len - 1 : 0);
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        const int pos = tt * SP::TT + u * TILE + t;
        const bool valid = whole || pos < w.len;
        const float a_k = sk[u] * 512.f;
        wsc[u] = sv[u] * p2lp;
        if (!valid) { wsc[u] = 0.f; zv[u] = 0.f; }
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float xv;
          if constexpr (KG == 2)
            xv = fmaf(head_k[h] * a_k, __uint_as_float(raw[RS * u + h]),
                      fmaf(head_k[h] * (sk1[u] * 512.f), __uint_as_float(raw[RS * u + 8 + h]),
                           fmaf(head_k[8 + h], zk[u], head_k[16 + h] * zk1[u])));
          else
            xv = fmaf(head_k[h] * a_k, __uint_as_float(raw[RS * u + h]), head_k[8 + h] * zk[u]);
          x[u][h] = valid ? xv : -INFINITY;
          over = fmaxf(over, x[u][h] - m[h]);
        }
      }
      if constexpr (MQ) {
        if (!whole) mask_lagged_columns<NT, GP>(P, w.len, w.ht, tt * SP::TT + t, TILE, x, m, over);
      }
      // (a group's first tile of an item always takes the exact maximum: with several query
      // tokens every score of that tile can be masked, which would leave m at -inf)
      if (named_barrier_or(1 + wg, 128, over > MAX_LAG || (MQ && m[0] == -INFINITY))) {
        const int buf = n & 1;
        float* wmax = red_max + ((wg * 2 + buf) * 4 + wq) * 8;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const float wm = warp_max_f32(NT == 2 ? fmaxf(x[0][h], x[NT - 1][h]) : x[0][h]);
          if (lane == 0) wmax[h] = wm;
        }
        named_barrier(1 + wg, 128);
        const float* gm = red_max + (wg * 2 + buf) * 4 * 8;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          // (floored so that a column with every score masked so far has a finite reference)
          float tm = fmaxf(m[h], fmaxf(fmaxf(gm[h], gm[8 + h]), fmaxf(gm[16 + h], gm[24 + h])));
          if constexpr (MQ) tm = fmaxf(tm, -1e30f);
          const float corr = m[h] == -INFINITY ? 0.f : fast_exp2(m[h] - tm);
          l[h] *= corr;
          c[h] *= corr;
          oacc[h] *= corr;   // holds every earlier tile's O (added above)
          m[h] = tm;
        }
      }
      // two heads per instruction in f16x2: p = 2^(x-m), w = p * s_v 2^lp, E4M3 hi + lo/16
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        pw[u][0] = pw[u][1] = pw[u][2] = pw[u][3] = 0u;
        const __half2 wsc2 = __float2half2_rn(wsc[u]);
#pragma unroll
        for (int h = 0; h < GP; h += 2) {
          const __half2 d2 = __floats2half2_rn(x[u][h] - m[h], x[u][h + 1] - m[h + 1]);
          const __half2 e2 = h2_exp2(d2);
          const float2 ef = __half22float2(e2);
          l[h] += ef.x;
          l[h + 1] += ef.y;
          c[h] = fmaf(ef.x, zv[u], c[h]);
          c[h + 1] = fmaf(ef.y, zv[u], c[h + 1]);
          const __half2 w2 = __hmul2(e2, wsc2);
          const uint32_t hi2 = f16x2_to_e4m3x2(w2);
          const __half2 r2 = __hmul2(__hsub2(w2, e4m3x2_to_f16x2(hi2)), __float2half2_rn(16.f));
          const uint32_t lo2 = f16x2_to_e4m3x2(r2);
          pw[u][h >> 2] |= hi2 << (16 * ((h >> 1) & 1));
          pw[u][2 + (h >> 2)] |= lo2 << (16 * ((h >> 1) & 1));
        }
      }
#endif
      FQ_STAMP(21);
      // the P row(s): bytes [hi_0..hi_7 | lo_0..lo_7], one plane of 128 rows per token of a lane;
      // with the V rows above they complete the PV MMA's operands
#pragma unroll
      for (int u = 0; u < NT; ++u)
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_row + u * TILE * 16),
                     "r"(pw[u][0]), "r"(pw[u][1]), "r"(pw[u][2]), "r"(pw[u][3])
                     : "memory");
      fence_proxy_async();
      FQ_STAMP(11);
      __syncwarp();
      if (lane == 0) mbar_arrive(bars.pv_ready(wg));
      FQ_STAMP(22);
      pending = true;
      // The previous split piece of this CTA is counted in here, a tile into the next item: its
      // partials have drained, and the fence and the atomic's round trip cost one thread of
      // one group a microsecond in mid-stream instead of stalling an item boundary. The wait
      // (long satisfied) is what orders every worker warp's partial stores before this
      // thread's release fence and atomic.
      if (wg == 0 && t == 0 && pend_k > 0 && seen < 0) {
        mbar_wait(bars.stored(), pend_phase, abort_flag, status, 29, wprof);
        __threadfence();
        seen = atomicAdd(P.a.unit_counters + pend_unit, 1);
      }
    }
    it0 += nt;
    FQ_ITEM_STAMP(24);
    if (pending) accumulate();
    FQ_ITEM_STAMP(27);

    // ---- item epilogue. First, the count-in of the previous split piece (see step 1 below)
    if (wg == 0 && t == 0 && pend_k > 0 && seen < 0) {   // group 0 had no tile in this item
      mbar_wait(bars.stored(), pend_phase, abort_flag, status, 29, wprof);
      __threadfence();
      seen = atomicAdd(P.a.unit_counters + pend_unit, 1);
    }
    // group sums, then the groups' states through shared memory
    float* rs = red_sum + (wg * 4 + wq) * 16;
#pragma unroll
    for (int h = 0; h < GP; ++h) {
      float ls = l[h], cs = c[h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ls += __shfl_xor_sync(0xFFFFFFFFu, ls, o);
        cs += __shfl_xor_sync(0xFFFFFFFFu, cs, o);
      }
      if (lane == 0) { rs[h] = ls; rs[8 + h] = cs; }
    }
    named_barrier(1 + wg, 128);
    const float* gs = red_sum + wg * 4 * 16;
#pragma unroll
    for (int h = 0; h < GP; ++h) {
      l[h] = (gs[h] + gs[16 + h]) + (gs[32 + h] + gs[48 + h]);
      c[h] = (gs[8 + h] + gs[24 + h]) + (gs[40 + h] + gs[56 + h]);
    }
    {   // every group leaves its state in shared memory
      float* xo = reinterpret_cast<float*>(smem + SP::XCHG_OFF + wg * SP::XCHG_STRIDE);
      float* xmeta = xo + TILE * 8;
#pragma unroll
      for (int h = 0; h < GP; ++h) xo[h * TILE + t] = oacc[h];   // head-major: no bank conflicts
      if (t == 0) {
#pragma unroll
        for (int h = 0; h < GP; ++h) { xmeta[h] = m[h]; xmeta[8 + h] = l[h]; xmeta[16 + h] = c[h]; }
      }
    }
    named_barrier(1 + G, 128 * G);
    FQ_ITEM_STAMP(30);
    // The groups' states are merged in fixed order (group 0, then 1, 2, 3), each group taking a
    // share of the heads; the loop over the groups is unrolled so that its loads go out together.
    // (The results go to global memory only after the barrier below: a barrier that follows
    // global stores waits for them to be acknowledged, about 2 us under this load.)
    constexpr int HPG = (GP + G - 1) / G;   // heads a group merges
    float rM[HPG], rL[HPG], rO[HPG];
#pragma unroll
    for (int i = 0; i < HPG; ++i) {
      const int h = wg + i * G;
      float M = -INFINITY, L = 0.f, C = 0.f, O = 0.f;
      if (h < GP) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float* xo = reinterpret_cast<const float*>(smem + SP::XCHG_OFF +
                                                           g * SP::XCHG_STRIDE);
          const float* xmeta = xo + TILE * 8;
          const float m1 = xmeta[h], l1 = xmeta[8 + h], c1 = xmeta[16 + h];
          // at two tokens per lane, channel t's sum is split over rows t and t + 64
          float o1 = xo[h * TILE + t];
          if (SP::PAIR && t < 64) o1 += xo[h * TILE + t + 64];
          const float Mn = fmaxf(M, m1);
          const float f0 = M == -INFINITY ? 0.f : exp2f(M - Mn);
          const float f1 = m1 == -INFINITY ? 0.f : exp2f(m1 - Mn);
          L = L * f0 + l1 * f1;
          C = C * f0 + c1 * f1;
          O = O * f0 + o1 * f1;
          M = Mn;
        }
        O = O * (o_mul * v_position_scale<BITS>(t)) + C;
      }
      rM[i] = M; rL[i] = L; rO[i] = O;
    }
    FQ_ITEM_STAMP(28);
    // ---- in-kernel merge, step 1. A split piece is counted in (release fence + one atomic on
    // its unit's counter) not here but a tile into the NEXT item (above), or after the last
    // item. Whoever finds the count complete makes the CTA merge that unit after the barrier
    // below.
    if (wg == 0 && t == 0) {
      int km = 0;
      if (pend_k > 0 && seen == pend_k - 1) {
        P.a.unit_counters[pend_unit] = 0;   // nobody touches it again before the next launch
        km = pend_k;
      }
      merge_info[0] = km; merge_info[1] = pend_b; merge_info[2] = pend_kvh; merge_info[3] = pend_ht;
      pend_k = 0;
      seen = -1;
      if (w.slot >= 0 && P.a.unit_counters != nullptr) {
        pend_unit = (w.b * P.p.num_kv_heads + w.kvh) * P.head_tiles + w.ht;
        pend_k = this_k;
        pend_b = w.b; pend_kvh = w.kvh; pend_ht = w.ht;
        pend_phase = static_cast<uint32_t>(ik & 1);
      }
    }
    FQ_ITEM_STAMP(31);
    // the exchange buffers are reused by the next item
    named_barrier(1 + G, 128 * G);
    FQ_ITEM_STAMP(25);
    // ---- in-kernel merge, step 2: every group takes its share of the unit's heads (the words
    // are next written after the next item's first all-group barrier, which this read precedes)
    if (w.slot != -2) {
      const int ch = channel_of_expanded_pos<BITS>(t);
      const bool on = t < D;   // head_dim 64: the upper half of the O rows is padding
#pragma unroll
      for (int i = 0; i < HPG; ++i) {
        const int h = wg + i * G;
        const int hl = w.ht * 8 + h;
        if (h >= GP || hl >= P.heads_per_kv) continue;
        const float M = rM[i], L = rL[i], O = rO[i];
        const long long head = static_cast<long long>(w.kvh) * P.heads_per_kv + hl;
        const long long row = static_cast<long long>(w.b) * P.a.num_qo_heads + head;
        if (w.slot < 0) {
          const long long orow = caller_row<MQ>(P, w.b, w.kvh, hl);
          const float val = L > 0.f ? O / L * P.a.o_scale : 0.f;
          if (on) store_value(P.a.out, P.a.out_dtype, orow * D + ch, val);
          if (t == 0 && P.a.lse != nullptr)
            P.a.lse[orow] = L > 0.f ? (M + log2f(L)) * LN2 : -INFINITY;
        } else {
          const long long prow =
              static_cast<long long>(w.slot) * P.a.batch * P.a.num_qo_heads + row;
          if (on) P.a.o_partial[prow * D + ch] = O;
          if (t == 0) { P.a.l_partial[prow] = L; P.a.m_partial[prow] = M; }
        }
      }
    }
    // this warp's stores of the item are issued
    __syncwarp();
    if (lane == 0) mbar_arrive(bars.stored());
    if (merge_info[0] > 0)
      merge_unit(merge_info[0], merge_info[1], merge_info[2], merge_info[3], wg, G);
    FQ_ITEM_STAMP(26);
  }
  // The last split piece of this CTA is counted in here; if that completes its unit, the CTA
  // merges it (every group its share of the heads, as above).
  {
    volatile int* last_info = merge_info + 4;   // slow groups may still be reading merge_info
    if (wg == 0 && t == 0) {
      int km = 0;
      if (pend_k > 0) {
        if (seen < 0) {
          mbar_wait(bars.stored(), pend_phase, abort_flag, status, 29, wprof);
          __threadfence();
          seen = atomicAdd(P.a.unit_counters + pend_unit, 1);
        }
        if (seen == pend_k - 1) {
          P.a.unit_counters[pend_unit] = 0;
          km = pend_k;
        }
      }
      last_info[0] = km; last_info[1] = pend_b; last_info[2] = pend_kvh; last_info[3] = pend_ht;
    }
    named_barrier(1 + G, 128 * G);
    if (last_info[0] > 0)
      merge_unit(last_info[0], last_info[1], last_info[2], last_info[3], wg, G);
  }
}

}  // namespace

template <int BITS, int D, int GP, int KG, bool MQ>
__global__ void __launch_bounds__(decode_threads(BITS, D), ctas_per_sm(BITS, D)) decode_kernel(const DecodeParams P) {
  // KG: 1 whole-head K with f32 records, 3 the same with bf16 pairs, 2 two 64-channel K groups
  static_assert(KG == 1 || KG == 3 || (KG == 2 && D == 128),
                "K groups of 64 channels at head_dim 128");
  static_assert(D == 64 || D == 128, "this build tiles head_dim 64 and 128");
  using SP = SmemPlan<BITS, D>;
  using TP = TmemPlan<BITS, D>;
  constexpr int G = SP::G;
  constexpr int W_PRODUCER = 4 * G, W_S = W_PRODUCER + 1, W_PV = W_PRODUCER + 2,
                W_PRODUCER2 = W_PRODUCER + 3;
  static_assert(decode_threads(BITS, D) == 32 * (W_PRODUCER2 + 1), "warp roles and block size disagree");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem = smem_raw + (smem0 - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NS = P.ring_stages;
  Bars<G> bars{smem0 + SP::BAR_OFF, NS};
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SP::BAR_OFF + 1024);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SP::BAR_OFF + 1016);
  int* status = P.a.status;
#ifdef FQ_WAIT_PROFILE
  const long long kernel_t0 = clock64();
  if (threadIdx.x < WAIT_SITES) const_cast<int*>(abort_flag)[4 + threadIdx.x] = 0;
#endif

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    set_wait_budget(abort_flag, P.wait_budget);
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
    mbar_init(bars.stored(), 4 * G);   // one arrival per worker warp
    fence_barrier_init();
  }
  if (warp == W_S) tmem_alloc(smem_u32(tmem_slot), TP::ALLOC);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Everything above touched only this CTA's shared and tensor memory. Under a programmatic
  // launch it may have run while the launch before this one in the stream was still finishing:
  // wait for that launch (complete and flushed) before the first global access, and let the
  // launch after this one start its own set-up as SMs free up. Both are no-ops otherwise.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const ItemRange items = item_range(P);
  // The CTA's first items, decoded by one thread each: their dependent loads (row, length, table
  // offset) go out side by side, once, instead of in every role at every item boundary.
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
  int wprof[WAIT_SITES] = {};   // used by the diagnostic build only
#ifdef FQ_WAIT_PROFILE
  if (threadIdx.x == 0) wprof[22] = static_cast<int>(clock64() - kernel_t0);   // set-up
#endif

  if (warp == W_PRODUCER || warp == W_PRODUCER2) {
    // ------------------------------------------------------------------ producers
    // Two warps take alternate tiles. A tile's two pages (K codes, V codes, scale records of
    // one KV head) arrive as 16-byte cp.async copies issued by all 32 lanes: measured on B200,
    // a cp.async.bulk costs its issuing warp ~200 cycles whatever its size, so six 1-2 KB bulk
    // copies per tile cap the ring near 2.5 TB/s, while 20 cp.async per lane cost ~370 cycles.
    // Page ids are fetched 32 at a time, one per lane, a chunk ahead of the tiles that use them.
    // The first producer also stages each item's query rows, in expansion order, as the S MMA's
    // B operand; it runs a ring's depth ahead of the MMAs, which hides the load.
    const int pi = warp == W_PRODUCER ? 0 : 1;
    const uint64_t stream_policy = l2_evict_first_policy();
    int it = 0, qi = 0;
    RingPos rp;
    for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
      const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
      if (w.t1 <= w.t0) continue;
      constexpr int PPT = SP::PPT;   // pages per tile
      const int npages = (w.len + PAGE - 1) / PAGE;
      const int pend = min(PPT * w.t1, npages);
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
      int cur = fetch(PPT * w.t0);
      if (pi == 0) {
        const int qb = qi & 1;
        mbar_wait(bars.q_empty(qb), ((qi >> 1) & 1) ^ 1, abort_flag, status, 7, wprof);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int chunk = lane + 32 * j;      // 16 rows of eight 16-byte chunks
          const int r = chunk >> 3, cc = chunk & 7;
          uint4 v = make_uint4(0, 0, 0, 0);
          // At two tokens per lane rows 0-7 carry the heads against the first token's half of
          // the K row (bytes 0-63) and rows 8-15 the same heads against the second's (64-127).
          // With two K groups of 64 channels (one token per lane) the same split of the rows
          // yields each group's partial product in its own S column.
          constexpr bool SPLIT = SP::PAIR || KG == 2;
          const int hl = w.ht * 8 + (SPLIT ? (r & 7) : r);  // head inside the KV head's group
          const bool live = (SPLIT || r < 8) && hl < P.heads_per_kv;
          const long long qrow = live ? caller_row<MQ>(P, w.b, w.kvh, hl) : 0;
          const bool mine = SPLIT ? ((r < 8) == (cc < 4)) : 16 * cc < D;
          const int src = SP::PAIR ? (cc & 3) : cc;
          float qsum = 0.f;
          if (live && mine) {
            const uint4 in = __ldg(reinterpret_cast<const uint4*>(
                static_cast<const uint8_t*>(P.a.q) +
                qrow * D + 16 * src));
            const uint32_t words[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 lo = e4m3x2_to_f32x2(words[i] & 0xFFFF);
              const float2 hi = e4m3x2_to_f32x2(words[i] >> 16);
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
          *reinterpret_cast<uint4*>(smem + SP::Q_OFF + qb * SP::Q_BYTES + r * 128 +
                                    ((cc ^ (r & 7)) << 4)) = v;
          if (j < 2 || KG == 2) {
            // the row's eight chunks sit in eight neighbouring lanes: per-head constants
            // (rows 8-15: the second K group's query sums)
            qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, 1);
            qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, 2);
            qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, 4);
            if (cc == 0) {
              float scale = 0.f;
              if (live) {
                scale = P.a.sm_scale * 1.4426950408889634f;
                if (P.a.q_descale != nullptr)
                  scale *= caller_descale<MQ>(P, w.b, w.kvh, hl);
              }
              float* hc = reinterpret_cast<float*>(smem + SP::HEADC_OFF) + qb * 24;
              if (r < 8) {
                hc[r] = scale;
                hc[8 + r] = scale * qsum;
              } else {
                hc[16 + (r - 8)] = scale * qsum;
              }
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars.q_full(qb));
      }
      ++qi;
      for (int base = PPT * w.t0; base < PPT * w.t1; base += 32) {
        const int nxt = base + 32 < PPT * w.t1 ? fetch(base + 32) : -1;
        for (int k = 0; k < 32 / PPT && base + PPT * k < PPT * w.t1; ++k, ++it) {
          const int s = rp.s;
          const uint32_t eph = rp.ph ^ 1u;
          rp.next(NS);
          if ((it & 1) != pi) continue;
          int ids[PPT];
#pragma unroll
          for (int j = 0; j < PPT; ++j) ids[j] = __shfl_sync(0xFFFFFFFFu, cur, PPT * k + j);
          mbar_wait(bars.ring_empty(s), eph, abort_flag, status, 0, wprof);
          const uint32_t full = bars.ring_full(s);
          // code chunks go to their swizzled place in the row (SmemPlan::row_swizzle); a lane's
          // 16 bytes are chunk lane % CHUNKS of row lane / CHUNKS (+ a multiple of 8 rows)
          const int code_lane = (lane & ~(SP::CHUNKS - 1)) |
                                ((lane & (SP::CHUNKS - 1)) ^ SP::row_swizzle(lane / SP::CHUNKS));
          const uint32_t dst = ring0 + s * SP::STAGE + 16 * code_lane;
          const uint32_t dst_rec = ring0 + s * SP::STAGE + 16 * lane;
#pragma unroll
          for (int j = 0; j < PPT; ++j) {
            const int id = ids[j];
            if (id < 0 || (FQ_STUB_ROLES & 8)) continue;
            const long long blk = static_cast<long long>(id) * P.p.num_kv_heads + w.kvh;
            const uint8_t* ks = P.p.k_codes + blk * SP::CODE_PAGE + 16 * lane;
            const uint8_t* vs = P.p.v_codes + blk * SP::CODE_PAGE + 16 * lane;
            // records: 16 B per token in an f32 pool, 8 B in a bf16 pool (same slot in the ring)
            // (with two K groups: 8 B of K pairs per token, then 4 B of V pairs per token)
            constexpr int scale_page =
                KG == 2 ? 12 * PAGE : (KG == 3 ? SP::SCALE_PAGE / 2 : SP::SCALE_PAGE);
            const uint8_t* ss = static_cast<const uint8_t*>(P.p.scales) + blk * scale_page +
                                16 * lane;
#pragma unroll
            for (int c = 0; c < SP::CODE_PAGE; c += 512)
              cp_async16_stream(dst + SP::K_OFF + j * SP::CODE_PAGE + c, ks + c, stream_policy);
#pragma unroll
            for (int c = 0; c < SP::CODE_PAGE; c += 512)
              cp_async16_stream(dst + SP::V_OFF + j * SP::CODE_PAGE + c, vs + c, stream_policy);
#pragma unroll
            for (int c = 0; c < SP::SCALE_PAGE; c += 512)
              if (c + 16 * lane < scale_page)
                cp_async16_stream(dst_rec + SP::S_OFF + j * SP::SCALE_PAGE + c, ss + c,
                                  stream_policy);
          }
          cp_async_arrive(full);
        }
        cur = nxt;
      }
    }
    // drain: every copy this warp issued has landed once its stage reports full
    for (int back = 0; back < NS && back < it; ++back) {
      if (--rp.s < 0) { rp.s = NS - 1; rp.ph ^= 1u; }
      mbar_wait_drain(bars.ring_full(rp.s), rp.ph, P.wait_budget / 16);
    }
  } else if (warp == W_S) {
    // ------------------------------------------------------------------ S issuer
    // One thread issues S = C_K . Q^T for every tile, in tile order. The loop is kept to a few
    // dozen scalar instructions per tile: descriptor high words, the instruction descriptor and
    // the accumulate flags are immediates, and the group index is a counter.
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc_e4m3(128, 16, 0, 0);
      constexpr uint32_t Q_HI = smem_desc_hi(1024, 2);
      int qi = 0, g = 0;   // tiles go to the groups in turn
      uint32_t gph = 0;    // phase of the groups' barriers: flips once per round of G tiles
      for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
        const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
        if (w.t1 <= w.t0) continue;
        const int qb = qi & 1;
        mbar_wait(bars.q_full(qb), (qi >> 1) & 1, abort_flag, status, 1, wprof);
        const uint32_t q_lo = smem_desc_lo(smem0 + SP::Q_OFF + qb * SP::Q_BYTES, 16);
        for (int t = w.t0; t < w.t1; ++t) {
          mbar_wait(bars.k_ready(g), gph, abort_flag, status, 2, wprof);
          tc_fence_after();
          // (with a 128-byte row per token, a chain and a 16-column S buffer per token)
#pragma unroll
          for (int u = 0; u < (SP::TWO ? 2 : 1); ++u) {
            const uint32_t sd = tmem + TP::S + g * TP::S_COLS + 16 * u;
            const uint32_t ka = tmem + TP::KOP + g * TP::KOP_COLS + (D / 4) * u;
            umma_ts_c<Q_HI, IDESC_S, false>(sd, ka, q_lo);
#pragma unroll
            for (int k = 1; k < ((FQ_STUB_ROLES & 16) ? 1 : (SP::PAIR ? 2 : 1) * D / 32); ++k)
              umma_ts_c<Q_HI, IDESC_S, true>(sd, ka + 8 * k, q_lo + 2 * k);
          }
          tc_commit(bars.s_done(g));
          if (t == w.t1 - 1) tc_commit(bars.q_empty(qb));
          if (++g == G) { g = 0; gph ^= 1u; }
        }
        ++qi;
      }
    }
    __syncwarp();
  } else if (warp == W_PV) {
    // ------------------------------------------------------------------ PV issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_PV = make_idesc_e4m3(128, 16, 1, 1);
      constexpr uint32_t V_HI = smem_desc_hi(1024, 2), P_HI = smem_desc_hi(128, 0);
      const uint32_t v_lo0 = smem_desc_lo(smem0 + SP::VOP_OFF, 16);
      const uint32_t p_lo0 = smem_desc_lo(smem0 + SP::P_OFF, 128);
      int g = 0;
      uint32_t gph = 0;
      for (int wi = items.begin, ik = 0; wi < items.end; wi += items.step, ++ik) {
        const WorkItem w = item_at(P, item_cache, item_more, SP::ITEM_SLOTS, ik, wi);
        for (int t = w.t0; t < w.t1; ++t) {
          mbar_wait(bars.pv_ready(g), gph, abort_flag, status, 4, wprof);
          tc_fence_after();
          const uint32_t v_lo = v_lo0 + g * (SP::VOP_STAGE >> 4);
          const uint32_t p_lo = p_lo0 + g * (SP::P_BYTES >> 4);
          const uint32_t od = tmem + TP::O + g * TP::O_COLS;
          // one accumulator per token of a lane: the same V rows against that token's P plane
#pragma unroll
          for (int u = 0; u < (SP::PAIR ? 2 : 1); ++u) {
            const uint32_t pu = p_lo + u * (TILE * 16 >> 4);
            umma_ss_c<V_HI, P_HI, IDESC_PV, false>(od + 16 * u, v_lo, pu);
#pragma unroll
            for (int k = 1; k < ((FQ_STUB_ROLES & 32) ? 1 : (SP::TWO ? 2 : 1) * TILE / 32); ++k)
              umma_ss_c<V_HI, P_HI, IDESC_PV, true>(od + 16 * u, v_lo + k * (32 * SP::ROW >> 4),
                                                    pu + k * (32 * 16 >> 4));
          }
          tc_commit(bars.pv_done(g));
          if (++g == G) { g = 0; gph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ workers
    worker_role<BITS, D, GP, KG, MQ>(P, smem, smem0, tmem, bars, abort_flag, items, wprof);
#ifdef FQ_WAIT_PROFILE
    if (threadIdx.x == 0) wprof[21] = static_cast<int>(clock64() - kernel_t0);   // workers done
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (warp == W_S) {
    tc_fence_after();
    tmem_dealloc(tmem, TP::ALLOC);
  }
#ifdef FQ_WAIT_PROFILE
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < WAIT_SITES; ++i)
      if (wprof[i]) atomicAdd(const_cast<int*>(abort_flag) + 4 + i, wprof[i] >> 4);
  }
  __syncthreads();
  if (g_wait_profile != nullptr && threadIdx.x < WAIT_SITES) {
    int v = const_cast<int*>(abort_flag)[4 + threadIdx.x];
    if (threadIdx.x == 23) v = static_cast<int>((clock64() - kernel_t0) >> 4);
    g_wait_profile[blockIdx.x * WAIT_SITES + threadIdx.x] = v;
  }
#endif
}

// Tensor-core self test (see foscar_b200.h): one tile of both contractions on given operands.
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(int mode, const uint8_t* k_bytes, const uint8_t* q_bytes,
                     const uint8_t* v_bytes, const uint8_t* p_bytes, float* s_out, float* o_out,
                     int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem = smem_raw + (smem0 - smem_u32(smem_raw));
  constexpr int KOFF = 0, VOFF = 16384, QOFF = 32768, POFF = 34816, MISC = 36864;   // MISC: barrier, tensor-memory slot, abort flag + wait budget
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + MISC + 16);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + MISC + 8);
  const uint32_t bar = smem0 + MISC;
  if (t == 0) {
    *abort_flag = 0;
    set_wait_budget(abort_flag, WAIT_BUDGET_CYCLES);
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;
  // operands: K row t (128 bytes), V row t, P row t, Q chunk
  uint32_t kr[32];
  for (int i = 0; i < 32; ++i) kr[i] = reinterpret_cast<const uint32_t*>(k_bytes + t * 128)[i];
  if (mode == 0) {
    for (int v = 0; v < 4; ++v) tmem_st8(tmem + lane_base + 8 * v, kr + 8 * v);
    tmem_st_wait();
  } else {
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<uint4*>(smem + KOFF + t * 128 + ((c ^ (t & 7)) << 4)) =
          make_uint4(kr[4 * c], kr[4 * c + 1], kr[4 * c + 2], kr[4 * c + 3]);
  }
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(smem + VOFF + t * 128 + ((c ^ (t & 7)) << 4)) =
        reinterpret_cast<const uint4*>(v_bytes + t * 128)[c];
  *reinterpret_cast<uint4*>(smem + POFF + t * 16) = reinterpret_cast<const uint4*>(p_bytes)[t];
  {
    const int r = t >> 3, c = t & 7;
    *reinterpret_cast<uint4*>(smem + QOFF + r * 128 + ((c ^ (r & 7)) << 4)) =
        reinterpret_cast<const uint4*>(q_bytes + r * 128)[c];
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  if (t == 0) {
    tc_fence_after();
    constexpr uint32_t IDESC_S = make_idesc_e4m3(128, 16, 0, 0);
    constexpr uint32_t IDESC_PV = make_idesc_e4m3(128, 16, 1, 1);
    for (int k = 0; k < 4; ++k) {
      const uint64_t bd = make_smem_desc(smem0 + QOFF + k * 32, 16, 1024, 2);
      if (mode == 0) {
        umma_ts(tmem + 32, tmem + k * 8, bd, IDESC_S, k > 0);
      } else {
        const uint64_t ad = make_smem_desc(smem0 + KOFF + k * 32, 16, 1024, 2);
        umma_ss(tmem + 32, ad, bd, IDESC_S, k > 0);
      }
    }
    for (int k = 0; k < 4; ++k) {
      const uint64_t ad = make_smem_desc(smem0 + VOFF + k * 4096, 16, 1024, 2);
      const uint64_t bd = make_smem_desc(smem0 + POFF + k * 512, 128, 128, 0);
      umma_ss(tmem + 48, ad, bd, IDESC_PV, k > 0);
    }
    tc_commit(bar);
  }
  mbar_wait(bar, 0, abort_flag, status);
  tc_fence_after();
  uint32_t r16[16];
  tmem_ld16(tmem + lane_base + 32, r16);
  tmem_ld_wait();
  for (int i = 0; i < 16; ++i) s_out[t * 16 + i] = __uint_as_float(r16[i]);
  tmem_ld16(tmem + lane_base + 48, r16);
  tmem_ld_wait();
  for (int i = 0; i < 16; ++i) o_out[t * 16 + i] = __uint_as_float(r16[i]);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
}

// Wait self test (see foscar_b200.h): every thread waits, with the given cycle budget, for a
// barrier phase that nothing completes. The first waiter to run out raises the CTA's abort flag
// and FQ_STATUS_TIMEOUT; the others fall through; the kernel returns.
__global__ void __launch_bounds__(64, 1) wait_selftest_kernel(long long budget, int* status,
                                                              int* gave_up) {
  __shared__ __align__(8) unsigned long long bar_word;
  __shared__ __align__(8) int ctl_words[4];
  volatile int* abort_flag = ctl_words;
  const uint32_t bar = smem_u32(&bar_word);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    set_wait_budget(abort_flag, budget);
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  mbar_wait(bar, 0, abort_flag, status);    // runs out
  mbar_wait(bar, 0, abort_flag, status);    // returns at once: the CTA has given up
  __syncthreads();
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = *abort_flag;
}

}  // namespace fq

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
#include <algorithm>
#include <cstdlib>

namespace fq {

static int device_sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 148;
  return sms > 0 ? sms : 148;
}

template <int BITS, int D, int GP, int KG = 1, bool MQ = false>
static int launch_decode(DecodeParams& P, cudaStream_t stream) {
  using SP = SmemPlan<BITS, D>;
  constexpr int THREADS = decode_threads(BITS, D);
  int stages = SP::max_ring_stages();
  if (stages > 20) stages = 20;
  if (const char* env = getenv("FOSCAR_B200_RING_STAGES")) {   // tuning knob for experiments
    const int want = atoi(env);
    if (want >= SP::G && want < stages) stages = want;
  }
  // An even ring: the two producers take alternate tiles, so with an even stage count a stage
  // always belongs to the same producer, which then sees every release of it. With an odd count
  // a producer meets a stage every second lap only and waits on a phase parity that an older,
  // still outstanding release also satisfies (a 5-stage ring hung on exactly that).
  stages &= ~1;
  if (stages < SP::G) return FQ_ERR_UNSUPPORTED;  // a group steps the ring by one lap at most
  P.ring_stages = stages;
  P.tile_tokens = SP::TT;
  P.wait_budget = P.a.wait_budget_cycles > 0 ? P.a.wait_budget_cycles : WAIT_BUDGET_CYCLES;
  // Shared memory the ring leaves over holds more decoded work items (32 bytes each), up to
  // one per thread of the CTA's start-up pass.
  constexpr int LIMIT = smem_limit(BITS, D);
  const int spare = LIMIT - 1024 - SP::RING_OFF - stages * SP::STAGE;
  const int more = std::max(0, std::min(spare / 32, THREADS - SP::ITEM_SLOTS));
  P.item_slots = SP::ITEM_SLOTS + more;
  const int smem = SP::RING_OFF + stages * SP::STAGE + more * 32 + 1024;
  static bool configured[64] = {};  // per (BITS, D, GP) instantiation and device
  auto kernel = decode_kernel<BITS, D, GP, KG, MQ>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         LIMIT);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  int ctas = P.a.max_ctas > 0 ? P.a.max_ctas : device_sm_count() * ctas_per_sm(BITS, D);
  int grid = P.a.worklist ? ctas : std::min(ctas, P.num_items);
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

}  // namespace fq


using namespace fq;

extern "C" int fq_ctas_per_sm(int32_t bits, int32_t head_dim) {
  if ((bits != 2 && bits != 4) || (head_dim != 64 && head_dim != 128 && head_dim != 256))
    return FQ_ERR_UNSUPPORTED;
  return head_dim == 256 ? 1 : ctas_per_sm(bits, head_dim);
}

extern "C" int fq_tile_tokens(int32_t bits, int32_t head_dim) {
  if ((bits != 2 && bits != 4) || (head_dim != 64 && head_dim != 128 && head_dim != 256))
    return FQ_ERR_UNSUPPORTED;
  return tile_tokens(bits, head_dim);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int fq_decode(const fq_pools* pools, const fq_decode_args* args, void* stream) {
  if (!pools || !args) return FQ_ERR_BAD_ARG;
  if (!pools->k_codes || !pools->v_codes || !pools->scales) return FQ_ERR_BAD_ARG;
  if (pools->num_kv_heads <= 0 || pools->num_pages <= 0) return FQ_ERR_BAD_ARG;
  // the kernels read these with 16-byte vector loads and copies
  if (!aligned16(pools->k_codes) || !aligned16(pools->v_codes) || !aligned16(pools->scales) ||
      !aligned16(args->q) || (args->worklist && !aligned16(args->worklist)))
    return FQ_ERR_BAD_ARG;
  // sub-head K groups: 64-channel groups at head_dim 128 (bf16 pair rings)
  if (pools->k_groups != 1 &&
      !(pools->k_groups == 2 && pools->head_dim == 128 && pools->scale_bf16))
    return FQ_ERR_UNSUPPORTED;
  if (pools->head_dim != 64 && pools->head_dim != 128 && pools->head_dim != 256)
    return FQ_ERR_UNSUPPORTED;
  if (pools->head_dim == 256 && pools->k_groups != 1) return FQ_ERR_UNSUPPORTED;
  if (pools->bits != 2 && pools->bits != 4) return FQ_ERR_UNSUPPORTED;
  const fq_decode_args& a = *args;
  if (a.batch <= 0 || a.num_qo_heads <= 0 || a.num_qo_heads % pools->num_kv_heads) return FQ_ERR_BAD_ARG;
  if (!a.seq_lens || !a.page_table || !a.table_offsets || !a.q || !a.out) return FQ_ERR_BAD_ARG;
  if (a.out_dtype < 0 || a.out_dtype > 2) return FQ_ERR_BAD_ARG;
  DecodeParams P{};
  P.p = *pools;
  P.a = a;
  // several query tokens per request ride as further columns of their KV head's unit
  P.q_len = a.q_len > 1 ? a.q_len : 1;
  if (P.q_len > 64) return FQ_ERR_BAD_ARG;
  P.gqa = a.num_qo_heads / pools->num_kv_heads;
  P.gqa_inv = (65536 + P.gqa - 1) / P.gqa;
  P.hq = a.num_qo_heads;
  if (P.gqa * P.q_len > 512) return FQ_ERR_TOO_LARGE;   // (column_token's range)
  P.heads_per_kv = P.gqa * P.q_len;
  P.a.num_qo_heads = a.num_qo_heads * P.q_len;
  P.head_tiles = (P.heads_per_kv + 7) / 8;
  // the separate merge launch writes rows in [B, HQ] order only
  if (P.q_len > 1 && (a.worklist ? a.max_splits > 1 : a.kv_splits > 1) && !a.unit_counters)
    return FQ_ERR_UNSUPPORTED;
  const long long units = static_cast<long long>(a.batch) * pools->num_kv_heads * P.head_tiles;
  if (a.worklist) {
    if (a.num_work <= 0 || a.max_splits < 1) return FQ_ERR_BAD_ARG;
    if (!a.o_partial || !a.l_partial || !a.m_partial) return FQ_ERR_BAD_ARG;
    P.num_items = a.num_work;  // capacity; the live row count is read from the list's header
  } else {
    if (a.kv_splits < 1) return FQ_ERR_BAD_ARG;
    if (a.kv_splits > 1 && (!a.o_partial || !a.l_partial || !a.m_partial ||
                            a.kv_splits > a.max_splits))
      return FQ_ERR_BAD_ARG;
    if (units * a.kv_splits > 0x7FFFFFFFLL) return FQ_ERR_TOO_LARGE;
    P.num_items = static_cast<int>(units * a.kv_splits);
  }
  const int gp = std::min(P.heads_per_kv, 8) <= 4 ? 4 : 8;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pools->head_dim == 256) return launch_decode_wide(P, s);
#define FQ_DISPATCH(DD, KK, MM)                                                               \
  do {                                                                                        \
    if (pools->bits == 2)                                                                     \
      return gp == 4 ? launch_decode<2, DD, 4, KK, MM>(P, s)                                  \
                     : launch_decode<2, DD, 8, KK, MM>(P, s);                                 \
    return gp == 4 ? launch_decode<4, DD, 4, KK, MM>(P, s)                                    \
                   : launch_decode<4, DD, 8, KK, MM>(P, s);                                   \
  } while (0)
  // several query tokens per request: builds of their own for whole-head K (f32 or bf16
  // records), so that the one-token builds stay as they are
  if (P.q_len > 1) {
    if (pools->k_groups != 1) return FQ_ERR_UNSUPPORTED;
    if (pools->head_dim == 64) {
      if (pools->scale_bf16) FQ_DISPATCH(64, 3, true);
      FQ_DISPATCH(64, 1, true);
    }
    if (pools->scale_bf16) FQ_DISPATCH(128, 3, true);
    FQ_DISPATCH(128, 1, true);
  }
  if (pools->k_groups == 2) FQ_DISPATCH(128, 2, false);
  if (pools->head_dim == 64) {
    if (pools->scale_bf16) FQ_DISPATCH(64, 3, false);
    FQ_DISPATCH(64, 1, false);
  }
  if (pools->scale_bf16) FQ_DISPATCH(128, 3, false);
  FQ_DISPATCH(128, 1, false);
#undef FQ_DISPATCH
}

// ---------------------------------------------------------------------------------------------
// Split decode for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
namespace fq {
// Scratch for the split partials (o, l, m) of fq_decode_split_static. It lives in the library
// image: every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) float g_static_partials[FQ_STATIC_SCRATCH_BYTES / 4];
}  // namespace fq

extern "C" int fq_decode_split_static(const fq_pools* pools, const fq_decode_args* args,
                                      void* stream) {
  if (!pools || !args) return FQ_ERR_BAD_ARG;
  if (args->worklist != nullptr || args->kv_splits < 1) return FQ_ERR_BAD_ARG;
  if (args->batch <= 0 || args->num_qo_heads <= 0) return FQ_ERR_BAD_ARG;
  if (args->q_len > 1) return FQ_ERR_UNSUPPORTED;   // fq_merge below writes [B, HQ] rows
  const long long rows = static_cast<long long>(args->kv_splits) * args->batch * args->num_qo_heads;
  const long long need = rows * (pools->head_dim + 2) * 4;
  if (need > static_cast<long long>(FQ_STATIC_SCRATCH_BYTES)) return FQ_ERR_SCRATCH_TOO_SMALL;
  // In host code the array's name is only a handle: the device address is asked for once per
  // device, with that device current, and cached.
  static float* base_of_device[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return FQ_ERR_UNSUPPORTED;
  if (base_of_device[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, fq::g_static_partials);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (p == nullptr) return FQ_ERR_UNSUPPORTED;
    base_of_device[dev] = static_cast<float*>(p);
  }
  fq_decode_args a = *args;
  a.unit_counters = nullptr;  // partials are merged by fq_merge below
  a.split_counts = nullptr;
  a.max_splits = a.kv_splits;
  a.o_partial = base_of_device[dev];
  a.l_partial = a.o_partial + rows * pools->head_dim;
  a.m_partial = a.l_partial + rows;
  const int rc = fq_decode(pools, &a, stream);
  if (rc != 0 || a.kv_splits == 1) return rc;
  return fq_merge(a.o_partial, a.l_partial, a.m_partial, nullptr, a.kv_splits, a.kv_splits,
                  a.batch, a.num_qo_heads, pools->num_kv_heads, pools->head_dim, a.o_scale, a.out,
                  a.out_dtype, a.lse, stream);
}

#ifdef FQ_WAIT_PROFILE
extern "C" int fq_debug_set_wait_profile(void* buffer) {
  return static_cast<int>(cudaMemcpyToSymbol(fq::g_wait_profile, &buffer, sizeof(buffer)));
}
#endif

extern "C" int fq_umma_selftest(int32_t mode, const uint8_t* k_bytes, const uint8_t* q_bytes,
                                const uint8_t* v_bytes, const uint8_t* p_bytes, float* s_out,
                                float* o_out, int32_t* status, void* stream) {
  if (!k_bytes || !q_bytes || !v_bytes || !p_bytes || !s_out || !o_out) return FQ_ERR_BAD_ARG;
  const int smem = 36864 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      mode, k_bytes, q_bytes, v_bytes, p_bytes, s_out, o_out, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fq_wait_selftest(int64_t budget_cycles, int32_t* status, int32_t* gave_up,
                                void* stream) {
  if (budget_cycles < 1 || budget_cycles > WAIT_BUDGET_CYCLES) return FQ_ERR_BAD_ARG;
  wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(budget_cycles, status,
                                                                         gave_up);
  return static_cast<int>(cudaGetLastError());
}
