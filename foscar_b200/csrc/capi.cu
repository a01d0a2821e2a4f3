// Host side of the C ABI for the decode path: argument checks, launch configuration, the
// split planners (pure host arithmetic) and small queries.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "decode.cuh"

using namespace fq;

extern "C" const char* fq_version(void) { return "foscar_b200 0.1.0 (sm_100a)"; }

extern "C" const char* fq_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case FQ_ERR_BAD_ARG: return "bad argument";
    case FQ_ERR_UNSUPPORTED: return "unsupported configuration";
    case FQ_ERR_TOO_LARGE: return "problem too large for one launch";
    case FQ_ERR_SCRATCH_TOO_SMALL:
      return "the split partials exceed the library's built-in scratch buffer "
             "(kv_splits * batch * num_qo_heads * (head_dim + 2) * 4 > FQ_STATIC_SCRATCH_BYTES)";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown";
  }
}

extern "C" int64_t fq_workspace_bytes(int32_t max_splits, int32_t batch, int32_t num_qo_heads,
                                      int32_t head_dim) {
  if (max_splits < 1 || batch < 1 || num_qo_heads < 1 || head_dim < 1) return FQ_ERR_BAD_ARG;
  return 4ll * max_splits * batch * num_qo_heads * (head_dim + 2);
}

// Fixed cost of a piece in tile units (pipeline refill, the merge of the groups' states and the
// output), as measured on B200 against the cost of streaming one tile (about 4.7 us against
// 0.34 us per 128-token INT2 tile at head_dim 128).
static long long piece_overhead(int bits, int head_dim) {
  long long ovh = bits == 4 && head_dim == 128 ? 10 : 14;
  if (two_token_build(bits, head_dim)) ovh = 7;   // the same time in 256-token tiles
  if (const char* env = getenv("FOSCAR_B200_PIECE_OVERHEAD")) {   // tuning knob for experiments
    const int v = atoi(env);
    if (v >= 0 && v <= 256) ovh = v;
  }
  return ovh;
}

extern "C" int fq_piece_overhead(int32_t bits, int32_t head_dim) {
  if (bits != 2 && bits != 4) return FQ_ERR_BAD_ARG;
  return static_cast<int>(piece_overhead(bits, head_dim));
}

// Cost, in tile units, of running `base` units cut into s pieces each on `sms` CTAs: the form
// (waves x (tiles + per-piece) + merge) is the one the reference's planner uses
// (src/foscar/_sm100/scheduler.py:101-127); the constants are the balanced planner's: the
// per-piece overhead above, and a merge of s slots by the unit's last piece (about 2 us plus
// 0.1 us a slot).
static double split_cost(long long base, int tiles, int s, long long ovh, int sms) {
  const double waves = std::ceil(static_cast<double>(base) * s / sms);
  return waves * (std::ceil(static_cast<double>(tiles) / s) + static_cast<double>(ovh)) +
         (s > 1 ? 6.0 + 0.3 * s : 0.0);
}

extern "C" int fq_plan_splits(int32_t batch, int32_t num_kv_heads, int32_t head_tiles,
                              int32_t max_kv_len, int32_t bits, int32_t head_dim,
                              int32_t sm_count) {
  if (batch < 1 || num_kv_heads < 1 || head_tiles < 1 || sm_count < 1) return FQ_ERR_BAD_ARG;
  if (bits != 2 && bits != 4) return FQ_ERR_BAD_ARG;
  const long long base = static_cast<long long>(batch) * num_kv_heads * head_tiles;
  const long long ovh = piece_overhead(bits, head_dim);
  const int tt = tile_tokens(bits, head_dim);
  const int tiles = std::max(1, (max_kv_len + tt - 1) / tt);
  int best = 1;
  double best_cost = split_cost(base, tiles, 1, ovh, sm_count);
  for (int s = 2; s <= 64; ++s) {
    if (tiles / s < 4) break;  // at least four tiles per piece
    const double c = split_cost(base, tiles, s, ovh, sm_count);
    // more pieces only for a gain of a few percent: every piece adds partial traffic
    if (c < 0.97 * best_cost) { best = s; best_cost = c; }
  }
  return best;
}

// Words an explicit list needs for `units` units on `num_ctas` CTAs (a cut adds one piece).
static long long worklist_words(long long units, int num_ctas) {
  const long long starts = (static_cast<long long>(num_ctas) + 1 + 7) / 8 * 8;
  return WORK_WORDS + starts + WORK_WORDS * (units + num_ctas);
}

// Balanced plan: every piece (a unit, or a part of a unit cut between CTAs) costs its tile count
// plus a fixed overhead. The units (request, KV head, head tile) are dealt to the CTAs in order;
// a CTA takes tiles until its share of the total cost is used up, and the unit in hand continues
// on the next CTA as a new piece. No unit is cut into more than max_splits pieces: the share is
// raised until the longest unit fits that many, and a unit's last allowed piece takes all that
// is left of it (the CTAs after it then take less). List layout (int32 words):
// header {pieces, units, ctas, rows' word offset, 0...}, cta_start[ctas + 1] padded to 8 words,
// then one row of 8 words per piece.
extern "C" int fq_plan_worklist(const int32_t* seq_lens, int32_t batch, int32_t num_kv_heads,
                                int32_t head_tiles, int32_t num_ctas, int32_t max_splits,
                                int32_t* worklist, int32_t max_words, int32_t* split_counts,
                                int32_t bits, int32_t head_dim) {
  if (!seq_lens || !worklist || !split_counts) return FQ_ERR_BAD_ARG;
  if (batch < 1 || num_kv_heads < 1 || head_tiles < 1 || num_ctas < 1 || max_splits < 1)
    return FQ_ERR_BAD_ARG;
  if (bits != 2 && bits != 4) return FQ_ERR_BAD_ARG;
  const long long OVH = piece_overhead(bits, head_dim);
  const long long MIN_PIECE = 4;   // a CTA with less room than this for tiles passes the unit on
  const int upr = num_kv_heads * head_tiles;
  const int tt = tile_tokens(bits, head_dim);
  const long long units = static_cast<long long>(batch) * upr;
  if (worklist_words(units, num_ctas) > max_words) return FQ_ERR_TOO_LARGE;
  auto tiles_of = [&](int b) -> long long {
    return seq_lens[b] > 0 ? (static_cast<long long>(seq_lens[b]) + tt - 1) / tt : 0;
  };
  long long total = 0, longest = 0;
  for (int b = 0; b < batch; ++b) {
    total += (tiles_of(b) + OVH) * upr;
    longest = std::max(longest, tiles_of(b));
  }
  total += OVH * (num_ctas - 1);   // about one cut, hence one more piece, per CTA boundary
  long long share = std::max<long long>(OVH + 1, (total + num_ctas - 1) / num_ctas);
  // The longest unit in so many pieces: one may be the remainder of a CTA, the others full.
  // Beyond the caller's cap, a unit of T tiles is not worth more than about sqrt(2 T) pieces:
  // every piece adds a slot to the unit's merge, which the unit's last piece runs alone (a
  // 32K-token context alone on the GPU was otherwise cut into 40 to 60 pieces of two tiles).
  const int worth = std::max(2, static_cast<int>(std::sqrt(2.0 * static_cast<double>(longest))));
  const long long full_pieces = std::max(1, std::min(max_splits, worth) - 1);
  share = std::max(share, OVH + (longest + full_pieces - 1) / full_pieces);
  const int starts_words = (num_ctas + 1 + 7) / 8 * 8;
  int32_t* cta_start = worklist + WORK_WORDS;
  int32_t* rows = worklist + WORK_WORDS + starts_words;
  std::memset(worklist, 0, sizeof(int32_t) * (WORK_WORDS + starts_words));
  int pieces_total = 0, cta = 0;
  long long room = share;   // cost the CTA in hand can still take
  cta_start[0] = 0;
  for (long long u = 0; u < units; ++u) {
    const int b = static_cast<int>(u / upr), kvh = static_cast<int>(u % upr) / head_tiles,
              ht = static_cast<int>(u % upr) % head_tiles;
    const int tiles = static_cast<int>(tiles_of(b));
    const int first_row = pieces_total;
    int t0 = 0, pieces = 0;
    for (;;) {
      const bool last_cta = cta == num_ctas - 1;
      const bool last_piece = pieces == max_splits - 1;   // the unit may not be cut again
      // room for the overhead plus a worthwhile number of tiles, or the rest of the unit
      if (!last_cta && room < OVH + std::min<long long>(MIN_PIECE, tiles - t0) &&
          !(last_piece && pieces > 0 && room > OVH)) {
        cta_start[++cta] = pieces_total;
        room = share + std::min<long long>(room, 0);   // an overfull CTA is paid for by the next
        continue;
      }
      int t1 = tiles;
      if (!last_cta && !last_piece && OVH + (tiles - t0) > room)
        t1 = t0 + static_cast<int>(room - OVH);
      int32_t* row = rows + static_cast<long long>(WORK_WORDS) * pieces_total;
      row[0] = b; row[1] = kvh; row[2] = ht; row[3] = t0; row[4] = t1; row[5] = pieces;
      row[6] = 0; row[7] = 0;
      ++pieces_total;
      ++pieces;
      room -= OVH + (t1 - t0);
      t0 = t1;
      if (t0 >= tiles) break;
    }
    if (pieces > max_splits) return FQ_ERR_TOO_LARGE;   // cannot happen; kept as a check
    if (pieces == 1) rows[static_cast<long long>(WORK_WORDS) * first_row + 5] = -1;
    split_counts[u] = pieces;
  }
  while (cta < num_ctas) cta_start[++cta] = pieces_total;
  worklist[0] = pieces_total;
  worklist[1] = static_cast<int32_t>(units);
  worklist[2] = num_ctas;
  worklist[3] = WORK_WORDS + starts_words;
  return pieces_total;
}

extern "C" int fq_worklist_attach_requests(int32_t* worklist, int64_t words,
                                           const int32_t* seq_lens,
                                           const int32_t* table_offsets, int32_t batch) {
  if (!worklist || !seq_lens || !table_offsets || batch < 1 || words < WORK_WORDS)
    return FQ_ERR_BAD_ARG;
  const long long pieces = worklist[0], rows_off = worklist[3];
  if (pieces < 0 || rows_off < WORK_WORDS || rows_off + pieces * WORK_WORDS > words)
    return FQ_ERR_BAD_ARG;
  int32_t* rows = worklist + rows_off;
  for (long long i = 0; i < pieces; ++i) {
    int32_t* row = rows + i * WORK_WORDS;
    if (row[0] < 0 || row[0] >= batch) return FQ_ERR_BAD_ARG;
    row[6] = seq_lens[row[0]];
    row[7] = table_offsets[row[0]];
  }
  worklist[4] = 1;
  return 0;
}

extern "C" int64_t fq_worklist_words(int32_t batch, int32_t num_kv_heads, int32_t head_tiles,
                                     int32_t num_ctas) {
  if (batch < 1 || num_kv_heads < 1 || head_tiles < 1 || num_ctas < 1) return FQ_ERR_BAD_ARG;
  return worklist_words(static_cast<long long>(batch) * num_kv_heads * head_tiles, num_ctas);
}
