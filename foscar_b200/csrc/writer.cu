// Cache writer: quantizes bf16 K/V rows (or lays out engine-quantized rows) into the packed
// INT2/INT4 pools with their per-token scale records, and keeps the per-page V-scale maxima
// and their exponent count table.
//
// Result contract (what a launch leaves in the pools) follows the reference writer,
// src/foscar/_append_core.py:18-22 (runs), :73-109 (tail clear, page maxima), :533-587
// (quantizer arithmetic), :589-628 (records); code placement src/foscar/_sm100/code_layout.py.
//
// Structure is this library's own. Two stream-ordered launches:
//   1. page_start_kernel: every token at in-page position 0 begins a new use of its page: the
//      page's scale records are zeroed and its maximum cell is cleared (count moved out).
//   2. append_kernel: a half-warp per row (K and V of a (token, KV head) pair side by side in a
//      warp, four pairs per pass) quantizes, packs, stores the row and the record, and raises
//      the page maximum with atomicMax, moving the count between bins.
// Zero-then-overwrite leaves exactly the bytes "clear every position no token of the launch
// writes" leaves, and needs no scan of the slot map. HBM-bound: 2*D*2 bytes read per (token,
// head), coalesced 16-byte-per-lane-group loads.
#include <algorithm>

#include "common.cuh"

namespace fq {

constexpr float S_CLAMP = 1.0e-8f;
constexpr float ENVELOPE = 18446744073709551616.0f;       // 2^64
constexpr float DIVIDEND_FLOOR = 8.673617379884035e-19f;  // 2^-60

struct WriterArgs {
  fq_pools p;
  const void* k;
  const void* v;
  long long k_stride, v_stride;  // token strides in elements
  const float* k_scale;
  const float* k_zero;
  const float* v_scale;
  const float* v_zero;
  const long long* slots;
  // page-group mode (slots == nullptr): token i is row i % 64 of group i / 64, which goes to
  // page page_ids[i / 64]; rows at or past valid[i / 64] are skipped
  const int* page_ids;
  const int* valid;
  int num_tokens;
  int k_clip, v_clip;
  int* status;
};

// Where a token goes: its slot (page * 64 + position), negative for a token to skip.
__device__ inline long long slot_of(const WriterArgs& a, int token) {
  if (a.slots != nullptr) return a.slots[token];
  const int group = token >> 6, pos = token & (PAGE - 1);
  if (a.valid != nullptr && pos >= __ldg(a.valid + group)) return -1;
  const int page = __ldg(a.page_ids + group);
  // a page id outside the pool is reported by the row pass as a slot outside the cache
  if (page < 0) return static_cast<long long>(a.p.num_pages) * PAGE;
  return static_cast<long long>(page) * PAGE + pos;
}

__device__ inline float warp_group_min(float x, int lanes) {
  for (int o = lanes >> 1; o > 0; o >>= 1) x = fminf(x, __shfl_xor_sync(0xFFFFFFFFu, x, o));
  return x;
}
__device__ inline float warp_group_max(float x, int lanes) {
  for (int o = lanes >> 1; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xFFFFFFFFu, x, o));
  return x;
}

// Bytes of one (page, head) scale block and where a token's records sit in it.
__device__ inline long long scale_block_bytes(const fq_pools& p) {
  const int esz = p.scale_bf16 ? 2 : 4;
  int elems = p.k_groups == 1 ? 4 * PAGE : 2 * p.k_groups * PAGE + 2 * PAGE;
  if (p.k_channel_group != 0) elems = 2 * PAGE + 2 * p.head_dim;   // V ring, K channel rows
  return static_cast<long long>(elems) * esz;
}

// Move one cell's count in the table when the cell went from `old` to `now`.
__device__ inline void settle_count(uint32_t* hist, uint32_t old, uint32_t now) {
  const bool c_old = (old & 0x7FFFFFFFu) != 0, c_new = (now & 0x7FFFFFFFu) != 0;
  const uint32_t b_old = vmax_bucket(old), b_new = vmax_bucket(now);
  if (c_old && c_new && b_old == b_new) return;
  if (c_new) atomicAdd(hist + b_new, 1u);
  if (c_old) atomicAdd(hist + b_old, 0xFFFFFFFFu);
}

// The same into a block-local table of signed deltas (flushed once per block): the pool's counts
// live in a handful of bins, and a global atomic per raised cell serialises on those addresses.
__device__ inline void settle_count_local(int* local, uint32_t old, uint32_t now) {
  const bool c_old = (old & 0x7FFFFFFFu) != 0, c_new = (now & 0x7FFFFFFFu) != 0;
  const uint32_t b_old = vmax_bucket(old), b_new = vmax_bucket(now);
  if (c_old && c_new && b_old == b_new) return;
  if (c_new) atomicAdd(local + b_new, 1);
  if (c_old) atomicAdd(local + b_old, -1);
}

// -------------------------------------------------------------------------------------------
// 1. page starts
// -------------------------------------------------------------------------------------------
__global__ void page_start_kernel(WriterArgs a) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int hkv = a.p.num_kv_heads;
  if (warp >= a.num_tokens * hkv) return;
  const int token = warp / hkv, head = warp % hkv;
  const long long slot = slot_of(a, token);
  if (slot < 0 || (slot & (PAGE - 1)) != 0) return;
  const long long page = slot >> 6;
  if (page >= a.p.num_pages) return;  // reported by append_kernel
  const long long bb = scale_block_bytes(a.p);
  uint4* block = reinterpret_cast<uint4*>(static_cast<char*>(a.p.scales) +
                                          (page * hkv + head) * bb);
  for (int i = lane; i < bb / 16; i += 32) block[i] = make_uint4(0, 0, 0, 0);
  if (lane == 0 && a.p.v_page_max != nullptr) {
    const uint32_t old = atomicExch(a.p.v_page_max + page * hkv + head, 0u);
    if ((old & 0x7FFFFFFFu) != 0) atomicAdd(a.p.v_max_hist + vmax_bucket(old), 0xFFFFFFFFu);
  }
}

// -------------------------------------------------------------------------------------------
// 2. rows
// -------------------------------------------------------------------------------------------

// A half-warp holds one row: lanes 0-15 a token's K row, lanes 16-31 its V row, D/16 channels a
// lane. The two rows' reductions, scale divisions, packing and record hand-over then share their
// instructions, and a warp takes ROWS_PER_WARP (token, head) pairs per pass with all their loads
// issued before the first is used (at one warp per pair the kernel spent most of its time in the
// per-pair fixed part and in waiting for two small loads).
constexpr int ROWS_PER_WARP = 4;

// Reduce over the `lanes` (16, 8 or 4) neighbouring lanes of a half-warp group; every lane of the
// warp executes all four exchanges.
__device__ __forceinline__ void group_min_max(float& mn, float& mx, int lanes) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {
    const float a = __shfl_xor_sync(0xFFFFFFFFu, mn, o), b = __shfl_xor_sync(0xFFFFFFFFu, mx, o);
    if (o < lanes) {
      mn = fminf(mn, a);
      mx = fmaxf(mx, b);
    }
  }
}

// Per-row clip threshold: the element at `index` of the row's |x| sorted ascending, found by a
// radix select over the 15 value bits of a bf16 magnitude (bits 30..16 of the f32 pattern). The
// row sits in the 16 lanes of a half-warp.
template <int CH>
__device__ inline float clip_threshold(const float (&x)[CH], int index) {
  uint32_t prefix = 0;
  int rank = index;
  for (int bit = 30; bit >= 16; --bit) {
    const uint32_t decided = 0x80000000u - (1u << bit);  // bits 30..bit
    int count = 0;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const uint32_t mag = __float_as_uint(x[i]) & 0x7FFFFFFFu;
      count += ((mag & decided) == prefix) ? 1 : 0;
    }
    for (int o = 8; o > 0; o >>= 1) count += __shfl_xor_sync(0xFFFFFFFFu, count, o);
    if (rank >= count) {
      rank -= count;
      prefix |= 1u << bit;
    }
  }
  return __uint_as_float(prefix);
}

// Quantize the CH values of this lane against its group's (s, z) into the lane's part of the
// row's code words: WPL whole words, or its fields of a word shared with neighbouring lanes.
template <int BITS, int CH, int WPL>
__device__ inline void quantize_fields(const float (&x)[CH], float s, float z, int c0, bool inside,
                                       uint32_t (&word)[WPL]) {
  constexpr int QMAX = (1 << BITS) - 1;
  constexpr int W = 32 / BITS;
#pragma unroll
  for (int j = 0; j < WPL; ++j) word[j] = 0;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    float xv = x[i];
    if (!inside) xv = fminf(fmaxf(xv, -ENVELOPE), ENVELOPE);
    const float dividend = fmaxf(__fsub_rn(xv, z), DIVIDEND_FLOOR);
    int q = __float2int_rn(__fdiv_rn(dividend, s));
    q = min(q, QMAX);
    word[WPL == 1 ? 0 : i / W] |= static_cast<uint32_t>(q) << (code_bit_offset<BITS>(c0 + i) & 31);
  }
}

template <int BITS, int D, bool PREQ>
__device__ __forceinline__ void append_rows(const WriterArgs& a, int* hist_delta, long long first,
                                            long long total);

template <int BITS, int D, bool PREQ>
__global__ void __launch_bounds__(256) append_kernel(WriterArgs a) {
  __shared__ int hist_delta[FQ_VMAX_BINS];
  // A launch that follows this one under programmatic stream serialization (the decode of the
  // same step, flags bit 0 of fq_decode_args) may begin its on-chip set-up now; it waits for
  // this grid to complete before its first global access (the reference's writer does the
  // same, src/foscar/_append_core.py:1154-1159). A no-op otherwise.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int i = threadIdx.x; i < FQ_VMAX_BINS; i += blockDim.x) hist_delta[i] = 0;
  __syncthreads();
  // resident CTAs, every warp striding over the (token, head) pairs ROWS_PER_WARP at a time
  const long long total = static_cast<long long>(a.num_tokens) * a.p.num_kv_heads;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (long long first = warp * ROWS_PER_WARP; first < total; first += warps * ROWS_PER_WARP)
    append_rows<BITS, D, PREQ>(a, hist_delta, first, total);
  __syncthreads();
  if (a.p.v_max_hist != nullptr)
    for (int i = threadIdx.x; i < FQ_VMAX_BINS; i += blockDim.x)
      if (hist_delta[i] != 0) atomicAdd(a.p.v_max_hist + i, static_cast<uint32_t>(hist_delta[i]));
}

template <int BITS, int D, bool PREQ>
__device__ __forceinline__ void append_rows(const WriterArgs& a, int* hist_delta, long long first,
                                            long long total) {
  constexpr int R = ROWS_PER_WARP;
  constexpr int CH = D / 16;                   // channels per lane: 4, 8 or 16
  constexpr int W = 32 / BITS;                 // codes per word
  constexpr int WPL = CH >= W ? CH / W : 1;    // whole words per lane ...
  constexpr int LPW = CH >= W ? 1 : W / CH;    // ... or lanes sharing one word
  constexpr int RB = D * BITS / 8;             // row bytes
  constexpr int QMAX = (1 << BITS) - 1;
  constexpr int IN_WORDS = PREQ ? CH / 4 : CH / 2;   // 32-bit words of a lane's input
  const int lane = threadIdx.x & 31;
  const int half = lane >> 4, hl = lane & 15;  // half 0: the K row, half 1: the V row
  const int c0 = hl * CH;
  const int hkv = a.p.num_kv_heads;
  const int kg = a.p.k_groups;
  const bool kch = a.p.k_channel_group != 0;   // K goes by whole pages (append_k_channel_kernel)
  const bool idle = kch && half == 0;
  const int glanes = half == 0 ? 16 / kg : 16; // lanes of this lane's quantization group

  // ---- every pair's slot and rows are requested before any is used
  int token[R], head[R];
  long long slot[R];
  uint32_t in[R][IN_WORDS];
  // (pairs are numbered token-major and a launch has fewer than 2^31 of them: one 32-bit
  // division per pass, the pass's other pairs by stepping the head)
  int tok = static_cast<int>(static_cast<uint32_t>(first) / static_cast<uint32_t>(hkv));
  int hd = static_cast<int>(first) - tok * hkv;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const bool live = first + r < total;
    token[r] = live ? tok : 0;
    head[r] = live ? hd : 0;
    if (++hd == hkv) { hd = 0; ++tok; }
    slot[r] = live ? slot_of(a, token[r]) : -1;
#pragma unroll
    for (int i = 0; i < IN_WORDS; ++i) in[r][i] = 0;
    if (!live || idle) continue;
    if (!PREQ) {
      const __nv_bfloat16* row = static_cast<const __nv_bfloat16*>(half ? a.v : a.k) +
                                 token[r] * (half ? a.v_stride : a.k_stride) +
                                 static_cast<long long>(head[r]) * D + c0;
      if constexpr (CH == 4) {
        const uint2 t = __ldg(reinterpret_cast<const uint2*>(row));
        in[r][0] = t.x; in[r][1] = t.y;
      } else {
#pragma unroll
        for (int i = 0; i < CH / 8; ++i) {
          const uint4 t = __ldg(reinterpret_cast<const uint4*>(row) + i);
          in[r][4 * i] = t.x; in[r][4 * i + 1] = t.y; in[r][4 * i + 2] = t.z; in[r][4 * i + 3] = t.w;
        }
      }
    } else {
      // engine-quantized: one code per byte
      const uint8_t* row = static_cast<const uint8_t*>(half ? a.v : a.k) +
                           (static_cast<long long>(token[r]) * hkv + head[r]) * D + c0;
#pragma unroll
      for (int i = 0; i < IN_WORDS; ++i) in[r][i] = __ldg(reinterpret_cast<const uint32_t*>(row) + i);
    }
  }
  // the pages' current maxima, wanted only at the very end of each pair
  uint32_t cell_seen[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    cell_seen[r] = 0;
    const long long page = slot[r] >> 6;
    if (lane == 0 && slot[r] >= 0 && page < a.p.num_pages && a.p.v_page_max != nullptr)
      cell_seen[r] = *reinterpret_cast<volatile uint32_t*>(a.p.v_page_max + page * hkv + head[r]);
  }

#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (slot[r] < 0) continue;                 // (warp-uniform)
    const long long page = slot[r] >> 6;
    const int pos = static_cast<int>(slot[r] & (PAGE - 1));
    if (page >= a.p.num_pages) {
      if (lane == 0 && a.status) atomicOr(a.status, FQ_STATUS_BAD_SLOT);
      continue;
    }
    float s, z;               // this lane's group's record
    uint32_t word[WPL];
    if (!PREQ) {
      float x[CH];
#pragma unroll
      for (int i = 0; i < CH / 2; ++i) {
        x[2 * i] = __uint_as_float(in[r][i] << 16);
        x[2 * i + 1] = __uint_as_float(in[r][i] & 0xFFFF0000u);
      }
      if (a.k_clip >= 0 || a.v_clip >= 0) {
        const int index = half ? a.v_clip : a.k_clip;
        const float t = clip_threshold<CH>(x, index < 0 ? 0 : index);
        if (index >= 0) {
#pragma unroll
          for (int i = 0; i < CH; ++i) x[i] = fminf(fmaxf(x[i], -t), t);
        }
      }
      float mn = x[0], mx = x[0];
#pragma unroll
      for (int i = 1; i < CH; ++i) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
      }
      group_min_max(mn, mx, glanes);
      const bool inside = mx <= ENVELOPE && mn >= -ENVELOPE;
      z = fminf(fmaxf(mn, -ENVELOPE), ENVELOPE);
      const float top = fminf(fmaxf(mx, -ENVELOPE), ENVELOPE);
      s = __fdiv_rn(fmaxf(__fsub_rn(top, z), S_CLAMP), static_cast<float>(QMAX));
      quantize_fields<BITS, CH, WPL>(x, s, z, c0, inside, word);
    } else {
      // codes masked to the stored width; records saturated
#pragma unroll
      for (int j = 0; j < WPL; ++j) word[j] = 0;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const uint32_t q = (in[r][i / 4] >> (8 * (i % 4))) & QMAX;
        word[WPL == 1 ? 0 : i / W] |= q << (code_bit_offset<BITS>(c0 + i) & 31);
      }
      const float s_lo = __fdiv_rn(S_CLAMP, static_cast<float>(QMAX));
      const float s_hi = __fdiv_rn(2.0f * ENVELOPE, static_cast<float>(QMAX));
      const long long row = static_cast<long long>(token[r]) * hkv + head[r];
      const long long rec = half ? row : row * kg + hl / (16 / kg);
      // (K by whole pages: the K half has neither codes nor a record of its own here)
      s = idle ? s_lo : fminf(fmaxf(__ldg((half ? a.v_scale : a.k_scale) + rec), s_lo), s_hi);
      z = idle ? 0.f
               : fminf(fmaxf(__ldg((half ? a.v_zero : a.k_zero) + rec), -ENVELOPE), ENVELOPE);
    }

    // code words shared by neighbouring lanes are assembled, then one lane per word stores
#pragma unroll
    for (int o = 1; o < LPW; o <<= 1) word[0] |= __shfl_xor_sync(0xFFFFFFFFu, word[0], o);
    const long long row_index = (page * hkv + head[r]) * PAGE + pos;
    if (!idle && hl % LPW == 0) {
      uint32_t* dst = reinterpret_cast<uint32_t*>((half ? a.p.v_codes : a.p.k_codes) +
                                                  row_index * RB) + c0 / W;
      if constexpr (WPL == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(word[0], word[1]);
      else dst[0] = word[0];
    }

    // the records meet in lane 0: V's from lane 16, the K groups' from their first lanes
    const float sv = __shfl_sync(0xFFFFFFFFu, s, 16), zv = __shfl_sync(0xFFFFFFFFu, z, 16);
    const float sk = s, zk = z;
    float sk1 = 0.f, zk1 = 0.f, sk2 = 0.f, zk2 = 0.f, sk3 = 0.f, zk3 = 0.f;
    if (kg > 1) {   // (warp-uniform)
      sk1 = __shfl_sync(0xFFFFFFFFu, s, (16 / kg) * 1 % 16);
      zk1 = __shfl_sync(0xFFFFFFFFu, z, (16 / kg) * 1 % 16);
      sk2 = __shfl_sync(0xFFFFFFFFu, s, (16 / kg) * 2 % 16);
      zk2 = __shfl_sync(0xFFFFFFFFu, z, (16 / kg) * 2 % 16);
      sk3 = __shfl_sync(0xFFFFFFFFu, s, (16 / kg) * 3 % 16);
      zk3 = __shfl_sync(0xFFFFFFFFu, z, (16 / kg) * 3 % 16);
    }
    if (lane == 0) {
      char* block = static_cast<char*>(a.p.scales) +
                    (page * hkv + head[r]) * scale_block_bytes(a.p);
      uint32_t sv_bits;
      if (kch) {
        // V ring at the front of the block: token t's (s_v, z_v) at element 2t
        if (!a.p.scale_bf16) {
          reinterpret_cast<float2*>(block)[pos] = make_float2(sv, zv);
          sv_bits = __float_as_uint(sv);
        } else {
          const __nv_bfloat162 h = __floats2bfloat162_rn(sv, zv);
          const uint32_t vrec = *reinterpret_cast<const uint32_t*>(&h);
          reinterpret_cast<uint32_t*>(block)[pos] = vrec;
          sv_bits = vrec << 16;
        }
      } else if (!a.p.scale_bf16) {
        // f32 pool: whole-head K only
        reinterpret_cast<float4*>(block)[pos] = make_float4(sk, zk, sv, zv);
        sv_bits = __float_as_uint(sv);
      } else {
        auto pack = [](float s_, float z_) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(s_, z_);
          return *reinterpret_cast<const uint32_t*>(&h);
        };
        const uint32_t vrec = pack(sv, zv);
        sv_bits = vrec << 16;
        if (kg == 1) {
          reinterpret_cast<uint2*>(block)[pos] = make_uint2(pack(sk, zk), vrec);
        } else {
          uint32_t* kring = reinterpret_cast<uint32_t*>(block) + kg * pos;
          kring[0] = pack(sk, zk);
          kring[1] = pack(sk1, zk1);
          if (kg == 4) {
            kring[2] = pack(sk2, zk2);
            kring[3] = pack(sk3, zk3);
          }
          reinterpret_cast<uint32_t*>(block + 2 * kg * PAGE * 2)[pos] = vrec;
        }
      }
      if (a.p.v_page_max != nullptr) {
        uint32_t* cell = a.p.v_page_max + page * hkv + head[r];
        if (sv_bits > cell_seen[r]) {   // a stale (smaller) reading only costs a redundant atomicMax
          const uint32_t old = atomicMax(cell, sv_bits);
          if (old < sv_bits) settle_count_local(hist_delta, old, sv_bits);
        }
      }
    }
  }
}

// A channel's record after the block's V ring: row 0 s_d, row 1 z_d, in the pool's record type.
template <int D>
__device__ inline void store_channel_record(const fq_pools& p, long long blk, int d, float s,
                                            float z) {
  char* block = static_cast<char*>(p.scales) + blk * scale_block_bytes(p);
  if (!p.scale_bf16) {
    float* rec = reinterpret_cast<float*>(block) + 2 * PAGE;
    rec[d] = s;
    rec[D + d] = z;
  } else {
    __nv_bfloat16* rec = reinterpret_cast<__nv_bfloat16*>(block) + 2 * PAGE;
    rec[d] = __float2bfloat16_rn(s);
    rec[D + d] = __float2bfloat16_rn(z);
  }
}

// A page's first n token rows from one code byte per (token, channel) in shared memory: field f
// of word w holds channel W*w + f/2 + (W/2)*(f%2) (src/foscar/_sm100/code_layout.py:24-43).
template <int BITS, int D>
__device__ inline void store_packed_rows(const uint8_t* codes, int n, uint8_t* page_rows) {
  constexpr int W = 32 / BITS;             // codes per word
  constexpr int WORDS = D * BITS / 32;     // words per token row
  uint32_t* rows = reinterpret_cast<uint32_t*>(page_rows);
  for (int i = threadIdx.x; i < n * WORDS; i += blockDim.x) {
    const int j = i / WORDS, w = i % WORDS;
    const uint8_t* src = codes + j * D + W * w;
    uint32_t word = 0;
#pragma unroll
    for (int f = 0; f < W; ++f)
      word |= static_cast<uint32_t>(src[(f >> 1) + (W / 2) * (f & 1)]) << (BITS * f);
    rows[j * WORDS + w] = word;
  }
}

// -------------------------------------------------------------------------------------------
// 3. K per channel over a page's tokens
// -------------------------------------------------------------------------------------------
// One CTA per (page group, KV head): the group's K rows go to shared memory; thread d takes
// channel d through the token-wise quantizer's arithmetic along the token axis (exact min/max
// over the valid tokens, z = clamp(min), s = max(max - z, 1e-8) / qmax, codes from the f32 s)
// and leaves one code byte per (token, channel); the CTA then assembles the packed token rows
// (src/foscar/_sm100/code_layout.py:24-43) and stores them and the channel records.
template <int BITS, int D>
__global__ void __launch_bounds__(256) append_k_channel_kernel(WriterArgs a) {
  constexpr int QMAX = (1 << BITS) - 1;
  extern __shared__ __align__(16) uint8_t smem_k[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_k);   // [64][D]
  uint8_t* codes = smem_k + PAGE * D * 2;                            // [64][D]
  const int hkv = a.p.num_kv_heads;
  const int group = blockIdx.x / hkv, head = blockIdx.x % hkv;
  int n = a.valid != nullptr ? __ldg(a.valid + group) : PAGE;
  if (n > PAGE) n = PAGE;
  if (n <= 0) return;
  const int page = __ldg(a.page_ids + group);
  if (page < 0 || page >= a.p.num_pages) return;   // reported by the row pass
  // the group's rows, 16 bytes per thread and step
  constexpr int CPR = D / 8;   // 16-byte chunks per row
  for (int i = threadIdx.x; i < n * CPR; i += blockDim.x) {
    const int j = i / CPR, c = i % CPR;
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(a.k) +
                               (static_cast<long long>(group) * PAGE + j) * a.k_stride +
                               static_cast<long long>(head) * D + 8 * c;
    reinterpret_cast<uint4*>(tile + j * D)[c] = __ldg(reinterpret_cast<const uint4*>(src));
  }
  __syncthreads();
  const long long blk = static_cast<long long>(page) * hkv + head;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float mn = __bfloat162float(tile[d]), mx = mn;
    for (int j = 1; j < n; ++j) {
      const float x = __bfloat162float(tile[j * D + d]);
      mn = fminf(mn, x);
      mx = fmaxf(mx, x);
    }
    const bool inside = mx <= ENVELOPE && mn >= -ENVELOPE;
    const float z = fminf(fmaxf(mn, -ENVELOPE), ENVELOPE);
    const float top = fminf(fmaxf(mx, -ENVELOPE), ENVELOPE);
    const float s = __fdiv_rn(fmaxf(__fsub_rn(top, z), S_CLAMP), static_cast<float>(QMAX));
    for (int j = 0; j < n; ++j) {
      float x = __bfloat162float(tile[j * D + d]);
      if (!inside) x = fminf(fmaxf(x, -ENVELOPE), ENVELOPE);
      const float dividend = fmaxf(__fsub_rn(x, z), DIVIDEND_FLOOR);
      const int q = min(__float2int_rn(__fdiv_rn(dividend, s)), QMAX);
      codes[j * D + d] = static_cast<uint8_t>(q);
    }
    store_channel_record<D>(a.p, blk, d, s, z);
  }
  __syncthreads();
  store_packed_rows<BITS, D>(codes, n, a.p.k_codes + blk * PAGE * (D * BITS / 8));
}

// The same pages from an engine that quantized them itself: K codes one per byte
// [P * 64, HKV, D] with f32 (s_d, z_d) [P, HKV, D] per page and channel. One CTA per (page
// group, KV head) masks the codes to the stored width, packs the token rows and stores the
// channel records, saturated like the token-wise records of fq_append_quantized.
template <int BITS, int D>
__global__ void __launch_bounds__(256) pack_k_channel_kernel(WriterArgs a) {
  constexpr int QMAX = (1 << BITS) - 1;
  __shared__ __align__(16) uint8_t codes[PAGE * D];
  const int hkv = a.p.num_kv_heads;
  const int group = blockIdx.x / hkv, head = blockIdx.x % hkv;
  int n = a.valid != nullptr ? __ldg(a.valid + group) : PAGE;
  if (n > PAGE) n = PAGE;
  if (n <= 0) return;
  const int page = __ldg(a.page_ids + group);
  if (page < 0 || page >= a.p.num_pages) return;   // reported by the row pass
  constexpr int WPR = D / 4;   // 32-bit words of a token's code bytes
  for (int i = threadIdx.x; i < n * WPR; i += blockDim.x) {
    const int j = i / WPR, c = i % WPR;
    const uint8_t* src = static_cast<const uint8_t*>(a.k) +
                         ((static_cast<long long>(group) * PAGE + j) * hkv + head) * D;
    reinterpret_cast<uint32_t*>(codes + j * D)[c] =
        __ldg(reinterpret_cast<const uint32_t*>(src) + c) & (0x01010101u * QMAX);
  }
  const long long blk = static_cast<long long>(page) * hkv + head;
  const float s_lo = __fdiv_rn(S_CLAMP, static_cast<float>(QMAX));
  const float s_hi = __fdiv_rn(2.0f * ENVELOPE, static_cast<float>(QMAX));
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const long long rec = (static_cast<long long>(group) * hkv + head) * D + d;
    const float s = fminf(fmaxf(__ldg(a.k_scale + rec), s_lo), s_hi);
    const float z = fminf(fmaxf(__ldg(a.k_zero + rec), -ENVELOPE), ENVELOPE);
    store_channel_record<D>(a.p, blk, d, s, z);
  }
  __syncthreads();
  store_packed_rows<BITS, D>(codes, n, a.p.k_codes + blk * PAGE * (D * BITS / 8));
}

// -------------------------------------------------------------------------------------------
// recount
// -------------------------------------------------------------------------------------------
__global__ void recount_kernel(uint32_t* cells, long long n, uint32_t* hist) {
  __shared__ uint32_t local[FQ_VMAX_BINS];
  for (int i = threadIdx.x; i < FQ_VMAX_BINS; i += blockDim.x) local[i] = 0;
  __syncthreads();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t v = cells[i] & 0x7FFFFFFFu;
    cells[i] = v;
    if (v != 0) atomicAdd(&local[vmax_bucket(v)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < FQ_VMAX_BINS; i += blockDim.x)
    if (local[i]) atomicAdd(hist + i, local[i]);
}

template <bool PREQ>
static int launch_append(const WriterArgs& a, cudaStream_t stream) {
  const long long pairs = static_cast<long long>(a.num_tokens) * a.p.num_kv_heads;
  if (pairs == 0) return 0;
  const int threads = 256;
  const long long start_blocks = (pairs * 32 + threads - 1) / threads;   // a warp per pair
  if (start_blocks > 0x7FFFFFFFLL || pairs > 0x7FFFFFFFLL) return FQ_ERR_TOO_LARGE;
  page_start_kernel<<<static_cast<unsigned>(start_blocks), threads, 0, stream>>>(a);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    sms = 148;
  // the row pass: resident CTAs, a warp taking ROWS_PER_WARP pairs per pass
  const long long want = (pairs + 8 * ROWS_PER_WARP - 1) / (8 * ROWS_PER_WARP);
#define FQ_LAUNCH(B, DD)                                                                      \
  if (a.p.bits == B && a.p.head_dim == DD) {                                                  \
    int per_sm = 0;                                                                           \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, append_kernel<B, DD, PREQ>,    \
                                                      threads, 0) != cudaSuccess || per_sm < 1) \
      per_sm = 2;                                                                             \
    const long long grid = std::min<long long>(want, static_cast<long long>(sms) * per_sm);   \
    append_kernel<B, DD, PREQ><<<static_cast<unsigned>(grid), threads, 0, stream>>>(a);       \
    return static_cast<int>(cudaGetLastError());                                              \
  }
  FQ_LAUNCH(2, 64) FQ_LAUNCH(2, 128) FQ_LAUNCH(2, 256)
  FQ_LAUNCH(4, 64) FQ_LAUNCH(4, 128) FQ_LAUNCH(4, 256)
#undef FQ_LAUNCH
  return FQ_ERR_UNSUPPORTED;
}

template <int BITS, int D>
static int launch_k_channel(const WriterArgs& a, int groups, cudaStream_t stream) {
  const int smem = PAGE * D * 3;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(append_k_channel_kernel<BITS, D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  append_k_channel_kernel<BITS, D>
      <<<static_cast<unsigned>(groups) * a.p.num_kv_heads, 256, smem, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

static int check_pools(const fq_pools* p) {
  if (!p || !p->k_codes || !p->v_codes || !p->scales) return FQ_ERR_BAD_ARG;
  if (p->k_channel_group != 0 && (p->k_channel_group != PAGE || p->k_groups != 1))
    return FQ_ERR_UNSUPPORTED;
  if (p->bits != 2 && p->bits != 4) return FQ_ERR_UNSUPPORTED;
  if (p->head_dim != 64 && p->head_dim != 128 && p->head_dim != 256) return FQ_ERR_UNSUPPORTED;
  if (p->k_groups != 1 && p->k_groups != 2 && p->k_groups != 4) return FQ_ERR_UNSUPPORTED;
  if (p->head_dim / p->k_groups < 64) return FQ_ERR_UNSUPPORTED;
  if (p->k_groups > 1 && !p->scale_bf16) return FQ_ERR_UNSUPPORTED;
  if (p->num_kv_heads <= 0 || p->num_pages <= 0) return FQ_ERR_BAD_ARG;
  if ((p->v_page_max == nullptr) != (p->v_max_hist == nullptr)) return FQ_ERR_BAD_ARG;
  return 0;
}

}  // namespace fq

extern "C" int fq_append_page_groups(const fq_pools* pools, const void* k, const void* v,
                                     int64_t k_token_stride, int64_t v_token_stride,
                                     const int32_t* page_ids, const int32_t* valid,
                                     int32_t num_page_groups, int32_t* status, void* stream) {
  if (int e = fq::check_pools(pools)) return e;
  if (pools->k_channel_group != FQ_PAGE_SIZE) return FQ_ERR_UNSUPPORTED;
  if (num_page_groups < 0 || (num_page_groups > 0 && (!k || !v || !page_ids)))
    return FQ_ERR_BAD_ARG;
  if (num_page_groups == 0) return 0;
  if (num_page_groups > (0x7FFFFFFF >> 6)) return FQ_ERR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (k_token_stride * 2) % 16 || (v_token_stride * 2) % 16)
    return FQ_ERR_BAD_ARG;
  fq::WriterArgs a{};
  a.p = *pools;
  a.k = k; a.v = v;
  a.k_stride = k_token_stride; a.v_stride = v_token_stride;
  a.page_ids = page_ids;
  a.valid = valid;
  a.num_tokens = num_page_groups * FQ_PAGE_SIZE;
  a.k_clip = a.v_clip = -1;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // V rows, V records, page maxima: the token-wise row pass (it skips K for these pools)
  if (int e = fq::launch_append<false>(a, s)) return e;
#define FQ_LAUNCH(B, DD) \
  if (pools->bits == B && pools->head_dim == DD) return fq::launch_k_channel<B, DD>(a, num_page_groups, s);
  FQ_LAUNCH(2, 64) FQ_LAUNCH(2, 128) FQ_LAUNCH(2, 256)
  FQ_LAUNCH(4, 64) FQ_LAUNCH(4, 128) FQ_LAUNCH(4, 256)
#undef FQ_LAUNCH
  return FQ_ERR_UNSUPPORTED;
}

extern "C" int fq_append_quantized_page_groups(const fq_pools* pools, const uint8_t* k_codes,
                                               const float* k_scale, const float* k_zero,
                                               const uint8_t* v_codes, const float* v_scale,
                                               const float* v_zero, const int32_t* page_ids,
                                               const int32_t* valid, int32_t num_page_groups,
                                               int32_t* status, void* stream) {
  if (int e = fq::check_pools(pools)) return e;
  if (pools->k_channel_group != FQ_PAGE_SIZE) return FQ_ERR_UNSUPPORTED;
  if (num_page_groups < 0 ||
      (num_page_groups > 0 && (!k_codes || !v_codes || !k_scale || !k_zero || !v_scale ||
                               !v_zero || !page_ids)))
    return FQ_ERR_BAD_ARG;
  if (num_page_groups == 0) return 0;
  if (num_page_groups > (0x7FFFFFFF >> 6)) return FQ_ERR_TOO_LARGE;
  // the code rows are read four bytes at a time
  if ((reinterpret_cast<uintptr_t>(k_codes) | reinterpret_cast<uintptr_t>(v_codes)) & 3)
    return FQ_ERR_BAD_ARG;
  fq::WriterArgs a{};
  a.p = *pools;
  a.k = k_codes; a.v = v_codes;
  a.k_scale = k_scale; a.k_zero = k_zero; a.v_scale = v_scale; a.v_zero = v_zero;
  a.page_ids = page_ids;
  a.valid = valid;
  a.num_tokens = num_page_groups * FQ_PAGE_SIZE;
  a.k_clip = a.v_clip = -1;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // V rows, V records, page maxima: the layout-only row pass (it skips K for these pools)
  if (int e = fq::launch_append<true>(a, s)) return e;
#define FQ_LAUNCH(B, DD)                                                                   \
  if (pools->bits == B && pools->head_dim == DD) {                                         \
    fq::pack_k_channel_kernel<B, DD>                                                       \
        <<<static_cast<unsigned>(num_page_groups) * pools->num_kv_heads, 256, 0, s>>>(a);  \
    return static_cast<int>(cudaGetLastError());                                           \
  }
  FQ_LAUNCH(2, 64) FQ_LAUNCH(2, 128) FQ_LAUNCH(2, 256)
  FQ_LAUNCH(4, 64) FQ_LAUNCH(4, 128) FQ_LAUNCH(4, 256)
#undef FQ_LAUNCH
  return FQ_ERR_UNSUPPORTED;
}

extern "C" int fq_append(const fq_pools* pools, const void* k, const void* v,
                         int64_t k_token_stride, int64_t v_token_stride,
                         const int64_t* slot_mapping, int32_t num_tokens, int32_t k_clip,
                         int32_t v_clip, int32_t* status, void* stream) {
  if (int e = fq::check_pools(pools)) return e;
  if (pools->k_channel_group != 0) return FQ_ERR_UNSUPPORTED;   // fq_append_page_groups
  if ((reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (k_token_stride * 2) % 16 || (v_token_stride * 2) % 16)
    return FQ_ERR_BAD_ARG;
  if (num_tokens < 0 || (num_tokens > 0 && (!k || !v || !slot_mapping))) return FQ_ERR_BAD_ARG;
  if (k_clip >= pools->head_dim || v_clip >= pools->head_dim) return FQ_ERR_BAD_ARG;
  fq::WriterArgs a{};
  a.p = *pools;
  a.k = k; a.v = v;
  a.k_stride = k_token_stride; a.v_stride = v_token_stride;
  a.slots = reinterpret_cast<const long long*>(slot_mapping);
  a.num_tokens = num_tokens;
  a.k_clip = k_clip < 0 ? -1 : k_clip;
  a.v_clip = v_clip < 0 ? -1 : v_clip;
  a.status = status;
  return fq::launch_append<false>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int fq_append_quantized(const fq_pools* pools, const uint8_t* k_codes,
                                   const float* k_scale, const float* k_zero,
                                   const uint8_t* v_codes, const float* v_scale,
                                   const float* v_zero, const int64_t* slot_mapping,
                                   int32_t num_tokens, int32_t* status, void* stream) {
  if (int e = fq::check_pools(pools)) return e;
  if (pools->k_channel_group != 0) return FQ_ERR_UNSUPPORTED;
  if (num_tokens < 0 || (num_tokens > 0 && (!k_codes || !v_codes || !k_scale || !k_zero ||
                                            !v_scale || !v_zero || !slot_mapping)))
    return FQ_ERR_BAD_ARG;
  // the code rows are read four bytes at a time
  if ((reinterpret_cast<uintptr_t>(k_codes) | reinterpret_cast<uintptr_t>(v_codes)) & 3)
    return FQ_ERR_BAD_ARG;
  fq::WriterArgs a{};
  a.p = *pools;
  a.k = k_codes; a.v = v_codes;
  a.k_scale = k_scale; a.k_zero = k_zero; a.v_scale = v_scale; a.v_zero = v_zero;
  a.slots = reinterpret_cast<const long long*>(slot_mapping);
  a.num_tokens = num_tokens;
  a.k_clip = a.v_clip = -1;
  a.status = status;
  return fq::launch_append<true>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int fq_recount_vmax(const fq_pools* pools, void* stream) {
  if (int e = fq::check_pools(pools)) return e;
  if (!pools->v_page_max) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemsetAsync(pools->v_max_hist, 0, FQ_VMAX_BINS * sizeof(uint32_t), s);
  if (err != cudaSuccess) return static_cast<int>(err);
  const long long n = static_cast<long long>(pools->num_pages) * pools->num_kv_heads;
  const int blocks = static_cast<int>(n / 1024 + 1 < 592 ? n / 1024 + 1 : 592);
  fq::recount_kernel<<<blocks, 256, 0, s>>>(pools->v_page_max, n, pools->v_max_hist);
  return static_cast<int>(cudaGetLastError());
}
