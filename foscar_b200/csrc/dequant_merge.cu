// Read-back (packed codes -> bf16 rows) and the log-sum-exp merges.
//
// Read-back follows src/foscar/_dequant_core.py:19-25 (out = bf16_rne(fma.rn(s, q, z)), rows
// t < seq_lens[b] only) with the reference's device traps replaced by status bits. The split
// merge follows src/foscar/_sm100/gqa_decode.py:666-761 (max in the log2 domain, fixed slot
// order, rows with no finite maximum give zeros). All three kernels are plain HBM streams.
#include <algorithm>

#include "common.cuh"

namespace fq {

struct DequantArgs {
  fq_pools p;
  __nv_bfloat16* k_out;
  __nv_bfloat16* v_out;
  long long k_stride, v_stride, num_rows;
  const int* page_indptr;
  const int* page_indices;
  const int* seq_lens;
  const void* out_indptr;
  int out_indptr_64;
  int batch;
  int num_entries;
  int* status;
};

// The BITS-wide field at bit POS of w (POS + BITS <= 23) as an exact float, without the
// integer-to-float conversion unit: the field is placed in the mantissa of 2^(23-POS), whose
// unit in the last place is 2^-POS, and 2^(23-POS) is subtracted again.
template <int BITS, int POS>
__device__ __forceinline__ float field_as_float(uint32_t w) {
  constexpr uint32_t MASK = ((1u << BITS) - 1) << POS;
  constexpr uint32_t ONE = static_cast<uint32_t>(150 - POS) << 23;
  return __uint_as_float((w & MASK) | ONE) - __uint_as_float(ONE);
}

// The eight codes of eight adjacent channels (first channel a multiple of 8). INT4: one word,
// channel j at bit 8j (j < 4) or 8(j-4)+4. INT2: half a word, the caller having shifted it so
// that channel j sits at bit 4j.
template <int BITS>
__device__ __forceinline__ void eight_codes(uint32_t w, float (&q)[8]) {
  const uint32_t hi = w >> 16;
  if constexpr (BITS == 2) {
    q[0] = field_as_float<2, 0>(w);   q[1] = field_as_float<2, 4>(w);
    q[2] = field_as_float<2, 8>(w);   q[3] = field_as_float<2, 12>(w);
    q[4] = field_as_float<2, 0>(hi);  q[5] = field_as_float<2, 4>(hi);
    q[6] = field_as_float<2, 8>(hi);  q[7] = field_as_float<2, 12>(hi);
  } else {
    q[0] = field_as_float<4, 0>(w);   q[1] = field_as_float<4, 8>(w);
    q[2] = field_as_float<4, 0>(hi);  q[3] = field_as_float<4, 8>(hi);
    q[4] = field_as_float<4, 4>(w);   q[5] = field_as_float<4, 12>(w);
    q[6] = field_as_float<4, 4>(hi);  q[7] = field_as_float<4, 12>(hi);
  }
}

__device__ __forceinline__ uint32_t bf16_pair(float lo, float hi) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}

__device__ __forceinline__ void plain_store(uint4* p, uint4 v) { *p = v; }
#ifndef FQ_DQ_STORE
#define FQ_DQ_STORE __stcs
#endif
#ifndef FQ_DQ_CTAS
#define FQ_DQ_CTAS 8
#endif
// What one (page entry, KV head) item reads and writes; rows == 0: nothing to do.
struct PageJob {
  int rows;
  int page;
  long long out0;   // output row of the page's first token
};

// Resolve item `entry` against the batch: the owning request (last b with page_indptr[b] <=
// entry), the tokens it has on this page, the physical page and the first output row.
__device__ __forceinline__ PageJob page_job(const DequantArgs& a, long long entry, bool live) {
  PageJob j{0, 0, 0};
  if (!live) return j;
  int lo = 0, hi = a.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(a.page_indptr + mid) <= entry) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int first = __ldg(a.page_indptr + b), last = __ldg(a.page_indptr + b + 1);
  if (entry < first || entry >= last) return j;  // an entry no request owns
  const int len = __ldg(a.seq_lens + b);
  if (len < 0 || (static_cast<long long>(len) + PAGE - 1) / PAGE > last - first) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, FQ_STATUS_BAD_LENGTH);
    return j;
  }
  const int k = static_cast<int>(entry) - first;
  const int remaining = len - k * PAGE;
  if (remaining <= 0) return j;
  const int page = __ldg(a.page_indices + entry);
  if (page < 0 || page >= a.p.num_pages) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, FQ_STATUS_BAD_PAGE);
    return j;
  }
  j.rows = remaining < PAGE ? remaining : PAGE;
  j.page = page;
  j.out0 = (a.out_indptr_64 ? static_cast<const long long*>(a.out_indptr)[b]
                            : static_cast<const int*>(a.out_indptr)[b]) +
           static_cast<long long>(k) * PAGE;
  return j;
}

// Persistent CTAs of 4 warps over the (page entry, KV head) items, item i = entry * HKV + head.
// An item's K codes, V codes and scale block are copied into shared memory with 16-byte
// asynchronous copies one item ahead of the arithmetic (two buffers), and the item after that
// is resolved while the copies fly, so no warp waits on a dependent global load per row. In the
// arithmetic a lane owns eight adjacent channels (one 16-byte store) of a row, D/8 lanes cover
// a row and a warp pass covers 256/D rows.
template <int BITS, int D>
__global__ void __launch_bounds__(128, FQ_DQ_CTAS) dequant_kernel(DequantArgs a, long long items) {
  constexpr int RB = D * BITS / 8;
  constexpr int LPR = D / 8;                 // lanes per row
  constexpr int RPW = 32 / LPR;              // rows per warp pass
  constexpr int PASSES = PAGE / (4 * RPW);   // passes per warp over the page
  constexpr int CODES = PAGE * RB;           // bytes of one page of K (or V) codes of one head
  constexpr int SB_MAX = (2 * PAGE + 2 * D) * 4 > 4 * PAGE * 4 ? (2 * PAGE + 2 * D) * 4
                                                               : 4 * PAGE * 4;
  constexpr int BUF = 2 * CODES + SB_MAX;
  __shared__ __align__(16) uint8_t stage[2 * BUF];
  const int hkv = a.p.num_kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kg = a.p.k_groups;
  const bool bf = a.p.scale_bf16 != 0;
  const bool kch = a.p.k_channel_group != 0;   // K records per channel of the page
  const int block_elems =
      kch ? 2 * PAGE + 2 * D : (kg == 1 ? 4 * PAGE : 2 * kg * PAGE + 2 * PAGE);
  const int sb_bytes = block_elems * (bf ? 2 : 4);
  const int sub = lane / LPR, c0 = (lane % LPR) * 8;
  const int grp = c0 / (D / kg);
  // this lane's word of a code row, and how far to shift it (INT2: the odd half of a word)
  const int word = BITS == 4 ? c0 / 8 : c0 / 16;
  const int align = BITS == 4 ? 0 : 2 * ((c0 / 8) & 1);
  const uint32_t stage0 = smem_u32(stage);

  auto fetch = [&](const PageJob& j, long long item, int buf) {
    if (j.rows > 0) {
      const long long blk = static_cast<long long>(j.page) * hkv + item % hkv;
      const uint32_t dst = stage0 + buf * BUF;
      const uint8_t* ksrc = a.p.k_codes + blk * CODES;
      const uint8_t* vsrc = a.p.v_codes + blk * CODES;
      const uint8_t* ssrc = static_cast<const uint8_t*>(a.p.scales) + blk * sb_bytes;
      const int code_chunks = (j.rows * RB + 15) >> 4;   // the rows the request has on the page
      for (int c = threadIdx.x; c < code_chunks; c += 128) {
        cp_async16(dst + 16 * c, ksrc + 16 * c);
        cp_async16(dst + CODES + 16 * c, vsrc + 16 * c);
      }
      for (int c = threadIdx.x; c < (sb_bytes >> 4); c += 128)
        cp_async16(dst + 2 * CODES + 16 * c, ssrc + 16 * c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const long long step = gridDim.x;
  long long item = blockIdx.x;
  PageJob cur = page_job(a, item / hkv, item < items);
  fetch(cur, item, 0);
  PageJob nxt = page_job(a, (item + step) / hkv, item + step < items);
  for (int n = 0; item < items; item += step, ++n) {
    const int buf = n & 1;
    fetch(nxt, item + step, buf ^ 1);
    const PageJob nxt2 = page_job(a, (item + 2 * step) / hkv, item + 2 * step < items);
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    if (cur.rows > 0) {
      const uint8_t* kbuf = stage + buf * BUF;
      const uint8_t* vbuf = kbuf + CODES;
      const uint8_t* sblock = kbuf + 2 * CODES;
      const int head = static_cast<int>(item % hkv);
      __nv_bfloat16* kbase = a.k_out + static_cast<long long>(head) * D + c0;
      __nv_bfloat16* vbase = a.v_out + static_cast<long long>(head) * D + c0;
      // channel-wise K: this lane's channels' (s_d, z_d), the same for every row of the page
      float sch[8], zch[8];
      if (kch) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (!bf) {
            const float* rec = reinterpret_cast<const float*>(sblock) + 2 * PAGE;
            sch[i] = rec[c0 + i];
            zch[i] = rec[D + c0 + i];
          } else {
            const __nv_bfloat16* rec = reinterpret_cast<const __nv_bfloat16*>(sblock) + 2 * PAGE;
            sch[i] = __bfloat162float(rec[c0 + i]);
            zch[i] = __bfloat162float(rec[D + c0 + i]);
          }
        }
      }
#pragma unroll 2
      for (int p = 0; p < PASSES; ++p) {
        const int t = (p * 4 + warp) * RPW + sub;
        if (t >= cur.rows) continue;
        const long long orow = cur.out0 + t;
        if (orow < 0 || orow >= a.num_rows) {
          if (a.status) atomicOr(a.status, FQ_STATUS_BAD_ROW);
          continue;
        }
        const uint32_t kw = reinterpret_cast<const uint32_t*>(kbuf + t * RB)[word] >> align;
        const uint32_t vw = reinterpret_cast<const uint32_t*>(vbuf + t * RB)[word] >> align;
        float sk = 0.f, zk = 0.f, sv, zv;
        if (kch) {
          if (!bf) {
            const float2 r = reinterpret_cast<const float2*>(sblock)[t];
            sv = r.x; zv = r.y;
          } else {
            const uint32_t vr = reinterpret_cast<const uint32_t*>(sblock)[t];
            sv = __uint_as_float(vr << 16); zv = __uint_as_float(vr & 0xFFFF0000u);
          }
        } else if (!bf) {
          const float4 r = reinterpret_cast<const float4*>(sblock)[t];
          sk = r.x; zk = r.y; sv = r.z; zv = r.w;
        } else {
          uint32_t kr, vr;
          if (kg == 1) {
            const uint2 r = reinterpret_cast<const uint2*>(sblock)[t];
            kr = r.x; vr = r.y;
          } else {
            kr = reinterpret_cast<const uint32_t*>(sblock)[kg * t + grp];
            vr = reinterpret_cast<const uint32_t*>(sblock + 2 * kg * PAGE * 2)[t];
          }
          sk = __uint_as_float(kr << 16); zk = __uint_as_float(kr & 0xFFFF0000u);
          sv = __uint_as_float(vr << 16); zv = __uint_as_float(vr & 0xFFFF0000u);
        }
        float qk[8], qv[8];
        eight_codes<BITS>(kw, qk);
        eight_codes<BITS>(vw, qv);
        float ko[8], vo[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ko[i] = kch ? __fmaf_rn(sch[i], qk[i], zch[i]) : __fmaf_rn(sk, qk[i], zk);
          vo[i] = __fmaf_rn(sv, qv[i], zv);
        }
        FQ_DQ_STORE(reinterpret_cast<uint4*>(kbase + orow * a.k_stride),
               make_uint4(bf16_pair(ko[0], ko[1]), bf16_pair(ko[2], ko[3]),
                          bf16_pair(ko[4], ko[5]), bf16_pair(ko[6], ko[7])));
        FQ_DQ_STORE(reinterpret_cast<uint4*>(vbase + orow * a.v_stride),
               make_uint4(bf16_pair(vo[0], vo[1]), bf16_pair(vo[2], vo[3]),
                          bf16_pair(vo[4], vo[5]), bf16_pair(vo[6], vo[7])));
      }
    }
    __syncthreads();   // the buffer is refilled by the next iteration's copies
    cur = nxt;
    nxt = nxt2;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// A negative length (or one longer than the request's pages) is also reported for requests
// that own no entry, which no page CTA visits.
__global__ void dequant_check_kernel(DequantArgs a) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= a.batch) return;
  const int len = a.seq_lens[b];
  const int pages = a.page_indptr[b + 1] - a.page_indptr[b];
  if (len < 0 || pages < 0 || (static_cast<long long>(len) + PAGE - 1) / PAGE > pages)
    if (a.status) atomicOr(a.status, FQ_STATUS_BAD_LENGTH);
}

__device__ inline void store_out(void* out, int dtype, long long idx, float v) {
  if (dtype == 0) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else if (dtype == 1) static_cast<__half*>(out)[idx] = __float2half_rn(v);
  else static_cast<float*>(out)[idx] = v;
}

// Split-KV merge: grid (B*HQ), block = head_dim threads (one channel each). Partials are
// [max_splits, B, HQ, D] / [max_splits, B, HQ]; slots [0, k) of the request are combined in
// slot order, so the result is run-to-run identical.
__global__ void merge_kernel(const float* __restrict__ o_partial,
                             const float* __restrict__ l_partial,
                             const float* __restrict__ m_partial,
                             const int* __restrict__ split_counts, int kv_splits, int batch,
                             int hq, int hkv, int d, float o_scale, void* out, int out_dtype,
                             float* lse) {
  const int row = blockIdx.x;  // b*HQ + h
  const int b = row / hq, h = row % hq;
  int k = kv_splits;
  if (split_counts) {
    // counts are per unit (request, KV head, head tile of eight query heads); a unit with one
    // piece wrote its final output itself
    const int ratio = hq / hkv, tiles = (ratio + 7) / 8;
    k = split_counts[(b * hkv + h / ratio) * tiles + (h % ratio) / 8];
    if (k <= 1) return;
  }
  const long long rows = static_cast<long long>(batch) * hq;
  float M = -INFINITY;
  for (int s = 0; s < k; ++s) M = fmaxf(M, __ldg(m_partial + s * rows + row));
  float den = 0.f, acc = 0.f;
  const int c = threadIdx.x;
  if (M > -INFINITY) {
    for (int s = 0; s < k; ++s) {
      const float w = exp2f(__ldg(m_partial + s * rows + row) - M);
      den += w * __ldg(l_partial + s * rows + row);
      if (c < d) acc += w * __ldg(o_partial + (s * rows + row) * d + c);
    }
  }
  const bool live = den > 0.f;
  if (c < d) store_out(out, out_dtype, static_cast<long long>(row) * d + c,
                       live ? acc / den * o_scale : 0.f);
  if (c == 0 && lse) lse[row] = live ? (M + log2f(den)) * 0.6931471805599453f : -INFINITY;
}

// Merge of attention states held as (normalised o, natural-log lse) from R sequence shards.
__global__ void merge_states_kernel(const float* __restrict__ o, const float* __restrict__ lse_in,
                                    int shards, long long rows, int d, long long o_stride,
                                    long long lse_stride, void* out, int out_dtype, float* lse) {
  const int row = blockIdx.x;
  const int c = threadIdx.x;
  float L = -INFINITY;
  for (int r = 0; r < shards; ++r) L = fmaxf(L, __ldg(lse_in + (r * rows + row) * lse_stride));
  float den = 0.f, acc = 0.f;
  if (L > -INFINITY) {
    for (int r = 0; r < shards; ++r) {
      const float w = expf(__ldg(lse_in + (r * rows + row) * lse_stride) - L);
      den += w;
      if (c < d) acc += w * __ldg(o + (r * rows + row) * o_stride + c);
    }
  }
  const bool live = den > 0.f;
  if (c < d) store_out(out, out_dtype, static_cast<long long>(row) * d + c,
                       live ? acc / den : 0.f);
  if (c == 0 && lse) lse[row] = live ? L + logf(den) : -INFINITY;
}

}  // namespace fq

extern "C" int fq_dequantize(const fq_pools* pools, void* k_out, void* v_out,
                             int64_t k_row_stride, int64_t v_row_stride, int64_t num_out_rows,
                             const int32_t* page_indptr, const int32_t* page_indices,
                             int32_t num_entries, const int32_t* seq_lens,
                             const void* out_indptr, int32_t out_indptr_64, int32_t batch,
                             int32_t* status, void* stream) {
  if (!pools || !pools->k_codes || !pools->v_codes || !pools->scales) return FQ_ERR_BAD_ARG;
  if (batch < 0 || num_entries < 0) return FQ_ERR_BAD_ARG;
  if (batch == 0) return 0;
  if (!k_out || !v_out || !page_indptr || !seq_lens || !out_indptr) return FQ_ERR_BAD_ARG;
  if (num_entries > 0 && !page_indices) return FQ_ERR_BAD_ARG;
  // rows leave as 16-byte stores of eight channels, pages arrive as 16-byte copies
  if ((reinterpret_cast<uintptr_t>(k_out) | reinterpret_cast<uintptr_t>(v_out) |
       reinterpret_cast<uintptr_t>(pools->k_codes) | reinterpret_cast<uintptr_t>(pools->v_codes) |
       reinterpret_cast<uintptr_t>(pools->scales)) & 15 ||
      k_row_stride % 8 || v_row_stride % 8)
    return FQ_ERR_BAD_ARG;
  const long long blocks = static_cast<long long>(num_entries) * pools->num_kv_heads;
  if (blocks > 0x7FFFFFFFLL) return FQ_ERR_TOO_LARGE;
  fq::DequantArgs a{};
  a.p = *pools;
  a.k_out = static_cast<__nv_bfloat16*>(k_out);
  a.v_out = static_cast<__nv_bfloat16*>(v_out);
  a.k_stride = k_row_stride; a.v_stride = v_row_stride; a.num_rows = num_out_rows;
  a.page_indptr = page_indptr; a.page_indices = page_indices; a.seq_lens = seq_lens;
  a.out_indptr = out_indptr; a.out_indptr_64 = out_indptr_64;
  a.batch = batch; a.num_entries = num_entries; a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  fq::dequant_check_kernel<<<(batch + 255) / 256, 256, 0, s>>>(a);
  if (blocks == 0) return static_cast<int>(cudaGetLastError());
  // persistent CTAs: as many as stay resident, every one looping over its share of the items
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    sms = 148;
#define FQ_LAUNCH(B, DD)                                                                      \
  if (pools->bits == B && pools->head_dim == DD) {                                            \
    int per_sm = 0;                                                                           \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fq::dequant_kernel<B, DD>,    \
                                                      128, 0) != cudaSuccess || per_sm < 1)   \
      per_sm = 4;                                                                             \
    const long long grid = std::min<long long>(blocks, static_cast<long long>(sms) * per_sm); \
    fq::dequant_kernel<B, DD><<<static_cast<unsigned>(grid), 128, 0, s>>>(a, blocks);         \
    return static_cast<int>(cudaGetLastError());                                              \
  }
  FQ_LAUNCH(2, 64) FQ_LAUNCH(2, 128) FQ_LAUNCH(2, 256)
  FQ_LAUNCH(4, 64) FQ_LAUNCH(4, 128) FQ_LAUNCH(4, 256)
#undef FQ_LAUNCH
  return FQ_ERR_UNSUPPORTED;
}

extern "C" int fq_merge(const float* o_partial, const float* l_partial, const float* m_partial,
                        const int32_t* split_counts, int32_t kv_splits, int32_t max_splits,
                        int32_t batch, int32_t num_qo_heads, int32_t num_kv_heads,
                        int32_t head_dim, float o_scale,
                        void* out, int32_t out_dtype, float* lse, void* stream) {
  if (!o_partial || !l_partial || !m_partial || !out) return FQ_ERR_BAD_ARG;
  if (batch <= 0 || num_qo_heads <= 0 || head_dim <= 0 || head_dim > 1024) return FQ_ERR_BAD_ARG;
  if (num_kv_heads <= 0 || num_qo_heads % num_kv_heads) return FQ_ERR_BAD_ARG;
  if (!split_counts && (kv_splits < 1 || kv_splits > max_splits)) return FQ_ERR_BAD_ARG;
  if (out_dtype < 0 || out_dtype > 2) return FQ_ERR_BAD_ARG;
  const int threads = (head_dim + 31) / 32 * 32;
  fq::merge_kernel<<<batch * num_qo_heads, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      o_partial, l_partial, m_partial, split_counts, kv_splits, batch, num_qo_heads,
      num_kv_heads, head_dim, o_scale, out, out_dtype, lse);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fq_merge_states(const float* o_shards, const float* lse_shards,
                               int32_t num_shards, int32_t batch, int32_t num_qo_heads,
                               int32_t head_dim, void* out, int32_t out_dtype, float* lse,
                               int64_t o_row_stride, int64_t lse_stride, void* stream) {
  if (!o_shards || !lse_shards || !out || num_shards < 1) return FQ_ERR_BAD_ARG;
  if (batch <= 0 || num_qo_heads <= 0 || head_dim <= 0 || head_dim > 1024) return FQ_ERR_BAD_ARG;
  if (out_dtype < 0 || out_dtype > 2) return FQ_ERR_BAD_ARG;
  const int threads = (head_dim + 31) / 32 * 32;
  fq::merge_states_kernel<<<batch * num_qo_heads, threads, 0,
                            static_cast<cudaStream_t>(stream)>>>(
      o_shards, lse_shards, num_shards, static_cast<long long>(batch) * num_qo_heads, head_dim,
      o_row_stride > 0 ? o_row_stride : head_dim, lse_stride > 0 ? lse_stride : 1, out, out_dtype,
      lse);
  return static_cast<int>(cudaGetLastError());
}
