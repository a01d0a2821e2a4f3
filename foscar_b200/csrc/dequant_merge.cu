// Read-back (packed codes -> bf16 rows) and the log-sum-exp merges.
//
// Read-back follows src/foscar/_dequant_core.py:19-25 (out = bf16_rne(fma.rn(s, q, z)), rows
// t < seq_lens[b] only) with the reference's device traps replaced by status bits. The split
// merge follows src/foscar/_sm100/gqa_decode.py:666-761 (max in the log2 domain, fixed slot
// order, rows with no finite maximum give zeros). All three kernels are plain HBM streams.
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

// One CTA of 4 warps per (page entry, KV head); a warp writes whole rows, lane l the channels
// [l*CH, (l+1)*CH), so every store instruction covers one contiguous 2*D-byte row.
template <int BITS, int D>
__global__ void __launch_bounds__(128) dequant_kernel(DequantArgs a) {
  constexpr int CH = D / 32;
  constexpr int RB = D * BITS / 8;
  constexpr uint32_t MASK = (1u << BITS) - 1;
  const int hkv = a.p.num_kv_heads;
  const int entry = blockIdx.x / hkv, head = blockIdx.x % hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // request owning this entry: last b with page_indptr[b] <= entry
  int lo = 0, hi = a.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(a.page_indptr + mid) <= entry) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int first = __ldg(a.page_indptr + b), last = __ldg(a.page_indptr + b + 1);
  if (entry < first || entry >= last) return;  // an entry no request owns
  const int len = __ldg(a.seq_lens + b);
  if (len < 0 || (static_cast<long long>(len) + PAGE - 1) / PAGE > last - first) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, FQ_STATUS_BAD_LENGTH);
    return;
  }
  const int j = entry - first;
  const int remaining = len - j * PAGE;
  if (remaining <= 0) return;
  const int rows = remaining < PAGE ? remaining : PAGE;
  const int page = __ldg(a.page_indices + entry);
  if (page < 0 || page >= a.p.num_pages) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, FQ_STATUS_BAD_PAGE);
    return;
  }
  const long long out0 = (a.out_indptr_64 ? static_cast<const long long*>(a.out_indptr)[b]
                                          : static_cast<const int*>(a.out_indptr)[b]) +
                         static_cast<long long>(j) * PAGE;
  const long long blk = static_cast<long long>(page) * hkv + head;
  const int kg = a.p.k_groups;
  const int esz = a.p.scale_bf16 ? 2 : 4;
  const bool kch = a.p.k_channel_group != 0;   // K records per channel of the page
  const long long block_elems =
      kch ? 2 * PAGE + 2 * D : (kg == 1 ? 4 * PAGE : 2 * kg * PAGE + 2 * PAGE);
  const char* sblock = static_cast<const char*>(a.p.scales) + blk * block_elems * esz;
  const int c0 = lane * CH;
  const int grp = lane / (32 / kg);
  // channel-wise K: this lane's channels' (s_d, z_d), the same for every row of the page
  float sch[CH], zch[CH];
  if (kch) {
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      if (!a.p.scale_bf16) {
        const float* rec = reinterpret_cast<const float*>(sblock) + 2 * PAGE;
        sch[i] = __ldg(rec + c0 + i);
        zch[i] = __ldg(rec + D + c0 + i);
      } else {
        const __nv_bfloat16* rec = reinterpret_cast<const __nv_bfloat16*>(sblock) + 2 * PAGE;
        sch[i] = __bfloat162float(rec[c0 + i]);
        zch[i] = __bfloat162float(rec[D + c0 + i]);
      }
    }
  }

  for (int t = warp; t < rows; t += 4) {
    const long long orow = out0 + t;
    if (orow < 0 || orow >= a.num_rows) {
      if (lane == 0 && a.status) atomicOr(a.status, FQ_STATUS_BAD_ROW);
      continue;
    }
    float sk = 0.f, zk = 0.f, sv, zv;
    if (kch) {
      if (!a.p.scale_bf16) {
        const float2 r = __ldg(reinterpret_cast<const float2*>(sblock) + t);
        sv = r.x; zv = r.y;
      } else {
        const uint32_t vr = __ldg(reinterpret_cast<const uint32_t*>(sblock) + t);
        sv = __uint_as_float(vr << 16); zv = __uint_as_float(vr & 0xFFFF0000u);
      }
    } else if (!a.p.scale_bf16) {
      const float4 r = __ldg(reinterpret_cast<const float4*>(sblock) + t);
      sk = r.x; zk = r.y; sv = r.z; zv = r.w;
    } else {
      uint32_t kr, vr;
      if (kg == 1) {
        const uint2 r = __ldg(reinterpret_cast<const uint2*>(sblock) + t);
        kr = r.x; vr = r.y;
      } else {
        kr = __ldg(reinterpret_cast<const uint32_t*>(sblock) + kg * t + grp);
        vr = __ldg(reinterpret_cast<const uint32_t*>(sblock + 2 * kg * PAGE * 2) + t);
      }
      sk = __uint_as_float(kr << 16); zk = __uint_as_float(kr & 0xFFFF0000u);
      sv = __uint_as_float(vr << 16); zv = __uint_as_float(vr & 0xFFFF0000u);
    }
    const uint32_t* krow =
        reinterpret_cast<const uint32_t*>(a.p.k_codes + (blk * PAGE + t) * RB);
    const uint32_t* vrow =
        reinterpret_cast<const uint32_t*>(a.p.v_codes + (blk * PAGE + t) * RB);
    __nv_bfloat16 ko[CH], vo[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int off = code_bit_offset<BITS>(c0 + i);
      const uint32_t qk = (__ldg(krow + (off >> 5)) >> (off & 31)) & MASK;
      const uint32_t qv = (__ldg(vrow + (off >> 5)) >> (off & 31)) & MASK;
      ko[i] = __float2bfloat16_rn(kch ? __fmaf_rn(sch[i], static_cast<float>(qk), zch[i])
                                      : __fmaf_rn(sk, static_cast<float>(qk), zk));
      vo[i] = __float2bfloat16_rn(__fmaf_rn(sv, static_cast<float>(qv), zv));
    }
    __nv_bfloat16* kd = a.k_out + orow * a.k_stride + static_cast<long long>(head) * D + c0;
    __nv_bfloat16* vd = a.v_out + orow * a.v_stride + static_cast<long long>(head) * D + c0;
    if constexpr (CH == 8) {
      *reinterpret_cast<uint4*>(kd) = *reinterpret_cast<uint4*>(ko);
      *reinterpret_cast<uint4*>(vd) = *reinterpret_cast<uint4*>(vo);
    } else if constexpr (CH == 4) {
      *reinterpret_cast<uint2*>(kd) = *reinterpret_cast<uint2*>(ko);
      *reinterpret_cast<uint2*>(vd) = *reinterpret_cast<uint2*>(vo);
    } else {
      *reinterpret_cast<uint32_t*>(kd) = *reinterpret_cast<uint32_t*>(ko);
      *reinterpret_cast<uint32_t*>(vd) = *reinterpret_cast<uint32_t*>(vo);
    }
  }
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
#define FQ_LAUNCH(B, DD)                                                          \
  if (pools->bits == B && pools->head_dim == DD) {                                \
    fq::dequant_kernel<B, DD><<<static_cast<unsigned>(blocks), 128, 0, s>>>(a);   \
    return static_cast<int>(cudaGetLastError());                                  \
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
