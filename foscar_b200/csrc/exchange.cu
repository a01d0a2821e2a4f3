// Cross-GPU step of a sequence-split decode: every rank holds the attention state (o, lse) of
// its token range; one launch per rank writes its rows into a staging slot in EVERY rank's
// memory, raises a flag there, waits (bounded) for the other ranks' flags in its own memory and
// merges the gathered rows locally:   out = sum_r exp(lse_r - L) o_r,  L = logsumexp_r lse_r.
//
// The reference is a single-GPU library and has no counterpart; the merge arithmetic is its
// attention-state merge (src/foscar/_sm100/gqa_decode.py:666-761) in the natural-log domain.
//
// Peers are reached with ordinary st.global / ld.volatile through peer-mapped pointers (buffers
// of torch's symmetric memory): no bulk or tensor copies, no multicast, no library kernel is
// handed a peer pointer. The staging area is double-buffered by the step's parity, so a rank
// that is already on step s + 1 never overwrites rows another rank still merges for step s
// (a rank reaches step s + 2 only after every rank has posted step s + 1, i.e. finished s).
//
// Layout of one rank's staging buffer (floats unless said): for parity p in {0, 1}:
//   rows  [world][rows_per_rank][d + 1]   (o row, then lse), slot r written by rank r
// then  flags int64 [2][world]  (the step a rank has posted for that parity), then words used by
// this rank's own launches only: arrival counters int32 [2], an exit counter int32 and the
// number of steps this rank has run int64. With step == 0 a launch takes its step from that
// count (every rank launches the same number of times), so that a captured launch can be
// replayed: nothing the host passes changes from step to step.
#include "common.cuh"

namespace fq {

constexpr int MAX_RANKS = 16;

struct ExchangeArgs {
  float* staging[MAX_RANKS];   // every rank's staging buffer as mapped in this process
  const float* o_local;        // [rows][d] f32, normalised
  const float* lse_local;      // [rows] f32, natural log
  void* out;
  float* lse_out;
  int* status;
  long long step;              // 1, 2, 3, ...: the same on every rank
  long long budget;            // cycle budget of the wait for the peers
  int rows, d, rank, world, out_dtype;
};

__host__ __device__ inline long long exchange_rows_floats(int world, int rows, int d) {
  return static_cast<long long>(world) * rows * (d + 1);
}
__host__ __device__ inline long long exchange_bytes(int world, int rows, int d) {
  const long long data = 2 * exchange_rows_floats(world, rows, d) * 4;
  return (data + 15) / 16 * 16 + 2 * world * 8 + 32;
}

__device__ inline void store_out_x(void* out, int out_dtype, long long idx, float val) {
  if (out_dtype == 0) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(val);
  else if (out_dtype == 1) static_cast<__half*>(out)[idx] = __float2half_rn(val);
  else static_cast<float*>(out)[idx] = val;
}

// All CTAs of the launch are resident at once (the host keeps the grid at or below the SM
// count): they wait on one another through a counter and on the peers through flags.
__global__ void __launch_bounds__(256) exchange_merge_kernel(ExchangeArgs a) {
  __shared__ long long s_step;
  {
    const long long par_f = exchange_rows_floats(a.world, a.rows, a.d);
    char* own = reinterpret_cast<char*>(a.staging[a.rank]) + (2 * par_f * 4 + 15) / 16 * 16 +
                2 * a.world * 8;
    volatile long long* steps_run = reinterpret_cast<volatile long long*>(own + 16);
    if (threadIdx.x == 0) s_step = a.step > 0 ? a.step : *steps_run + 1;
    __syncthreads();
    a.step = s_step;
  }
  const int par = static_cast<int>(a.step & 1);
  const long long slot_floats = static_cast<long long>(a.rows) * (a.d + 1);
  const long long par_floats = exchange_rows_floats(a.world, a.rows, a.d);
  const long long data_bytes = (2 * par_floats * 4 + 15) / 16 * 16;
  auto flags_of = [&](float* base) {
    return reinterpret_cast<volatile long long*>(reinterpret_cast<char*>(base) + data_bytes) +
           par * a.world;
  };
  float* mine = a.staging[a.rank];
  int* counter = reinterpret_cast<int*>(reinterpret_cast<char*>(mine) + data_bytes +
                                        2 * a.world * 8) + par;
  __shared__ int s_flag;

  // 1. this rank's rows into slot `rank` of every rank's staging area (its own included)
  const int row_words = a.d + 1;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    for (int c = threadIdx.x; c < row_words; c += blockDim.x) {
      const float v = c < a.d ? a.o_local[static_cast<long long>(row) * a.d + c]
                              : a.lse_local[row];
      const long long off = par * par_floats + a.rank * slot_floats +
                            static_cast<long long>(row) * row_words + c;
      for (int r = 0; r < a.world; ++r) a.staging[r][off] = v;
    }
  }
  // 2. when every CTA's rows are out, one thread posts the step on every rank
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(counter, 1);
    if (arrived == static_cast<int>(gridDim.x) - 1) {
      *counter = 0;   // this launch's last CTA: ready for the launch two steps on
      __threadfence_system();
      for (int r = 0; r < a.world; ++r) flags_of(a.staging[r])[a.rank] = a.step;
      __threadfence_system();
    }
    // 3. wait for every rank's post in this rank's own memory, bounded
    volatile long long* flags = flags_of(mine);
    const long long t0 = clock64();
    int ok = 1;
    for (int r = 0; r < a.world && ok; ++r) {
      while (flags[r] < a.step) {
        if (clock64() - t0 > a.budget) {
          ok = 0;
          if (a.status) atomicOr(a.status, FQ_STATUS_TIMEOUT);
          break;
        }
      }
    }
    __threadfence_system();
    s_flag = ok;
  }
  __syncthreads();
  // 4. merge the gathered rows (all in this rank's memory); a peer that never posted leaves the
  // output as it was
  if (s_flag) {
  const float* base = mine + par * par_floats;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    float L = -INFINITY;
    for (int r = 0; r < a.world; ++r)
      L = fmaxf(L, __ldcv(base + r * slot_floats + static_cast<long long>(row) * row_words + a.d));
    for (int c = threadIdx.x; c < a.d; c += blockDim.x) {
      float den = 0.f, acc = 0.f;
      if (L > -INFINITY) {
        for (int r = 0; r < a.world; ++r) {
          const float* src = base + r * slot_floats + static_cast<long long>(row) * row_words;
          const float w = expf(__ldcv(src + a.d) - L);
          den += w;
          acc += w * __ldcv(src + c);
        }
      }
      store_out_x(a.out, a.out_dtype, static_cast<long long>(row) * a.d + c,
                  den > 0.f ? acc / den : 0.f);
      if (c == 0 && a.lse_out != nullptr)
        a.lse_out[row] = den > 0.f ? L + logf(den) : -INFINITY;
    }
  }
  }
  // 5. the launch's last CTA to leave counts the step (every CTA has read the count by now)
  if (threadIdx.x == 0) {
    int* exits = counter - par + 2;
    if (atomicAdd(exits, 1) == static_cast<int>(gridDim.x) - 1) {
      *exits = 0;
      *reinterpret_cast<volatile long long*>(reinterpret_cast<char*>(counter - par) + 16) = a.step;
    }
  }
}

}  // namespace fq

extern "C" int64_t fq_exchange_bytes(int32_t world, int32_t batch, int32_t num_qo_heads,
                                     int32_t head_dim) {
  if (world < 1 || world > fq::MAX_RANKS || batch < 1 || num_qo_heads < 1 || head_dim < 1)
    return FQ_ERR_BAD_ARG;
  return fq::exchange_bytes(world, batch * num_qo_heads, head_dim);
}

extern "C" int fq_exchange_merge(void* const* staging, int32_t rank, int32_t world,
                                 const float* o_local, const float* lse_local, int32_t batch,
                                 int32_t num_qo_heads, int32_t head_dim, int64_t step, void* out,
                                 int32_t out_dtype, float* lse_out, int64_t wait_budget_cycles,
                                 int32_t* status, void* stream) {
  if (!staging || !o_local || !lse_local || !out) return FQ_ERR_BAD_ARG;
  if (world < 1 || world > fq::MAX_RANKS || rank < 0 || rank >= world) return FQ_ERR_BAD_ARG;
  if (batch < 1 || num_qo_heads < 1 || head_dim < 1 || step < 0) return FQ_ERR_BAD_ARG;
  if (out_dtype < 0 || out_dtype > 2) return FQ_ERR_BAD_ARG;
  fq::ExchangeArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!staging[r] || (reinterpret_cast<uintptr_t>(staging[r]) & 15)) return FQ_ERR_BAD_ARG;
    a.staging[r] = static_cast<float*>(staging[r]);
  }
  a.o_local = o_local; a.lse_local = lse_local;
  a.out = out; a.lse_out = lse_out; a.status = status;
  a.step = step;
  a.budget = wait_budget_cycles > 0 ? wait_budget_cycles : fq::WAIT_BUDGET_CYCLES;
  a.rows = batch * num_qo_heads; a.d = head_dim; a.rank = rank; a.world = world;
  a.out_dtype = out_dtype;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    sms = 148;
  // every CTA must be resident while it waits: a grid well inside one wave
  int grid = a.rows < sms / 2 ? a.rows : sms / 2;
  if (grid < 1) grid = 1;
  fq::exchange_merge_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}
