// What it costs the issuing warp to move a page-sized chunk from global to shared memory on
// sm_100a: one `cp.async.bulk` (the untiled TMA copy, completion counted in bytes on an mbarrier)
// against 16-byte `cp.async` from all 32 lanes (completion by `cp.async.mbarrier.arrive.noinc`),
// the two candidates for the decode kernel's ring. One CTA per SM fills 128 KB of shared memory
// once (no stage is reused, so the issue loop never waits), then waits, bounded, for the bytes.
// Prints, per chunk size and method, the cycles the issuing warp spent per chunk and the rate of
// the whole grid. Every address and size is a multiple of 16 bytes; plain copies into this
// CTA's own shared memory, one GPU.
#include <cstdio>
#include <cstdlib>

#include "../../foscar_b200/csrc/common.cuh"

using namespace fq;

__device__ inline void expect_bytes(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ inline void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

constexpr int RING_BYTES = 128 * 1024;
constexpr int MAX_CHUNKS = 128;

// method 0: one lane issues each chunk as one bulk copy; 1: six lanes issue a chunk each;
// 2: all lanes issue 16-byte cp.async
__global__ void __launch_bounds__(128, 1)
probe(const uint8_t* src, long long src_bytes, int bytes, int method, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  const uint32_t ring = (smem_u32(raw) + 1023u) & ~1023u;
  __shared__ __align__(8) unsigned long long bars[MAX_CHUNKS];
  __shared__ __align__(8) int abort_flag[4];
  const int chunks = RING_BYTES / bytes;
  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    set_wait_budget(abort_flag, 200000000LL);   // a tenth of a second
    for (int i = 0; i < chunks; ++i) mbar_init(smem_u32(&bars[i]), method == 2 ? 32 : 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const long long span = src_bytes - RING_BYTES;
  const uint8_t* from = src + (static_cast<long long>(blockIdx.x) * 7919 * 4096) % span;
  const long long t0 = clock64();
  if (method == 2) {
    for (int c = 0; c < chunks; ++c) {
      for (int i = lane; i < bytes / 16; i += 32)
        cp_async16(ring + c * bytes + 16 * i, from + static_cast<long long>(c) * bytes + 16 * i);
      cp_async_arrive(smem_u32(&bars[c]));
    }
  } else {
    const int lanes = method == 0 ? 1 : 6;
    for (int c0 = 0; c0 < chunks; c0 += lanes) {
      const int c = c0 + lane;
      if (lane < lanes && c < chunks) {
        expect_bytes(smem_u32(&bars[c]), bytes);
        bulk_copy(ring + c * bytes, from + static_cast<long long>(c) * bytes, bytes,
                  smem_u32(&bars[c]));
      }
      __syncwarp();
    }
  }
  const long long t1 = clock64();
  for (int c = 0; c < chunks; ++c) mbar_wait(smem_u32(&bars[c]), 0, abort_flag, status);
  const long long t2 = clock64();
  if (lane == 0 && blockIdx.x == 0) {
    out[0] = t1 - t0;
    out[1] = t2 - t0;
  }
}

int main() {
  long long* d_out;
  int* d_status;
  uint8_t* src;
  const long long src_bytes = 1ll << 30;
  if (cudaMalloc(&d_out, 16) || cudaMalloc(&d_status, 4) || cudaMalloc(&src, src_bytes)) return 2;
  cudaMemset(src, 1, src_bytes);
  cudaMemset(d_status, 0, 4);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_BYTES + 1024);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  const char* names[3] = {"cp.async.bulk, 1 lane", "cp.async.bulk, 6 lanes", "cp.async 16 B x 32 lanes"};
  for (int bytes : {1024, 2048, 4096, 8192})
    for (int method = 0; method < 3; ++method) {
      cudaEvent_t e0, e1;
      cudaEventCreate(&e0);
      cudaEventCreate(&e1);
      probe<<<sms, 128, RING_BYTES + 1024>>>(src, src_bytes, bytes, method, d_out, d_status);
      cudaEventRecord(e0);
      probe<<<sms, 128, RING_BYTES + 1024>>>(src, src_bytes, bytes, method, d_out, d_status);
      cudaEventRecord(e1);
      const cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) {
        printf("error %s\n", cudaGetErrorString(e));
        return 1;
      }
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      long long h[2];
      int st = 0;
      cudaMemcpy(h, d_out, 16, cudaMemcpyDeviceToHost);
      cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
      const int chunks = RING_BYTES / bytes;
      printf("chunk %5d B  %-26s issue %7.1f cycles/chunk  %6.1f cycles/KB  filled in %7.0f cycles"
             "  grid %6.0f GB/s  status %d\n",
             bytes, names[method], static_cast<double>(h[0]) / chunks,
             static_cast<double>(h[0]) / (RING_BYTES / 1024), static_cast<double>(h[1]),
             static_cast<double>(sms) * RING_BYTES / ms / 1e6, st);
      if (st != 0) return 3;
    }
  return 0;
}
