// Microbenchmark: how fast can tcgen05.mma be issued on one SM?
//
// One CTA per SM.  `issuers` threads (lane 0 of the warps listed in `issuer_warps`) each issue `iters` MMAs of
// 128 x N x 16 (bf16 operands in shared memory, all zeros, K-major rows of 64 bytes) into their own TMEM
// columns, commit to their own mbarrier and wait for it (a bounded wait).  Printed per configuration: cycles per
// MMA as the issuing thread sees them, cycles per MMA over all issuers, and multiply-accumulates per cycle and SM
// (the tensor pipe's dense bf16 rate is 4096 per cycle and SM).
//
// What it showed on a B200: a thread issues one MMA every 148 cycles in this loop whatever N is (75-110 in the
// kernels, whose loops are unrolled), issuers in different warps add up (two: twice the MMAs; four: 48 cycles per
// N = 64 MMA, and the pipe's full rate from N = 128 on), two issuers on the same warp scheduler (warps 1 and 5)
// lose 7 %, and one thread that alternates between accumulators gains nothing.
//
// Not part of the library.  Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue_rate mma_issue_rate.cu && ./mma_issue_rate
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../ptx_sm100.cuh"

using namespace nb::ptx;

#define CK(x)                                                                                 \
  do {                                                                                        \
    cudaError_t e_ = (x);                                                                     \
    if (e_ != cudaSuccess) {                                                                  \
      printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__);         \
      exit(2);                                                                                \
    }                                                                                         \
  } while (0)

struct RateParams {
  int issuers;          // 1..4
  int issuer_warps[4];  // which warps of the 12 issue
  int N;                // MMA width: 32 .. 256, issuers * accumulators * N <= 512 TMEM columns
  int accumulators;     // TMEM accumulators one issuer cycles through
  int iters;
  long long* cycles;  // [issuer][2]: issue loop, issue loop + completion (block 0 only)
  int* status;        // set to 1 when a wait ran out
};

constexpr int kThreads = 384;
constexpr int kSmemBytes = 64 * 1024;

__global__ void __launch_bounds__(kThreads, 1) k_mma_issue_rate(const RateParams p) {
  extern __shared__ uint8_t raw[];
  __shared__ __align__(8) uint64_t bar[4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  for (int i = threadIdx.x; i < kSmemBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(raw)[i] = 0u;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1);
    fence_mbar_init();
  }
  if (warp == 11) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  int me = -1;
  for (int i = 0; i < p.issuers; ++i)
    if (p.issuer_warps[i] == warp) me = i;
  if (me >= 0 && lane == 0) {
    const uint32_t idesc = instr_desc(1u, 1u, 128u, static_cast<uint32_t>(p.N));
    // A: 128 rows of 64 bytes at `base`, B: N rows of 64 bytes behind it (every issuer reads the same tiles)
    const uint64_t a = smem_desc_kmajor(base, 64);
    const uint64_t b = smem_desc_kmajor(base + 128u * 64u, 64);
    const uint32_t d = tmem_base + static_cast<uint32_t>(me * p.accumulators * p.N);
    const long long t0 = clock64();
    for (int i = 0; i < p.iters; ++i) {
      const uint64_t k_step = 2u * (i & 1);  // a 64-byte row holds two K steps of 32 bytes (2 units of 16 bytes)
      mma_f16(d + static_cast<uint32_t>((i % p.accumulators) * p.N), a + k_step, b + k_step, idesc,
              i >= p.accumulators ? 1u : 0u);
    }
    const long long t1 = clock64();
    tc_commit(smem_u32(&bar[me]));
    const bool ok = mbar_wait_bounded(smem_u32(&bar[me]), 0, &abort_flag, 2000000000ull);
    const long long t2 = clock64();
    if (!ok) atomicExch(p.status, 1);
    if (blockIdx.x == 0) {
      p.cycles[me * 2] = t1 - t0;
      p.cycles[me * 2 + 1] = t2 - t0;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 11) tmem_dealloc(tmem_base, 512);
}

static void run(int grid, int issuers, const int (&warps)[4], int N, int accumulators, long long* d_cycles, int* d_status) {
  if (issuers * accumulators * N > 512) return;
  RateParams p{};
  p.issuers = issuers;
  for (int i = 0; i < 4; ++i) p.issuer_warps[i] = warps[i];
  p.N = N;
  p.accumulators = accumulators;
  p.iters = 2000;
  p.cycles = d_cycles;
  p.status = d_status;
  CK(cudaMemset(d_cycles, 0, 64));
  k_mma_issue_rate<<<grid, kThreads, kSmemBytes + 1024>>>(p);
  CK(cudaDeviceSynchronize());
  long long h[8];
  int st;
  CK(cudaMemcpy(h, d_cycles, 64, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost));
  long long done = 0, issue = 0;
  for (int w = 0; w < issuers; ++w) {
    if (h[2 * w + 1] > done) done = h[2 * w + 1];
    if (h[2 * w] > issue) issue = h[2 * w];
  }
  printf("CTAs %3d  N %3d  issuers %d (warps %d %d %d %d)  accumulators %d:  %.1f clk/MMA per issuer, %.1f clk/MMA overall, %.0f MAC/clk/SM%s\n",
         grid, N, issuers, warps[0], issuers > 1 ? warps[1] : -1, issuers > 2 ? warps[2] : -1, issuers > 3 ? warps[3] : -1,
         accumulators, double(issue) / p.iters, double(done) / (double(p.iters) * issuers),
         128.0 * N * 16 * p.iters * issuers / double(done), st ? "  (a wait ran out)" : "");
}

int main() {
  long long* d_cycles;
  int* d_status;
  CK(cudaMalloc(&d_cycles, 64));
  CK(cudaMalloc(&d_status, 4));
  CK(cudaMemset(d_status, 0, 4));
  CK(cudaFuncSetAttribute(k_mma_issue_rate, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes + 1024));
  const int first_four[4] = {0, 1, 2, 3};
  for (int grid : {1, 148})
    for (int N : {32, 64, 128, 256})
      for (int issuers : {1, 2, 4}) run(grid, issuers, first_four, N, 1, d_cycles, d_status);
  // one issuer over several accumulators
  for (int accumulators : {2, 4}) run(148, 1, first_four, 64, accumulators, d_cycles, d_status);
  // where the issuing warps sit: different schedulers (1 and 10, 2 and 7), the same scheduler (1 and 5)
  const int placements[3][4] = {{1, 10, 0, 0}, {2, 7, 0, 0}, {1, 5, 0, 0}};
  for (const auto& w : placements) run(148, 2, w, 64, 1, d_cycles, d_status);
  return 0;
}
