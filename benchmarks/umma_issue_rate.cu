// Cycles per tcgen05.mma as a function of how the issuing thread is selected, the tile width N and the operand
// layout.  Operands are zeroed shared memory; only the timing matters.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -o /tmp/umma_issue_rate benchmarks/umma_issue_rate.cu && /tmp/umma_issue_rate
//
// Result on a B200 (1.9 GHz): with the loop inside `if (threadIdx.x == 32)` / `if (lane == 0)` every MMA costs
// 142 cycles whatever its size (N = 8 ... 256, M = 64 or 128, K-major or MN-major operands): the issue path is the
// limit, not the tensor pipe.  With the loop inside `if (elect.sync ...)` of a converged warp the cost is N / 2 cycles
// down to a floor of 60 cycles (N = 256: 128.0, N = 128: 64.1, N = 64: 59.6), i.e. the tensor pipe's full rate.
// Electing inside the loop (elect + __syncwarp per MMA) costs 243 cycles.  The kernels of this backend therefore put
// their TMA-producer and MMA-issue loops under one elect.sync.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include "../csrc/device/tcgen05.cuh"
using namespace b200;

struct Cfg { int a_mn, b_mn, M, N, nacc, lbo_b, kstep, how; };  // how: 0 lane test, 1 elect inside the loop, 2 elect around the loop
constexpr int ITERS = 2000;

__device__ __forceinline__ void issue_loop(const Cfg& c, uint32_t tmem, uint32_t a0, uint32_t a_hi, uint32_t b0, uint32_t b_hi,
                                           uint32_t idesc) {
  for (int i = 0; i < ITERS; ++i) {
    const uint32_t k = (uint32_t)(i & 3) * (uint32_t)c.kstep;  // step along K inside the tile like a real loop
    uint64_t ad, bd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ad) : "r"(a0 + k), "r"(a_hi));
    asm("mov.b64 %0, {%1, %2};" : "=l"(bd) : "r"(b0 + k), "r"(b_hi));
    umma_f16(tmem + (uint32_t)((i % c.nacc) * c.N), ad, bd, idesc, i >= c.nacc ? 1u : 0u);
  }
}

__global__ void __launch_bounds__(128, 1) probe(Cfg c, long long* out, int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  if (warp == 1) tmem_alloc(&slot, 512);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (warp == 2) {
    const uint32_t idesc = make_idesc(1, 1, 1, c.a_mn, c.b_mn, c.M, c.N);
    uint32_t a_lo, a_hi, b_lo, b_hi;
    split_desc(c.a_mn ? make_smem_desc_sw128(0, 16384, 1024) : make_smem_desc_sw128(0, 16, 1024), &a_lo, &a_hi);
    split_desc(c.b_mn ? make_smem_desc_sw128(0, c.lbo_b, 1024) : make_smem_desc_sw128(0, 16, 1024), &b_lo, &b_hi);
    const uint32_t s16 = smem_u32(smem) >> 4;
    const uint32_t a0 = a_lo + s16, b0 = b_lo + s16 + (32768 >> 4);
    const long long t0 = clock64();
    if (c.how == 0) {
      if ((threadIdx.x & 31) == 0) issue_loop(c, tmem, a0, a_hi, b0, b_hi, idesc);
    } else if (c.how == 1) {
      for (int i = 0; i < ITERS; ++i) {
        uint64_t ad, bd;
        asm("mov.b64 %0, {%1, %2};" : "=l"(ad) : "r"(a0), "r"(a_hi));
        asm("mov.b64 %0, {%1, %2};" : "=l"(bd) : "r"(b0), "r"(b_hi));
        if (elect_one()) umma_f16(tmem + (uint32_t)((i % c.nacc) * c.N), ad, bd, idesc, i >= c.nacc ? 1u : 0u);
        __syncwarp();
      }
    } else {
      if (elect_one()) issue_loop(c, tmem, a0, a_hi, b0, b_hi, idesc);
    }
    __syncwarp();
    const long long t1 = clock64();
    if (elect_one()) {
      umma_commit(&bar);
      const bool ok = mbar_wait(&bar, 0, err, 1);  // bounded wait
      const long long t2 = clock64();
      if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ok; }
    }
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

int main() {
  long long* out; int* err;
  cudaMallocManaged(&out, 64); cudaMallocManaged(&err, 4); *err = 0;
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const Cfg cfgs[] = {
      {0, 0, 128, 256, 1, 0, 2, 0},    {0, 0, 128, 256, 1, 0, 2, 1},    {0, 0, 128, 256, 1, 0, 2, 2},    {0, 0, 128, 256, 2, 0, 2, 2},
      {0, 0, 128, 192, 1, 0, 2, 2},    {0, 0, 128, 128, 1, 0, 2, 0},    {0, 0, 128, 128, 1, 0, 2, 2},    {0, 0, 128, 64, 1, 0, 2, 0},
      {0, 0, 128, 64, 1, 0, 2, 2},     {0, 0, 128, 64, 4, 0, 2, 2},     {0, 0, 128, 16, 1, 0, 2, 2},     {0, 0, 64, 256, 1, 0, 2, 2},
      {1, 1, 128, 256, 1, 8192, 128, 0}, {1, 1, 128, 256, 1, 8192, 128, 2}, {1, 1, 128, 192, 1, 8192, 128, 2}, {1, 1, 128, 192, 1, 1024, 128, 2},
      {1, 1, 128, 192, 2, 1024, 128, 2}, {1, 1, 128, 64, 1, 8192, 128, 2},
  };
  printf("   M    N a_mn b_mn nacc lbo_b how | issue clk/mma | total clk/mma | N/2\n");
  for (const Cfg& c : cfgs) {
    probe<<<148, 128, 170 * 1024>>>(c, out, err);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
    printf("%4d %4d %4d %4d %4d %5d %3d | %13.1f | %13.1f | %3d  (completed=%lld, error flag=%d)\n", c.M, c.N, c.a_mn, c.b_mn, c.nacc,
           c.lbo_b, c.how, (double)out[0] / ITERS, (double)out[1] / ITERS, c.N / 2, out[2], *err);
  }
  return 0;
}
