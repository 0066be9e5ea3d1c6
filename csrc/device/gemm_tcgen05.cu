// Persistent, warp-specialised GEMM on the 5th-generation tensor cores.
//
//   D[M,N] = act(alpha * A[M,K] * B[N,K]^T + bias + beta * R)
//
// Replaces cnnlMatMul / cnnlBatchMatMulBCast of the reference
// (torch_mlu/csrc/aten/operators/cnnl/internal/matmul_internal.cpp:106,
// bmm_internal.cpp:89) and is the main loop the convolution kernels reuse.
//
// Structure (one CTA per SM, 320 threads):
//   warp 0    : TMA producer -- per k-block one expect_tx + tiled tensor-map loads
//               of the A (128 x 128 B) and B (tile_n x 128 B) tiles, 128-byte swizzle
//   warp 1    : allocates 512 tensor-memory columns, issues tcgen05.mma (one elected
//               thread), commits to the stage's "empty" barrier and, after the last
//               k-block of a tile, to the accumulator's "full" barrier
//   warps 2-9 : epilogue (two warps per lane quarter, alternate chunks) -- tcgen05.ld 32 columns at a time, alpha/bias/residual/
//               activation in registers, cast, 16-byte global stores
// The accumulator is double buffered (2 x 256 columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.  All waits are bounded (see tcgen05.cuh).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"
#include "tcgen05.cuh"
#include "tma_util.cuh"

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_EPI_WARPS = 8;  // two epilogue warps per tensor-memory lane quarter
constexpr int GEMM_EPI_THREADS = GEMM_EPI_WARPS * 32;
constexpr int GEMM_THREADS = 64 + GEMM_EPI_THREADS;
constexpr int GEMM_MAX_STAGES = 8;
constexpr int GEMM_A_STAGE_BYTES = GEMM_BM * 128;  // 16 KB
constexpr int GEMM_TMEM_COLS = 512;
constexpr int GEMM_ACC_STRIDE = 256;  // columns per accumulator buffer

struct GemmKernelArgs {
  int M, N, K, batch;
  int tile_n, stages, k_blocks, tiles_m, tiles_n;
  int elem_bytes;       // 1 (int8), 2 or 4
  int kind;             // 0 f16/bf16, 1 tf32, 2 int8
  const float* col_scale;
  int a_mn, b_mn;
  uint32_t idesc;
  int mn_lbo, mn_sbo, mn_kstep;  // descriptor fields of MN-major operands (bytes)
  void* D;
  int64_t ldd, stride_d, stride_d2;
  int batch_inner;      // the batch index bz splits into (bz / batch_inner, bz % batch_inner): two batch strides per operand
  int d_dtype;
  const void* bias;
  int bias_dtype, bias_per_row;
  const void* residual;
  int64_t ldr, stride_r, stride_r2;
  int res_dtype;
  float alpha, beta;
  int act;
  int coef_bytes;       // shared memory reserved for column scale / bias (0 or 2048)
  int tma_store;        // epilogue stages 64-column blocks in shared memory and stores them by TMA
  int epi_bufs;         // staging buffers per epilogue warp (1 or 2)
  int reduce_add;       // fp32 D += result: 32 x 32 blocks are added to global memory with tensor-map reductions
  int splits;           // the K loop is divided among `splits` work items per output tile (reduce_add only)
  int kb_per_split;
  int* err;
};

__device__ __forceinline__ float load_scalar(const void* p, int64_t i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return v > 0.f ? v : 0.f;
  if (act == 2) return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
  return v;
}

// 32 floats -> 16 words of packed bf16 / fp16 pairs (element 2i in the low half).
__device__ __forceinline__ void pack16(const float (&v)[32], uint32_t (&pk)[16], int dt) {
  if (dt == B200_BF16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      pk[j] = *reinterpret_cast<const uint32_t*>(&h2);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __half2 h2 = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      pk[j] = *reinterpret_cast<const uint32_t*>(&h2);
    }
  }
}

// v[j] = v[j] * scale[j] + bias[j] for 32 consecutive columns; the coefficients sit in shared memory.
__device__ __forceinline__ void apply_coef(float (&v)[32], const float* sc, const float* bi) {
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 s4 = *reinterpret_cast<const float4*>(sc + j);
    const float4 b4 = *reinterpret_cast<const float4*>(bi + j);
    v[j] = fmaf(v[j], s4.x, b4.x); v[j + 1] = fmaf(v[j + 1], s4.y, b4.y);
    v[j + 2] = fmaf(v[j + 2], s4.z, b4.z); v[j + 3] = fmaf(v[j + 3], s4.w, b4.w);
  }
}

// v[j] += beta * residual[j] for `valid` (<= 32) consecutive elements starting at rp.
__device__ __forceinline__ void add_residual(float (&v)[32], const uint8_t* rp, int valid, int dt, float beta) {
  if (valid == 32 && dt != B200_F32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
    alignas(16) uint16_t hh[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(hh)[j] = __ldg(reinterpret_cast<const uint4*>(rp) + j);
    if (dt == B200_BF16) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += beta * __bfloat162float(__ushort_as_bfloat16(hh[j]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += beta * __half2float(__ushort_as_half(hh[j]));
    }
  } else if (valid == 32 && dt == B200_F32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 r4 = __ldg(reinterpret_cast<const float4*>(rp) + j / 4);
      v[j] += beta * r4.x; v[j + 1] += beta * r4.y; v[j + 2] += beta * r4.z; v[j + 3] += beta * r4.w;
    }
  } else {
    // constant indices keep v[] in registers
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) v[j] += beta * load_scalar(rp, j, dt);
  }
}

// GENERAL: the staged-store epilogue applies alpha / per-column scale and bias / per-row bias / residual / activation /
// the int32 conversion; without it an accumulator is only rounded to the output type (compile-time switch: with
// run-time flags the compiler predicated the unrolled blocks of every option instead of branching around them).
template <bool GENERAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmD, const GemmKernelArgs g) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int b_stage_bytes = g.tile_n * 128;
  const int stage_bytes = GEMM_A_STAGE_BYTES + b_stage_bytes;
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)g.stages * stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + GEMM_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * GEMM_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  // per-tile column coefficients (scale, bias); present only when the launch has any
  float* coef = reinterpret_cast<float*>(tiles + (size_t)g.stages * stage_bytes + 1024);
  uint8_t* stage_out = tiles + (size_t)g.stages * stage_bytes + 1024 + g.coef_bytes;  // 8 warps x 2 buffers x 4 KB, 128-byte swizzled

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], GEMM_EPI_THREADS);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc(tmem_slot, GEMM_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_batch = g.tiles_m * g.tiles_n;
  // a work item is (output tile, K split); splits of one tile are adjacent so that they run at the same time
  const int total_tiles = tiles_per_batch * g.batch * g.splits;
  const int bk_elems = 128 / g.elem_bytes;          // K elements per k-block
  const int mn_block = 128 / g.elem_bytes;          // MN elements per 128-byte row (MN-major)
  bool failed = false;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = (uint32_t)stage_bytes;
      for (int item = blockIdx.x; item < total_tiles && !failed; item += gridDim.x) {
        const int tile = item / g.splits, split = item - tile * g.splits;
        const int bz = tile / tiles_per_batch;
        const int bo = bz / g.batch_inner, bi = bz - bo * g.batch_inner;
        const int t = tile - bz * tiles_per_batch;
        const int m0 = (t % g.tiles_m) * GEMM_BM;
        const int n0 = (t / g.tiles_m) * g.tile_n;
        const int kb0 = split * g.kb_per_split, kb1 = min(g.k_blocks, kb0 + g.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, g.err, ERR_TIMEOUT_EMPTY)) { failed = true; break; }
          mbar_arrive_expect_tx(&full_bar[stage], tx_bytes);
          uint8_t* sa = tiles + (size_t)stage * stage_bytes;
          uint8_t* sb = sa + GEMM_A_STAGE_BYTES;
          const int k0 = kb * bk_elems;
          if (!g.a_mn) {
            tma_load_4d(sa, &tmA, &full_bar[stage], k0, m0, bi, bo);
          } else {
            const int blk_bytes = bk_elems * 128;
            for (int i = 0; i < GEMM_BM / mn_block; ++i)
              tma_load_4d(sa + i * blk_bytes, &tmA, &full_bar[stage], m0 + i * mn_block, k0, bi, bo);
          }
          if (!g.b_mn) {
            tma_load_4d(sb, &tmB, &full_bar[stage], k0, n0, bi, bo);
          } else {
            const int blk_bytes = bk_elems * 128;
            for (int i = 0; i < g.tile_n / mn_block; ++i)
              tma_load_4d(sb + i * blk_bytes, &tmB, &full_bar[stage], n0 + i * mn_block, k0, bi, bo);
          }
          if (++stage == g.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      // descriptor templates and addresses in 16-byte units: per K block the issue loop only adds
      uint32_t a_lo0, a_hi, b_lo0, b_hi;
      split_desc(g.a_mn ? make_smem_desc_sw128(0, g.mn_lbo, g.mn_sbo) : make_smem_desc_sw128(0, 16, 1024), &a_lo0, &a_hi);
      split_desc(g.b_mn ? make_smem_desc_sw128(0, g.mn_lbo, g.mn_sbo) : make_smem_desc_sw128(0, 16, 1024), &b_lo0, &b_hi);
      const uint32_t a_step = g.a_mn ? (uint32_t)g.mn_kstep >> 4 : 2u, b_step = g.b_mn ? (uint32_t)g.mn_kstep >> 4 : 2u;
      const uint32_t tiles_16 = smem_u32(tiles) >> 4, stage_16 = (uint32_t)stage_bytes >> 4;
      for (int item = blockIdx.x; item < total_tiles && !failed; item += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, g.err, ERR_TIMEOUT_TMEM_EMPTY)) { failed = true; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * GEMM_ACC_STRIDE;
        const int split = item % g.splits;
        const int kb0 = split * g.kb_per_split, kb1 = min(g.k_blocks, kb0 + g.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, g.err, ERR_TIMEOUT_FULL)) { failed = true; break; }
          tc_fence_after();
          const uint32_t sa_16 = tiles_16 + (uint32_t)stage * stage_16;
          const uint32_t sb_16 = sa_16 + (GEMM_A_STAGE_BYTES >> 4);
          const uint32_t accum = kb > kb0 ? 1u : 0u;
          if (g.kind == 1) umma_x4<1>(d_tmem, a_lo0 + sa_16, a_hi, a_step, b_lo0 + sb_16, b_hi, b_step, g.idesc, accum);
          else if (g.kind == 2) umma_x4<2>(d_tmem, a_lo0 + sa_16, a_hi, a_step, b_lo0 + sb_16, b_hi, b_step, g.idesc, accum);
          else umma_x4<0>(d_tmem, a_lo0 + sa_16, a_hi, a_step, b_lo0 + sb_16, b_hi, b_step, g.idesc, accum);
          umma_commit(&empty_bar[stage]);  // frees the smem stage once the MMAs have read it
          if (++stage == g.stages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // tcgen05.ld: warp w may touch lanes [32*(w%4), +32)
    const int colhalf = (warp - 2) >> 2;  // the two warps of a quarter take alternate 32-column chunks
    int acc = 0;
    int sbuf_sel = 0;
    uint32_t acc_phase = 0;
    uint32_t tile_iter = 0;
    const bool has_coef = g.col_scale != nullptr || (g.bias != nullptr && !g.bias_per_row);
    for (int item = blockIdx.x; item < total_tiles && !failed; item += gridDim.x, ++tile_iter) {
      const int tile = item / g.splits;
      const int bz = tile / tiles_per_batch;
      const int bo = bz / g.batch_inner, bi = bz - bo * g.batch_inner;
      const int t = tile - bz * tiles_per_batch;
      const int m0 = (t % g.tiles_m) * GEMM_BM;
      const int n0 = (t / g.tiles_m) * g.tile_n;
      const float* cs = coef;
      if (has_coef) {
        // every thread has passed a barrier after its last read of the previous tile's coefficients
        float* wsc = coef;
        for (int ci = threadIdx.x - 64; ci < g.tile_n; ci += GEMM_EPI_THREADS) {
          const int n = n0 + ci;
          wsc[ci] = (g.col_scale && n < g.N) ? g.col_scale[n] : 1.f;
          wsc[256 + ci] = (g.bias && !g.bias_per_row && n < g.N) ? load_scalar(g.bias, n, g.bias_dtype) : 0.f;
        }
        named_barrier(2, GEMM_EPI_THREADS);
      }
      if (!mbar_wait(&acc_full[acc], acc_phase, g.err, ERR_TIMEOUT_TMEM_FULL)) { failed = true; break; }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < g.M;
      const float row_bias = (g.bias && g.bias_per_row && row_ok) ? load_scalar(g.bias, row, g.bias_dtype) : 0.f;
      uint8_t* drow = static_cast<uint8_t*>(g.D) +
                      ((size_t)bi * g.stride_d + (size_t)bo * g.stride_d2 + (size_t)row * g.ldd) * (g.d_dtype == B200_F32 ? 4 : 2);
      const uint8_t* rrow = g.residual ? static_cast<const uint8_t*>(g.residual) +
                                             ((size_t)bi * g.stride_r + (size_t)bo * g.stride_r2 + (size_t)row * g.ldr) *
                                                 (g.res_dtype == B200_F32 ? 4 : 2)
                                       : nullptr;
      if (g.reduce_add) {
        // fp32 accumulation into global memory: each warp stages 32 rows x 32 fp32 columns (4 KB, 128-byte swizzle) and
        // adds them with one tensor-map reduction; rows / columns outside the matrix are clipped.  K splits of one tile and
        // whatever the destination already holds simply add up.
        uint8_t* sbuf0 = stage_out + (warp - 2) * 4096 * g.epi_bufs;
        const uint32_t t_addr = tmem_base + acc * GEMM_ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
        for (int c = colhalf * 32; c < g.tile_n; c += 64) {
          uint32_t r[32];
          tmem_ld32(t_addr + c, r);
          tmem_ld_wait();
          if (n0 + c >= g.N) continue;  // warp-uniform
          if (g.alpha != 1.f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * g.alpha);
          }
          if (lane == 0) {
            if (g.epi_bufs == 2) tma_store_wait_read<1>();
            else tma_store_wait_read<0>();
          }
          __syncwarp();
          uint8_t* sbuf = sbuf0 + sbuf_sel * 4096;
          if (g.epi_bufs == 2) sbuf_sel ^= 1;
          uint8_t* srow = sbuf + lane * 128;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            *reinterpret_cast<uint4*>(srow + ((k ^ (lane & 7)) * 16)) = make_uint4(r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_reduce_add_4d(&tmD, sbuf, n0 + c, m0 + quarter * 32, bi, bo);
            tma_store_commit();
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        if (has_coef) named_barrier(2, GEMM_EPI_THREADS);
        continue;
      }
      if (g.tma_store) {
        // Each epilogue warp stages its own 32 rows x 64 columns (4 KB, 128-byte swizzle) and issues its own
        // tensor-map store; the two warps of a lane quarter take alternate 64-column blocks.  No barrier
        // across warps is needed.
        uint8_t* sbuf0 = stage_out + (warp - 2) * 4096 * g.epi_bufs;  // two buffers per warp when they fit: convert while the last store is read
        auto finish = [&](const uint32_t (&r)[32], int c, float (&v)[32]) {
          const int n_base = n0 + c;
          if (!GENERAL) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) v[jj] = __uint_as_float(r[jj]);
            return;
          }
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) v[jj] = g.kind == 2 ? (float)(int)r[jj] : __uint_as_float(r[jj]);
          if (g.alpha != 1.f) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) v[jj] *= g.alpha;
          }
          if (has_coef) apply_coef(v, cs + c, cs + 256 + c);
          if (g.bias && g.bias_per_row) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) v[jj] += row_bias;
          }
          if (rrow && row_ok && n_base < g.N)
            add_residual(v, rrow + (size_t)n_base * (g.res_dtype == B200_F32 ? 4 : 2), min(32, g.N - n_base), g.res_dtype, g.beta);
          if (g.act) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) v[jj] = apply_act(v[jj], g.act);
          }
        };
        const uint32_t t_addr = tmem_base + acc * GEMM_ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
        for (int cb = colhalf * 64; cb < g.tile_n; cb += 128) {
          uint32_t ra[32], rb[32];
          tmem_ld32(t_addr + cb, ra);
          tmem_ld32(t_addr + cb + 32, rb);
          tmem_ld_wait();
          if (lane == 0) {  // the store that last used this buffer has read it
            if (g.epi_bufs == 2) tma_store_wait_read<1>();
            else tma_store_wait_read<0>();
          }
          __syncwarp();
          uint8_t* sbuf = sbuf0 + sbuf_sel * 4096;
          if (g.epi_bufs == 2) sbuf_sel ^= 1;
          uint8_t* srow = sbuf + lane * 128;
          // one copy of the code for both 32-column halves (the second half is moved into the first half's
          // registers); not unrolled, to keep the hot code small
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            float v[32];
            uint32_t pk[16];
            finish(ra, cb + 32 * h, v);
            pack16(v, pk, g.d_dtype);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              *reinterpret_cast<uint4*>(srow + (((4 * h + k) ^ (lane & 7)) * 16)) = make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
#pragma unroll
            for (int j = 0; j < 32; ++j) ra[j] = rb[j];
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tmD, sbuf, n0 + cb, m0 + quarter * 32, bi, bo);  // rows / columns outside the matrix are clipped
            tma_store_commit();
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        if (has_coef) named_barrier(2, GEMM_EPI_THREADS);
        continue;
      }
      for (int c = colhalf * 32; c < g.tile_n; c += 64) {
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * GEMM_ACC_STRIDE + ((uint32_t)(quarter * 32) << 16) + c, r);
        tmem_ld_wait();
        const int n_base = n0 + c;
        if (!row_ok || n_base >= g.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = g.kind == 2 ? (float)(int)r[j] : __uint_as_float(r[j]);
        if (g.alpha != 1.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= g.alpha;
        }
        const int valid = min(32, g.N - n_base);
        if (has_coef) apply_coef(v, cs + c, cs + 256 + c);
        if (g.bias && g.bias_per_row) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += row_bias;
        }
        if (rrow) add_residual(v, rrow + (size_t)n_base * (g.res_dtype == B200_F32 ? 4 : 2), valid, g.res_dtype, g.beta);
        if (g.act) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], g.act);
        }
        if (g.d_dtype == B200_F32) {
          float* o = reinterpret_cast<float*>(drow) + n_base;
          if (valid == 32 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) o[j] = v[j];
          }
        } else {
          uint32_t pk[16];
          pack16(v, pk, g.d_dtype);
          uint16_t* o = reinterpret_cast<uint16_t*>(drow) + n_base;
          if (valid == 32 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(o)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) o[j] = (uint16_t)(pk[j >> 1] >> ((j & 1) * 16));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (has_coef) named_barrier(2, GEMM_EPI_THREADS);
    }
  }

  // ---------------------------------------------------------------- teardown
  if ((g.tma_store || g.reduce_add) && warp >= 2 && lane == 0) tma_store_wait_all<0>();  // every issuing lane drains its own stores
  if (*((volatile int*)g.err) != 0) {
    // Error path: give copies that are still in flight time to land before the
    // shared memory goes away.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, GEMM_TMEM_COLS);
  }
}

static int pick_tile_n(int M, int N, int sms) {
  // Candidates are multiples of 32 up to 256; prefer the one with the fewest
  // waves of CTAs, then the least padding, then the widest tile.
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  int best = 256;
  double best_cost = 1e30;
  for (int tn = 256; tn >= 32; tn -= 32) {
    const int tiles_n = (N + tn - 1) / tn;
    const long tiles = (long)tiles_m * tiles_n;
    const long waves = (tiles + sms - 1) / sms;
    // cost ~ time: waves * (tile_n work) with a fixed per-tile overhead
    const double cost = (double)waves * (tn + 24);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = tn;
    }
  }
  return best;
}

}  // namespace b200

extern "C" int b200_gemm(const B200GemmParams* p, void* stream) {
  using namespace b200;
  if (p->M <= 0 || p->N <= 0 || p->batch <= 0) return 0;
  if (p->K <= 0) return (int)cudaErrorInvalidValue;
  const int es = p->ab_dtype == B200_F32 ? 4 : (p->ab_dtype == B200_I8 ? 1 : 2);
  if (es == 1 && (p->a_mn_major || p->b_mn_major)) return (int)cudaErrorInvalidValue;  // int8 operands are K-major
  // fp32 operands run as tf32 and must be K-major (the host layer transposes).
  if (es == 4 && (p->a_mn_major || p->b_mn_major)) return (int)cudaErrorInvalidValue;
  const CUtensorMapDataType dt = p->ab_dtype == B200_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : p->ab_dtype == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : p->ab_dtype == B200_I8  ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                           : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  auto ok16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!ok16(p->A) || !ok16(p->B) || (p->lda * es) % 16 || (p->ldb * es) % 16 || (p->stride_a * es) % 16 ||
      (p->stride_b * es) % 16 || (p->stride_a2 * es) % 16 || (p->stride_b2 * es) % 16)
    return (int)cudaErrorInvalidValue;
  // batch = outer x inner; with batch_inner == 0 (the usual case) there is one batch stride per operand
  const int inner = p->batch_inner > 0 ? p->batch_inner : p->batch;
  if (p->batch % inner) return (int)cudaErrorInvalidValue;
  const int outer = p->batch / inner;

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int bk = 128 / es;
  const int mn_block = 128 / es;

  GemmKernelArgs g{};
  g.M = p->M; g.N = p->N; g.K = p->K; g.batch = p->batch;
  g.tile_n = p->tile_n > 0 ? p->tile_n : pick_tile_n(p->M, p->N, sms);
  if (p->b_mn_major && g.tile_n % mn_block) g.tile_n = (g.tile_n + mn_block - 1) / mn_block * mn_block;
  if (g.tile_n > 256 || g.tile_n % 32) return (int)cudaErrorInvalidValue;
  g.k_blocks = (p->K + bk - 1) / bk;
  g.tiles_m = (p->M + GEMM_BM - 1) / GEMM_BM;
  g.tiles_n = (p->N + g.tile_n - 1) / g.tile_n;
  g.elem_bytes = es;
  g.a_mn = p->a_mn_major; g.b_mn = p->b_mn_major;
  const int fmt = p->ab_dtype == B200_F32 ? 2 : ((p->ab_dtype == B200_BF16 || p->ab_dtype == B200_I8) ? 1 : 0);
  g.kind = es == 4 ? 1 : (es == 1 ? 2 : 0);
  g.col_scale = p->col_scale;
  g.idesc = make_idesc(g.kind == 2 ? 2 : 1, fmt, fmt, g.a_mn, g.b_mn, GEMM_BM, g.tile_n);
  // MN-major: 8-row K groups are 1024 B apart, 128-byte MN blocks are one
  // k-block (bk rows x 128 B) apart, one MMA consumes 32 B of K = (32/es) rows.
  g.mn_sbo = 1024;
  g.mn_lbo = bk * 128;
  g.mn_kstep = (32 / es) * 128;
  g.D = p->D; g.ldd = p->ldd; g.stride_d = p->stride_d; g.stride_d2 = p->stride_d2; g.d_dtype = p->d_dtype;
  g.batch_inner = inner;
  g.bias = p->bias; g.bias_dtype = p->bias_dtype; g.bias_per_row = p->bias_per_row;
  g.residual = p->residual; g.ldr = p->ldr; g.stride_r = p->stride_r; g.stride_r2 = p->stride_r2; g.res_dtype = p->res_dtype;
  g.alpha = p->alpha; g.beta = p->beta; g.act = p->act;
  g.err = error_flag_ptr();
  if (!g.err) return (int)cudaErrorInvalidDevice;

  const int stage_bytes = GEMM_A_STAGE_BYTES + g.tile_n * 128;
  g.tma_store = (p->d_dtype != B200_F32 && g.tile_n % 64 == 0 && (p->ldd * 2) % 16 == 0 && (p->stride_d * 2) % 16 == 0 &&
                 (p->stride_d2 * 2) % 16 == 0 &&
                 (reinterpret_cast<uintptr_t>(p->D) & 15) == 0)
                    ? 1 : 0;
  g.reduce_add = 0;
  g.splits = 1;
  g.kb_per_split = g.k_blocks;
  if (p->accumulate) {
    // D (fp32) += alpha * A * B: no bias / residual / activation (they would be applied once per K split)
    if (p->d_dtype != B200_F32 || p->bias || p->residual || p->act || p->col_scale || (p->ldd * 4) % 16 || (p->stride_d * 4) % 16 ||
        (reinterpret_cast<uintptr_t>(p->D) & 15))
      return (int)cudaErrorInvalidValue;
    g.reduce_add = 1;
    g.tma_store = 0;
    int splits = p->splits;
    if (splits <= 0) {
      // fill the GPU once: as many K splits as it takes for every SM to have a work item, at least 4 K blocks each
      const long tiles = (long)g.tiles_m * g.tiles_n * g.batch;
      splits = (int)(sms / tiles);
      const int max_splits = (g.k_blocks + 3) / 4;
      if (splits > max_splits) splits = max_splits;
      if (splits < 1) splits = 1;
    }
    if (splits > g.k_blocks) splits = g.k_blocks;
    g.kb_per_split = (g.k_blocks + splits - 1) / splits;
    g.splits = (g.k_blocks + g.kb_per_split - 1) / g.kb_per_split;
  }
  g.coef_bytes = (p->col_scale || (p->bias && !p->bias_per_row)) ? 2048 : 0;
  const bool staged = g.tma_store || g.reduce_add;
  int smem_budget = 227 * 1024 - 2048 - g.coef_bytes - (staged ? 32768 : 0);
  g.epi_bufs = 1;
  if (staged && (smem_budget - 32768) / stage_bytes >= 4) {  // a second staging buffer per warp when four stages still fit
    g.epi_bufs = 2;
    smem_budget -= 32768;
  }
  g.stages = smem_budget / stage_bytes;
  if (g.stages > GEMM_MAX_STAGES) g.stages = GEMM_MAX_STAGES;
  if (g.stages > g.kb_per_split + 1) g.stages = g.kb_per_split + 1 < 2 ? 2 : g.kb_per_split + 1;
  if (g.stages < 2) g.stages = 2;
  const size_t smem = (size_t)g.stages * stage_bytes + 1024 /*align*/ + 1024 /*barriers*/ + g.coef_bytes +
                      (staged ? 32768 * g.epi_bufs : 0);

  CUtensorMap tmA, tmB;
  // batch strides: a single-level batch of one matrix still needs a non-zero, 16-byte-multiple stride in the map
  auto bstride = [&](int64_t given, int64_t dflt) { return (uint64_t)((given > 0 ? given : dflt) * es); };
  const int64_t span_a = (int64_t)p->lda * (p->a_mn_major ? p->K : p->M), span_b = (int64_t)p->ldb * (p->b_mn_major ? p->K : p->N);
  const uint64_t ba1 = bstride(p->stride_a, span_a), ba2 = bstride(p->stride_a2, span_a * inner);
  const uint64_t bb1 = bstride(p->stride_b, span_b), bb2 = bstride(p->stride_b2, span_b * inner);
  int rc;
  if (!p->a_mn_major) {
    uint64_t dims[4] = {(uint64_t)p->K, (uint64_t)p->M, (uint64_t)inner, (uint64_t)outer};
    uint64_t str[3] = {(uint64_t)p->lda * es, ba1, ba2};
    uint32_t box[4] = {(uint32_t)bk, GEMM_BM, 1, 1};
    rc = encode_tiled(&tmA, dt, 4, p->A, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    uint64_t dims[4] = {(uint64_t)p->M, (uint64_t)p->K, (uint64_t)inner, (uint64_t)outer};
    uint64_t str[3] = {(uint64_t)p->lda * es, ba1, ba2};
    uint32_t box[4] = {(uint32_t)mn_block, (uint32_t)bk, 1, 1};
    rc = encode_tiled(&tmA, dt, 4, p->A, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc) return rc;
  if (!p->b_mn_major) {
    uint64_t dims[4] = {(uint64_t)p->K, (uint64_t)p->N, (uint64_t)inner, (uint64_t)outer};
    uint64_t str[3] = {(uint64_t)p->ldb * es, bb1, bb2};
    uint32_t box[4] = {(uint32_t)bk, (uint32_t)g.tile_n, 1, 1};
    rc = encode_tiled(&tmB, dt, 4, p->B, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    uint64_t dims[4] = {(uint64_t)p->N, (uint64_t)p->K, (uint64_t)inner, (uint64_t)outer};
    uint64_t str[3] = {(uint64_t)p->ldb * es, bb1, bb2};
    uint32_t box[4] = {(uint32_t)mn_block, (uint32_t)bk, 1, 1};
    rc = encode_tiled(&tmB, dt, 4, p->B, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc) return rc;

  const int64_t span_d = (int64_t)p->ldd * p->M;
  g.stride_d = p->stride_d > 0 ? p->stride_d : span_d;
  g.stride_d2 = p->stride_d2 > 0 ? p->stride_d2 : g.stride_d * inner;
  if (p->residual) {
    g.stride_r = p->batch > 1 ? p->stride_r : 0;
    g.stride_r2 = p->stride_r2 > 0 ? p->stride_r2 : g.stride_r * inner;
  }
  CUtensorMap tmD = tmA;
  if (g.tma_store) {
    const CUtensorMapDataType ddt = p->d_dtype == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    uint64_t dims[4] = {(uint64_t)p->N, (uint64_t)p->M, (uint64_t)inner, (uint64_t)outer};
    uint64_t str[3] = {(uint64_t)p->ldd * 2, (uint64_t)g.stride_d * 2, (uint64_t)g.stride_d2 * 2};
    uint32_t box[4] = {64, 32, 1, 1};  // one epilogue warp stores 32 rows at a time
    rc = encode_tiled(&tmD, ddt, 4, p->D, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  if (g.reduce_add) {
    uint64_t dims[4] = {(uint64_t)p->N, (uint64_t)p->M, (uint64_t)inner, (uint64_t)outer};
    uint64_t str[3] = {(uint64_t)p->ldd * 4, (uint64_t)g.stride_d * 4, (uint64_t)g.stride_d2 * 4};
    uint32_t box[4] = {32, 32, 1, 1};
    rc = encode_tiled(&tmD, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p->D, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  const bool general = !(g.tma_store && g.kind != 2 && g.alpha == 1.f && !g.col_scale && !g.bias && !g.residual && !g.act);
  typedef void (*Kernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmKernelArgs);
  const Kernel kernel = general ? gemm_tcgen05_kernel<true> : gemm_tcgen05_kernel<false>;
  static bool attr_set[2][64] = {};
  if (!attr_set[general ? 1 : 0][dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set[general ? 1 : 0][dev & 63] = true;
  }
  const long total_tiles = (long)g.tiles_m * g.tiles_n * g.batch * g.splits;
  int ctas = p->max_ctas > 0 ? p->max_ctas : sms;
  if (ctas > total_tiles) ctas = (int)total_tiles;
  kernel<<<ctas, GEMM_THREADS, smem, (cudaStream_t)stream>>>(tmA, tmB, tmD, g);
  return (int)cudaGetLastError();
}
