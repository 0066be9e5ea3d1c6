// Implicit-GEMM convolution (forward / data gradient) and weight gradient on
// tcgen05 tensor cores with tensor-memory accumulators.
//
// Replaces cnnlConvolutionForward / BackwardData / BackwardFilter of the reference
// (torch_mlu/csrc/aten/operators/cnnl/internal/convolution_float_forward_internal.cpp:136,
// convolution_float_backward_internal.cpp:89,162).
//
// Forward (and dgrad):  M = 128 output pixels (a BW x BH x BNI box of the pixel
// grid), N = tile_n output channels, K loop = taps x 64-channel blocks.  Warp roles
// are those of the GEMM kernel (TMA producer / MMA issuer / 8 epilogue warps, two
// accumulator buffers); each epilogue warp stages and stores its own 32 pixels, so the
// store path has no CTA-wide barrier.  When the weights of one output-channel tile are
// small they stay resident in shared memory and the pipeline stages hold activations only.  The A tile of a tap is ONE 4-D tiled tensor-map load whose
// origin is the tile's pixel origin plus the tap offset; halo elements outside the
// view are zero-filled by the copy engine, so no im2col buffer exists anywhere.
//
// Wgrad: M = 128 output channels, N = up to four 64-wide blocks of the flattened
// (tap, input-channel) axis, K = pixels (64 per stage).  Both operands are MN-major
// (channels contiguous) straight out of the NHWC tensors.  CTAs split the pixel
// range and add their partial tiles to an fp32 buffer.
#include <algorithm>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"
#include "tcgen05.cuh"
#include "tma_util.cuh"

namespace b200 {

constexpr int CONV_THREADS = 192;        // weight-gradient kernel: TMA warp, MMA warp, 4 epilogue warps
constexpr int CONV_EPI_WARPS = 8;          // forward kernel: two epilogue warps per tensor-memory lane quarter
constexpr int CONV_EPI_THREADS = CONV_EPI_WARPS * 32;
constexpr int CONV_FPROP_THREADS = 64 + CONV_EPI_THREADS;
constexpr int CONV_MAX_STAGES = 12;
constexpr int CONV_A_BYTES = 128 * 128;

struct ConvArgs {
  int N, P, Q, Cin, Cout;
  int bw, bh, bni;              // pixel box (bw*bh*bni == 128)
  int tiles_q, tiles_p, tiles_n, tiles_co, tile_n;
  int c_blocks;                 // Cin / cblk (rounded up)
  int cblk;                     // input channels per 128-byte row: 64 (16-bit) or 128 (int8)
  int kind;                     // 0 f16/bf16, 2 int8
  int ntaps, stages, b_mn;
  uint32_t idesc;
  B200ConvTap taps[B200_CONV_MAX_TAPS];
  void* out;
  int out_dtype;
  long long o_sn, o_sh, o_sw;
  int o_mul_h, o_off_h, o_mul_w, o_off_w;
  const float* scale;
  const void* bias;
  int bias_dtype;
  const void* residual;
  int res_dtype;
  int act;
  float alpha;
  double* stats;                // optional [2 * Cout]: per-channel sum and sum of squares of the stored outputs
  float out_qscale;             // int8 outputs: multiplier before rounding
  // Halo mode (single channel block, every tap on one view, resident weights): per pixel tile (8 wide,
  // 16 high) one column tile of 8 x halo_h pixels is loaded for each distinct horizontal tap offset; a
  // tap's A operand is the window of its column tile shifted down by whole pixel rows (8 x 128 bytes =
  // one swizzle repeat, so the window stays aligned).  Activations cross L2 -> shared memory once per
  // horizontal offset instead of once per tap.  (A single tile with windows shifted sideways by 128-byte
  // steps was tried: a descriptor that starts off the 1024-byte swizzle repeat gave wrong products even
  // with its base-offset field set, so that variant is not used.)
  int halo, halo_h, halo_stage_bytes, dw_min, dh_min;
  int halo_ndw, halo_col_bytes;
  int b_res_bytes;              // > 0: weights of one output-channel tile stay resident in shared memory
  int coef_bytes;               // shared memory reserved for per-channel scale / bias (0 or 2048)
  int tma_store;                // epilogue stages 64-channel blocks in shared memory and stores them by TMA
  int epi_bufs;                 // staging buffers per epilogue warp (2 when shared memory allows: conversion overlaps the store)
  int* err;
};

struct ConvMaps {
  CUtensorMap a[B200_CONV_MAX_MAPS];
  CUtensorMap w;
  CUtensorMap out;
};

__device__ __forceinline__ float ld_scalar(const void* p, long long i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
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

// v[j] = v[j] * scale[j] + bias[j] for 32 consecutive channels; the coefficients sit in shared memory.
__device__ __forceinline__ void apply_coef(float (&v)[32], const float* sc, const float* bi) {
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 s4 = *reinterpret_cast<const float4*>(sc + j);
    const float4 b4 = *reinterpret_cast<const float4*>(bi + j);
    v[j] = fmaf(v[j], s4.x, b4.x); v[j + 1] = fmaf(v[j + 1], s4.y, b4.y);
    v[j + 2] = fmaf(v[j + 2], s4.z, b4.z); v[j + 3] = fmaf(v[j + 3], s4.w, b4.w);
  }
}

// v[j] += residual[j] for `valid` (<= 32) consecutive elements starting at rp.
__device__ __forceinline__ void add_residual(float (&v)[32], const uint8_t* rp, int valid, int dt) {
  if (valid == 32 && dt != B200_F32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
    alignas(16) uint16_t hh[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(hh)[j] = __ldg(reinterpret_cast<const uint4*>(rp) + j);
    if (dt == B200_BF16) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(__ushort_as_bfloat16(hh[j]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += __half2float(__ushort_as_half(hh[j]));
    }
  } else {
    // constant indices keep v[] in registers
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) v[j] += ld_scalar(rp, j, dt);
  }
}

// GENERAL: the epilogue applies alpha / per-channel scale and bias / residual / activation (I8: the accumulators
// are int32); without it an accumulator is only rounded to the output type.  STATS: channel sums for a following
// batch norm.  Compile-time switches: with run-time flags the compiler predicated the unrolled 32-element blocks of
// every option instead of branching around them, and the plain 64 -> 256 channel 1x1 layer spent a third of its time
// on instructions of options it did not use (145 -> 99 us).
template <bool GENERAL, bool STATS, bool I8, bool RES>
__global__ void __launch_bounds__(CONV_FPROP_THREADS, 1)
conv_fprop_kernel(const __grid_constant__ ConvMaps maps, const __grid_constant__ ConvArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Layout: [resident weights (b_res_bytes, may be 0)] [stages] [barriers 1 KB] [coefficients] [output staging 32 KB]
  // Streaming mode: a stage holds an A tile (16 KB) and the tap's weight tile.
  // Resident mode : a stage holds only the A tile; the weights of the current output-channel
  //                 tile (all taps, all channel blocks) stay in shared memory across pixel tiles.
  const int b_blk_bytes = g.tile_n * 128;
  const int stage_bytes = g.halo ? g.halo_stage_bytes : CONV_A_BYTES + (g.b_res_bytes ? 0 : b_blk_bytes);
  uint8_t* bres = smem;
  uint8_t* stage0 = smem + g.b_res_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + (size_t)g.stages * stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + CONV_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * CONV_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* b_full = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_full + 1);
  float* coef = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 1024);
  // eight 4 KB staging buffers (32 pixels x 64 channels, 128-byte swizzle), one per epilogue warp
  uint8_t* stage_out = reinterpret_cast<uint8_t*>(bars) + 1024 + g.coef_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], CONV_EPI_THREADS); }
    mbar_init(b_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&maps.w);
    if (g.tma_store) tma_prefetch_desc(&maps.out);
    tma_prefetch_desc(&maps.a[0]);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int pix_tiles = g.tiles_q * g.tiles_p * g.tiles_n;
  const int total_tiles = pix_tiles * g.tiles_co;
  const int k_iters = g.ntaps * g.c_blocks;
  bool failed = false;

  if (warp == 0) {
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0; uint32_t phase = 0;
      int cur_ct = -1;
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
        // pixel tiles vary fastest so concurrently running CTAs share the weight tile
        const int pt = tile % pix_tiles, ct = tile / pix_tiles;
        const int q0 = (pt % g.tiles_q) * g.bw;
        const int p0 = ((pt / g.tiles_q) % g.tiles_p) * g.bh;
        const int n0 = (pt / (g.tiles_q * g.tiles_p)) * g.bni;
        const int co0 = ct * g.tile_n;
        if (g.b_res_bytes && ct != cur_ct) {
          // Every MMA that read the previous weights has finished once all stages are empty.
          for (int i = 0; i < g.stages && !failed; ++i) {
            const int s = stage + i < g.stages ? stage + i : stage + i - g.stages;
            const uint32_t par = s >= stage ? (phase ^ 1) : phase;
            if (!mbar_wait(&empty_bar[s], par, g.err, ERR_TIMEOUT_EMPTY)) failed = true;
          }
          if (failed) break;
          mbar_arrive_expect_tx(b_full, (uint32_t)g.b_res_bytes);
          for (int it = 0; it < k_iters; ++it) {
            const int tap = it / g.c_blocks, cb = it - tap * g.c_blocks;
            uint8_t* sb = bres + (size_t)it * b_blk_bytes;
            if (!g.b_mn) {
              tma_load_3d(sb, &maps.w, b_full, cb * g.cblk, co0, g.taps[tap].wtap);
            } else {
              for (int j = 0; j < g.tile_n / 64; ++j)
                tma_load_3d(sb + j * 8192, &maps.w, b_full, co0 + j * 64, cb * 64, g.taps[tap].wtap);
            }
          }
          cur_ct = ct;
        }
        if (g.halo) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, g.err, ERR_TIMEOUT_EMPTY)) { failed = true; break; }
          // channel coordinate 0; the pixel origin may be negative (zero filled)
          mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)(g.halo_ndw * g.halo_col_bytes));
          for (int j = 0; j < g.halo_ndw; ++j)
            tma_load_4d(stage0 + (size_t)stage * stage_bytes + (size_t)j * g.halo_col_bytes, &maps.a[1], &full_bar[stage], 0,
                        q0 + g.dw_min + j, p0 + g.dh_min, n0);
          if (++stage == g.stages) { stage = 0; phase ^= 1; }
          continue;
        }
        for (int it = 0; it < k_iters; ++it) {
          const int tap = it / g.c_blocks, cb = it - tap * g.c_blocks;
          const B200ConvTap tp = g.taps[tap];
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, g.err, ERR_TIMEOUT_EMPTY)) { failed = true; break; }
          mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)stage_bytes);
          uint8_t* sa = stage0 + (size_t)stage * stage_bytes;
          tma_load_4d(sa, &maps.a[tp.map], &full_bar[stage], cb * g.cblk, q0 + tp.dw, p0 + tp.dh, n0);
          if (!g.b_res_bytes) {
            if (!g.b_mn) {
              tma_load_3d(sa + CONV_A_BYTES, &maps.w, &full_bar[stage], cb * g.cblk, co0, tp.wtap);
            } else {
              for (int j = 0; j < g.tile_n / 64; ++j)
                tma_load_3d(sa + CONV_A_BYTES + j * 8192, &maps.w, &full_bar[stage], co0 + j * 64, cb * 64, tp.wtap);
            }
          }
          if (++stage == g.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0;
      int cur_ct = -1; uint32_t b_phase = 0;
      // descriptor templates and addresses in 16-byte units: per K block the issue loop only adds
      uint32_t a_lo0, a_hi, b_lo0, b_hi;
      split_desc(make_smem_desc_sw128(0, 16, 1024), &a_lo0, &a_hi);
      split_desc(g.b_mn ? make_smem_desc_sw128(0, 8192, 1024) : make_smem_desc_sw128(0, 16, 1024), &b_lo0, &b_hi);
      const uint32_t b_step = g.b_mn ? 128u : 2u;  // 2048 or 32 bytes per K = 16 step
      const uint32_t stage0_16 = smem_u32(stage0) >> 4, stage_16 = (uint32_t)stage_bytes >> 4;
      const uint32_t bres_16 = smem_u32(bres) >> 4, bblk_16 = (uint32_t)b_blk_bytes >> 4;
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
        const int ct = tile / pix_tiles;
        if (g.b_res_bytes && ct != cur_ct) {
          if (!mbar_wait(b_full, b_phase, g.err, ERR_TIMEOUT_FULL)) { failed = true; break; }
          b_phase ^= 1;
          cur_ct = ct;
        }
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, g.err, ERR_TIMEOUT_TMEM_EMPTY)) { failed = true; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        if (g.halo) {
          if (!mbar_wait(&full_bar[stage], phase, g.err, ERR_TIMEOUT_FULL)) { failed = true; break; }
          tc_fence_after();
          const uint32_t tile0_16 = stage0_16 + (uint32_t)stage * stage_16;
          for (int tap = 0; tap < g.ntaps; ++tap) {
            const B200ConvTap tp = g.taps[tap];
            // column tile of this tap's dw, shifted down by (dh - dh_min) pixel rows of 1024 bytes
            const uint32_t a0_16 = tile0_16 + (uint32_t)(((tp.dw - g.dw_min) * g.halo_col_bytes + (tp.dh - g.dh_min) * 1024) >> 4);
            umma_x4<0>(d_tmem, a_lo0 + a0_16, a_hi, 2, b_lo0 + bres_16 + (uint32_t)tap * bblk_16, b_hi, b_step, g.idesc,
                       tap > 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == g.stages) { stage = 0; phase ^= 1; }
          umma_commit(&acc_full[acc]);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          continue;
        }
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait(&full_bar[stage], phase, g.err, ERR_TIMEOUT_FULL)) { failed = true; break; }
          tc_fence_after();
          const uint32_t sa_16 = stage0_16 + (uint32_t)stage * stage_16;
          const uint32_t sb_16 = g.b_res_bytes ? bres_16 + (uint32_t)it * bblk_16 : sa_16 + (CONV_A_BYTES >> 4);
          if (g.kind == 2)
            umma_x4<2>(d_tmem, a_lo0 + sa_16, a_hi, 2, b_lo0 + sb_16, b_hi, b_step, g.idesc, it > 0 ? 1u : 0u);
          else
            umma_x4<0>(d_tmem, a_lo0 + sa_16, a_hi, 2, b_lo0 + sb_16, b_hi, b_step, g.idesc, it > 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == g.stages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // Eight epilogue warps.  tcgen05.ld lets warp w touch tensor-memory lanes [32*(w%4), +32),
    // so two warps share each quarter of the tile's 128 pixels and take alternate column blocks.
    // Nothing in the store path synchronises across warps: each warp stages its own 32 pixels
    // x 64 channels (4 KB, 128-byte swizzle) and issues its own tensor-map store.
    const int quarter = warp & 3;
    const int colhalf = (warp - 2) >> 2;
    // two 4 KB staging buffers per warp: the next block is converted while the copy engine still reads the last one
    uint8_t* sbuf0 = stage_out + (warp - 2) * 4096 * g.epi_bufs;
    int sbuf_sel = 0;
    int acc = 0; uint32_t acc_phase = 0;
    const int esz = g.out_dtype == B200_F32 ? 4 : g.out_dtype == B200_I8 ? 1 : 2;
    const int rsz = g.res_dtype == B200_F32 ? 4 : 2;
    const bool has_coef = g.scale != nullptr || g.bias != nullptr;
    const int r = quarter * 32 + lane;
    // origin of this warp's 32 pixels inside the tile's pixel box (all extents are powers of two)
    const int w_off = (quarter * 32) % g.bw, h_off = ((quarter * 32) / g.bw) % g.bh, n_off = (quarter * 32) / (g.bw * g.bh);
    // Channel statistics (for a following batch norm): lane L keeps the running sum and sum of
    // squares of channels 2L, 2L+1 of each 64-channel block this warp stores, over all pixel
    // tiles of one output-channel tile, and adds them to the fp64 totals when that tile changes.
    float st_s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, st_q[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    int st_ct = -1;
    auto flush_stats = [&]() {
      if (st_ct < 0) return;
#pragma unroll
      for (int bi = 0; bi < 2; ++bi) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int ch = st_ct * g.tile_n + colhalf * 64 + bi * 128 + 2 * lane + e;
          if (colhalf * 64 + bi * 128 < g.tile_n && ch < g.Cout) {
            atomicAdd(g.stats + ch, (double)st_s[bi][e]);
            atomicAdd(g.stats + g.Cout + ch, (double)st_q[bi][e]);
          }
          st_s[bi][e] = 0.f; st_q[bi][e] = 0.f;
        }
      }
    };
    for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
      const int pt = tile % pix_tiles, ct = tile / pix_tiles;
      if (STATS && ct != st_ct) { flush_stats(); st_ct = ct; }
      const int q0 = (pt % g.tiles_q) * g.bw;
      const int p0 = ((pt / g.tiles_q) % g.tiles_p) * g.bh;
      const int n0 = (pt / (g.tiles_q * g.tiles_p)) * g.bni;
      const int co0 = ct * g.tile_n;
      const int q = q0 + r % g.bw, p = p0 + (r / g.bw) % g.bh, n = n0 + r / (g.bw * g.bh);
      const bool row_ok = q < g.Q && p < g.P && n < g.N;
      const long long off = (long long)n * g.o_sn + (long long)(p * g.o_mul_h + g.o_off_h) * g.o_sh +
                            (long long)(q * g.o_mul_w + g.o_off_w) * g.o_sw;
      const float* cs = coef;
      const float* cbias = cs + 256;
      if (has_coef) {
        // Every epilogue thread passes the barrier at the end of a tile after its last read of
        // the coefficients, so they can be overwritten here.
        for (int t = threadIdx.x - 64; t < g.tile_n; t += CONV_EPI_THREADS) {
          const int co = co0 + t;
          coef[t] = (g.scale && co < g.Cout) ? g.scale[co] : 1.f;
          coef[256 + t] = (g.bias && co < g.Cout) ? ld_scalar(g.bias, co, g.bias_dtype) : 0.f;
        }
        named_barrier(2, CONV_EPI_THREADS);
      }
      if (!mbar_wait(&acc_full[acc], acc_phase, g.err, ERR_TIMEOUT_TMEM_FULL)) { failed = true; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * 256 + ((uint32_t)(quarter * 32) << 16);

      // accumulator chunk (32 channels starting at tile column c) -> alpha, scale/bias, residual, activation
      auto finish = [&](const uint32_t (&rr)[32], int c, float (&v)[32]) {
        if (I8) {  // int32 accumulators of the int8 kind
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = (float)(int)rr[j];
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[j]);
        }
        if (GENERAL) {
          if (g.alpha != 1.f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= g.alpha;
          }
          if (has_coef) apply_coef(v, cs + c, cbias + c);
          const int cbase = co0 + c;
          if (g.residual && row_ok && cbase < g.Cout)
            add_residual(v, static_cast<const uint8_t*>(g.residual) + (off + cbase) * rsz, min(32, g.Cout - cbase), g.res_dtype);
          if (g.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
          }
        } else if (RES) {  // only a residual (a gradient that arrived over another path) is added
          const int cbase = co0 + c;
          if (row_ok && cbase < g.Cout)
            add_residual(v, static_cast<const uint8_t*>(g.residual) + (off + cbase) * rsz, min(32, g.Cout - cbase), g.res_dtype);
        }
        if (STATS && !row_ok) {
          // pixels outside the output are clipped by the store but must not count in the statistics
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
      };

      if (g.tma_store) {
        // not unrolled: the body is large and the epilogue warps share the instruction cache with the
        // producer and MMA roles
#pragma unroll 1
        for (int bi = 0; bi < 2; ++bi) {
          const int cb = colhalf * 64 + bi * 128;
          if (cb >= g.tile_n) break;
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
          // the two 32-column halves run through one copy of the code (the second half is moved into the
          // first half's registers): the loop is deliberately not unrolled to keep the kernel's hot code small
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            float v[32];
            uint32_t pk[16];
            finish(ra, cb + 32 * h, v);
            pack16(v, pk, g.out_dtype);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              *reinterpret_cast<uint4*>(srow + (((4 * h + k) ^ (lane & 7)) * 16)) = make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
#pragma unroll
            for (int j = 0; j < 32; ++j) ra[j] = rb[j];
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (STATS) {
            // Column sums over the 32 staged pixels (the rounded values that were stored; pixels
            // outside the tensor were zeroed above).
            // packed fp32 pairs: one add and one fma per two elements
            unsigned long long s2 = 0ull, q2 = 0ull;
#pragma unroll 8
            for (int rw = 0; rw < 32; ++rw) {
              const uint32_t w2 = *reinterpret_cast<const uint32_t*>(sbuf + rw * 128 + (((lane >> 2) ^ (rw & 7)) * 16) + (lane & 3) * 4);
              uint32_t lo, hi;
              if (g.out_dtype == B200_BF16) {
                lo = w2 << 16; hi = w2 & 0xffff0000u;
              } else {
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w2));
                lo = __float_as_uint(f2.x); hi = __float_as_uint(f2.y);
              }
              unsigned long long ab;
              asm("mov.b64 %0, {%1, %2};" : "=l"(ab) : "r"(lo), "r"(hi));
              asm("add.rn.f32x2 %0, %0, %1;" : "+l"(s2) : "l"(ab));
              asm("fma.rn.f32x2 %0, %1, %1, %0;" : "+l"(q2) : "l"(ab));
            }
            uint32_t s_lo, s_hi, q_lo, q_hi;
            asm("mov.b64 {%0, %1}, %2;" : "=r"(s_lo), "=r"(s_hi) : "l"(s2));
            asm("mov.b64 {%0, %1}, %2;" : "=r"(q_lo), "=r"(q_hi) : "l"(q2));
            const float s0 = __uint_as_float(s_lo), s1 = __uint_as_float(s_hi);
            const float q0s = __uint_as_float(q_lo), q1s = __uint_as_float(q_hi);
            // bi is a run-time loop index: select the accumulator set explicitly so that both stay in registers
            if (bi == 0) { st_s[0][0] += s0; st_s[0][1] += s1; st_q[0][0] += q0s; st_q[0][1] += q1s; }
            else { st_s[1][0] += s0; st_s[1][1] += s1; st_q[1][0] += q0s; st_q[1][1] += q1s; }
          }
          if (lane == 0) {
            // rows / channels outside the tensor are clipped by the store
            tma_store_4d(&maps.out, sbuf, co0 + cb, q0 + w_off, p0 + h_off, n0 + n_off);
            tma_store_commit();
          }
        }
      } else {
        for (int c = colhalf * 32; c < g.tile_n; c += 64) {
          uint32_t rr[32];
          tmem_ld32(t_addr + c, rr);
          tmem_ld_wait();
          const int cbase = co0 + c;
          if (!row_ok || cbase >= g.Cout) continue;
          const int valid = min(32, g.Cout - cbase);
          float v[32];
          finish(rr, c, v);
          uint8_t* op = static_cast<uint8_t*>(g.out) + (off + cbase) * esz;
          if (g.out_dtype == B200_I8) {
            // quantized for the consumer: four signed bytes per word
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint32_t w = 0;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float qv = fminf(fmaxf(rintf(v[4 * j + e] * g.out_qscale), -127.f), 127.f);
                w |= ((uint32_t)(int)qv & 0xffu) << (8 * e);
              }
              pk[j] = w;
            }
            if (valid == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
              reinterpret_cast<uint4*>(op)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              reinterpret_cast<uint4*>(op)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) op[j] = (uint8_t)(pk[j >> 2] >> ((j & 3) * 8));
            }
          } else if (g.out_dtype == B200_F32) {
            float* o = reinterpret_cast<float*>(op);
            if (valid == 32 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) o[j] = v[j];
            }
          } else {
            uint32_t pk[16];
            pack16(v, pk, g.out_dtype);
            uint16_t* o = reinterpret_cast<uint16_t*>(op);
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
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (has_coef) named_barrier(2, CONV_EPI_THREADS);
    }
    if (STATS) flush_stats();
    if (g.tma_store && lane == 0) tma_store_wait_all<0>();  // stores must be complete before shared memory goes away
  }

  if (*((volatile int*)g.err) != 0) {
    // give loads that may still be in flight time to land before shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ------------------------------------------------------------------------- wgrad
struct WgradArgs {
  int N, P, Q, Cin, Cout;
  int bw, bh, bni;               // pixel box, bw*bh*bni == 64
  int tiles_q, tiles_p, tiles_n; // pixel chunks
  int m_tiles;                   // ceil(Cout / 128)
  int n_blocks_total;            // ntaps * (Cin / 64)
  int n_blocks_per_tile;         // <= 4
  int n_tiles;
  int c_blocks;                  // Cin / 64
  int splits, chunks_per_split;
  int stages, ntaps;
  uint32_t idesc;
  B200ConvTap taps[B200_CONV_MAX_TAPS];
  float* dw_acc;
  long long dw_ld;               // wtaps * Cin
  int* err;
};
struct WgradMaps {
  CUtensorMap x[B200_CONV_MAX_MAPS];
  CUtensorMap dy;
  CUtensorMap dw;  // fp32 [Cout][wtaps * Cin] accumulation buffer, box 32 x 32
};

__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_wgrad_kernel(const __grid_constant__ WgradMaps maps, const __grid_constant__ WgradArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // stage: A = 2 blocks (128 out-channels) x (64 pixels x 128 B); B = n_blocks x 8 KB
  const int blk_bytes = 64 * 128;
  const int stage_bytes = 2 * blk_bytes + g.n_blocks_per_tile * blk_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)g.stages * stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + CONV_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * CONV_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);
  // four 4 KB staging buffers (32 channels x 32 fp32 columns, 128-byte swizzle), one per epilogue warp
  uint8_t* stage_out = reinterpret_cast<uint8_t*>(bars) + 1024;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_full[0], 1);
    mbar_fence_init();
    tma_prefetch_desc(&maps.dy);
    tma_prefetch_desc(&maps.dw);
    tma_prefetch_desc(&maps.x[0]);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // One work item per CTA: (m tile, n tile, split).
  const int item = blockIdx.x;
  const int split = item % g.splits;
  const int nt = (item / g.splits) % g.n_tiles;
  const int mt = item / (g.splits * g.n_tiles);
  const int total_chunks = g.tiles_q * g.tiles_p * g.tiles_n;
  const int chunk_begin = split * g.chunks_per_split;
  const int chunk_end = min(total_chunks, chunk_begin + g.chunks_per_split);
  const int nb0 = nt * g.n_blocks_per_tile;
  const int nblk = min(g.n_blocks_per_tile, g.n_blocks_total - nb0);
  const int co0 = mt * 128;
  bool failed = false;

  if (warp == 0) {
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0; uint32_t phase = 0;
      for (int ch = chunk_begin; ch < chunk_end; ++ch) {
        const int q0 = (ch % g.tiles_q) * g.bw;
        const int p0 = ((ch / g.tiles_q) % g.tiles_p) * g.bh;
        const int n0 = (ch / (g.tiles_q * g.tiles_p)) * g.bni;
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, g.err, ERR_TIMEOUT_EMPTY)) { failed = true; break; }
        mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)((2 + nblk) * blk_bytes));
        uint8_t* sa = smem + (size_t)stage * stage_bytes;
        tma_load_4d(sa, &maps.dy, &full_bar[stage], co0, q0, p0, n0);
        tma_load_4d(sa + blk_bytes, &maps.dy, &full_bar[stage], co0 + 64, q0, p0, n0);
        for (int j = 0; j < nblk; ++j) {
          const int nb = nb0 + j;
          const int tap = nb / g.c_blocks, cb = nb - tap * g.c_blocks;
          const B200ConvTap tp = g.taps[tap];
          tma_load_4d(sa + (2 + j) * blk_bytes, &maps.x[tp.map], &full_bar[stage], cb * 64, q0 + tp.dw, p0 + tp.dh, n0);
        }
        if (++stage == g.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0; uint32_t phase = 0;
      uint32_t d_lo0, d_hi;
      split_desc(make_smem_desc_sw128(0, blk_bytes, 1024), &d_lo0, &d_hi);
      const uint32_t smem0_16 = smem_u32(smem) >> 4, stage_16 = (uint32_t)stage_bytes >> 4;
      for (int ch = chunk_begin; ch < chunk_end; ++ch) {
        if (!mbar_wait(&full_bar[stage], phase, g.err, ERR_TIMEOUT_FULL)) { failed = true; break; }
        tc_fence_after();
        // MN-major operands: 16 pixels (K) per MMA = 2048 B; blocks of 64 channels 8 KB apart.
        const uint32_t sa_16 = smem0_16 + (uint32_t)stage * stage_16;
        umma_x4<0>(tmem_base, d_lo0 + sa_16, d_hi, 128, d_lo0 + sa_16 + (uint32_t)(2 * blk_bytes >> 4), d_hi, 128, g.idesc,
                   ch > chunk_begin ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == g.stages) { stage = 0; phase ^= 1; }
      }
      if (!failed) umma_commit(&acc_full[0]);
    }
  } else if (chunk_end > chunk_begin) {
    const int quarter = warp & 3;
    if (mbar_wait(&acc_full[0], 0, g.err, ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      // Each warp adds its 32 output channels x 32 columns at a time into the fp32 buffer with one
      // tensor-map reduction (full 128-byte lines) instead of per-thread 16-byte atomics.  Channels past
      // Cout and columns past the row end are clipped; columns past Cin inside a tap slot are zero
      // (their input channels were zero filled), so adding them into the next tap's columns is harmless.
      uint8_t* sbuf = stage_out + (warp - 2) * 4096;
      const int ncols = nblk * 64;
      for (int c = 0; c < ncols; c += 32) {
        uint32_t rr[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, rr);
        tmem_ld_wait();
        // flattened column -> (tap slot, channel): blocks never straddle a tap
        const int nb = nb0 + c / 64;
        const int tap = nb / g.c_blocks, cb = nb - tap * g.c_blocks;
        const int ci = cb * 64 + (c % 64);
        if (ci >= g.Cin) continue;  // warp-uniform
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        uint8_t* srow = sbuf + lane * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          *reinterpret_cast<uint4*>(srow + ((k ^ (lane & 7)) * 16)) = make_uint4(rr[4 * k], rr[4 * k + 1], rr[4 * k + 2], rr[4 * k + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_2d(&maps.dw, sbuf, g.taps[tap].wtap * g.Cin + ci, co0 + quarter * 32);
          tma_store_commit();
        }
      }
      if (lane == 0) tma_store_wait_all<0>();
    }
  }
  if (*((volatile int*)g.err) != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// Choose a power-of-two pixel box bw*bh*bni == total that wastes the fewest rows.
static void pick_box(int total, int N, int P, int Q, int* bw, int* bh, int* bni) {
  double best = 1e30;
  for (int w = 1; w <= total; w *= 2) {
    for (int h = 1; w * h <= total; h *= 2) {
      const int n = total / (w * h);
      if (w > 256 || h > 256 || n > 256) continue;
      const double tiles = (double)((Q + w - 1) / w) * ((P + h - 1) / h) * ((N + n - 1) / n);
      const double cost = tiles - 1e-3 * w - 1e-5 * h;  // ties: wider, then taller boxes
      if (cost < best) { best = cost; *bw = w; *bh = h; *bni = n; }
    }
  }
}

static int encode_view(CUtensorMap* m, const B200ConvView& v, CUtensorMapDataType dt, int boxc, int bw, int bh, int bni,
                       int es = 2) {
  uint64_t dims[4] = {(uint64_t)v.dims[0], (uint64_t)v.dims[1], (uint64_t)v.dims[2], (uint64_t)v.dims[3]};
  uint64_t str[3] = {(uint64_t)v.strides[0] * es, (uint64_t)v.strides[1] * es, (uint64_t)v.strides[2] * es};
  uint32_t box[4] = {(uint32_t)boxc, (uint32_t)bw, (uint32_t)bh, (uint32_t)bni};
  return encode_tiled(m, dt, 4, v.base, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
}

static int set_smem_attr_once(const void* fn, int dev, bool* done) {
  if (done[dev & 63]) return 0;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return (int)e;
  done[dev & 63] = true;
  return 0;
}

}  // namespace b200

// A pointwise (single centred tap) convolution over densely packed pixels is a plain GEMM:
// fold batch, rows and columns into one pixel axis so that every A tile is one contiguous
// 128-pixel run for the copy engine instead of a small 3-D box.
static bool flatten_pointwise(B200ConvParams* q) {
  if (q->ntaps != 1 || q->num_views != 1 || q->taps[0].dh != 0 || q->taps[0].dw != 0 || q->taps[0].map != 0) return false;
  const B200ConvView& v = q->views[0];
  if (v.dims[1] != q->Q || v.dims[2] != q->P || v.dims[3] != q->N) return false;
  if (v.strides[1] != v.strides[0] * v.dims[1] || v.strides[2] != v.strides[1] * v.dims[2]) return false;
  if (q->o_mul_h != 1 || q->o_mul_w != 1 || q->o_off_h != 0 || q->o_off_w != 0) return false;
  if (q->o_sh != q->o_sw * q->Q || q->o_sn != q->o_sh * q->P) return false;
  const long long pixels = (long long)q->N * q->P * q->Q;
  if (pixels > 0x7fffffffLL) return false;
  q->views[0].dims[1] = pixels; q->views[0].dims[2] = 1; q->views[0].dims[3] = 1;
  q->views[0].strides[1] = v.strides[0] * pixels; q->views[0].strides[2] = v.strides[0] * pixels;
  q->Q = (int)pixels; q->P = 1; q->N = 1;
  q->o_sh = q->o_sw * pixels; q->o_sn = q->o_sh;
  return true;
}

extern "C" int b200_conv_fprop(const B200ConvParams* p_in, void* stream) {
  using namespace b200;
  if (p_in->N <= 0 || p_in->P <= 0 || p_in->Q <= 0 || p_in->Cout <= 0) return 0;
  B200ConvParams flat = *p_in;
  flatten_pointwise(&flat);
  const B200ConvParams* p = &flat;
  if (p->ntaps <= 0 || p->ntaps > B200_CONV_MAX_TAPS || p->num_views <= 0 || p->num_views > B200_CONV_MAX_MAPS)
    return (int)cudaErrorInvalidValue;
  const int es = p->ab_dtype == B200_I8 ? 1 : 2;
  if ((p->Cin * es) % 16 || p->ab_dtype == B200_F32) return (int)cudaErrorInvalidValue;
  const CUtensorMapDataType dt = p->ab_dtype == B200_I8    ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : p->ab_dtype == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                           : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUtensorMapDataType out_dt = p->out_dtype == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);

  ConvArgs g{};
  g.N = p->N; g.P = p->P; g.Q = p->Q; g.Cin = p->Cin; g.Cout = p->Cout;
  pick_box(128, p->N, p->P, p->Q, &g.bw, &g.bh, &g.bni);
  g.tiles_q = (p->Q + g.bw - 1) / g.bw;
  g.tiles_p = (p->P + g.bh - 1) / g.bh;
  g.tiles_n = (p->N + g.bni - 1) / g.bni;
  long pix_tiles = (long)g.tiles_q * g.tiles_p * g.tiles_n;
  if (p->tile_n > 0) {
    g.tile_n = p->tile_n;
  } else {
    // widest tile that still leaves every SM with work; never wider than Cout needs
    int tn = 256;
    while (tn > 32 && (tn / 2 >= p->Cout || (pix_tiles * ((p->Cout + tn - 1) / tn) < sms && tn > 64))) tn /= 2;
    if (p->Cout <= 32) tn = 32;
    g.tile_n = tn;
  }
  g.b_mn = p->w_stride_n == 1 && p->w_stride_k != 1;
  if (g.b_mn && g.tile_n < 64) g.tile_n = 64;
  if (g.tile_n % 32 || g.tile_n > 256 || (g.b_mn && g.tile_n % 64)) return (int)cudaErrorInvalidValue;
  g.tiles_co = (p->Cout + g.tile_n - 1) / g.tile_n;
  g.cblk = 128 / es;
  g.kind = es == 1 ? 2 : 0;
  if (g.kind == 2 && g.b_mn) return (int)cudaErrorInvalidValue;
  g.c_blocks = (p->Cin + g.cblk - 1) / g.cblk;
  g.ntaps = p->ntaps;
  for (int i = 0; i < p->ntaps; ++i) g.taps[i] = p->taps[i];
  const int fmt = (p->ab_dtype == B200_BF16 || p->ab_dtype == B200_I8) ? 1 : 0;
  g.idesc = make_idesc(g.kind == 2 ? 2 : 1, fmt, fmt, 0, g.b_mn, 128, g.tile_n);
  g.out = p->out; g.out_dtype = p->out_dtype;
  g.o_sn = p->o_sn; g.o_sh = p->o_sh; g.o_sw = p->o_sw;
  g.o_mul_h = p->o_mul_h; g.o_off_h = p->o_off_h; g.o_mul_w = p->o_mul_w; g.o_off_w = p->o_off_w;
  g.scale = static_cast<const float*>(p->scale);
  g.bias = p->bias; g.bias_dtype = p->bias_dtype;
  g.residual = p->residual; g.res_dtype = p->res_dtype; g.act = p->act;
  g.stats = static_cast<double*>(p->stats);
  g.alpha = p->alpha == 0.f ? 1.f : p->alpha;
  g.err = error_flag_ptr();
  if (!g.err) return (int)cudaErrorInvalidDevice;
  g.out_qscale = p->out_qscale;
  if (p->out_dtype == B200_I8 && !(p->out_qscale > 0.f)) return (int)cudaErrorInvalidValue;
  g.tma_store = (p->out_dtype != B200_F32 && p->out_dtype != B200_I8 && g.tile_n % 64 == 0 && p->Cout % 8 == 0) ? 1 : 0;
  g.coef_bytes = (p->scale || p->bias) ? 2048 : 0;
  // one 4 KB staging buffer per epilogue warp; a second one is added below when the pipeline keeps enough stages
  g.epi_bufs = 1;
  int smem_cap = 227 * 1024 - 2048 - g.coef_bytes - (g.tma_store ? 32768 : 0);
  // Weights of one output-channel tile (every tap and channel block) stay in shared memory when
  // they are small and each CTA reuses them over several pixel tiles; the stages then hold only
  // activations, which puts more of them in flight.
  if (g.stats && !g.tma_store) return (int)cudaErrorInvalidValue;  // statistics come from the staged tiles
  const long b_tile_bytes = (long)g.ntaps * g.c_blocks * g.tile_n * 128;
  g.b_res_bytes = (b_tile_bytes <= 96 * 1024 && pix_tiles >= 2L * sms) ? (int)b_tile_bytes : 0;
  // Halo mode: see ConvArgs.  The pixel box is fixed to 8 x 16 x 1 so that the 16 row groups of the
  // MMA's A operand are the 16 image rows of the tile.
  g.halo = 0;
  if (g.b_res_bytes && g.c_blocks == 1 && g.ntaps > 1 && p->num_views == 1 && g.kind == 0 && p->Q >= 8 && p->P >= 8) {
    int dw0 = 1 << 20, dw1 = -(1 << 20), dh0 = 1 << 20, dh1 = -(1 << 20);
    bool one_view = true;
    for (int i = 0; i < p->ntaps; ++i) {
      dw0 = std::min<int>(dw0, p->taps[i].dw); dw1 = std::max<int>(dw1, p->taps[i].dw);
      dh0 = std::min<int>(dh0, p->taps[i].dh); dh1 = std::max<int>(dh1, p->taps[i].dh);
      one_view = one_view && p->taps[i].map == 0;
    }
    const int hh = 16 + dh1 - dh0;
    if (one_view && hh <= 24 && dw1 - dw0 < 4) {
      g.halo = 1; g.halo_h = hh; g.dw_min = dw0; g.dh_min = dh0;
      g.halo_ndw = dw1 - dw0 + 1; g.halo_col_bytes = 8 * hh * 128;
      g.halo_stage_bytes = g.halo_ndw * g.halo_col_bytes;
      g.bw = 8; g.bh = 16; g.bni = 1;
      g.tiles_q = (p->Q + 7) / 8; g.tiles_p = (p->P + 15) / 16; g.tiles_n = p->N;
      pix_tiles = (long)g.tiles_q * g.tiles_p * g.tiles_n;
    }
  }
  const int stage_bytes = g.halo ? g.halo_stage_bytes : CONV_A_BYTES + (g.b_res_bytes ? 0 : g.tile_n * 128);
  if (g.tma_store && (smem_cap - 32768 - g.b_res_bytes) / stage_bytes >= (g.halo ? 2 : 4)) {
    g.epi_bufs = 2;
    smem_cap -= 32768;
  }
  g.stages = (smem_cap - g.b_res_bytes) / stage_bytes;
  if (g.stages > CONV_MAX_STAGES) g.stages = CONV_MAX_STAGES;
  if (g.stages < 2) g.stages = 2;

  ConvMaps maps;
  maps.out = CUtensorMap{};
  if (g.tma_store) {
    B200ConvView ov;
    ov.base = static_cast<const char*>(p->out) + ((long long)p->o_off_h * p->o_sh + (long long)p->o_off_w * p->o_sw) * 2;
    ov.dims[0] = p->Cout; ov.dims[1] = p->Q; ov.dims[2] = p->P; ov.dims[3] = p->N;
    ov.strides[0] = p->o_sw * p->o_mul_w; ov.strides[1] = p->o_sh * p->o_mul_h; ov.strides[2] = p->o_sn;
    // each epilogue warp stores its own 32 pixels: the first 32 rows of the (bw, bh, bni) box order
    const int sw = g.bw < 32 ? g.bw : 32;
    const int sh = g.bh < 32 / sw ? g.bh : 32 / sw;
    const int sn = 32 / (sw * sh);
    int rc = encode_view(&maps.out, ov, out_dt, 64, sw, sh, sn);
    if (rc) return rc;
  }
  for (int i = 0; i < p->num_views; ++i) {
    int rc = encode_view(&maps.a[i], p->views[i], dt, g.cblk, g.bw, g.bh, g.bni, es);
    if (rc) return rc;
  }
  for (int i = p->num_views; i < B200_CONV_MAX_MAPS; ++i) maps.a[i] = maps.a[0];
  if (g.halo) {
    int rc = encode_view(&maps.a[1], p->views[0], dt, g.cblk, 8, g.halo_h, 1, es);
    if (rc) return rc;
  }
  {
    int rc;
    if (!g.b_mn) {
      uint64_t dims[3] = {(uint64_t)p->Cin, (uint64_t)p->Cout, (uint64_t)p->wtaps};
      uint64_t str[2] = {(uint64_t)p->w_stride_n * es, (uint64_t)p->w_stride_tap * es};
      uint32_t box[3] = {(uint32_t)g.cblk, (uint32_t)g.tile_n, 1};
      rc = encode_tiled(&maps.w, dt, 3, p->weight, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      uint64_t dims[3] = {(uint64_t)p->Cout, (uint64_t)p->Cin, (uint64_t)p->wtaps};
      uint64_t str[2] = {(uint64_t)p->w_stride_k * 2, (uint64_t)p->w_stride_tap * 2};
      uint32_t box[3] = {64, 64, 1};
      rc = encode_tiled(&maps.w, dt, 3, p->weight, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc) return rc;
  }
  const bool general = g.kind == 2 || g.alpha != 1.f || g.scale || g.bias || g.act != 0;
  const bool stats = g.stats != nullptr;
  const bool res = g.residual != nullptr;
  typedef void (*Kernel)(const ConvMaps, const ConvArgs);
  const bool i8 = g.kind == 2;
  Kernel kernel;
  if (i8) kernel = stats ? conv_fprop_kernel<true, true, true, false> : conv_fprop_kernel<true, false, true, false>;
  else if (general) kernel = stats ? conv_fprop_kernel<true, true, false, false> : conv_fprop_kernel<true, false, false, false>;
  else if (res) kernel = stats ? conv_fprop_kernel<false, true, false, true> : conv_fprop_kernel<false, false, false, true>;
  else kernel = stats ? conv_fprop_kernel<false, true, false, false> : conv_fprop_kernel<false, false, false, false>;
  int rc = 0;
  {
    static bool done[16][64] = {};
    rc = set_smem_attr_once((const void*)kernel, dev, done[(i8 ? 8 : 0) + (general ? 4 : 0) + (res ? 2 : 0) + (stats ? 1 : 0)]);
  }
  if (rc) return rc;
  const size_t smem = 1024 /*align*/ + (size_t)g.b_res_bytes + (size_t)g.stages * stage_bytes + 1024 /*barriers*/ +
                      g.coef_bytes + (g.tma_store ? 32768 * g.epi_bufs : 0);
  const long total_tiles = pix_tiles * g.tiles_co;
  const int ctas = (int)(total_tiles < sms ? total_tiles : sms);
  kernel<<<ctas, CONV_FPROP_THREADS, smem, (cudaStream_t)stream>>>(maps, g);
  return (int)cudaGetLastError();
}

namespace b200 {
bool try_wgrad_halo(const B200ConvWgradParams* p, void* stream, int* rc);  // conv_wgrad_halo.cu
}

extern "C" int b200_conv_wgrad(const B200ConvWgradParams* p, void* stream) {
  using namespace b200;
  if (p->N <= 0 || p->P <= 0 || p->Q <= 0 || p->Cout <= 0 || p->Cin <= 0) return 0;
  if (p->ntaps <= 0 || p->ntaps > B200_CONV_MAX_TAPS || p->num_views <= 0 || p->num_views > B200_CONV_MAX_MAPS)
    return (int)cudaErrorInvalidValue;
  {
    // stride-1 multi-tap filters: shared activation windows (about half the L2 -> SM traffic)
    int rc = 0;
    if (try_wgrad_halo(p, stream, &rc)) return rc;
  }
  if (p->Cin % 8 || p->Cout % 8 || p->ab_dtype == B200_F32) return (int)cudaErrorInvalidValue;
  const CUtensorMapDataType dt = p->ab_dtype == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);

  WgradArgs g{};
  g.N = p->N; g.P = p->P; g.Q = p->Q; g.Cin = p->Cin; g.Cout = p->Cout;
  pick_box(64, p->N, p->P, p->Q, &g.bw, &g.bh, &g.bni);
  g.tiles_q = (p->Q + g.bw - 1) / g.bw;
  g.tiles_p = (p->P + g.bh - 1) / g.bh;
  g.tiles_n = (p->N + g.bni - 1) / g.bni;
  g.m_tiles = (p->Cout + 127) / 128;
  g.c_blocks = (p->Cin + 63) / 64;
  g.n_blocks_total = p->ntaps * g.c_blocks;
  g.n_blocks_per_tile = g.n_blocks_total < 4 ? g.n_blocks_total : 4;
  g.n_tiles = (g.n_blocks_total + g.n_blocks_per_tile - 1) / g.n_blocks_per_tile;
  const long chunks = (long)g.tiles_q * g.tiles_p * g.tiles_n;
  const long base_items = (long)g.m_tiles * g.n_tiles;
  int splits = p->splits;
  if (splits <= 0) {
    // one wave of CTAs: a second wave doubles the partial tiles that have to be added into the buffer and
    // measured slower on every layer shape (e.g. 256x14x14 3x3: 138 us -> 103 us)
    splits = (int)(sms / base_items);
    const long max_splits = (chunks + 15) / 16;                // at least 16 chunks per split
    if (splits > max_splits) splits = (int)max_splits;
    if (splits < 1) splits = 1;
  }
  if (splits > chunks) splits = (int)chunks;
  g.chunks_per_split = (int)((chunks + splits - 1) / splits);
  g.splits = (int)((chunks + g.chunks_per_split - 1) / g.chunks_per_split);
  g.ntaps = p->ntaps;
  for (int i = 0; i < p->ntaps; ++i) g.taps[i] = p->taps[i];
  const int fmt = p->ab_dtype == B200_BF16 ? 1 : 0;
  g.idesc = make_idesc(1, fmt, fmt, 1, 1, 128, g.n_blocks_per_tile * 64);
  g.dw_acc = p->dw_acc;
  g.dw_ld = (long long)p->wtaps * p->Cin;
  g.err = error_flag_ptr();
  if (!g.err) return (int)cudaErrorInvalidDevice;
  const int stage_bytes = (2 + g.n_blocks_per_tile) * 64 * 128;
  g.stages = (227 * 1024 - 2048 - 4 * 4096 - 1024) / stage_bytes;
  if (g.stages > CONV_MAX_STAGES) g.stages = CONV_MAX_STAGES;

  WgradMaps maps;
  for (int i = 0; i < p->num_views; ++i) {
    int rc = encode_view(&maps.x[i], p->views[i], dt, 64, g.bw, g.bh, g.bni);
    if (rc) return rc;
  }
  for (int i = p->num_views; i < B200_CONV_MAX_MAPS; ++i) maps.x[i] = maps.x[0];
  {
    B200ConvView v;
    v.base = p->dy;
    v.dims[0] = p->Cout; v.dims[1] = p->Q; v.dims[2] = p->P; v.dims[3] = p->N;
    v.strides[0] = p->dy_sw; v.strides[1] = p->dy_sh; v.strides[2] = p->dy_sn;
    int rc = encode_view(&maps.dy, v, dt, 64, g.bw, g.bh, g.bni);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)g.dw_ld, (uint64_t)p->Cout};
    uint64_t str[1] = {(uint64_t)g.dw_ld * 4};
    uint32_t box[2] = {32, 32};
    int rc = encode_tiled(&maps.dw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p->dw_acc, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  static bool attr_done[64] = {false};
  int rc = set_smem_attr_once((const void*)conv_wgrad_kernel, dev, attr_done);
  if (rc) return rc;
  const size_t smem = (size_t)g.stages * stage_bytes + 1024 /*align*/ + 1024 /*barriers*/ + 4 * 4096 /*staging*/;
  const long items = base_items * g.splits;
  conv_wgrad_kernel<<<(int)items, CONV_THREADS, smem, (cudaStream_t)stream>>>(maps, g);
  return (int)cudaGetLastError();
}
