// Weight gradient of stride-1 multi-tap convolutions (3x3 and the like) with shared activation windows.
//
// dW[co][tap][ci] = sum over pixels dy[pix][co] * x[pix + tap][ci] as a GEMM with M = 128 output channels,
// K = pixels, N = (vertical taps) x (input-channel blocks).  The plain weight-gradient kernel loads one
// activation tile per (tap, channel block), so every activation crosses L2 -> shared memory nine times for a
// 3x3 filter and once more per output-channel tile.  Here one work item owns ONE horizontal tap offset dw and
// loads, per pixel chunk (8 wide, bh high, bni images), a single column tile of 8 x (bh + 2) pixels per channel
// block; the three vertical taps are windows of that tile shifted down by whole pixel rows.  A pixel row of 8
// pixels x 64 channels is exactly one 1024-byte swizzle repeat, so every window starts on a repeat boundary, and
// the three windows are one MN-major B operand of N = 192 whose 64-column blocks lie 1024 bytes apart (the
// descriptor's leading-dimension offset), i.e. they overlap in shared memory.  With two channel blocks per item
// the accumulator is 128 x 384 fp32 in tensor memory.  L2 -> SM traffic drops from
// (128 + 256) * 2 bytes per pixel and 128 x 256 tile to (128 * 2 + 2 * 64 * 2 * (bh + 2) / bh) bytes per pixel
// and 128 x 384 tile: about 2x less on ResNet's 3x3 layers.
//
// Replaces cnnlConvolutionBackwardFilter of the reference for these shapes
// (torch_mlu/csrc/aten/operators/cnnl/internal/convolution_float_backward_internal.cpp:162).
#include <algorithm>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"
#include "tcgen05.cuh"
#include "tma_util.cuh"

namespace b200 {

constexpr int WH_THREADS = 192;   // TMA warp, MMA warp, 4 epilogue warps
constexpr int WH_MAX_STAGES = 8;
constexpr int WH_MAX_STEPS = 8;   // K steps of 16 pixels per chunk (chunks hold at most 128 pixels)

struct WgradHaloArgs {
  int N, P, Q, Cin, Cout;
  int bh, bni, rows;              // chunk = 8 x bh x bni pixels = `rows` pixel rows of 8
  int tiles_q, tiles_p, tiles_n;
  int m_tiles, c_blocks, c_groups, ncb;
  int ndw, ndh, dw_min, dh_min;
  int splits, chunks_per_split, stages;
  int a_blk_bytes;                // rows * 1024: one 64-channel block of dy
  int col_bytes;                  // bni * (bh + ndh - 1) * 1024: one activation column tile
  int stage_bytes;
  int sep_mma;                    // 1: one N = 64 MMA per (vertical tap, channel block) instead of one N = ndh * 64
  uint32_t idesc;
  short wtap[4][4];               // [dw - dw_min][dh - dh_min] -> weight tap slot, -1 = no such tap
  float* dw_acc;
  long long dw_ld;
  int* err;
};
struct WgradHaloMaps {
  CUtensorMap x, dy, dw;
};

__global__ void __launch_bounds__(WH_THREADS, 1)
conv_wgrad_halo_kernel(const __grid_constant__ WgradHaloMaps maps, const __grid_constant__ WgradHaloArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)g.stages * g.stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + WH_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * WH_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);
  // per K step: offset of the first pixel row inside a column tile (16-byte units) and the descriptor high word
  // (it carries the distance to the second pixel row, which is larger when the step straddles two images)
  uint32_t* step_b_off = reinterpret_cast<uint32_t*>(bars) + 64;
  uint32_t* step_b_hi = step_b_off + WH_MAX_STEPS;
  uint8_t* stage_out = reinterpret_cast<uint8_t*>(bars) + 1024;  // 4 warps x 2 buffers x 4 KB
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int steps = g.rows >> 1;
  const int tile_rows = g.bh + g.ndh - 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_full[0], 1);
    mbar_fence_init();
    tma_prefetch_desc(&maps.dy);
    tma_prefetch_desc(&maps.dw);
    tma_prefetch_desc(&maps.x);
    for (int s = 0; s < steps; ++s) {
      const int g0 = 2 * s, g1 = 2 * s + 1;
      const int o0 = (g0 / g.bh) * tile_rows + g0 % g.bh, o1 = (g1 / g.bh) * tile_rows + g1 % g.bh;
      uint32_t lo, hi;
      split_desc(make_smem_desc_sw128(0, 1024, (uint32_t)(o1 - o0) * 1024u), &lo, &hi);
      step_b_off[s] = (uint32_t)o0 * 64u;  // rows of 1024 bytes in 16-byte units
      step_b_hi[s] = hi;
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // work item: (output-channel tile, horizontal tap offset, channel-block group, pixel split)
  int item = blockIdx.x;
  const int split = item % g.splits; item /= g.splits;
  const int cg = item % g.c_groups; item /= g.c_groups;
  const int dwi = item % g.ndw;
  const int mt = item / g.ndw;
  const int co0 = mt * 128;
  const int cb0 = cg * g.ncb;
  const int ncb = min(g.ncb, g.c_blocks - cb0);
  const int total_chunks = g.tiles_q * g.tiles_p * g.tiles_n;
  const int chunk_begin = split * g.chunks_per_split;
  const int chunk_end = min(total_chunks, chunk_begin + g.chunks_per_split);
  bool failed = false;

  if (warp == 0) {
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0; uint32_t phase = 0;
      const uint32_t tx = (uint32_t)(2 * g.a_blk_bytes + ncb * g.col_bytes);
      for (int ch = chunk_begin; ch < chunk_end; ++ch) {
        const int q0 = (ch % g.tiles_q) * 8;
        const int p0 = ((ch / g.tiles_q) % g.tiles_p) * g.bh;
        const int n0 = (ch / (g.tiles_q * g.tiles_p)) * g.bni;
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, g.err, ERR_TIMEOUT_EMPTY)) { failed = true; break; }
        mbar_arrive_expect_tx(&full_bar[stage], tx);
        uint8_t* sa = smem + (size_t)stage * g.stage_bytes;
        tma_load_4d(sa, &maps.dy, &full_bar[stage], co0, q0, p0, n0);
        tma_load_4d(sa + g.a_blk_bytes, &maps.dy, &full_bar[stage], co0 + 64, q0, p0, n0);  // zero filled past Cout
        for (int j = 0; j < ncb; ++j)
          tma_load_4d(sa + 2 * g.a_blk_bytes + j * g.col_bytes, &maps.x, &full_bar[stage], (cb0 + j) * 64,
                      q0 + g.dw_min + dwi, p0 + g.dh_min, n0);
        if (++stage == g.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {  // one elected lane of the converged warp: the compiler keeps the issue path uniform
      int stage = 0; uint32_t phase = 0;
      uint32_t a_lo0, a_hi, b_lo0, b_hi_unused;
      split_desc(make_smem_desc_sw128(0, (uint32_t)g.a_blk_bytes, 1024), &a_lo0, &a_hi);
      split_desc(make_smem_desc_sw128(0, 1024, 1024), &b_lo0, &b_hi_unused);
      const uint32_t smem0_16 = smem_u32(smem) >> 4, stage_16 = (uint32_t)g.stage_bytes >> 4;
      const uint32_t a_blk2_16 = (uint32_t)(2 * g.a_blk_bytes) >> 4, col_16 = (uint32_t)g.col_bytes >> 4;
      const int ncols_j = g.ndh * 64;
      for (int ch = chunk_begin; ch < chunk_end; ++ch) {
        if (!mbar_wait(&full_bar[stage], phase, g.err, ERR_TIMEOUT_FULL)) { failed = true; break; }
        tc_fence_after();
        const uint32_t sa_16 = smem0_16 + (uint32_t)stage * stage_16;
        for (int s = 0; s < steps; ++s) {
          const uint32_t acc = (ch > chunk_begin || s > 0) ? 1u : 0u;
          uint64_t ad;
          asm("mov.b64 %0, {%1, %2};" : "=l"(ad) : "r"(a_lo0 + sa_16 + (uint32_t)s * 128u), "r"(a_hi));
          const uint32_t boff = step_b_off[s], bhi = step_b_hi[s];
          for (int j = 0; j < ncb; ++j) {
            const uint32_t b_lo = b_lo0 + sa_16 + a_blk2_16 + (uint32_t)j * col_16 + boff;
            if (!g.sep_mma) {
              uint64_t bd;
              asm("mov.b64 %0, {%1, %2};" : "=l"(bd) : "r"(b_lo), "r"(bhi));
              umma_f16(tmem_base + (uint32_t)(j * ncols_j), ad, bd, g.idesc, acc);
            } else {
              for (int t = 0; t < g.ndh; ++t) {
                uint64_t bd;
                asm("mov.b64 %0, {%1, %2};" : "=l"(bd) : "r"(b_lo + (uint32_t)t * 64u), "r"(bhi));
                umma_f16(tmem_base + (uint32_t)(j * ncols_j + t * 64), ad, bd, g.idesc, acc);
              }
            }
          }
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == g.stages) { stage = 0; phase ^= 1; }
      }
      if (!failed) umma_commit(&acc_full[0]);
    }
  } else if (chunk_end > chunk_begin) {
    const int quarter = warp & 3;
    if (mbar_wait(&acc_full[0], 0, g.err, ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      // 32 output channels x 32 columns per tensor-map reduce-add; two staging buffers per warp so that the next
      // block is converted while the previous one is still being read by the copy engine
      uint8_t* sbuf0 = stage_out + (warp - 2) * 8192;
      const int ncols = ncb * g.ndh * 64;
      int buf = 0;
      for (int c = 0; c < ncols; c += 32) {
        const int blk = c >> 6;
        const int j = blk / g.ndh, t = blk - j * g.ndh;
        const int tap = g.wtap[dwi][t];
        if (tap < 0 || co0 + quarter * 32 >= g.Cout) continue;  // warp-uniform: no such tap / rows past Cout
        uint32_t rr[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, rr);
        tmem_ld_wait();
        if (lane == 0) tma_store_wait_read<1>();  // the buffer written two blocks ago has been read
        __syncwarp();
        uint8_t* sbuf = sbuf0 + buf * 4096;
        uint8_t* srow = sbuf + lane * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          *reinterpret_cast<uint4*>(srow + ((k ^ (lane & 7)) * 16)) = make_uint4(rr[4 * k], rr[4 * k + 1], rr[4 * k + 2], rr[4 * k + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int ci = (cb0 + j) * 64 + (c & 63);
          tma_reduce_add_2d(&maps.dw, sbuf, tap * g.Cin + ci, co0 + quarter * 32);
          tma_store_commit();
        }
        buf ^= 1;
      }
      if (lane == 0) tma_store_wait_all<0>();
    }
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

// 0 off, 1 on (default), 2 on with separate N = 64 MMAs; CATCH_B200_WGRAD_HALO sets the initial value
static int g_halo_mode = [] {
  const char* e = std::getenv("CATCH_B200_WGRAD_HALO");
  return e ? std::atoi(e) : 1;
}();

// Returns true when the halo kernel took the problem (*rc holds the launch result).
bool try_wgrad_halo(const B200ConvWgradParams* p, void* stream, int* rc) {
  const int mode = g_halo_mode;
  if (mode == 0) return false;
  if (p->num_views != 1 || p->ntaps < 2 || p->Cin % 64 || p->Cout % 8 || p->ab_dtype == B200_F32) return false;
  int dw0 = 1 << 20, dw1 = -(1 << 20), dh0 = 1 << 20, dh1 = -(1 << 20);
  for (int i = 0; i < p->ntaps; ++i) {
    if (p->taps[i].map != 0) return false;
    dw0 = std::min<int>(dw0, p->taps[i].dw); dw1 = std::max<int>(dw1, p->taps[i].dw);
    dh0 = std::min<int>(dh0, p->taps[i].dh); dh1 = std::max<int>(dh1, p->taps[i].dh);
  }
  const int ndw = dw1 - dw0 + 1, ndh = dh1 - dh0 + 1;
  if (ndw > 4 || ndh > 4 || ndh < 2 || p->Q < 4) return false;
  const B200ConvView& v = p->views[0];

  WgradHaloArgs g{};
  g.N = p->N; g.P = p->P; g.Q = p->Q; g.Cin = p->Cin; g.Cout = p->Cout;
  g.ndw = ndw; g.ndh = ndh; g.dw_min = dw0; g.dh_min = dh0;
  for (int a = 0; a < 4; ++a)
    for (int b = 0; b < 4; ++b) g.wtap[a][b] = -1;
  for (int i = 0; i < p->ntaps; ++i) g.wtap[p->taps[i].dw - dw0][p->taps[i].dh - dh0] = p->taps[i].wtap;
  g.c_blocks = p->Cin / 64;
  g.ncb = (g.c_blocks >= 2 && ndh * 64 * 2 <= 512) ? 2 : 1;
  g.c_groups = (g.c_blocks + g.ncb - 1) / g.ncb;
  g.m_tiles = (p->Cout + 127) / 128;
  // pixel chunk 8 x bh x bni: an even number of pixel rows (K steps of 16 pixels), at most 128 pixels; cheapest in
  // bytes fetched per useful pixel (gradient rows + activation rows with their halo), ties to the larger chunk
  double best = 1e30;
  for (int bh = 1; bh <= 16 && bh <= p->P; ++bh) {
    for (int bni = 1; bni <= 8; ++bni) {
      const int rows = bh * bni;
      if (rows % 2 || rows > 2 * WH_MAX_STEPS || rows < 4) continue;
      const double waste = (double)((p->P + bh - 1) / bh) * bh / p->P * (double)((p->N + bni - 1) / bni) * bni / p->N;
      const double bytes = waste * (2.0 * 128 + g.ncb * 128.0 * (bh + ndh - 1) / bh);
      const double cost = bytes - 1e-3 * rows;
      if (cost < best) { best = cost; g.bh = bh; g.bni = bni; }
    }
  }
  if (g.bh == 0) return false;
  g.rows = g.bh * g.bni;
  g.tiles_q = (p->Q + 7) / 8;
  g.tiles_p = (p->P + g.bh - 1) / g.bh;
  g.tiles_n = (p->N + g.bni - 1) / g.bni;
  g.a_blk_bytes = g.rows * 1024;
  g.col_bytes = g.bni * (g.bh + ndh - 1) * 1024;
  g.stage_bytes = 2 * g.a_blk_bytes + g.ncb * g.col_bytes;
  const int smem_cap = 227 * 1024 - 1024 /*align*/ - 1024 /*barriers*/ - 32768 /*staging*/;
  g.stages = smem_cap / g.stage_bytes;
  if (g.stages > WH_MAX_STAGES) g.stages = WH_MAX_STAGES;
  if (g.stages < 2) return false;
  g.sep_mma = (mode & 3) == 2 ? 1 : 0;

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long chunks = (long)g.tiles_q * g.tiles_p * g.tiles_n;
  const long base_items = (long)g.m_tiles * g.ndw * g.c_groups;
  int splits = p->splits;
  if (splits <= 0) {
    splits = (int)(sms / base_items);  // one wave of CTAs
    const long max_splits = (chunks + 7) / 8;
    if (splits > max_splits) splits = (int)max_splits;
    if (splits < 1) splits = 1;
  }
  if (splits > chunks) splits = (int)chunks;
  g.chunks_per_split = (int)((chunks + splits - 1) / splits);
  g.splits = (int)((chunks + g.chunks_per_split - 1) / g.chunks_per_split);
  const int fmt = p->ab_dtype == B200_BF16 ? 1 : 0;
  g.idesc = make_idesc(1, fmt, fmt, 1, 1, 128, g.sep_mma ? 64 : ndh * 64);
  g.dw_acc = p->dw_acc;
  g.dw_ld = (long long)p->wtaps * p->Cin;
  g.err = error_flag_ptr();
  if (!g.err) { *rc = (int)cudaErrorInvalidDevice; return true; }

  const CUtensorMapDataType dt = p->ab_dtype == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  WgradHaloMaps maps;
  {
    uint64_t dims[4] = {(uint64_t)v.dims[0], (uint64_t)v.dims[1], (uint64_t)v.dims[2], (uint64_t)v.dims[3]};
    uint64_t str[3] = {(uint64_t)v.strides[0] * 2, (uint64_t)v.strides[1] * 2, (uint64_t)v.strides[2] * 2};
    uint32_t box[4] = {64, 8, (uint32_t)(g.bh + ndh - 1), (uint32_t)g.bni};
    *rc = encode_tiled(&maps.x, dt, 4, v.base, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    if (*rc) return true;
  }
  {
    uint64_t dims[4] = {(uint64_t)p->Cout, (uint64_t)p->Q, (uint64_t)p->P, (uint64_t)p->N};
    uint64_t str[3] = {(uint64_t)p->dy_sw * 2, (uint64_t)p->dy_sh * 2, (uint64_t)p->dy_sn * 2};
    uint32_t box[4] = {64, 8, (uint32_t)g.bh, (uint32_t)g.bni};
    *rc = encode_tiled(&maps.dy, dt, 4, p->dy, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    if (*rc) return true;
  }
  {
    uint64_t dims[2] = {(uint64_t)g.dw_ld, (uint64_t)p->Cout};
    uint64_t str[1] = {(uint64_t)g.dw_ld * 4};
    uint32_t box[2] = {32, 32};
    *rc = encode_tiled(&maps.dw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p->dw_acc, dims, str, box, nullptr, CU_TENSOR_MAP_SWIZZLE_128B);
    if (*rc) return true;
  }
  static bool attr_done[64] = {false};
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute((const void*)conv_wgrad_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) { *rc = (int)e; return true; }
    attr_done[dev & 63] = true;
  }
  const size_t smem = (size_t)g.stages * g.stage_bytes + 1024 + 1024 + 32768;
  const long items = base_items * g.splits;
  conv_wgrad_halo_kernel<<<(int)items, WH_THREADS, smem, (cudaStream_t)stream>>>(maps, g);
  *rc = (int)cudaGetLastError();
  return true;
}

}  // namespace b200

extern "C" int b200_conv_wgrad_halo_mode(int mode) {
  const int prev = b200::g_halo_mode;
  if (mode >= 0) b200::g_halo_mode = mode;
  return prev;
}
