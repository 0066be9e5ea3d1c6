// Sorting rows of any length and any orderable dtype, and prefix sums.
//
// The reference sorts with cnnlTopKTensor (torch_mlu/csrc/aten/operators/cnnl/internal/topk_internal.cpp:71,118)
// and finds unique values with cnnlUnique* (unique_internal.cpp:53-92); here the long-row path is a bitonic
// network over (key, position) pairs held in a workspace:
//   * every element is encoded as an order-preserving 64-bit key (floats: sign-flipped bit pattern with NaN
//     as the largest value; integers: biased) next to its position in the row, rows padded to a power of two;
//   * tiles of 2048 pairs are sorted in shared memory; larger compare-exchange distances run as one
//     grid-wide pass each, and every remaining distance inside a tile is finished by one shared-memory pass;
//   * pairs compare by (key, position), so equal keys keep their original order (a stable sort) although the
//     network itself is not stable.
// The inclusive scan (cumsum over int64) is the usual three phases: per-CTA scan + totals, scan of the
// totals by one CTA, add the offsets.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"

namespace {

constexpr int TILE = 2048;       // pairs per shared-memory tile (32 KB)
constexpr int SORT_THREADS = 1024;

struct Pair {
  unsigned long long key;
  long long pos;
};

__device__ __forceinline__ unsigned long long encode_key(const void* x, long long i, int dt) {
  switch (dt) {
    case B200_F32: case B200_F16: case B200_BF16: {
      float v;
      if (dt == B200_F32) v = static_cast<const float*>(x)[i];
      else if (dt == B200_F16) v = __half2float(static_cast<const __half*>(x)[i]);
      else v = __bfloat162float(static_cast<const __nv_bfloat16*>(x)[i]);
      if (v != v) return 0xffffffffffffffffull;  // NaN: the largest key
      unsigned u = __float_as_uint(v);
      u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
      return (unsigned long long)u;
    }
    case B200_F64: {
      const double v = static_cast<const double*>(x)[i];
      if (v != v) return 0xffffffffffffffffull;
      unsigned long long u = (unsigned long long)__double_as_longlong(v);
      return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
    }
    case B200_I64: return (unsigned long long)static_cast<const long long*>(x)[i] ^ 0x8000000000000000ull;
    case B200_I32: return (unsigned long long)((long long)static_cast<const int*>(x)[i]) ^ 0x8000000000000000ull;
    case B200_I16: return (unsigned long long)((long long)static_cast<const short*>(x)[i]) ^ 0x8000000000000000ull;
    case B200_I8: return (unsigned long long)((long long)static_cast<const signed char*>(x)[i]) ^ 0x8000000000000000ull;
    default: return (unsigned long long)static_cast<const unsigned char*>(x)[i];  // uint8 / bool
  }
}

// "a goes before b" in the requested order; padding (pos < 0) always goes last
__device__ __forceinline__ bool before(const Pair& a, const Pair& b, int descending) {
  if ((a.pos < 0) != (b.pos < 0)) return b.pos < 0;
  if (a.key != b.key) return descending ? a.key > b.key : a.key < b.key;
  return a.pos < b.pos;
}

__global__ void sort_encode_kernel(const void* x, int dt, long long rows, long long len, long long padded, Pair* ws) {
  const long long total = rows * padded;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / padded, c = i - r * padded;
    Pair p;
    if (c < len) { p.key = encode_key(x, r * len + c, dt); p.pos = c; }
    else { p.key = 0; p.pos = -1; }
    ws[i] = p;
  }
}

// Sorts every TILE-sized tile completely (alternating directions so that consecutive tiles form bitonic
// sequences), or, with k_start > TILE, finishes the distances < TILE of the merge stage `k_start`.
__global__ void __launch_bounds__(SORT_THREADS) sort_tile_kernel(Pair* ws, long long padded, int descending, long long k_start) {
  __shared__ Pair sh[TILE];
  const long long tile0 = (long long)blockIdx.x * TILE;   // tiles never straddle rows: padded is a multiple of TILE
  const long long in_row = tile0 % padded;
  for (int i = threadIdx.x; i < TILE; i += SORT_THREADS) sh[i] = ws[tile0 + i];
  __syncthreads();
  const long long k_first = k_start > TILE ? k_start : 2;
  for (long long k = k_first; k <= (k_start > TILE ? k_start : (long long)TILE); k <<= 1) {
    for (int j = (int)((k > TILE ? (long long)TILE : k) >> 1); j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < TILE / 2; t += SORT_THREADS) {
        const int lo = 2 * t - (t & (j - 1));
        const int hi = lo + j;
        const bool up = ((in_row + lo) & k) == 0;
        const Pair a = sh[lo], b = sh[hi];
        if (before(a, b, descending) != up) { sh[lo] = b; sh[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < TILE; i += SORT_THREADS) ws[tile0 + i] = sh[i];
}

// one compare-exchange distance j >= TILE of merge stage k, over all rows
__global__ void sort_global_kernel(Pair* ws, long long rows, long long padded, long long k, long long j, int descending) {
  const long long half = padded / 2, total = rows * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / half, t = i - r * half;
    const long long lo = 2 * t - (t & (j - 1)), hi = lo + j;
    const bool up = (lo & k) == 0;
    Pair* row = ws + r * padded;
    const Pair a = row[lo], b = row[hi];
    if (before(a, b, descending) != up) { row[lo] = b; row[hi] = a; }
  }
}

__global__ void sort_write_kernel(const Pair* ws, const void* x, int elem_bytes, long long rows, long long len, long long padded,
                                  long long k, void* values, long long* indices) {
  const long long total = rows * k;
  const char* xin = static_cast<const char*>(x);
  char* vout = static_cast<char*>(values);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / k, c = i - r * k;
    const long long src = ws[r * padded + c].pos;
    if (indices) indices[i] = src;
    if (values) {
      const char* s = xin + (r * len + src) * elem_bytes;
      char* d = vout + i * elem_bytes;
      for (int b = 0; b < elem_bytes; ++b) d[b] = s[b];
    }
  }
}

// ---- inclusive scan of int64 ------------------------------------------------------------------------
constexpr int SCAN_THREADS = 512, SCAN_ITEMS = 8, SCAN_CHUNK = SCAN_THREADS * SCAN_ITEMS;

__device__ long long block_scan_inclusive(long long v, long long* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const long long n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) warp_sums[warp] = v;
  __syncthreads();
  if (warp == 0) {
    long long s = lane < SCAN_THREADS / 32 ? warp_sums[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long n = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += n;
    }
    if (lane < SCAN_THREADS / 32) warp_sums[lane] = s;
  }
  __syncthreads();
  if (warp > 0) v += warp_sums[warp - 1];
  __syncthreads();
  return v;
}

// phase 1: each CTA scans one chunk and records its total
__global__ void __launch_bounds__(SCAN_THREADS) scan_chunk_kernel(const long long* in, long long* out, long long n, long long* totals) {
  __shared__ long long warp_sums[32];
  const long long base = (long long)blockIdx.x * SCAN_CHUNK + (long long)threadIdx.x * SCAN_ITEMS;
  long long v[SCAN_ITEMS], run = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    v[k] = base + k < n ? in[base + k] : 0;
    run += v[k];
    v[k] = run;
  }
  const long long incl = block_scan_inclusive(run, warp_sums);
  const long long excl = incl - run;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k)
    if (base + k < n) out[base + k] = v[k] + excl;
  if (threadIdx.x == SCAN_THREADS - 1) totals[blockIdx.x] = incl;
}
// phase 2: one CTA turns the chunk totals into exclusive offsets
__global__ void __launch_bounds__(SCAN_THREADS) scan_totals_kernel(long long* totals, long long chunks) {
  __shared__ long long warp_sums[32];
  __shared__ long long carry_sh;
  if (threadIdx.x == 0) carry_sh = 0;
  __syncthreads();
  for (long long base = 0; base < chunks; base += SCAN_THREADS) {
    const long long i = base + threadIdx.x;
    const long long v = i < chunks ? totals[i] : 0;
    const long long incl = block_scan_inclusive(v, warp_sums);
    const long long carry = carry_sh;
    __syncthreads();
    if (i < chunks) totals[i] = carry + incl - v;
    if (threadIdx.x == SCAN_THREADS - 1) carry_sh = carry + incl;
    __syncthreads();
  }
}
// phase 3
__global__ void scan_add_kernel(long long* out, long long n, const long long* totals) {
  const long long off = totals[blockIdx.x];
  const long long base = (long long)blockIdx.x * SCAN_CHUNK;
  for (int t = threadIdx.x; t < SCAN_CHUNK; t += blockDim.x)
    if (base + t < n) out[base + t] += off;
}

inline int grid1d(long long n, int threads, int cap) {
  long long g = (n + threads - 1) / threads;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}
inline long long pad_len(long long len) {
  long long p = TILE;
  while (p < len) p <<= 1;
  return p;
}

}  // namespace

extern "C" long long b200_sort_long_workspace_bytes(long long rows, long long len) {
  return rows * pad_len(len) * (long long)sizeof(Pair);
}

// Sorts each of `rows` contiguous rows of `len` elements (any length); writes the first k sorted values
// (dtype of x; may be null) and their int64 positions (may be null).  Equal keys keep their order.
extern "C" int b200_sort_long(const void* x, int dtype, int elem_bytes, long long rows, long long len, int descending,
                              long long k, void* values, long long* indices, void* workspace, void* stream) {
  if (rows <= 0 || len <= 0 || k <= 0) return 0;
  if (k > len || !workspace) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  Pair* ws = static_cast<Pair*>(workspace);
  const long long padded = pad_len(len);
  const long long tiles = rows * padded / TILE;
  if (tiles > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  sort_encode_kernel<<<grid1d(rows * padded, 256, 148 * 16), 256, 0, s>>>(x, dtype, rows, len, padded, ws);
  sort_tile_kernel<<<(unsigned)tiles, SORT_THREADS, 0, s>>>(ws, padded, descending, 0);
  for (long long kk = 2LL * TILE; kk <= padded; kk <<= 1) {
    for (long long j = kk >> 1; j >= TILE; j >>= 1)
      sort_global_kernel<<<grid1d(rows * padded / 2, 256, 148 * 16), 256, 0, s>>>(ws, rows, padded, kk, j, descending);
    sort_tile_kernel<<<(unsigned)tiles, SORT_THREADS, 0, s>>>(ws, padded, descending, kk);
  }
  sort_write_kernel<<<grid1d(rows * k, 256, 148 * 16), 256, 0, s>>>(ws, x, elem_bytes, rows, len, padded, k, values, indices);
  return (int)cudaGetLastError();
}

extern "C" long long b200_scan_workspace_elems(long long n) { return (n + SCAN_CHUNK - 1) / SCAN_CHUNK + 1; }

// out[i] = in[0] + ... + in[i] (int64).  `workspace` holds b200_scan_workspace_elems(n) int64 values.
extern "C" int b200_inclusive_scan_i64(const long long* in, long long* out, long long n, long long* workspace, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const long long chunks = (n + SCAN_CHUNK - 1) / SCAN_CHUNK;
  if (chunks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  scan_chunk_kernel<<<(unsigned)chunks, SCAN_THREADS, 0, s>>>(in, out, n, workspace);
  if (chunks > 1) {
    scan_totals_kernel<<<1, SCAN_THREADS, 0, s>>>(workspace, chunks);
    scan_add_kernel<<<(unsigned)chunks, 256, 0, s>>>(out, n, workspace);
  }
  return (int)cudaGetLastError();
}
