// Indexing, sorting and resampling kernels: gather / scatter along a dimension, row
// gather / scatter for advanced indexing, nonzero, arange, tril / triu, row sort (top-k),
// nearest / bilinear 2-D resampling, NMS and depthwise convolution.
//
// Behavioural parity: the reference reaches these through CNNL (index_select.cpp,
// index.cpp, index_put.cpp, masked_select / nonzero, topk.cpp, sort.cpp,
// upsample_nearest2d.cpp, upsample_bilinear2d.cpp, nms.cpp under
// torch_mlu/csrc/aten/operators/cnnl/).  Here they are plain CUDA kernels: none of them
// is GEMM shaped, all are bound by memory traffic or by latency on small inputs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include "kernels_api.h"

namespace {

constexpr int kMaxDims = 8;

template <int BYTES> struct Word;
template <> struct Word<1> { using T = uint8_t; };
template <> struct Word<2> { using T = uint16_t; };
template <> struct Word<4> { using T = uint32_t; };
template <> struct Word<8> { using T = uint64_t; };

__device__ __forceinline__ float load_as_float(const void* p, long long i, int dt) {
  switch (dt) {
    case B200_F32: return static_cast<const float*>(p)[i];
    case B200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    case B200_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case B200_F64: return (float)static_cast<const double*>(p)[i];
    case B200_I64: return (float)static_cast<const long long*>(p)[i];
    case B200_I32: return (float)static_cast<const int*>(p)[i];
    case B200_U8: case B200_BOOL: return (float)static_cast<const uint8_t*>(p)[i];
    case B200_I8: return (float)static_cast<const int8_t*>(p)[i];
    default: return 0.f;
  }
}
__device__ __forceinline__ void store_from_float(void* p, long long i, int dt, float v) {
  switch (dt) {
    case B200_F32: static_cast<float*>(p)[i] = v; break;
    case B200_BF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v); break;
    case B200_F16: static_cast<__half*>(p)[i] = __float2half(v); break;
    case B200_F64: static_cast<double*>(p)[i] = v; break;
    default: break;
  }
}

inline unsigned grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = 148LL * 32;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

// ---- gather / scatter along one dimension ---------------------------------------------
struct DimIndexArgs {
  int ndim, dim;
  long long sizes[kMaxDims];        // shape of the index tensor (contiguous)
  long long a_strides[kMaxDims];    // element strides of the indexed tensor
  long long b_strides[kMaxDims];    // element strides of the tensor shaped like the index (src of scatter / out of gather)
  long long dim_size;               // extent of the indexed tensor along `dim`
};

// mode 0: b[i] = a[index]; 1: a[index] = b[i]; 2: a[index] += b[i] (fp32 only)
template <typename W>
__global__ void dim_index_kernel(W* a, W* b, const long long* index, long long n, DimIndexArgs g, int mode, int* bad) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, aoff = 0, boff = 0;
    for (int d = g.ndim - 1; d >= 0; --d) {
      const long long c = rem % g.sizes[d];
      rem /= g.sizes[d];
      boff += c * g.b_strides[d];
      if (d != g.dim) aoff += c * g.a_strides[d];
    }
    long long ix = index[i];
    if (ix < 0) ix += g.dim_size;
    if (ix < 0 || ix >= g.dim_size) { *bad = 1; continue; }
    aoff += ix * g.a_strides[g.dim];
    if (mode == 0) b[boff] = a[aoff];
    else if (mode == 1) a[aoff] = b[boff];
    else atomicAdd(reinterpret_cast<float*>(a) + aoff, reinterpret_cast<const float*>(b)[boff]);
  }
}

// ---- rows: out[o][n][:] = src[o][idx[n]][:]  and the scatter counterpart ---------------
__global__ void take_rows_kernel(const char* src, const long long* idx, long long outer, long long n_src, long long n_idx,
                                 long long row_bytes, char* out, int* bad) {
  const long long rows = outer * n_idx;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long o = r / n_idx, n = r - o * n_idx;
    long long ix = idx[n];
    if (ix < 0) ix += n_src;
    if (ix < 0 || ix >= n_src) { if (threadIdx.x == 0) *bad = 1; continue; }
    const char* s = src + (o * n_src + ix) * row_bytes;
    char* d = out + r * row_bytes;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d) | (uintptr_t)row_bytes) & 15) == 0) {
      for (long long b = threadIdx.x * 16LL; b < row_bytes; b += blockDim.x * 16LL)
        *reinterpret_cast<uint4*>(d + b) = *reinterpret_cast<const uint4*>(s + b);
    } else {
      for (long long b = threadIdx.x; b < row_bytes; b += blockDim.x) d[b] = s[b];
    }
  }
}
// accumulate == 0: dst[o][idx[n]][:] = val[o][n][:] (word copies); accumulate == 1: fp32 atomic add
__global__ void put_rows_kernel(char* dst, const long long* idx, long long outer, long long n_dst, long long n_idx,
                                long long row_elems, int elem_bytes, const char* val, int accumulate, int* bad) {
  const long long rows = outer * n_idx;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long o = r / n_idx, n = r - o * n_idx;
    long long ix = idx[n];
    if (ix < 0) ix += n_dst;
    if (ix < 0 || ix >= n_dst) { if (threadIdx.x == 0) *bad = 1; continue; }
    char* d = dst + (o * n_dst + ix) * row_elems * elem_bytes;
    const char* s = val + r * row_elems * elem_bytes;
    if (accumulate) {
      for (long long e = threadIdx.x; e < row_elems; e += blockDim.x)
        atomicAdd(reinterpret_cast<float*>(d) + e, reinterpret_cast<const float*>(s)[e]);
    } else {
      const long long nb = row_elems * elem_bytes;
      for (long long b = threadIdx.x; b < nb; b += blockDim.x) d[b] = s[b];
    }
  }
}

// ---- nonzero ----------------------------------------------------------------------------
constexpr int kNzBlock = 1024;
template <typename W>
__global__ void nz_count_kernel(const W* x, long long n, int is_float_bits, long long* counts) {
  __shared__ int warp_cnt[32];
  const long long i = blockIdx.x * (long long)kNzBlock + threadIdx.x;
  bool nz = false;
  if (i < n) {
    const W v = x[i];
    // floating types: -0.0 is zero; its bit pattern is only the sign bit
    nz = is_float_bits ? (static_cast<W>(v << 1) != 0) : (v != 0);
  }
  const unsigned m = __ballot_sync(0xffffffffu, nz);
  if ((threadIdx.x & 31) == 0) warp_cnt[threadIdx.x >> 5] = __popc(m);
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < kNzBlock / 32; ++w) s += warp_cnt[w];
    counts[blockIdx.x] = s;
  }
}
// exclusive scan of `counts` in place by one block; total goes to counts[nblocks]
__global__ void nz_scan_kernel(long long* counts, long long nblocks) {
  __shared__ long long part[1024];
  const long long per = (nblocks + blockDim.x - 1) / blockDim.x;
  const long long lo = threadIdx.x * per, hi = lo + per < nblocks ? lo + per : nblocks;
  long long s = 0;
  for (long long i = lo; i < hi; ++i) s += counts[i];
  part[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int t = 0; t < blockDim.x; ++t) { const long long v = part[t]; part[t] = run; run += v; }
    counts[nblocks] = run;
  }
  __syncthreads();
  long long run = part[threadIdx.x];
  for (long long i = lo; i < hi; ++i) { const long long v = counts[i]; counts[i] = run; run += v; }
}
template <typename W>
__global__ void nz_write_kernel(const W* x, long long n, int is_float_bits, const long long* offsets, int ndim,
                                DimIndexArgs g, long long* out) {
  __shared__ int warp_off[32];
  const long long i = blockIdx.x * (long long)kNzBlock + threadIdx.x;
  bool nz = false;
  if (i < n) {
    const W v = x[i];
    nz = is_float_bits ? (static_cast<W>(v << 1) != 0) : (v != 0);
  }
  const unsigned m = __ballot_sync(0xffffffffu, nz);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_off[warp] = __popc(m);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int w = 0; w < kNzBlock / 32; ++w) { const int v = warp_off[w]; warp_off[w] = run; run += v; }
  }
  __syncthreads();
  if (nz) {
    const long long pos = offsets[blockIdx.x] + warp_off[warp] + __popc(m & ((1u << lane) - 1));
    long long rem = i;
    for (int d = ndim - 1; d >= 0; --d) {
      out[pos * ndim + d] = rem % g.sizes[d];
      rem /= g.sizes[d];
    }
  }
}

// ---- arange, tril / triu ------------------------------------------------------------------
__global__ void arange_kernel(void* out, int dt, long long n, double start, double step) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const double v = start + step * (double)i;
    switch (dt) {
      case B200_I64: static_cast<long long*>(out)[i] = (long long)v; break;
      case B200_I32: static_cast<int*>(out)[i] = (int)v; break;
      case B200_F64: static_cast<double*>(out)[i] = v; break;
      default: store_from_float(out, i, dt, (float)v); break;
    }
  }
}
// keeps the lower (upper == 0) or upper triangle relative to diagonal k of [batch, rows, cols] contiguous matrices
template <typename W>
__global__ void tri_kernel(const W* in, W* out, long long n, long long rows, long long cols, long long k, int upper) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long c = i % cols, r = (i / cols) % rows;
    const bool keep = upper ? (c - r >= k) : (c - r <= k);
    out[i] = keep ? in[i] : W(0);
  }
}

}  // namespace

static int check_dims(int ndim) { return (ndim < 0 || ndim > kMaxDims) ? (int)cudaErrorInvalidValue : 0; }

extern "C" int b200_dim_index(void* a, void* b, int elem_bytes, const long long* index, int ndim, int dim,
                              const long long* sizes, const long long* a_strides, const long long* b_strides,
                              long long dim_size, int mode, int* bad_flag, void* stream) {
  if (check_dims(ndim)) return (int)cudaErrorInvalidValue;
  DimIndexArgs g{};
  g.ndim = ndim; g.dim = dim; g.dim_size = dim_size;
  long long n = 1;
  for (int d = 0; d < ndim; ++d) { g.sizes[d] = sizes[d]; g.a_strides[d] = a_strides[d]; g.b_strides[d] = b_strides[d]; n *= sizes[d]; }
  if (n <= 0) return 0;
  if (mode == 2 && elem_bytes != 4) return (int)cudaErrorInvalidValue;
  const unsigned grid = grid_for(n, 256);
  cudaStream_t s = (cudaStream_t)stream;
  switch (elem_bytes) {
    case 1: dim_index_kernel<uint8_t><<<grid, 256, 0, s>>>((uint8_t*)a, (uint8_t*)b, index, n, g, mode, bad_flag); break;
    case 2: dim_index_kernel<uint16_t><<<grid, 256, 0, s>>>((uint16_t*)a, (uint16_t*)b, index, n, g, mode, bad_flag); break;
    case 4: dim_index_kernel<uint32_t><<<grid, 256, 0, s>>>((uint32_t*)a, (uint32_t*)b, index, n, g, mode, bad_flag); break;
    case 8: dim_index_kernel<uint64_t><<<grid, 256, 0, s>>>((uint64_t*)a, (uint64_t*)b, index, n, g, mode, bad_flag); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_take_rows(const void* src, const long long* idx, long long outer, long long n_src, long long n_idx,
                              long long row_bytes, void* out, int* bad_flag, void* stream) {
  if (outer * n_idx <= 0 || row_bytes <= 0) return 0;
  const long long rows = outer * n_idx;
  const unsigned grid = (unsigned)(rows < 148 * 16 ? rows : 148 * 16);
  take_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const char*)src, idx, outer, n_src, n_idx, row_bytes, (char*)out, bad_flag);
  return (int)cudaGetLastError();
}
extern "C" int b200_put_rows(void* dst, const long long* idx, long long outer, long long n_dst, long long n_idx,
                             long long row_elems, int elem_bytes, const void* values, int accumulate, int* bad_flag,
                             void* stream) {
  if (outer * n_idx <= 0 || row_elems <= 0) return 0;
  if (accumulate && elem_bytes != 4) return (int)cudaErrorInvalidValue;
  const long long rows = outer * n_idx;
  const unsigned grid = (unsigned)(rows < 148 * 16 ? rows : 148 * 16);
  put_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((char*)dst, idx, outer, n_dst, n_idx, row_elems, elem_bytes,
                                                           (const char*)values, accumulate, bad_flag);
  return (int)cudaGetLastError();
}

extern "C" long long b200_nonzero_workspace_elems(long long n) { return (n + kNzBlock - 1) / kNzBlock + 1; }
// pass 1: per-block counts and their exclusive scan; workspace[nblocks] receives the total
extern "C" int b200_nonzero_count(const void* x, int elem_bytes, int is_float, long long n, long long* workspace, void* stream) {
  const long long nblocks = (n + kNzBlock - 1) / kNzBlock;
  cudaStream_t s = (cudaStream_t)stream;
  if (nblocks > 0) {
    switch (elem_bytes) {
      case 1: nz_count_kernel<uint8_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint8_t*)x, n, is_float, workspace); break;
      case 2: nz_count_kernel<uint16_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint16_t*)x, n, is_float, workspace); break;
      case 4: nz_count_kernel<uint32_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint32_t*)x, n, is_float, workspace); break;
      case 8: nz_count_kernel<uint64_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint64_t*)x, n, is_float, workspace); break;
      default: return (int)cudaErrorInvalidValue;
    }
  }
  nz_scan_kernel<<<1, 1024, 0, s>>>(workspace, nblocks);
  return (int)cudaGetLastError();
}
// pass 2: coordinates of the nonzero elements in row-major order, out is [total, ndim] int64
extern "C" int b200_nonzero_write(const void* x, int elem_bytes, int is_float, long long n, const long long* workspace,
                                  int ndim, const long long* sizes, long long* out, void* stream) {
  if (check_dims(ndim)) return (int)cudaErrorInvalidValue;
  const long long nblocks = (n + kNzBlock - 1) / kNzBlock;
  if (nblocks <= 0) return 0;
  DimIndexArgs g{};
  g.ndim = ndim;
  for (int d = 0; d < ndim; ++d) g.sizes[d] = sizes[d];
  cudaStream_t s = (cudaStream_t)stream;
  switch (elem_bytes) {
    case 1: nz_write_kernel<uint8_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint8_t*)x, n, is_float, workspace, ndim, g, out); break;
    case 2: nz_write_kernel<uint16_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint16_t*)x, n, is_float, workspace, ndim, g, out); break;
    case 4: nz_write_kernel<uint32_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint32_t*)x, n, is_float, workspace, ndim, g, out); break;
    case 8: nz_write_kernel<uint64_t><<<(unsigned)nblocks, kNzBlock, 0, s>>>((const uint64_t*)x, n, is_float, workspace, ndim, g, out); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_arange(void* out, int dtype, long long n, double start, double step, void* stream) {
  if (n <= 0) return 0;
  arange_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(out, dtype, n, start, step);
  return (int)cudaGetLastError();
}
extern "C" int b200_tri(const void* in, void* out, int elem_bytes, long long batch, long long rows, long long cols,
                        long long k, int upper, void* stream) {
  const long long n = batch * rows * cols;
  if (n <= 0) return 0;
  const unsigned grid = grid_for(n, 256);
  cudaStream_t s = (cudaStream_t)stream;
  switch (elem_bytes) {
    case 1: tri_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)in, (uint8_t*)out, n, rows, cols, k, upper); break;
    case 2: tri_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)in, (uint16_t*)out, n, rows, cols, k, upper); break;
    case 4: tri_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)in, (uint32_t*)out, n, rows, cols, k, upper); break;
    case 8: tri_kernel<uint64_t><<<grid, 256, 0, s>>>((const uint64_t*)in, (uint64_t*)out, n, rows, cols, k, upper); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

// =========================================================================================
// Row sort (bitonic, one block per row, rows of up to 4096 elements) -- serves sort and topk
// =========================================================================================
namespace {
constexpr int kSortMax = 4096;

__device__ __forceinline__ bool sort_before(float ka, int ia, float kb, int ib, int descending) {
  if (ka == kb) return ia < ib;
  return descending ? (ka > kb) : (ka < kb);
}

__global__ void sort_rows_kernel(const void* x, int dt, int len, int padded, int descending, int k, void* values,
                                 int elem_bytes, long long* indices) {
  extern __shared__ unsigned char sort_smem[];
  float* keys = reinterpret_cast<float*>(sort_smem);
  int* idx = reinterpret_cast<int*>(keys + padded);
  const long long row = blockIdx.x;
  const float pad_key = descending ? -INFINITY : INFINITY;
  for (int i = threadIdx.x; i < padded; i += blockDim.x) {
    float v = pad_key;
    if (i < len) {
      v = load_as_float(x, row * len + i, dt);
      if (v != v) v = INFINITY;  // NaN sorts as the largest value
    }
    keys[i] = v;
    idx[i] = i < len ? i : 0x7fffffff;  // padding loses every tie
  }
  __syncthreads();
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < padded / 2; t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;  // direction of this bitonic block
        const float ka = keys[lo], kb = keys[hi];
        const int ia = idx[lo], ib = idx[hi];
        const bool in_order = sort_before(ka, ia, kb, ib, descending);
        if (in_order != up) { keys[lo] = kb; keys[hi] = ka; idx[lo] = ib; idx[hi] = ia; }
      }
      __syncthreads();
    }
  }
  const char* xin = static_cast<const char*>(x);
  char* vout = static_cast<char*>(values);
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int src = idx[j];
    indices[row * k + j] = src;
    for (int b = 0; b < elem_bytes; ++b) vout[(row * k + j) * elem_bytes + b] = xin[(row * len + src) * elem_bytes + b];
  }
}

// ---- 2-D resampling ---------------------------------------------------------------------
struct ResampleArgs {
  long long N, C, H, W, OH, OW;
  long long in_s[4], out_s[4];  // element strides (n, c, h, w)
  float scale_h, scale_w;       // input step per output pixel
  int align_corners;
};
__device__ __forceinline__ float src_coord(long long o, float scale, int align, long long in_size) {
  if (align) return scale * (float)o;
  const float s = scale * ((float)o + 0.5f) - 0.5f;
  return s < 0.f ? 0.f : s;
}
// mode 0 nearest, 1 bilinear.  backward == 0: out <- in;  backward == 1: in_acc (fp32, contiguous NCHW) += out gradient
__global__ void resample_kernel(const void* in, void* out, int dt, ResampleArgs g, int mode, int backward, float* in_acc) {
  const long long n_out = g.N * g.C * g.OH * g.OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_out; i += (long long)gridDim.x * blockDim.x) {
    const long long ow = i % g.OW, oh = (i / g.OW) % g.OH, c = (i / (g.OW * g.OH)) % g.C, n = i / (g.OW * g.OH * g.C);
    const long long ooff = n * g.out_s[0] + c * g.out_s[1] + oh * g.out_s[2] + ow * g.out_s[3];
    const long long ibase = n * g.in_s[0] + c * g.in_s[1];
    const long long abase = (n * g.C + c) * g.H * g.W;
    if (mode == 0) {
      long long ih = (long long)floorf((float)oh * g.scale_h), iw = (long long)floorf((float)ow * g.scale_w);
      ih = ih < g.H - 1 ? ih : g.H - 1;
      iw = iw < g.W - 1 ? iw : g.W - 1;
      if (!backward) store_from_float(out, ooff, dt, load_as_float(in, ibase + ih * g.in_s[2] + iw * g.in_s[3], dt));
      else atomicAdd(in_acc + abase + ih * g.W + iw, load_as_float(out, ooff, dt));
    } else {
      const float fh = src_coord(oh, g.scale_h, g.align_corners, g.H), fw = src_coord(ow, g.scale_w, g.align_corners, g.W);
      long long h0 = (long long)fh, w0 = (long long)fw;
      h0 = h0 < g.H - 1 ? h0 : g.H - 1;
      w0 = w0 < g.W - 1 ? w0 : g.W - 1;
      const long long h1 = h0 < g.H - 1 ? h0 + 1 : h0, w1 = w0 < g.W - 1 ? w0 + 1 : w0;
      const float lh = fh - (float)h0, lw = fw - (float)w0;
      const float c00 = (1.f - lh) * (1.f - lw), c01 = (1.f - lh) * lw, c10 = lh * (1.f - lw), c11 = lh * lw;
      if (!backward) {
        const float v = c00 * load_as_float(in, ibase + h0 * g.in_s[2] + w0 * g.in_s[3], dt) +
                        c01 * load_as_float(in, ibase + h0 * g.in_s[2] + w1 * g.in_s[3], dt) +
                        c10 * load_as_float(in, ibase + h1 * g.in_s[2] + w0 * g.in_s[3], dt) +
                        c11 * load_as_float(in, ibase + h1 * g.in_s[2] + w1 * g.in_s[3], dt);
        store_from_float(out, ooff, dt, v);
      } else {
        const float gv = load_as_float(out, ooff, dt);
        atomicAdd(in_acc + abase + h0 * g.W + w0, c00 * gv);
        atomicAdd(in_acc + abase + h0 * g.W + w1, c01 * gv);
        atomicAdd(in_acc + abase + h1 * g.W + w0, c10 * gv);
        atomicAdd(in_acc + abase + h1 * g.W + w1, c11 * gv);
      }
    }
  }
}

// ---- NMS: suppression bit matrix over boxes sorted by score ----------------------------
// mask[i * col_blocks + j] has bit b set when box i overlaps box j*64+b (a later box) by more than `thr`.
__global__ void nms_mask_kernel(const float* boxes, int n, float thr, unsigned long long* mask, int col_blocks) {
  const int row_start = blockIdx.y, col_start = blockIdx.x;
  if (row_start > col_start) return;
  const int row_size = min(n - row_start * 64, 64), col_size = min(n - col_start * 64, 64);
  __shared__ float cb[64 * 4];
  if (threadIdx.x < col_size) {
    for (int k = 0; k < 4; ++k) cb[threadIdx.x * 4 + k] = boxes[(col_start * 64 + threadIdx.x) * 4 + k];
  }
  __syncthreads();
  if (threadIdx.x < row_size) {
    const int i = row_start * 64 + threadIdx.x;
    const float x1 = boxes[i * 4], y1 = boxes[i * 4 + 1], x2 = boxes[i * 4 + 2], y2 = boxes[i * 4 + 3];
    const float area = (x2 - x1) * (y2 - y1);
    unsigned long long bits = 0;
    const int start = row_start == col_start ? threadIdx.x + 1 : 0;
    for (int j = start; j < col_size; ++j) {
      const float xx1 = fmaxf(x1, cb[j * 4]), yy1 = fmaxf(y1, cb[j * 4 + 1]);
      const float xx2 = fminf(x2, cb[j * 4 + 2]), yy2 = fminf(y2, cb[j * 4 + 3]);
      const float w = fmaxf(xx2 - xx1, 0.f), h = fmaxf(yy2 - yy1, 0.f);
      const float inter = w * h;
      const float area_j = (cb[j * 4 + 2] - cb[j * 4]) * (cb[j * 4 + 3] - cb[j * 4 + 1]);
      if (inter > thr * (area + area_j - inter)) bits |= 1ull << j;
    }
    mask[(long long)i * col_blocks + col_start] = bits;
  }
}

// ---- depthwise convolution (one filter per output channel; out channel k reads input channel k / mult) ----
struct DwArgs {
  long long N, C, H, W, K, P, Q;  // K = C * mult output channels
  int R, S, sh, sw, ph, pw, mult;
  long long x_s[4], y_s[4];       // element strides (n, c, h, w) of input and output / their gradients
};
__global__ void dw_fwd_kernel(const void* x, const void* w, void* y, int dt, DwArgs g) {
  const long long n_out = g.N * g.K * g.P * g.Q;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_out; i += (long long)gridDim.x * blockDim.x) {
    // channel fastest: adjacent threads read adjacent channels of channels-last tensors
    const long long k = i % g.K, q = (i / g.K) % g.Q, p = (i / (g.K * g.Q)) % g.P, n = i / (g.K * g.Q * g.P);
    const long long c = k / g.mult;
    float acc = 0.f;
    for (int r = 0; r < g.R; ++r) {
      const long long h = p * g.sh - g.ph + r;
      if (h < 0 || h >= g.H) continue;
      for (int s = 0; s < g.S; ++s) {
        const long long ww = q * g.sw - g.pw + s;
        if (ww < 0 || ww >= g.W) continue;
        acc += load_as_float(x, n * g.x_s[0] + c * g.x_s[1] + h * g.x_s[2] + ww * g.x_s[3], dt) *
               load_as_float(w, (k * g.R + r) * g.S + s, dt);
      }
    }
    store_from_float(y, n * g.y_s[0] + k * g.y_s[1] + p * g.y_s[2] + q * g.y_s[3], dt, acc);
  }
}
__global__ void dw_dgrad_kernel(const void* dy, const void* w, void* dx, int dt, DwArgs g) {
  const long long n_in = g.N * g.C * g.H * g.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_in; i += (long long)gridDim.x * blockDim.x) {
    const long long c = i % g.C, ww = (i / g.C) % g.W, h = (i / (g.C * g.W)) % g.H, n = i / (g.C * g.W * g.H);
    float acc = 0.f;
    for (int m = 0; m < g.mult; ++m) {
      const long long k = c * g.mult + m;
      for (int r = 0; r < g.R; ++r) {
        const long long hp = h + g.ph - r;
        if (hp < 0 || hp % g.sh) continue;
        const long long p = hp / g.sh;
        if (p >= g.P) continue;
        for (int s = 0; s < g.S; ++s) {
          const long long wq = ww + g.pw - s;
          if (wq < 0 || wq % g.sw) continue;
          const long long q = wq / g.sw;
          if (q >= g.Q) continue;
          acc += load_as_float(dy, n * g.y_s[0] + k * g.y_s[1] + p * g.y_s[2] + q * g.y_s[3], dt) *
                 load_as_float(w, (k * g.R + r) * g.S + s, dt);
        }
      }
    }
    store_from_float(dx, n * g.x_s[0] + c * g.x_s[1] + h * g.x_s[2] + ww * g.x_s[3], dt, acc);
  }
}
// one block per (output channel, tap): dw[k][r][s] = sum over n, p, q
__global__ void dw_wgrad_kernel(const void* dy, const void* x, float* dw, int dt, DwArgs g) {
  __shared__ float part[256];
  const long long k = blockIdx.x / (g.R * g.S);
  const int r = (int)((blockIdx.x / g.S) % g.R), s = (int)(blockIdx.x % g.S);
  const long long c = k / g.mult;
  const long long total = g.N * g.P * g.Q;
  float acc = 0.f;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const long long q = i % g.Q, p = (i / g.Q) % g.P, n = i / (g.Q * g.P);
    const long long h = p * g.sh - g.ph + r, ww = q * g.sw - g.pw + s;
    if (h < 0 || h >= g.H || ww < 0 || ww >= g.W) continue;
    acc += load_as_float(dy, n * g.y_s[0] + k * g.y_s[1] + p * g.y_s[2] + q * g.y_s[3], dt) *
           load_as_float(x, n * g.x_s[0] + c * g.x_s[1] + h * g.x_s[2] + ww * g.x_s[3], dt);
  }
  part[threadIdx.x] = acc;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) dw[blockIdx.x] = part[0];
}

}  // namespace

namespace {
template <typename E>
__global__ void index_fill_kernel(E* dst, const long long* idx, long long outer, long long n_dst, long long n_idx, long long inner,
                                  E fill, int* bad_flag) {
  const long long total = outer * n_idx * inner;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long in = i % inner, j = (i / inner) % n_idx, o = i / (inner * n_idx);
    long long t = idx[j];
    if (t < 0) t += n_dst;
    if (t < 0 || t >= n_dst) { if (bad_flag) *bad_flag = 1; continue; }
    dst[(o * n_dst + t) * inner + in] = fill;
  }
}
}  // namespace

extern "C" int b200_index_fill(void* dst, int elem_bytes, const long long* idx, long long outer, long long n_dst,
                               long long n_idx, long long inner, unsigned long long fill_bits, int* bad_flag, void* stream) {
  const long long total = outer * n_idx * inner;
  if (total <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = grid_for(total, 256);
  switch (elem_bytes) {
    case 1: index_fill_kernel<unsigned char><<<grid, 256, 0, s>>>((unsigned char*)dst, idx, outer, n_dst, n_idx, inner, (unsigned char)fill_bits, bad_flag); break;
    case 2: index_fill_kernel<unsigned short><<<grid, 256, 0, s>>>((unsigned short*)dst, idx, outer, n_dst, n_idx, inner, (unsigned short)fill_bits, bad_flag); break;
    case 4: index_fill_kernel<unsigned><<<grid, 256, 0, s>>>((unsigned*)dst, idx, outer, n_dst, n_idx, inner, (unsigned)fill_bits, bad_flag); break;
    case 8: index_fill_kernel<unsigned long long><<<grid, 256, 0, s>>>((unsigned long long*)dst, idx, outer, n_dst, n_idx, inner, fill_bits, bad_flag); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_sort_rows_max_len(void) { return kSortMax; }
// Sorts each of `rows` rows of `len` (<= 4096) elements; writes the first k sorted values (dtype of x)
// and their int64 positions.  Ties keep the lower position first.
extern "C" int b200_sort_rows(const void* x, int dtype, int elem_bytes, long long rows, int len, int descending, int k,
                              void* values, long long* indices, void* stream) {
  if (rows <= 0 || len <= 0 || k <= 0) return 0;
  if (len > kSortMax || k > len) return (int)cudaErrorInvalidValue;
  int padded = 2;
  while (padded < len) padded <<= 1;
  const int threads = padded / 2 < 1024 ? (padded / 2 < 32 ? 32 : padded / 2) : 1024;
  sort_rows_kernel<<<(unsigned)rows, threads, (size_t)padded * 8, (cudaStream_t)stream>>>(x, dtype, len, padded, descending, k,
                                                                                        values, elem_bytes, indices);
  return (int)cudaGetLastError();
}

extern "C" int b200_resample2d(const void* in, void* out, int dtype, const long long* sizes /*N,C,H,W,OH,OW*/,
                               const long long* in_strides, const long long* out_strides, double scale_h, double scale_w,
                               int align_corners, int mode, int backward, float* in_acc, void* stream) {
  ResampleArgs g{};
  g.N = sizes[0]; g.C = sizes[1]; g.H = sizes[2]; g.W = sizes[3]; g.OH = sizes[4]; g.OW = sizes[5];
  for (int d = 0; d < 4; ++d) { g.in_s[d] = in_strides ? in_strides[d] : 0; g.out_s[d] = out_strides[d]; }
  g.scale_h = (float)scale_h; g.scale_w = (float)scale_w; g.align_corners = align_corners;
  const long long n = g.N * g.C * g.OH * g.OW;
  if (n <= 0) return 0;
  resample_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(in, out, dtype, g, mode, backward, in_acc);
  return (int)cudaGetLastError();
}

extern "C" int b200_nms_mask(const float* sorted_boxes, int n, float iou_threshold, unsigned long long* mask, void* stream) {
  if (n <= 0) return 0;
  const int cb = (n + 63) / 64;
  dim3 grid(cb, cb);
  nms_mask_kernel<<<grid, 64, 0, (cudaStream_t)stream>>>(sorted_boxes, n, iou_threshold, mask, cb);
  return (int)cudaGetLastError();
}

static DwArgs make_dw(const long long* dims, const int* conv, const long long* x_strides, const long long* y_strides) {
  DwArgs g{};
  g.N = dims[0]; g.C = dims[1]; g.H = dims[2]; g.W = dims[3]; g.K = dims[4]; g.P = dims[5]; g.Q = dims[6];
  g.R = conv[0]; g.S = conv[1]; g.sh = conv[2]; g.sw = conv[3]; g.ph = conv[4]; g.pw = conv[5];
  g.mult = (int)(g.K / g.C);
  for (int d = 0; d < 4; ++d) { g.x_s[d] = x_strides[d]; g.y_s[d] = y_strides[d]; }
  return g;
}
// dims = {N, C, H, W, K, P, Q}; conv = {R, S, stride_h, stride_w, pad_h, pad_w}; weight is contiguous [K][1][R][S].
// pass 0: y = conv(x, w); 1: dx from dy; 2: dw (fp32 [K][R][S]) from dy and x.
extern "C" int b200_depthwise_conv(int pass, const void* x, const void* w, void* y, int dtype, const long long* dims,
                                   const int* conv, const long long* x_strides, const long long* y_strides, void* stream) {
  const DwArgs g = make_dw(dims, conv, x_strides, y_strides);
  cudaStream_t s = (cudaStream_t)stream;
  if (g.N * g.K * g.P * g.Q <= 0 || g.C <= 0) return 0;
  if (pass == 0) {
    dw_fwd_kernel<<<grid_for(g.N * g.K * g.P * g.Q, 256), 256, 0, s>>>(x, w, y, dtype, g);
  } else if (pass == 1) {
    // here `x` is the gradient buffer to fill and `y` the incoming output gradient
    dw_dgrad_kernel<<<grid_for(g.N * g.C * g.H * g.W, 256), 256, 0, s>>>(y, w, const_cast<void*>(x), dtype, g);
  } else {
    // here `w` is the fp32 weight-gradient buffer and `y` the incoming output gradient
    dw_wgrad_kernel<<<(unsigned)(g.K * g.R * g.S), 256, 0, s>>>(y, x, static_cast<float*>(const_cast<void*>(w)), dtype, g);
  }
  return (int)cudaGetLastError();
}
