// Counter-based Philox 4x32-10 random numbers keyed by (seed, subsequence, offset): the generator state of the
// device (the reference keeps an MTGP32 state tensor instead, torch_mlu/csrc/aten/core/generator_impl.cpp:183-205).
#pragma once
#include <cuda_runtime.h>

struct Philox {
  unsigned int key[2];
  unsigned int ctr[4];
};
__device__ __forceinline__ void philox_round(unsigned int* c, const unsigned int* k) {
  const unsigned int M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const unsigned int hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const unsigned int hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const unsigned int n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ uint4 philox4(unsigned long long seed, unsigned long long subsequence, unsigned long long offset) {
  unsigned int k[2] = {(unsigned int)seed, (unsigned int)(seed >> 32)};
  unsigned int c[4] = {(unsigned int)offset, (unsigned int)(offset >> 32), (unsigned int)subsequence,
                       (unsigned int)(subsequence >> 32)};
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c, k);
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
  }
  return make_uint4(c[0], c[1], c[2], c[3]);
}
__device__ __forceinline__ float u01(unsigned int x) { return ((x >> 8) + 0.5f) * (1.0f / 16777216.0f); }  // (0,1)

