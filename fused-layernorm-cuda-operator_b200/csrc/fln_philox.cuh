// Philox4x32-10 (Salmon, Moraes, Dror, Shaw, SC'11) and the keep masks of the fused dropout:
// one 128-bit output serves 8 consecutive elements, 16 bits each; see fln_dropout.cu for the
// layout of counter, key and mask.
#pragma once
#include "fln_common.cuh"

namespace fln {

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = (unsigned long long)0xD2511F53u * c.x;
    const unsigned long long p1 = (unsigned long long)0xCD9E8D57u * c.z;
    c = make_uint4((unsigned int)(p1 >> 32) ^ c.y ^ k.x, (unsigned int)p1, (unsigned int)(p0 >> 32) ^ c.w ^ k.y,
                   (unsigned int)p0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

// keep mask (8 bits) of group g
__device__ __forceinline__ unsigned int keep_mask8(unsigned long long g, unsigned long long seed, unsigned long long offset,
                                                   unsigned int threshold) {
  const uint4 r = philox4x32_10(make_uint4((unsigned int)g, (unsigned int)(g >> 32), (unsigned int)offset,
                                           (unsigned int)(offset >> 32)),
                                make_uint2((unsigned int)seed, (unsigned int)(seed >> 32)));
  const unsigned int w[4] = {r.x, r.y, r.z, r.w};
  unsigned int m = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const unsigned int v = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    m |= (v >= threshold ? 1u : 0u) << j;
  }
  return m;
}

// the same mask as 16-bit lanes: word w covers elements 2w (low half) and 2w + 1 (high half), all
// ones where the element is kept; returns the 8-bit mask
__device__ __forceinline__ unsigned int keep_lanes8(unsigned long long g, unsigned long long seed,
                                                    unsigned long long offset, unsigned int threshold,
                                                    unsigned int (&lanes)[4]) {
  const uint4 r = philox4x32_10(make_uint4((unsigned int)g, (unsigned int)(g >> 32), (unsigned int)offset,
                                           (unsigned int)(offset >> 32)),
                                make_uint2((unsigned int)seed, (unsigned int)(seed >> 32)));
  const unsigned int w[4] = {r.x, r.y, r.z, r.w};
  unsigned int m = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const bool lo = (w[j] & 0xffffu) >= threshold, hi = (w[j] >> 16) >= threshold;
    lanes[j] = (lo ? 0xffffu : 0u) | (hi ? 0xffff0000u : 0u);
    m |= (lo ? 1u : 0u) << (2 * j) | (hi ? 1u : 0u) << (2 * j + 1);
  }
  return m;
}

}  // namespace fln
