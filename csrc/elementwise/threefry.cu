// Synthetic token ids from a counter-based generator: element i of the stream is a function of (key, i) only, so
// each rank writes its own rows of the global batch directly on the device (Threefry-2x32, 20 rounds; two 32-bit
// draws per element combined as in jax.random.randint to avoid modulo bias).
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"

namespace mt {
namespace {

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int r) { return __funnelshift_l(x, x, r); }

__device__ __forceinline__ uint32_t threefry_bits(uint32_t k0, uint32_t k1, uint32_t x0, uint32_t x1) {
  const uint32_t ks[3] = {k0, k1, k0 ^ k1 ^ 0x1BD11BDAu};
  x0 += ks[0];
  x1 += ks[1];
#pragma unroll
  for (int g = 0; g < 5; ++g) {
    if (g % 2 == 0) {
      x0 += x1; x1 = rotl32(x1, 13) ^ x0;
      x0 += x1; x1 = rotl32(x1, 15) ^ x0;
      x0 += x1; x1 = rotl32(x1, 26) ^ x0;
      x0 += x1; x1 = rotl32(x1, 6) ^ x0;
    } else {
      x0 += x1; x1 = rotl32(x1, 17) ^ x0;
      x0 += x1; x1 = rotl32(x1, 29) ^ x0;
      x0 += x1; x1 = rotl32(x1, 16) ^ x0;
      x0 += x1; x1 = rotl32(x1, 24) ^ x0;
    }
    x0 += ks[(g + 1) % 3];
    x1 += ks[(g + 2) % 3] + (uint32_t)(g + 1);
  }
  return x0 ^ x1;
}

__global__ void threefry_randint_kernel(int64_t* __restrict__ out, int64_t count, uint32_t a0, uint32_t a1,
                                        uint32_t b0, uint32_t b1, uint64_t start, uint32_t span, uint32_t mult) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t c = start + (uint64_t)i;
    const uint32_t hi = threefry_bits(a0, a1, (uint32_t)(c >> 32), (uint32_t)c);
    const uint32_t lo = threefry_bits(b0, b1, (uint32_t)(c >> 32), (uint32_t)c);
    const uint32_t off = (hi % span) * mult + (lo % span);  // wraps modulo 2^32 like the reference arithmetic
    out[i] = (int64_t)(off % span);
  }
}

}  // namespace

void threefry_randint(int64_t* out, int64_t count, uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1, uint64_t start,
                      uint32_t span, cudaStream_t stream) {
  if (count <= 0) return;
  uint32_t mult = (uint32_t)((1u << 16) % span);
  mult = (uint32_t)(((uint64_t)mult * mult) % span);
  const int threads = 256;
  const int64_t blocks = (count + threads - 1) / threads;
  threefry_randint_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), threads, 0, stream>>>(
      out, count, a0, a1, b0, b1, start, span, mult);
}

}  // namespace mt
