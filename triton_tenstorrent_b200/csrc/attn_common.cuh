// Pieces shared by the attention forward kernels (single-CTA and CTA-pair): tile constants and the
// exponential sequence of the base-2 online softmax (examples/fused-attn/06-fused-attention.py:57-68).
#pragma once
#include <stdint.h>

#include "ptx.cuh"

namespace b200k {

constexpr int AT_BM = 128;            // rows per Q tile
constexpr int AT_BN = 128;            // keys per K/V block
constexpr int AT_BOX_BYTES = 16384;   // one TMA box: 128 rows x 64 columns of bf16

// The running maximum used as the exponent base only advances (and O is only rescaled) when a row maximum
// outgrows it by more than this many powers of two.
constexpr float AT_RESCALE_THRESHOLD = 8.0f;  // log2 units

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// In place: s[i] <- exp2(s[i] * scale - m) for 32 scores (fp32 bits), adding the results to two pair sums.
// Pass 1: 16 packed multiply-subtracts; pass 2: 32 exponentials; pass 3: 16 packed adds.
__device__ __forceinline__ void exp_block32(uint32_t (&s)[32], uint64_t scale2, uint64_t negm2, uint64_t& sum_a,
                                            uint64_t& sum_b) {
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    float x0, x1;
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[2 * c]), __uint_as_float(s[2 * c + 1])), scale2, negm2), x0, x1);
    s[2 * c] = __float_as_uint(x0);
    s[2 * c + 1] = __float_as_uint(x1);
  }
#pragma unroll
  for (int c = 0; c < 32; ++c) s[c] = __float_as_uint(ex2_approx(__uint_as_float(s[c])));
#pragma unroll
  for (int c = 0; c < 16; c += 2) {
    sum_a = add_f32x2(sum_a, pack_f32x2(__uint_as_float(s[2 * c]), __uint_as_float(s[2 * c + 1])));
    sum_b = add_f32x2(sum_b, pack_f32x2(__uint_as_float(s[2 * c + 2]), __uint_as_float(s[2 * c + 3])));
  }
}

}  // namespace b200k
