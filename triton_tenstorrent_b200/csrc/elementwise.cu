// Elementwise fp32 kernels: add, sin, mul-add.  HBM-bound: every thread keeps several independent
// 128-bit loads in flight, accesses are coalesced (a warp touches 512 contiguous bytes per load);
// each CTA handles one tile of 1024 float4 per operand (grid-stride only beyond a very large grid).  A scalar path handles
// pointers that are not 16-byte aligned and the n % 4 tail.
//
// Math follows the reference kernels op by op:
//   add      python/tutorials/01-vector-add.py:47-54     out = x + y          (one IEEE fp32 add)
//   sin      examples/01-sin-kernel.py:25-29              out = sin(x)         (precise sinf, <= 1 ulp)
//   mul_add  python/tutorials/01-vector-mul-add.py        out = x * y + z      (two roundings, no FMA)
//   add bf16 python/tutorials/01-vector-add.loop.py:29-66 (run on bf16 tensors, :102-103): the exact sum
//            rounded once to nearest even; computed as an fp32 add of the widened operands and one
//            RNE downcast, which gives the same bits (the fp32 sum of two bf16 values can only be
//            inexact when the smaller operand is far below half a bf16 ulp of the larger)
#include "launch.h"
#include "ptx.cuh"

namespace b200k {

enum class EwOp { Add, Sin, MulAdd, Copy };

template <EwOp OP>
constexpr bool ew_unary() { return OP == EwOp::Sin || OP == EwOp::Copy; }

template <EwOp OP>
__device__ __forceinline__ float ew_apply(float x, float y, float z) {
  if constexpr (OP == EwOp::Add) {
    return x + y;
  } else if constexpr (OP == EwOp::Sin) {
    return sinf(x);
  } else if constexpr (OP == EwOp::Copy) {
    return x;   // bits preserved: a float move never quiets a NaN payload
  } else {
    return __fadd_rn(__fmul_rn(x, y), z);  // keep the two roundings of the reference's x*y then +z
  }
}

template <EwOp OP>
__device__ __forceinline__ float4 ew_apply4(float4 x, float4 y, float4 z) {
  float4 r;
  r.x = ew_apply<OP>(x.x, y.x, z.x);
  r.y = ew_apply<OP>(x.y, y.y, z.y);
  r.z = ew_apply<OP>(x.z, y.z, z.z);
  r.w = ew_apply<OP>(x.w, y.w, z.w);
  return r;
}

// Streaming 128-bit accesses: data is touched exactly once, so bypass L1 allocation.
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

#ifndef B200K_EW_THREADS
#define B200K_EW_THREADS 256
#endif
#ifndef B200K_EW_UNROLL
#define B200K_EW_UNROLL 4
#endif
// Grid cap in CTAs per SM.  Measured at n = 2^26 on B200: a cap of 8 (one resident wave, long grid-stride
// loops) gives 6260 / 5880 GB/s for add / sin, 32 gives 6620 / 6390, 64 gives 6660 / 6570, and in effect no cap
// (one 16 KB-per-operand tile per CTA, handed out by the hardware scheduler) 6800 / 6675 GB/s.
#ifndef B200K_EW_CTAS_PER_SM
#define B200K_EW_CTAS_PER_SM 1024
#endif
constexpr int EW_THREADS = B200K_EW_THREADS;
constexpr int EW_UNROLL = B200K_EW_UNROLL;  // independent float4 per operand per thread per iteration

template <EwOp OP>
__global__ void __launch_bounds__(EW_THREADS) ew_vec4_kernel(const float4* __restrict__ x, const float4* __restrict__ y,
                                                             const float4* __restrict__ z, float4* __restrict__ out,
                                                             int64_t n4) {
  constexpr bool HAS_Y = !ew_unary<OP>();
  constexpr bool HAS_Z = (OP == EwOp::MulAdd);
  const int64_t tile = static_cast<int64_t>(EW_THREADS) * EW_UNROLL;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * tile;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n4; base += stride) {
    float4 xv[EW_UNROLL], yv[EW_UNROLL], zv[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + threadIdx.x + static_cast<int64_t>(u) * EW_THREADS;
      if (i < n4) {
        xv[u] = ld_stream(x + i);
        if constexpr (HAS_Y) yv[u] = ld_stream(y + i);
        if constexpr (HAS_Z) zv[u] = ld_stream(z + i);
      }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + threadIdx.x + static_cast<int64_t>(u) * EW_THREADS;
      if (i < n4) st_stream(out + i, ew_apply4<OP>(xv[u], HAS_Y ? yv[u] : xv[u], HAS_Z ? zv[u] : xv[u]));
    }
  }
}

// Scalar grid-stride path: unaligned pointers and the (< 4 element) tail.
template <EwOp OP>
__global__ void __launch_bounds__(EW_THREADS) ew_scalar_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                               const float* __restrict__ z, float* __restrict__ out,
                                                               int64_t begin, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float xv = x[i];
    const float yv = !ew_unary<OP>() ? y[i] : 0.f;
    const float zv = (OP == EwOp::MulAdd) ? z[i] : 0.f;
    out[i] = ew_apply<OP>(xv, yv, zv);
  }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <EwOp OP>
static int ew_launch(const float* x, const float* y, const float* z, float* out, int64_t n, cudaStream_t stream) {
  if (n == 0) return B200K_OK;
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  const bool vec_ok = aligned16(x) && aligned16(out) && (ew_unary<OP>() || aligned16(y)) &&
                      (OP != EwOp::MulAdd || aligned16(z));
  const int64_t n4 = vec_ok ? (n / 4) : 0;
  if (n4 > 0) {
    const int64_t tile = static_cast<int64_t>(EW_THREADS) * EW_UNROLL;
    const int64_t want = (n4 + tile - 1) / tile;
    // One tile per CTA up to the cap, then grid-stride.
    const int64_t cap = static_cast<int64_t>(dev->sm_count) * B200K_EW_CTAS_PER_SM;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    ew_vec4_kernel<OP><<<grid, EW_THREADS, 0, stream>>>(reinterpret_cast<const float4*>(x),
                                                        reinterpret_cast<const float4*>(y),
                                                        reinterpret_cast<const float4*>(z),
                                                        reinterpret_cast<float4*>(out), n4);
    count_launch();
    B200K_CHECK_LAUNCH("elementwise vec4 kernel");
  }
  const int64_t done = n4 * 4;
  if (done < n) {
    const int64_t rest = n - done;
    int64_t want = (rest + EW_THREADS - 1) / EW_THREADS;
    const int64_t cap = static_cast<int64_t>(dev->sm_count) * 8;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    ew_scalar_kernel<OP><<<grid, EW_THREADS, 0, stream>>>(x, y, z, out, done, n);
    count_launch();
    B200K_CHECK_LAUNCH("elementwise scalar kernel");
  }
  return B200K_OK;
}

// ---- bf16 add: 8 elements per 128-bit access, same tiling as the fp32 kernels
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  return pack_bf16x2(bf16_bits_to_f32(a & 0xFFFFu) + bf16_bits_to_f32(b & 0xFFFFu),
                     bf16_bits_to_f32(a >> 16) + bf16_bits_to_f32(b >> 16));
}

__global__ void __launch_bounds__(EW_THREADS) ew_add_bf16_vec8_kernel(const uint4* __restrict__ x,
                                                                      const uint4* __restrict__ y,
                                                                      uint4* __restrict__ out, int64_t n8) {
  const int64_t tile = static_cast<int64_t>(EW_THREADS) * EW_UNROLL;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * tile;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n8; base += stride) {
    uint4 xv[EW_UNROLL], yv[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + threadIdx.x + static_cast<int64_t>(u) * EW_THREADS;
      if (i < n8) {
        xv[u] = __ldcs(x + i);
        yv[u] = __ldcs(y + i);
      }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + threadIdx.x + static_cast<int64_t>(u) * EW_THREADS;
      if (i < n8)
        __stcs(out + i, make_uint4(add_bf16x2(xv[u].x, yv[u].x), add_bf16x2(xv[u].y, yv[u].y),
                                   add_bf16x2(xv[u].z, yv[u].z), add_bf16x2(xv[u].w, yv[u].w)));
    }
  }
}

__global__ void __launch_bounds__(EW_THREADS) ew_add_bf16_scalar_kernel(const uint16_t* __restrict__ x,
                                                                        const uint16_t* __restrict__ y,
                                                                        uint16_t* __restrict__ out, int64_t begin,
                                                                        int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = static_cast<uint16_t>(pack_bf16x2(bf16_bits_to_f32(x[i]) + bf16_bits_to_f32(y[i]), 0.f) & 0xFFFFu);
}

int add_bf16(const uint16_t* x, const uint16_t* y, uint16_t* out, int64_t n, cudaStream_t stream) {
  if (n == 0) return B200K_OK;
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  const bool vec_ok = aligned16(x) && aligned16(y) && aligned16(out);
  const int64_t n8 = vec_ok ? (n / 8) : 0;
  if (n8 > 0) {
    const int64_t tile = static_cast<int64_t>(EW_THREADS) * EW_UNROLL;
    const int64_t want = (n8 + tile - 1) / tile;
    const int64_t cap = static_cast<int64_t>(dev->sm_count) * B200K_EW_CTAS_PER_SM;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    ew_add_bf16_vec8_kernel<<<grid, EW_THREADS, 0, stream>>>(reinterpret_cast<const uint4*>(x),
                                                             reinterpret_cast<const uint4*>(y),
                                                             reinterpret_cast<uint4*>(out), n8);
    count_launch();
    B200K_CHECK_LAUNCH("bf16 add vec8 kernel");
  }
  const int64_t done = n8 * 8;
  if (done < n) {
    const int64_t rest = n - done;
    const int64_t want = (rest + EW_THREADS - 1) / EW_THREADS;
    const int64_t cap = static_cast<int64_t>(dev->sm_count) * 8;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    ew_add_bf16_scalar_kernel<<<grid, EW_THREADS, 0, stream>>>(x, y, out, done, n);
    count_launch();
    B200K_CHECK_LAUNCH("bf16 add scalar kernel");
  }
  return B200K_OK;
}

int add_f32(const float* x, const float* y, float* out, int64_t n, cudaStream_t s) {
  return ew_launch<EwOp::Add>(x, y, nullptr, out, n, s);
}
int sin_f32(const float* x, float* out, int64_t n, cudaStream_t s) {
  return ew_launch<EwOp::Sin>(x, nullptr, nullptr, out, n, s);
}
int copy_f32(const float* x, float* out, int64_t n, cudaStream_t s) {
  return ew_launch<EwOp::Copy>(x, nullptr, nullptr, out, n, s);
}
int mul_add_f32(const float* x, const float* y, const float* z, float* out, int64_t n, cudaStream_t s) {
  return ew_launch<EwOp::MulAdd>(x, y, z, out, n, s);
}

}  // namespace b200k
