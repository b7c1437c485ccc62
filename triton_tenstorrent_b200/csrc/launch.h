// Host-side plumbing shared by the kernel launchers: error reporting for the C-ABI, per-device
// information, the per-device status word, tensor-map (TMA descriptor) creation with a cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "../../include/b200k.h"

namespace b200k {

// Stores a printf-formatted message for b200k_last_error() (thread-local) and returns `code`.
int set_error(int code, const char* fmt, ...);
void clear_error();

struct DeviceInfo {
  int device;
  int sm_count;
  int cc_major, cc_minor;
  int max_smem_optin;
  uint32_t* status_word;  // device memory, 8 words, zero-initialised; word 0 = first failure code
};
// Information about the current device (created on first use; nullptr + error set on failure).
const DeviceInfo* current_device_info();

void count_launch();

#define B200K_CHECK_LAUNCH(what)                                                                   \
  do {                                                                                             \
    cudaError_t e__ = cudaGetLastError();                                                          \
    if (e__ != cudaSuccess) return set_error(B200K_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e__)); \
  } while (0)

#define B200K_CHECK_CUDA(expr)                                                                       \
  do {                                                                                               \
    cudaError_t e__ = (expr);                                                                        \
    if (e__ != cudaSuccess) return set_error(B200K_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `ld` elements,
// box = box_inner x box_outer elements, 128-byte swizzle (box_inner * 2 bytes at most 128; narrower rows are
// padded to 128 bytes in shared memory),
// out-of-bounds reads fill with zero.  Cached per (base, dims, pitch, box).
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
// 3-D bf16 tensor map of a contiguous [batch][rows][inner] tensor, box = 1 x box_rows x box_inner, 128-byte swizzle.
// A box that runs past `rows` is zero-filled on loads and clipped on stores, so that it never touches the next
// batch entry.
int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
                      uint32_t box_inner, uint32_t box_rows);
// 4-D tensor map of a `rows` x `cols` matrix stored tile-major (contiguous 32 x 32 tiles, tiles in
// row-major order; rows and cols multiples of 32): dimensions (column in tile, tile column, row in
// tile, tile row), box = box_rows x 32 elements (one tile column, box_rows a multiple of 32),
// 64-byte swizzle, so the box lands as box_rows dense rows of 64 bytes.
// row_pairs: the two 64-byte rows of a pair are fetched as ONE 128-byte line (half as many requests to
// L2) with the 128-byte swizzle.  Read back as a 64-byte-swizzled image this is the same data except that
// rows r and r ^ 1 have changed places wherever bit 3 of r is set (the two swizzles differ in address bit 9
// only): usable for the K-major A operand, whose row order only permutes the rows of the accumulator.
int make_tmap_tile32(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint32_t box_rows,
                     bool row_pairs = false);

// Tensor maps of additional destinations of a kernel's output.  Every output tile is stored to the
// caller's primary destination and to each of these, straight from the epilogue's staging buffer: the
// destinations may be buffers of other GPUs mapped into this process (peer memory), which turns the
// epilogue into the sending side of an all-gather that overlaps the main loop of the following tiles.
constexpr int MAX_EXTRA_DESTS = 7;
struct alignas(64) ExtraMaps {
  CUtensorMap m[MAX_EXTRA_DESTS];
};

// Kernel launchers (one translation unit each).
int add_f32(const float* x, const float* y, float* out, int64_t n, cudaStream_t s);
int add_bf16(const uint16_t* x, const uint16_t* y, uint16_t* out, int64_t n, cudaStream_t s);
int sin_f32(const float* x, float* out, int64_t n, cudaStream_t s);
int copy_f32(const float* x, float* out, int64_t n, cudaStream_t s);
int mul_add_f32(const float* x, const float* y, const float* z, float* out, int64_t n, cudaStream_t s);

struct MatmulArgs {
  const void* A;
  const void* B;
  void* C;
  int M, N, K;
  int64_t lda, ldb, ldc;
  const void* bias;
  int bias_kind;
  int64_t ldbias;
  int act;
  int round_before_bias;
  int dtype;  // 0 = bf16, 1 = fp16 (A, B, C and a full [M,N] bias)
  int tile32; // 1 = A, B and C are stored tile-major (32 x 32 tiles); lda/ldb/ldc are ignored, no bias
  void* const* extra_C;  // n_extra further [M,N] destinations with leading dimension ldc (host array of device pointers)
  int n_extra;
};
// status_override: device word the kernel reports bounded-wait failures to (nullptr = the
// per-device word from current_device_info()).
int matmul_bf16(const MatmulArgs& a, cudaStream_t s, uint32_t* status_override);
// How the CTA-pair matmul runs the `rest` tiles left after the full waves of `pairs` pairs: 0 = as whole tiles,
// 1 = each cut in two column halves.  Pure host code.
int matmul_tail_mode(int rest, int pairs);
// out[0..5) = mode, leftover tiles, pairs, full waves, work items of the last wave.
int matmul_tail_plan(int M, int N, int K, int sm_count, int* out);

struct AttnArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse2;
  int Z, H, N_CTX, D;
  int causal;
  float sm_scale;
  void* const* extra_o;  // n_extra further [Z,H,N_CTX,D] destinations of O (host array of device pointers)
  int n_extra;
};
int attn_fwd_bf16(const AttnArgs& a, cudaStream_t s);
struct AttnBwdArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse2;   // M of the forward
  void* dq;
  void* dk;
  void* dv;
  float* delta;        // caller-provided scratch, Z*H*N_CTX floats
  int Z, H, N_CTX, D;
  int causal;
  float sm_scale;
};
int attn_bwd_bf16(const AttnBwdArgs& a, cudaStream_t s);
int attn_bwd_supported(int D, int N_CTX);
int attn_supported(int D, int N_CTX);
// Work-queue simulation that assigns the causal items (ZH * num_pairs, head-major, longest first) to `grid` CTAs:
// returns the table [rounds][grid] of item numbers (-1 = none).  Pure host code.
std::vector<int> attn_schedule(int ZH, int num_pairs, int num_mblk, int ntile, int grid, int* rounds_out);
int selftest_wait_timeout(long long budget_cycles, cudaStream_t s);
// The same self-test reporting into `status_words` (device memory, at least two words: status, kernel's own outcome).
int selftest_wait_timeout_at(uint32_t* status_words, long long budget_cycles, cudaStream_t s);

}  // namespace b200k
