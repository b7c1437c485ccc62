// Persistent, warp-specialised bf16 matmul for sm_100a:  C = epilogue(A[M,K] . B[K,N]).
//
//   warp 0      TMA producer: A tile 128x64 (K-major) and B tile 64xBN (N-major, as B is row-major
//               [K,N]) into a STAGES-deep shared-memory ring, 128-byte swizzle, completion on mbarriers
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128 x BN x 16 per instruction,
//               fp32 accumulators in TMEM, two accumulator buffers so the epilogue of tile i overlaps
//               the main loop of tile i+1) and tcgen05.commit to release ring slots / publish tiles
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32-lane quarter), fused bias /
//               activation / rounding, swizzled staging in shared memory, TMA store of C
//
// The grid is one CTA per SM; CTA c walks tiles c, c+G, c+2G, ... of the reference's grouped tile
// order (examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py:116-124), which is the
// strided form of the persistent block loop the reference's compiler adds around the kernel
// (cpu/lib/Dialect/TritonCPU/Transforms/MakePersistentKernel.cpp:144-198).
// Contraction semantics follow matmul_kernel_tma (.ttnn.py:126-143): zero fill outside [M,K]/[K,N],
// fp32 accumulation, one RNE downcast, stores outside [M,N] dropped.
//
// Operands may also be stored tile-major (contiguous 32 x 32 tiles), the layout the reference's
// pointer-based matmul_kernel addresses (examples/matmul/03-matrix-multiplication.py:333-386): the
// same kernels then fetch boxes of one tile column through 4-D tensor maps into 64-byte-swizzled
// operand images; only tensor maps, boxes per stage and descriptor constants differ.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "launch.h"
#include "ptx.cuh"

namespace b200k {

constexpr int MM_BM = 128;
constexpr int MM_BK = 64;       // 64 bf16 = 128 bytes = one swizzle row
constexpr int MM_UMMA_K = 16;
constexpr int MM_THREADS = 192;
constexpr int MM_EPI_WARPS = 4;
constexpr int MM_A_STAGE_BYTES = MM_BM * MM_BK * 2;            // 16 KB
constexpr int MM_B_BOX_BYTES = MM_BK * 64 * 2;                 // 8 KB: 64 k-rows x 64 n
constexpr int MM_C_BUF_BYTES = 32 * 128;                       // 32 rows x 64 bf16
constexpr int MM_C_STAGING_BYTES = MM_EPI_WARPS * 2 * MM_C_BUF_BYTES;  // 32 KB

struct MatmulParams {
  int M, N, K;
  int num_pid_m, num_pid_n, group_m;
  int serpentine;   // odd groups of tile rows walk the tile columns backwards
  int num_tiles, num_kb;
  // CTA-pair kernel: work items [0, full_work) are whole 256 x 256 tiles; items beyond are the tiles of the last,
  // less than half full wave cut in two 256 x 128 halves, so that twice as many pairs share it (num_work items in all)
  int num_work, full_work;
  uint32_t idesc_half;             // instruction descriptor of the 256 x 128 MMA
  const float* bias_row;      // [N] fp32 or nullptr
  const uint16_t* bias_full;  // [M, ldbias] bf16 or nullptr
  int64_t ldbias;
  int act;
  int round_before_bias;
  // Operand images in shared memory (bytes).  Row-major operands: 128-byte swizzle, A rows of 64 k
  // (k step +32 B), B boxes of 64 k-rows x 64 n.  Tile-major operands: 64-byte swizzle, A as two
  // 128 x 32 halves, B boxes of 64 k-rows x 32 n.
  uint32_t swz;                    // UMMA layout type of both operands
  uint32_t a_sbo, a_khalf;         // A: 8-row group pitch; offset of k-steps 2,3 (k >= 32) from k-steps 0,1
  uint32_t b_lbo, b_sbo, b_kstep;  // MN-major B: pitch of N chunks, of 8 k-row groups, of one k step (16 rows)
  int f16;                         // operands, bias[M,N] and C are fp16 instead of bf16
  uint32_t idesc;                  // UMMA instruction descriptor (tile shape, operand formats and majors)
  int l2_hint;                     // CTA-pair kernel: 0 = no hints, 1 = A evict_last / B evict_first, 2 = A evict_last only
  int tile32;                      // A, B, C stored as contiguous 32 x 32 tiles (4-D tensor maps, tile coordinates)
  int n_extra;                     // further copies of C the epilogue stores every tile to (ExtraMaps; row-major only)
  uint32_t* status;
};

constexpr int MM_MAX_EXTRA = MAX_EXTRA_DESTS;

template <int BN, int STAGES>
struct MatmulSmem {
  static constexpr int B_STAGE_BYTES = (BN / 64) * MM_B_BOX_BYTES;
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = STAGES * MM_A_STAGE_BYTES;
  static constexpr int C_OFF = B_OFF + STAGES * B_STAGE_BYTES;
  static constexpr int BAR_OFF = C_OFF + MM_C_STAGING_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem_ptr, abort
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = BAR_OFF + BAR_BYTES + 1024;  // + slack to align the base to 1024
};

__device__ __forceinline__ void tile_coords(const MatmulParams& p, int tile, int& pid_m, int& pid_n) {
  const int num_pid_in_group = p.group_m * p.num_pid_n;
  const int group_id = tile / num_pid_in_group;
  const int first_pid_m = group_id * p.group_m;
  const int group_size_m = min(p.num_pid_m - first_pid_m, p.group_m);
  const int in_group = tile - group_id * num_pid_in_group;
  pid_m = first_pid_m + (in_group % group_size_m);
  pid_n = in_group / group_size_m;
  // the next group of rows starts with the B columns the previous group finished with (still in L2)
  if (p.serpentine && (group_id & 1)) pid_n = p.num_pid_n - 1 - pid_n;
}

// 16-bit element <-> fp32 in the operand type of the launch (bf16 or fp16; warp-uniform flag)
__device__ __forceinline__ float h16_to_f32(uint32_t bits16, int f16) {
  return f16 ? f16_bits_to_f32(bits16) : bf16_bits_to_f32(bits16);
}
__device__ __forceinline__ uint32_t pack_h16x2(float lo, float hi, int f16) {
  return f16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}

__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == B200K_ACT_RELU) return fmaxf(x, 0.f);
  if (act == B200K_ACT_LEAKY_RELU) return x >= 0.f ? x : 0.01f * x;
  return x;
}

// One 64-column chunk of a warp's 32 accumulator rows: fused bias / activation / downcast, swizzled
// staging in shared memory, TMA store.  v0/v1 hold columns [0,32) and [32,64) of the chunk as fp32
// bits; `row` is this thread's global row, `row0_warp` the warp's first row, `col0` the chunk's
// first global column; `buf` toggles between the warp's two staging buffers.
__device__ __forceinline__ void epilogue_chunk(const MatmulParams& p, const CUtensorMap* tmap_c,
                                               const CUtensorMap* extra_maps,
                                               const uint32_t (&v0)[32], const uint32_t (&v1)[32], int row,
                                               int row0_warp, int col0, uint8_t* my_stage, int& buf, uint32_t lane) {
    float f[64];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      f[j] = __uint_as_float(v0[j]);
      f[32 + j] = __uint_as_float(v1[j]);
    }
    // ---- fused epilogue
    if (p.bias_row != nullptr) {
      if (col0 + 64 <= p.N) {
        const float4* bp = reinterpret_cast<const float4*>(p.bias_row + col0);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float4 b = __ldg(bp + j);
          f[4 * j + 0] += b.x;
          f[4 * j + 1] += b.y;
          f[4 * j + 2] += b.z;
          f[4 * j + 3] += b.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (col0 + j < p.N) f[j] += __ldg(p.bias_row + col0 + j);
      }
    }
    float bfull[64];
    const bool has_full = (p.bias_full != nullptr);
    if (has_full) {
      const bool row_ok = row < p.M;
      const uint16_t* brow = p.bias_full + static_cast<int64_t>(row_ok ? row : 0) * p.ldbias + col0;
      if (row_ok && col0 + 64 <= p.N && (p.ldbias & 7) == 0 &&
          (reinterpret_cast<uintptr_t>(p.bias_full) & 15u) == 0) {
        const uint4* bp = reinterpret_cast<const uint4*>(brow);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 b = __ldg(bp + j);
          bfull[8 * j + 0] = h16_to_f32(b.x & 0xFFFFu, p.f16);
          bfull[8 * j + 1] = h16_to_f32(b.x >> 16, p.f16);
          bfull[8 * j + 2] = h16_to_f32(b.y & 0xFFFFu, p.f16);
          bfull[8 * j + 3] = h16_to_f32(b.y >> 16, p.f16);
          bfull[8 * j + 4] = h16_to_f32(b.z & 0xFFFFu, p.f16);
          bfull[8 * j + 5] = h16_to_f32(b.z >> 16, p.f16);
          bfull[8 * j + 6] = h16_to_f32(b.w & 0xFFFFu, p.f16);
          bfull[8 * j + 7] = h16_to_f32(b.w >> 16, p.f16);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          bfull[j] = (row_ok && col0 + j < p.N) ? h16_to_f32(__ldg(brow + j), p.f16) : 0.f;
      }
      if (!p.round_before_bias) {
#pragma unroll
        for (int j = 0; j < 64; ++j) f[j] += bfull[j];
      }
    }
    if (p.act != B200K_ACT_NONE) {
#pragma unroll
      for (int j = 0; j < 64; ++j) f[j] = apply_act(f[j], p.act);
    }
    uint32_t packed[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) packed[j] = pack_h16x2(f[2 * j], f[2 * j + 1], p.f16);
    if (has_full && p.round_before_bias) {
      // 16-bit add after the downcast: bf16(float(bf16(acc)) + float(bias))
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float lo = h16_to_f32(packed[j] & 0xFFFFu, p.f16) + bfull[2 * j];
        const float hi = h16_to_f32(packed[j] >> 16, p.f16) + bfull[2 * j + 1];
        packed[j] = pack_h16x2(lo, hi, p.f16);
      }
    }
    // ---- staging buffer `buf` must no longer be read by the TMA store issued two chunks ago
    if (lane == 0) tma_store_wait_read<1>();
    __syncwarp();
    uint8_t* stage_buf = my_stage + buf * MM_C_BUF_BYTES;
    if (p.tile32) {
      // two 32 x 32 tiles side by side, each 32 rows of 64 bytes with the 64-byte swizzle.  A was fetched as
      // 128-byte row pairs (make_tmap_tile32, row_pairs): accumulator row r holds the result row r ^ 1 wherever
      // bit 3 of r is set, which is undone here by the choice of the staging row.
      const uint32_t srow = lane ^ ((lane >> 3) & 1u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 val = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        *reinterpret_cast<uint4*>(stage_buf + (j >> 2) * 2048 + srow * 64 + (((j & 3) ^ ((srow >> 1) & 3)) << 4)) = val;
      }
    } else {
      uint8_t* dst = stage_buf + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 val = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = val;
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (row0_warp < p.M && col0 < p.N) {
        if (p.tile32) {
          tma_store_tile32(tmap_c, stage_buf, col0 >> 5, row0_warp >> 5);
          if (col0 + 32 < p.N) tma_store_tile32(tmap_c, stage_buf + 2048, (col0 >> 5) + 1, row0_warp >> 5);
        } else {
          tma_store_2d(tmap_c, stage_buf, col0, row0_warp);
          for (int d = 0; d < p.n_extra; ++d) tma_store_2d(extra_maps + d, stage_buf, col0, row0_warp);
        }
      }
      tma_store_commit();
    }
    buf ^= 1;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(MM_THREADS, 1)
matmul_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ ExtraMaps extra,
                           const MatmulParams p) {
  using L = MatmulSmem<BN, STAGES>;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 256) ? 256 : 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem + L::A_OFF;
  uint8_t* smem_b = smem + L::B_OFF;
  uint8_t* smem_c = smem + L::C_OFF;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;  // warp-uniform
  const uint32_t lane = lane_id();
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], MM_EPI_WARPS);
    }
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp_idx == 1) {
    tmem_alloc(tmem_ptr_smem, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp_idx == 0) {
    // ---------------------------------------------------------------- TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      int pid_m, pid_n;
      tile_coords(p, tile, pid_m, pid_n);
      const int m0 = pid_m * MM_BM, n0 = pid_n * BN;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        ok = mbar_wait(&empty_bar[stage], phase ^ 1u, ctx, 1);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&full_bar[stage], MM_A_STAGE_BYTES + L::B_STAGE_BYTES);
          if (p.tile32) {
            // tile-major operands: A as two 128 x 32 halves, B as BN/32 boxes of 64 k-rows x 32 n; tile coordinates
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_tile32(smem_a + stage * MM_A_STAGE_BYTES + j * (MM_A_STAGE_BYTES / 2), &tmap_a, &full_bar[stage],
                              kb * 2 + j, m0 >> 5);
#pragma unroll
            for (int i = 0; i < BN / 32; ++i)
              tma_load_tile32(smem_b + stage * L::B_STAGE_BYTES + i * (MM_B_BOX_BYTES / 2), &tmap_b, &full_bar[stage],
                              (n0 >> 5) + i, kb * 2);
          } else {
            tma_load_2d(smem_a + stage * MM_A_STAGE_BYTES, &tmap_a, &full_bar[stage], kb * MM_BK, m0);
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(smem_b + stage * L::B_STAGE_BYTES + i * MM_B_BOX_BYTES, &tmap_b, &full_bar[stage],
                          n0 + i * 64, kb * MM_BK);
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp_idx == 1) {
    // ---------------------------------------------------------------- MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, ctx, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        ok = mbar_wait(&full_bar[stage], phase, ctx, 3);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem_a + stage * MM_A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + stage * L::B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < MM_BK / MM_UMMA_K; ++k) {
            const uint64_t a_desc = umma_smem_desc(a_addr + (k >> 1) * p.a_khalf + (k & 1) * (MM_UMMA_K * 2), 16,
                                                   p.a_sbo, p.swz);
            const uint64_t b_desc = umma_smem_desc(b_addr + k * p.b_kstep, p.b_lbo, p.b_sbo, p.swz);
            umma_ss(d_tmem, a_desc, b_desc, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // slot reusable once these MMAs have read it
          if (kb == p.num_kb - 1) umma_commit(&tmem_full_bar[acc]);  // accumulator complete
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp_idx & 3;  // TMEM lane quarter this warp may read
    const int ew = warp_idx - 2;
    uint8_t* my_stage = smem_c + ew * 2 * MM_C_BUF_BYTES;
    int it = 0;
    int buf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
      int pid_m, pid_n;
      tile_coords(p, tile, pid_m, pid_n);
      const int m0 = pid_m * MM_BM, n0 = pid_n * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(&tmem_full_bar[acc], acc_phase, ctx, 4);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + q * 32 + static_cast<int>(lane);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(t_row + c * 64, v0);
        tmem_ld_x32(t_row + c * 64 + 32, v1);
        tmem_wait_ld();
        if (c == BN / 64 - 1) {
          // whole accumulator is in registers / already stored: hand the TMEM buffer back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        }
        epilogue_chunk(p, &tmap_c, extra.m, v0, v1, row, m0 + q * 32, n0 + c * 64, my_stage, buf, lane);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown
  drain_after_abort(abort_smem);
  tc_fence_before();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// =============================================================================================
// CTA-pair variant (cta_group::2): two CTAs of a cluster share one 256 x 256 output tile.
// CTA r of the pair loads its own 128 rows of A and its own 128-column half of B (so each SM moves
// 32 KB per K block instead of 48 KB), the pair leader issues one M = 256 MMA per K step that reads
// both CTAs' shared memory, and each CTA's tensor memory receives its 128 rows x 256 columns of the
// accumulator.  Loads of both CTAs are counted on the leader's "full" barrier; the leader's commits
// release the ring slot in both CTAs and publish the accumulator to both epilogues.
// =============================================================================================
constexpr int MM2_BN = 256;                                  // tile columns (both CTAs)

struct PairWork {
  int pid_m, pid_n;
  int col0;    // first column of the work item
  int width;   // 256, or 128 for a half tile
};
__device__ __forceinline__ PairWork pair_work(const MatmulParams& p, int w) {
  PairWork r;
  int tile = w, half = 0;
  r.width = MM2_BN;
  if (w >= p.full_work) {
    const int t = w - p.full_work;
    tile = p.full_work + (t >> 1);
    half = t & 1;
    r.width = MM2_BN / 2;
  }
  tile_coords(p, tile, r.pid_m, r.pid_n);
  r.col0 = r.pid_n * MM2_BN + half * (MM2_BN / 2);
  return r;
}
constexpr int MM2_B_STAGE_BYTES = 2 * MM_B_BOX_BYTES;        // this CTA's 64 x 128 half of B: 16 KB
constexpr int MM2_STAGE_BYTES = MM_A_STAGE_BYTES + MM2_B_STAGE_BYTES;  // 32 KB per CTA per K block

template <int STAGES>
struct Matmul2Smem {
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = STAGES * MM_A_STAGE_BYTES;
  static constexpr int C_OFF = B_OFF + STAGES * MM2_B_STAGE_BYTES;
  static constexpr int BAR_OFF = C_OFF + MM_C_STAGING_BYTES;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = BAR_OFF + BAR_BYTES + 1024;
};

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MM_THREADS, 1)
matmul_bf16_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ ExtraMaps extra,
                                const MatmulParams p) {
  using L = Matmul2Smem<STAGES>;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem + L::A_OFF;
  uint8_t* smem_b = smem + L::B_OFF;
  uint8_t* smem_c = smem + L::C_OFF;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);   // used in the leader only
  uint64_t* empty_bar = full_bar + STAGES;                               // one set per CTA
  uint64_t* tmem_full_bar = empty_bar + STAGES;                          // one set per CTA
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;                          // used in the leader only
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_ctarank();      // 0 = pair leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);       // the leader's producer arrives once (with the byte count of both CTAs)
      mbar_init(&empty_bar[s], 1);      // one commit from the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);                   // one commit from the leader's MMA thread
      mbar_init(&tmem_empty_bar[a], 2 * MM_EPI_WARPS);   // epilogue warps of both CTAs
    }
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp_idx == 1) {
    tmem_alloc_2cta(tmem_ptr_smem, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must exist before either CTA signals the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp_idx == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // The A row panel of a tile group is re-read by every tile column of the sweep; B tiles stream.
    const uint64_t pol_a = p.l2_hint ? l2_policy_evict_last() : l2_policy_evict_normal();
    const uint64_t pol_b = p.l2_hint == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
    for (int work = pair; ok && work < p.num_work; work += num_pairs) {
      const PairWork wk = pair_work(p, work);
      const int m0 = wk.pid_m * 256 + static_cast<int>(rank) * MM_BM;
      const int n0 = wk.col0 + static_cast<int>(rank) * (wk.width / 2);   // this CTA's half of the item's columns
      const int b_boxes = wk.width / 128;                                  // 64-column boxes this CTA loads
      for (int kb = 0; kb < p.num_kb; ++kb) {
        ok = mbar_wait(&empty_bar[stage], phase ^ 1u, ctx, 41);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t leader_full = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * (MM_A_STAGE_BYTES + b_boxes * MM_B_BOX_BYTES));
          if (p.tile32) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_tile32_2cta_hint(smem_a + stage * MM_A_STAGE_BYTES + j * (MM_A_STAGE_BYTES / 2), &tmap_a,
                                        leader_full, kb * 2 + j, m0 >> 5, pol_a);
            for (int i = 0; i < 2 * b_boxes; ++i)
              tma_load_tile32_2cta_hint(smem_b + stage * MM2_B_STAGE_BYTES + i * (MM_B_BOX_BYTES / 2), &tmap_b,
                                        leader_full, (n0 >> 5) + i, kb * 2, pol_b);
          } else {
            tma_load_2d_2cta_hint(smem_a + stage * MM_A_STAGE_BYTES, &tmap_a, leader_full, kb * MM_BK, m0, pol_a);
            for (int i = 0; i < b_boxes; ++i)
              tma_load_2d_2cta_hint(smem_b + stage * MM2_B_STAGE_BYTES + i * MM_B_BOX_BYTES, &tmap_b, leader_full,
                                    n0 + i * 64, kb * MM_BK, pol_b);
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp_idx == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int work = pair; ok && work < p.num_work; work += num_pairs, ++it) {
        const uint32_t idesc = work >= p.full_work ? p.idesc_half : p.idesc;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, ctx, 42);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * MM2_BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, ctx, 43);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_addr = smem_u32(smem_a + stage * MM_A_STAGE_BYTES);
            const uint32_t b_addr = smem_u32(smem_b + stage * MM2_B_STAGE_BYTES);
#pragma unroll
            for (int k = 0; k < MM_BK / MM_UMMA_K; ++k) {
              const uint64_t a_desc = umma_smem_desc(a_addr + (k >> 1) * p.a_khalf + (k & 1) * (MM_UMMA_K * 2), 16,
                                                     p.a_sbo, p.swz);
              const uint64_t b_desc = umma_smem_desc(b_addr + k * p.b_kstep, p.b_lbo, p.b_sbo, p.swz);
              umma_ss_2cta(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            // release this ring slot in both CTAs once the MMAs above have read it
            const uint32_t e = smem_u32(&empty_bar[stage]);
            umma_commit_2cta(mapa_shared(e, 0));
            umma_commit_2cta(mapa_shared(e, 1));
            if (kb == p.num_kb - 1) {  // accumulator complete: wake both epilogues
              const uint32_t f = smem_u32(&tmem_full_bar[acc]);
              umma_commit_2cta(mapa_shared(f, 0));
              umma_commit_2cta(mapa_shared(f, 1));
            }
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int q = warp_idx & 3;
    const int ew = warp_idx - 2;
    uint8_t* my_stage = smem_c + ew * 2 * MM_C_BUF_BYTES;
    int it = 0;
    int buf = 0;
    bool ok = true;
    for (int work = pair; ok && work < p.num_work; work += num_pairs, ++it) {
      const PairWork wk = pair_work(p, work);
      const int m0 = wk.pid_m * 256 + static_cast<int>(rank) * MM_BM;
      const int n0 = wk.col0;
      const int chunks = wk.width / 64;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(&tmem_full_bar[acc], acc_phase, ctx, 44);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + q * 32 + static_cast<int>(lane);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * MM2_BN;
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_x32(t_row + c * 64, v0);
        tmem_ld_x32(t_row + c * 64 + 32, v1);
        tmem_wait_ld();
        if (c == chunks - 1) {
          // this warp's part of the accumulator has left tensor memory: tell the leader's MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&tmem_empty_bar[acc]), 0));   // tensor-memory data only: CTA-scope release
        }
        epilogue_chunk(p, &tmap_c, extra.m, v0, v1, row, m0 + q * 32, n0 + c * 64, my_stage, buf, lane);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown
  drain_after_abort(abort_smem);
  // Neither CTA may exit (or free tensor memory) while its partner can still signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp_idx == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Host launcher
// ---------------------------------------------------------------------------------------------
// Tensor maps of A, B and C.  Row-major: boxes of 128 x 64, 64 x 64 and 32 x 64 elements, 128-byte swizzle.
// Tile-major: boxes of 128 x 32, 64 x 32 and 32 x 32 elements (one tile column), 64-byte swizzle.
static void set_operand_images(MatmulParams* p, int tile32) {
  if (tile32) {
    p->swz = UMMA_LAYOUT_SW64;
    p->a_sbo = 512;                     // 8 rows of 64 bytes
    p->a_khalf = MM_A_STAGE_BYTES / 2;  // k = 32..63 live in the second 128 x 32 half
    p->b_lbo = MM_B_BOX_BYTES / 2;      // next 32-column chunk of N = next 4 KB box
    p->b_sbo = 512;                     // next group of 8 k-rows
    p->b_kstep = MM_UMMA_K * 64;        // 16 k-rows of 64 bytes
  } else {
    p->swz = UMMA_LAYOUT_SW128;
    p->a_sbo = 1024;                    // 8 rows of 128 bytes
    p->a_khalf = 2 * MM_UMMA_K * 2;     // one row holds all 64 k: k-steps advance by 32 bytes
    p->b_lbo = MM_B_BOX_BYTES;          // next 64-column chunk of N = next 8 KB box
    p->b_sbo = 1024;                    // next group of 8 k-rows
    p->b_kstep = MM_UMMA_K * 128;       // 16 k-rows of 128 bytes
  }
}

static int make_operand_tmaps(const MatmulArgs& a, CUtensorMap* ta, CUtensorMap* tb, CUtensorMap* tc, ExtraMaps* extra) {
  int rc;
  memset(extra, 0, sizeof(*extra));
  for (int d = 0; d < a.n_extra; ++d)
    if ((rc = make_tmap_bf16_2d(&extra->m[d], a.extra_C[d], a.N, a.M, a.ldc, 64, 32)) != 0) return rc;
  if (a.tile32) {
    if ((rc = make_tmap_tile32(ta, a.A, a.K, a.M, MM_BM, /*row_pairs=*/true)) != 0) return rc;
    if ((rc = make_tmap_tile32(tb, a.B, a.N, a.K, MM_BK)) != 0) return rc;
    return make_tmap_tile32(tc, a.C, a.N, a.M, 32);
  }
  if ((rc = make_tmap_bf16_2d(ta, a.A, a.K, a.M, a.lda, 64, MM_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(tb, a.B, a.N, a.K, a.ldb, 64, MM_BK)) != 0) return rc;
  return make_tmap_bf16_2d(tc, a.C, a.N, a.M, a.ldc, 64, 32);
}

template <int BN, int STAGES>
static int launch_matmul(const MatmulArgs& a, const DeviceInfo* dev, cudaStream_t stream, uint32_t* status) {
  using L = MatmulSmem<BN, STAGES>;
  static_assert(L::TOTAL <= 232448, "shared memory budget exceeded");
  CUtensorMap ta, tb, tc;
  int rc;
  ExtraMaps extra;
  if ((rc = make_operand_tmaps(a, &ta, &tb, &tc, &extra)) != 0) return rc;

  MatmulParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.num_pid_m = (a.M + MM_BM - 1) / MM_BM;
  p.num_pid_n = (a.N + BN - 1) / BN;
  p.group_m = 16;  // 16 tile rows of 128 = 2048 rows of A (33.5 MB at K = 8192) stay hot in L2
  if (const char* g = getenv("B200K_MATMUL_GROUP_M")) { int v = atoi(g); if (v > 0) p.group_m = v; }
  p.serpentine = 1;
  if (const char* g = getenv("B200K_MATMUL_SERPENTINE")) p.serpentine = atoi(g) != 0;
  p.num_tiles = p.num_pid_m * p.num_pid_n;
  p.num_kb = (a.K + MM_BK - 1) / MM_BK;
  p.bias_row = (a.bias_kind == B200K_BIAS_ROW_F32) ? static_cast<const float*>(a.bias) : nullptr;
  p.bias_full = (a.bias_kind == B200K_BIAS_FULL_BF16) ? static_cast<const uint16_t*>(a.bias) : nullptr;
  p.ldbias = a.ldbias;
  p.act = a.act;
  p.round_before_bias = a.round_before_bias;
  set_operand_images(&p, a.tile32);
  p.l2_hint = 0;
  p.f16 = a.dtype;
  p.tile32 = a.tile32;
  p.n_extra = a.n_extra;
  p.idesc = umma_idesc_16bit_f32(MM_BM, BN, /*a_mn_major=*/0, /*b_mn_major=*/1, a.dtype);
  p.idesc_half = p.idesc;   // the pair kernel's fields, unused here
  p.num_work = p.full_work = p.num_tiles;
  p.status = status;

  // per device (function attributes belong to the current context), cheap enough to repeat
  B200K_CHECK_CUDA(cudaFuncSetAttribute(matmul_bf16_tcgen05_kernel<BN, STAGES>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  matmul_bf16_tcgen05_kernel<BN, STAGES><<<grid, MM_THREADS, L::TOTAL, stream>>>(ta, tb, tc, extra, p);
  count_launch();
  B200K_CHECK_LAUNCH("matmul_bf16_tcgen05_kernel");
  return B200K_OK;
}

// How the CTA-pair kernel runs the `rest` tiles left after the full waves of `pairs` pairs, from measured costs in
// units of one whole-tile wave (M x 8192 x 8192 on one B200, whole / column halves):
//   whole tiles     1     always possible
//   column halves   each leftover tile as two 256 x 128 items on twice as many pairs; possible when 2 * rest <= pairs;
//                   about 0.55-0.6 of a wave (M = 1280, 12 left: 135.1 -> 130.6 us; 2048, 34 left: 199.0 -> 186.1;
//                   3072, 14 left: 291.3 -> 281.0)
// A third form was built and measured and is NOT used: the leftover tiles' K blocks dealt out in equal shares, one per
// pair, with fp32 partial sums through a workspace (M = 1024, 54 left: 99.8 -> 115.5 us; 8192, 62 left: 794 -> 838;
// correct to 1 bf16 ulp, but the shares break the locality of all pairs sweeping K together, and two epilogues plus
// the round trip through the workspace end up on the critical path).
// Returns 0 = whole tiles, 1 = column halves.
int matmul_tail_mode(int rest, int pairs) {
  if (rest <= 0 || rest >= pairs) return 0;
  return 2 * rest <= pairs ? 1 : 0;
}

int matmul_tail_plan(int M, int N, int K, int sm_count, int* out) {
  const int tiles = ((M + 255) / 256) * ((N + MM2_BN - 1) / MM2_BN);
  const int max_pairs = sm_count / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  const int rest = pairs > 0 ? tiles % pairs : 0;
  const int mode = matmul_tail_mode(rest, pairs);
  out[0] = mode;
  out[1] = rest;
  out[2] = pairs;
  out[3] = tiles / (pairs > 0 ? pairs : 1);                  // full waves
  out[4] = mode == 1 ? 2 * rest : rest;                      // work items of the last wave
  (void)K;
  return 0;
}

template <int STAGES>
static int launch_matmul_2cta(const MatmulArgs& a, const DeviceInfo* dev, cudaStream_t stream, uint32_t* status) {
  using L = Matmul2Smem<STAGES>;
  static_assert(L::TOTAL <= 232448, "shared memory budget exceeded");
  CUtensorMap ta, tb, tc;
  int rc;
  ExtraMaps extra;
  if ((rc = make_operand_tmaps(a, &ta, &tb, &tc, &extra)) != 0) return rc;

  MatmulParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.num_pid_m = (a.M + 255) / 256;
  p.num_pid_n = (a.N + MM2_BN - 1) / MM2_BN;
  p.group_m = 8;  // 8 tile rows of 256 = 2048 rows of A stay hot in L2 while the tile columns stream
  if (const char* g = getenv("B200K_MATMUL_GROUP_M")) { int v = atoi(g); if (v > 0) p.group_m = v; }
  p.serpentine = 1;
  if (const char* g = getenv("B200K_MATMUL_SERPENTINE")) p.serpentine = atoi(g) != 0;
  p.num_tiles = p.num_pid_m * p.num_pid_n;
  p.num_kb = (a.K + MM_BK - 1) / MM_BK;
  p.bias_row = (a.bias_kind == B200K_BIAS_ROW_F32) ? static_cast<const float*>(a.bias) : nullptr;
  p.bias_full = (a.bias_kind == B200K_BIAS_FULL_BF16) ? static_cast<const uint16_t*>(a.bias) : nullptr;
  p.ldbias = a.ldbias;
  p.act = a.act;
  p.round_before_bias = a.round_before_bias;
  set_operand_images(&p, a.tile32);
  p.f16 = a.dtype;
  p.tile32 = a.tile32;
  p.n_extra = a.n_extra;
  p.idesc = umma_idesc_16bit_f32(256, MM2_BN, /*a_mn_major=*/0, /*b_mn_major=*/1, a.dtype);
  p.idesc_half = umma_idesc_16bit_f32(256, MM2_BN / 2, /*a_mn_major=*/0, /*b_mn_major=*/1, a.dtype);
  p.l2_hint = 2;  // keep the group's A row panel in L2 (measured +2 % at 8192^3 over no hint; B evict_first loses)
  if (const char* h = getenv("B200K_MATMUL_L2_HINT")) p.l2_hint = atoi(h);
  p.status = status;

  B200K_CHECK_CUDA(cudaFuncSetAttribute(matmul_bf16_tcgen05_2cta_kernel<STAGES>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  const int max_pairs = dev->sm_count / 2;
  const int pairs = p.num_tiles < max_pairs ? p.num_tiles : max_pairs;
  // The last wave: if its tiles occupy at most half of the pairs, cut them in two so that it takes half as long
  // (4096^3: 256 tiles on 74 pairs = 3 waves + 34 tiles -> 3 waves + 68 half tiles).
  p.num_work = p.full_work = p.num_tiles;
  const int rest = p.num_tiles % pairs;
  const char* split_env = getenv("B200K_MATMUL_SPLIT_TAIL");
  if (matmul_tail_mode(rest, pairs) == 1 && !(split_env != nullptr && atoi(split_env) == 0)) {
    p.full_work = p.num_tiles - rest;
    p.num_work = p.full_work + 2 * rest;
  }
  matmul_bf16_tcgen05_2cta_kernel<STAGES><<<2 * pairs, MM_THREADS, L::TOTAL, stream>>>(ta, tb, tc, extra, p);
  count_launch();
  B200K_CHECK_LAUNCH("matmul_bf16_tcgen05_2cta_kernel");
  return B200K_OK;
}

int matmul_bf16(const MatmulArgs& a, cudaStream_t stream, uint32_t* status_override) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return set_error(B200K_ERR_INVALID_ARG, "matmul: M, N, K must be positive (got %d, %d, %d)", a.M, a.N, a.K);
  if (a.A == nullptr || a.B == nullptr || a.C == nullptr) return set_error(B200K_ERR_INVALID_ARG, "matmul: null operand pointer");
  if (a.tile32) {
    if ((a.M & 31) || (a.N & 31) || (a.K & 31))
      return set_error(B200K_ERR_INVALID_ARG, "matmul: tile-major operands need M, N, K multiples of 32 (got %d, %d, %d)", a.M, a.N, a.K);
    if (a.bias_kind != B200K_BIAS_NONE) return set_error(B200K_ERR_INVALID_ARG, "matmul: tile-major operands take no bias");
    if (a.n_extra != 0) return set_error(B200K_ERR_INVALID_ARG, "matmul: tile-major operands take no extra destinations");
  } else {
    if (a.lda < a.K || a.ldb < a.N || a.ldc < a.N) return set_error(B200K_ERR_INVALID_ARG, "matmul: leading dimension smaller than the row length");
    if ((a.lda & 7) || (a.ldb & 7) || (a.ldc & 7))
      return set_error(B200K_ERR_INVALID_ARG, "matmul: lda/ldb/ldc must be multiples of 8 elements (16-byte rows for TMA); got %lld, %lld, %lld",
                       (long long)a.lda, (long long)a.ldb, (long long)a.ldc);
  }
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B) | reinterpret_cast<uintptr_t>(a.C)) & 15u)
    return set_error(B200K_ERR_INVALID_ARG, "matmul: A, B and C must be 16-byte aligned");
  if (a.n_extra < 0 || a.n_extra > MM_MAX_EXTRA || (a.n_extra > 0 && a.extra_C == nullptr))
    return set_error(B200K_ERR_INVALID_ARG, "matmul: 0..%d extra destinations supported (got %d)", MM_MAX_EXTRA, a.n_extra);
  for (int d = 0; d < a.n_extra; ++d)
    if (a.extra_C[d] == nullptr || (reinterpret_cast<uintptr_t>(a.extra_C[d]) & 15u))
      return set_error(B200K_ERR_INVALID_ARG, "matmul: extra destination %d is null or not 16-byte aligned", d);
  if (a.bias_kind < B200K_BIAS_NONE || a.bias_kind > B200K_BIAS_FULL_BF16) return set_error(B200K_ERR_INVALID_ARG, "matmul: bad bias_kind %d", a.bias_kind);
  if (a.dtype != 0 && a.dtype != 1) return set_error(B200K_ERR_INVALID_ARG, "matmul: bad element type %d", a.dtype);
  if (a.act < B200K_ACT_NONE || a.act > B200K_ACT_LEAKY_RELU) return set_error(B200K_ERR_INVALID_ARG, "matmul: bad act %d", a.act);
  if (a.bias_kind != B200K_BIAS_NONE && a.bias == nullptr) return set_error(B200K_ERR_INVALID_ARG, "matmul: bias_kind %d needs a bias pointer", a.bias_kind);
  if (a.bias_kind == B200K_BIAS_ROW_F32 && (reinterpret_cast<uintptr_t>(a.bias) & 15u))
    return set_error(B200K_ERR_INVALID_ARG, "matmul: bias[N] must be 16-byte aligned");
  if (a.bias_kind == B200K_BIAS_FULL_BF16 && a.ldbias < a.N) return set_error(B200K_ERR_INVALID_ARG, "matmul: ldbias smaller than N");
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  if (dev->cc_major != 10) return set_error(B200K_ERR_NO_DEVICE, "matmul: needs an sm_100 device (found sm_%d%d)", dev->cc_major, dev->cc_minor);
  uint32_t* status = status_override ? status_override : dev->status_word;

  // 128x256 tiles unless that leaves SMs idle and narrower tiles would not.
  const int64_t tiles256 = static_cast<int64_t>((a.M + MM_BM - 1) / MM_BM) * ((a.N + 255) / 256);
  bool narrow = (a.N <= 128) || (tiles256 < dev->sm_count);
  if (const char* f = getenv("B200K_MATMUL_BN")) { int v = atoi(f); if (v == 128) narrow = true; if (v == 256) narrow = false; }
  // CTA pairs on 256 x 256 tiles when there are enough of them to occupy every pair of SMs.
  const int64_t tiles2 = static_cast<int64_t>((a.M + 255) / 256) * ((a.N + 255) / 256);
  bool pair = tiles2 >= dev->sm_count / 2;
  if (const char* f = getenv("B200K_MATMUL_2CTA")) pair = atoi(f) != 0;
  if (pair) return launch_matmul_2cta<6>(a, dev, stream, status);
  if (narrow) return launch_matmul<128, 6>(a, dev, stream, status);
  return launch_matmul<256, 4>(a, dev, stream, status);
}

}  // namespace b200k
