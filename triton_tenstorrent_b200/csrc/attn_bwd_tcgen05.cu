// Fused attention backward for sm_100a, HEAD_DIM 128, N_CTX a multiple of 128: dQ, dK, dV from Q, K, V, O, dO and the
// row statistics M = m + log2(l) that the forward saves for exactly this purpose
// (examples/fused-attn/06-fused-attention.py:238,269: `ctx.save_for_backward(q, k, v, o, M)`).  The reference stops
// there (it has no backward kernel); this file completes the pair with the algorithm of the Triton tutorial the
// reference's forward was taken from, in the forward's own conventions (base-2 domain, scale applied in fp32 after
// the MMA, 16-bit rounding only where a value becomes a tensor-core operand):
//   delta_i = sum_d O_id dO_id                                  (fp32, a small kernel of its own)
//   P_ij    = exp2(qk_scale * (Q K^T)_ij - M_i)                 (already normalised: M carries log2 l)
//   dV_j    = sum_i bf16(P_ij) dO_i
//   dP_ij   = dO_i . V_j
//   dS_ij   = P_ij (dP_ij - delta_i)                            (P in fp32 here, as in the tutorial)
//   dK_j    = sm_scale * sum_i bf16(dS_ij) Q_i        dQ_i = sm_scale * sum_j bf16(dS_ij) K_j
// Two kernels, both deterministic (no atomics): one CTA per 128-key block accumulates dK and dV over the query blocks,
// one CTA per 128-query block accumulates dQ over the key blocks; each recomputes S and dP with tcgen05 MMAs.
//
//   warps 0-7  two threads per row of the score tile (warps 0-3 columns 0-63, warps 4-7 columns 64-127; the backward has
//              no row reductions, M and delta are given, so the two halves never talk): tcgen05.ld S and dP,
//              exponentials, dS, bf16 results written back over S / dP in tensor memory; epilogue (scale, downcast,
//              swizzled staging, TMA store), again one 64-column half each.  Two warps per scheduler instead
//              of one: 4.48 -> 4.30 ms at Z=4, H=32, N_CTX=4096
//   warp 8     TMA producer (the item's resident tiles; a two-stage ring of the tiles that stream)
//   warp 9     tensor-memory owner and tcgen05.mma issuer
// Tensor memory: dK/dV kernel S^T | dP^T | dV | dK (128 fp32 columns each, rows = keys); dQ kernel S | dP | dQ.
// Per streamed block the chain MMA(S, dP) -> exponentials -> MMA(gradients) is serial (tensor memory holds one block),
// only the loads run ahead.
#include <math.h>
#include <string.h>

#include "attn_common.cuh"
#include "launch.h"
#include "ptx.cuh"

namespace b200k {

constexpr int BW_D = 128;
constexpr int BW_THREADS = 320;
constexpr int BW_SCORE_WARPS = 8;
constexpr int BW_WARP_TMA = 8, BW_WARP_MMA = 9;
constexpr int BW_TILE_BYTES = AT_BM * BW_D * 2;       // 32 KB: two boxes of 128 rows x 64 columns
constexpr int BW_NSTAGE = 2;

struct BwdParams {
  int ZH, N_CTX, num_blk;
  int num_items;        // ZH * num_blk
  int causal;
  float qk_scale;       // sm_scale * 1.44269504
  float sm_scale;
  const float* lse2;    // M of the forward, [ZH, N_CTX]
  const float* delta;   // [ZH, N_CTX]
  uint32_t* status;
};

// ---------------------------------------------------------------------------------------------------------------
// delta = rowsum(O * dO): one warp per row of 128 bf16 values
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const uint2* __restrict__ o, const uint2* __restrict__ d_o,
                                                             float* __restrict__ delta, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const uint2 a = __ldg(o + row * 32 + lane), b = __ldg(d_o + row * 32 + lane);   // four bf16 each
    float s = bf16_bits_to_f32(a.x & 0xFFFFu) * bf16_bits_to_f32(b.x & 0xFFFFu);
    s = fmaf(bf16_bits_to_f32(a.x >> 16), bf16_bits_to_f32(b.x >> 16), s);
    s = fmaf(bf16_bits_to_f32(a.y & 0xFFFFu), bf16_bits_to_f32(b.y & 0xFFFFu), s);
    s = fmaf(bf16_bits_to_f32(a.y >> 16), bf16_bits_to_f32(b.y >> 16), s);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    if (lane == 0) delta[row] = s;
  }
}

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Offsets (bytes) of the k-step `kk` (16 elements of the contraction) inside a 128 x 128 tile of two 64-column boxes:
// contraction along the tile's columns (K-major operand) / along its rows (MN-major operand).
__device__ __forceinline__ uint64_t koff_cols(int kk) {
  return static_cast<uint64_t>(((kk >> 2) * AT_BOX_BYTES + (kk & 3) * 32) >> 4);
}
__device__ __forceinline__ uint64_t koff_rows(int kk) { return static_cast<uint64_t>((kk * 2048) >> 4); }

// One 128 x 128 tile: two TMA boxes.
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row) {
  tma_load_2d(dst, m, bar, 0, row);
  tma_load_2d(dst + AT_BOX_BYTES, m, bar, 64, row);
}

// Epilogue of one accumulator: 128 rows x 128 fp32 columns of tensor memory -> x scale -> bf16 -> swizzled staging in
// shared memory (a tile that is no longer needed); the caller issues the TMA stores of its 32 rows.
// Tensor-memory column (relative to the fp32 score tile) of the bf16 operand's k-step kk (16 scores = 8 columns): the
// two column halves are each packed at the start of their own 64 columns, so that no warp writes where another reads.
__device__ __forceinline__ constexpr uint32_t bf16_col(int kk) { return kk < 4 ? kk * 8 : 64 + (kk - 4) * 8; }

__device__ __forceinline__ void store_acc(uint32_t t_acc, float scale, uint8_t* stage, int r, int half) {
#pragma unroll 1
  for (int c4 = 2 * half; c4 < 2 * half + 2; ++c4) {   // this thread's 64 columns = one 64-column box
    uint32_t o[32];
    tmem_ld_x32(t_acc + c4 * 32, o);
    tmem_wait_ld();
    uint8_t* row_ptr = stage + (c4 >> 1) * AT_BOX_BYTES + r * 128;
    const int chunk0 = (c4 & 1) * 4;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      uint4 val;
      val.x = pack_bf16x2(__uint_as_float(o[8 * jj + 0]) * scale, __uint_as_float(o[8 * jj + 1]) * scale);
      val.y = pack_bf16x2(__uint_as_float(o[8 * jj + 2]) * scale, __uint_as_float(o[8 * jj + 3]) * scale);
      val.z = pack_bf16x2(__uint_as_float(o[8 * jj + 4]) * scale, __uint_as_float(o[8 * jj + 5]) * scale);
      val.w = pack_bf16x2(__uint_as_float(o[8 * jj + 6]) * scale, __uint_as_float(o[8 * jj + 7]) * scale);
      *reinterpret_cast<uint4*>(row_ptr + (((chunk0 + jj) ^ (r & 7)) << 4)) = val;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dK and dV: one item = (batch*head, key block n); the query blocks m stream (m >= n when causal)
// ---------------------------------------------------------------------------------------------------------------
constexpr int KV_STAGE_BYTES = 2 * BW_TILE_BYTES + 1024;          // Q tile, dO tile, 128 M values, 128 delta values
constexpr int KV_RES_OFF = 0;                                     // K tile, V tile (resident per item)
constexpr int KV_STAGE_OFF = 2 * BW_TILE_BYTES;
constexpr int KV_BAR_OFF = KV_STAGE_OFF + BW_NSTAGE * KV_STAGE_BYTES;
constexpr int KV_NBAR = 2 + 2 * BW_NSTAGE + 4;
constexpr int KV_SMEM_TOTAL = KV_BAR_OFF + KV_NBAR * 8 + 16 + 1024;
static_assert(KV_SMEM_TOTAL <= 232448, "attention backward (dK/dV) shared memory budget exceeded");

__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dkdv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                             const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                             const __grid_constant__ CUtensorMap tmap_dk, const __grid_constant__ CUtensorMap tmap_dv,
                             const BwdParams p) {
  constexpr uint32_t IDESC_SS = umma_idesc_bf16_f32(AT_BM, AT_BN, 0, 0);   // both operands K-major
  constexpr uint32_t IDESC_TS = umma_idesc_bf16_f32(AT_BM, BW_D, 0, 1);    // A in tensor memory, B MN-major
  constexpr uint32_t C_ST = 0, C_DPT = 128, C_DV = 256, C_DK = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_k = smem + KV_RES_OFF;
  uint8_t* smem_v = smem_k + BW_TILE_BYTES;
  uint8_t* smem_stage = smem + KV_STAGE_OFF;
  uint64_t* res_full = reinterpret_cast<uint64_t*>(smem + KV_BAR_OFF);   // K and V tiles have arrived
  uint64_t* res_empty = res_full + 1;                                    // ... may be overwritten (4 warps)
  uint64_t* st_full = res_empty + 1;                                     // [stage] Q, dO, M, delta have arrived
  uint64_t* st_empty = st_full + BW_NSTAGE;                              // [stage] released by the MMA issuer
  uint64_t* x_full = st_empty + BW_NSTAGE;                               // S^T and dP^T are in tensor memory
  uint64_t* p_ready = x_full + 1;                                        // P^T and dS^T written (4 warps)
  uint64_t* acc_full = p_ready + 1;                                      // dV and dK complete
  uint64_t* acc_empty = acc_full + 1;                                    // ... read out (4 warps)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 1);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    mbar_init(res_full, 1);
    mbar_init(res_empty, BW_SCORE_WARPS);
    for (int s = 0; s < BW_NSTAGE; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&st_empty[s], 1);
    }
    mbar_init(x_full, 1);
    mbar_init(p_ready, BW_SCORE_WARPS);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, BW_SCORE_WARPS);
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
  }
  if (warp_idx == BW_WARP_MMA) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp_idx == BW_WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t stage_phase = 0, items = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      const int hz = item / p.num_blk, n = item - hz * p.num_blk;
      const int row_base = hz * p.N_CTX;
      ok = mbar_wait(res_empty, (items & 1u) ^ 1u, ctx, 80);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(res_full, 2 * BW_TILE_BYTES);
        load_tile(smem_k, &tmap_k, res_full, row_base + n * AT_BN);
        load_tile(smem_v, &tmap_v, res_full, row_base + n * AT_BN);
      }
      __syncwarp();
      for (int m = p.causal ? n : 0; ok && m < p.num_blk; ++m) {
        ok = mbar_wait(&st_empty[stage], stage_phase ^ 1u, ctx, 81);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* dst = smem_stage + stage * KV_STAGE_BYTES;
          mbar_expect_tx(&st_full[stage], 2 * BW_TILE_BYTES + 1024);
          load_tile(dst, &tmap_q, &st_full[stage], row_base + m * AT_BM);
          load_tile(dst + BW_TILE_BYTES, &tmap_do, &st_full[stage], row_base + m * AT_BM);
          bulk_load_1d(dst + 2 * BW_TILE_BYTES, p.lse2 + row_base + m * AT_BM, 512, &st_full[stage]);
          bulk_load_1d(dst + 2 * BW_TILE_BYTES + 512, p.delta + row_base + m * AT_BM, 512, &st_full[stage]);
        }
        __syncwarp();
        if (++stage == BW_NSTAGE) { stage = 0; stage_phase ^= 1u; }
      }
    }
  } else if (warp_idx == BW_WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t stage_phase = 0, items = 0, blocks = 0;
    bool ok = true;
    const uint64_t k_desc = umma_smem_desc_sw128(smem_u32(smem_k), 16, 1024);
    const uint64_t v_desc = umma_smem_desc_sw128(smem_u32(smem_v), 16, 1024);
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      const int hz = item / p.num_blk, n = item - hz * p.num_blk;
      ok = mbar_wait(res_full, items & 1u, ctx, 82);
      if (!ok) break;
      bool first = true;
      for (int m = p.causal ? n : 0; ok && m < p.num_blk; ++m, ++blocks) {
        ok = mbar_wait(&st_full[stage], stage_phase, ctx, 83);
        if (!ok) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(smem_stage + stage * KV_STAGE_BYTES);
        const uint32_t do_addr = q_addr + BW_TILE_BYTES;
        if (lane == 0) {
          // S^T = K Q^T and dP^T = V dO^T: rows = keys, columns = queries, contraction over the head dimension
          const uint64_t qk = umma_smem_desc_sw128(q_addr, 16, 1024), dok = umma_smem_desc_sw128(do_addr, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BW_D / 16; ++kk)
            umma_ss(tmem_base + C_ST, k_desc + koff_cols(kk), qk + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < BW_D / 16; ++kk)
            umma_ss(tmem_base + C_DPT, v_desc + koff_cols(kk), dok + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
          umma_commit(x_full);
        }
        __syncwarp();
        ok = mbar_wait(p_ready, blocks & 1u, ctx, 84);
        if (!ok) break;
        if (first) {   // the previous item's dV / dK must have left tensor memory before they are overwritten
          ok = mbar_wait(acc_empty, (items & 1u) ^ 1u, ctx, 85);
          if (!ok) break;
        }
        tc_fence_after();
        if (lane == 0) {
          // dV += P^T dO and dK += dS^T Q: A from tensor memory (bf16, 8 columns per k-step), contraction over the queries
          const uint64_t qn = umma_smem_desc_sw128(q_addr, AT_BOX_BYTES, 1024);
          const uint64_t don = umma_smem_desc_sw128(do_addr, AT_BOX_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < AT_BM / 16; ++kk)
            umma_ts(tmem_base + C_DV, tmem_base + C_ST + bf16_col(kk), don + koff_rows(kk), IDESC_TS, (!first || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < AT_BM / 16; ++kk)
            umma_ts(tmem_base + C_DK, tmem_base + C_DPT + bf16_col(kk), qn + koff_rows(kk), IDESC_TS, (!first || kk > 0) ? 1u : 0u);
          umma_commit(&st_empty[stage]);
          if (m == p.num_blk - 1) umma_commit(acc_full);
        }
        __syncwarp();
        first = false;
        if (++stage == BW_NSTAGE) { stage = 0; stage_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ score rows (warps 0..7): thread = (key, column half)
    const int q = warp_idx & 3;          // tensor-memory lane quarter
    const int half = warp_idx >> 2;      // columns [64 * half, 64 * half + 64)
    const int r = q * 32 + static_cast<int>(lane);
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_st = tmem_base + lane_field + C_ST, t_dpt = tmem_base + lane_field + C_DPT;
    int stage = 0;
    uint32_t stage_phase = 0, items = 0, blocks = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      const int hz = item / p.num_blk, n = item - hz * p.num_blk;
      for (int m = p.causal ? n : 0; ok && m < p.num_blk; ++m, ++blocks) {
        // the stage's M and delta vectors are read from shared memory below: observe their arrival directly
        ok = mbar_wait(&st_full[stage], stage_phase, ctx, 88);
        if (!ok) break;
        ok = mbar_wait(x_full, blocks & 1u, ctx, 86);
        if (!ok) break;
        tc_fence_after();
        const float* mv = reinterpret_cast<const float*>(smem_stage + stage * KV_STAGE_BYTES + 2 * BW_TILE_BYTES);
        const float* dv = mv + 128;
        const bool diag = p.causal && m == n;
#pragma unroll 1
        for (int c4 = 2 * half; c4 < 2 * half + 2; ++c4) {
          uint32_t s[32], d[32];
          tmem_ld_x32(t_st + c4 * 32, s);
          tmem_ld_x32(t_dpt + c4 * 32, d);
          tmem_wait_ld();
          uint32_t pp[16], ds[16];
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 m4 = *reinterpret_cast<const float4*>(mv + c4 * 32 + c);
            const float4 d4 = *reinterpret_cast<const float4*>(dv + c4 * 32 + c);
            const float mm[4] = {m4.x, m4.y, m4.z, m4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
            float pv[4], dsv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float pe = ex2_approx(fmaf(__uint_as_float(s[c + e]), p.qk_scale, -mm[e]));
              if (diag && c4 * 32 + c + e < r) pe = 0.f;          // query index < key index
              pv[e] = pe;
              dsv[e] = pe * (__uint_as_float(d[c + e]) - dd[e]);
            }
            pp[c / 2] = pack_bf16x2(pv[0], pv[1]);
            pp[c / 2 + 1] = pack_bf16x2(pv[2], pv[3]);
            ds[c / 2] = pack_bf16x2(dsv[0], dsv[1]);
            ds[c / 2 + 1] = pack_bf16x2(dsv[2], dsv[3]);
          }
          // the bf16 results land in columns this thread has already read (16 columns per 32 scores, packed from
          // the start of the thread's own 64-column half: the other half's warps run at their own pace)
          tmem_st_x16(t_st + bf16_col(c4 * 2), pp);
          tmem_st_x16(t_dpt + bf16_col(c4 * 2), ds);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
        if (++stage == BW_NSTAGE) { stage = 0; stage_phase ^= 1u; }
      }
      if (!ok) break;
      // ---- epilogue: dV and sm_scale * dK -> bf16 -> staging in the K / V tiles (no longer needed) -> TMA store
      ok = mbar_wait(acc_full, items & 1u, ctx, 87);
      if (!ok) break;
      tc_fence_after();
      store_acc(tmem_base + lane_field + C_DV, 1.0f, smem_k, r, half);
      store_acc(tmem_base + lane_field + C_DK, p.sm_scale, smem_v, r, half);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(acc_empty);
        const int y = hz * p.N_CTX + n * AT_BN + q * 32;
        tma_store_2d(&tmap_dv, smem_k + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y);
        tma_store_2d(&tmap_dk, smem_v + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y);
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(res_empty);
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown
  drain_after_abort(abort_smem);
  tc_fence_before();
  __syncthreads();
  if (warp_idx == BW_WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dQ: one item = (batch*head, query block m); the key blocks n stream (n <= m when causal)
// ---------------------------------------------------------------------------------------------------------------
constexpr int DQ_STAGE_BYTES = 2 * BW_TILE_BYTES;                 // K tile, V tile
constexpr int DQ_STAGE_OFF = 2 * BW_TILE_BYTES;                   // after the resident Q and dO tiles
constexpr int DQ_BAR_OFF = DQ_STAGE_OFF + BW_NSTAGE * DQ_STAGE_BYTES;
constexpr int DQ_SMEM_TOTAL = DQ_BAR_OFF + KV_NBAR * 8 + 16 + 1024;
static_assert(DQ_SMEM_TOTAL <= 232448, "attention backward (dQ) shared memory budget exceeded");

__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                           const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  constexpr uint32_t IDESC_SS = umma_idesc_bf16_f32(AT_BM, AT_BN, 0, 0);
  constexpr uint32_t IDESC_TS = umma_idesc_bf16_f32(AT_BM, BW_D, 0, 1);
  constexpr uint32_t C_S = 0, C_DP = 128, C_DQ = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;
  uint8_t* smem_do = smem + BW_TILE_BYTES;
  uint8_t* smem_stage = smem + DQ_STAGE_OFF;
  uint64_t* res_full = reinterpret_cast<uint64_t*>(smem + DQ_BAR_OFF);
  uint64_t* res_empty = res_full + 1;
  uint64_t* st_full = res_empty + 1;
  uint64_t* st_empty = st_full + BW_NSTAGE;
  uint64_t* x_full = st_empty + BW_NSTAGE;
  uint64_t* p_ready = x_full + 1;
  uint64_t* acc_full = p_ready + 1;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 1);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    mbar_init(res_full, 1);
    mbar_init(res_empty, BW_SCORE_WARPS);
    for (int s = 0; s < BW_NSTAGE; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&st_empty[s], 1);
    }
    mbar_init(x_full, 1);
    mbar_init(p_ready, BW_SCORE_WARPS);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, BW_SCORE_WARPS);
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
  }
  if (warp_idx == BW_WARP_MMA) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // causal items take m + 1 blocks: hand out the long ones first
  auto item_block = [&](int item, int& hz, int& m) {
    hz = item / p.num_blk;
    m = item - hz * p.num_blk;
    if (p.causal) m = p.num_blk - 1 - m;
  };

  if (warp_idx == BW_WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t stage_phase = 0, items = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, m;
      item_block(item, hz, m);
      const int row_base = hz * p.N_CTX;
      ok = mbar_wait(res_empty, (items & 1u) ^ 1u, ctx, 90);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(res_full, 2 * BW_TILE_BYTES);
        load_tile(smem_q, &tmap_q, res_full, row_base + m * AT_BM);
        load_tile(smem_do, &tmap_do, res_full, row_base + m * AT_BM);
      }
      __syncwarp();
      const int n_end = p.causal ? m + 1 : p.num_blk;
      for (int n = 0; ok && n < n_end; ++n) {
        ok = mbar_wait(&st_empty[stage], stage_phase ^ 1u, ctx, 91);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* dst = smem_stage + stage * DQ_STAGE_BYTES;
          mbar_expect_tx(&st_full[stage], 2 * BW_TILE_BYTES);
          load_tile(dst, &tmap_k, &st_full[stage], row_base + n * AT_BN);
          load_tile(dst + BW_TILE_BYTES, &tmap_v, &st_full[stage], row_base + n * AT_BN);
        }
        __syncwarp();
        if (++stage == BW_NSTAGE) { stage = 0; stage_phase ^= 1u; }
      }
    }
  } else if (warp_idx == BW_WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t stage_phase = 0, items = 0, blocks = 0;
    bool ok = true;
    const uint64_t q_desc = umma_smem_desc_sw128(smem_u32(smem_q), 16, 1024);
    const uint64_t do_desc = umma_smem_desc_sw128(smem_u32(smem_do), 16, 1024);
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, m;
      item_block(item, hz, m);
      ok = mbar_wait(res_full, items & 1u, ctx, 92);
      if (!ok) break;
      const int n_end = p.causal ? m + 1 : p.num_blk;
      for (int n = 0; ok && n < n_end; ++n, ++blocks) {
        ok = mbar_wait(&st_full[stage], stage_phase, ctx, 93);
        if (!ok) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem_stage + stage * DQ_STAGE_BYTES);
        const uint32_t v_addr = k_addr + BW_TILE_BYTES;
        if (lane == 0) {
          // S = Q K^T and dP = dO V^T: rows = queries, columns = keys
          const uint64_t kk_desc = umma_smem_desc_sw128(k_addr, 16, 1024), vk_desc = umma_smem_desc_sw128(v_addr, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BW_D / 16; ++kk)
            umma_ss(tmem_base + C_S, q_desc + koff_cols(kk), kk_desc + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < BW_D / 16; ++kk)
            umma_ss(tmem_base + C_DP, do_desc + koff_cols(kk), vk_desc + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
          umma_commit(x_full);
        }
        __syncwarp();
        ok = mbar_wait(p_ready, blocks & 1u, ctx, 94);
        if (!ok) break;
        if (n == 0) {
          ok = mbar_wait(acc_empty, (items & 1u) ^ 1u, ctx, 95);
          if (!ok) break;
        }
        tc_fence_after();
        if (lane == 0) {
          // dQ += dS K: A = dS (bf16 in tensor memory over S), contraction over the keys
          const uint64_t kn_desc = umma_smem_desc_sw128(k_addr, AT_BOX_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < AT_BN / 16; ++kk)
            umma_ts(tmem_base + C_DQ, tmem_base + C_S + bf16_col(kk), kn_desc + koff_rows(kk), IDESC_TS, (n > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&st_empty[stage]);
          if (n == n_end - 1) umma_commit(acc_full);
        }
        __syncwarp();
        if (++stage == BW_NSTAGE) { stage = 0; stage_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ score rows (warps 0..7): thread = (query, column half)
    const int q = warp_idx & 3;          // tensor-memory lane quarter
    const int half = warp_idx >> 2;      // columns [64 * half, 64 * half + 64)
    const int r = q * 32 + static_cast<int>(lane);
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + C_S, t_dp = tmem_base + lane_field + C_DP;
    uint32_t items = 0, blocks = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, m;
      item_block(item, hz, m);
      const int64_t my_row = static_cast<int64_t>(hz) * p.N_CTX + m * AT_BM + r;
      const float m_i = __ldg(p.lse2 + my_row), d_i = __ldg(p.delta + my_row);
      const int n_end = p.causal ? m + 1 : p.num_blk;
      for (int n = 0; ok && n < n_end; ++n, ++blocks) {
        ok = mbar_wait(x_full, blocks & 1u, ctx, 96);
        if (!ok) break;
        tc_fence_after();
        const bool diag = p.causal && n == m;
#pragma unroll 1
        for (int c4 = 2 * half; c4 < 2 * half + 2; ++c4) {
          uint32_t s[32], d[32];
          tmem_ld_x32(t_s + c4 * 32, s);
          tmem_ld_x32(t_dp + c4 * 32, d);
          tmem_wait_ld();
          uint32_t ds[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(s[c]), p.qk_scale, -m_i));
            float p1 = ex2_approx(fmaf(__uint_as_float(s[c + 1]), p.qk_scale, -m_i));
            if (diag && c4 * 32 + c > r) p0 = 0.f;                 // key index > query index
            if (diag && c4 * 32 + c + 1 > r) p1 = 0.f;
            ds[c / 2] = pack_bf16x2(p0 * (__uint_as_float(d[c]) - d_i), p1 * (__uint_as_float(d[c + 1]) - d_i));
          }
          tmem_st_x16(t_s + bf16_col(c4 * 2), ds);   // packed inside this thread's own column half
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      }
      if (!ok) break;
      // ---- epilogue: sm_scale * dQ -> bf16 -> staging in the Q tile -> TMA store
      ok = mbar_wait(acc_full, items & 1u, ctx, 97);
      if (!ok) break;
      tc_fence_after();
      store_acc(tmem_base + lane_field + C_DQ, p.sm_scale, smem_q, r, half);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(acc_empty);
        const int y = hz * p.N_CTX + m * AT_BM + q * 32;
        tma_store_2d(&tmap_dq, smem_q + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y);
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(res_empty);
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown
  drain_after_abort(abort_smem);
  tc_fence_before();
  __syncthreads();
  if (warp_idx == BW_WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Host
// ---------------------------------------------------------------------------------------------------------------
int attn_bwd_supported(int D, int N_CTX) { return (D == BW_D && N_CTX >= AT_BM && N_CTX % AT_BM == 0) ? 1 : 0; }

int attn_bwd_bf16(const AttnBwdArgs& a, cudaStream_t stream) {
  if (a.Z <= 0 || a.H <= 0 || a.N_CTX <= 0) return set_error(B200K_ERR_INVALID_ARG, "attention backward: Z, H, N_CTX must be positive");
  if (!attn_bwd_supported(a.D, a.N_CTX))
    return set_error(B200K_ERR_UNSUPPORTED, "attention backward: HEAD_DIM %d / N_CTX %d not supported (HEAD_DIM 128, N_CTX a multiple of 128)", a.D, a.N_CTX);
  const void* ptrs[] = {a.q, a.k, a.v, a.o, a.d_o, a.lse2, a.dq, a.dk, a.dv, a.delta};
  for (const void* ptr : ptrs) {
    if (ptr == nullptr) return set_error(B200K_ERR_INVALID_ARG, "attention backward: null pointer");
    if (reinterpret_cast<uintptr_t>(ptr) & 15u) return set_error(B200K_ERR_INVALID_ARG, "attention backward: every buffer must be 16-byte aligned");
  }
  const int64_t zh = static_cast<int64_t>(a.Z) * a.H;
  if (zh > 0x7FFFFFFF || zh * a.N_CTX > 0x7FFFFFFF) return set_error(B200K_ERR_INVALID_ARG, "attention backward: Z*H*N_CTX exceeds 2^31-1 rows");
  if (!(a.sm_scale > 0.f) || !isfinite(a.sm_scale)) return set_error(B200K_ERR_INVALID_ARG, "attention backward: sm_scale must be positive and finite");
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  if (dev->cc_major != 10) return set_error(B200K_ERR_NO_DEVICE, "attention backward: needs an sm_100 device (found sm_%d%d)", dev->cc_major, dev->cc_minor);

  const uint64_t rows = static_cast<uint64_t>(zh) * a.N_CTX;
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tq, a.q, BW_D, rows, BW_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tk, a.k, BW_D, rows, BW_D, 64, AT_BN)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tv, a.v, BW_D, rows, BW_D, 64, AT_BN)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tdo, a.d_o, BW_D, rows, BW_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tdq, a.dq, BW_D, rows, BW_D, 64, 32)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tdk, a.dk, BW_D, rows, BW_D, 64, 32)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tdv, a.dv, BW_D, rows, BW_D, 64, 32)) != 0) return rc;

  BwdParams p;
  p.ZH = static_cast<int>(zh);
  p.N_CTX = a.N_CTX;
  p.num_blk = a.N_CTX / AT_BM;
  p.num_items = p.ZH * p.num_blk;
  p.causal = a.causal ? 1 : 0;
  p.sm_scale = a.sm_scale;
  p.qk_scale = a.sm_scale * 1.44269504f;
  p.lse2 = a.lse2;
  p.delta = a.delta;
  p.status = dev->status_word;

  const int64_t delta_warps = static_cast<int64_t>(rows);
  int delta_grid = static_cast<int>((delta_warps * 32 + 255) / 256);
  if (delta_grid > dev->sm_count * 8) delta_grid = dev->sm_count * 8;
  attn_bwd_delta_kernel<<<delta_grid, 256, 0, stream>>>(static_cast<const uint2*>(a.o), static_cast<const uint2*>(a.d_o),
                                                        a.delta, static_cast<int64_t>(rows));
  count_launch();
  B200K_CHECK_LAUNCH("attn_bwd_delta_kernel");

  const int grid = p.num_items < dev->sm_count ? p.num_items : dev->sm_count;
  B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM_TOTAL));
  attn_bwd_dkdv_tcgen05_kernel<<<grid, BW_THREADS, KV_SMEM_TOTAL, stream>>>(tq, tk, tv, tdo, tdk, tdv, p);
  count_launch();
  B200K_CHECK_LAUNCH("attn_bwd_dkdv_tcgen05_kernel");

  B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_dq_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM_TOTAL));
  attn_bwd_dq_tcgen05_kernel<<<grid, BW_THREADS, DQ_SMEM_TOTAL, stream>>>(tq, tk, tv, tdo, tdq, p);
  count_launch();
  B200K_CHECK_LAUNCH("attn_bwd_dq_tcgen05_kernel");
  return B200K_OK;
}

}  // namespace b200k
