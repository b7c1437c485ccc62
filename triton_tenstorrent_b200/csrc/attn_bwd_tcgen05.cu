// Fused attention backward for sm_100a, HEAD_DIM 64 or 128, any N_CTX: dQ, dK, dV from Q, K, V, O, dO and the
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
//   warps 0-7  two threads per row of the 128 x 128 score tile (warps 0-3 columns 0-63, warps 4-7 columns 64-127; the
//              backward has no row reductions, M and delta are given, so the halves never talk).  Phase 1: tcgen05.ld
//              S, p = exp2(qk_scale S - M) kept in fp32 registers (dK/dV: bf16 P stored).  Phase 2: tcgen05.ld dP,
//              dS = p (dP - delta) stored as bf16.  bf16 results go over the first 32 of the 64 columns the thread
//              itself has read, so no warp writes where another still reads.  Epilogue: scale, downcast, swizzled
//              staging, TMA store, one 64-column box per half
//   warp 8     TMA producer
//   warp 9     tensor-memory owner and tcgen05.mma issuer
//   warps 10-11 no role; their registers go to the score warps (setmaxnreg: 208 per score thread, 88 for the others)
// All MMAs are 128 x 128 x 16: a 128 x 64 x 16 instruction occupies the tensor pipe for 46 cycles against 64 (measured),
// so stepping the streamed dimension by 64 rows (which would let two whole score buffers fit in tensor memory) makes the
// score products cost 1.4 times as much; that version ran at 3.30 ms (Z=4, H=32, N_CTX=4096), the serial whole-block
// version before it at 4.30 ms.  Instead the 512 columns are used so that the pipe always has work that does not depend
// on the phase the score warps are in:
//   dK/dV  S^T | dP^T | dV | dK.  Phase 1 leaves p in registers, so the issuer can run the NEXT block's S^T while phase 2
//          works; phase 2 writes dS^T and P^T over the dP^T columns it has read, then the issuer runs dV += P^T dO,
//          dK += dS^T Q and the next dP^T (while the next phase 1 runs).
//   dQ     S (buffer 0) | S (buffer 1) | dP | dQ.  The next block's S is always ready; after phase 2 (dS over S) the
//          issuer runs the next dP, dQ += dS K and the S after next.
// Measured (Z=4, H=32, N_CTX=4096): 2.9 ms = 940 TFLOP/s of the algorithm's flop; cycle stamps show the dQ kernel bound
// by its score warps (phase 1 1240 + phase 2 430 cycles per block, hand-offs 300-450) and the dK/dV kernel by the chain
// phase 2 -> 16 gradient MMAs + 8 for dP^T -> phase 2.  A microbenchmark of the issue loop puts the MMAs themselves at
// 64-67 cycles whatever the other warps do (exponentials, tcgen05.ld / st, TMA fills); each dependent group of 8 costs
// about 420 cycles more between the barrier that releases it and the barrier it completes.
#include <math.h>
#include <string.h>

#include "attn_common.cuh"
#include "launch.h"
#include "ptx.cuh"

namespace b200k {

constexpr int BW_THREADS = 384;           // warps 10 and 11 have no role: they only donate their registers
constexpr int BW_REGS_SCORE = 208, BW_REGS_OTHER = 88;   // 8 x 32 x 208 + 4 x 32 x 88 = 384 x 168
constexpr int BW_SCORE_WARPS = 8;
constexpr int BW_WARP_TMA = 8, BW_WARP_MMA = 9;
// A tile is 128 rows x HEAD_DIM columns of bf16: HEAD_DIM / 64 TMA boxes of 128 rows x 64 columns (16 KB each).
constexpr int bw_tile_bytes(int D) { return AT_BM * D * 2; }

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
// delta = rowsum(O * dO): one warp per row of D bf16 values (D / 4 lanes load four values each)
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const uint2* __restrict__ o, const uint2* __restrict__ d_o,
                                                             float* __restrict__ delta, int64_t rows, int d4) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += nwarps) {
    float s = 0.f;
    if (lane < d4) {
      const uint2 a = __ldg(o + row * d4 + lane), b = __ldg(d_o + row * d4 + lane);   // four bf16 each
      s = bf16_bits_to_f32(a.x & 0xFFFFu) * bf16_bits_to_f32(b.x & 0xFFFFu);
      s = fmaf(bf16_bits_to_f32(a.x >> 16), bf16_bits_to_f32(b.x >> 16), s);
      s = fmaf(bf16_bits_to_f32(a.y & 0xFFFFu), bf16_bits_to_f32(b.y & 0xFFFFu), s);
      s = fmaf(bf16_bits_to_f32(a.y >> 16), bf16_bits_to_f32(b.y >> 16), s);
    }
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

// Descriptor offsets (16-byte units) of the k-step `kk` (16 elements of the contraction) inside a 128 x 128 tile of two
// 64-column boxes: contraction along the tile's columns (K-major operand) / along its rows (MN-major operand).
__device__ __forceinline__ uint64_t koff_cols(int kk) {
  return static_cast<uint64_t>(((kk >> 2) * AT_BOX_BYTES + (kk & 3) * 32) >> 4);
}
__device__ __forceinline__ uint64_t koff_rows(int kk) { return static_cast<uint64_t>((kk * 2048) >> 4); }

// One 128 x D tile: D / 64 TMA boxes; rows [row, row + 128) of batch*head hz.  RAGGED (N_CTX not a multiple of 128): the
// tensor maps are three-dimensional (column, row in the head, head), so rows past the end of a head read as zero and
// are not written, instead of spilling into the next head.
template <int D, bool RAGGED>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int hz, int row, int n_ctx) {
#pragma unroll
  for (int bx = 0; bx < D / 64; ++bx) {
    if (RAGGED) tma_load_3d(dst + bx * AT_BOX_BYTES, m, bar, bx * 64, row, hz);
    else tma_load_2d(dst + bx * AT_BOX_BYTES, m, bar, bx * 64, hz * n_ctx + row);
  }
}

// Tensor-memory column (relative to a 128-column fp32 tile) of the bf16 operand's k-step kk (16 values = 8 columns):
// each column half is packed over the first 32 of its own 64 columns.
__device__ __forceinline__ constexpr uint32_t bf16_col(int kk) { return kk < 4 ? kk * 8 : 64 + (kk - 4) * 8; }

// Epilogue of one accumulator: 128 rows x 128 fp32 columns of tensor memory -> x scale -> bf16 -> swizzled staging in
// shared memory (a resident tile that is no longer needed); each thread takes the 64-column box `half` of its row and
// the caller issues the TMA stores of its warp's 32 rows.
__device__ __forceinline__ void store_acc(uint32_t t_acc, float scale, uint8_t* stage, int r, int half) {
#pragma unroll 1
  for (int c4 = 2 * half; c4 < 2 * half + 2; ++c4) {
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

// Phase 1 of a thread's 64 scores at tensor-memory address t_s: p = exp2(qk_scale * s - M), fp32, into pr[].  All 64
// columns are requested at once and waited for once (1.2 % faster than sixteen at a time with the next sixteen in
// flight: every tcgen05.wait::ld is a round trip); pairs go through the packed fp32 instructions (each lane rounds
// like the scalar form) because the issue slots beside the exponentials are what bounds this loop.
//   COLS (dK/dV: rows = keys): M differs per column, read from shared memory (mvec); masked where query < key
//   !COLS (dQ: rows = queries): M is this thread's (m_i); masked where key > query
// col0 is the index of the thread's first column inside the block, r the thread's row.
template <bool COLS, bool MASKED>
__device__ __forceinline__ void score_phase1(uint32_t t_s, const float* mvec, float qk_scale, float m_i, int col0, int r,
                                             float (&pr)[64]) {
  const uint64_t scale2 = COLS ? pack_f32x2(-qk_scale, -qk_scale) : pack_f32x2(qk_scale, qk_scale);
  const uint64_t negm2 = pack_f32x2(-m_i, -m_i);
  uint32_t in[4][16];
#pragma unroll
  for (int k = 0; k < 4; ++k) tmem_ld_x16(t_s + k * 16, in[k]);
  tmem_wait_ld();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t(&sk)[16] = in[k];
    float4 m4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      const uint64_t s2 = pack_f32x2(__uint_as_float(sk[c]), __uint_as_float(sk[c + 1]));
      float x0, x1, p0, p1;
      if (COLS) {
        if ((c & 2) == 0) m4 = *reinterpret_cast<const float4*>(mvec + k * 16 + c);   // one 16-byte load per four scores
        const uint64_t m2 = (c & 2) == 0 ? pack_f32x2(m4.x, m4.y) : pack_f32x2(m4.z, m4.w);
        unpack_f32x2(fma_f32x2(s2, scale2, m2), x0, x1);                          // M - s * qk_scale
        p0 = ex2_approx(-x0);
        p1 = ex2_approx(-x1);
        if (MASKED) {
          if (col0 + k * 16 + c < r) p0 = 0.f;
          if (col0 + k * 16 + c + 1 < r) p1 = 0.f;
        }
      } else {
        unpack_f32x2(fma_f32x2(s2, scale2, negm2), x0, x1);
        p0 = ex2_approx(x0);
        p1 = ex2_approx(x1);
        if (MASKED) {
          if (col0 + k * 16 + c > r) p0 = 0.f;
          if (col0 + k * 16 + c + 1 > r) p1 = 0.f;
        }
      }
      pr[k * 16 + c] = p0;
      pr[k * 16 + c + 1] = p1;
    }
  }
}

// Phase 2: dS = p * (dP - delta) for the thread's 64 values of dP at t_dp; bf16 result to the 32 columns at t_dst.
template <bool COLS>
__device__ __forceinline__ void score_phase2(uint32_t t_dp, uint32_t t_dst, const float* dvec, float d_i, const float (&pr)[64]) {
  const uint64_t negd2 = pack_f32x2(-d_i, -d_i);
  const uint64_t minus1 = pack_f32x2(-1.0f, -1.0f);
  uint32_t in[4][16];
  uint32_t ds[16];
#pragma unroll
  for (int k = 0; k < 4; ++k) tmem_ld_x16(t_dp + k * 16, in[k]);
  tmem_wait_ld();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t(&dk)[16] = in[k];
    float4 dl4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      const uint64_t d2 = pack_f32x2(__uint_as_float(dk[c]), __uint_as_float(dk[c + 1]));
      uint64_t t2;
      if (COLS) {
        if ((c & 2) == 0) dl4 = *reinterpret_cast<const float4*>(dvec + k * 16 + c);
        const uint64_t dl2 = (c & 2) == 0 ? pack_f32x2(dl4.x, dl4.y) : pack_f32x2(dl4.z, dl4.w);
        t2 = fma_f32x2(dl2, minus1, d2);                                          // dP - delta
      } else {
        t2 = add_f32x2(d2, negd2);
      }
      float y0, y1;
      unpack_f32x2(mul_f32x2(pack_f32x2(pr[k * 16 + c], pr[k * 16 + c + 1]), t2), y0, y1);
      ds[(k & 1) * 8 + c / 2] = pack_bf16x2(y0, y1);
    }
    if (k & 1) tmem_st_x16(t_dst + (k >> 1) * 16, ds);
  }
}

// Common epilogue of a score warp: one or two accumulators -> staging in the resident tiles -> TMA stores of the
// warp's 32 rows x 64 columns; then the resident tiles and the accumulators are handed back.
template <bool RAGGED>
__device__ __forceinline__ void epilogue_store(uint32_t t_acc0, float scale0, uint8_t* stage0, const CUtensorMap* out0,
                                               bool two, uint32_t t_acc1, float scale1, uint8_t* stage1,
                                               const CUtensorMap* out1, int r, int q, int half, int hz, int y, int n_ctx,
                                               uint32_t lane, uint64_t* acc_empty, uint64_t* res_empty, bool active) {
  // HEAD_DIM 128: each half stores its 64-column box; HEAD_DIM 64: the one box is stored by the first half alone
  if (active) {
    store_acc(t_acc0, scale0, stage0, r, half);
    if (two) store_acc(t_acc1, scale1, stage1, r, half);
  }
  tc_fence_before();
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    mbar_arrive(acc_empty);
    if (active) {
      // RAGGED: rows past the end of the head are clipped by the 3-D map (a warp whose 32 rows all lie past it stores nothing)
      if (RAGGED) {
        if (y < n_ctx) {
          tma_store_3d(out0, stage0 + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y, hz);
          if (two) tma_store_3d(out1, stage1 + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y, hz);
        }
      } else {
        tma_store_2d(out0, stage0 + half * AT_BOX_BYTES + q * 32 * 128, half * 64, hz * n_ctx + y);
        if (two) tma_store_2d(out1, stage1 + half * AT_BOX_BYTES + q * 32 * 128, half * 64, hz * n_ctx + y);
      }
      tma_store_commit();
      tma_store_wait_read<0>();
    }
    mbar_arrive(res_empty);
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------------------------
// dK and dV: one item = (batch*head, key block n); K, V resident; the query blocks m stream (m >= n when causal).
// Rows of the score tiles are keys: S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q.
// ---------------------------------------------------------------------------------------------------------------
constexpr int KV_NSTAGE = 2;
constexpr int KV_NBAR = 2 + 4 * KV_NSTAGE + 6;
// shared memory: K, V | Q stages | dO stages | per stage 128 M values and 128 delta values | barriers
constexpr int kv_vec_off(int D) { return (2 + 2 * KV_NSTAGE) * bw_tile_bytes(D); }
constexpr int kv_bar_off(int D) { return kv_vec_off(D) + KV_NSTAGE * 1024; }
constexpr int kv_smem_total(int D) { return kv_bar_off(D) + KV_NBAR * 8 + 16 + 1024; }
static_assert(kv_smem_total(128) <= 232448, "attention backward (dK/dV) shared memory budget exceeded");

template <int BW_D, bool RAGGED>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dkdv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                             const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                             const __grid_constant__ CUtensorMap tmap_dk, const __grid_constant__ CUtensorMap tmap_dv,
                             const BwdParams p) {
  constexpr uint32_t IDESC_SS = umma_idesc_bf16_f32(AT_BM, AT_BN, 0, 0);   // both operands K-major
  constexpr uint32_t IDESC_TS = umma_idesc_bf16_f32(AT_BM, BW_D, 0, 1);    // A in tensor memory, B MN-major
  constexpr uint32_t C_ST = 0, C_DPT = 128, C_DV = 256, C_DK = 256 + BW_D;
  constexpr int BW_TILE_BYTES = bw_tile_bytes(BW_D);
  constexpr int KV_Q_OFF = 2 * BW_TILE_BYTES, KV_DO_OFF = KV_Q_OFF + KV_NSTAGE * BW_TILE_BYTES;
  constexpr int KV_VEC_OFF = kv_vec_off(BW_D), KV_BAR_OFF = kv_bar_off(BW_D);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_k = smem;
  uint8_t* smem_v = smem + BW_TILE_BYTES;
  uint8_t* smem_q = smem + KV_Q_OFF;
  uint8_t* smem_do = smem + KV_DO_OFF;
  float* smem_vec = reinterpret_cast<float*>(smem + KV_VEC_OFF);
  uint64_t* res_full = reinterpret_cast<uint64_t*>(smem + KV_BAR_OFF);   // K and V tiles have arrived
  uint64_t* res_empty = res_full + 1;                                    // ... may be overwritten (8 warps)
  uint64_t* q_full = res_empty + 1;                                      // [stage] Q tile, M and delta vectors
  uint64_t* q_empty = q_full + KV_NSTAGE;                                // [stage] released after dK += dS^T Q
  uint64_t* do_full = q_empty + KV_NSTAGE;                               // [stage] dO tile
  uint64_t* do_empty = do_full + KV_NSTAGE;                              // [stage] released after dV += P^T dO
  uint64_t* s_full = do_empty + KV_NSTAGE;                               // S^T is in tensor memory
  uint64_t* dp_full = s_full + 1;                                        // dP^T is in tensor memory
  uint64_t* p1_ready = dp_full + 1;                                      // S^T consumed (8 warps)
  uint64_t* p2_ready = p1_ready + 1;                                     // dS^T and P^T written over dP^T (8 warps)
  uint64_t* acc_full = p2_ready + 1;                                     // dV and dK complete
  uint64_t* acc_empty = acc_full + 1;                                    // ... read out (8 warps)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 1);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    mbar_init(res_full, 1);
    mbar_init(res_empty, BW_SCORE_WARPS);
    for (int s = 0; s < KV_NSTAGE; ++s) {
      mbar_init(&q_full[s], RAGGED ? 2 : 1);   // RAGGED: the producer warp copies the M / delta vectors itself
      mbar_init(&q_empty[s], 1);
      mbar_init(&do_full[s], 1);
      mbar_init(&do_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p1_ready, BW_SCORE_WARPS);
    mbar_init(p2_ready, BW_SCORE_WARPS);
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

  // Every role walks the same sequence of (item, block) and counts blocks in `g`: stage g % 2 (use g / 2 of it), and
  // the g-th completion of the single barriers.
  if (warp_idx >= BW_SCORE_WARPS) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(BW_REGS_OTHER));   // all four warps, one instruction
   if (warp_idx == BW_WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t items = 0, g = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      const int hz = item / p.num_blk, n = item - hz * p.num_blk;
      const int row_base = hz * p.N_CTX;
      ok = mbar_wait(res_empty, (items & 1u) ^ 1u, ctx, 80);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(res_full, 2 * BW_TILE_BYTES);
        load_tile<BW_D, RAGGED>(smem_k, &tmap_k, res_full, hz, n * AT_BN, p.N_CTX);
        load_tile<BW_D, RAGGED>(smem_v, &tmap_v, res_full, hz, n * AT_BN, p.N_CTX);
      }
      __syncwarp();
      for (int m = p.causal ? n : 0; ok && m < p.num_blk; ++m, ++g) {
        const uint32_t st = g & 1u, ph = (g >> 1) & 1u;
        const int row = row_base + m * AT_BM;
        ok = mbar_wait(&q_empty[st], ph ^ 1u, ctx, 81);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&q_full[st], BW_TILE_BYTES + (RAGGED ? 0 : 1024));
          load_tile<BW_D, RAGGED>(smem_q + st * BW_TILE_BYTES, &tmap_q, &q_full[st], hz, m * AT_BM, p.N_CTX);
          if (!RAGGED) {
            bulk_load_1d(smem_vec + st * 256, p.lse2 + row, 512, &q_full[st]);
            bulk_load_1d(smem_vec + st * 256 + 128, p.delta + row, 512, &q_full[st]);
          }
        }
        if (RAGGED) {
          // the block's M and delta values, zero past the end of the head (a bulk copy would run into the next head, or
          // off the buffer): four of each per lane, then a second arrival on the stage's barrier
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int idx = static_cast<int>(lane) * 4 + e, qi = m * AT_BM + idx;
            const bool in = qi < p.N_CTX;
            smem_vec[st * 256 + idx] = in ? __ldg(p.lse2 + row_base + qi) : 0.f;
            smem_vec[st * 256 + 128 + idx] = in ? __ldg(p.delta + row_base + qi) : 0.f;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&q_full[st]);
        }
        __syncwarp();
        ok = mbar_wait(&do_empty[st], ph ^ 1u, ctx, 82);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&do_full[st], BW_TILE_BYTES);
          load_tile<BW_D, RAGGED>(smem_do + st * BW_TILE_BYTES, &tmap_do, &do_full[st], hz, m * AT_BM, p.N_CTX);
        }
        __syncwarp();
      }
    }
  } else if (warp_idx == BW_WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t items = 0, g = 0;
    bool ok = true;
    const uint64_t k_desc = umma_smem_desc_sw128(smem_u32(smem_k), 16, 1024);
    const uint64_t v_desc = umma_smem_desc_sw128(smem_u32(smem_v), 16, 1024);
    // S^T = K Q^T / dP^T = V dO^T of the block in stage st: rows = keys, columns = queries, contraction over d
    auto issue_st = [&](uint32_t st) {
      const uint64_t qk = umma_smem_desc_sw128(smem_u32(smem_q + st * BW_TILE_BYTES), 16, 1024);
#pragma unroll
      for (int kk = 0; kk < BW_D / 16; ++kk)
        umma_ss(tmem_base + C_ST, k_desc + koff_cols(kk), qk + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
      umma_commit(s_full);
    };
    auto issue_dpt = [&](uint32_t st) {
      const uint64_t dok = umma_smem_desc_sw128(smem_u32(smem_do + st * BW_TILE_BYTES), 16, 1024);
#pragma unroll
      for (int kk = 0; kk < BW_D / 16; ++kk)
        umma_ss(tmem_base + C_DPT, v_desc + koff_cols(kk), dok + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
      umma_commit(dp_full);
    };
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      const int hz = item / p.num_blk, n = item - hz * p.num_blk;
      (void)hz;
      const int nb = p.num_blk - (p.causal ? n : 0);
      ok = mbar_wait(res_full, items & 1u, ctx, 83);
      if (!ok) break;
      // the item's first block: both score products up front
      ok = mbar_wait(&q_full[g & 1u], (g >> 1) & 1u, ctx, 84);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) issue_st(g & 1u);
      __syncwarp();
      ok = mbar_wait(&do_full[g & 1u], (g >> 1) & 1u, ctx, 85);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) issue_dpt(g & 1u);
      __syncwarp();
      for (int j = 0; ok && j < nb; ++j, ++g) {
        const uint32_t st = g & 1u, nst = (g + 1) & 1u, nph = ((g + 1) >> 1) & 1u;
        const bool more = j + 1 < nb;
        // ---- after phase 1 (S^T is in the score warps' registers): the next block's S^T
        ok = mbar_wait(p1_ready, g & 1u, ctx, 86);
        if (!ok) break;
        if (more) {
          ok = mbar_wait(&q_full[nst], nph, ctx, 84);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) issue_st(nst);
          __syncwarp();
        }
        // ---- after phase 2 (dS^T | P^T in the dP^T columns): dV += P^T dO, dK += dS^T Q, then the next block's dP^T
        ok = mbar_wait(p2_ready, g & 1u, ctx, 88);
        if (!ok) break;
        if (j == 0) {   // the previous item's dV / dK must have left tensor memory before they are overwritten
          ok = mbar_wait(acc_empty, (items & 1u) ^ 1u, ctx, 87);
          if (!ok) break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint64_t don = umma_smem_desc_sw128(smem_u32(smem_do + st * BW_TILE_BYTES), AT_BOX_BYTES, 1024);
          const uint64_t qn = umma_smem_desc_sw128(smem_u32(smem_q + st * BW_TILE_BYTES), AT_BOX_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < AT_BM / 16; ++kk)
            umma_ts(tmem_base + C_DV, tmem_base + C_DPT + 32 + bf16_col(kk), don + koff_rows(kk), IDESC_TS, (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&do_empty[st]);
#pragma unroll
          for (int kk = 0; kk < AT_BM / 16; ++kk)
            umma_ts(tmem_base + C_DK, tmem_base + C_DPT + bf16_col(kk), qn + koff_rows(kk), IDESC_TS, (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&q_empty[st]);
          if (!more) umma_commit(acc_full);
        }
        __syncwarp();
        if (more) {
          ok = mbar_wait(&do_full[nst], nph, ctx, 85);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) issue_dpt(nst);
          __syncwarp();
        }
      }
    }
   }  // warps 10 and 11 have no role
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(BW_REGS_SCORE));
    // ------------------------------------------------------------------ score rows (warps 0..7): thread = (key, column half)
    const int q = warp_idx & 3;          // tensor-memory lane quarter
    const int half = warp_idx >> 2;      // queries [64 * half, 64 * half + 64) of the block
    const int r = q * 32 + static_cast<int>(lane);
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + C_ST + half * 64, t_dp = tmem_base + lane_field + C_DPT + half * 64;
    uint32_t items = 0, g = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      const int hz = item / p.num_blk, n = item - hz * p.num_blk;
      for (int m = p.causal ? n : 0; ok && m < p.num_blk; ++m, ++g) {
        const uint32_t st = g & 1u;
        const float* mvec = smem_vec + st * 256 + half * 64;
        const bool diag = p.causal && m == n;
        float pr[64];
        // the M and delta vectors are read from shared memory below: observe their arrival directly
        ok = mbar_wait(&q_full[st], (g >> 1) & 1u, ctx, 89);
        if (!ok) break;
        ok = mbar_wait(s_full, g & 1u, ctx, 90);
        if (!ok) break;
        tc_fence_after();
        if (diag) score_phase1<true, true>(t_s, mvec, p.qk_scale, 0.f, half * 64, r, pr);
        else score_phase1<true, false>(t_s, mvec, p.qk_scale, 0.f, half * 64, r, pr);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p1_ready);      // S^T is in registers: the next block's S^T may overwrite it
        uint32_t pp[32];                           // bf16 P^T, packed while dP^T is still on its way
#pragma unroll
        for (int c = 0; c < 32; ++c) pp[c] = pack_bf16x2(pr[2 * c], pr[2 * c + 1]);
        ok = mbar_wait(dp_full, g & 1u, ctx, 91);
        if (!ok) break;
        tc_fence_after();
        score_phase2<true>(t_dp, t_dp, mvec + 128, 0.f, pr);   // dS^T over the first 32 of the thread's dP^T columns
        tmem_st_x32(t_dp + 32, pp);                            // P^T over the other 32 (all 64 have been read)
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p2_ready);
      }
      if (!ok) break;
      // ---- epilogue: dV and sm_scale * dK -> bf16 -> staging in the K / V tiles (no longer needed) -> TMA store
      ok = mbar_wait(acc_full, items & 1u, ctx, 92);
      if (!ok) break;
      tc_fence_after();
      epilogue_store<RAGGED>(tmem_base + lane_field + C_DV, 1.0f, smem_k, &tmap_dv, true, tmem_base + lane_field + C_DK,
                             p.sm_scale, smem_v, &tmap_dk, r, q, half, hz, n * AT_BN + q * 32, p.N_CTX, lane, acc_empty,
                             res_empty, BW_D == 128 || half == 0);
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
// dQ: one item = (batch*head, query block m); Q, dO resident; the key blocks n stream (n <= m when causal).
// Rows of the score tiles are queries: S = Q K^T (two buffers), dP = dO V^T, dQ += dS K.
// ---------------------------------------------------------------------------------------------------------------
constexpr int DQ_NK = 3, DQ_NV = 2;                                   // K lives until dQ += dS K, V only until dP
constexpr int DQ_NBAR = 2 + 2 * DQ_NK + 2 * DQ_NV + 6;
// shared memory: Q, dO | K slots | V slots | barriers
constexpr int dq_bar_off(int D) { return (2 + DQ_NK + DQ_NV) * bw_tile_bytes(D); }
constexpr int dq_smem_total(int D) { return dq_bar_off(D) + DQ_NBAR * 8 + 16 + 1024; }
static_assert(dq_smem_total(128) <= 232448, "attention backward (dQ) shared memory budget exceeded");

template <int BW_D, bool RAGGED>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                           const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  constexpr uint32_t IDESC_SS = umma_idesc_bf16_f32(AT_BM, AT_BN, 0, 0);
  constexpr uint32_t IDESC_TS = umma_idesc_bf16_f32(AT_BM, BW_D, 0, 1);
  constexpr uint32_t C_S = 0 /* buffer 1 at 128 */, C_DP = 256, C_DQ = 384;
  constexpr int BW_TILE_BYTES = bw_tile_bytes(BW_D);
  constexpr int DQ_K_OFF = 2 * BW_TILE_BYTES, DQ_V_OFF = DQ_K_OFF + DQ_NK * BW_TILE_BYTES, DQ_BAR_OFF = dq_bar_off(BW_D);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;
  uint8_t* smem_do = smem + BW_TILE_BYTES;
  uint8_t* smem_k = smem + DQ_K_OFF;
  uint8_t* smem_v = smem + DQ_V_OFF;
  uint64_t* res_full = reinterpret_cast<uint64_t*>(smem + DQ_BAR_OFF);
  uint64_t* res_empty = res_full + 1;
  uint64_t* k_full = res_empty + 1;
  uint64_t* k_empty = k_full + DQ_NK;                                    // [slot] released after dQ += dS K
  uint64_t* v_full = k_empty + DQ_NK;
  uint64_t* v_empty = v_full + DQ_NV;                                    // [slot] released after dP = dO V^T
  uint64_t* s_full = v_empty + DQ_NV;                                    // [buffer] S is in tensor memory
  uint64_t* dp_full = s_full + 2;                                        // dP is in tensor memory
  uint64_t* p_ready = dp_full + 1;                                       // dS written over S; S and dP consumed (8 warps)
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
    for (int s = 0; s < DQ_NK; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < DQ_NV; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
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

  // Every role counts the blocks it has walked in `g`: S buffer g % 2, K slot g % 3, V slot g % 2.
  if (warp_idx >= BW_SCORE_WARPS) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(BW_REGS_OTHER));   // all four warps, one instruction
   if (warp_idx == BW_WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t items = 0, g = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, m;
      item_block(item, hz, m);
      ok = mbar_wait(res_empty, (items & 1u) ^ 1u, ctx, 100);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(res_full, 2 * BW_TILE_BYTES);
        load_tile<BW_D, RAGGED>(smem_q, &tmap_q, res_full, hz, m * AT_BM, p.N_CTX);
        load_tile<BW_D, RAGGED>(smem_do, &tmap_do, res_full, hz, m * AT_BM, p.N_CTX);
      }
      __syncwarp();
      const int n_end = p.causal ? m + 1 : p.num_blk;
      for (int n = 0; ok && n < n_end; ++n, ++g) {
        const uint32_t ks = g % DQ_NK, kph = (g / DQ_NK) & 1u, vs = g % DQ_NV, vph = (g / DQ_NV) & 1u;
        ok = mbar_wait(&k_empty[ks], kph ^ 1u, ctx, 101);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&k_full[ks], BW_TILE_BYTES);
          load_tile<BW_D, RAGGED>(smem_k + ks * BW_TILE_BYTES, &tmap_k, &k_full[ks], hz, n * AT_BN, p.N_CTX);
        }
        __syncwarp();
        ok = mbar_wait(&v_empty[vs], vph ^ 1u, ctx, 102);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&v_full[vs], BW_TILE_BYTES);
          load_tile<BW_D, RAGGED>(smem_v + vs * BW_TILE_BYTES, &tmap_v, &v_full[vs], hz, n * AT_BN, p.N_CTX);
        }
        __syncwarp();
      }
    }
  } else if (warp_idx == BW_WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    uint32_t items = 0, g = 0;
    bool ok = true;
    const uint64_t q_desc = umma_smem_desc_sw128(smem_u32(smem_q), 16, 1024);
    const uint64_t do_desc = umma_smem_desc_sw128(smem_u32(smem_do), 16, 1024);
    // S = Q K^T of block gg into buffer gg % 2; dP = dO V^T of block gg (each waits for its tile first)
    auto issue_s = [&](uint32_t gg) -> bool {
      const uint32_t ks = gg % DQ_NK;
      if (!mbar_wait(&k_full[ks], (gg / DQ_NK) & 1u, ctx, 103)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint64_t kd = umma_smem_desc_sw128(smem_u32(smem_k + ks * BW_TILE_BYTES), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < BW_D / 16; ++kk)
          umma_ss(tmem_base + C_S + (gg & 1u) * 128, q_desc + koff_cols(kk), kd + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[gg & 1u]);
      }
      __syncwarp();
      return true;
    };
    auto issue_dp = [&](uint32_t gg) -> bool {
      const uint32_t vs = gg % DQ_NV;
      if (!mbar_wait(&v_full[vs], (gg / DQ_NV) & 1u, ctx, 104)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint64_t vd = umma_smem_desc_sw128(smem_u32(smem_v + vs * BW_TILE_BYTES), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < BW_D / 16; ++kk)
          umma_ss(tmem_base + C_DP, do_desc + koff_cols(kk), vd + koff_cols(kk), IDESC_SS, kk > 0 ? 1u : 0u);
        umma_commit(dp_full);
        umma_commit(&v_empty[vs]);
      }
      __syncwarp();
      return true;
    };
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, m;
      item_block(item, hz, m);
      const int nb = p.causal ? m + 1 : p.num_blk;
      ok = mbar_wait(res_full, items & 1u, ctx, 105);
      if (!ok) break;
      ok = issue_s(g) && issue_dp(g);
      if (ok && nb > 1) ok = issue_s(g + 1);
      for (int j = 0; ok && j < nb; ++j, ++g) {
        // all warps have read S and dP of block g and written dS over S
        ok = mbar_wait(p_ready, g & 1u, ctx, 106);
        if (!ok) break;
        if (j == 0) {
          ok = mbar_wait(acc_empty, (items & 1u) ^ 1u, ctx, 107);
          if (!ok) break;
        }
        if (j + 1 < nb) {   // first what the score warps wait for next
          ok = issue_dp(g + 1);
          if (!ok) break;
        }
        tc_fence_after();
        if (lane == 0) {
          // dQ += dS K: A = dS (bf16 over S of buffer g % 2), contraction over the keys
          const uint32_t ks = g % DQ_NK;
          const uint64_t kn = umma_smem_desc_sw128(smem_u32(smem_k + ks * BW_TILE_BYTES), AT_BOX_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < AT_BN / 16; ++kk)
            umma_ts(tmem_base + C_DQ, tmem_base + C_S + (g & 1u) * 128 + bf16_col(kk), kn + koff_rows(kk), IDESC_TS,
                    (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&k_empty[ks]);
          if (j == nb - 1) umma_commit(acc_full);
        }
        __syncwarp();
        if (j + 2 < nb) {   // the freed buffer takes the S after next (after the MMAs above have read dS: in order)
          ok = issue_s(g + 2);
          if (!ok) break;
        }
      }
    }
   }  // warps 10 and 11 have no role
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(BW_REGS_SCORE));
    // ------------------------------------------------------------------ score rows (warps 0..7): thread = (query, column half)
    const int q = warp_idx & 3;
    const int half = warp_idx >> 2;      // keys [64 * half, 64 * half + 64) of the block
    const int r = q * 32 + static_cast<int>(lane);
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_dp = tmem_base + lane_field + C_DP + half * 64;
    uint32_t items = 0, g = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, m;
      item_block(item, hz, m);
      const int64_t my_row = static_cast<int64_t>(hz) * p.N_CTX + m * AT_BM + r;
      const bool row_in = !RAGGED || m * AT_BM + r < p.N_CTX;     // rows past the end of the head: computed, never stored
      const float m_i = row_in ? __ldg(p.lse2 + my_row) : 0.f, d_i = row_in ? __ldg(p.delta + my_row) : 0.f;
      const int n_end = p.causal ? m + 1 : p.num_blk;
      for (int n = 0; ok && n < n_end; ++n, ++g) {
        const uint32_t t_s = tmem_base + lane_field + C_S + (g & 1u) * 128 + half * 64;
        const bool diag = p.causal && n == m;
        float pr[64];
        ok = mbar_wait(&s_full[g & 1u], (g >> 1) & 1u, ctx, 108);
        if (!ok) break;
        tc_fence_after();
        if (diag) score_phase1<false, true>(t_s, nullptr, p.qk_scale, m_i, half * 64, r, pr);
        else score_phase1<false, false>(t_s, nullptr, p.qk_scale, m_i, half * 64, r, pr);
        ok = mbar_wait(dp_full, g & 1u, ctx, 109);
        if (!ok) break;
        tc_fence_after();
        score_phase2<false>(t_dp, t_s, nullptr, d_i, pr);      // dS over the first 32 of the thread's S columns
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      }
      if (!ok) break;
      // ---- epilogue: sm_scale * dQ -> bf16 -> staging in the Q tile -> TMA store
      ok = mbar_wait(acc_full, items & 1u, ctx, 110);
      if (!ok) break;
      tc_fence_after();
      epilogue_store<RAGGED>(tmem_base + lane_field + C_DQ, p.sm_scale, smem_q, &tmap_dq, false, 0, 0.f, nullptr, nullptr, r, q,
                             half, hz, m * AT_BM + q * 32, p.N_CTX, lane, acc_empty, res_empty, BW_D == 128 || half == 0);
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
int attn_bwd_supported(int D, int N_CTX) { return ((D == 64 || D == 128) && N_CTX >= 1) ? 1 : 0; }

int attn_bwd_bf16(const AttnBwdArgs& a, cudaStream_t stream) {
  if (a.Z <= 0 || a.H <= 0 || a.N_CTX <= 0) return set_error(B200K_ERR_INVALID_ARG, "attention backward: Z, H, N_CTX must be positive");
  if (!attn_bwd_supported(a.D, a.N_CTX))
    return set_error(B200K_ERR_UNSUPPORTED, "attention backward: HEAD_DIM %d / N_CTX %d not supported (HEAD_DIM 64 or 128)", a.D, a.N_CTX);
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
  // N_CTX a multiple of 128: one 2-D map over all rows; otherwise per-head 3-D maps (column, row in the head, head)
  const bool ragged = a.N_CTX % AT_BM != 0;
  auto make_map = [&](CUtensorMap* m, const void* base, uint32_t box_rows) {
    return ragged ? make_tmap_bf16_3d(m, base, a.D, a.N_CTX, zh, 64, box_rows)
                  : make_tmap_bf16_2d(m, base, a.D, rows, a.D, 64, box_rows);
  };
  if ((rc = make_map(&tq, a.q, AT_BM)) != 0) return rc;
  if ((rc = make_map(&tk, a.k, AT_BM)) != 0) return rc;
  if ((rc = make_map(&tv, a.v, AT_BM)) != 0) return rc;
  if ((rc = make_map(&tdo, a.d_o, AT_BM)) != 0) return rc;
  if ((rc = make_map(&tdq, a.dq, 32)) != 0) return rc;
  if ((rc = make_map(&tdk, a.dk, 32)) != 0) return rc;
  if ((rc = make_map(&tdv, a.dv, 32)) != 0) return rc;

  BwdParams p;
  p.ZH = static_cast<int>(zh);
  p.N_CTX = a.N_CTX;
  p.num_blk = (a.N_CTX + AT_BM - 1) / AT_BM;
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
                                                        a.delta, static_cast<int64_t>(rows), a.D / 4);
  count_launch();
  B200K_CHECK_LAUNCH("attn_bwd_delta_kernel");

  const int grid = p.num_items < dev->sm_count ? p.num_items : dev->sm_count;
#define B200K_BWD_LAUNCH(DD, RR)                                                                                              \
  do {                                                                                                                       \
    B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_tcgen05_kernel<DD, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                          kv_smem_total(DD)));                                                               \
    attn_bwd_dkdv_tcgen05_kernel<DD, RR><<<grid, BW_THREADS, kv_smem_total(DD), stream>>>(tq, tk, tv, tdo, tdk, tdv, p);     \
    count_launch();                                                                                                          \
    B200K_CHECK_LAUNCH("attn_bwd_dkdv_tcgen05_kernel");                                                                      \
    B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_dq_tcgen05_kernel<DD, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                          dq_smem_total(DD)));                                                               \
    attn_bwd_dq_tcgen05_kernel<DD, RR><<<grid, BW_THREADS, dq_smem_total(DD), stream>>>(tq, tk, tv, tdo, tdq, p);            \
    count_launch();                                                                                                          \
    B200K_CHECK_LAUNCH("attn_bwd_dq_tcgen05_kernel");                                                                        \
  } while (0)
  if (a.D == 64) {
    if (ragged) B200K_BWD_LAUNCH(64, true);
    else B200K_BWD_LAUNCH(64, false);
  } else {
    if (ragged) B200K_BWD_LAUNCH(128, true);
    else B200K_BWD_LAUNCH(128, false);
  }
#undef B200K_BWD_LAUNCH
  return B200K_OK;
}

}  // namespace b200k
