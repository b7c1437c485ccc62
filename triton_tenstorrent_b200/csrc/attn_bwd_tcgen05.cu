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
//   warps 0-7  one thread per row of a step's score tile; warps 0-3 take the even steps, warps 4-7 the odd ones (the
//              backward has no row reductions, M and delta are given): tcgen05.ld S and dP, exponentials, dS, bf16
//              results written back over S / dP in tensor memory (packed over columns the thread has already read);
//              epilogue (scale, downcast, swizzled staging, TMA store), one 64-column half per group
//   warp 8     TMA producer (the item's resident tiles; a four-stage ring of the half-tiles that stream)
//   warp 9     tensor-memory owner and tcgen05.mma issuer
// Both kernels are one template.  The streamed dimension advances in steps of 64 rows (queries for dK/dV, keys for
// dQ), so that a step's scores take 64 + 64 tensor-memory columns and two steps fit beside the accumulators:
//   columns   0..127  step buffer 0: S | dP (64 fp32 columns each; bf16 P / dS packed over them)
//   columns 128..255  step buffer 1
//   columns 256..511  dK/dV kernel: dV | dK;  dQ kernel: dQ | Q, dO as bf16 MMA A operands (64 columns each)
// The issuer runs one step ahead: MMA(S, dP) of step j+1 and the gradient MMAs of step j-1 execute while a score group
// works on step j.  With whole 128-row blocks tensor memory held one block and the chain MMA -> exponentials -> MMA was
// serial: 4.30 ms at Z=4, H=32, N_CTX=4096 against 3.30 ms now (dK/dV 1.95, dQ 1.29, delta 0.05).
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
constexpr int BW_TILE_BYTES = AT_BM * BW_D * 2;       // 32 KB: two boxes of 128 rows x 64 columns (resident tiles)
constexpr int BW_SUB = 64;                            // streamed rows per step
constexpr int BW_SUB_BOX = BW_SUB * 128;              // 8 KB: 64 rows x 64 columns
constexpr int BW_SUB_TILE = 2 * BW_SUB_BOX;           // 16 KB: 64 rows x 128 columns
constexpr int BW_NSTAGE = 4;
static_assert(BW_NSTAGE % 2 == 0, "the two score groups own alternate stages");
constexpr int BW_STAGE_BYTES = 2 * BW_SUB_TILE + 1024;   // two half-tiles, then 64 M values and 64 delta values (dK/dV)
constexpr int BW_STAGE_OFF = 2 * BW_TILE_BYTES;          // after the two resident tiles
constexpr int BW_BAR_OFF = BW_STAGE_OFF + BW_NSTAGE * BW_STAGE_BYTES;
constexpr int BW_NBAR = 2 + 2 * BW_NSTAGE + 2 + 2 + 2 + 1;
constexpr int BW_SMEM_TOTAL = BW_BAR_OFF + BW_NBAR * 8 + 16 + 1024;
static_assert(BW_SMEM_TOTAL <= 232448, "attention backward shared memory budget exceeded");

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

// Descriptor offsets (16-byte units) of the k-step `kk` (16 elements of the contraction) inside a tile of two
// 64-column boxes of `box_bytes` each: contraction along the tile's columns (K-major operand) / along its rows
// (MN-major operand).
__device__ __forceinline__ uint64_t koff_cols(int kk, int box_bytes) {
  return static_cast<uint64_t>(((kk >> 2) * box_bytes + (kk & 3) * 32) >> 4);
}
__device__ __forceinline__ uint64_t koff_rows(int kk) { return static_cast<uint64_t>((kk * 2048) >> 4); }

// A tile of `rows` x 128 columns: two TMA boxes of 64 columns.
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row, int box_bytes) {
  tma_load_2d(dst, m, bar, 0, row);
  tma_load_2d(dst + box_bytes, m, bar, 64, row);
}

// Tensor-memory column (relative to a step's fp32 score tile of 64 columns) of the bf16 operand's k-step kk (16 scores
// = 8 columns): each thread packs its 32 scores at the start of its own 32 columns, so no warp writes where another
// still reads.
__device__ __forceinline__ constexpr uint32_t bf16_col(int kk) { return (kk >> 1) * 32 + (kk & 1) * 8; }

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

// The score work of one thread for one step: its row's 64 fp32 scores S and 64 values dP in the step buffer `t_buf`
// (S at columns 0..63, dP at 64..127) become bf16 dS (and P for dK/dV), packed over the first 16 columns of every 32
// just read.  Sixteen columns at a time, the next sixteen in flight meanwhile; pairs of scores go through the packed
// fp32 instructions (each lane rounds like the scalar form), because the issue slots beside the exponentials are
// what bounds this loop (about 9 cycles per exponential with two other instructions, 14 with four).
//   dK/dV (rows = keys): M and delta differ per column and come from shared memory: p = exp2(-(M - s * qk_scale)),
//                        dS = p * (dP - delta); masked (diagonal block) where query < key
//   dQ (rows = queries): M and delta are this thread's: p = exp2(s * qk_scale - M); masked where key > query
template <bool DKDV, bool MASKED>
__device__ __forceinline__ void score_step(uint32_t t_buf, const float* vec, float qk_scale, float m_i, float d_i, int col0,
                                           int r) {
  const uint64_t scale2 = DKDV ? pack_f32x2(-qk_scale, -qk_scale) : pack_f32x2(qk_scale, qk_scale);
  const uint64_t negm2 = pack_f32x2(-m_i, -m_i), negd2 = pack_f32x2(-d_i, -d_i);
  const uint64_t minus1 = pack_f32x2(-1.0f, -1.0f);
  uint32_t s[2][16], d[2][16];
  uint32_t pp[16], ds[16];
  tmem_ld_x16(t_buf, s[0]);
  tmem_ld_x16(t_buf + 64, d[0]);
  tmem_wait_ld();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (k + 1 < 4) {
      tmem_ld_x16(t_buf + (k + 1) * 16, s[(k + 1) & 1]);
      tmem_ld_x16(t_buf + 64 + (k + 1) * 16, d[(k + 1) & 1]);
    }
    const uint32_t(&sk)[16] = s[k & 1];
    const uint32_t(&dk)[16] = d[k & 1];
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      const uint64_t s2 = pack_f32x2(__uint_as_float(sk[c]), __uint_as_float(sk[c + 1]));
      const uint64_t d2 = pack_f32x2(__uint_as_float(dk[c]), __uint_as_float(dk[c + 1]));
      float x0, x1, p0, p1;
      uint64_t t2;
      if (DKDV) {
        const float2 m2 = *reinterpret_cast<const float2*>(vec + k * 16 + c);
        const float2 dl2 = *reinterpret_cast<const float2*>(vec + 64 + k * 16 + c);
        unpack_f32x2(fma_f32x2(s2, scale2, pack_f32x2(m2.x, m2.y)), x0, x1);     // M - s * qk_scale
        p0 = ex2_approx(-x0);
        p1 = ex2_approx(-x1);
        t2 = fma_f32x2(pack_f32x2(dl2.x, dl2.y), minus1, d2);                     // dP - delta
        if (MASKED) {
          if (col0 + k * 16 + c < r) p0 = 0.f;                                    // query index < key index
          if (col0 + k * 16 + c + 1 < r) p1 = 0.f;
        }
        pp[(k & 1) * 8 + c / 2] = pack_bf16x2(p0, p1);
      } else {
        unpack_f32x2(fma_f32x2(s2, scale2, negm2), x0, x1);
        p0 = ex2_approx(x0);
        p1 = ex2_approx(x1);
        t2 = add_f32x2(d2, negd2);
        if (MASKED) {
          if (col0 + k * 16 + c > r) p0 = 0.f;                                    // key index > query index
          if (col0 + k * 16 + c + 1 > r) p1 = 0.f;
        }
      }
      float y0, y1;
      unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), t2), y0, y1);
      ds[(k & 1) * 8 + c / 2] = pack_bf16x2(y0, y1);
    }
    if (k & 1) {   // 32 scores done: 16 columns of bf16 over the start of the 32 columns they came from
      if (DKDV) {
        tmem_st_x16(t_buf + (k >> 1) * 32, pp);
        tmem_st_x16(t_buf + 64 + (k >> 1) * 32, ds);
      } else {
        tmem_st_x16(t_buf + (k >> 1) * 32, ds);
      }
    }
    if (k + 1 < 4) tmem_wait_ld();
  }
}

// ---------------------------------------------------------------------------------------------------------------
// DKDV = true:  one item = (batch*head, key block n); resident K, V; the queries stream (blocks m >= n when causal):
//               S^T = K Qs^T, dP^T = V dOs^T (rows = keys), dV += P^T dOs, dK += dS^T Qs.
// DKDV = false: one item = (batch*head, query block m); resident Q, dO; the keys stream (blocks n <= m when causal):
//               S = Q Ks^T, dP = dO Vs^T (rows = queries), dQ += dS Ks.
// "res0/res1" are the resident pair, "str0/str1" the streamed pair (the factor of res0 / res1 in the score products),
// "out0/out1" the results (dV, dK or dQ, -).
// ---------------------------------------------------------------------------------------------------------------
template <bool DKDV>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_res0, const __grid_constant__ CUtensorMap tmap_res1,
                        const __grid_constant__ CUtensorMap tmap_str0, const __grid_constant__ CUtensorMap tmap_str1,
                        const __grid_constant__ CUtensorMap tmap_out0, const __grid_constant__ CUtensorMap tmap_out1,
                        const BwdParams p) {
  constexpr uint32_t IDESC_X = umma_idesc_bf16_f32(AT_BM, BW_SUB, 0, 0);   // scores: both operands K-major, N = 64
  constexpr uint32_t IDESC_G = umma_idesc_bf16_f32(AT_BM, BW_D, 0, 1);     // gradients: A in tensor memory, B MN-major
  constexpr uint32_t C_ACC0 = 256, C_ACC1 = 384;
  // dQ has one accumulator, so its resident tiles (Q, dO) fit in tensor memory as bf16 A operands (64 columns each):
  // the score MMAs then read only the streamed half-tile from shared memory (32 KB per step instead of 96 KB; shared
  // memory bandwidth, 128 bytes per clock, is what bounds these MMAs at N = 64).  dK/dV has no columns to spare.
  constexpr bool RES_TMEM = !DKDV;
  constexpr uint32_t C_RES0 = 384, C_RES1 = 448;
  constexpr uint32_t STAGE_TX = 2 * BW_SUB_TILE + (DKDV ? 512 : 0);
  // wait sites: 80.. for dK/dV, 90.. for dQ
  constexpr uint32_t SITE = DKDV ? 80 : 90;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_res0 = smem;
  uint8_t* smem_res1 = smem + BW_TILE_BYTES;
  uint8_t* smem_stage = smem + BW_STAGE_OFF;
  uint64_t* res_full = reinterpret_cast<uint64_t*>(smem + BW_BAR_OFF);   // resident tiles have arrived
  uint64_t* res_empty = res_full + 1;                                    // ... may be overwritten (8 warps)
  uint64_t* st_full = res_empty + 1;                                     // [stage] the step's half-tiles have arrived
  uint64_t* st_empty = st_full + BW_NSTAGE;                              // [stage] released by the MMA issuer
  uint64_t* x_full = st_empty + BW_NSTAGE;                               // [buffer] S and dP are in tensor memory
  uint64_t* p_ready = x_full + 2;                                        // [buffer] bf16 P / dS written (4 warps)
  uint64_t* acc_full = p_ready + 2;                                      // accumulators complete
  uint64_t* acc_empty = acc_full + 1;                                    // ... read out (8 warps)
  uint64_t* res_ready = acc_empty + 1;                                   // resident tiles copied to tensor memory (8 warps)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(res_ready + 1);
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
    for (int b = 0; b < 2; ++b) {
      mbar_init(&x_full[b], 1);
      mbar_init(&p_ready[b], BW_SCORE_WARPS / 2);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, BW_SCORE_WARPS);
    mbar_init(res_ready, BW_SCORE_WARPS);
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_res0);
    prefetch_tmap(&tmap_res1);
    prefetch_tmap(&tmap_str0);
    prefetch_tmap(&tmap_str1);
  }
  if (warp_idx == BW_WARP_MMA) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // item -> (batch*head, resident block, range of streamed blocks).  Causal items differ in length: the long ones
  // are handed out first (dK/dV: small n; dQ: large m).
  auto item_range = [&](int item, int& hz, int& blk, int& s_begin, int& s_end) {
    hz = item / p.num_blk;
    blk = item - hz * p.num_blk;
    if (DKDV) {
      s_begin = p.causal ? blk : 0;
      s_end = p.num_blk;
    } else {
      if (p.causal) blk = p.num_blk - 1 - blk;
      s_begin = 0;
      s_end = p.causal ? blk + 1 : p.num_blk;
    }
  };

  if (warp_idx == BW_WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t stage_phase = 0, items = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, blk, s_begin, s_end;
      item_range(item, hz, blk, s_begin, s_end);
      const int row_base = hz * p.N_CTX;
      ok = mbar_wait(res_empty, (items & 1u) ^ 1u, ctx, SITE + 0);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(res_full, 2 * BW_TILE_BYTES);
        load_tile(smem_res0, &tmap_res0, res_full, row_base + blk * AT_BM, AT_BOX_BYTES);
        load_tile(smem_res1, &tmap_res1, res_full, row_base + blk * AT_BM, AT_BOX_BYTES);
      }
      __syncwarp();
      for (int step = 2 * s_begin; ok && step < 2 * s_end; ++step) {
        ok = mbar_wait(&st_empty[stage], stage_phase ^ 1u, ctx, SITE + 1);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* dst = smem_stage + stage * BW_STAGE_BYTES;
          const int row = row_base + step * BW_SUB;
          mbar_expect_tx(&st_full[stage], STAGE_TX);
          load_tile(dst, &tmap_str0, &st_full[stage], row, BW_SUB_BOX);
          load_tile(dst + BW_SUB_TILE, &tmap_str1, &st_full[stage], row, BW_SUB_BOX);
          if (DKDV) {
            bulk_load_1d(dst + 2 * BW_SUB_TILE, p.lse2 + row, 256, &st_full[stage]);
            bulk_load_1d(dst + 2 * BW_SUB_TILE + 256, p.delta + row, 256, &st_full[stage]);
          }
        }
        __syncwarp();
        if (++stage == BW_NSTAGE) { stage = 0; stage_phase ^= 1u; }
      }
    }
  } else if (warp_idx == BW_WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    int xs = 0, gs = 0;                 // ring positions of the next score step / the next gradient step
    uint32_t xs_phase = 0, items = 0, blocks = 0;
    bool ok = true;
    const uint64_t r0_desc = umma_smem_desc_sw128(smem_u32(smem_res0), 16, 1024);
    const uint64_t r1_desc = umma_smem_desc_sw128(smem_u32(smem_res1), 16, 1024);
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, blk, s_begin, s_end;
      item_range(item, hz, blk, s_begin, s_end);
      ok = mbar_wait(RES_TMEM ? res_ready : res_full, items & 1u, ctx, SITE + 2);
      if (!ok) break;
      tc_fence_after();
      const int total = 2 * (s_end - s_begin);
      for (int j = 0; ok && j <= total; ++j) {
        if (j < total) {
          // scores of step j into buffer j & 1.  Its previous user (step j - 2) has been read by the score warps
          // (p_ready was observed) and its gradient MMAs were issued before these; the tensor pipe runs in order
          ok = mbar_wait(&st_full[xs], xs_phase, ctx, SITE + 3);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a0 = smem_u32(smem_stage + xs * BW_STAGE_BYTES);
            const uint64_t s0 = umma_smem_desc_sw128(a0, 16, 1024), s1 = umma_smem_desc_sw128(a0 + BW_SUB_TILE, 16, 1024);
            const uint32_t t = tmem_base + (j & 1) * 128;
            if (RES_TMEM) {
#pragma unroll
              for (int kk = 0; kk < BW_D / 16; ++kk)
                umma_ts(t, tmem_base + C_RES0 + kk * 8, s0 + koff_cols(kk, BW_SUB_BOX), IDESC_X, kk > 0 ? 1u : 0u);
#pragma unroll
              for (int kk = 0; kk < BW_D / 16; ++kk)
                umma_ts(t + 64, tmem_base + C_RES1 + kk * 8, s1 + koff_cols(kk, BW_SUB_BOX), IDESC_X, kk > 0 ? 1u : 0u);
            } else {
#pragma unroll
              for (int kk = 0; kk < BW_D / 16; ++kk)
                umma_ss(t, r0_desc + koff_cols(kk, AT_BOX_BYTES), s0 + koff_cols(kk, BW_SUB_BOX), IDESC_X, kk > 0 ? 1u : 0u);
#pragma unroll
              for (int kk = 0; kk < BW_D / 16; ++kk)
                umma_ss(t + 64, r1_desc + koff_cols(kk, AT_BOX_BYTES), s1 + koff_cols(kk, BW_SUB_BOX), IDESC_X, kk > 0 ? 1u : 0u);
            }
            umma_commit(&x_full[j & 1]);
          }
          __syncwarp();
          if (++xs == BW_NSTAGE) { xs = 0; xs_phase ^= 1u; }
        }
        if (j > 0) {
          // gradients of step j - 1: A = bf16 P / dS in tensor memory (8 columns per k-step of 16 streamed rows)
          const int jj = j - 1;
          ok = mbar_wait(&p_ready[jj & 1], (blocks + (jj >> 1)) & 1u, ctx, SITE + 4);
          if (!ok) break;
          if (jj == 0) {   // the previous item's accumulators must have left tensor memory before they are overwritten
            ok = mbar_wait(acc_empty, (items & 1u) ^ 1u, ctx, SITE + 5);
            if (!ok) break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a0 = smem_u32(smem_stage + gs * BW_STAGE_BYTES);
            const uint64_t n0 = umma_smem_desc_sw128(a0, BW_SUB_BOX, 1024);
            const uint64_t n1 = umma_smem_desc_sw128(a0 + BW_SUB_TILE, BW_SUB_BOX, 1024);
            const uint32_t t = tmem_base + (jj & 1) * 128;
            if (DKDV) {
#pragma unroll
              for (int kk = 0; kk < BW_SUB / 16; ++kk)   // dV += P^T dOs
                umma_ts(tmem_base + C_ACC0, t + bf16_col(kk), n1 + koff_rows(kk), IDESC_G, (jj > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
              for (int kk = 0; kk < BW_SUB / 16; ++kk)   // dK += dS^T Qs
                umma_ts(tmem_base + C_ACC1, t + 64 + bf16_col(kk), n0 + koff_rows(kk), IDESC_G, (jj > 0 || kk > 0) ? 1u : 0u);
            } else {
#pragma unroll
              for (int kk = 0; kk < BW_SUB / 16; ++kk)   // dQ += dS Ks
                umma_ts(tmem_base + C_ACC0, t + bf16_col(kk), n0 + koff_rows(kk), IDESC_G, (jj > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(&st_empty[gs]);
            if (jj == total - 1) umma_commit(acc_full);
          }
          __syncwarp();
          if (++gs == BW_NSTAGE) gs = 0;
        }
      }
      blocks += static_cast<uint32_t>(s_end - s_begin);
    }
  } else {
    // ------------------------------------------------------------------ score rows (warps 0..7)
    // warps 0-3 take the even steps (buffer 0), warps 4-7 the odd ones (buffer 1): the two warps that share a scheduler
    // are half a period apart, so one computes while the other waits for its MMAs, loads and stores
    const int q = warp_idx & 3;          // tensor-memory lane quarter
    const int half = warp_idx >> 2;      // step buffer; in the epilogue the 64-column box
    const int r = q * 32 + static_cast<int>(lane);
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_buf = tmem_base + lane_field + half * 128;
    int stage = half;                    // ring position of this group's next step (steps alternate between the groups)
    uint32_t stage_phase = 0, items = 0, blocks = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x, ++items) {
      int hz, blk, s_begin, s_end;
      item_range(item, hz, blk, s_begin, s_end);
      float m_i = 0.f, d_i = 0.f;
      if (!DKDV) {
        const int64_t my_row = static_cast<int64_t>(hz) * p.N_CTX + blk * AT_BM + r;
        m_i = __ldg(p.lse2 + my_row);
        d_i = __ldg(p.delta + my_row);
      }
      if (RES_TMEM) {
        // group 0 copies Q, group 1 dO: each thread its row, 128 bf16 -> 64 columns (two values per column, the layout
        // of an MMA A operand in tensor memory).  The previous item's MMAs have all completed (acc_full was observed)
        ok = mbar_wait(res_full, items & 1u, ctx, SITE + 9);
        if (!ok) break;
        const uint8_t* src = (half == 0 ? smem_res0 : smem_res1) + r * 128;
        const uint32_t t_res = tmem_base + lane_field + (half == 0 ? C_RES0 : C_RES1);
#pragma unroll
        for (int bx = 0; bx < 2; ++bx) {
          uint32_t w[32];
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint4 v4 = *reinterpret_cast<const uint4*>(src + bx * AT_BOX_BYTES + ((ch ^ (r & 7)) << 4));
            w[4 * ch] = v4.x; w[4 * ch + 1] = v4.y; w[4 * ch + 2] = v4.z; w[4 * ch + 3] = v4.w;
          }
          tmem_st_x32(t_res + bx * 32, w);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(res_ready);
      }
      for (int sb = s_begin; ok && sb < s_end; ++sb, ++blocks) {
        const bool diag = p.causal && sb == blk;
        if (DKDV) {   // the step's M and delta vectors are read from shared memory below: observe their arrival directly
          ok = mbar_wait(&st_full[stage], stage_phase, ctx, SITE + 8);
          if (!ok) break;
        }
        ok = mbar_wait(&x_full[half], blocks & 1u, ctx, SITE + 6);
        if (!ok) break;
        tc_fence_after();
        {
          const float* vec = DKDV ? reinterpret_cast<const float*>(smem_stage + stage * BW_STAGE_BYTES + 2 * BW_SUB_TILE) : nullptr;
          const int col0 = half * BW_SUB;               // the step's first score, as an index into the streamed block
          if (diag) score_step<DKDV, true>(t_buf, vec, p.qk_scale, m_i, d_i, col0, r);
          else score_step<DKDV, false>(t_buf, vec, p.qk_scale, m_i, d_i, col0, r);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[half]);
        stage += 2;                       // BW_NSTAGE is even: a group stays on stages of its own parity
        if (stage >= BW_NSTAGE) { stage -= BW_NSTAGE; stage_phase ^= 1u; }
      }
      if (!ok) break;
      // ---- epilogue: accumulators -> x scale -> bf16 -> staging in the resident tiles (no longer needed) -> TMA store
      ok = mbar_wait(acc_full, items & 1u, ctx, SITE + 7);
      if (!ok) break;
      tc_fence_after();
      store_acc(tmem_base + lane_field + C_ACC0, DKDV ? 1.0f : p.sm_scale, smem_res0, r, half);
      if (DKDV) store_acc(tmem_base + lane_field + C_ACC1, p.sm_scale, smem_res1, r, half);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(acc_empty);
        const int y = hz * p.N_CTX + blk * AT_BM + q * 32;
        tma_store_2d(&tmap_out0, smem_res0 + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y);
        if (DKDV) tma_store_2d(&tmap_out1, smem_res1 + half * AT_BOX_BYTES + q * 32 * 128, half * 64, y);
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
  // resident tiles: boxes of 128 rows; streamed half-tiles: boxes of 64 rows; results: boxes of 32 rows (one warp's)
  CUtensorMap tq_s, tk_s, tv_s, tdo_s;
  if ((rc = make_tmap_bf16_2d(&tq, a.q, BW_D, rows, BW_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tk, a.k, BW_D, rows, BW_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tv, a.v, BW_D, rows, BW_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tdo, a.d_o, BW_D, rows, BW_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tq_s, a.q, BW_D, rows, BW_D, 64, BW_SUB)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tk_s, a.k, BW_D, rows, BW_D, 64, BW_SUB)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tv_s, a.v, BW_D, rows, BW_D, 64, BW_SUB)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tdo_s, a.d_o, BW_D, rows, BW_D, 64, BW_SUB)) != 0) return rc;
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
  B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BW_SMEM_TOTAL));
  attn_bwd_tcgen05_kernel<true><<<grid, BW_THREADS, BW_SMEM_TOTAL, stream>>>(tk, tv, tq_s, tdo_s, tdv, tdk, p);
  count_launch();
  B200K_CHECK_LAUNCH("attn_bwd_tcgen05_kernel<dK, dV>");

  B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BW_SMEM_TOTAL));
  attn_bwd_tcgen05_kernel<false><<<grid, BW_THREADS, BW_SMEM_TOTAL, stream>>>(tq, tdo, tk_s, tv_s, tdq, tdq, p);
  count_launch();
  B200K_CHECK_LAUNCH("attn_bwd_tcgen05_kernel<dQ>");
  return B200K_OK;
}

}  // namespace b200k
