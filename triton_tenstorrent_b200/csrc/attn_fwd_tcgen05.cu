// Fused attention forward for sm_100a: O = softmax(Q K^T * sm_scale [+ causal mask]) V, bf16 in/out,
// HEAD_DIM 16, 32, 64, 128 or 256, blockwise online softmax in the base-2 domain exactly like the reference kernel
// (examples/fused-attn/06-fused-attention.py:33-90 inner loop, :143-215 prologue/epilogue).
//
// One CTA owns a pair of adjacent 128-row Q tiles of one (batch, head) (a single tile for HEAD_DIM 256,
// where tensor memory and shared memory hold one) and walks the K/V blocks of 128 keys once for both:
//   warps 0-3   softmax group of Q tile 0     warps 4-7   softmax group of Q tile 1
//   warp 8      TMA producer (Q tiles, K/V ring of three 32 KB slots in the order K0 V0 K1 V1 ...)
//   warp 9      tensor-memory owner and tcgen05.mma issuer
//   warps 10-11 idle (they complete the third warpgroup so that it can release registers)
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  S = Q K^T is produced
// by an SS MMA; each softmax thread owns one row (tcgen05.ld 32x32b), so row max / row sum need no
// cross-thread exchange; P is rounded to bf16 (the reference's p.to(dtype), :81) and written back
// over the first 64 columns of S; O += P V is a TS MMA with P read from tensor memory and V
// consumed row-major (MN-major B operand).  While one tile's softmax runs, the tensor pipe works on
// the other tile.
//
// Rescaling of O: the reference multiplies the accumulator by alpha = 2^(m_old - m_new) in every
// block (:66-78).  Here the running maximum used for the exponentials is only advanced when it
// would grow by more than 2^8 for some row of the warp (a warp vote), and O (in tensor memory) is
// rescaled only then; P and l are scaled by the same power of two, so O/l is unchanged up to fp32
// rounding, and M = m + log2(l) is unchanged.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <utility>
#include <vector>

#include "attn_common.cuh"
#include "attn_fwd_2cta.cuh"
#include "launch.h"
#include "ptx.cuh"

namespace b200k {

constexpr int AT_THREADS = 384;         // three warpgroups: softmax 0, softmax 1, {TMA, MMA, 2 idle warps}
constexpr int AT_MAX_NSLOT = 3;       // K/V ring slots (2 for head dimension 256).  Measured at D = 128, S = 4096:
                                      // 3 slots 1269 / 1004 TFLOP/s (full / causal), 4: 1264 / 980, 5: 1253 / 970,
                                      // 2: 1223 / 1004 -- a deeper prefetch only adds traffic ahead of its use
constexpr int AT_NBAR = 2 + 2 + 2 * AT_MAX_NSLOT + 2 + 2 + 2 + 2;
// Shared-memory layout for head dimension D: Q0 | Q1 | K/V ring | barriers.  A 128 x D tile is
// max(D/64, 1) boxes of 128 rows x 128 bytes.  For D < 64 a row only fills its first 2*D bytes: TMA pads
// every box row to the 128-byte swizzle span, the MMAs and the TMA store touch only the filled part.
// D = 256 leaves tensor memory (S 128 + O 256 columns) and shared memory for ONE Q tile per CTA.
template <int D>
struct AttnCfg {
  static_assert(D == 16 || D == 32 || D == 64 || D == 128 || D == 256, "head dimension");
  static constexpr int NBOX = D >= 64 ? D / 64 : 1;
  static constexpr int BOX_COLS = D >= 64 ? 64 : D;        // elements per box row
  static constexpr int TILE_BYTES = NBOX * AT_BOX_BYTES;   // footprint in shared memory: 16 .. 64 KB
  static constexpr int TX_BYTES = AT_BM * D * 2;           // bytes a tile load delivers
  static constexpr int NTILE = D <= 128 ? 2 : 1;           // Q tiles per CTA
  static constexpr int NSLOT = D <= 128 ? AT_MAX_NSLOT : 2;
  static constexpr int O_COL0 = NTILE * 128;               // first tensor-memory column of the O accumulators
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = NTILE * TILE_BYTES;
  static constexpr int BAR_OFF = KV_OFF + NSLOT * TILE_BYTES;
  static constexpr int SMEM_TOTAL = BAR_OFF + AT_NBAR * 8 + 16 + 1024;
  static_assert(SMEM_TOTAL <= 232448, "attention shared memory budget exceeded");
  static_assert(O_COL0 + NTILE * (D < 128 ? 128 : D) <= 512, "attention tensor memory budget exceeded");
};

// Two refinements of the softmax path, both measured at Z=4, H=32, N_CTX=4096 (non-causal TFLOP/s at HEAD_DIM 128 / 64;
// with neither: 1261 / 683):
//   halves       P reaches the MMA issuer in two halves of 64 keys, so that half of the PV product runs while the last
//                exponentials are computed and only 4 + 8 MMAs stand between the end of a block's softmax and the next
//                block's scores: 1293-1324 / 766-771.  Always on (B200K_ATTN_P_HALVES=0 builds the whole-block form).
//   early start  the first 32 exponentials start with the current exponent base while the row maximum is still being
//                computed, and are redone from tensor memory when the base has to move: 1287 / 747 alone, 1255 / 795
//                together with the halves.  On for HEAD_DIM <= 64 only, where the exponentials are the bound.
// Tried and dropped: handing P over as 64 + 32 + 32 keys (-10 %: the extra hand-off costs the softmax warps more than
// the two MMAs it moves), and interleaving the scale / sum / pack instructions by hand between the ex2 instructions
// (one warp's mix of 2-3 other instructions per ex2 runs at 9-12 cycles per ex2 however it is ordered; measured with
// a microbenchmark and in the kernel).
#ifndef B200K_ATTN_P_HALVES
#define B200K_ATTN_P_HALVES 1
#endif

struct AttnParams {
  int ZH, N_CTX;
  int num_mblk, num_pairs, num_items;
  int rounds;        // items per CTA (the longest list)
  const int* sched;  // [rounds][grid] item of CTA c in round k (-1 = none); nullptr: item k * grid + c
  int ntile;       // Q tiles per item (2, or 1 for head dimension 256)
  int causal;
  float qk_scale;  // sm_scale * 1.44269504 (fp32 product, as the reference computes it)
  float* lse2;
  uint32_t* status;
  int n_extra;     // further copies of O the epilogue stores every tile to (ExtraMaps)
};

struct AttnItem {
  int hz;
  int mblk[2];
  int nblk[2];  // K/V blocks each tile consumes (0 = tile absent)
  int n;        // K/V blocks loaded
};

__device__ __forceinline__ AttnItem attn_item(const AttnParams& p, int item) {
  AttnItem it;
  it.hz = item / p.num_pairs;
  int pr = item - it.hz * p.num_pairs;
  if (p.causal) pr = p.num_pairs - 1 - pr;  // longest rows first
  it.mblk[0] = p.ntile * pr;
  it.mblk[1] = p.ntile * pr + 1;
  const bool valid1 = p.ntile == 2 && it.mblk[1] < p.num_mblk;
  it.nblk[0] = p.causal ? it.mblk[0] + 1 : p.num_mblk;
  it.nblk[1] = valid1 ? (p.causal ? it.mblk[1] + 1 : p.num_mblk) : 0;
  it.n = it.nblk[1] > it.nblk[0] ? it.nblk[1] : it.nblk[0];
  return it;
}

// The item of this CTA in round k, or -1.  Causal launches read a table made by the host (a list schedule that
// balances the unequal item lengths, see attn_schedule); otherwise items are strided over the CTAs.
__device__ __forceinline__ int attn_round_item(const AttnParams& p, int k) {
  const int idx = k * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
  const int item = p.sched != nullptr ? __ldg(p.sched + idx) : idx;
  return item < p.num_items ? item : -1;
}

// 12 warps start with 168 registers each (16384 per scheduler partition / 96 threads).  The third
// warpgroup then returns registers to the CTA's pool and the softmax warpgroups take them
// (setmaxnreg), so that a softmax thread can hold a whole row of scores plus the packed P values
// without spilling.  Only what the CTA was given at launch can be redistributed:
// 2 x (216 - 168) = 168 - 72 per thread triple.
constexpr int AT_REGS_SOFTMAX = 216;
constexpr int AT_REGS_OTHER = 72;

// RAGGED: N_CTX is not a multiple of 128.  The tensor maps are then three-dimensional, one entry per (batch, head), so
// that tiles and blocks running past N_CTX are zero-filled / clipped instead of touching the next head, and the keys
// past N_CTX are masked.  The unragged instantiation keeps two-dimensional maps over all rows (measured 2 % faster at
// the workload size than the three-dimensional form).
template <int D, bool RAGGED>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                             const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                             const __grid_constant__ ExtraMaps extra, const AttnParams p) {
  constexpr uint32_t IDESC_S = umma_idesc_bf16_f32(AT_BM, AT_BN, 0, 0);   // Q (K-major) x K^T (K-major)
  constexpr uint32_t IDESC_PV = umma_idesc_bf16_f32(AT_BM, D, 0, 1);      // P (TMEM) x V (N-major)
  using Cfg = AttnCfg<D>;
  constexpr int AT_TILE_BYTES = Cfg::TILE_BYTES;
  constexpr int AT_NSLOT = Cfg::NSLOT;
  constexpr bool EARLY_START = D <= 64;   // see the note on the softmax refinements above

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem + Cfg::Q_OFF;
  uint8_t* smem_kv = smem + Cfg::KV_OFF;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* q_empty = q_full + 2;
  uint64_t* kv_full = q_empty + 2;
  uint64_t* kv_empty = kv_full + AT_MAX_NSLOT;
  uint64_t* s_full = kv_empty + AT_MAX_NSLOT;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint64_t* p_half = o_full + 2;    // first 64 keys of P are in tensor memory
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(p_half + 2);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&q_empty[t], 4);
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&p_half[t], 4);
      mbar_init(&o_full[t], 1);
    }
    for (int s = 0; s < AT_NSLOT; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_o);
  }
  if (warp_idx == 9) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // Each role's code is dominated by its warpgroup's setmaxnreg so that the compiler knows its budget.
  if (warp_idx >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(AT_REGS_OTHER));  // all four warps, one instruction
   if (warp_idx == 8) {
    // ------------------------------------------------------------------ TMA producer
    int slot = 0;
    uint32_t slot_phase = 0;
    uint32_t q_loads[2] = {0, 0};
    bool ok = true;
    for (int round = 0; ok && round < p.rounds; ++round) {
      const int item = attn_round_item(p, round);
      if (item < 0) continue;
      const AttnItem it = attn_item(p, item);
      for (int step = 0; ok && step < 2 * it.n; ++step) {
        // Q tiles are interleaved with the first K/V blocks: Q0 K0 Q1 V0 K1 V1 ...
        if (step < 2 && it.nblk[step] > 0) {
          const int t = step;
          ok = mbar_wait(&q_empty[t], (q_loads[t] & 1u) ^ 1u, ctx, 10);
          if (!ok) break;
          if (lane == 0) {
            mbar_expect_tx(&q_full[t], Cfg::TX_BYTES);
            const int row = it.mblk[t] * AT_BM;   // within the (batch, head): rows past N_CTX are zero-filled
#pragma unroll
            for (int bx = 0; bx < Cfg::NBOX; ++bx) {
              uint8_t* dst = smem_q + t * AT_TILE_BYTES + bx * AT_BOX_BYTES;
              if constexpr (RAGGED) tma_load_3d(dst, &tmap_q, &q_full[t], bx * 64, row, it.hz);
              else tma_load_2d(dst, &tmap_q, &q_full[t], bx * 64, it.hz * p.N_CTX + row);
            }
          }
          __syncwarp();
          ++q_loads[t];
        }
        const int j = step >> 1;
        const bool is_v = (step & 1) != 0;
        ok = mbar_wait(&kv_empty[slot], slot_phase ^ 1u, ctx, 11);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(&kv_full[slot], Cfg::TX_BYTES);
          const CUtensorMap* tm = is_v ? &tmap_v : &tmap_k;
          const int row = j * AT_BN;
          uint8_t* dst = smem_kv + slot * AT_TILE_BYTES;
#pragma unroll
          for (int bx = 0; bx < Cfg::NBOX; ++bx) {
            if constexpr (RAGGED) tma_load_3d(dst + bx * AT_BOX_BYTES, tm, &kv_full[slot], bx * 64, row, it.hz);
            else tma_load_2d(dst + bx * AT_BOX_BYTES, tm, &kv_full[slot], bx * 64, it.hz * p.N_CTX + row);
          }
        }
        __syncwarp();
        if (++slot == AT_NSLOT) { slot = 0; slot_phase ^= 1u; }
      }
    }
   } else if (warp_idx == 9) {
    // ------------------------------------------------------------------ MMA issuer
    int slot = 0;                 // next ring slot to consume (K0 V0 K1 V1 ...)
    uint32_t slot_phase = 0;
    uint32_t q_cnt[2] = {0, 0};   // Q tiles consumed per tile index
    uint32_t p_cnt[2] = {0, 0};   // P blocks consumed per tile index
    bool ok = true;
    const uint32_t q_addr[2] = {smem_u32(smem_q), smem_u32(smem_q + AT_TILE_BYTES)};
    const uint32_t kv_addr0 = smem_u32(smem_kv);

    // Descriptors differ from one MMA to the next only in the start-address field (bits 0..13, in
    // units of 16 bytes): build one per operand base and add the offset, so that issuing an MMA
    // costs a couple of integer instructions and the issue thread stays ahead of the tensor pipe.
    const uint64_t q_desc[2] = {umma_smem_desc_sw128(q_addr[0], 16, 1024), umma_smem_desc_sw128(q_addr[1], 16, 1024)};
    const uint64_t k_desc0 = umma_smem_desc_sw128(kv_addr0, 16, 1024);            // K block: K-major
    const uint64_t v_desc0 = umma_smem_desc_sw128(kv_addr0, AT_BOX_BYTES, 1024);  // V block: N-major
    auto issue_s = [&](int t, int slot_idx) {
      // S_t = Q_t K^T : D/16 MMAs of K = 16 over the head dimension (64-column boxes)
      if (lane == 0) {
        const uint64_t kd = k_desc0 + static_cast<uint64_t>((slot_idx * AT_TILE_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = static_cast<uint64_t>(((k >> 2) * AT_BOX_BYTES + (k & 3) * 32) >> 4);
          umma_ss(tmem_base + t * 128, q_desc[t] + off, kd + off, IDESC_S, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      }
      __syncwarp();
    };
    auto issue_pv = [&](int t, int slot_idx, bool accumulate, int k0, int k1) {
      // O_t (+)= P_t V for the key steps [k0, k1) of the block's 8 (K = 16 keys each); P_t is bf16 in TMEM
      // (8 columns per step)
      if (lane == 0) {
        const uint64_t vd = v_desc0 + static_cast<uint64_t>((slot_idx * AT_TILE_BYTES) >> 4);
#pragma unroll
        for (int k = k0; k < k1; ++k)
          umma_ts(tmem_base + Cfg::O_COL0 + t * 128, tmem_base + t * 128 + k * 8, vd + static_cast<uint64_t>((k * 2048) >> 4),
                  IDESC_PV, (accumulate || k > 0) ? 1u : 0u);
      }
      __syncwarp();
    };

    for (int round = 0; ok && round < p.rounds; ++round) {
      const int item = attn_round_item(p, round);
      if (item < 0) continue;
      const AttnItem it = attn_item(p, item);
      // ---- block 0 scores
      ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 20);
      if (!ok) break;
      int k_slot = slot;
      if (++slot == AT_NSLOT) { slot = 0; slot_phase ^= 1u; }
      for (int t = 0; ok && t < 2; ++t) {
        if (it.nblk[t] == 0) continue;
        ok = mbar_wait(&q_full[t], q_cnt[t] & 1u, ctx, 21);
        if (!ok) break;
        ++q_cnt[t];
        tc_fence_after();
        issue_s(t, k_slot);
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&kv_empty[k_slot]);
      __syncwarp();
      // ---- main loop
      for (int j = 0; ok && j < it.n; ++j) {
        ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 22);  // V_j
        if (!ok) break;
        const int v_slot = slot;
        if (++slot == AT_NSLOT) { slot = 0; slot_phase ^= 1u; }
        const bool have_next = (j + 1 < it.n);
        bool next_k_ready = false;
        for (int t = 0; ok && t < 2; ++t) {
          if (j < it.nblk[t]) {
#if B200K_ATTN_P_HALVES
            // the first 64 keys of P arrive while the softmax group still works on the other 64
            ok = mbar_wait(&p_half[t], p_cnt[t] & 1u, ctx, 26);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, v_slot, j > 0, 0, AT_BN / 32);
#endif
            ok = mbar_wait(&p_full[t], p_cnt[t] & 1u, ctx, 23);
            if (!ok) break;
            ++p_cnt[t];
            tc_fence_after();
            issue_pv(t, v_slot, j > 0, B200K_ATTN_P_HALVES ? AT_BN / 32 : 0, AT_BN / 16);
            if (j == it.nblk[t] - 1) {
              if (lane == 0) umma_commit(&o_full[t]);
              __syncwarp();
            }
          }
          if (t == 1) {
            if (lane == 0) umma_commit(&kv_empty[v_slot]);  // every PV of block j has been issued
            __syncwarp();
          }
          if (j + 1 < it.nblk[t]) {
            if (!next_k_ready) {
              ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 24);  // K_{j+1}
              if (!ok) break;
              next_k_ready = true;
              tc_fence_after();
            }
            issue_s(t, slot);
          }
        }
        if (!ok) break;
        if (have_next) {
          if (!next_k_ready) {  // no tile used K_{j+1} (cannot happen while have_next, kept for safety)
            ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 25);
            if (!ok) break;
          }
          if (lane == 0) umma_commit(&kv_empty[slot]);
          __syncwarp();
          if (++slot == AT_NSLOT) { slot = 0; slot_phase ^= 1u; }
        }
      }
    }
   }  // warps 10 and 11 have no role
  } else {
    // ------------------------------------------------------------------ softmax groups (warps 0..7)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(AT_REGS_SOFTMAX));
    const int t = warp_idx >> 2;        // Q tile of this group
    const int q = warp_idx & 3;         // TMEM lane quarter
    const int r = q * 32 + static_cast<int>(lane);  // row within the tile
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + t * 128;        // S_t / P_t
    const uint32_t t_o = tmem_base + lane_field + Cfg::O_COL0 + t * 128;  // O_t
    uint8_t* stage = smem_q + t * AT_TILE_BYTES;                  // O staging reuses the Q tile
    const float scale = p.qk_scale;
    uint32_t blk_cnt = 0, item_cnt = 0;
    bool ok = true;
    for (int round = 0; ok && round < p.rounds; ++round) {
      const int item = attn_round_item(p, round);
      if (item < 0) continue;
      const AttnItem it = attn_item(p, item);
      const int n_me = it.nblk[t];
      if (n_me == 0) continue;
      float m_used = -INFINITY;
      float l = 0.f;
      for (int j = 0; j < n_me; ++j) {
        ok = mbar_wait(&s_full[t], blk_cnt & 1u, ctx, 30);
        if (!ok) break;
        ++blk_cnt;
        tc_fence_after();
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_x32(t_s + 0, s0);
        tmem_ld_x32(t_s + 32, s1);
        tmem_ld_x32(t_s + 64, s2);
        tmem_ld_x32(t_s + 96, s3);
        tmem_wait_ld();
        // Keys of this block a row may see: all 128, except in the diagonal block of a causal launch (key index >
        // query index is masked: the reference adds -1e6 before the max, after exp2 both give exactly 0) and in the
        // last block of a head whose N_CTX is not a multiple of 128 (the keys past N_CTX do not exist; their scores
        // come from zero-filled K rows).  `lim` >= 1 in both cases, so no row is ever fully masked.
        int lim = AT_BN;
        bool masked = p.causal && j == n_me - 1;
        if (masked) lim = r + 1;
        if constexpr (RAGGED) {
          if (p.N_CTX - j * AT_BN < lim) lim = p.N_CTX - j * AT_BN;
          masked = __any_sync(0xFFFFFFFFu, lim < AT_BN);
        }
        if (masked) {
          const uint32_t ninf = 0xFF800000u;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c >= lim) s0[c] = ninf;
            if (c + 32 >= lim) s1[c] = ninf;
            if (c + 64 >= lim) s2[c] = ninf;
            if (c + 96 >= lim) s3[c] = ninf;
          }
        }
        const uint64_t scale2 = pack_f32x2(scale, scale);
        uint64_t negm2 = pack_f32x2(-m_used, -m_used);
        uint64_t sum_a = 0, sum_b = 0;  // bit pattern of (0.f, 0.f)
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        if constexpr (EARLY_START) {
        // The exponent base m_used only moves when a row maximum outgrows it by 2^8, which after the first block
        // of an item is rare.  So the first 32 exponentials are started with the current base while the row maximum
        // over the other 96 scores is still being computed (the max instructions fill the issue slots the ex2 unit
        // leaves free); if the vote below then finds that the base must move, those 32 are recomputed from the
        // scores still in tensor memory.  The first block of an item (m_used = -inf) always takes that path.
#pragma unroll
        for (int c = 0; c < 32; c += 2) mx0 = fmax3(mx0, __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s0[2 * c]), __uint_as_float(s0[2 * c + 1])), scale2, negm2), x0, x1);
          s0[2 * c] = __float_as_uint(x0);
          s0[2 * c + 1] = __float_as_uint(x1);
        }
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          s0[c] = __float_as_uint(ex2_approx(__uint_as_float(s0[c])));
          s0[c + 1] = __float_as_uint(ex2_approx(__uint_as_float(s0[c + 1])));
          mx1 = fmax3(mx1, __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
          mx2 = fmax3(mx2, __uint_as_float(s2[c]), __uint_as_float(s2[c + 1]));
          mx3 = fmax3(mx3, __uint_as_float(s3[c]), __uint_as_float(s3[c + 1]));
        }
#pragma unroll
        for (int c = 0; c < 16; c += 2) {
          sum_a = add_f32x2(sum_a, pack_f32x2(__uint_as_float(s0[2 * c]), __uint_as_float(s0[2 * c + 1])));
          sum_b = add_f32x2(sum_b, pack_f32x2(__uint_as_float(s0[2 * c + 2]), __uint_as_float(s0[2 * c + 3])));
        }
        } else {
#pragma unroll
        for (int c = 0; c < 32; c += 2) {  // 3-input max: two new scores per instruction
          mx0 = fmax3(mx0, __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
          mx1 = fmax3(mx1, __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
          mx2 = fmax3(mx2, __uint_as_float(s2[c]), __uint_as_float(s2[c + 1]));
          mx3 = fmax3(mx3, __uint_as_float(s3[c]), __uint_as_float(s3[c + 1]));
        }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float m_new = fmaxf(m_used, mx * scale);
        const bool need = (m_new - m_used) > AT_RESCALE_THRESHOLD;  // true for j == 0 (m_used = -inf)
        if (__any_sync(0xFFFFFFFFu, need)) {
          const float alpha = (j == 0) ? 0.f : ex2_approx(m_used - m_new);
          m_used = m_new;
          l *= alpha;
          if (j > 0) {
            // the PV MMA of block j-1 has completed (its completion precedes s_full of block j)
            if constexpr (D >= 32) {
#pragma unroll 1
              for (int c4 = 0; c4 < D / 32; ++c4) {
                uint32_t o[32];
                tmem_ld_x32(t_o + c4 * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                tmem_st_x32(t_o + c4 * 32, o);
              }
            } else {
              uint32_t o[16];
              tmem_ld_x16(t_o, o);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tmem_st_x16(t_o, o);
            }
          }
          negm2 = pack_f32x2(-m_used, -m_used);
          if constexpr (EARLY_START) {
          // redo the first 32 exponentials with the new base: their scores are still in tensor memory
          tmem_ld_x32(t_s + 0, s0);
          tmem_wait_ld();
          if (masked) {
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (c >= lim) s0[c] = 0xFF800000u;
          }
          sum_a = 0;
          sum_b = 0;
          exp_block32(s0, scale2, negm2, sum_a, sum_b);
          }
        }
        // p = exp2(s * scale - m): the multiply-subtract and the row sum run two lanes per instruction
        // (fma.rn.f32x2 / add.rn.f32x2); each lane rounds exactly like the scalar fma / add.
        // Three passes per 32 scores, each over independent registers, so that the latency of the
        // special-function unit is covered by the other exponentials instead of by stalls.
        if constexpr (!EARLY_START) exp_block32(s0, scale2, negm2, sum_a, sum_b);
        exp_block32(s1, scale2, negm2, sum_a, sum_b);
        {
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            pk[c] = pack_bf16x2(__uint_as_float(s0[2 * c]), __uint_as_float(s0[2 * c + 1]));
            pk[16 + c] = pack_bf16x2(__uint_as_float(s1[2 * c]), __uint_as_float(s1[2 * c + 1]));
          }
          tmem_st_x32(t_s, pk);
        }
        exp_block32(s2, scale2, negm2, sum_a, sum_b);
#if B200K_ATTN_P_HALVES
        // the first 64 keys of P have had the time of 32 exponentials to land in tensor memory: hand them over, so
        // that half of the PV product runs while the last 32 exponentials are computed
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_half[t]);
#endif
        exp_block32(s3, scale2, negm2, sum_a, sum_b);
        {
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            pk[c] = pack_bf16x2(__uint_as_float(s2[2 * c]), __uint_as_float(s2[2 * c + 1]));
            pk[16 + c] = pack_bf16x2(__uint_as_float(s3[2 * c]), __uint_as_float(s3[2 * c + 1]));
          }
          tmem_st_x32(t_s + 32, pk);
        }
        {
          float sa0, sa1, sb0, sb1;
          unpack_f32x2(sum_a, sa0, sa1);
          unpack_f32x2(sum_b, sb0, sb1);
          l += (sa0 + sa1) + (sb0 + sb1);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      if (!ok) break;
      // ---- epilogue: O / l -> bf16 -> swizzled staging (the Q tile's buffer) -> TMA store; M = m + log2(l)
      ok = mbar_wait(&o_full[t], item_cnt & 1u, ctx, 31);
      if (!ok) break;
      ++item_cnt;
      tc_fence_after();
      const float inv_l = 1.0f / l;
      if constexpr (D >= 32) {
#pragma unroll 1
        for (int c4 = 0; c4 < D / 32; ++c4) {
          uint32_t o[32];
          tmem_ld_x32(t_o + c4 * 32, o);
          tmem_wait_ld();
          uint8_t* row_ptr = stage + (c4 >> 1) * AT_BOX_BYTES + r * 128;
          const int chunk0 = (c4 & 1) * 4;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint4 val;
            val.x = pack_bf16x2(__uint_as_float(o[8 * jj + 0]) * inv_l, __uint_as_float(o[8 * jj + 1]) * inv_l);
            val.y = pack_bf16x2(__uint_as_float(o[8 * jj + 2]) * inv_l, __uint_as_float(o[8 * jj + 3]) * inv_l);
            val.z = pack_bf16x2(__uint_as_float(o[8 * jj + 4]) * inv_l, __uint_as_float(o[8 * jj + 5]) * inv_l);
            val.w = pack_bf16x2(__uint_as_float(o[8 * jj + 6]) * inv_l, __uint_as_float(o[8 * jj + 7]) * inv_l);
            *reinterpret_cast<uint4*>(row_ptr + (((chunk0 + jj) ^ (r & 7)) << 4)) = val;
          }
        }
      } else {
        uint32_t o[16];
        tmem_ld_x16(t_o, o);
        tmem_wait_ld();
        uint8_t* row_ptr = stage + r * 128;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          uint4 val;
          val.x = pack_bf16x2(__uint_as_float(o[8 * jj + 0]) * inv_l, __uint_as_float(o[8 * jj + 1]) * inv_l);
          val.y = pack_bf16x2(__uint_as_float(o[8 * jj + 2]) * inv_l, __uint_as_float(o[8 * jj + 3]) * inv_l);
          val.z = pack_bf16x2(__uint_as_float(o[8 * jj + 4]) * inv_l, __uint_as_float(o[8 * jj + 5]) * inv_l);
          val.w = pack_bf16x2(__uint_as_float(o[8 * jj + 6]) * inv_l, __uint_as_float(o[8 * jj + 7]) * inv_l);
          *reinterpret_cast<uint4*>(row_ptr + ((jj ^ (r & 7)) << 4)) = val;
        }
      }
      tc_fence_before();
      const int row_in_head = it.mblk[t] * AT_BM;
      if (!RAGGED || row_in_head + r < p.N_CTX)    // the last tile of a head may run past N_CTX: those rows do not exist
        p.lse2[static_cast<int64_t>(it.hz) * p.N_CTX + row_in_head + r] = m_used + log2f(l);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int y = row_in_head + q * 32;   // rows past N_CTX are clipped by the store
        auto store_to = [&](const CUtensorMap* m) {
#pragma unroll
          for (int bx = 0; bx < Cfg::NBOX; ++bx) {
            const uint8_t* src = stage + bx * AT_BOX_BYTES + q * 32 * 128;
            if constexpr (RAGGED) tma_store_3d(m, src, bx * 64, y, it.hz);
            else tma_store_2d(m, src, bx * 64, it.hz * p.N_CTX + y);
          }
        };
        if (!RAGGED || y < p.N_CTX) {
          store_to(&tmap_o);
          for (int d = 0; d < p.n_extra; ++d) store_to(&extra.m[d]);
        }
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(&q_empty[t]);  // the Q buffer may be refilled
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // -------------------------------------------------------------------- teardown
  drain_after_abort(abort_smem);
  tc_fence_before();
  __syncthreads();
  if (warp_idx == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int attn_supported(int D, int N_CTX) {
  const bool d_ok = D == 16 || D == 32 || D == 64 || D == 128 || D == 256;   // the reference's set (06-fused-attention.py:233)
  // any sequence length: tensor maps are per (batch, head), so tiles and blocks that run past N_CTX are zero-filled
  // on loads, clipped on stores, and their keys masked (the reference itself walks whole BLOCK_M / BLOCK_N blocks
  // and is only meaningful for multiples of them: 32, 64 or 128 depending on the configuration it picks, :110-121)
  return (d_ok && N_CTX >= 1) ? 1 : 0;
}

static int pick_grid(int sm_count, int num_items, int num_pairs, bool causal) {
  int grid = num_items < sm_count ? num_items : sm_count;
  if (causal && num_pairs > 1 && grid > 1) {
    // Items are strided over CTAs; with a stride that shares a factor with the number of row pairs
    // per head a CTA would only ever see a few of the (unequally long) causal row positions.
    auto gcd = [](int a, int b) { while (b) { int t = a % b; a = b; b = t; } return a; };
    while (grid > 1 && gcd(grid, num_pairs) != 1) --grid;
  }
  return grid;
}

// Argument checks shared by the entry points.
static int attn_check_args(const AttnArgs& a) {
  if (a.Z <= 0 || a.H <= 0 || a.N_CTX <= 0) return set_error(B200K_ERR_INVALID_ARG, "attention: Z, H, N_CTX must be positive");
  if (!attn_supported(a.D, a.N_CTX))
    return set_error(B200K_ERR_UNSUPPORTED, "attention: HEAD_DIM %d / N_CTX %d not supported (HEAD_DIM 16, 32, 64, 128 or 256; N_CTX >= 1)", a.D, a.N_CTX);
  if (a.q == nullptr || a.k == nullptr || a.v == nullptr || a.o == nullptr || a.lse2 == nullptr)
    return set_error(B200K_ERR_INVALID_ARG, "attention: null pointer");
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
       reinterpret_cast<uintptr_t>(a.o)) & 15u)
    return set_error(B200K_ERR_INVALID_ARG, "attention: q, k, v, o must be 16-byte aligned");
  if (a.n_extra < 0 || a.n_extra > MAX_EXTRA_DESTS || (a.n_extra > 0 && a.extra_o == nullptr))
    return set_error(B200K_ERR_INVALID_ARG, "attention: 0..%d extra destinations supported (got %d)", MAX_EXTRA_DESTS, a.n_extra);
  for (int d = 0; d < a.n_extra; ++d)
    if (a.extra_o[d] == nullptr || (reinterpret_cast<uintptr_t>(a.extra_o[d]) & 15u))
      return set_error(B200K_ERR_INVALID_ARG, "attention: extra destination %d is null or not 16-byte aligned", d);
  // Z*H first (two positive ints cannot overflow 64 bits), then the row count
  const int64_t zh = static_cast<int64_t>(a.Z) * a.H;
  if (zh > 0x7FFFFFFF || zh * a.N_CTX > 0x7FFFFFFF) return set_error(B200K_ERR_INVALID_ARG, "attention: Z*H*N_CTX exceeds 2^31-1 rows");
  if (!(a.sm_scale > 0.f) || !isfinite(a.sm_scale)) return set_error(B200K_ERR_INVALID_ARG, "attention: sm_scale must be positive and finite");
  return B200K_OK;
}

// Causal items differ in length (2 to 2 * num_pairs K/V blocks), so dealing them out with a fixed stride leaves
// some CTAs with up to 12 % more work than the average.  The host instead simulates a work queue: items are taken
// in launch order (head by head, longest row position first, so that the CTAs running at the same time share
// the K/V of a few heads in L2) by whichever CTA becomes free first.  The resulting table [rounds][grid] lives in
// device memory, one per (shape, grid, device), created at the first launch of that shape.
struct SchedKey {
  int device, ZH, num_pairs, num_mblk, ntile, grid;
  bool operator<(const SchedKey& o) const {
    return std::tie(device, ZH, num_pairs, num_mblk, ntile, grid) <
           std::tie(o.device, o.ZH, o.num_pairs, o.num_mblk, o.ntile, o.grid);
  }
};
struct SchedTable {
  int* dev;
  int rounds;
};
static std::map<SchedKey, SchedTable> g_sched;
static std::mutex g_sched_mutex;

// K/V blocks a causal item walks: its last Q tile's diagonal block is the last one (items hold ntile tiles:
// 1 for head dimension 256, 2 in the single-CTA kernel, 4 in the CTA-pair kernel).
static int causal_item_blocks(int item, int num_pairs, int num_mblk, int ntile) {
  const int pr = num_pairs - 1 - item % num_pairs;
  const int n = ntile * (pr + 1);
  return n < num_mblk ? n : num_mblk;
}

std::vector<int> attn_schedule(int ZH, int num_pairs, int num_mblk, int ntile, int grid, int* rounds_out) {
  const int num_items = ZH * num_pairs;
  std::vector<std::vector<int>> lists(grid);
  // (time at which the CTA is free, CTA): smallest first
  std::priority_queue<std::pair<double, int>, std::vector<std::pair<double, int>>, std::greater<std::pair<double, int>>> free_at;
  for (int c = 0; c < grid; ++c) free_at.push({0.0, c});
  // Launch order: head by head, longest row position first; the items of the last few heads (about one and a half
  // rounds) are merged and taken longest first across those heads, so that the queue ends with the shortest items.
  std::vector<int> order;
  order.reserve(num_items);
  int tail_heads = (3 * grid / 2 + num_pairs - 1) / num_pairs;
  if (tail_heads > ZH) tail_heads = ZH;
  for (int item = 0; item < (ZH - tail_heads) * num_pairs; ++item) order.push_back(item);
  for (int level = 0; level < num_pairs; ++level)
    for (int hz = ZH - tail_heads; hz < ZH; ++hz) order.push_back(hz * num_pairs + level);
  for (int item : order) {
    auto [t, c] = free_at.top();
    free_at.pop();
    lists[c].push_back(item);
    // one period per K/V block plus about one for loading Q, the first scores and the epilogue
    free_at.push({t + causal_item_blocks(item, num_pairs, num_mblk, ntile) + 1.0, c});
  }
  size_t rounds = 0;
  for (const auto& l : lists) rounds = l.size() > rounds ? l.size() : rounds;
  std::vector<int> table(rounds * grid, -1);
  for (int c = 0; c < grid; ++c)
    for (size_t k = 0; k < lists[c].size(); ++k) table[k * grid + c] = lists[c][k];
  *rounds_out = static_cast<int>(rounds);
  return table;
}

// At most this many schedule tables are kept per process; a caller that walks through more shapes than that gets
// the tables rebuilt (after a device synchronisation, so that no launch in flight still reads a freed one).
constexpr size_t AT_MAX_SCHEDULES = 64;

static int get_schedule(const SchedKey& key, cudaStream_t stream, const int** dev_table, int* rounds) {
  std::lock_guard<std::mutex> lock(g_sched_mutex);
  auto it = g_sched.find(key);
  if (it == g_sched.end()) {
    if (g_sched.size() >= AT_MAX_SCHEDULES) {
      B200K_CHECK_CUDA(cudaDeviceSynchronize());
      for (auto& kv : g_sched) {
        int cur = 0;
        if (cudaGetDevice(&cur) == cudaSuccess && cur == kv.first.device) {
          cudaFree(kv.second.dev);
        } else if (cudaSetDevice(kv.first.device) == cudaSuccess) {
          cudaDeviceSynchronize();
          cudaFree(kv.second.dev);
          cudaSetDevice(cur);
        }
      }
      g_sched.clear();
    }
    int r = 0;
    const std::vector<int> table = attn_schedule(key.ZH, key.num_pairs, key.num_mblk, key.ntile, key.grid, &r);
    int* dev = nullptr;
    B200K_CHECK_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev), table.size() * sizeof(int)));
    // Upload on the launch stream and wait for it: a copy from pageable memory on the legacy stream is not ordered
    // with a non-blocking stream, so the first launch of a shape on a side stream could otherwise read the table
    // before it has arrived.  First use of a shape only.
    cudaError_t e = cudaMemcpyAsync(dev, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
      cudaFree(dev);
      return set_error(B200K_ERR_CUDA, "attention: uploading the causal schedule failed: %s", cudaGetErrorString(e));
    }
    it = g_sched.emplace(key, SchedTable{dev, r}).first;
  }
  *dev_table = it->second.dev;
  *rounds = it->second.rounds;
  return B200K_OK;
}

// The CTA-pair kernel (attn_fwd_2cta.cuh): head dimension 128, whole groups of four Q tiles.
// Not the default: it measures slightly slower than the single-CTA kernel (see the note in that file).
static bool attn2_applies(const AttnArgs& a) {
  if (a.D != A2_D || a.N_CTX % (4 * AT_BM) != 0) return false;
  const char* e = getenv("B200K_ATTN_2CTA");
  return e != nullptr && atoi(e) != 0;
}

static int attn2_launch(const AttnArgs& a, cudaStream_t stream, int sm_count, uint32_t* status, bool may_allocate) {
  const int64_t rows = static_cast<int64_t>(a.Z) * a.H * a.N_CTX;
  CUtensorMap tq, tk, tv, to;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tq, a.q, A2_D, rows, A2_D, 64, AT_BM)) != 0) return rc;
  if ((rc = make_tmap_bf16_2d(&tk, a.k, A2_D, rows, A2_D, 64, AT_BN / 2)) != 0) return rc;   // half of a block's keys
  if ((rc = make_tmap_bf16_2d(&tv, a.v, A2_D, rows, A2_D, 64, AT_BN)) != 0) return rc;       // half of the columns
  if ((rc = make_tmap_bf16_2d(&to, a.o, A2_D, rows, A2_D, 64, 32)) != 0) return rc;
  ExtraMaps extra;
  memset(&extra, 0, sizeof(extra));
  for (int d = 0; d < a.n_extra; ++d)
    if ((rc = make_tmap_bf16_2d(&extra.m[d], a.extra_o[d], A2_D, rows, A2_D, 64, 32)) != 0) return rc;

  Attn2Params p;
  p.ZH = a.Z * a.H;
  p.N_CTX = a.N_CTX;
  p.num_mblk = a.N_CTX / AT_BM;
  p.num_quads = p.num_mblk / 4;
  p.num_items = p.ZH * p.num_quads;
  p.causal = a.causal ? 1 : 0;
  p.qk_scale = a.sm_scale * 1.44269504f;
  p.lse2 = a.lse2;
  p.status = status;
  p.n_extra = a.n_extra;

  const int max_pairs = sm_count / 2;
  int pairs = pick_grid(max_pairs, p.num_items, p.num_quads, p.causal != 0);
  p.sched = nullptr;
  p.rounds = (p.num_items + pairs - 1) / pairs;
  const char* sched_env = getenv("B200K_ATTN_SCHEDULE");
  if (p.causal && p.num_quads > 1 && may_allocate && !(sched_env != nullptr && atoi(sched_env) == 0)) {
    pairs = p.num_items < max_pairs ? p.num_items : max_pairs;   // the table balances any grid: use every pair
    int dev = 0;
    B200K_CHECK_CUDA(cudaGetDevice(&dev));
    if ((rc = get_schedule(SchedKey{dev, p.ZH, p.num_quads, p.num_mblk, 4, pairs}, stream, &p.sched, &p.rounds)) != 0) return rc;
  }
  B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_bf16_tcgen05_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        A2_SMEM_TOTAL));
  attn_fwd_bf16_tcgen05_2cta_kernel<<<2 * pairs, A2_THREADS, A2_SMEM_TOTAL, stream>>>(tq, tk, tv, to, extra, p);
  count_launch();
  B200K_CHECK_LAUNCH("attn_fwd_bf16_tcgen05_2cta_kernel");
  return B200K_OK;
}

// Encodes the tensor maps and launches the kernel on `sm_count` SMs, reporting to `status`.
static int attn_launch(const AttnArgs& a, cudaStream_t stream, int sm_count, uint32_t* status, bool may_allocate) {
  if (attn2_applies(a) && sm_count >= 2) return attn2_launch(a, stream, sm_count, status, may_allocate);
  CUtensorMap tq, tk, tv, to;
  int rc;
  const uint64_t D = static_cast<uint64_t>(a.D);
  const uint32_t box_cols = a.D >= 64 ? 64u : static_cast<uint32_t>(a.D);
  // ragged sequence lengths: [Z*H][N_CTX][D], one tensor-map entry per (batch, head); otherwise all rows as one matrix
  const uint64_t zh = static_cast<uint64_t>(a.Z) * a.H, n_ctx = static_cast<uint64_t>(a.N_CTX);
  const bool ragged = (a.N_CTX % AT_BM) != 0;
  auto make_map = [&](CUtensorMap* m, const void* base, uint32_t box_rows) {
    return ragged ? make_tmap_bf16_3d(m, base, D, n_ctx, zh, box_cols, box_rows)
                  : make_tmap_bf16_2d(m, base, D, zh * n_ctx, D, box_cols, box_rows);
  };
  if ((rc = make_map(&tq, a.q, AT_BM)) != 0) return rc;
  if ((rc = make_map(&tk, a.k, AT_BN)) != 0) return rc;
  if ((rc = make_map(&tv, a.v, AT_BN)) != 0) return rc;
  if ((rc = make_map(&to, a.o, 32)) != 0) return rc;
  ExtraMaps extra;
  memset(&extra, 0, sizeof(extra));
  for (int d = 0; d < a.n_extra; ++d)
    if ((rc = make_map(&extra.m[d], a.extra_o[d], 32)) != 0) return rc;

  AttnParams p;
  p.ZH = a.Z * a.H;
  p.N_CTX = a.N_CTX;
  p.num_mblk = (a.N_CTX + AT_BM - 1) / AT_BM;
  p.ntile = a.D <= 128 ? 2 : 1;
  p.num_pairs = (p.num_mblk + p.ntile - 1) / p.ntile;
  p.num_items = p.ZH * p.num_pairs;
  p.causal = a.causal ? 1 : 0;
  p.qk_scale = a.sm_scale * 1.44269504f;
  p.lse2 = a.lse2;
  p.status = status;
  p.n_extra = a.n_extra;

  int grid = pick_grid(sm_count, p.num_items, p.num_pairs, p.causal != 0);
  if (const char* g = getenv("B200K_ATTN_GRID")) { int v = atoi(g); if (v > 0 && v <= p.num_items) grid = v; }
  p.sched = nullptr;
  p.rounds = (p.num_items + grid - 1) / grid;
  const char* sched_env = getenv("B200K_ATTN_SCHEDULE");
  if (p.causal && p.num_pairs > 1 && may_allocate && !(sched_env != nullptr && atoi(sched_env) == 0)) {
    grid = p.num_items < sm_count ? p.num_items : sm_count;   // the table balances any grid: use every SM
    int dev = 0;
    B200K_CHECK_CUDA(cudaGetDevice(&dev));
    if ((rc = get_schedule(SchedKey{dev, p.ZH, p.num_pairs, p.num_mblk, p.ntile, grid}, stream, &p.sched, &p.rounds)) != 0) return rc;
  }
  // function attributes belong to the current context (per device); cheap enough to repeat
#define B200K_ATTN_LAUNCH_R(DD, RR)                                                                                   \
  do {                                                                                                              \
    B200K_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_bf16_tcgen05_kernel<DD, RR>,                                     \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<DD>::SMEM_TOTAL));   \
    attn_fwd_bf16_tcgen05_kernel<DD, RR><<<grid, AT_THREADS, AttnCfg<DD>::SMEM_TOTAL, stream>>>(tq, tk, tv, to, extra, p); \
  } while (0)
#define B200K_ATTN_LAUNCH(DD)                     \
  case DD:                                        \
    if (ragged) B200K_ATTN_LAUNCH_R(DD, true);    \
    else B200K_ATTN_LAUNCH_R(DD, false);          \
    break;
  switch (a.D) {
    B200K_ATTN_LAUNCH(16)
    B200K_ATTN_LAUNCH(32)
    B200K_ATTN_LAUNCH(64)
    B200K_ATTN_LAUNCH(128)
    B200K_ATTN_LAUNCH(256)
    default:
      return set_error(B200K_ERR_UNSUPPORTED, "attention: HEAD_DIM %d not built", a.D);
  }
#undef B200K_ATTN_LAUNCH_R
#undef B200K_ATTN_LAUNCH
  count_launch();
  B200K_CHECK_LAUNCH("attn_fwd_bf16_tcgen05_kernel");
  return B200K_OK;
}

int attn_fwd_bf16(const AttnArgs& a, cudaStream_t stream) {
  const int rc = attn_check_args(a);
  if (rc != B200K_OK) return rc;
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  if (dev->cc_major != 10) return set_error(B200K_ERR_NO_DEVICE, "attention: needs an sm_100 device (found sm_%d%d)", dev->cc_major, dev->cc_minor);
  return attn_launch(a, stream, dev->sm_count, dev->status_word, /*may_allocate=*/true);
}

}  // namespace b200k

// ---------------------------------------------------------------------------------------------
// Attention forward for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
// b200k_attn_fwd_bf16 needs two pieces of device memory besides q, k, v and o: the row statistics
// M (one fp32 per query row, which the caller must allocate even when it only wants O) and the
// library's status word, which the first call on a device obtains with cudaMalloc.  Some callers can
// do neither: code running under a memory pool that forbids raw CUDA allocations, a plugin that is
// handed fixed buffers by its host application, or a serving loop that must not touch the allocator
// once it is warm.  For them the same kernel is launched with both pieces placed in the static device
// array below, which every GPU that loads this library holds from module load until exit.
//
// Layout: words [0, 64) status block (the kernel uses word 0), then one fp32 per query row.
#define B200K_ATTN_NOALLOC_MAX_ROWS 524288  /* Z*H*N_CTX; 2 MiB of row statistics (+256 B) per GPU */
static __device__ __align__(256) uint32_t g_attn_noalloc_scratch[64 + B200K_ATTN_NOALLOC_MAX_ROWS];

namespace b200k {

struct NoAllocDevice {
  uint32_t* scratch;  // device address of g_attn_noalloc_scratch on that device
  int sm_count;
  int cc_major;
};
static NoAllocDevice g_noalloc_dev[64];
static std::atomic<int> g_noalloc_ready[64];
static std::mutex g_noalloc_mutex;

// Per-device set-up (first call on a device, with that device current): the array's name is only a
// host-side handle, so its device address is looked up once and cached.  Nothing is allocated.
// Returns B200K_OK and the device record, or the status code that matches the error message.
static int noalloc_device(const NoAllocDevice** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return set_error(B200K_ERR_NO_DEVICE, "attention (no-alloc): no usable current device (%s)", cudaGetErrorString(e));
  if (!g_noalloc_ready[dev].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ready[dev].load(std::memory_order_acquire)) {
      NoAllocDevice d{};
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_attn_noalloc_scratch);
      if (e != cudaSuccess || ptr == nullptr)
        return set_error(B200K_ERR_CUDA, "attention (no-alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      d.scratch = static_cast<uint32_t*>(ptr);
      if ((e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
          (e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
        return set_error(B200K_ERR_CUDA, "attention (no-alloc): cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
      g_noalloc_dev[dev] = d;
      g_noalloc_ready[dev].store(1, std::memory_order_release);
    }
  }
  if (g_noalloc_dev[dev].cc_major != 10)
    return set_error(B200K_ERR_NO_DEVICE, "attention (no-alloc): needs an sm_100 device");
  *out = &g_noalloc_dev[dev];
  return B200K_OK;
}

}  // namespace b200k

extern "C" int b200k_attn_fwd_bf16_noalloc(const void* q, const void* k, const void* v, void* o, int Z, int H, int N_CTX,
                                           int D, int causal, float sm_scale, void* stream) {
  using namespace b200k;
  clear_error();
  if (Z > 0 && H > 0 && N_CTX > 0) {
    // Z*H first: the product of two positive ints fits 64 bits, and once it is within the limit so does the row count
    const int64_t zh = static_cast<int64_t>(Z) * H;
    if (zh > B200K_ATTN_NOALLOC_MAX_ROWS || zh * N_CTX > B200K_ATTN_NOALLOC_MAX_ROWS)
      return set_error(B200K_ERR_INVALID_ARG,
                       "attention (no-alloc): Z*H*N_CTX = %d*%d*%d query rows exceed the %d rows the static scratch holds; "
                       "split the batch or use b200k_attn_fwd_bf16 with a caller-provided M buffer",
                       Z, H, N_CTX, B200K_ATTN_NOALLOC_MAX_ROWS);
  }
  // dummy non-null M so that the shared checks apply unchanged; replaced below
  AttnArgs a{q, k, v, o, reinterpret_cast<float*>(uintptr_t(16)), Z, H, N_CTX, D, causal, sm_scale};
  int rc = attn_check_args(a);
  if (rc != B200K_OK) return rc;
  const NoAllocDevice* dev = nullptr;
  if ((rc = noalloc_device(&dev)) != B200K_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // A failure that an earlier call recorded stays in word 0 until b200k_attn_noalloc_status has reported it (the
  // kernel records only into a zero word), so nothing is cleared here; the row statistics are write-only.
  a.lse2 = reinterpret_cast<float*>(dev->scratch + 64);
  return attn_launch(a, s, dev->sm_count, dev->scratch, /*may_allocate=*/false);  // strided items, no schedule table
}

// The status word of the no-allocation path lives in the static array (word 0), where b200k_device_status, which
// reads the library's allocated per-device word, never looks.  This reader copies it to the caller's host word on
// `stream`, waits for the stream, and clears it after reporting a failure.  It allocates nothing either.
extern "C" int b200k_attn_noalloc_status(void* stream, uint32_t* code) {
  using namespace b200k;
  clear_error();
  const NoAllocDevice* dev = nullptr;
  const int rc = noalloc_device(&dev);
  if (rc != B200K_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t host = 0;
  B200K_CHECK_CUDA(cudaMemcpyAsync(&host, dev->scratch, sizeof(host), cudaMemcpyDeviceToHost, s));
  B200K_CHECK_CUDA(cudaStreamSynchronize(s));
  if (code != nullptr) *code = host;
  if (host != 0) {
    B200K_CHECK_CUDA(cudaMemsetAsync(dev->scratch, 0, 2 * sizeof(uint32_t), s));
    B200K_CHECK_CUDA(cudaStreamSynchronize(s));
    return set_error(B200K_ERR_DEVICE_TIMEOUT, "a bounded device-side wait of the no-allocation attention gave up (site %u)", host >> 8);
  }
  return B200K_OK;
}

// The bounded-wait self-test (a wait on a barrier that nothing completes, with a small cycle budget) reporting into the
// static array's status block instead of the allocated per-device word: shows that a wait which gives up on the
// no-allocation path is visible through b200k_attn_noalloc_status.  Faults nothing; the kernel returns normally.
extern "C" int b200k_attn_noalloc_selftest(int64_t budget_cycles, void* stream) {
  using namespace b200k;
  clear_error();
  const NoAllocDevice* dev = nullptr;
  const int rc = noalloc_device(&dev);
  if (rc != B200K_OK) return rc;
  return selftest_wait_timeout_at(dev->scratch, budget_cycles, static_cast<cudaStream_t>(stream));
}
