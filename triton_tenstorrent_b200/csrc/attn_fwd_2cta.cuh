// Fused attention forward on CTA pairs (tcgen05 cta_group::2), HEAD_DIM 128, N_CTX a multiple of 512.
// Same arithmetic as the single-CTA kernel (attn_fwd_tcgen05.cu: base-2 online softmax of
// examples/fused-attn/06-fused-attention.py:33-90, P rounded to bf16 before P V, lazy rescale of O); what
// changes is who holds which operand:
//
//   A cluster of two CTAs owns FOUR adjacent 128-row Q tiles of one (batch, head).  MMA "tile" t (t = 0, 1) is
//   256 rows tall: rows [256 t, 256 t + 128) belong to CTA 0, rows [256 t + 128, 256 t + 256) to CTA 1, and one
//   tcgen05.mma.cta_group::2 instruction (M = 256) issued by CTA 0 computes both halves.
//   S = Q K^T : each CTA supplies its own Q tile (A, 128 rows) and HALF of the K block (B: 64 of the 128 keys).
//   O += P V  : each CTA supplies its own P from its tensor memory (A) and HALF of the V block (B: 64 of the 128
//               head-dimension columns).
//   So every SM reads 6 KB (scores) / 2 KB (PV) of shared memory per MMA instead of 8 KB / 4 KB, and loads half of
//   every K/V block.
//
// MEASURED, and the reason this kernel is NOT the default (B200K_ATTN_2CTA=1 selects it): at Z=4, H=32, N_CTX=4096 it
// reaches 1305 TFLOP/s against the single-CTA kernel's 1340 (causal 1082 against 1180, where the 512-row items also
// balance worse).  A microbenchmark of back-to-back tcgen05.mma shows why nothing is gained on the tensor pipe: an
// M = 128 per SM, N = 128, K = 16 instruction takes 64 cycles whether A comes from shared or tensor memory and
// whether it is cta_group::1 or ::2 (N = 256: 128 cycles; N = 64: 45-48, never 32), so the single-CTA kernel's MMAs
// are not limited by shared-memory reads, and both kernels are bound by the same per-tile chain
// softmax -> PV -> next scores.  Two things learnt on the way, both kept:
//   * the softmax warps of CTA 1 must arrive on CTA 0's barriers with the default CTA-scope release
//     (mbar_arrive_remote); with mbarrier.arrive.release.cluster each arrival cost about 650 cycles (881 TFLOP/s);
//   * the two tiles' softmax groups share the ex2 units, and the offset they start an item with persists for the
//     whole item, so tile 1's first scores are issued only when tile 0's first P half has arrived.
//
// Roles per CTA (384 threads) are those of the single-CTA kernel: warps 0-3 / 4-7 softmax of the CTA's two Q tiles,
// warp 8 TMA producer (own Q tiles, own halves of K and V: a ring of six 16 KB slots), warp 9 MMA issuer (CTA 0
// only), warps 10-11 donate registers.  Tensor memory per CTA: S0 | S1 | O0 | O1 (its own 128 rows of each).
// Barriers: loads of both CTAs are counted on CTA 0's "full" barriers; CTA 0's tcgen05.commit releases ring slots and
// publishes scores / outputs on the barriers of both CTAs; the softmax warps of both CTAs arrive on CTA 0's
// "P ready" barriers.  No multicast loads.
//
// Causal: tile t of the pair needs the K/V blocks 0 .. 4 q + 2 t + 1 (q = index of the 512-row group); CTA 0's rows
// end one block earlier than CTA 1's, so its last block is fully masked: it hands over P = 0 without computing.
#pragma once
#include "attn_common.cuh"
#include "launch.h"
#include "ptx.cuh"

namespace b200k {

#ifndef B200K_ATTN2_STAGGER
#define B200K_ATTN2_STAGGER 1
#endif

constexpr int A2_D = 128;
constexpr int A2_THREADS = 384;
constexpr int A2_TILE_BYTES = AT_BM * A2_D * 2;   // one Q tile: 32 KB (two boxes of 128 rows x 64 columns)
constexpr int A2_SLOT_BYTES = 16384;              // half a K block (64 keys x 128) or half a V block (128 keys x 64)
constexpr int A2_NSLOT = 6;
constexpr int A2_NBAR = 2 + 2 + 2 * A2_NSLOT + 2 + 2 + 2 + 2;
constexpr int A2_Q_OFF = 0;
constexpr int A2_KV_OFF = 2 * A2_TILE_BYTES;
constexpr int A2_BAR_OFF = A2_KV_OFF + A2_NSLOT * A2_SLOT_BYTES;
constexpr int A2_SMEM_TOTAL = A2_BAR_OFF + A2_NBAR * 8 + 16 + 1024;
static_assert(A2_SMEM_TOTAL <= 232448, "attention (CTA pair) shared memory budget exceeded");
constexpr int A2_O_COL0 = 256;                    // tensor-memory columns: S0 0, S1 128, O0 256, O1 384
constexpr int A2_REGS_SOFTMAX = 216;
constexpr int A2_REGS_OTHER = 72;

struct Attn2Params {
  int ZH, N_CTX;
  int num_mblk;      // 128-row tiles per head
  int num_quads;     // 512-row groups per head
  int num_items;     // ZH * num_quads
  int rounds;        // items per pair (the longest list)
  const int* sched;  // [rounds][pairs] item of pair c in round k (-1 = none); nullptr: item k * pairs + c
  int causal;
  float qk_scale;
  float* lse2;
  uint32_t* status;
  int n_extra;
};

struct Attn2Item {
  int hz;
  int quad;     // 512-row group (longest first when causal)
  int nblk[2];  // K/V blocks MMA tile t consumes
  int n;        // K/V blocks loaded
};

__device__ __forceinline__ Attn2Item attn2_item(const Attn2Params& p, int item) {
  Attn2Item it;
  it.hz = item / p.num_quads;
  int q = item - it.hz * p.num_quads;
  if (p.causal) q = p.num_quads - 1 - q;
  it.quad = q;
  it.nblk[0] = p.causal ? 4 * q + 2 : p.num_mblk;
  it.nblk[1] = p.causal ? 4 * q + 4 : p.num_mblk;
  it.n = it.nblk[1];
  return it;
}

__device__ __forceinline__ int attn2_round_item(const Attn2Params& p, int k, int pair, int num_pairs) {
  const int idx = k * num_pairs + pair;
  const int item = p.sched != nullptr ? __ldg(p.sched + idx) : idx;
  return item < p.num_items ? item : -1;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(A2_THREADS, 1)
attn_fwd_bf16_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                                  const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                                  const __grid_constant__ ExtraMaps extra, const Attn2Params p) {
  constexpr uint32_t IDESC_S = umma_idesc_bf16_f32(256, AT_BN, 0, 0);    // Q (K-major) x K^T (K-major), both CTAs
  constexpr uint32_t IDESC_PV = umma_idesc_bf16_f32(256, A2_D, 0, 1);    // P (TMEM) x V (N-major), both CTAs

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem + A2_Q_OFF;
  uint8_t* smem_kv = smem + A2_KV_OFF;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + A2_BAR_OFF);   // used in CTA 0 (loads of both CTAs)
  uint64_t* q_empty = q_full + 2;                                      // per CTA
  uint64_t* kv_full = q_empty + 2;                                     // used in CTA 0
  uint64_t* kv_empty = kv_full + A2_NSLOT;                             // per CTA
  uint64_t* s_full = kv_empty + A2_NSLOT;                              // per CTA
  uint64_t* p_half = s_full + 2;                                       // used in CTA 0 (softmax warps of both CTAs)
  uint64_t* p_full = p_half + 2;                                       // used in CTA 0
  uint64_t* o_full = p_full + 2;                                       // per CTA
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(o_full + 2);
  uint32_t* abort_smem = tmem_ptr_smem + 1;

  const int warp_idx = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  WaitCtx ctx{abort_smem, p.status};

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);    // CTA 0's producer arrives once, with the byte count of both CTAs
      mbar_init(&q_empty[t], 4);   // this CTA's four softmax warps of tile t
      mbar_init(&s_full[t], 1);    // one commit from CTA 0's MMA thread
      mbar_init(&p_half[t], 8);    // the softmax warps of tile t in both CTAs
      mbar_init(&p_full[t], 8);
      mbar_init(&o_full[t], 1);
    }
    for (int s = 0; s < A2_NSLOT; ++s) {
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
    tmem_alloc_2cta(tmem_ptr_smem, 512);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must exist before either CTA signals the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp_idx >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(A2_REGS_OTHER));
   if (warp_idx == 8) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    int slot = 0;
    uint32_t slot_phase = 0;
    uint32_t q_loads[2] = {0, 0};
    bool ok = true;
    for (int round = 0; ok && round < p.rounds; ++round) {
      const int item = attn2_round_item(p, round, pair, num_pairs);
      if (item < 0) continue;
      const Attn2Item it = attn2_item(p, item);
      const int row_base = it.hz * p.N_CTX;
      for (int step = 0; ok && step < 2 * it.n; ++step) {
        // this CTA's Q tiles are interleaved with the first K/V blocks: Q0 K0 Q1 V0 K1 V1 ...
        if (step < 2) {
          const int t = step;
          ok = mbar_wait(&q_empty[t], (q_loads[t] & 1u) ^ 1u, ctx, 50);
          if (!ok) break;
          if (lane == 0) {
            const uint32_t bar = mapa_shared(smem_u32(&q_full[t]), 0);
            if (rank == 0) mbar_expect_tx(&q_full[t], 2 * A2_TILE_BYTES);
            const int row = row_base + (4 * it.quad + 2 * t + static_cast<int>(rank)) * AT_BM;
#pragma unroll
            for (int bx = 0; bx < 2; ++bx)
              tma_load_2d_2cta(smem_q + t * A2_TILE_BYTES + bx * AT_BOX_BYTES, &tmap_q, bar, bx * 64, row);
          }
          __syncwarp();
          ++q_loads[t];
        }
        const int j = step >> 1;
        const bool is_v = (step & 1) != 0;
        ok = mbar_wait(&kv_empty[slot], slot_phase ^ 1u, ctx, 51);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = mapa_shared(smem_u32(&kv_full[slot]), 0);
          if (rank == 0) mbar_expect_tx(&kv_full[slot], 2 * A2_SLOT_BYTES);
          uint8_t* dst = smem_kv + slot * A2_SLOT_BYTES;
          if (is_v) {
            // this CTA's 64 head-dimension columns of the 128 keys of block j
            tma_load_2d_2cta(dst, &tmap_v, bar, 64 * static_cast<int>(rank), row_base + j * AT_BN);
          } else {
            // this CTA's 64 keys of block j: two boxes of 64 rows x 64 columns
            const int row = row_base + j * AT_BN + 64 * static_cast<int>(rank);
            tma_load_2d_2cta(dst, &tmap_k, bar, 0, row);
            tma_load_2d_2cta(dst + 8192, &tmap_k, bar, 64, row);
          }
        }
        __syncwarp();
        if (++slot == A2_NSLOT) { slot = 0; slot_phase ^= 1u; }
      }
    }
   } else if (warp_idx == 9 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (CTA 0 only)
    int slot = 0;
    uint32_t slot_phase = 0;
    uint32_t q_cnt[2] = {0, 0};
    uint32_t p_cnt[2] = {0, 0};
    bool ok = true;
    const uint32_t q_addr[2] = {smem_u32(smem_q), smem_u32(smem_q + A2_TILE_BYTES)};
    const uint32_t kv_addr0 = smem_u32(smem_kv);
    const uint64_t q_desc[2] = {umma_smem_desc_sw128(q_addr[0], 16, 1024), umma_smem_desc_sw128(q_addr[1], 16, 1024)};
    const uint64_t k_desc0 = umma_smem_desc_sw128(kv_addr0, 16, 1024);            // K half: K-major, 64 rows
    const uint64_t v_desc0 = umma_smem_desc_sw128(kv_addr0, AT_BOX_BYTES, 1024);  // V half: N-major, one 64-column chunk
    // commits go to the same barrier in both CTAs
    auto commit_both = [&](uint64_t* bar) {
      const uint32_t a = smem_u32(bar);
      umma_commit_2cta(mapa_shared(a, 0));
      umma_commit_2cta(mapa_shared(a, 1));
    };
    auto issue_s = [&](int t, int slot_idx) {
      if (lane == 0) {
        const uint64_t kd = k_desc0 + static_cast<uint64_t>((slot_idx * A2_SLOT_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < A2_D / 16; ++k) {
          const uint64_t qoff = static_cast<uint64_t>(((k >> 2) * AT_BOX_BYTES + (k & 3) * 32) >> 4);
          const uint64_t koff = static_cast<uint64_t>(((k >> 2) * 8192 + (k & 3) * 32) >> 4);
          umma_ss_2cta(tmem_base + t * 128, q_desc[t] + qoff, kd + koff, IDESC_S, k > 0 ? 1u : 0u);
        }
        commit_both(&s_full[t]);
      }
      __syncwarp();
    };
    auto issue_pv = [&](int t, int slot_idx, bool accumulate, int k0, int k1) {
      if (lane == 0) {
        const uint64_t vd = v_desc0 + static_cast<uint64_t>((slot_idx * A2_SLOT_BYTES) >> 4);
#pragma unroll
        for (int k = k0; k < k1; ++k)
          umma_ts_2cta(tmem_base + A2_O_COL0 + t * 128, tmem_base + t * 128 + k * 8,
                       vd + static_cast<uint64_t>((k * 2048) >> 4), IDESC_PV, (accumulate || k > 0) ? 1u : 0u);
      }
      __syncwarp();
    };

    for (int round = 0; ok && round < p.rounds; ++round) {
      const int item = attn2_round_item(p, round, pair, num_pairs);
      if (item < 0) continue;
      const Attn2Item it = attn2_item(p, item);
      // ---- block 0 scores
      ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 60);
      if (!ok) break;
      const int k_slot = slot;
      if (++slot == A2_NSLOT) { slot = 0; slot_phase ^= 1u; }
      for (int t = 0; ok && t < 2; ++t) {
        ok = mbar_wait(&q_full[t], q_cnt[t] & 1u, ctx, 61);
        if (!ok) break;
        ++q_cnt[t];
#if B200K_ATTN2_STAGGER
        // The two tiles' softmax groups share the ex2 units, and whatever offset they start an item with persists
        // (each tile's cycle has the same length).  Started together they compete for the whole item; so tile 1's
        // first scores wait until tile 0's softmax is well under way (this wait does not consume the phase: the
        // main loop waits for the same completion again).
        if (t == 1) {
          ok = mbar_wait(B200K_ATTN2_STAGGER == 1 ? &p_half[0] : &p_full[0], p_cnt[0] & 1u, ctx, 67);
          if (!ok) break;
        }
#endif
        tc_fence_after();
        issue_s(t, k_slot);
      }
      if (!ok) break;
      if (lane == 0) commit_both(&kv_empty[k_slot]);
      __syncwarp();
      // ---- main loop
      for (int j = 0; ok && j < it.n; ++j) {
        ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 62);  // V_j
        if (!ok) break;
        const int v_slot = slot;
        if (++slot == A2_NSLOT) { slot = 0; slot_phase ^= 1u; }
        const bool have_next = (j + 1 < it.n);
        bool next_k_ready = false;
        for (int t = 0; ok && t < 2; ++t) {
          if (j < it.nblk[t]) {
            ok = mbar_wait(&p_half[t], p_cnt[t] & 1u, ctx, 66);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, v_slot, j > 0, 0, 4);
            ok = mbar_wait(&p_full[t], p_cnt[t] & 1u, ctx, 63);
            if (!ok) break;
            ++p_cnt[t];
            tc_fence_after();
            issue_pv(t, v_slot, j > 0, 4, 8);
            if (j == it.nblk[t] - 1) {
              if (lane == 0) commit_both(&o_full[t]);
              __syncwarp();
            }
          }
          if (t == 1) {
            if (lane == 0) commit_both(&kv_empty[v_slot]);  // every PV of block j has been issued
            __syncwarp();
          }
          if (j + 1 < it.nblk[t]) {
            if (!next_k_ready) {
              ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 64);  // K_{j+1}
              if (!ok) break;
              next_k_ready = true;
              tc_fence_after();
            }
            issue_s(t, slot);
          }
        }
        if (!ok) break;
        if (have_next) {
          if (!next_k_ready) {
            ok = mbar_wait(&kv_full[slot], slot_phase, ctx, 65);
            if (!ok) break;
          }
          if (lane == 0) commit_both(&kv_empty[slot]);
          __syncwarp();
          if (++slot == A2_NSLOT) { slot = 0; slot_phase ^= 1u; }
        }
      }
    }
   }  // warps 10 and 11 (and warp 9 of CTA 1) have no role
  } else {
    // ------------------------------------------------------------------ softmax groups (warps 0..7, both CTAs)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(A2_REGS_SOFTMAX));
    const int t = warp_idx >> 2;        // MMA tile of this group
    const int q = warp_idx & 3;         // TMEM lane quarter
    const int r = q * 32 + static_cast<int>(lane);  // row within the tile
    const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + t * 128;             // S_t / P_t
    const uint32_t t_o = tmem_base + lane_field + A2_O_COL0 + t * 128;  // O_t
    uint8_t* stage = smem_q + t * A2_TILE_BYTES;                       // O staging reuses the Q tile
    const uint32_t p_half_leader = mapa_shared(smem_u32(&p_half[t]), 0);
    const uint32_t p_full_leader = mapa_shared(smem_u32(&p_full[t]), 0);
    const float scale = p.qk_scale;
    uint32_t blk_cnt = 0, item_cnt = 0;
    bool ok = true;
    for (int round = 0; ok && round < p.rounds; ++round) {
      const int item = attn2_round_item(p, round, pair, num_pairs);
      if (item < 0) continue;
      const Attn2Item it = attn2_item(p, item);
      const int n_me = it.nblk[t];
      const int mblk = 4 * it.quad + 2 * t + static_cast<int>(rank);   // this group's 128-row tile of the head
      float m_used = -INFINITY;
      float l = 0.f;
      for (int j = 0; j < n_me; ++j) {
        ok = mbar_wait(&s_full[t], blk_cnt & 1u, ctx, 70);
        if (!ok) break;
        ++blk_cnt;
        tc_fence_after();
        if (p.causal && j > mblk) {
          // every key of this block lies beyond this tile's rows (the other CTA's rows still need it): P = 0
          uint32_t z[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) z[c] = 0u;
          tmem_st_x32(t_s, z);
          tmem_st_x32(t_s + 32, z);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_remote(p_half_leader);
            mbar_arrive_remote(p_full_leader);
          }
          continue;
        }
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_x32(t_s + 0, s0);
        tmem_ld_x32(t_s + 32, s1);
        tmem_ld_x32(t_s + 64, s2);
        tmem_ld_x32(t_s + 96, s3);
        tmem_wait_ld();
        if (p.causal && j == mblk) {
          // diagonal block: key index > query index is masked (reference adds -1e6 before the max;
          // after exp2 both give exactly 0)
          const uint32_t ninf = 0xFF800000u;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c > r) s0[c] = ninf;
            if (c + 32 > r) s1[c] = ninf;
            if (c + 64 > r) s2[c] = ninf;
            if (c + 96 > r) s3[c] = ninf;
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 32; c += 2) {  // 3-input max: two new scores per instruction
          mx0 = fmax3(mx0, __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
          mx1 = fmax3(mx1, __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
          mx2 = fmax3(mx2, __uint_as_float(s2[c]), __uint_as_float(s2[c + 1]));
          mx3 = fmax3(mx3, __uint_as_float(s3[c]), __uint_as_float(s3[c + 1]));
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
#pragma unroll 1
            for (int c4 = 0; c4 < A2_D / 32; ++c4) {
              uint32_t o[32];
              tmem_ld_x32(t_o + c4 * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tmem_st_x32(t_o + c4 * 32, o);
            }
          }
        }
        const uint64_t scale2 = pack_f32x2(scale, scale);
        const uint64_t negm2 = pack_f32x2(-m_used, -m_used);
        uint64_t sum_a = 0, sum_b = 0;  // bit pattern of (0.f, 0.f)
        exp_block32(s0, scale2, negm2, sum_a, sum_b);
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
        // the first 64 keys of P have had the time of 32 exponentials to land in tensor memory: hand them over, so
        // that half of the PV product runs while the last 32 exponentials are computed
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(p_half_leader);
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
        if (lane == 0) mbar_arrive_remote(p_full_leader);
      }
      if (!ok) break;
      // ---- epilogue: O / l -> bf16 -> swizzled staging (the Q tile's buffer) -> TMA store; M = m + log2(l)
      ok = mbar_wait(&o_full[t], item_cnt & 1u, ctx, 71);
      if (!ok) break;
      ++item_cnt;
      tc_fence_after();
      const float inv_l = 1.0f / l;
#pragma unroll 1
      for (int c4 = 0; c4 < A2_D / 32; ++c4) {
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
      tc_fence_before();
      const int64_t out_row = static_cast<int64_t>(it.hz) * p.N_CTX + mblk * AT_BM;
      p.lse2[out_row + r] = m_used + log2f(l);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int y = static_cast<int>(out_row) + q * 32;
#pragma unroll
        for (int bx = 0; bx < 2; ++bx) tma_store_2d(&tmap_o, stage + bx * AT_BOX_BYTES + q * 32 * 128, bx * 64, y);
        for (int d = 0; d < p.n_extra; ++d) {
#pragma unroll
          for (int bx = 0; bx < 2; ++bx)
            tma_store_2d(&extra.m[d], stage + bx * AT_BOX_BYTES + q * 32 * 128, bx * 64, y);
        }
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(&q_empty[t]);  // this CTA's Q buffer may be refilled
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // -------------------------------------------------------------------- teardown
  drain_after_abort(abort_smem);
  // Neither CTA may exit (or free tensor memory) while its partner can still signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp_idx == 9) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

}  // namespace b200k
