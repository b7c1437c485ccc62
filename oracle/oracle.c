/*
 * oracle.c — CPU restatement of the reference kernels.  TEST INFRASTRUCTURE ONLY: it is the checker
 * for the CUDA path (tests/, the smoke test) and the timed CPU baseline of the benchmark; nothing in
 * the shipped package imports, links or calls it.
 *
 * Parity pin: the functions below are checked against golden vectors produced by executing the
 * reference's own kernel sources with Triton's CPU interpreter (tests/golden/make_golden.py).
 * The reference's CPU/NPU back ends themselves cannot be built without LLVM/MLIR and tt-mlir.
 *
 * Each function cites the reference lines it restates (paths relative to the reference project).
 * Plain C + OpenMP; work is split over threads with the reference's contiguous block ranges
 * (npu/lib/TritonNPUToTenstorrent/D2M/SPMDOpToD2M.cpp:77-113): base = nb / W, rem = nb % W, worker w
 * gets [w*base + min(w,rem), ... + base + (w < rem)), and every worker runs the persistent loop
 * `for block in [start, end)` that cpu/lib/Dialect/TritonCPU/Transforms/MakePersistentKernel.cpp:144-198
 * wraps around a kernel body.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------------- */
/* 16-bit float helpers                                                                         */
/* ------------------------------------------------------------------------------------------- */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
/* round to nearest even; NaN stays NaN */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float f16_to_f32(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}
static inline uint16_t f32_to_f16(float f) {
  _Float16 x = (_Float16)f; /* round to nearest even */
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}
/* dtype: 0 = bf16, 1 = fp16 */
static inline float h_to_f32(uint16_t h, int dtype) { return dtype ? f16_to_f32(h) : bf16_to_f32(h); }
static inline uint16_t f32_to_h(float f, int dtype) { return dtype ? f32_to_f16(f) : f32_to_bf16(f); }

/* ------------------------------------------------------------------------------------------- */
/* Block-range partition                                                                         */
/* ------------------------------------------------------------------------------------------- */
void oracle_block_range(int64_t num_blocks, int workers, int w, int64_t* start, int64_t* end) {
  const int64_t base = num_blocks / workers, rem = num_blocks % workers;
  const int64_t s = (int64_t)w * base + (w < rem ? w : rem);
  *start = s;
  *end = s + base + (w < rem ? 1 : 0);
}

/* Overrides OMP_NUM_THREADS (launchers such as torchrun set it to 1 for every rank). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------------------------- */
/* Elementwise kernels                                                                          */
/* ------------------------------------------------------------------------------------------- */
/* add_kernel, python/tutorials/01-vector-add.py:29-54: program pid handles offsets
 * pid*BLOCK + [0,BLOCK) under the mask offsets < n (:41-47), out = x + y (:51). */
void oracle_add_f32(const float* x, const float* y, float* out, int64_t n, int block, int workers) {
  const int64_t nb = (n + block - 1) / block;
  if (workers <= 0) workers = oracle_max_threads();
#pragma omp parallel for num_threads(workers) schedule(static, 1)
  for (int w = 0; w < workers; ++w) {
    int64_t bs, be;
    oracle_block_range(nb, workers, w, &bs, &be);
    for (int64_t b = bs; b < be; ++b) {
      const int64_t lo = b * block;
      const int64_t hi = lo + block < n ? lo + block : n;
      for (int64_t i = lo; i < hi; ++i) out[i] = x[i] + y[i];
    }
  }
}

/* add_kernel of python/tutorials/01-vector-add.loop.py:29-66, one program at a time: program pid owns
 * the element range [pid*BLOCK*row_count, min(+BLOCK*row_count, n)) (:46-48) and walks it in
 * lrow_count = cdiv(range, BLOCK) rows of BLOCK elements under the mask offsets < n (:49-66); a
 * program whose range starts at or beyond n does nothing (cdiv of a non-positive length, :49).
 * Elements no program owns are left untouched.  dtype 0 = fp32, 1 = bf16 bit patterns (the tutorial
 * runs bf16, :102-103; a bf16 add is the exact sum rounded to nearest even). */
void oracle_add_loop(const void* xv, const void* yv, void* outv, int64_t n, int64_t row_count, int block, int grid,
                     int dtype) {
#pragma omp parallel for schedule(static)
  for (int pid = 0; pid < grid; ++pid) {
    int64_t block_start = (int64_t)pid * block * row_count;
    int64_t block_end = block_start + (int64_t)block * row_count;
    if (block_end > n) block_end = n;
    const int64_t block_diff = block_end - block_start;
    const int64_t lrow_count = block_diff > 0 ? (block_diff + block - 1) / block : 0;
    for (int64_t idx = 0; idx < lrow_count; ++idx) {
      for (int64_t i = block_start; i < block_start + block; ++i) {
        if (i >= n) continue;
        if (dtype == 0) {
          ((float*)outv)[i] = ((const float*)xv)[i] + ((const float*)yv)[i];
        } else {
          const float sum = bf16_to_f32(((const uint16_t*)xv)[i]) + bf16_to_f32(((const uint16_t*)yv)[i]);
          ((uint16_t*)outv)[i] = f32_to_bf16(sum);
        }
      }
      block_start += block;
    }
  }
}

/* sin_kernel, examples/01-sin-kernel.py:17-29; tl.sin lowers to llvm.sin.f32, i.e. the C library's
 * sinf, on the reference's CPU path (cpu/lib/TritonCPUToLLVM/TritonCPUToLLVM.cpp:130). */
void oracle_sin_f32(const float* x, float* out, int64_t n, int block, int workers) {
  const int64_t nb = (n + block - 1) / block;
  if (workers <= 0) workers = oracle_max_threads();
#pragma omp parallel for num_threads(workers) schedule(static, 1)
  for (int w = 0; w < workers; ++w) {
    int64_t bs, be;
    oracle_block_range(nb, workers, w, &bs, &be);
    for (int64_t b = bs; b < be; ++b) {
      const int64_t lo = b * block;
      const int64_t hi = lo + block < n ? lo + block : n;
      for (int64_t i = lo; i < hi; ++i) out[i] = sinf(x[i]);
    }
  }
}

/* memcpy_kernel, python/tutorials/gluon/01-intro.py:84-93: program pid copies elements [pid*XBLOCK, min(.., xnumel))
 * one at a time (gl.load / gl.store of a scalar); words are moved as integers so that no NaN payload can change. */
void oracle_memcpy_f32(const float* in, float* out, int64_t xnumel, int xblock, int workers) {
  const uint32_t* src = (const uint32_t*)in;
  uint32_t* dst = (uint32_t*)out;
  const int64_t nb = (xnumel + xblock - 1) / xblock;
  if (workers <= 0) workers = oracle_max_threads();
#pragma omp parallel for num_threads(workers) schedule(static, 1)
  for (int w = 0; w < workers; ++w) {
    int64_t bs, be;
    oracle_block_range(nb, workers, w, &bs, &be);
    for (int64_t pid = bs; pid < be; ++pid) {
      const int64_t start = pid * xblock;
      const int64_t end = start + xblock < xnumel ? start + xblock : xnumel;
      for (int64_t i = start; i < end; ++i) dst[i] = src[i];
    }
  }
}

/* Correctly rounded reference for the ulp bound: sin in double, rounded once to fp32. */
void oracle_sin_f64_to_f32(const float* x, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = (float)sin((double)x[i]);
}

/* python/tutorials/01-vector-mul-add.py: out = x * y + z as two Triton ops (two roundings). */
void oracle_mul_add_f32(const float* x, const float* y, const float* z, float* out, int64_t n, int block, int workers) {
  const int64_t nb = (n + block - 1) / block;
  if (workers <= 0) workers = oracle_max_threads();
#pragma omp parallel for num_threads(workers) schedule(static, 1)
  for (int w = 0; w < workers; ++w) {
    int64_t bs, be;
    oracle_block_range(nb, workers, w, &bs, &be);
    for (int64_t b = bs; b < be; ++b) {
      const int64_t lo = b * block;
      const int64_t hi = lo + block < n ? lo + block : n;
      for (int64_t i = lo; i < hi; ++i) {
        volatile float prod = x[i] * y[i]; /* keep the product's own rounding (no FMA contraction) */
        out[i] = prod + z[i];
      }
    }
  }
}

/* ------------------------------------------------------------------------------------------- */
/* Matmul                                                                                       */
/* ------------------------------------------------------------------------------------------- */
/* Epilogue modes of oracle_golden_matmul:
 *   0  C = h(sum)                                      golden_matmul, examples/matmul_tensor_descriptor/matmul_multi_core_tma.cpp:31-51
 *                                                      == matmul_kernel_tma's acc.to(dtype), 09-persistent-matmul.ttnn.py:139
 *   1  C = h(sum + float(bias[i,j]))                   golden_matmul with bias, examples/matmul_fused/matmul_fused_add.cpp:31-52 (:49)
 *   2  C = h(float(h(sum)) + float(bias[i,j]))         matmul_kernel_fused, python/tutorials/09-matmul-fused.py:139-146 (add after downcast)
 *   3  C = h(act(sum + biasrow[j]))                    [N] fp32 bias + activation on the fp32 accumulator
 *                                                      (activation placement as examples/matmul/03-matrix-multiplication.py:372-374)
 * act: 0 none, 1 relu, 2 leaky_relu (x >= 0 ? x : 0.01 x, 03-matrix-multiplication.py:393-395); applied in modes 0 and 3.
 * The contraction is the reference's loop: for each (i,j) a sequential fp32 sum over k of
 * float(a[i,k]) * float(b[k,j]) (products of 16-bit values are exact in fp32).
 */
static inline float act_apply(float x, int act) {
  if (act == 1) return x > 0.f ? x : 0.f;
  if (act == 2) return x >= 0.f ? x : 0.01f * x;
  return x;
}

void oracle_golden_matmul(const uint16_t* a, const uint16_t* b, uint16_t* out, int64_t M, int64_t N, int64_t K,
                          int dtype, int mode, const uint16_t* bias_full, const float* bias_row, int act) {
  /* Widen B once, transposed, so that the k loop streams; summation order over k is unchanged. */
  float* bt = (float*)malloc((size_t)N * K * sizeof(float));
  float* af = (float*)malloc((size_t)M * K * sizeof(float));
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < N; ++j)
    for (int64_t k = 0; k < K; ++k) bt[j * K + k] = h_to_f32(b[k * N + j], dtype);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M * K; ++i) af[i] = h_to_f32(a[i], dtype);
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      float sum = 0.0f;
      const float* ar = af + i * K;
      const float* br = bt + j * K;
      for (int64_t k = 0; k < K; ++k) sum += ar[k] * br[k];
      float r;
      switch (mode) {
        case 1: r = sum + h_to_f32(bias_full[i * N + j], dtype); break;
        case 2: r = h_to_f32(f32_to_h(sum, dtype), dtype) + h_to_f32(bias_full[i * N + j], dtype); break;
        case 3: r = act_apply(sum + bias_row[j], act); break;
        default: r = act_apply(sum, act); break;
      }
      out[i * N + j] = f32_to_h(r, dtype);
    }
  }
  free(bt);
  free(af);
}

/* The reference's golden_matmul exactly as written (strided B access, no staging), used as the timed
 * CPU baseline: examples/matmul_tensor_descriptor/matmul_multi_core_tma.cpp:31-51. */
void oracle_golden_matmul_naive(const uint16_t* a, const uint16_t* b, uint16_t* out, uint32_t M, uint32_t N, uint32_t K) {
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t i = 0; i < M; ++i) {
    for (uint32_t j = 0; j < N; ++j) {
      float sum = 0.0f;
      const size_t ia = (size_t)i * K;
      for (uint32_t k = 0; k < K; ++k) sum += bf16_to_f32(a[ia + k]) * bf16_to_f32(b[(size_t)k * N + j]);
      out[(size_t)i * N + j] = f32_to_bf16(sum);
    }
  }
}

/* matmul_kernel, examples/matmul/03-matrix-multiplication.py:241-395, one program (pid_m, pid_n) at a
 * time with the reference's only configuration BLOCK_SIZE_M = BLOCK_SIZE_N = BLOCK_SIZE_K = 32 (:217-222).
 * The kernel addresses its operands TILE-MAJOR and ignores the strides it is given:
 *   A (:333-344)  offset(m, k) = ((m/32) * num_tiles_k + k/32) * 1024 + (m%32) * 32 + k%32, m = offs_m % M (:310)
 *   B (:354-362)  offset(k, n) = ((k/32) * num_tiles_n + n/32) * 1024 + (k%32) * 32 + n%32, n = offs_n % N (:311)
 *   C (:378-386)  offset(m, n) = ((m/32) * num_tiles_n + n/32) * 1024 + (m%32) * 32 + n%32
 * loads are masked with k < K and read 0 otherwise (:347-349,364-366); the accumulator is fp32 over
 * the k tiles in order (:323-369); optional leaky_relu on the accumulator (:372-373), one downcast
 * (:374), store masked with m < M and n < N (:388-389).  dtype 1 = fp16 (the reference), 0 = bf16. */
void oracle_matmul_kernel_tile32(const uint16_t* a, const uint16_t* b, uint16_t* c, int64_t M, int64_t N, int64_t K,
                                 int dtype, int act) {
  const int64_t T = 32;
  const int64_t ntm = (M + T - 1) / T, ntn = (N + T - 1) / T, ntk = (K + T - 1) / T;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t pid_m = 0; pid_m < ntm; ++pid_m) {
    for (int64_t pid_n = 0; pid_n < ntn; ++pid_n) {
      float acc[32][32];
      for (int i = 0; i < 32; ++i)
        for (int j = 0; j < 32; ++j) acc[i][j] = 0.0f;
      for (int64_t kt = 0; kt < ntk; ++kt) {
        float at[32][32], bt[32][32];
        for (int i = 0; i < 32; ++i) {
          const int64_t m = (pid_m * T + i) % M;
          for (int kk = 0; kk < 32; ++kk) {
            const int64_t k = kt * T + kk;
            const int64_t off = ((m / T) * ntk + k / T) * (T * T) + (m % T) * T + k % T;
            at[i][kk] = (k < K) ? h_to_f32(a[off], dtype) : 0.0f;
          }
        }
        for (int kk = 0; kk < 32; ++kk) {
          const int64_t k = kt * T + kk;
          for (int j = 0; j < 32; ++j) {
            const int64_t n = (pid_n * T + j) % N;
            const int64_t off = ((k / T) * ntn + n / T) * (T * T) + (k % T) * T + n % T;
            bt[kk][j] = (k < K) ? h_to_f32(b[off], dtype) : 0.0f;
          }
        }
        for (int i = 0; i < 32; ++i)
          for (int j = 0; j < 32; ++j) {
            float sum = acc[i][j];
            for (int kk = 0; kk < 32; ++kk) sum += at[i][kk] * bt[kk][j];
            acc[i][j] = sum;
          }
      }
      for (int i = 0; i < 32; ++i) {
        const int64_t om = pid_m * T + i;
        const int64_t m = om % M;
        for (int j = 0; j < 32; ++j) {
          const int64_t on = pid_n * T + j;
          const int64_t n = on % N;
          if (om < M && on < N) {
            const int64_t off = ((m / T) * ntn + n / T) * (T * T) + (m % T) * T + n % T;
            c[off] = f32_to_h(act_apply(acc[i][j], act), dtype);
          }
        }
      }
    }
  }
}

/* ------------------------------------------------------------------------------------------- */
/* Fused attention forward                                                                      */
/* ------------------------------------------------------------------------------------------- */
/* _attn_fwd + _attn_fwd_inner, examples/fused-attn/06-fused-attention.py:33-90,143-215, one program
 * (start_m, off_hz) at a time, op by op:
 *   qk_scale = sm_scale * 1.44269504 (:188-189); m_i = -inf, l_i = 1, acc = 0 (:184-186);
 *   off-band blocks (:62-64): m_ij = max(m_i, max(qk) * qk_scale); qk = qk * qk_scale - m_ij
 *   diagonal blocks (:56-61): qk = qk * qk_scale + (offs_m >= start_n + offs_n ? 0 : -1e6);
 *                             m_ij = max(m_i, max(qk)); qk -= m_ij
 *   p = exp2(qk); alpha = exp2(m_i - m_ij); l_ij = sum(p) (:65-68); acc *= alpha (:78);
 *   acc += bf16(p) . v (:80-83); l_i = l_i * alpha + l_ij; m_i = m_ij (:86-87)
 *   causal: STAGE 3 runs the off-band pass over [0, start_m*BM) then the diagonal pass over
 *   [start_m*BM, (start_m+1)*BM) in steps of BLOCK_N (:41-48,195-209)
 *   epilogue (:211-215): M = m_i + log2(l_i); O = bf16(acc / l_i)
 * q,k,v,o: bf16 bit patterns, contiguous [Z,H,N_CTX,D]; M: fp32 [Z,H,N_CTX].
 */
void oracle_attn_fwd_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* o, float* Mout, int Z, int H,
                          int N_CTX, int D, int causal, float sm_scale, int BLOCK_M, int BLOCK_N) {
  const int num_m = (N_CTX + BLOCK_M - 1) / BLOCK_M;
  float qk_scale = sm_scale;
  qk_scale *= 1.44269504f;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int off_hz = 0; off_hz < Z * H; ++off_hz) {
    for (int start_m = 0; start_m < num_m; ++start_m) {
      const size_t base = (size_t)off_hz * N_CTX * D;
      float* acc = (float*)calloc((size_t)BLOCK_M * D, sizeof(float));
      float* qk = (float*)malloc((size_t)BLOCK_M * BLOCK_N * sizeof(float));
      float* qf = (float*)malloc((size_t)BLOCK_M * D * sizeof(float));
      float* kf = (float*)malloc((size_t)BLOCK_N * D * sizeof(float));
      float* vf = (float*)malloc((size_t)BLOCK_N * D * sizeof(float));
      float* m_i = (float*)malloc(BLOCK_M * sizeof(float));
      float* l_i = (float*)malloc(BLOCK_M * sizeof(float));
      for (int r = 0; r < BLOCK_M; ++r) { m_i[r] = -INFINITY; l_i[r] = 1.0f; }
      const int rows = (start_m + 1) * BLOCK_M <= N_CTX ? BLOCK_M : N_CTX - start_m * BLOCK_M;
      for (int r = 0; r < BLOCK_M; ++r)
        for (int d = 0; d < D; ++d)
          qf[r * D + d] = r < rows ? bf16_to_f32(q[base + (size_t)(start_m * BLOCK_M + r) * D + d]) : 0.f;
      /* stage list: non-causal -> one pass [0, N_CTX) without mask; causal -> off-band then diagonal */
      for (int pass = 0; pass < 2; ++pass) {
        int lo, hi, diag;
        if (!causal) {
          if (pass == 1) break;
          lo = 0; hi = N_CTX; diag = 0;
        } else if (pass == 0) {
          lo = 0; hi = start_m * BLOCK_M; diag = 0;
        } else {
          lo = start_m * BLOCK_M; hi = (start_m + 1) * BLOCK_M; diag = 1;
        }
        for (int start_n = lo; start_n < hi; start_n += BLOCK_N) {
          for (int c = 0; c < BLOCK_N; ++c)
            for (int d = 0; d < D; ++d) {
              const int key = start_n + c;
              const int in = key < N_CTX;
              kf[c * D + d] = in ? bf16_to_f32(k[base + (size_t)key * D + d]) : 0.f;
              vf[c * D + d] = in ? bf16_to_f32(v[base + (size_t)key * D + d]) : 0.f;
            }
          for (int r = 0; r < BLOCK_M; ++r) {
            float* qkr = qk + (size_t)r * BLOCK_N;
            for (int c = 0; c < BLOCK_N; ++c) {
              float s = 0.f;
              for (int d = 0; d < D; ++d) s += qf[r * D + d] * kf[c * D + d];
              qkr[c] = s;
            }
            float m_ij;
            if (diag) {
              float mx = -INFINITY;
              for (int c = 0; c < BLOCK_N; ++c) {
                const int offs_m = start_m * BLOCK_M + r;
                qkr[c] = qkr[c] * qk_scale + (offs_m >= start_n + c ? 0.f : -1.0e6f);
                mx = fmaxf(mx, qkr[c]);
              }
              m_ij = fmaxf(m_i[r], mx);
              for (int c = 0; c < BLOCK_N; ++c) qkr[c] -= m_ij;
            } else {
              float mx = -INFINITY;
              for (int c = 0; c < BLOCK_N; ++c) mx = fmaxf(mx, qkr[c]);
              m_ij = fmaxf(m_i[r], mx * qk_scale);
              for (int c = 0; c < BLOCK_N; ++c) qkr[c] = qkr[c] * qk_scale - m_ij;
            }
            float l_ij = 0.f;
            for (int c = 0; c < BLOCK_N; ++c) {
              qkr[c] = exp2f(qkr[c]);
              l_ij += qkr[c];
            }
            const float alpha = exp2f(m_i[r] - m_ij);
            float* ar = acc + (size_t)r * D;
            for (int d = 0; d < D; ++d) ar[d] *= alpha;
            for (int c = 0; c < BLOCK_N; ++c) {
              const float pb = bf16_to_f32(f32_to_bf16(qkr[c])); /* p.to(dtype) */
              if (pb != 0.f)
                for (int d = 0; d < D; ++d) ar[d] += pb * vf[c * D + d];
            }
            l_i[r] = l_i[r] * alpha + l_ij;
            m_i[r] = m_ij;
          }
        }
      }
      for (int r = 0; r < rows; ++r) {
        const size_t row = (size_t)off_hz * N_CTX + (size_t)start_m * BLOCK_M + r;
        Mout[row] = m_i[r] + log2f(l_i[r]);
        for (int d = 0; d < D; ++d) o[row * D + d] = f32_to_bf16(acc[(size_t)r * D + d] / l_i[r]);
      }
      free(acc); free(qk); free(qf); free(kf); free(vf); free(m_i); free(l_i);
    }
  }
}

/* ------------------------------------------------------------------------------------------- */
/* Fused attention backward.  PARITY UNPINNED: the reference has no backward kernel (its forward */
/* only saves q, k, v, o, M: examples/fused-attn/06-fused-attention.py:238,269), so there is no   */
/* reference output or golden vector to pin this against.  It restates the algorithm of the      */
/* Triton tutorial the reference's forward comes from, in the forward's conventions:             */
/*   delta_i = sum_d o_id do_id;  p_ij = exp2(qk_scale * q_i.k_j - M_i)  (0 above the diagonal)   */
/*   dv_j = sum_i bf16(p_ij) do_i;  ds_ij = p_ij (do_i.v_j - delta_i)                             */
/*   dk_j = sm_scale sum_i bf16(ds_ij) q_i;  dq_i = sm_scale sum_j bf16(ds_ij) k_j                */
/* all sums in fp32, one round-to-nearest-even downcast of each gradient at the end.             */
/* The tests check it against fp32 automatic differentiation of the attention definition.        */
/* ------------------------------------------------------------------------------------------- */
void oracle_attn_bwd_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* o, const uint16_t* d_o,
                          const float* M, uint16_t* dq, uint16_t* dk, uint16_t* dv, int Z, int H, int N_CTX, int D,
                          int causal, float sm_scale) {
  float qk_scale = sm_scale;
  qk_scale *= 1.44269504f;
  const size_t rows = (size_t)Z * H * N_CTX;
  float* delta = (float*)malloc(rows * sizeof(float));
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < (long long)rows; ++r) {
    float s = 0.f;
    for (int d = 0; d < D; ++d) s += bf16_to_f32(o[r * D + d]) * bf16_to_f32(d_o[r * D + d]);
    delta[r] = s;
  }
  /* pass over the keys: dk_j, dv_j */
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
  for (int hz = 0; hz < Z * H; ++hz) {
    for (int j = 0; j < N_CTX; ++j) {
      const size_t base = (size_t)hz * N_CTX;
      float accv[256], acck[256];
      for (int d = 0; d < D; ++d) { accv[d] = 0.f; acck[d] = 0.f; }
      for (int i = causal ? j : 0; i < N_CTX; ++i) {
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < D; ++d) {
          s += bf16_to_f32(q[(base + i) * D + d]) * bf16_to_f32(k[(base + j) * D + d]);
          dp += bf16_to_f32(d_o[(base + i) * D + d]) * bf16_to_f32(v[(base + j) * D + d]);
        }
        const float p = exp2f(s * qk_scale - M[base + i]);
        const float ds = p * (dp - delta[base + i]);
        const float pb = bf16_to_f32(f32_to_bf16(p)), dsb = bf16_to_f32(f32_to_bf16(ds));
        for (int d = 0; d < D; ++d) {
          accv[d] += pb * bf16_to_f32(d_o[(base + i) * D + d]);
          acck[d] += dsb * bf16_to_f32(q[(base + i) * D + d]);
        }
      }
      for (int d = 0; d < D; ++d) {
        dv[(base + j) * D + d] = f32_to_bf16(accv[d]);
        dk[(base + j) * D + d] = f32_to_bf16(acck[d] * sm_scale);
      }
    }
  }
  /* pass over the queries: dq_i */
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
  for (int hz = 0; hz < Z * H; ++hz) {
    for (int i = 0; i < N_CTX; ++i) {
      const size_t base = (size_t)hz * N_CTX;
      float accq[256];
      for (int d = 0; d < D; ++d) accq[d] = 0.f;
      const int j_end = causal ? i + 1 : N_CTX;
      for (int j = 0; j < j_end; ++j) {
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < D; ++d) {
          s += bf16_to_f32(q[(base + i) * D + d]) * bf16_to_f32(k[(base + j) * D + d]);
          dp += bf16_to_f32(d_o[(base + i) * D + d]) * bf16_to_f32(v[(base + j) * D + d]);
        }
        const float p = exp2f(s * qk_scale - M[base + i]);
        const float dsb = bf16_to_f32(f32_to_bf16(p * (dp - delta[base + i])));
        for (int d = 0; d < D; ++d) accq[d] += dsb * bf16_to_f32(k[(base + j) * D + d]);
      }
      for (int d = 0; d < D; ++d) dq[(base + i) * D + d] = f32_to_bf16(accq[d] * sm_scale);
    }
  }
  free(delta);
}
