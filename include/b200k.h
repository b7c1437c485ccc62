/*
 * b200k.h — C-ABI of libb200kernels.so: hand-written sm_100a kernels for the
 * example kernels of kernelize-ai/triton-tenstorrent (vector add, sin,
 * tensor-descriptor bf16 matmul, fused-epilogue matmul, fused-attention forward).
 *
 * Conventions
 *   - Every pointer named below as "device" is a CUDA device pointer on the
 *     CURRENT device; the caller owns all buffers.  `stream` is a cudaStream_t
 *     passed as void* (NULL = legacy default stream).  Calls are asynchronous.
 *   - Every function returns B200K_OK (0) or a negative b200k_status code; the
 *     human-readable reason of the last failure on the calling thread is
 *     returned by b200k_last_error().  No C++ exception crosses this boundary.
 *   - The reference launches are synchronous (backend/driver.py:168 schedule.run(),
 *     :361 ttrt.runtime.wait); callers that want that behaviour synchronise the
 *     stream after the call.
 */
#ifndef B200K_H_
#define B200K_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200k_status {
  B200K_OK = 0,
  B200K_ERR_INVALID_ARG = -1,   /* shape / stride / alignment / enum out of range   */
  B200K_ERR_CUDA = -2,          /* a CUDA runtime or driver call failed              */
  B200K_ERR_UNSUPPORTED = -3,   /* valid request this build has no kernel for        */
  B200K_ERR_NO_DEVICE = -4,     /* no CUDA device / not an sm_100 device             */
  B200K_ERR_DEVICE_TIMEOUT = -5 /* a bounded device-side wait gave up (see b200k_device_status) */
} b200k_status;

/* Bias operand of the fused matmul epilogue. */
enum { B200K_BIAS_NONE = 0, B200K_BIAS_ROW_F32 = 1 /* bias[N] fp32 */, B200K_BIAS_FULL_BF16 = 2 /* bias[M,N] bf16 */ };
/* Activation applied to the fp32 accumulator (after a fp32 bias add). */
enum { B200K_ACT_NONE = 0, B200K_ACT_RELU = 1, B200K_ACT_LEAKY_RELU = 2 /* x>=0 ? x : 0.01x */ };

/* Library ABI version (major*100+minor). */
int b200k_version(void);
/* Reason of the last failed call on this thread ("" if none). */
const char* b200k_last_error(void);

/*
 * out[i] = x[i] + y[i], fp32, i in [0,n).
 * Replaces: add_kernel, python/tutorials/01-vector-add.py:29-54 (launch :75).
 * `block` is the reference's BLOCK_SIZE constexpr; it is validated (>0) and used only to
 * report the equivalent reference grid — the result does not depend on it.
 */
int b200k_add_f32(const float* x, const float* y, float* out, int64_t n, int block, void* stream);

/*
 * out[i] = x[i] + y[i] on bf16 tensors: the exact sum rounded once to nearest even.
 * Replaces: add_kernel of python/tutorials/01-vector-add.loop.py:29-66, which that tutorial runs on
 * bf16 tensors (:102-103).  Its row_count loop (each program walks row_count consecutive blocks) is a
 * work partition, not arithmetic: through b200k_launch the kernel "add_kernel" accepts the extra
 * row_count argument and checks that grid * row_count * BLOCK_SIZE covers n.
 */
int b200k_add_bf16(const void* x, const void* y, void* out, int64_t n, int block, void* stream);

/*
 * out[i] = sinf(x[i]), fp32 (CUDA precise sinf, <= 1 ulp).
 * Replaces: sin_kernel, examples/01-sin-kernel.py:17-29 (launch :36).
 */
int b200k_sin_f32(const float* x, float* out, int64_t n, int block, void* stream);

/*
 * out[i] = x[i] for i < n, fp32 words copied bit for bit (NaN payloads included).  x and out must not overlap.
 * Replaces: memcpy_kernel, python/tutorials/gluon/01-intro.py:84-93 (launch :96-99; XBLOCK = block) and
 * copy_scalar_kernel of the same file (:60-63, n = 1).
 */
int b200k_copy_f32(const float* x, float* out, int64_t n, int block, void* stream);

/*
 * out[i] = x[i] * y[i] + z[i] (one fused multiply-add is NOT used: product and sum are
 * rounded separately like the reference's two Triton ops).
 * Replaces: python/tutorials/01-vector-mul-add.py (x*y+z variant of add_kernel).
 */
int b200k_mul_add_f32(const float* x, const float* y, const float* z, float* out, int64_t n, int block, void* stream);

/*
 * C[M,N] = epilogue(A[M,K] . B[K,N]); A, B, C bf16 row-major with leading dimensions
 * lda/ldb/ldc in ELEMENTS (multiples of 8; base pointers 16-byte aligned), fp32 accumulate,
 * one round-to-nearest-even to bf16.
 *   bias_kind = B200K_BIAS_NONE      : C = act(acc)
 *   bias_kind = B200K_BIAS_ROW_F32   : C = bf16(act(acc + bias[n])), bias fp32[N]
 *   bias_kind = B200K_BIAS_FULL_BF16 : bias bf16 [M,N] with leading dimension ldbias;
 *        round_before_bias = 1 : C = bf16(float(bf16(act(acc))) + float(bias[m,n]))
 *                                (python/tutorials/09-matmul-fused.py:139-146: add after the downcast)
 *        round_before_bias = 0 : C = bf16(act(acc + float(bias[m,n])))
 *                                (examples/matmul_fused/matmul_fused_add.cpp:49: add in fp32)
 * Replaces: matmul_kernel_tma, examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py:105-143;
 *           matmul_kernel_fused, python/tutorials/09-matmul-fused.py:105-148;
 *           the contraction + leaky_relu of matmul_kernel, examples/matmul/03-matrix-multiplication.py:241-395.
 * Loads outside [M,K]/[K,N] read zero and stores outside [M,N] are dropped, like the reference's
 * tensor descriptors (npu/lib/Dialect/TritonTenstorrent/Transforms/ConvertTensorDescToLoadStore.cpp:57-105).
 */
int b200k_matmul_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                      int64_t lda, int64_t ldb, int64_t ldc,
                      const void* bias, int bias_kind, int64_t ldbias,
                      int act, int round_before_bias, void* stream);

/*
 * The same contraction and epilogues with fp16 operands (A, B, C and a full [M,N] bias in fp16; fp32
 * accumulate, one round-to-nearest-even to fp16).  The reference's matmul_kernel_fused hard-codes fp16
 * (python/tutorials/09-matmul-fused.py:115) and its pointer-based matmul_kernel stores fp16
 * (examples/matmul/03-matrix-multiplication.py:374,410); its fp16 tensor-descriptor twin is
 * examples/matmul_tensor_descriptor/09-persistent-matmul.py:107-145.
 */
int b200k_matmul_f16(const void* A, const void* B, void* C, int M, int N, int K,
                     int64_t lda, int64_t ldb, int64_t ldc,
                     const void* bias, int bias_kind, int64_t ldbias,
                     int act, int round_before_bias, void* stream);

/*
 * b200k_matmul_bf16 whose epilogue stores every output tile to n_dests destination matrices
 * C_dests[0..n_dests) (1 <= n_dests <= 8; all [M,N] bf16 with the same leading dimension ldc, 16-byte
 * aligned) instead of one: the single c_desc.store of the reference kernel
 * (examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py:143) becomes n_dests TMA stores from
 * the same staging buffer.  The destinations may be buffers of other GPUs mapped into this process
 * (CUDA IPC or peer-mapped allocations): with C_dests[r] = peer r's full C + this GPU's row offset,
 * every GPU holds the complete C once all ranks' launches have finished, i.e. the M-row-sharded
 * matmul and the all-gather of C are one kernel whose NVLink traffic overlaps the main loop.
 * C_dests is a HOST array of device pointers; it is read before the call returns.
 * The caller orders readers of remote destinations after the launch (a stream-ordered collective or
 * a host barrier after synchronising the stream).
 */
int b200k_matmul_bf16_multi(const void* A, const void* B, void* const* C_dests, int n_dests, int M, int N, int K,
                            int64_t lda, int64_t ldb, int64_t ldc,
                            const void* bias, int bias_kind, int64_t ldbias,
                            int act, int round_before_bias, void* stream);

/*
 * C = act(A . B) with A, B and C stored TILE-MAJOR, the memory layout the reference's pointer-based
 * matmul_kernel addresses (examples/matmul/03-matrix-multiplication.py:333-344 A, :354-362 B,
 * :378-386 C): the logical [R,S] matrix is cut into 32 x 32 tiles, tile (tr, ts) occupies the 1024
 * contiguous elements starting at (tr * (S/32) + ts) * 1024, row-major inside the tile
 * (BLOCK_SIZE_M = BLOCK_SIZE_N = BLOCK_SIZE_K = 32 is the reference's only configuration, :217-222).
 * M, N, K must be multiples of 32 and the base pointers 16-byte aligned.  f16 = 1: fp16 operands and
 * output (what the reference kernel stores, :374); f16 = 0: bf16.  act: B200K_ACT_NONE,
 * B200K_ACT_LEAKY_RELU (the reference's ACTIVATION="leaky_relu", :372-373,391-392) or B200K_ACT_RELU,
 * applied to the fp32 accumulator before the single round-to-nearest-even downcast.
 * The tiles go through 4-dimensional TMA tensor maps straight into 64-byte-swizzled operand images in
 * shared memory (and C tiles back out the same way); there is no separate layout-conversion pass.
 */
int b200k_matmul_tile32(const void* A, const void* B, void* C, int M, int N, int K, int act, int f16, void* stream);

/*
 * O = softmax(Q K^T * sm_scale [+ causal mask]) V per (batch, head); q,k,v,o bf16 contiguous
 * [Z,H,N_CTX,D]; lse2[Z,H,N_CTX] fp32 receives m_i + log2(l_i) (base-2 log-sum-exp of the
 * scaled scores), exactly the `M` tensor of the reference.  D must be 16, 32, 64, 128 or 256 (the reference's set,
 * 06-fused-attention.py:233); other head sizes return B200K_ERR_UNSUPPORTED (b200k_attn_supported tells).  N_CTX may
 * be any length >= 1: the reference walks whole BLOCK_M x BLOCK_N blocks (32, 64 or 128 rows, :110-121) and is only
 * meaningful for multiples of them; here keys past N_CTX are masked and rows past it are neither computed into M
 * nor stored, so lengths such as 96, 192 or 320 (multiples of the reference's smaller blocks) and ragged ones work.
 * Replaces: _attn_fwd / _attn_fwd_inner, examples/fused-attn/06-fused-attention.py:33-90,143-215
 *           (host wrapper _attention.forward :224-273).
 */
int b200k_attn_fwd_bf16(const void* q, const void* k, const void* v, void* o, float* lse2,
                        int Z, int H, int N_CTX, int D, int causal, float sm_scale, void* stream);
/*
 * The same attention forward for callers that cannot allocate device memory (no counterpart in the
 * reference).  b200k_attn_fwd_bf16 makes its caller allocate the M buffer even when only O is wanted,
 * and its first call on a device obtains the library's status word with cudaMalloc.  Hosts that run
 * under an allocator they must not bypass, plugins that only ever see buffers handed to them, and warm
 * serving loops that may not allocate can call this entry point instead: M and the status word live in
 * a static device array inside the library (2 MiB + 256 B on every GPU that loads it, held until exit),
 * and the call performs no cudaMalloc, cudaFree or other allocating call.  O is identical to
 * b200k_attn_fwd_bf16's; M is not returned.
 *   - Limit: Z*H*N_CTX <= 524288 query rows (the static array's capacity); larger problems are rejected
 *     with B200K_ERR_INVALID_ARG.  Other argument rules are those of b200k_attn_fwd_bf16.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that
 *     device current; make that first call before any stream capture begins.
 *   - All calls on one device share the array and it keeps the last call's contents: the row statistics are
 *     write-only, the status word starts at zero (module load) and is only ever cleared by
 *     b200k_attn_noalloc_status.  Two calls whose kernels overlap on the GPU (different streams) race on the
 *     row statistics, so serialise calls per device.
 *   - A bounded device-side wait that gives up on this path is recorded in the array, not in the word that
 *     b200k_device_status reads (that function allocates on a device's first use): query it with
 *     b200k_attn_noalloc_status.
 */
int b200k_attn_fwd_bf16_noalloc(const void* q, const void* k, const void* v, void* o,
                                int Z, int H, int N_CTX, int D, int causal, float sm_scale, void* stream);
/*
 * Status of the no-allocation attention path on the current device (no counterpart in the reference): copies
 * the status word kept in the static array to *code on `stream`, synchronises the stream, and returns
 * B200K_OK when it is zero, or B200K_ERR_DEVICE_TIMEOUT after clearing it when a bounded wait of an earlier
 * b200k_attn_fwd_bf16_noalloc call gave up (that call's O is then incomplete).  Allocates nothing.
 */
int b200k_attn_noalloc_status(void* stream, uint32_t* code);
/*
 * b200k_selftest_wait_timeout reporting into the static array of the no-allocation path instead of the
 * library's allocated status word (no counterpart in the reference): a one-warp kernel waits `budget_cycles`
 * on a barrier nothing completes, gives up, records that and returns normally; b200k_attn_noalloc_status then
 * reports B200K_ERR_DEVICE_TIMEOUT once.  Nothing faults or hangs.
 */
int b200k_attn_noalloc_selftest(int64_t budget_cycles, void* stream);
/*
 * b200k_attn_fwd_bf16 whose epilogue stores every O tile to n_dests destinations o_dests[0..n_dests)
 * (1 <= n_dests <= 8, each a contiguous [Z,H,N_CTX,D] bf16 block, 16-byte aligned) instead of one; the
 * row statistics go to lse2 only.  As with b200k_matmul_bf16_multi the further destinations may be buffers
 * of other GPUs mapped into this process, so a (batch, head)-sharded attention leaves the complete O on
 * every GPU without a separate all-gather.  o_dests is a HOST array of device pointers.
 */
int b200k_attn_fwd_bf16_multi(const void* q, const void* k, const void* v, void* const* o_dests, int n_dests,
                              float* lse2, int Z, int H, int N_CTX, int D, int causal, float sm_scale, void* stream);

/* 1 if b200k_attn_fwd_bf16 has a kernel for this (D, N_CTX), else 0. */
int b200k_attn_supported(int D, int N_CTX);

/*
 * Attention backward: dq, dk, dv (bf16, contiguous [Z,H,N_CTX,D]) from q, k, v, the forward's o and lse2 (its `M`
 * output) and the gradient d_o of o.  This is the consumer of what the reference's forward saves for a backward pass,
 * `ctx.save_for_backward(q, k, v, o, M)` (examples/fused-attn/06-fused-attention.py:238,269); the reference itself has
 * no backward kernel, so there is no reference function this replaces: the algorithm is that of the Triton tutorial the
 * reference's forward comes from (delta = rowsum(o * d_o); P recomputed as exp2(qk_scale * q.k - M); dv = P^T d_o;
 * dS = P (d_o.v - delta); dk = sm_scale dS^T q; dq = sm_scale dS k), with P and dS rounded to bf16 where they enter a
 * tensor-core product and everything else in fp32.  delta_scratch: Z*H*N_CTX floats the caller provides (the
 * library allocates nothing).  D must be 64 or 128, N_CTX any length >= 1 (b200k_attn_bwd_supported tells); every
 * buffer 16-byte aligned; dq, dk, dv and delta_scratch must not overlap any input or each other (they are written
 * while other CTAs still read q, k, v, o, d_o).  Three kernel launches on `stream`, deterministic (no atomics).
 */
int b200k_attn_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                        void* dq, void* dk, void* dv, float* delta_scratch, int Z, int H, int N_CTX, int D, int causal,
                        float sm_scale, void* stream);
int b200k_attn_bwd_supported(int D, int N_CTX);

/*
 * Generic launch mirroring the argument list the reference launcher builds
 * (backend/driver.py:98-170 TTLauncher.__call__: constexprs dropped, tensors as pointers,
 * TensorDescriptor flattened to base, shape.., strides.., padding flag, shape.., strides..).
 * kernel_name is one of: "add_kernel", "sin_kernel", "mul_add_kernel", "memcpy_kernel", "copy_scalar_kernel",
 * "matmul_kernel_tma", "matmul_kernel_fused", "matmul_kernel", "_attn_fwd", optionally followed by ":KEY=VALUE,..." with the constexpr values
 * the reference bakes into the compiled kernel (BLOCK_SIZE, XBLOCK, BLOCK_SIZE_M/N, STAGE, and F16=1 for the
 * matmul kernels when the descriptors point at fp16 data).  The grid is validated against the problem size
 * implied by the arguments; it does not change the result.
 */
typedef enum b200k_arg_kind { B200K_ARG_PTR = 0, B200K_ARG_I32 = 1, B200K_ARG_I64 = 2, B200K_ARG_F32 = 3 } b200k_arg_kind;
typedef struct b200k_arg {
  int32_t kind; /* b200k_arg_kind */
  int32_t _pad;
  union {
    void* ptr;
    int32_t i32;
    int64_t i64;
    float f32;
  } v;
} b200k_arg;
int b200k_launch(const char* kernel_name, int grid_x, int grid_y, int grid_z, void* stream,
                 const b200k_arg* args, int nargs);

/*
 * Device properties in the shape of TTUtils.get_device_properties (backend/driver.py:76-82).
 */
typedef struct b200k_props {
  int32_t multiprocessor_count;
  int32_t max_shared_mem;     /* opt-in bytes per block */
  int32_t max_num_regs;       /* 32-bit registers per SM */
  int32_t warp_size;
  int32_t cc_major, cc_minor;
  int64_t total_mem;
  char name[128];
} b200k_props;
int b200k_device_props(int device, b200k_props* out);

/*
 * Sharing a device buffer between the per-GPU processes of one box, for b200k_matmul_bf16_multi's remote
 * destinations.  b200k_ipc_export describes the allocation that contains `ptr` (a CUDA IPC handle of the
 * allocation, the offset of `ptr` inside it, the device); the 88 bytes can be sent to another process by any
 * means.  b200k_ipc_open maps that allocation into the CALLING device's context with peer access enabled and
 * returns the address corresponding to `ptr`; repeated opens of one allocation reuse the mapping, which stays
 * until the process exits (the exporter must keep the allocation alive as long as importers use it).  Fails
 * with B200K_ERR_UNSUPPORTED when the current device cannot access the exporting device directly.
 */
typedef struct b200k_ipc_handle {
  unsigned char handle[64];
  int64_t offset;
  int64_t size;   /* bytes of the allocation */
  int32_t device; /* exporting device ordinal */
  int32_t _pad;
} b200k_ipc_handle;
int b200k_ipc_export(const void* ptr, b200k_ipc_handle* out);
int b200k_ipc_open(const b200k_ipc_handle* h, void** ptr);

/*
 * The static schedule of a causal attention launch, for inspection and tests (pure host arithmetic, no device):
 * Z*H heads, N_CTX rows, head dimension D, `ctas` CTAs.  Items are (head, pair of 128-row Q tiles), numbered
 * head * pairs + level with level 0 the longest row position; table[k * ctas + c] is the item CTA c
 * processes k-th (-1 = none).  *rounds receives the number of rows of the table; fails with
 * B200K_ERR_INVALID_ARG when `capacity` (in ints) is too small.  The reference leaves this to its persistent
 * block loop over equal blocks (cpu/lib/Dialect/TritonCPU/Transforms/MakePersistentKernel.cpp:144-198); causal
 * attention items are not equal, hence a work-queue order instead of equal ranges.
 */
int b200k_attn_causal_schedule(int ZH, int N_CTX, int D, int ctas, int* table, int capacity, int* rounds);

/*
 * Contiguous block range of worker `w` out of `workers` over `num_blocks` blocks:
 * base = nb / W, rem = nb % W, worker w gets [w*base + min(w,rem), +base + (w<rem)).
 * Replaces: the per-core partition of npu/lib/TritonNPUToTenstorrent/D2M/SPMDOpToD2M.cpp:53-113.
 * Pure host arithmetic (no device needed).
 */
int b200k_block_range(int64_t num_blocks, int workers, int w, int64_t* block_start, int64_t* block_end);

/*
 * How b200k_matmul_bf16 runs the output tiles that are left over after the full waves of 256 x 256 tiles (host
 * arithmetic only; it refines, below the block, the partition the reference's runtime makes by dealing whole
 * blocks to cores, npu/lib/TritonNPUToTenstorrent/D2M/SPMDOpToD2M.cpp:77-113).  For an M x N x K problem on
 * `sm_count` SMs out5 receives: mode (0 = whole tiles, 1 = each leftover tile as two column halves on twice as
 * many CTA pairs), leftover tiles, CTA pairs, full waves, work items of the last wave.
 */
int b200k_matmul_tail_plan(int M, int N, int K, int sm_count, int* out5);

/*
 * Reads (synchronously, after synchronising `stream`) the per-device status word that the
 * matmul/attention kernels set when one of their bounded waits gives up.  *code receives 0 when
 * healthy, else (site<<8 | role); the word is cleared.  Returns B200K_ERR_DEVICE_TIMEOUT if non-zero.
 */
int b200k_device_status(void* stream, uint32_t* code);

/*
 * Failure-detection self-test: launches a one-warp kernel whose only wait can never be satisfied and
 * has a budget of `budget_cycles` SM cycles (a few million = about a millisecond).  The wait gives up,
 * the kernel returns normally, and the next b200k_device_status reports B200K_ERR_DEVICE_TIMEOUT with
 * site 99.  Exercises, without faulting or hanging anything, the same bounded-wait code the matmul and
 * attention kernels use.  No counterpart in the reference (its launches have no device-side waits).
 */
int b200k_selftest_wait_timeout(int64_t budget_cycles, void* stream);

/* Number of kernel launches issued by this library in the calling process (all threads). */
int64_t b200k_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200K_H_ */
