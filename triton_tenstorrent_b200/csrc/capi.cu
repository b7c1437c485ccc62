// C-ABI of libb200kernels.so (declared in include/b200k.h) and the host plumbing behind it.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "launch.h"

namespace b200k {

// ---------------------------------------------------------------------------------------------
// Errors
// ---------------------------------------------------------------------------------------------
static thread_local char g_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_error[0] = '\0'; }

static std::atomic<int64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---------------------------------------------------------------------------------------------
// Devices
// ---------------------------------------------------------------------------------------------
static constexpr int kMaxDevices = 64;
static DeviceInfo g_devices[kMaxDevices];
static std::atomic<int> g_device_ready[kMaxDevices];
static std::mutex g_device_mutex;

const DeviceInfo* current_device_info() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_error(B200K_ERR_NO_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    set_error(B200K_ERR_NO_DEVICE, "device index %d out of range", dev);
    return nullptr;
  }
  if (g_device_ready[dev].load(std::memory_order_acquire)) return &g_devices[dev];
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (g_device_ready[dev].load(std::memory_order_acquire)) return &g_devices[dev];
  DeviceInfo d{};
  d.device = dev;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    set_error(B200K_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    return nullptr;
  }
  d.sm_count = prop.multiProcessorCount;
  d.cc_major = prop.major;
  d.cc_minor = prop.minor;
  d.max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
  e = cudaMalloc(reinterpret_cast<void**>(&d.status_word), 8 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(d.status_word, 0, 8 * sizeof(uint32_t));
  // the memset runs on the legacy stream, which non-blocking streams are not ordered with: wait for it (first use only)
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error(B200K_ERR_CUDA, "status word allocation: %s", cudaGetErrorString(e));
    return nullptr;
  }
  g_devices[dev] = d;
  g_device_ready[dev].store(1, std::memory_order_release);
  return &g_devices[dev];
}

// ---------------------------------------------------------------------------------------------
// Tensor maps
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct TmapKey {
  uintptr_t base;
  uint64_t inner, outer, ld;
  uint32_t box_inner, box_outer;
  uint32_t kind;  // 0 = row-major 2-D, 1 = tile-major 4-D
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld && box_inner == o.box_inner &&
           box_outer == o.box_outer && kind == o.kind;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&h](uint64_t v) { h = (h ^ v) * 1099511628211ull; };
    mix(k.base); mix(k.inner); mix(k.outer); mix(k.ld); mix(k.box_inner); mix(k.box_outer); mix(k.kind);
    return static_cast<size_t>(h);
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
static std::mutex g_tmap_mutex;

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  TmapKey key{reinterpret_cast<uintptr_t>(base), inner, outer, ld, box_inner, box_outer, 0};
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) {
      *out = it->second;
      return B200K_OK;
    }
  }
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld * 2) % 16 != 0)
    return set_error(B200K_ERR_INVALID_ARG, "tensor map: base and row pitch must be 16-byte aligned");
  // a box row narrower than the 128-byte swizzle span is padded to it in shared memory by TMA
  if (box_inner == 0 || box_inner * 2 > 128 || (box_inner * 2) % 16 != 0 || box_outer == 0 || box_outer > 256)
    return set_error(B200K_ERR_INVALID_ARG, "tensor map: box %ux%u not supported", box_inner, box_outer);
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, pitch %llu, box %u x %u)",
                     static_cast<int>(r), (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld,
                     box_inner, box_outer);
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (g_tmaps.size() > 4096) g_tmaps.clear();
    g_tmaps.emplace(key, *out);
  }
  return B200K_OK;
}

int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
                      uint32_t box_inner, uint32_t box_rows) {
  TmapKey key{reinterpret_cast<uintptr_t>(base), inner, rows, batch, box_inner, box_rows, 3};
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) {
      *out = it->second;
      return B200K_OK;
    }
  }
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (inner * 2) % 16 != 0)
    return set_error(B200K_ERR_INVALID_ARG, "tensor map: base and row pitch must be 16-byte aligned");
  if (box_inner == 0 || box_inner * 2 > 128 || (box_inner * 2) % 16 != 0 || box_rows == 0 || box_rows > 256)
    return set_error(B200K_ERR_INVALID_ARG, "tensor map: box %ux%u not supported", box_inner, box_rows);
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {inner * 2, rows * inner * 2};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d (dims %llu x %llu x %llu, box %u x %u)",
                     static_cast<int>(r), (unsigned long long)inner, (unsigned long long)rows, (unsigned long long)batch,
                     box_inner, box_rows);
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (g_tmaps.size() > 4096) g_tmaps.clear();
    g_tmaps.emplace(key, *out);
  }
  return B200K_OK;
}

int make_tmap_tile32(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint32_t box_rows,
                     bool row_pairs) {
  const uint32_t box_cols = 32;
  TmapKey key{reinterpret_cast<uintptr_t>(base), cols, rows, 0, box_cols, box_rows, row_pairs ? 2u : 1u};
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) {
      *out = it->second;
      return B200K_OK;
    }
  }
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return set_error(B200K_ERR_INVALID_ARG, "tensor map: base must be 16-byte aligned");
  if (cols == 0 || rows == 0 || (cols & 31) || (rows & 31))
    return set_error(B200K_ERR_INVALID_ARG, "tile-major tensor map: %llu x %llu is not a whole number of 32 x 32 tiles",
                     (unsigned long long)rows, (unsigned long long)cols);
  if (box_rows == 0 || (box_rows & 31) || box_rows > 256)
    return set_error(B200K_ERR_INVALID_ARG, "tile-major tensor map: box %u x %u not supported", box_rows, box_cols);
  const uint64_t tile_bytes = 32 * 32 * 2;
  // (column in tile, tile column, row in tile, tile row); with row_pairs the two rows of a pair form one
  // 128-byte line: (element in line, tile column, line in tile, tile row)
  cuuint64_t dims[4] = {32, cols / 32, 32, rows / 32};
  cuuint64_t strides[3] = {tile_bytes, 32 * 2, (cols / 32) * tile_bytes};  // next tile column, next row in tile, next tile row
  cuuint32_t box[4] = {32, 1, 32, box_rows / 32};
  if (row_pairs) {
    dims[0] = 64; dims[2] = 16;
    strides[1] = 64 * 2;
    box[0] = 64; box[2] = 16;
  }
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, row_pairs ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled (tile-major) failed with CUresult %d (%llu x %llu, box %u x %u)",
                     static_cast<int>(r), (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (g_tmaps.size() > 4096) g_tmaps.clear();
    g_tmaps.emplace(key, *out);
  }
  return B200K_OK;
}

// ---------------------------------------------------------------------------------------------
// Generic launch: parse the reference launcher's flattened argument list
// ---------------------------------------------------------------------------------------------
struct ArgCursor {
  const b200k_arg* args;
  int n;
  int i = 0;
  bool fail = false;
  void* ptr() {
    if (i >= n || args[i].kind != B200K_ARG_PTR) { fail = true; ++i; return nullptr; }
    return args[i++].v.ptr;
  }
  int64_t integer() {
    if (i >= n) { fail = true; ++i; return 0; }
    const b200k_arg& a = args[i++];
    if (a.kind == B200K_ARG_I32) return a.v.i32;
    if (a.kind == B200K_ARG_I64) return a.v.i64;
    fail = true;
    return 0;
  }
  float f32() {
    if (i >= n || args[i].kind != B200K_ARG_F32) { fail = true; ++i; return 0.f; }
    return args[i++].v.f32;
  }
};

// base, shape[2], strides[2], padding flag, shape[2], strides[2]   (backend/driver.py:141-159)
struct Desc2D {
  void* base;
  int64_t shape[2], strides[2];
  int64_t padding;
};
static bool read_desc2d(ArgCursor& c, Desc2D* d) {
  d->base = c.ptr();
  d->shape[0] = c.integer(); d->shape[1] = c.integer();
  d->strides[0] = c.integer(); d->strides[1] = c.integer();
  d->padding = c.integer();
  const int64_t s0 = c.integer(), s1 = c.integer(), t0 = c.integer(), t1 = c.integer();
  if (c.fail) return false;
  return s0 == d->shape[0] && s1 == d->shape[1] && t0 == d->strides[0] && t1 == d->strides[1];
}

// "name:KEY=VAL,KEY=VAL" -> value of KEY or `dflt`.  The suffix carries the constexpr
// specialisation that the reference bakes into the compiled function.
static long spec_value(const char* spec, const char* key, long dflt) {
  if (spec == nullptr) return dflt;
  const size_t klen = strlen(key);
  const char* s = spec;
  while (*s) {
    if (strncmp(s, key, klen) == 0 && s[klen] == '=') return strtol(s + klen + 1, nullptr, 10);
    const char* comma = strchr(s, ',');
    if (comma == nullptr) break;
    s = comma + 1;
  }
  return dflt;
}

static int generic_launch(const char* kernel_name, int gx, int gy, int gz, cudaStream_t stream, const b200k_arg* args,
                          int nargs) {
  if (kernel_name == nullptr) return set_error(B200K_ERR_INVALID_ARG, "launch: null kernel name");
  if (gx <= 0 || gy <= 0 || gz <= 0) return set_error(B200K_ERR_INVALID_ARG, "launch: grid (%d,%d,%d) must be positive", gx, gy, gz);
  if (nargs < 0 || (nargs > 0 && args == nullptr)) return set_error(B200K_ERR_INVALID_ARG, "launch: bad argument list");
  std::string name(kernel_name);
  const char* spec = nullptr;
  const size_t colon = name.find(':');
  std::string spec_str;
  if (colon != std::string::npos) {
    spec_str = name.substr(colon + 1);
    name = name.substr(0, colon);
    spec = spec_str.c_str();
  }
  ArgCursor c{args, nargs};
  if (name == "muladd_kernel") name = "mul_add_kernel";   // the spelling of python/tutorials/01-vector-mul-add.py:29
  if (name == "memcpy_kernel" || name == "copy_scalar_kernel") {
    // python/tutorials/gluon/01-intro.py: memcpy_kernel(in_ptr, out_ptr, xnumel, XBLOCK: constexpr) :84-93 and
    // copy_scalar_kernel(in_ptr, out_ptr) :50-53 (one element, one program)
    if (gy != 1 || gz != 1) return set_error(B200K_ERR_INVALID_ARG, "launch %s: 1-D grid expected", name.c_str());
    void* src = c.ptr();
    void* dst = c.ptr();
    const int64_t n = name == "memcpy_kernel" ? c.integer() : 1;
    if (c.fail || c.i != nargs) return set_error(B200K_ERR_INVALID_ARG, "launch %s: expected two pointers%s, got %d arguments", name.c_str(), name == "memcpy_kernel" ? " and xnumel" : "", nargs);
    if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "launch %s: negative xnumel", name.c_str());
    const long block = spec_value(spec, "XBLOCK", 0);
    if (block > 0 && static_cast<int64_t>(gx) * block < n)
      return set_error(B200K_ERR_INVALID_ARG, "launch %s: grid %d x XBLOCK %ld does not cover xnumel=%lld", name.c_str(), gx, block, (long long)n);
    if (n > 0 && (src == nullptr || dst == nullptr)) return set_error(B200K_ERR_INVALID_ARG, "launch %s: null pointer", name.c_str());
    return copy_f32((const float*)src, (float*)dst, n, stream);
  }
  if (name == "add_kernel" || name == "sin_kernel" || name == "mul_add_kernel") {
    if (gy != 1 || gz != 1) return set_error(B200K_ERR_INVALID_ARG, "launch %s: 1-D grid expected", name.c_str());
    const int nptr = name == "add_kernel" ? 3 : (name == "sin_kernel" ? 2 : 4);
    void* p[4] = {nullptr, nullptr, nullptr, nullptr};
    for (int i = 0; i < nptr; ++i) p[i] = c.ptr();
    const int64_t n = c.integer();
    // add_kernel of python/tutorials/01-vector-add.loop.py:29-35 takes one more scalar: row_count, the
    // number of consecutive blocks each program walks
    int64_t row_count = 1;
    if (name == "add_kernel" && c.i + 1 == nargs) {
      row_count = c.integer();
      if (row_count <= 0) return set_error(B200K_ERR_INVALID_ARG, "launch add_kernel: row_count must be positive (got %lld)", (long long)row_count);
    }
    if (c.fail || c.i != nargs) return set_error(B200K_ERR_INVALID_ARG, "launch %s: expected %d pointers and n_elements, got %d arguments", name.c_str(), nptr, nargs);
    const long block = spec_value(spec, "BLOCK_SIZE", 0);
    if (block > 0 && static_cast<int64_t>(gx) * block * row_count < n)
      return set_error(B200K_ERR_INVALID_ARG, "launch %s: grid %d x BLOCK_SIZE %ld x row_count %lld does not cover n=%lld", name.c_str(), gx, block, (long long)row_count, (long long)n);
    if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "launch %s: negative n", name.c_str());
    const bool bf16 = spec_value(spec, "BF16", 0) != 0;
    if (bf16 && name != "add_kernel") return set_error(B200K_ERR_UNSUPPORTED, "launch %s: only add_kernel has a bf16 form", name.c_str());
    if (name == "add_kernel") {
      if (bf16) return add_bf16((const uint16_t*)p[0], (const uint16_t*)p[1], (uint16_t*)p[2], n, stream);
      return add_f32((const float*)p[0], (const float*)p[1], (float*)p[2], n, stream);
    }
    if (name == "sin_kernel") return sin_f32((const float*)p[0], (float*)p[1], n, stream);
    return mul_add_f32((const float*)p[0], (const float*)p[1], (const float*)p[2], (float*)p[3], n, stream);
  }
  if (name == "matmul_kernel_tma" || name == "matmul_kernel_fused") {
    const bool fused = name == "matmul_kernel_fused";
    Desc2D a, b, cd, bias{};
    bool ok = read_desc2d(c, &a) && read_desc2d(c, &b) && read_desc2d(c, &cd);
    if (ok && fused) ok = read_desc2d(c, &bias);
    const int64_t M = c.integer(), N = c.integer(), K = c.integer();
    if (!ok || c.fail || c.i != nargs)
      return set_error(B200K_ERR_INVALID_ARG, "launch %s: malformed flattened descriptor list (%d arguments)", name.c_str(), nargs);
    if (a.shape[0] != M || a.shape[1] != K || b.shape[0] != K || b.shape[1] != N || cd.shape[0] != M || cd.shape[1] != N)
      return set_error(B200K_ERR_INVALID_ARG, "launch %s: descriptor shapes do not match M,N,K", name.c_str());
    if (a.strides[1] != 1 || b.strides[1] != 1 || cd.strides[1] != 1 || (fused && bias.strides[1] != 1))
      return set_error(B200K_ERR_INVALID_ARG, "launch %s: descriptors must have unit inner stride", name.c_str());
    if (fused && (bias.shape[0] != M || bias.shape[1] != N))
      return set_error(B200K_ERR_INVALID_ARG, "launch %s: bias descriptor must be [M,N]", name.c_str());
    if (gy != 1 || gz != 1) return set_error(B200K_ERR_INVALID_ARG, "launch %s: 1-D grid expected", name.c_str());
    const long bm = spec_value(spec, "BLOCK_SIZE_M", 0), bn = spec_value(spec, "BLOCK_SIZE_N", 0);
    if (bm > 0 && bn > 0) {
      const int64_t need = ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
      if (gx < need) return set_error(B200K_ERR_INVALID_ARG, "launch %s: grid %d smaller than the %lld output tiles", name.c_str(), gx, (long long)need);
    }
    MatmulArgs ma{};
    ma.A = a.base; ma.B = b.base; ma.C = cd.base;
    ma.M = (int)M; ma.N = (int)N; ma.K = (int)K;
    ma.lda = a.strides[0]; ma.ldb = b.strides[0]; ma.ldc = cd.strides[0];
    if (fused) {
      ma.bias = bias.base; ma.bias_kind = B200K_BIAS_FULL_BF16; ma.ldbias = bias.strides[0];
      ma.round_before_bias = 1;  // the Triton kernel adds the bias after the downcast
    }
    ma.dtype = spec_value(spec, "F16", 0) ? 1 : 0;  // descriptors do not carry the element type
    return matmul_bf16(ma, stream, nullptr);
  }
  if (name == "matmul_kernel") {
    // a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn
    // (examples/matmul/03-matrix-multiplication.py:413-420).  TILE32=1: the buffers are tile-major, as the
    // reference kernel addresses them (it ignores the strides); otherwise row-major with the given strides.
    void* pa = c.ptr(); void* pb = c.ptr(); void* pc = c.ptr();
    const int64_t M = c.integer(), N = c.integer(), K = c.integer();
    int64_t st[6];
    for (int i = 0; i < 6; ++i) st[i] = c.integer();
    if (c.fail || c.i != nargs)
      return set_error(B200K_ERR_INVALID_ARG, "launch matmul_kernel: expected 3 pointers, M, N, K and 6 strides, got %d arguments", nargs);
    if (gy != 1 || gz != 1) return set_error(B200K_ERR_INVALID_ARG, "launch matmul_kernel: 1-D grid expected");
    const long bm = spec_value(spec, "BLOCK_SIZE_M", 0), bn = spec_value(spec, "BLOCK_SIZE_N", 0);
    if (bm > 0 && bn > 0) {
      const int64_t need = ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
      if (gx < need) return set_error(B200K_ERR_INVALID_ARG, "launch matmul_kernel: grid %d smaller than the %lld output tiles", gx, (long long)need);
    }
    const long act = spec_value(spec, "ACTIVATION", B200K_ACT_NONE);
    MatmulArgs ma{};
    ma.A = pa; ma.B = pb; ma.C = pc;
    ma.M = (int)M; ma.N = (int)N; ma.K = (int)K;
    ma.act = (int)act;
    ma.dtype = spec_value(spec, "F16", 1) ? 1 : 0;  // the reference kernel stores fp16
    ma.tile32 = spec_value(spec, "TILE32", 0) ? 1 : 0;
    if (!ma.tile32) {
      if (st[1] != 1 || st[3] != 1 || st[5] != 1)
        return set_error(B200K_ERR_INVALID_ARG, "launch matmul_kernel: row-major operands must have unit inner stride");
      ma.lda = st[0]; ma.ldb = st[2]; ma.ldc = st[4];
    }
    return matmul_bf16(ma, stream, nullptr);
  }
  if (name == "_attn_fwd") {
    const float sm_scale = c.f32();
    float* lse = static_cast<float*>(c.ptr());
    const int64_t Z = c.integer(), H = c.integer();
    Desc2D q, k, v, o;
    const bool ok = read_desc2d(c, &q) && read_desc2d(c, &k) && read_desc2d(c, &v) && read_desc2d(c, &o);
    const int64_t n_ctx = c.integer();
    if (!ok || c.fail || c.i != nargs)
      return set_error(B200K_ERR_INVALID_ARG, "launch _attn_fwd: malformed argument list (%d arguments)", nargs);
    const int64_t D = q.shape[1];
    const int64_t y = Z * H * n_ctx;
    const Desc2D* all[4] = {&q, &k, &v, &o};
    for (const Desc2D* d : all)
      if (d->shape[0] != y || d->shape[1] != D || d->strides[0] != D || d->strides[1] != 1)
        return set_error(B200K_ERR_INVALID_ARG, "launch _attn_fwd: descriptors must be contiguous [Z*H*N_CTX, HEAD_DIM]");
    if (gy != Z * H || gz != 1) return set_error(B200K_ERR_INVALID_ARG, "launch _attn_fwd: grid must be (cdiv(N_CTX,BLOCK_M), Z*H, 1)");
    const long block_m = spec_value(spec, "BLOCK_M", 0);
    if (block_m > 0 && gx != (n_ctx + block_m - 1) / block_m)
      return set_error(B200K_ERR_INVALID_ARG, "launch _attn_fwd: grid x = %d, expected cdiv(N_CTX=%lld, BLOCK_M=%ld)", gx, (long long)n_ctx, block_m);
    const long stage = spec_value(spec, "STAGE", 1);
    if (stage != 1 && stage != 3) return set_error(B200K_ERR_INVALID_ARG, "launch _attn_fwd: STAGE must be 1 or 3");
    AttnArgs aa{q.base, k.base, v.base, o.base, lse, (int)Z, (int)H, (int)n_ctx, (int)D, stage == 3 ? 1 : 0, sm_scale};
    return attn_fwd_bf16(aa, stream);
  }
  return set_error(B200K_ERR_UNSUPPORTED, "launch: unknown kernel '%s'", name.c_str());
}

}  // namespace b200k

// ---------------------------------------------------------------------------------------------
// extern "C"
// ---------------------------------------------------------------------------------------------
using namespace b200k;

extern "C" {

int b200k_version(void) { return 100; }

const char* b200k_last_error(void) { return g_error; }

int b200k_add_f32(const float* x, const float* y, float* out, int64_t n, int block, void* stream) {
  clear_error();
  if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "add: n must be >= 0 (got %lld)", (long long)n);
  if (block <= 0) return set_error(B200K_ERR_INVALID_ARG, "add: BLOCK_SIZE must be positive (got %d)", block);
  if (n > 0 && (x == nullptr || y == nullptr || out == nullptr)) return set_error(B200K_ERR_INVALID_ARG, "add: null pointer");
  return add_f32(x, y, out, n, static_cast<cudaStream_t>(stream));
}

int b200k_add_bf16(const void* x, const void* y, void* out, int64_t n, int block, void* stream) {
  clear_error();
  if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "add: n must be >= 0 (got %lld)", (long long)n);
  if (block <= 0) return set_error(B200K_ERR_INVALID_ARG, "add: BLOCK_SIZE must be positive (got %d)", block);
  if (n > 0 && (x == nullptr || y == nullptr || out == nullptr)) return set_error(B200K_ERR_INVALID_ARG, "add: null pointer");
  return add_bf16(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(y), static_cast<uint16_t*>(out), n,
                  static_cast<cudaStream_t>(stream));
}

int b200k_sin_f32(const float* x, float* out, int64_t n, int block, void* stream) {
  clear_error();
  if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "sin: n must be >= 0 (got %lld)", (long long)n);
  if (block <= 0) return set_error(B200K_ERR_INVALID_ARG, "sin: BLOCK_SIZE must be positive (got %d)", block);
  if (n > 0 && (x == nullptr || out == nullptr)) return set_error(B200K_ERR_INVALID_ARG, "sin: null pointer");
  return sin_f32(x, out, n, static_cast<cudaStream_t>(stream));
}

int b200k_copy_f32(const float* x, float* out, int64_t n, int block, void* stream) {
  clear_error();
  if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "copy: n must be >= 0 (got %lld)", (long long)n);
  if (block <= 0) return set_error(B200K_ERR_INVALID_ARG, "copy: XBLOCK must be positive (got %d)", block);
  if (n > 0 && (x == nullptr || out == nullptr)) return set_error(B200K_ERR_INVALID_ARG, "copy: null pointer");
  return copy_f32(x, out, n, static_cast<cudaStream_t>(stream));
}

int b200k_mul_add_f32(const float* x, const float* y, const float* z, float* out, int64_t n, int block, void* stream) {
  clear_error();
  if (n < 0) return set_error(B200K_ERR_INVALID_ARG, "mul_add: n must be >= 0 (got %lld)", (long long)n);
  if (block <= 0) return set_error(B200K_ERR_INVALID_ARG, "mul_add: BLOCK_SIZE must be positive (got %d)", block);
  if (n > 0 && (x == nullptr || y == nullptr || z == nullptr || out == nullptr))
    return set_error(B200K_ERR_INVALID_ARG, "mul_add: null pointer");
  return mul_add_f32(x, y, z, out, n, static_cast<cudaStream_t>(stream));
}

int b200k_matmul_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                      const void* bias, int bias_kind, int64_t ldbias, int act, int round_before_bias, void* stream) {
  clear_error();
  MatmulArgs a{A, B, C, M, N, K, lda, ldb, ldc, bias, bias_kind, ldbias, act, round_before_bias, 0};
  return matmul_bf16(a, static_cast<cudaStream_t>(stream), nullptr);
}

int b200k_matmul_f16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                     const void* bias, int bias_kind, int64_t ldbias, int act, int round_before_bias, void* stream) {
  clear_error();
  MatmulArgs a{A, B, C, M, N, K, lda, ldb, ldc, bias, bias_kind, ldbias, act, round_before_bias, 1};
  return matmul_bf16(a, static_cast<cudaStream_t>(stream), nullptr);
}

int b200k_matmul_bf16_multi(const void* A, const void* B, void* const* C_dests, int n_dests, int M, int N, int K,
                            int64_t lda, int64_t ldb, int64_t ldc, const void* bias, int bias_kind, int64_t ldbias,
                            int act, int round_before_bias, void* stream) {
  clear_error();
  if (C_dests == nullptr || n_dests < 1 || n_dests > 8)
    return set_error(B200K_ERR_INVALID_ARG, "matmul_multi: 1..8 destinations expected (got %d)", n_dests);
  MatmulArgs a{A, B, C_dests[0], M, N, K, lda, ldb, ldc, bias, bias_kind, ldbias, act, round_before_bias, 0, 0,
               C_dests + 1, n_dests - 1};
  return matmul_bf16(a, static_cast<cudaStream_t>(stream), nullptr);
}

int b200k_matmul_tile32(const void* A, const void* B, void* C, int M, int N, int K, int act, int f16, void* stream) {
  clear_error();
  if (f16 != 0 && f16 != 1) return set_error(B200K_ERR_INVALID_ARG, "matmul_tile32: f16 must be 0 or 1 (got %d)", f16);
  MatmulArgs a{A, B, C, M, N, K, 0, 0, 0, nullptr, B200K_BIAS_NONE, 0, act, 0, f16, 1};
  return matmul_bf16(a, static_cast<cudaStream_t>(stream), nullptr);
}

int b200k_attn_fwd_bf16(const void* q, const void* k, const void* v, void* o, float* lse2, int Z, int H, int N_CTX,
                        int D, int causal, float sm_scale, void* stream) {
  clear_error();
  AttnArgs a{q, k, v, o, lse2, Z, H, N_CTX, D, causal, sm_scale};
  return attn_fwd_bf16(a, static_cast<cudaStream_t>(stream));
}

int b200k_attn_fwd_bf16_multi(const void* q, const void* k, const void* v, void* const* o_dests, int n_dests,
                              float* lse2, int Z, int H, int N_CTX, int D, int causal, float sm_scale, void* stream) {
  clear_error();
  if (o_dests == nullptr || n_dests < 1 || n_dests > 8)
    return set_error(B200K_ERR_INVALID_ARG, "attn_multi: 1..8 destinations expected (got %d)", n_dests);
  AttnArgs a{q, k, v, o_dests[0], lse2, Z, H, N_CTX, D, causal, sm_scale, o_dests + 1, n_dests - 1};
  return attn_fwd_bf16(a, static_cast<cudaStream_t>(stream));
}

int b200k_attn_causal_schedule(int ZH, int N_CTX, int D, int ctas, int* table, int capacity, int* rounds) {
  clear_error();
  if (ZH <= 0 || ctas <= 0 || table == nullptr || rounds == nullptr || !attn_supported(D, N_CTX))
    return set_error(B200K_ERR_INVALID_ARG, "attn_causal_schedule: bad arguments");
  const int ntile = D <= 128 ? 2 : 1;
  const int num_mblk = (N_CTX + 127) / 128;
  const int num_pairs = (num_mblk + ntile - 1) / ntile;
  int r = 0;
  const std::vector<int> t = attn_schedule(ZH, num_pairs, num_mblk, ntile, ctas, &r);
  if (static_cast<size_t>(capacity) < t.size())
    return set_error(B200K_ERR_INVALID_ARG, "attn_causal_schedule: table needs %zu ints", t.size());
  memcpy(table, t.data(), t.size() * sizeof(int));
  *rounds = r;
  return B200K_OK;
}

int b200k_attn_supported(int D, int N_CTX) { return attn_supported(D, N_CTX); }

int b200k_attn_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                        void* dq, void* dk, void* dv, float* delta_scratch, int Z, int H, int N_CTX, int D, int causal,
                        float sm_scale, void* stream) {
  clear_error();
  AttnBwdArgs a{q, k, v, o, d_o, lse2, dq, dk, dv, delta_scratch, Z, H, N_CTX, D, causal, sm_scale};
  return attn_bwd_bf16(a, static_cast<cudaStream_t>(stream));
}

int b200k_attn_bwd_supported(int D, int N_CTX) { return attn_bwd_supported(D, N_CTX); }

int b200k_launch(const char* kernel_name, int grid_x, int grid_y, int grid_z, void* stream, const b200k_arg* args,
                 int nargs) {
  clear_error();
  return generic_launch(kernel_name, grid_x, grid_y, grid_z, static_cast<cudaStream_t>(stream), args, nargs);
}

int b200k_device_props(int device, b200k_props* out) {
  clear_error();
  if (out == nullptr) return set_error(B200K_ERR_INVALID_ARG, "device_props: null output");
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return set_error(B200K_ERR_NO_DEVICE, "cudaGetDeviceProperties(%d): %s", device, cudaGetErrorString(e));
  memset(out, 0, sizeof(*out));
  out->multiprocessor_count = prop.multiProcessorCount;
  out->max_shared_mem = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->max_num_regs = prop.regsPerMultiprocessor;
  out->warp_size = prop.warpSize;
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  strncpy(out->name, prop.name, sizeof(out->name) - 1);
  return B200K_OK;
}

// ---- CUDA IPC: one mapping per imported allocation, kept for the life of the process
namespace {
struct IpcMapping {
  unsigned char handle[64];
  int importer_device;
  void* base;
};
std::vector<IpcMapping> g_ipc_mappings;
std::mutex g_ipc_mutex;
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
}  // namespace

int b200k_ipc_export(const void* ptr, b200k_ipc_handle* out) {
  clear_error();
  if (ptr == nullptr || out == nullptr) return set_error(B200K_ERR_INVALID_ARG, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle size");
  cudaPointerAttributes attr;
  B200K_CHECK_CUDA(cudaPointerGetAttributes(&attr, ptr));
  if (attr.type != cudaMemoryTypeDevice) return set_error(B200K_ERR_INVALID_ARG, "ipc_export: not a device pointer");
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPointByVersion("cuMemGetAddressRange", &fn, 12000, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || fn == nullptr)
    return set_error(B200K_ERR_CUDA, "ipc_export: cuMemGetAddressRange is not available from this driver");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = reinterpret_cast<GetAddressRangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) return set_error(B200K_ERR_CUDA, "ipc_export: cuMemGetAddressRange failed with CUresult %d", (int)r);
  memset(out, 0, sizeof(*out));
  cudaIpcMemHandle_t h;
  B200K_CHECK_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(out->handle, &h, 64);
  out->offset = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  out->size = static_cast<int64_t>(size);
  out->device = attr.device;
  return B200K_OK;
}

int b200k_ipc_open(const b200k_ipc_handle* h, void** ptr) {
  clear_error();
  if (h == nullptr || ptr == nullptr) return set_error(B200K_ERR_INVALID_ARG, "ipc_open: null argument");
  if (h->offset < 0 || h->offset >= h->size) return set_error(B200K_ERR_INVALID_ARG, "ipc_open: offset outside the allocation");
  int dev = -1;
  B200K_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev != h->device) {
    int can = 0;
    B200K_CHECK_CUDA(cudaDeviceCanAccessPeer(&can, dev, h->device));
    if (!can) return set_error(B200K_ERR_UNSUPPORTED, "ipc_open: device %d cannot access device %d directly", dev, h->device);
  }
  std::lock_guard<std::mutex> lock(g_ipc_mutex);
  for (const IpcMapping& m : g_ipc_mappings)
    if (m.importer_device == dev && memcmp(m.handle, h->handle, 64) == 0) {
      *ptr = static_cast<char*>(m.base) + h->offset;
      return B200K_OK;
    }
  cudaIpcMemHandle_t ch;
  memcpy(&ch, h->handle, 64);
  void* base = nullptr;
  B200K_CHECK_CUDA(cudaIpcOpenMemHandle(&base, ch, cudaIpcMemLazyEnablePeerAccess));
  IpcMapping m;
  memcpy(m.handle, h->handle, 64);
  m.importer_device = dev;
  m.base = base;
  g_ipc_mappings.push_back(m);
  *ptr = static_cast<char*>(base) + h->offset;
  return B200K_OK;
}

int b200k_block_range(int64_t num_blocks, int workers, int w, int64_t* block_start, int64_t* block_end) {
  clear_error();
  if (num_blocks < 0 || workers <= 0 || w < 0 || w >= workers || block_start == nullptr || block_end == nullptr)
    return set_error(B200K_ERR_INVALID_ARG, "block_range: need num_blocks >= 0, 0 <= w < workers and output pointers");
  const int64_t base = num_blocks / workers, rem = num_blocks % workers;
  const int64_t start = w * base + (w < rem ? w : rem);
  *block_start = start;
  *block_end = start + base + (w < rem ? 1 : 0);
  return B200K_OK;
}

int b200k_matmul_tail_plan(int M, int N, int K, int sm_count, int* out5) {
  clear_error();
  if (M <= 0 || N <= 0 || K <= 0 || sm_count < 2 || out5 == nullptr)
    return set_error(B200K_ERR_INVALID_ARG, "matmul_tail_plan: bad arguments");
  return matmul_tail_plan(M, N, K, sm_count, out5);
}

int b200k_device_status(void* stream, uint32_t* code) {
  clear_error();
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t host = 0;
  B200K_CHECK_CUDA(cudaMemcpyAsync(&host, dev->status_word, sizeof(host), cudaMemcpyDeviceToHost, s));
  B200K_CHECK_CUDA(cudaStreamSynchronize(s));
  if (code != nullptr) *code = host;
  if (host != 0) {
    B200K_CHECK_CUDA(cudaMemsetAsync(dev->status_word, 0, sizeof(uint32_t), s));
    B200K_CHECK_CUDA(cudaStreamSynchronize(s));
    return set_error(B200K_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (site %u)", host >> 8);
  }
  return B200K_OK;
}

int b200k_selftest_wait_timeout(int64_t budget_cycles, void* stream) {
  clear_error();
  return selftest_wait_timeout(budget_cycles, static_cast<cudaStream_t>(stream));
}

int64_t b200k_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
