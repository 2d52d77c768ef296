// Host-side TMA descriptor encoding and the library-wide error string.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <mutex>

namespace kwu {

static thread_local char g_err[512] = {0};
static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_total() { return g_launches.load(); }
const char* last_error() { return g_err; }
void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    // off unless asked for: on the dense training step the early starts measured 0.7 % SLOWER (the step runs
    // at the board's power limit; the extra resident CTAs cost more clock than the hidden launch gaps save)
    const char* e = getenv("KWU_PDL");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on == 1;
}

// Status word of each device (set by the host binding), for kernels whose entry point carries no status
// argument of its own.
static int* g_status_word[64] = {nullptr};
void set_device_status_word(int* p) {
  int dev = 0;
  cudaGetDevice(&dev);
  __atomic_store_n(&g_status_word[dev & 63], p, __ATOMIC_RELEASE);
}
int* device_status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  return __atomic_load_n(&g_status_word[dev & 63], __ATOMIC_ACQUIRE);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_kind, uint64_t rows, uint64_t cols,
                   uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, int swizzle) {
  // The driver call needs a context bound to THIS thread (autograd runs backward on its own threads,
  // which may not have touched the runtime yet): binding the current device's primary context is cheap.
  static thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaSetDevice(dev);
    cudaFree(nullptr);
    bound = true;
  }
  EncodeTiledFn fn = get_encode();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point unavailable");
    return 1;
  }
  CUtensorMapDataType dt;
  uint64_t eb;
  switch (elem_kind) {
    case ELEM_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; eb = 2; break;
    case ELEM_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; eb = 2; break;
    case ELEM_U8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; eb = 1; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; eb = 4; break;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld_elems * eb) & 15)) {
    set_last_error("TMA operand must be 16-byte aligned with a 16-byte multiple pitch (base %p pitch %llu B)",
                   base, (unsigned long long)(ld_elems * eb));
    return 2;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld_elems * eb};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(swizzle),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with %d (rows %llu cols %llu ld %llu box %ux%u)",
                   (int)r, (unsigned long long)rows, (unsigned long long)cols,
                   (unsigned long long)ld_elems, box_rows, box_cols);
    return 3;
  }
  return 0;
}

}  // namespace kwu

KWU_API const char* kwu_last_error() { return kwu::last_error(); }

// Registers the int32 status word of the CURRENT device (0 = ok; kernels write an error code into it when a
// bounded wait gives up). Entry points that take a status pointer use that one; the others use this.
KWU_API void kwu_set_status_word(int* word) { kwu::set_device_status_word(word); }

// Number of kernels this library has launched in this process (for launch accounting in benchmarks).
KWU_API long long kwu_launch_count() { return kwu::launch_total(); }
