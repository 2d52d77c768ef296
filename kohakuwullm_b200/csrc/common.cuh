// Shared device/host helpers for the sm_100a kernels of this library.
//
// Everything here is inline PTX for Blackwell (tcgen05 / TMEM / TMA / mbarrier) plus the
// conventions every kernel follows:
//   * every wait on an mbarrier or a flag is BOUNDED: after a time limit the waiter records
//     an error code in a status word that the host reads, raises a CTA-wide abort flag, and
//     every role of the kernel leaves its loop, waits for copies in flight, frees its TMEM
//     and returns. A kernel never spins for ever and never traps.
//   * TMA loads are plain per-CTA `cp.async.bulk.tensor` (no cluster multicast anywhere).
//   * the x coordinate of every TMA copy is a multiple of 16 bytes by construction.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda.h>
#include <stdint.h>

namespace kwu {

// ------------------------------------------------------------------ status word
// Error codes written by kernels into the int32 status word (0 = ok).
enum : int {
  KWU_OK = 0,
  KWU_ERR_TIMEOUT_FULL = 1,    // consumer waited for a TMA stage that never arrived
  KWU_ERR_TIMEOUT_EMPTY = 2,   // producer waited for a stage that was never released
  KWU_ERR_TIMEOUT_ACC_FULL = 3,
  KWU_ERR_TIMEOUT_ACC_EMPTY = 4,
  KWU_ERR_TIMEOUT_FLAG = 5,    // a peer / test flag never arrived
  KWU_ERR_TIMEOUT_MISC = 6,
  KWU_ERR_BAD_ARG = 7,
  KWU_ERR_EP_OVERFLOW = 8,     // an expert-parallel receive buffer was too small for the routed rows
};

// Wait limit in SM clock cycles (about 2 s at 2 GHz; tests shorten it). The clock is only read once
// per 1024 failed polls, so a wait that succeeds quickly never pays for it.
#ifndef KWU_WAIT_LIMIT_CYCLES
#define KWU_WAIT_LIMIT_CYCLES 4000000000ll
#endif

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Work item of a persistent CTA in round r of a cost-sorted (heaviest first) list: rounds alternate
// direction, so the CTA that got the heaviest item of one round gets the lightest of the next (static
// boustrophedon assignment; per-CTA totals come within a few percent of a greedy dynamic queue).
__device__ __forceinline__ int snake_item(int r) {
  const int G = static_cast<int>(gridDim.x), b = static_cast<int>(blockIdx.x);
  return r * G + ((r & 1) ? G - 1 - b : b);
}

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with `launch_k` (host side, below) may START while the kernel before it in the stream is
// still running: its CTAs become resident as SMs free up and run their set-up (barrier init, TMEM allocation,
// descriptor prefetch). `pdl_wait` blocks until the preceding kernels have completed and their memory is
// visible; NOTHING that another kernel produced may be read before it. `pdl_launch_dependents` lets the NEXT
// kernel in the stream begin its own early start; it is called right after the wait, so at most one successor
// is resident and waiting at any time. Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() {
  pdl_wait();
  pdl_launch_dependents();
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One probe of the barrier. A thread whose phase is not complete yet is suspended by the hardware until the
// phase completes or `KWU_WAIT_SUSPEND_NS` have passed, whichever is first, so a waiting warp costs no issue
// slots and no ALU cycles while it waits (a busy loop of probes took a large share of both from the warps
// that had work).
#ifndef KWU_WAIT_SUSPEND_NS
#define KWU_WAIT_SUSPEND_NS 20000
#endif
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(static_cast<uint32_t>(KWU_WAIT_SUSPEND_NS))
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` lives in shared memory and is shared by every role of the CTA.
// Returns false when the wait was abandoned (own time-out or somebody else's abort). Every failed probe
// has already slept for up to the suspend time, so the abort flag and the clock are read after each one.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > KWU_WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

// ------------------------------------------------------------------ TMA
// Untiled bulk copy global -> shared (this CTA), completion counted on an mbarrier. Both addresses 16-byte
// aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared (this CTA only), completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x),
        "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x),
        "r"(y), "r"(z)
      : "memory");
}
// 2-D tiled store shared -> global.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x,
                                             int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05 ops issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], 16-bit inputs (kind::f16 covers f16 and bf16).
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Block-scaled e4m3 x e4m3 with UE8M0 scales held in TMEM (one scale per 32 along K).
__device__ __forceinline__ void mma_mxf8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem)
      : "memory");
}
// Copy 32 rows x 128 bit of scale factors from shared memory into TMEM, replicated into the
// four 32-lane quarters.
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}

// tcgen05.ld 32 lanes x 32 bit, N consecutive columns per thread.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// fp32 vector reduction into global memory (no return value)
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (sm_100 flavour: version field = 1).
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version (1)
//   bits 61-63 swizzle: 0 none, 2 128B, 4 64B, 6 32B
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(swizzle & 7) << 61;
  return d;
}
constexpr uint32_t SWZ_NONE = 0, SWZ_128B = 2, SWZ_64B = 4, SWZ_32B = 6;

// Instruction descriptor for kind::f16 (dense, fp32 accumulate).
//   fmt: 0 = f16, 1 = bf16; major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, int fmt, int a_major,
                                                      int b_major) {
  return (1u << 4)                               // D = f32
         | (static_cast<uint32_t>(fmt) << 7)     // A format
         | (static_cast<uint32_t>(fmt) << 10)    // B format
         | (static_cast<uint32_t>(a_major) << 15) | (static_cast<uint32_t>(b_major) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
// Instruction descriptor for kind::mxf8f6f4.block_scale, e4m3 x e4m3, UE8M0 scales, K = 32.
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int M, int N, int a_sf_id, int b_sf_id) {
  return (static_cast<uint32_t>(b_sf_id) << 4) | (0u << 7) | (0u << 10) |
         (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(M >> 4) << 24) | (static_cast<uint32_t>(a_sf_id) << 29);
}

// ------------------------------------------------------------------ small math helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// 2^x on the special-function unit, no range fix-ups (inputs here are <= 0 or already bounded)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32 pairs (one instruction works on two floats held in a 64-bit register pair): the softmax loops
// of the attention kernels are bound by the number of issued instructions, not by the arithmetic.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 16 bytes from shared memory as two 64-bit words (fp32 pairs), addressed in the shared window: a generic
// pointer derived from an aligned-up dynamic-shared-memory base makes the compiler emit generic loads
__device__ __forceinline__ ulonglong2 lds_u64x2(uint32_t saddr) {
  ulonglong2 v;
  asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(saddr));
  return v;
}
// 1/x on the special-function unit (about 1 ulp; the IEEE division of the plain `/` costs ~10 instructions)
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));  // low half = a, high half = b
  return r;
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

}  // namespace kwu

// ------------------------------------------------------------------ host side
#define KWU_API extern "C" __attribute__((visibility("default")))

namespace kwu {
// Encode a 2-D row-major tensor map: `rows` x `cols` elements of `elem_bytes`, row pitch
// `ld_elems` elements, box `box_rows` x `box_cols`, with the given swizzle
// (CU_TENSOR_MAP_SWIZZLE_*). Returns 0 on success. Implemented in tensormap.cu through the
// driver entry point fetched at run time (no link-time dependency on libcuda).
int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_kind, uint64_t rows, uint64_t cols,
                   uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, int swizzle);
enum : int { ELEM_BF16 = 0, ELEM_F16 = 1, ELEM_U8 = 2, ELEM_F32 = 3 };
const char* last_error();
// Function attributes (`cudaFuncSetAttribute`) take effect per DEVICE, so "already set" is remembered per
// device: one bit per device ordinal, read and written atomically. Two threads that race both apply the
// attribute, which is idempotent.
struct PerDeviceOnce {
  unsigned long long done = 0;
  bool pending() const {
    int dev = 0;
    cudaGetDevice(&dev);
    return !(__atomic_load_n(&done, __ATOMIC_ACQUIRE) & (1ull << (dev & 63)));
  }
  void mark() {
    int dev = 0;
    cudaGetDevice(&dev);
    __atomic_fetch_or(&done, 1ull << (dev & 63), __ATOMIC_RELEASE);
  }
};
bool pdl_enabled();   // programmatic dependent launch for kernels started through launch_k (KWU_PDL=1 turns it on)
void set_device_status_word(int* p);
int* device_status_word();   // the current device's registered status word, or null
void count_launch(int n = 1);
long long launch_total();  // bumps the library-wide kernel launch counter
void set_last_error(const char* fmt, ...);
}  // namespace kwu

namespace kwu {
// Launch `kern` with the programmatic-stream-serialization attribute (see pdl_wait above). Only for kernels
// that call pdl_sync() / pdl_wait() before their first read of another kernel's output.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
}  // namespace kwu
