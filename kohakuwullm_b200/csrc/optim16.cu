// 16-bit optimizer kernels: AdamW with state in the parameter dtype, and stochastic rounding.
//
//   adamw16        p, m and sqrt(v) stored in bf16; all math in fp32 registers; decoupled weight decay;
//                  optional stochastic rounding of p and m on the way back.
//   sr_cast        fp32 -> bf16 by stochastic rounding: 16 random bits are added to the 16 bits that the
//                  conversion discards, then the value is truncated. E[SR(x)] = x.
//   sr_update      p = SR(p * (1 - decay) + alpha * u)   (fused write-back of an fp32 update into bf16 params)
//   sr_grouped     the same for a whole model in ONE launch: a table of (param ptr, update ptr, numel,
//                  running element offset) chunks; element i of tensor t draws random number
//                  offset[t] + i, so the result is bit-identical to the per-tensor loop.
// Randomness is Philox4x32-10 keyed by (seed, counter = element index / 8: eight 16-bit draws per block); `draws` (optional) injects the
// 16-bit draws directly, which is how the PyTorch reference checks the kernels bit for bit.
// Reference: src/kohakuwullm/kernels/optim/adamw16.py:16-168, stochastic_round.py:44-270,
// stochastic_round_grouped.py:22-176.
#include "common.cuh"

namespace kwu {

__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
  uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c[0], c[1], c[2], c[3]);
}

// 16 random bits for flat element index i
__device__ __forceinline__ uint32_t draw16(unsigned long long seed, unsigned long long i, const uint16_t* draws) {
  if (draws) return draws[i];
  const unsigned long long ctr = i >> 3;  // 8 draws of 16 bits per Philox block
  const uint4 r = philox4x32_10(static_cast<uint32_t>(ctr), static_cast<uint32_t>(ctr >> 32),
                                static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  const uint32_t words[4] = {r.x, r.y, r.z, r.w};
  const uint32_t w = words[(i >> 1) & 3];
  return (i & 1) ? (w >> 16) : (w & 0xffffu);
}

__device__ __forceinline__ __nv_bfloat16 sr_round(float x, uint32_t r16) {
  uint32_t bits = __float_as_uint(x);
  if ((bits & 0x7f800000u) != 0x7f800000u) bits += r16;  // leave inf / nan alone
  return __ushort_as_bfloat16(static_cast<unsigned short>(bits >> 16));
}

__global__ void __launch_bounds__(256)
sr_cast_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n, unsigned long long seed,
               unsigned long long offset, const uint16_t* __restrict__ draws) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = sr_round(x[i], draw16(seed, offset + i, draws ? draws : nullptr));
}

__global__ void __launch_bounds__(256)
sr_update_kernel(__nv_bfloat16* __restrict__ p, const float* __restrict__ u, long long n, float decay, float alpha,
                 unsigned long long seed, unsigned long long offset, const uint16_t* __restrict__ draws) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(p[i]) * (1.f - decay) + alpha * u[i];
    p[i] = sr_round(v, draw16(seed, offset + i, draws));
  }
}

struct SrChunk {
  __nv_bfloat16* p;
  const float* u;
  long long numel;
  unsigned long long rng_offset;  // cumulative element count of the tensors before this one
  float decay, alpha;
};

__global__ void __launch_bounds__(256)
sr_grouped_kernel(const SrChunk* __restrict__ chunks, unsigned long long seed) {
  const SrChunk c = chunks[blockIdx.y];
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < c.numel;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(c.p[i]) * (1.f - c.decay) + c.alpha * c.u[i];
    c.p[i] = sr_round(v, draw16(seed, c.rng_offset + i, nullptr));
  }
}

// g: gradient in the parameter dtype (bf16) or fp32 (g32). v is stored as sqrt(v).
__global__ void __launch_bounds__(256)
adamw16_kernel(__nv_bfloat16* __restrict__ p, __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ sv,
               const __nv_bfloat16* __restrict__ g16, const float* __restrict__ g32, long long n, float lr,
               float beta1, float beta2, float eps, float wd, float bc1_inv, float bc2_inv_sqrt, float grad_scale,
               int stochastic, unsigned long long seed, unsigned long long offset) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = (g32 ? g32[i] : __bfloat162float(g16[i])) * grad_scale;
    float pv = __bfloat162float(p[i]);
    float mv = __bfloat162float(m[i]);
    const float s = __bfloat162float(sv[i]);
    mv = beta1 * mv + (1.f - beta1) * g;
    const float vv = beta2 * s * s + (1.f - beta2) * g * g;
    const float root = sqrtf(vv);
    pv = pv * (1.f - lr * wd) - lr * (mv * bc1_inv) / (root * bc2_inv_sqrt + eps);
    if (stochastic) {
      p[i] = sr_round(pv, draw16(seed, offset + 2 * i, nullptr));
      m[i] = sr_round(mv, draw16(seed, offset + 2 * i + 1, nullptr));
    } else {
      p[i] = __float2bfloat16(pv);
      m[i] = __float2bfloat16(mv);
    }
    sv[i] = __float2bfloat16(root);
  }
}

static inline int grid1d(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return static_cast<int>(g < 1 ? 1 : g);
}
static inline int chk(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("%s launch: %s", what, cudaGetErrorString(e)); return 11; }
  return 0;
}

}  // namespace kwu

using namespace kwu;

KWU_API int kwu_sr_cast(const float* x, void* out, long long n, unsigned long long seed, unsigned long long offset,
                        const void* draws, void* stream) {
  if (n <= 0) return 0;
  sr_cast_kernel<<<grid1d(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, (__nv_bfloat16*)out, n, seed, offset, (const uint16_t*)draws); kwu::count_launch();
  return chk("sr_cast");
}

KWU_API int kwu_sr_update(void* p, const float* u, long long n, float decay, float alpha, unsigned long long seed,
                          unsigned long long offset, const void* draws, void* stream) {
  if (n <= 0) return 0;
  sr_update_kernel<<<grid1d(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)p, u, n, decay, alpha, seed, offset, (const uint16_t*)draws); kwu::count_launch();
  return chk("sr_update");
}

// chunks: device array of `n_chunks` records {p, u, numel, rng_offset, decay, alpha} (40 bytes each, see SrChunk)
KWU_API int kwu_sr_grouped(const void* chunks, int n_chunks, unsigned long long seed, void* stream) {
  if (n_chunks <= 0) return 0;
  sr_grouped_kernel<<<dim3(64, n_chunks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((const SrChunk*)chunks, seed); kwu::count_launch();
  return chk("sr_grouped");
}
KWU_API int kwu_sr_chunk_bytes() { return static_cast<int>(sizeof(SrChunk)); }

KWU_API int kwu_adamw16(void* p, void* m, void* sv, const void* g16, const float* g32, long long n, float lr, float beta1,
                        float beta2, float eps, float wd, int step, float grad_scale, int stochastic,
                        unsigned long long seed, unsigned long long offset, void* stream) {
  if (n <= 0) return 0;
  const float bc1_inv = 1.f / (1.f - powf(beta1, (float)step));
  const float bc2_inv_sqrt = 1.f / sqrtf(1.f - powf(beta2, (float)step));
  adamw16_kernel<<<grid1d(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (__nv_bfloat16*)p, (__nv_bfloat16*)m, (__nv_bfloat16*)sv, (const __nv_bfloat16*)g16, g32, n, lr, beta1, beta2, eps, wd,
      bc1_inv, bc2_inv_sqrt, grad_scale, stochastic, seed, offset); kwu::count_launch();
  return chk("adamw16");
}
