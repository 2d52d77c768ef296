// Optimizer kernels over FLAT buffers: the whole model is one launch.
//
//   adamw_flat     fp32 master / exp_avg / exp_avg_sq + fp32 gradient -> updated master and the
//                  low-precision (bf16) parameter copy; the gradient buffer is zeroed on the way out
//                  so the next accumulation starts clean without a separate memset pass.
//   sumsq_flat     sum of squares of the gradient (two-stage, deterministic) for global-norm clipping.
//   clip_coef      turns the norm into the multiplier min(1, max_norm / (norm + eps)) on the device,
//                  so clipping never needs a host round trip.
// Per-tensor hyper-parameters (weight decay, lr multiplier) come from a segment table: segment s
// covers elements [seg_start[s], seg_start[s+1]).
// Replaces torch._fused_adamw_ (src/kohakuwullm/training/optim/fused_adamw.py:139-172) and the
// per-tensor Triton AdamW (src/kohakuwullm/kernels/optim/adamw16.py:16-77) of the reference.
#include "common.cuh"

namespace kwu {

struct AdamHyper {
  float lr, beta1, beta2, eps;
  float bc1_inv;       // 1 / (1 - beta1^t)
  float bc2_inv_sqrt;  // 1 / sqrt(1 - beta2^t)
};

__device__ __forceinline__ int find_segment(const long long* __restrict__ seg_start, int nseg, long long i) {
  int lo = 0, hi = nseg - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seg_start[mid] <= i) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// All buffers are indexed by the same flat element index. `param_lp` may be null (fp32-only group).
// grad_scale (device scalar, may be null) multiplies the gradient before use (token count / clip).
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                  float* __restrict__ grad, __nv_bfloat16* __restrict__ param_lp,
                  const long long* __restrict__ seg_start, const float* __restrict__ seg_wd,
                  const float* __restrict__ seg_lr_mult, int nseg, long long n,
                  const float* __restrict__ grad_scale, AdamHyper hp, int zero_grad) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  // Each block walks ONE contiguous range of the buffers (not a grid-wide stride): with five streams of several
  // gigabytes each, a grid-stride loop has every block on a new 2 MB page of every stream at every iteration.
  const long long vecs = n >> 2;
  const long long per_block = ((vecs + gridDim.x - 1) / gridDim.x + 31) & ~31LL;   // whole 512-byte lines of fp32
  const long long v_begin = static_cast<long long>(blockIdx.x) * per_block;
  const long long v_end = v_begin + per_block < vecs ? v_begin + per_block : vecs;
  for (long long vi = v_begin + threadIdx.x; vi < v_end; vi += blockDim.x) {
    const long long i = vi << 2;
    // segments start on multiples of 4 elements, so one lookup serves the whole vector
    const int s = find_segment(seg_start, nseg, i);
    const float wd = seg_wd[s];
    const float lr = hp.lr * seg_lr_mult[s];
    float4 g4 = *reinterpret_cast<const float4*>(grad + i);
    float4 p4 = *reinterpret_cast<const float4*>(master + i);
    float4 m4 = *reinterpret_cast<const float4*>(m + i);
    float4 v4 = *reinterpret_cast<const float4*>(v + i);
    float g[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
    float p[4] = {p4.x, p4.y, p4.z, p4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mm[e] = hp.beta1 * mm[e] + (1.f - hp.beta1) * g[e];
      vv[e] = hp.beta2 * vv[e] + (1.f - hp.beta2) * g[e] * g[e];
      const float denom = sqrtf(vv[e]) * hp.bc2_inv_sqrt + hp.eps;
      p[e] = p[e] * (1.f - lr * wd) - lr * (mm[e] * hp.bc1_inv) / denom;
    }
    *reinterpret_cast<float4*>(master + i) = make_float4(p[0], p[1], p[2], p[3]);
    *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (param_lp) {
      uint2 o;
      o.x = pack_bf16(p[0], p[1]);
      o.y = pack_bf16(p[2], p[3]);
      *reinterpret_cast<uint2*>(param_lp + i) = o;
    }
    if (zero_grad) *reinterpret_cast<float4*>(grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Stage 1: per-block partial sums of squares. Stage 2 (one block) adds them in a fixed order.
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float s_red[8];
  float acc = 0.f;
  // one contiguous range per block, four independent 16-byte loads in flight per thread: a single load per
  // thread and iteration left the kernel at half of the copy bandwidth (bound by latency, not by bytes)
  const long long vecs = n >> 2;
  const long long per_block = ((vecs + gridDim.x - 1) / gridDim.x + 31) & ~31LL;
  const long long v_begin = static_cast<long long>(blockIdx.x) * per_block;
  const long long v_end = v_begin + per_block < vecs ? v_begin + per_block : vecs;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long vi = v_begin + threadIdx.x; vi < v_end; vi += 4LL * blockDim.x) {
    float4 a[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long idx = vi + static_cast<long long>(u) * blockDim.x;
      a[u] = idx < v_end ? x4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) acc += a[u].x * a[u].x + a[u].y * a[u].y + a[u].z * a[u].z + a[u].w * a[u].w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long j = vecs << 2; j < n; ++j) acc += x[j] * x[j];   // up to three trailing elements
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = s_red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}

__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nblocks, float* __restrict__ out,
                                   int accumulate) {
  __shared__ float s_red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) *out = accumulate ? *out + t : t;
  }
}

// base = *base_scale (device scalar, e.g. 1 / global token count; 1 when null)
// coef = base * min(1, max_norm / (sqrt(sumsq) * base + eps)); norm_out = sqrt(sumsq) * base
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, const float* __restrict__ base_scale_ptr,
                                 float max_norm, float* __restrict__ coef, float* __restrict__ norm_out) {
  const float base_scale = base_scale_ptr ? *base_scale_ptr : 1.f;
  const float norm = sqrtf(*sumsq) * base_scale;
  if (norm_out) *norm_out = norm;
  float c = base_scale;
  if (max_norm > 0.f) c *= fminf(1.f, max_norm / (norm + 1e-6f));
  *coef = c;
}

}  // namespace kwu

using namespace kwu;

KWU_API int kwu_adamw_flat(float* master, float* m, float* v, float* grad, void* param_lp,
                           const long long* seg_start, const float* seg_wd, const float* seg_lr_mult,
                           int nseg, long long n, const float* grad_scale, float lr, float beta1,
                           float beta2, float eps, int step, int zero_grad, void* stream) {
  if (n <= 0) return 0;
  if (n % 4) { set_last_error("adamw_flat: element count must be a multiple of 4"); return 7; }
  AdamHyper hp;
  hp.lr = lr; hp.beta1 = beta1; hp.beta2 = beta2; hp.eps = eps;
  hp.bc1_inv = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  hp.bc2_inv_sqrt = 1.f / sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  adamw_flat_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, reinterpret_cast<__nv_bfloat16*>(param_lp), seg_start, seg_wd, seg_lr_mult, nseg,
      n, grad_scale, hp, zero_grad); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("adamw_flat launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

KWU_API int kwu_sumsq_blocks() { return 148 * 8; }

// out (+)= sum(x^2); `partial` is scratch of kwu_sumsq_blocks() floats.
KWU_API int kwu_sumsq_flat(const float* x, long long n, float* partial, float* out, int accumulate,
                           void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int blocks = kwu_sumsq_blocks();
  sumsq_partial_kernel<<<blocks, 256, 0, st>>>(x, n, partial); kwu::count_launch();
  sumsq_final_kernel<<<1, 1024, 0, st>>>(partial, blocks, out, accumulate); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("sumsq launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

KWU_API int kwu_clip_coef(const float* sumsq, const float* base_scale, float max_norm, float* coef,
                          float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sumsq, base_scale, max_norm, coef, norm_out); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("clip_coef launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}
