// Mixture-of-experts routing and dispatch kernels.
//
//   moe_router_fwd   gate logits (fp32 SIMT tile GEMM, or read from a buffer the tensor cores filled) -> score (sigmoid | softmax | sqrt-softplus) ->
//                    selection over score + bias (bias steers SELECTION only) -> top-k by repeated warp
//                    arg-max -> gate weight from the UNBIASED score, optionally normalised over the k picks
//                    and scaled -> per-call histogram `counts` and the running `load_accum`.
//   moe_plan         counts -> expert row offsets padded to 128 rows, the grouped-GEMM tile table and
//                    zeroed cursors (one block, no host synchronisation; list lengths are host bounds).
//   moe_place        every (token, slot) pair takes a row inside its expert's padded range.
//   moe_gather       expert-sorted activation rows (padding rows are zero).
//   moe_combine      out[t] = sum_slot w[t,slot] * rows[pos(t,slot)]: a per-token gather-sum, so the result
//                    does not depend on the order in which pairs were placed (no atomics on the output).
//   moe_combine_bwd  d_rows[pos] = w * dout[t] (padding rows zero), d_w[t,slot] = <rows[pos], dout[t]>.
// Reference: src/kohakuwullm/kernels/moe/router.py:76-194, moe_dispatch.py:14-130.
#include "common.cuh"
#include "mx_quant.cuh"

namespace kwu {

constexpr int RT_BT = 32;     // tokens per block
constexpr int RT_BD = 32;     // reduction chunk
constexpr int RT_MAXE = 128;

enum : int { SCORE_SIGMOID = 0, SCORE_SOFTMAX = 1, SCORE_SQRTSOFTPLUS = 2 };

__global__ void __launch_bounds__(256)
moe_router_fwd_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ W,
                      const float* __restrict__ bias, float* __restrict__ logits_out, int* __restrict__ idx_out,
                      float* __restrict__ weight_out, int* __restrict__ counts, float* __restrict__ load_accum,
                      int T, int D, int E, int top_k, int score_fn, int norm_topk, float scaling) {
  __shared__ float s_x[RT_BT][RT_BD + 1];
  __shared__ float s_w[RT_MAXE][RT_BD + 1];
  __shared__ float s_logit[RT_BT][RT_MAXE + 1];
  const int t0 = blockIdx.x * RT_BT;
  const int tid = threadIdx.x;
  // thread -> (token ty, experts tx, tx + 8, ...): 256 threads = 32 tokens x 8 expert lanes
  const int ty = tid >> 3, tx = tid & 7;
  float acc[RT_MAXE / 8];
#pragma unroll
  for (int j = 0; j < RT_MAXE / 8; ++j) acc[j] = 0.f;
  if (x == nullptr) {
    // logits were already formed on the tensor cores (two bf16 GEMMs over a hi/lo split of W): read them
#pragma unroll
    for (int j = 0; j < RT_MAXE / 8; ++j)
      if (tx + 8 * j < E && t0 + ty < T) acc[j] = logits_out[static_cast<size_t>(t0 + ty) * E + tx + 8 * j];
  }
  for (int d0 = 0; x != nullptr && d0 < D; d0 += RT_BD) {
    for (int i = tid; i < RT_BT * RT_BD; i += 256) {
      const int r = i / RT_BD, c = i % RT_BD;
      const int t = t0 + r;
      s_x[r][c] = (t < T && d0 + c < D) ? __bfloat162float(x[static_cast<size_t>(t) * ldx + d0 + c]) : 0.f;
    }
    for (int i = tid; i < E * RT_BD; i += 256) {
      const int r = i / RT_BD, c = i % RT_BD;
      s_w[r][c] = (d0 + c < D) ? W[static_cast<size_t>(r) * D + d0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < RT_BD; ++c) {
      const float xv = s_x[ty][c];
#pragma unroll
      for (int j = 0; j < RT_MAXE / 8; ++j)
        if (tx + 8 * j < E) acc[j] += xv * s_w[tx + 8 * j][c];
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < RT_MAXE / 8; ++j)
    if (tx + 8 * j < E) s_logit[ty][tx + 8 * j] = acc[j];
  __syncthreads();

  // top-k: one warp handles 4 tokens; lane l owns experts l, l+32, l+64, l+96
  const int warp = tid >> 5, lane = tid & 31;
  for (int r = warp * 4; r < warp * 4 + 4; ++r) {
    const int t = t0 + r;
    if (t >= T) continue;
    float sc[4], sel[4];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = lane + 32 * j;
      const float lg = e < E ? s_logit[r][e] : -INFINITY;
      if (logits_out && e < E) logits_out[static_cast<size_t>(t) * E + e] = lg;
      sc[j] = lg;
      mx = fmaxf(mx, lg);
    }
    if (score_fn == SCORE_SOFTMAX) {
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sc[j] = (lane + 32 * j < E) ? __expf(sc[j] - mx) : 0.f;
        sum += sc[j];
      }
      sum = warp_sum(sum);
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[j] /= sum;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lg = sc[j];
        if (score_fn == SCORE_SIGMOID) sc[j] = 1.f / (1.f + __expf(-lg));
        else sc[j] = sqrtf(lg > 20.f ? lg : log1pf(__expf(lg)));
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = lane + 32 * j;
      sel[j] = e < E ? sc[j] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    float wsum = 0.f;
    float my_w = 0.f;
    int my_e = -1;
    for (int k = 0; k < top_k; ++k) {
      // warp arg-max over 4 candidates per lane; ties go to the lower expert index
      float best = -INFINITY;
      int be = RT_MAXE;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = lane + 32 * j;
        if (sel[j] > best || (sel[j] == best && e < be)) { best = sel[j]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
      }
      // the owner lane reports the unbiased score and retires the expert
      const int owner = be & 31, slot = be >> 5;
      float score = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j == slot) score = sc[j];
      score = __shfl_sync(0xffffffffu, score, owner);
      if (lane == owner) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j == slot) sel[j] = -INFINITY;
      }
      if (lane == k) { my_w = score; my_e = be; }
      wsum += score;
    }
    if (lane < top_k) {
      float w = my_w;
      if (norm_topk) w = w / (wsum + 1e-20f);
      w *= scaling;
      idx_out[static_cast<size_t>(t) * top_k + lane] = my_e;
      weight_out[static_cast<size_t>(t) * top_k + lane] = w;
      atomicAdd(&counts[my_e], 1);
      if (load_accum) atomicAdd(&load_accum[my_e], 1.f);
    }
  }
}

// One block. offsets[e] = start row of expert e (multiples of 128), offsets[E] = rows in use.
// tiles: (m0, expert, valid, 0) for every 128-row tile; entries past the used rows are invalid.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                int* __restrict__ cursors, int4* __restrict__ tiles, int max_tiles,
                                int* __restrict__ pair_of, int max_rows) {
  __shared__ int s_off[RT_MAXE + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E) cursors[e] = 0;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int m0 = s_off[e], i = s_off[e] / 128; m0 < s_off[e + 1] && i < max_tiles; m0 += 128, ++i)
      tiles[i] = make_int4(m0, e, 1, 0);
  for (int i = s_off[E] / 128 + threadIdx.x; i < max_tiles; i += blockDim.x) tiles[i] = make_int4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) pair_of[i] = -1;
}

__global__ void moe_place_kernel(const int* __restrict__ idx, int n_pairs, const int* __restrict__ offsets,
                                 int* __restrict__ cursors, int* __restrict__ pos_of, int* __restrict__ pair_of) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = idx[i];
  const int pos = offsets[e] + atomicAdd(&cursors[e], 1);
  pos_of[i] = pos;
  pair_of[pos] = i;
}

// rows[pos] = x[pair_of[pos] / k] (zero when the row is padding). One warp per row. With `mx` the MXFP8 copy of
// the gathered rows (what the first expert GEMM consumes) is written in the same pass: sort + quantise + place.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ pair_of, int top_k,
                  __nv_bfloat16* __restrict__ rows, int D, int max_rows, const int* __restrict__ offsets, int E,
                  const MxOut mx) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int used = offsets[E];
  const int nvec = D / 8;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < used; r += gridDim.x * wpb) {
    const int pair = pair_of[r];
    uint4* dst = reinterpret_cast<uint4*>(rows + static_cast<size_t>(r) * D);
    const uint4* src = pair < 0 ? nullptr : reinterpret_cast<const uint4*>(x + static_cast<size_t>(pair / top_k) * ldx);
    for (int v0 = 0; v0 < nvec; v0 += 32) {   // uniform trip count: the fp8 emission shuffles inside
      const int v = v0 + lane;
      const bool in = v < nvec;
      const uint4 a = (in && src) ? src[v] : make_uint4(0, 0, 0, 0);
      if (in) dst[v] = a;
      if (mx.q) {
        float f[8];
        unpack8(a, f);
        mx_emit8(f, in, r, 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
      }
    }
  }
}

// out[t] = sum_slot w[t,slot] * rows[pos_of[t,slot]]  (w null: plain sum, used as the gather backward)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ pos_of,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int ldo, int T, int top_k, int D) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    for (int v = lane; v < D / 8; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < top_k; ++s) {
        const int pos = pos_of[t * top_k + s];
        const float ws = w ? w[t * top_k + s] : 1.f;
        const uint4 a = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(pos) * D)[v];
        float2 f;
        f = unpack_bf16(a.x); acc[0] += ws * f.x; acc[1] += ws * f.y;
        f = unpack_bf16(a.y); acc[2] += ws * f.x; acc[3] += ws * f.y;
        f = unpack_bf16(a.z); acc[4] += ws * f.x; acc[5] += ws * f.y;
        f = unpack_bf16(a.w); acc[6] += ws * f.x; acc[7] += ws * f.y;
      }
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ldo)[v] =
          make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    }
  }
}

// d_rows[pos] = w[pair] * dout[token(pair)] (0 for padding); d_w[pair] = <rows[pos], dout[token]>
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ rows, const __nv_bfloat16* __restrict__ dout, int lddo,
                       const int* __restrict__ pair_of, const float* __restrict__ w, __nv_bfloat16* __restrict__ d_rows,
                       float* __restrict__ d_w, int top_k, int D, const int* __restrict__ offsets, int E,
                       const MxOut mx) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int used = offsets[E];
  const int nvec = D / 8;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < used; r += gridDim.x * wpb) {
    const int pair = pair_of[r];
    uint4* dst = reinterpret_cast<uint4*>(d_rows + static_cast<size_t>(r) * D);
    const float ws = pair < 0 ? 0.f : w[pair];
    const uint4* g = pair < 0 ? nullptr : reinterpret_cast<const uint4*>(dout + static_cast<size_t>(pair / top_k) * lddo);
    const uint4* y = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(r) * D);
    float dot = 0.f;
    for (int v0 = 0; v0 < nvec; v0 += 32) {   // uniform trip count: the fp8 emission shuffles inside
      const int v = v0 + lane;
      const bool in = v < nvec;
      uint32_t o[4] = {0u, 0u, 0u, 0u};
      if (in && g) {
        const uint4 gv = g[v], yv = y[v];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 gf = unpack_bf16(gw[e]), yf = unpack_bf16(yw[e]);
          dot += gf.x * yf.x + gf.y * yf.y;
          o[e] = pack_bf16(ws * gf.x, ws * gf.y);
        }
      }
      if (in) dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
      if (mx.q) {
        float f[8];
        unpack8(make_uint4(o[0], o[1], o[2], o[3]), f);
        mx_emit8(f, in, r, 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
      }
    }
    dot = warp_sum(dot);
    if (lane == 0 && d_w && pair >= 0) d_w[pair] = dot;
  }
}

static inline int moe_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("%s launch: %s", what, cudaGetErrorString(e)); return 11; }
  return 0;
}

}  // namespace kwu

using namespace kwu;

KWU_API int kwu_moe_router_fwd(const void* x, int ldx, const float* W, const float* bias, float* logits,
                               int* idx, float* weight, int* counts, float* load_accum, int T, int D, int E,
                               int top_k, int score_fn, int norm_topk, float scaling, void* stream) {
  if (E > RT_MAXE || E % 8 || top_k > 32 || top_k > E) { set_last_error("moe_router: need E <= 128, E %% 8 == 0, k <= 32"); return 7; }
  if (T <= 0) return 0;
  moe_router_fwd_kernel<<<(T + RT_BT - 1) / RT_BT, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, ldx, W, bias, logits, idx, weight, counts, load_accum, T, D, E, top_k, score_fn,
      norm_topk, scaling); kwu::count_launch();
  return moe_check("moe_router_fwd");
}

// Host bounds used to size the buffers: rows = pairs + E*127 rounded up to 128; tiles = rows / 128.
KWU_API int kwu_moe_max_rows(int n_pairs, int E) { return (n_pairs + E * 127 + 127) / 128 * 128; }

KWU_API int kwu_moe_plan_and_place(const int* counts, const int* idx, int n_pairs, int E, int* offsets, int* cursors,
                                   void* tiles, int max_tiles, int* pos_of, int* pair_of, int max_rows, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (E > RT_MAXE) { set_last_error("moe_plan: E must be <= 128"); return 7; }
  moe_plan_kernel<<<1, 1024, 0, st>>>(counts, E, offsets, cursors, reinterpret_cast<int4*>(tiles), max_tiles, pair_of, max_rows); kwu::count_launch();
  if (n_pairs > 0) {
    moe_place_kernel<<<(n_pairs + 255) / 256, 256, 0, st>>>(idx, n_pairs, offsets, cursors, pos_of, pair_of); kwu::count_launch();
  }
  return moe_check("moe_plan_and_place");
}

static MxOut moe_mx(void* q, void* sf, int D) {
  MxOut m;
  m.q = reinterpret_cast<uint8_t*>(q); m.ldq = D; m.sf = reinterpret_cast<uint8_t*>(sf); m.n_kchunks = D >> 7;
  return m;
}

// q / sf (optional, D %% 128 == 0): MXFP8 copy of the gathered rows, written in the same pass.
KWU_API int kwu_moe_gather(const void* x, int ldx, const int* pair_of, int top_k, void* rows, int D, int max_rows,
                           const int* offsets, int E, void* q, void* sf, void* stream) {
  if (D % 8) { set_last_error("moe_gather: D must be a multiple of 8"); return 7; }
  if (q && D % 128) { set_last_error("moe_gather: the fp8 copy needs D %% 128 == 0"); return 7; }
  moe_gather_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, ldx, pair_of, top_k, (__nv_bfloat16*)rows, D, max_rows, offsets, E, moe_mx(q, sf, D)); kwu::count_launch();
  return moe_check("moe_gather");
}

KWU_API int kwu_moe_combine(const void* rows, const int* pos_of, const float* w, void* out, int ldo, int T, int top_k,
                            int D, void* stream) {
  if (D % 8) { set_last_error("moe_combine: D must be a multiple of 8"); return 7; }
  if (T <= 0) return 0;
  int grid = (T + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_combine_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)rows, pos_of, w, (__nv_bfloat16*)out, ldo, T, top_k, D); kwu::count_launch();
  return moe_check("moe_combine");
}

// q / sf (optional, D %% 128 == 0): MXFP8 copy of d_rows, written in the same pass.
KWU_API int kwu_moe_combine_bwd(const void* rows, const void* dout, int lddo, const int* pair_of, const float* w,
                                void* d_rows, float* d_w, int top_k, int D, const int* offsets, int E, void* q,
                                void* sf, void* stream) {
  if (D % 8) { set_last_error("moe_combine_bwd: D must be a multiple of 8"); return 7; }
  if (q && D % 128) { set_last_error("moe_combine_bwd: the fp8 copy needs D %% 128 == 0"); return 7; }
  moe_combine_bwd_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)rows, (const __nv_bfloat16*)dout, lddo, pair_of, w, (__nv_bfloat16*)d_rows, d_w, top_k, D,
      offsets, E, moe_mx(q, sf, D)); kwu::count_launch();
  return moe_check("moe_combine_bwd");
}

// ------------------------------------------------------------------------------------ router backward
// Gradient of the gate weights with respect to the logits, then the two gate-matrix products, all fp32:
//   dlogits[t,e]  from d_weight[t,k] through (normalise over the k picks, scale) and the score function
//                 (sigmoid / sqrt-softplus touch only the picked experts; softmax is dense over E);
//                 an incoming dense logit gradient (auxiliary / z-loss terms) is added;
//   dx[t,:]  = dlogits[t,:] W          (T,E) x (E,D)
//   dW[e,:] += dlogits[:,e]^T x        reduced over tokens with fp32 atomics
// The contraction sizes (E <= 128) are far too small for tensor-core tiles to matter; these are SIMT tile
// loops. Reference: src/kohakuwullm/kernels/moe/router.py:197-280 and the two fp32 matmuls at :415-420.
namespace kwu {

__global__ void __launch_bounds__(256)
moe_router_dlogits_kernel(const float* __restrict__ logits, const int* __restrict__ idx,
                          const float* __restrict__ d_weight, const float* __restrict__ dlogits_in,
                          float* __restrict__ dlogits, __nv_bfloat16* __restrict__ dlogits_bf16, int T, int E,
                          int top_k, int score_fn, int norm_topk, float scaling) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    const float* lg = logits + static_cast<size_t>(t) * E;
    float* out = dlogits + static_cast<size_t>(t) * E;
    // scores of this lane's experts (lane, lane+32, ...) and, for softmax, the row statistics
    float sc[4];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = lane + 32 * j;
      sc[j] = e < E ? lg[e] : -INFINITY;
      mx = fmaxf(mx, sc[j]);
    }
    if (score_fn == SCORE_SOFTMAX) {
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sc[j] = (lane + 32 * j < E) ? __expf(sc[j] - mx) : 0.f;
        sum += sc[j];
      }
      sum = warp_sum(sum);
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[j] /= sum;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float l = sc[j];
        if (lane + 32 * j >= E) { sc[j] = 0.f; continue; }
        sc[j] = (score_fn == SCORE_SIGMOID) ? 1.f / (1.f + __expf(-l)) : sqrtf(l > 20.f ? l : log1pf(__expf(l)));
      }
    }
    // lane k (< top_k) owns pick k: its expert, unbiased score and incoming gradient
    int my_e = -1;
    float my_s = 0.f, my_g = 0.f;
    if (lane < top_k) {
      my_e = idx[static_cast<size_t>(t) * top_k + lane];
      my_g = d_weight[static_cast<size_t>(t) * top_k + lane];
    }
    for (int k = 0; k < top_k; ++k) {
      const int e = __shfl_sync(0xffffffffu, my_e, k);
      const int owner = e & 31, slot = e >> 5;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j == slot) s = sc[j];
      s = __shfl_sync(0xffffffffu, s, owner);
      if (lane == k) my_s = s;
    }
    // d(weight)/d(score) over the picks
    float ssum = warp_sum(lane < top_k ? my_s : 0.f);
    float gs = warp_sum(lane < top_k ? my_g * my_s : 0.f);
    float ds_pick = 0.f;
    if (lane < top_k) {
      if (norm_topk) {
        const float S = ssum + 1e-20f;
        ds_pick = scaling * (my_g / S - gs / (S * S));
      } else {
        ds_pick = scaling * my_g;
      }
    }
    // scatter the pick gradients onto this lane's experts
    float ds[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top_k; ++k) {
      const int e = __shfl_sync(0xffffffffu, my_e, k);
      const float d = __shfl_sync(0xffffffffu, ds_pick, k);
      if ((e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j == (e >> 5)) ds[j] += d;
      }
    }
    float dot = 0.f;
    if (score_fn == SCORE_SOFTMAX) {
#pragma unroll
      for (int j = 0; j < 4; ++j) dot += ds[j] * sc[j];
      dot = warp_sum(dot);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = lane + 32 * j;
      if (e >= E) continue;
      float dl;
      if (score_fn == SCORE_SOFTMAX) {
        dl = sc[j] * (ds[j] - dot);
      } else if (score_fn == SCORE_SIGMOID) {
        dl = ds[j] * sc[j] * (1.f - sc[j]);
      } else {  // s = sqrt(softplus(l)): ds/dl = sigmoid(l) / (2 s)
        const float sg = 1.f / (1.f + __expf(-lg[e]));
        dl = sc[j] > 0.f ? ds[j] * sg / (2.f * sc[j]) : 0.f;
      }
      if (dlogits_in) dl += dlogits_in[static_cast<size_t>(t) * E + e];
      out[e] = dl;
      if (dlogits_bf16) dlogits_bf16[static_cast<size_t>(t) * E + e] = __float2bfloat16(dl);
    }
  }
}

constexpr int RB_BT = 32, RB_BD = 128, RB_BE = 32;

// dx[t, d] = sum_e dl[t, e] W[e, d]; block = 32 tokens x 128 columns, thread = 1 token-row slice of 16 columns
__global__ void __launch_bounds__(256)
moe_router_dx_kernel(const float* __restrict__ dl, const float* __restrict__ W, __nv_bfloat16* __restrict__ dx,
                     int lddx, int T, int D, int E) {
  __shared__ float s_dl[RB_BT][RB_BE + 1];
  __shared__ float s_w[RB_BE][RB_BD + 1];
  const int t0 = blockIdx.x * RB_BT, d0 = blockIdx.y * RB_BD;
  const int ty = threadIdx.x >> 3, tx = threadIdx.x & 7;  // 32 token rows x 8 column lanes (16 columns each, stride 8)
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  for (int e0 = 0; e0 < E; e0 += RB_BE) {
    for (int i = threadIdx.x; i < RB_BT * RB_BE; i += 256) {
      const int r = i / RB_BE, c = i % RB_BE;
      s_dl[r][c] = (t0 + r < T && e0 + c < E) ? dl[static_cast<size_t>(t0 + r) * E + e0 + c] : 0.f;
    }
    for (int i = threadIdx.x; i < RB_BE * RB_BD; i += 256) {
      const int r = i / RB_BD, c = i % RB_BD;
      s_w[r][c] = (e0 + r < E && d0 + c < D) ? W[static_cast<size_t>(e0 + r) * D + d0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int e = 0; e < RB_BE; ++e) {
      const float a = s_dl[ty][e];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] += a * s_w[e][tx + 8 * j];
    }
    __syncthreads();
  }
  const int t = t0 + ty;
  if (t < T)
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int d = d0 + tx + 8 * j;
      if (d < D) dx[static_cast<size_t>(t) * lddx + d] = __float2bfloat16(acc[j]);
    }
}

constexpr int RW_BT = 32, RW_BD = 64;

// dW[e, d] += sum_{t in chunk} dl[t, e] x[t, d]; block = one 64-column slab and a strided set of 64-token chunks
__global__ void __launch_bounds__(256)
moe_router_dw_kernel(const float* __restrict__ dl, const __nv_bfloat16* __restrict__ x, int ldx,
                     float* __restrict__ dW, int T, int D, int E) {
  __shared__ float s_dl[RW_BT][RT_MAXE + 1];
  __shared__ float s_x[RW_BT][RW_BD + 1];
  const int d0 = blockIdx.x * RW_BD;
  // thread -> column tx (0..63) and expert lanes ey, ey + 4, ... (E / 4 experts each)
  const int tx = threadIdx.x & 63, ey = threadIdx.x >> 6;
  float acc[RT_MAXE / 4];
#pragma unroll
  for (int j = 0; j < RT_MAXE / 4; ++j) acc[j] = 0.f;
  for (int t0 = blockIdx.y * RW_BT; t0 < T; t0 += gridDim.y * RW_BT) {
    for (int i = threadIdx.x; i < RW_BT * E; i += 256) {
      const int r = i / E, c = i % E;
      s_dl[r][c] = (t0 + r < T) ? dl[static_cast<size_t>(t0 + r) * E + c] : 0.f;
    }
    for (int i = threadIdx.x; i < RW_BT * RW_BD; i += 256) {
      const int r = i / RW_BD, c = i % RW_BD;
      s_x[r][c] = (t0 + r < T && d0 + c < D) ? __bfloat162float(x[static_cast<size_t>(t0 + r) * ldx + d0 + c]) : 0.f;
    }
    __syncthreads();
    for (int r = 0; r < RW_BT; ++r) {
      const float xv = s_x[r][tx];
#pragma unroll
      for (int j = 0; j < RT_MAXE / 4; ++j)
        if (ey + 4 * j < E) acc[j] += s_dl[r][ey + 4 * j] * xv;
    }
    __syncthreads();
  }
  if (d0 + tx < D)
#pragma unroll
    for (int j = 0; j < RT_MAXE / 4; ++j)
      if (ey + 4 * j < E) atomicAdd(&dW[static_cast<size_t>(ey + 4 * j) * D + d0 + tx], acc[j]);
}

}  // namespace kwu

// dlogits: (T,E) fp32 scratch/output. dx (T,D) bf16 or null. dW (E,D) fp32, ACCUMULATED into (zero it first
// for a plain gradient), or null.
// dlogits_bf16 (optional): a bf16 copy of the logit gradient, the operand of the tensor-core products
// dx = dl W and dW += dl^T x when the caller forms them with the GEMM kernel instead of passing dx / dW here.
KWU_API int kwu_moe_router_bwd(const float* logits, const int* idx, const float* d_weight, const float* dlogits_in,
                               float* dlogits, void* dlogits_bf16, const void* x, int ldx, const float* W, void* dx,
                               int lddx, float* dW, int T, int D, int E, int top_k, int score_fn, int norm_topk,
                               float scaling, void* stream) {
  if (E > RT_MAXE || top_k > 32) { set_last_error("moe_router_bwd: need E <= 128 and k <= 32"); return 7; }
  if (T <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = (T + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_router_dlogits_kernel<<<grid, 256, 0, st>>>(logits, idx, d_weight, dlogits_in, dlogits,
                                                 (__nv_bfloat16*)dlogits_bf16, T, E, top_k, score_fn, norm_topk,
                                                 scaling); kwu::count_launch();
  if (dx) {
    dim3 g((T + RB_BT - 1) / RB_BT, (D + RB_BD - 1) / RB_BD);
    moe_router_dx_kernel<<<g, 256, 0, st>>>(dlogits, W, (__nv_bfloat16*)dx, lddx, T, D, E); kwu::count_launch();
  }
  if (dW) {
    int chunks = (T + RW_BT - 1) / RW_BT;
    if (chunks > 64) chunks = 64;
    dim3 g((D + RW_BD - 1) / RW_BD, chunks);
    moe_router_dw_kernel<<<g, 256, 0, st>>>(dlogits, (const __nv_bfloat16*)x, ldx, dW, T, D, E); kwu::count_launch();
  }
  return moe_check("moe_router_bwd");
}
