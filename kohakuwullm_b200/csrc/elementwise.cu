// Bandwidth-bound kernels: RMSNorm (+residual add), per-head QK-RMSNorm fused with RoPE, SwiGLU.
//
// All of them read and write bf16 with fp32 math, use 16-byte vector accesses and size their
// grids from the row count. They take the place of the reference's Triton kernels
// src/kohakuwullm/kernels/elementwise/rmsnorm.py:20-128, swiglu.py:49-119 and
// src/kohakuwullm/kernels/attention/rope.py:27-89.
#include "common.cuh"
#include "mx_quant.cuh"

namespace kwu {

// --------------------------------------------------------------------------- RMSNorm
// One warp per row. y = x * rstd * w   (w fp32, optional; `one_plus` selects the Gemma (1+w) form)
// Optional fused residual: h = x + res is formed first, written to `h_out`, and normalised.
template <bool HAS_RES>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows,
                   int cols, float eps, int one_plus, const MxOut mx) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;  // cols % 8 == 0 (checked on the host)
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * cols);
    const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * cols) : nullptr;
    uint4* hr = HAS_RES ? reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * cols) : nullptr;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      uint4 a = xr[v];
      float2 f0 = unpack_bf16(a.x), f1 = unpack_bf16(a.y), f2 = unpack_bf16(a.z), f3 = unpack_bf16(a.w);
      if (HAS_RES) {
        const uint4 b = rr[v];
        const float2 g0 = unpack_bf16(b.x), g1 = unpack_bf16(b.y), g2 = unpack_bf16(b.z), g3 = unpack_bf16(b.w);
        a.x = pack_bf16(f0.x + g0.x, f0.y + g0.y);
        a.y = pack_bf16(f1.x + g1.x, f1.y + g1.y);
        a.z = pack_bf16(f2.x + g2.x, f2.y + g2.y);
        a.w = pack_bf16(f3.x + g3.x, f3.y + g3.y);
        hr[v] = a;
        // normalise the value that was stored (bf16-rounded), so backward sees the same h
        f0 = unpack_bf16(a.x); f1 = unpack_bf16(a.y); f2 = unpack_bf16(a.z); f3 = unpack_bf16(a.w);
      }
      ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y +
            f3.x * f3.x + f3.y * f3.y;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / static_cast<float>(cols) + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    if (HAS_RES) __syncwarp();
    const uint4* src = HAS_RES ? reinterpret_cast<const uint4*>(hr) : xr;
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * cols);
    for (int v0 = 0; v0 < nvec; v0 += 32) {  // uniform trip count: the fp8 emission shuffles inside
      const int v = v0 + lane;
      const bool in = v < nvec;
      const uint4 a = in ? src[v] : make_uint4(0, 0, 0, 0);
      float f[8];
      float2 t;
      t = unpack_bf16(a.x); f[0] = t.x; f[1] = t.y;
      t = unpack_bf16(a.y); f[2] = t.x; f[3] = t.y;
      t = unpack_bf16(a.z); f[4] = t.x; f[5] = t.y;
      t = unpack_bf16(a.w); f[6] = t.x; f[7] = t.y;
      if (w && in) {
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v];
        const float4 w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = f[e] * rstd * (one_plus ? 1.f + ww[e] : ww[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= rstd;
      }
      uint4 o;
      o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
      o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
      if (in) yr[v] = o;
      if (mx.q) {  // the fp8 copy is made from the stored (bf16-rounded) values
        float fr[8];
        unpack8(o, fr);
        mx_emit8(fr, in, row, 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
      }
    }
  }
}

// Backward. dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w_eff,  xhat = x * rstd.
// Optional `dres` is added into dx (gradient arriving on the residual path), which fuses the
// residual-add backward. Each block accumulates a dW partial over its rows in shared memory and
// writes it to dw_partial[block, cols]; a second kernel sums the partials.
// Register-resident variant for rows of at most 32 * NV vectors (8 bf16 each): a lane loads its NV vectors
// of x and dy once (all loads issued before the first use), forms the row's dot product, and produces dx
// and the weight-gradient partial from the same registers, so every byte is read exactly once.
constexpr int RMS_BWD_THREADS = 384;   // up to 12 warps at <= 170 registers; the launcher uses them when every warp gets many rows
// STAGED: rows come through shared memory, fetched one row ahead with bulk copies (issued by lane 0 of the warp
// that uses them), so the next row's bytes are in flight while this one is reduced, combined and written;
// measured with clock stamps, a warp otherwise spent 3700 of ~9000 cycles per row waiting for its loads.
// Shared memory then is 256 bytes of barriers and, per warp, two stages of three rows (x, dy, dres); the
// stage area doubles as the warp's parking row for the column sums at the end.
template <int NV, bool STAGED>
__global__ void __launch_bounds__(RMS_BWD_THREADS)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                       const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, float* __restrict__ dw_direct, int rows, int cols,
                       int one_plus, const MxOut mx, int* __restrict__ status) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  extern __shared__ float s_dw[];  // unstaged: one parking row of cols floats per warp
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = cols >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * 2u;
  uint8_t* smem_base = reinterpret_cast<uint8_t*>(s_dw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_base);                         // STAGED: [warps][2]
  uint8_t* my_area = smem_base + 256 + static_cast<size_t>(warp) * 6 * row_bytes;   // STAGED: 2 stages x 3 rows
  const int row_step = gridDim.x * warps_per_block;
  const int first_row = blockIdx.x * warps_per_block + warp;
  auto fetch = [&](int row, int st) {   // lane 0 only
    uint64_t* bar = &bars[warp * 2 + st];
    uint8_t* dst = my_area + static_cast<size_t>(st) * 3 * row_bytes;
    mbar_expect_tx(bar, (dres ? 3u : 2u) * row_bytes);
    bulk_g2s(dst, x + static_cast<size_t>(row) * cols, row_bytes, bar);
    bulk_g2s(dst + row_bytes, dy + static_cast<size_t>(row) * cols, row_bytes, bar);
    if (dres) bulk_g2s(dst + 2 * row_bytes, dres + static_cast<size_t>(row) * cols, row_bytes, bar);
  };
  if (STAGED) {
    if (lane == 0) {
      mbar_init(&bars[warp * 2], 1);
      mbar_init(&bars[warp * 2 + 1], 1);
      mbar_fence_init();
      if (first_row < rows) fetch(first_row, 0);
    }
    __syncwarp();
  }
  uint64_t dw2[NV][4];   // column sums of g * xhat for this lane's columns, as fp32 pairs
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) dw2[j][e] = pack_f32x2(0.f, 0.f);
  const float inv_cols = 1.f / static_cast<float>(cols);
  int pass = 0;
  for (int row = first_row; row < rows; row += row_step, ++pass) {
    uint4 a[NV], g[NV], r[NV];
    if (STAGED) {
      const int st = pass & 1;
      if (lane == 0 && row + row_step < rows) fetch(row + row_step, st ^ 1);
      // bounded wait: a copy that never lands ends the loop instead of hanging the kernel, and the host
      // learns of it through the status word (the rows this warp did not reach stay unwritten)
      bool landed = false;
      for (int tries = 0; tries < 400000 && !landed; ++tries) landed = mbar_try_wait(&bars[warp * 2 + st], (pass >> 1) & 1);
      if (!__all_sync(0xffffffffu, landed)) {
        if (lane == 0 && status) atomicCAS(status, 0, KWU_ERR_TIMEOUT_MISC);
        // the next row's copy was issued above into the other stage: give it a bounded time to land before
        // the stage area is reused as the parking row and the CTA exits
        if (row + row_step < rows) {
          bool other = false;
          for (int tries = 0; tries < 100000 && !other; ++tries)
            other = mbar_try_wait(&bars[warp * 2 + (st ^ 1)], ((pass + 1) >> 1) & 1);
        }
        __syncwarp();
        break;
      }
      const uint4* xs = reinterpret_cast<const uint4*>(my_area + static_cast<size_t>(st) * 3 * row_bytes);
      const uint4* gs = reinterpret_cast<const uint4*>(my_area + static_cast<size_t>(st) * 3 * row_bytes + row_bytes);
      const uint4* rs = reinterpret_cast<const uint4*>(my_area + static_cast<size_t>(st) * 3 * row_bytes + 2 * row_bytes);
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = lane + 32 * j;
        const bool in = v < nvec;
        a[j] = in ? xs[v] : make_uint4(0, 0, 0, 0);
        g[j] = in ? gs[v] : make_uint4(0, 0, 0, 0);
        r[j] = (in && dres) ? rs[v] : make_uint4(0, 0, 0, 0);
      }
      __syncwarp();   // every lane holds its copy: the next pass may refill this stage
    } else {
      const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * cols);
      const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * cols);
      const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * cols) : nullptr;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = lane + 32 * j;
        const bool in = v < nvec;
        a[j] = in ? xr[v] : make_uint4(0, 0, 0, 0);
        g[j] = in ? gr[v] : make_uint4(0, 0, 0, 0);
        r[j] = (in && rr) ? rr[v] : make_uint4(0, 0, 0, 0);
      }
    }
    const float rstd = rstd_in[row];
    // packed fp32 pairs throughout: a bf16x2 word becomes one 64-bit operand, every multiply / fused
    // multiply-add works on both halves (the row costs about a third fewer issue slots)
    auto bf2 = [](uint32_t u) { return pack_f32x2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u)); };
    const uint64_t one2 = pack_f32x2(1.f, 1.f);
    auto wpair = [&](int v, int e) -> uint64_t {
      if (!w) return one2;
      const uint64_t wv = *reinterpret_cast<const uint64_t*>(w + 8 * v + 2 * e);
      return one_plus ? add_f32x2(wv, one2) : wv;
    };
    uint64_t dot2 = pack_f32x2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      if (v < nvec) {
        const uint32_t aw[4] = {a[j].x, a[j].y, a[j].z, a[j].w}, gw[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) dot2 = fma_f32x2(mul_f32x2(bf2(gw[e]), wpair(v, e)), bf2(aw[e]), dot2);
      }
    }
    float dlo, dhi;
    unpack_f32x2(dot2, dlo, dhi);
    const float dot = warp_sum(dlo + dhi) * rstd * inv_cols;
    const uint64_t rstd2 = pack_f32x2(rstd, rstd), ndot2 = pack_f32x2(-dot, -dot);
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * cols);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      uint32_t o[4] = {0u, 0u, 0u, 0u};
      if (v < nvec) {
        const uint32_t aw[4] = {a[j].x, a[j].y, a[j].z, a[j].w}, gw[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
        const uint32_t rw[4] = {r[j].x, r[j].y, r[j].z, r[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint64_t g2 = bf2(gw[e]);
          const uint64_t xh2 = mul_f32x2(bf2(aw[e]), rstd2);                          // normalised input
          const uint64_t t2 = fma_f32x2(xh2, ndot2, mul_f32x2(g2, wpair(v, e)));      // g*w - xhat*dot
          float o0, o1;
          unpack_f32x2(fma_f32x2(t2, rstd2, bf2(rw[e])), o0, o1);                     // rstd*(...) + residual grad
          o[e] = pack_bf16(o0, o1);
          dw2[j][e] = fma_f32x2(g2, xh2, dw2[j][e]);
        }
        dxr[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
      if (mx.q && 32 * j < nvec) {  // warp-uniform condition: all lanes take part in the block maximum
        float fr[8];
        unpack8(make_uint4(o[0], o[1], o[2], o[3]), fr);
        mx_emit8(fr, v < nvec, row, 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
      }
    }
  }
  if (dw_partial) {
    // every warp parks its column sums in its own shared-memory row, then each column is summed over the
    // warps by one thread (shared-memory float atomics from 40 values per lane took 4 us of a 24 us launch)
    float* mine = STAGED ? reinterpret_cast<float*>(my_area) : s_dw + static_cast<size_t>(warp) * cols;
    if (STAGED) __syncwarp();   // the warp's last stage reads are done (each pass ends its reads with a warp barrier)
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      if (v < nvec) {
        float d[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) unpack_f32x2(dw2[j][e], d[2 * e], d[2 * e + 1]);
        *reinterpret_cast<float4*>(mine + 8 * v) = make_float4(d[0], d[1], d[2], d[3]);
        *reinterpret_cast<float4*>(mine + 8 * v + 4) = make_float4(d[4], d[5], d[6], d[7]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      float t = 0.f;
      for (int wp = 0; wp < warps_per_block; ++wp)
        t += STAGED ? reinterpret_cast<const float*>(smem_base + 256 + static_cast<size_t>(wp) * 6 * row_bytes)[i]
                    : s_dw[static_cast<size_t>(wp) * cols + i];
      if (dw_direct) atomicAdd(&dw_direct[i], t);
      else dw_partial[static_cast<size_t>(blockIdx.x) * cols + i] = t;
    }
  }
}

__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int cols, int one_plus) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  extern __shared__ float s_dw[];  // cols floats
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  if (dw_partial)
    for (int i = threadIdx.x; i < cols; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  // a lane always owns the same columns (vectors lane, lane+32, ...), so the weight gradient of up to
  // RMS_REG_VECS vectors per lane is summed over the warp's rows in registers and flushed once
  constexpr int RMS_REG_VECS = 8;   // covers cols <= 2048; wider rows fall back to shared atomics
  const bool reg_dw = dw_partial && nvec <= 32 * RMS_REG_VECS;
  float dw_acc[RMS_REG_VECS][8];
#pragma unroll
  for (int j = 0; j < RMS_REG_VECS; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[j][e] = 0.f;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * cols);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 a = xr[v], g = gr[v];
      float xf[8], gf[8];
      float2 t;
      t = unpack_bf16(a.x); xf[0] = t.x; xf[1] = t.y; t = unpack_bf16(a.y); xf[2] = t.x; xf[3] = t.y;
      t = unpack_bf16(a.z); xf[4] = t.x; xf[5] = t.y; t = unpack_bf16(a.w); xf[6] = t.x; xf[7] = t.y;
      t = unpack_bf16(g.x); gf[0] = t.x; gf[1] = t.y; t = unpack_bf16(g.y); gf[2] = t.x; gf[3] = t.y;
      t = unpack_bf16(g.z); gf[4] = t.x; gf[5] = t.y; t = unpack_bf16(g.w); gf[6] = t.x; gf[7] = t.y;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float we = 1.f;
        if (w) we = one_plus ? 1.f + w[8 * v + e] : w[8 * v + e];
        dot += gf[e] * we * xf[e] * rstd;
      }
    }
    dot = warp_sum(dot) / static_cast<float>(cols);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * cols) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * cols);
#pragma unroll
    for (int jj = 0; jj < RMS_REG_VECS + 1; ++jj) {
     for (int v = lane + 32 * jj; v < nvec; v += (jj == RMS_REG_VECS ? 32 : nvec)) {
      const uint4 a = xr[v], g = gr[v];
      float xf[8], gf[8], rf[8];
      float2 t;
      t = unpack_bf16(a.x); xf[0] = t.x; xf[1] = t.y; t = unpack_bf16(a.y); xf[2] = t.x; xf[3] = t.y;
      t = unpack_bf16(a.z); xf[4] = t.x; xf[5] = t.y; t = unpack_bf16(a.w); xf[6] = t.x; xf[7] = t.y;
      t = unpack_bf16(g.x); gf[0] = t.x; gf[1] = t.y; t = unpack_bf16(g.y); gf[2] = t.x; gf[3] = t.y;
      t = unpack_bf16(g.z); gf[4] = t.x; gf[5] = t.y; t = unpack_bf16(g.w); gf[6] = t.x; gf[7] = t.y;
      if (rr) {
        const uint4 r = rr[v];
        t = unpack_bf16(r.x); rf[0] = t.x; rf[1] = t.y; t = unpack_bf16(r.y); rf[2] = t.x; rf[3] = t.y;
        t = unpack_bf16(r.z); rf[4] = t.x; rf[5] = t.y; t = unpack_bf16(r.w); rf[6] = t.x; rf[7] = t.y;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) rf[e] = 0.f;
      }
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float we = 1.f;
        if (w) we = one_plus ? 1.f + w[8 * v + e] : w[8 * v + e];
        const float xhat = xf[e] * rstd;
        o[e] = rstd * (gf[e] * we - xhat * dot) + rf[e];
        if (dw_partial) {
          if (reg_dw && jj < RMS_REG_VECS) dw_acc[jj < RMS_REG_VECS ? jj : 0][e] += gf[e] * xhat;
          else atomicAdd(&s_dw[8 * v + e], gf[e] * xhat);
        }
      }
      uint4 ov;
      ov.x = pack_bf16(o[0], o[1]); ov.y = pack_bf16(o[2], o[3]);
      ov.z = pack_bf16(o[4], o[5]); ov.w = pack_bf16(o[6], o[7]);
      dxr[v] = ov;
     }
    }
  }
  if (reg_dw) {
#pragma unroll
    for (int j = 0; j < RMS_REG_VECS; ++j) {
      const int v = lane + 32 * j;
      if (v < nvec)
#pragma unroll
        for (int e = 0; e < 8; ++e) atomicAdd(&s_dw[8 * v + e], dw_acc[j][e]);
    }
  }
  if (dw_partial) {
    __syncthreads();
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
      dw_partial[static_cast<size_t>(blockIdx.x) * cols + i] = s_dw[i];
  }
}

// dw[c] (+)= sum_b partial[b, c]
__global__ void colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                       int nblocks, int cols, int accumulate) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[static_cast<size_t>(b) * cols + c];
  dw[c] = accumulate ? dw[c] + s : s;
}

// --------------------------------------------------------------------------- QK-norm + RoPE
// One warp per (token, head) row of HEAD_DIM = 64: lane i owns elements i and i+32, which are
// exactly the rotate-half partners. Reads rows from a strided source (the fused qkv projection
// output), applies RMSNorm over the head (optional fp32 weight[64]) and then rotary embedding
// with per-token cos/sin half tables (T, rot/2) fp32; elements beyond `rot` pass through.
//   forward : dst = rope(norm(src))
//   backward: dsrc = norm_bwd(rope_bwd(ddst)); dweight partials accumulated with atomics.
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ src, int src_ld,
                       __nv_bfloat16* __restrict__ dst, int dst_ld,
                       const float* __restrict__ weight, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int tokens, int heads, int rot_half,
                       float eps, int do_norm) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(tokens) * heads;
  const int wpb = blockDim.x >> 5;
  for (long r = static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < total;
       r += static_cast<long>(gridDim.x) * wpb) {
    const int t = static_cast<int>(r / heads);
    const int h = static_cast<int>(r % heads);
    const __nv_bfloat16* s = src + static_cast<size_t>(t) * src_ld + h * 64;
    float a = __bfloat162float(s[lane]);
    float b = __bfloat162float(s[lane + 32]);
    if (do_norm) {
      const float ss = warp_sum(a * a + b * b);
      const float rstd = rsqrtf(ss * (1.f / 64.f) + eps);
      a *= rstd;
      b *= rstd;
      if (weight) {
        a *= weight[lane];
        b *= weight[lane + 32];
      }
      // the reference rounds the normalised value to the storage dtype before rotating
      a = __bfloat162float(__float2bfloat16(a));
      b = __bfloat162float(__float2bfloat16(b));
    }
    float oa = a, ob = b;
    if (rot_half == 32) {
      const float c = cos_t[static_cast<size_t>(t) * 32 + lane];
      const float sn = sin_t[static_cast<size_t>(t) * 32 + lane];
      oa = a * c - b * sn;
      ob = b * c + a * sn;
    } else if (rot_half > 0) {
      // partial rotary: element j < rot_half pairs with j + rot_half; the tail passes through
      const float other_a = __shfl_sync(0xffffffffu, a, (lane + rot_half) & 31);
      const float other_b = __shfl_sync(0xffffffffu, a, (lane - rot_half) & 31);
      if (lane < rot_half) {
        const float c = cos_t[static_cast<size_t>(t) * rot_half + lane];
        const float sn = sin_t[static_cast<size_t>(t) * rot_half + lane];
        oa = a * c - other_a * sn;
      } else if (lane < 2 * rot_half) {
        const float c = cos_t[static_cast<size_t>(t) * rot_half + lane - rot_half];
        const float sn = sin_t[static_cast<size_t>(t) * rot_half + lane - rot_half];
        oa = a * c + other_b * sn;
      }
    }
    __nv_bfloat16* d = dst + static_cast<size_t>(t) * dst_ld + h * 64;
    d[lane] = __float2bfloat16(oa);
    d[lane + 32] = __float2bfloat16(ob);
  }
}

__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ src, int src_ld,
                       const __nv_bfloat16* __restrict__ dout, int dout_ld,
                       __nv_bfloat16* __restrict__ dsrc, int dsrc_ld,
                       const float* __restrict__ weight, float* __restrict__ dweight,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens,
                       int heads, int rot_half, float eps, int do_norm) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  __shared__ float s_dw[64];
  if (threadIdx.x < 64) s_dw[threadIdx.x] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(tokens) * heads;
  const int wpb = blockDim.x >> 5;
  float dwa = 0.f, dwb = 0.f;
  for (long r = static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < total;
       r += static_cast<long>(gridDim.x) * wpb) {
    const int t = static_cast<int>(r / heads);
    const int h = static_cast<int>(r % heads);
    const __nv_bfloat16* g = dout + static_cast<size_t>(t) * dout_ld + h * 64;
    float ga = __bfloat162float(g[lane]);
    float gb = __bfloat162float(g[lane + 32]);
    // rotary backward = rotation by the negated angle
    float da = ga, db = gb;
    if (rot_half == 32) {
      const float c = cos_t[static_cast<size_t>(t) * 32 + lane];
      const float sn = sin_t[static_cast<size_t>(t) * 32 + lane];
      da = ga * c + gb * sn;
      db = gb * c - ga * sn;
    } else if (rot_half > 0) {
      const float other_a = __shfl_sync(0xffffffffu, ga, (lane + rot_half) & 31);
      const float other_b = __shfl_sync(0xffffffffu, ga, (lane - rot_half) & 31);
      if (lane < rot_half) {
        const float c = cos_t[static_cast<size_t>(t) * rot_half + lane];
        const float sn = sin_t[static_cast<size_t>(t) * rot_half + lane];
        da = ga * c + other_a * sn;
      } else if (lane < 2 * rot_half) {
        const float c = cos_t[static_cast<size_t>(t) * rot_half + lane - rot_half];
        const float sn = sin_t[static_cast<size_t>(t) * rot_half + lane - rot_half];
        da = ga * c - other_b * sn;
      }
    }
    if (do_norm) {
      const __nv_bfloat16* s = src + static_cast<size_t>(t) * src_ld + h * 64;
      const float xa = __bfloat162float(s[lane]);
      const float xb = __bfloat162float(s[lane + 32]);
      const float ss = warp_sum(xa * xa + xb * xb);
      const float rstd = rsqrtf(ss * (1.f / 64.f) + eps);
      const float ha = xa * rstd, hb = xb * rstd;
      const float wa = weight ? weight[lane] : 1.f, wb = weight ? weight[lane + 32] : 1.f;
      if (dweight) {
        dwa += da * ha;
        dwb += db * hb;
      }
      const float g1 = da * wa, g2 = db * wb;
      const float dot = warp_sum(g1 * ha + g2 * hb) * (1.f / 64.f);
      da = rstd * (g1 - ha * dot);
      db = rstd * (g2 - hb * dot);
    }
    __nv_bfloat16* d = dsrc + static_cast<size_t>(t) * dsrc_ld + h * 64;
    d[lane] = __float2bfloat16(da);
    d[lane + 32] = __float2bfloat16(db);
  }
  if (dweight) {
    atomicAdd(&s_dw[lane], dwa);
    atomicAdd(&s_dw[lane + 32], dwb);
    __syncthreads();
    if (threadIdx.x < 64) atomicAdd(&dweight[threadIdx.x], s_dw[threadIdx.x]);
  }
}

// Vector form for full rotary (rot_half == 32) or no rotary: eight lanes per 64-element row, 16-byte accesses,
// four rows per warp pass. Lane sub-index j holds elements [8j, 8j+8); its rotate-half partner is lane j ^ 4.
__device__ __forceinline__ float row8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__global__ void __launch_bounds__(256)
qknorm_rope_fwd_vec_kernel(const __nv_bfloat16* __restrict__ src, int src_ld,
                           __nv_bfloat16* __restrict__ dst, int dst_ld,
                           const float* __restrict__ weight, const float* __restrict__ cos_t,
                           const float* __restrict__ sin_t, int tokens, int heads, int rot_half,
                           float eps, int do_norm) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int lane = threadIdx.x & 31, sub = lane & 7, slot = lane >> 3;
  const long total = static_cast<long>(tokens) * heads;
  const int wpb = blockDim.x >> 5;
  float w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = (do_norm && weight) ? weight[8 * sub + i] : 1.f;
  for (long r0 = (static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5)) * 4; r0 < total;
       r0 += static_cast<long>(gridDim.x) * wpb * 4) {
    const long r = r0 + slot;
    const bool live = r < total;
    const int t = live ? static_cast<int>(r / heads) : 0;
    const int h = live ? static_cast<int>(r % heads) : 0;
    float x[8];
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * src_ld + h * 64 + 8 * sub);
    unpack8(raw, x);
    uint32_t xw[4] = {raw.x, raw.y, raw.z, raw.w};
    if (do_norm) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
      const float rstd = rsqrtf(row8_sum(ss) * (1.f / 64.f) + eps);
      // the reference rounds the normalised value to the storage dtype before rotating
#pragma unroll
      for (int i = 0; i < 4; ++i) xw[i] = pack_bf16(x[2 * i] * rstd * w[2 * i], x[2 * i + 1] * rstd * w[2 * i + 1]);
      unpack8(make_uint4(xw[0], xw[1], xw[2], xw[3]), x);
    }
    if (rot_half == 32) {
      float y[8];
      uint32_t pw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pw[i] = __shfl_xor_sync(0xffffffffu, xw[i], 4);
      unpack8(make_uint4(pw[0], pw[1], pw[2], pw[3]), y);
      const float sign = (sub < 4) ? -1.f : 1.f;
      const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(t) * 32 + 8 * (sub & 3));
      const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(t) * 32 + 8 * (sub & 3));
      const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = x[i] * c[i] + sign * y[i] * sn[i];
    }
    if (live) {
      uint4 o;
      o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
      o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
      *reinterpret_cast<uint4*>(dst + static_cast<size_t>(t) * dst_ld + h * 64 + 8 * sub) = o;
    }
  }
}

__global__ void __launch_bounds__(256)
qknorm_rope_bwd_vec_kernel(const __nv_bfloat16* __restrict__ src, int src_ld,
                           const __nv_bfloat16* __restrict__ dout, int dout_ld,
                           __nv_bfloat16* __restrict__ dsrc, int dsrc_ld,
                           const float* __restrict__ weight, float* __restrict__ dweight,
                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens,
                           int heads, int rot_half, float eps, int do_norm) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  __shared__ float s_dw[64];
  if (threadIdx.x < 64) s_dw[threadIdx.x] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, sub = lane & 7, slot = lane >> 3;
  const long total = static_cast<long>(tokens) * heads;
  const int wpb = blockDim.x >> 5;
  float w[8], dw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = (do_norm && weight) ? weight[8 * sub + i] : 1.f;
    dw[i] = 0.f;
  }
  for (long r0 = (static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5)) * 4; r0 < total;
       r0 += static_cast<long>(gridDim.x) * wpb * 4) {
    const long r = r0 + slot;
    const bool live = r < total;
    const int t = live ? static_cast<int>(r / heads) : 0;
    const int h = live ? static_cast<int>(r % heads) : 0;
    uint4 graw = make_uint4(0, 0, 0, 0), xraw = make_uint4(0, 0, 0, 0);
    if (live) {
      graw = *reinterpret_cast<const uint4*>(dout + static_cast<size_t>(t) * dout_ld + h * 64 + 8 * sub);
      if (do_norm) xraw = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * src_ld + h * 64 + 8 * sub);
    }
    float d[8];
    unpack8(graw, d);
    if (rot_half == 32) {
      // rotary backward = rotation by the negated angle
      float y[8];
      const uint32_t gw[4] = {graw.x, graw.y, graw.z, graw.w};
      uint32_t pw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pw[i] = __shfl_xor_sync(0xffffffffu, gw[i], 4);
      unpack8(make_uint4(pw[0], pw[1], pw[2], pw[3]), y);
      const float sign = (sub < 4) ? 1.f : -1.f;
      const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(t) * 32 + 8 * (sub & 3));
      const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(t) * 32 + 8 * (sub & 3));
      const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) d[i] = d[i] * c[i] + sign * y[i] * sn[i];
    }
    if (do_norm) {
      float x[8];
      unpack8(xraw, x);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
      const float rstd = rsqrtf(row8_sum(ss) * (1.f / 64.f) + eps);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] *= rstd;                 // normalised input
        dw[i] += d[i] * x[i];         // dead rows carry zeros
        d[i] *= w[i];
        dot += d[i] * x[i];
      }
      dot = row8_sum(dot) * (1.f / 64.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) d[i] = rstd * (d[i] - x[i] * dot);
    }
    if (live) {
      uint4 o;
      o.x = pack_bf16(d[0], d[1]); o.y = pack_bf16(d[2], d[3]);
      o.z = pack_bf16(d[4], d[5]); o.w = pack_bf16(d[6], d[7]);
      *reinterpret_cast<uint4*>(dsrc + static_cast<size_t>(t) * dsrc_ld + h * 64 + 8 * sub) = o;
    }
  }
  if (dweight && do_norm) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // the four row slots of a warp hold the same columns: fold them before the shared atomics
      float v = dw[i];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      if (slot == 0) atomicAdd(&s_dw[8 * sub + i], v);
    }
    __syncthreads();
    if (threadIdx.x < 64) atomicAdd(&dweight[threadIdx.x], s_dw[threadIdx.x]);
  }
}

// Query and key heads of a fused qkv projection in ONE launch (rows = tokens x (Hq + Hkv); the q and k slices
// are adjacent in `src`, so head h of token t sits at src + t * src_ld + 64 h for both). At 4096 tokens each
// of the two separate launches is a few microseconds of work behind a launch; one launch halves that.
// Vector form only: full rotary (rot_half == 32) or none.
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_qk_kernel(const __nv_bfloat16* __restrict__ src, int src_ld, __nv_bfloat16* __restrict__ dst_q,
                          __nv_bfloat16* __restrict__ dst_k, const float* __restrict__ wq_p,
                          const float* __restrict__ wk_p, const float* __restrict__ cos_t,
                          const float* __restrict__ sin_t, int tokens, int Hq, int Hkv, int rot_half, float eps,
                          int do_norm) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int lane = threadIdx.x & 31, sub = lane & 7, slot = lane >> 3;
  const int HT = Hq + Hkv;
  const long total = static_cast<long>(tokens) * HT;
  const int wpb = blockDim.x >> 5;
  float wq[8], wk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    wq[i] = (do_norm && wq_p) ? wq_p[8 * sub + i] : 1.f;
    wk[i] = (do_norm && wk_p) ? wk_p[8 * sub + i] : 1.f;
  }
  // Two rows per 8-lane group and iteration (8 rows per warp): both rows' loads (data and rotary tables) are
  // issued before either row's arithmetic, so a lane has ten 16-byte loads in flight instead of five. At 4096
  // tokens a warp runs the loop once or twice only, and the kernel's time is that chain's latency.
  for (long r0 = (static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5)) * 8; r0 < total;
       r0 += static_cast<long>(gridDim.x) * wpb * 8) {
    long rr[2];
    bool live[2], is_k[2];
    int tt[2], hh[2];
    uint4 raw[2];
    float4 c0[2], c1[2], s0[2], s1[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      rr[u] = r0 + slot + 4 * u;
      live[u] = rr[u] < total;
      tt[u] = live[u] ? static_cast<int>(rr[u] / HT) : 0;
      hh[u] = live[u] ? static_cast<int>(rr[u] % HT) : 0;
      is_k[u] = hh[u] >= Hq;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (live[u]) raw[u] = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(tt[u]) * src_ld + hh[u] * 64 + 8 * sub);
      if (rot_half == 32) {
        const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(tt[u]) * 32 + 8 * (sub & 3));
        const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(tt[u]) * 32 + 8 * (sub & 3));
        c0[u] = cp[0]; c1[u] = cp[1]; s0[u] = sp[0]; s1[u] = sp[1];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float x[8];
      unpack8(raw[u], x);
      uint32_t xw[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
      if (do_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
        const float rstd = rsqrtf(row8_sum(ss) * (1.f / 64.f) + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float w0 = is_k[u] ? wk[2 * i] : wq[2 * i], w1 = is_k[u] ? wk[2 * i + 1] : wq[2 * i + 1];
          xw[i] = pack_bf16(x[2 * i] * rstd * w0, x[2 * i + 1] * rstd * w1);
        }
        unpack8(make_uint4(xw[0], xw[1], xw[2], xw[3]), x);
      }
      if (rot_half == 32) {
        float y[8];
        uint32_t pw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pw[i] = __shfl_xor_sync(0xffffffffu, xw[i], 4);
        unpack8(make_uint4(pw[0], pw[1], pw[2], pw[3]), y);
        const float sign = (sub < 4) ? -1.f : 1.f;
        const float c[8] = {c0[u].x, c0[u].y, c0[u].z, c0[u].w, c1[u].x, c1[u].y, c1[u].z, c1[u].w};
        const float sn[8] = {s0[u].x, s0[u].y, s0[u].z, s0[u].w, s1[u].x, s1[u].y, s1[u].z, s1[u].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = x[i] * c[i] + sign * y[i] * sn[i];
      }
      if (live[u]) {
        uint4 o;
        o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
        o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
        __nv_bfloat16* d = is_k[u] ? dst_k + (static_cast<size_t>(tt[u]) * Hkv + (hh[u] - Hq)) * 64
                                   : dst_q + (static_cast<size_t>(tt[u]) * Hq + hh[u]) * 64;
        *reinterpret_cast<uint4*>(d + 8 * sub) = o;
      }
    }
  }
}

// Backward of the above for q and k in one launch, writing into the fused gradient buffer `dsrc` (the layout of
// the qkv projection output). With `mx.q` set it also emits the MXFP8 copy (bytes + scales) of the WHOLE
// gradient row, v slice included: the v slice was written into `dsrc` by the attention backward before this
// kernel runs and is only read back here, so the consumer (the qkv projection's dgrad) needs no quantise pass.
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_qk_kernel(const __nv_bfloat16* __restrict__ src, int src_ld, const __nv_bfloat16* __restrict__ dq,
                          const __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dsrc, int dsrc_ld,
                          const float* __restrict__ wq_p, const float* __restrict__ wk_p,
                          float* __restrict__ dwq_out, float* __restrict__ dwk_out,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens, int Hq,
                          int Hkv, int rot_half, float eps, int do_norm, const MxOut mx, int q_blocks) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  // Blocks [0, q_blocks) take the query heads, the rest the key heads (and, with emission, the value heads,
  // which are only read back and quantised): a block then needs ONE weight vector and ONE gradient
  // accumulator in registers (both roles in every thread cost 99 registers and a third of the occupancy).
  __shared__ float s_dw[64];
  if (threadIdx.x < 64) s_dw[threadIdx.x] = 0.f;
  __syncthreads();
  const bool q_role = static_cast<int>(blockIdx.x) < q_blocks;
  const int role_block = q_role ? blockIdx.x : blockIdx.x - q_blocks;
  const int role_blocks = q_role ? q_blocks : gridDim.x - q_blocks;
  const int lane = threadIdx.x & 31, sub = lane & 7, slot = lane >> 3;
  const int H = q_role ? Hq : (mx.q ? 2 * Hkv : Hkv);   // heads this role walks per token
  const int h_base = q_role ? 0 : Hq;                   // first head of the role inside a qkv row
  const int H_norm = q_role ? Hq : Hkv;                 // heads of the role that are normalised / rotated
  const __nv_bfloat16* gsrc = q_role ? dq : dk;
  const float* w_p = q_role ? wq_p : wk_p;
  float* dw_out = q_role ? dwq_out : dwk_out;
  const long total = static_cast<long>(tokens) * H;
  const int wpb = blockDim.x >> 5;
  float w[8], dw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = (do_norm && w_p) ? w_p[8 * sub + i] : 1.f;
    dw[i] = 0.f;
  }
  // uniform trip count per warp: the emission shuffles inside the loop
  for (long r0 = (static_cast<long>(role_block) * wpb + (threadIdx.x >> 5)) * 4; r0 < total;
       r0 += static_cast<long>(role_blocks) * wpb * 4) {
    const long r = r0 + slot;
    const bool live = r < total;
    const int t = live ? static_cast<int>(r / H) : 0;
    const int hl = live ? static_cast<int>(r % H) : 0;
    const bool is_v = hl >= H_norm;
    const int h = h_base + hl;
    uint4 o = make_uint4(0, 0, 0, 0);
    uint4 graw = make_uint4(0, 0, 0, 0), xraw = make_uint4(0, 0, 0, 0);
    if (live) {
      if (is_v) {
        o = *reinterpret_cast<const uint4*>(dsrc + static_cast<size_t>(t) * dsrc_ld + h * 64 + 8 * sub);
      } else {
        graw = *reinterpret_cast<const uint4*>(gsrc + (static_cast<size_t>(t) * H_norm + hl) * 64 + 8 * sub);
        if (do_norm) xraw = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * src_ld + h * 64 + 8 * sub);
      }
    }
    float d[8];
    unpack8(graw, d);
    if (rot_half == 32) {
      float y[8];
      const uint32_t gw[4] = {graw.x, graw.y, graw.z, graw.w};
      uint32_t pw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pw[i] = __shfl_xor_sync(0xffffffffu, gw[i], 4);
      unpack8(make_uint4(pw[0], pw[1], pw[2], pw[3]), y);
      const float sign = (sub < 4) ? 1.f : -1.f;
      const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(t) * 32 + 8 * (sub & 3));
      const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(t) * 32 + 8 * (sub & 3));
      const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) d[i] = d[i] * c[i] + sign * y[i] * sn[i];
    }
    if (do_norm) {
      float x[8];
      unpack8(xraw, x);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
      const float rstd = rsqrtf(row8_sum(ss) * (1.f / 64.f) + eps);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] *= rstd;
        dw[i] += d[i] * x[i];         // dead and value rows carry zeros
        d[i] *= w[i];
        dot += d[i] * x[i];
      }
      dot = row8_sum(dot) * (1.f / 64.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) d[i] = rstd * (d[i] - x[i] * dot);
    }
    if (!is_v) {
      o.x = pack_bf16(d[0], d[1]); o.y = pack_bf16(d[2], d[3]);
      o.z = pack_bf16(d[4], d[5]); o.w = pack_bf16(d[6], d[7]);
      if (live) *reinterpret_cast<uint4*>(dsrc + static_cast<size_t>(t) * dsrc_ld + h * 64 + 8 * sub) = o;
    }
    if (mx.q) {
      float fr[8];
      unpack8(o, fr);   // the rounded values, as a quantise pass over the stored tensor would see them
      mx_emit8(fr, live, t, h * 64 + 8 * sub, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
    }
  }
  if (do_norm && dw_out) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a = dw[i];
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      if (slot == 0) atomicAdd(&s_dw[8 * sub + i], a);
    }
    __syncthreads();
    if (threadIdx.x < 64) atomicAdd(&dw_out[threadIdx.x], s_dw[threadIdx.x]);
  }
}

// --------------------------------------------------------------------------- SwiGLU
// in: (rows, 2H) with the gate in columns [0,H) and the value in [H,2H); out (rows, H).
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, int in_ld, __nv_bfloat16* __restrict__ out,
                  int out_ld, int rows, int H, const MxOut mx) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int nvec = H >> 3;
  const long total = static_cast<long>(rows) * nvec;
  // uniform trip count for the whole block: the optional fp8 emission shuffles inside the loop
  for (long base = static_cast<long>(blockIdx.x) * blockDim.x; base < total;
       base += static_cast<long>(gridDim.x) * blockDim.x) {
    const long i = base + threadIdx.x;
    const bool in_range = i < total;
    const int r = in_range ? static_cast<int>(i / nvec) : 0;
    const int v = in_range ? static_cast<int>(i % nvec) : 0;
    uint32_t ow[4] = {0u, 0u, 0u, 0u};
    if (in_range) {
      const uint4 g = *reinterpret_cast<const uint4*>(in + static_cast<size_t>(r) * in_ld + 8 * v);
      const uint4 u = *reinterpret_cast<const uint4*>(in + static_cast<size_t>(r) * in_ld + H + 8 * v);
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 gf = unpack_bf16(gw[e]), uf = unpack_bf16(uw[e]);
        const float s0 = gf.x * fast_rcp(1.f + __expf(-gf.x)), s1 = gf.y * fast_rcp(1.f + __expf(-gf.y));
        ow[e] = pack_bf16(s0 * uf.x, s1 * uf.y);
      }
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * out_ld + 8 * v) =
          make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    if (mx.q) {
      float fr[8];
      unpack8(make_uint4(ow[0], ow[1], ow[2], ow[3]), fr);
      mx_emit8(fr, in_range, r, 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
    }
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, int in_ld,
                  const __nv_bfloat16* __restrict__ dout, int dout_ld,
                  __nv_bfloat16* __restrict__ din, int din_ld, int rows, int H, const MxOut mx) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int nvec = H >> 3;
  const long total = static_cast<long>(rows) * nvec;
  for (long base = static_cast<long>(blockIdx.x) * blockDim.x; base < total;
       base += static_cast<long>(gridDim.x) * blockDim.x) {
    const long i = base + threadIdx.x;
    const bool in_range = i < total;
    const int r = in_range ? static_cast<int>(i / nvec) : 0;
    const int v = in_range ? static_cast<int>(i % nvec) : 0;
    uint32_t og[4] = {0u, 0u, 0u, 0u}, ou[4] = {0u, 0u, 0u, 0u};
    if (in_range) {
      const uint4 g = *reinterpret_cast<const uint4*>(in + static_cast<size_t>(r) * in_ld + 8 * v);
      const uint4 u = *reinterpret_cast<const uint4*>(in + static_cast<size_t>(r) * in_ld + H + 8 * v);
      const uint4 d = *reinterpret_cast<const uint4*>(dout + static_cast<size_t>(r) * dout_ld + 8 * v);
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w},
                     dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 gf = unpack_bf16(gw[e]), uf = unpack_bf16(uw[e]), df = unpack_bf16(dw[e]);
        const float sg0 = fast_rcp(1.f + __expf(-gf.x)), sg1 = fast_rcp(1.f + __expf(-gf.y));
        const float si0 = gf.x * sg0, si1 = gf.y * sg1;
        const float dg0 = df.x * uf.x * (sg0 * (1.f + gf.x * (1.f - sg0)));
        const float dg1 = df.y * uf.y * (sg1 * (1.f + gf.y * (1.f - sg1)));
        og[e] = pack_bf16(dg0, dg1);
        ou[e] = pack_bf16(df.x * si0, df.y * si1);
      }
      *reinterpret_cast<uint4*>(din + static_cast<size_t>(r) * din_ld + 8 * v) =
          make_uint4(og[0], og[1], og[2], og[3]);
      *reinterpret_cast<uint4*>(din + static_cast<size_t>(r) * din_ld + H + 8 * v) =
          make_uint4(ou[0], ou[1], ou[2], ou[3]);
    }
    if (mx.q) {  // din is quantised along its 2H columns: gate half and value half are separate blocks
      float fr[8];
      unpack8(make_uint4(og[0], og[1], og[2], og[3]), fr);
      mx_emit8(fr, in_range, r, 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
      unpack8(make_uint4(ou[0], ou[1], ou[2], ou[3]), fr);
      mx_emit8(fr, in_range, r, H + 8 * v, mx.q, mx.ldq, mx.sf, mx.n_kchunks);
    }
  }
}

static inline int grid_for(long work_items, int per_block, int cap = 148 * 8) {
  long g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

static inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s launch: %s", what, cudaGetErrorString(e));
    return 11;
  }
  return 0;
}

}  // namespace kwu

using namespace kwu;

static MxOut make_mx(void* q, int ldq, void* sf, int cols) {
  MxOut m;
  m.q = reinterpret_cast<uint8_t*>(q); m.ldq = ldq; m.sf = reinterpret_cast<uint8_t*>(sf); m.n_kchunks = cols >> 7;
  return m;
}
// The fused fp8 copy needs whole 128-row scale tiles and 128-column chunks.
static bool mx_shape_ok(const char* what, int rows, int cols) {
  if (rows % 128 || cols % 128) {
    set_last_error("%s: fp8 emission needs rows and cols that are multiples of 128 (got %d x %d)", what, rows, cols);
    return false;
  }
  return true;
}

static int rmsnorm_fwd_impl(const void* x, const void* res, const float* w, void* y, void* h_out,
                            float* rstd, int rows, int cols, float eps, int one_plus, const MxOut mx, void* stream) {
  if (cols % 8) { set_last_error("rmsnorm: cols must be a multiple of 8"); return 7; }
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows, 8);
  if (res) {
    launch_k(rmsnorm_fwd_kernel<true>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w,
                                                  (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows,
                                                  cols, eps, one_plus, mx); kwu::count_launch();
  } else {
    launch_k(rmsnorm_fwd_kernel<false>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, nullptr, w, (__nv_bfloat16*)y,
                                                   nullptr, rstd, rows, cols, eps, one_plus, mx); kwu::count_launch();
  }
  return check_launch("rmsnorm_fwd");
}

KWU_API int kwu_rmsnorm_fwd(const void* x, const void* res, const float* w, void* y, void* h_out,
                            float* rstd, int rows, int cols, float eps, int one_plus, void* stream) {
  return rmsnorm_fwd_impl(x, res, w, y, h_out, rstd, rows, cols, eps, one_plus, make_mx(nullptr, 0, nullptr, cols), stream);
}

// Same, and also writes the MXFP8 copy of y (e4m3 bytes `q` with pitch ldq, scale chunks `sf`).
KWU_API int kwu_rmsnorm_fwd_mx(const void* x, const void* res, const float* w, void* y, void* h_out,
                               float* rstd, int rows, int cols, float eps, int one_plus, void* q, int ldq, void* sf,
                               void* stream) {
  if (!mx_shape_ok("rmsnorm_fwd_mx", rows, cols)) return 7;
  return rmsnorm_fwd_impl(x, res, w, y, h_out, rstd, rows, cols, eps, one_plus, make_mx(q, ldq, sf, cols), stream);
}

// dw_partial: scratch of `kwu_rmsnorm_bwd_blocks(rows)` x cols floats (may be null when w is null).
KWU_API int kwu_rmsnorm_bwd_blocks(int rows) { return grid_for(rows, 8, 296); }

static int rmsnorm_bwd_impl(const void* x, const float* w, const float* rstd, const void* dy,
                            const void* dres, void* dx, float* dw, float* dw_partial, int rows,
                            int cols, int one_plus, int accumulate_dw, const MxOut mx, void* stream,
                            int max_blocks = 296) {
  if (cols % 8) { set_last_error("rmsnorm: cols must be a multiple of 8"); return 7; }
  if (mx.q && cols > 2048) { set_last_error("rmsnorm_bwd_mx: rows wider than 2048 columns are not supported"); return 7; }
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = grid_for(rows, 8, max_blocks);
  const bool want_dw = (w != nullptr && dw != nullptr && dw_partial != nullptr);
  const size_t dw_smem = want_dw ? cols * sizeof(float) : 0;
  // 12 warps per CTA keep more rows in flight (8 % faster at 32768 rows) but leave the 4096-row case with an uneven
  // 2-or-3 rows per warp; there 8 warps are faster
  const int threads = rows >= 148 * 12 * 6 ? RMS_BWD_THREADS : 256;
  const size_t dw_smem_reg = want_dw ? static_cast<size_t>(threads / 32) * cols * sizeof(float) : 0;   // one row per warp
  const int nv = (cols / 8 + 31) / 32;
  if (nv <= 8 && grid > 148) grid = 148;  // the register-resident kernels run one CTA per SM
  // dw += ... : the register-resident kernels add their column sums to dw themselves
  float* direct = (want_dw && accumulate_dw && nv <= 8) ? dw : nullptr;
#define KWU_RMS_BWD_HEAD (const __nv_bfloat16*)x, w, rstd, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres, \
      (__nv_bfloat16*)dx, want_dw ? dw_partial : nullptr
#define KWU_RMS_BWD_TAIL rows, cols, one_plus
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const size_t stage_smem = 256 + static_cast<size_t>(threads / 32) * 6 * cols * 2;
  const bool staged = al16(x) && al16(dy) && (!dres || al16(dres)) && stage_smem <= 220 * 1024;
  static PerDeviceOnce reg_attr;
  if (reg_attr.pending()) {
    const int lim = 220 * 1024;
#define KWU_RMS_ATTR(NVV)                                                                                      \
    cudaFuncSetAttribute(rmsnorm_bwd_reg_kernel<NVV, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim); \
    cudaFuncSetAttribute(rmsnorm_bwd_reg_kernel<NVV, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim)
    KWU_RMS_ATTR(2); KWU_RMS_ATTR(4); KWU_RMS_ATTR(5); KWU_RMS_ATTR(6); KWU_RMS_ATTR(8);
#undef KWU_RMS_ATTR
    reg_attr.mark();
  }
#define KWU_RMS_LAUNCH(NVV)                                                                                         \
  do {                                                                                                              \
    if (staged)                                                                                                     \
      launch_k(rmsnorm_bwd_reg_kernel<NVV, true>, dim3(grid), dim3(threads), stage_smem, st, KWU_RMS_BWD_HEAD, direct, KWU_RMS_BWD_TAIL, mx, kwu::device_status_word()); \
    else                                                                                                            \
      launch_k(rmsnorm_bwd_reg_kernel<NVV, false>, dim3(grid), dim3(threads), dw_smem_reg, st, KWU_RMS_BWD_HEAD, direct, KWU_RMS_BWD_TAIL, mx, nullptr); \
  } while (0)
  if (nv <= 2) KWU_RMS_LAUNCH(2);
  else if (nv <= 4) KWU_RMS_LAUNCH(4);
  else if (nv <= 5) KWU_RMS_LAUNCH(5);
  else if (nv <= 6) KWU_RMS_LAUNCH(6);
  else if (nv <= 8) KWU_RMS_LAUNCH(8);
  else launch_k(rmsnorm_bwd_kernel, dim3(grid), dim3(256), dw_smem, st, KWU_RMS_BWD_HEAD, KWU_RMS_BWD_TAIL);
#undef KWU_RMS_LAUNCH
#undef KWU_RMS_BWD_HEAD
#undef KWU_RMS_BWD_TAIL
  kwu::count_launch();
  if (int rc = check_launch("rmsnorm_bwd")) return rc;
  if (want_dw && !direct) {
    launch_k(colsum_partials_kernel, dim3((cols + 255) / 256), dim3(256), 0, st, dw_partial, dw, grid, cols, accumulate_dw); kwu::count_launch();
    return check_launch("rmsnorm_dw");
  }
  return 0;
}

KWU_API int kwu_rmsnorm_bwd(const void* x, const float* w, const float* rstd, const void* dy,
                            const void* dres, void* dx, float* dw, float* dw_partial, int rows,
                            int cols, int one_plus, int accumulate_dw, void* stream) {
  return rmsnorm_bwd_impl(x, w, rstd, dy, dres, dx, dw, dw_partial, rows, cols, one_plus, accumulate_dw,
                          make_mx(nullptr, 0, nullptr, cols), stream);
}

// Same, and also writes the MXFP8 copy of dx (the gradient that the previous projection's dgrad consumes).
KWU_API int kwu_rmsnorm_bwd_mx(const void* x, const float* w, const float* rstd, const void* dy,
                               const void* dres, void* dx, float* dw, float* dw_partial, int rows,
                               int cols, int one_plus, int accumulate_dw, void* q, int ldq, void* sf, void* stream) {
  if (!mx_shape_ok("rmsnorm_bwd_mx", rows, cols)) return 7;
  return rmsnorm_bwd_impl(x, w, rstd, dy, dres, dx, dw, dw_partial, rows, cols, one_plus, accumulate_dw,
                          make_mx(q, ldq, sf, cols), stream);
}

KWU_API int kwu_qknorm_rope_fwd(const void* src, int src_ld, void* dst, int dst_ld, const float* weight,
                                const float* cos_t, const float* sin_t, int tokens, int heads,
                                int head_dim, int rot_half, float eps, int do_norm, void* stream) {
  if (head_dim != 64) { set_last_error("qknorm_rope: head_dim must be 64"); return 7; }
  if (rot_half != 32 && rot_half != 16 && rot_half != 8 && rot_half != 0) {
    set_last_error("qknorm_rope: rotary half must be 0, 8, 16 or 32");
    return 7;
  }
  if (tokens <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (rot_half == 32 || rot_half == 0) && src_ld % 8 == 0 && dst_ld % 8 == 0 && al16(src) && al16(dst) &&
                   (rot_half == 0 || (al16(cos_t) && al16(sin_t))) && (!weight || al16(weight));
  if (vec) {
    const int grid = grid_for(static_cast<long>(tokens) * heads, 32, 148 * 16);
    launch_k(qknorm_rope_fwd_vec_kernel, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)src, src_ld, (__nv_bfloat16*)dst,
                                                    dst_ld, weight, cos_t, sin_t, tokens, heads, rot_half,
                                                    eps, do_norm); kwu::count_launch();
    return check_launch("qknorm_rope_fwd");
  }
  const int grid = grid_for(static_cast<long>(tokens) * heads, 8, 148 * 16);
  launch_k(qknorm_rope_fwd_kernel, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)src, src_ld, (__nv_bfloat16*)dst,
                                              dst_ld, weight, cos_t, sin_t, tokens, heads, rot_half,
                                              eps, do_norm); kwu::count_launch();
  return check_launch("qknorm_rope_fwd");
}

KWU_API int kwu_qknorm_rope_bwd(const void* src, int src_ld, const void* dout, int dout_ld, void* dsrc,
                                int dsrc_ld, const float* weight, float* dweight, const float* cos_t,
                                const float* sin_t, int tokens, int heads, int head_dim, int rot_half,
                                float eps, int do_norm, void* stream) {
  if (head_dim != 64) { set_last_error("qknorm_rope: head_dim must be 64"); return 7; }
  if (tokens <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (rot_half == 32 || rot_half == 0) && src_ld % 8 == 0 && dout_ld % 8 == 0 && dsrc_ld % 8 == 0 &&
                   al16(src) && al16(dout) && al16(dsrc) && (rot_half == 0 || (al16(cos_t) && al16(sin_t)));
  if (vec) {
    // few blocks: each one ends with 64 global atomics for the norm weight gradient (148 x 16 blocks measured 15 % slower)
    const int grid = grid_for(static_cast<long>(tokens) * heads, 32, 148 * 4);
    launch_k(qknorm_rope_bwd_vec_kernel, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)src, src_ld,
                                                    (const __nv_bfloat16*)dout, dout_ld, (__nv_bfloat16*)dsrc,
                                                    dsrc_ld, weight, dweight, cos_t, sin_t, tokens, heads,
                                                    rot_half, eps, do_norm); kwu::count_launch();
    return check_launch("qknorm_rope_bwd");
  }
  const int grid = grid_for(static_cast<long>(tokens) * heads, 8, 148 * 4);
  launch_k(qknorm_rope_bwd_kernel, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)src, src_ld,
                                              (const __nv_bfloat16*)dout, dout_ld, (__nv_bfloat16*)dsrc,
                                              dsrc_ld, weight, dweight, cos_t, sin_t, tokens, heads,
                                              rot_half, eps, do_norm); kwu::count_launch();
  return check_launch("qknorm_rope_bwd");
}

// q and k heads of a fused qkv buffer in one launch. dst_q (T, Hq, 64) and dst_k (T, Hkv, 64) are contiguous.
// Needs rot_half 32 or 0 and 16-byte aligned operands (returns 7 otherwise: use the per-tensor entry points).
KWU_API int kwu_qknorm_rope_fwd_qk(const void* src, int src_ld, void* dst_q, void* dst_k, const float* wq,
                                   const float* wk, const float* cos_t, const float* sin_t, int tokens, int Hq,
                                   int Hkv, int rot_half, float eps, int do_norm, void* stream) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if ((rot_half != 32 && rot_half != 0) || src_ld % 8 || !al16(src) || !al16(dst_q) || !al16(dst_k) ||
      (rot_half && (!al16(cos_t) || !al16(sin_t)))) {
    set_last_error("qknorm_rope_fwd_qk: needs full or no rotary and 16-byte aligned operands");
    return 7;
  }
  if (tokens <= 0) return 0;
  const int grid = grid_for(static_cast<long>(tokens) * (Hq + Hkv), 64, 148 * 8);
  launch_k(qknorm_rope_fwd_qk_kernel, dim3(grid), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)src, src_ld, (__nv_bfloat16*)dst_q, (__nv_bfloat16*)dst_k, wq, wk, cos_t, sin_t, tokens,
      Hq, Hkv, rot_half, eps, do_norm); kwu::count_launch();
  return check_launch("qknorm_rope_fwd_qk");
}

// Backward for q and k in one launch; dq (T, Hq, 64) and dk (T, Hkv, 64) contiguous, results written into the
// q and k slices of dsrc (T, dsrc_ld). dwq / dwk (64 floats each, optional) are ADDED to. With q8 / sf non-null
// the MXFP8 copy of all (Hq + 2 Hkv) * 64 columns of dsrc is written too (the v slice must already hold its
// final values); tokens must then be a multiple of 128 and the column count a multiple of 128.
KWU_API int kwu_qknorm_rope_bwd_qk(const void* src, int src_ld, const void* dq, const void* dk, void* dsrc,
                                   int dsrc_ld, const float* wq, const float* wk, float* dwq, float* dwk,
                                   const float* cos_t, const float* sin_t, int tokens, int Hq, int Hkv,
                                   int rot_half, float eps, int do_norm, void* q8, int ldq, void* sf,
                                   void* stream) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if ((rot_half != 32 && rot_half != 0) || src_ld % 8 || dsrc_ld % 8 || !al16(src) || !al16(dq) || !al16(dk) ||
      !al16(dsrc) || (rot_half && (!al16(cos_t) || !al16(sin_t)))) {
    set_last_error("qknorm_rope_bwd_qk: needs full or no rotary and 16-byte aligned operands");
    return 7;
  }
  if (tokens <= 0) return 0;
  const int cols = (Hq + 2 * Hkv) * 64;
  if (q8 && (tokens % 128 || cols % 128 || ldq % 8)) {
    set_last_error("qknorm_rope_bwd_qk: the fp8 copy needs tokens and columns in multiples of 128");
    return 7;
  }
  const int kv_heads = q8 ? 2 * Hkv : Hkv;
  const int grid = grid_for(static_cast<long>(tokens) * (Hq + kv_heads), 32, 148 * 8);
  // blocks are dealt to the two roles in proportion to their rows (at least one each)
  int q_blocks = static_cast<int>(static_cast<long>(grid) * Hq / (Hq + kv_heads));
  if (q_blocks < 1) q_blocks = 1;
  const int total_blocks = q_blocks + (grid - q_blocks < 1 ? 1 : grid - q_blocks);
  launch_k(qknorm_rope_bwd_qk_kernel, dim3(total_blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)src, src_ld, (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (__nv_bfloat16*)dsrc,
      dsrc_ld, wq, wk, dwq, dwk, cos_t, sin_t, tokens, Hq, Hkv, rot_half, eps, do_norm,
      make_mx(q8, ldq, sf, cols), q_blocks); kwu::count_launch();
  return check_launch("qknorm_rope_bwd_qk");
}

static int swiglu_fwd_impl(const void* in, int in_ld, void* out, int out_ld, int rows, int H, const MxOut mx,
                           void* stream) {
  if (H % 8 || in_ld % 8 || out_ld % 8) { set_last_error("swiglu: H and pitches must be multiples of 8"); return 7; }
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(static_cast<long>(rows) * (H / 8), 256);
  launch_k(swiglu_fwd_kernel, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)in, in_ld, (__nv_bfloat16*)out, out_ld,
                                         rows, H, mx); kwu::count_launch();
  return check_launch("swiglu_fwd");
}

KWU_API int kwu_swiglu_fwd(const void* in, int in_ld, void* out, int out_ld, int rows, int H,
                           void* stream) {
  return swiglu_fwd_impl(in, in_ld, out, out_ld, rows, H, make_mx(nullptr, 0, nullptr, H), stream);
}

// Same, and also writes the MXFP8 copy of the (rows, H) output.
KWU_API int kwu_swiglu_fwd_mx(const void* in, int in_ld, void* out, int out_ld, int rows, int H, void* q, int ldq,
                              void* sf, void* stream) {
  if (!mx_shape_ok("swiglu_fwd_mx", rows, H)) return 7;
  return swiglu_fwd_impl(in, in_ld, out, out_ld, rows, H, make_mx(q, ldq, sf, H), stream);
}

static int swiglu_bwd_impl(const void* in, int in_ld, const void* dout, int dout_ld, void* din,
                           int din_ld, int rows, int H, const MxOut mx, void* stream) {
  if (H % 8 || in_ld % 8 || dout_ld % 8 || din_ld % 8) { set_last_error("swiglu: H and pitches must be multiples of 8"); return 7; }
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(static_cast<long>(rows) * (H / 8), 256);
  launch_k(swiglu_bwd_kernel, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)in, in_ld, (const __nv_bfloat16*)dout,
                                         dout_ld, (__nv_bfloat16*)din, din_ld, rows, H, mx); kwu::count_launch();
  return check_launch("swiglu_bwd");
}

KWU_API int kwu_swiglu_bwd(const void* in, int in_ld, const void* dout, int dout_ld, void* din,
                           int din_ld, int rows, int H, void* stream) {
  return swiglu_bwd_impl(in, in_ld, dout, dout_ld, din, din_ld, rows, H, make_mx(nullptr, 0, nullptr, 2 * H), stream);
}

// Same, and also writes the MXFP8 copy of the (rows, 2H) input gradient.
KWU_API int kwu_swiglu_bwd_mx(const void* in, int in_ld, const void* dout, int dout_ld, void* din,
                              int din_ld, int rows, int H, void* q, int ldq, void* sf, void* stream) {
  if (!mx_shape_ok("swiglu_bwd_mx", rows, 2 * H) || H % 32) { set_last_error("swiglu_bwd_mx: bad shape"); return 7; }
  return swiglu_bwd_impl(in, in_ld, dout, dout_ld, din, din_ld, rows, H, make_mx(q, ldq, sf, 2 * H), stream);
}

// --------------------------------------------------------------------------- allocation-free variant
// kwu_rmsnorm_bwd_noalloc: RMSNorm backward for callers that cannot obtain device memory themselves.
// See kwu_noalloc.h for who those callers are and for the contract. The weight-gradient partial sums
// that kwu_rmsnorm_bwd takes as a caller-provided buffer live here in a fixed array inside the
// library image; every GPU that loads the library carries it until the process exits.
#include "kwu_noalloc.h"

#include <mutex>

namespace kwu {

static __device__ __align__(256) float g_noalloc_dw_partial[KWU_NOALLOC_MAX_BLOCKS * KWU_NOALLOC_MAX_COLS];

// In host code the array's name is only a handle for the runtime, not a device address, so the
// address is asked for once per device (with that device current) and cached.
static float* noalloc_scratch_address() {
  static std::mutex mu;
  static float* per_device[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_error("rmsnorm_bwd_noalloc: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_dw_partial);
    if (e != cudaSuccess || !ptr) {
      set_last_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    per_device[dev] = ptr;
  }
  return per_device[dev];
}

}  // namespace kwu

KWU_API int kwu_rmsnorm_bwd_noalloc(const void* x, const float* w, const float* rstd, const void* dy,
                                    const void* dres, void* dx, float* dw, int rows, int cols,
                                    int one_plus, int accumulate_dw, void* stream) {
  if (cols % 8) { set_last_error("rmsnorm_bwd_noalloc: cols must be a multiple of 8 (got %d)", cols); return 7; }
  if (cols > KWU_NOALLOC_MAX_COLS) {
    set_last_error("rmsnorm_bwd_noalloc: cols %d exceeds the built-in scratch (at most %d columns); "
                   "use kwu_rmsnorm_bwd with a caller-provided buffer", cols, KWU_NOALLOC_MAX_COLS);
    return 7;
  }
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool want_dw = (w != nullptr && dw != nullptr);
  float* partial = nullptr;
  if (want_dw) {
    partial = noalloc_scratch_address();
    if (!partial) return 12;
  }
  // same kernels and the same choice between them as kwu_rmsnorm_bwd; only the scratch differs. Every block
  // overwrites its own row of the scratch before the column sum reads it, so nothing in the array has to
  // start at zero even though it still holds the previous call's partial sums
  return rmsnorm_bwd_impl(x, w, rstd, dy, dres, dx, want_dw ? dw : nullptr, partial, rows, cols, one_plus,
                          accumulate_dw, make_mx(nullptr, 0, nullptr, cols), stream, KWU_NOALLOC_MAX_BLOCKS);
}

// --------------------------------------------------------------------------- embedding
// Forward: out[t, :] = W[token[t], :] * scale (one warp per token row, 16-byte vectors).
// Backward: dW[token[t], :] += dout[t, :] * scale with vector fp32 reductions straight into the fp32 gradient
// buffer: no dense (vocab x dim) temporary and no separate accumulation pass. Takes the place of
// nn.Embedding's gather and embedding_dense_backward (src/kohakuwullm/models/backbone.py:73-122 uses nn.Embedding).
namespace kwu {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ W,
                     __nv_bfloat16* __restrict__ out, int T, int D, int V, float scale) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    long long id = tokens[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(W + static_cast<size_t>(id) * D);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * D);
    for (int v = lane; v < D / 8; v += 32) {
      uint4 a = src[v];
      if (scale != 1.f) {
        float f[8];
        float2 x;
        x = unpack_bf16(a.x); f[0] = x.x; f[1] = x.y; x = unpack_bf16(a.y); f[2] = x.x; f[3] = x.y;
        x = unpack_bf16(a.z); f[4] = x.x; f[5] = x.y; x = unpack_bf16(a.w); f[6] = x.x; f[7] = x.y;
        a = make_uint4(pack_bf16(f[0] * scale, f[1] * scale), pack_bf16(f[2] * scale, f[3] * scale),
                       pack_bf16(f[4] * scale, f[5] * scale), pack_bf16(f[6] * scale, f[7] * scale));
      }
      dst[v] = a;
    }
  }
}

__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ dout,
                     float* __restrict__ dW, int T, int D, int V, float scale) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    const long long id = tokens[t];
    if (id < 0 || id >= V) continue;
    const uint4* src = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(t) * D);
    float* dst = dW + static_cast<size_t>(id) * D;
    for (int v = lane; v < D / 8; v += 32) {
      const uint4 a = src[v];
      const float2 f0 = unpack_bf16(a.x), f1 = unpack_bf16(a.y), f2 = unpack_bf16(a.z), f3 = unpack_bf16(a.w);
      red_add_f32x4(dst + 8 * v, f0.x * scale, f0.y * scale, f1.x * scale, f1.y * scale);
      red_add_f32x4(dst + 8 * v + 4, f2.x * scale, f2.y * scale, f3.x * scale, f3.y * scale);
    }
  }
}

}  // namespace kwu

KWU_API int kwu_embedding_fwd(const long long* tokens, const void* W, void* out, int T, int D, int V, float scale,
                              void* stream) {
  if (D % 8) { set_last_error("embedding: dim must be a multiple of 8"); return 7; }
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<grid_for(T, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      tokens, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, T, D, V, scale); kwu::count_launch();
  return check_launch("embedding_fwd");
}

// dW: fp32 (V, D), accumulated into.
KWU_API int kwu_embedding_bwd(const long long* tokens, const void* dout, float* dW, int T, int D, int V, float scale,
                              void* stream) {
  if (D % 8) { set_last_error("embedding: dim must be a multiple of 8"); return 7; }
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<grid_for(T, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      tokens, (const __nv_bfloat16*)dout, dW, T, D, V, scale); kwu::count_launch();
  return check_launch("embedding_bwd");
}
