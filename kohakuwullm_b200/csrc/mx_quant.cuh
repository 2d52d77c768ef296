// MXFP8 quantisation helpers shared by the stand-alone quantise kernels and by producers that emit the
// fp8 copy of their output directly (RMSNorm, SwiGLU). Rule and layout are described in mxfp8.cu.
#pragma once
#include "common.cuh"

namespace kwu {

__device__ __forceinline__ uint32_t ue8m0_from_amax(float amax) {
  amax = fmaxf(amax, 1e-30f);
  const float v = amax * (1.0f / 448.0f);
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = (bits >> 23) & 0xffu;
  if (bits & 0x7fffffu) e += 1;  // ceil(log2(v))
  return min(e, 254u);
}
__device__ __forceinline__ float inv_scale_from_ue8m0(uint32_t e) {
  // 2^-(e-127) = 2^(127-e): biased exponent 254 - e (e = 254 would be a denormal; clamp)
  const uint32_t be = (e >= 254u) ? 1u : (254u - e);
  return __uint_as_float(be << 23);
}
__device__ __forceinline__ size_t sf_offset(int row, int kblock, int n_kchunks) {
  const int rt = row >> 7, r = row & 127;
  return (static_cast<size_t>(rt) * n_kchunks + (kblock >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 +
         (kblock & 3);
}

// Tile-local scale layout of a B operand (a weight) whose GEMM tiles are `bn` rows wide, bn in (128, 256]: the
// rows [tile * bn, (tile + 1) * bn) of the matrix own TWO consecutive 512-byte chunks per 128-column k-chunk
// (rows 0..127 of the tile in the first, rows 128..bn-1 in the second), ordered [tile][k_chunk][2]. A tile's
// scales then always start at TMEM column 0 of the scale area, whatever bn is (with the plain 128-row chunks
// a tile that starts inside a chunk needs a column offset, and odd offsets are not addressable).
__device__ __forceinline__ size_t sf_offset_tiled(int row, int kblock, int n_kchunks, int bn) {
  const int tile = row / bn, r = row - tile * bn;
  return ((static_cast<size_t>(tile) * n_kchunks + (kblock >> 2)) * 2 + (r >> 7)) * 512 + (r & 31) * 16 +
         ((r & 127) >> 5) * 4 + (kblock & 3);
}
__device__ __forceinline__ size_t sf_offset_any(int row, int kblock, int n_kchunks, int bn) {
  return bn > 128 ? sf_offset_tiled(row, kblock, n_kchunks, bn) : sf_offset(row, kblock, n_kchunks);
}

// Eight consecutive values of one row held by this lane; the aligned group of four lanes holds one
// 32-element block. Every lane of the warp must call this (the block maximum is formed with shuffles);
// lanes whose `active` is false contribute zeros and store nothing. `col` is the first of the 8 columns.
__device__ __forceinline__ void mx_emit8(const float (&f)[8], bool active, int row, int col, uint8_t* __restrict__ q,
                                         int ldq, uint8_t* __restrict__ sf, int n_kchunks) {
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, active ? fabsf(f[e]) : 0.f);
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!active) return;
  const uint32_t e8 = ue8m0_from_amax(amax);
  const float inv = inv_scale_from_ue8m0(e8);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int e = 0; e < 4; e += 2) {
    const __nv_fp8x2_storage_t a2 = __nv_cvt_float2_to_fp8x2(make_float2(f[e] * inv, f[e + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t b2 = __nv_cvt_float2_to_fp8x2(make_float2(f[e + 4] * inv, f[e + 5] * inv), __NV_SATFINITE, __NV_E4M3);
    lo |= static_cast<uint32_t>(a2) << (8 * e);
    hi |= static_cast<uint32_t>(b2) << (8 * e);
  }
  *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * ldq + col) = make_uint2(lo, hi);
  if ((threadIdx.x & 3) == 0) sf[sf_offset(row, col >> 5, n_kchunks)] = static_cast<uint8_t>(e8);
}

// Values of a packed bf16x8 vector as floats (what a later quantise pass of the stored tensor would see).
__device__ __forceinline__ void unpack8(const uint4& a, float (&f)[8]) {
  float2 t;
  t = unpack_bf16(a.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16(a.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16(a.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16(a.w); f[6] = t.x; f[7] = t.y;
}

struct MxOut {
  uint8_t* q;   // (rows, ldq) e4m3 bytes, null: no emission
  int ldq;
  uint8_t* sf;  // scale chunks of a (rows, cols) operand
  int n_kchunks;
};

}  // namespace kwu
