// MXFP8: e4m3 values with one UE8M0 (power-of-two) scale per 32 elements along the contraction axis.
//
//   kwu_mxfp8_quantize     (M,K) bf16 -> (M,K) e4m3 + scales, blocks along K (rows stay rows)
//   kwu_mxfp8_quantize_t   (R,C) bf16 -> (C,R) e4m3 + scales, blocks along R: the transposed copy a
//                          dgrad needs (dx = dy W contracts over the rows of W)
//   kwu_gemm_mxfp8         C[M,N] (+)= A[M,K] B[N,K]^T with tcgen05.mma.kind::mxf8f6f4.block_scale
//
// Scale layout: the one the tensor core consumes from TMEM. For every 128-row x 128-column tile of
// the matrix there is one 512-byte chunk; inside it the scale of row r, 32-block j sits at byte
// (r % 32) * 16 + (r / 32) * 4 + j. Chunks are ordered [row_tile][k_chunk]. A chunk is moved
// global -> shared by one bulk copy and shared -> TMEM by one tcgen05.cp.32x128b.warpx4.
// Exponent rule: exp = max(ceil(log2(amax / 448)), -127) (round UP so nothing saturates), amax
// clamped at 1e-30, stored as exp + 127; values are divided by 2^exp and rounded to e4m3 (satfinite).
// Rows beyond M inside the last 128-row tile get the neutral scale byte 127 so that padded rows can
// never inject a NaN scale. Reference: src/kohakuwullm/kernels/mxfp8/quantize.py:39-215 and the
// cuBLASLt path behind src/kohakuwullm/kernels/mxfp8/linear.py:49-126.
#include "common.cuh"
#include "mx_quant.cuh"

namespace kwu {

// ------------------------------------------------------------------------------------ quantise
// One thread = 8 consecutive elements; 4 threads = one 32-block; a warp covers 256 columns of a row.
__global__ void __launch_bounds__(256)
mxfp8_quantize_kernel(const __nv_bfloat16* __restrict__ x, int ldx, uint8_t* __restrict__ q, int ldq,
                      uint8_t* __restrict__ sf, int M, int K, int M_pad, int sf_bn) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int lane = threadIdx.x & 31;
  const int n_kchunks = K >> 7;
  const int segs = (K + 255) >> 8;  // 256-column segments per row
  const long total = static_cast<long>(M_pad) * segs;
  const int wpb = blockDim.x >> 5;
  for (long w = static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5); w < total;
       w += static_cast<long>(gridDim.x) * wpb) {
    const int row = static_cast<int>(w / segs);
    const int col = static_cast<int>(w % segs) * 256 + lane * 8;
    const bool in_col = col < K;
    float f[8];
    if (row < M && in_col) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx + col);
      float2 t;
      t = unpack_bf16(a.x); f[0] = t.x; f[1] = t.y;
      t = unpack_bf16(a.y); f[2] = t.x; f[3] = t.y;
      t = unpack_bf16(a.z); f[4] = t.x; f[5] = t.y;
      t = unpack_bf16(a.w); f[6] = t.x; f[7] = t.y;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t e8 = (row < M) ? ue8m0_from_amax(amax) : 127u;
    if (in_col) {
      if (row < M) {
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
      }
      // tile-local layout (sf_bn > 128): only real rows are written, the buffer's padding keeps its neutral fill
      if ((lane & 3) == 0 && (sf_bn <= 128 || row < M))
        sf[sf_offset_any(row, col >> 5, n_kchunks, sf_bn)] = static_cast<uint8_t>(e8);
    }
  }
}

// Transposed quantise: input (R, C) row-major, output qT (C, R) with blocks of 32 along R.
// A block handles a 32 (rows) x 64 (cols) input tile: thread t < 64 owns column c0 + t.
__global__ void __launch_bounds__(64)
mxfp8_quantize_t_kernel(const __nv_bfloat16* __restrict__ x, int ldx, uint8_t* __restrict__ qT, int ldq,
                        uint8_t* __restrict__ sf, int R, int C, int C_pad, long long x_batch, long long q_batch,
                        long long sf_batch, int sf_bn) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  // blockIdx.z: independent matrices (the experts of a stacked weight) at fixed strides
  x += static_cast<size_t>(blockIdx.z) * x_batch;
  qT += static_cast<size_t>(blockIdx.z) * q_batch;
  sf += static_cast<size_t>(blockIdx.z) * sf_batch;
  const int r0 = blockIdx.y * 32;
  const int c = blockIdx.x * 64 + threadIdx.x;
  if (c >= C_pad) return;
  const int n_kchunks = (R + 127) >> 7;  // contraction axis of the output is R
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int r = r0 + i;
    v[i] = (r < R && c < C) ? __bfloat162float(x[static_cast<size_t>(r) * ldx + c]) : 0.f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  const uint32_t e8 = (c < C) ? ue8m0_from_amax(amax) : 127u;
  if (r0 < R && (sf_bn <= 128 || c < C)) sf[sf_offset_any(c, r0 >> 5, n_kchunks, sf_bn)] = static_cast<uint8_t>(e8);
  if (c < C) {
    const float inv = inv_scale_from_ue8m0(e8);
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_fp8x2_storage_t a2 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t b2 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      w[j] = static_cast<uint32_t>(a2) | (static_cast<uint32_t>(b2) << 16);
    }
    uint4* dst = reinterpret_cast<uint4*>(qT + static_cast<size_t>(c) * ldq + r0);
    if (r0 + 32 <= R) {
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
      uint8_t* d8 = qT + static_cast<size_t>(c) * ldq + r0;
      for (int i = 0; i < 32 && r0 + i < R; ++i) d8[i] = static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3)));
    }
  }
}

// ------------------------------------------------------------------------------------ GEMM
constexpr int MX_BM = 128;
constexpr int MX_BK = 128;  // 128 e4m3 = one 128-byte swizzle row = four K=32 MMAs = one scale chunk
constexpr int MX_THREADS = 192;

struct MxGemmParams {
  int M, N, K;
  int ldc;
  int out_fp32, accumulate;
  float alpha;
  const uint8_t* sfa;  // scale chunks of A: [ceil(M/128)][K/128][512]
  const uint8_t* sfb;  // scale chunks of B: [ceil(N/128)][K/128][512]
  int tiles_m, tiles_n;
  // grouped mode (rows of A grouped by expert): tile table entries (m0, expert, valid, 0); B holds the
  // experts' matrices stacked along its rows, `group_n` rows each (a multiple of 128)
  const int4* group_tiles;
  int group_n;
  int sfb_chunk_rows;  // number of 128-row scale chunks B has (chunk indices are clamped to it)
  int sfb_tiled;       // B scales are in the tile-local layout of mx_quant.cuh (two chunks per BN-row tile)
  const long long* row_ptrs;  // bf16 output: row r is stored at this byte address (0: dropped) instead of C + r*ldc
  int* status;
};

// Tile -> (A row offset, B row offset, output column offset); false: nothing to do for this entry.
__device__ __forceinline__ bool mx_decode_tile(const MxGemmParams& p, int tile, int BN, int& m0, int& n0, int& b_row0) {
  const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
  n0 = tn * BN;
  if (p.group_tiles) {
    const int4 t = p.group_tiles[tm];
    if (!t.z) return false;
    m0 = t.x;
    b_row0 = t.y * p.group_n + n0;
  } else {
    m0 = tm * MX_BM;
    b_row0 = n0;
  }
  return true;
}

template <int BN>
struct MxSmem {
  static constexpr int A_BYTES = MX_BM * MX_BK;
  static constexpr int B_BYTES = BN * MX_BK;
  // a tile whose width is not a multiple of 128 can start inside a scale chunk and then touches one more
  static constexpr int SFB_CHUNKS = (BN % 128 == 0) ? BN / 128 : BN / 128 + 1;
  static constexpr int SF_BYTES = 512 + SFB_CHUNKS * 512;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + (SF_BYTES + 1023) / 1024 * 1024;  // data + scale area
  // as many stages as fit under 227 KB of shared memory (with 2 KB of barriers and alignment slack), at most 6
  static constexpr int FIT = (227 * 1024 - 2048) / STAGE_BYTES;
  static constexpr int STAGES = FIT > 6 ? 6 : FIT;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + 1024;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

template <int BN>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  void* __restrict__ Cout, const MxGemmParams p) {
  using S = MxSmem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t SFA_COL = 2 * BN;
  constexpr uint32_t SFB_COL = 2 * BN + 4;
  static_assert(2 * BN + 4 + 4 * S::SFB_CHUNKS <= 512, "accumulators + scales must fit in TMEM");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bar_area = smem + STAGES * S::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = p.K / MX_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync();   // set-up above overlapped the previous kernel's tail; operands are read from here on

  if (warp == 0) {
    // warp-uniform loop, one elected lane issues (see the MMA warp below)
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m0, n0, b_row0;
      if (!mx_decode_tile(p, tile, BN, m0, n0, b_row0)) continue;
      const int tm = m0 / MX_BM;
      // scale chunks of this tile's rows: A rows [m0, m0+128) are row tile tm; B rows [n0, n0+BN)
      // start at 128-row tile n0/128 (BN is a multiple of 16, n0 may start mid-chunk only when
      // BN is not a multiple of 128: the chunk pair covering [n0, n0+BN) is loaded and the row
      // offset inside it is applied through the TMEM lane/column arithmetic below).
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY));
        if (!ok) break;
        uint8_t* sa = smem + stage * S::STAGE_BYTES;
        uint8_t* sb = sa + S::A_BYTES;
        uint8_t* ssf = sb + S::B_BYTES;
        if (leader) {
          mbar_expect_tx(&full_bar[stage], S::A_BYTES + S::B_BYTES + S::SF_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * MX_BK, m0);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * MX_BK, b_row0);
          bulk_load_1d(ssf, p.sfa + (static_cast<size_t>(tm) * num_kb + kb) * 512, 512, &full_bar[stage]);
          if (p.sfb_tiled) {
            // the tile's own pair of chunks, contiguous in global memory
            bulk_load_1d(ssf + 512, p.sfb + (static_cast<size_t>(n0 / BN) * num_kb + kb) * 1024, S::SFB_CHUNKS * 512,
                         &full_bar[stage]);
          } else
#pragma unroll
          for (int c = 0; c < S::SFB_CHUNKS; ++c) {
            // rows past the end of B belong to masked output columns: any valid chunk will do for them
            const int chunk = min(b_row0 / 128 + c, p.sfb_chunk_rows - 1);
            bulk_load_1d(ssf + 512 + c * 512, p.sfb + (static_cast<size_t>(chunk) * num_kb + kb) * 512, 512,
                         &full_bar[stage]);
          }
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop so that stage addresses, descriptors and counters stay warp-uniform (under
    // a single-lane branch every operand of every tcgen05 instruction is first moved from a per-thread to a
    // uniform register, and with 128-wide tiles the issue of 2-3 scale copies + 4 MMAs per k-block then takes
    // longer than their execution); one elected lane issues.
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m0, n0, b_row0;
      if (!mx_decode_tile(p, tile, BN, m0, n0, b_row0)) continue;
      // the tile's first B row sits (b_row0 % 128) / 32 columns into its first scale chunk
      const uint32_t sfb_off = p.sfb_tiled ? 0u : static_cast<uint32_t>((b_row0 & 127) >> 5);
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      ++it;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[as], aphase ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_EMPTY));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + as * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL));
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
        const uint32_t sb = sa + S::A_BYTES;
        const uint32_t ssf = sb + S::B_BYTES;
        const uint64_t ad = make_smem_desc(sa, 16, 1024, SWZ_128B);
        const uint64_t bd = make_smem_desc(sb, 16, 1024, SWZ_128B);
        const uint64_t sfd = make_smem_desc(ssf, 16, 128, SWZ_NONE);
        const uint32_t acc0 = kb > 0 ? 1u : 0u;
        if (leader) {
          // scale chunks: shared -> TMEM (32 rows x 16 B each, 8-row groups 128 B apart, no swizzle);
          // 512 bytes further in shared memory is +32 in the descriptor's address field
          tc_cp_32x128b_warpx4(tmem_base + SFA_COL, sfd);
#pragma unroll
          for (int c = 0; c < S::SFB_CHUNKS; ++c) tc_cp_32x128b_warpx4(tmem_base + SFB_COL + 4 * c, sfd + 32 * (c + 1));
          // 32 fp8 elements along K per instruction: +32 bytes = +2 in the address field
          mma_mxf8_ss(d_tmem, ad, bd, make_idesc_mxf8(MX_BM, BN, 0, 0), tmem_base + SFA_COL,
                      tmem_base + SFB_COL + sfb_off, acc0);
#pragma unroll
          for (int k = 1; k < MX_BK / 32; ++k)
            mma_mxf8_ss(d_tmem, ad + 2 * k, bd + 2 * k, make_idesc_mxf8(MX_BM, BN, k, k), tmem_base + SFA_COL,
                        tmem_base + SFB_COL + sfb_off, 1u);
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && leader) tc_commit(&acc_full[as]);
      __syncwarp();
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m0, n0, b_row0;
      if (!mx_decode_tile(p, tile, BN, m0, n0, b_row0)) continue;
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      ++it;
      ok = mbar_wait(&acc_full[as], aphase, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BN;
#pragma unroll 1
      for (int c = 0; c < (BN + 31) / 32; ++c) {
        uint32_t r[32];
        // a tile width that is an odd multiple of 16 ends in a 16-column chunk
        const int width = (BN % 32 != 0 && c == BN / 32) ? 16 : 32;
        if (width == 32) {
          tmem_ld_x32(t_row + c * 32, r);
        } else {
          tmem_ld_x16(t_row + c * 32, r);
#pragma unroll
          for (int j = 16; j < 32; ++j) r[j] = 0u;
        }
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        const int col_end = min(col0 + width, p.N);   // columns past the tile or the matrix are not stored
        if (row < p.M && col0 < col_end) {
          const bool full = (col_end - col0 == 32);
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(Cout) + static_cast<size_t>(row) * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (full || col0 + j < col_end) {
                float v = __uint_as_float(r[j]) * p.alpha;
                if (p.accumulate) v += dst[j];
                dst[j] = v;
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * p.ldc + col0;
            if (p.row_ptrs) {
              const long long base = p.row_ptrs[row];
              if (!base) continue;
              dst = reinterpret_cast<__nv_bfloat16*>(base) + col0;
            }
            const int nvec = (col_end - col0) >> 3;   // whole 8-column vectors (N and the tile edges are multiples of 8)
            if ((col_end - col0) % 8 == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (j < nvec) {
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]) * p.alpha;
                  uint4* d4 = reinterpret_cast<uint4*>(dst) + j;
                  if (p.accumulate) {
                    const uint4 o = *d4;
                    const float2 o0 = unpack_bf16(o.x), o1 = unpack_bf16(o.y), o2 = unpack_bf16(o.z), o3 = unpack_bf16(o.w);
                    f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                    f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                  }
                  *d4 = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < col_end) {
                  float v = __uint_as_float(r[j]) * p.alpha;
                  if (p.accumulate) v += __bfloat162float(dst[j]);
                  dst[j] = __float2bfloat16(v);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN>
static int launch_mx(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                     const uint8_t* sfa, const uint8_t* sfb, int out_fp32, int accumulate, float alpha,
                     cudaStream_t stream, int* status, const int4* group_tiles = nullptr, int n_group_tiles = 0,
                     int n_groups = 1, const long long* row_ptrs = nullptr, int sfb_tiled = 0) {
  using S = MxSmem<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = encode_tmap_2d(&tmA, A, ELEM_U8, M, K, lda, MX_BM, MX_BK, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_tmap_2d(&tmB, B, ELEM_U8, static_cast<long long>(N) * n_groups, K, ldb, BN, MX_BK,
                           CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  MxGemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha;
  p.sfa = sfa; p.sfb = sfb;
  p.tiles_m = group_tiles ? n_group_tiles : (M + MX_BM - 1) / MX_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_tiles = group_tiles;
  p.group_n = N;
  p.sfb_chunk_rows = static_cast<int>((static_cast<long long>(N) * n_groups + 127) / 128);
  p.row_ptrs = out_fp32 ? nullptr : row_ptrs;
  p.sfb_tiled = sfb_tiled;
  p.status = status;
  auto kern = gemm_mxfp8_kernel<BN>;
  static PerDeviceOnce attr_set;
  if (attr_set.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) { set_last_error("gemm_mxfp8 attr: %s", cudaGetErrorString(e)); return 10; }
    attr_set.mark();
  }
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = p.tiles_m * p.tiles_n;
  if (grid > sms) grid = sms;
  launch_k(kern, dim3(grid), dim3(MX_THREADS), S::TOTAL, stream, tmA, tmB, C, p); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("gemm_mxfp8 launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

// Tile width. 128 works with the plain scale layout (a tile always starts on a chunk boundary). Wider tiles
// (multiples of 16 up to 240: two accumulators plus the scale columns must fit in 512 TMEM columns) need the B
// operand's scales in the tile-local layout, which only an operand quantised for that width has (weights).
// Why wider: per 128-deep k-block a 128 x BN tile moves 16 KB + BN * 128 B through shared memory for
// 128 * BN * 128 multiply-adds, and the kernel is bound by that traffic, so the cost per output column falls
// from 0.25 (BN 128) to 0.196 (BN 224); and the width can be chosen so that the tile count fills whole waves
// of SMs (4096 x 1280: 320 tiles of 128 = 2.16 waves -> 3 rounds; 288 tiles of 144 = 1.95 waves -> 2 rounds).
// A variant that kept the plain layout and offset the scale address by (first row % 128) / 32 TMEM columns
// faulted ("misaligned address") at width 160, where that offset is odd; width 192 (offsets 0 and 2) ran
// correctly, so odd column offsets of the scale address are the cause, and no path here uses an offset.
static bool bn_supported(int bn) { return bn == 128 || (bn > 128 && bn <= 240 && bn % 16 == 0); }

}  // namespace kwu

using namespace kwu;

// Bytes of the scale buffer of a (rows, K) operand.
KWU_API long long kwu_mxfp8_sf_bytes(int rows, int K) {
  return static_cast<long long>((rows + 127) / 128) * (K / 128) * 512;
}

KWU_API int kwu_mxfp8_quantize(const void* x, int ldx, void* q, int ldq, void* sf, int M, int K, void* stream) {
  if (K % 128) { set_last_error("mxfp8_quantize: K must be a multiple of 128 (got %d)", K); return 7; }
  if (M <= 0) return 0;
  const int M_pad = (M + 127) / 128 * 128;
  long warps = static_cast<long>(M_pad) * ((K + 255) / 256);
  long grid = (warps + 7) / 8;
  if (grid > 148 * 16) grid = 148 * 16;
  launch_k(mxfp8_quantize_kernel, dim3(static_cast<int>(grid)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (uint8_t*)sf, M, K, M_pad, 0); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_quantize launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

// x (R, C) -> qT (C, R) quantised along R; sf has kwu_mxfp8_sf_bytes(C, R) bytes. R % 128 == 0.
KWU_API int kwu_mxfp8_quantize_t(const void* x, int ldx, void* qT, int ldq, void* sf, int R, int C, void* stream) {
  if (R % 128) { set_last_error("mxfp8_quantize_t: R must be a multiple of 128 (got %d)", R); return 7; }
  if (C <= 0) return 0;
  const int C_pad = (C + 127) / 128 * 128;
  dim3 grid((C_pad + 63) / 64, R / 32);
  launch_k(mxfp8_quantize_t_kernel, dim3(grid), dim3(64), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)x, ldx, (uint8_t*)qT, ldq, (uint8_t*)sf, R, C, C_pad, 0, 0, 0, 0); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_quantize_t launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

// Weight forms: as kwu_mxfp8_quantize / kwu_mxfp8_quantize_t, with the scales in the tile-local layout for GEMM
// tiles `sf_bn` rows wide (sf_bn <= 128: plain layout). The scale buffer has kwu_mxfp8_sf_bytes_tiled bytes and
// must be pre-filled with the neutral byte 127: only the scales of real rows are written.
KWU_API long long kwu_mxfp8_sf_bytes_tiled(int rows, int K, int sf_bn) {
  if (sf_bn <= 128) return kwu_mxfp8_sf_bytes(rows, K);
  return static_cast<long long>((rows + sf_bn - 1) / sf_bn) * (K / 128) * 1024;
}

KWU_API int kwu_mxfp8_quantize_w(const void* x, int ldx, void* q, int ldq, void* sf, int M, int K, int sf_bn,
                                 void* stream) {
  if (K % 128) { set_last_error("mxfp8_quantize_w: K must be a multiple of 128 (got %d)", K); return 7; }
  if (!bn_supported(sf_bn)) { set_last_error("mxfp8_quantize_w: unsupported tile width %d", sf_bn); return 7; }
  if (M <= 0) return 0;
  const int M_pad = (M + 127) / 128 * 128;
  long warps = static_cast<long>(M_pad) * ((K + 255) / 256);
  long grid = (warps + 7) / 8;
  if (grid > 148 * 16) grid = 148 * 16;
  launch_k(mxfp8_quantize_kernel, dim3(static_cast<int>(grid)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (uint8_t*)sf, M, K, M_pad, sf_bn); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_quantize_w launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

KWU_API int kwu_mxfp8_quantize_t_w(const void* x, int ldx, void* qT, int ldq, void* sf, int R, int C, int sf_bn,
                                   void* stream) {
  if (R % 128) { set_last_error("mxfp8_quantize_t_w: R must be a multiple of 128 (got %d)", R); return 7; }
  if (!bn_supported(sf_bn)) { set_last_error("mxfp8_quantize_t_w: unsupported tile width %d", sf_bn); return 7; }
  if (C <= 0) return 0;
  const int C_pad = (C + 127) / 128 * 128;
  dim3 grid((C_pad + 63) / 64, R / 32);
  launch_k(mxfp8_quantize_t_kernel, dim3(grid), dim3(64), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)x, ldx, (uint8_t*)qT, ldq, (uint8_t*)sf, R, C, C_pad, 0, 0, 0, sf_bn); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_quantize_t_w launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

// `batch` matrices x[b] (R, C) at stride R*ldx -> qT[b] (C, R) at stride C*ldq, scale buffers at stride
// kwu_mxfp8_sf_bytes(C, R). C must be a multiple of 128 so that the stacked outputs stay chunk-aligned.
KWU_API int kwu_mxfp8_quantize_t_batched(const void* x, int ldx, void* qT, int ldq, void* sf, int R, int C, int batch,
                                         void* stream) {
  if (R % 128 || C % 128) { set_last_error("mxfp8_quantize_t_batched: R and C must be multiples of 128"); return 7; }
  if (batch <= 0) return 0;
  dim3 grid(C / 64, R / 32, batch);
  launch_k(mxfp8_quantize_t_kernel, dim3(grid), dim3(64), 0, reinterpret_cast<cudaStream_t>(stream), 
      (const __nv_bfloat16*)x, ldx, (uint8_t*)qT, ldq, (uint8_t*)sf, R, C, C, static_cast<long long>(R) * ldx,
      static_cast<long long>(C) * ldq, kwu_mxfp8_sf_bytes(C, R), 0); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_quantize_t_batched launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

// Grouped form: rows of A are grouped by expert in 128-row-aligned ranges described by `tiles`
// ((m0, expert, valid, 0) per 128-row tile); B stacks the experts' (N, K) matrices along its rows.
// out[rows of expert e] = A[rows] B[e]^T. N must be a multiple of 128.
// row_ptrs (optional): per output row the byte address it is stored at (0 = skip); C is then not written.
KWU_API int kwu_gemm_mxfp8_grouped(const void* A, const void* sfa, const void* B, const void* sfb, void* C,
                                   int M, int N, int K, int lda, int ldb, int ldc, int n_experts,
                                   const void* tiles, int n_tiles, const long long* row_ptrs, void* stream,
                                   int* status) {
  if (M <= 0 || N <= 0 || n_tiles <= 0) return 0;
  if (K % 128 || N % 128) { set_last_error("gemm_mxfp8_grouped: K and N must be multiples of 128 (got %d, %d)", K, N); return 7; }
  return launch_mx<128>(A, B, C, M, N, K, lda, ldb, ldc, (const uint8_t*)sfa, (const uint8_t*)sfb, 0, 0, 1.f,
                        reinterpret_cast<cudaStream_t>(stream), status, reinterpret_cast<const int4*>(tiles),
                        n_tiles, n_experts, row_ptrs);
}

KWU_API int kwu_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M,
                           int N, int K, int lda, int ldb, int ldc, int out_fp32, int accumulate,
                           float alpha, int bn, void* stream, int* status) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128) { set_last_error("gemm_mxfp8: K must be a multiple of 128 (got %d)", K); return 7; }
  if (bn <= 0) bn = 128;
  if (!bn_supported(bn)) { set_last_error("gemm_mxfp8: tile width %d is not 128 or a multiple of 16 in (128, 240]", bn); return 7; }
#define KWU_MX_CASE(W)                                                                                              \
  case W:                                                                                                           \
    return launch_mx<W>(A, B, C, M, N, K, lda, ldb, ldc, (const uint8_t*)sfa, (const uint8_t*)sfb, out_fp32,        \
                        accumulate, alpha, reinterpret_cast<cudaStream_t>(stream), status, nullptr, 0, 1, nullptr, \
                        W > 128 ? 1 : 0)
  switch (bn) {
    KWU_MX_CASE(128); KWU_MX_CASE(144); KWU_MX_CASE(160); KWU_MX_CASE(176); KWU_MX_CASE(192);
    KWU_MX_CASE(208); KWU_MX_CASE(224); KWU_MX_CASE(240);
  }
#undef KWU_MX_CASE
  return 7;
}

// ------------------------------------------------------------------------------------ attention operands
// Per-head MXFP8 quantisation of q / k for attention (head_dim 64 = two 32-blocks per (token, head) row):
//   mxfp8_column_mean   mu[h, d] = mean over the T tokens of the pack of x[t, h, d]  (key smoothing: scores
//                       change by q . mu, a constant along the key axis, which softmax ignores)
//   mxfp8_quant_heads   x[t, h, :] (- mu[h, :]) -> e4m3 bytes + two UE8M0 scale bytes per row, and the
//                       dequantised bf16 copy (e4m3 x 2^e is exact in bf16) that the attention kernels read.
// Reference: src/kohakuwullm/kernels/mxfp8/attention_quant.py:17-78.
namespace kwu {

__global__ void __launch_bounds__(256)
mxfp8_column_mean_kernel(const __nv_bfloat16* __restrict__ x, long long ld_t, int T, int H, float* __restrict__ mu) {
  // block = one head; thread = (channel d = tid % 64, token lane = tid / 64)
  __shared__ float s_part[4][64];
  const int h = blockIdx.x, d = threadIdx.x & 63, tl = threadIdx.x >> 6;
  float acc = 0.f;
  for (int t = tl; t < T; t += 4) acc += __bfloat162float(x[static_cast<size_t>(t) * ld_t + h * 64 + d]);
  s_part[tl][d] = acc;
  __syncthreads();
  if (tl == 0) mu[h * 64 + d] = (s_part[0][d] + s_part[1][d] + s_part[2][d] + s_part[3][d]) / static_cast<float>(T);
}

// One lane = 8 channels; 8 lanes = one (token, head) row; a warp covers 4 rows.
__global__ void __launch_bounds__(256)
mxfp8_quant_heads_kernel(const __nv_bfloat16* __restrict__ x, long long ld_t, const float* __restrict__ mu,
                         uint8_t* __restrict__ q8, uint8_t* __restrict__ sf, __nv_bfloat16* __restrict__ deq,
                         long long rows, int H) {
  const int lane = threadIdx.x & 31;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r0 = wid * 4; r0 < rows; r0 += nwarps * 4) {
    const long long row = r0 + (lane >> 3);
    const int c = (lane & 7) * 8;
    const bool in = row < rows;
    const long long t = in ? row / H : 0;
    const int h = in ? static_cast<int>(row % H) : 0;
    float f[8];
    if (in) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ld_t + h * 64 + c);
      unpack8(a, f);
      if (mu) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] -= mu[h * 64 + c + e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!in) continue;
    const uint32_t e8 = ue8m0_from_amax(amax);
    const float inv = inv_scale_from_ue8m0(e8);
    const float scale = __uint_as_float(e8 << 23);  // 2^(e8 - 127); e8 >= 1 here because amax >= 1e-30
    uint32_t lo = 0, hi = 0;
    float d[8];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const __nv_fp8x2_storage_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(f[e] * inv, f[e + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p2, __NV_E4M3);
      const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      d[e] = back.x * scale;
      d[e + 1] = back.y * scale;
      if (e < 4) lo |= static_cast<uint32_t>(p2) << (8 * e);
      else hi |= static_cast<uint32_t>(p2) << (8 * (e - 4));
    }
    if (q8) *reinterpret_cast<uint2*>(q8 + static_cast<size_t>(row) * 64 + c) = make_uint2(lo, hi);
    if (sf && (lane & 3) == 0) sf[static_cast<size_t>(row) * 2 + (c >> 5)] = static_cast<uint8_t>(e8);
    *reinterpret_cast<uint4*>(deq + static_cast<size_t>(row) * 64 + c) =
        make_uint4(pack_bf16(d[0], d[1]), pack_bf16(d[2], d[3]), pack_bf16(d[4], d[5]), pack_bf16(d[6], d[7]));
  }
}

}  // namespace kwu

// x: (T, H, 64) bf16 view with token pitch ld_t elements (heads contiguous). mu: (H, 64) fp32 out.
KWU_API int kwu_mxfp8_column_mean(const void* x, long long ld_t, int T, int H, float* mu, void* stream) {
  if (T <= 0 || H <= 0) return 0;
  mxfp8_column_mean_kernel<<<H, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((const __nv_bfloat16*)x, ld_t, T, H, mu); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_column_mean launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

// q8 (T,H,64) bytes and sf (T,H,2) bytes are optional; deq (T,H,64) bf16 contiguous is always written.
KWU_API int kwu_mxfp8_quant_heads(const void* x, long long ld_t, const float* mu, void* q8, void* sf, void* deq, int T,
                                  int H, void* stream) {
  if (T <= 0 || H <= 0) return 0;
  const long long rows = static_cast<long long>(T) * H;
  long long grid = (rows + 31) / 32;
  if (grid > 148 * 16) grid = 148 * 16;
  mxfp8_quant_heads_kernel<<<static_cast<int>(grid), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, ld_t, mu, (uint8_t*)q8, (uint8_t*)sf, (__nv_bfloat16*)deq, rows, H); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("mxfp8_quant_heads launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}
