// Persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores.
//
//   C[M,N] (+)= A * B      fp32 accumulation in TMEM, bf16 or fp32 output
//
// Operand storage (each operand independently):
//   A "K-major":  A stored [M,K] row-major.      A "MN-major": A stored [K,M] row-major.
//   B "K-major":  B stored [N,K] row-major.      B "MN-major": B stored [K,N] row-major.
// so y = x W^T, dx = dy W and dW = dy^T x all run without a transpose pass.
//
// Structure of one CTA (192 threads, one CTA per SM, static round-robin tile schedule):
//   warp 0      TMA producer: cp.async.bulk.tensor tiles into a 128B-swizzled smem ring
//   warp 1      allocates TMEM; one lane issues tcgen05.mma and tcgen05.commit
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, convert, store to global
// Two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
// Takes the role of the cuBLAS calls behind nn.Linear in the reference
// (src/kohakuwullm/models/components/attention.py:77-89, mlp.py:15-126).
#include "common.cuh"

#include <cstdio>
#include <mutex>
#include <unordered_map>

namespace kwu {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  int ldc;
  int out_fp32;     // 0: bf16 output, 1: fp32 output
  int accumulate;   // 1: C += A*B (read-modify-write in the epilogue)
  float alpha;      // scale applied to the product
  // descriptor constants, computed on the host
  uint32_t a_lbo, a_sbo, a_kadv;
  uint32_t b_lbo, b_sbo, b_kadv;
  uint32_t idesc;
  int tiles_m, tiles_n;
  int* status;
  // split-K (group_mode 0 only): the contraction is cut into `splits` ranges handled by different CTAs,
  // each adding its partial product into the fp32 output with vector reductions (needs out_fp32 and
  // C += semantics). Used by weight gradients, whose outputs have too few tiles to fill the GPU.
  int splits;
  // stream-K (group_mode 0 only, fp32 C += semantics): the (tile, k-block) work units are cut into
  // `streamk` equal contiguous ranges, one per CTA; a CTA adds the partial product of every tile its range
  // touches into the output with vector reductions, so all SMs finish together whatever the tile count.
  int streamk;
  // grouped (mixture-of-experts) modes
  //   1: rows grouped by expert: row tile t reads group_tiles[t] = (m0, expert, valid); the expert picks
  //      a block of `group_b_rows` rows of B (K-major: output rows; MN-major: contraction rows)
  //   2: contraction grouped by expert (weight gradients): C[e] (+)= A[rows_e]^T B[rows_e] with
  //      rows_e = [group_offsets[e], group_offsets[e+1]); C advances by c_group_stride elements per expert
  int group_mode;
  const int4* group_tiles;
  const int* group_offsets;
  int group_b_rows;
  int num_groups;
  long long c_group_stride;
  // scatter epilogue (bf16 EPI_STORE only): output row r goes to the byte address row_ptrs[r] (0: row is
  // dropped) instead of C + r*ldc. The addresses may be peer-mapped memory of another GPU: the expert-
  // parallel combine / gradient return is then done by the GEMM's own epilogue stores, tile by tile.
  const long long* row_ptrs;
  // fused cross-entropy epilogues (EPI_LSE / EPI_DLOGITS)
  const int* labels;     // (M) target column per row, negative = ignored row
  float2* partial;       // EPI_LSE: (tiles_n, M) running (max, sum-exp) per row and column tile
  float* target_logit;   // EPI_LSE: (M) logit of the target column
  const float* lse;      // EPI_DLOGITS: (M) log-sum-exp of the full row
  const float* coef_p;   // EPI_DLOGITS: (M) factor on the probabilities
  const float* coef_y;   // EPI_DLOGITS: (M) factor on the one-hot target
};

constexpr int EPI_STORE = 0;    // C (+)= alpha * acc
constexpr int EPI_LSE = 1;      // no C: per-row (max, sum-exp) partials and the target logit
constexpr int EPI_DLOGITS = 2;  // C = coef_p * exp(acc - lse) - coef_y * onehot   (bf16)

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 256) ? 4 : ((BN >= 192) ? 5 : 6);
  static constexpr int BAR_BYTES = 1024;
  // per epilogue warp a 32 x 32 fp32 patch (rows padded to 36 floats) through which the fp32 reductions are
  // transposed, so that one warp instruction adds to 4 rows x 128 contiguous bytes instead of 32 rows x 16 bytes
  static constexpr int RED_STAGE_BYTES = 4 * 32 * 36 * 4;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + RED_STAGE_BYTES + 1024;  // +1024 alignment slack
};

struct TileInfo {
  int m0, n0;        // output tile origin
  int b_row_off;     // added to B's row coordinate (expert selection)
  int k_begin, nkb;  // contraction range in elements / 64-blocks
  long long c_off;   // added to the output pointer (elements)
};

constexpr int GEMM_RASTER_M = 16;

// Same decoding in every role of the CTA. Returns false for tiles that carry no work.
template <int BN>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, int tile, int num_kb, TileInfo& t) {
  t.b_row_off = 0; t.k_begin = 0; t.nkb = num_kb; t.c_off = 0;
  if (p.group_mode == 2) {
    const int per = p.tiles_m * p.tiles_n;
    const int e = tile / per, r = tile % per;
    t.m0 = (r / p.tiles_n) * GEMM_BM;
    t.n0 = (r % p.tiles_n) * BN;
    t.k_begin = p.group_offsets[e];
    t.nkb = (p.group_offsets[e + 1] - t.k_begin) / GEMM_BK;
    t.c_off = static_cast<long long>(e) * p.c_group_stride;
    return t.nkb > 0;
  }
  if (p.splits > 1) {
    const int per = p.tiles_m * p.tiles_n;
    const int sidx = tile / per;
    tile = tile % per;
    const int kb0 = static_cast<int>(static_cast<long long>(num_kb) * sidx / p.splits);
    const int kb1 = static_cast<int>(static_cast<long long>(num_kb) * (sidx + 1) / p.splits);
    t.k_begin = kb0 * GEMM_BK;
    t.nkb = kb1 - kb0;
  }
  if (p.group_mode == 1) {
    const int tm = tile / p.tiles_n;
    t.n0 = (tile % p.tiles_n) * BN;
    const int4 g = p.group_tiles[tm];
    t.m0 = g.x;
    t.b_row_off = g.y * p.group_b_rows;
    return g.z != 0;
  }
  // Raster order: panels of GEMM_RASTER_M row tiles, rows fastest inside a panel. The tiles that run at the
  // same time then share a few B tiles and one A panel, which stays in L2; with columns fastest every wave
  // of a wide product (a 65536-row vocabulary matrix) streams a different stretch of B from HBM for every
  // row tile, 32 times the matrix in total.
  const int span = GEMM_RASTER_M * p.tiles_n;
  const int panel = tile / span, within = tile - panel * span;
  const int gm = min(GEMM_RASTER_M, p.tiles_m - panel * GEMM_RASTER_M);
  t.m0 = (panel * GEMM_RASTER_M + within % gm) * GEMM_BM;
  t.n0 = (within / gm) * BN;
  return true;
}

// Work item number `i` of this CTA. 0: none left; 1: `t` holds work; 2: nothing to do for this index, go on.
template <int BN>
__device__ __forceinline__ int next_work(const GemmParams& p, int i, int num_tiles, int num_kb, TileInfo& t) {
  if (p.streamk > 0) {
    const long long units = static_cast<long long>(p.tiles_m) * p.tiles_n * num_kb;
    const long long u0 = units * blockIdx.x / p.streamk, u1 = units * (blockIdx.x + 1) / p.streamk;
    const long long tile = u0 / num_kb + i;
    const long long start = max(u0, tile * num_kb), end = min(u1, (tile + 1) * num_kb);
    if (start >= end) return 0;
    t.b_row_off = 0; t.c_off = 0;
    t.m0 = static_cast<int>(tile / p.tiles_n) * GEMM_BM;
    t.n0 = static_cast<int>(tile % p.tiles_n) * BN;
    t.k_begin = static_cast<int>(start - tile * num_kb) * GEMM_BK;
    t.nkb = static_cast<int>(end - start);
    return 1;
  }
  const int tile = blockIdx.x + i * gridDim.x;
  if (tile >= num_tiles) return 0;
  return decode_tile<BN>(p, tile, num_kb, t) ? 1 : 2;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 void* __restrict__ Cbase, const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 256) ? 256 : 512;

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
  float* red_stage = reinterpret_cast<float*>(bar_area + S::BAR_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n * (p.group_mode == 2 ? p.num_groups : 1) * (p.splits > 1 ? p.splits : 1);
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;

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
    // ------------------------------------------------------------ TMA producer
    // warp-uniform loop, one elected lane issues (coordinates, addresses and the tensor-map pointers stay
    // in uniform registers; the MN-major operands need up to six loads per k-block)
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int wi = 0; ok; ++wi) {
      TileInfo ti;
      const int got = next_work<BN>(p, wi, num_tiles, num_kb, ti);
      if (got == 0) break;
      if (got == 2) continue;
      const int m0 = ti.m0, n0 = ti.n0;
      for (int kb = 0; kb < ti.nkb; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY));
        if (!ok) break;
        uint8_t* sa = smem + stage * S::STAGE_BYTES;
        uint8_t* sb = sa + S::A_BYTES;
        const int k0 = ti.k_begin + kb * GEMM_BK;
        if (leader) {
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c)
              tma_load_2d(sa + c * 8192, &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0 + ti.b_row_off);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * 8192, &tmB, &full_bar[stage], n0 + c * 64, k0 + ti.b_row_off);
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
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop so that stage addresses, descriptors and counters stay warp-uniform
    // (a single-lane branch keeps them in per-thread registers and pays a move into the uniform registers
    // for every operand of every tcgen05.mma); one elected lane issues.
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    bool ok = true;
    // the descriptors of one k-block differ only in the address field: +(bytes >> 4) per 16-wide K step
    const uint32_t a_step = static_cast<uint32_t>(p.a_kadv) >> 4, b_step = static_cast<uint32_t>(p.b_kadv) >> 4;
    for (int wi = 0; ok; ++wi) {
      TileInfo ti;
      const int got = next_work<BN>(p, wi, num_tiles, num_kb, ti);
      if (got == 0) break;
      if (got == 2) continue;
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      ++it;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[as], aphase ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_EMPTY));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + as * BN;
      for (int kb = 0; kb < ti.nkb; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL));
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
        const uint64_t ad = make_smem_desc(sa, p.a_lbo, p.a_sbo, SWZ_128B);
        const uint64_t bd = make_smem_desc(sa + S::A_BYTES, p.b_lbo, p.b_sbo, SWZ_128B);
        const uint32_t acc0 = kb > 0 ? 1u : 0u;
        if (leader) {
          mma_f16_ss(d_tmem, ad, bd, p.idesc, acc0);
#pragma unroll
          for (int k = 1; k < GEMM_BK / 16; ++k) mma_f16_ss(d_tmem, ad + k * a_step, bd + k * b_step, p.idesc, 1u);
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
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int wi = 0; ok; ++wi) {
      TileInfo ti;
      const int got = next_work<BN>(p, wi, num_tiles, num_kb, ti);
      if (got == 0) break;
      if (got == 2) continue;
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      ++it;
      const int m0 = ti.m0, n0 = ti.n0;
      void* Cout = reinterpret_cast<uint8_t*>(Cbase) + ti.c_off * (p.out_fp32 ? 4 : 2);
      ok = mbar_wait(&acc_full[as], aphase, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);  // the TMEM loads below are warp-collective
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BN;
      // per-row state of the cross-entropy epilogues
      float run_max = -INFINITY, run_sum = 0.f, tgt = 0.f;
      bool tgt_here = false;
      int label = -1;
      float row_lse = 0.f, row_cp = 0.f, row_cy = 0.f;
      if (EPI != EPI_STORE && row < p.M) {
        label = p.labels ? p.labels[row] : -1;
        if (EPI == EPI_DLOGITS) {
          row_lse = p.lse[row];
          row_cp = p.coef_p[row];
          row_cy = p.coef_y[row];
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (EPI == EPI_LSE) {
          if (row < p.M && col0 < p.N) {
            // the column bound and the label only matter in one chunk of a row each: handled outside the
            // per-element loops, which are a scale, a maximum, and one fused multiply-add + exp2 per logit
            if (col0 + 32 > p.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j >= p.N) r[j] = __float_as_uint(-INFINITY);
            }
            if (label >= col0 && label < col0 + 32) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j == label) { tgt = __uint_as_float(r[j]) * p.alpha; tgt_here = true; }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], __uint_as_float(r[j]));
            // alpha > 0 commutes with the maximum
            const float cmax = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.alpha;
            const float nm = fmaxf(run_max, cmax);
            const float a2 = p.alpha * 1.4426950408889634f, nb = -nm * 1.4426950408889634f;
            const uint64_t a2p = pack_f32x2(a2, a2), nbp = pack_f32x2(nb, nb);
            uint64_t acc2[2] = {pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f)};
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float e0, e1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), a2p, nbp), e0, e1);
              acc2[(j >> 1) & 1] = add_f32x2(acc2[(j >> 1) & 1], pack_f32x2(fast_exp2(e0), fast_exp2(e1)));
            }
            float c0, c1, c2, c3;
            unpack_f32x2(acc2[0], c0, c1);
            unpack_f32x2(acc2[1], c2, c3);
            run_sum = run_sum * fast_exp2((run_max - nm) * 1.4426950408889634f) + ((c0 + c1) + (c2 + c3));
            run_max = nm;
          }
        } else if (EPI == EPI_DLOGITS) {
          if (row < p.M && col0 < p.N) {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * p.ldc + col0;
            float f[32];
            {
              // g = coef_p * exp2(acc * alpha * log2e - lse * log2e); the one-hot term is applied afterwards, in
              // the one chunk of the row that holds the label
              const float a2 = p.alpha * 1.4426950408889634f, nb = -row_lse * 1.4426950408889634f;
              const uint64_t a2p = pack_f32x2(a2, a2), nbp = pack_f32x2(nb, nb), cpp = pack_f32x2(row_cp, row_cp);
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                float e0, e1;
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), a2p, nbp), e0, e1);
                unpack_f32x2(mul_f32x2(pack_f32x2(fast_exp2(e0), fast_exp2(e1)), cpp), f[j], f[j + 1]);
              }
              if (label >= col0 && label < col0 + 32) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j == label) f[j] -= row_cy;
              }
            }
            if (col0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16(f[8 * j + 0], f[8 * j + 1]);
                v.y = pack_bf16(f[8 * j + 2], f[8 * j + 3]);
                v.z = pack_bf16(f[8 * j + 4], f[8 * j + 5]);
                v.w = pack_bf16(f[8 * j + 6], f[8 * j + 7]);
                reinterpret_cast<uint4*>(dst)[j] = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dst[j] = __float2bfloat16(f[j]);
            }
          }
        } else if (p.out_fp32 && (p.splits > 1 || p.streamk > 0 || (p.group_mode == 2 && p.accumulate))) {
          // Several CTAs add into the same tile (split-K, stream-K), or the tile is short in K and a
          // read-modify-write would leave the epilogue waiting on loads (per-expert weight gradients):
          // fire-and-forget vector reductions. The accumulator has one row per lane; the patch goes through
          // shared memory so that the lanes of one reduction instruction cover whole 128-byte row segments.
          if (col0 < p.N) {   // warp-uniform
            float* stg = red_stage + (warp - 2) * (32 * 36);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(stg + lane * 36 + 4 * j) =
                  make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                              __uint_as_float(r[4 * j + 2]) * p.alpha, __uint_as_float(r[4 * j + 3]) * p.alpha);
            __syncwarp();
            const int c4 = (lane & 7) * 4;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3);
              const int grow = m0 + quarter * 32 + rr;
              const float4 v = *reinterpret_cast<const float4*>(stg + rr * 36 + c4);
              if (grow < p.M) {
                float* dst = reinterpret_cast<float*>(Cout) + static_cast<size_t>(grow) * p.ldc + col0 + c4;
                if (col0 + c4 + 4 <= p.N) {
                  red_add_f32x4(dst, v.x, v.y, v.z, v.w);
                } else {
                  const float f[4] = {v.x, v.y, v.z, v.w};
                  for (int e = 0; e < 4; ++e)
                    if (col0 + c4 + e < p.N) atomicAdd(dst + e, f[e]);
                }
              }
            }
            __syncwarp();
          }
        } else if (row < p.M && col0 < p.N) {
          const bool full = (col0 + 32 <= p.N);
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(Cout) + static_cast<size_t>(row) * p.ldc + col0;
            if (full) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v;
                v.x = __uint_as_float(r[4 * j + 0]) * p.alpha;
                v.y = __uint_as_float(r[4 * j + 1]) * p.alpha;
                v.z = __uint_as_float(r[4 * j + 2]) * p.alpha;
                v.w = __uint_as_float(r[4 * j + 3]) * p.alpha;
                float4* d4 = reinterpret_cast<float4*>(dst) + j;
                if (p.accumulate) {
                  const float4 o = *d4;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *d4 = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float v = __uint_as_float(r[j]) * p.alpha;
                  if (p.accumulate) v += dst[j];
                  dst[j] = v;
                }
              }
            }
          } else {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * p.ldc + col0;
            if (p.row_ptrs) {
              const long long base = p.row_ptrs[row];
              if (!base) continue;
              dst = reinterpret_cast<__nv_bfloat16*>(base) + col0;
            }
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]) * p.alpha;
                uint4* d4 = reinterpret_cast<uint4*>(dst) + j;
                if (p.accumulate) {
                  const uint4 o = *d4;
                  const float2 o0 = unpack_bf16(o.x), o1 = unpack_bf16(o.y), o2 = unpack_bf16(o.z),
                               o3 = unpack_bf16(o.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                uint4 v;
                v.x = pack_bf16(f[0], f[1]);
                v.y = pack_bf16(f[2], f[3]);
                v.z = pack_bf16(f[4], f[5]);
                v.w = pack_bf16(f[6], f[7]);
                *d4 = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float v = __uint_as_float(r[j]) * p.alpha;
                  if (p.accumulate) v += __bfloat162float(dst[j]);
                  dst[j] = __float2bfloat16(v);
                }
              }
            }
          }
        }
      }
      if (EPI == EPI_LSE && row < p.M) {
        p.partial[static_cast<size_t>(n0 / BN) * p.M + row] = make_float2(run_max, run_sum);
        if (tgt_here) p.target_logit[row] = tgt;
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
    }
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the CTA's smem goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host launcher
static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

struct DescOverride {
  int active = 0;
  uint32_t a_lbo, a_sbo, a_kadv, b_lbo, b_sbo, b_kadv;
};
static DescOverride g_override;

struct GroupArgs {
  int mode = 0;
  const int4* tiles = nullptr;
  const int* offsets = nullptr;
  int b_rows = 0;
  int num_groups = 1;
  long long c_stride = 0;
  int row_tiles = 0;  // mode 1: number of entries in `tiles`
  const long long* row_ptrs = nullptr;
};

struct EpiArgs {
  const int* labels = nullptr;
  float2* partial = nullptr;
  float* target_logit = nullptr;
  const float* lse = nullptr;
  const float* coef_p = nullptr;
  const float* coef_y = nullptr;
};

template <int BN, bool A_MN, bool B_MN, int EPI = EPI_STORE>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                       int ldc, int out_fp32, int accumulate, float alpha, int max_ctas,
                       cudaStream_t stream, int* status, const EpiArgs& ea = EpiArgs(),
                       const GroupArgs& ga = GroupArgs(), int b_total_rows = 0, int splits = 1, bool streamk = false) {
  using S = GemmSmem<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = encode_tmap_2d(&tmA, A, ELEM_BF16, M, K, lda, GEMM_BM, GEMM_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = encode_tmap_2d(&tmA, A, ELEM_BF16, K, M, lda, GEMM_BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  // with expert groups B is the stack of all experts' matrices: b_total_rows rows in storage order
  if (!B_MN)
    rc = encode_tmap_2d(&tmB, B, ELEM_BF16, b_total_rows ? b_total_rows : N, K, ldb, BN, GEMM_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = encode_tmap_2d(&tmB, B, ELEM_BF16, b_total_rows ? b_total_rows : K, N, ldb, GEMM_BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha;
  // K-major, 128B swizzle: rows are 128 B, 8-row groups 1024 B apart, K advances 32 B per MMA.
  // MN-major, 128B swizzle: 64-element chunks along MN are whole 8 KB boxes, 8-row K groups are
  // 1024 B apart, K advances 16 rows = 2048 B per MMA.
  p.a_lbo = A_MN ? 8192 : 16; p.a_sbo = 1024; p.a_kadv = A_MN ? 2048 : 32;
  p.b_lbo = B_MN ? 8192 : 16; p.b_sbo = 1024; p.b_kadv = B_MN ? 2048 : 32;
  if (g_override.active) {
    if (A_MN) { p.a_lbo = g_override.a_lbo; p.a_sbo = g_override.a_sbo; p.a_kadv = g_override.a_kadv; }
    if (B_MN) { p.b_lbo = g_override.b_lbo; p.b_sbo = g_override.b_sbo; p.b_kadv = g_override.b_kadv; }
  }
  p.idesc = make_idesc_f16(GEMM_BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
  p.tiles_m = ga.mode == 1 ? ga.row_tiles : (M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.status = status;
  p.splits = (ga.mode == 0 && out_fp32 && accumulate) ? splits : 1;
  p.streamk = 0;
  p.group_mode = ga.mode; p.group_tiles = ga.tiles; p.group_offsets = ga.offsets;
  p.group_b_rows = ga.b_rows; p.num_groups = ga.num_groups; p.c_group_stride = ga.c_stride;
  p.row_ptrs = (EPI == EPI_STORE && !out_fp32) ? ga.row_ptrs : nullptr;
  p.labels = ea.labels; p.partial = ea.partial; p.target_logit = ea.target_logit;
  p.lse = ea.lse; p.coef_p = ea.coef_p; p.coef_y = ea.coef_y;

  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, EPI>;
  static PerDeviceOnce attr_set;
  if (attr_set.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) {
      set_last_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 10;
    }
    attr_set.mark();
  }
  long grid_l = static_cast<long>(p.tiles_m) * p.tiles_n * (ga.mode == 2 ? ga.num_groups : 1) * (p.splits > 1 ? p.splits : 1);
  int grid = grid_l > (1 << 30) ? (1 << 30) : static_cast<int>(grid_l);
  int cap = num_sms();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  if (streamk && ga.mode == 0 && out_fp32 && accumulate && EPI == EPI_STORE) {
    const long long units = static_cast<long long>(p.tiles_m) * p.tiles_n * ((K + GEMM_BK - 1) / GEMM_BK);
    grid = static_cast<int>(units < cap ? units : cap);
    p.splits = 1;
    p.streamk = grid;
  }
  launch_k(kern, dim3(grid), dim3(GEMM_THREADS), S::TOTAL, stream, tmA, tmB, C, p); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("gemm launch: %s", cudaGetErrorString(e));
    return 11;
  }
  return 0;
}

static int pick_bn(int M, int N, int forced) {
  if (forced == 128 || forced == 256) return forced;
  const int sms = num_sms();
  const int tm = (M + GEMM_BM - 1) / GEMM_BM;
  const long t256 = static_cast<long>(tm) * ((N + 255) / 256);
  const long t128 = static_cast<long>(tm) * ((N + 127) / 128);
  const long c256 = ((t256 + sms - 1) / sms) * 256;
  const long c128 = ((t128 + sms - 1) / sms) * 128;
  // a wide tile re-reads A half as often; prefer it unless the narrow one saves a real wave
  return (c128 * 100 < c256 * 92) ? 128 : 256;
}

}  // namespace kwu

// C[M,N] (+)= alpha * op(A) op(B). a_mn / b_mn select the storage described at the top of the file.
// lda/ldb/ldc are row pitches in elements of the STORED matrices. bn: 0 = choose, 128 or 256.
KWU_API int kwu_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                          int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, float alpha,
                          int bn, int max_ctas, void* stream, int* status) {
  using namespace kwu;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int BN = pick_bn(M, N, bn);
  int splits = 1;
  bool streamk = false;
  if (out_fp32 && accumulate && bn == 0 && K >= 1024) {
    // weight-gradient shape: few output tiles, long contraction, C += semantics. Wide tiles, and the
    // (tile, k-block) units are dealt out evenly over the SMs (stream-K) unless the tiles already fill
    // whole waves.
    const int sms = num_sms();
    const long t256 = static_cast<long>((M + GEMM_BM - 1) / GEMM_BM) * ((N + 255) / 256);
    BN = 256;
    streamk = (t256 % sms) != 0;
  }
#define KWU_GEMM_CASE(bnv, amn, bmn)                                                              \
  if (BN == bnv && a_mn == amn && b_mn == bmn)                                                    \
    return launch_gemm<bnv, amn != 0, bmn != 0>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32,        \
                                                accumulate, alpha, max_ctas, st, status, EpiArgs(), \
                                                GroupArgs(), 0, splits, streamk);
  KWU_GEMM_CASE(128, 0, 0) KWU_GEMM_CASE(128, 0, 1) KWU_GEMM_CASE(128, 1, 0) KWU_GEMM_CASE(128, 1, 1)
  KWU_GEMM_CASE(256, 0, 0) KWU_GEMM_CASE(256, 0, 1) KWU_GEMM_CASE(256, 1, 0) KWU_GEMM_CASE(256, 1, 1)
#undef KWU_GEMM_CASE
  set_last_error("kwu_gemm_bf16: unsupported variant");
  return 20;
}

// Test hook: override the MN-major descriptor constants (used once to pin the layout rules).
KWU_API void kwu_gemm_debug_override(int active, unsigned a_lbo, unsigned a_sbo, unsigned a_kadv,
                                     unsigned b_lbo, unsigned b_sbo, unsigned b_kadv) {
  kwu::g_override.active = active;
  kwu::g_override.a_lbo = a_lbo; kwu::g_override.a_sbo = a_sbo; kwu::g_override.a_kadv = a_kadv;
  kwu::g_override.b_lbo = b_lbo; kwu::g_override.b_sbo = b_sbo; kwu::g_override.b_kadv = b_kadv;
}


// ------------------------------------------------------------------ fused linear cross-entropy
// Forward: logits = alpha * h W^T are never written. Every (row, 256-column tile) leaves one
// (max, sum-exp) pair in partial[tile, row]; the target logit of each row is captured on the way.
// kwu_ce_combine then folds the partials into lse[row].
KWU_API int kwu_ce_tiles_n(int V) { return (V + 255) / 256; }

KWU_API int kwu_gemm_lse(const void* H, const void* W, int T, int V, int D, int ldh, int ldw,
                         const int* labels, void* partial, float* target_logit, float alpha,
                         void* stream, int* status) {
  using namespace kwu;
  if (T <= 0) return 0;
  EpiArgs ea;
  ea.labels = labels;
  ea.partial = reinterpret_cast<float2*>(partial);
  ea.target_logit = target_logit;
  return launch_gemm<256, false, false, EPI_LSE>(H, W, nullptr, T, V, D, ldh, ldw, 0, 0, 0, alpha, 0,
                                                 reinterpret_cast<cudaStream_t>(stream), status, ea);
}

// Backward recompute: dlogits[row, col] = coef_p[row] * exp(logit - lse[row]) - coef_y[row] * onehot,
// written as bf16 with row pitch ldd.
KWU_API int kwu_gemm_dlogits(const void* H, const void* W, void* dlogits, int T, int V, int D, int ldh,
                             int ldw, int ldd, const int* labels, const float* lse,
                             const float* coef_p, const float* coef_y, float alpha, void* stream,
                             int* status) {
  using namespace kwu;
  if (T <= 0) return 0;
  EpiArgs ea;
  ea.labels = labels;
  ea.lse = lse;
  ea.coef_p = coef_p;
  ea.coef_y = coef_y;
  return launch_gemm<256, false, false, EPI_DLOGITS>(H, W, dlogits, T, V, D, ldh, ldw, ldd, 0, 0, alpha,
                                                     0, reinterpret_cast<cudaStream_t>(stream), status, ea);
}

namespace kwu {
__global__ void ce_combine_kernel(const float2* __restrict__ partial, int tiles_n, int M,
                                  float* __restrict__ lse) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float m = -INFINITY, s = 0.f;
  for (int t = 0; t < tiles_n; ++t) {
    const float2 v = partial[static_cast<size_t>(t) * M + row];
    const float nm = fmaxf(m, v.x);
    s = s * __expf(m - nm) + v.y * __expf(v.x - nm);
    m = nm;
  }
  lse[row] = m + __logf(s);
}
}  // namespace kwu

KWU_API int kwu_ce_combine(const void* partial, int tiles_n, int M, float* lse, void* stream) {
  if (M <= 0) return 0;
  kwu::ce_combine_kernel<<<(M + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2*>(partial), tiles_n, M, lse); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { kwu::set_last_error("ce_combine launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}


// ------------------------------------------------------------------ grouped (mixture-of-experts) GEMMs
// Rows grouped by expert (forward and dgrad):  C[rows of tile] = A[rows of tile] * op(B[expert]).
//   A (M_pad, K) K-major. b_mn = 0: B is (E*N, K), expert e owns rows [e*N, (e+1)*N)  -> y = x W_e^T
//                         b_mn = 1: B is (E*Kc, N) with Kc = K,  expert e owns rows [e*K, (e+1)*K) -> dx = dy W_e
//   tiles: (row_tiles, 4) int32 entries (m0, expert, valid, unused) built by kwu_moe_plan.
//   row_ptrs (optional, bf16 output only): per output row the byte address it is stored at (0 = skip the row);
//   C is then not written.
KWU_API int kwu_gemm_bf16_grouped_rows(const void* A, const void* B, void* C, int M_pad, int N, int K, int lda,
                                       int ldb, int ldc, int b_mn, int num_experts, const void* tiles,
                                       int row_tiles, int out_fp32, const long long* row_ptrs, void* stream,
                                       int* status) {
  using namespace kwu;
  if (M_pad <= 0 || row_tiles <= 0) return 0;
  GroupArgs ga;
  ga.mode = 1;
  ga.row_ptrs = row_ptrs;
  ga.tiles = reinterpret_cast<const int4*>(tiles);
  ga.row_tiles = row_tiles;
  ga.b_rows = b_mn ? K : N;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int total_rows = num_experts * ga.b_rows;
  if (b_mn)
    return launch_gemm<128, false, true>(A, B, C, M_pad, N, K, lda, ldb, ldc, out_fp32, 0, 1.f, 0, st, status,
                                         EpiArgs(), ga, total_rows);
  return launch_gemm<128, false, false>(A, B, C, M_pad, N, K, lda, ldb, ldc, out_fp32, 0, 1.f, 0, st, status,
                                        EpiArgs(), ga, total_rows);
}

// Contraction grouped by expert (weight gradients): dW[e] (N_out, K_out) (+)= dY[rows_e]^T X[rows_e].
//   dY (M_pad, N_out) and X (M_pad, K_out) row-major; offsets: (E+1) padded row offsets (multiples of 128).
KWU_API int kwu_gemm_bf16_grouped_wgrad(const void* dY, const void* X, void* dW, int M_pad, int N_out, int K_out,
                                        int lddy, int ldx, int num_experts, const int* offsets, int out_fp32,
                                        int accumulate, void* stream, int* status) {
  using namespace kwu;
  if (M_pad <= 0) return 0;
  GroupArgs ga;
  ga.mode = 2;
  ga.offsets = offsets;
  ga.num_groups = num_experts;
  ga.c_stride = static_cast<long long>(N_out) * K_out;
  return launch_gemm<128, true, true>(dY, X, dW, N_out, K_out, M_pad, lddy, ldx, K_out, out_fp32, accumulate, 1.f,
                                      0, reinterpret_cast<cudaStream_t>(stream), status, EpiArgs(), ga, 0);
}
