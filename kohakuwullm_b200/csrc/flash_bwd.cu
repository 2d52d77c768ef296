// Varlen causal / sliding-window flash attention backward for head_dim 64, bf16, on tcgen05.
//
// Three launches, no atomics, deterministic:
//   1. delta[h,t] = sum_d out[t,h,d] * dout[t,h,d]
//   2. dK/dV kernel: persistent CTAs over (128-key tile, query head) items. Scores are formed TRANSPOSED
//      (S^T = K Q^T, dP^T = V dO^T, keys on the TMEM lanes) so that P^T and dS^T are directly the
//      A operands of dV += P^T dO and dK += dS^T Q. The CTA loops over every query head of its GQA
//      group and every 64-query tile that can see the key tile, accumulating in TMEM.
//   3. dQ kernel: persistent CTAs over (128-query tile, query head) items, each looping over 64-key tiles:
//      S = Q K^T, dP = dO V^T, dS = P o (dP - delta) * scale written to TMEM as bf16,
//      dQ += dS K accumulated in TMEM.
// The stored lse already contains the sink term, so P = exp(S*scale - lse) is the sink-aware
// probability and nothing else changes (sink columns carry a zero value).
// Replaces src/kohakuwullm/kernels/attention/flash_attn_bwd.py:16-348 of the reference (which
// accumulates GQA groups with fp32 atomics).
#include "common.cuh"

namespace kwu {

constexpr int FB_D = 64;
constexpr int FB_THREADS = 320;  // 8 softmax warps (two per TMEM lane quarter) + TMA warp + MMA warp
constexpr float FB_LOG2E = 1.4426950408889634f;
template <bool V> struct BoolC { static constexpr bool value = V; };   // compile-time switch for the tile bodies

// ------------------------------------------------------------------------------------ delta
__global__ void __launch_bounds__(256)
flash_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                   float* __restrict__ delta, int T, int Hq) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  // eight lanes per (t, h) row of 64 (one 16-byte load of each operand per lane), four rows per warp pass
  const int lane = threadIdx.x & 31, sub = lane & 7, slot = lane >> 3;
  const long total = static_cast<long>(T) * Hq;
  const int wpb = blockDim.x >> 5;
  for (long r0 = (static_cast<long>(blockIdx.x) * wpb + (threadIdx.x >> 5)) * 4; r0 < total;
       r0 += static_cast<long>(gridDim.x) * wpb * 4) {
    const long r = r0 + slot;
    float s = 0.f;
    if (r < total) {
      const uint4 a = reinterpret_cast<const uint4*>(out + r * 64)[sub];
      const uint4 b = reinterpret_cast<const uint4*>(dout + r * 64)[sub];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = unpack_bf16(aw[i]), fb = unpack_bf16(bw[i]);
        s += fa.x * fb.x + fa.y * fb.y;
      }
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (sub == 0 && r < total) {
      const int t = static_cast<int>(r / Hq), h = static_cast<int>(r % Hq);
      delta[static_cast<size_t>(h) * T + t] = s;
    }
  }
}

struct FlashBwdParams {
  const float* lse;     // (Hq, T), natural log, sink term included
  const float* delta;   // (Hq, T)
  __nv_bfloat16* dq;    // (T, Hq, 64)
  __nv_bfloat16* dk;    // (T, Hkv, 64)
  __nv_bfloat16* dv;    // (T, Hkv, 64)
  float* dk_part;       // (T, Hq, 64) per-query-head partials when Hq > Hkv, else null
  float* dv_part;
  const int4* plan;
  int n_tiles;
  int dk_ld, dv_ld;     // row pitch (elements per token) of dk / dv, so they can land inside a fused dqkv buffer
  int T, Hq, Hkv, window;
  float scale;
  int* status;
};

// ------------------------------------------------------------------------------------ dK / dV
// smem: 2 x K tile 16 KB, V tile 16 KB, 3 stages x (Q 8 KB + dO 8 KB).
// Persistent: a CTA walks items (key tile, query head) blockIdx.x, blockIdx.x + gridDim.x, ...; barrier
// phases run on counters that continue across items, and the producer warp loads the next item's K / V
// and first Q / dO tiles while the current item's accumulators are being written out.
// Inside an item the score product of query tile i + 1 is issued right after dV of tile i (the softmax warps
// keep P in registers for their second phase, so the score columns are free by then): the softmax warps find
// the next scores ready when they finish a tile instead of waiting for a product that starts only then.
// At an item boundary the chain used to be: last dK done -> K / V of the next item loaded -> first S -> softmax
// (about 7000 cycles on a CTA that spends 3300 per tile, so short documents paid more for the boundary than
// for their tiles). K is double-buffered and loaded during the previous item, the item's first Q / dO tile is
// loaded before its V, so the first S of an item is issued the moment the previous item's products are out,
// and V (needed only for dP, one softmax phase later) arrives under that first phase.
constexpr int FBK_STAGES = 3;
constexpr int FBK_SMEM = 3 * 16384 + FBK_STAGES * 16384 + 2048 + 1024 + 1024;

struct DkdvItem {
  int kv0, de, h, hk, q_begin, q_end, n_it;
};

__device__ __forceinline__ bool dkdv_decode(const FlashBwdParams& p, int item, DkdvItem& it) {
  const int4 job = p.plan[p.n_tiles + item / p.Hq];   // second list: key tiles seen by the most queries first
  if (!job.w) return false;
  it.kv0 = job.x; it.de = job.z;
  it.h = item % p.Hq;                      // one item per query head; GQA partials are summed afterwards
  it.hk = it.h / (p.Hq / p.Hkv);
  it.q_begin = it.kv0;
  it.q_end = it.de;
  if (p.window > 0) it.q_end = min(it.de, it.kv0 + 127 + p.window);
  it.n_it = (it.q_end - it.q_begin + 63) / 64;
  return it.n_it > 0;
}

__global__ void __launch_bounds__(FB_THREADS, 2)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmDO64,
                      const __grid_constant__ CUtensorMap tmK128, const __grid_constant__ CUtensorMap tmV128,
                      const FlashBwdParams p) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;                                // 2 x 16 KB: item n in buffer n & 1
  uint8_t* sV = smem + 32768;
  uint8_t* sQ = smem + 49152;                        // FBK_STAGES x 8 KB
  uint8_t* sDO = smem + 49152 + FBK_STAGES * 8192;   // FBK_STAGES x 8 KB
  float* sLse = reinterpret_cast<float*>(smem + 49152 + FBK_STAGES * 16384);   // per stage 64: -lse * log2(e)
  float* sDelta = sLse + FBK_STAGES * 64;                                      // per stage 64: -delta * scale
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 49152 + FBK_STAGES * 16384 + 2048);
  uint64_t* k_full = bars + 0;    // [2]
  uint64_t* k_empty = bars + 2;   // [2] the item's last products have read this K buffer
  uint64_t* qd_full = bars + 4;   // [3]
  uint64_t* qd_empty = bars + 7;  // [3]
  uint64_t* sdp_full = bars + 10;
  uint64_t* p_ready = bars + 11;
  uint64_t* acc_done = bars + 12;
  uint64_t* v_full = bars + 13;
  uint64_t* v_empty = bars + 14;   // the item's last products have read V
  uint64_t* acc_free = bars + 15;  // the item's dK / dV accumulators have been read out
  uint64_t* dp_full = bars + 16;   // dP^T is in TMEM (S^T has its own barrier, so the exponentials start earlier)
  uint64_t* ds_ready = bars + 17;  // dS^T has been written (P^T has its own barrier, so dV starts earlier)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_items = p.n_tiles * p.Hq;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    for (int s = 0; s < FBK_STAGES; ++s) {
      mbar_init(&qd_full[s], 1);
      mbar_init(&qd_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(dp_full, 1);
    mbar_init(ds_ready, 256);
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 256);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 64, tDV = tmem_base + 128, tDK = tmem_base + 192;
  // the next item of this CTA at or after round `rnd` (rounds whose slot is empty or past the list are skipped)
  auto next_item = [&](int& rnd, DkdvItem& it) -> bool {
    for (; rnd * static_cast<int>(gridDim.x) < n_items; ++rnd) {
      const int item = snake_item(rnd);
      if (item < n_items && dkdv_decode(p, item, it)) {
        ++rnd;
        return true;
      }
    }
    return false;
  };

  if (warp == 8) {
    int g = 0, ic = 0, rnd = 0;
    int ok = 1;
    DkdvItem it, nx;
    bool have = next_item(rnd, it);
    auto load_k = [&](const DkdvItem& d, int n) {   // lane 0: K of the CTA's n-th item into buffer n & 1
      if (!mbar_wait(&k_empty[n & 1], ((n >> 1) & 1) ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY)) return 0;
      mbar_expect_tx(&k_full[n & 1], 16384);
      tma_load_2d(sK + (n & 1) * 16384, &tmK128, &k_full[n & 1], d.hk * FB_D, d.kv0);
      return 1;
    };
    auto load_q = [&](const DkdvItem& d, int i) {    // whole warp: the i-th Q / dO tile of item d and its statistics
      const int s = g % FBK_STAGES;
      const uint32_t ph = (g / FBK_STAGES) & 1;
      const int q_lo = d.q_begin + i * 64;
      if (lane == 0) ok = mbar_wait(&qd_empty[s], ph ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return;
      const float* lse_h = p.lse + static_cast<size_t>(d.h) * p.T;
      const float* dl_h = p.delta + static_cast<size_t>(d.h) * p.T;
      // per-query softmax statistics of this tile, staged once for all 128 key rows
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int qc = min(q_lo + lane + 32 * u, p.T - 1);
        sLse[s * 64 + lane + 32 * u] = -lse_h[qc] * FB_LOG2E;    // negated: they enter as FMA addends
        sDelta[s * 64 + lane + 32 * u] = -dl_h[qc] * p.scale;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_expect_tx(&qd_full[s], 16384);
        tma_load_2d(sQ + s * 8192, &tmQ64, &qd_full[s], d.h * FB_D, q_lo);
        tma_load_2d(sDO + s * 8192, &tmDO64, &qd_full[s], d.h * FB_D, q_lo);
      }
      ++g;
    };
    if (have) {
      if (lane == 0) ok = load_k(it, 0);
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    while (have && ok) {
      const bool have_next = next_item(rnd, nx);
      load_q(it, 0);                     // with K (loaded during the previous item) this is all the first S needs
      if (!ok) break;
      if (lane == 0) {
        ok = mbar_wait(v_empty, (ic & 1) ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY) ? 1 : 0;
        if (ok) {
          mbar_expect_tx(v_full, 16384);
          tma_load_2d(sV, &tmV128, v_full, it.hk * FB_D, it.kv0);
        }
        if (ok && have_next) ok = load_k(nx, ic + 1);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      for (int i = 1; i < it.n_it && ok; ++i) load_q(it, i);
      it = nx;
      have = have_next;
      ++ic;
    }
  } else if (warp == 9) {
    // The whole warp walks the loop, so that addresses, descriptors and loop counters stay warp-uniform
    // (a single-lane branch would keep them in per-thread registers and pay a transfer into the uniform
    // registers for every operand of every tcgen05.mma); one elected lane issues the tensor-core work.
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_f16(128, 64, 1, 0, 0);   // S^T, dP^T: N = 64 queries
    const uint32_t idesc_a = make_idesc_f16(128, 64, 1, 0, 1);   // dV, dK: B is MN-major
    const uint64_t dV0 = make_smem_desc(smem_u32(sV), 16, 1024, SWZ_128B);
    int g = 0, ic = 0, rnd = 0;
    bool ok = true;
    DkdvItem it;
    while (ok && next_item(rnd, it)) {
      const uint64_t dK0 = make_smem_desc(smem_u32(sK + (ic & 1) * 16384), 16, 1024, SWZ_128B);
      ok = __all_sync(0xffffffffu, mbar_wait(&k_full[ic & 1], (ic >> 1) & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL));
      // Order of the products of an item: S(0) | dP(i), [P ready] dV(i), S(i+1), [dS ready] dK(i) | ...
      // K-major operands advance 32 bytes per 16-wide K step (+2 in the descriptor's address field),
      // MN-major ones 2048 bytes (+128)
      auto issue_s = [&](int gi) -> bool {
        const int s = gi % FBK_STAGES;
        const uint32_t ph = (gi / FBK_STAGES) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&qd_full[s], ph, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL)))
          return false;
        tc_fence_after();
        const uint64_t dQk = make_smem_desc(smem_u32(sQ + s * 8192), 16, 1024, SWZ_128B);
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16_ss(tS, dK0 + 2 * k, dQk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
          tc_commit(sdp_full);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(g);
      for (int i = 0; i < it.n_it && ok; ++i) {
        const int gi = g + i;
        const int s = gi % FBK_STAGES;
        const uint64_t dDOk = make_smem_desc(smem_u32(sDO + s * 8192), 16, 1024, SWZ_128B);
        const uint64_t dQm = make_smem_desc(smem_u32(sQ + s * 8192), 8192, 1024, SWZ_128B);
        const uint64_t dDOm = make_smem_desc(smem_u32(sDO + s * 8192), 8192, 1024, SWZ_128B);
        if (i == 0) {   // V arrives after the first Q / dO tile; S(0) did not need it
          ok = __all_sync(0xffffffffu, mbar_wait(v_full, ic & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL));
          if (!ok) break;
          tc_fence_after();
        }
        // dP^T of this tile: its columns were last read by dK of the previous tile, issued before this
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16_ss(tDP, dV0 + 2 * k, dDOk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
          tc_commit(dp_full);
        }
        __syncwarp();
        ok = __all_sync(0xffffffffu, mbar_wait(p_ready, gi & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_MISC));
        if (!ok) break;
        if (i == 0) {
          // the first products of an item overwrite dV / dK: the previous item's must have been read out
          ok = __all_sync(0xffffffffu,
                          mbar_wait(acc_free, (ic & 1) ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_EMPTY));
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t acc = i > 0 ? 1u : 0u;
        // dV needs only P^T: it is issued while the softmax warps are still forming dS^T
        if (leader) {
          // 16 queries per step: steps 0, 1 read columns [0,16) of the score block, steps 2, 3 columns [32,48)
          mma_f16_ts(tDV, tS, dDOm, idesc_a, acc);
#pragma unroll
          for (int k = 1; k < 4; ++k)
            mma_f16_ts(tDV, tS + (k >> 1) * 32 + (k & 1) * 8, dDOm + 128 * k, idesc_a, 1u);
        }
        __syncwarp();
        if (i + 1 < it.n_it) {
          ok = issue_s(gi + 1);   // the score columns are free once dV (issued just above) has read P^T
          if (!ok) break;
        }
        ok = __all_sync(0xffffffffu, mbar_wait(ds_ready, gi & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_MISC));
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          mma_f16_ts(tDK, tDP, dQm, idesc_a, acc);
#pragma unroll
          for (int k = 1; k < 4; ++k)
            mma_f16_ts(tDK, tDP + (k >> 1) * 32 + (k & 1) * 8, dQm + 128 * k, idesc_a, 1u);
          tc_commit(&qd_empty[s]);
        }
        __syncwarp();
      }
      if (ok && leader) {
        tc_commit(acc_done);
        tc_commit(&k_empty[ic & 1]);
        tc_commit(v_empty);
      }
      __syncwarp();
      g += it.n_it;
      ++ic;
    }
  } else {
    // two threads per key row: warp w handles query columns [0,32) of the tile, warp w+4 columns [32,64)
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c_log2 = p.scale * FB_LOG2E;
    int g = 0, ic = 0;
    bool ok = true;
    for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items && ok; ++rnd) {
      const int item = snake_item(rnd);
      if (item >= n_items) continue;
      DkdvItem it;
      if (!dkdv_decode(p, item, it)) continue;
      const int kj = it.kv0 + row;
      const int de = it.de, q_end = it.q_end, h = it.h, hk = it.hk;
      for (int i = 0; i < it.n_it; ++i) {
        const int gi = g + i;
        const int q_lo = it.q_begin + i * 64;
        const int st = gi % FBK_STAGES;
        const uint32_t lse_sa = smem_u32(sLse + st * 64), dl_sa = smem_u32(sDelta + st * 64);
        // observe the producer's barrier directly so its smem writes are visible here
        ok = mbar_wait(&qd_full[st], (gi / FBK_STAGES) & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL);
        if (ok) ok = mbar_wait(sdp_full, gi & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // query columns of this tile that key row kj may attend to: [c_lo, c_hi]
        const int c_lo_q = kj - q_lo;                                           // causal: qi >= kj
        int c_hi_q = min(q_end, p.window > 0 ? kj + p.window : q_end) - 1 - q_lo;  // window and document end
        if (kj >= de) c_hi_q = -1;
        // Whole warps branch on whether any of their rows needs the mask: off the diagonal and away from the
        // window / document edges the loop carries no compares or selects at all.
        const bool need_mask = __any_sync(0xffffffffu, (c_lo_q > 0) || (c_hi_q < 63));
        auto tile = [&](auto masked) -> bool {
          constexpr bool MASK = decltype(masked)::value;
          const int c = half;
          // phase 1: P^T = exp2(S^T * c - lse), kept in fp32 in place of the scores and stored as bf16
          uint32_t sv[32], pp[16];
          tmem_ld_x32(tS + lane_addr + c * 32, sv);
          tmem_ld_wait();
          const uint64_t c2 = pack_f32x2(c_log2, c_log2), sc2 = pack_f32x2(p.scale, p.scale);
#pragma unroll
          for (int e4 = 0; e4 < 32; e4 += 4) {
            // the per-query statistics are the same for every key row: one 16-byte shared load covers four
            // columns, already as two fp32 pairs
            const ulonglong2 nl = lds_u64x2(lse_sa + (c * 32 + e4) * 4);
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int e = e4 + 2 * h2;
              float p0, p1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), c2,
                                     h2 ? nl.y : nl.x), p0, p1);
              p0 = fast_exp2(p0);
              p1 = fast_exp2(p1);
              if constexpr (MASK) {
                const int col = c * 32 + e;
                p0 = (col >= c_lo_q && col <= c_hi_q) ? p0 : 0.f;
                p1 = (col + 1 >= c_lo_q && col + 1 <= c_hi_q) ? p1 : 0.f;
              }
              sv[e] = __float_as_uint(p0);
              sv[e + 1] = __float_as_uint(p1);
              pp[e / 2] = pack_bf16(p0, p1);
            }
          }
          // P^T as bf16 overwrites the first half of the 32 score columns that THIS thread read (never columns
          // that the row's other thread may still have to read): queries [32c, 32c+32) sit in columns [32c, 32c+16)
          tmem_st_x16(tS + lane_addr + c * 32, pp);
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(p_ready);
          // phase 2: dS^T = P^T o (dP^T * scale - delta)
          bool fine = mbar_wait(dp_full, gi & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
          fine = __all_sync(0xffffffffu, fine);
          if (!fine) return false;
          tc_fence_after();
          uint32_t dp[32], dd[16];
          tmem_ld_x32(tDP + lane_addr + c * 32, dp);
          tmem_ld_wait();
#pragma unroll
          for (int e4 = 0; e4 < 32; e4 += 4) {
            const ulonglong2 nd = lds_u64x2(dl_sa + (c * 32 + e4) * 4);
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int e = e4 + 2 * h2;
              float d0, d1;
              const uint64_t t2 = fma_f32x2(pack_f32x2(__uint_as_float(dp[e]), __uint_as_float(dp[e + 1])), sc2,
                                            h2 ? nd.y : nd.x);
              unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), t2), d0, d1);
              dd[e / 2] = pack_bf16(d0, d1);
            }
          }
          tmem_st_x16(tDP + lane_addr + c * 32, dd);
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(ds_ready);
          return true;
        };
        ok = need_mask ? tile(BoolC<true>{}) : tile(BoolC<false>{});
        if (!ok) break;
      }
      if (ok) {
        ok = mbar_wait(acc_done, ic & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (!ok) break;
      tc_fence_after();
      {
        const int which = half;  // the first thread of a row writes dV, the second dK
        uint32_t o[64];
        const uint32_t src = (which == 0 ? tDV : tDK) + lane_addr;
        tmem_ld_x32(src, o);
        tmem_ld_x32(src + 32, o + 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(acc_free);   // the next item's first products may overwrite the accumulators now
        if (kj < de) {
          if (p.dk_part) {
            float4* dst = reinterpret_cast<float4*>((which == 0 ? p.dv_part : p.dk_part) +
                                                    (static_cast<size_t>(kj) * p.Hq + h) * FB_D);
#pragma unroll
            for (int v = 0; v < 16; ++v)
              dst[v] = make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                   __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
          } else {
            __nv_bfloat16* base = (which == 0 ? p.dv + static_cast<size_t>(kj) * p.dv_ld
                                              : p.dk + static_cast<size_t>(kj) * p.dk_ld) + hk * FB_D;
            uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1]));
              w.y = pack_bf16(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3]));
              w.z = pack_bf16(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5]));
              w.w = pack_bf16(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7]));
              dst[v] = w;
            }
          }
        }
      }
      g += it.n_it;
      ++ic;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------ dQ
// smem: Q 16 KB, dO 16 KB, 3 stages x (K 8 KB + V 8 KB). Persistent over (query tile, query head) items,
// heaviest first, like the forward kernel. The score accumulator is double-buffered in TMEM: S of key tile
// j + 1 is issued while the softmax warps still work on tile j, so inside an item they never wait for a
// score product (the chain per tile was S -> P -> dS -> dQ, one after the other).
constexpr int FBQ_STAGES = 3;
constexpr int FBQ_SMEM = 2 * 16384 + FBQ_STAGES * 16384 + 1024 + 1024;

struct DqItem {
  int q0, de, h, hk, q_hi, lo, n_kv;
};

__device__ __forceinline__ bool dq_decode(const FlashBwdParams& p, int item, DqItem& it) {
  const int4 job = p.plan[item / p.Hq];   // first list: query tiles that see the most keys first
  if (!job.w) return false;
  it.q0 = job.x; it.de = job.z;
  it.h = item % p.Hq;
  it.hk = it.h / (p.Hq / p.Hkv);
  it.q_hi = min(it.q0 + 128, it.de);
  it.lo = job.y;
  if (p.window > 0) it.lo = max(job.y, it.q0 - p.window + 1);
  it.n_kv = (it.q_hi - it.lo + 63) / 64;
  return it.n_kv > 0;
}

__global__ void __launch_bounds__(FB_THREADS, 2)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ128, const __grid_constant__ CUtensorMap tmDO128,
                    const __grid_constant__ CUtensorMap tmK64, const __grid_constant__ CUtensorMap tmV64,
                    const FlashBwdParams p) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + 16384;
  uint8_t* sK = smem + 32768;                        // FBQ_STAGES x 8 KB
  uint8_t* sV = smem + 32768 + FBQ_STAGES * 8192;    // FBQ_STAGES x 8 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 32768 + FBQ_STAGES * 16384);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;   // [3]
  uint64_t* kv_empty = bars + 4;  // [3]
  uint64_t* sdp_full = bars + 7;  // [2], one per score buffer: S of the next tile may complete early
  uint64_t* p_ready = bars + 9;
  uint64_t* acc_done = bars + 10;
  uint64_t* q_empty = bars + 11;  // the item's last products have read Q and dO
  uint64_t* acc_free = bars + 12; // the item's dQ accumulator has been read out
  uint64_t* dp_full = bars + 13;  // dP is in TMEM (S has its own barrier, so the exponentials start earlier)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_items = p.n_tiles * p.Hq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FBQ_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&sdp_full[0], 1);
    mbar_init(&sdp_full[1], 1);
    mbar_init(p_ready, 256);
    mbar_init(dp_full, 1);
    mbar_init(acc_done, 1);
    mbar_init(q_empty, 1);
    mbar_init(acc_free, 256);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ = tmem_base + 192;   // tS: two buffers of 64 columns

  if (warp == 8) {
    if (lane == 0) {
      int g = 0, ic = 0;
      bool ok = true;
      for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items && ok; ++rnd) {
        const int item = snake_item(rnd);
        if (item >= n_items) continue;
        DqItem it;
        if (!dq_decode(p, item, it)) continue;
        if (!mbar_wait(q_empty, (ic & 1) ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY)) break;
        ++ic;
        mbar_expect_tx(q_full, 32768);
        tma_load_2d(sQ, &tmQ128, q_full, it.h * FB_D, it.q0);
        tma_load_2d(sDO, &tmDO128, q_full, it.h * FB_D, it.q0);
        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const int s = g % FBQ_STAGES;
          const uint32_t ph = (g / FBQ_STAGES) & 1;
          if (!mbar_wait(&kv_empty[s], ph ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&kv_full[s], 16384);
          tma_load_2d(sK + s * 8192, &tmK64, &kv_full[s], it.hk * FB_D, it.lo + j * 64);
          tma_load_2d(sV + s * 8192, &tmV64, &kv_full[s], it.hk * FB_D, it.lo + j * 64);
        }
      }
    }
  } else if (warp == 9) {
    // warp-uniform loop, one elected lane issues (see the dK / dV kernel)
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_f16(128, 64, 1, 0, 0);
    const uint32_t idesc_q = make_idesc_f16(128, 64, 1, 0, 1);
    const uint64_t dQ0 = make_smem_desc(smem_u32(sQ), 16, 1024, SWZ_128B);
    const uint64_t dDO0 = make_smem_desc(smem_u32(sDO), 16, 1024, SWZ_128B);
    int g = 0, ic = 0;
    bool ok = true;
    for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items && ok; ++rnd) {
      const int item = snake_item(rnd);
      if (item >= n_items) continue;
      DqItem it;
      if (!dq_decode(p, item, it)) continue;
      ok = __all_sync(0xffffffffu, mbar_wait(q_full, ic & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL));
      // Order of the products of an item: S(0) | dP(j), S(j+1), [softmax of tile j done] dQ(j) | ...
      // S(j+1) goes to the other score buffer, whose last reader, dQ(j-1), was issued before it.
      auto issue_s = [&](int gj) -> bool {
        const int s = gj % FBQ_STAGES;
        const uint32_t ph = (gj / FBQ_STAGES) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&kv_full[s], ph, abort_flag, p.status, KWU_ERR_TIMEOUT_FULL)))
          return false;
        tc_fence_after();
        const uint64_t dKk = make_smem_desc(smem_u32(sK + s * 8192), 16, 1024, SWZ_128B);
        const uint32_t dst = tS + (gj & 1) * 64;
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16_ss(dst, dQ0 + 2 * k, dKk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
          tc_commit(&sdp_full[gj & 1]);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(g);
      for (int j = 0; j < it.n_kv && ok; ++j) {
        const int gj = g + j;
        const int s = gj % FBQ_STAGES;
        const uint64_t dVk = make_smem_desc(smem_u32(sV + s * 8192), 16, 1024, SWZ_128B);
        const uint64_t dKm = make_smem_desc(smem_u32(sK + s * 8192), 8192, 1024, SWZ_128B);
        // the softmax warps have read dP of the previous tile (its p_ready was waited for below)
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16_ss(tDP, dDO0 + 2 * k, dVk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
          tc_commit(dp_full);
        }
        __syncwarp();
        if (j + 1 < it.n_kv) {
          ok = issue_s(gj + 1);
          if (!ok) break;
        } else if (leader) {
          tc_commit(q_empty);   // Q and dO are free once the products issued so far are done
        }
        __syncwarp();
        ok = __all_sync(0xffffffffu, mbar_wait(p_ready, gj & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_MISC));
        if (!ok) break;
        if (j == 0) {
          ok = __all_sync(0xffffffffu,
                          mbar_wait(acc_free, (ic & 1) ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_EMPTY));
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t acc = j > 0 ? 1u : 0u;
        const uint32_t tSj = tS + (gj & 1) * 64;
        if (leader) {
          mma_f16_ts(tDQ, tSj, dKm, idesc_q, acc);
#pragma unroll
          for (int k = 1; k < 4; ++k)
            mma_f16_ts(tDQ, tSj + (k >> 1) * 32 + (k & 1) * 8, dKm + 128 * k, idesc_q, 1u);
          tc_commit(&kv_empty[s]);
        }
        __syncwarp();
      }
      if (ok && leader) tc_commit(acc_done);
      __syncwarp();
      g += it.n_kv;
      ++ic;
    }
  } else {
    const int quarter = warp & 3, half = warp >> 2;   // two threads per query row, 32 key columns each
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c_log2 = p.scale * FB_LOG2E;
    int g = 0, ic = 0;
    bool ok = true;
    for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items && ok; ++rnd) {
      const int item = snake_item(rnd);
      if (item >= n_items) continue;
      DqItem it;
      if (!dq_decode(p, item, it)) continue;
      const int qi = it.q0 + row;
      const int q_hi = it.q_hi, h = it.h;
      const int qc = min(qi, p.T - 1);
      const float lse_q = p.lse[static_cast<size_t>(h) * p.T + qc] * FB_LOG2E;
      const float dl_q = p.delta[static_cast<size_t>(h) * p.T + qc] * p.scale;
      for (int j = 0; j < it.n_kv; ++j) {
        const int gj = g + j;
        const int kv0 = it.lo + j * 64;
        const uint32_t tSj = tS + (gj & 1) * 64;
        ok = mbar_wait(&sdp_full[gj & 1], (gj >> 1) & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // key columns of this tile that query row qi may attend to: [c_lo, c_hi]
        const int c_hi_k = (qi < q_hi) ? (qi - kv0) : -1;
        const int c_lo_k = (p.window > 0) ? (qi - p.window + 1 - kv0) : 0;
        const bool need_mask = __any_sync(0xffffffffu, (c_hi_k < 63) || (c_lo_k > 0));
        auto tile = [&](auto masked) -> bool {
          constexpr bool MASK = decltype(masked)::value;
          const int c = half;
          // phase 1: P = exp2(S * c - lse) in fp32, in place of the scores
          uint32_t sv[32];
          tmem_ld_x32(tSj + lane_addr + c * 32, sv);
          tmem_ld_wait();
          const uint64_t c2 = pack_f32x2(c_log2, c_log2), sc2 = pack_f32x2(p.scale, p.scale);
          const uint64_t nl2 = pack_f32x2(-lse_q, -lse_q), nd2 = pack_f32x2(-dl_q, -dl_q);
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float p0, p1;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), c2, nl2), p0, p1);
            p0 = fast_exp2(p0);
            p1 = fast_exp2(p1);
            if constexpr (MASK) {
              const int col = c * 32 + e;
              p0 = (col >= c_lo_k && col <= c_hi_k) ? p0 : 0.f;
              p1 = (col + 1 >= c_lo_k && col + 1 <= c_hi_k) ? p1 : 0.f;
            }
            sv[e] = __float_as_uint(p0);
            sv[e + 1] = __float_as_uint(p1);
          }
          // phase 2: dS = P o (dP * scale - delta), stored as bf16 over the first half of this thread's score columns
          bool fine = mbar_wait(dp_full, gj & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
          fine = __all_sync(0xffffffffu, fine);
          if (!fine) return false;
          tc_fence_after();
          uint32_t dp[32], dd[16];
          tmem_ld_x32(tDP + lane_addr + c * 32, dp);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float d0, d1;
            const uint64_t t2 = fma_f32x2(pack_f32x2(__uint_as_float(dp[e]), __uint_as_float(dp[e + 1])), sc2, nd2);
            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), t2), d0, d1);
            dd[e / 2] = pack_bf16(d0, d1);
          }
          tmem_st_x16(tSj + lane_addr + c * 32, dd);
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(p_ready);
          return true;
        };
        ok = need_mask ? tile(BoolC<true>{}) : tile(BoolC<false>{});
        if (!ok) break;
      }
      if (ok) {
        ok = mbar_wait(acc_done, ic & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (!ok) break;
      tc_fence_after();
      uint32_t o[32];
      tmem_ld_x32(tDQ + lane_addr + half * 32, o);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(acc_free);
      if (qi < q_hi) {
        uint4* dst = reinterpret_cast<uint4*>(p.dq + (static_cast<size_t>(qi) * p.Hq + h) * FB_D + half * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1]));
          w.y = pack_bf16(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3]));
          w.z = pack_bf16(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5]));
          w.w = pack_bf16(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7]));
          dst[v] = w;
        }
      }
      g += it.n_kv;
      ++ic;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// dk[t, hk, :] = sum over the query heads of group hk of part[t, h, :]   (same for dv)
__global__ void __launch_bounds__(256)
flash_group_reduce_kernel(const float* __restrict__ dk_part, const float* __restrict__ dv_part,
                          __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, int dk_ld,
                          int dv_ld, int T, int Hq, int Hkv) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  const int group = Hq / Hkv;
  const long total = static_cast<long>(T) * Hkv * 16;  // float4 lanes
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i & 15);
    const long th = i >> 4;
    const int hk = static_cast<int>(th % Hkv);
    const long t = th / Hkv;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    for (int g = 0; g < group; ++g) {
      const size_t off = ((static_cast<size_t>(t) * Hq + hk * group + g) * 64) / 4 + v;
      const float4 x = reinterpret_cast<const float4*>(dk_part)[off];
      const float4 y = reinterpret_cast<const float4*>(dv_part)[off];
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
      b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
    }
    reinterpret_cast<uint2*>(dk + static_cast<size_t>(t) * dk_ld + hk * 64)[v] =
        make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
    reinterpret_cast<uint2*>(dv + static_cast<size_t>(t) * dv_ld + hk * 64)[v] =
        make_uint2(pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
  }
}

}  // namespace kwu

using namespace kwu;

// Scratch for the GQA partial sums: 2 * T * Hq * 64 floats when Hq > Hkv (0 otherwise).
KWU_API long long kwu_flash_bwd_scratch_floats(int T, int Hq, int Hkv) {
  return Hq > Hkv ? 2ll * T * Hq * 64 : 0;
}

KWU_API int kwu_flash_bwd(const void* q, int q_ld, const void* k, int k_ld, const void* v, int v_ld,
                          const void* out, const void* dout, const float* lse, float* delta,
                          void* dq, void* dk, int dk_ld, void* dv, int dv_ld, float* scratch, const void* plan,
                          int n_tiles, int T, int Hq, int Hkv, int window, float scale, void* stream,
                          int* status) {
  if (T <= 0 || n_tiles <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    long rows = static_cast<long>(T) * Hq;
    long g = (rows + 31) / 32;
    if (g > 148 * 16) g = 148 * 16;
    launch_k(flash_delta_kernel, dim3(static_cast<int>(g)), dim3(256), 0, st, (const __nv_bfloat16*)out,
                                                          (const __nv_bfloat16*)dout, delta, T, Hq); kwu::count_launch();
  }
  CUtensorMap tmQ64, tmDO64, tmK128, tmV128, tmQ128, tmDO128, tmK64, tmV64;
  int rc;
  const uint64_t wq = (uint64_t)Hq * FB_D, wk = (uint64_t)Hkv * FB_D;
  const int SW = CU_TENSOR_MAP_SWIZZLE_128B;
  if ((rc = encode_tmap_2d(&tmQ64, q, ELEM_BF16, T, wq, q_ld, 64, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmDO64, dout, ELEM_BF16, T, wq, wq, 64, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmK128, k, ELEM_BF16, T, wk, k_ld, 128, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmV128, v, ELEM_BF16, T, wk, v_ld, 128, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmQ128, q, ELEM_BF16, T, wq, q_ld, 128, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmDO128, dout, ELEM_BF16, T, wq, wq, 128, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmK64, k, ELEM_BF16, T, wk, k_ld, 64, 64, SW))) return rc;
  if ((rc = encode_tmap_2d(&tmV64, v, ELEM_BF16, T, wk, v_ld, 64, 64, SW))) return rc;
  static PerDeviceOnce attr;
  if (attr.pending()) {
    cudaError_t e1 = cudaFuncSetAttribute(flash_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FBK_SMEM);
    cudaError_t e2 = cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FBQ_SMEM);
    if (e1 != cudaSuccess || e2 != cudaSuccess) { set_last_error("flash_bwd attr failed"); return 10; }
    attr.mark();
  }
  FlashBwdParams p;
  p.lse = lse; p.delta = delta;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.plan = reinterpret_cast<const int4*>(plan);
  p.n_tiles = n_tiles;
  p.dk_ld = dk_ld; p.dv_ld = dv_ld;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.window = window; p.scale = scale; p.status = status;
  if (Hq > Hkv) {
    if (!scratch) { set_last_error("flash_bwd: GQA needs the scratch buffer"); return 7; }
    p.dk_part = scratch;
    p.dv_part = scratch + static_cast<size_t>(T) * Hq * 64;
  } else {
    p.dk_part = p.dv_part = nullptr;
  }
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long items = static_cast<long long>(n_tiles) * Hq;
  const int pgrid = static_cast<int>(items < 2LL * sms ? items : 2LL * sms);   // two resident CTAs per SM walk the items
  launch_k(flash_bwd_dkdv_kernel, dim3(pgrid), dim3(FB_THREADS), FBK_SMEM, st, tmQ64, tmDO64, tmK128, tmV128, p); kwu::count_launch();
  if (Hq > Hkv) {
    long g = (static_cast<long>(T) * Hkv * 16 + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    launch_k(flash_group_reduce_kernel, dim3(static_cast<int>(g)), dim3(256), 0, st, p.dk_part, p.dv_part, p.dk, p.dv, dk_ld, dv_ld, T, Hq, Hkv); kwu::count_launch();
  }
  launch_k(flash_bwd_dq_kernel, dim3(pgrid), dim3(FB_THREADS), FBQ_SMEM, st, tmQ128, tmDO128, tmK64, tmV64, p); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("flash_bwd launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}
