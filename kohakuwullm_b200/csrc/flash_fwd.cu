// Varlen causal / sliding-window flash attention forward for head_dim 64, bf16, on tcgen05.
//
// Persistent CTAs (two per SM) walk a heaviest-first list of (128-row query tile, query head) items. Roles:
//   warps 0..7  softmax: two threads per query row (64 key columns each); read S from TMEM, online
//               softmax in fp32, write P (bf16) back to TMEM, rescale the O accumulator when the max moves
//   warp 8      TMA producer: Q per item, K and V tiles through two-stage rings (runs ahead into the next item)
//   warp 9      issues tcgen05.mma:  S = Q K^T (smem x smem)  and  O += P V (TMEM x smem)
// TMEM columns: S [0,128) fp32, P [128,192) packed bf16, O [192,256) fp32. Two CTAs fit per SM, so
// one CTA's softmax overlaps the other's tensor-core work.
//
// Documents never attend across their boundary: a tile's key range is clipped to its own document
// and (with a window) to the last `window` positions. Sinks enter as sink_lse[h] = logsumexp of the
// head's sink logits: the stored lse is logaddexp(lse, sink_lse) and the output is scaled to match.
// Replaces src/kohakuwullm/kernels/attention/flash_attn_fwd.py:35-154 and the vendor FA2 call at
// src/kohakuwullm/models/components/attention.py:170-188 of the reference.
#include "common.cuh"
#include "mx_quant.cuh"

namespace kwu {

constexpr int FA_BM = 128;   // query rows per CTA
constexpr int FA_BN = 128;   // keys per tile
constexpr int FA_D = 64;
constexpr int FA_THREADS = 320;  // 8 softmax warps + TMA warp + MMA warp
constexpr int FA_TILE_BYTES = 128 * 64 * 2;  // 16 KB
constexpr int FA_SMEM = 5 * FA_TILE_BYTES + 1024 + 3072 + 1024;  // tiles + barriers + row-max exchange + alignment slack
constexpr float FA_NEG = -1.0e30f;
template <bool V> struct FwdBoolC { static constexpr bool value = V; };

struct FlashFwdParams {
  __nv_bfloat16* out;   // (T, Hq, 64)
  float* lse;           // (Hq, T)
  const int4* plan;     // (q0, doc_start, doc_end, valid)
  int n_tiles;
  int T, Hq, Hkv, window;
  const float* sink_lse;  // (Hq) or null
  float scale_log2;       // softmax scale * log2(e)
  int* status;
  // optional MXFP8 copy of `out` seen as a (T, Hq * 64) matrix: e4m3 bytes + UE8M0 scale chunks (the layout of
  // mxfp8.cu), for an MXFP8 output projection. Each epilogue thread holds exactly one 32-element block.
  uint8_t* q8;
  uint8_t* sf;
};

// Tile lists for packed batches: for every document, ceil(len/tile) entries (q0, doc_start, doc_end, valid),
// written twice: plan[0, max_tiles) sorted by the number of keys a QUERY tile sees (descending: the order
// of the forward and dQ kernels), plan[max_tiles, 2*max_tiles) sorted by the number of queries that see a
// KEY tile (descending: the dK / dV kernel). Unused entries sort last. One block; a rank sort, since the
// list has at most a few hundred entries.
__global__ void attn_plan_kernel(const int* __restrict__ cu, int ndocs, int tile, int4* __restrict__ plan,
                                 int max_tiles) {
  extern __shared__ int4 s_plan[];                                   // max_tiles entries in token order
  int* s_off = reinterpret_cast<int*>(s_plan + max_tiles);           // ndocs + 1
  for (int d = threadIdx.x; d < ndocs; d += blockDim.x) {
    const int len = cu[d + 1] - cu[d];
    s_off[d + 1] = (len + tile - 1) / tile;
  }
  if (threadIdx.x == 0) s_off[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int d = 0; d < ndocs; ++d) s_off[d + 1] += s_off[d];
  __syncthreads();
  const int used = s_off[ndocs];
  for (int d = threadIdx.x; d < ndocs; d += blockDim.x) {
    const int s = cu[d], e = cu[d + 1];
    int idx = s_off[d];
    for (int q0 = s; q0 < e && idx < max_tiles; q0 += tile, ++idx) s_plan[idx] = make_int4(q0, s, e, 1);
  }
  for (int i = used + threadIdx.x; i < max_tiles; i += blockDim.x) s_plan[i] = make_int4(0, 0, 0, 0);
  __syncthreads();
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) {
    const int4 me = s_plan[i];
    const int cq = me.w ? min(me.x + tile, me.z) - me.y : -1;   // keys visible to the tile's last query row
    const int ck = me.w ? me.z - me.x : -1;                     // queries that can see the tile's first key
    int rq = 0, rk = 0;
    for (int j = 0; j < max_tiles; ++j) {
      const int4 o = s_plan[j];
      const int oq = o.w ? min(o.x + tile, o.z) - o.y : -1;
      const int ok = o.w ? o.z - o.x : -1;
      rq += (oq > cq) || (oq == cq && j < i);
      rk += (ok > ck) || (ok == ck && j < i);
    }
    plan[rq] = me;
    plan[max_tiles + rk] = me;
  }
}

// Work item = (query tile, query head). A CTA walks items blockIdx.x, blockIdx.x + gridDim.x, ... of the
// heaviest-first list, so TMEM allocation, barrier set-up and the tensor-map fetch are paid once per CTA,
// and the producer warp is already loading the next item's Q and K while the softmax warps finish the
// current one. Barrier phases run on counters that continue across items.
struct FwdItem {
  int q0, ds, de, h, hk, lo, n_kv, q_hi;
};

__device__ __forceinline__ bool fwd_decode(const FlashFwdParams& p, int item, FwdItem& it) {
  const int4 job = p.plan[item / p.Hq];   // the list is sorted: query tiles that see the most keys first
  if (!job.w) return false;
  it.q0 = job.x; it.ds = job.y; it.de = job.z;
  it.h = item % p.Hq;
  it.hk = it.h / (p.Hq / p.Hkv);
  it.q_hi = min(it.q0 + FA_BM, it.de);            // one past the last valid query row
  it.lo = it.ds;
  if (p.window > 0) it.lo = max(it.ds, it.q0 - p.window + 1);
  it.n_kv = (it.q_hi - it.lo + FA_BN - 1) / FA_BN;
  return it.n_kv > 0;
}

__global__ void __launch_bounds__(FA_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashFwdParams p) {
  pdl_sync();   // nothing of the previous kernel is read above this line
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + FA_TILE_BYTES;       // 2 stages
  uint8_t* sV = smem + 3 * FA_TILE_BYTES;   // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 5 * FA_TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 10;
  uint64_t* o_done = bars + 11;
  uint64_t* q_empty = bars + 12;  // the item's last S product has read Q
  uint64_t* o_free = bars + 13;   // the softmax warps have read the item's O accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_rowmax = reinterpret_cast<float*>(smem + 5 * FA_TILE_BYTES + 1024);  // 2 x 256 max + 256 sums

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_items = p.n_tiles * p.Hq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 256);
    mbar_init(o_done, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_free, 256);
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
  const uint32_t tS = tmem_base, tP = tmem_base + 128, tO = tmem_base + 192;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      int g = 0, ic = 0;   // K/V tiles and items issued so far by this CTA
      bool ok = true;
      for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items && ok; ++rnd) {
        const int item = snake_item(rnd);
        if (item >= n_items) continue;
        FwdItem it;
        if (!fwd_decode(p, item, it)) continue;
        if (!mbar_wait(q_empty, (ic & 1) ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY)) break;
        ++ic;
        mbar_expect_tx(q_full, FA_TILE_BYTES);
        tma_load_2d(sQ, &tmQ, q_full, it.h * FA_D, it.q0);
        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const int s = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          const int kv0 = it.lo + j * FA_BN;
          if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&k_full[s], FA_TILE_BYTES);
          tma_load_2d(sK + s * FA_TILE_BYTES, &tmK, &k_full[s], it.hk * FA_D, kv0);
          if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, p.status, KWU_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&v_full[s], FA_TILE_BYTES);
          tma_load_2d(sV + s * FA_TILE_BYTES, &tmV, &v_full[s], it.hk * FA_D, kv0);
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop, so that descriptors and counters stay warp-uniform (a single-lane
    // branch keeps them in per-thread registers and pays a transfer into the uniform registers for every
    // operand of every tcgen05.mma, on the critical path between two softmax tiles); one elected lane issues.
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_f16(128, 128, 1, 0, 0);
    const uint32_t idesc_o = make_idesc_f16(128, 64, 1, 0, 1);
    const uint64_t dQ0 = make_smem_desc(smem_u32(sQ), 16, 1024, SWZ_128B);
    int g = 0, ic = 0;
    bool ok = true;
    auto issue_s = [&](int gj, bool last_of_item) {
      const int s = gj & 1;
      const uint64_t dK = make_smem_desc(smem_u32(sK + s * FA_TILE_BYTES), 16, 1024, SWZ_128B);
      if (leader) {
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) mma_f16_ss(tS, dQ0 + 2 * k, dK + 2 * k, idesc_s, k > 0 ? 1u : 0u);
        tc_commit(s_full);
        tc_commit(&k_empty[s]);
        if (last_of_item) tc_commit(q_empty);
      }
      __syncwarp();
    };
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, p.status, code));
    };
    for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items && ok; ++rnd) {
      const int item = snake_item(rnd);
      if (item >= n_items) continue;
      FwdItem it;
      if (!fwd_decode(p, item, it)) continue;
      const int n_kv = it.n_kv;
      ok = wait_all(q_full, ic & 1, KWU_ERR_TIMEOUT_FULL);
      if (ok) ok = wait_all(&k_full[g & 1], (g >> 1) & 1, KWU_ERR_TIMEOUT_FULL);
      if (!ok) break;
      tc_fence_after();
      // S of the previous item has been read (its last p_full was waited for below) and P is rewritten
      // by the softmax warps only after they have waited for the previous item's last o_done
      issue_s(g, n_kv == 1);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int gj = g + j;
        const int s = gj & 1;
        const uint32_t ph = (gj >> 1) & 1;
        if (j + 1 < n_kv) {
          ok = wait_all(&k_full[(gj + 1) & 1], ((gj + 1) >> 1) & 1, KWU_ERR_TIMEOUT_FULL);
          if (!ok) break;
        }
        // P_j written (and S_j fully read) by the softmax warps
        ok = wait_all(p_full, gj & 1, KWU_ERR_TIMEOUT_MISC);
        if (!ok) break;
        tc_fence_after();
        if (j + 1 < n_kv) issue_s(gj + 1, j + 2 == n_kv);
        ok = wait_all(&v_full[s], ph, KWU_ERR_TIMEOUT_FULL);
        if (!ok) break;
        if (j == 0) {
          // the first product of an item overwrites O: the previous item's epilogue must have read it
          ok = wait_all(o_free, (ic & 1) ^ 1, KWU_ERR_TIMEOUT_ACC_EMPTY);
          if (!ok) break;
        }
        tc_fence_after();
        const uint64_t dV = make_smem_desc(smem_u32(sV + s * FA_TILE_BYTES), 8192, 1024, SWZ_128B);
        const uint32_t acc = j > 0 ? 1u : 0u;
        if (leader) {
          mma_f16_ts(tO, tP, dV, idesc_o, acc);
#pragma unroll
          for (int k = 1; k < FA_BN / 16; ++k) mma_f16_ts(tO, tP + k * 8, dV + 128 * k, idesc_o, 1u);
          tc_commit(o_done);
          tc_commit(&v_empty[s]);
        }
        __syncwarp();
      }
      g += n_kv;
      ++ic;
    }
  } else {
    // ---------------------------------------------------------------- softmax (warps 0..7)
    // Two threads per query row: warp w and warp w+4 share TMEM lane quarter w%4; the first takes key
    // columns [0,64) of the tile, the second [64,128). They exchange only the row maximum (through
    // shared memory, once per tile); each keeps its own partial row sum until the epilogue.
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;     // query row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t col_base = half * 64;
    int g = 0;
    bool ok = true;
    for (int rnd = 0; rnd * static_cast<int>(gridDim.x) < n_items; ++rnd) {
      const int item = snake_item(rnd);
      if (item >= n_items) continue;
      FwdItem it;
      if (!fwd_decode(p, item, it)) continue;
      const int q0 = it.q0, n_kv = it.n_kv, h = it.h;
      const int qi = q0 + row;
      float m = FA_NEG, l = 0.f;
      for (int j = 0; j < n_kv; ++j) {
        const int gj = g + j;
        const int kv0 = it.lo + j * FA_BN;
        // after a time-out the loops keep running (so every warp still meets the named barrier below)
        // but do no work; the waits return at once because the abort flag is set
        if (ok) {
          ok = mbar_wait(s_full, gj & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
          ok = __all_sync(0xffffffffu, ok);
        }
        tc_fence_after();
        const bool need_mask = (kv0 + FA_BN - 1 > q0) || (p.window > 0 && (q0 + FA_BM - 1 - kv0) >= p.window);
        // key columns this row may see inside the tile: [c_lo, c_hi]
        const int c_hi = qi - kv0;
        const int c_lo = (p.window > 0) ? (qi - p.window + 1 - kv0) : -1;
        // pass 1: maximum of the raw scores of this thread's 64 columns (the positive scale commutes with max)
        float mx4[4] = {FA_NEG, FA_NEG, FA_NEG, FA_NEG};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (!ok) break;
          uint32_t r[32];
          tmem_ld_x32(tS + lane_addr + col_base + c * 32, r);
          tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = col_base + c * 32 + e;
              const float sv = (col <= c_hi && col >= c_lo) ? __uint_as_float(r[e]) : FA_NEG;
              mx4[e & 3] = fmaxf(mx4[e & 3], sv);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(r[e]));
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // exchange with the thread that owns the other half of the row (buffers alternate per tile)
        float* xbuf = s_rowmax + (gj & 1) * 256;
        xbuf[half * 128 + row] = mx;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        mx = fmaxf(fmaxf(mx, xbuf[(half ^ 1) * 128 + row]), m);
        if (!ok) continue;
        const float alpha = fast_exp2((m - mx) * p.scale_log2);
        m = mx;
        const float neg_ms = -mx * p.scale_log2;
        // pass 2: probabilities p = 2^(s*c - m*c), packed to bf16
        uint32_t pk[32];
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        // the mask is needed only on diagonal / window-edge tiles (the same for the whole CTA): two copies
        // of the loop, so that the common one carries no compares or selects
        auto pass2 = [&](auto masked) {
          constexpr bool MASK = decltype(masked)::value;
          const uint64_t sl2 = pack_f32x2(p.scale_log2, p.scale_log2), nm2 = pack_f32x2(neg_ms, neg_ms);
          uint64_t acc2[2] = {pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f)};
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld_x32(tS + lane_addr + col_base + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float p0, p1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), sl2, nm2), p0, p1);
              p0 = fast_exp2(p0);
              p1 = fast_exp2(p1);
              if constexpr (MASK) {
                const int col = col_base + c * 32 + e;
                p0 = (col <= c_hi && col >= c_lo) ? p0 : 0.f;
                p1 = (col + 1 <= c_hi && col + 1 >= c_lo) ? p1 : 0.f;
              }
              acc2[(e >> 1) & 1] = add_f32x2(acc2[(e >> 1) & 1], pack_f32x2(p0, p1));
              pk[c * 16 + e / 2] = pack_bf16(p0, p1);
            }
          }
          unpack_f32x2(acc2[0], sum4[0], sum4[1]);
          unpack_f32x2(acc2[1], sum4[2], sum4[3]);
        };
        if (need_mask) pass2(FwdBoolC<true>{}); else pass2(FwdBoolC<false>{});
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        // the previous P V product must be complete before P is overwritten and O is touched; for the
        // first tile of an item that product belongs to the previous item and was waited for in its epilogue
        if (j > 0) {
          ok = mbar_wait(o_done, (gj - 1) & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_EMPTY);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) continue;
          tc_fence_after();
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            // this thread rescales its half of the row's 64 output columns
            uint32_t o[32];
            tmem_ld_x32(tO + lane_addr + half * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_x32(tO + lane_addr + half * 32, o);
          }
        }
        tmem_st_x32(tP + lane_addr + half * 32, pk);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(p_full);
      }
      // ---------------------------------------------------------------- epilogue of the item
      if (ok) {
        ok = mbar_wait(o_done, (g + n_kv - 1) & 1, abort_flag, p.status, KWU_ERR_TIMEOUT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      // total row sum = own partial + the partner's (both are relative to the same final maximum)
      float* lbuf = s_rowmax + 512;
      lbuf[half * 128 + row] = l;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      l += lbuf[(half ^ 1) * 128 + row];
      if (ok) {
        tc_fence_after();
        uint32_t o[32];
        tmem_ld_x32(tO + lane_addr + half * 32, o);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(o_free);   // the next item's first product may overwrite O now
        float lse = (m * p.scale_log2 + log2f(l)) * 0.6931471805599453f;  // natural log
        float inv = 1.f / l;
        if (p.sink_lse) {
          const float sl = p.sink_lse[h];
          const float tot = fmaxf(lse, sl) + log1pf(__expf(-fabsf(lse - sl)));
          inv *= __expf(lse - tot);
          lse = tot;
        }
        if (qi < it.q_hi) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(qi) * p.Hq + h) * FA_D + half * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
            dst[v] = w;
            // keep the rounded values (what a quantise pass over the stored tensor would read)
            o[8 * v + 0] = w.x << 16; o[8 * v + 1] = w.x & 0xffff0000u;
            o[8 * v + 2] = w.y << 16; o[8 * v + 3] = w.y & 0xffff0000u;
            o[8 * v + 4] = w.z << 16; o[8 * v + 5] = w.z & 0xffff0000u;
            o[8 * v + 6] = w.w << 16; o[8 * v + 7] = w.w & 0xffff0000u;
          }
          if (p.q8) {
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(__uint_as_float(o[e])));
            const uint32_t e8 = ue8m0_from_amax(amax);
            const float qs = inv_scale_from_ue8m0(e8);
            uint32_t b[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(o[4 * j]) * qs, __uint_as_float(o[4 * j + 1]) * qs), __NV_SATFINITE, __NV_E4M3);
              const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(o[4 * j + 2]) * qs, __uint_as_float(o[4 * j + 3]) * qs), __NV_SATFINITE, __NV_E4M3);
              b[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
            }
            const int ncols = p.Hq * FA_D;
            uint4* qd = reinterpret_cast<uint4*>(p.q8 + static_cast<size_t>(qi) * ncols + h * FA_D + half * 32);
            qd[0] = make_uint4(b[0], b[1], b[2], b[3]);
            qd[1] = make_uint4(b[4], b[5], b[6], b[7]);
            p.sf[sf_offset(qi, h * 2 + half, ncols >> 7)] = static_cast<uint8_t>(e8);
          }
          if (half == 0) p.lse[static_cast<size_t>(h) * p.T + qi] = lse;
        }
      }
      g += n_kv;
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

}  // namespace kwu

using namespace kwu;

KWU_API int kwu_attn_plan(const int* cu_seqlens, int ndocs, int tile, void* plan, int max_tiles,
                          void* stream) {
  if (ndocs <= 0 || max_tiles <= 0) return 0;
  const size_t smem = static_cast<size_t>(max_tiles) * sizeof(int4) + (ndocs + 1) * sizeof(int);
  if (smem > 96 * 1024) {
    set_last_error("attn_plan: too many tiles / documents (%d / %d)", max_tiles, ndocs);
    return 7;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static PerDeviceOnce attr;
  if (smem > 48 * 1024 && attr.pending()) {
    cudaFuncSetAttribute(attn_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr.mark();
  }
  attn_plan_kernel<<<1, 256, smem, st>>>(cu_seqlens, ndocs, tile, reinterpret_cast<int4*>(plan), max_tiles); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("attn_plan launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

static int flash_fwd_impl(const void* q, int q_ld, const void* k, int k_ld, const void* v, int v_ld,
                          void* out, float* lse, const void* plan, int n_tiles, int T, int Hq, int Hkv,
                          int window, const float* sink_lse, float scale, void* q8, void* sf, void* stream,
                          int* status) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (q8 && (T % 128 || (Hq * FA_D) % 128 || !sf)) {
    set_last_error("flash_fwd: the fp8 copy needs tokens and Hq * 64 in multiples of 128");
    return 7;
  }
  if (Hq % Hkv) { set_last_error("flash_fwd: Hq must be a multiple of Hkv"); return 7; }
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if ((rc = encode_tmap_2d(&tmQ, q, ELEM_BF16, T, (uint64_t)Hq * FA_D, q_ld, FA_BM, FA_D, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_tmap_2d(&tmK, k, ELEM_BF16, T, (uint64_t)Hkv * FA_D, k_ld, FA_BN, FA_D, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_tmap_2d(&tmV, v, ELEM_BF16, T, (uint64_t)Hkv * FA_D, v_ld, FA_BN, FA_D, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  static PerDeviceOnce attr;
  if (attr.pending()) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM);
    if (e != cudaSuccess) { set_last_error("flash_fwd attr: %s", cudaGetErrorString(e)); return 10; }
    attr.mark();
  }
  FlashFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.plan = reinterpret_cast<const int4*>(plan);
  p.n_tiles = n_tiles;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.window = window;
  p.sink_lse = sink_lse;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.q8 = reinterpret_cast<uint8_t*>(q8);
  p.sf = reinterpret_cast<uint8_t*>(sf);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long items = static_cast<long long>(n_tiles) * Hq;
  int grid = static_cast<int>(items < 2LL * sms ? items : 2LL * sms);   // two resident CTAs per SM, each walks the item list
  launch_k(flash_fwd_kernel, dim3(grid), dim3(FA_THREADS), FA_SMEM, reinterpret_cast<cudaStream_t>(stream), tmQ, tmK, tmV, p); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("flash_fwd launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

KWU_API int kwu_flash_fwd(const void* q, int q_ld, const void* k, int k_ld, const void* v, int v_ld,
                          void* out, float* lse, const void* plan, int n_tiles, int T, int Hq, int Hkv,
                          int window, const float* sink_lse, float scale, void* stream, int* status) {
  return flash_fwd_impl(q, q_ld, k, k_ld, v, v_ld, out, lse, plan, n_tiles, T, Hq, Hkv, window, sink_lse, scale,
                        nullptr, nullptr, stream, status);
}

// As kwu_flash_fwd, and also writes the MXFP8 copy of `out` viewed as (T, Hq * 64): q8 (T, Hq * 64) e4m3 bytes and
// sf, kwu_mxfp8_sf_bytes(T, Hq * 64) bytes of scale chunks. T must be a multiple of 128 (every row of every
// scale chunk is then written: each token belongs to exactly one query tile).
KWU_API int kwu_flash_fwd_mx(const void* q, int q_ld, const void* k, int k_ld, const void* v, int v_ld,
                             void* out, float* lse, const void* plan, int n_tiles, int T, int Hq, int Hkv,
                             int window, const float* sink_lse, float scale, void* q8, void* sf, void* stream,
                             int* status) {
  return flash_fwd_impl(q, q_ld, k, k_ld, v, v_ld, out, lse, plan, n_tiles, T, Hq, Hkv, window, sink_lse, scale,
                        q8, sf, stream, status);
}
