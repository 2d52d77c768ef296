// Expert-parallel dispatch and combine over NVLink peer memory (plain peer loads and stores; no
// multimem, no TMA on peer memory).
//
// E experts are split over W ranks (El = E / W consecutive experts per rank). Every rank routes its own
// T tokens, then:
//
//   ep_plan      each rank writes its per-expert pair counts into every peer's `table[src][E]` and raises
//                a flag; after all W rows have arrived every rank derives, from the same table and hence
//                identically, (a) as a DESTINATION: 128-row-padded offsets of its El experts, the tile
//                table for the grouped GEMMs and the number of real rows per expert (inside an expert's
//                range the rows are ordered by source rank); (b) as a SOURCE: for every global expert the
//                first row, inside the owner's receive buffer, of the segment reserved for this rank.
//   ep_dispatch  every (token, slot) pair takes the next row of its segment and the token's activation
//                row is written straight into the owner's receive buffer with 16-byte peer stores.
//   ep_barrier   "my stores to you are finished" / "my outputs are ready": one flag per (kind, peer),
//                holding a monotonically increasing epoch that lives on the device, so the same launch
//                sequence can be replayed from a CUDA graph.
//   ep_copy_rows receive buffer -> private rows (padding rows zeroed), or private rows -> output buffer.
//   scatter map  ep_copy_rows also turns the (source rank, pair) tag that ep_dispatch left beside every row into
//                the address of that pair's slot in the SOURCE's per-pair buffer. The expert GEMMs take the map
//                as their epilogue target (gemm_bf16.cu / mxfp8.cu `row_ptrs`): the second expert GEMM stores
//                its output rows, and in backward the first GEMM's dgrad its input-gradient rows, straight into
//                the sources' memory while later tiles are still in the tensor cores. The source then only
//                sums its own k slots per token (moe_combine on local memory).
//   ep_combine   out[t] = sum_slot w[t,slot] * yout_owner[pos(t,slot)], read with 16-byte peer loads: a
//                per-token gather-sum (no atomics, result independent of arrival order). Optionally keeps
//                the gathered rows for the gate-weight gradient.
//   ep_combine_bwd  pushes w * dout[t] into the owner's receive buffer and forms d_w = <y_row, dout[t]>.
//
// Buffer reuse across layers is safe without further barriers: a source only starts the next layer's
// dispatch after its combine, which follows the owner's "outputs ready" flag, which the owner raises
// after it has copied its received rows out of the receive buffer.
// A rank whose receive rows would exceed `cap` records KWU_ERR_EP_OVERFLOW in the status word; pairs
// beyond the capacity are dropped (pos = -1) and counted, never written out of bounds.
// All waits are bounded (clock64 limit -> KWU_ERR_TIMEOUT_FLAG in the status word, kernel returns).
// Takes the place of the all-to-all dispatch/combine around the reference's expert GEMMs
// (src/kohakuwullm/kernels/moe/moe_dispatch.py:14-130; expert parallelism itself has no reference
// implementation, only the config row that names it).
#include "common.cuh"

namespace kwu {

constexpr int EP_MAX_WORLD = 8;
constexpr int EP_MAX_E = 128;
enum : int { EP_FLAG_COUNTS = 0, EP_FLAG_ARRIVED = 1, EP_FLAG_OUTPUT = 2, EP_NUM_FLAGS = 3 };

struct EpPeers {
  int* table[EP_MAX_WORLD];            // [W][E] int32 on every rank
  int* flags[EP_MAX_WORLD];            // [EP_NUM_FLAGS][W] int32 on every rank
  __nv_bfloat16* xrecv[EP_MAX_WORLD];  // [cap][D] rows arriving at the owner
  __nv_bfloat16* yout[EP_MAX_WORLD];   // [cap][D] rows the sources read back
  int* meta[EP_MAX_WORLD];             // [cap] (source rank << 28 | pair index) of every row at the owner
  __nv_bfloat16* ypairs[EP_MAX_WORLD]; // [T*k][D] per-pair rows at the SOURCE, written by the owners' GEMM epilogues
};

__device__ __forceinline__ void ep_st_release(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ep_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Signal every peer's flag (kind, my rank) with the next epoch and wait for all peers' signals.
// Must be called by all threads of a block with blockDim.x >= world. Returns false on time-out.
__device__ bool ep_signal_and_wait(const EpPeers& pe, int* epochs, int kind, int rank, int world, int* status,
                                   long long limit_cycles) {
  __shared__ int s_epoch, s_ok;
  if (threadIdx.x == 0) {
    s_epoch = epochs[kind] + 1;
    epochs[kind] = s_epoch;
    s_ok = 1;
  }
  __threadfence_system();
  __syncthreads();
  const int epoch = s_epoch;
  if (threadIdx.x < world) {
    ep_st_release(pe.flags[threadIdx.x] + kind * world + rank, epoch);
    const int* f = pe.flags[rank] + kind * world + threadIdx.x;
    const long long t0 = clock64();
    while (ep_ld_acquire(f) < epoch) {
      if (clock64() - t0 > limit_cycles) {
        s_ok = 0;
        if (status) atomicCAS(status, 0, KWU_ERR_TIMEOUT_FLAG);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

struct EpPlanArgs {
  EpPeers peers;
  const int* counts;   // [E] pairs of this rank per global expert
  int* epochs;         // [EP_NUM_FLAGS] device-resident epoch counters
  int rank, world, E, El, cap;
  int* offsets;        // [El + 1] padded row offsets of the local experts; offsets[El] = rows in use
  int* totals;         // [El] real rows per local expert
  int4* tiles;         // [max_tiles] (m0, local expert, valid, 0)
  int max_tiles;
  int* send_base;      // [E] first row of this rank's segment in the owner's buffer
  int* cursors;        // [E] zeroed
  long long limit_cycles;
  int fatal_overflow;  // 1: an owner over capacity sets the overflow code; 0: the excess pairs are dropped and counted
  int* status;
};

__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpPlanArgs a) {
  __shared__ int s_tab[EP_MAX_WORLD * EP_MAX_E];
  __shared__ int s_off[EP_MAX_E + EP_MAX_WORLD];  // padded offset of every global expert inside its owner
  const int W = a.world, E = a.E, El = a.El;
  // publish this rank's counts into every peer's table row `rank`
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) {
    const int p = i / E, e = i % E;
    a.peers.table[p][a.rank * E + e] = a.counts[e];
  }
  const bool ok = ep_signal_and_wait(a.peers, a.epochs, EP_FLAG_COUNTS, a.rank, W, a.status, a.limit_cycles);
  for (int i = threadIdx.x; i < W * E; i += blockDim.x)
    s_tab[i] = ok ? ep_ld_acquire(a.peers.table[a.rank] + i) : 0;
  __syncthreads();
  // per owner: exclusive prefix over its local experts of the 128-padded totals
  if (threadIdx.x < W) {
    const int r = threadIdx.x;
    int acc = 0;
    for (int le = 0; le < El; ++le) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += s_tab[s * E + r * El + le];
      s_off[r * El + le] = acc;
      acc += (tot + 127) / 128 * 128;
    }
    s_off[E + r] = acc;  // rows in use on owner r
    if (acc > a.cap && a.status && a.fatal_overflow) atomicCAS(a.status, 0, KWU_ERR_EP_OVERFLOW);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < a.rank; ++s) before += s_tab[s * E + e];
    a.send_base[e] = s_off[e] + before;
    a.cursors[e] = 0;
  }
  // destination side
  const int used = min(s_off[E + a.rank], a.cap / 128 * 128);
  for (int le = threadIdx.x; le <= El; le += blockDim.x) {
    if (le < El) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += s_tab[s * E + a.rank * El + le];
      a.totals[le] = tot;
      a.offsets[le] = min(s_off[a.rank * El + le], used);
    } else {
      a.offsets[El] = used;
    }
  }
  for (int i = threadIdx.x; i < a.max_tiles; i += blockDim.x) {
    const int m0 = i * 128;
    int4 t = make_int4(0, 0, 0, 0);
    if (m0 < used) {
      int le = 0;
      while (le + 1 < El && s_off[a.rank * El + le + 1] <= m0) ++le;
      t = make_int4(m0, le, 1, 0);
    }
    a.tiles[i] = t;
  }
}

// One warp per (token, slot) pair.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const EpPeers pe, const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ idx,
                   int n_pairs, int top_k, const int* __restrict__ send_base, int* __restrict__ cursors,
                   int* __restrict__ pos_of, int D, int El, int cap, int rank, int* __restrict__ dropped) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * wpb) {
    const int e = idx[i];
    int pos = 0;
    if (lane == 0) pos = send_base[e] + atomicAdd(&cursors[e], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= cap) {
      if (lane == 0) {
        pos_of[i] = -1;
        if (dropped) atomicAdd(dropped, 1);   // pairs of this rank that found no room at their owner
      }
      continue;
    }
    if (lane == 0) {
      pos_of[i] = pos;
      pe.meta[e / El][pos] = (rank << 28) | i;   // where the owner's GEMM epilogues send this row's results
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(i / top_k) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(pe.xrecv[e / El] + static_cast<size_t>(pos) * D);
    for (int v = lane; v < D / 8; v += 32) dst[v] = src[v];
  }
}

__global__ void ep_barrier_kernel(const EpPeers pe, int* epochs, int kind, int rank, int world, int* status,
                                  long long limit_cycles) {
  ep_signal_and_wait(pe, epochs, kind, rank, world, status, limit_cycles);
}

// dst[r] = (r is a real row) ? src[r] : 0 for r < offsets[El]. zero_pad = 0 copies everything in use.
__global__ void __launch_bounds__(256)
ep_copy_rows_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                    const int* __restrict__ offsets, const int* __restrict__ totals, int El, int D, int zero_pad,
                    const EpPeers pe, const int* __restrict__ meta, long long* __restrict__ row_ptrs) {
  __shared__ int s_off[EP_MAX_E + 1], s_tot[EP_MAX_E];
  for (int i = threadIdx.x; i <= El; i += blockDim.x) {
    s_off[i] = offsets[i];
    if (i < El) s_tot[i] = totals[i];
  }
  __syncthreads();
  const int used = s_off[El];
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < used; r += gridDim.x * wpb) {
    bool real = true;
    if (zero_pad) {
      int le = 0;
      while (le + 1 < El && s_off[le + 1] <= r) ++le;
      real = (r - s_off[le]) < s_tot[le];
    }
    if (row_ptrs && lane == 0) {
      // where this row's results go: the source rank's per-pair buffer, seen through THIS rank's mapping
      long long addr = 0;
      if (real) {
        const int tag = meta[r];
        addr = reinterpret_cast<long long>(pe.ypairs[tag >> 28] + static_cast<size_t>(tag & 0x0fffffff) * D);
      }
      row_ptrs[r] = addr;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * D);
    uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * D);
    for (int v = lane; v < D / 8; v += 32) d[v] = real ? s[v] : make_uint4(0, 0, 0, 0);
  }
}

// out[t] = sum_slot w * yout_owner[pos]; w null: plain sum. keep (optional): gathered rows per pair.
__global__ void __launch_bounds__(256)
ep_combine_kernel(const EpPeers pe, const int* __restrict__ pos_of, const int* __restrict__ idx,
                  const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int ldo,
                  __nv_bfloat16* __restrict__ keep, int T, int top_k, int D, int El) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    for (int v = lane; v < D / 8; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < top_k; ++s) {
        const int pair = t * top_k + s;
        const int pos = pos_of[pair];
        uint4 a = make_uint4(0, 0, 0, 0);
        if (pos >= 0) a = reinterpret_cast<const uint4*>(pe.yout[idx[pair] / El] + static_cast<size_t>(pos) * D)[v];
        if (keep) reinterpret_cast<uint4*>(keep + static_cast<size_t>(pair) * D)[v] = a;
        const float ws = w ? w[pair] : 1.f;
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

// One warp per pair: owner.xrecv[pos] = w * dout[t]; d_w[pair] = <kept_row, dout[t]>.
__global__ void __launch_bounds__(256)
ep_combine_bwd_kernel(const EpPeers pe, const __nv_bfloat16* __restrict__ dout, int lddo,
                      const __nv_bfloat16* __restrict__ kept, const int* __restrict__ pos_of,
                      const int* __restrict__ idx, const float* __restrict__ w, float* __restrict__ d_w,
                      int n_pairs, int top_k, int D, int El) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * wpb) {
    const int pos = pos_of[i];
    if (pos < 0) {
      if (lane == 0 && d_w) d_w[i] = 0.f;
      continue;
    }
    const float ws = w[i];
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(i / top_k) * lddo);
    const uint4* y = reinterpret_cast<const uint4*>(kept + static_cast<size_t>(i) * D);
    uint4* dst = reinterpret_cast<uint4*>(pe.xrecv[idx[i] / El] + static_cast<size_t>(pos) * D);
    float dot = 0.f;
    for (int v = lane; v < D / 8; v += 32) {
      const uint4 gv = g[v], yv = y[v];
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 gf = unpack_bf16(gw[e]), yf = unpack_bf16(yw[e]);
        dot += gf.x * yf.x + gf.y * yf.y;
        o[e] = pack_bf16(ws * gf.x, ws * gf.y);
      }
      dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    dot = warp_sum(dot);
    if (lane == 0 && d_w) d_w[i] = dot;
  }
}

static inline int ep_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("%s launch: %s", what, cudaGetErrorString(e)); return 11; }
  return 0;
}

static bool ep_fill(EpPeers& pe, const long long* table, const long long* flags, const long long* xrecv,
                    const long long* yout, const long long* meta, const long long* ypairs, int world) {
  if (world < 1 || world > EP_MAX_WORLD) { set_last_error("ep: world size %d not in [1, 8]", world); return false; }
  for (int p = 0; p < EP_MAX_WORLD; ++p) {
    const bool in = p < world;
    pe.table[p] = in ? reinterpret_cast<int*>(table[p]) : nullptr;
    pe.flags[p] = in ? reinterpret_cast<int*>(flags[p]) : nullptr;
    pe.xrecv[p] = in ? reinterpret_cast<__nv_bfloat16*>(xrecv[p]) : nullptr;
    pe.yout[p] = in ? reinterpret_cast<__nv_bfloat16*>(yout[p]) : nullptr;
    pe.meta[p] = in ? reinterpret_cast<int*>(meta[p]) : nullptr;
    pe.ypairs[p] = in ? reinterpret_cast<__nv_bfloat16*>(ypairs[p]) : nullptr;
  }
  return true;
}

}  // namespace kwu

using namespace kwu;

// Sizes of the symmetric blocks, in int32 elements.
KWU_API int kwu_ep_table_ints(int world, int E) { return world * E; }
KWU_API int kwu_ep_flag_ints() { return EP_NUM_FLAGS * EP_MAX_WORLD; }

KWU_API int kwu_ep_plan(const long long* table_ptrs, const long long* flag_ptrs, const long long* xrecv_ptrs,
                        const long long* yout_ptrs, const long long* meta_ptrs, const long long* ypairs_ptrs, const int* counts, int* epochs, int rank, int world, int E,
                        int cap, int* offsets, int* totals, void* tiles, int max_tiles, int* send_base,
                        int* cursors, long long limit_cycles, int fatal_overflow, void* stream, int* status) {
  EpPlanArgs a;
  if (!ep_fill(a.peers, table_ptrs, flag_ptrs, xrecv_ptrs, yout_ptrs, meta_ptrs, ypairs_ptrs, world)) return 7;
  if (E > EP_MAX_E || E % world) { set_last_error("ep_plan: need E <= 128 and E %% world == 0"); return 7; }
  a.counts = counts; a.epochs = epochs; a.rank = rank; a.world = world; a.E = E; a.El = E / world; a.cap = cap;
  a.offsets = offsets; a.totals = totals; a.tiles = reinterpret_cast<int4*>(tiles); a.max_tiles = max_tiles;
  a.send_base = send_base; a.cursors = cursors;
  a.limit_cycles = limit_cycles > 0 ? limit_cycles : KWU_WAIT_LIMIT_CYCLES;
  a.fatal_overflow = fatal_overflow;
  a.status = status;
  ep_plan_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a); kwu::count_launch();
  return ep_check("ep_plan");
}

KWU_API int kwu_ep_dispatch(const long long* table_ptrs, const long long* flag_ptrs, const long long* xrecv_ptrs,
                            const long long* yout_ptrs, const long long* meta_ptrs, const long long* ypairs_ptrs, int world, const void* x, int ldx, const int* idx,
                            int n_pairs, int top_k, const int* send_base, int* cursors, int* pos_of, int D, int El,
                            int cap, int rank, int* dropped, void* stream) {
  EpPeers pe;
  if (!ep_fill(pe, table_ptrs, flag_ptrs, xrecv_ptrs, yout_ptrs, meta_ptrs, ypairs_ptrs, world)) return 7;
  if (D % 8) { set_last_error("ep_dispatch: D must be a multiple of 8"); return 7; }
  if (n_pairs >= (1 << 28)) { set_last_error("ep_dispatch: too many pairs for the row tags"); return 7; }
  if (n_pairs <= 0) return 0;
  ep_dispatch_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pe, (const __nv_bfloat16*)x, ldx, idx, n_pairs, top_k, send_base, cursors, pos_of, D, El, cap, rank, dropped); kwu::count_launch();
  return ep_check("ep_dispatch");
}

KWU_API int kwu_ep_barrier(const long long* table_ptrs, const long long* flag_ptrs, const long long* xrecv_ptrs,
                           const long long* yout_ptrs, const long long* meta_ptrs, const long long* ypairs_ptrs, int* epochs, int kind, int rank, int world,
                           long long limit_cycles, void* stream, int* status) {
  EpPeers pe;
  if (!ep_fill(pe, table_ptrs, flag_ptrs, xrecv_ptrs, yout_ptrs, meta_ptrs, ypairs_ptrs, world)) return 7;
  if (kind < 0 || kind >= EP_NUM_FLAGS) { set_last_error("ep_barrier: unknown flag kind %d", kind); return 7; }
  ep_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pe, epochs, kind, rank, world, status, limit_cycles > 0 ? limit_cycles : KWU_WAIT_LIMIT_CYCLES); kwu::count_launch();
  return ep_check("ep_barrier");
}

// row_ptrs (optional, with zero_pad = 1 on the receive buffer): for every row the address, in this rank's mapping,
// of the per-pair slot at the row's source rank (0 for padding rows); the grouped GEMMs take it as their scatter map.
KWU_API int kwu_ep_copy_rows(const long long* table_ptrs, const long long* flag_ptrs, const long long* xrecv_ptrs,
                             const long long* yout_ptrs, const long long* meta_ptrs, const long long* ypairs_ptrs,
                             int world, int rank, const void* src, void* dst, const int* offsets, const int* totals,
                             int El, int D, int zero_pad, long long* row_ptrs, void* stream) {
  EpPeers pe;
  if (!ep_fill(pe, table_ptrs, flag_ptrs, xrecv_ptrs, yout_ptrs, meta_ptrs, ypairs_ptrs, world)) return 7;
  if (D % 8 || El > EP_MAX_E) { set_last_error("ep_copy_rows: D %% 8 != 0 or too many local experts"); return 7; }
  ep_copy_rows_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, offsets, totals, El, D, zero_pad, pe, pe.meta[rank], row_ptrs); kwu::count_launch();
  return ep_check("ep_copy_rows");
}

KWU_API int kwu_ep_combine(const long long* table_ptrs, const long long* flag_ptrs, const long long* xrecv_ptrs,
                           const long long* yout_ptrs, const long long* meta_ptrs, const long long* ypairs_ptrs, int world, const int* pos_of, const int* idx, const float* w,
                           void* out, int ldo, void* keep, int T, int top_k, int D, int El, void* stream) {
  EpPeers pe;
  if (!ep_fill(pe, table_ptrs, flag_ptrs, xrecv_ptrs, yout_ptrs, meta_ptrs, ypairs_ptrs, world)) return 7;
  if (D % 8) { set_last_error("ep_combine: D must be a multiple of 8"); return 7; }
  if (T <= 0) return 0;
  int grid = (T + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  ep_combine_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pe, pos_of, idx, w, (__nv_bfloat16*)out, ldo, (__nv_bfloat16*)keep, T, top_k, D, El); kwu::count_launch();
  return ep_check("ep_combine");
}

KWU_API int kwu_ep_combine_bwd(const long long* table_ptrs, const long long* flag_ptrs, const long long* xrecv_ptrs,
                               const long long* yout_ptrs, const long long* meta_ptrs, const long long* ypairs_ptrs, int world, const void* dout, int lddo, const void* kept,
                               const int* pos_of, const int* idx, const float* w, float* d_w, int n_pairs, int top_k,
                               int D, int El, void* stream) {
  EpPeers pe;
  if (!ep_fill(pe, table_ptrs, flag_ptrs, xrecv_ptrs, yout_ptrs, meta_ptrs, ypairs_ptrs, world)) return 7;
  if (D % 8) { set_last_error("ep_combine_bwd: D must be a multiple of 8"); return 7; }
  if (n_pairs <= 0) return 0;
  ep_combine_bwd_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pe, (const __nv_bfloat16*)dout, lddo, (const __nv_bfloat16*)kept, pos_of, idx, w, d_w, n_pairs, top_k, D, El); kwu::count_launch();
  return ep_check("ep_combine_bwd");
}
