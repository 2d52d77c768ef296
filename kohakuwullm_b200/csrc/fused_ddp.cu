// Data-parallel gradient reduce-scatter, partitioned AdamW and parameter all-gather as two kernels
// over NVLink peer memory (plain peer loads and stores; no multimem, no TMA).
//
// Every rank keeps its flat fp32 gradient buffer and its flat parameter buffer in symmetric
// (peer-mapped) memory. Rank r owns the contiguous shard [r*n/W, (r+1)*n/W) of every buffer:
//
//   ddp_reduce_shard      waits until every peer's gradients are final (flag epoch), then for each
//                         element of the OWN shard sums the W peers' gradients with 16-byte peer loads
//                         in a fixed rank order (so every rank would compute bit-identical sums),
//                         stores the sum into the local buffer, accumulates the shard's sum of squares
//                         deterministically, and publishes it to every peer's slot table.
//   ddp_adamw_allgather   waits for all W slots (which also proves every peer has finished READING this
//                         rank's gradients), forms the global norm and the clip coefficient
//                         scale = inv_tokens * min(1, max_norm / norm), applies AdamW to the own shard
//                         (fp32 master / exp_avg / exp_avg_sq live only on the owner), stores the new
//                         low-precision parameters into EVERY peer's parameter buffer with 16-byte peer
//                         stores, zeroes the whole local gradient buffer, and finally signals and waits
//                         for the closing barrier so that kernel completion implies that all peers'
//                         shards have landed in this rank's parameters.
//
// Flag protocol: flags only ever hold the step's epoch number (monotonically increasing), so nothing
// is reset between steps. All waits are bounded; on a time-out the kernel records
// KWU_ERR_TIMEOUT_FLAG in the status word and returns, and a reduction that timed out (or that found the
// status word already set) does not publish its norm, so no rank applies the update of that step. The division by the global trained-token count
// happens here (inv_tokens is a device scalar), which is what makes gradient accumulation token-exact
// without a host round trip. Takes the place of torch DDP's bucketed NCCL all-reduce followed by a
// separate optimizer pass (scripts/train/lm.py:383-398, src/kohakuwullm/training/optim/fused_adamw.py
// of the reference).
#include "common.cuh"

namespace kwu {

constexpr int DDP_MAX_WORLD = 8;

struct DdpPeers {
  const float* grad[DDP_MAX_WORLD];  // every rank's gradient buffer (peer-mapped), own rank included
  void* param[DDP_MAX_WORLD];        // every rank's parameter buffer
  int* flags[DDP_MAX_WORLD];         // every rank's flag block: [ready W][sq_flag W][done W] ints
  float* slots[DDP_MAX_WORLD];       // every rank's sum-of-squares slots: W floats
};

constexpr int FLAG_READY = 0, FLAG_SQ = 1, FLAG_DONE = 2;

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until flags[kind*W + p] >= epoch for every p. One thread per peer polls; returns false on time-out.
__device__ bool wait_all_flags(const int* flags, int kind, int world, int epoch, int* status,
                               long long limit_cycles) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* f = flags + kind * world + threadIdx.x;
    const long long t0 = clock64();
    while (ld_acquire_sys(f) < epoch) {
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

struct ReduceArgs {
  DdpPeers peers;
  int rank, world, epoch;
  long long lo, n;          // own shard [lo, lo + n) in elements (n % 4 == 0)
  float* local_grad;        // == peers.grad[rank], writable
  float* partial;           // gridDim.x floats
  unsigned int* counter;    // zero-initialised, self-resetting
  float* sumsq;             // local device scalar accumulated across calls of one step
  int first, publish;       // first: overwrite sumsq; publish: send sumsq to all peers afterwards
  int signal_ready;         // announce "my gradients are final" (once per step)
  long long limit_cycles;
  int* status;
};

__global__ void __launch_bounds__(512)
ddp_reduce_shard_kernel(const ReduceArgs a) {
  __shared__ float s_red[16];
  __shared__ int s_last;
  if (a.signal_ready && blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.peers.flags[threadIdx.x] + FLAG_READY * a.world + a.rank, a.epoch);
  }
  const bool ok = wait_all_flags(a.peers.flags[a.rank], FLAG_READY, a.world, a.epoch, a.status, a.limit_cycles);
  float acc = 0.f;
  if (ok) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < a.n; i += stride) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < DDP_MAX_WORLD; ++p) {
        if (p < a.world) {
          const float4 v = *reinterpret_cast<const float4*>(a.peers.grad[p] + a.lo + i);
          s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
      }
      *reinterpret_cast<float4*>(a.local_grad + a.lo + i) = s;
      acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  }
  // deterministic two-level sum of squares: block partials, then the last block adds them in order
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += s_red[w];
    a.partial[blockIdx.x] = t;
    __threadfence();
    const unsigned int done = atomicAdd(a.counter, 1u);
    s_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence();
    float t = 0.f;
    for (unsigned int b = 0; b < gridDim.x; ++b) t += a.partial[b];
    const float total = a.first ? t : (*a.sumsq + t);
    *a.sumsq = total;
    *a.counter = 0;
    // A block whose wait ran out has written the status word before it added itself to the counter. The sum is
    // then NOT published: every rank's ddp_adamw_allgather runs out of time waiting for it and leaves the
    // parameters untouched, instead of stepping on gradients that were never reduced.
    const bool healthy = !a.status || *reinterpret_cast<volatile int*>(a.status) == 0;
    if (a.publish && healthy) {
      for (int p = 0; p < a.world; ++p) a.peers.slots[p][a.rank] = total;
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) st_release_sys(a.peers.flags[p] + FLAG_SQ * a.world + a.rank, a.epoch);
    }
  }
}

struct AdamArgs {
  DdpPeers peers;
  int rank, world, epoch;
  long long lo, n, total;   // shard [lo, lo+n), whole buffer length
  float* local_grad;
  float* master;            // shard-local fp32 master (null: the fp32 parameters are their own master)
  float* m;
  float* v;
  int param_is_bf16;
  const long long* seg_start;   // whole-buffer coordinates
  const float* seg_wd;
  const float* seg_lr_mult;
  int nseg;
  const float* inv_tokens;  // device scalar
  float max_norm;
  float* norm_out;          // device scalar (optional)
  float lr, beta1, beta2, eps, bc1_inv, bc2_inv_sqrt;
  unsigned int* counter;
  int wait_sq, finish;      // wait_sq: first group of the step; finish: closing barrier after this group
  int zero_all_grads;
  long long limit_cycles;
  int* status;
};

__device__ __forceinline__ int seg_of(const long long* __restrict__ seg_start, int nseg, long long i) {
  int lo = 0, hi = nseg - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seg_start[mid] <= i) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(512)
ddp_adamw_allgather_kernel(const AdamArgs a) {
  __shared__ int s_last;
  const bool ok = wait_all_flags(a.peers.flags[a.rank], FLAG_SQ, a.world, a.epoch, a.status, a.limit_cycles);
  if (ok) {
    float total = 0.f;
    for (int p = 0; p < a.world; ++p) total += a.peers.slots[a.rank][p];
    const float inv = *a.inv_tokens;
    const float norm = sqrtf(total) * inv;
    float scale = inv;
    if (a.max_norm > 0.f) scale *= fminf(1.f, a.max_norm / (norm + 1e-6f));
    if (a.norm_out && blockIdx.x == 0 && threadIdx.x == 0) *a.norm_out = norm;

    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < a.n; i += stride) {
      const long long gi = a.lo + i;
      const int s = seg_of(a.seg_start, a.nseg, gi);  // tensors start on multiples of 128 elements
      const float wd = a.seg_wd[s];
      const float lr = a.lr * a.seg_lr_mult[s];
      float g[8], p[8], mm[8], vv[8];
      *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(a.local_grad + gi);
      *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(a.local_grad + gi + 4);
      if (a.zero_all_grads) {  // the owner clears its shard as it consumes it
        *reinterpret_cast<float4*>(a.local_grad + gi) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(a.local_grad + gi + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float* mst = a.master ? a.master + i : reinterpret_cast<float*>(a.peers.param[a.rank]) + gi;
      *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(mst);
      *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(mst + 4);
      *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(a.m + i);
      *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(a.m + i + 4);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(a.v + i);
      *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(a.v + i + 4);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float ge = g[e] * scale;
        mm[e] = a.beta1 * mm[e] + (1.f - a.beta1) * ge;
        vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * ge * ge;
        const float denom = sqrtf(vv[e]) * a.bc2_inv_sqrt + a.eps;
        p[e] = p[e] * (1.f - lr * wd) - lr * (mm[e] * a.bc1_inv) / denom;
      }
      *reinterpret_cast<float4*>(a.m + i) = *reinterpret_cast<float4*>(mm);
      *reinterpret_cast<float4*>(a.m + i + 4) = *reinterpret_cast<float4*>(mm + 4);
      *reinterpret_cast<float4*>(a.v + i) = *reinterpret_cast<float4*>(vv);
      *reinterpret_cast<float4*>(a.v + i + 4) = *reinterpret_cast<float4*>(vv + 4);
      if (a.master) {
        *reinterpret_cast<float4*>(a.master + i) = *reinterpret_cast<float4*>(p);
        *reinterpret_cast<float4*>(a.master + i + 4) = *reinterpret_cast<float4*>(p + 4);
      }
      // all-gather: the owner writes the updated values into every rank's parameter buffer
      if (a.param_is_bf16) {
        const uint4 o = make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
#pragma unroll
        for (int r = 0; r < DDP_MAX_WORLD; ++r)
          if (r < a.world) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.peers.param[r]) + gi) = o;
      } else {
#pragma unroll
        for (int r = 0; r < DDP_MAX_WORLD; ++r) {
          if (r < a.world) {
            float* dst = reinterpret_cast<float*>(a.peers.param[r]) + gi;
            *reinterpret_cast<float4*>(dst) = *reinterpret_cast<float4*>(p);
            *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<float4*>(p + 4);
          }
        }
      }
    }
    if (a.zero_all_grads) {
      // every peer has published its slot, i.e. has finished reading this rank's gradients
      const long long zs = static_cast<long long>(gridDim.x) * blockDim.x * 4;
      for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < a.total; i += zs)
        if (i < a.lo || i >= a.lo + a.n)  // the own shard is cleared element by element above
          *reinterpret_cast<float4*>(a.local_grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  __threadfence_system();  // this thread's peer stores are performed before anything that follows
  if (!a.finish) return;
  // closing barrier: the last block to finish tells every peer "my stores to you are done" and waits
  // for the same message from all of them
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(a.counter, 1u);
    s_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *a.counter = 0;
    if (threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys(a.peers.flags[threadIdx.x] + FLAG_DONE * a.world + a.rank, a.epoch);
    }
    wait_all_flags(a.peers.flags[a.rank], FLAG_DONE, a.world, a.epoch, a.status, a.limit_cycles);
  }
}

// Single-GPU check of the bounded wait: nothing ever sets the flag, so the kernel must give up after
// `limit_cycles`, record the time-out in the status word and return.
__global__ void ddp_wait_probe_kernel(const int* flags, int world, int epoch, int* status, long long limit_cycles,
                                      int* result) {
  const bool ok = wait_all_flags(flags, FLAG_READY, world, epoch, status, limit_cycles);
  if (threadIdx.x == 0) *result = ok ? 1 : 0;
}

}  // namespace kwu

using namespace kwu;

static void fill_peers(DdpPeers& pe, const long long* grad, const long long* param, const long long* flags,
                       const long long* slots, int world) {
  for (int p = 0; p < DDP_MAX_WORLD; ++p) {
    const bool in = p < world;
    pe.grad[p] = in ? reinterpret_cast<const float*>(grad[p]) : nullptr;
    pe.param[p] = in ? reinterpret_cast<void*>(param[p]) : nullptr;
    pe.flags[p] = in ? reinterpret_cast<int*>(flags[p]) : nullptr;
    pe.slots[p] = in ? reinterpret_cast<float*>(slots[p]) : nullptr;
  }
}

KWU_API int kwu_ddp_blocks() { return 148 * 2; }

// Pointer tables are host arrays of `world` device addresses (as 64-bit integers).
KWU_API int kwu_ddp_reduce_shard(const long long* grad_ptrs, const long long* param_ptrs, const long long* flag_ptrs,
                                 const long long* slot_ptrs, int rank, int world, int epoch, long long lo,
                                 long long n, float* partial, unsigned int* counter, float* sumsq, int first,
                                 int publish, int signal_ready, long long limit_cycles, void* stream, int* status) {
  if (world < 1 || world > DDP_MAX_WORLD) { set_last_error("ddp: world size %d not in [1, 8]", world); return 7; }
  if (n % 8 || lo % 8) { set_last_error("ddp: shard bounds must be multiples of 8 elements"); return 7; }
  ReduceArgs a;
  fill_peers(a.peers, grad_ptrs, param_ptrs, flag_ptrs, slot_ptrs, world);
  a.rank = rank; a.world = world; a.epoch = epoch; a.lo = lo; a.n = n;
  a.local_grad = const_cast<float*>(a.peers.grad[rank]);
  a.partial = partial; a.counter = counter; a.sumsq = sumsq; a.first = first; a.publish = publish;
  a.signal_ready = signal_ready;
  a.limit_cycles = limit_cycles > 0 ? limit_cycles : KWU_WAIT_LIMIT_CYCLES;
  a.status = status;
  ddp_reduce_shard_kernel<<<kwu_ddp_blocks(), 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("ddp_reduce_shard launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

KWU_API int kwu_ddp_adamw_allgather(const long long* grad_ptrs, const long long* param_ptrs,
                                    const long long* flag_ptrs, const long long* slot_ptrs, int rank, int world,
                                    int epoch, long long lo, long long n, long long total, float* master, float* m,
                                    float* v, int param_is_bf16, const long long* seg_start, const float* seg_wd,
                                    const float* seg_lr_mult, int nseg, const float* inv_tokens, float max_norm,
                                    float* norm_out, float lr, float beta1, float beta2, float eps, int step,
                                    unsigned int* counter, int finish, int zero_all_grads, long long limit_cycles,
                                    void* stream, int* status) {
  if (world < 1 || world > DDP_MAX_WORLD) { set_last_error("ddp: world size %d not in [1, 8]", world); return 7; }
  if (n % 8 || lo % 8 || total % 4) { set_last_error("ddp: shard bounds must be multiples of 8 elements"); return 7; }
  AdamArgs a;
  fill_peers(a.peers, grad_ptrs, param_ptrs, flag_ptrs, slot_ptrs, world);
  a.rank = rank; a.world = world; a.epoch = epoch; a.lo = lo; a.n = n; a.total = total;
  a.local_grad = const_cast<float*>(a.peers.grad[rank]);
  a.master = master; a.m = m; a.v = v; a.param_is_bf16 = param_is_bf16;
  a.seg_start = seg_start; a.seg_wd = seg_wd; a.seg_lr_mult = seg_lr_mult; a.nseg = nseg;
  a.inv_tokens = inv_tokens; a.max_norm = max_norm; a.norm_out = norm_out;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps;
  a.bc1_inv = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  a.bc2_inv_sqrt = 1.f / sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  a.counter = counter; a.wait_sq = 1; a.finish = finish; a.zero_all_grads = zero_all_grads;
  a.limit_cycles = limit_cycles > 0 ? limit_cycles : KWU_WAIT_LIMIT_CYCLES;
  a.status = status;
  ddp_adamw_allgather_kernel<<<kwu_ddp_blocks(), 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("ddp_adamw_allgather launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

KWU_API int kwu_ddp_wait_probe(const int* flags, int world, int epoch, int* status, long long limit_cycles,
                               int* result, void* stream) {
  ddp_wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flags, world, epoch, status, limit_cycles, result); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("ddp_wait_probe launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}
