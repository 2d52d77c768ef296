// Single-token decode attention over a KV cache (head_dim 64, bf16, GQA).
//
//   q      (B, H, 64)                 the new token's queries (already normalised and rotated)
//   kcache (B, L_max, Hkv, 64), vcache same; only keys [lo, kv_len) are read, lo = kv_len - window when
//                                     the layer has a sliding window (the query sits at kv_len - 1)
//   out    (B, H, 64) bf16, lse (B, H) fp32 (natural log, sink included when given)
//
// The op is bandwidth bound: every key/value row of the cache is read exactly once per KV head and
// shared by the `group = H / Hkv` query heads of that KV head. Split-KV: one CTA per (256-key chunk, KV
// head, batch row):
//   phase 1  thread t owns key lo + chunk*256 + t: its 128-byte K row is read with eight 16-byte loads
//            and dotted with the group's queries (staged in shared memory as fp32, scale * log2e folded);
//   phase 2  chunk max / exp2 / sum per head in shared memory;
//   phase 3  lane = pair of output channels, warps stride over the keys: V rows are read as coalesced
//            128-byte lines, p-weighted sums for all heads of the group stay in registers, warps reduce
//            through shared memory.
// Partials (m, l, acc[64]) go to a scratch buffer; `decode_combine` merges the chunks, folds the learned
// sink logits into the denominator and writes bf16. No tensor cores: one query row per head has no
// contraction worth a tile. Takes the place of the mask-free one-row SDPA decode path of the reference
// (src/kohakuwullm/models/components/attention.py:224-291).
#include "common.cuh"

namespace kwu {

constexpr int DEC_D = 64;
constexpr int DEC_CHUNK = 256;
constexpr int DEC_MAX_GROUP = 8;

struct DecodeParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  long long q_sb, q_sh;             // element strides of q: batch, head
  long long k_sb, k_sl, k_sh;       // element strides of the caches: batch, position, kv head
  long long v_sb, v_sl, v_sh;
  int B, H, Hkv, group;
  int kv_len, lo;                   // keys [lo, kv_len)
  int n_chunks;
  float scale_log2e;
  float* part;                      // [B][H][n_chunks][66]: m, l, acc[64]
};

__global__ void __launch_bounds__(DEC_CHUNK)
decode_chunk_kernel(const DecodeParams p) {
  __shared__ float s_q[DEC_MAX_GROUP][DEC_D];
  __shared__ float s_p[DEC_MAX_GROUP][DEC_CHUNK];
  __shared__ float s_red[DEC_MAX_GROUP][8];
  __shared__ float s_m[DEC_MAX_GROUP], s_l[DEC_MAX_GROUP];
  __shared__ float s_acc[8][DEC_MAX_GROUP][DEC_D];
  const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.group;
  for (int i = tid; i < G * DEC_D; i += DEC_CHUNK) {
    const int g = i / DEC_D, d = i % DEC_D;
    s_q[g][d] = __bfloat162float(p.q[b * p.q_sb + (hk * G + g) * p.q_sh + d]) * p.scale_log2e;
  }
  __syncthreads();
  // phase 1: scores (log2 domain)
  const int key = p.lo + chunk * DEC_CHUNK + tid;
  const bool valid = key < p.kv_len;
  float s[DEC_MAX_GROUP];
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) s[g] = 0.f;
  if (valid) {
    const uint4* kr = reinterpret_cast<const uint4*>(p.k + b * p.k_sb + static_cast<long long>(key) * p.k_sl + hk * p.k_sh);
#pragma unroll
    for (int c = 0; c < DEC_D / 8; ++c) {
      const uint4 a = kr[c];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16(w[e]);
#pragma unroll
        for (int g = 0; g < DEC_MAX_GROUP; ++g)
          if (g < G) s[g] += f.x * s_q[g][c * 8 + 2 * e] + f.y * s_q[g][c * 8 + 2 * e + 1];
      }
    }
  }
  // phase 2: chunk max, exp2, sum per head
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) {
    if (g < G) {
      const float m = warp_max(valid ? s[g] : -INFINITY);
      if (lane == 0) s_red[g][warp] = m;
    }
  }
  __syncthreads();
  if (tid < G) {
    float m = -INFINITY;
    for (int w = 0; w < 8; ++w) m = fmaxf(m, s_red[tid][w]);
    s_m[tid] = m;
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) {
    if (g < G) {
      const float m = s_m[g];
      const float pv = (valid && m > -INFINITY) ? exp2f(s[g] - m) : 0.f;
      s_p[g][tid] = pv;
      const float sum = warp_sum(pv);
      if (lane == 0) s_red[g][warp] = sum;  // safe: every thread passed the barrier after reading s_red
    }
  }
  __syncthreads();
  if (tid < G) {
    float l = 0.f;
    for (int w = 0; w < 8; ++w) l += s_red[tid][w];
    s_l[tid] = l;
  }
  // phase 3: acc[g][d] = sum_j p[g][j] * V[j][d]; lane owns channels 2*lane, 2*lane+1
  float acc[DEC_MAX_GROUP][2];
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) acc[g][0] = acc[g][1] = 0.f;
  const int n_here = min(DEC_CHUNK, p.kv_len - (p.lo + chunk * DEC_CHUNK));
  for (int j = warp; j < n_here; j += 8) {
    const long long pos = p.lo + chunk * DEC_CHUNK + j;
    const uint32_t vv = *reinterpret_cast<const uint32_t*>(p.v + b * p.v_sb + pos * p.v_sl + hk * p.v_sh + 2 * lane);
    const float2 f = unpack_bf16(vv);
#pragma unroll
    for (int g = 0; g < DEC_MAX_GROUP; ++g) {
      if (g < G) {
        const float pj = s_p[g][j];
        acc[g][0] += pj * f.x;
        acc[g][1] += pj * f.y;
      }
    }
  }
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) {
    if (g < G) {
      s_acc[warp][g][2 * lane] = acc[g][0];
      s_acc[warp][g][2 * lane + 1] = acc[g][1];
    }
  }
  __syncthreads();
  for (int i = tid; i < G * DEC_D; i += DEC_CHUNK) {
    const int g = i / DEC_D, d = i % DEC_D;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += s_acc[w][g][d];
    float* dst = p.part + ((static_cast<size_t>(b) * p.H + hk * G + g) * p.n_chunks + chunk) * 66;
    dst[2 + d] = t;
    if (d == 0) {
      dst[0] = s_m[g];
      dst[1] = s_l[g];
    }
  }
}

// One block of 64 threads per (batch, head): merge the chunks.
__global__ void __launch_bounds__(64)
decode_combine_kernel(const float* __restrict__ part, int n_chunks, const float* __restrict__ sink, int n_sinks,
                      __nv_bfloat16* __restrict__ out, long long o_sb, long long o_sh, float* __restrict__ lse,
                      int H) {
  const int bh = blockIdx.x;
  const int b = bh / H, h = bh % H;
  const int d = threadIdx.x;
  const float* base = part + static_cast<size_t>(bh) * n_chunks * 66;
  float m = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) m = fmaxf(m, base[c * 66]);
  float l = 0.f, acc = 0.f;
  if (m > -INFINITY) {
    for (int c = 0; c < n_chunks; ++c) {
      const float mc = base[c * 66];
      if (mc == -INFINITY) continue;
      const float w = exp2f(mc - m);
      l += base[c * 66 + 1] * w;
      acc += base[c * 66 + 2 + d] * w;
    }
  }
  // learned sink logits join the denominator only (natural-log logits; m is in the log2 domain)
  constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  float m2 = m;
  if (sink) {
    for (int s = 0; s < n_sinks; ++s) m2 = fmaxf(m2, sink[h * n_sinks + s] * LOG2E);
  }
  float denom = (m > -INFINITY) ? l * exp2f(m - m2) : 0.f;
  if (sink)
    for (int s = 0; s < n_sinks; ++s) denom += exp2f(sink[h * n_sinks + s] * LOG2E - m2);
  const float o = (denom > 0.f && m > -INFINITY) ? acc * exp2f(m - m2) / denom : 0.f;
  out[b * o_sb + h * o_sh + d] = __float2bfloat16(o);
  if (d == 0 && lse) lse[bh] = (denom > 0.f) ? (m2 + log2f(denom)) * LN2 : -INFINITY;
}

}  // namespace kwu

using namespace kwu;

// Floats of scratch needed for (B, H) rows and up to `max_keys` attended keys.
KWU_API long long kwu_decode_scratch_floats(int B, int H, int max_keys) {
  const long long chunks = (max_keys + DEC_CHUNK - 1) / DEC_CHUNK;
  return static_cast<long long>(B) * H * (chunks > 0 ? chunks : 1) * 66;
}

// Strides are in elements. window <= 0: all keys [0, kv_len). sink: (H, n_sinks) fp32 logits or null.
KWU_API int kwu_decode_attention(const void* q, long long q_sb, long long q_sh, const void* k, long long k_sb,
                                 long long k_sl, long long k_sh, const void* v, long long v_sb, long long v_sl,
                                 long long v_sh, void* out, long long o_sb, long long o_sh, float* lse, float* scratch,
                                 int B, int H, int Hkv, int kv_len, int window, float scale, const float* sink,
                                 int n_sinks, void* stream) {
  if (Hkv <= 0 || H % Hkv || H / Hkv > DEC_MAX_GROUP) { set_last_error("decode_attention: need H %% Hkv == 0 and group <= 8"); return 7; }
  if (kv_len <= 0 || B <= 0) { set_last_error("decode_attention: empty cache"); return 7; }
  if ((k_sl % 8) || (k_sh % 8) || (k_sb % 8) || (v_sl % 2) || (v_sh % 2)) { set_last_error("decode_attention: cache rows must be 16-byte aligned"); return 7; }
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.q_sb = q_sb; p.q_sh = q_sh; p.k_sb = k_sb; p.k_sl = k_sl; p.k_sh = k_sh; p.v_sb = v_sb; p.v_sl = v_sl; p.v_sh = v_sh;
  p.B = B; p.H = H; p.Hkv = Hkv; p.group = H / Hkv;
  p.kv_len = kv_len;
  p.lo = (window > 0 && kv_len > window) ? kv_len - window : 0;
  p.n_chunks = (kv_len - p.lo + DEC_CHUNK - 1) / DEC_CHUNK;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.part = scratch;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  decode_chunk_kernel<<<dim3(p.n_chunks, Hkv, B), DEC_CHUNK, 0, st>>>(p); kwu::count_launch();
  decode_combine_kernel<<<B * H, 64, 0, st>>>(scratch, p.n_chunks, sink, n_sinks, (__nv_bfloat16*)out, o_sb, o_sh, lse, H); kwu::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_last_error("decode_attention launch: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}
