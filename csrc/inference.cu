// Serving kernels for sm_100a: single-query (decode) attention against a grouped-query KV cache, and batched token
// sampling.  Both are memory / latency bound (no tensor-core shape), so they are plain CUDA-core kernels laid out so
// that every K / V byte of the cache is read exactly once per step.
//
// * ats_decode_attn: one new query token per sequence.  Grid (key chunk of 256, kv head, sequence); a CTA scores its
//   256 keys for every query head of the group (K read once per group, not once per query head), does the softmax of
//   the chunk in shared memory and reduces P V; a second kernel merges the chunks (flash-decoding).  The new token's
//   K / V are written into the cache by the CTA whose chunk contains that position, so no separate append is needed.
// * ats_sample: repetition penalty -> temperature -> top-k -> top-p -> multinomial (or arg-max when temperature <= 0) for
//   one row of logits per CTA, without sorting: the top-k and top-p cut-offs are found by bisection on the order-preserving
//   integer image of the floats.
//
// The reference has no KV cache (it re-runs the whole context for every token, reference Chat.py:379-452) and samples
// with eager tensor ops (reference Chat.py:391-425); the order of the sampling steps follows that code.
#include "common.cuh"

namespace ats {

constexpr int DEC_CHUNK = 256;
constexpr int DEC_THREADS = 256;

struct DecodeArgs {
  const __nv_bfloat16* q;      // [B, *] packed projection of the new token; head h at q + b * ld_qkv + q_col0 + h * D
  const __nv_bfloat16* k_new;  // same buffer, k_col0 / v_col0
  const __nv_bfloat16* v_new;
  long long ld_qkv;
  __nv_bfloat16* k_cache;  // [B, max_len, Hkv, D]
  __nv_bfloat16* v_cache;
  long long cache_b_stride;  // elements between sequences
  const int* lengths;        // [B] tokens already cached per sequence, or nullptr -> `length` for all
  int length;
  int B, Hq, Hkv, D, max_len;
  float scale;
  float* part_o;   // [B, Hq, n_chunks, D]
  float* part_ml;  // [B, Hq, n_chunks, 2]
  int n_chunks;
  __nv_bfloat16* out;  // [B, Hq * D]
};

template <int D, int REP>
__global__ void __launch_bounds__(DEC_THREADS) decode_attn_kernel(const DecodeArgs p) {
  __shared__ float s_q[REP][D];
  __shared__ float s_p[REP][DEC_CHUNK];
  __shared__ float s_red[DEC_THREADS / (D / 2)][REP][D];
  const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_old = p.lengths ? p.lengths[b] : p.length;
  const int n_tot = n_old + 1;  // the new token attends to itself
  const int k0 = chunk * DEC_CHUNK;
  const bool active = k0 < n_tot;
  const int k_end = min(k0 + DEC_CHUNK, n_tot);

  // query heads of the group -> shared memory (fp32, pre-scaled)
  for (int i = tid; i < REP * D; i += DEC_THREADS) {
    const int h = i / D, d = i % D;
    s_q[h][d] = __bfloat162float(p.q[(long long)b * p.ld_qkv + (hk * REP + h) * D + d]) * p.scale;
  }
  // the new token's K / V row goes into the cache (by the CTA that owns its position)
  __nv_bfloat16* kc = p.k_cache + (long long)b * p.cache_b_stride + (long long)hk * D;
  __nv_bfloat16* vc = p.v_cache + (long long)b * p.cache_b_stride + (long long)hk * D;
  const long long row_stride = (long long)p.Hkv * D;
  if (active && n_old >= k0 && n_old < k0 + DEC_CHUNK && n_old < p.max_len) {
    for (int d = tid; d < D; d += DEC_THREADS) {
      kc[n_old * row_stride + d] = p.k_new[(long long)b * p.ld_qkv + hk * D + d];
      vc[n_old * row_stride + d] = p.v_new[(long long)b * p.ld_qkv + hk * D + d];
    }
  }
  __syncthreads();

  // ---- scores: thread t <-> key k0 + t
  float acc[REP];
#pragma unroll
  for (int h = 0; h < REP; ++h) acc[h] = -INFINITY;
  const int key = k0 + tid;
  if (active && key < k_end) {
#pragma unroll
    for (int h = 0; h < REP; ++h) acc[h] = 0.f;
    const __nv_bfloat16* krow = (key == n_old) ? p.k_new + (long long)b * p.ld_qkv + hk * D : kc + key * row_stride;
#pragma unroll
    for (int d8 = 0; d8 < D / 8; ++d8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(krow + d8 * 8);
      const float2 a = unpack_bf16x2(kv.x), bq = unpack_bf16x2(kv.y), c = unpack_bf16x2(kv.z), e = unpack_bf16x2(kv.w);
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float* qh = &s_q[h][d8 * 8];
        acc[h] += a.x * qh[0] + a.y * qh[1] + bq.x * qh[2] + bq.y * qh[3] + c.x * qh[4] + c.y * qh[5] + e.x * qh[6] + e.y * qh[7];
      }
    }
  }
#pragma unroll
  for (int h = 0; h < REP; ++h) s_p[h][tid] = acc[h];
  __syncthreads();
  // ---- chunk softmax: warp h handles head h (REP <= 8 = number of warps)
  if (warp < REP) {
    float m = -INFINITY;
    for (int i = lane; i < DEC_CHUNK; i += 32) m = fmaxf(m, s_p[warp][i]);
    m = warp_max(m);
    float l = 0.f;
    for (int i = lane; i < DEC_CHUNK; i += 32) {
      const float e = (m == -INFINITY) ? 0.f : __expf(s_p[warp][i] - m);
      s_p[warp][i] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) {
      float* ml = p.part_ml + (((long long)b * p.Hq + hk * REP + warp) * p.n_chunks + chunk) * 2;
      ml[0] = m;
      ml[1] = l;
    }
  }
  __syncthreads();
  // ---- P V: thread (g, dp) sums keys g, g + G, ... for dims 2 dp, 2 dp + 1 of every head
  constexpr int TPR = D / 2, G = DEC_THREADS / TPR;
  const int g = tid / TPR, dp = tid % TPR;
  float o0[REP], o1[REP];
#pragma unroll
  for (int h = 0; h < REP; ++h) o0[h] = o1[h] = 0.f;
  if (active) {
    for (int kk = k0 + g; kk < k_end; kk += G) {
      const __nv_bfloat16* vrow = (kk == n_old) ? p.v_new + (long long)b * p.ld_qkv + hk * D : vc + kk * row_stride;
      const float2 vv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(vrow + 2 * dp));
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float pr = s_p[h][kk - k0];
        o0[h] += pr * vv.x;
        o1[h] += pr * vv.y;
      }
    }
  }
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    s_red[g][h][2 * dp] = o0[h];
    s_red[g][h][2 * dp + 1] = o1[h];
  }
  __syncthreads();
  for (int i = tid; i < REP * D; i += DEC_THREADS) {
    const int h = i / D, d = i % D;
    float t = 0.f;
#pragma unroll
    for (int gg = 0; gg < G; ++gg) t += s_red[gg][h][d];
    p.part_o[(((long long)b * p.Hq + hk * REP + h) * p.n_chunks + chunk) * D + d] = t;
  }
}

// one warp per (sequence, query head): merge the chunk partials
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int BH, int n_chunks, int D) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= BH) return;
  const float* ml = part_ml + (long long)w * n_chunks * 2;
  float m = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) m = fmaxf(m, ml[2 * c]);
  float l = 0.f;
  for (int c = 0; c < n_chunks; ++c) l += ml[2 * c + 1] * ((ml[2 * c] == -INFINITY) ? 0.f : __expf(ml[2 * c] - m));
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = lane; d < D; d += 32) {
    float t = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
      const float f = (ml[2 * c] == -INFINITY) ? 0.f : __expf(ml[2 * c] - m);
      t += part_o[((long long)w * n_chunks + c) * D + d] * f;
    }
    out[(long long)w * D + d] = __float2bfloat16(t * inv);
  }
}

// ------------------------------------------------------------------------------------------------ sampling
__device__ __forceinline__ uint32_t f2key(float f) {  // order-preserving map float -> uint
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int SMP_THREADS = 1024;

struct SampleArgs {
  const void* logits;  // [B, V] bf16 or fp32
  int logits_fp32;
  long long ld;
  float* work;  // [B, V] fp32 scratch (penalised, temperature-scaled logits)
  const long long* history;  // [B, hist_len] token ids or nullptr
  int hist_len, hist_ld;
  const float* uniform;  // [B] in [0, 1)
  long long* out;        // [B]
  int V;
  float temperature, top_p, rep_penalty;
  int top_k;
};

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const SampleArgs p) {
  __shared__ float red[33];
  __shared__ int s_arg, s_pick;
  __shared__ float s_scan[SMP_THREADS / 32 + 1];
  const int b = blockIdx.x, tid = threadIdx.x, V = p.V;
  float* w = p.work + (long long)b * V;
  // pass 0: copy to fp32
  for (int i = tid; i < V; i += SMP_THREADS)
    w[i] = p.logits_fp32 ? static_cast<const float*>(p.logits)[b * p.ld + i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p.logits)[b * p.ld + i]);
  __syncthreads();
  // repetition penalty on the distinct tokens of the window (a token listed twice is penalised once)
  if (p.history && p.rep_penalty != 1.f) {
    for (int j = tid; j < p.hist_len; j += SMP_THREADS) {
      const long long tok = p.history[(long long)b * p.hist_ld + j];
      bool first = tok >= 0 && tok < V;
      for (int jj = 0; first && jj < j; ++jj) first = p.history[(long long)b * p.hist_ld + jj] != tok;
      if (first) {
        const float x = w[tok];
        w[tok] = x > 0.f ? x / p.rep_penalty : x * p.rep_penalty;
      }
    }
    __syncthreads();
  }
  // arg-max (lowest index on ties) -- also the greedy answer
  float mx = -INFINITY;
  for (int i = tid; i < V; i += SMP_THREADS) mx = fmaxf(mx, w[i]);
  mx = block_max(mx, red);
  if (tid == 0) s_arg = V;
  __syncthreads();
  for (int i = tid; i < V; i += SMP_THREADS)
    if (w[i] == mx) atomicMin(&s_arg, i);
  __syncthreads();
  if (p.temperature <= 0.f) {
    if (tid == 0) p.out[b] = s_arg;
    return;
  }
  const float inv_t = 1.f / p.temperature;
  // top-k cut-off: largest key t with count(key >= t) >= k  (bisection over the 32 key bits)
  uint32_t cut = 0u;
  if (p.top_k > 0 && p.top_k < V) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t trial = cut | (1u << bit);
      int c = 0;
      for (int i = tid; i < V; i += SMP_THREADS) c += f2key(w[i]) >= trial;
      const float tot = block_sum(float(c), red);  // counts <= 2^24 are exact in fp32
      if (tot >= float(p.top_k)) cut = trial;
    }
  }
  // normaliser over the top-k set, at temperature
  float z = 0.f;
  for (int i = tid; i < V; i += SMP_THREADS)
    if (f2key(w[i]) >= cut) z += __expf((w[i] - mx) * inv_t);
  z = block_sum(z, red);
  // top-p cut-off: smallest key t with mass(key > t) <= top_p * z; elements with key >= t are kept
  uint32_t pcut = cut;
  if (p.top_p < 1.f) {
    // bisection for the smallest t in [cut, max key] satisfying the predicate (it holds at t = max key: mass above is 0)
    uint32_t lo = cut, hi = f2key(mx);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      float above = 0.f;
      for (int i = tid; i < V; i += SMP_THREADS) {
        const uint32_t kk = f2key(w[i]);
        if (kk > mid) above += __expf((w[i] - mx) * inv_t);
      }
      above = block_sum(above, red);
      if (above <= p.top_p * z) hi = mid;
      else lo = mid + 1;
    }
    pcut = lo;
  }
  // multinomial over the kept set, in index order: contiguous segment per thread + block scan
  const int seg = (V + SMP_THREADS - 1) / SMP_THREADS;
  const int i0 = tid * seg, i1 = min(i0 + seg, V);
  float local = 0.f;
  for (int i = i0; i < i1; ++i)
    if (f2key(w[i]) >= pcut) local += __expf((w[i] - mx) * inv_t);
  // inclusive scan over threads
  float incl = local;
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    float v = s_scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    s_scan[lane] = v;
    if (lane == 31) s_scan[32] = v;
  }
  __syncthreads();
  const float base = (warp ? s_scan[warp - 1] : 0.f) + incl - local;
  const float total = s_scan[32];
  const float target = p.uniform[b] * total;
  if (tid == 0) s_pick = V;
  __syncthreads();
  if (local > 0.f && target >= base && target < base + local) {
    float run = base;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      if (f2key(w[i]) >= pcut) {
        run += __expf((w[i] - mx) * inv_t);
        pick = i;
        if (target < run) break;
      }
    }
    if (pick >= 0) atomicMin(&s_pick, pick);
  }
  __syncthreads();
  // rounding can leave the target just past the last kept element: fall back to the arg-max, which is always kept
  if (tid == 0) p.out[b] = s_pick < V ? s_pick : s_arg;
}

}  // namespace ats

using namespace ats;

template <int D, int REP>
static int launch_decode(const DecodeArgs& p, cudaStream_t s) {
  dim3 grid(p.n_chunks, p.Hkv, p.B);
  decode_attn_kernel<D, REP><<<grid, DEC_THREADS, 0, s>>>(p);
  return int(cudaGetLastError());
}

// Scratch sizes for `ats_decode_attn`: floats needed for part_o and part_ml with a cache of `max_len` positions.
ATS_API int ats_decode_attn_chunks(int max_len) { return (max_len + DEC_CHUNK - 1) / DEC_CHUNK; }

// qkv: packed projection of the new token [B, ld_qkv]; caches [B, max_len, Hkv, D] (batch stride cache_b_stride elements).
// lengths: per-sequence cached lengths (device int32) or nullptr for the common `length`.  out: [B, Hq * D] bf16.
ATS_API int ats_decode_attn(const void* qkv, long long ld_qkv, int q_col0, int k_col0, int v_col0, void* k_cache, void* v_cache,
                            long long cache_b_stride, const int* lengths, int length, int max_tokens, int B, int Hq, int Hkv, int D,
                            int max_len, float* part_o, float* part_ml, void* out, void* stream) {
  if ((D != 64 && D != 128) || Hq % Hkv || ((q_col0 | k_col0 | v_col0) & 7) || (ld_qkv & 7)) return 1003;
  const int rep = Hq / Hkv;
  DecodeArgs p;
  const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(qkv);
  p.q = base + q_col0; p.k_new = base + k_col0; p.v_new = base + v_col0;
  p.ld_qkv = ld_qkv;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache); p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.cache_b_stride = cache_b_stride;
  p.lengths = lengths; p.length = length;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.max_len = max_len;
  p.scale = 1.f / sqrtf(float(D));
  p.part_o = part_o; p.part_ml = part_ml;
  // chunks to launch: enough for the longest sequence (+ the new token)
  p.n_chunks = (min(max_tokens + 1, max_len) + DEC_CHUNK - 1) / DEC_CHUNK;
  if (p.n_chunks < 1) p.n_chunks = 1;
  p.out = static_cast<__nv_bfloat16*>(out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int e = 1004;
#define ATS_DEC(DD, RR) if (D == DD && rep == RR) e = launch_decode<DD, RR>(p, s);
  ATS_DEC(64, 1) ATS_DEC(64, 2) ATS_DEC(64, 4) ATS_DEC(64, 8) ATS_DEC(128, 1) ATS_DEC(128, 2) ATS_DEC(128, 4) ATS_DEC(128, 8)
#undef ATS_DEC
  if (e) return e;
  const int BH = B * Hq;
  decode_merge_kernel<<<(BH * 32 + 255) / 256, 256, 0, s>>>(part_o, part_ml, p.out, BH, p.n_chunks, D);
  return int(cudaGetLastError());
}

// logits [B, V] (row pitch ld elements; fp32 when logits_fp32 else bf16) -> out [B] int64.  work: [B, V] fp32 scratch;
// history: [B, hist_len] int64 (row pitch hist_ld) or nullptr; uniform: [B] fp32 in [0, 1).
ATS_API int ats_sample(const void* logits, int logits_fp32, long long ld, float* work, const long long* history, int hist_len,
                       int hist_ld, const float* uniform, long long* out, int B, int V, float temperature, int top_k, float top_p,
                       float rep_penalty, void* stream) {
  if (B <= 0 || V <= 0) return 1003;
  SampleArgs p;
  p.logits = logits; p.logits_fp32 = logits_fp32; p.ld = ld; p.work = work;
  p.history = history; p.hist_len = hist_len; p.hist_ld = hist_ld;
  p.uniform = uniform; p.out = out; p.V = V;
  p.temperature = temperature; p.top_p = top_p; p.rep_penalty = rep_penalty; p.top_k = top_k;
  sample_kernel<<<B, SMP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return int(cudaGetLastError());
}
