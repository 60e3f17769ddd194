// Mixture-of-Depths token routing for training: router scores, selection bookkeeping, row gather, weighted scatter-add and
// their backward passes.  All of it is memory-bound row movement around the dense SwiGLU GEMMs of the selected tokens:
//   forward   scores[t] = (h[t] . w + b) / temperature                      (one pass over h, warp per token)
//             sel = the `keep` best positions of every sequence, ascending  (mod_rank_kernel + mod_compact_kernel in moe.cu)
//             picked[j] = h[token(j)], weight[j] = sigmoid(scores[token(j)]), slot_of[token(j)] = j
//             aux = mean binary cross-entropy of sigmoid(scores) against membership in the selected set
//             out[t] = base[t] + (slot_of[t] >= 0 ? weight[slot] * y[slot] : 0)
//   backward  dy[j] = weight[j] * dout[token(j)],  dweight[j] = <dout[token(j)], y[j]>
//             ds[t] = (daux * (sigmoid(s) - member) / T + (member ? dweight * sigmoid'(s) : 0)) / temperature
//             dh[t] = ds[t] * w + (member ? dpicked[slot] : 0)               (one pass, written once)
//             dw = sum_t ds[t] h[t],  db = sum_t ds[t]
// The reference does this with eager PyTorch (core/model.py:860-1020: nn.Linear router, torch.topk over the whole batch,
// boolean-mask gather, index_add scatter).
#include "common.cuh"

namespace ats {

constexpr int kModMaxHidden = 16384;

// ---- scores ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mod_scores_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                  float* __restrict__ scores, long long tokens, int hidden, float inv_temp) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const float b = bias ? __bfloat162float(bias[0]) : 0.f;
  for (long long t = warp; t < tokens; t += nwarps) {
    const uint4* row = reinterpret_cast<const uint4*>(h + t * hidden);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    float acc = 0.f;
    for (int c = lane; c < hidden / 8; c += 32) {
      const uint4 p = row[c], q = __ldg(wr + c);
      const float2 p0 = unpack_bf16x2(p.x), p1 = unpack_bf16x2(p.y), p2 = unpack_bf16x2(p.z), p3 = unpack_bf16x2(p.w);
      const float2 q0 = unpack_bf16x2(q.x), q1 = unpack_bf16x2(q.y), q2 = unpack_bf16x2(q.z), q3 = unpack_bf16x2(q.w);
      acc += p0.x * q0.x + p0.y * q0.y + p1.x * q1.x + p1.y * q1.y + p2.x * q2.x + p2.y * q2.y + p3.x * q3.x + p3.y * q3.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) scores[t] = (acc + b) * inv_temp;
  }
}

// ---- gather of the selected rows -------------------------------------------------------------------------------------
// One warp per selected slot j = b * keep + i: token = b * seq_len + sel[j].
__global__ void __launch_bounds__(256)
mod_gather_kernel(const __nv_bfloat16* __restrict__ h, const int* __restrict__ sel, const float* __restrict__ scores,
                  __nv_bfloat16* __restrict__ picked, float* __restrict__ weight, int* __restrict__ slot_of, long long slots, int keep,
                  int seq_len, int hidden) {
  const int lane = threadIdx.x & 31;
  const long long j = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j >= slots) return;
  const int pos = sel[j];
  if (!ATS_DBG_CHECK(pos >= 0 && pos < seq_len, kDbgModRows, j)) return;
  const long long t = (j / keep) * seq_len + pos;
  const uint4* src = reinterpret_cast<const uint4*>(h + t * hidden);
  uint4* dst = reinterpret_cast<uint4*>(picked + j * hidden);
  for (int c = lane; c < hidden / 8; c += 32) dst[c] = src[c];
  if (lane == 0) {
    weight[j] = 1.f / (1.f + __expf(-scores[t]));
    slot_of[t] = int(j);
  }
}

// ---- auxiliary loss: mean BCE-with-logits against membership -------------------------------------------------------------
__global__ void __launch_bounds__(1024)
mod_aux_kernel(const float* __restrict__ scores, const int* __restrict__ slot_of, float* __restrict__ aux, long long tokens) {
  __shared__ float red[33];
  float acc = 0.f;
  for (long long t = threadIdx.x; t < tokens; t += blockDim.x) {
    const float s = scores[t];
    const float y = slot_of[t] >= 0 ? 1.f : 0.f;
    acc += fmaxf(s, 0.f) - s * y + log1pf(__expf(-fabsf(s)));  // the numerically stable form of BCE-with-logits
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) aux[0] = acc / float(tokens);
}

// ---- out = base + scatter(weight * y) ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mod_scatter_kernel(const __nv_bfloat16* __restrict__ base, const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_of,
                   const float* __restrict__ weight, __nv_bfloat16* __restrict__ out, long long tokens, int hidden) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long t = warp; t < tokens; t += nwarps) {
    const int slot = slot_of[t];
    uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
    if (slot < 0) {
      if (base) {
        const uint4* src = reinterpret_cast<const uint4*>(base + t * hidden);
        for (int c = lane; c < hidden / 8; c += 32) dst[c] = src[c];
      } else {
        for (int c = lane; c < hidden / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      }
      continue;
    }
    const float wgt = weight[slot];
    const uint4* yr = reinterpret_cast<const uint4*>(y + (long long)slot * hidden);
    const uint4* src = base ? reinterpret_cast<const uint4*>(base + t * hidden) : nullptr;
    for (int c = lane; c < hidden / 8; c += 32) {
      const uint4 v = yr[c];
      const uint4 r = src ? src[c] : make_uint4(0, 0, 0, 0);
      const float2 v0 = unpack_bf16x2(v.x), v1 = unpack_bf16x2(v.y), v2 = unpack_bf16x2(v.z), v3 = unpack_bf16x2(v.w);
      const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
      uint4 o;
      o.x = pack_bf16x2(r0.x + wgt * v0.x, r0.y + wgt * v0.y);
      o.y = pack_bf16x2(r1.x + wgt * v1.x, r1.y + wgt * v1.y);
      o.z = pack_bf16x2(r2.x + wgt * v2.x, r2.y + wgt * v2.y);
      o.w = pack_bf16x2(r3.x + wgt * v3.x, r3.y + wgt * v3.y);
      dst[c] = o;
    }
  }
}

// ---- backward of the scatter: dy and the gradient of the token weight -----------------------------------------------------
__global__ void __launch_bounds__(256)
mod_scatter_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y, const int* __restrict__ sel,
                       const float* __restrict__ weight, __nv_bfloat16* __restrict__ dy, float* __restrict__ dweight, long long slots,
                       int keep, int seq_len, int hidden) {
  const int lane = threadIdx.x & 31;
  const long long j = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j >= slots) return;
  const int pos = sel[j];
  if (!ATS_DBG_CHECK(pos >= 0 && pos < seq_len, kDbgModRows, j)) return;
  const long long t = (j / keep) * seq_len + pos;
  const float wgt = weight[j];
  const uint4* g = reinterpret_cast<const uint4*>(dout + t * hidden);
  const uint4* yr = reinterpret_cast<const uint4*>(y + j * hidden);
  uint4* dst = reinterpret_cast<uint4*>(dy + j * hidden);
  float dot = 0.f;
  for (int c = lane; c < hidden / 8; c += 32) {
    const uint4 a = g[c], v = yr[c];
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 v0 = unpack_bf16x2(v.x), v1 = unpack_bf16x2(v.y), v2 = unpack_bf16x2(v.z), v3 = unpack_bf16x2(v.w);
    dot += a0.x * v0.x + a0.y * v0.y + a1.x * v1.x + a1.y * v1.y + a2.x * v2.x + a2.y * v2.y + a3.x * v3.x + a3.y * v3.y;
    uint4 o;
    o.x = pack_bf16x2(wgt * a0.x, wgt * a0.y);
    o.y = pack_bf16x2(wgt * a1.x, wgt * a1.y);
    o.z = pack_bf16x2(wgt * a2.x, wgt * a2.y);
    o.w = pack_bf16x2(wgt * a3.x, wgt * a3.y);
    dst[c] = o;
  }
  dot = warp_sum(dot);
  if (lane == 0) dweight[j] = dot;
}

// ---- backward of the routing: the one dh tensor and the score gradient ---------------------------------------------------------
__global__ void __launch_bounds__(256)
mod_route_bwd_kernel(const __nv_bfloat16* __restrict__ dpicked, const int* __restrict__ slot_of, const float* __restrict__ scores,
                     const float* __restrict__ dweight, const float* __restrict__ daux, const float* __restrict__ dscores_ext,
                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ dh, float* __restrict__ ds_out, long long tokens,
                     int hidden, float inv_temp) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const float ga = daux ? daux[0] / float(tokens) : 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (long long t = warp; t < tokens; t += nwarps) {
    const int slot = slot_of[t];
    const float s = scores[t];
    const float sg = 1.f / (1.f + __expf(-s));
    float ds = ga * (sg - (slot >= 0 ? 1.f : 0.f));
    if (slot >= 0 && dweight) ds += dweight[slot] * sg * (1.f - sg);
    if (dscores_ext) ds += dscores_ext[t];
    ds *= inv_temp;  // scores = raw / temperature
    if (lane == 0) ds_out[t] = ds;
    const uint4* dp = (slot >= 0 && dpicked) ? reinterpret_cast<const uint4*>(dpicked + (long long)slot * hidden) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(dh + t * hidden);
    for (int c = lane; c < hidden / 8; c += 32) {
      const uint4 q = __ldg(wr + c);
      const uint4 r = dp ? dp[c] : make_uint4(0, 0, 0, 0);
      const float2 q0 = unpack_bf16x2(q.x), q1 = unpack_bf16x2(q.y), q2 = unpack_bf16x2(q.z), q3 = unpack_bf16x2(q.w);
      const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
      uint4 o;
      o.x = pack_bf16x2(r0.x + ds * q0.x, r0.y + ds * q0.y);
      o.y = pack_bf16x2(r1.x + ds * q1.x, r1.y + ds * q1.y);
      o.z = pack_bf16x2(r2.x + ds * q2.x, r2.y + ds * q2.y);
      o.w = pack_bf16x2(r3.x + ds * q3.x, r3.y + ds * q3.y);
      dst[c] = o;
    }
  }
}

// ---- router weight gradient: dw[c] = sum_t ds[t] h[t, c], db = sum_t ds[t] ------------------------------------------------------
// Every CTA walks a contiguous run of tokens; a thread owns 8 columns (looping when hidden > 8 * blockDim) and writes its sums into
// the CTA's row of `partial` [gridDim.x, hidden + 8] (column `hidden` holds the CTA's sum of ds); a second launch adds the rows up.
__global__ void __launch_bounds__(256)
mod_router_wgrad_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ ds, float* __restrict__ partial, long long tokens,
                        int hidden, int rows_per_cta) {
  const long long t0 = (long long)blockIdx.x * rows_per_cta;
  const long long t1 = t0 + rows_per_cta < tokens ? t0 + rows_per_cta : tokens;
  float* prow = partial + (long long)blockIdx.x * (hidden + 8);
  for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (long long t = t0; t < t1; ++t) {
      const float d = ds[t];
      const uint4 p = reinterpret_cast<const uint4*>(h + t * hidden)[c];
      const float2 p0 = unpack_bf16x2(p.x), p1 = unpack_bf16x2(p.y), p2 = unpack_bf16x2(p.z), p3 = unpack_bf16x2(p.w);
      acc[0] += d * p0.x; acc[1] += d * p0.y; acc[2] += d * p1.x; acc[3] += d * p1.y;
      acc[4] += d * p2.x; acc[5] += d * p2.y; acc[6] += d * p3.x; acc[7] += d * p3.y;
    }
    *reinterpret_cast<float4*>(prow + c * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(prow + c * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (long long t = t0; t < t1; ++t) s += ds[t];
    prow[hidden] = s;
  }
}

__global__ void __launch_bounds__(256)
mod_colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int width, int pitch) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += partial[(long long)r * pitch + c];
  out[c] = s;
}

}  // namespace ats

using namespace ats;

static inline unsigned warp_grid(long long warps, unsigned cap) {
  const long long blocks = (warps + 7) / 8;
  return unsigned(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

ATS_API int ats_mod_scores(const void* h, const void* w, const void* bias, float* scores, long long tokens, int hidden, float inv_temp,
                           void* stream) {
  if ((hidden & 7) || hidden > kModMaxHidden) return 1003;
  if (tokens == 0) return 0;
  mod_scores_kernel<<<warp_grid(tokens, 148 * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias), scores, tokens,
      hidden, inv_temp);
  return int(cudaGetLastError());
}

// slot_of must hold -1 everywhere on entry; aux may be null.
ATS_API int ats_mod_gather(const void* h, const int* sel, const float* scores, void* picked, float* weight, int* slot_of, float* aux,
                           int batch, int seq_len, int keep, int hidden, void* stream) {
  if ((hidden & 7) || keep > seq_len) return 1003;
  const long long slots = (long long)batch * keep, tokens = (long long)batch * seq_len;
  if (slots == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  mod_gather_kernel<<<unsigned((slots + 7) / 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(h), sel, scores,
                                                              static_cast<__nv_bfloat16*>(picked), weight, slot_of, slots, keep, seq_len,
                                                              hidden);
  if (aux) mod_aux_kernel<<<1, 1024, 0, s>>>(scores, slot_of, aux, tokens);
  return int(cudaGetLastError());
}

ATS_API int ats_mod_scatter(const void* base, const void* y, const int* slot_of, const float* weight, void* out, long long tokens,
                            int hidden, void* stream) {
  if (hidden & 7) return 1003;
  if (tokens == 0) return 0;
  mod_scatter_kernel<<<warp_grid(tokens, 148 * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(base), static_cast<const __nv_bfloat16*>(y), slot_of, weight, static_cast<__nv_bfloat16*>(out),
      tokens, hidden);
  return int(cudaGetLastError());
}

ATS_API int ats_mod_scatter_bwd(const void* dout, const void* y, const int* sel, const float* weight, void* dy, float* dweight, int batch,
                                int seq_len, int keep, int hidden, void* stream) {
  if ((hidden & 7) || keep > seq_len) return 1003;
  const long long slots = (long long)batch * keep;
  if (slots == 0) return 0;
  mod_scatter_bwd_kernel<<<unsigned((slots + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(y), sel, weight, static_cast<__nv_bfloat16*>(dy), dweight,
      slots, keep, seq_len, hidden);
  return int(cudaGetLastError());
}

// dwb: hidden + 1 floats (router weight gradient, then the bias gradient); partial: scratch of ats_mod_wgrad_ctas() * (hidden + 8)
// floats; dpicked, dweight, daux, dscores_ext may each be null.
ATS_API int ats_mod_wgrad_ctas() { return 296; }
ATS_API int ats_mod_route_bwd(const void* h, const void* dpicked, const int* slot_of, const float* scores, const float* dweight,
                              const float* daux, const float* dscores_ext, const void* w, void* dh, float* ds, float* dwb, float* partial,
                              long long tokens, int hidden, float inv_temp, void* stream) {
  if ((hidden & 7) || hidden > kModMaxHidden) return 1003;
  if (tokens == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  mod_route_bwd_kernel<<<warp_grid(tokens, 148 * 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dpicked), slot_of, scores, dweight,
                                                                   daux, dscores_ext, static_cast<const __nv_bfloat16*>(w),
                                                                   static_cast<__nv_bfloat16*>(dh), ds, tokens, hidden, inv_temp);
  const int ctas = int(tokens < 296 ? tokens : 296);
  const int rows = int((tokens + ctas - 1) / ctas);
  const int used = int((tokens + rows - 1) / rows);
  mod_router_wgrad_kernel<<<used, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(h), ds, partial, tokens, hidden, rows);
  mod_colsum_kernel<<<(hidden + 1 + 255) / 256, 256, 0, s>>>(partial, dwb, used, hidden + 1, hidden + 8);
  return int(cudaGetLastError());
}
