// LayerNorm (forward / backward) and scaled masked soft-max (padding-mask and causal forms, forward / backward) for
// sm_100a.  All are HBM-bound row kernels: one warp-group per row, bf16 in / out, fp32 arithmetic, 16-byte accesses.
//
// The transformer itself uses RMSNorm and flash attention, so nothing on the training hot path calls these; they
// exist because the model file of the reference exports a LayerNorm module (reference core/model.py:307-327) and its
// vendored kernel set ships a LayerNorm (colossalai extensions csrc/cuda/layer_norm_cuda_kernel.cu:255-474) and the
// Megatron soft-max pair (scaled_masked_softmax_cuda.cu, scaled_upper_triang_masked_softmax_cuda.cu), which the eager
// attention fallback and user models built on the framework's layers rely on.
#include "common.cuh"

namespace ats {

constexpr int LN_THREADS = 256;

// y = (x - mean) * rstd * gamma + beta; saves mean / rstd (fp32) for the backward.
__global__ void __launch_bounds__(LN_THREADS) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                                                   const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                                                   float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows,
                                                                   int H, float eps) {
  __shared__ float red[33];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* xr = x + r * H;
    float s = 0.f, ss = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += LN_THREADS * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]);
        s += f.x + f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
    s = block_sum(s, red);
    ss = block_sum(ss, red);
    const float mean = s / H;
    const float rstd = rsqrtf(fmaxf(ss / H - mean * mean, 0.f) + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[r] = mean;
      if (rstd_out) rstd_out[r] = rstd;
    }
    for (int i = threadIdx.x * 8; i < H; i += LN_THREADS * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
      const uint4 g = *reinterpret_cast<const uint4*>(gamma + i);
      uint4 bb = make_uint4(0, 0, 0, 0);
      if (beta) bb = *reinterpret_cast<const uint4*>(beta + i);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w}, gu[4] = {g.x, g.y, g.z, g.w}, bu[4] = {bb.x, bb.y, bb.z, bb.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]), gg = unpack_bf16x2(gu[j]), be = unpack_bf16x2(bu[j]);
        o[j] = pack_bf16x2((f.x - mean) * rstd * gg.x + be.x, (f.y - mean) * rstd * gg.y + be.y);
      }
      *reinterpret_cast<uint4*>(y + r * H + i) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = dy * gamma; per-CTA partial dgamma / dbeta rows go to
// `partials` [gridDim.x, 2, H] and are summed by colsum (two-stage, deterministic).
__global__ void __launch_bounds__(LN_THREADS) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                                                                   const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                                                   float* __restrict__ partials, long long rows, int H) {
  __shared__ float red[33];
  float* pg = partials + (long long)blockIdx.x * 2 * H;
  float* pb = pg + H;
  for (int i = threadIdx.x; i < 2 * H; i += LN_THREADS) pg[i] = 0.f;
  __syncthreads();
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
    for (int i = threadIdx.x * 2; i < H; i += LN_THREADS * 2) {
      const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + r * H + i));
      const float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + r * H + i));
      const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(gamma + i));
      const float h0 = (xv.x - mu) * rs, h1 = (xv.y - mu) * rs;
      s1 += d.x * g.x + d.y * g.y;
      s2 += d.x * g.x * h0 + d.y * g.y * h1;
    }
    s1 = block_sum(s1, red) / H;
    s2 = block_sum(s2, red) / H;
    for (int i = threadIdx.x * 2; i < H; i += LN_THREADS * 2) {
      const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + r * H + i));
      const float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + r * H + i));
      const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(gamma + i));
      const float h0 = (xv.x - mu) * rs, h1 = (xv.y - mu) * rs;
      *reinterpret_cast<uint32_t*>(dx + r * H + i) = pack_bf16x2(rs * (d.x * g.x - s1 - h0 * s2), rs * (d.y * g.y - s1 - h1 * s2));
      pg[i] += d.x * h0;      // each thread owns its columns of the CTA's partial row: no atomics
      pg[i + 1] += d.y * h1;
      pb[i] += d.x;
      pb[i + 1] += d.y;
    }
  }
}

__global__ void ln_colsum_kernel(const float* __restrict__ partials, int nparts, int H, float* __restrict__ dgamma, float* __restrict__ dbeta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * H) return;
  float t = 0.f;
  for (int p = 0; p < nparts; ++p) t += partials[(long long)p * 2 * H + i];
  if (i < H) dgamma[i] = t;
  else if (dbeta) dbeta[i - H] = t;
}

// ------------------------------------------------------------------------------------------------ soft-max
// x: [rows, n] scores with rows = batch * heads * queries.  mask (uint8, 1 = masked out) is [batch, queries, n] shared by the
// heads, or null; causal != 0 masks key j > query index (row % queries) + (n - queries).  y = softmax(scale * x).
// A fully masked row yields zeros.
__global__ void __launch_bounds__(256) masked_softmax_fwd_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ mask,
                                                                 __nv_bfloat16* __restrict__ y, long long rows, int n, int heads, int queries,
                                                                 float scale, int causal) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int qi = int(row % queries);
  const long long b = row / ((long long)heads * queries);
  const uint8_t* mrow = mask ? mask + (b * queries + qi) * n : nullptr;
  const int limit = causal ? qi + (n - queries) : n - 1;  // last visible key
  const __nv_bfloat16* xr = x + row * n;
  float m = -INFINITY;
  for (int j = lane; j < n; j += 32) {
    const bool vis = j <= limit && !(mrow && mrow[j]);
    if (vis) m = fmaxf(m, __bfloat162float(xr[j]) * scale);
  }
  m = warp_max(m);
  float l = 0.f;
  for (int j = lane; j < n; j += 32) {
    const bool vis = j <= limit && !(mrow && mrow[j]);
    if (vis) l += __expf(__bfloat162float(xr[j]) * scale - m);
  }
  l = warp_sum(l);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int j = lane; j < n; j += 32) {
    const bool vis = j <= limit && !(mrow && mrow[j]);
    y[row * n + j] = __float2bfloat16(vis ? __expf(__bfloat162float(xr[j]) * scale - m) * inv : 0.f);
  }
}

// dx = scale * y * (dy - sum(dy * y)); masked positions have y = 0 and so dx = 0.
__global__ void __launch_bounds__(256) masked_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                                                                 __nv_bfloat16* __restrict__ dx, long long rows, int n, float scale) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float dot = 0.f;
  for (int j = lane; j < n; j += 32) dot += __bfloat162float(dy[row * n + j]) * __bfloat162float(y[row * n + j]);
  dot = warp_sum(dot);
  for (int j = lane; j < n; j += 32) {
    const float yy = __bfloat162float(y[row * n + j]);
    dx[row * n + j] = __float2bfloat16(scale * yy * (__bfloat162float(dy[row * n + j]) - dot));
  }
}

}  // namespace ats

using namespace ats;

ATS_API int ats_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, long long rows, int H,
                              float eps, void* stream) {
  if (H % 8) return 1003;
  const int blocks = int(rows < 1184 ? rows : 1184);
  if (blocks == 0) return 0;
  layernorm_fwd_kernel<<<blocks, LN_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta),
      static_cast<__nv_bfloat16*>(y), mean, rstd, rows, H, eps);
  return int(cudaGetLastError());
}

// partials: fp32 scratch [blocks, 2, H]; dgamma / dbeta: fp32 [H] (dbeta may be null).
ATS_API int ats_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                              float* partials, int blocks, float* dgamma, float* dbeta, long long rows, int H, void* stream) {
  if (H % 2 || blocks <= 0) return 1003;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  layernorm_bwd_kernel<<<blocks, LN_THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                                                     static_cast<const __nv_bfloat16*>(gamma), mean, rstd, static_cast<__nv_bfloat16*>(dx),
                                                     partials, rows, H);
  ln_colsum_kernel<<<(2 * H + 255) / 256, 256, 0, s>>>(partials, blocks, H, dgamma, dbeta);
  return int(cudaGetLastError());
}

ATS_API int ats_masked_softmax_fwd(const void* x, const unsigned char* mask, void* y, long long rows, int n, int heads, int queries,
                                   float scale, int causal, void* stream) {
  if (rows <= 0) return 0;
  masked_softmax_fwd_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), mask, static_cast<__nv_bfloat16*>(y), rows, n, heads, queries, scale, causal);
  return int(cudaGetLastError());
}

ATS_API int ats_masked_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int n, float scale, void* stream) {
  if (rows <= 0) return 0;
  masked_softmax_bwd_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(dx), rows, n, scale);
  return int(cudaGetLastError());
}
