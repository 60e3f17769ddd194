// Cross-entropy (+accuracy, +in-place gradient) over bf16 logits, global gradient norm, clip coefficient,
// partitioned AdamW on fp32 master/m/v with bf16 parameter write-back.
//
// Counterparts in the reference: training/fused_loss.cu:67-167 (forward-only fp32 CE), training/
// fused_grad_clip.cu:26-101, torch.optim.AdamW(fused=True) (training/trainer.py:2227) and the vendored
// multi_tensor_adam.cu:30-116.  Here the learning rate, the step count and the gradient scale are read from
// device memory, so an LR change by the orchestrator or a clip coefficient never forces a host round trip.
#include "common.cuh"

namespace ats {

// One CTA per row.  Pass 1: online max / sum-exp / argmax.  Pass 2 (row_scale != nullptr): logits are replaced
// in place by (softmax - onehot) * row_scale[row]; rows whose label is ignore_index get zeros.
__global__ void __launch_bounds__(256)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                  const float* __restrict__ row_scale, float* __restrict__ loss_row, float* __restrict__ correct,
                  float* __restrict__ lse_out, int vocab, long long ld, long long ignore_index) {
  __shared__ float red[33];
  __shared__ float s_best[8];
  __shared__ int s_idx[8];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long label = labels[row];
  const bool valid = label != ignore_index && label >= 0 && label < vocab;
  const int nvec = vocab >> 3;
  float m = -INFINITY, s = 0.f, best = -INFINITY;
  int best_i = 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 a = reinterpret_cast<const uint4*>(lr)[v];
    float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
    float f[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
    float vm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) vm = fmaxf(vm, f[e]);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f[e] > best) {
        best = f[e];
        best_i = v * 8 + e;
      }
    const float nm = fmaxf(m, vm);
    float add = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) add += __expf(f[e] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int j = (nvec << 3) + threadIdx.x; j < vocab; j += blockDim.x) {  // tail when vocab % 8 != 0
    float f = __bfloat162float(lr[j]);
    if (f > best) {
      best = f;
      best_i = j;
    }
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max(m, red);
  const float gs = block_sum(m == -INFINITY ? 0.f : s * __expf(m - gm), red);
  // argmax: lowest index among maxima
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s_best[threadIdx.x >> 5] = best;
    s_idx[threadIdx.x >> 5] = best_i;
  }
  __syncthreads();
  const float lse = gm + __logf(gs);
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (s_best[w] > best || (s_best[w] == best && s_idx[w] < best_i)) {
        best = s_best[w];
        best_i = s_idx[w];
      }
    float l = 0.f;
    if (valid) l = lse - __bfloat162float(lr[label]);
    if (!(l == l)) l = 0.f;
    loss_row[row] = l;
    if (correct) correct[row] = (valid && best_i == label) ? 1.f : 0.f;
    if (lse_out) lse_out[row] = lse;
  }
  if (!row_scale) return;
  __syncthreads();
  const float sc = valid ? row_scale[row] : 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 a = reinterpret_cast<const uint4*>(lr)[v];
    uint32_t u[4] = {a.x, a.y, a.z, a.w}, o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = unpack_bf16x2(u[e]);
      const int j = v * 8 + 2 * e;
      float p0 = __expf(f.x - lse) - (j == label ? 1.f : 0.f);
      float p1 = __expf(f.y - lse) - (j + 1 == label ? 1.f : 0.f);
      o[e] = pack_bf16x2(p0 * sc, p1 * sc);
    }
    reinterpret_cast<uint4*>(lr)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int j = (nvec << 3) + threadIdx.x; j < vocab; j += blockDim.x) {
    float p = __expf(__bfloat162float(lr[j]) - lse) - (j == label ? 1.f : 0.f);
    lr[j] = __float2bfloat16(p * sc);
  }
}

// sum of squares of a bf16 (or fp32) buffer -> one partial per block, then a single-block finish that adds
// into out[0] (so several buffers can be folded into one norm).
template <typename T>
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const T* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[33];
  float acc = 0.f;
  if constexpr (sizeof(T) == 2) {
    const long long nvec = n >> 3;
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
      uint4 a = reinterpret_cast<const uint4*>(g)[v];
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
    }
    if (blockIdx.x == 0)
      for (long long j = (nvec << 3) + threadIdx.x; j < n; j += blockDim.x) {
        float f = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[j]);
        acc += f * f;
      }
  } else {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
      float f = reinterpret_cast<const float*>(g)[i];
      acc += f * f;
    }
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(256) sumsq_finish_kernel(const float* __restrict__ partial, int n, float* out, int accumulate) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

// state[0] = grad scale to apply inside AdamW, state[1] = global norm, state[2] = skip flag (non-finite norm).
//   norm = sqrt(sumsq) * pre_scale ; coef = min(1, max_norm / (norm + 1e-6)) ; state[0] = pre_scale * coef
__global__ void clip_coef_kernel(const float* sumsq, float pre_scale, float max_norm, float* state) {
  const float norm = sqrtf(sumsq[0]) * pre_scale;
  const bool finite = isfinite(norm);
  float coef = 1.f;
  if (max_norm > 0.f && finite) coef = fminf(1.f, max_norm / (norm + 1e-6f));
  state[0] = finite ? pre_scale * coef : 0.f;
  state[1] = norm;
  state[2] = finite ? 0.f : 1.f;
}

// AdamW with decoupled weight decay on a flat shard.  hyper = {lr, beta1, beta2, eps, weight_decay, step}
// lives in device memory; clip_state as produced by clip_coef_kernel (may be nullptr).
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             const __nv_bfloat16* __restrict__ grad, __nv_bfloat16* __restrict__ param, long long n,
             const float* __restrict__ hyper, const float* __restrict__ clip_state, float wd_mult) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4] * wd_mult, step = hyper[5];
  float gscale = 1.f;
  if (clip_state) {
    if (clip_state[2] != 0.f) return;  // non-finite gradients: skip the step
    gscale = clip_state[0];
  }
  const float bc1 = 1.f - __powf(b1, step), bc2 = 1.f - __powf(b2, step);
  const float step_size = lr / bc1;
  const float inv_bc2_sqrt = rsqrtf(bc2);
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 3 < n) {
      float4 p = *reinterpret_cast<float4*>(master + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      uint2 gq = *reinterpret_cast<const uint2*>(grad + i);
      float2 g0 = unpack_bf16x2(gq.x), g1 = unpack_bf16x2(gq.y);
      float g[4] = {g0.x * gscale, g0.y * gscale, g1.x * gscale, g1.y * gscale};
      float pp[4] = {p.x, p.y, p.z, p.w}, pm[4] = {mm.x, mm.y, mm.z, mm.w}, pv[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pm[e] = b1 * pm[e] + (1.f - b1) * g[e];
        pv[e] = b2 * pv[e] + (1.f - b2) * g[e] * g[e];
        const float denom = sqrtf(pv[e]) * inv_bc2_sqrt + eps;
        pp[e] = pp[e] * (1.f - lr * wd) - step_size * pm[e] / denom;
      }
      *reinterpret_cast<float4*>(master + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(pm[0], pm[1], pm[2], pm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(pv[0], pv[1], pv[2], pv[3]);
      *reinterpret_cast<uint2*>(param + i) = make_uint2(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]));
    } else {
      for (long long j = i; j < n; ++j) {
        const float g = __bfloat162float(grad[j]) * gscale;
        const float nm = b1 * m[j] + (1.f - b1) * g;
        const float nv = b2 * v[j] + (1.f - b2) * g * g;
        const float denom = sqrtf(nv) * inv_bc2_sqrt + eps;
        const float np = master[j] * (1.f - lr * wd) - step_size * nm / denom;
        m[j] = nm; v[j] = nv; master[j] = np;
        param[j] = __float2bfloat16(np);
      }
    }
  }
}

}  // namespace ats

using namespace ats;

ATS_API int ats_ce_fwd_bwd(void* logits, const long long* labels, const float* row_scale, float* loss_row, float* correct,
                           float* lse, long long rows, int vocab, long long ld, long long ignore_index, void* stream) {
  if (rows == 0) return 0;
  if (ld & 7) return 1003;
  ce_fwd_bwd_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), labels, row_scale, loss_row, correct, lse, vocab, ld, ignore_index);
  return int(cudaGetLastError());
}

// partial: scratch of >= 1024 floats.
ATS_API int ats_sumsq(const void* g, long long n, int is_fp32, float* partial, float* out, int accumulate, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int blocks = int((n / 8 + 255) / 256);
  if (blocks < 1) blocks = 1;
  if (blocks > 1024) blocks = 1024;
  if (is_fp32) sumsq_partial_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(g), n, partial);
  else sumsq_partial_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(g), n, partial);
  sumsq_finish_kernel<<<1, 256, 0, s>>>(partial, blocks, out, accumulate);
  return int(cudaGetLastError());
}

ATS_API int ats_clip_coef(const float* sumsq, float pre_scale, float max_norm, float* state, void* stream) {
  clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, pre_scale, max_norm, state);
  return int(cudaGetLastError());
}

ATS_API int ats_adamw(float* master, float* m, float* v, const void* grad, void* param, long long n, const float* hyper,
                      const float* clip_state, float wd_mult, void* stream) {
  if (n == 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  adamw_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, m, v, static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(param), n, hyper, clip_state, wd_mult);
  return int(cudaGetLastError());
}
