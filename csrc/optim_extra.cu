// Optimiser kernels beside AdamW, all on the flat fp32 master shard of a ZeRO bucket with bf16 gradients in and bf16
// parameters out, hyper-parameters read from device memory (so a learning-rate change needs no new launch arguments)
// and the clip state {grad scale, norm, skip flag} honoured exactly as the AdamW kernel does:
//
//   * SGD with momentum / dampening / Nesterov / weight decay;
//   * LAMB in two stages: stage 1 forms the Adam direction u = m^ / (sqrt(v^) + eps) + wd * w and the per-tensor sums of
//     w^2 and u^2; stage 2 applies w -= lr * trust * u with trust = |w| / |u| per tensor.  Tensors are segments of the flat
//     shard; the host cuts the shard into chunks that never straddle a tensor, so a CTA knows its tensor without a search;
//   * scale with overflow flag (unscale of loss-scaled gradients) and absolute maximum (max-norm).
//
// The vendored optimiser kernels of the reference do the same work over lists of tensor pointers
// (colossalai extensions csrc/cuda/multi_tensor_sgd_kernel.cu, multi_tensor_lamb.cu:40-354, multi_tensor_scale_kernel.cu,
// multi_tensor_l2norm_kernel.cu); here the parameters already live in one flat buffer, so one launch covers them all.
#include "common.cuh"

namespace ats {

// hyper = {lr, momentum, dampening, weight_decay, nesterov (0/1), first_step (0/1)}
__global__ void __launch_bounds__(256) sgd_kernel(float* __restrict__ master, float* __restrict__ mom, const __nv_bfloat16* __restrict__ grad,
                                                  __nv_bfloat16* __restrict__ param, long long n, const float* __restrict__ hyper,
                                                  const float* __restrict__ clip_state, float wd_mult) {
  const float lr = hyper[0], mu = hyper[1], damp = hyper[2], wd = hyper[3] * wd_mult;
  const bool nesterov = hyper[4] != 0.f, first = hyper[5] != 0.f;
  float gscale = 1.f;
  if (clip_state) {
    if (clip_state[2] != 0.f) return;
    gscale = clip_state[0];
  }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float w = master[i];
    float g = __bfloat162float(grad[i]) * gscale + wd * w;
    if (mu != 0.f) {
      const float b = first ? g : mu * mom[i] + (1.f - damp) * g;
      mom[i] = b;
      g = nesterov ? g + mu * b : b;
    }
    const float nw = w - lr * g;
    master[i] = nw;
    param[i] = __float2bfloat16(nw);
  }
}

constexpr int LAMB_CHUNK = 4096;

// hyper = {lr, beta1, beta2, eps, weight_decay, step}.  chunk c covers [chunk_start[c], chunk_start[c] + chunk_len[c]) of tensor
// chunk_seg[c].  seg_sums: [n_seg, 2] (sum w^2, sum u^2), zeroed by the caller.
__global__ void __launch_bounds__(256) lamb_stage1_kernel(const float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                          const __nv_bfloat16* __restrict__ grad, float* __restrict__ update,
                                                          const long long* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                                                          const int* __restrict__ chunk_seg, float* __restrict__ seg_sums,
                                                          const float* __restrict__ hyper, const float* __restrict__ clip_state, float wd_mult) {
  __shared__ float red[33];
  const float b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4] * wd_mult, step = hyper[5];
  float gscale = 1.f;
  if (clip_state) {
    if (clip_state[2] != 0.f) return;
    gscale = clip_state[0];
  }
  const float bc1 = 1.f - __powf(b1, step), bc2 = 1.f - __powf(b2, step);
  const int c = blockIdx.x;
  const long long s = chunk_start[c];
  const int len = chunk_len[c];
  float sw = 0.f, su = 0.f;
  for (int i = threadIdx.x; i < len; i += 256) {
    const long long j = s + i;
    const float g = __bfloat162float(grad[j]) * gscale;
    const float nm = b1 * m[j] + (1.f - b1) * g;
    const float nv = b2 * v[j] + (1.f - b2) * g * g;
    m[j] = nm;
    v[j] = nv;
    const float w = master[j];
    const float u = (nm / bc1) / (sqrtf(nv / bc2) + eps) + wd * w;
    update[j] = u;
    sw += w * w;
    su += u * u;
  }
  sw = block_sum(sw, red);
  su = block_sum(su, red);
  if (threadIdx.x == 0) {
    atomicAdd(&seg_sums[2 * chunk_seg[c]], sw);
    atomicAdd(&seg_sums[2 * chunk_seg[c] + 1], su);
  }
}

__global__ void __launch_bounds__(256) lamb_stage2_kernel(float* __restrict__ master, const float* __restrict__ update,
                                                          __nv_bfloat16* __restrict__ param, const long long* __restrict__ chunk_start,
                                                          const int* __restrict__ chunk_len, const int* __restrict__ chunk_seg,
                                                          const float* __restrict__ seg_sums, const float* __restrict__ hyper,
                                                          const float* __restrict__ clip_state) {
  if (clip_state && clip_state[2] != 0.f) return;
  const float lr = hyper[0];
  const int c = blockIdx.x;
  const float wn = sqrtf(seg_sums[2 * chunk_seg[c]]), un = sqrtf(seg_sums[2 * chunk_seg[c] + 1]);
  const float trust = (wn > 0.f && un > 0.f) ? wn / un : 1.f;
  const long long s = chunk_start[c];
  const int len = chunk_len[c];
  for (int i = threadIdx.x; i < len; i += 256) {
    const long long j = s + i;
    const float nw = master[j] - lr * trust * update[j];
    master[j] = nw;
    param[j] = __float2bfloat16(nw);
  }
}

// out = in * scale (bf16 or fp32 in, fp32 out); flag[0] set to 1 when any input is inf / nan.
template <typename T>
__global__ void __launch_bounds__(256) scale_check_kernel(const T* __restrict__ in, float* __restrict__ out, long long n, const float* scale_ptr,
                                                          float scale, int* __restrict__ flag) {
  const float sc = scale_ptr ? scale_ptr[0] * scale : scale;
  bool bad = false;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float x = float(in[i]);
    bad |= !isfinite(x);
    out[i] = x * sc;
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) *flag = 1;
}

template <typename T>
__global__ void __launch_bounds__(256) absmax_kernel(const T* __restrict__ in, long long n, float* __restrict__ out) {
  __shared__ float red[33];
  float m = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) m = fmaxf(m, fabsf(float(in[i])));
  m = block_max(m, red);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));  // non-negative floats order like ints
}

}  // namespace ats

using namespace ats;

static unsigned grid_for(long long n) {
  long long b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return unsigned(b);
}

ATS_API int ats_sgd(float* master, float* mom, const void* grad, void* param, long long n, const float* hyper, const float* clip_state,
                    float wd_mult, void* stream) {
  if (n == 0) return 0;
  sgd_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(master, mom, static_cast<const __nv_bfloat16*>(grad),
                                                                        static_cast<__nv_bfloat16*>(param), n, hyper, clip_state, wd_mult);
  return int(cudaGetLastError());
}

ATS_API int ats_lamb_chunk() { return LAMB_CHUNK; }

// update: fp32 scratch [n]; seg_sums: fp32 [n_seg, 2]; chunk tables as built by the host (chunks <= ats_lamb_chunk() elements).
// stage 0 = both stages; 1 = direction and per-tensor sums only; 2 = apply only (a sharded optimiser all-reduces seg_sums between).
ATS_API int ats_lamb(float* master, float* m, float* v, const void* grad, void* param, float* update, const long long* chunk_start,
                     const int* chunk_len, const int* chunk_seg, int n_chunks, float* seg_sums, int n_seg, const float* hyper,
                     const float* clip_state, float wd_mult, int stage, void* stream) {
  if (n_chunks == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (stage != 2) {
    cudaError_t e = cudaMemsetAsync(seg_sums, 0, sizeof(float) * 2 * n_seg, s);
    if (e != cudaSuccess) return int(e);
    lamb_stage1_kernel<<<n_chunks, 256, 0, s>>>(master, m, v, static_cast<const __nv_bfloat16*>(grad), update, chunk_start, chunk_len,
                                                chunk_seg, seg_sums, hyper, clip_state, wd_mult);
  }
  if (stage != 1)
    lamb_stage2_kernel<<<n_chunks, 256, 0, s>>>(master, update, static_cast<__nv_bfloat16*>(param), chunk_start, chunk_len, chunk_seg, seg_sums,
                                                hyper, clip_state);
  return int(cudaGetLastError());
}

ATS_API int ats_scale_check(const void* in, int is_fp32, float* out, long long n, const float* scale_ptr, float scale, int* flag, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_fp32) scale_check_kernel<float><<<grid_for(n), 256, 0, s>>>(static_cast<const float*>(in), out, n, scale_ptr, scale, flag);
  else scale_check_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), out, n, scale_ptr, scale, flag);
  return int(cudaGetLastError());
}

// out[0] = max(out[0], max |in|); the caller zeroes out[0] first.
ATS_API int ats_absmax(const void* in, int is_fp32, long long n, float* out, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_fp32) absmax_kernel<float><<<grid_for(n), 256, 0, s>>>(static_cast<const float*>(in), n, out);
  else absmax_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), n, out);
  return int(cudaGetLastError());
}
