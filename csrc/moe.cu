// Mixture-of-Experts routing kernels: gate projection (small-N GEMM) with its two gradients, fused
// softmax / top-k / renormalise, deterministic capacity-limited slot planning, row dispatch into per-expert
// buffers (local or on a peer GPU through a pointer table), weighted combine, and the per-slot dot product that
// gives the combine-weight gradient.
//
// Counterparts in the reference: core/moe_cuda_ops.cu:47-310 (atomics-ordered top-k / dispatch / combine) and the
// eager routing in core/model.py:1169-1263.  Differences: softmax runs over all experts before the top-k and the
// kept probabilities are renormalised (the documented semantics), slot order is token order (deterministic), and
// capacity is enforced.
#include "common.cuh"

namespace ats {

// ------------------------------------------------------------------------------------------------
// gate projection: logits[t, e] = sum_h x[t, h] * wg[e, h]       (fp32 out), one warp per token
// ------------------------------------------------------------------------------------------------
template <int EMAX>
__global__ void __launch_bounds__(256)
gate_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, float* __restrict__ logits,
                long long tokens, int hidden, int experts) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  float acc[EMAX];
#pragma unroll
  for (int e = 0; e < EMAX; ++e) acc[e] = 0.f;
  const int nvec = hidden >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + t * hidden);
  for (int v = lane; v < nvec; v += 32) {
    uint4 a = xr[v];
    float2 x0 = unpack_bf16x2(a.x), x1 = unpack_bf16x2(a.y), x2 = unpack_bf16x2(a.z), x3 = unpack_bf16x2(a.w);
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      if (e < experts) {
        uint4 b = reinterpret_cast<const uint4*>(wg + (long long)e * hidden)[v];
        float2 w0 = unpack_bf16x2(b.x), w1 = unpack_bf16x2(b.y), w2 = unpack_bf16x2(b.z), w3 = unpack_bf16x2(b.w);
        acc[e] += x0.x * w0.x + x0.y * w0.y + x1.x * w1.x + x1.y * w1.y + x2.x * w2.x + x2.y * w2.y + x3.x * w3.x + x3.y * w3.y;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < EMAX; ++e) {
    if (e < experts) {
      float s = warp_sum(acc[e]);
      if (lane == 0) logits[t * experts + e] = s;
    }
  }
}

// Same product with the router weight staged once per CTA in shared memory and two tokens per warp step, so that a weight
// vector read from shared memory is used for two tokens (used when E * hidden * 2 bytes fit in 64 KB).
template <int EMAX>
__global__ void __launch_bounds__(256)
gate_fwd_smem_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, float* __restrict__ logits,
                     long long tokens, int hidden, int experts) {
  extern __shared__ uint4 s_w[];  // [experts][hidden / 8]
  const int nvec = hidden >> 3;
  for (int i = threadIdx.x; i < experts * nvec; i += blockDim.x) s_w[i] = reinterpret_cast<const uint4*>(wg)[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long t0 = ((long long)blockIdx.x * wpb + warp) * 2; t0 < tokens; t0 += (long long)gridDim.x * wpb * 2) {
    const bool two = t0 + 1 < tokens;
    float acc0[EMAX], acc1[EMAX];
#pragma unroll
    for (int e = 0; e < EMAX; ++e) acc0[e] = acc1[e] = 0.f;
    const uint4* xr0 = reinterpret_cast<const uint4*>(x + t0 * hidden);
    const uint4* xr1 = reinterpret_cast<const uint4*>(x + (t0 + (two ? 1 : 0)) * hidden);
    for (int v = lane; v < nvec; v += 32) {
      const uint4 a = xr0[v], b = xr1[v];
      const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
      const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
#pragma unroll
      for (int e = 0; e < EMAX; ++e) {
        if (e < experts) {
          const uint4 w = s_w[e * nvec + v];
          const float2 w0 = unpack_bf16x2(w.x), w1 = unpack_bf16x2(w.y), w2 = unpack_bf16x2(w.z), w3 = unpack_bf16x2(w.w);
          acc0[e] += a0.x * w0.x + a0.y * w0.y + a1.x * w1.x + a1.y * w1.y + a2.x * w2.x + a2.y * w2.y + a3.x * w3.x + a3.y * w3.y;
          acc1[e] += b0.x * w0.x + b0.y * w0.y + b1.x * w1.x + b1.y * w1.y + b2.x * w2.x + b2.y * w2.y + b3.x * w3.x + b3.y * w3.y;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      if (e < experts) {
        const float s0 = warp_sum(acc0[e]), s1 = warp_sum(acc1[e]);
        if (lane == 0) {
          logits[t0 * experts + e] = s0;
          if (two) logits[(t0 + 1) * experts + e] = s1;
        }
      }
    }
  }
}

// dx[t, h] (+)= sum_e dlogits[t, e] * wg[e, h]
__global__ void __launch_bounds__(256)
gate_bwd_dx_kernel(const float* __restrict__ dlogits, const __nv_bfloat16* __restrict__ wg, __nv_bfloat16* __restrict__ dx,
                   long long tokens, int hidden, int experts, int accumulate) {
  const int vpr = hidden >> 3;
  const long long total = tokens * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = int(i - t * vpr);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int e = 0; e < experts; ++e) {
      const float d = dlogits[t * experts + e];
      uint4 b = reinterpret_cast<const uint4*>(wg + (long long)e * hidden)[v];
      float2 w0 = unpack_bf16x2(b.x), w1 = unpack_bf16x2(b.y), w2 = unpack_bf16x2(b.z), w3 = unpack_bf16x2(b.w);
      acc[0] += d * w0.x; acc[1] += d * w0.y; acc[2] += d * w1.x; acc[3] += d * w1.y;
      acc[4] += d * w2.x; acc[5] += d * w2.y; acc[6] += d * w3.x; acc[7] += d * w3.y;
    }
    uint4* dst = reinterpret_cast<uint4*>(dx + t * hidden) + v;
    if (accumulate) {
      uint4 o = *dst;
      float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z), f3 = unpack_bf16x2(o.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    *dst = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// Same for up to eight experts with the weights in registers: a thread owns eight columns and walks over tokens, so a token
// costs eight broadcast loads of dlogits, 64 FMAs and one 16-byte store instead of eight more weight loads.
__global__ void __launch_bounds__(256)
gate_bwd_dx_reg_kernel(const float* __restrict__ dlogits, const __nv_bfloat16* __restrict__ wg, __nv_bfloat16* __restrict__ dx,
                       long long tokens, int hidden, int experts, int accumulate) {
  const int v = blockIdx.y * 256 + threadIdx.x;
  if (v >= (hidden >> 3)) return;
  float w[8][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    uint4 b = e < experts ? reinterpret_cast<const uint4*>(wg + (long long)e * hidden)[v] : make_uint4(0, 0, 0, 0);
    float2 w0 = unpack_bf16x2(b.x), w1 = unpack_bf16x2(b.y), w2 = unpack_bf16x2(b.z), w3 = unpack_bf16x2(b.w);
    w[e][0] = w0.x; w[e][1] = w0.y; w[e][2] = w1.x; w[e][3] = w1.y; w[e][4] = w2.x; w[e][5] = w2.y; w[e][6] = w3.x; w[e][7] = w3.y;
  }
  for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (e < experts) {
        const float d = dlogits[t * experts + e];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] += d * w[e][c];
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(dx + t * hidden) + v;
    if (accumulate) {
      uint4 o = *dst;
      float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z), f3 = unpack_bf16x2(o.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    *dst = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// dwg partial: block b sums tokens [b*chunk, (b+1)*chunk): partial[b][e][h] = sum_t dlogits[t,e] * x[t,h]
__global__ void __launch_bounds__(256)
gate_bwd_dw_kernel(const float* __restrict__ dlogits, const __nv_bfloat16* __restrict__ x, float* __restrict__ partial,
                   long long tokens, int hidden, int experts, int chunk) {
  const long long t0 = (long long)blockIdx.x * chunk;
  const long long t1 = min(t0 + chunk, tokens);
  for (int e0 = 0; e0 < experts; e0 += 8) {
    for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x) {
      float acc[8][8];
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;
      // four tokens per step, their rows requested before any arithmetic: one load in flight per thread left HBM idle
      for (long long tb = t0; tb < t1; tb += 4) {
        uint4 q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          q[j] = tb + j < t1 ? reinterpret_cast<const uint4*>(x + (tb + j) * hidden)[v] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (tb + j >= t1) break;
          const long long t = tb + j;
          float2 x0 = unpack_bf16x2(q[j].x), x1 = unpack_bf16x2(q[j].y), x2 = unpack_bf16x2(q[j].z), x3 = unpack_bf16x2(q[j].w);
          float xs[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
#pragma unroll
          for (int a = 0; a < 8; ++a) {
            if (e0 + a < experts) {
              const float d = dlogits[t * experts + e0 + a];
#pragma unroll
              for (int b = 0; b < 8; ++b) acc[a][b] += d * xs[b];
            }
          }
        }
      }
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        if (e0 + a < experts) {
          float* dst = partial + ((long long)blockIdx.x * experts + e0 + a) * hidden + v * 8;
          reinterpret_cast<float4*>(dst)[0] = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
          reinterpret_cast<float4*>(dst)[1] = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// softmax over all experts (after temperature), top-k, renormalise.  One thread per token, experts <= 64.
//   probs[t, e]   : softmax(logits / temperature)                         (kept for backward)
//   topk_idx[t,k] : expert ids, descending probability, ties -> lower id
//   topk_w[t, k]  : probs of the kept experts / their sum
// ------------------------------------------------------------------------------------------------
__global__ void topk_softmax_kernel(const float* __restrict__ logits, float* __restrict__ probs, int* __restrict__ topk_idx,
                                    float* __restrict__ topk_w, long long tokens, int experts, int k, float inv_temp) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float p[64];
  float m = -INFINITY;
  for (int e = 0; e < experts; ++e) {
    p[e] = logits[t * experts + e] * inv_temp;
    m = fmaxf(m, p[e]);
  }
  float s = 0.f;
  for (int e = 0; e < experts; ++e) {
    p[e] = __expf(p[e] - m);
    s += p[e];
  }
  const float inv = 1.f / s;
  for (int e = 0; e < experts; ++e) {
    p[e] *= inv;
    probs[t * experts + e] = p[e];
  }
  unsigned long long taken = 0ull;
  float wsum = 0.f;
  float wk[8];
  int ik[8];
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0;
    for (int e = 0; e < experts; ++e)
      if (!((taken >> e) & 1ull) && p[e] > best) {
        best = p[e];
        bi = e;
      }
    taken |= 1ull << bi;
    wk[j] = best;
    ik[j] = bi;
    wsum += best;
  }
  const float wi = 1.f / fmaxf(wsum, 1e-20f);
  for (int j = 0; j < k; ++j) {
    topk_idx[t * k + j] = ik[j];
    topk_w[t * k + j] = wk[j] * wi;
  }
}

// ------------------------------------------------------------------------------------------------
// Fused routing for training: soft-max of the logits (probabilities at temperature 1 for the balance loss, at 1 / inv_temp
// for the routing), top-k, renormalised weights, and per-block partial sums of the clean probabilities and of the expert
// picks (summed in a fixed order by route_finish_kernel -> deterministic).  One thread per token.
//   aux = E * sum_e (picks_e / (T k)) * (sum_t p_clean[t, e] / T) * weight, clamped to <= 1
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
route_fwd_kernel(const float* __restrict__ logits, float* __restrict__ probs, float* __restrict__ clean, int* __restrict__ topk_idx,
                 float* __restrict__ topk_w, float* __restrict__ part, long long tokens, int experts, int k, float inv_temp) {
  __shared__ float s_p[8][64], s_c[64];
  if (threadIdx.x < 64) s_c[threadIdx.x] = 0.f;
  __syncthreads();
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float c[64];
  for (int e = 0; e < experts; ++e) c[e] = 0.f;
  if (t < tokens) {
    float p[64];
    float m = -INFINITY;
    for (int e = 0; e < experts; ++e) {
      c[e] = logits[t * experts + e];
      m = fmaxf(m, c[e]);
    }
    float sc = 0.f, sp = 0.f;
    for (int e = 0; e < experts; ++e) {
      p[e] = __expf((c[e] - m) * inv_temp);
      c[e] = __expf(c[e] - m);
      sc += c[e];
      sp += p[e];
    }
    const float ic = 1.f / sc, ip = 1.f / sp;
    for (int e = 0; e < experts; ++e) {
      p[e] *= ip;
      c[e] *= ic;
      probs[t * experts + e] = p[e];
      if (clean) clean[t * experts + e] = c[e];
    }
    unsigned long long taken = 0ull;
    float wsum = 0.f, wk[8];
    int ik[8];
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int bi = 0;
      for (int e = 0; e < experts; ++e)
        if (!((taken >> e) & 1ull) && p[e] > best) {
          best = p[e];
          bi = e;
        }
      taken |= 1ull << bi;
      wk[j] = best;
      ik[j] = bi;
      wsum += best;
      atomicAdd(&s_c[bi], 1.f);
    }
    const float wi = 1.f / fmaxf(wsum, 1e-20f);
    for (int j = 0; j < k; ++j) {
      topk_idx[t * k + j] = ik[j];
      topk_w[t * k + j] = wk[j] * wi;
    }
  }
  // clean-probability sums: shuffle tree per warp, then the warps in order (fixed order -> reproducible bits);
  // the pick counts are integers, so their atomics are exact
  for (int e = 0; e < experts; ++e) {
    const float ws = warp_sum(c[e]);
    if (lane == 0) s_p[warp][e] = ws;
  }
  __syncthreads();
  if (threadIdx.x < experts) {
    float sp = 0.f;
    for (int w = 0; w < 8; ++w) sp += s_p[w][threadIdx.x];
    part[(long long)blockIdx.x * 2 * experts + threadIdx.x] = sp;
    part[(long long)blockIdx.x * 2 * experts + experts + threadIdx.x] = s_c[threadIdx.x];
  }
}

// stats[0..E) = mean clean probability, stats[E..2E) = pick fraction f_e, stats[2E] = aux, stats[2E + 1] = 1 if clamped
__global__ void route_finish_kernel(const float* __restrict__ part, int nblocks, float* __restrict__ stats, long long tokens, int experts,
                                    int k, float weight) {
  __shared__ float prod[64];
  const int e = threadIdx.x;
  if (e < experts) {
    float sp = 0.f, sc = 0.f;
    for (int b = 0; b < nblocks; ++b) {
      sp += part[(long long)b * 2 * experts + e];
      sc += part[(long long)b * 2 * experts + experts + e];
    }
    const float pm = sp / float(tokens), f = sc / float(tokens * k);
    stats[e] = pm;
    stats[experts + e] = f;
    prod[e] = pm * f;
  }
  __syncthreads();
  if (e == 0) {
    float a = 0.f;
    for (int x = 0; x < experts; ++x) a += prod[x];
    a *= float(experts) * weight;
    stats[2 * experts + 1] = a > 1.f ? 1.f : 0.f;
    stats[2 * experts] = fminf(a, 1.f);
  }
}

// dlogits = softmax_bwd(clean, dclean) + softmax_bwd(probs, dprobs) * inv_temp with
//   dclean[e] = daux * E * weight * f_e / T (0 when the loss was clamped),
//   dprobs[i_j] = (dw_j - sum_m dw_m w_m) / S,  S = sum of the kept probabilities.
__global__ void __launch_bounds__(256)
route_bwd_kernel(const float* __restrict__ probs, const float* __restrict__ clean, const int* __restrict__ topk_idx,
                 const float* __restrict__ topk_w, const float* __restrict__ dw, const float* __restrict__ daux,
                 const float* __restrict__ stats, float* __restrict__ dlogits, long long tokens, int experts, int k, float inv_temp,
                 float weight) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float g[64];
  for (int e = 0; e < experts; ++e) g[e] = 0.f;
  if (dw) {
    float S = 0.f, dot = 0.f;
    for (int j = 0; j < k; ++j) {
      S += probs[t * experts + topk_idx[t * k + j]];
      dot += dw[t * k + j] * topk_w[t * k + j];
    }
    const float iS = 1.f / fmaxf(S, 1e-20f);
    for (int j = 0; j < k; ++j) g[topk_idx[t * k + j]] = (dw[t * k + j] - dot) * iS;
    float pg = 0.f;
    for (int e = 0; e < experts; ++e) pg += probs[t * experts + e] * g[e];
    for (int e = 0; e < experts; ++e) g[e] = probs[t * experts + e] * (g[e] - pg) * inv_temp;
  }
  if (daux && stats[2 * experts + 1] == 0.f) {
    const float scale = daux[0] * float(experts) * weight / float(tokens);
    const float* cl = clean ? clean : probs;
    float pg = 0.f;
    for (int e = 0; e < experts; ++e) pg += cl[t * experts + e] * scale * stats[experts + e];
    for (int e = 0; e < experts; ++e) g[e] += cl[t * experts + e] * (scale * stats[experts + e] - pg);
  }
  for (int e = 0; e < experts; ++e) dlogits[t * experts + e] = g[e];
}

// ------------------------------------------------------------------------------------------------
// Slot planning (single CTA, deterministic): slot s = t*k + j goes to expert e = topk_idx[s]; its rank is the
// number of earlier slots with the same expert.  rank >= capacity -> dropped (pos = -1).
//   slot_pos[s] = rank (row inside the expert's region)   counts[e] = min(total_e, capacity)
//   totals[e]   = un-clamped demand (for statistics / aux loss)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
plan_slots_kernel(const int* __restrict__ topk_idx, int* __restrict__ slot_pos, int* __restrict__ counts,
                  int* __restrict__ totals, long long slots, int experts, int capacity) {
  __shared__ int running[64];
  __shared__ int warp_cnt[32][64 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x < 64) running[threadIdx.x] = 0;
  __syncthreads();
  for (long long base = 0; base < slots; base += blockDim.x) {
    const long long s = base + threadIdx.x;
    int e = s < slots ? topk_idx[s] : -1;
    if (e >= 0 && !ATS_DBG_CHECK(e < experts, kDbgPlanSlots, e)) e = -1;
    int my_rank_in_warp = 0;
    for (int x = 0; x < experts; ++x) {
      const unsigned mask = __ballot_sync(0xffffffffu, e == x);
      if (e == x) my_rank_in_warp = __popc(mask & ((1u << lane) - 1u));
      if (lane == 0) warp_cnt[warp][x] = __popc(mask);
    }
    __syncthreads();
    int before = 0;
    if (e >= 0) {
      for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
      const int rank = running[e] + before + my_rank_in_warp;
      slot_pos[s] = rank < capacity ? rank : -1;
    }
    __syncthreads();
    if (threadIdx.x < experts) {
      int tot = 0;
      for (int w = 0; w < nwarps; ++w) tot += warp_cnt[w][threadIdx.x];
      running[threadIdx.x] += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x < experts) {
    const int tot = running[threadIdx.x];
    counts[threadIdx.x] = tot < capacity ? tot : capacity;
    if (totals) totals[threadIdx.x] = tot;
  }
}

// Multi-CTA form of the same plan (same ranks, so still deterministic): chunks of 1024 slots; pass 1 counts the experts of
// every chunk, pass 2 adds the counts of the earlier chunks to the rank inside the chunk.
__device__ __forceinline__ void chunk_ranks(int e, int experts, int (*warp_cnt)[64 + 1], int& rank_in_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  rank_in_warp = 0;
  for (int x = 0; x < experts; ++x) {
    const unsigned mask = __ballot_sync(0xffffffffu, e == x);
    if (e == x) rank_in_warp = __popc(mask & ((1u << lane) - 1u));
    if (lane == 0) warp_cnt[warp][x] = __popc(mask);
  }
}

__global__ void __launch_bounds__(1024)
plan_count_kernel(const int* __restrict__ topk_idx, int* __restrict__ chunk_cnt, long long slots, int experts) {
  __shared__ int warp_cnt[32][64 + 1];
  const long long s = (long long)blockIdx.x * 1024 + threadIdx.x;
  const int e = s < slots ? topk_idx[s] : -1;
  int r;
  chunk_ranks(e, experts, warp_cnt, r);
  __syncthreads();
  if (threadIdx.x < experts) {
    int tot = 0;
    for (int w = 0; w < 32; ++w) tot += warp_cnt[w][threadIdx.x];
    chunk_cnt[blockIdx.x * experts + threadIdx.x] = tot;
  }
}

__global__ void __launch_bounds__(1024)
plan_rank_kernel(const int* __restrict__ topk_idx, const int* __restrict__ chunk_cnt, int* __restrict__ slot_pos,
                 int* __restrict__ counts, int* __restrict__ totals, long long slots, int experts, int capacity) {
  __shared__ int warp_cnt[32][64 + 1];
  __shared__ int before_chunk[64];
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x < experts) {
    int acc = 0;
    for (int c = 0; c < int(blockIdx.x); ++c) acc += chunk_cnt[c * experts + threadIdx.x];
    before_chunk[threadIdx.x] = acc;
    if (blockIdx.x == gridDim.x - 1) {  // the last chunk knows the totals
      const int tot = acc + chunk_cnt[blockIdx.x * experts + threadIdx.x];
      counts[threadIdx.x] = tot < capacity ? tot : capacity;
      if (totals) totals[threadIdx.x] = tot;
    }
  }
  const long long s = (long long)blockIdx.x * 1024 + threadIdx.x;
  const int e = s < slots ? topk_idx[s] : -1;
  int r;
  chunk_ranks(e, experts, warp_cnt, r);
  __syncthreads();
  if (e >= 0) {
    int before = before_chunk[e];
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
    const int rank = before + r;
    slot_pos[s] = rank < capacity ? rank : -1;
  }
}

// ------------------------------------------------------------------------------------------------
// Dispatch: for every kept slot copy (optionally scaled) row src[t] into dst_base[e] + pos * hidden, where
// dst_base is a table of per-expert base pointers (a peer GPU's receive buffer under expert parallelism).
// The last blocks zero the pad rows [count_e, round_up_128(count_e)) so that whole 128-row tiles are defined.
// One warp per slot.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dispatch_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ topk_idx,
                     const int* __restrict__ slot_pos, const float* __restrict__ slot_scale,
                     __nv_bfloat16* const* __restrict__ dst_base, const int* __restrict__ counts,
                     int* const* __restrict__ count_dst, long long slots, int k, int hidden, int experts, int capacity) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int vpr = hidden >> 3;
  // publish how many rows each expert receives from this rank (the expert's owner may be a peer GPU)
  if (count_dst && blockIdx.x == 0 && threadIdx.x < experts) *count_dst[threadIdx.x] = counts[threadIdx.x];
  if (w < slots) {
    const int pos = slot_pos[w];
    if (pos < 0) return;
    const int e = topk_idx[w];
    if (!ATS_DBG_CHECK(e >= 0 && e < experts && pos < capacity, kDbgDispatch, e < 0 || e >= experts ? e : pos)) return;
    const long long t = w / k;
    const uint4* s = reinterpret_cast<const uint4*>(src + t * hidden);
    uint4* d = reinterpret_cast<uint4*>(dst_base[e] + (long long)pos * hidden);
    if (slot_scale) {
      const float sc = slot_scale[w];
      for (int v = lane; v < vpr; v += 32) {
        uint4 a = s[v];
        float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
        d[v] = make_uint4(pack_bf16x2(f0.x * sc, f0.y * sc), pack_bf16x2(f1.x * sc, f1.y * sc),
                          pack_bf16x2(f2.x * sc, f2.y * sc), pack_bf16x2(f3.x * sc, f3.y * sc));
      }
    } else {
      for (int v = lane; v < vpr; v += 32) d[v] = s[v];
    }
    return;
  }
  // pad rows: warp index beyond the slots enumerates (expert, pad row) pairs, at most 127 per expert
  const long long pw = w - slots;
  const int e = int(pw / 128);
  if (e >= experts) return;
  const int c = counts[e];
  const int padded = min((c + 127) & ~127, capacity);
  const int row = c + int(pw % 128);
  if (row >= padded) return;
  uint4* d = reinterpret_cast<uint4*>(dst_base[e] + (long long)row * hidden);
  for (int v = lane; v < vpr; v += 32) d[v] = make_uint4(0, 0, 0, 0);
}

// Combine: out[t] = (res[t]) + sum_j w[t,j] * rows[e_j][pos_j]   over kept slots; one warp per token.
__global__ void __launch_bounds__(256)
combine_rows_kernel(__nv_bfloat16* const* __restrict__ src_base, __nv_bfloat16* const* __restrict__ copy_base,
                    const int* __restrict__ topk_idx, const int* __restrict__ slot_pos, const float* __restrict__ topk_w,
                    const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ out, long long tokens, int k, int hidden) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const int vpr = hidden >> 3;
  for (int v = lane; v < vpr; v += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (res) {
      uint4 a = reinterpret_cast<const uint4*>(res + t * hidden)[v];
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
    }
    for (int j = 0; j < k; ++j) {
      const int pos = slot_pos[t * k + j];
      if (pos < 0) continue;
      const float wt = topk_w ? topk_w[t * k + j] : 1.f;
      const int e = topk_idx[t * k + j];
      if (!ATS_DBG_CHECK(e >= 0 && e < 64, kDbgCombine, e)) continue;
      uint4 a = reinterpret_cast<const uint4*>(src_base[e] + (long long)pos * hidden)[v];
      // rows pulled from a peer GPU are kept in a local copy for the backward pass (gate-weight gradient)
      if (copy_base) reinterpret_cast<uint4*>(copy_base[e] + (long long)pos * hidden)[v] = a;
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] += wt * f0.x; acc[1] += wt * f0.y; acc[2] += wt * f1.x; acc[3] += wt * f1.y;
      acc[4] += wt * f2.x; acc[5] += wt * f2.y; acc[6] += wt * f3.x; acc[7] += wt * f3.y;
    }
    reinterpret_cast<uint4*>(out + t * hidden)[v] =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// dw[t, j] = < dout[t], rows[e_j][pos_j] >  (0 for dropped slots); one warp per slot.
__global__ void __launch_bounds__(256)
slot_dot_kernel(__nv_bfloat16* const* __restrict__ src_base, const int* __restrict__ topk_idx,
                const int* __restrict__ slot_pos, const __nv_bfloat16* __restrict__ dout, float* __restrict__ dw,
                long long slots, int k, int hidden) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= slots) return;
  const int pos = slot_pos[w];
  float acc = 0.f;
  if (pos >= 0 && ATS_DBG_CHECK(topk_idx[w] >= 0 && topk_idx[w] < 64, kDbgSlotDot, topk_idx[w])) {
    const long long t = w / k;
    const uint4* a = reinterpret_cast<const uint4*>(dout + t * hidden);
    const uint4* b = reinterpret_cast<const uint4*>(src_base[topk_idx[w]] + (long long)pos * hidden);
    for (int v = lane; v < (hidden >> 3); v += 32) {
      uint4 p = a[v], q = b[v];
      float2 p0 = unpack_bf16x2(p.x), p1 = unpack_bf16x2(p.y), p2 = unpack_bf16x2(p.z), p3 = unpack_bf16x2(p.w);
      float2 q0 = unpack_bf16x2(q.x), q1 = unpack_bf16x2(q.y), q2 = unpack_bf16x2(q.z), q3 = unpack_bf16x2(q.w);
      acc += p0.x * q0.x + p0.y * q0.y + p1.x * q1.x + p1.y * q1.y + p2.x * q2.x + p2.y * q2.y + p3.x * q3.x + p3.y * q3.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dw[w] = acc;
}

// Per-sequence top-k token selection for Mixture-of-Depths: scores[b, l] -> the `keep` largest per sequence, emitted in
// ascending position order (so causal attention / RoPE positions stay ordered), L <= 8192.  Two launches: (1) rank by counting,
// a CTA per 256 positions of a sequence with the whole sequence's scores in shared memory (ties go to the earlier position);
// (2) ordered compaction of the membership flags, one CTA per sequence.  sel[b, i] = position, i < keep.
__global__ void __launch_bounds__(256)
mod_rank_kernel(const float* __restrict__ scores, int* __restrict__ member, int seq_len, int keep) {
  // 64 positions per CTA, four threads per position: each counts every fourth score, a shuffle adds the four counts
  extern __shared__ float s_sc[];
  const float* sc = scores + (long long)blockIdx.y * seq_len;
  for (int i = threadIdx.x; i < seq_len; i += blockDim.x) s_sc[i] = sc[i];
  __syncthreads();
  const int i = blockIdx.x * 64 + (threadIdx.x >> 2), part = threadIdx.x & 3;
  const bool live = i < seq_len;
  const float v = live ? s_sc[i] : 0.f;
  int rank = 0;
  if (live) {
    // the four threads of a position take every fourth score: the four addresses of a step are neighbours (no bank conflict)
#pragma unroll 8
    for (int j = part; j < seq_len; j += 4) {
      const float o = s_sc[j];
      rank += (o > v) || (o == v && j < i);
    }
  }
  rank += __shfl_xor_sync(0xffffffffu, rank, 1);
  rank += __shfl_xor_sync(0xffffffffu, rank, 2);
  if (live && part == 0) member[(long long)blockIdx.y * seq_len + i] = rank < keep;
}

__global__ void __launch_bounds__(1024)
mod_compact_kernel(const int* __restrict__ member, int* __restrict__ sel, int seq_len, int keep) {
  __shared__ int s_base;
  __shared__ int wsum[32];
  const int* flag = member + (long long)blockIdx.x * seq_len;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < seq_len; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int f = i < seq_len ? flag[i] : 0;
    const unsigned mask = __ballot_sync(0xffffffffu, f);
    if (lane == 0) wsum[warp] = __popc(mask);
    __syncthreads();
    int before = s_base;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    const int pos = before + __popc(mask & ((1u << lane) - 1u));
    if (f && ATS_DBG_CHECK(pos < keep, kDbgModRows, i)) sel[(long long)blockIdx.x * keep + pos] = i;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < (blockDim.x >> 5); ++w) tot += wsum[w];
      s_base += tot;
    }
    __syncthreads();
  }
}

}  // namespace ats

using namespace ats;

ATS_API int ats_gate_fwd(const void* x, const void* wg, float* logits, long long tokens, int hidden, int experts, void* stream) {
  if ((hidden & 7) || experts > 64) return 1003;
  if (tokens == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = unsigned((tokens * 32 + 255) / 256);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(wg);
  const size_t w_bytes = size_t(experts) * hidden * 2;
  if (experts <= 16 && w_bytes <= 65536) {
    static bool attr8 = false, attr16 = false;
    const unsigned grid = 148 * 3;
    if (experts <= 8) {
      if (!attr8) {
        cudaFuncSetAttribute(gate_fwd_smem_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
        attr8 = true;
      }
      gate_fwd_smem_kernel<8><<<grid, 256, w_bytes, s>>>(X, W, logits, tokens, hidden, experts);
    } else {
      if (!attr16) {
        cudaFuncSetAttribute(gate_fwd_smem_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
        attr16 = true;
      }
      gate_fwd_smem_kernel<16><<<grid, 256, w_bytes, s>>>(X, W, logits, tokens, hidden, experts);
    }
    return int(cudaGetLastError());
  }
  if (experts <= 8) gate_fwd_kernel<8><<<blocks, 256, 0, s>>>(X, W, logits, tokens, hidden, experts);
  else if (experts <= 16) gate_fwd_kernel<16><<<blocks, 256, 0, s>>>(X, W, logits, tokens, hidden, experts);
  else gate_fwd_kernel<64><<<blocks, 256, 0, s>>>(X, W, logits, tokens, hidden, experts);
  return int(cudaGetLastError());
}

ATS_API int ats_gate_bwd_dx(const float* dlogits, const void* wg, void* dx, long long tokens, int hidden, int experts,
                            int accumulate, void* stream) {
  if (hidden & 7) return 1003;
  if (tokens == 0) return 0;
  if (experts <= 8) {
    const unsigned col_blocks = unsigned(((hidden >> 3) + 255) / 256);
    unsigned row_blocks = 148 * 8 / col_blocks;
    if ((long long)row_blocks > tokens) row_blocks = unsigned(tokens);
    gate_bwd_dx_reg_kernel<<<dim3(row_blocks, col_blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        dlogits, static_cast<const __nv_bfloat16*>(wg), static_cast<__nv_bfloat16*>(dx), tokens, hidden, experts, accumulate);
    return int(cudaGetLastError());
  }
  long long work = tokens * (hidden >> 3);
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  gate_bwd_dx_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dlogits, static_cast<const __nv_bfloat16*>(wg), static_cast<__nv_bfloat16*>(dx), tokens, hidden, experts, accumulate);
  return int(cudaGetLastError());
}

// partial: fp32 scratch [nblocks, experts, hidden]; reduce with ats_colsum_partial(partial, nblocks, experts*hidden, ...).
ATS_API int ats_gate_bwd_dw(const float* dlogits, const void* x, float* partial, int nblocks, long long tokens, int hidden,
                            int experts, void* stream) {
  if (hidden & 7) return 1003;
  const int chunk = int((tokens + nblocks - 1) / nblocks);
  gate_bwd_dw_kernel<<<nblocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(dlogits, static_cast<const __nv_bfloat16*>(x),
                                                                           partial, tokens, hidden, experts, chunk > 0 ? chunk : 1);
  return int(cudaGetLastError());
}

ATS_API int ats_topk_softmax(const float* logits, float* probs, int* topk_idx, float* topk_w, long long tokens, int experts,
                             int k, float temperature, void* stream) {
  if (experts > 64 || k > 8 || k > experts) return 1003;
  if (tokens == 0) return 0;
  topk_softmax_kernel<<<unsigned((tokens + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, probs, topk_idx, topk_w, tokens, experts, k, 1.f / temperature);
  return int(cudaGetLastError());
}

// Fused training router.  clean: [T, E] or null when temperature == 1 (then probs doubles as the clean probabilities).
// part: fp32 scratch [ceil(T / 256), 2, E]; stats: fp32 [2 E + 2] (see route_finish_kernel).
ATS_API int ats_route_fwd(const float* logits, float* probs, float* clean, int* topk_idx, float* topk_w, float* part, float* stats,
                          long long tokens, int experts, int k, float temperature, float weight, void* stream) {
  if (experts > 64 || k > 8 || k > experts) return 1003;
  if (tokens == 0) return 0;
  const int nblocks = int((tokens + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  route_fwd_kernel<<<nblocks, 256, 0, s>>>(logits, probs, clean, topk_idx, topk_w, part, tokens, experts, k, 1.f / temperature);
  route_finish_kernel<<<1, 64, 0, s>>>(part, nblocks, stats, tokens, experts, k, weight);
  return int(cudaGetLastError());
}

ATS_API int ats_route_bwd(const float* probs, const float* clean, const int* topk_idx, const float* topk_w, const float* dw,
                          const float* daux, const float* stats, float* dlogits, long long tokens, int experts, int k,
                          float temperature, float weight, void* stream) {
  if (experts > 64 || k > 8) return 1003;
  if (tokens == 0) return 0;
  route_bwd_kernel<<<unsigned((tokens + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      probs, clean, topk_idx, topk_w, dw, daux, stats, dlogits, tokens, experts, k, 1.f / temperature, weight);
  return int(cudaGetLastError());
}

ATS_API int ats_plan_slots(const int* topk_idx, int* slot_pos, int* counts, int* totals, long long slots, int experts,
                           int capacity, void* stream) {
  if (experts > 64) return 1003;
  plan_slots_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(topk_idx, slot_pos, counts, totals, slots, experts, capacity);
  return int(cudaGetLastError());
}

// Same result from two multi-CTA passes.  chunk_cnt: int32 scratch of ceil(slots / 1024) * experts entries.
ATS_API int ats_plan_slots_chunked(const int* topk_idx, int* slot_pos, int* counts, int* totals, int* chunk_cnt, long long slots,
                                   int experts, int capacity, void* stream) {
  if (experts > 64 || slots <= 0) return 1003;
  const unsigned chunks = unsigned((slots + 1023) / 1024);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  plan_count_kernel<<<chunks, 1024, 0, s>>>(topk_idx, chunk_cnt, slots, experts);
  plan_rank_kernel<<<chunks, 1024, 0, s>>>(topk_idx, chunk_cnt, slot_pos, counts, totals, slots, experts, capacity);
  return int(cudaGetLastError());
}

ATS_API int ats_dispatch_rows(const void* src, const int* topk_idx, const int* slot_pos, const float* slot_scale,
                              void* const* dst_base, const int* counts, void* const* count_dst, long long slots, int k,
                              int hidden, int experts, int capacity, int zero_pad, void* stream) {
  if ((hidden & 7) || experts > 256) return 1003;
  const long long warps = slots + (zero_pad ? (long long)experts * 128 : 0);
  if (warps == 0) return 0;
  dispatch_rows_kernel<<<unsigned((warps * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), topk_idx, slot_pos, slot_scale,
      reinterpret_cast<__nv_bfloat16* const*>(dst_base), counts, reinterpret_cast<int* const*>(count_dst), slots, k, hidden,
      experts, capacity);
  return int(cudaGetLastError());
}

ATS_API int ats_combine_rows(void* const* src_base, void* const* copy_base, const int* topk_idx, const int* slot_pos, const float* topk_w,
                             const void* res, void* out, long long tokens, int k, int hidden, void* stream) {
  if (hidden & 7) return 1003;
  if (tokens == 0) return 0;
  combine_rows_kernel<<<unsigned((tokens * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16* const*>(src_base), reinterpret_cast<__nv_bfloat16* const*>(copy_base), topk_idx, slot_pos, topk_w,
      static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(out), tokens, k, hidden);
  return int(cudaGetLastError());
}

ATS_API int ats_slot_dot(void* const* src_base, const int* topk_idx, const int* slot_pos, const void* dout, float* dw,
                         long long slots, int k, int hidden, void* stream) {
  if (hidden & 7) return 1003;
  if (slots == 0) return 0;
  slot_dot_kernel<<<unsigned((slots * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16* const*>(src_base), topk_idx, slot_pos, static_cast<const __nv_bfloat16*>(dout), dw, slots, k,
      hidden);
  return int(cudaGetLastError());
}

// member: batch * seq_len ints of scratch (the membership flags; left filled for the caller).
ATS_API int ats_mod_select(const float* scores, int* sel, int* member, int batch, int seq_len, int keep, void* stream) {
  if (seq_len > 8192 || keep > seq_len || !member) return 1003;
  if (batch == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  mod_rank_kernel<<<dim3((seq_len + 63) / 64, batch), 256, seq_len * 4, s>>>(scores, member, seq_len, keep);
  mod_compact_kernel<<<batch, 1024, 0, s>>>(member, sel, seq_len, keep);
  return int(cudaGetLastError());
}
