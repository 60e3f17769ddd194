// Memory-bound kernels: RMSNorm / LayerNorm (fwd, bwd), half-split RoPE, SwiGLU (fwd, bwd), embedding
// (gather * scale, sorted-segment gradient), casts.  bf16 in/out, fp32 math, 16-byte vector accesses.
//
// Counterparts in the reference: core/transformer_ops.cu:61-315 (fp32 CUDA-core RMSNorm / RoPE / SwiGLU) and
// the eager PyTorch paths in core/model.py:228-304, 470-524, 1082-1088, 1924-1931.
#include "common.cuh"
#include <cstdlib>

namespace ats {

// ------------------------------------------------------------------------------------------------
// RMSNorm forward:  y = (x [+ res]) * rsqrt(mean((x+res)^2) + eps) * w ; optionally writes x+res.
// One CTA per row; cols % 8 == 0.
// ------------------------------------------------------------------------------------------------
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd, int cols, float eps) {
  __shared__ float red[33];
  pdl_prologue();
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * cols) : nullptr;
  const int nvec = cols >> 3;
  constexpr int MAXV = 4;  // up to 4 vectors per thread are cached in registers (cols <= THREADS*32)
  float cache[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      uint4 a = xr[v];
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      float f[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
      if (rr) {
        uint4 b = rr[v];
        float2 g0 = unpack_bf16x2(b.x), g1 = unpack_bf16x2(b.y), g2 = unpack_bf16x2(b.z), g3 = unpack_bf16x2(b.w);
        f[0] += g0.x; f[1] += g0.y; f[2] += g1.x; f[3] += g1.y; f[4] += g2.x; f[5] += g2.y; f[6] += g3.x; f[7] += g3.y;
        if (sum_out) {
          uint4 o = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
          reinterpret_cast<uint4*>(sum_out + row * cols)[v] = o;
          // keep the bf16-rounded residual stream so forward and recompute agree
          float2 q0 = unpack_bf16x2(o.x), q1 = unpack_bf16x2(o.y), q2 = unpack_bf16x2(o.z), q3 = unpack_bf16x2(o.w);
          f[0] = q0.x; f[1] = q0.y; f[2] = q1.x; f[3] = q1.y; f[4] = q2.x; f[5] = q2.y; f[6] = q3.x; f[7] = q3.y;
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        cache[i][e] = f[e];
        ss += f[e] * f[e];
      }
    }
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / cols + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * cols);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      uint4 a = wr[v];
      float2 w0 = unpack_bf16x2(a.x), w1 = unpack_bf16x2(a.y), w2 = unpack_bf16x2(a.z), w3 = unpack_bf16x2(a.w);
      const float* f = cache[i];
      yr[v] = make_uint4(pack_bf16x2(f[0] * r * w0.x, f[1] * r * w0.y), pack_bf16x2(f[2] * r * w1.x, f[3] * r * w1.y),
                         pack_bf16x2(f[4] * r * w2.x, f[5] * r * w2.y), pack_bf16x2(f[6] * r * w3.x, f[7] * r * w3.y));
    }
  }
}

// RMSNorm backward. Each CTA walks rows blockIdx.x, +gridDim.x, ...; dx per row, dw partial per CTA (fp32),
// reduced by rmsnorm_dw_reduce_kernel.  dx = rstd * (dy*w - xhat * mean(dy*w*xhat)), xhat = x * rstd.
// If dres_in is given it is added to dx (gradient arriving through the residual branch).
// NV = 16-byte vectors per thread (THREADS * NV * 8 >= cols): the per-thread arrays are sized by it, so the common widths
// get a small register footprint and enough CTAs per SM to keep HBM busy (one CTA has one row in flight).
template <int THREADS, int NV = 4>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int cols) {
  __shared__ float red[33];
  constexpr int MAXV = NV;
  const int nvec = cols >> 3;
  float dwacc[MAXV][8];
  float wreg[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
    if (v < nvec) {
      uint4 a = reinterpret_cast<const uint4*>(w)[v];
      float2 w0 = unpack_bf16x2(a.x), w1 = unpack_bf16x2(a.y), w2 = unpack_bf16x2(a.z), w3 = unpack_bf16x2(a.w);
      wreg[i][0] = w0.x; wreg[i][1] = w0.y; wreg[i][2] = w1.x; wreg[i][3] = w1.y;
      wreg[i][4] = w2.x; wreg[i][5] = w2.y; wreg[i][6] = w3.x; wreg[i][7] = w3.y;
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float r = rstd[row];
    float xh[MAXV][8], g[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) {
        uint4 a = reinterpret_cast<const uint4*>(x + row * cols)[v];
        uint4 b = reinterpret_cast<const uint4*>(dy + row * cols)[v];
        float2 x0 = unpack_bf16x2(a.x), x1 = unpack_bf16x2(a.y), x2 = unpack_bf16x2(a.z), x3 = unpack_bf16x2(a.w);
        float2 d0 = unpack_bf16x2(b.x), d1 = unpack_bf16x2(b.y), d2 = unpack_bf16x2(b.z), d3 = unpack_bf16x2(b.w);
        float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
        float dv[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] = xv[e] * r;
          g[i][e] = dv[e] * wreg[i][e];
          dot += g[i][e] * xh[i][e];
          dwacc[i][e] += dv[e] * xh[i][e];
        }
      }
    }
    dot = block_sum(dot, red) / cols;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = r * (g[i][e] - xh[i][e] * dot);
        if (dres_in) {
          uint4 c = reinterpret_cast<const uint4*>(dres_in + row * cols)[v];
          float2 c0 = unpack_bf16x2(c.x), c1 = unpack_bf16x2(c.y), c2 = unpack_bf16x2(c.z), c3 = unpack_bf16x2(c.w);
          o[0] += c0.x; o[1] += c0.y; o[2] += c1.x; o[3] += c1.y; o[4] += c2.x; o[5] += c2.y; o[6] += c3.x; o[7] += c3.y;
        }
        reinterpret_cast<uint4*>(dx + row * cols)[v] =
            make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
      }
    }
  }
  float* out = dw_partial + (long long)blockIdx.x * cols;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      reinterpret_cast<float4*>(out)[2 * v] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      reinterpret_cast<float4*>(out)[2 * v + 1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// Warp-per-row form of the RMSNorm backward for rows of up to 32 * 8 * NV elements: a warp keeps its whole row (x, dy and
// the residual-branch gradient) in registers as packed bf16, reduces with shuffles only and never meets a CTA barrier
// inside the row loop, so every warp keeps 3 * NV 16-byte loads in flight.  The weight-gradient partials of the four warps
// of a CTA are folded in shared memory (fixed order) into one partial row per CTA.
template <int NV>
__global__ void __launch_bounds__(128, 2)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                        const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw_partial, int rows, int cols) {
  extern __shared__ float fold[];  // [4][cols] fp32, then the weight row as bf16 (zero-padded to 256 * NV elements)
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int nvec = cols >> 3;
  const float inv_cols = 1.f / float(cols);
  uint4* wsm = reinterpret_cast<uint4*>(fold + 4 * cols);
  for (int v = threadIdx.x; v < 32 * NV; v += 128) wsm[v] = v < nvec ? reinterpret_cast<const uint4*>(w)[v] : make_uint4(0, 0, 0, 0);
  __syncthreads();
  float dwacc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
  }
  for (long long row = blockIdx.x * 4 + wib; row < rows; row += 4LL * gridDim.x) {
    const float r = rstd[row];
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + row * cols);
    const uint4* cr = dres_in ? reinterpret_cast<const uint4*>(dres_in + row * cols) : nullptr;
    uint4 a[NV], b[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      const bool in = v < nvec;
      a[i] = in ? xr[v] : make_uint4(0, 0, 0, 0);
      b[i] = in ? dr[v] : make_uint4(0, 0, 0, 0);
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const uint4 wq = wsm[lane + 32 * i];
      const uint32_t au[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, bu[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
      const uint32_t wu[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 xv = unpack_bf16x2(au[e]), dv = unpack_bf16x2(bu[e]), ww = unpack_bf16x2(wu[e]);
        const float xh0 = xv.x * r, xh1 = xv.y * r;
        dot += dv.x * ww.x * xh0 + dv.y * ww.y * xh1;
        dwacc[i][2 * e] += dv.x * xh0;
        dwacc[i][2 * e + 1] += dv.y * xh1;
      }
    }
    dot = warp_sum(dot) * inv_cols;
    uint4* outr = reinterpret_cast<uint4*>(dx + row * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      const uint4 wq = wsm[v];
      const uint4 cq = (cr && v < nvec) ? cr[v] : make_uint4(0, 0, 0, 0);
      const uint32_t au[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, bu[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
      const uint32_t wu[4] = {wq.x, wq.y, wq.z, wq.w}, cu[4] = {cq.x, cq.y, cq.z, cq.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 xv = unpack_bf16x2(au[e]), dv = unpack_bf16x2(bu[e]), ww = unpack_bf16x2(wu[e]), cc = unpack_bf16x2(cu[e]);
        o[e] = pack_bf16x2(r * (dv.x * ww.x - xv.x * r * dot) + cc.x, r * (dv.y * ww.y - xv.y * r * dot) + cc.y);
      }
      if (v < nvec) outr[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float* f = fold + wib * cols + 8 * v;
      reinterpret_cast<float4*>(f)[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      reinterpret_cast<float4*>(f)[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
  __syncthreads();
  float* out = dw_partial + (long long)blockIdx.x * cols;
  for (int col = threadIdx.x; col < cols; col += 128) out[col] = (fold[col] + fold[cols + col]) + (fold[2 * cols + col] + fold[3 * cols + col]);
}

// dw[c] (+)= sum_b partial[b][c]; output bf16 or fp32.  One CTA per 32 columns: 8 row lanes x 32 columns read the partials
// with 128-byte coalesced accesses, then the row lanes are folded through shared memory (fixed order: deterministic).
__global__ void __launch_bounds__(256) colsum_partial_kernel(const float* __restrict__ partial, int nblocks, int cols,
                                                             __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ out_f32, int accumulate) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < cols)
    for (int b = rl; b < nblocks; b += 8) s += partial[(long long)b * cols + c];
  red[rl][lane] = s;
  __syncthreads();
  if (rl == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += red[j][lane];
    if (out_f32) out_f32[c] = accumulate ? out_f32[c] + t : t;
    if (out_bf16) out_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[c]) + t : t);
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE, half-split layout, in place on a packed projection buffer [tokens, row_stride] whose first
// (n_heads * d) columns starting at col_offset are heads of width d.  cos/sin: [max_pos, d/2] fp32.
// position of token t = pos[t] if pos != nullptr else pos_offset + (t % seq_len).  sign = -1 -> inverse (backward).
// ------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, int tokens, int seq_len,
                            int pos_offset, int row_stride, int col_offset, int n_heads, int d, float sign) {
  pdl_prologue();
  const int half = d >> 1;
  const int vec_per_head = half >> 3;  // 8 pairs per 16-byte vector
  const long long total = (long long)tokens * n_heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % vec_per_head);
    const int h = int((i / vec_per_head) % n_heads);
    const long long t = i / ((long long)vec_per_head * n_heads);
    const int p = pos ? pos[t] : pos_offset + int(t % seq_len);
    __nv_bfloat16* base = buf + t * row_stride + col_offset + h * d + v * 8;
    uint4 a = *reinterpret_cast<uint4*>(base);
    uint4 b = *reinterpret_cast<uint4*>(base + half);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)p * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)p * half + v * 8);
    float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    float c[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    float s[8] = {sa.x * sign, sa.y * sign, sa.z * sign, sa.w * sign, sb.x * sign, sb.y * sign, sb.z * sign, sb.w * sign};
    uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 x1 = unpack_bf16x2(au[e]), x2 = unpack_bf16x2(bu[e]);
      o1[e] = pack_bf16x2(x1.x * c[2 * e] - x2.x * s[2 * e], x1.y * c[2 * e + 1] - x2.y * s[2 * e + 1]);
      o2[e] = pack_bf16x2(x1.x * s[2 * e] + x2.x * c[2 * e], x1.y * s[2 * e + 1] + x2.y * c[2 * e + 1]);
    }
    *reinterpret_cast<uint4*>(base) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(base + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU on a fused projection gu[rows, 2I] (gate = first I columns): h = silu(g) * u.
// Backward: given dh, writes dgu in the same [rows, 2I] layout and (optionally) recomputes h.
// ------------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long rows,
                                  int inter) {
  const int vpr = inter >> 3;
  const long long total = rows * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int v = int(i - r * vpr);
    const __nv_bfloat16* row = gu + r * 2 * inter;
    uint4 g = reinterpret_cast<const uint4*>(row)[v];
    uint4 u = reinterpret_cast<const uint4*>(row + inter)[v];
    uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 a = unpack_bf16x2(gg[e]), b = unpack_bf16x2(uu[e]);
      o[e] = pack_bf16x2(silu_f(a.x) * b.x, silu_f(a.y) * b.y);
    }
    reinterpret_cast<uint4*>(h + r * inter)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// counts != nullptr: the rows form groups of `cap` rows (expert capacity layout, blockIdx.y = group) of which only the first
// round_up_128(counts[g]) are in use; the rest is neither read nor written (the ragged GEMMs never look at it).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, __nv_bfloat16* __restrict__ h_out, long long rows,
                                  int inter, const int* __restrict__ counts, int cap) {
  const int vpr = inter >> 3;
  long long row0 = 0;
  if (counts) {
    row0 = (long long)blockIdx.y * cap;
    rows = min((counts[blockIdx.y] + 127) & ~127, cap);
  }
  const long long total = rows * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = row0 + i / vpr;
    const int v = int(i % vpr);
    const __nv_bfloat16* row = gu + r * 2 * inter;
    uint4 g = reinterpret_cast<const uint4*>(row)[v];
    uint4 u = reinterpret_cast<const uint4*>(row + inter)[v];
    uint4 d = reinterpret_cast<const uint4*>(dh + r * inter)[v];
    uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w}, dd[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4], oh[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 a = unpack_bf16x2(gg[e]), b = unpack_bf16x2(uu[e]), c = unpack_bf16x2(dd[e]);
      float s0 = 1.f / (1.f + __expf(-a.x)), s1 = 1.f / (1.f + __expf(-a.y));
      float si0 = a.x * s0, si1 = a.y * s1;
      // d silu(x)/dx = s + x*s*(1-s)
      og[e] = pack_bf16x2(c.x * b.x * (s0 + si0 * (1.f - s0)), c.y * b.y * (s1 + si1 * (1.f - s1)));
      ou[e] = pack_bf16x2(c.x * si0, c.y * si1);
      oh[e] = pack_bf16x2(si0 * b.x, si1 * b.y);
    }
    __nv_bfloat16* orow = dgu + r * 2 * inter;
    reinterpret_cast<uint4*>(orow)[v] = make_uint4(og[0], og[1], og[2], og[3]);
    reinterpret_cast<uint4*>(orow + inter)[v] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    if (h_out) reinterpret_cast<uint4*>(h_out + r * inter)[v] = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding: out[t] = table[clamp(ids[t])] * scale.  Gradient: ids sorted on the host side of the op
// (sorted_ids, order); one warp per run of equal ids sums its rows in fp32 -> deterministic, no atomics.
// ------------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long tokens, int hidden, int vocab, float scale) {
  pdl_prologue();
  const int vpr = hidden >> 3;
  const long long total = tokens * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = int(i - t * vpr);
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    uint4 a = reinterpret_cast<const uint4*>(table + id * hidden)[v];
    if (scale != 1.f) {
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      a = make_uint4(pack_bf16x2(f0.x * scale, f0.y * scale), pack_bf16x2(f1.x * scale, f1.y * scale),
                     pack_bf16x2(f2.x * scale, f2.y * scale), pack_bf16x2(f3.x * scale, f3.y * scale));
    }
    reinterpret_cast<uint4*>(out + t * hidden)[v] = a;
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ order,
                                     const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dtable,
                                     long long tokens, int hidden, int vocab, float scale, int accumulate) {
  const long long warp_global = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= tokens) return;
  long long id = sorted_ids[warp_global];
  if (warp_global > 0 && sorted_ids[warp_global - 1] == id) return;  // not the start of a run
  long long cid = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const int vpr = hidden >> 3;
  for (int v = lane; v < vpr; v += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long j = warp_global; j < tokens && sorted_ids[j] == id; ++j) {
      uint4 a = reinterpret_cast<const uint4*>(dout + order[j] * hidden)[v];
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    uint4* dst = reinterpret_cast<uint4*>(dtable + cid * hidden) + v;
    if (accumulate) {
      uint4 o = *dst;
      float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z), f3 = unpack_bf16x2(o.w);
      *dst = make_uint4(pack_bf16x2(f0.x + acc[0] * scale, f0.y + acc[1] * scale), pack_bf16x2(f1.x + acc[2] * scale, f1.y + acc[3] * scale),
                        pack_bf16x2(f2.x + acc[4] * scale, f2.y + acc[5] * scale), pack_bf16x2(f3.x + acc[6] * scale, f3.y + acc[7] * scale));
    } else {
      *dst = make_uint4(pack_bf16x2(acc[0] * scale, acc[1] * scale), pack_bf16x2(acc[2] * scale, acc[3] * scale),
                        pack_bf16x2(acc[4] * scale, acc[5] * scale), pack_bf16x2(acc[6] * scale, acc[7] * scale));
    }
  }
}

// fp32 -> bf16 cast (optionally accumulating into the destination)
__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n,
                                     int accumulate, float scale) {
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 3 < n) {
      float4 a = *reinterpret_cast<const float4*>(in + i);
      float o[4] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale};
      if (accumulate) {
        uint2 p = *reinterpret_cast<uint2*>(out + i);
        float2 p0 = unpack_bf16x2(p.x), p1 = unpack_bf16x2(p.y);
        o[0] += p0.x; o[1] += p0.y; o[2] += p1.x; o[3] += p1.y;
      }
      *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    } else {
      for (long long j = i; j < n; ++j) {
        float o = in[j] * scale + (accumulate ? __bfloat162float(out[j]) : 0.f);
        out[j] = __float2bfloat16(o);
      }
    }
  }
}

static inline int grid_for(long long work_items, int threads, int cap = 148 * 16) {
  long long b = (work_items + threads - 1) / threads;
  if (b < 1) b = 1;
  return int(b < cap ? b : cap);
}

}  // namespace ats

using namespace ats;

ATS_API int ats_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd,
                            long long rows, int cols, float eps, void* stream) {
  if (cols & 7) return 1003;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(res);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto S = static_cast<__nv_bfloat16*>(sum_out);
  if (rows == 0) return 0;
  if (rows <= 1024 && cols <= 256 * 32) {  // decode-sized: the launch overlaps the tail of the kernel before it
    cudaError_t ce = cols <= 128 * 32 ? launch_pdl(rmsnorm_fwd_kernel<128>, dim3((unsigned)rows), dim3(128), 0, s, X, R, W, Y, S, rstd, cols, eps)
                                      : launch_pdl(rmsnorm_fwd_kernel<256>, dim3((unsigned)rows), dim3(256), 0, s, X, R, W, Y, S, rstd, cols, eps);
    return int(ce != cudaSuccess ? ce : cudaGetLastError());
  }
  if (cols <= 128 * 32) rmsnorm_fwd_kernel<128><<<(unsigned)rows, 128, 0, s>>>(X, R, W, Y, S, rstd, cols, eps);
  else if (cols <= 256 * 32) rmsnorm_fwd_kernel<256><<<(unsigned)rows, 256, 0, s>>>(X, R, W, Y, S, rstd, cols, eps);
  else if (cols <= 512 * 32) rmsnorm_fwd_kernel<512><<<(unsigned)rows, 512, 0, s>>>(X, R, W, Y, S, rstd, cols, eps);
  else return 1003;
  return int(cudaGetLastError());
}

// dw_partial: fp32 scratch of nblocks*cols; dw written as bf16 (dw_bf16) and/or fp32 (dw_f32).
static int rmsnorm_bwd_launch(const void* x, const void* w, const void* dy, const float* rstd, const void* dres_in, void* dx,
                              float* dw_partial, int nblocks, void* dw_bf16, float* dw_f32, int accumulate, long long rows,
                              int cols, void* stream, bool warp_rows) {
  if (cols & 7) return 1003;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto DR = static_cast<const __nv_bfloat16*>(dres_in);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  static const bool warp_rows_on = [] {
    const char* e = getenv("ATS_NORM_WARP_ROWS");  // "0" keeps the CTA-per-row kernels everywhere (for comparisons)
    return !(e && e[0] == '0');
  }();
  if (warp_rows && warp_rows_on && cols <= 2048 && rows >= 1024 && nblocks >= 1) {
    // many rows of moderate width: one warp per row, two CTAs of four warps per SM
    const int nb = nblocks < 296 ? nblocks : 296;
    const size_t sm = size_t(4) * cols * sizeof(float) + (cols <= 1024 ? 4 : 8) * 512;
    if (cols <= 1024) rmsnorm_bwd_warp_kernel<4><<<nb, 128, sm, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
    else rmsnorm_bwd_warp_kernel<8><<<nb, 128, sm, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
    colsum_partial_kernel<<<(cols + 31) / 32, 256, 0, s>>>(dw_partial, nb, cols, static_cast<__nv_bfloat16*>(dw_bf16), dw_f32, accumulate);
    return int(cudaGetLastError());
  }
  if (cols <= 128 * 8) rmsnorm_bwd_kernel<128, 1><<<nblocks, 128, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
  else if (cols <= 128 * 16) rmsnorm_bwd_kernel<128, 2><<<nblocks, 128, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
  else if (cols <= 128 * 32) rmsnorm_bwd_kernel<128><<<nblocks, 128, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
  else if (cols <= 256 * 32) rmsnorm_bwd_kernel<256><<<nblocks, 256, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
  else if (cols <= 512 * 32) rmsnorm_bwd_kernel<512><<<nblocks, 512, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, (int)rows, cols);
  else return 1003;
  colsum_partial_kernel<<<(cols + 31) / 32, 256, 0, s>>>(dw_partial, nblocks, cols, static_cast<__nv_bfloat16*>(dw_bf16),
                                                          dw_f32, accumulate);
  return int(cudaGetLastError());
}

ATS_API int ats_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres_in, void* dx,
                            float* dw_partial, int nblocks, void* dw_bf16, float* dw_f32, int accumulate, long long rows,
                            int cols, void* stream) {
  return rmsnorm_bwd_launch(x, w, dy, rstd, dres_in, dx, dw_partial, nblocks, dw_bf16, dw_f32, accumulate, rows, cols, stream, true);
}

ATS_API int ats_colsum_partial(const float* partial, int nblocks, int cols, void* out_bf16, float* out_f32, int accumulate,
                               void* stream) {
  colsum_partial_kernel<<<(cols + 31) / 32, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partial, nblocks, cols, static_cast<__nv_bfloat16*>(out_bf16), out_f32, accumulate);
  return int(cudaGetLastError());
}

ATS_API int ats_rope(void* buf, const float* cos_t, const float* sin_t, const int* pos, long long tokens, int seq_len,
                     int pos_offset, int row_stride, int col_offset, int n_heads, int d, int inverse, void* stream) {
  if ((d & 15) || (row_stride & 7) || (col_offset & 7)) return 1003;
  const long long work = tokens * n_heads * (d >> 4);
  if (work == 0) return 0;
  if (tokens <= 1024) {
    cudaError_t ce = launch_pdl(rope_kernel, dim3(grid_for(work, 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                static_cast<__nv_bfloat16*>(buf), cos_t, sin_t, pos, (int)tokens, seq_len, pos_offset, row_stride,
                                col_offset, n_heads, d, inverse ? -1.f : 1.f);
    return int(ce != cudaSuccess ? ce : cudaGetLastError());
  }
  rope_kernel<<<grid_for(work, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(buf), cos_t, sin_t, pos, (int)tokens, seq_len, pos_offset, row_stride, col_offset, n_heads, d,
      inverse ? -1.f : 1.f);
  return int(cudaGetLastError());
}

ATS_API int ats_swiglu_fwd(const void* gu, void* h, long long rows, int inter, void* stream) {
  if (inter & 7) return 1003;
  if (rows == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(rows * (inter >> 3), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), rows, inter);
  return int(cudaGetLastError());
}

ATS_API int ats_swiglu_bwd(const void* gu, const void* dh, void* dgu, void* h_out, long long rows, int inter, void* stream) {
  if (inter & 7) return 1003;
  if (rows == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(rows * (inter >> 3), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(dgu),
      static_cast<__nv_bfloat16*>(h_out), rows, inter, nullptr, 0);
  return int(cudaGetLastError());
}

// Capacity layout [groups, cap, *]: only the first round_up_128(counts[g]) rows of every group are processed.
ATS_API int ats_swiglu_bwd_grouped(const void* gu, const void* dh, void* dgu, void* h_out, int groups, int cap, const int* counts, int inter,
                                   void* stream) {
  if ((inter & 7) || groups > 65535) return 1003;
  if (groups == 0 || cap == 0) return 0;
  unsigned gx = grid_for((long long)cap * (inter >> 3), 256);
  const unsigned per_group = (148u * 16u + groups - 1) / groups;  // about 16 CTAs per SM over all groups
  if (gx > per_group) gx = per_group;
  swiglu_bwd_kernel<<<dim3(gx, groups), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(dgu),
      static_cast<__nv_bfloat16*>(h_out), 0, inter, counts, cap);
  return int(cudaGetLastError());
}

ATS_API int ats_embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int hidden, int vocab,
                              float scale, void* stream) {
  if (hidden & 7) return 1003;
  if (tokens == 0) return 0;
  if (tokens <= 1024) {
    cudaError_t ce = launch_pdl(embedding_fwd_kernel, dim3(grid_for(tokens * (hidden >> 3), 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), tokens, hidden, vocab, scale);
    return int(ce != cudaSuccess ? ce : cudaGetLastError());
  }
  embedding_fwd_kernel<<<grid_for(tokens * (hidden >> 3), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), tokens, hidden, vocab, scale);
  return int(cudaGetLastError());
}

ATS_API int ats_embedding_bwd(const long long* sorted_ids, const long long* order, const void* dout, void* dtable,
                              long long tokens, int hidden, int vocab, float scale, int accumulate, void* stream) {
  if (hidden & 7) return 1003;
  if (tokens == 0) return 0;
  const int threads = 256;
  const long long blocks = (tokens * 32 + threads - 1) / threads;
  embedding_bwd_kernel<<<(unsigned)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      sorted_ids, order, static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dtable), tokens, hidden, vocab,
      scale, accumulate);
  return int(cudaGetLastError());
}

ATS_API int ats_cast_f32_bf16(const float* in, void* out, long long n, int accumulate, float scale, void* stream) {
  if (n == 0) return 0;
  cast_f32_bf16_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      in, static_cast<__nv_bfloat16*>(out), n, accumulate, scale);
  return int(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in ats_noalloc.h).
//
// ats_rmsnorm_bwd needs an fp32 scratch of nblocks * cols floats for the per-block weight-gradient partials and
// leaves its allocation to the caller.  Some callers cannot allocate at all: code running inside a CUDA-graph
// capture or another region where cudaMalloc is illegal, a real-time loop that must not touch the driver's
// allocator, a host application that hands this library a fixed memory budget.  For them the partials live in
// the file-scope device array below, which every GPU that loads this library keeps until the process exits
// (kNoAllocMaxBlocks * kNoAllocMaxCols * 4 bytes = 4 MiB).
// ------------------------------------------------------------------------------------------------
namespace ats {
constexpr int kNoAllocMaxBlocks = 128;
constexpr int kNoAllocMaxCols = 8192;
constexpr int kNoAllocMaxDevices = 64;
static __device__ __align__(256) float g_rmsnorm_bwd_partials[kNoAllocMaxBlocks * kNoAllocMaxCols];
// Device address of the array above, per device.  The array's name is only a host-side handle in host code;
// the address a kernel can use comes from cudaGetSymbolAddress with that device current.
static float* g_rmsnorm_bwd_partials_addr[kNoAllocMaxDevices] = {};
}  // namespace ats

ATS_API int ats_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, const void* dres_in,
                                    void* dx, void* dw_bf16, float* dw_f32, int accumulate, long long rows, int cols,
                                    void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7)) return 1003;
  if (rows > 2147483647LL) return 1003;     // the kernels index rows with 32-bit integers
  if (cols > kNoAllocMaxCols) return 2001;  // ATS_ERR_NOALLOC_TOO_LARGE
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return int(e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) return 2002;  // ATS_ERR_NOALLOC_DEVICE
  if (!g_rmsnorm_bwd_partials_addr[dev]) {
    // first call on this device: resolve the device address once (do this before any stream capture)
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_bwd_partials);
    if (e != cudaSuccess) return int(e);
    g_rmsnorm_bwd_partials_addr[dev] = p;
  }
  float* partial = g_rmsnorm_bwd_partials_addr[dev];
  const int nblocks = rows < kNoAllocMaxBlocks ? int(rows) : kNoAllocMaxBlocks;
  // Every partial that the reduction reads (nblocks rows of cols floats) is written by the first kernel of this
  // same call, so nothing has to be cleared even though the array still holds the previous call's values.
  return rmsnorm_bwd_launch(x, w, dy, rstd, dres_in, dx, partial, nblocks, dw_bf16, dw_f32, accumulate, rows, cols, stream, false);
}

ATS_API void ats_rmsnorm_bwd_noalloc_limits(int* max_cols, long long* scratch_bytes) {
  if (max_cols) *max_cols = kNoAllocMaxCols;
  if (scratch_bytes) *scratch_bytes = (long long)kNoAllocMaxBlocks * kNoAllocMaxCols * 4;
}

ATS_API const char* ats_noalloc_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case 1003: return "bad shape: rows and cols must be positive, rows at most 2^31 - 1 and cols a multiple of 8";
    case 2001: return "problem too large for the built-in scratch: cols exceeds the limit reported by ats_rmsnorm_bwd_noalloc_limits";
    case 2002: return "device ordinal outside the range this library keeps scratch addresses for";
    default: return "CUDA runtime error (the code is a cudaError_t)";
  }
}

// ------------------------------------------------------------------------------------------------ fp8 quantisation
#include <cuda_fp8.h>

namespace ats {

// One CTA per row: scale = amax / 448 (e4m3 max), q = x / scale.  The row is read twice (second time from L1 / L2).
__global__ void __launch_bounds__(256) quantize_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ x, long long ld, uint8_t* __restrict__ q,
                                                                 long long ldq, float* __restrict__ scale, int cols) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ld;
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < cols; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = block_max(amax, red);
  const float sc = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float inv = 1.f / sc;
  if (threadIdx.x == 0) scale[row] = sc;
  uint8_t* qr = q + row * ldq;
  for (int i = threadIdx.x * 8; i < cols; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    uint16_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]);
      o[j] = __nv_cvt_float2_to_fp8x2(make_float2(f.x * inv, f.y * inv), __NV_SATFINITE, __NV_E4M3);
    }
    *reinterpret_cast<uint2*>(qr + i) = make_uint2(uint32_t(o[0]) | (uint32_t(o[1]) << 16), uint32_t(o[2]) | (uint32_t(o[3]) << 16));
  }
}

// One CTA per row: scale = amax / 127, q = round(x / scale) as signed bytes.  inv_smooth (optional, [cols] bf16): the row is
// multiplied by it first (SmoothQuant: the per-channel factors that were folded into the weight are divided out of the activations).
__global__ void __launch_bounds__(256) quantize_rows_int8_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int8_t* __restrict__ q,
                                                                 long long ldq, float* __restrict__ scale, int cols,
                                                                 const __nv_bfloat16* __restrict__ inv_smooth) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ld;
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < cols; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint4 sm = inv_smooth ? *reinterpret_cast<const uint4*>(inv_smooth + i) : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w}, w[4] = {sm.x, sm.y, sm.z, sm.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]), g = unpack_bf16x2(w[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x * g.x), fabsf(f.y * g.y)));
    }
  }
  amax = block_max(amax, red);
  const float sc = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
  const float inv = 1.f / sc;
  if (threadIdx.x == 0) scale[row] = sc;
  int8_t* qr = q + row * ldq;
  for (int i = threadIdx.x * 8; i < cols; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint4 sm = inv_smooth ? *reinterpret_cast<const uint4*>(inv_smooth + i) : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w}, w[4] = {sm.x, sm.y, sm.z, sm.w};
    uint32_t o[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]), g = unpack_bf16x2(w[j]);
      const int a = max(-127, min(127, __float2int_rn(f.x * g.x * inv))), b = max(-127, min(127, __float2int_rn(f.y * g.y * inv)));
      o[j >> 1] |= (uint32_t(a & 0xff) | (uint32_t(b & 0xff) << 8)) << (16 * (j & 1));
    }
    *reinterpret_cast<uint2*>(qr + i) = make_uint2(o[0], o[1]);
  }
}

}  // namespace ats

// x: bf16 [rows, cols] with pitch ld; q: e4m3 bytes [rows, cols] with pitch ldq; scale: fp32 [rows].  cols % 8 == 0.
ATS_API int ats_quantize_rows_e4m3(const void* x, long long ld, void* q, long long ldq, float* scale, long long rows, int cols, void* stream) {
  if ((cols & 7) || (ld & 7) || (ldq & 7)) return 1003;
  if (rows == 0) return 0;
  ats::quantize_rows_e4m3_kernel<<<unsigned(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ld, static_cast<uint8_t*>(q), ldq, scale, cols);
  return int(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------ debug build
#ifdef ATS_DEBUG
namespace ats {
__device__ int g_debug_report[4] = {0, 0, 0, 0};
}
#endif
// out4 = {code, kernel id, block, detail} of the first bounds check that failed since the last call (all zero: none), and the
// report is cleared.  Returns 1 in the debug build, 0 in the release build (which has no checks).
ATS_API int ats_debug_report(int* out4) {
#ifdef ATS_DEBUG
  int zero[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(out4, ats::g_debug_report, sizeof(zero)) != cudaSuccess) return -1;
  if (cudaMemcpyToSymbol(ats::g_debug_report, zero, sizeof(zero)) != cudaSuccess) return -1;
  return 1;
#else
  for (int i = 0; i < 4; ++i) out4[i] = 0;
  return 0;
#endif
}

ATS_API int ats_quantize_rows_int8(const void* x, long long ld, void* q, long long ldq, float* scale, long long rows, int cols,
                                   const void* inv_smooth, void* stream) {
  if ((cols & 7) || (ld & 7) || (ldq & 7)) return 1003;
  if (rows == 0) return 0;
  ats::quantize_rows_int8_kernel<<<unsigned(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ld, static_cast<int8_t*>(q), ldq, scale, cols, static_cast<const __nv_bfloat16*>(inv_smooth));
  return int(cudaGetLastError());
}
