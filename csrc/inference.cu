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
#include <stdlib.h>

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
  int* chunk_done;     // [B, Hkv] arrival counters (zero between launches) or nullptr: the last CTA of a (sequence, KV head) merges
};

template <int D, int REP>
__global__ void __launch_bounds__(DEC_THREADS) decode_attn_kernel(const DecodeArgs p) {
  __shared__ float s_q[REP][D];
  __shared__ float s_p[REP][DEC_CHUNK];
  __shared__ float s_red[DEC_THREADS / 32][REP][D];
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

  // ---- scores: D / 8 lanes share a key row (one 16-byte load each, so a warp's load covers whole rows: with one thread per
  // row every load instruction touched 32 cache lines and the kernel was bound by L1 wavefronts at a third of HBM speed);
  // the partial dot products are folded with shuffles.  Four rows per lane group are requested before the first is used.
  {
    constexpr int LPR = D / 8, RPW = 32 / LPR, ROWS_PER_PASS = (DEC_THREADS / 32) * RPW, SUNR = 4;
    const int sub = lane / LPR, l8 = lane % LPR;
    float q[REP][8];
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) q[h][e] = s_q[h][8 * l8 + e];
    for (int r0 = warp * RPW + sub; r0 < DEC_CHUNK; r0 += ROWS_PER_PASS * SUNR) {
      uint4 kv[SUNR];
#pragma unroll
      for (int u = 0; u < SUNR; ++u) {
        const int key = k0 + r0 + u * ROWS_PER_PASS;
        if (active && key < k_end) {
          const __nv_bfloat16* krow = (key == n_old) ? p.k_new + (long long)b * p.ld_qkv + hk * D : kc + key * row_stride;
          kv[u] = *reinterpret_cast<const uint4*>(krow + 8 * l8);
        } else {
          kv[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < SUNR; ++u) {
        const int r = r0 + u * ROWS_PER_PASS;
        const float2 a = unpack_bf16x2(kv[u].x), bq = unpack_bf16x2(kv[u].y), c = unpack_bf16x2(kv[u].z), e = unpack_bf16x2(kv[u].w);
        float part[REP];
#pragma unroll
        for (int h = 0; h < REP; ++h)
          part[h] = a.x * q[h][0] + a.y * q[h][1] + bq.x * q[h][2] + bq.y * q[h][3] + c.x * q[h][4] + c.y * q[h][5] + e.x * q[h][6] + e.y * q[h][7];
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1)
#pragma unroll
          for (int h = 0; h < REP; ++h) part[h] += __shfl_xor_sync(0xffffffffu, part[h], off);
        if (l8 == 0 && r < DEC_CHUNK) {
          const bool valid = active && (k0 + r) < k_end;
#pragma unroll
          for (int h = 0; h < REP; ++h) s_p[h][r] = valid ? part[h] : -INFINITY;
        }
      }
    }
  }
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
  // ---- P V: thread (g, d8) sums keys g, g + G, ... for the eight dims 8 d8 .. 8 d8 + 7 of every head.  A row is read by
  // D / 8 threads with 16-byte loads and four rows are requested before the first is used: the loop is bound by the number of
  // bytes in flight, not by arithmetic.
  constexpr int TPR = D / 8, G = DEC_THREADS / TPR;  // threads per row, row groups
  const int g = tid / TPR, d8 = tid % TPR;
  float o[REP][8];
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int e = 0; e < 8; ++e) o[h][e] = 0.f;
  if (active) {
    constexpr int UNR = 4;
    for (int kk = k0 + g; kk < k_end; kk += G * UNR) {
      uint4 vv[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int kr = kk + u * G;
        if (kr < k_end) {
          const __nv_bfloat16* vrow = (kr == n_old) ? p.v_new + (long long)b * p.ld_qkv + hk * D : vc + kr * row_stride;
          vv[u] = *reinterpret_cast<const uint4*>(vrow + 8 * d8);
        } else {
          vv[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int kr = kk + u * G;
        if (kr >= k_end) break;
        const float2 v0 = unpack_bf16x2(vv[u].x), v1 = unpack_bf16x2(vv[u].y), v2 = unpack_bf16x2(vv[u].z), v3 = unpack_bf16x2(vv[u].w);
#pragma unroll
        for (int h = 0; h < REP; ++h) {
          const float pr = s_p[h][kr - k0];
          o[h][0] += pr * v0.x; o[h][1] += pr * v0.y; o[h][2] += pr * v1.x; o[h][3] += pr * v1.y;
          o[h][4] += pr * v2.x; o[h][5] += pr * v2.y; o[h][6] += pr * v3.x; o[h][7] += pr * v3.y;
        }
      }
    }
  }
  // fold the row groups that share a warp (lanes d8 and d8 + TPR, ...), then the warps through shared memory
#pragma unroll
  for (int off = TPR; off < 32; off <<= 1)
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) o[h][e] += __shfl_xor_sync(0xffffffffu, o[h][e], off);
  if (lane < TPR) {
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) s_red[warp][h][8 * d8 + e] = o[h][e];
  }
  __syncthreads();
  for (int i = tid; i < REP * D; i += DEC_THREADS) {
    const int h = i / D, d = i % D;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) t += s_red[w][h][d];
    p.part_o[(((long long)b * p.Hq + hk * REP + h) * p.n_chunks + chunk) * D + d] = t;
  }
}

// ------------------------------------------------------------------------------------------------
// Tensor-core form of the same kernel (default).  With fp32 FMAs the kernel above issues ~1300 warp instructions per 32 keys
// (four query heads per KV head, D = 128) and is bound by instruction issue at a third of HBM speed; both products are
// therefore done with warp-level MMAs (m16n8k16, bf16 in, fp32 out) whose 16 rows hold the query heads of the group.  A
// decode step is bandwidth-bound, so the warp-level MMA is enough; no shared-memory staging or transposing loads are needed:
//
// * S = Q K^T: the sum over the head dimension does not care about the order of its terms, so the dimension index is permuted
//   such that the 16-byte piece a lane loads from a key row IS its B fragment for two consecutive k-steps (words 0,1 and 2,3);
//   the Q fragments are read from global memory with the same permutation.
// * O = P V: B wants two KEYS of one dimension in a register, memory holds two DIMENSIONS of one key in a word.  A lane loads
//   16 bytes (four such words) of four keys and two byte permutes per word turn them into the fragments of TWO column tiles, one
//   holding the even and one the odd dimension of the words; output columns are just another order of the dimensions.
// Every warp handles 32 keys of the chunk for all dimensions; the warps' partial outputs are folded through shared memory.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// OCC: CTAs per SM the register allocation is cut for (2: 116 registers, no spills; 3: 80 registers, about 240 bytes of spills
// but half again as many loads in flight).
template <int D, int REP, int OCC = 2>
__global__ void __launch_bounds__(DEC_THREADS, OCC) decode_attn_mma_kernel(const DecodeArgs p) {
  pdl_prologue();
  static_assert(REP <= 8 && D % 32 == 0, "query heads of a group sit in rows 0..7 of the MMA");
  __shared__ float s_p[REP][DEC_CHUNK];
  __shared__ __align__(16) float s_red[DEC_THREADS / 32][REP][D];
  const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  int n_old = p.lengths ? p.lengths[b] : p.length;
  if (!ATS_DBG_CHECK(n_old >= 0 && n_old < p.max_len, kDbgDecodeAttn, n_old)) return;
  const int n_tot = n_old + 1;  // the new token attends to itself
  const int k0 = chunk * DEC_CHUNK;
  const bool active = k0 < n_tot;
  const int k_end = min(k0 + DEC_CHUNK, n_tot);
  __nv_bfloat16* kc = p.k_cache + (long long)b * p.cache_b_stride + (long long)hk * D;
  __nv_bfloat16* vc = p.v_cache + (long long)b * p.cache_b_stride + (long long)hk * D;
  const long long row_stride = (long long)p.Hkv * D;
  const __nv_bfloat16* k_new = p.k_new + (long long)b * p.ld_qkv + hk * D;
  const __nv_bfloat16* v_new = p.v_new + (long long)b * p.ld_qkv + hk * D;
  // the new token's K / V row goes into the cache (by the CTA that owns its position); this CTA reads it from the projection
  if (active && n_old >= k0 && n_old < k0 + DEC_CHUNK && n_old < p.max_len) {
    for (int d = tid; d < D; d += DEC_THREADS) {
      kc[n_old * row_stride + d] = k_new[d];
      vc[n_old * row_stride + d] = v_new[d];
    }
  }
  const int kw0 = warp * 32;  // this warp's keys inside the chunk

  // ---- S = Q K^T
  {
    uint32_t qa[D / 16][2];  // A fragments (rows g < REP): [virtual k-step][a0, a2]
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(p.q + (long long)b * p.ld_qkv + (hk * REP + (g < REP ? g : 0)) * D);
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      uint4 w = make_uint4(0, 0, 0, 0);
      if (g < REP) w = *reinterpret_cast<const uint4*>(qrow + 4 * (4 * j + t));
      qa[2 * j][0] = w.x; qa[2 * j][1] = w.y; qa[2 * j + 1][0] = w.z; qa[2 * j + 1][1] = w.w;
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int r = kw0 + nt * 8 + g;  // the key whose row this lane loads (column g of the tile)
      const int key = k0 + r;
      const bool ok = active && key < k_end;
      const __nv_bfloat16* krow = (key == n_old) ? k_new : kc + key * row_stride;
      uint4 kv[D / 32];
#pragma unroll
      for (int j = 0; j < D / 32; ++j) kv[j] = ok ? *reinterpret_cast<const uint4*>(krow + 8 * (4 * j + t)) : make_uint4(0, 0, 0, 0);
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < D / 32; ++j) {
        mma_16816_bf16(c, qa[2 * j][0], 0u, qa[2 * j][1], 0u, kv[j].x, kv[j].y);
        mma_16816_bf16(c, qa[2 * j + 1][0], 0u, qa[2 * j + 1][1], 0u, kv[j].z, kv[j].w);
      }
      if (g < REP) {  // c[0], c[1]: head g, keys 2t and 2t + 1 of the tile
        const int c0 = kw0 + nt * 8 + 2 * t;
        s_p[g][c0] = (active && k0 + c0 < k_end) ? c[0] * p.scale : -INFINITY;
        s_p[g][c0 + 1] = (active && k0 + c0 + 1 < k_end) ? c[1] * p.scale : -INFINITY;
      }
    }
  }
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
  // ---- O = P V over this warp's 32 keys (two blocks of 16), all dimensions.  Lane (g, t) loads 16 bytes (dims 64 rd + 8 g .. + 7)
  // of four keys: eight lanes cover 128 contiguous bytes of a row.  Word i of the piece holds dims 8 g + 2 i, + 1: the low halves of
  // two keys form the B fragment of the column tile "even dims of word i", the high halves that of "odd dims of word i".
  constexpr int RD = D / 64;
  float oe[RD][4][4], oo[RD][4][4];
#pragma unroll
  for (int rd = 0; rd < RD; ++rd)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) oe[rd][i][e] = oo[rd][i][e] = 0.f;
  if (active && k0 + kw0 < k_end) {
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      const int kk0 = kw0 + kb * 16;
      if (k0 + kk0 >= k_end) break;
      uint32_t pa0 = 0u, pa2 = 0u;  // P fragments (bf16 pairs): keys 2t, 2t + 1 and 2t + 8, 2t + 9 of head g
      if (g < REP) {
        pa0 = pack_bf16x2(s_p[g][kk0 + 2 * t], s_p[g][kk0 + 2 * t + 1]);
        pa2 = pack_bf16x2(s_p[g][kk0 + 2 * t + 8], s_p[g][kk0 + 2 * t + 9]);
      }
      uint4 w[RD][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = k0 + kk0 + 2 * t + (i & 1) + (i >> 1) * 8;
        const __nv_bfloat16* vrow = (key == n_old) ? v_new : vc + key * row_stride;
#pragma unroll
        for (int rd = 0; rd < RD; ++rd)
          w[rd][i] = key < k_end ? *reinterpret_cast<const uint4*>(vrow + 64 * rd + 8 * g) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int rd = 0; rd < RD; ++rd) {
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&w[rd][0]);
        const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&w[rd][1]);
        const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&w[rd][2]);
        const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&w[rd][3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mma_16816_bf16(oe[rd][i], pa0, 0u, pa2, 0u, __byte_perm(w0[i], w1[i], 0x5410), __byte_perm(w2[i], w3[i], 0x5410));
          mma_16816_bf16(oo[rd][i], pa0, 0u, pa2, 0u, __byte_perm(w0[i], w1[i], 0x7632), __byte_perm(w2[i], w3[i], 0x7632));
        }
      }
    }
  }
  // lane (g, t), head g: accumulator column 2t is dim 64 rd + 16 t + 2 i (+ 1 for the odd tile), column 2t + 1 eight dims further
  if (g < REP) {
#pragma unroll
    for (int rd = 0; rd < RD; ++rd) {
      float* dst = &s_red[warp][g][64 * rd + 16 * t];
      *reinterpret_cast<float4*>(dst) = make_float4(oe[rd][0][0], oo[rd][0][0], oe[rd][1][0], oo[rd][1][0]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(oe[rd][2][0], oo[rd][2][0], oe[rd][3][0], oo[rd][3][0]);
      *reinterpret_cast<float4*>(dst + 8) = make_float4(oe[rd][0][1], oo[rd][0][1], oe[rd][1][1], oo[rd][1][1]);
      *reinterpret_cast<float4*>(dst + 12) = make_float4(oe[rd][2][1], oo[rd][2][1], oe[rd][3][1], oo[rd][3][1]);
    }
  }
  __syncthreads();
  for (int i = tid; i < REP * D; i += DEC_THREADS) {
    const int h = i / D, d = i % D;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) acc += s_red[w][h][d];
    p.part_o[(((long long)b * p.Hq + hk * REP + h) * p.n_chunks + chunk) * D + d] = acc;
  }
  if (p.chunk_done == nullptr) return;
  // The CTA that arrives last for this (sequence, KV head) merges the chunk partials of its query heads: no separate merge launch.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* cnt = p.chunk_done + b * p.Hkv + hk;
    s_last = atomicAdd(cnt, 1) == int(gridDim.x) - 1;
    if (s_last) *cnt = 0;  // every CTA of this launch has arrived: ready for the next launch on the stream
  }
  __syncthreads();
  if (!s_last || warp >= REP) return;
  __threadfence();
  const long long wq = (long long)b * p.Hq + hk * REP + warp;
  const float* ml = p.part_ml + wq * p.n_chunks * 2;
  float m = -INFINITY;
  for (int c = 0; c < p.n_chunks; ++c) m = fmaxf(m, __ldcg(ml + 2 * c));
  float l = 0.f;
  for (int c = 0; c < p.n_chunks; ++c) {
    const float mc = __ldcg(ml + 2 * c);
    l += __ldcg(ml + 2 * c + 1) * ((mc == -INFINITY) ? 0.f : __expf(mc - m));
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (int c = 0; c < p.n_chunks; ++c) {
      const float mc = __ldcg(ml + 2 * c);
      const float f = (mc == -INFINITY) ? 0.f : __expf(mc - m);
      acc += __ldcg(p.part_o + (wq * p.n_chunks + c) * D + d) * f;
    }
    p.out[wq * D + d] = __float2bfloat16(acc * inv);
  }
}

// one warp per (sequence, query head): merge the chunk partials
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int BH, int n_chunks, int D) {
  pdl_prologue();
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
  pdl_prologue();
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


// ------------------------------------------------------------------------------------------------
// Mixture-of-experts routing of a decode-sized step (at most 1024 (token, k) slots): three launches around the two grouped
// GEMMs instead of gate GEMM + soft-max + top-k + slot plan + dispatch + pointer tables.
//
// serve_gate_route_kernel    one CTA per token: gate logits (one warp per expert row, fp32 accumulation), soft-max of
//                            logits / temperature over ALL experts, top-k, kept probabilities renormalised to sum to one
//                            (reference core/model.py:1169-1217).
// serve_plan_dispatch_kernel one warp per slot: its rank among the earlier slots of the same expert (token order, so the
//                            result equals the training-time plan), then the row copy into the expert's block; the block may
//                            live on a peer GPU (dst_table) or be e * dst_stride elements into a local buffer.
// serve_combine_kernel       one CTA per token: out = residual + sum_j w_j * row_j, rows read through the same addressing.
// ------------------------------------------------------------------------------------------------
constexpr int SRV_MAX_E = 64, SRV_MAX_K = 8;

__global__ void __launch_bounds__(256) serve_gate_route_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg,
                                                               int* __restrict__ topk_idx, float* __restrict__ topk_w, int hidden,
                                                               int experts, int k, float inv_temp) {
  pdl_prologue();
  __shared__ float s_logit[SRV_MAX_E];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)t * hidden);
  const int nvec = hidden >> 3;
  for (int e = warp; e < experts; e += nwarps) {
    const uint4* wr = reinterpret_cast<const uint4*>(wg + (long long)e * hidden);
    float acc = 0.f;
#pragma unroll 8
    for (int v = lane; v < nvec; v += 32) {  // unrolled: the loads of several iterations are in flight together
      const uint4 a = xr[v], b = wr[v];
      const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
      const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
      acc += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) s_logit[e] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float p[SRV_MAX_E];
    float m = -INFINITY;
    for (int e = 0; e < experts; ++e) m = fmaxf(m, s_logit[e]);
    float sum = 0.f;
    for (int e = 0; e < experts; ++e) {
      p[e] = __expf((s_logit[e] - m) * inv_temp);
      sum += p[e];
    }
    const float inv = 1.f / sum;
    unsigned long long taken = 0ull;
    float wk[SRV_MAX_K], wsum = 0.f;
    int ik[SRV_MAX_K];
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int bi = 0;
      for (int e = 0; e < experts; ++e)
        if (!((taken >> e) & 1ull) && p[e] * inv > best) {
          best = p[e] * inv;
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
}

__global__ void __launch_bounds__(256) serve_plan_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                                                  int* __restrict__ slot_pos, int* __restrict__ counts,
                                                                  int* __restrict__ totals, __nv_bfloat16* const* __restrict__ dst_table,
                                                                  __nv_bfloat16* dst0, long long dst_stride, int slots, int k, int hidden,
                                                                  int experts, int capacity) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int s = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // this warp's slot
  if (blockIdx.x == 0 && (counts || totals)) {
    // per-expert demand (block 0 only; any order gives the same sums)
    __shared__ int s_cnt[SRV_MAX_E];
    if (threadIdx.x < SRV_MAX_E) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < slots; i += blockDim.x) atomicAdd(&s_cnt[topk_idx[i]], 1);
    __syncthreads();
    if (threadIdx.x < experts) {
      const int tot = s_cnt[threadIdx.x];
      if (counts) counts[threadIdx.x] = tot < capacity ? tot : capacity;
      if (totals) totals[threadIdx.x] = tot;
    }
  }
  if (s >= slots) return;
  const int e = topk_idx[s];
  if (!ATS_DBG_CHECK(e >= 0 && e < experts, kDbgServeDispatch, e)) return;
  int rank = 0;
  for (int i = lane; i < s; i += 32) rank += topk_idx[i] == e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
  const int pos = rank < capacity ? rank : -1;
  if (lane == 0) slot_pos[s] = pos;
  if (pos < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(s / k) * hidden);
  __nv_bfloat16* base = dst_table ? dst_table[e] : dst0 + (long long)e * dst_stride;
  uint4* d = reinterpret_cast<uint4*>(base + (long long)pos * hidden);
#pragma unroll 8
  for (int v = lane; v < (hidden >> 3); v += 32) d[v] = src[v];
}

__device__ __forceinline__ float sumsq_bf16x8(const uint4& o) {
  const float2 f0 = unpack_bf16x2(o.x), f1 = unpack_bf16x2(o.y), f2 = unpack_bf16x2(o.z), f3 = unpack_bf16x2(o.w);
  return f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
}
// x * rstd * w for eight bf16 values (the arithmetic of rmsnorm_fwd_kernel)
__device__ __forceinline__ uint4 scale_bf16x8(const uint4& o, const uint4& w, float rstd) {
  const uint32_t xs[4] = {o.x, o.y, o.z, o.w}, ws[4] = {w.x, w.y, w.z, w.w};
  uint32_t r[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 x = unpack_bf16x2(xs[e]), g = unpack_bf16x2(ws[e]);
    r[e] = pack_bf16x2(x.x * rstd * g.x, x.y * rstd * g.y);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

__global__ void __launch_bounds__(256) serve_combine_kernel(__nv_bfloat16* const* __restrict__ src_table, const __nv_bfloat16* src0,
                                                            long long src_stride, const int* __restrict__ topk_idx,
                                                            const int* __restrict__ slot_pos, const float* __restrict__ topk_w,
                                                            const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ out, int k,
                                                            int hidden, const __nv_bfloat16* __restrict__ norm_w,
                                                            __nv_bfloat16* __restrict__ norm_out, float eps,
                                                            const int* __restrict__ ready_flags, const int* __restrict__ epoch_counter,
                                                            int experts_per_rank, unsigned long long budget_ns, int* status) {
  pdl_prologue();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int nvec = hidden >> 3;
  if (ready_flags) {
    // the rows are pulled from the experts' owners: wait (bounded) until each owner this token needs has raised its flag for this
    // call -- the flag is written by the launch that folded the owner's down projection, so no barrier launch sits in between
    if (threadIdx.x < k) {
      const int e = topk_idx[t * k + threadIdx.x];
      if (slot_pos[t * k + threadIdx.x] >= 0 && e >= 0) {
        const int want = *epoch_counter;  // this rank's own fold of this call has already counted
        const int* f = ready_flags + e / experts_per_rank;
        const uint64_t t0 = globaltimer_ns();
        int v;
        do {
          asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
          if (v >= want) break;
          if (globaltimer_ns() - t0 > budget_ns) {
            if (status) atomicCAS(status, 0, int(kTimeoutPeerFlag));
            break;
          }
        } while (true);
      }
    }
    __syncthreads();
  }
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (res) {
      const uint4 a = reinterpret_cast<const uint4*>(res + (long long)t * hidden)[v];
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
    }
    for (int j = 0; j < k; ++j) {
      const int pos = slot_pos[t * k + j];
      if (pos < 0) continue;
      const int e = topk_idx[t * k + j];
      if (!ATS_DBG_CHECK(e >= 0 && e < SRV_MAX_E, kDbgServeCombine, e)) continue;
      const float wt = topk_w[t * k + j];
      const __nv_bfloat16* base = src_table ? src_table[e] : src0 + (long long)e * src_stride;
      const uint4 a = reinterpret_cast<const uint4*>(base + (long long)pos * hidden)[v];
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] += wt * f0.x; acc[1] += wt * f0.y; acc[2] += wt * f1.x; acc[3] += wt * f1.y;
      acc[4] += wt * f2.x; acc[5] += wt * f2.y; acc[6] += wt * f3.x; acc[7] += wt * f3.y;
    }
    const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    reinterpret_cast<uint4*>(out + (long long)t * hidden)[v] = o;
    if (norm_out) ss += sumsq_bf16x8(o);
  }
  if (norm_out) {
    // RMSNorm of the row just written (the next block's input norm), on the bf16-rounded values as the separate kernel sees them
    const float rstd = rsqrtf(block_sum(ss, red) / float(hidden) + eps);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 o = reinterpret_cast<const uint4*>(out + (long long)t * hidden)[v];  // written by this thread above
      reinterpret_cast<uint4*>(norm_out + (long long)t * hidden)[v] = scale_bf16x8(o, reinterpret_cast<const uint4*>(norm_w)[v], rstd);
    }
  }
}

// ---- fold of the reduction slices of the packed projection + rotary embedding of the q / k heads, one CTA per token ---------------
// part: [splits, tokens, N] fp32 partial products; out: [tokens, N] bf16 with q and k heads rotated at position pos[t].
__global__ void __launch_bounds__(256) fold_rope_kernel(const float* __restrict__ part, int splits, long long slice_stride,
                                                        __nv_bfloat16* __restrict__ out, const float* __restrict__ cos_t,
                                                        const float* __restrict__ sin_t, const int* __restrict__ pos, int N, int n_q,
                                                        int n_kv, int d) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int half = d >> 1, vph = half >> 3;
  const int rope_items = (n_q + n_kv) * vph;  // an item: 8 elements of a head's first half and the matching 8 of its second half
  const int v_items = n_kv * (d >> 3);
  const float* row = part + (long long)t * N;
  __nv_bfloat16* orow = out + (long long)t * N;
  const int p = pos[t];
  auto fold8 = [&](int col, float (&a)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
#pragma unroll 4
    for (int sl = 0; sl < splits; ++sl) {
      const float4* src = reinterpret_cast<const float4*>(row + sl * slice_stride + col);
      const float4 x = src[0], y = src[1];
      a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w; a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
    }
  };
  for (int i = threadIdx.x; i < rope_items + v_items; i += blockDim.x) {
    float a[8];
    if (i >= rope_items) {
      const int col = (n_q + n_kv) * d + (i - rope_items) * 8;
      fold8(col, a);
      *reinterpret_cast<uint4*>(orow + col) = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
      continue;
    }
    const int head = i / vph, v = i - head * vph;
    const int col = head * d + v * 8;
    float b[8];
    fold8(col, a);
    fold8(col + half, b);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)p * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)p * half + v * 8);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    const float c[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float sn[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // rounded to bf16 first: the same values the separate fold and rotation kernels exchange through memory
      const float2 x1 = unpack_bf16x2(pack_bf16x2(a[2 * e], a[2 * e + 1])), x2 = unpack_bf16x2(pack_bf16x2(b[2 * e], b[2 * e + 1]));
      o1[e] = pack_bf16x2(x1.x * c[2 * e] - x2.x * sn[2 * e], x1.y * c[2 * e + 1] - x2.y * sn[2 * e + 1]);
      o2[e] = pack_bf16x2(x1.x * sn[2 * e] + x2.x * c[2 * e], x1.y * sn[2 * e + 1] + x2.y * c[2 * e + 1]);
    }
    *reinterpret_cast<uint4*>(orow + col) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(orow + col + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

// ---- fold of the reduction slices of the output projection + residual + RMSNorm, one CTA per token ---------------------------------
// x_out = sum of the slices + residual (bf16); h_out = RMSNorm(x_out) * w.
__global__ void __launch_bounds__(256) fold_add_norm_kernel(const float* __restrict__ part, int splits, long long slice_stride,
                                                            const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ w,
                                                            __nv_bfloat16* __restrict__ x_out, __nv_bfloat16* __restrict__ h_out,
                                                            int hidden, float eps) {
  pdl_prologue();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int nvec = hidden >> 3;
  const float* row = part + (long long)t * hidden;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (res) {
      const uint4 r = reinterpret_cast<const uint4*>(res + (long long)t * hidden)[v];
      const float2 f0 = unpack_bf16x2(r.x), f1 = unpack_bf16x2(r.y), f2 = unpack_bf16x2(r.z), f3 = unpack_bf16x2(r.w);
      a[0] = f0.x; a[1] = f0.y; a[2] = f1.x; a[3] = f1.y; a[4] = f2.x; a[5] = f2.y; a[6] = f3.x; a[7] = f3.y;
    }
#pragma unroll 4
    for (int sl = 0; sl < splits; ++sl) {
      const float4* src = reinterpret_cast<const float4*>(row + sl * slice_stride + v * 8);
      const float4 x = src[0], y = src[1];
      a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w; a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
    }
    const uint4 o = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
    reinterpret_cast<uint4*>(x_out + (long long)t * hidden)[v] = o;
    ss += sumsq_bf16x8(o);
  }
  const float rstd = rsqrtf(block_sum(ss, red) / float(hidden) + eps);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 o = reinterpret_cast<const uint4*>(x_out + (long long)t * hidden)[v];  // written by this thread above
    reinterpret_cast<uint4*>(h_out + (long long)t * hidden)[v] = scale_bf16x8(o, reinterpret_cast<const uint4*>(w)[v], rstd);
  }
}

}  // namespace ats

using namespace ats;

// 1 (default): warp-level tensor-core kernel; 0: the fp32 CUDA-core kernel (kept for comparison, ATS_DECODE_ATTN_MMA=0)
static int g_decode_mma = -1;
static int g_decode_occ = 2;  // ATS_DECODE_ATTN_OCC=3 selects the 80-register build of the tensor-core kernel
template <int D, int REP>
static int launch_decode(const DecodeArgs& p, cudaStream_t s) {
  if (g_decode_mma < 0) {
    const char* e = getenv("ATS_DECODE_ATTN_MMA");
    g_decode_mma = (e && e[0] == '0') ? 0 : 1;
    const char* o = getenv("ATS_DECODE_ATTN_OCC");
    if (o && o[0] == '3') g_decode_occ = 3;
  }
  dim3 grid(p.n_chunks, p.Hkv, p.B);
  if (g_decode_mma && g_decode_occ == 3) decode_attn_mma_kernel<D, REP, 3><<<grid, DEC_THREADS, 0, s>>>(p);
  else if (g_decode_mma) {
    cudaError_t ce = launch_pdl(decode_attn_mma_kernel<D, REP, 2>, grid, dim3(DEC_THREADS), 0, s, p);
    return int(ce != cudaSuccess ? ce : cudaGetLastError());
  }
  else decode_attn_kernel<D, REP><<<grid, DEC_THREADS, 0, s>>>(p);
  return int(cudaGetLastError());
}

// Scratch sizes for `ats_decode_attn`: floats needed for part_o and part_ml with a cache of `max_len` positions.
ATS_API int ats_decode_attn_chunks(int max_len) { return (max_len + DEC_CHUNK - 1) / DEC_CHUNK; }

// qkv: packed projection of the new token [B, ld_qkv]; caches [B, max_len, Hkv, D] (batch stride cache_b_stride elements).
// lengths: per-sequence cached lengths (device int32) or nullptr for the common `length`.  out: [B, Hq * D] bf16.
ATS_API int ats_decode_attn(const void* qkv, long long ld_qkv, int q_col0, int k_col0, int v_col0, void* k_cache, void* v_cache,
                            long long cache_b_stride, const int* lengths, int length, int max_tokens, int B, int Hq, int Hkv, int D,
                            int max_len, float* part_o, float* part_ml, int* chunk_done, void* out, void* stream) {
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
  if (g_decode_mma < 0) {
    const char* ev = getenv("ATS_DECODE_ATTN_MMA");
    g_decode_mma = (ev && ev[0] == '0') ? 0 : 1;
    const char* o = getenv("ATS_DECODE_ATTN_OCC");
    if (o && o[0] == '3') g_decode_occ = 3;
  }
  const bool merge_inside = chunk_done != nullptr && g_decode_mma == 1 && g_decode_occ == 2;
  p.chunk_done = merge_inside ? chunk_done : nullptr;
  int e = 1004;
#define ATS_DEC(DD, RR) if (D == DD && rep == RR) e = launch_decode<DD, RR>(p, s);
  ATS_DEC(64, 1) ATS_DEC(64, 2) ATS_DEC(64, 4) ATS_DEC(64, 8) ATS_DEC(128, 1) ATS_DEC(128, 2) ATS_DEC(128, 4) ATS_DEC(128, 8)
#undef ATS_DEC
  if (e) return e;
  if (merge_inside) return int(cudaGetLastError());
  const int BH = B * Hq;
  launch_pdl(decode_merge_kernel, dim3((BH * 32 + 255) / 256), dim3(256), 0, s, (const float*)part_o, (const float*)part_ml, p.out, BH, p.n_chunks, D);
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
  launch_pdl(sample_kernel, dim3(B), dim3(SMP_THREADS), 0, static_cast<cudaStream_t>(stream), p);
  return int(cudaGetLastError());
}

// ---- decode-sized mixture-of-experts routing (see the kernels above) ----------------------------------------------
ATS_API int ats_serve_gate_route(const void* x, const void* wg, int* topk_idx, float* topk_w, int tokens, int hidden, int experts, int k,
                                 float temperature, void* stream) {
  if (tokens <= 0 || experts < 1 || experts > SRV_MAX_E || k < 1 || k > SRV_MAX_K || k > experts || (hidden & 7)) return 1003;
  launch_pdl(serve_gate_route_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(wg), topk_idx, topk_w, hidden, experts, k, 1.f / temperature);
  return int(cudaGetLastError());
}

// dst_table: device array of `experts` base pointers (blocks on peer GPUs), or null with dst0 + e * dst_stride (elements).
ATS_API int ats_serve_plan_dispatch(const void* x, const int* topk_idx, int* slot_pos, int* counts, int* totals, void* const* dst_table,
                                    void* dst0, long long dst_stride, int tokens, int k, int hidden, int experts, int capacity,
                                    void* stream) {
  const int slots = tokens * k;
  if (slots <= 0 || slots > 1024 || experts < 1 || experts > SRV_MAX_E || (hidden & 7) || (!dst_table && !dst0)) return 1003;
  launch_pdl(serve_plan_dispatch_kernel, dim3((slots * 32 + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(x), topk_idx, slot_pos, counts, totals, reinterpret_cast<__nv_bfloat16* const*>(dst_table),
             static_cast<__nv_bfloat16*>(dst0), dst_stride, slots, k, hidden, experts, capacity);
  return int(cudaGetLastError());
}

// norm_w / norm_out (both or neither): also write RMSNorm(out) * norm_w, the input of the next block.
// ready_flags / epoch_counter / experts_per_rank (all or none): the kernel itself waits for the owners of the rows it pulls (see
// ats_splitk_reduce_signal) instead of relying on a barrier launch before it.
ATS_API unsigned long long ats_get_wait_budget_ns();  // comm.cu
ATS_API int ats_serve_combine(void* const* src_table, const void* src0, long long src_stride, const int* topk_idx, const int* slot_pos,
                              const float* topk_w, const void* residual, void* out, int tokens, int k, int hidden, const void* norm_w,
                              void* norm_out, float eps, const int* ready_flags, const int* epoch_counter, int experts_per_rank, int* status,
                              void* stream) {
  if (tokens <= 0 || (hidden & 7) || (!src_table && !src0) || ((norm_w == nullptr) != (norm_out == nullptr))) return 1003;
  if (ready_flags && (!epoch_counter || experts_per_rank < 1 || k > 32)) return 1003;
  launch_pdl(serve_combine_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream),
             reinterpret_cast<__nv_bfloat16* const*>(src_table), static_cast<const __nv_bfloat16*>(src0), src_stride, topk_idx, slot_pos, topk_w,
             static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), k, hidden, static_cast<const __nv_bfloat16*>(norm_w),
             static_cast<__nv_bfloat16*>(norm_out), eps, ready_flags, epoch_counter, experts_per_rank,
             (unsigned long long)ats_get_wait_budget_ns(), status);
  return int(cudaGetLastError());
}

ATS_API int ats_fold_rope(const float* part, int splits, void* out, const float* cos_t, const float* sin_t, const int* pos, int tokens, int N,
                          int n_q, int n_kv, int d, void* stream) {
  if (tokens <= 0 || splits < 1 || (d & 15) || N != (n_q + 2 * n_kv) * d || !pos) return 1003;
  launch_pdl(fold_rope_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream), part, splits, (long long)tokens * N,
             static_cast<__nv_bfloat16*>(out), cos_t, sin_t, pos, N, n_q, n_kv, d);
  return int(cudaGetLastError());
}

ATS_API int ats_fold_add_norm(const float* part, int splits, const void* residual, const void* norm_w, void* x_out, void* h_out, int tokens,
                              int hidden, float eps, void* stream) {
  if (tokens <= 0 || splits < 1 || (hidden & 7) || !norm_w || !x_out || !h_out) return 1003;
  launch_pdl(fold_add_norm_kernel, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream), part, splits, (long long)tokens * hidden,
             static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(norm_w), static_cast<__nv_bfloat16*>(x_out),
             static_cast<__nv_bfloat16*>(h_out), hidden, eps);
  return int(cudaGetLastError());
}
