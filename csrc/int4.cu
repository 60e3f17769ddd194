// Weight-only 4-bit linear layers (W4A16, group-wise asymmetric quantisation as produced by GPTQ or round-to-nearest).
//
// A decode step of a few tokens reads every weight once and does almost no arithmetic with it, so the step time is the weight
// bytes divided by the HBM rate: 4-bit weights cut it to a quarter of bf16.  tcgen05 wants at least 64 token rows and operands
// in shared memory in its own layout; for one to sixteen tokens the warp-level MMA (m16n8k16, bf16 in, fp32 out) is the right tool:
// the WEIGHTS are the 16-row A operand, the tokens the 8 columns of B, so no tensor row is wasted, and the packed format is laid
// out such that the 16 bytes a lane loads ARE its A fragments of four consecutive k-steps:
//
//   tile T = 16 output features, super-step S = 64 reduction indices, lane (g, t) = (lane / 4, lane % 4), word j = 0..3:
//   nibble i of word [S][T][lane][j] holds feature 16 T + g + 8 (i & 1), reduction index 64 S + 16 t + 4 j + 2 ((i >> 1) & 1) + (i >> 2)
//
// The super-step is the OUTER index of the stored array: CTAs own tiles, start together and advance at the same pace, so at any
// time the CTAs in flight read one contiguous window of the array per warp slot, as a copy kernel does (measured against the
// tile-outermost order: no difference at these sizes; kept because it is the order that stays sequential as K grows).
//
// (the sum over the reduction index does not care about the order of its terms, so inside a k-step the MMA's logical indices
// 2t, 2t+1, 2t+8, 2t+9 are mapped to the four consecutive actual indices 16 t + 4 j .. + 3: the B fragment of a lane is then 8
// consecutive bytes of a token's row, and the 32 bytes it loads per super-step serve four k-steps).  `(w >> 4 r) & 0x000f000f |
// 0x43004300` turns two nibbles into the bf16 pair (128 + q_lo, 128 + q_hi) exactly.  The streaming kernel feeds these raw
// pairs to the MMA and takes zero point and scale out of the sum: per 64-channel step (inside one group) it accumulates
// sum((128 + q) x) and, with an all-ones A operand, sum(x), and adds scale * (sum((128 + q) x) - (128 + zero) * sum(x)) to the
// running result in fp32, which is the exact product with (q - zero) * scale.  The dequantise kernel subtracts the bf16 pair
// (128 + zero) (exact) and multiplies by the bf16 scale (one rounding): the bf16 weight a prompt-sized GEMM then reads.
// Per (group, feature) one 32-bit word: low half the bf16 scale, high half bf16(128 + zero).
//
// ats_gemv_int4: up to 16 tokens (one or two token tiles of eight), optional residual add, optional SwiGLU over the two halves of the features.
// ats_dequant_int4: the bf16 matrix for prompt-sized products, which then run on the tcgen05 GEMM.
//
// Counterparts in the reference: the GPTQ hook of training/trainer.py:681-710 (AutoGPTQ, 4 bits, group 128) and the Triton GPTQ
// matmul of its vendored inference engine (colossalai/kernel/triton/gptq_triton.py).
#include "common.cuh"

namespace ats {

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (128 + q) pairs -> (q - zero) * scale, in bf16 pairs.  The integer ALU issues a warp instruction every other cycle and is the
// pipe this kernel fills first (measured: 60 % busy with the plain C++ form, 15 of its instructions per packed word), so the
// extraction is pinned to one logic operation per pair, (w' & mask) | magic with both constants in registers, and the three
// shifts of a word are done as multiply-high by a power of two on the FMA pipe, which has room (no measurable change by
// itself: the kernel was waiting for memory then, see the copy ring below).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t shr_mulhi(uint32_t w, uint32_t two_pow_32_minus_shift) {
  uint32_t d;
  asm("mul.hi.u32 %0, %1, %2;" : "=r"(d) : "r"(w), "r"(two_pow_32_minus_shift));
  return d;
}
__device__ __forceinline__ uint32_t dq_scale(uint32_t v, uint32_t zero2, uint32_t scale2) {
  const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&zero2));
  const __nv_bfloat162 r = __hmul2(d, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
  return *reinterpret_cast<const uint32_t*>(&r);
}
struct Int4Consts {
  uint32_t mask, magic, m4, m8, m12, ones;  // 0x000f000f, 0x43004300 (bf16 128.0 twice), 2^28, 2^24, 2^20, bf16 1.0 twice
};
// one packed word -> the four A-fragment registers of a k-step (rows g / g + 8 alternate)
__device__ __forceinline__ void dq_word(uint32_t w, const Int4Consts& k, uint32_t zA, uint32_t sA, uint32_t zB, uint32_t sB, uint32_t (&a)[4]) {
  a[0] = dq_scale(and_or(w, k.mask, k.magic), zA, sA);
  a[1] = dq_scale(and_or(shr_mulhi(w, k.m4), k.mask, k.magic), zB, sB);
  a[2] = dq_scale(and_or(shr_mulhi(w, k.m8), k.mask, k.magic), zA, sA);
  a[3] = dq_scale(and_or(shr_mulhi(w, k.m12), k.mask, k.magic), zB, sB);
}

constexpr int GEMV_WARPS = 8;

// Asynchronous copies global -> shared (each lane copies into slots only it reads back, so no barrier is involved: a lane waits
// for its own copy groups).  Loads into registers did not pipeline here: with five loads per step and stage the kernel waited
// a full round trip to memory in every step whatever the prefetch depth (1.9 TB/s, warps 68 % of the time on the long
// scoreboard); copy groups are counted, not score-boarded.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(smem))), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16_or_zero(void* smem, const void* gmem, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(uint32_t(__cvta_generic_to_shared(smem))), "l"(gmem), "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(uint32_t(__cvta_generic_to_shared(smem))), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// bytes one warp holds per stage: packed words and scale words of R tiles, 16 activations per lane and token tile
__host__ __device__ constexpr int int4_stage_bytes(int R, int NT) { return 32 * (R * 16 + R * 8 + NT * 32); }
__host__ __device__ constexpr int int4_ring_bytes(int R, int NT, int DEPTH) { return GEMV_WARPS * DEPTH * int4_stage_bytes(R, NT); }

// R tiles per CTA: one, or with SWIGLU the gate tile and the up tile of the same features.  The warps split the super-steps;
// every warp keeps the copies of DEPTH of its super-steps in flight (a ring in shared memory), so that a CTA's few microseconds
// are spent streaming and not waiting for one round trip to memory per step.  One tile per CTA and MINB resident CTAs per SM keep
// the grid fine-grained: with two tiles and 72 registers the 28,672-feature projection ran as 2.02 waves of CTAs, i.e. three.
// NT: token tiles of eight rows (the code fragments of a step feed NT MMAs).
template <int R, bool SWIGLU, int NT, int DEPTH, int MINB>
__global__ void __launch_bounds__(GEMV_WARPS * 32, MINB)
gemv_int4_kernel(const uint4* __restrict__ wq, const uint32_t* __restrict__ meta, const __nv_bfloat16* __restrict__ x, long long ldx,
                 const __nv_bfloat16* __restrict__ add, long long ld_add, __nv_bfloat16* __restrict__ out, long long ld_out,
                 int M, int N, int K, int group_shift) {
  pdl_prologue();
  __shared__ float s_red[GEMV_WARPS][R][8 * NT][16];  // [warp][tile][token][feature of the tile]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n_super = K >> 6, n_tiles = N >> 4;
  // constants the extraction wants in registers; built from a kernel argument so that they are not folded back into immediates
  const uint32_t one = uint32_t(group_shift > 0);
  const Int4Consts kc = {0x000f000fu * one, 0x43004300u * one, one << 28, one << 24, one << 20, 0x3f803f80u * one};
  int tile[R];
#pragma unroll
  for (int r = 0; r < R; ++r) tile[r] = SWIGLU ? int(blockIdx.x) + r * (N >> 5) : int(blockIdx.x) * R + r;
  float c[R][NT][4];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int n = 0; n < NT; ++n) c[r][n][0] = c[r][n][1] = c[r][n][2] = c[r][n][3] = 0.f;
  bool tok[NT];             // this lane supplies token g of token tile n
  const uint4* xrow[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    tok[n] = 8 * n + g < M;
    xrow[n] = reinterpret_cast<const uint4*>(x + (long long)(tok[n] ? 8 * n + g : 0) * ldx + 16 * t);
  }

  extern __shared__ __align__(16) unsigned char ring[];
  constexpr int STAGE = int4_stage_bytes(R, NT);
  unsigned char* my_ring = ring + warp * DEPTH * STAGE;
  // slots of this lane inside a stage: [R][32] packed words (16 B), [R][32] scale words (2 x 4 B), [2 NT][32] activations (16 B)
  auto w_slot = [&](int d, int r) { return my_ring + d * STAGE + r * 512 + lane * 16; };
  auto m_slot = [&](int d, int r) { return my_ring + d * STAGE + R * 512 + r * 256 + lane * 8; };
  auto x_slot = [&](int d, int i) { return my_ring + d * STAGE + R * 768 + i * 512 + lane * 16; };
  auto issue = [&](int d, int S) {
    const long long grp = S >> (group_shift - 6);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      cp_async16(w_slot(d, r), wq + ((long long)S * n_tiles + tile[r]) * 32 + lane);
      const uint32_t* mrow = meta + grp * N + tile[r] * 16 + g;
      cp_async4(m_slot(d, r), mrow);
      cp_async4(m_slot(d, r) + 4, mrow + 8);
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {  // lanes without a token get zeros
      cp_async16_or_zero(x_slot(d, 2 * n), xrow[n] + S * 8, tok[n]);
      cp_async16_or_zero(x_slot(d, 2 * n + 1), xrow[n] + S * 8 + 1, tok[n]);
    }
  };
  auto compute = [&](int d) {
    uint32_t xw[NT][8];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const uint4 x0 = *reinterpret_cast<const uint4*>(x_slot(d, 2 * n)), x1 = *reinterpret_cast<const uint4*>(x_slot(d, 2 * n + 1));
      xw[n][0] = x0.x; xw[n][1] = x0.y; xw[n][2] = x0.z; xw[n][3] = x0.w;
      xw[n][4] = x1.x; xw[n][5] = x1.y; xw[n][6] = x1.z; xw[n][7] = x1.w;
    }
    // sum of the step's activations per token: a product with an all-ones A operand (every row of the result holds it)
    float cx[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      cx[n][0] = cx[n][1] = cx[n][2] = cx[n][3] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) mma_16816(cx[n], kc.ones, kc.ones, kc.ones, kc.ones, xw[n][2 * j], xw[n][2 * j + 1]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      // bf16 -> fp32 is a shift: scale, and 128 + zero, of features g (A) and g + 8 (B)
      const uint2 mAB = *reinterpret_cast<const uint2*>(m_slot(d, r));
      const float sA = __uint_as_float(mAB.x << 16), zA = __uint_as_float(mAB.x & 0xffff0000u);
      const float sB = __uint_as_float(mAB.y << 16), zB = __uint_as_float(mAB.y & 0xffff0000u);
      const uint4 wv = *reinterpret_cast<const uint4*>(w_slot(d, r));
      const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
      float cq[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) cq[n][0] = cq[n][1] = cq[n][2] = cq[n][3] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a0 = and_or(w4[j], kc.mask, kc.magic), a1 = and_or(shr_mulhi(w4[j], kc.m4), kc.mask, kc.magic);
        const uint32_t a2 = and_or(shr_mulhi(w4[j], kc.m8), kc.mask, kc.magic), a3 = and_or(shr_mulhi(w4[j], kc.m12), kc.mask, kc.magic);
#pragma unroll
        for (int n = 0; n < NT; ++n) mma_16816(cq[n], a0, a1, a2, a3, xw[n][2 * j], xw[n][2 * j + 1]);
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        c[r][n][0] = fmaf(sA, fmaf(-zA, cx[n][0], cq[n][0]), c[r][n][0]);
        c[r][n][1] = fmaf(sA, fmaf(-zA, cx[n][1], cq[n][1]), c[r][n][1]);
        c[r][n][2] = fmaf(sB, fmaf(-zB, cx[n][2], cq[n][2]), c[r][n][2]);
        c[r][n][3] = fmaf(sB, fmaf(-zB, cx[n][3], cq[n][3]), c[r][n][3]);
      }
    }
  };

  // group i of this lane's copies holds super-step warp + 8 i; one group is committed per step, empty past the end
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {
    if (warp + d * GEMV_WARPS < n_super) issue(d, warp + d * GEMV_WARPS);
    cp_async_commit();
  }
  for (int S0 = warp; S0 < n_super; S0 += GEMV_WARPS * DEPTH) {
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      const int S = S0 + d * GEMV_WARPS;
      if (S < n_super) {  // the same for every lane of the warp
        cp_async_wait<DEPTH - 1>();  // all but the DEPTH - 1 youngest groups have landed: this step's is among them
        compute(d);
        const int Sn = S + GEMV_WARPS * DEPTH;
        if (Sn < n_super) issue(d, Sn);  // the slots just read are refilled (their values are in registers by now)
        cp_async_commit();
      }
    }
  }
  cp_async_wait<0>();
  // accumulator of token tile n: c[0], c[1] = feature g, tokens 8 n + 2t and + 1; c[2], c[3] = feature g + 8
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      s_red[warp][r][8 * n + 2 * t][g] = c[r][n][0];
      s_red[warp][r][8 * n + 2 * t + 1][g] = c[r][n][1];
      s_red[warp][r][8 * n + 2 * t][g + 8] = c[r][n][2];
      s_red[warp][r][8 * n + 2 * t + 1][g + 8] = c[r][n][3];
    }
  __syncthreads();
  constexpr int OUT_TILES = SWIGLU ? 1 : R;
  for (int e = tid; e < OUT_TILES * NT * 128; e += GEMV_WARPS * 32) {
    const int r = e / (NT * 128), m = (e >> 4) & (8 * NT - 1), f = e & 15;
    if (m >= M) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) v += s_red[w][r][m][f];
    const int col = (SWIGLU ? int(blockIdx.x) : int(blockIdx.x) * R + r) * 16 + f;
    if (SWIGLU) {
      float u = 0.f;
#pragma unroll
      for (int w = 0; w < GEMV_WARPS; ++w) u += s_red[w][R - 1][m][f];
      // the gate and up products are rounded to bf16 first, as the unfused form stores them
      const float gf = __bfloat162float(__float2bfloat16(v)), uf = __bfloat162float(__float2bfloat16(u));
      v = gf / (1.f + __expf(-gf)) * uf;
    }
    if (add) v += __bfloat162float(add[(long long)m * ld_add + col]);
    out[(long long)m * ld_out + col] = __float2bfloat16(v);
  }
}

// one thread per (tile, super-step, lane): 16 + 16 consecutive values of features g and g + 8
__global__ void __launch_bounds__(256)
dequant_int4_kernel(const uint4* __restrict__ wq, const uint32_t* __restrict__ meta, __nv_bfloat16* __restrict__ out, long long ld,
                    int N, int K, int group_shift, long long n_items) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_items) return;
  const int lane = int(i & 31), g = lane >> 2, t = lane & 3;
  // consecutive warps walk the steps of one tile: the bf16 rows (four fifths of the traffic) are written as contiguous runs
  const int n_super = K >> 6, n_tiles = N >> 4;
  const int S = int((i >> 5) % n_super), T = int((i >> 5) / n_super);
  const uint4 w = __ldcs(wq + ((long long)S * n_tiles + T) * 32 + lane);
  const long long grp = S >> (group_shift - 6);
  const uint32_t* mrow = meta + grp * N + T * 16 + g;
  const uint32_t mA = __ldg(mrow), mB = __ldg(mrow + 8);
  const uint32_t sA = __byte_perm(mA, mA, 0x1010), zA = __byte_perm(mA, mA, 0x3232);
  const uint32_t sB = __byte_perm(mB, mB, 0x1010), zB = __byte_perm(mB, mB, 0x3232);
  const uint32_t w4[4] = {w.x, w.y, w.z, w.w};
  const Int4Consts kc = {0x000f000fu, 0x43004300u, 1u << 28, 1u << 24, 1u << 20, 0x3f803f80u};
  uint32_t ra[8], rb[8];  // features g and g + 8: word 2 j = indices 4 j, 4 j + 1; word 2 j + 1 = indices 4 j + 2, 4 j + 3
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t a[4];
    dq_word(w4[j], kc, zA, sA, zB, sB, a);
    ra[2 * j] = a[0];
    rb[2 * j] = a[1];
    ra[2 * j + 1] = a[2];
    rb[2 * j + 1] = a[3];
  }
  __nv_bfloat16* pa = out + (long long)(T * 16 + g) * ld + (S << 6) + 16 * t;
  __nv_bfloat16* pb = pa + 8 * ld;
  reinterpret_cast<uint4*>(pa)[0] = make_uint4(ra[0], ra[1], ra[2], ra[3]);
  reinterpret_cast<uint4*>(pa)[1] = make_uint4(ra[4], ra[5], ra[6], ra[7]);
  reinterpret_cast<uint4*>(pb)[0] = make_uint4(rb[0], rb[1], rb[2], rb[3]);
  reinterpret_cast<uint4*>(pb)[1] = make_uint4(rb[4], rb[5], rb[6], rb[7]);
}

}  // namespace ats

// groups are powers of two of at least 64 input channels (a super-step never straddles two groups)
static bool int4_shape_ok(int N, int K, int group) {
  return N > 0 && K > 0 && group >= 64 && (group & (group - 1)) == 0 && (N % 16) == 0 && (K % 64) == 0 && (K % group) == 0;
}
static int int4_group_shift(int group) {
  int s = 0;
  while ((1 << s) < group) ++s;
  return s;
}

// out[M, N or N / 2] = x[M, K] @ W^T (+ add), M <= 16.  swiglu: W = [gate; up], out = silu(gate) * up (N % 32 == 0).
ATS_API int ats_gemv_int4(const void* wq, const void* meta, const void* x, long long ldx, const void* add, long long ld_add, void* out,
                          long long ld_out, int M, int N, int K, int group, int swiglu, void* stream) {
  if (!int4_shape_ok(N, K, group) || M < 1 || M > 16 || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return 1003;
  if (swiglu && (N % 32)) return 1003;
  auto s = static_cast<cudaStream_t>(stream);
  const auto* w4 = static_cast<const uint4*>(wq);
  const auto* mt = static_cast<const uint32_t*>(meta);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* ap = static_cast<const __nv_bfloat16*>(add);
  auto* op = static_cast<__nv_bfloat16*>(out);
  const int tiles = N / 16;
  const int gs = int4_group_shift(group);
  cudaError_t err;
  const dim3 block(ats::GEMV_WARPS * 32);
#define ATS_GEMV4(R_, SW_, NT_, D_, B_, GRID_)                                                                                        \
  [&]() -> cudaError_t {                                                                                                             \
    constexpr int kRing = ats::int4_ring_bytes(R_, NT_, D_);                                                                         \
    static bool attr_set = false;                                                                                                    \
    if (!attr_set) {                                                                                                                 \
      cudaError_t ce = cudaFuncSetAttribute(ats::gemv_int4_kernel<R_, SW_, NT_, D_, B_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                            kRing);                                                                                  \
      if (ce != cudaSuccess) return ce;                                                                                              \
      attr_set = true;                                                                                                               \
    }                                                                                                                                \
    return ats::launch_pdl(ats::gemv_int4_kernel<R_, SW_, NT_, D_, B_>, dim3(GRID_), block, kRing, s, w4, mt, xp, ldx, ap, ld_add,  \
                           op, ld_out, M, N, K, gs);                                                                                 \
  }()
  const bool two = M > 8;
  if (swiglu)
    err = two ? ATS_GEMV4(2, true, 2, 3, 2, tiles / 2) : ATS_GEMV4(2, true, 1, 4, 2, tiles / 2);
  else
    err = two ? ATS_GEMV4(1, false, 2, 4, 2, tiles) : ATS_GEMV4(1, false, 1, 4, 3, tiles);
#undef ATS_GEMV4
  return int(err);
}

ATS_API int ats_dequant_int4(const void* wq, const void* meta, void* out, long long ld, int N, int K, int group, void* stream) {
  if (!int4_shape_ok(N, K, group) || (ld & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return 1003;
  const long long n_items = (long long)(N / 16) * (K / 64) * 32;
  ats::dequant_int4_kernel<<<unsigned((n_items + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(wq), static_cast<const uint32_t*>(meta), static_cast<__nv_bfloat16*>(out), ld, N, K, int4_group_shift(group), n_items);
  return int(cudaGetLastError());
}
