// Causal grouped-query flash attention forward for sm_100a, two query tiles per CTA.
//
// One CTA owns 256 consecutive queries of one head as two 128-row tiles (A, B).  Both tiles score against the same
// K / V stream (every K / V tile is fetched once for 256 queries) and ping-pong on the tensor cores: while the four
// soft-max warps of tile A work on S_A(j), the tensor cores compute S_B(j) and the P V product of the tile that finished
// before.  The output accumulators O_A / O_B stay in tensor memory for the whole row sweep; a soft-max thread rescales
// its row of O only when the running maximum has grown by more than 2^8 (a stale maximum cancels in O / l, so the result
// is exact), which removes the per-block round trip of the accumulator.
//
//   warps 0..3   soft-max of tile A, one query row per thread (S row read from TMEM in one go)
//   warps 4..7   soft-max of tile B
//   warp 8       TMA producer: Q_A, Q_B once, then K_j / V_j through a multi-stage ring
//   warp 9       TMEM owner and MMA issuer, order per block: P V (A), S_A(j+1), P V (B), S_B(j+1)
// A soft-max thread holds a whole 128-element score row in registers (168 registers per thread, no spills); the rare
// accumulator rescale works in 16-column pieces to stay inside that budget.
//
// PT = true keeps P in tensor memory (bf16 pairs written over the first 64 columns of the S tile, read by the MMA as
// its A operand); PT = false stages P through shared memory in the 128-byte-swizzled K-major layout.
// Every wait is bounded (status word + clean unwind); no load uses cluster multicast.
// Replaces flash_attn_func of the reference model (reference core/model.py:763-768) without expanding K / V per query head.
#include "common.cuh"

namespace ats {

// max of three floats in one instruction (sm_100: max.f32 with three sources)
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}


constexpr int A2_THREADS = 320;  // soft-max A (warps 0-3), soft-max B (4-7), TMA (8), MMA (9)

struct Attn2Args {
  int B, L, Hq, Hkv;
  int q_col0, k_col0, v_col0;
  __nv_bfloat16* out;  // [B, L, Hq, D]
  float* lse;          // [B, Hq, L]
  float scale_log2;
  int* status;
  long long* prof;  // optional [16]: cycle totals per phase of CTA (0,0,0) (diagnostics; null in normal use)
};

template <int D, bool PT>
struct Attn2Smem {
  static constexpr int TB = 128 * D * 2;
  static constexpr int KST = (D == 64) ? 3 : 2;
  static constexpr int VST = (D == 64) ? 3 : (PT ? 2 : 1);
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = 2 * TB;
  static constexpr int V_OFF = K_OFF + KST * TB;
  static constexpr int P_OFF = V_OFF + VST * TB;
  static constexpr int BAR_OFF = P_OFF + (PT ? 0 : 65536);
  static constexpr int TOTAL = BAR_OFF + 512 + 1024;
};

// exp2 on the FMA pipe: round-to-nearest range reduction with the 1.5 * 2^23 trick, degree-3 polynomial on [-0.5, 0.5]
// (relative error 6e-4, below the bf16 rounding of P), exponent added with one integer shift-add.  The 16 MUFU lanes of an SM
// are the bottleneck of the forward pass at D = 64, so part of the exponentials is computed this way.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, magic);
  const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 p = __ffma2_rn(f, make_float2(0.0555041f, 0.0555041f), make_float2(0.2402265f, 0.2402265f));
  p = __ffma2_rn(p, f, make_float2(0.6931472f, 0.6931472f));
  p = __ffma2_rn(p, f, make_float2(1.f, 1.f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                     __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
}

// POLY: 0 = every exponential on the MUFU; n > 0 = one pair of every n goes through exp2_poly2.
template <int D, bool PT, bool PROF, int POLY>
__global__ void __launch_bounds__(A2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const Attn2Args p) {
  using SM = Attn2Smem<D, PT>;
  constexpr int TB = SM::TB, KST = SM::KST, VST = SM::VST;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + SM::Q_OFF;
  uint8_t* sK = smem + SM::K_OFF;
  uint8_t* sV = smem + SM::V_OFF;
  uint8_t* sP = smem + SM::P_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars;         // 1
  uint64_t* k_full = bars + 1;     // [3]
  uint64_t* k_empty = bars + 4;    // [3]
  uint64_t* v_full = bars + 7;     // [3]
  uint64_t* v_empty = bars + 10;   // [3]
  uint64_t* s_full = bars + 13;    // [2] per tile
  uint64_t* s_empty = bars + 15;   // [2] per tile, 4 arrivals (PT = false only)
  uint64_t* p_full = bars + 17;    // [2] per tile, 4 arrivals
  uint64_t* o_done = bars + 19;    // [2] per tile: last P V finished
  uint64_t* pv_done = bars + 21;   // [2] per tile: every P V (EARLY mode: P buffer free again, O stable)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
  // SEP: P has tensor-memory columns of its own (D = 64 leaves room), so the scores of block j + 1 can be computed while the
  // soft-max of block j is still running; the same holds when P is staged in shared memory.  Otherwise P overwrites S.
  constexpr bool SEP = PT && D == 64;
  constexpr bool EARLY = !PT || SEP;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid = (heads, batch, tile pairs): x is handed out fastest, so all CTAs of the heaviest pair index start first
  const int t = gridDim.z - 1 - blockIdx.z;  // pair index, heaviest first
  const int h = blockIdx.x, b = blockIdx.y;
  const int hk = h / (p.Hq / p.Hkv);
  const int nbA = 2 * t + 1, nbB = 2 * t + 2;  // key blocks seen by tile A / tile B
  const int row0 = b * p.L + t * 256;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&s_full[x], 1);
      mbar_init(&s_empty[x], 4);
      mbar_init(&p_full[x], 4);
      mbar_init(&o_done[x], 1);
      mbar_init(&pv_done[x], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S_A [0,128)  S_B [128,256)  O_A [256, 256+D)  O_B [256+D, 256+2D)  and, when SEP, P_A [384,448)  P_B [448,512)

  if (warp == 8) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer
      mbar_expect_tx(q_full, 2 * TB);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(sQ + x * TB + c * 16384, &map_q, q_full, p.q_col0 + h * D + 64 * c, row0 + x * 128);
      for (int j = 0; j < nbB; ++j) {
        const int krow = b * p.L + j * 128;
        const int sk = j % KST, sv = j % VST;
        if (!mbar_wait_bounded(&k_empty[sk], ((j / KST) & 1) ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[sk], TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(sK + sk * TB + c * 16384, &map_k, &k_full[sk], p.k_col0 + hk * D + 64 * c, krow);
        if (!mbar_wait_bounded(&v_empty[sv], ((j / VST) & 1) ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&v_full[sv], TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(sV + sv * TB + c * 16384, &map_v, &v_full[sv], p.v_col0 + hk * D + 64 * c, krow);
      }
      if (*abort_flag) {  // give copies already in flight time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 20000ull) {
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc_s = make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t idesc_o = make_idesc(128, D, 1, 1, 0, 1);
      // base descriptors are built once; inside the loops a descriptor is a base plus a constant, because the issue rate
      // of this one thread bounds the kernel when the MMAs are as small as 128 x 64 x 16
      const uint64_t q_k = make_smem_desc_sw128(smem_u32(sQ), 16, 1024), k_k = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t v_mn = make_smem_desc_sw128(smem_u32(sV), 16384, 1024), p_k = make_smem_desc_sw128(smem_u32(sP), 16, 1024);
      auto issue_s = [&](int x, int j) {
        const uint64_t q_d = desc_advance(q_k, uint32_t(x) * TB), k_d = desc_advance(k_k, uint32_t(j % KST) * TB);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(tmem_base + x * 128, desc_advance(q_d, off), desc_advance(k_d, off), idesc_s, k != 0);
        }
        tc_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j) {
        const uint64_t v_d = desc_advance(v_mn, uint32_t(j % VST) * TB);  // MN-major: D contiguous
        const uint32_t o_tmem = tmem_base + 256 + x * D;
        const uint64_t p_d = desc_advance(p_k, uint32_t(x) * 32768);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (PT) tc_mma_f16_ts(o_tmem, (SEP ? tmem_base + 384 + x * 64 : tmem_base + x * 128) + k * 8, desc_advance(v_d, k * 2048), idesc_o, (j | k) != 0);
          else tc_mma_f16(o_tmem, desc_advance(p_d, (k >> 2) * 16384 + (k & 3) * 32), desc_advance(v_d, k * 2048), idesc_o, (j | k) != 0);
        }
      };
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, kTimeoutFull);
      ok = ok && mbar_wait_bounded(&k_full[0], 0, abort_flag, p.status, kTimeoutFull);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_s(1, 0);
        tc_commit(&k_empty[0]);
      }
      const bool rec = PROF && p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
      long long w_load = 0, w_p = 0, t_issue = 0, c0 = 0, c1 = 0;
      const long long t_begin = clock64();
      if (EARLY) {
        for (int j = 0; ok && j < nbB; ++j) {
          const int nk = (j + 1) % KST, nk_ph = ((j + 1) / KST) & 1;
          if (rec) c0 = clock64();
          // scores of the next block first: they only need the S tiles to have been read into registers
          if (j + 1 < nbB) {
            if (!mbar_wait_bounded(&k_full[nk], nk_ph, abort_flag, p.status, kTimeoutFull)) break;
            if (j + 1 < nbA) {
              if (!mbar_wait_bounded(&s_empty[0], j & 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
              tc_fence_after();
              issue_s(0, j + 1);
            }
            if (!mbar_wait_bounded(&s_empty[1], j & 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
            tc_fence_after();
            issue_s(1, j + 1);
            tc_commit(&k_empty[nk]);
          }
          if (!mbar_wait_bounded(&v_full[j % VST], (j / VST) & 1, abort_flag, p.status, kTimeoutFull)) break;
          if (rec) { c1 = clock64(); w_load += c1 - c0; }
          if (j < nbA) {
            if (!mbar_wait_bounded(&p_full[0], j & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
            if (rec) { c0 = clock64(); w_p += c0 - c1; c1 = c0; }
            tc_fence_after();
            issue_pv(0, j);
            tc_commit(&pv_done[0]);
          }
          if (!mbar_wait_bounded(&p_full[1], j & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
          if (rec) { c0 = clock64(); w_p += c0 - c1; }
          tc_fence_after();
          issue_pv(1, j);
          tc_commit(&pv_done[1]);
          tc_commit(&v_empty[j % VST]);
          if (rec) { c1 = clock64(); t_issue += c1 - c0; }
        }
      } else
      for (int j = 0; ok && j < nbB; ++j) {
        const int nk = (j + 1) % KST, nk_ph = ((j + 1) / KST) & 1;
        if (rec) c0 = clock64();
        if (!mbar_wait_bounded(&v_full[j % VST], (j / VST) & 1, abort_flag, p.status, kTimeoutFull)) break;
        if (rec) { c1 = clock64(); w_load += c1 - c0; }
        if (j < nbA) {
          if (!mbar_wait_bounded(&p_full[0], j & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
          if (rec) { c0 = clock64(); w_p += c0 - c1; }
          tc_fence_after();
          issue_pv(0, j);
          if (j == nbA - 1) tc_commit(&o_done[0]);
          if (j + 1 < nbA) {
            if (!mbar_wait_bounded(&k_full[nk], nk_ph, abort_flag, p.status, kTimeoutFull)) break;
            if (!PT && !mbar_wait_bounded(&s_empty[0], j & 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
            tc_fence_after();
            issue_s(0, j + 1);
          }
          if (rec) { c1 = clock64(); t_issue += c1 - c0; }
        }
        if (rec) c0 = clock64();
        if (!mbar_wait_bounded(&p_full[1], j & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
        if (rec) { c1 = clock64(); w_p += c1 - c0; }
        tc_fence_after();
        issue_pv(1, j);
        tc_commit(&v_empty[j % VST]);
        if (j == nbB - 1) tc_commit(&o_done[1]);
        if (j + 1 < nbB) {
          if (!mbar_wait_bounded(&k_full[nk], nk_ph, abort_flag, p.status, kTimeoutFull)) break;
          if (!PT && !mbar_wait_bounded(&s_empty[1], j & 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
          tc_fence_after();
          issue_s(1, j + 1);
          tc_commit(&k_empty[nk]);
        }
        if (rec) { c0 = clock64(); t_issue += c0 - c1; }
      }
      if (rec) {
        p.prof[0] = clock64() - t_begin; p.prof[1] = w_load; p.prof[2] = w_p; p.prof[3] = t_issue; p.prof[4] = nbB;
      }
    }
  } else if (warp < 8) {
    // -------------------------------------------------------------------- soft-max groups
    const int x = warp >> 2;        // 0 = tile A, 1 = tile B
    const int quad = warp & 3;      // TMEM lane quadrant this warp may touch
    const int r = quad * 32 + lane;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t tmem_S = tmem_base + x * 128 + lane_base;
    const uint32_t tmem_O = tmem_base + 256 + x * D + lane_base;
    const int qt = 2 * t + x;
    const int nb = qt + 1;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    const bool rec = PROF && p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 4 && lane == 0;
    long long w_s = 0, t_ld = 0, t_max = 0, t_exp = 0, t_sig = 0, c0 = 0, c1 = 0;
    for (int i = 0; i < nb; ++i) {
      if (rec) c0 = clock64();
      if (!mbar_wait_bounded(&s_full[x], i & 1, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      if (rec) { c1 = clock64(); w_s += c1 - c0; }
      tc_fence_after();
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_S + c * 32, reinterpret_cast<uint32_t(&)[32]>(v[c * 32]));
      tmem_ld_wait();
      if (rec) { c0 = clock64(); t_ld += c0 - c1; }
      if (EARLY) {  // the S tile may be overwritten as soon as every row is in registers
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[x]);
      }
      if (i == qt) {
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (c > r) v[c] = 0xff800000u;  // -inf above the diagonal
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 128; c += 8) {  // three-input max: two new scores per instruction, four independent chains
        mx0 = max3f(mx0, __uint_as_float(v[c]), __uint_as_float(v[c + 1]));
        mx1 = max3f(mx1, __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
        mx2 = max3f(mx2, __uint_as_float(v[c + 4]), __uint_as_float(v[c + 5]));
        mx3 = max3f(mx3, __uint_as_float(v[c + 6]), __uint_as_float(v[c + 7]));
      }
      const float mnew = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
      // The previous P V of this tile must be finished before O is rescaled (rare) or the P buffer is written again.  The
      // exponentials of the first quarter of the row do not depend on it, so the wait sits behind them.
      bool pv_waited = !(EARLY && i > 0);
      if (i == 0) {
        m = mnew;
      } else if (__any_sync(0xffffffffu, mnew > m + 8.f)) {
        if (!pv_waited) {
          if (!mbar_wait_bounded(&pv_done[x], (i - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          pv_waited = true;
        }
        // the previous P V of this tile has completed (implied by S(i) being ready when P aliases S, waited for above otherwise)
        const float alpha = exp2f(m - mnew);
        m = mnew;
        l *= alpha;
#pragma unroll 1
        for (int c = 0; c < D / 16; ++c) {  // rare path: narrow pieces keep its register footprint small
          uint32_t o[16];
          tmem_ld_32x16(tmem_O + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st_32x16(tmem_O + c * 16, o);
        }
        tmem_st_wait();
      }
      if (rec) { c1 = clock64(); t_max += c1 - c0; }
      // exp2(x * scale - m) with packed fp32x2 arithmetic (one FMA and one ADD per two elements); the row sum is taken
      // over the fp32 probabilities
      float2 rsa = make_float2(0.f, 0.f), rsb = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m, -m);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 xs = __ffma2_rn(make_float2(__uint_as_float(v[c * 32 + 2 * e]), __uint_as_float(v[c * 32 + 2 * e + 1])), sc2, nm2);
          const float2 pr = (POLY > 0 && (e % (POLY > 0 ? POLY : 1)) == (POLY > 0 ? POLY : 1) - 1) ? exp2_poly2(xs) : make_float2(exp2f(xs.x), exp2f(xs.y));
          pk[e] = pack_bf16x2(pr.x, pr.y);
          if (e & 1) rsb = __fadd2_rn(rsb, pr);
          else rsa = __fadd2_rn(rsa, pr);
        }
        if (!pv_waited) {  // first quarter done in registers: now the P buffer must be free
          ok = mbar_wait_bounded(&pv_done[x], (i - 1) & 1, abort_flag, p.status, kTimeoutTmemFull);
          tc_fence_after();
          pv_waited = true;
        }
        if (!ok) continue;
        if (PT) {
          tmem_st_32x16((SEP ? tmem_base + 384 + x * 64 + lane_base : tmem_S) + c * 16, pk);
        } else {
          uint8_t* prow = sP + x * 32768 + (c >> 1) * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = (c & 1) * 4 + g;
            *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
          }
        }
      }
      if (!ok) break;
      l += (rsa.x + rsa.y) + (rsb.x + rsb.y);
      if (rec) { c0 = clock64(); t_exp += c0 - c1; }
      if (PT) tmem_st_wait();
      tc_fence_before();
      if (!PT) fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
      if (rec) { c1 = clock64(); t_sig += c1 - c0; }
    }
    if (rec) {
      p.prof[8] = w_s; p.prof[9] = t_ld; p.prof[10] = t_max; p.prof[11] = t_exp; p.prof[12] = t_sig;
    }
    if (ok && (EARLY ? mbar_wait_bounded(&pv_done[x], (nb - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)
                     : mbar_wait_bounded(&o_done[x], 0, abort_flag, p.status, kTimeoutTmemFull))) {
      tc_fence_after();
      const float inv = 1.f / l;
      const long long tok = (long long)row0 + x * 128 + r;
      __nv_bfloat16* orow = p.out + (tok * p.Hq + h) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_O + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) =
              make_uint4(pack_bf16x2(__uint_as_float(o[8 * g]) * inv, __uint_as_float(o[8 * g + 1]) * inv),
                         pack_bf16x2(__uint_as_float(o[8 * g + 2]) * inv, __uint_as_float(o[8 * g + 3]) * inv),
                         pack_bf16x2(__uint_as_float(o[8 * g + 4]) * inv, __uint_as_float(o[8 * g + 5]) * inv),
                         pack_bf16x2(__uint_as_float(o[8 * g + 6]) * inv, __uint_as_float(o[8 * g + 7]) * inv));
      }
      if (p.lse) p.lse[((long long)b * p.Hq + h) * p.L + (long long)qt * 128 + r] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ats

using namespace ats;

static int g_fwd2_poly = 0;  // measured on B200: the polynomial path does not pay off (0.284 ms vs 0.291 / 0.302 ms at every 4th / 2nd pair)

template <int D, bool PT, bool PROF, int POLY>
static int launch_fwd2_impl(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Attn2Args& p, int B, int L, int Hq,
                       cudaStream_t s) {
  using SM = Attn2Smem<D, PT>;
  cudaError_t ce = cudaFuncSetAttribute(attn_fwd2_kernel<D, PT, PROF, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
  if (ce != cudaSuccess) return int(ce);
  dim3 grid(Hq, B, L / 256);
  attn_fwd2_kernel<D, PT, PROF, POLY><<<grid, A2_THREADS, SM::TOTAL, s>>>(mq, mk, mv, p);
  return int(cudaGetLastError());
}

template <int D, bool PT>
static int launch_fwd2(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Attn2Args& p, int B, int L, int Hq,
                       cudaStream_t s) {
  // the instrumented build of the kernel runs only when a profile buffer is given
  if (p.prof) return launch_fwd2_impl<D, PT, true, 0>(mq, mk, mv, p, B, L, Hq, s);
  if (g_fwd2_poly == 2) return launch_fwd2_impl<D, PT, false, 2>(mq, mk, mv, p, B, L, Hq, s);
  if (g_fwd2_poly == 4) return launch_fwd2_impl<D, PT, false, 4>(mq, mk, mv, p, B, L, Hq, s);
  return launch_fwd2_impl<D, PT, false, 0>(mq, mk, mv, p, B, L, Hq, s);
}

// Share of the forward pass's exponentials computed on the FMA pipe: 0 = none, 2 = every second pair, 4 = every fourth.
ATS_API int ats_attn_fwd2_set_poly(int every) {
  if (every != 0 && every != 2 && every != 4) return 1003;
  g_fwd2_poly = every;
  return 0;
}

// Same contract as ats_attn_fwd, for L a multiple of 256.  p_in_tmem selects where the probabilities are staged.
// prof: null, or 16 int64 that receive per-phase cycle totals of CTA (0,0,0) (diagnostics).
ATS_API int ats_attn_fwd2(const void* q, long long ld_q, long long q_cols, int q_col0, const void* k, long long ld_k,
                          long long k_cols, int k_col0, const void* v, long long ld_v, long long v_cols, int v_col0,
                          void* out, float* lse, int B, int L, int Hq, int Hkv, int D, int p_in_tmem, int* status, long long* prof, void* stream) {
  if ((D != 64 && D != 128) || (L % 256) || Hq % Hkv || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7)) return 1003;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  CUtensorMap mq, mk, mv;
  int e;
  const unsigned long long rows = (unsigned long long)B * L;
  if ((e = make_tmap_2d(&mq, q, rows, q_cols, ld_q, 2, 64, 128))) return e;
  if ((e = make_tmap_2d(&mk, k, rows, k_cols, ld_k, 2, 64, 128))) return e;
  if ((e = make_tmap_2d(&mv, v, rows, v_cols, ld_v, 2, 64, 128))) return e;
  Attn2Args p;
  p.B = B; p.L = L; p.Hq = Hq; p.Hkv = Hkv;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse;
  p.scale_log2 = 1.4426950408889634f / sqrtf(float(D));
  p.status = status;
  p.prof = prof;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128) return p_in_tmem ? launch_fwd2<128, true>(mq, mk, mv, p, B, L, Hq, s) : launch_fwd2<128, false>(mq, mk, mv, p, B, L, Hq, s);
  return p_in_tmem ? launch_fwd2<64, true>(mq, mk, mv, p, B, L, Hq, s) : launch_fwd2<64, false>(mq, mk, mv, p, B, L, Hq, s);
}
