// Causal grouped-query flash attention backward for sm_100a on tcgen05 tensor cores.
//
// Two passes share one kernel template (plus a tiny pre-pass delta = rowsum(dO * O)):
//   MODE 0 (dK, dV): one CTA per (128-key tile j, kv head, batch).  K_j and V_j stay in shared memory; for every query
//           head of the group and every query tile i >= j the CTA streams Q_i and dO_i, recomputes S = Q K^T and
//           dP = dO V^T on the tensor cores, forms P = exp(S - lse) and dS = P * (dP - delta) * scale in registers, and
//           accumulates dV += P^T dO and dK += dS^T Q in TMEM across all iterations (no atomics, deterministic).
//   MODE 1 (dQ):     one CTA per (128-query tile i, query head, batch).  Q_i and dO_i stay resident, K_j / V_j stream for
//           j <= i, and dQ += dS K accumulates in TMEM; dS goes back to tensor memory as bf16 and is the MMA's A operand.
// S and dP are recomputed in both passes (7 tile products per tile pair instead of 5) in exchange for an atomics-free,
// deterministic dQ.  P and dS live in shared memory as [query x key] bf16 tiles in the 128-byte-swizzled layout, which
// the same bytes serve both as a K-major operand (dS K) and as an MN-major operand (P^T dO, dS^T Q).
//
//   warp 0: TMA producer   warp 1: TMEM owner + MMA issuer   warps 2..9: two threads per query row (64 key columns each)
// Every wait is bounded (status word + clean unwind); no load uses cluster multicast.
//
// Replaces the flash-attn / SDPA backward the reference relies on (reference core/model.py:763-768).
#include "common.cuh"

namespace ats {

#ifndef ATS_AB_SPLIT
#define ATS_AB_SPLIT 2
#endif
constexpr int AB_SPLIT = ATS_AB_SPLIT;             // threads per query row in the softmax-gradient stage (2 or 4)
constexpr int AB_COLS = 128 / AB_SPLIT;           // key columns per thread
constexpr int AB_THREADS = 64 + 128 * AB_SPLIT;   // TMA warp, MMA warp, 4 * AB_SPLIT softmax-gradient warps

struct AttnBwdArgs {
  int B, L, Hq, Hkv, D;
  int q_col0, k_col0, v_col0;
  const float* lse;    // [B, Hq, L] natural log
  const float* delta;  // [B, Hq, L]
  __nv_bfloat16* dq;   // row = token, pitch ld_dq elements, head h at column h * D
  __nv_bfloat16* dk;   // row = token, pitch ld_dkv
  __nv_bfloat16* dv;
  long long ld_dq, ld_dkv;
  float scale, scale_log2;
  int* status;
  long long* prof;  // optional [16]: cycle totals per phase, written by one CTA (diagnostics; null in normal use)
};

template <int D, int MODE>
struct AttnBwdSmem {
  // streamed stages: a stage is held until the gradient products that read it have finished, and a refill takes a
  // TMA round trip, so the ring must be deep enough to have the next tiles in flight meanwhile
  static constexpr int ST = (D == 64) ? 4 : (MODE == 1 ? 2 : 1);
  static constexpr int TB = 128 * D * 2;
  static constexpr int R1 = 0, R2 = TB;
  static constexpr int T1 = 2 * TB;            // ST stages
  static constexpr int T2 = T1 + ST * TB;      // ST stages
  static constexpr int P_OFF = T2 + ST * TB;   // MODE 0 only
  static constexpr int DS_OFF = P_OFF + (MODE == 0 ? 32768 : 0);
  static constexpr int BAR_OFF = DS_OFF + (MODE == 0 ? 32768 : 0);  // the dQ pass keeps dS in tensor memory
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// delta[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d].  Eight elements (16 bytes) per thread, D / 8 threads per row, so a
// warp covers 32 / (D / 8) rows with fully coalesced 512-byte accesses.
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                                         float* __restrict__ delta, int B, int L, int Hq, int D) {
  const int tpr = D >> 3;  // threads per row: 8 (D = 64) or 16 (D = 128)
  const long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long row = g / tpr;  // (token, head) row
  const int part = int(g % tpr);
  const long long total = (long long)B * L * Hq;
  float acc = 0.f;
  if (row < total) {
    const uint4 a = reinterpret_cast<const uint4*>(dout + row * D)[part];
    const uint4 o = reinterpret_cast<const uint4*>(out + row * D)[part];
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 o0 = unpack_bf16x2(o.x), o1 = unpack_bf16x2(o.y), o2 = unpack_bf16x2(o.z), o3 = unpack_bf16x2(o.w);
    acc = a0.x * o0.x + a0.y * o0.y + a1.x * o1.x + a1.y * o1.y + a2.x * o2.x + a2.y * o2.y + a3.x * o3.x + a3.y * o3.y;
  }
  for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < total && part == 0) {
    const int h = int(row % Hq);
    const long long tok = row / Hq;
    const int b = int(tok / L), i = int(tok % L);
    delta[((long long)b * Hq + h) * L + i] = acc;
  }
}

template <int D, int MODE>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const AttnBwdArgs p) {
  using SM = AttnBwdSmem<D, MODE>;
  constexpr int ST = SM::ST;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sR1 = smem + SM::R1;
  uint8_t* sR2 = smem + SM::R2;
  uint8_t* sT1 = smem + SM::T1;
  uint8_t* sT2 = smem + SM::T2;
  uint8_t* sP = smem + SM::P_OFF;
  uint8_t* sDS = smem + SM::DS_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* res_full = bars;       // 1
  uint64_t* t_full = bars + 1;     // [4]
  uint64_t* t_empty = bars + 5;    // [4]
  uint64_t* s_full = bars + 9;     // S and dP ready
  uint64_t* sd_free = bars + 10;   // one arrival per softmax warp: S / dP read out of TMEM
  uint64_t* pds_full = bars + 11;  // one arrival per softmax warp: P / dS written to shared memory
  uint64_t* pds_free = bars + 12;  // accumulate MMAs have consumed P / dS
  uint64_t* acc_done = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = p.L / 128;
  const int rep = p.Hq / p.Hkv;
  // Grid = (heads, batch, tiles): CTAs are handed out x-fastest, so with the tile index slowest every CTA of the heaviest
  // tile (of all heads and sequences) starts before any lighter one.  With the tile index fastest, a heavy tile of the
  // last heads started late and the causal imbalance left SMs idle for a quarter of the dK/dV pass.
  const int b = blockIdx.y;
  // fixed tile of this CTA and iteration space
  int fixed, head, n_iter;
  if (MODE == 0) {
    fixed = blockIdx.z;  // key tile j (j = 0 has the most work)
    head = blockIdx.x;   // kv head
    n_iter = rep * (nq - fixed);
  } else {
    fixed = nq - 1 - blockIdx.z;  // query tile i (the last one has the most work)
    head = blockIdx.x;            // query head
    n_iter = fixed + 1;
  }
  const int hk = MODE == 0 ? head : head / rep;

  if (threadIdx.x == 0) {
    mbar_init(res_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&t_full[s], 1);
      mbar_init(&t_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(sd_free, 4 * AB_SPLIT);
    mbar_init(pds_full, 4 * AB_SPLIT);
    mbar_init(pds_free, 1);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_A1 = tmem_base + 256, tmem_A2 = tmem_base + 256 + D;
  const uint32_t tmem_dS = tmem_base + 384;  // MODE 1: dS as bf16 pairs, 64 columns, the A operand of dQ += dS K

  // iteration t -> (query head, query tile, key tile)
  auto decode = [&](int t, int& h, int& qi, int& kj) {
    if (MODE == 0) {
      const int per = nq - fixed;
      h = head * rep + t / per;
      qi = fixed + t % per;
      kj = fixed;
    } else {
      h = head;
      qi = fixed;
      kj = t;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer
      mbar_expect_tx(res_full, 2 * SM::TB);
      if (MODE == 0) {
        const int row = b * p.L + fixed * 128;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(sR1 + c * 16384, &map_k, res_full, p.k_col0 + hk * D + 64 * c, row);
          tma_load_2d(sR2 + c * 16384, &map_v, res_full, p.v_col0 + hk * D + 64 * c, row);
        }
      } else {
        const int row = b * p.L + fixed * 128;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(sR1 + c * 16384, &map_q, res_full, p.q_col0 + head * D + 64 * c, row);
          tma_load_2d(sR2 + c * 16384, &map_do, res_full, head * D + 64 * c, row);
        }
      }
      for (int t = 0; t < n_iter; ++t) {
        const int s = t % ST, ph = (t / ST) & 1;
        int h, qi, kj;
        decode(t, h, qi, kj);
        if (!mbar_wait_bounded(&t_empty[s], ph ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&t_full[s], 2 * SM::TB);
        if (MODE == 0) {
          const int row = b * p.L + qi * 128;
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_2d(sT1 + s * SM::TB + c * 16384, &map_q, &t_full[s], p.q_col0 + h * D + 64 * c, row);
            tma_load_2d(sT2 + s * SM::TB + c * 16384, &map_do, &t_full[s], h * D + 64 * c, row);
          }
        } else {
          const int row = b * p.L + kj * 128;
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_2d(sT1 + s * SM::TB + c * 16384, &map_k, &t_full[s], p.k_col0 + hk * D + 64 * c, row);
            tma_load_2d(sT2 + s * SM::TB + c * 16384, &map_v, &t_full[s], p.v_col0 + hk * D + 64 * c, row);
          }
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 20000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc_s = make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t idesc_acc0 = make_idesc(128, D, 1, 1, 1, 1);  // A^T B with both operands MN-major
      const uint32_t idesc_acc1 = make_idesc(128, D, 1, 1, 0, 1);  // dS (K-major) x K (MN-major)
      // Descriptors are built once: per operand one base descriptor for the K-major view and one for the MN-major view;
      // inside the loops a descriptor is the base plus a constant (the issue rate of this one thread bounds the kernel).
      const uint64_t r1_k = make_smem_desc_sw128(smem_u32(sR1), 16, 1024), r2_k = make_smem_desc_sw128(smem_u32(sR2), 16, 1024);
      const uint64_t r1_mn = make_smem_desc_sw128(smem_u32(sR1), 16384, 1024), r2_mn = make_smem_desc_sw128(smem_u32(sR2), 16384, 1024);
      const uint64_t t1_k = make_smem_desc_sw128(smem_u32(sT1), 16, 1024), t2_k = make_smem_desc_sw128(smem_u32(sT2), 16, 1024);
      const uint64_t t1_mn = make_smem_desc_sw128(smem_u32(sT1), 16384, 1024), t2_mn = make_smem_desc_sw128(smem_u32(sT2), 16384, 1024);
      const uint64_t p_mn = make_smem_desc_sw128(smem_u32(sP), 16384, 1024), ds_mn = make_smem_desc_sw128(smem_u32(sDS), 16384, 1024);
      auto issue_scores = [&](int t) {  // S = Q K^T and dP = dO V^T of iteration t
        const uint32_t so = uint32_t(t % ST) * SM::TB;
        const uint64_t q_d = MODE == 0 ? desc_advance(t1_k, so) : r1_k, do_d = MODE == 0 ? desc_advance(t2_k, so) : r2_k;
        const uint64_t k_d = MODE == 0 ? r1_k : desc_advance(t1_k, so), v_d = MODE == 0 ? r2_k : desc_advance(t2_k, so);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(tmem_S, desc_advance(q_d, off), desc_advance(k_d, off), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(tmem_dP, desc_advance(do_d, off), desc_advance(v_d, off), idesc_s, k != 0);
        }
        tc_commit(s_full);
      };
      auto issue_acc = [&](int t) {  // the gradient products that consume P / dS of iteration t
        const int s = t % ST;
        const uint32_t so = uint32_t(s) * SM::TB;
        if (MODE == 0) {
          const uint64_t do_d = desc_advance(t2_mn, so), q_d = desc_advance(t1_mn, so);
#pragma unroll
          for (int k = 0; k < 8; ++k)  // reduction over the 128 queries, 16 per step
            tc_mma_f16(tmem_A1, desc_advance(p_mn, k * 2048), desc_advance(do_d, k * 2048), idesc_acc0, (t | k) != 0);
#pragma unroll
          for (int k = 0; k < 8; ++k) tc_mma_f16(tmem_A2, desc_advance(ds_mn, k * 2048), desc_advance(q_d, k * 2048), idesc_acc0, (t | k) != 0);
        } else {
          const uint64_t k_d = desc_advance(t1_mn, so);
#pragma unroll
          for (int k = 0; k < 8; ++k)  // reduction over the 128 keys; dS is read from tensor memory (8 columns per 16 keys)
            tc_mma_f16_ts(tmem_A1, tmem_dS + k * 8, desc_advance(k_d, k * 2048), idesc_acc1, (t | k) != 0);
        }
        tc_commit(pds_free);
        tc_commit(&t_empty[s]);
      };
      bool ok = mbar_wait_bounded(res_full, 0, abort_flag, p.status, kTimeoutFull);
      if (ST >= 2) {
        // The scores of iteration t + 1 are issued as soon as the soft-max threads have S / dP of iteration t in registers,
        // so the tensor cores work on them while those threads do the exponentials of iteration t.
        ok = ok && mbar_wait_bounded(&t_full[0], 0, abort_flag, p.status, kTimeoutFull);
        if (ok) {
          tc_fence_after();
          issue_scores(0);
        }
        const bool rec = p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        long long w_tfull = 0, w_sdfree = 0, w_pdsfull = 0, t_issue = 0, c0 = 0, c1 = 0;
        const long long t_begin = clock64();
        for (int t = 0; ok && t < n_iter; ++t) {
          if (t + 1 < n_iter) {
            if (rec) c0 = clock64();
            if (!mbar_wait_bounded(&t_full[(t + 1) % ST], ((t + 1) / ST) & 1, abort_flag, p.status, kTimeoutFull)) break;
            if (rec) { c1 = clock64(); w_tfull += c1 - c0; }
            if (!mbar_wait_bounded(sd_free, t & 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
            if (rec) { c0 = clock64(); w_sdfree += c0 - c1; }
            tc_fence_after();
            issue_scores(t + 1);
            if (rec) { c1 = clock64(); t_issue += c1 - c0; }
          }
          if (rec) c0 = clock64();
          if (!mbar_wait_bounded(pds_full, t & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
          if (rec) { c1 = clock64(); w_pdsfull += c1 - c0; }
          tc_fence_after();
          issue_acc(t);
          if (rec) { c0 = clock64(); t_issue += c0 - c1; }
        }
        if (rec) {
          p.prof[0] = clock64() - t_begin;
          p.prof[1] = w_tfull; p.prof[2] = w_sdfree; p.prof[3] = w_pdsfull; p.prof[4] = t_issue; p.prof[5] = n_iter;
        }
      } else {
        // one streamed stage: the next tile can only be fetched after this iteration's products, so the order is serial
        for (int t = 0; ok && t < n_iter; ++t) {
          if (!mbar_wait_bounded(&t_full[0], t & 1, abort_flag, p.status, kTimeoutFull)) break;
          if (!mbar_wait_bounded(sd_free, (t & 1) ^ 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
          tc_fence_after();
          issue_scores(t);
          if (!mbar_wait_bounded(pds_full, t & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
          tc_fence_after();
          issue_acc(t);
        }
      }
      tc_commit(acc_done);
    }
  } else {
    // ---------------------------------------- softmax-gradient threads: a TMEM lane quadrant is open to warps with the
    // same (warp % 4), so the AB_SPLIT warps w, w + 4, ... share 32 query rows and take AB_COLS key columns each
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // which AB_COLS key columns of the 128
    const int r = quad * 32 + lane;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    bool ok = true;
    // log-sum-exp and delta of this thread's query row, fetched one iteration ahead so the loads never sit on the critical path
    auto row_stats = [&](int t, float& l2, float& d) {
      int h, qi, kj;
      decode(t, h, qi, kj);
      const long long idx = ((long long)b * p.Hq + h) * p.L + qi * 128 + r;
      l2 = p.lse[idx] * 1.4426950408889634f;
      d = p.delta[idx];
    };
    float lse2 = 0.f, dl = 0.f, lse2_n = 0.f, dl_n = 0.f;
    if (n_iter > 0) row_stats(0, lse2_n, dl_n);
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), scale2 = make_float2(p.scale, p.scale);
    const bool rec = p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 2 && lane == 0;
    long long w_sfull = 0, t_load = 0, t_math = 0, w_pdsfree = 0, t_store = 0, c0 = 0, c1 = 0;
    for (int t = 0; t < n_iter; ++t) {
      int h, qi, kj;
      decode(t, h, qi, kj);
      lse2 = lse2_n;
      dl = dl_n;
      if (t + 1 < n_iter && (MODE == 0)) row_stats(t + 1, lse2_n, dl_n);  // MODE 1 keeps the same query rows throughout
      if (rec) c0 = clock64();
      if (!mbar_wait_bounded(s_full, t & 1, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      if (rec) { c1 = clock64(); w_sfull += c1 - c0; }
      tc_fence_after();
      // this thread's columns of S, then of dP; the exponentials start while the dP load is still in flight
      uint32_t sv[AB_COLS], dv[AB_COLS];
#pragma unroll
      for (int c = 0; c < AB_COLS / 32; ++c) tmem_ld_32x32(tmem_S + lane_base + part * AB_COLS + c * 32, reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
      tmem_ld_wait();
      if (rec) { c0 = clock64(); t_load += c0 - c1; }
#pragma unroll
      for (int c = 0; c < AB_COLS / 32; ++c) tmem_ld_32x32(tmem_dP + lane_base + part * AB_COLS + c * 32, reinterpret_cast<uint32_t(&)[32]>(dv[c * 32]));
      const float2 nl2 = make_float2(-lse2, -lse2), ndl2 = make_float2(-dl, -dl);
      const bool diag = (qi == kj);
      float2 pr[AB_COLS / 2];
      uint32_t pk[AB_COLS / 2], dk[AB_COLS / 2];
#pragma unroll
      for (int i = 0; i < AB_COLS / 2; ++i) {
        const float2 xs = __ffma2_rn(make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), sc2, nl2);
        pr[i] = make_float2(exp2f(xs.x), exp2f(xs.y));
        if (diag) {
          if (part * AB_COLS + 2 * i > r) pr[i].x = 0.f;
          if (part * AB_COLS + 2 * i + 1 > r) pr[i].y = 0.f;
        }
        pk[i] = pack_bf16x2(pr[i].x, pr[i].y);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sd_free);  // S and dP are in registers: the tensor cores may start the next scores
#pragma unroll
      for (int i = 0; i < AB_COLS / 2; ++i) {
        const float2 dd = __fmul2_rn(__fmul2_rn(pr[i], scale2), __fadd2_rn(make_float2(__uint_as_float(dv[2 * i]), __uint_as_float(dv[2 * i + 1])), ndl2));
        dk[i] = pack_bf16x2(dd.x, dd.y);
      }
      // the gradient products of the previous iteration must be done with P / dS before they are overwritten
      if (rec) { c1 = clock64(); t_math += c1 - c0; }
      if (!mbar_wait_bounded(pds_free, (t & 1) ^ 1, abort_flag, p.status, kTimeoutTmemEmpty)) {
        ok = false;
        break;
      }
      if (rec) { c0 = clock64(); w_pdsfree += c0 - c1; }
      if (MODE == 1) {
        // dQ pass: dS never touches shared memory
        if (AB_COLS == 64) tmem_st_32x32(tmem_dS + lane_base + part * 32, reinterpret_cast<uint32_t(&)[32]>(dk[0]));
        else tmem_st_32x16(tmem_dS + lane_base + part * 16, reinterpret_cast<uint32_t(&)[16]>(dk[0]));
        tmem_st_wait();
        tc_fence_before();
      } else {
        constexpr int CH = AB_COLS / 8;  // 16-byte chunks per thread
        const int col0 = part * AB_COLS;
        const int roff = (col0 >> 6) * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int g = 0; g < CH; ++g) {
          const int chunk = ((((col0 & 63) >> 3) + g) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(sP + roff + chunk) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
          *reinterpret_cast<uint4*>(sDS + roff + chunk) = make_uint4(dk[4 * g], dk[4 * g + 1], dk[4 * g + 2], dk[4 * g + 3]);
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (rec) { c1 = clock64(); t_store += c1 - c0; }
    }
    if (rec) {
      p.prof[8] = w_sfull; p.prof[9] = t_load; p.prof[10] = t_math; p.prof[11] = w_pdsfree; p.prof[12] = t_store;
    }
    if (ok && mbar_wait_bounded(acc_done, 0, abort_flag, p.status, kTimeoutTmemFull)) {
      tc_fence_after();
      const long long tok = (long long)b * p.L + fixed * 128 + r;
      __nv_bfloat16* o1 = MODE == 0 ? p.dv + tok * p.ld_dkv + head * D : p.dq + tok * p.ld_dq + head * D;
      __nv_bfloat16* o2 = MODE == 0 ? p.dk + tok * p.ld_dkv + head * D : nullptr;
      // the AB_SPLIT threads of a row store D / AB_SPLIT columns each, 16 at a time
      constexpr int PIECES = D / 16 / AB_SPLIT;
#pragma unroll
      for (int c = part * PIECES; c < (part + 1) * PIECES; ++c) {
        uint32_t v[16];
        tmem_ld_32x16(tmem_A1 + lane_base + c * 16, v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 2; ++g)
          *reinterpret_cast<uint4*>(o1 + c * 16 + g * 8) =
              make_uint4(pack_bf16x2(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1])), pack_bf16x2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3])),
                         pack_bf16x2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5])), pack_bf16x2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7])));
        if (MODE == 0) {
          tmem_ld_32x16(tmem_A2 + lane_base + c * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 2; ++g)
            *reinterpret_cast<uint4*>(o2 + c * 16 + g * 8) =
                make_uint4(pack_bf16x2(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1])), pack_bf16x2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3])),
                           pack_bf16x2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5])), pack_bf16x2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7])));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ats

using namespace ats;

template <int D, int MODE>
static int launch_attn_bwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                           const AttnBwdArgs& p, cudaStream_t s) {
  using SM = AttnBwdSmem<D, MODE>;
  cudaError_t ce = cudaFuncSetAttribute(attn_bwd_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
  if (ce != cudaSuccess) return int(ce);
  dim3 grid(MODE == 0 ? p.Hkv : p.Hq, p.B, p.L / 128);
  attn_bwd_kernel<D, MODE><<<grid, AB_THREADS, SM::TOTAL, s>>>(mq, mk, mv, mdo, p);
  return int(cudaGetLastError());
}

// q/k/v as for ats_attn_fwd; out, dout: [B, L, Hq, D] contiguous; lse [B, Hq, L]; delta: fp32 scratch [B, Hq, L];
// dq: rows = tokens with pitch ld_dq, dk / dv with pitch ld_dkv (so all three can be slices of one packed gradient).
// prof: null, or 32 int64 that receive per-phase cycle totals of CTA (0,0,0) of each pass (diagnostics).
ATS_API int ats_attn_bwd(const void* q, long long ld_q, long long q_cols, int q_col0, const void* k, long long ld_k,
                         long long k_cols, int k_col0, const void* v, long long ld_v, long long v_cols, int v_col0,
                         const void* out, const void* dout, const float* lse, float* delta, void* dq, void* dk, void* dv,
                         long long ld_dq, long long ld_dkv, int B, int L, int Hq, int Hkv, int D, int* status, long long* prof, void* stream) {
  if ((D != 64 && D != 128) || (L % 128) || Hq % Hkv || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7) || (ld_dq & 7) || (ld_dkv & 7))
    return 1003;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap mq, mk, mv, mdo;
  int e;
  const unsigned long long rows = (unsigned long long)B * L;
  if ((e = make_tmap_2d(&mq, q, rows, q_cols, ld_q, 2, 64, 128))) return e;
  if ((e = make_tmap_2d(&mk, k, rows, k_cols, ld_k, 2, 64, 128))) return e;
  if ((e = make_tmap_2d(&mv, v, rows, v_cols, ld_v, 2, 64, 128))) return e;
  if ((e = make_tmap_2d(&mdo, dout, rows, (unsigned long long)Hq * D, (unsigned long long)Hq * D, 2, 64, 128))) return e;
  const long long delta_threads = (long long)B * L * Hq * (D / 8);
  attn_delta_kernel<<<unsigned((delta_threads + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dout),
                                                                      static_cast<const __nv_bfloat16*>(out), delta, B, L, Hq, D);
  AttnBwdArgs p;
  p.B = B; p.L = L; p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.lse = lse; p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq); p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
  p.ld_dq = ld_dq; p.ld_dkv = ld_dkv;
  p.scale = 1.f / sqrtf(float(D));
  p.scale_log2 = 1.4426950408889634f * p.scale;
  p.status = status;
  p.prof = prof;
  if (D == 128) {
    if ((e = launch_attn_bwd<128, 0>(mq, mk, mv, mdo, p, s))) return e;
    if (prof) p.prof = prof + 16;
    return launch_attn_bwd<128, 1>(mq, mk, mv, mdo, p, s);
  }
  if ((e = launch_attn_bwd<64, 0>(mq, mk, mv, mdo, p, s))) return e;
  if (prof) p.prof = prof + 16;
  return launch_attn_bwd<64, 1>(mq, mk, mv, mdo, p, s);
}
