// Causal grouped-query flash attention forward for sm_100a on tcgen05 tensor cores.
//
//   O[b, i, h, :] = softmax_j<=i( Q[b,i,h,:] . K[b,j,g(h),:] / sqrt(D) ) V[b,j,g(h),:]        g(h) = h / (Hq / Hkv)
//
// One CTA per (128-query tile, query head, batch).  K and V tiles of 128 keys stream through a 2-stage TMA pipeline
// and are shared by nothing else: the query heads of a group read the same K/V straight from global memory / L2,
// no expanded copy of K/V is ever made (the reference materialises it with repeat_interleave, core/model.py:705-707).
//
//   warp 0      TMA producer (Q once, then K_j, V_j)
//   warp 1      owns TMEM; issues S_j = Q K_j^T (fp32 in TMEM, double-buffered) and O_j = P_j V_j
//   warps 2..5  one query row per thread: read S_j from TMEM, online softmax in the log2 domain, write P_j (bf16)
//               into shared memory in the 128-byte-swizzled K-major layout the MMA reads, then fold O_j into the
//               fp32 accumulator kept in registers.
//
// Q/K/V are addressed through 2-D tensor maps over the packed projection buffer (row = token, column = head*D + d),
// so the attention reads the QKV GEMM's output in place.  Output: O [B, L, Hq, D] bf16 and the log-sum-exp
// [B, Hq, L] fp32 for the backward pass.  Every wait is bounded (status word + clean unwind).
#include "common.cuh"

namespace ats {

constexpr int ATT_BM = 128;  // queries per CTA
constexpr int ATT_BN = 128;  // keys per block
constexpr int ATT_THREADS = 192;

struct AttnArgs {
  int B, L, Hq, Hkv, D;
  int q_col0, k_col0, v_col0;  // first column of head 0 of each operand inside its tensor map
  __nv_bfloat16* out;          // [B, L, Hq, D]
  float* lse;                  // [B, Hq, L]
  float scale_log2;            // log2(e) / sqrt(D)
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int TILE_BYTES = 128 * D * 2;          // one 128-row operand tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE_BYTES;                // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE_BYTES;    // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * TILE_BYTES;    // 128 x 128 bf16
  static constexpr int BAR_OFF = P_OFF + 128 * 128 * 2;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;      // barriers + alignment slack
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const AttnArgs p) {
  using SM = AttnSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + SM::Q_OFF;
  uint8_t* sK = smem + SM::K_OFF;
  uint8_t* sV = smem + SM::V_OFF;
  uint8_t* sP = smem + SM::P_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* v_full = bars + 3;      // [2]
  uint64_t* k_empty = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* s_empty = bars + 11;    // [2], 4 arrivals
  uint64_t* p_full = bars + 13;     // 4 arrivals
  uint64_t* pv_done = bars + 14;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid = (heads, batch, query tiles): x is handed out fastest, so all CTAs of the heaviest tile index start first
  const int qt = gridDim.z - 1 - blockIdx.z;  // heaviest tiles first
  const int h = blockIdx.x, b = blockIdx.y;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_blocks = qt + 1;
  const int row0 = b * p.L + qt * ATT_BM;     // token row of the first query

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;        // two buffers of 128 columns
  const uint32_t tmem_O = tmem_base + 256;  // D columns

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer
      mbar_expect_tx(q_full, SM::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_2d(sQ + c * 16384, &map_q, q_full, p.q_col0 + h * D + 64 * c, row0);
      bool ok = true;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int s = j & 1, ph = (j >> 1) & 1;
        const int krow = b * p.L + j * ATT_BN;
        if (!mbar_wait_bounded(&k_empty[s], ph ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[s], SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(sK + s * SM::TILE_BYTES + c * 16384, &map_k, &k_full[s], p.k_col0 + hk * D + 64 * c, krow);
        if (!mbar_wait_bounded(&v_empty[s], ph ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&v_full[s], SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(sV + s * SM::TILE_BYTES + c * 16384, &map_v, &v_full[s], p.v_col0 + hk * D + 64 * c, krow);
      }
      if (*abort_flag) {  // give copies already in flight time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 20000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc_s = make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t idesc_o = make_idesc(128, D, 1, 1, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&k_full[s], ph, abort_flag, p.status, kTimeoutFull)) return false;
        if (!mbar_wait_bounded(&s_empty[s], ph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * SM::TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(tmem_S + s * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                     make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, k != 0);
        }
        tc_commit(&s_full[s]);
        tc_commit(&k_empty[s]);
        return true;
      };
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, kTimeoutFull);
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_blocks; ++j) {
        if (j + 1 < n_blocks && !issue_s(j + 1)) break;
        const int s = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&v_full[s], ph, abort_flag, p.status, kTimeoutFull)) break;
        if (!mbar_wait_bounded(p_full, j & 1, abort_flag, p.status, kTimeoutTmemFull)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * SM::TILE_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(p_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(v_addr + k * 2048, 16384, 1024);  // MN-major: D contiguous
          tc_mma_f16(tmem_O, adesc, bdesc, idesc_o, k != 0);
        }
        tc_commit(pv_done);
        tc_commit(&v_empty[s]);
      }
    }
  } else {
    // -------------------------------------------------------------------- softmax + accumulate (one row per thread)
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // query row inside the tile
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const int s = j & 1, ph = (j >> 1) & 1;
      if (!mbar_wait_bounded(&s_full[s], ph, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool diag = (j == qt);
      // pass 1: row maximum
      // four independent running maxima / sums: with one softmax warp per scheduler a 128-long dependent chain
      // would expose the full ALU latency on every element
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_S + s * 128 + lane_base + c * 32, v);
        tmem_ld_wait();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > r) v[i] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(v[i]));
          mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(v[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
        }
      }
      // raw maxima are scaled once (scale > 0); the carried maximum m is already in the log2 domain
      const float mx = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
      const float alpha = exp2f(m - mx);
      m = mx;
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
      // pass 2: probabilities -> P tile in shared memory (K-major, 128-byte swizzle: chunk ^= row % 8)
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_S + s * 128 + lane_base + c * 32, v);
        tmem_ld_wait();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > r) v[i] = 0xff800000u;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          // exp2(x * scale - mx) as one FMA + ex2; exp2(-inf) = 0 handles the causal mask
          const float p0 = exp2f(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, -mx));
          const float p1 = exp2f(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, -mx));
          pk[i] = pack_bf16x2(p0, p1);
          const float2 q = unpack_bf16x2(pk[i]);  // sum what the MMA will actually see
          if (i & 1) {
            rs2 += q.x;
            rs3 += q.y;
          } else {
            rs0 += q.x;
            rs1 += q.y;
          }
        }
        uint8_t* prow = sP + (c >> 1) * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c & 1) * 4 + g;  // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        }
      }
      const float rs = (rs0 + rs1) + (rs2 + rs3);
      l = l * alpha + rs;
      tc_fence_before();
      fence_proxy_async_smem();  // P was written with generic stores, the MMA reads it through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[s]);
        mbar_arrive(p_full);
      }
      // fold O_j into the accumulator once the P V product is done
      if (!mbar_wait_bounded(pv_done, j & 1, abort_flag, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_base + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = acc[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
    }
    if (ok) {
      const float inv = 1.f / l;
      const long long tok = (long long)row0 + r;
      __nv_bfloat16* orow = p.out + (tok * p.Hq + h) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<uint4*>(orow + i * 8) =
            make_uint4(pack_bf16x2(acc[8 * i] * inv, acc[8 * i + 1] * inv), pack_bf16x2(acc[8 * i + 2] * inv, acc[8 * i + 3] * inv),
                       pack_bf16x2(acc[8 * i + 4] * inv, acc[8 * i + 5] * inv), pack_bf16x2(acc[8 * i + 6] * inv, acc[8 * i + 7] * inv));
      }
      if (p.lse) p.lse[((long long)b * p.Hq + h) * p.L + qt * ATT_BM + r] = (m + log2f(l)) * 0.6931471805599453f;
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

// q/k/v: bf16 views whose rows are tokens (b * L + i) with pitch ld_* elements; *_cols = number of columns reachable
// from the base pointer (for the tensor map), *_col0 = column of head 0.  out [B, L, Hq, D], lse [B, Hq, L].
ATS_API int ats_attn_fwd(const void* q, long long ld_q, long long q_cols, int q_col0, const void* k, long long ld_k,
                         long long k_cols, int k_col0, const void* v, long long ld_v, long long v_cols, int v_col0,
                         void* out, float* lse, int B, int L, int Hq, int Hkv, int D, int* status, void* stream) {
  if ((D != 64 && D != 128) || (L % 128) || Hq % Hkv || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7)) return 1003;
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
  AttnArgs p;
  p.B = B; p.L = L; p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse;
  p.scale_log2 = 1.4426950408889634f / sqrtf(float(D));
  p.status = status;
  dim3 grid(Hq, B, L / ATT_BM);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t ce;
  if (D == 128) {
    ce = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<128>::TOTAL);
    if (ce != cudaSuccess) return int(ce);
    attn_fwd_kernel<128><<<grid, ATT_THREADS, AttnSmem<128>::TOTAL, s>>>(mq, mk, mv, p);
  } else {
    ce = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<64>::TOTAL);
    if (ce != cudaSuccess) return int(ce);
    attn_fwd_kernel<64><<<grid, ATT_THREADS, AttnSmem<64>::TOTAL, s>>>(mq, mk, mv, p);
  }
  return int(cudaGetLastError());
}
