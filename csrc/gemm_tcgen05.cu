// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128-byte swizzle) ->
// tcgen05.mma with fp32 accumulators in TMEM -> epilogue from TMEM.
//
//   D[g] (M x N) = alpha * A[g] (M x K) * B[g]^T (N x K)      for every group g
//
// * Either operand may be K-major (reduction index contiguous in global memory) or MN-major (output index
//   contiguous).  Forward linear is K/K, dgrad is K/MN, wgrad is MN/MN, so no transposed copy of an
//   activation or weight is ever materialised.
// * Grouped mode walks `groups` problems that share one pair of tensor maps; per-group coordinate shifts
//   select the expert.  `ragged == 1`: the row count of group g is counts[g] rounded up to 128 (capacity
//   layout [E, C, *], pad rows are zero).  `ragged == 2`: the reduction length is counts[g] rounded up to 128
//   (expert weight gradients).
// * Epilogues: store bf16 | add bf16 C | fp32 store/accumulate | SwiGLU (gate and up halves of the accumulator
//   are combined, optionally also writing the pre-activations for backward).
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue
// (one TMEM lane quadrant each).  Two 256-column accumulators ping-pong so the epilogue of tile i overlaps
// the main loop of tile i+1.  No load in this file uses cluster multicast.
//
// Replaces the cuBLAS calls behind every nn.Linear of the reference (reference core/model.py:686-718,
// 1082-1088, 1229-1240, 1957-1973).
#include "common.cuh"
#include <stdio.h>

namespace ats {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UK = 16;   // K per tcgen05.mma for 16-bit inputs
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_THREADS = 256;  // TMA, MMA, 4 epilogue warps, 2 copy warps (idle unless B is gathered from peers)
constexpr int MAX_GROUPS = 256;
constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + (MAX_GROUPS + 1) * 4;

enum Epilogue : int { kStore = 0, kAddC = 1, kF32 = 2, kSwiGLU = 3, kSwiGLUBwd = 4 };

struct GemmArgs {
  int M, N, K;
  int groups, ragged;
  const int* counts;
  int a_gs_mn, a_gs_k, b_gs_mn, b_gs_k;  // per-group coordinate shifts (elements)
  long long d_gs, c_gs, aux_gs;          // per-group element offsets of D / C / aux
  __nv_bfloat16* D;
  const __nv_bfloat16* C;
  __nv_bfloat16* aux;
  float* Df32;
  int ldd, ldc, ldaux;
  int a_mn, b_mn;        // operand majors: 0 = K-major, 1 = MN-major
  int epilogue;
  int up_offset;         // SwiGLU: row offset of the "up" half inside B (= intermediate size)
  float alpha;
  int beta;              // kF32: accumulate into Df32
  int b_div;             // B operand of group g belongs to weight g / b_div (several token blocks per expert)
  int k_split;           // > 1: group index = problem * k_split + slice; slice s reduces over [s * K, (s + 1) * K) of the problem's
                         // reduction dimension and owns its own D block (fp32 partial products that a small kernel folds)
  int k_segs;            // ragged == 2: the reduction of group g runs over k_segs blocks of rows, seg_stride apart,
  int seg_stride;        //              block s holding counts[g * k_segs + s] rows
  void* const* d_table;  // optional per-group output base pointers (e.g. buffers on peer GPUs)
  // kF32 with scatter_rows > 0: reduce-scatter inside the epilogue.  Row r of the product belongs to rank r / scatter_rows, whose fp32
  // buffer d_table[r / scatter_rows] receives the row at (r % scatter_rows) * ldd with vector atomic adds (`red.add.v4.f32`, which
  // travel over NVLink for rows owned by peers): every rank of a data-parallel group adds its partial weight gradient straight
  // into the owner's gradient shard while the main loop of the next tile runs.
  int scatter_rows;
  // fp8 (e4m3) operands: one byte per element, 128 elements per swizzle row and per K block, kind::f8f6f4 MMAs (K = 32).
  // The fp32 accumulator is multiplied by row_scale[row] * col_scale[col] in the epilogue (per-token activation scales,
  // per-output-channel weight scales), so the main loop needs no per-block promotion.
  // All-gather fused into the GEMM (n_copy != 0): two warps of every CTA pull B, shard by shard, from the GPUs that own it
  // (peer memory) into the local buffer that map_b covers and count every 4 KB piece into b_ready[chunk] (chunks of
  // `ready_rows` rows).  The TMA producer waits (bounded) until the chunks its tile reads are complete (counter >= epoch),
  // and tiles start at the columns of this rank's own shard, which is read in place: each remote byte crosses NVLink once
  // while the tensor cores are already working.
  int n_copy;
  const void* const* b_src;  // [b_shards] base address of every rank's shard
  long long shard_bytes, chunk_bytes;
  uint8_t* b_dst;
  int* b_ready;
  int ready_rows, n_chunks, epoch, first_chunk, n_rot;
  // own chunks whose 128-row box is not entirely inside this rank's shard (a shard of 64-row chunks can begin or end in the
  // middle of a box): they are copied into the staging buffer like remote chunks and their boxes are read from there
  int n_edge, edge_chunk[2];
  int own_row0, own_rows;    // rows of B that live in this rank's shard (read through map_b_own)
  long long* prof;           // optional [8]: cycle totals of CTA 0's MMA thread (total, wait for stage, wait for accumulator, issue, k-blocks)
  // kSwiGLUBwd: the product is dh (gradient of h = silu(gate) * up); `aux` holds the saved pre-activations [gate | up] (read),
  // D receives [dgate | dup] in the same layout and out2 the recomputed h, so dh itself never goes to memory.
  __nv_bfloat16* out2;
  int ldout2;
  long long out2_gs;
  // b_packed: the K-major B operand is stored tile by tile ([weights][N / 128][K / 64][128 rows][64 elements], one 16 KB box
  // contiguous in memory) so that streaming a weight that is read once (decode) touches whole DRAM pages; b_kblocks = K / 64.
  int b_packed, b_kblocks;
  int wide;                // D (and aux) rows are 32-byte aligned at every 16th column: the bf16 epilogues store whole sectors
  int fp8;
  const float* row_scale;  // [groups * rs_gs] or null
  const float* col_scale;  // [weights * cs_gs] or null
  long long rs_gs, cs_gs;
  int* status;
  unsigned long long wait_budget_ns;  // budget of the waits on peers' data (gathered B), set by the host from ats_get_wait_budget_ns()
};

struct TileCoord {
  int g, m0, n0, k_iters, valid;
};

__device__ __forceinline__ int round_up_128(int v) { return (v + 127) & ~127; }

// Rows of D and reduction length of group g.
__device__ __forceinline__ void group_extents(const GemmArgs& p, int g, int& mg, int& kg) {
  mg = p.M;
  kg = p.K;
  if (p.ragged == 1) {
    const int cnt = p.counts[g / p.k_split];
    mg = ATS_DBG_CHECK(cnt >= 0 && cnt <= p.M, kDbgGemmGroups, cnt) ? min(round_up_128(cnt), p.M) : 0;
  }
  if (p.ragged == 2) {
    kg = 0;
    for (int s = 0; s < p.k_segs; ++s) kg += min(round_up_128(p.counts[g * p.k_segs + s]), p.K);
  }
}
__device__ __forceinline__ int seg_iters_of(const GemmArgs& p, int g, int s, int k_iters) {
  if (p.ragged != 2) return k_iters;
  return min(round_up_128(p.counts[g * p.k_segs + s]), p.K) / BK;
}

__device__ __forceinline__ int tiles_n_of(const GemmArgs& p) {
  return p.epilogue == kSwiGLU ? (p.N + 127) / 128 : (p.N + BN - 1) / BN;
}

__device__ __forceinline__ TileCoord decode_tile(const GemmArgs& p, const int* prefix, int tile, int& g_hint, int bm = BM) {
  TileCoord t;
  int g = g_hint;
  while (g + 1 < p.groups && tile >= prefix[g + 1]) ++g;
  g_hint = g;
  int local = tile - prefix[g];
  int tn = tiles_n_of(p);
  int mg, kg;
  group_extents(p, g, mg, kg);
  // Rasterisation: panels of PANEL_N tile columns, rows fastest-varying across panels' columns, so that the ~148
  // tiles in flight touch about as many rows of A as of B (keeps both operands L2-resident per wave).
#ifndef ATS_PANEL_N
#define ATS_PANEL_N 8
#endif
  constexpr int PANEL_N = ATS_PANEL_N;
  const int tm = (mg + bm - 1) / bm;
  const int panel = local / (PANEL_N * tm);
  const int within = local - panel * PANEL_N * tm;
  const int width = min(PANEL_N, tn - panel * PANEL_N);
  const int mt = within / width;
  int nt = panel * PANEL_N + (within - mt * width);
  if (p.n_rot) nt = (nt + p.n_rot) % tn;  // gathered B: begin with the columns whose rows are already local
  t.g = g;
  t.m0 = mt * bm;
  t.n0 = nt * (p.epilogue == kSwiGLU ? 128 : BN);
  const int bk = p.fp8 ? 2 * BK : BK;  // elements per K block (always 128 bytes)
  t.k_iters = (kg + bk - 1) / bk;
  t.valid = mg;
  return t;
}

// Copy warps of a launch that gathers B from its owners: two warps of every CTA pull the remote shards into the local staging
// buffer, 4 KB per warp and step, in the order in which the tiles will need them; consecutive pieces of a chunk go to different
// CTAs, so the ~300 copy warps of the grid keep more than a megabyte in flight on NVLink.  A chunk's counter grows by one per piece.
__device__ __forceinline__ void copy_remote_shards(const GemmArgs& p, int copy_warp, int lane) {
  const long long cps = p.shard_bytes / p.chunk_bytes;
  const long long per_chunk = p.chunk_bytes / 4096;
  const long long total = (long long)(p.n_chunks - cps + p.n_edge) * per_chunk;
  const int own_hi = p.first_chunk + int(cps);
  for (long long i = copy_warp + 2LL * blockIdx.x; i < total; i += 2LL * gridDim.x) {
    const long long ci = i / per_chunk, pi = i - ci * per_chunk;
    // the edge chunks of the own shard first (the first tiles read them), then the remote chunks in the order of the tiles
    const int chunk = ci < p.n_edge ? p.edge_chunk[ci] : int((own_hi + (ci - p.n_edge)) % p.n_chunks);
    const long long off = (chunk % cps) * p.chunk_bytes + pi * 4096 + lane * 16;
    const uint8_t* src = static_cast<const uint8_t*>(p.b_src[chunk / cps]) + off;
    uint8_t* dst = p.b_dst + (long long)chunk * p.chunk_bytes + pi * 4096 + lane * 16;
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = *reinterpret_cast<const uint4*>(src + j * 512);
#pragma unroll
    for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(dst + j * 512) = v[j];
    __threadfence();
    asm volatile("fence.proxy.async;" ::: "memory");  // the tiles are read through the async proxy (TMA)
    __syncwarp();
    if (lane == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.b_ready + chunk) : "memory");
  }
}

// Chunks of gathered B that the calling producer thread already knows to be present (a contiguous range), and the bounded wait for
// one more: returns false when the wait was abandoned.
struct ChunkRange {
  int lo = 0, hi = -1;
};
__device__ __forceinline__ bool wait_chunk(const GemmArgs& p, ChunkRange& r, int c, volatile int* abort_flag) {
  if (c >= p.n_chunks) c = p.n_chunks - 1;
  if (c >= r.lo && c <= r.hi) return true;
  if (c >= p.first_chunk && c < p.first_chunk + int(p.shard_bytes / p.chunk_bytes) &&
      !((p.n_edge > 0 && c == p.edge_chunk[0]) || (p.n_edge > 1 && c == p.edge_chunk[1])))
    return true;  // own shard, whole box inside it: read in place
  const uint64_t t0 = globaltimer_ns();
  int v;
  do {
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.b_ready + c) : "memory");
    if (v >= p.epoch) break;  // epoch = pieces per chunk x number of calls so far
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > p.wait_budget_ns) {
      *abort_flag = 1;
      if (p.status) atomicCAS(p.status, 0, int(kTimeoutPeerFlag));
      return false;
    }
  } while (true);
  if (c == r.hi + 1) r.hi = c;
  else r.lo = r.hi = c;
  asm volatile("fence.proxy.async;" ::: "memory");  // the data was written through the generic proxy of another CTA, TMA reads it
  return true;
}

// Epilogue of one tile for one warp: `taddr` = TMEM address of the accumulator at this warp's lane quadrant, `row_in_tile` =
// the accumulator row (TMEM lane) that this thread owns.
__device__ __forceinline__ void epilogue_tile(const GemmArgs& p, const TileCoord& t, uint32_t taddr, int row_in_tile) {
  const int row = t.m0 + row_in_tile;
  const bool row_ok = row < t.valid;
  const bool have_acc = t.k_iters > 0;
  const float rs = (p.row_scale && row_ok) ? p.row_scale[p.rs_gs * t.g + row] * p.alpha : p.alpha;
  const float* cs = p.col_scale ? p.col_scale + p.cs_gs * (t.g / p.k_split / p.b_div) : nullptr;
  if (p.epilogue == kSwiGLU) {
    __nv_bfloat16* dbase = p.d_table ? static_cast<__nv_bfloat16*>(p.d_table[t.g]) : p.D + p.d_gs * t.g;
    __nv_bfloat16* drow = dbase + (long long)row * p.ldd;
    __nv_bfloat16* arow = p.aux ? p.aux + p.aux_gs * t.g + (long long)row * p.ldaux : nullptr;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t gr[32], ur[32];
      tmem_ld_32x32(taddr + c * 32, gr);
      tmem_ld_32x32(taddr + 128 + c * 32, ur);
      tmem_ld_wait();
      if (p.fp8 == 2) {  // int8 operands: the accumulator columns hold s32
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          gr[i] = __float_as_uint(__int2float_rn(int(gr[i])));
          ur[i] = __float_as_uint(__int2float_rn(int(ur[i])));
        }
      }
      if (row_ok) {
        // eight columns: h, gate and up as four packed bf16 pairs each
        auto piece = [&](int v, int col, uint4& hq, uint4& gq4, uint4& uq4) {
          uint32_t h[4], gg[4], uu[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float g0 = __uint_as_float(gr[v * 8 + 2 * e]) * rs, g1 = __uint_as_float(gr[v * 8 + 2 * e + 1]) * rs;
            float u0 = __uint_as_float(ur[v * 8 + 2 * e]) * rs, u1 = __uint_as_float(ur[v * 8 + 2 * e + 1]) * rs;
            if (cs) {
              g0 *= cs[col + 2 * e];
              g1 *= cs[col + 2 * e + 1];
              u0 *= cs[p.up_offset + col + 2 * e];
              u1 *= cs[p.up_offset + col + 2 * e + 1];
            }
            gg[e] = pack_bf16x2(g0, g1);
            uu[e] = pack_bf16x2(u0, u1);
            // activation on the bf16-rounded values so a separate SwiGLU pass gives identical bits
            float2 gq = unpack_bf16x2(gg[e]), uq = unpack_bf16x2(uu[e]);
            h[e] = pack_bf16x2(silu_f(gq.x) * uq.x, silu_f(gq.y) * uq.y);
          }
          hq = make_uint4(h[0], h[1], h[2], h[3]);
          gq4 = make_uint4(gg[0], gg[1], gg[2], gg[3]);
          uq4 = make_uint4(uu[0], uu[1], uu[2], uu[3]);
        };
        if (p.wide) {
#pragma unroll
          for (int v = 0; v < 4; v += 2) {
            const int col = t.n0 + c * 32 + v * 8;
            if (col + 16 <= p.N) {
              uint4 h0, g0, u0, h1, g1, u1;
              piece(v, col, h0, g0, u0);
              piece(v + 1, col + 8, h1, g1, u1);
              st_global_32B(drow + col, h0, h1);
              if (arow) {
                st_global_32B(arow + col, g0, g1);
                st_global_32B(arow + p.up_offset + col, u0, u1);
              }
            } else if (col < p.N) {
              uint4 h0, g0, u0;
              piece(v, col, h0, g0, u0);
              *reinterpret_cast<uint4*>(drow + col) = h0;
              if (arow) {
                *reinterpret_cast<uint4*>(arow + col) = g0;
                *reinterpret_cast<uint4*>(arow + p.up_offset + col) = u0;
              }
            }
          }
        } else {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = t.n0 + c * 32 + v * 8;
            if (col < p.N) {
              uint4 h0, g0, u0;
              piece(v, col, h0, g0, u0);
              *reinterpret_cast<uint4*>(drow + col) = h0;
              if (arow) {
                *reinterpret_cast<uint4*>(arow + col) = g0;
                *reinterpret_cast<uint4*>(arow + p.up_offset + col) = u0;
              }
            }
          }
        }
      }
    }
  } else if (p.epilogue == kSwiGLUBwd) {
    __nv_bfloat16* dbase = p.D + p.d_gs * t.g + (long long)row * p.ldd;
    const __nv_bfloat16* arow = p.aux + p.aux_gs * t.g + (long long)row * p.ldaux;
    __nv_bfloat16* hrow = p.out2 ? p.out2 + p.out2_gs * t.g + (long long)row * p.ldout2 : nullptr;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint4 g[4], u[4];  // the chunk's 32 gate and 32 up values, requested before the accumulator is read
      if (p.wide && row_ok) {
#pragma unroll
        for (int v = 0; v < 4; v += 2) {
          const int col = t.n0 + c * 32 + v * 8;
          if (col + 16 <= p.N) {
            ld_global_32B(arow + col, g[v], g[v + 1]);
            ld_global_32B(arow + p.up_offset + col, u[v], u[v + 1]);
          } else if (col < p.N) {
            g[v] = *reinterpret_cast<const uint4*>(arow + col);
            u[v] = *reinterpret_cast<const uint4*>(arow + p.up_offset + col);
          }
        }
      }
      uint32_t r[32];
      if (have_acc) {
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0;
      }
      if (!row_ok) continue;
      // eight columns from the saved gate / up values and the accumulator
      auto piece = [&](int v, const uint4& gq, const uint4& uq, uint4& og4, uint4& ou4, uint4& oh4) {
        const uint32_t gg[4] = {gq.x, gq.y, gq.z, gq.w}, uu[4] = {uq.x, uq.y, uq.z, uq.w};
        uint32_t og[4], ou[4], oh[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // dh rounded to bf16 first: bit-identical to writing dh and running the separate backward kernel
          const float2 d = unpack_bf16x2(pack_bf16x2(__uint_as_float(r[v * 8 + 2 * e]) * rs, __uint_as_float(r[v * 8 + 2 * e + 1]) * rs));
          const float2 a = unpack_bf16x2(gg[e]), b = unpack_bf16x2(uu[e]);
          const float s0 = 1.f / (1.f + __expf(-a.x)), s1 = 1.f / (1.f + __expf(-a.y));
          const float si0 = a.x * s0, si1 = a.y * s1;
          og[e] = pack_bf16x2(d.x * b.x * (s0 + si0 * (1.f - s0)), d.y * b.y * (s1 + si1 * (1.f - s1)));
          ou[e] = pack_bf16x2(d.x * si0, d.y * si1);
          oh[e] = pack_bf16x2(si0 * b.x, si1 * b.y);
        }
        og4 = make_uint4(og[0], og[1], og[2], og[3]);
        ou4 = make_uint4(ou[0], ou[1], ou[2], ou[3]);
        oh4 = make_uint4(oh[0], oh[1], oh[2], oh[3]);
      };
      if (p.wide) {
#pragma unroll
        for (int v = 0; v < 4; v += 2) {
          const int col = t.n0 + c * 32 + v * 8;
          uint4 a0, b0, c0, a1, b1, c1;
          if (col + 16 <= p.N) {
            piece(v, g[v], u[v], a0, b0, c0);
            piece(v + 1, g[v + 1], u[v + 1], a1, b1, c1);
            st_global_32B(dbase + col, a0, a1);
            st_global_32B(dbase + p.up_offset + col, b0, b1);
            if (hrow) st_global_32B(hrow + col, c0, c1);
          } else if (col < p.N) {
            piece(v, g[v], u[v], a0, b0, c0);
            *reinterpret_cast<uint4*>(dbase + col) = a0;
            *reinterpret_cast<uint4*>(dbase + p.up_offset + col) = b0;
            if (hrow) *reinterpret_cast<uint4*>(hrow + col) = c0;
          }
        }
      } else {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int col = t.n0 + c * 32 + v * 8;
          if (col < p.N) {
            uint4 a0, b0, c0;
            piece(v, *reinterpret_cast<const uint4*>(arow + col), *reinterpret_cast<const uint4*>(arow + p.up_offset + col), a0, b0, c0);
            *reinterpret_cast<uint4*>(dbase + col) = a0;
            *reinterpret_cast<uint4*>(dbase + p.up_offset + col) = b0;
            if (hrow) *reinterpret_cast<uint4*>(hrow + col) = c0;
          }
        }
      }
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      if (have_acc) {
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (p.fp8 == 2) {  // int8 operands: the accumulator columns hold s32
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__int2float_rn(int(r[i])));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0;
      }
      if (!row_ok) continue;
      const int colbase = t.n0 + c * 32;
      if (p.epilogue == kF32 && p.scatter_rows > 0) {
        const int owner = row / p.scatter_rows;
        float* drow = static_cast<float*>(p.d_table[owner]) + (long long)(row - owner * p.scatter_rows) * p.ldd;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const int col = colbase + v * 4;
          if (col < p.N)
            asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(drow + col), "f"(__uint_as_float(r[v * 4]) * p.alpha),
                         "f"(__uint_as_float(r[v * 4 + 1]) * p.alpha), "f"(__uint_as_float(r[v * 4 + 2]) * p.alpha),
                         "f"(__uint_as_float(r[v * 4 + 3]) * p.alpha)
                         : "memory");
        }
      } else if (p.epilogue == kF32) {
        float* drow = p.Df32 + p.d_gs * t.g + (long long)row * p.ldd;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const int col = colbase + v * 4;
          if (col < p.N) {
            // rs = alpha (x the row scale of an 8-bit product); cs = its column scales: both distribute over the sum of the slices
            float4 o = make_float4(__uint_as_float(r[v * 4]) * rs, __uint_as_float(r[v * 4 + 1]) * rs,
                                   __uint_as_float(r[v * 4 + 2]) * rs, __uint_as_float(r[v * 4 + 3]) * rs);
            if (cs) {
              const float4 c4 = *reinterpret_cast<const float4*>(cs + col);
              o.x *= c4.x; o.y *= c4.y; o.z *= c4.z; o.w *= c4.w;
            }
            if (p.beta) {
              float4 old = *reinterpret_cast<float4*>(drow + col);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(drow + col) = o;
          }
        }
      } else {
        __nv_bfloat16* dbase = p.d_table ? static_cast<__nv_bfloat16*>(p.d_table[t.g]) : p.D + p.d_gs * t.g;
        __nv_bfloat16* drow = dbase + (long long)row * p.ldd;
        const __nv_bfloat16* crow =
            p.epilogue == kAddC ? p.C + p.c_gs * t.g + (long long)row * p.ldc : nullptr;
        auto piece = [&](int v, int col, const uint4& cv) -> uint4 {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * rs;
          if (cs) {
            const float4 c0 = *reinterpret_cast<const float4*>(cs + col), c1 = *reinterpret_cast<const float4*>(cs + col + 4);
            f[0] *= c0.x; f[1] *= c0.y; f[2] *= c0.z; f[3] *= c0.w;
            f[4] *= c1.x; f[5] *= c1.y; f[6] *= c1.z; f[7] *= c1.w;
          }
          if (crow) {
            float2 c0 = unpack_bf16x2(cv.x), c1 = unpack_bf16x2(cv.y), c2 = unpack_bf16x2(cv.z), c3 = unpack_bf16x2(cv.w);
            f[0] += c0.x; f[1] += c0.y; f[2] += c1.x; f[3] += c1.y;
            f[4] += c2.x; f[5] += c2.y; f[6] += c3.x; f[7] += c3.y;
          }
          return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        };
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        if (p.wide) {
#pragma unroll
          for (int v = 0; v < 4; v += 2) {
            const int col = colbase + v * 8;
            if (col + 16 <= p.N) {
              uint4 c0 = zero4, c1 = zero4;
              if (crow) ld_global_32B(crow + col, c0, c1);
              st_global_32B(drow + col, piece(v, col, c0), piece(v + 1, col + 8, c1));
            } else if (col < p.N) {
              *reinterpret_cast<uint4*>(drow + col) = piece(v, col, crow ? *reinterpret_cast<const uint4*>(crow + col) : zero4);
            }
          }
        } else {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = colbase + v * 8;
            if (col < p.N) *reinterpret_cast<uint4*>(drow + col) = piece(v, col, crow ? *reinterpret_cast<const uint4*>(crow + col) : zero4);
          }
        }
      }
    }
  }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_b_own, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_prologue();  // decode-sized products are launched programmatically dependent on the kernel before them
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + STAGES;          // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;      // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* prefix = reinterpret_cast<int*>(smem + STAGES * STAGE_BYTES + 256);  // [groups + 1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    // tile prefix sums (groups is small)
    int acc = 0;
    int tn = tiles_n_of(p);
    for (int g = 0; g < p.groups; ++g) {
      prefix[g] = acc;
      int mg, kg;
      group_extents(p, g, mg, kg);
      acc += ((mg + BM - 1) / BM) * tn;
    }
    prefix[p.groups] = acc;
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.n_copy) tma_prefetch_desc(&map_b_own);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = prefix[p.groups];
  const int first_tile = int(blockIdx.x);
  const int tile_step = int(gridDim.x);

  if (warp >= 6) {
    // ------------------------------------------------------------------ copy warps (gathered B only)
    // Two warps of every CTA pull the remote shards of B into the local staging buffer, 4 KB per warp and step, in the
    // order in which the tiles will need them; consecutive pieces of a chunk go to different CTAs, so the ~300 copy
    // warps of the grid keep more than a megabyte in flight on NVLink.  A chunk's counter grows by one per piece.
    if (p.n_copy) copy_remote_shards(p, warp - 6, lane);
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0, phase = 0, g_hint = 0;
      uint32_t armed = 0, armed_phase = 0;
      bool ok = true;
      ChunkRange ready;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        TileCoord t = decode_tile(p, prefix, tile, g_hint);
        if (p.n_copy) {
          const int r0 = t.n0, r1 = p.epilogue == kSwiGLU ? t.n0 + p.up_offset : t.n0 + 128;
          ok = wait_chunk(p, ready, r0 / p.ready_rows, abort_flag) && wait_chunk(p, ready, (r0 + 127) / p.ready_rows, abort_flag) &&
               wait_chunk(p, ready, r1 / p.ready_rows, abort_flag) && wait_chunk(p, ready, (r1 + 127) / p.ready_rows, abort_flag);
          if (!ok) break;
        }
        const int ge = t.g / p.k_split, k_off = (t.g - ge * p.k_split) * p.K;  // problem and reduction slice of this group
        const int a_mn_c = t.m0 + p.a_gs_mn * ge, a_k_c = p.a_gs_k * ge + k_off;
        const int gb = ge / p.b_div;
        const int b_mn_c = t.n0 + p.b_gs_mn * gb, b_k_c = p.b_gs_k * gb + k_off;
        int seg = 0, seg_left = seg_iters_of(p, t.g, 0, t.k_iters), kpos = 0;
        for (int kb = 0; kb < t.k_iters; ++kb) {
          while (seg_left == 0) {
            ++seg;
            seg_left = seg_iters_of(p, t.g, seg, t.k_iters);
            kpos = 0;
          }
          if (!mbar_wait_bounded(&empty[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmpty)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (uint32_t(phase) << stage);
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
          const int k0 = seg * p.seg_stride + kpos * (p.fp8 ? 2 * BK : BK);
          ++kpos;
          --seg_left;
          if (!p.a_mn) {
            tma_load_2d(a_dst, &map_a, &full[stage], a_k_c + k0, a_mn_c);  // box 64 x 128
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)  // box 64 (MN) x 64 (K rows)
              tma_load_2d(a_dst + j * (BK * 128), &map_a, &full[stage], a_mn_c + 64 * j, a_k_c + k0);
          }
          if (!p.b_mn) {
            // two boxes of 64 x 128 rows; SwiGLU takes the second from the "up" half
            const int second = p.epilogue == kSwiGLU ? b_mn_c + p.up_offset : b_mn_c + 128;
            if (p.n_copy) {
              // gathered B: rows of this rank's own shard are read in place, the others from the staging buffer
              const int o0 = b_mn_c - p.own_row0, o1 = second - p.own_row0;
              if (o0 >= 0 && o0 + 128 <= p.own_rows) tma_load_2d(b_dst, &map_b_own, &full[stage], k0, o0);
              else tma_load_2d(b_dst, &map_b, &full[stage], k0, b_mn_c);
              if (o1 >= 0 && o1 + 128 <= p.own_rows) tma_load_2d(b_dst + 128 * 128, &map_b_own, &full[stage], k0, o1);
              else tma_load_2d(b_dst + 128 * 128, &map_b, &full[stage], k0, second);
            } else if (p.b_packed) {
              const int kb_idx = (k0 + k_off) >> 6;
              tma_load_2d(b_dst, &map_b, &full[stage], 0, ((b_mn_c >> 7) * p.b_kblocks + kb_idx) << 7);
              tma_load_2d(b_dst + 128 * 128, &map_b, &full[stage], 0, ((second >> 7) * p.b_kblocks + kb_idx) << 7);
            } else {
              tma_load_2d(b_dst, &map_b, &full[stage], b_k_c + k0, b_mn_c);
              tma_load_2d(b_dst + 128 * 128, &map_b, &full[stage], b_k_c + k0, second);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * (BK * 128), &map_b, &full[stage], b_mn_c + 64 * j, b_k_c + k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // let copies that were already issued land before the CTA gives its shared memory back
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed >> s & 1)) continue;
          uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full[s], (armed_phase >> s) & 1) && globaltimer_ns() - t0 < 10000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = p.fp8 == 2 ? make_idesc_i8(BM, BN)           // s8 x s8 -> s32, both K-major
                             : p.fp8 ? make_idesc(BM, BN, 0, 0, 0, 0)   // e4m3 x e4m3, both K-major
                                     : make_idesc(BM, BN, 1, 1, p.a_mn, p.b_mn);
      int stage = 0, phase = 0, acc = 0, acc_phase = 0, g_hint = 0;
      bool ok = true;
      // K-major operand: 32 bytes per MMA along the swizzle row; MN-major: 16 K-rows of 128 bytes per MMA
      const uint64_t a_desc0 = p.a_mn ? make_smem_desc_sw128(smem_u32(sA), BK * 128, 1024) : make_smem_desc_sw128(smem_u32(sA), 16, 1024);
      const uint64_t b_desc0 = p.b_mn ? make_smem_desc_sw128(smem_u32(sB), BK * 128, 1024) : make_smem_desc_sw128(smem_u32(sB), 16, 1024);
      const uint64_t a_step16 = (p.a_mn ? UK * 128 : UK * 2) >> 4, b_step16 = (p.b_mn ? UK * 128 : UK * 2) >> 4;
      const bool rec = p.prof != nullptr && blockIdx.x == 0;
      long long w_full = 0, w_acc = 0, t_issue = 0, n_kb = 0, c0 = 0, c1 = 0;
      const long long t_begin = clock64();
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        TileCoord t = decode_tile(p, prefix, tile, g_hint);
        if (rec) c0 = clock64();
        if (!mbar_wait_bounded(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
        if (rec) { c1 = clock64(); w_acc += c1 - c0; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_iters; ++kb) {
          if (rec) c0 = clock64();
          if (!mbar_wait_bounded(&full[stage], phase, abort_flag, p.status, kTimeoutFull)) {
            ok = false;
            break;
          }
          if (rec) { c1 = clock64(); w_full += c1 - c0; ++n_kb; }
          tc_fence_after();
          // descriptors: one base per operand (built before the tile loop), advanced by constants
          const uint64_t adesc = desc_advance(a_desc0, uint32_t(stage) * A_STAGE_BYTES);
          const uint64_t bdesc = desc_advance(b_desc0, uint32_t(stage) * B_STAGE_BYTES);
          if (p.fp8) {
            if (p.fp8 == 2) {
#pragma unroll
              for (int k = 0; k < BK / UK; ++k) tc_mma_i8(d_tmem, adesc + k * a_step16, bdesc + k * b_step16, idesc, (kb | k) != 0);
            } else {
#pragma unroll
              for (int k = 0; k < BK / UK; ++k) tc_mma_f8(d_tmem, adesc + k * a_step16, bdesc + k * b_step16, idesc, (kb | k) != 0);
            }
          } else {
#pragma unroll
            for (int k = 0; k < BK / UK; ++k) tc_mma_f16(d_tmem, adesc + k * a_step16, bdesc + k * b_step16, idesc, (kb | k) != 0);
          }
          tc_commit(&empty[stage]);  // the stage is free once these MMAs have read it
          if (rec) t_issue += clock64() - c1;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (t.k_iters > 0) tc_commit(&tfull[acc]);
        else mbar_arrive(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (rec) {
        p.prof[0] = clock64() - t_begin; p.prof[1] = w_full; p.prof[2] = w_acc; p.prof[3] = t_issue; p.prof[4] = n_kb;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0, acc_phase = 0, g_hint = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step) {
      TileCoord t = decode_tile(p, prefix, tile, g_hint);
      if (!mbar_wait_bounded(&tfull[acc], acc_phase, abort_flag, p.status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quad * 32) << 16);
      epilogue_tile(p, t, taddr, row_in_tile);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
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

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (two SMs) works on one 256 x 256 tile with `tcgen05.mma.cta_group::2`.
// Each CTA stages its own 128 rows of A and only HALF of the B tile (128 of the 256 rows), so a pair pulls 64 KB per
// k-block from L2 where two independent CTAs pull 96 KB, and a stage is 32 KB, which makes room for six stages.
// One thread of the leader CTA (cluster rank 0) issues every MMA; both CTAs hold their 128 accumulator rows in
// their own TMEM and run their own epilogue.
//
//   full[s]   leader's barrier: its producer arrives with the byte count of BOTH CTAs, the loads of both CTAs
//             (`.cta_group::2`, no multicast) complete on it
//   empty[s]  one per CTA: freed by the leader's commit, delivered to both CTAs
//   tfull[a]  one per CTA: accumulator ready (same commit form)
//   tempty[a] leader's barrier: the epilogue warps of both CTAs arrive (the partner's through its cluster address)
// ------------------------------------------------------------------------------------------------
constexpr int PAIR_BM = 2 * BM;
#ifndef ATS_PAIR_STAGES
#define ATS_PAIR_STAGES 6
#endif
constexpr int PAIR_STAGES = ATS_PAIR_STAGES;
constexpr int PAIR_B_STAGE_BYTES = (BN / 2) * BK * 2;
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_STAGE_BYTES;
constexpr int PAIR_THREADS = 192;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 + (MAX_GROUPS + 1) * 4;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS + 64, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_b_own, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + PAIR_STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
  uint64_t* full = bars;                         // [PAIR_STAGES]
  uint64_t* empty = bars + PAIR_STAGES;          // [PAIR_STAGES]
  uint64_t* tfull = bars + 2 * PAIR_STAGES;      // [2]
  uint64_t* tempty = bars + 2 * PAIR_STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PAIR_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* prefix = reinterpret_cast<int*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES + 256);  // [groups + 1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = leader

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 8);  // four epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    int acc = 0;
    const int tn = tiles_n_of(p);
    for (int g = 0; g < p.groups; ++g) {
      prefix[g] = acc;
      int mg, kg;
      group_extents(p, g, mg, kg);
      acc += ((mg + PAIR_BM - 1) / PAIR_BM) * tn;
    }
    prefix[p.groups] = acc;
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.n_copy) tma_prefetch_desc(&map_b_own);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = prefix[p.groups];
  const int first_tile = int(cluster_id_x());
  const int tile_step = int(cluster_count_x());

  if (warp >= 6) {
    // ------------------------------------------------------------------ copy warps (launches that gather B from its owners)
    if (p.n_copy) copy_remote_shards(p, warp - 6, lane);
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0, phase = 0, g_hint = 0;
      bool ok = true;
      ChunkRange ready;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        TileCoord t = decode_tile(p, prefix, tile, g_hint, PAIR_BM);
        const int ge = t.g / p.k_split, k_off = (t.g - ge * p.k_split) * p.K;  // problem and reduction slice of this group
        const int a_mn_c = t.m0 + int(rank) * BM + p.a_gs_mn * ge, a_k_c = p.a_gs_k * ge + k_off;
        const int gb = ge / p.b_div;
        const int b_k_c = p.b_gs_k * gb + k_off;
        // this CTA's half of the B tile: rows n0 .. n0+127 for the leader, the next 128 (SwiGLU: the "up" rows) for the partner
        const int b_mn_c = t.n0 + p.b_gs_mn * gb + (rank ? (p.epilogue == kSwiGLU ? p.up_offset : 128) : 0);
        const CUtensorMap* bmap = &map_b;
        int b_row = b_mn_c;
        if (p.n_copy) {
          // gathered B: rows of this rank's own shard are read in place, the others from the staging buffer once they are there
          ok = wait_chunk(p, ready, b_mn_c / p.ready_rows, abort_flag) && wait_chunk(p, ready, (b_mn_c + 127) / p.ready_rows, abort_flag);
          if (!ok) break;
          const int o = b_mn_c - p.own_row0;
          if (o >= 0 && o + 128 <= p.own_rows) {  // the whole box lies in this rank's shard
            bmap = &map_b_own;
            b_row = o;
          }
        }
        int seg = 0, seg_left = seg_iters_of(p, t.g, 0, t.k_iters), kpos = 0;
        for (int kb = 0; kb < t.k_iters; ++kb) {
          while (seg_left == 0) {
            ++seg;
            seg_left = seg_iters_of(p, t.g, seg, t.k_iters);
            kpos = 0;
          }
          if (!mbar_wait_bounded(&empty[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmpty)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * PAIR_STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
          uint8_t* b_dst = sB + stage * PAIR_B_STAGE_BYTES;
          const int k0 = seg * p.seg_stride + kpos * (p.fp8 ? 2 * BK : BK);
          ++kpos;
          --seg_left;
          if (!p.a_mn) {
            tma_load_2d_pair(a_dst, &map_a, bar, a_k_c + k0, a_mn_c);  // box 64 x 128
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)  // box 64 (MN) x 64 (K rows)
              tma_load_2d_pair(a_dst + j * (BK * 128), &map_a, bar, a_mn_c + 64 * j, a_k_c + k0);
          }
          if (!p.b_mn) {
            if (p.b_packed) tma_load_2d_pair(b_dst, bmap, bar, 0, ((b_row >> 7) * p.b_kblocks + ((k0 + k_off) >> 6)) << 7);
            else tma_load_2d_pair(b_dst, bmap, bar, b_k_c + k0, b_row);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tma_load_2d_pair(b_dst + j * (BK * 128), &map_b, bar, b_mn_c + 64 * j, b_k_c + k0);
          }
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // a wait ran out: give the copies issued last time to land before this CTA's shared memory goes away
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = p.fp8 == 2 ? make_idesc_i8(PAIR_BM, BN)
                             : p.fp8 ? make_idesc(PAIR_BM, BN, 0, 0, 0, 0) : make_idesc(PAIR_BM, BN, 1, 1, p.a_mn, p.b_mn);
      int stage = 0, phase = 0, acc = 0, acc_phase = 0, g_hint = 0;
      bool ok = true;
      const uint64_t a_desc0 = p.a_mn ? make_smem_desc_sw128(smem_u32(sA), BK * 128, 1024) : make_smem_desc_sw128(smem_u32(sA), 16, 1024);
      const uint64_t b_desc0 = p.b_mn ? make_smem_desc_sw128(smem_u32(sB), BK * 128, 1024) : make_smem_desc_sw128(smem_u32(sB), 16, 1024);
      const uint64_t a_step16 = (p.a_mn ? UK * 128 : UK * 2) >> 4, b_step16 = (p.b_mn ? UK * 128 : UK * 2) >> 4;
      const bool rec = p.prof != nullptr && blockIdx.x == 0;
      long long w_full = 0, w_acc = 0, t_issue = 0, n_kb = 0, c0 = 0, c1 = 0;
      const long long t_begin = clock64();
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        TileCoord t = decode_tile(p, prefix, tile, g_hint, PAIR_BM);
        if (rec) c0 = clock64();
        if (!mbar_wait_bounded(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
        if (rec) { c1 = clock64(); w_acc += c1 - c0; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_iters; ++kb) {
          if (rec) c0 = clock64();
          if (!mbar_wait_bounded(&full[stage], phase, abort_flag, p.status, kTimeoutFull)) {
            ok = false;
            break;
          }
          if (rec) { c1 = clock64(); w_full += c1 - c0; ++n_kb; }
          tc_fence_after();
          const uint64_t adesc = desc_advance(a_desc0, uint32_t(stage) * A_STAGE_BYTES);
          const uint64_t bdesc = desc_advance(b_desc0, uint32_t(stage) * PAIR_B_STAGE_BYTES);
          if (p.fp8) {
            if (p.fp8 == 2) {
#pragma unroll
              for (int k = 0; k < BK / UK; ++k) tc_mma_i8_pair(d_tmem, adesc + k * a_step16, bdesc + k * b_step16, idesc, (kb | k) != 0);
            } else {
#pragma unroll
              for (int k = 0; k < BK / UK; ++k) tc_mma_f8_pair(d_tmem, adesc + k * a_step16, bdesc + k * b_step16, idesc, (kb | k) != 0);
            }
          } else {
#pragma unroll
            for (int k = 0; k < BK / UK; ++k) tc_mma_f16_pair(d_tmem, adesc + k * a_step16, bdesc + k * b_step16, idesc, (kb | k) != 0);
          }
          tc_commit_pair(&empty[stage], 3);  // both CTAs get their stage back once these MMAs have read it
          if (rec) t_issue += clock64() - c1;
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (t.k_iters > 0) {
          tc_commit_pair(&tfull[acc], 3);
        } else {
          mbar_arrive(&tfull[acc]);
          mbar_arrive_cluster(mapa_shared(smem_u32(&tfull[acc]), 1));
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (rec) {
        p.prof[0] = clock64() - t_begin; p.prof[1] = w_full; p.prof[2] = w_acc; p.prof[3] = t_issue; p.prof[4] = n_kb;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0, acc_phase = 0, g_hint = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step) {
      TileCoord t = decode_tile(p, prefix, tile, g_hint, PAIR_BM);
      t.m0 += int(rank) * BM;
      if (!mbar_wait_bounded(&tfull[acc], acc_phase, abort_flag, p.status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quad * 32) << 16);
      epilogue_tile(p, t, taddr, row_in_tile);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // Neither CTA may leave (or give TMEM back) while its partner can still signal its barriers or read its shared memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------------
EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, int elem_bytes,
                 uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return 1000;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * elem_bytes) & 15)) return 1001;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1100 + int(r);
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

}  // namespace ats

using namespace ats;

ATS_API unsigned long long ats_get_wait_budget_ns();  // comm.cu
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& p, int epilogue, int groups, int M, int N,
                       int max_ctas, void* stream, const CUtensorMap* mb_own = nullptr);
static long long* g_gemm_prof = nullptr;

// Diagnostics: device buffer of 8 int64 that the next bf16 GEMM launches fill with cycle totals of CTA 0's MMA thread
// (total, wait for a loaded stage, wait for a free accumulator, issue, k-blocks); null switches it off.
ATS_API void ats_gemm_set_profile(long long* buf) { g_gemm_prof = buf; }
// 1 (default): bf16 products with at least 256 rows run on CTA pairs (cta_group::2); 0: one CTA per 128 x 256 tile everywhere.
static int g_gemm_pair = 1;
// 1 (default): bf16 epilogues write 32 bytes per store where the output layout allows it; 0: 16-byte stores everywhere.
static int g_gemm_wide = 1;
ATS_API void ats_gemm_set_wide_stores(int on) { g_gemm_wide = on; }
ATS_API void ats_gemm_set_pair(int on) { g_gemm_pair = on; }

// Generic entry point. The global 2-D extents of both operands are given explicitly (rows x cols, cols contiguous,
// pitch ld elements); for a K-major operand cols is the reduction dimension, for an MN-major operand rows is.
// Returns 0 or an error code (>= 1000: tensor-map encode, otherwise cudaError_t of the launch).
ATS_API int ats_gemm_bf16(const void* A, long long a_rows, long long a_cols, long long lda, int a_mn,
                          const void* B, long long b_rows, long long b_cols, long long ldb, int b_mn,
                          void* D, int ldd, const void* C, int ldc, void* aux, int ldaux,
                          int M, int N, int K, float alpha, int beta, int epilogue, int up_offset,
                          int groups, int ragged, const int* counts,
                          int a_gs_mn, int a_gs_k, int b_gs_mn, int b_gs_k,
                          long long d_gs, long long c_gs, long long aux_gs,
                          int b_div, int k_segs, int seg_stride, void* const* d_table, int k_split, int scatter_rows,
                          int* status, int max_ctas, void* stream) {
  // The tensor-map encoder is a driver call: make sure this thread (autograd runs backward on its own threads)
  // has the primary context bound before the first use.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  if (groups < 1 || groups > MAX_GROUPS) return 1002;
  if ((N & 7) || (a_gs_mn & 7) || (a_gs_k & 7) || (b_gs_mn & 7) || (b_gs_k & 7) || (ldd & 7) || (d_gs & 7)) return 1003;
  const int b_packed = b_mn == 2 ? 1 : 0;  // K-major, stored tile by tile (see GemmArgs::b_packed)
  if (b_packed) {
    b_mn = 0;
    if ((b_rows & 127) || (b_cols & 63) || (b_gs_mn & 127) || b_gs_k || ragged == 2 || (epilogue == kSwiGLU && (up_offset & 127))) return 1007;
  }
  if (epilogue == kSwiGLU && (b_mn || (up_offset & 7))) return 1004;
  if (ragged && !counts) return 1005;
  if (b_div < 1 || k_segs < 1 || (seg_stride & 7) || (k_segs > 1 && ragged != 2)) return 1006;
  // reduction slices: whole K blocks per slice, fp32 partial outputs, every `k_split` consecutive groups are one problem
  if (k_split < 1 || (k_split > 1 && (epilogue != kF32 || ragged == 2 || (K & 63) || groups % k_split || d_table))) return 1008;
  // reduce-scatter epilogue: one problem, fp32 atomic adds into per-owner buffers, whole 16-byte vectors
  if (scatter_rows < 0 || (scatter_rows > 0 && (epilogue != kF32 || groups != 1 || !d_table || (N & 3) || (ldd & 3) || M % scatter_rows))) return 1009;
  CUtensorMap ma, mb;
  int e;
  if ((e = make_tmap_2d(&ma, A, a_rows, a_cols, lda, 2, 64, a_mn ? 64 : 128))) return e;
  if (b_packed) {
    if ((e = make_tmap_2d(&mb, B, (uint64_t)b_rows * (uint64_t)(b_cols / 64), 64, 64, 2, 64, 128))) return e;
  } else if ((e = make_tmap_2d(&mb, B, b_rows, b_cols, ldb, 2, 64, b_mn ? 64 : 128))) {
    return e;
  }
  GemmArgs p;
  p.b_packed = b_packed; p.b_kblocks = int(b_cols / 64);
  p.M = M; p.N = N; p.K = K; p.groups = groups; p.ragged = ragged; p.counts = counts;
  p.a_gs_mn = a_gs_mn; p.a_gs_k = a_gs_k; p.b_gs_mn = b_gs_mn; p.b_gs_k = b_gs_k;
  p.d_gs = d_gs; p.c_gs = c_gs; p.aux_gs = aux_gs;
  p.D = static_cast<__nv_bfloat16*>(D); p.C = static_cast<const __nv_bfloat16*>(C);
  p.aux = static_cast<__nv_bfloat16*>(aux); p.Df32 = static_cast<float*>(D);
  p.ldd = ldd; p.ldc = ldc; p.ldaux = ldaux; p.a_mn = a_mn; p.b_mn = b_mn; p.epilogue = epilogue;
  p.up_offset = up_offset; p.alpha = alpha; p.beta = beta; p.status = status;
  p.b_div = b_div; p.k_segs = k_segs; p.seg_stride = seg_stride; p.d_table = d_table; p.k_split = k_split; p.scatter_rows = scatter_rows;
  p.fp8 = 0; p.row_scale = nullptr; p.col_scale = nullptr; p.rs_gs = 0; p.cs_gs = 0;
  p.n_copy = 0; p.n_rot = 0; p.own_row0 = 0; p.own_rows = 0; p.prof = g_gemm_prof;
  p.n_edge = 0; p.edge_chunk[0] = p.edge_chunk[1] = -1;
  p.out2 = nullptr; p.ldout2 = 0; p.out2_gs = 0;
  if (epilogue == kSwiGLUBwd) {
    // second output (h) travels in the C slot of this entry point: C / ldc / c_gs
    if (!aux || (up_offset & 7) || (ldaux & 7)) return 1004;
    p.out2 = static_cast<__nv_bfloat16*>(const_cast<void*>(C)); p.ldout2 = ldc; p.out2_gs = c_gs;
    p.C = nullptr;
  }
  return launch_gemm(ma, mb, p, epilogue, groups, M, N, max_ctas, stream);
}

// Fold of the fp32 partial products that reduction slices leave (k_split > 1, or the dense form with one group per slice):
// out[o, i] = sum_s part[(o * splits + s) * n_inner + i] (+ add[o, i]) as bf16, i < n_inner (a multiple of 8), o < n_outer.
namespace ats {
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int splits, long long n_inner, long long n_outer,
                                                            __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ add) {
  pdl_prologue();
  const long long nvec = n_inner >> 3, total = nvec * n_outer;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const long long o = v / nvec, i = (v - o * nvec) << 3;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (add) {
      const uint4 a = *reinterpret_cast<const uint4*>(add + o * n_inner + i);
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
    }
    const float* src = part + (o * splits) * n_inner + i;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 a = *reinterpret_cast<const float4*>(src + s * n_inner), b = *reinterpret_cast<const float4*>(src + s * n_inner + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    *reinterpret_cast<uint4*>(out + o * n_inner + i) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}
}  // namespace ats

ATS_API int ats_splitk_reduce(const float* part, int splits, long long n_inner, long long n_outer, void* out, const void* add, void* stream) {
  if (splits < 1 || n_inner <= 0 || n_outer <= 0 || (n_inner & 7)) return 1003;
  long long blocks = ((n_inner >> 3) * n_outer + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaError_t ce = launch_pdl(splitk_reduce_kernel, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream), part, splits,
                              n_inner, n_outer, static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(add));
  return int(ce != cudaSuccess ? ce : cudaGetLastError());
}

// fp8 (e4m3) A [groups x M, K] and B [weights x N, K], both K-major and row-quantised: D = (A_q B_q^T) * row_scale * col_scale.
// a_gs_mn / b_gs_mn: row shift per group / per weight inside the 2-D operand; rs_gs / cs_gs: scale offsets per group / weight.
// Epilogues: store, +C, SwiGLU (up_offset as in the bf16 entry).  ragged: 0, or 1 with per-group row counts.
static int gemm_8bit(int kind, const void* A, long long a_rows, long long a_cols, long long lda, const void* B, long long b_rows,
                     long long b_cols, long long ldb, void* D, int ldd, const void* C, int ldc, void* aux, int ldaux, int M,
                     int N, int K, float alpha, int epilogue, int up_offset, int groups, int ragged, const int* counts,
                     int a_gs_mn, int b_gs_mn, long long d_gs, long long c_gs, long long aux_gs, int b_div,
                     const float* row_scale, long long rs_gs, const float* col_scale, long long cs_gs, int a_gs_k, int b_gs_k, int* status,
                     int max_ctas, void* stream) {
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  if (groups < 1 || groups > MAX_GROUPS) return 1002;
  if ((N & 7) || (K & 15) || (lda & 15) || (ldb & 15) || (ldd & 7) || (d_gs & 7) || (a_gs_mn & 7) || (b_gs_mn & 7)) return 1003;
  if ((epilogue == kSwiGLU && (up_offset & 7)) || (epilogue == kF32 && ((ldd & 3) || (N & 3)))) return 1004;
  if ((ragged && !counts) || ragged > 1 || b_div < 1 || (a_gs_k & 127) || (b_gs_k & 127)) return 1005;
  CUtensorMap ma, mb;
  int e;
  if ((e = make_tmap_2d(&ma, A, a_rows, a_cols, lda, 1, 128, 128))) return e;
  if ((e = make_tmap_2d(&mb, B, b_rows, b_cols, ldb, 1, 128, 128))) return e;
  GemmArgs p;
  p.M = M; p.N = N; p.K = K; p.groups = groups; p.ragged = ragged; p.counts = counts;
  p.a_gs_mn = a_gs_mn; p.a_gs_k = a_gs_k; p.b_gs_mn = b_gs_mn; p.b_gs_k = b_gs_k;  // K shifts per group: reduction slices
  p.d_gs = d_gs; p.c_gs = c_gs; p.aux_gs = aux_gs;
  p.D = static_cast<__nv_bfloat16*>(D); p.C = static_cast<const __nv_bfloat16*>(C);
  p.aux = static_cast<__nv_bfloat16*>(aux); p.Df32 = epilogue == kF32 ? static_cast<float*>(D) : nullptr;
  p.ldd = ldd; p.ldc = ldc; p.ldaux = ldaux; p.a_mn = 0; p.b_mn = 0; p.epilogue = epilogue;
  p.up_offset = up_offset; p.alpha = alpha; p.beta = 0; p.status = status;
  p.b_div = b_div; p.k_segs = 1; p.seg_stride = 0; p.d_table = nullptr; p.k_split = 1; p.scatter_rows = 0;
  p.b_packed = 0; p.b_kblocks = 0;
  p.fp8 = kind; p.row_scale = row_scale; p.col_scale = col_scale; p.rs_gs = rs_gs; p.cs_gs = cs_gs;
  p.n_copy = 0; p.n_rot = 0; p.own_row0 = 0; p.own_rows = 0; p.prof = nullptr;
  p.n_edge = 0; p.edge_chunk[0] = p.edge_chunk[1] = -1;
  p.out2 = nullptr; p.ldout2 = 0; p.out2_gs = 0;
  return launch_gemm(ma, mb, p, epilogue, groups, M, N, max_ctas, stream);
}

ATS_API int ats_gemm_fp8(const void* A, long long a_rows, long long a_cols, long long lda, const void* B, long long b_rows,
                         long long b_cols, long long ldb, void* D, int ldd, const void* C, int ldc, void* aux, int ldaux, int M,
                         int N, int K, float alpha, int epilogue, int up_offset, int groups, int ragged, const int* counts,
                         int a_gs_mn, int b_gs_mn, long long d_gs, long long c_gs, long long aux_gs, int b_div,
                         const float* row_scale, long long rs_gs, const float* col_scale, long long cs_gs, int a_gs_k, int b_gs_k,
                         int* status, int max_ctas, void* stream) {
  return gemm_8bit(1, A, a_rows, a_cols, lda, B, b_rows, b_cols, ldb, D, ldd, C, ldc, aux, ldaux, M, N, K, alpha, epilogue, up_offset, groups,
                   ragged, counts, a_gs_mn, b_gs_mn, d_gs, c_gs, aux_gs, b_div, row_scale, rs_gs, col_scale, cs_gs, a_gs_k, b_gs_k, status, max_ctas,
                   stream);
}

// Signed 8-bit operands (W8A8: activations quantised per token, weights per output channel), s32 accumulation on `kind::i8`,
// both scales applied in the epilogue.  Same arguments and epilogues as the e4m3 entry.
ATS_API int ats_gemm_int8(const void* A, long long a_rows, long long a_cols, long long lda, const void* B, long long b_rows,
                          long long b_cols, long long ldb, void* D, int ldd, const void* C, int ldc, void* aux, int ldaux, int M,
                          int N, int K, float alpha, int epilogue, int up_offset, int groups, int ragged, const int* counts,
                          int a_gs_mn, int b_gs_mn, long long d_gs, long long c_gs, long long aux_gs, int b_div,
                          const float* row_scale, long long rs_gs, const float* col_scale, long long cs_gs, int a_gs_k, int b_gs_k,
                          int* status, int max_ctas, void* stream) {
  return gemm_8bit(2, A, a_rows, a_cols, lda, B, b_rows, b_cols, ldb, D, ldd, C, ldc, aux, ldaux, M, N, K, alpha, epilogue, up_offset, groups,
                   ragged, counts, a_gs_mn, b_gs_mn, d_gs, c_gs, aux_gs, b_div, row_scale, rs_gs, col_scale, cs_gs, a_gs_k, b_gs_k, status, max_ctas,
                   stream);
}

// All-gather + GEMM in one kernel: D = A [M, K] * B^T with B [b_rows, K] row-sharded over `b_shards` GPUs.  `b_src` is a DEVICE
// array of the shards' base addresses (peer memory; entry `my_rank` is local), `B_local` the [b_rows, K] staging buffer on this
// GPU that the copy CTAs fill with the REMOTE shards and the GEMM reads (this rank's rows are read in place from `own_shard`), `b_ready` an int32 array of b_rows / ready_rows flags that only ever grow
// (`calls` = how many times this weight has been gathered with these flags, this call included).  Epilogues: store, +C, SwiGLU.
ATS_API int ats_gemm_bf16_gathered(const void* A, long long lda, const void* B_local, const void* own_shard, long long b_rows, const void* const* b_src,
                                   int b_shards, int my_rank, int ready_rows, int* b_ready, int calls, void* D, int ldd,
                                   const void* C, int ldc, void* aux, int ldaux, int M, int N, int K, int epilogue, int up_offset,
                                   int* status, void* stream) {
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  if (b_shards < 1 || my_rank < 0 || my_rank >= b_shards || ready_rows < 64 || calls < 1) return 1002;
  if (((long long)ready_rows * K * 2) % 4096) return 1003;
  if ((N & 7) || (K & 7) || (ldd & 7) || (b_rows % b_shards) || ((b_rows / b_shards) % ready_rows)) return 1003;
  if (ready_rows != 64 && ready_rows % 128) return 1003;  // chunks are halves or multiples of the 128-row boxes B is read in
  if (epilogue == kF32 || (epilogue == kSwiGLU && (up_offset & 7))) return 1004;
  CUtensorMap ma, mb;
  int e;
  if ((e = make_tmap_2d(&ma, A, M, K, lda, 2, 64, 128))) return e;
  if ((e = make_tmap_2d(&mb, B_local, b_rows, K, K, 2, 64, 128))) return e;
  CUtensorMap mb_own;
  if ((e = make_tmap_2d(&mb_own, own_shard, b_rows / b_shards, K, K, 2, 64, 128))) return e;
  GemmArgs p;
  p.M = M; p.N = N; p.K = K; p.groups = 1; p.ragged = 0; p.counts = nullptr;
  p.a_gs_mn = 0; p.a_gs_k = 0; p.b_gs_mn = 0; p.b_gs_k = 0; p.d_gs = 0; p.c_gs = 0; p.aux_gs = 0;
  p.D = static_cast<__nv_bfloat16*>(D); p.C = static_cast<const __nv_bfloat16*>(C);
  p.aux = static_cast<__nv_bfloat16*>(aux); p.Df32 = nullptr;
  p.ldd = ldd; p.ldc = ldc; p.ldaux = ldaux; p.a_mn = 0; p.b_mn = 0; p.epilogue = epilogue;
  p.up_offset = up_offset; p.alpha = 1.f; p.beta = 0; p.status = status;
  p.b_div = 1; p.k_segs = 1; p.seg_stride = 0; p.d_table = nullptr; p.k_split = 1; p.scatter_rows = 0;
  p.fp8 = 0; p.row_scale = nullptr; p.col_scale = nullptr; p.rs_gs = 0; p.cs_gs = 0;
  const long long shard_rows = b_rows / b_shards;
  p.b_packed = 0; p.b_kblocks = 0;
  p.n_copy = 1; p.b_src = b_src; p.b_dst = static_cast<uint8_t*>(const_cast<void*>(B_local));
  p.shard_bytes = shard_rows * K * 2; p.chunk_bytes = (long long)ready_rows * K * 2;
  p.b_ready = b_ready; p.ready_rows = ready_rows; p.n_chunks = int(b_rows / ready_rows);
  p.epoch = int(calls * (p.chunk_bytes / 4096));  // every call adds chunk_bytes / 4096 to each remote chunk's counter
  p.first_chunk = int(my_rank * (shard_rows / ready_rows));
  p.own_row0 = int(my_rank * shard_rows); p.own_rows = int(shard_rows); p.prof = nullptr;
  p.n_edge = 0; p.edge_chunk[0] = p.edge_chunk[1] = -1;
  if (b_shards > 1 && ready_rows == 64) {
    const int cps = int(shard_rows / ready_rows);
    if (p.own_row0 % 128) p.edge_chunk[p.n_edge++] = p.first_chunk;
    if ((p.own_row0 + p.own_rows) % 128 && !(p.n_edge && cps == 1)) p.edge_chunk[p.n_edge++] = p.first_chunk + cps - 1;
  }
  p.out2 = nullptr; p.ldout2 = 0; p.out2_gs = 0;
  const int tile_w = epilogue == kSwiGLU ? 128 : BN;
  p.n_rot = int((my_rank * shard_rows) % (epilogue == kSwiGLU ? (long long)up_offset : b_rows) / tile_w);
  return launch_gemm(ma, mb, p, epilogue, 1, M, N, 0, stream, &mb_own);
}

// Whole-sector stores need every row of D (and of aux for SwiGLU) to start 32-byte aligned at every 16th column.
static int sector_aligned_outputs(const GemmArgs& p) {
  if (!g_gemm_wide || p.d_table) return 0;
  if (p.epilogue == kF32) return 0;
  auto ok = [](const void* ptr, long long ld, long long gs) { return (reinterpret_cast<uintptr_t>(ptr) & 31) == 0 && (ld & 15) == 0 && (gs & 15) == 0; };
  if (!ok(p.D, p.ldd, p.d_gs)) return 0;
  if (p.epilogue == kAddC && !ok(p.C, p.ldc, p.c_gs)) return 0;
  if (p.epilogue == kSwiGLUBwd)
    return ok(p.aux, p.ldaux, p.aux_gs) && (p.up_offset & 15) == 0 && (!p.out2 || ok(p.out2, p.ldout2, p.out2_gs));
  if (p.epilogue == kSwiGLU && p.aux && (!ok(p.aux, p.ldaux, p.aux_gs) || (p.up_offset & 15))) return 0;
  return 1;
}

static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& p_in, int epilogue, int groups, int M, int N,
                       int max_ctas, void* stream, const CUtensorMap* mb_own) {
  GemmArgs p = p_in;
  p.wide = sector_aligned_outputs(p);
  p.wait_budget_ns = ats_get_wait_budget_ns();
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
    if (ce != cudaSuccess) return int(ce);
    attr_set = true;
  }
  const int tn = epilogue == kSwiGLU ? (N + 127) / 128 : (N + BN - 1) / BN;
  if (g_gemm_pair && M >= PAIR_BM) {
    // two SMs per 256 x 256 tile
    static int pair_clusters = -1;
    if (pair_clusters < 0) {
      cudaError_t ce = cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
      if (ce != cudaSuccess) return int(ce);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(unsigned(num_sms() & ~1));
      cfg.blockDim = dim3(PAIR_THREADS);
      cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
      int n = 0;
      ce = cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel, &cfg);
      if (ce != cudaSuccess) return int(ce);
      pair_clusters = n < 1 ? 1 : (n > num_sms() / 2 ? num_sms() / 2 : n);
    }
    const long long pair_tiles = (long long)groups * ((M + PAIR_BM - 1) / PAIR_BM) * tn;
    int clusters = pair_clusters;
    if (p.n_copy > 0) {
      // producers wait on the copy warps of other CTAs of this launch: keep the whole grid resident
    } else {
      if (max_ctas > 0 && max_ctas / 2 < clusters) clusters = max_ctas / 2 < 1 ? 1 : max_ctas / 2;
      if (pair_tiles < clusters) clusters = int(pair_tiles);
    }
    if (clusters < 1) return 0;
    // the two copy warps exist only in launches that gather B from peers
    gemm_bf16_pair_kernel<<<2 * clusters, p.n_copy ? PAIR_THREADS + 64 : PAIR_THREADS, PAIR_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
        ma, mb, mb_own ? *mb_own : mb, p);
    return int(cudaGetLastError());
  }
  long long upper = (long long)groups * ((M + BM - 1) / BM) * tn;
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (p.n_copy > 0) {
    // producers wait on the copy warps of other CTAs of this launch: keep the whole grid (one CTA per SM) resident
  } else if (upper < grid) {
    grid = int(upper);
  }
  if (grid < 1) return 0;
  if (M <= BM && p.n_copy == 0) {
    // a product of a decode step: its launch overlaps the tail of the kernel before it
    cudaError_t ce = launch_pdl(gemm_bf16_kernel, dim3(grid), dim3(GEMM_THREADS - 64), GEMM_SMEM_BYTES, static_cast<cudaStream_t>(stream), ma, mb,
                                mb_own ? *mb_own : mb, p);
    return int(ce != cudaSuccess ? ce : cudaGetLastError());
  }
  // the two copy warps exist only in launches that gather B from peers
  gemm_bf16_kernel<<<grid, p.n_copy ? GEMM_THREADS : GEMM_THREADS - 64, GEMM_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      ma, mb, mb_own ? *mb_own : mb, p);
  return int(cudaGetLastError());
}
