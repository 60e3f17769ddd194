// Peer-memory communication over NVLink / NVSwitch from inside kernels.
//
// * symmetric buffers: cudaMalloc + CUDA IPC handles, exchanged by the host through torch.distributed;
// * a flag barrier kernel (release/acquire at system scope, bounded spin, optional one-float payload to every
//   peer) -- all ranks launch it on their own GPU, it never waits on a kernel of the same GPU;
// * fused gradient path: every rank pulls its shard of the gradient bucket from all peers with plain 16-byte
//   loads, sums in fp32, keeps the reduced shard and its squared norm (reduce-scatter without a library call);
// * fused update path: AdamW on the owned fp32 shard whose bf16 result is pushed with 16-byte stores into the
//   parameter bucket of every peer (the all-gather happens inside the optimiser kernel).
//
// These replace the NCCL reduce-scatter / all-gather that DeepSpeed ZeRO, FSDP and the vendored LowLevelZero /
// Gemini engines issue around their optimiser step (reference training/trainer.py:2125-2183,
// backend/backend_fsdp.py:151-198, colossalai/zero/low_level/low_level_optim.py:370-449, 670-697).
// No load or store here uses cluster multicast; all peer traffic is ld.global / st.global on mapped peer memory.
#include "common.cuh"

namespace ats {

constexpr int MAX_PEERS = 16;
struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait budget of every peer wait in this library (nanoseconds of %globaltimer).  A host-side value handed to the kernels as
// an argument, so a test can make a wait give up after a few milliseconds and production runs can allow slow peers more
// than the one-second default.
static unsigned long long g_wait_budget_ns = ATS_WAIT_BUDGET_NS;

// flags.p[r] = base of rank r's flag array (int[world]).  The epoch lives in device memory (`epoch_counter`, private to
// this rank): thread 0 advances it, so a launch that is replayed from a CUDA graph still waits for a NEW arrival of
// every peer instead of re-using the epoch that was frozen into the captured arguments.  All ranks issue their barriers
// in the same order, so their counters agree.  Thread t: optionally stores the payload into peer t's payload slot
// [rank], releases the epoch into peer t's flags[rank], then waits (bounded) for flags[t] of its own array.
// `wait_ns` (optional, [MAX_PEERS + 1] int64 in this rank's memory): thread t adds the time it spent waiting for peer t, entry
// [MAX_PEERS] counts the calls -- how much of a step is spent waiting at barriers, and for whom, without a profiler.
__global__ void peer_barrier_kernel(PeerPtrs flags, PeerPtrs payload_dst, const float* payload_src, int rank, int world,
                                    int* epoch_counter, unsigned long long budget_ns, int* status, long long* wait_ns) {
  pdl_prologue();
  const int t = threadIdx.x;
  int epoch = 0;
  if (t == 0) {
    epoch = *epoch_counter + 1;
    *epoch_counter = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (t >= world) return;
  if (payload_src) {
    float v = *payload_src;
    reinterpret_cast<float*>(payload_dst.p[t])[rank] = v;
  }
  __threadfence_system();
  st_release_sys(reinterpret_cast<int*>(flags.p[t]) + rank, epoch);
  const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + t;
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(mine) < epoch) {
    if (globaltimer_ns() - t0 > budget_ns) {
      if (status) atomicCAS(status, 0, kTimeoutPeerFlag);
      return;
    }
    __nanosleep(64);
  }
  __threadfence_system();
  if (wait_ns) {
    wait_ns[t] += (long long)(globaltimer_ns() - t0);
    if (t == 0) wait_ns[MAX_PEERS] += 1;
  }
}

// out32[i] = sum_p grads_p[offset + i]  (i < n, n % 8 == 0); partial[block] = sum of squares of this block's part.
__global__ void __launch_bounds__(256)
peer_reduce_shard_kernel(PeerPtrs grads, int world, int rank, long long offset, long long n, float* __restrict__ out32,
                         float* __restrict__ partial, const int* __restrict__ status) {
  __shared__ float red[33];
  float ss = 0.f;
  // a barrier before this launch gave up on a peer: its gradients may be partial, so nothing is read or written
  // (the update kernel makes the same check; the host raises at its next status check)
  if (status && *status != 0) {
    if (threadIdx.x == 0) partial[blockIdx.x] = 0.f;
    return;
  }
  const long long nvec = n >> 3;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (int q = 0; q < world; ++q) {
      const int p = (rank + q) % world;  // start with the local copy, spread the remote reads over the peers
      const uint4 a = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[p]) + offset)[v];
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    reinterpret_cast<float4*>(out32)[2 * v] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    reinterpret_cast<float4*>(out32)[2 * v + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += acc[e] * acc[e];
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

__global__ void __launch_bounds__(256) sum_partials_kernel(const float* __restrict__ partial, int n, float* out, int accumulate) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

// clip state from `world` per-rank squared sums (slots written by the peers through the barrier payload)
__global__ void clip_coef_slots_kernel(const float* slots, int world, float pre_scale, float max_norm, float* state) {
  float s = 0.f;
  for (int i = 0; i < world; ++i) s += slots[i];
  const float norm = sqrtf(s) * pre_scale;
  const bool finite = isfinite(norm);
  float coef = 1.f;
  if (max_norm > 0.f && finite) coef = fminf(1.f, max_norm / (norm + 1e-6f));
  state[0] = finite ? pre_scale * coef : 0.f;
  state[1] = norm;
  state[2] = finite ? 0.f : 1.f;
}

// AdamW on the owned shard with fp32 gradients; the bf16 result goes to params.p[q] + offset for every rank q.
__global__ void __launch_bounds__(256)
adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g32,
                  PeerPtrs params, int world, int rank, long long offset, long long n, const float* __restrict__ hyper,
                  const float* __restrict__ clip_state, float wd_mult, const int* __restrict__ status) {
  if (status && *status != 0) return;  // a peer wait of this step gave up: keep master weights, moments and parameters as they are
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4] * wd_mult, step = hyper[5];
  float gscale = 1.f;
  if (clip_state) {
    if (clip_state[2] != 0.f) return;
    gscale = clip_state[0];
  }
  const float bc1 = 1.f - __powf(b1, step), bc2 = 1.f - __powf(b2, step);
  const float step_size = lr / bc1, inv_bc2_sqrt = rsqrtf(bc2);
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float pp[8], pm[8], pv[8], g[8];
    *reinterpret_cast<float4*>(pp) = reinterpret_cast<float4*>(master)[2 * i];
    *reinterpret_cast<float4*>(pp + 4) = reinterpret_cast<float4*>(master)[2 * i + 1];
    *reinterpret_cast<float4*>(pm) = reinterpret_cast<float4*>(m)[2 * i];
    *reinterpret_cast<float4*>(pm + 4) = reinterpret_cast<float4*>(m)[2 * i + 1];
    *reinterpret_cast<float4*>(pv) = reinterpret_cast<float4*>(v)[2 * i];
    *reinterpret_cast<float4*>(pv + 4) = reinterpret_cast<float4*>(v)[2 * i + 1];
    *reinterpret_cast<float4*>(g) = reinterpret_cast<const float4*>(g32)[2 * i];
    *reinterpret_cast<float4*>(g + 4) = reinterpret_cast<const float4*>(g32)[2 * i + 1];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ge = g[e] * gscale;
      pm[e] = b1 * pm[e] + (1.f - b1) * ge;
      pv[e] = b2 * pv[e] + (1.f - b2) * ge * ge;
      const float denom = sqrtf(pv[e]) * inv_bc2_sqrt + eps;
      pp[e] = pp[e] * (1.f - lr * wd) - step_size * pm[e] / denom;
    }
    reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(pp);
    reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(pp + 4);
    reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(pm);
    reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(pm + 4);
    reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(pv);
    reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(pv + 4);
    const uint4 o = make_uint4(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]), pack_bf16x2(pp[4], pp[5]), pack_bf16x2(pp[6], pp[7]));
    for (int q = 0; q < world; ++q) {
      const int p = (rank + q) % world;
      reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[p]) + offset)[i] = o;
    }
  }
}

// Plain peer copy (pull): dst[i] = src_peer[i], 16-byte vectors.  Used to stage a remote parameter shard locally.
__global__ void __launch_bounds__(256) peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// All-gather by pulling: dst[q * shard + i] = shards_q[i] for every rank q (this rank's own shard included), 16-byte vectors.
// Launched on a side stream with a bounded number of CTAs so that it overlaps the compute stream's GEMMs (ZeRO-3 prefetch).
// A read over NVLink takes a few microseconds, so every thread keeps eight 16-byte loads in flight: with one load per thread
// 24 CTAs moved 70 GB/s and the kernel stayed resident (and in the GEMMs' way) five times longer than the copy needs.
__global__ void __launch_bounds__(256) peer_gather_kernel(PeerPtrs shards, int world, uint4* __restrict__ dst, long long shard_vec,
                                                          const int* __restrict__ status) {
  if (status && *status != 0) return;
  constexpr int UNR = 8;
  const long long total = shard_vec * world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += stride * UNR) {
    uint4 v[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int q = int(i / shard_vec);
        v[u] = static_cast<const uint4*>(shards.p[q])[i - q * shard_vec];
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) dst[i] = v[u];
    }
  }
}

// Reduce-scatter by pulling, for one row-sharded matrix: out32[i] (+)= sum_q grads_q[offset + i], i < n (n, offset % 8 == 0).
// fp32 accumulation in registers; `accumulate` adds to what out32 holds (later micro-batches of one optimiser step).  Two
// vectors per thread, the loads of up to four peers for all of them issued before the first add (memory-level parallelism over
// NVLink) -- and no more than that, so that the kernel's registers leave room for a GEMM CTA on the same SM.
__global__ void __launch_bounds__(256)
peer_reduce_rows_kernel(PeerPtrs grads, int world, int rank, long long offset, long long n, float* __restrict__ out32, int accumulate,
                        const int* __restrict__ status) {
  if (status && *status != 0) return;
  constexpr int UNR = 2, PG = 4;
  const long long nvec = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * UNR) {
    float acc[UNR][8];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long v = v0 + u * stride;
      if (accumulate && v < nvec) {
        const float4 x = reinterpret_cast<const float4*>(out32)[2 * v], y = reinterpret_cast<const float4*>(out32)[2 * v + 1];
        acc[u][0] = x.x; acc[u][1] = x.y; acc[u][2] = x.z; acc[u][3] = x.w; acc[u][4] = y.x; acc[u][5] = y.y; acc[u][6] = y.z; acc[u][7] = y.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      }
    }
    for (int q0 = 0; q0 < world; q0 += PG) {
      uint4 a[UNR][PG];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long v = v0 + u * stride;
#pragma unroll
        for (int j = 0; j < PG; ++j) {
          a[u][j] = make_uint4(0, 0, 0, 0);
          if (q0 + j < world && v < nvec) {
            const int p = (rank + q0 + j) % world;  // start with the local copy, spread the remote reads over the peers
            a[u][j] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[p]) + offset)[v];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int j = 0; j < PG; ++j) {
          float2 f0 = unpack_bf16x2(a[u][j].x), f1 = unpack_bf16x2(a[u][j].y), f2 = unpack_bf16x2(a[u][j].z), f3 = unpack_bf16x2(a[u][j].w);
          acc[u][0] += f0.x; acc[u][1] += f0.y; acc[u][2] += f1.x; acc[u][3] += f1.y;
          acc[u][4] += f2.x; acc[u][5] += f2.y; acc[u][6] += f3.x; acc[u][7] += f3.y;
        }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long v = v0 + u * stride;
      if (v >= nvec) continue;
      reinterpret_cast<float4*>(out32)[2 * v] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
      reinterpret_cast<float4*>(out32)[2 * v + 1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
    }
  }
}

// Fold of the reduction slices of a grouped product (as ats_splitk_reduce) whose result peers will read: the CTA that finishes last
// raises this rank's flag on every peer (epoch = this rank's call counter), so that no barrier launch is needed between the
// product and the peers' reads.  done_counter: one int, zero between launches.  epoch_counter: one int in this rank's memory.
__global__ void __launch_bounds__(256)
splitk_reduce_signal_kernel(const float* __restrict__ part, int splits, long long n_inner, long long n_outer, __nv_bfloat16* __restrict__ out,
                            int* done_counter, int* epoch_counter, PeerPtrs flags, int rank, int world) {
  pdl_prologue();
  const long long nvec = n_inner >> 3, total = nvec * n_outer;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const long long o = v / nvec, i = (v - o * nvec) << 3;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const float* src = part + (o * splits) * n_inner + i;
    for (int s = 0; s < splits; ++s) {
      const float4 a = *reinterpret_cast<const float4*>(src + s * n_inner), b = *reinterpret_cast<const float4*>(src + s * n_inner + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    *reinterpret_cast<uint4*>(out + o * n_inner + i) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
  __threadfence_system();  // this CTA's rows are visible to the peers before it is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(done_counter, 1) == int(gridDim.x) - 1) {
      *done_counter = 0;
      const int e = *epoch_counter + 1;
      *epoch_counter = e;
      __threadfence_system();
      for (int t = 0; t < world; ++t)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(static_cast<int*>(flags.p[t]) + rank), "r"(e) : "memory");
    }
  }
}

static PeerPtrs to_peers(void* const* host_ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.p[i] = i < world ? host_ptrs[i] : nullptr;
  return pp;
}

}  // namespace ats

using namespace ats;

// ---- symmetric memory ----------------------------------------------------------------------------------
ATS_API int ats_ipc_alloc(unsigned long long bytes, void** ptr, unsigned char* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return int(e);
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return int(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return int(e);
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
ATS_API int ats_ipc_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return int(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
ATS_API int ats_ipc_close(void* ptr) { return int(cudaIpcCloseMemHandle(ptr)); }
ATS_API int ats_ipc_free(void* ptr) { return int(cudaFree(ptr)); }

// ---- kernels ------------------------------------------------------------------------------------------------
// flags / payload_dst: host arrays of `world` device pointers (one per rank, peer-mapped).
// epoch_counter: one int in this rank's device memory, zero before the first barrier of this flag set.
ATS_API int ats_peer_barrier(void* const* flags, void* const* payload_dst, const float* payload_src, int rank, int world,
                             int* epoch_counter, int* status, long long* wait_ns, void* stream) {
  if (world > MAX_PEERS || !epoch_counter) return 1003;
  PeerPtrs none = {};
  cudaError_t ce = launch_pdl(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), to_peers(flags, world),
                              payload_dst ? to_peers(payload_dst, world) : none, payload_src, rank, world, epoch_counter,
                              (unsigned long long)g_wait_budget_ns, status, wait_ns);
  return int(ce != cudaSuccess ? ce : cudaGetLastError());
}

// Budget of every peer wait launched after this call (0 restores the default of one second).
ATS_API void ats_set_wait_budget_ns(unsigned long long ns) { g_wait_budget_ns = ns ? ns : ATS_WAIT_BUDGET_NS; }
ATS_API unsigned long long ats_get_wait_budget_ns() { return g_wait_budget_ns; }

// Reduce this rank's shard [offset, offset + n) of the gradient buckets of all ranks into out32 and its squared sum
// into sumsq[0] (added when accumulate).  partial: >= 1184 floats of scratch.
ATS_API int ats_peer_reduce_shard(void* const* grads, int world, int rank, long long offset, long long n, float* out32,
                                  float* partial, float* sumsq, int accumulate, const int* status, void* stream) {
  if (world > MAX_PEERS || (n & 7) || (offset & 7)) return 1003;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long blocks = (n / 8 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  peer_reduce_shard_kernel<<<(unsigned)blocks, 256, 0, s>>>(to_peers(grads, world), world, rank, offset, n, out32, partial, status);
  sum_partials_kernel<<<1, 256, 0, s>>>(partial, (int)blocks, sumsq, accumulate);
  return int(cudaGetLastError());
}

ATS_API int ats_clip_coef_slots(const float* slots, int world, float pre_scale, float max_norm, float* state, void* stream) {
  clip_coef_slots_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(slots, world, pre_scale, max_norm, state);
  return int(cudaGetLastError());
}

ATS_API int ats_adamw_push(float* master, float* m, float* v, const float* g32, void* const* params, int world, int rank,
                           long long offset, long long n, const float* hyper, const float* clip_state, float wd_mult,
                           const int* status, void* stream) {
  if (world > MAX_PEERS || (n & 7) || (offset & 7)) return 1003;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  adamw_push_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(master, m, v, g32, to_peers(params, world),
                                                                                   world, rank, offset, n, hyper, clip_state, wd_mult, status);
  return int(cudaGetLastError());
}

ATS_API int ats_peer_copy(const void* src, void* dst, long long bytes, int max_blocks, void* stream) {
  if (bytes & 15) return 1003;
  long long nvec = bytes >> 4;
  long long blocks = (nvec + 255) / 256;
  if (blocks < 1) blocks = 1;
  const long long cap = max_blocks > 0 ? max_blocks : 148 * 4;
  if (blocks > cap) blocks = cap;
  peer_copy_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src),
                                                                                  static_cast<uint4*>(dst), nvec);
  return int(cudaGetLastError());
}

// shards: host array of `world` device pointers (every rank's shard, this rank's own included); dst: world * shard_bytes.
ATS_API int ats_peer_gather(void* const* shards, int world, void* dst, long long shard_bytes, int max_blocks, const int* status,
                            void* stream) {
  if (world < 1 || world > MAX_PEERS || (shard_bytes & 15) || shard_bytes <= 0) return 1003;
  const long long total = (shard_bytes >> 4) * world;
  long long blocks = (total + 255) / 256;
  const long long cap = max_blocks > 0 ? max_blocks : 148 * 4;
  if (blocks > cap) blocks = cap;
  peer_gather_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(to_peers(shards, world), world, static_cast<uint4*>(dst),
                                                                                      shard_bytes >> 4, status);
  return int(cudaGetLastError());
}

ATS_API int ats_peer_reduce_rows(void* const* grads, int world, int rank, long long offset, long long n, float* out32, int accumulate,
                                 const int* status, int max_blocks, void* stream) {
  if (world < 1 || world > MAX_PEERS || (n & 7) || (offset & 7) || n <= 0) return 1003;
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = max_blocks > 0 ? max_blocks : 148 * 4;
  if (blocks > cap) blocks = cap;
  peer_reduce_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(to_peers(grads, world), world, rank, offset, n, out32,
                                                                                           accumulate, status);
  return int(cudaGetLastError());
}

// flags: host array of `world` device pointers, entry t = the int32 flag array [world] in rank t's memory (peer-mapped).
ATS_API int ats_splitk_reduce_signal(const float* part, int splits, long long n_inner, long long n_outer, void* out, int* done_counter,
                                     int* epoch_counter, void* const* flags, int rank, int world, void* stream) {
  if (splits < 1 || n_inner <= 0 || n_outer <= 0 || (n_inner & 7) || world > MAX_PEERS || !done_counter || !epoch_counter) return 1003;
  long long blocks = ((n_inner >> 3) * n_outer + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaError_t ce = launch_pdl(splitk_reduce_signal_kernel, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream), part, splits,
                              n_inner, n_outer, static_cast<__nv_bfloat16*>(out), done_counter, epoch_counter, to_peers(flags, world), rank, world);
  return int(ce != cudaSuccess ? ce : cudaGetLastError());
}
