// Host-side AdamW for optimiser-state offload: fp32 master / m / v in (pinned) host memory, bf16 or fp32 gradients in,
// optional bf16 parameter copy out (the buffer that is copied back to the GPU).  OpenMP over tiles, AVX-512 when the CPU
// has it, AVX2 + FMA otherwise, scalar tail.  Same arithmetic as the device kernel (decoupled decay, bias correction,
// gradient pre-scale, skip on non-finite norm) so a run can move a bucket between device and host without a jump.
//
// The vendored counterpart of the reference is an AVX Adam with the same role
// (colossalai extensions csrc/cuda/cpu_adam.cpp:82-446, used by its CPU / hybrid Adam with Gemini offload).
#include <immintrin.h>
#include <omp.h>

#include <cmath>
#include <cstdint>
#include <cstring>

#define ATS_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = uint32_t(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {  // round to nearest even
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}

struct Hyper {
  float lr, b1, b2, eps, wd, step_size, inv_bc2_sqrt, gscale;
};

template <bool GRAD_BF16>
void tile_scalar(float* w, float* m, float* v, const void* g, uint16_t* p, long long lo, long long hi, const Hyper& h) {
  for (long long i = lo; i < hi; ++i) {
    const float gi = (GRAD_BF16 ? bf16_to_f32(static_cast<const uint16_t*>(g)[i]) : static_cast<const float*>(g)[i]) * h.gscale;
    const float nm = h.b1 * m[i] + (1.f - h.b1) * gi;
    const float nv = h.b2 * v[i] + (1.f - h.b2) * gi * gi;
    const float denom = std::sqrt(nv) * h.inv_bc2_sqrt + h.eps;
    const float nw = w[i] * (1.f - h.lr * h.wd) - h.step_size * nm / denom;
    m[i] = nm;
    v[i] = nv;
    w[i] = nw;
    if (p) p[i] = f32_to_bf16(nw);
  }
}

template <bool GRAD_BF16>
__attribute__((target("avx2,fma"))) void tile_avx2(float* w, float* m, float* v, const void* g, uint16_t* p, long long lo, long long hi,
                                                   const Hyper& h) {
  const __m256 b1 = _mm256_set1_ps(h.b1), ob1 = _mm256_set1_ps(1.f - h.b1), b2 = _mm256_set1_ps(h.b2), ob2 = _mm256_set1_ps(1.f - h.b2);
  const __m256 eps = _mm256_set1_ps(h.eps), decay = _mm256_set1_ps(1.f - h.lr * h.wd), ss = _mm256_set1_ps(h.step_size);
  const __m256 ibc = _mm256_set1_ps(h.inv_bc2_sqrt), gs = _mm256_set1_ps(h.gscale);
  long long i = lo;
  for (; i + 8 <= hi; i += 8) {
    __m256 gi;
    if (GRAD_BF16) {
      const __m128i raw = _mm_loadu_si128(reinterpret_cast<const __m128i*>(static_cast<const uint16_t*>(g) + i));
      gi = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(raw), 16));
    } else {
      gi = _mm256_loadu_ps(static_cast<const float*>(g) + i);
    }
    gi = _mm256_mul_ps(gi, gs);
    const __m256 nm = _mm256_fmadd_ps(b1, _mm256_loadu_ps(m + i), _mm256_mul_ps(ob1, gi));
    const __m256 nv = _mm256_fmadd_ps(b2, _mm256_loadu_ps(v + i), _mm256_mul_ps(ob2, _mm256_mul_ps(gi, gi)));
    const __m256 denom = _mm256_fmadd_ps(_mm256_sqrt_ps(nv), ibc, eps);
    const __m256 nw = _mm256_fnmadd_ps(ss, _mm256_div_ps(nm, denom), _mm256_mul_ps(_mm256_loadu_ps(w + i), decay));
    _mm256_storeu_ps(m + i, nm);
    _mm256_storeu_ps(v + i, nv);
    _mm256_storeu_ps(w + i, nw);
    if (p) {
      alignas(32) float tmp[8];
      _mm256_store_ps(tmp, nw);
      for (int k = 0; k < 8; ++k) p[i + k] = f32_to_bf16(tmp[k]);
    }
  }
  tile_scalar<GRAD_BF16>(w, m, v, g, p, i, hi, h);
}

template <bool GRAD_BF16>
__attribute__((target("avx512f,avx512bw"))) void tile_avx512(float* w, float* m, float* v, const void* g, uint16_t* p, long long lo,
                                                             long long hi, const Hyper& h) {
  const __m512 b1 = _mm512_set1_ps(h.b1), ob1 = _mm512_set1_ps(1.f - h.b1), b2 = _mm512_set1_ps(h.b2), ob2 = _mm512_set1_ps(1.f - h.b2);
  const __m512 eps = _mm512_set1_ps(h.eps), decay = _mm512_set1_ps(1.f - h.lr * h.wd), ss = _mm512_set1_ps(h.step_size);
  const __m512 ibc = _mm512_set1_ps(h.inv_bc2_sqrt), gs = _mm512_set1_ps(h.gscale);
  long long i = lo;
  for (; i + 16 <= hi; i += 16) {
    __m512 gi;
    if (GRAD_BF16) {
      const __m256i raw = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(static_cast<const uint16_t*>(g) + i));
      gi = _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(raw), 16));
    } else {
      gi = _mm512_loadu_ps(static_cast<const float*>(g) + i);
    }
    gi = _mm512_mul_ps(gi, gs);
    const __m512 nm = _mm512_fmadd_ps(b1, _mm512_loadu_ps(m + i), _mm512_mul_ps(ob1, gi));
    const __m512 nv = _mm512_fmadd_ps(b2, _mm512_loadu_ps(v + i), _mm512_mul_ps(ob2, _mm512_mul_ps(gi, gi)));
    const __m512 denom = _mm512_fmadd_ps(_mm512_sqrt_ps(nv), ibc, eps);
    const __m512 nw = _mm512_fnmadd_ps(ss, _mm512_div_ps(nm, denom), _mm512_mul_ps(_mm512_loadu_ps(w + i), decay));
    _mm512_storeu_ps(m + i, nm);
    _mm512_storeu_ps(v + i, nv);
    _mm512_storeu_ps(w + i, nw);
    if (p) {
      // round to nearest even in integer arithmetic (NaN handling is left to the scalar helper: weights are finite)
      const __m512i u = _mm512_castps_si512(nw);
      const __m512i lsb = _mm512_and_si512(_mm512_srli_epi32(u, 16), _mm512_set1_epi32(1));
      const __m512i r = _mm512_srli_epi32(_mm512_add_epi32(u, _mm512_add_epi32(lsb, _mm512_set1_epi32(0x7fff))), 16);
      _mm256_storeu_si256(reinterpret_cast<__m256i*>(p + i), _mm512_cvtepi32_epi16(r));
    }
  }
  tile_scalar<GRAD_BF16>(w, m, v, g, p, i, hi, h);
}

int g_isa = -1;  // 0 scalar, 1 avx2, 2 avx512
int isa() {
  if (g_isa < 0) {
    __builtin_cpu_init();
    if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw")) g_isa = 2;
    else if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) g_isa = 1;
    else g_isa = 0;
  }
  return g_isa;
}

template <bool GRAD_BF16>
void run(float* w, float* m, float* v, const void* g, uint16_t* p, long long n, const Hyper& h, int force_isa) {
  const int level = force_isa >= 0 ? (force_isa < isa() ? force_isa : isa()) : isa();
  constexpr long long TILE = 1 << 16;
  const long long tiles = (n + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < tiles; ++t) {
    const long long lo = t * TILE, hi = (lo + TILE < n) ? lo + TILE : n;
    if (level == 2) tile_avx512<GRAD_BF16>(w, m, v, g, p, lo, hi, h);
    else if (level == 1) tile_avx2<GRAD_BF16>(w, m, v, g, p, lo, hi, h);
    else tile_scalar<GRAD_BF16>(w, m, v, g, p, lo, hi, h);
  }
}

}  // namespace

// 0 = scalar, 1 = AVX2 + FMA, 2 = AVX-512 (what the running CPU supports).
ATS_HOST_API int ats_cpu_isa() { return isa(); }

// One AdamW step over n elements.  grad_bf16: gradients are bf16 (else fp32).  param_bf16 may be null.  step >= 1.
// grad_scale multiplies the gradient (clip coefficient x 1 / loss scale).  force_isa < 0: best available.
ATS_HOST_API int ats_cpu_adamw(float* master, float* m, float* v, const void* grad, int grad_bf16, void* param_bf16, long long n, float lr,
                               float beta1, float beta2, float eps, float weight_decay, long long step, float grad_scale, int force_isa) {
  if (n < 0 || step < 1) return 1;
  Hyper h;
  h.lr = lr; h.b1 = beta1; h.b2 = beta2; h.eps = eps; h.wd = weight_decay; h.gscale = grad_scale;
  const float bc1 = 1.f - std::pow(beta1, float(step)), bc2 = 1.f - std::pow(beta2, float(step));
  h.step_size = lr / bc1;
  h.inv_bc2_sqrt = 1.f / std::sqrt(bc2);
  if (grad_bf16) run<true>(master, m, v, grad, static_cast<uint16_t*>(param_bf16), n, h, force_isa);
  else run<false>(master, m, v, grad, static_cast<uint16_t*>(param_bf16), n, h, force_isa);
  return 0;
}
