// Host-side data-path helpers (C ABI, called through ctypes):
//   * ats_build_sample_index: cut a stream of tokenised documents into fixed-length training samples (each sample is
//     seq_len + 1 tokens; the last token of one sample is the first of the next, documents are concatenated in the given
//     order) and return, for every sample, the document and offset where it starts;
//   * ats_shuffle_index: seeded Fisher-Yates permutation (splitmix64), identical on every rank for the same seed;
//   * ats_pack_rows: gather ragged token lists into a padded [rows, width] int64 matrix plus mask, multi-threaded;
//   * ats_blend_index: interleave several datasets by weight with the greedy largest-deficit rule.
// The reference reaches this kind of code only through its vendored examples
// (colossalai examples/tutorial/sequence_parallel/data/datasets/helpers.cpp: sample / blending index builders).
#include <omp.h>

#include <cstdint>
#include <cstring>

#define ATS_HOST_API extern "C" __attribute__((visibility("default")))

// doc_lens[n_docs] tokens per document (in epoch order).  Returns the number of samples; fills sample_doc / sample_off
// (capacity `cap`; pass cap = 0 to only count).
ATS_HOST_API long long ats_build_sample_index(const int32_t* doc_lens, long long n_docs, int seq_len, long long* sample_doc,
                                              int32_t* sample_off, long long cap) {
  long long total = 0;
  for (long long i = 0; i < n_docs; ++i) total += doc_lens[i];
  if (total < 2 || seq_len < 1) return 0;
  const long long n_samples = (total - 1) / seq_len;
  if (cap == 0) return n_samples;
  long long doc = 0;
  int32_t off = 0;
  for (long long s = 0; s < n_samples && s < cap; ++s) {
    sample_doc[s] = doc;
    sample_off[s] = off;
    long long remaining = seq_len;  // advance by seq_len tokens (the +1 token overlaps with the next sample)
    while (remaining > 0) {
      const long long left = doc_lens[doc] - off;
      if (left > remaining) {
        off += int32_t(remaining);
        remaining = 0;
      } else {
        remaining -= left;
        ++doc;
        off = 0;
      }
    }
  }
  return n_samples;
}

static inline uint64_t splitmix64(uint64_t& s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

ATS_HOST_API void ats_shuffle_index(long long* idx, long long n, unsigned long long seed) {
  for (long long i = 0; i < n; ++i) idx[i] = i;
  uint64_t s = seed;
  for (long long i = n - 1; i > 0; --i) {
    const uint64_t j = splitmix64(s) % uint64_t(i + 1);
    const long long t = idx[i];
    idx[i] = idx[j];
    idx[j] = t;
  }
}

// tokens: concatenated rows; offsets[rows + 1].  Row r is truncated to `width`; padding cells get pad_id and mask 0.
ATS_HOST_API void ats_pack_rows(const int64_t* tokens, const long long* offsets, long long rows, int width, int64_t pad_id, int64_t* out,
                                uint8_t* mask) {
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < rows; ++r) {
    long long n = offsets[r + 1] - offsets[r];
    if (n > width) n = width;
    std::memcpy(out + r * width, tokens + offsets[r], size_t(n) * sizeof(int64_t));
    for (long long j = n; j < width; ++j) out[r * width + j] = pad_id;
    if (mask) {
      std::memset(mask + r * width, 1, size_t(n));
      std::memset(mask + r * width + n, 0, size_t(width - n));
    }
  }
}

// weights[n_sets] (any positive scale).  Fills which[n] (dataset of sample i) and within[n] (running index inside that
// dataset), always picking the dataset that is furthest behind its share.
ATS_HOST_API void ats_blend_index(const double* weights, int n_sets, long long n, int32_t* which, long long* within) {
  double wsum = 0;
  for (int d = 0; d < n_sets; ++d) wsum += weights[d];
  long long* taken = new long long[n_sets]();
  for (long long i = 0; i < n; ++i) {
    int best = 0;
    double best_err = -1e300;
    for (int d = 0; d < n_sets; ++d) {
      const double err = weights[d] / wsum * double(i + 1) - double(taken[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    which[i] = best;
    within[i] = taken[best]++;
  }
  delete[] taken;
}
