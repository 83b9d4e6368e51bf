// CPU dataset-index builders with a plain C ABI (loaded through ctypes; arrays are numpy buffers
// owned by the caller).  Counterpart of the pybind11 module megatron/data/helpers.cpp:
//   nx_build_sample_idx_{i32,i64}   GPT sample index (helpers.cpp:91-259)
//   nx_build_blending_indices       greedy largest-error dataset interleave (helpers.cpp:34-89)
//   nx_build_mapping                sentence-packing sample map, BERT style (helpers.cpp:270-511)
//   nx_build_blocks_mapping         block map for retrieval pre-training (helpers.cpp:514-747)
// The two-pass "count, allocate, fill" shape of the mapping builders is kept so the caller can
// size its numpy array: pass out == nullptr to get the number of rows.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

#define NX_EXPORT extern "C" __attribute__((visibility("default")))

template <typename IdxT>
static void build_sample_idx_impl(const int32_t* sizes, const int32_t* doc_idx, int64_t seq_length,
                                  int64_t num_epochs, int64_t tokens_per_epoch, IdxT* sample_idx,
                                  int64_t num_samples) {
  // sample i spans tokens [i * seq_length, (i + 1) * seq_length] of the concatenated, shuffled
  // document stream: seq_length + 1 tokens, the last one shared with the next sample.
  int64_t sample_index = 0;
  int64_t doc_idx_index = 0;
  int64_t doc_offset = 0;
  sample_idx[0] = static_cast<IdxT>(doc_idx_index);
  sample_idx[1] = static_cast<IdxT>(doc_offset);
  ++sample_index;
  while (sample_index <= num_samples) {
    int64_t remaining = seq_length + 1;
    while (remaining != 0) {
      const int64_t doc_id = doc_idx[doc_idx_index];
      const int64_t doc_length = static_cast<int64_t>(sizes[doc_id]) - doc_offset;
      remaining -= doc_length;
      if (remaining <= 0) {
        // the sample ends inside this document; "-1" re-reads its last token as the next
        // sample's first one
        doc_offset += (remaining + doc_length - 1);
        remaining = 0;
      } else {
        ++doc_idx_index;
        doc_offset = 0;
      }
    }
    sample_idx[2 * sample_index] = static_cast<IdxT>(doc_idx_index);
    sample_idx[2 * sample_index + 1] = static_cast<IdxT>(doc_offset);
    ++sample_index;
  }
  (void)num_epochs;
  (void)tokens_per_epoch;
}

NX_EXPORT int64_t nx_num_samples(int64_t seq_length, int64_t num_epochs, int64_t tokens_per_epoch) {
  return (num_epochs * tokens_per_epoch - 1) / seq_length;
}

// sample_idx: [(num_samples + 1), 2]
NX_EXPORT void nx_build_sample_idx_i32(const int32_t* sizes, const int32_t* doc_idx, int64_t seq_length,
                                       int64_t num_epochs, int64_t tokens_per_epoch, int32_t* sample_idx) {
  build_sample_idx_impl<int32_t>(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, sample_idx,
                                 nx_num_samples(seq_length, num_epochs, tokens_per_epoch));
}
NX_EXPORT void nx_build_sample_idx_i64(const int32_t* sizes, const int32_t* doc_idx, int64_t seq_length,
                                       int64_t num_epochs, int64_t tokens_per_epoch, int64_t* sample_idx) {
  build_sample_idx_impl<int64_t>(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, sample_idx,
                                 nx_num_samples(seq_length, num_epochs, tokens_per_epoch));
}

NX_EXPORT void nx_build_blending_indices(uint8_t* dataset_index, int64_t* dataset_sample_index,
                                         const double* weights, int32_t num_datasets, int64_t size,
                                         int32_t verbose) {
  std::vector<int64_t> current(num_datasets, 0);
  for (int64_t s = 0; s < size; ++s) {
    const double want = std::max(static_cast<double>(s), 1.0);
    int32_t best = 0;
    double best_err = weights[0] * want - static_cast<double>(current[0]);
    for (int32_t d = 1; d < num_datasets; ++d) {
      const double err = weights[d] * want - static_cast<double>(current[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    dataset_index[s] = static_cast<uint8_t>(best);
    dataset_sample_index[s] = current[best];
    current[best] += 1;
  }
  if (verbose) {
    printf(" > sample ratios:\n");
    for (int32_t d = 0; d < num_datasets; ++d)
      printf("   dataset %d, input: %g, achieved: %g\n", d, weights[d],
             static_cast<double>(current[d]) / static_cast<double>(size));
    fflush(stdout);
  }
}

static inline int32_t target_sample_len(int32_t short_seq_ratio, int32_t max_length, std::mt19937& gen) {
  const auto r = gen();
  if ((r % short_seq_ratio) == 0) return 2 + r % (max_length - 1);
  return max_length;
}

// Rows (start sentence, end sentence, target length). docs: [n_docs + 1] sentence boundaries; sizes: per
// sentence.  out == nullptr: returns the row count only; otherwise fills and shuffles `out` [rows, 3].
NX_EXPORT int64_t nx_build_mapping(const int64_t* docs, int64_t n_docs_plus_1, const int32_t* sizes,
                                   int32_t num_epochs, uint64_t max_num_samples, int32_t max_seq_length,
                                   double short_seq_prob, int32_t seed, int64_t* out) {
  const int32_t short_seq_ratio = static_cast<int32_t>(std::lround(1.0 / short_seq_prob));
  const int64_t n_docs = n_docs_plus_1 - 1;
  constexpr int32_t LONG_SENTENCE_LEN = 512;
  std::mt19937 gen(seed);
  uint64_t map_index = 0;
  for (int32_t epoch = 0; epoch < num_epochs; ++epoch) {
    if (map_index >= max_num_samples) break;
    for (int64_t doc = 0; doc < n_docs; ++doc) {
      const int64_t first = docs[doc], last = docs[doc + 1];
      int64_t remain = last - first;
      bool has_long = false;
      if (remain > 1)
        for (int64_t s = first; s < last; ++s)
          if (sizes[s] > LONG_SENTENCE_LEN) { has_long = true; break; }
      if (remain > 1 && !has_long) {
        int64_t prev_start = first;
        int32_t seq_len = 0, num_sent = 0;
        int32_t target = target_sample_len(short_seq_ratio, max_seq_length, gen);
        for (int64_t s = first; s < last; ++s) {
          seq_len += sizes[s];
          ++num_sent;
          --remain;
          if ((seq_len >= target && remain > 1 && num_sent > 1) || remain == 0) {
            if (out != nullptr) {
              out[3 * map_index] = prev_start;
              out[3 * map_index + 1] = s + 1;
              out[3 * map_index + 2] = target;
            }
            ++map_index;
            prev_start = s + 1;
            target = target_sample_len(short_seq_ratio, max_seq_length, gen);
            seq_len = 0;
            num_sent = 0;
          }
        }
      }
    }
  }
  const int64_t rows = static_cast<int64_t>(map_index);
  if (out != nullptr) {
    std::mt19937_64 gen64(seed + 1);
    for (int64_t i = rows - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(gen64() % static_cast<uint64_t>(i + 1));
      for (int c = 0; c < 3; ++c) std::swap(out[3 * i + c], out[3 * j + c]);
    }
  }
  return rows;
}

// Rows (start sentence, end sentence, document, block id). titles_sizes: per document.
NX_EXPORT int64_t nx_build_blocks_mapping(const int64_t* docs, int64_t n_docs_plus_1, const int32_t* sizes,
                                          const int32_t* titles_sizes, int32_t num_epochs,
                                          uint64_t max_num_samples, int32_t max_seq_length, int32_t seed,
                                          int32_t use_one_sent_blocks, int64_t* out) {
  const int64_t n_docs = n_docs_plus_1 - 1;
  constexpr int32_t LONG_SENTENCE_LEN = 512;
  const int32_t min_num_sent = use_one_sent_blocks ? 1 : 2;
  uint64_t map_index = 0;
  for (int32_t epoch = 0; epoch < num_epochs; ++epoch) {
    int64_t block_id = 0;
    if (map_index >= max_num_samples) break;
    for (int64_t doc = 0; doc < n_docs; ++doc) {
      const int64_t first = docs[doc], last = docs[doc + 1];
      const int32_t target = max_seq_length - titles_sizes[doc];
      int64_t remain = last - first;
      bool has_long = false;
      if (remain >= min_num_sent)
        for (int64_t s = first; s < last; ++s)
          if (sizes[s] > LONG_SENTENCE_LEN) { has_long = true; break; }
      if (remain >= min_num_sent && !has_long) {
        int64_t prev_start = first;
        int32_t seq_len = 0, num_sent = 0;
        for (int64_t s = first; s < last; ++s) {
          seq_len += sizes[s];
          ++num_sent;
          --remain;
          if ((seq_len >= target && remain >= min_num_sent && num_sent >= min_num_sent) || remain == 0) {
            if (out != nullptr) {
              out[4 * map_index] = prev_start;
              out[4 * map_index + 1] = s + 1;
              out[4 * map_index + 2] = doc;
              out[4 * map_index + 3] = block_id;
            }
            ++map_index;
            ++block_id;
            prev_start = s + 1;
            seq_len = 0;
            num_sent = 0;
          }
        }
      }
    }
  }
  const int64_t rows = static_cast<int64_t>(map_index);
  if (out != nullptr) {
    std::mt19937_64 gen64(seed + 1);
    for (int64_t i = rows - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(gen64() % static_cast<uint64_t>(i + 1));
      for (int c = 0; c < 4; ++c) std::swap(out[4 * i + c], out[4 * j + c]);
    }
  }
  return rows;
}
