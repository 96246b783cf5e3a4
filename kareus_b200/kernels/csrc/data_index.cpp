// Sample index of a GPT dataset: where in the shuffled stream of documents every training sample begins.
//
// The stream is the documents `doc_order[0], doc_order[1], ...` back to back.  Sample i covers tokens
// [i*seq_len, (i+1)*seq_len] of the stream (seq_len + 1 tokens: inputs and the labels shifted by one), so
// consecutive samples share one token.  out[2*i], out[2*i+1] = (position in doc_order, token offset inside
// that document) of sample i's first token, for i = 0..num_samples (the last entry closes the last sample).
// Same role as the index builder that Megatron compiles for its GPT dataset
// (3rdparty/Megatron-LM/megatron/core/datasets/helpers.cpp, build_sample_idx); written as one walk over
// the documents with 64-bit positions.
#include <stdint.h>

extern "C" int kb_build_sample_index(const int64_t* doc_len, const int64_t* doc_order, int64_t n_order,
                                     int64_t seq_len, int64_t num_samples, int64_t* out) {
  if (seq_len <= 0 || num_samples < 0 || n_order < 0) return 7;
  int64_t d = 0;          // position in doc_order
  int64_t off = 0;        // token offset inside that document
  // skip leading empty documents
  while (d < n_order && doc_len[doc_order[d]] == 0) ++d;
  for (int64_t i = 0; i <= num_samples; ++i) {
    if (d >= n_order) return 8;                 // the stream is too short for this many samples
    out[2 * i] = d;
    out[2 * i + 1] = off;
    if (i == num_samples) {
      // the closing entry must still have one token to give (the last label)
      break;
    }
    int64_t need = seq_len;                     // advance by seq_len tokens
    while (need > 0) {
      if (d >= n_order) return 8;
      const int64_t left = doc_len[doc_order[d]] - off;
      if (need < left) {
        off += need;
        need = 0;
      } else {
        need -= left;
        ++d;
        off = 0;
        while (d < n_order && doc_len[doc_order[d]] == 0) ++d;
      }
    }
  }
  return 0;
}

// Blend of several datasets: sample i of the blend comes from the dataset that is furthest behind its share
// (largest weight[d] * (i + 1) - taken[d]); out_ds[i] is that dataset and out_pos[i] how many samples it had
// given before.  Deterministic, and every prefix of the blend holds each dataset within one sample of its
// share.  Same role as Megatron's build_blending_indices (megatron/core/datasets/helpers.cpp).
extern "C" int kb_build_blend_index(const double* weights, int n_ds, int64_t n, int16_t* out_ds, int64_t* out_pos) {
  if (n_ds <= 0 || n_ds > 32767 || n < 0) return 7;
  int64_t taken[64];
  if (n_ds > 64) return 7;
  for (int d = 0; d < n_ds; ++d) taken[d] = 0;
  for (int64_t i = 0; i < n; ++i) {
    int best = 0;
    double best_err = -1e300;
    for (int d = 0; d < n_ds; ++d) {
      const double err = weights[d] * static_cast<double>(i + 1) - static_cast<double>(taken[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    out_ds[i] = static_cast<int16_t>(best);
    out_pos[i] = taken[best]++;
  }
  return 0;
}
