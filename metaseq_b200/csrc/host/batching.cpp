// Host-side helpers for the data pipeline and flat-parameter bookkeeping, exported with a
// C ABI and loaded through ctypes (libmsq_host.so).
//
//  * msq_batch_by_size        greedy token-budget batching (the reference's Cython
//                             batch_by_size_vec: metaseq/data/data_utils_fast.pyx:20-103)
//  * msq_batch_fixed_shapes   batching against a list of allowed (rows, longest) shapes
//                             (batch_fixed_shapes_fast: metaseq/data/data_utils_fast.pyx:124-172)
//  * msq_token_block_slices   cut a corpus of variable-length items into blocks for the
//                             break modes none / complete / complete_doc / eos
//                             (metaseq/data/token_block_utils_fast.pyx:52-105)
//  * msq_block_to_dataset_index  map each block to (first item, offset in it, last item)
//                             (token_block_utils_fast.pyx:111-138)
//  * msq_flatten / msq_unflatten  pack / unpack a list of host buffers into one flat buffer
//                             (apex_C flatten/unflatten: metaseq/modules/apex/flatten_unflatten.cpp)
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// num_tokens[n] in iteration order.  Writes the exclusive end position (in iteration order)
// of every batch to batch_ends and returns the number of batches.
long long msq_batch_by_size(const int64_t* num_tokens, long long n, long long max_tokens, long long max_sentences,
                            long long bsz_mult, int64_t* batch_ends) {
  long long nb = 0;
  long long start = 0;      // first element of the open batch
  long long rows = 0;       // elements in the open batch (excluding the candidate)
  int64_t longest = 0;      // longest element among open batch + candidate
  if (bsz_mult < 1) bsz_mult = 1;
  for (long long i = 0; i < n; ++i) {
    longest = std::max(longest, num_tokens[i]);
    const bool full = rows > 0 && ((max_sentences > 0 && rows == max_sentences) ||
                                   (max_tokens > 0 && (rows + 1) * longest > max_tokens));
    if (full) {
      const long long cut = std::max(bsz_mult * (rows / bsz_mult), rows % bsz_mult);
      start += cut;
      batch_ends[nb++] = start;
      rows -= cut;
      longest = 0;
      for (long long j = start; j <= i; ++j) longest = std::max(longest, num_tokens[j]);
    }
    ++rows;
  }
  if (rows > 0) batch_ends[nb++] = n;
  return nb;
}

// shapes[2 * s] = rows, shapes[2 * s + 1] = longest element allowed by shape s.  The open batch grows, in iteration
// order, while some shape holds it (rows and longest element both within the shape); the element that fits no shape
// together with the open batch closes it and opens the next one.  An element longer than every shape ends up alone.
// Writes the exclusive end position of every batch and returns their number.
long long msq_batch_fixed_shapes(const int64_t* num_tokens, long long n, const int64_t* shapes, long long n_shapes,
                                 int64_t* batch_ends) {
  long long nb = 0, rows = 0;
  int64_t longest = 0;
  // best[r] = the longest element that a batch of r rows may contain (0: no shape has r rows)
  int64_t max_rows = 0;
  for (long long s = 0; s < n_shapes; ++s) max_rows = std::max(max_rows, shapes[2 * s]);
  std::vector<int64_t> best(static_cast<size_t>(max_rows) + 2, 0);
  for (long long s = 0; s < n_shapes; ++s)
    for (int64_t r = 1; r <= shapes[2 * s]; ++r) best[r] = std::max(best[r], shapes[2 * s + 1]);
  for (long long i = 0; i < n; ++i) {
    const int64_t cand = std::max(longest, num_tokens[i]);
    const bool fits = rows + 1 <= max_rows && cand <= best[rows + 1];
    if (!fits && rows > 0) {
      batch_ends[nb++] = i;
      rows = 0;
      longest = 0;
    }
    ++rows;
    longest = std::max(longest, num_tokens[i]);
  }
  if (rows > 0) batch_ends[nb++] = n;
  return nb;
}

// mode: 0 none, 1 complete, 2 complete_doc, 3 eos.  sizes[n] item lengths.  Output rows of
// (start, end) token offsets into the concatenated corpus; returns the number of blocks.
// out must hold up to total_tokens / 1 + n rows in the worst case (caller sizes it as 2*(n + total/block + 2)).
long long msq_token_block_slices(const int64_t* sizes, long long n, long long block_size, int mode,
                                 long long document_sep_len, int64_t* out) {
  long long nb = 0;
  if (mode == 0) {
    long long total = 0;
    for (long long i = 0; i < n; ++i) total += sizes[i];
    for (long long s = 0; s < total; s += block_size) {
      out[2 * nb] = s;
      out[2 * nb + 1] = std::min(s + block_size, total);
      ++nb;
    }
    return nb;
  }
  if (mode == 3) {
    long long off = 0;
    for (long long i = 0; i < n; ++i) {
      // an item of length 1 is just the separator: it still forms its own (tiny) block
      out[2 * nb] = off;
      out[2 * nb + 1] = off + sizes[i];
      ++nb;
      off += sizes[i];
    }
    return nb;
  }
  // complete / complete_doc: whole items per block, never exceeding block_size unless a single
  // item is longer; complete_doc additionally closes the block at empty "document separator" items.
  long long tok = 0, cur = 0, start = 0;
  for (long long i = 0; i < n; ++i) {
    const long long sz = sizes[i];
    const bool doc_break = (mode == 2) && (sz == document_sep_len);
    if (doc_break) {
      if (cur > 0) {
        out[2 * nb] = start;
        out[2 * nb + 1] = tok;
        ++nb;
      }
      tok += sz;
      start = tok;
      cur = 0;
      continue;
    }
    if (cur > 0 && cur + sz > block_size) {
      out[2 * nb] = start;
      out[2 * nb + 1] = tok;
      ++nb;
      start = tok;
      cur = 0;
    }
    cur += sz;
    tok += sz;
  }
  if (cur > 0) {
    out[2 * nb] = start;
    out[2 * nb + 1] = tok;
    ++nb;
  }
  return nb;
}

// For every block (start, end): (index of first item, offset inside it, index of last item).
void msq_block_to_dataset_index(const int64_t* sizes, long long n, const int64_t* slices, long long nb,
                                int64_t* out) {
  std::vector<int64_t> cum(n + 1, 0);
  for (long long i = 0; i < n; ++i) cum[i + 1] = cum[i] + sizes[i];
  for (long long b = 0; b < nb; ++b) {
    const int64_t s = slices[2 * b], e = slices[2 * b + 1];
    const long long first = std::upper_bound(cum.begin(), cum.end(), s) - cum.begin() - 1;
    long long last = first;
    if (e > s) last = std::upper_bound(cum.begin(), cum.end(), e - 1) - cum.begin() - 1;
    out[3 * b] = first;
    out[3 * b + 1] = s - cum[first];
    out[3 * b + 2] = last;
  }
}

// Copies count buffers (srcs[i], nbytes[i]) back to back into dst; returns total bytes.
long long msq_flatten(const void* const* srcs, const int64_t* nbytes, long long count, void* dst) {
  long long off = 0;
  for (long long i = 0; i < count; ++i) {
    std::memcpy(static_cast<char*>(dst) + off, srcs[i], static_cast<size_t>(nbytes[i]));
    off += nbytes[i];
  }
  return off;
}

long long msq_unflatten(const void* src, void* const* dsts, const int64_t* nbytes, long long count) {
  long long off = 0;
  for (long long i = 0; i < count; ++i) {
    std::memcpy(dsts[i], static_cast<const char*>(src) + off, static_cast<size_t>(nbytes[i]));
    off += nbytes[i];
  }
  return off;
}

}  // extern "C"
