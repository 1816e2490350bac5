// Host-side index builders for a mixed prefill/decode step. The reference's scheduler crate is
// an empty scaffold (crates/sched/src/lib.rs:1-30), so these define the packing; the invariant
// they keep is the reference's only execution semantics, one sequence per call
// (crates/transformers/src/attention.rs:13-14): the packed step must equal running each sequence
// alone, so positions continue from each sequence's cached length and every new token gets the
// cache slot its (sequence, position) owns through the block table.
#include <cstdint>

#include "logismos_kernels.h"

extern "C" {

int64_t logismos_build_packing(const int32_t* cached_lens, const int32_t* new_lens, int32_t n_seqs,
                               const int32_t* block_tables, int32_t max_blocks, int32_t block_size,
                               int32_t n_pool_blocks, int32_t* cu_seqlens, int32_t* positions,
                               int64_t* slot_mapping, int32_t* seq_ids) {
  if (n_seqs < 0 || max_blocks < 0 || block_size <= 0) return -1;
  int64_t total = 0;
  cu_seqlens[0] = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    if (cached_lens[i] < 0 || new_lens[i] < 0) return -1;
    for (int32_t j = 0; j < new_lens[i]; ++j) {
      const int64_t pos = (int64_t)cached_lens[i] + j;
      const int64_t bi = pos / block_size;
      if (bi >= max_blocks) return -1;
      const int32_t blk = block_tables[(int64_t)i * max_blocks + bi];
      if (blk < 0 || blk >= n_pool_blocks) return -1;
      if (total >= 2147483647ll) return -1;
      positions[total] = (int32_t)pos;
      slot_mapping[total] = (int64_t)blk * block_size + pos % block_size;
      seq_ids[total] = i;
      ++total;
    }
    cu_seqlens[i + 1] = (int32_t)total;
  }
  return total;
}

int32_t logismos_build_decode_chunks(const int32_t* context_lens, int32_t n_seqs, int32_t chunk_tokens,
                                     int32_t* chunk_offsets) {
  if (n_seqs < 0 || chunk_tokens <= 0) return -1;
  int64_t total = 0;
  chunk_offsets[0] = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    const int64_t len = context_lens[i] > 0 ? context_lens[i] : 0;
    total += (len + chunk_tokens - 1) / chunk_tokens;
    if (total > 2147483647ll) return -1;
    chunk_offsets[i + 1] = (int32_t)total;
  }
  return (int32_t)total;
}

}  // extern "C"
