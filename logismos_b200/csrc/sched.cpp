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
    // a context counts the token being decoded, so it is never empty; the decode launch relies on it
    // (a sequence without a chunk would leave its output row unwritten)
    if (context_lens[i] < 1) return -1;
    const int64_t len = context_lens[i];
    total += (len + chunk_tokens - 1) / chunk_tokens;
    if (total > 2147483647ll) return -1;
    chunk_offsets[i + 1] = (int32_t)total;
  }
  return (int32_t)total;
}

// Tokens per chunk of the paged-attention decode launch for one step's contexts. Longer chunks mean
// fewer partial results to write and merge, as long as enough CTAs (chunks x kv heads) remain; measured
// on 148 SMs the largest of 512, 1024, 2048 that leaves at least 32768 / head_dim CTAs is the fastest:
// head_dim 128, 256 sequences log-uniform in [128, 32768]: 305 / 258 / 243 us; head_dim 256, 256
// sequences of 1-2 K tokens: 215 / 191 / 182 us; 32 such sequences: 38 / 33 / 53 us.
int32_t logismos_pick_decode_chunk(const int32_t* context_lens, int32_t n_seqs, int32_t n_kv_heads, int32_t head_dim) {
  int32_t best = 512;
  if (n_seqs <= 0 || n_kv_heads <= 0 || head_dim <= 0) return best;
  const int64_t min_ctas = 32768 / head_dim;
  const int32_t cands[2] = {1024, 2048};
  for (int32_t c : cands) {
    int64_t chunks = 0;
    for (int32_t i = 0; i < n_seqs; ++i) chunks += ((int64_t)(context_lens[i] > 0 ? context_lens[i] : 0) + c - 1) / c;
    if (chunks * n_kv_heads >= min_ctas) best = c;
  }
  return best;
}

}  // extern "C"
