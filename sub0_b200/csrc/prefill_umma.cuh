// Interface between the C-ABI entry point (prefill.cu) and the tcgen05 prefill kernel (prefill_umma.cu).
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace cda {

struct PrefillUmmaParams {
  const __half* q;
  __half* out;
  const int32_t* cu_q;
  const uint8_t* cache;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const float* cb_k;
  const float* cb_v;
  const __half* k_dense;   // dense source (k_bits == v_bits == 16): rotated-frame fp16 rows (row, H_kv, 128); seq_lens then
  const __half* v_dense;   // holds the number of valid keys per sequence and cu_k the first row of each sequence
  const int32_t* cu_k;
  unsigned long long wait_limit_ns;   // limit of every mbarrier wait (set by the launcher)
  int withhold_first_k;               // diagnostic: the producers keep back the first "K tile full" arrive
  int block_size, bs_shift, bt_stride, num_blocks;   // bs_shift: log2(block_size), or -1 if it is not a power of two
  int H_q, H_kv, group;
  float scale_log2;
};

// Launch the causal varlen prefill over the paged cache (k_bits, v_bits in {2, 4}) or over dense rotated rows (16, 16).
int dispatch_prefill_umma(const PrefillUmmaParams& p, int k_bits, int v_bits, int max_query_len, int B, cudaStream_t st);

}  // namespace cda
