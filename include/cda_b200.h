/*
 * cda_b200.h -- C ABI of the B200 (sm_100a) compressed-domain attention library, libcda_b200.so.
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream (passed as void*,
 * i.e. a cudaStream_t).  Unless a function says otherwise it allocates nothing, never synchronises,
 * only enqueues work on `stream` (so it can be captured into a CUDA graph) and returns CDA_OK or a
 * negative status; cda_b200_last_error_string() describes the most recent failure on the calling
 * thread.  The caller owns every buffer, including the split-KV workspace.
 *
 * Each declaration names the reference interface it stands in for.  The reference ships these as
 * closed pybind11 modules (cda/_prebuilt/ *.so) whose call sites are in
 * cda/kernels_cuda/wrappers.py and cda/kernels_cuda/fa2_cda.py; paths below are relative to the
 * reference project.
 *
 * Common conventions
 *   head_dim          128 (fixed, cda_attn_v2.py:51).
 *   k_bits / v_bits   4 (16-level codebook) or 2 (4-level codebook); codebooks are fp32 device arrays,
 *                     sorted ascending.
 *   slot layout       per token and KV head, `slot_bytes` = cda_b200_slot_bytes(k_bits, v_bits):
 *                       [ K indices 16*k_bits B | V indices 16*v_bits B | fp32 K norm | fp32 V norm | pad ]
 *                     indices packed MSB first (compression.py:163-188, 375-397); 144 B for k4v4
 *                     (cda_attn_v2.py:20-27, 51-60), 112 B for k4v2, 80 B for k2v2.
 *   paged cache       uint8 (num_slots, H_kv, slot_bytes); token n of sequence b lives in slot
 *                     block_table[b][n / block_size] * block_size + n % block_size; block_size % 16 == 0.
 *   rotation          the orthonormal 128-point Sylvester-Hadamard transform (compression.py:43-57),
 *                     applied inside the kernels by butterflies; no rotation matrix is passed.
 */
#ifndef CDA_B200_H_
#define CDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CDA_B200_ABI_VERSION 1
#define CDA_HEAD_DIM 128

enum cda_status {
  CDA_OK = 0,
  CDA_ERR_BAD_ARG = -1,       /* null pointer, negative size */
  CDA_ERR_BAD_SHAPE = -2,     /* H_q not a multiple of H_kv, block_size not a multiple of 16, ... */
  CDA_ERR_BAD_ALIGN = -3,     /* a pointer or slot width is not 16-byte aligned */
  CDA_ERR_UNSUPPORTED = -4,   /* bit width, group size or slot width outside the supported set */
  CDA_ERR_N_TOO_LARGE = -5,   /* sequence / token count exceeds an index range */
  CDA_ERR_WORKSPACE = -6,     /* workspace missing or smaller than *_workspace_bytes() */
  CDA_ERR_LAUNCH = -7         /* the CUDA runtime rejected a launch or attribute call */
};

/* Library version (CDA_B200_ABI_VERSION it was built with). */
int cda_b200_version(void);

/* Message for the last non-OK status returned on this thread ("" if none). */
const char* cda_b200_last_error_string(void);

/* Allocated bytes per (token, KV head) slot, or CDA_ERR_UNSUPPORTED.
 * Replaces the constants _DATA_BYTES_PER_TOKEN / _BYTES_PER_TOKEN (cda_attn_v2.py:56-58). */
int cda_b200_slot_bytes(int k_bits, int v_bits);

/* Fused paged encode: for each new token t and KV head h, Hadamard-rotate K[t,h,:] and V[t,h,:]
 * (result rounded to fp16 as Compressor.rotate does), take the fp32 L2 norm (floor 1e-12), divide,
 * clamp to [-1,1], pick the nearest codebook level with the reference's tie rule, pack and write
 * the payload bytes of slot slot_mapping[t].  Pad bytes are left untouched; entries of slot_mapping
 * that are negative or >= num_slots are skipped.
 *   K, V          (T, H_kv, 128) fp16 contiguous          slot_mapping  (T) int32
 *   flat_cache    (num_slots, H_kv, slot_bytes) uint8      cb_K, cb_V    fp32[16] or fp32[4]
 * Replaces cda_paged_encode_fused(K, V, slot_mapping, flat_cache, cb_K, cb_V), called at
 * cda/kernels_cuda/wrappers.py:153-156; algorithm cda/algorithm/compression.py:315-335. */
int cda_b200_paged_encode(const void* K, const void* V, const int32_t* slot_mapping, void* flat_cache,
                          const float* cb_K, const float* cb_V, int64_t T, int H_kv, int64_t num_slots,
                          int slot_bytes, int k_bits, int v_bits, void* stream);

/* The index-selection half of the encoder on caller-supplied rotated fp32 rows: norm, divide, clamp,
 * nearest level, pack.  idx_out (rows, 16*bits) uint8, norm_out (rows) fp32.  Shares its device code
 * with cda_b200_paged_encode; exists so that index parity can be checked on identical fp32 inputs.
 * Follows Compressor.quantize_unit / encode, cda/algorithm/compression.py:298-335. */
int cda_b200_quantize_rotated(const float* x_rot, int64_t rows, const float* cb, int bits,
                              uint8_t* idx_out, float* norm_out, void* stream);

/* y = scale * FHT128(x) on contiguous fp16 rows (fp32 butterflies, one rounding to fp16); x == y allowed.
 * Replaces hadamard128_fp16(x, y, scale), cda/kernels_cuda/fa2_cda.py:50-53. */
int cda_b200_hadamard128(const void* x, void* y, int64_t rows, float scale, void* stream);

/* Number of partial results per output row (key ranges per sequence) the decode entry points produce when
 * num_splits == 0 is passed.  The planned decomposition cuts the concatenation of all sequences into equal chunks,
 * one per SM, so this is the largest number of chunks one sequence touches.
 * Counterpart of the tile heuristic _choose_tile_n, cda/kernels_cuda/wrappers.py:41-76. */
int cda_b200_decode_plan_splits(int B, int H_kv, int max_seq_len, int device);

/* Bytes of workspace the decode entry points need for these sizes (num_splits == 0: the planned
 * count).  The reference kernel allocates this scratch itself (wrappers.py:97-99); here the caller does.
 * The first 256 bytes are a status block that the caller zeroes once; its first int collects, over the calls that use
 * the workspace:  bit 0 (1) a block-table entry was outside the cache and block 0 was read instead;  bit 1 (2) the
 * kernel's shared-memory window did not fit (empty partials were written);  bit 2 (4) a bounded wait for a cache copy
 * ran out of time;  bit 3 (8) cda_b200_decode_exchange waited in vain for another rank's row. */
size_t cda_b200_decode_workspace_bytes(int B, int H_q, int H_kv, int max_seq_len, int num_splits, int device);

/* Single-query GQA decode over the paged compressed cache: out[b,h,:] = softmax(scale * Hq.K^T) V H^T
 * with K, V decoded from codebook indices in the rotated frame, split over key ranges and merged by
 * log-sum-exp.  Q and out are un-rotated fp16 (B, H_q, 128); sequences with seq_lens[b] == 0 give zeros.
 *   block_table (B, block_table_stride) int32      seq_lens (B) int32, each <= max_seq_len
 *   workspace   >= cda_b200_decode_workspace_bytes(...) bytes, 16-byte aligned
 * Replaces cda_decode_full_hmma_v3(Q, kv_cache, block_table, seq_lens, cb_K, cb_V, rot_fp32, rot_fp16,
 * out, group_size, block_size, tile_N, max_seq_len, scale), cda/kernels_cuda/wrappers.py:115-124;
 * result defined by attention_compressed, cda/algorithm/attention.py:426-482. */
int cda_b200_decode(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                    const float* cb_K, const float* cb_V, void* out, void* workspace, size_t workspace_bytes,
                    int B, int H_q, int H_kv, int block_size, int block_table_stride, int max_seq_len,
                    int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale, int num_splits,
                    void* stream);

/* cda_b200_decode that also returns the log-sum-exp of the scaled scores, lse (B, H_q) fp32, natural log
 * (-inf for a sequence without keys): what an attention backend hands to a cross-rank LSE correction.
 * The reference backend cannot return it (can_return_lse_for_decode = False, cda_attn_v2.py:621). */
int cda_b200_decode_lse(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                        const float* cb_K, const float* cb_V, void* out, float* lse, void* workspace,
                        size_t workspace_bytes, int B, int H_q, int H_kv, int block_size, int block_table_stride,
                        int max_seq_len, int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale,
                        int num_splits, void* stream);

/* Same pass, but returns the un-normalised partial of the keys this cache holds, in the rotated frame:
 * O (B,H_q,128) fp32 = sum exp(s-m) V, m (B,H_q) fp32 = max s (natural-log domain, -inf if no key),
 * l (B,H_q) fp32 = sum exp(s-m).  This is what a sequence-sharded rank contributes.
 * The reference leaves this as NotImplementedError (cda_attn_v2.py:1697-1701); the contract is
 * attention_compressed_partial_reference, cda/algorithm/attention.py:349-384. */
int cda_b200_decode_partial(const void* Q, const void* kv_cache, const int32_t* block_table,
                            const int32_t* seq_lens, const float* cb_K, const float* cb_V, float* O, float* m,
                            float* l, void* workspace, size_t workspace_bytes, int B, int H_q, int H_kv,
                            int block_size, int block_table_stride, int max_seq_len, int64_t num_slots,
                            int slot_bytes, int k_bits, int v_bits, float scale, int num_splits, void* stream);

/* cda_b200_decode_partial writing one packed row per (sequence, query head): packed (B, H_q, 130) fp32 =
 * 128 un-normalised O values, then m, then l -- a single contiguous message for the all-gather of a
 * sequence-sharded decode.  packed must be 8-byte aligned.  Same contract as cda_b200_decode_partial. */
int cda_b200_decode_partial_packed(const void* Q, const void* kv_cache, const int32_t* block_table,
                                   const int32_t* seq_lens, const float* cb_K, const float* cb_V, float* packed,
                                   void* workspace, size_t workspace_bytes, int B, int H_q, int H_kv, int block_size,
                                   int block_table_stride, int max_seq_len, int64_t num_slots, int slot_bytes,
                                   int k_bits, int v_bits, float scale, int num_splits, void* stream);

/* Merge S partials per row: O (S,R,128), m (S,R), l (S,R) fp32 as produced by cda_b200_decode_partial
 * -> out (R,128) fp16; with unrotate != 0 the merged row is rounded to fp16 and rotated back to the model
 * frame (what decode does), otherwise it stays in the rotated frame.
 * Follows merge_partials, cda/algorithm/attention.py:239-272. */
int cda_b200_merge_partials(const float* O, const float* m, const float* l, int S, int64_t R, void* out,
                            int unrotate, void* stream);

/* cda_b200_merge_partials on packed partials (S, R, 130) fp32 as written by cda_b200_decode_partial_packed
 * (e.g. the all-gathered partials of S ranks).  Follows merge_partials, cda/algorithm/attention.py:239-272. */
int cda_b200_merge_partials_packed(const float* packed, int S, int64_t R, void* out, int unrotate, void* stream);

/* Sequence-sharded decode with the exchange inside the merge kernel (no collective library on the data path): every rank
 * holds a different key range of the same sequences and the same Q.  One call = the split kernel over the local keys +
 * one kernel that merges the local pieces, stores this rank's packed row (O[128], m, l, the call's tag) into EVERY rank's
 * exchange buffer with peer stores over NVLink, waits -- at most wait_ms per row -- until every rank's row of this call
 * has arrived in its own buffer, merges them (cda/algorithm/attention.py:239-272) and writes fp16 out (B,H_q,128).  It
 * replaces cda_b200_decode_partial_packed + all-gather + cda_b200_merge_partials_packed; the reference leaves the path as
 * NotImplementedError (cda_attn_v2.py:1697-1701).
 *   peer_buffers: DEVICE array of `world` device pointers; entry p is rank p's exchange buffer of
 *                 cda_b200_decode_exchange_bytes(B, H_q, world) bytes (entry `rank` is this rank's own), zeroed once,
 *                 16-byte aligned, mapped into this process (CUDA IPC or VMM) with peer access enabled;
 *   counters:     two uint64 in THIS rank's device memory, zeroed once (calls completed, rows finished);
 * every rank of the group must make the same sequence of calls with the same B and H_q.  A row that does not arrive in
 * time is left out of the merge and bit 3 of the workspace status word is set; nothing waits without a limit. */
size_t cda_b200_decode_exchange_bytes(int B, int H_q, int world);
/* Exchange buffers for cda_b200_decode_exchange: a zeroed device allocation on the current device (alloc / free), its
 * 64-byte CUDA IPC handle (export), and the mapping of another process's handle into this process with peer access
 * enabled on demand (import / close).  The handles are plain bytes: send them over any channel between the ranks. */
int cda_b200_exchange_alloc(size_t nbytes, void** ptr);
int cda_b200_exchange_free(void* ptr);
int cda_b200_exchange_export(const void* ptr, void* handle64);
int cda_b200_exchange_import(const void* handle64, void** ptr);
int cda_b200_exchange_close(void* ptr);
int cda_b200_decode_exchange(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                             const float* cb_K, const float* cb_V, void* out, void* workspace, size_t workspace_bytes,
                             void* const* peer_buffers, unsigned long long* counters, int rank, int world, int wait_ms,
                             int B, int H_q, int H_kv, int block_size, int block_table_stride, int max_seq_len,
                             int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale, int num_splits,
                             void* stream);

/* cda_b200_decode for callers that cannot hand over a workspace: the split-KV scratch is an 8 MiB array compiled into
 * the library (file-scope device memory; every GPU that loads the library holds it until the process exits).  Meant for
 * hosts where device allocation is off limits at call time -- a runtime whose memory pool is fixed at start-up and
 * handed out in full, a plugin that may only touch the buffers it is given, code running while the allocator is
 * locked.  The call itself allocates nothing (no cudaMalloc / cudaFree, no library that allocates): it clears the
 * 256-byte status block with a stream-ordered memset and launches the same two kernels as cda_b200_decode.
 *   num_splits   0 = planned decomposition; whatever is asked, the number of partials per row is lowered until they
 *                fit in 8 MiB.
 *   returns      CDA_ERR_WORKSPACE (with the sizes in the message) when even one partial per row does not fit, i.e.
 *                when B * H_q * 520 B + 256 (+ 8 when B * H_q is odd: the O rows stay 16-byte aligned) exceeds 8 MiB.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device current);
 * make that first call at start-up and outside any stream capture: with lazy module loading that first call is also
 * when the driver reserves the 8 MiB on that device, so it must come before the host hands out all device memory.  All calls share the one array and it keeps the previous call's
 * contents: calls whose kernels may overlap on the GPU (different streams, or graphs replayed concurrently) race on
 * it -- serialise them or use cda_b200_decode with separate workspaces.
 * Has no counterpart in the reference (its decode kernel allocates its scratch on every call, wrappers.py:97-99). */
int cda_b200_decode_static(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                           const float* cb_K, const float* cb_V, void* out, int B, int H_q, int H_kv, int block_size,
                           int block_table_stride, int max_seq_len, int64_t num_slots, int slot_bytes, int k_bits,
                           int v_bits, float scale, int num_splits, void* stream);
/* Status word of the most recent cda_b200_decode_static call on the current device (each call clears it first; same
 * bits as the caller-owned workspace: 0 block id out of range, 1 shared-memory window too small, 2 a copy wait ran out).
 * Synchronises the device. */
int cda_b200_decode_static_status(int* status);

/* Slow one-warp-per-query-head decode without tensor cores or splitting; decodes K/V exactly as
 * Compressor.decode does (cb[idx]*norm rounded to fp16).  A device-side cross-check, same arguments
 * and result as cda_b200_decode minus the workspace (out 8-byte aligned).  Contract: cda/algorithm/attention.py:426-482. */
int cda_b200_decode_scalar(const void* Q, const void* kv_cache, const int32_t* block_table,
                           const int32_t* seq_lens, const float* cb_K, const float* cb_V, void* out, int B,
                           int H_q, int H_kv, int block_size, int block_table_stride, int64_t num_slots,
                           int slot_bytes, int k_bits, int v_bits, float scale, void* stream);

/* Gather + decode every sequence to dense rotated-frame fp16: k_out, v_out (B*max_seq_len, H_kv, 128), 8-byte aligned,
 * rows at or beyond seq_lens[b] zero.
 * Replaces cda_fa2_paged_cache_to_dense_rotated(kv_cache, block_table, seq_lens, cb_K, cb_V, block_size,
 * max_seq_len), cda/kernels_cuda/fa2_cda.py:86-95 (there the kernel allocates the outputs). */
int cda_b200_cache_to_dense_rotated(const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                    const float* cb_K, const float* cb_V, void* k_out, void* v_out, int B,
                                    int H_kv, int block_size, int block_table_stride, int max_seq_len,
                                    int64_t num_slots, int slot_bytes, int k_bits, int v_bits, void* stream);

/* Causal variable-length prefill straight from the paged compressed cache: Q is rotated in the prologue,
 * K/V tiles are decoded from the cache into shared memory, the output is rotated back in the epilogue.
 * Query i of sequence b (0 <= i < q_len_b = cu_seqlens_q[b+1]-cu_seqlens_q[b]) attends keys
 * 0 .. seq_lens[b]-q_len_b+i (bottom-right alignment, fa2_cda.py:121-125).
 *   Q, out (T, H_q, 128) fp16, 16-byte aligned      cu_seqlens_q (B+1) int32      seq_lens (B) int32
 * Input errors the kernel meets (out-of-range block ids, q_len > seq_len) are reported by cda_b200_prefill_status().
 * Replaces fa2_cda_prefill_varlen_v1(..., fuse_fa2_epilogue=True), cda/kernels_cuda/fa2_cda.py:98-230,
 * i.e. cda_fa2_paged_cache_to_dense_rotated + cda_fa2_varlen_fwd_hadamard without the dense K/V round
 * trip through HBM; result defined by attention_compressed(causal=True), attention.py:426-482. */
int cda_b200_prefill_varlen(const void* Q, const void* kv_cache, const int32_t* block_table,
                            const int32_t* cu_seqlens_q, const int32_t* seq_lens, const float* cb_K,
                            const float* cb_V, void* out, int64_t T, int B, int H_q, int H_kv, int block_size,
                            int block_table_stride, int max_query_len, int max_seq_len, int64_t num_slots,
                            int slot_bytes, int k_bits, int v_bits, float scale, void* stream);

/* The same tcgen05 attention kernel on dense rotated-frame fp16 K/V (sequence b's rows start at cu_seqlens_k[b], valid
 * length seqused_k[b]; K/V 16-byte aligned); Q un-rotated in, out un-rotated.  q_len_b <= seqused_k[b].
 * Replaces cda_fa2_varlen_fwd_hadamard(Q, k_rot, v_rot, out, cu_q, cu_k, seqused_k, max_q, max_k, scale),
 * cda/kernels_cuda/fa2_cda.py:170-181. */
int cda_b200_varlen_fwd_hadamard(const void* Q, const void* k_rot, const void* v_rot, void* out,
                                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                 const int32_t* seqused_k, int64_t T, int B, int H_q, int H_kv,
                                 int max_query_len, int max_seq_len, float scale, void* stream);

/* cda_b200_varlen_fwd_hadamard on the FlashAttention-2-style mma.sync kernel instead of the tcgen05 one: same arguments,
 * same result within the path's tolerance.  An independent implementation kept as a cross-check (the main entry point
 * also falls back to it when Q or out is only 8-byte aligned).  Contract as above, cda/kernels_cuda/fa2_cda.py:170-181. */
int cda_b200_varlen_fwd_hadamard_mma(const void* Q, const void* k_rot, const void* v_rot, void* out,
                                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                     const int32_t* seqused_k, int64_t T, int B, int H_q, int H_kv,
                                     int max_query_len, int max_seq_len, float scale, void* stream);

/* Decode `rows` rows of packed indices (16*bits bytes each) and fp32 norms into fp16 rows of 128: out = fp16(cb[idx] * norm),
 * the rotated-frame K or V the "dequantise, then dense attention" baseline attends over.
 * Replaces the dequant op behind dequantize_compressed_kv(k_idx, k_norm, v_idx, v_norm, cb_k, cb_v),
 * cda/kernels_vllm_fa2_fork/interface.py:138-162 (one call per tensor). */
int cda_b200_dequantize_rows(const void* idx, const float* norm, const float* cb, void* out, int64_t rows, int bits,
                             void* stream);

/* The paged prefill kernel hands tiles between its warps through mbarriers with bounded waits.  A wait that gives up
 * ends its CTA, leaves that CTA's output rows unwritten and sets a per-device flag that makes later prefill CTAs and
 * launches return at once until cda_b200_prefill_clear_status() is called.  Returns 1 if the flag is set on the current
 * device, 0 if not, a negative status on a CUDA error.  Synchronises the device.  (No counterpart in the reference: its
 * kernels report nothing.) */
int cda_b200_prefill_fault(void);

/* What cda_b200_prefill_varlen saw in its inputs on the current device since the last clear (sticky bits; synchronises
 * the device):  bit 0 (1) a block-table entry was outside the cache and block 0 was read instead;  bit 2 (4) a bounded
 * wait gave up;  bit 3 (8) a sequence had more new tokens than tokens (q_len > seq_len) and its rows were left unwritten.
 * Negative status on a CUDA error.  (No counterpart in the reference.) */
int cda_b200_prefill_status(void);

/* Clear the bits of cda_b200_prefill_status and the flag of cda_b200_prefill_fault on the current device. */
int cda_b200_prefill_clear_status(void);

/* Diagnostic knobs for the prefill launches that follow in this process: the limit of every in-kernel wait in
 * microseconds (<= 0: the default, 50 ms) and, if withhold_first_k_arrive != 0, the producers keep back one "tile ready"
 * signal so that the waits behind it run out -- the way the tests exercise the give-up path without faulting anything. */
int cda_b200_prefill_debug(int wait_limit_us, int withhold_first_k_arrive);

#ifdef __cplusplus
}
#endif
#endif /* CDA_B200_H_ */
