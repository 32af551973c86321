// Dense helpers of the prefill path: (1) gather + decode of the paged cache to dense rotated-frame fp16 (and the flat
// variant for separately stored indices and norms), (2) causal variable-length flash attention over such dense
// rotated-frame K/V with the Hadamard rotation of Q fused in front and the inverse rotation of O fused behind, and the
// C-ABI entry points of the whole prefill path.  The fused paged prefill kernel itself lives in prefill_umma.cu.
//
// Attention kernel (dense_prefill_kernel): one CTA = 4 warps = 64 query rows of one (sequence, query head); each warp
// owns 16 rows, keeps its rotated Q fragments in registers and walks the allowed keys 64 at a time: tiles of decoded
// rotated K/V rows are copied with cp.async into XOR-swizzled [64][128] fp16 tiles; S = Q K^T and O += P V run on
// mma.m16n8k16 (fp16 in, fp32 accumulate) with ldmatrix operand loads.
// Epilogue: O/l is rounded to fp16, staged in shared memory, rotated back by butterflies and stored.
#include <cmath>

#include "common.cuh"
#include "prefill_umma.cuh"

namespace cda {

// ---- dense loader -----------------------------------------------------------------------------------------------------------
template <int KB, int VB>
__global__ void __launch_bounds__(256) cache_to_dense_kernel(const uint8_t* __restrict__ cache, const int32_t* __restrict__ block_table,
                                                             const int32_t* __restrict__ seq_lens, const float* __restrict__ cb_k,
                                                             const float* __restrict__ cb_v, __half* __restrict__ k_out,
                                                             __half* __restrict__ v_out, int64_t rows, int H_kv, int block_size,
                                                             int bt_stride, int max_seq_len, int num_blocks, int slot_bytes) {
  __shared__ float s_cb[2][16];
  if (threadIdx.x < 16) {
    s_cb[0][threadIdx.x] = threadIdx.x < (KB == 4 ? 16 : 4) ? cb_k[threadIdx.x] : 0.f;
    s_cb[1][threadIdx.x] = threadIdx.x < (VB == 4 ? 16 : 4) ? cb_v[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);   // ((b * max_seq_len) + n) * H_kv + h
  if (row >= rows) return;
  const int h = static_cast<int>(row % H_kv);
  const int64_t bn = row / H_kv;
  const int n = static_cast<int>(bn % max_seq_len), b = static_cast<int>(bn / max_seq_len);
  uint2 kz = make_uint2(0u, 0u), vz = make_uint2(0u, 0u);
  if (n < seq_lens[b]) {
    int blk = block_table[static_cast<int64_t>(b) * bt_stride + n / block_size];
    if (blk < 0 || blk >= num_blocks) blk = 0;
    const uint8_t* slot = cache + ((static_cast<int64_t>(blk) * block_size + n % block_size) * H_kv + h) * slot_bytes;
    const float nk = *reinterpret_cast<const float*>(slot + 16 * KB + 16 * VB);
    const float nv = *reinterpret_cast<const float*>(slot + 16 * KB + 16 * VB + 4);
    int ik[4], iv[4];
    if (KB == 4) { const uint8_t b0 = slot[2 * lane], b1 = slot[2 * lane + 1]; ik[0] = b0 >> 4; ik[1] = b0 & 15; ik[2] = b1 >> 4; ik[3] = b1 & 15; }
    else { const uint8_t b0 = slot[lane]; ik[0] = b0 >> 6; ik[1] = (b0 >> 4) & 3; ik[2] = (b0 >> 2) & 3; ik[3] = b0 & 3; }
    const uint8_t* vs = slot + 16 * KB;
    if (VB == 4) { const uint8_t b0 = vs[2 * lane], b1 = vs[2 * lane + 1]; iv[0] = b0 >> 4; iv[1] = b0 & 15; iv[2] = b1 >> 4; iv[3] = b1 & 15; }
    else { const uint8_t b0 = vs[lane]; iv[0] = b0 >> 6; iv[1] = (b0 >> 4) & 3; iv[2] = (b0 >> 2) & 3; iv[3] = b0 & 3; }
    float kf[4], vf[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { kf[i] = s_cb[0][ik[i]] * nk; vf[i] = s_cb[1][iv[i]] * nv; }   // Compressor.decode, compression.py:356-360
    kz = pack_half4(kf);
    vz = pack_half4(vf);
  }
  *reinterpret_cast<uint2*>(k_out + row * kHeadDim + 4 * lane) = kz;
  *reinterpret_cast<uint2*>(v_out + row * kHeadDim + 4 * lane) = vz;
}

// Flat variant for the "dequantise, then dense attention" baseline: one row = one (key, KV head); indices and norms in
// separate tensors (Compressor.encode's CompressedSlot, cda/algorithm/compression.py:196-205).
template <int BITS>
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const uint8_t* __restrict__ idx, const float* __restrict__ norm,
                                                              const float* __restrict__ cb, __half* __restrict__ out, int64_t rows) {
  __shared__ float s_cb[16];
  if (threadIdx.x < 16) s_cb[threadIdx.x] = threadIdx.x < (BITS == 4 ? 16 : 4) ? cb[threadIdx.x] : 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += static_cast<int64_t>(gridDim.x) * 8) {
    const uint8_t* src = idx + row * (16 * BITS);
    const float n = norm[row];
    int i4[4];
    if (BITS == 4) { const uint8_t b0 = src[2 * lane], b1 = src[2 * lane + 1]; i4[0] = b0 >> 4; i4[1] = b0 & 15; i4[2] = b1 >> 4; i4[3] = b1 & 15; }
    else { const uint8_t b0 = src[lane]; i4[0] = b0 >> 6; i4[1] = (b0 >> 4) & 3; i4[2] = (b0 >> 2) & 3; i4[3] = b0 & 3; }
    float f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = s_cb[i4[i]] * n;      // Compressor.decode, compression.py:356-360
    *reinterpret_cast<uint2*>(out + row * kHeadDim + 4 * lane) = pack_half4(f);
  }
}

// ---- attention ------------------------------------------------------------------------------------------------------------------
constexpr int kPfWarps = 4;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kBM = 64;    // query rows per CTA
constexpr int kBN = 64;    // keys per tile
constexpr int kTileBytes = kBN * kHeadDim * 2;   // 16 KB

struct PrefillParams {
  const __half* q;
  __half* out;
  const int32_t* cu_q;
  const __half* k_rot;
  const __half* v_rot;
  const int32_t* cu_k;
  const int32_t* seqused_k;
  int H_q, H_kv, group;
  float scale_log2;
};
constexpr int kDenseSmem = 2 * kTileBytes;     // [K tile | V tile]; Q and the output are staged in the K tile

// byte offset of 16-byte chunk `ch` (0..15) of row `row` in a swizzled [rows][128] fp16 tile
__device__ __forceinline__ int tile_off(int row, int ch) { return row * 256 + ((ch ^ (row & 7)) << 4); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__global__ void __launch_bounds__(kPfThreads) dense_prefill_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* k_tile = smem;
  uint8_t* v_tile = smem + kTileBytes;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int mblk = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int i0 = mblk * kBM;
  if (i0 >= q_len) return;
  const int k_len = p.seqused_k[b];
  const int offset = k_len - q_len;                     // query i sees keys 0 .. i + offset
  const int head = hq / p.group;
  int k_hi = i0 + kBM + offset;                         // exclusive bound of keys any row of this CTA may see
  k_hi = k_hi < k_len ? k_hi : k_len;
  const int n_tiles = k_hi > 0 ? (k_hi + kBN - 1) / kBN : 0;

  // ---- rotate the 16 query rows of this warp and stage them (swizzled) in the K tile ---------------------------------------
  for (int rr = 0; rr < 16; ++rr) {
    const int row = warp * 16 + rr, i = i0 + row;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (i < q_len) {
      load_half4(p.q + (static_cast<int64_t>(q_begin + i) * p.H_q + hq) * kHeadDim + 4 * lane, v);
      fht128_warp(v, lane);
#pragma unroll
      for (int t = 0; t < 4; ++t) v[t] *= kRsqrtD;
    }
    *reinterpret_cast<uint2*>(k_tile + tile_off(row, lane >> 1) + 8 * (lane & 1)) = pack_half4(v);
  }
  __syncwarp();
  uint32_t qa[8][4];
  {
    const uint32_t base = smem_addr(k_tile);
    const int row = warp * 16 + (lane & 15), chsel = lane >> 4;     // matrices: (rows 0-7,k lo) (rows 8-15,k lo) (rows 0-7,k hi) (rows 8-15,k hi)
#pragma unroll
    for (int s = 0; s < 8; ++s) ldmatrix_x4(base + tile_off(row, 2 * s + chsel), qa[s][0], qa[s][1], qa[s][2], qa[s][3]);
  }

  // ---- producer -------------------------------------------------------------------------------------------------------------------------
  auto issue_dense = [&](int kt) {        // fp16 rows of tile kt -> swizzled K and V tiles
    const int64_t k0 = p.cu_k[b];
    for (int ch = tid; ch < kBN * 16; ch += kPfThreads) {
      const int tok = ch >> 4, piece = ch & 15;
      const int n = kt * kBN + tok;
      if (n < k_len) {
        const int64_t off = ((k0 + n) * p.H_kv + head) * kHeadDim + piece * 8;
        cp_async16(smem_addr(k_tile + tile_off(tok, piece)), p.k_rot + off);
        cp_async16(smem_addr(v_tile + tile_off(tok, piece)), p.v_rot + off);
      } else {
        *reinterpret_cast<uint4*>(k_tile + tile_off(tok, piece)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(v_tile + tile_off(tok, piece)) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows r, r+8
  float oacc[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) oacc[n][i] = 0.f;

  __syncthreads();   // every warp has its Q fragments: the K tile may be overwritten

  const int row_lo = i0 + warp * 16 + r;     // query index of accumulator rows (c0,c1); (c2,c3) are row_lo + 8
#pragma unroll 1
  for (int kt = 0; kt < n_tiles; ++kt) {
    issue_dense(kt);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // ---- S = Q K^T (16 x 64 per warp) ---------------------------------------------------------------------------------------------------
    float sacc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) sacc[n][i] = 0.f;
    {
      const uint32_t kbase = smem_addr(k_tile);
      // one ldmatrix.x4 = two key octets x one k-step: lanes 0-7 (keys n0..+7, k lo) 8-15 (same keys, k hi) 16-23 (keys +8, k lo) 24-31 (keys +8, k hi)
      const int krow = (lane & 7) + ((lane >> 4) << 3), kch = (lane >> 3) & 1;
#pragma unroll
      for (int s = 0; s < 8; ++s)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(kbase + tile_off(np * 16 + krow, 2 * s + kch), b0, b1, b2, b3);
          mma_16816(sacc[2 * np], qa[s][0], qa[s][1], qa[s][2], qa[s][3], b0, b1);
          mma_16816(sacc[2 * np + 1], qa[s][0], qa[s][1], qa[s][2], qa[s][3], b2, b3);
        }
    }
    // ---- softmax scale * log2e, causal / length mask, online softmax ---------------------------------------------------------
    const int key0 = kt * kBN;
    const bool need_mask = key0 + kBN - 1 > i0 + warp * 16 + offset || key0 + kBN > k_len;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      sacc[n][0] *= p.scale_log2; sacc[n][1] *= p.scale_log2; sacc[n][2] *= p.scale_log2; sacc[n][3] *= p.scale_log2;
      if (need_mask) {
        const int key = key0 + n * 8 + 2 * c;
        const int lim0 = row_lo + offset, lim1 = row_lo + 8 + offset;    // last visible key of each row
        if (key > lim0 || key >= k_len) sacc[n][0] = -INFINITY;
        if (key + 1 > lim0 || key + 1 >= k_len) sacc[n][1] = -INFINITY;
        if (key > lim1 || key >= k_len) sacc[n][2] = -INFINITY;
        if (key + 1 > lim1 || key + 1 >= k_len) sacc[n][3] = -INFINITY;
      }
      mx[0] = fmaxf(mx[0], fmaxf(sacc[n][0], sacc[n][1]));
      mx[1] = fmaxf(mx[1], fmaxf(sacc[n][2], sacc[n][3]));
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    float ms[2], fs[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float mn = fmaxf(m_run[i], mx[i]);
      ms[i] = mn == -INFINITY ? 0.f : mn;
      fs[i] = fast_exp2(m_run[i] - ms[i]);
      m_run[i] = mn;
      l_run[i] *= fs[i];
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) { oacc[n][0] *= fs[0]; oacc[n][1] *= fs[0]; oacc[n][2] *= fs[1]; oacc[n][3] *= fs[1]; }

    uint32_t pa[4][4];   // probabilities as A fragments: k-step s covers keys 16s .. 16s+15
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = fast_exp2(sacc[n][0] - ms[0]), p1 = fast_exp2(sacc[n][1] - ms[0]);
      const float p2 = fast_exp2(sacc[n][2] - ms[1]), p3 = fast_exp2(sacc[n][3] - ms[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pa[n >> 1][(n & 1) * 2] = pack_half2(p0, p1);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_half2(p2, p3);
    }
    // ---- O += P V -----------------------------------------------------------------------------------------------------------------------------
    {
      const uint32_t vbase = smem_addr(v_tile);
      // transposed load: lanes 0-7 (keys k0..+7, dims d0..+7) 8-15 (keys +8, same dims) 16-23 (keys k0.., dims +8) 24-31 (keys +8, dims +8)
      const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3), vch = lane >> 4;
#pragma unroll
      for (int s = 0; s < 4; ++s)
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vbase + tile_off(s * 16 + vrow, 2 * dp + vch), b0, b1, b2, b3);
          mma_16816(oacc[2 * dp], pa[s][0], pa[s][1], pa[s][2], pa[s][3], b0, b1);
          mma_16816(oacc[2 * dp + 1], pa[s][0], pa[s][1], pa[s][2], pa[s][3], b2, b3);
        }
    }
    __syncthreads();   // the tiles are refilled at the top of the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();                 // all warps are done with the K/V tiles: reuse the K tile for the output

  // ---- epilogue: normalise, round to fp16, rotate back, store --------------------------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
  {
    const int row0 = warp * 16 + r, row1 = row0 + 8;
#pragma unroll
    for (int n = 0; n < 16; ++n) {     // accumulator n holds coordinates 8n + 2c, 8n + 2c + 1
      *reinterpret_cast<uint32_t*>(k_tile + tile_off(row0, n) + 4 * c) = pack_half2(oacc[n][0] * inv0, oacc[n][1] * inv0);
      *reinterpret_cast<uint32_t*>(k_tile + tile_off(row1, n) + 4 * c) = pack_half2(oacc[n][2] * inv1, oacc[n][3] * inv1);
    }
  }
  __syncwarp();
  for (int rr = 0; rr < 16; ++rr) {
    const int row = warp * 16 + rr, i = i0 + row;
    if (i >= q_len) break;
    float v[4];
    const uint2 raw = *reinterpret_cast<const uint2*>(k_tile + tile_off(row, lane >> 1) + 8 * (lane & 1));
    const __half2 lo = *reinterpret_cast<const __half2*>(&raw.x), hi = *reinterpret_cast<const __half2*>(&raw.y);
    v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
    fht128_warp(v, lane);
#pragma unroll
    for (int t = 0; t < 4; ++t) v[t] *= kRsqrtD;
    *reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(q_begin + i) * p.H_q + hq) * kHeadDim + 4 * lane) = pack_half4(v);
  }
}

static int launch_dense_prefill(const PrefillParams& p, int max_query_len, int B, cudaStream_t st) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(dense_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmem) != cudaSuccess)
      return check_launch("prefill: shared memory opt-in");
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid((max_query_len + kBM - 1) / kBM, p.H_q, B);
  dense_prefill_kernel<<<grid, kPfThreads, kDenseSmem, st>>>(p);
  return check_launch("dense prefill kernel");
}

}  // namespace cda

using namespace cda;

extern "C" int cda_b200_cache_to_dense_rotated(const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                               const float* cb_K, const float* cb_V, void* k_out, void* v_out, int B, int H_kv,
                                               int block_size, int block_table_stride, int max_seq_len, int64_t num_slots,
                                               int slot_bytes, int k_bits, int v_bits, void* stream) {
  if (B < 0 || H_kv <= 0 || max_seq_len < 0 || num_slots < 0) return fail(CDA_ERR_BAD_ARG, "cache_to_dense_rotated: bad size");
  if (!bits_ok(k_bits) || !bits_ok(v_bits)) return fail(CDA_ERR_UNSUPPORTED, "cache_to_dense_rotated: bits must be 2 or 4");
  if (slot_bytes != slot_bytes_for(k_bits, v_bits)) return fail(CDA_ERR_BAD_SHAPE, "cache_to_dense_rotated: slot width %d does not fit k%dv%d", slot_bytes, k_bits, v_bits);
  if (block_size <= 0 || block_size % 16) return fail(CDA_ERR_BAD_SHAPE, "cache_to_dense_rotated: block_size=%d is not a multiple of 16", block_size);
  if (static_cast<int64_t>(block_table_stride) * block_size < max_seq_len) return fail(CDA_ERR_BAD_SHAPE, "cache_to_dense_rotated: block table row shorter than max_seq_len");
  const int64_t rows = static_cast<int64_t>(B) * max_seq_len * H_kv;
  if (rows == 0) return CDA_OK;
  if (!kv_cache || !block_table || !seq_lens || !cb_K || !cb_V || !k_out || !v_out) return fail(CDA_ERR_BAD_ARG, "cache_to_dense_rotated: null pointer");
  if ((reinterpret_cast<uintptr_t>(k_out) & 7u) || (reinterpret_cast<uintptr_t>(v_out) & 7u))
    return fail(CDA_ERR_BAD_ALIGN, "cache_to_dense_rotated: k_out and v_out must be 8-byte aligned");
  const int64_t blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "cache_to_dense_rotated: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* c = static_cast<const uint8_t*>(kv_cache);
  __half* ko = static_cast<__half*>(k_out);
  __half* vo = static_cast<__half*>(v_out);
  const int nb = static_cast<int>(num_slots / block_size);
  const unsigned g = static_cast<unsigned>(blocks);
#define CDA_LAUNCH_DENSE(KBv, VBv) cache_to_dense_kernel<KBv, VBv><<<g, 256, 0, st>>>(c, block_table, seq_lens, cb_K, cb_V, ko, vo, rows, H_kv, block_size, block_table_stride, max_seq_len, nb, slot_bytes)
  if (k_bits == 4 && v_bits == 4) CDA_LAUNCH_DENSE(4, 4);
  else if (k_bits == 4 && v_bits == 2) CDA_LAUNCH_DENSE(4, 2);
  else if (k_bits == 2 && v_bits == 2) CDA_LAUNCH_DENSE(2, 2);
  else CDA_LAUNCH_DENSE(2, 4);
#undef CDA_LAUNCH_DENSE
  return check_launch("cache_to_dense_rotated");
}

extern "C" int cda_b200_dequantize_rows(const void* idx, const float* norm, const float* cb, void* out, int64_t rows, int bits,
                                       void* stream) {
  if (rows < 0) return fail(CDA_ERR_BAD_ARG, "dequantize_rows: negative rows");
  if (!bits_ok(bits)) return fail(CDA_ERR_UNSUPPORTED, "dequantize_rows: bits must be 2 or 4");
  if (rows == 0) return CDA_OK;
  if (!idx || !norm || !cb || !out) return fail(CDA_ERR_BAD_ARG, "dequantize_rows: null pointer");
  if (reinterpret_cast<uintptr_t>(out) & 7u) return fail(CDA_ERR_BAD_ALIGN, "dequantize_rows: out must be 8-byte aligned");
  const int64_t want = (rows + 7) / 8, cap = static_cast<int64_t>(device_sm_count(-1)) * 8;
  const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bits == 4)
    dequantize_rows_kernel<4><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(idx), norm, cb, static_cast<__half*>(out), rows);
  else
    dequantize_rows_kernel<2><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(idx), norm, cb, static_cast<__half*>(out), rows);
  return check_launch("dequantize_rows");
}

static int prefill_common_checks(const char* who, const void* Q, void* out, const int32_t* cu_q, int64_t T, int B, int H_q, int H_kv,
                                 int max_query_len) {
  if (T < 0 || B < 0 || H_q <= 0 || H_kv <= 0 || max_query_len < 0) return fail(CDA_ERR_BAD_ARG, "%s: bad size", who);
  if (H_q % H_kv) return fail(CDA_ERR_BAD_SHAPE, "%s: H_q=%d is not a multiple of H_kv=%d", who, H_q, H_kv);
  if (B == 0 || T == 0 || max_query_len == 0) return 1;   // nothing to do
  if (!Q || !out || !cu_q) return fail(CDA_ERR_BAD_ARG, "%s: null pointer", who);
  if ((reinterpret_cast<uintptr_t>(Q) & 7u) || (reinterpret_cast<uintptr_t>(out) & 7u)) return fail(CDA_ERR_BAD_ALIGN, "%s: Q/out must be 8-byte aligned", who);
  if (B > 65535 || H_q > 65535) return fail(CDA_ERR_N_TOO_LARGE, "%s: B or H_q exceeds the grid limit", who);
  return CDA_OK;
}

extern "C" int cda_b200_prefill_varlen(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* cu_seqlens_q,
                                       const int32_t* seq_lens, const float* cb_K, const float* cb_V, void* out, int64_t T, int B,
                                       int H_q, int H_kv, int block_size, int block_table_stride, int max_query_len, int max_seq_len,
                                       int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale, void* stream) {
  int rc = prefill_common_checks("prefill_varlen", Q, out, cu_seqlens_q, T, B, H_q, H_kv, max_query_len);
  if (rc == 1) return CDA_OK;
  if (rc != CDA_OK) return rc;
  if (!bits_ok(k_bits) || !bits_ok(v_bits)) return fail(CDA_ERR_UNSUPPORTED, "prefill_varlen: bits must be 2 or 4");
  if (slot_bytes != slot_bytes_for(k_bits, v_bits)) return fail(CDA_ERR_BAD_SHAPE, "prefill_varlen: slot width %d does not fit k%dv%d", slot_bytes, k_bits, v_bits);
  if (block_size <= 0 || block_size % 16) return fail(CDA_ERR_BAD_SHAPE, "prefill_varlen: block_size=%d is not a multiple of 16", block_size);
  if (static_cast<int64_t>(block_table_stride) * block_size < max_seq_len) return fail(CDA_ERR_BAD_SHAPE, "prefill_varlen: block table row shorter than max_seq_len");
  if (!kv_cache || !block_table || !seq_lens || !cb_K || !cb_V) return fail(CDA_ERR_BAD_ARG, "prefill_varlen: null pointer");
  if (!aligned16(kv_cache)) return fail(CDA_ERR_BAD_ALIGN, "prefill_varlen: cache must be 16-byte aligned");
  if (!aligned16(Q) || !aligned16(out)) return fail(CDA_ERR_BAD_ALIGN, "prefill_varlen: Q and out must be 16-byte aligned");
  if (H_q / H_kv > 8) return fail(CDA_ERR_UNSUPPORTED, "prefill_varlen: GQA group %d > 8", H_q / H_kv);
  PrefillUmmaParams p{};
  p.q = static_cast<const __half*>(Q); p.out = static_cast<__half*>(out); p.cu_q = cu_seqlens_q;
  p.cache = static_cast<const uint8_t*>(kv_cache); p.block_table = block_table; p.seq_lens = seq_lens;
  p.cb_k = cb_K; p.cb_v = cb_V; p.block_size = block_size; p.bt_stride = block_table_stride;
  p.bs_shift = -1;
  for (int sft = 4; sft < 31; ++sft) if ((1 << sft) == block_size) p.bs_shift = sft;
  p.num_blocks = static_cast<int>(num_slots / block_size);
  p.H_q = H_q; p.H_kv = H_kv; p.group = H_q / H_kv; p.scale_log2 = scale * kLog2e;
  return dispatch_prefill_umma(p, k_bits, v_bits, max_query_len, B, static_cast<cudaStream_t>(stream));
}

static int dense_mma_sync(const void* Q, const void* k_rot, const void* v_rot, void* out, const int32_t* cu_seqlens_q,
                          const int32_t* cu_seqlens_k, const int32_t* seqused_k, int B, int H_q, int H_kv, int max_query_len, float scale,
                          void* stream) {
  PrefillParams p{};
  p.q = static_cast<const __half*>(Q); p.out = static_cast<__half*>(out); p.cu_q = cu_seqlens_q;
  p.k_rot = static_cast<const __half*>(k_rot); p.v_rot = static_cast<const __half*>(v_rot);
  p.cu_k = cu_seqlens_k; p.seqused_k = seqused_k;
  p.H_q = H_q; p.H_kv = H_kv; p.group = H_q / H_kv; p.scale_log2 = scale * kLog2e;
  return launch_dense_prefill(p, max_query_len, B, static_cast<cudaStream_t>(stream));
}

extern "C" int cda_b200_varlen_fwd_hadamard(const void* Q, const void* k_rot, const void* v_rot, void* out, const int32_t* cu_seqlens_q,
                                            const int32_t* cu_seqlens_k, const int32_t* seqused_k, int64_t T, int B, int H_q, int H_kv,
                                            int max_query_len, int max_seq_len, float scale, void* stream) {
  (void)max_seq_len;
  int rc = prefill_common_checks("varlen_fwd_hadamard", Q, out, cu_seqlens_q, T, B, H_q, H_kv, max_query_len);
  if (rc == 1) return CDA_OK;
  if (rc != CDA_OK) return rc;
  if (!k_rot || !v_rot || !cu_seqlens_k || !seqused_k) return fail(CDA_ERR_BAD_ARG, "varlen_fwd_hadamard: null pointer");
  if (!aligned16(k_rot) || !aligned16(v_rot)) return fail(CDA_ERR_BAD_ALIGN, "varlen_fwd_hadamard: K/V must be 16-byte aligned");
  // The tcgen05 kernel with dense-source producers; it moves Q and the output in 16-byte pieces and serves GQA groups up to
  // 8.  Anything else (8-byte aligned Q / out, wider groups) goes to the mma.sync kernel.
  if (!aligned16(Q) || !aligned16(out) || H_q / H_kv > 8)
    return dense_mma_sync(Q, k_rot, v_rot, out, cu_seqlens_q, cu_seqlens_k, seqused_k, B, H_q, H_kv, max_query_len, scale, stream);
  PrefillUmmaParams p{};
  p.q = static_cast<const __half*>(Q); p.out = static_cast<__half*>(out); p.cu_q = cu_seqlens_q;
  p.seq_lens = seqused_k; p.cu_k = cu_seqlens_k;
  p.k_dense = static_cast<const __half*>(k_rot); p.v_dense = static_cast<const __half*>(v_rot);
  p.block_size = 16; p.bs_shift = 4;
  p.H_q = H_q; p.H_kv = H_kv; p.group = H_q / H_kv; p.scale_log2 = scale * kLog2e;
  return dispatch_prefill_umma(p, 16, 16, max_query_len, B, static_cast<cudaStream_t>(stream));
}

// The same contract on the FlashAttention-2-style mma.sync kernel: an independent implementation kept as a cross-check
// of the tcgen05 path (and used by it for inputs that are only 8-byte aligned).
extern "C" int cda_b200_varlen_fwd_hadamard_mma(const void* Q, const void* k_rot, const void* v_rot, void* out,
                                                const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* seqused_k,
                                                int64_t T, int B, int H_q, int H_kv, int max_query_len, int max_seq_len, float scale,
                                                void* stream) {
  (void)max_seq_len;
  int rc = prefill_common_checks("varlen_fwd_hadamard_mma", Q, out, cu_seqlens_q, T, B, H_q, H_kv, max_query_len);
  if (rc == 1) return CDA_OK;
  if (rc != CDA_OK) return rc;
  if (!k_rot || !v_rot || !cu_seqlens_k || !seqused_k) return fail(CDA_ERR_BAD_ARG, "varlen_fwd_hadamard_mma: null pointer");
  if (!aligned16(k_rot) || !aligned16(v_rot)) return fail(CDA_ERR_BAD_ALIGN, "varlen_fwd_hadamard_mma: K/V must be 16-byte aligned");
  return dense_mma_sync(Q, k_rot, v_rot, out, cu_seqlens_q, cu_seqlens_k, seqused_k, B, H_q, H_kv, max_query_len, scale, stream);
}
