// Prefill path: (1) gather + decode of the paged cache to dense rotated-frame fp16, and (2) causal variable-length
// flash attention whose K/V producer decodes codebook indices straight from the paged cache into shared memory,
// with the Hadamard rotation of Q fused in front and the inverse rotation of O fused behind.
//
// Attention kernel (prefill_kernel): one CTA = 4 warps = 64 query rows of one (sequence, query head); each warp
// owns 16 rows, keeps its rotated Q fragments in registers and walks the allowed keys 64 at a time:
//   * PAGED source: the 64 slots of the next tile are fetched with 16-byte cp.async copies into a double-buffered
//     staging area while the current tile is being multiplied; all threads then expand codes through fp16-pair
//     tables into XOR-swizzled [64][128] fp16 K and V tiles.  Norms are not folded into the tiles: the K norm
//     (times scale*log2e) multiplies score columns, the V norm multiplies probabilities.
//   * DENSE source: tiles of already decoded rotated K/V rows are copied with cp.async (norm factors are 1).
//   * S = Q K^T and O += P V run on mma.m16n8k16 (fp16 in, fp32 accumulate) with ldmatrix operand loads.
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
constexpr int kLutRep = 8;                       // table replication (conflict damping) in the prefill kernel

struct PrefillParams {
  const __half* q;
  __half* out;
  const int32_t* cu_q;
  // paged source
  const uint8_t* cache;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const float* cb_k;
  const float* cb_v;
  int block_size, bt_stride, num_blocks;
  // dense source
  const __half* k_rot;
  const __half* v_rot;
  const int32_t* cu_k;
  const int32_t* seqused_k;
  int H_q, H_kv, group;
  float scale_log2;
};

template <int KB, int VB>
struct PfGeom {
  static constexpr int kSlotBytes = 16 * KB + 16 * VB + 16;
  static constexpr int kStagingBytes = kBN * kSlotBytes;
  static constexpr int kLutKWords = (KB == 4 ? 256 : 16) * kLutRep;
  static constexpr int kLutVWords = (VB == 4 ? 256 : 16) * kLutRep;
  // layout: [K tile | V tile | norms (2 x 64 floats) | staging x 2 | lut K | lut V]; Q and the output are staged in the K/V tiles
  static constexpr int kNormOff = 2 * kTileBytes;
  static constexpr int kStageOff = kNormOff + 2 * kBN * 4;
  static constexpr int kLutOff = kStageOff + 2 * kStagingBytes;
  static constexpr int kSmemPaged = kLutOff + (kLutKWords + kLutVWords) * 4;
  static constexpr int kSmemDense = kStageOff;
};

// byte offset of 16-byte chunk `ch` (0..15) of row `row` in a swizzled [rows][128] fp16 tile
__device__ __forceinline__ int tile_off(int row, int ch) { return row * 256 + ((ch ^ (row & 7)) << 4); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <int BITS>
__device__ __forceinline__ void build_lut_rep(uint32_t* lut, const float* __restrict__ cb, int tid, float inv_alpha) {
  constexpr int L = BITS == 4 ? 16 : 4;
  constexpr int E = BITS == 4 ? 256 : 16;
  for (int w = tid; w < E * kLutRep; w += kPfThreads) {
    const int e = w / kLutRep;
    const int first = BITS == 4 ? (e >> 4) : (e >> 2);
    const int second = BITS == 4 ? (e & 15) : (e & 3);
    lut[w] = pack_half2(__ldg(cb + (first & (L - 1))) * inv_alpha, __ldg(cb + (second & (L - 1))) * inv_alpha);
  }
}

// Expand `nbytes` packed index bytes (one 64-coordinate half row when BITS == 4 and nbytes == 32; the whole
// row when BITS == 2) from `src` into the 8 16-byte chunks starting at chunk `ch0` of row `row` of a tile.
template <int BITS>
__device__ __forceinline__ void expand_half_row(const uint8_t* src, const uint32_t* lut, uint8_t* tile, int row, int ch0) {
  // BITS == 4: 32 bytes -> 64 values -> 8 chunks.  BITS == 2: 16 bytes -> 64 values -> 8 chunks.
  constexpr int kWords = BITS == 4 ? 8 : 4;
  uint32_t w[kWords];
#pragma unroll
  for (int i = 0; i < kWords / 4; ++i) {
    const uint4 t = *reinterpret_cast<const uint4*>(src + 16 * i);
    w[4 * i] = t.x; w[4 * i + 1] = t.y; w[4 * i + 2] = t.z; w[4 * i + 3] = t.w;
  }
#pragma unroll
  for (int chn = 0; chn < 8; ++chn) {
    uint32_t v[4];
    if (BITS == 4) {          // chunk = 8 values = 4 bytes = one word
      const uint32_t x = w[chn];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = lut[((x >> (8 * i)) & 0xffu) * kLutRep];
    } else {                  // chunk = 8 values = 2 bytes = half a word
      const uint32_t x = w[chn >> 1] >> (16 * (chn & 1));
      v[0] = lut[((x >> 4) & 0xfu) * kLutRep];
      v[1] = lut[(x & 0xfu) * kLutRep];
      v[2] = lut[((x >> 12) & 0xfu) * kLutRep];
      v[3] = lut[((x >> 8) & 0xfu) * kLutRep];
    }
    *reinterpret_cast<uint4*>(tile + tile_off(row, ch0 + chn)) = make_uint4(v[0], v[1], v[2], v[3]);
  }
}

template <int KB, int VB, bool PAGED>
__global__ void __launch_bounds__(kPfThreads) prefill_kernel(const PrefillParams p) {
  using Gm = PfGeom<KB, VB>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* k_tile = smem;
  uint8_t* v_tile = smem + kTileBytes;
  float* nk_s = reinterpret_cast<float*>(smem + Gm::kNormOff);
  float* nv_s = nk_s + kBN;
  uint8_t* staging = smem + Gm::kStageOff;
  uint32_t* lut_k = reinterpret_cast<uint32_t*>(smem + Gm::kLutOff);
  uint32_t* lut_v = lut_k + Gm::kLutKWords;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int mblk = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int i0 = mblk * kBM;
  if (i0 >= q_len) return;
  const int k_len = PAGED ? p.seq_lens[b] : p.seqused_k[b];
  const int offset = k_len - q_len;                     // query i sees keys 0 .. i + offset
  const int head = hq / p.group;
  int k_hi = i0 + kBM + offset;                         // exclusive bound of keys any row of this CTA may see
  k_hi = k_hi < k_len ? k_hi : k_len;
  const int n_tiles = k_hi > 0 ? (k_hi + kBN - 1) / kBN : 0;

  // fp16 tables hold level / alpha; alpha_k is folded into the score scale, alpha_v into the final normalisation
  float alpha_k = 1.f, alpha_v = 1.f;
  if (PAGED) {
    __shared__ float s_err[64];
    __shared__ int s_idx[64];
    find_table_scales<(KB == 4 ? 16 : 4), (VB == 4 ? 16 : 4)>(p.cb_k, p.cb_v, s_err, s_idx, alpha_k, alpha_v);
    build_lut_rep<KB>(lut_k, p.cb_k, tid, 1.0f / alpha_k);
    build_lut_rep<VB>(lut_v, p.cb_v, tid, 1.0f / alpha_v);
  }
  const float k_scale = p.scale_log2 * alpha_k;

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

  // ---- producer helpers ----------------------------------------------------------------------------------------------------------------
  const int32_t* bt_row = PAGED ? p.block_table + static_cast<int64_t>(b) * p.bt_stride : nullptr;
  auto issue_staging = [&](int kt) {      // PAGED: raw slots of tile kt -> staging[kt & 1]
    uint8_t* dst = staging + (kt & 1) * Gm::kStagingBytes;
    constexpr int kPieces = Gm::kSlotBytes / 16;
    for (int ch = tid; ch < kBN * kPieces; ch += kPfThreads) {
      const int tok = ch / kPieces, piece = ch - tok * kPieces;
      const int n = kt * kBN + tok;
      if (n < k_len) {
        int blk = __ldg(bt_row + n / p.block_size);
        if (blk < 0 || blk >= p.num_blocks) blk = 0;
        const uint8_t* src = p.cache + ((static_cast<int64_t>(blk) * p.block_size + n % p.block_size) * p.H_kv + head) * Gm::kSlotBytes + piece * 16;
        cp_async16(smem_addr(dst + tok * Gm::kSlotBytes + piece * 16), src);
      }
    }
  };
  auto issue_dense = [&](int kt) {        // DENSE: fp16 rows of tile kt -> swizzled K and V tiles
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

  if (PAGED && n_tiles > 0) issue_staging(0);
  cp_async_commit();
  __syncthreads();   // every warp has its Q fragments: the K tile may be overwritten; tables are visible

  const int row_lo = i0 + warp * 16 + r;     // query index of accumulator rows (c0,c1); (c2,c3) are row_lo + 8
#pragma unroll 1
  for (int kt = 0; kt < n_tiles; ++kt) {
    if (PAGED) {
      if (kt + 1 < n_tiles) issue_staging(kt + 1);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      // expand: thread -> (token = tid & 63, coordinate half = tid >> 6)
      const int tok = tid & 63, half = tid >> 6;
      const uint8_t* slot = staging + (kt & 1) * Gm::kStagingBytes + tok * Gm::kSlotBytes;
      expand_half_row<KB>(slot + half * (8 * KB), lut_k + (lane & (kLutRep - 1)), k_tile, tok, 8 * half);
      expand_half_row<VB>(slot + 16 * KB + half * (8 * VB), lut_v + (lane & (kLutRep - 1)), v_tile, tok, 8 * half);
      if (half == 0) {
        const bool ok = kt * kBN + tok < k_len;
        const float2 nn = *reinterpret_cast<const float2*>(slot + 16 * KB + 16 * VB);
        nk_s[tok] = ok ? nn.x * k_scale : 0.f;
        nv_s[tok] = ok ? nn.y : 0.f;
      }
    } else {
      issue_dense(kt);
      cp_async_commit();
      if (tid < kBN) { nk_s[tid] = p.scale_log2; nv_s[tid] = 1.f; }
      cp_async_wait<0>();
    }
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
    // ---- column scale (K norm * scale * log2e), causal / length mask, online softmax ---------------------------------------------------------
    const int key0 = kt * kBN;
    const bool need_mask = key0 + kBN - 1 > i0 + warp * 16 + offset || key0 + kBN > k_len;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float2 f = *reinterpret_cast<const float2*>(nk_s + n * 8 + 2 * c);
      sacc[n][0] *= f.x; sacc[n][1] *= f.y; sacc[n][2] *= f.x; sacc[n][3] *= f.y;
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

    uint32_t pa[4][4];   // probabilities (times V norm) as A fragments: k-step s covers keys 16s .. 16s+15
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = fast_exp2(sacc[n][0] - ms[0]), p1 = fast_exp2(sacc[n][1] - ms[0]);
      const float p2 = fast_exp2(sacc[n][2] - ms[1]), p3 = fast_exp2(sacc[n][3] - ms[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      const float2 g = *reinterpret_cast<const float2*>(nv_s + n * 8 + 2 * c);
      pa[n >> 1][(n & 1) * 2] = pack_half2(p0 * g.x, p1 * g.y);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_half2(p2 * g.x, p3 * g.y);
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
    if (!PAGED) __syncthreads();   // dense tiles are refilled at the top of the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();                 // all warps are done with the K/V tiles: reuse the K tile for the output

  // ---- epilogue: normalise, round to fp16, rotate back, store --------------------------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  const float inv0 = l_run[0] > 0.f ? alpha_v / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? alpha_v / l_run[1] : 0.f;
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

template <int KB, int VB, bool PAGED>
static int launch_prefill(const PrefillParams& p, int max_query_len, int B, cudaStream_t st) {
  using Gm = PfGeom<KB, VB>;
  constexpr int smem = PAGED ? Gm::kSmemPaged : Gm::kSmemDense;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(prefill_kernel<KB, VB, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return check_launch("prefill: shared memory opt-in");
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid((max_query_len + kBM - 1) / kBM, p.H_q, B);
  prefill_kernel<KB, VB, PAGED><<<grid, kPfThreads, smem, st>>>(p);
  return check_launch("prefill kernel");
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
  if (H_q / H_kv > 8) return fail(CDA_ERR_UNSUPPORTED, "prefill_varlen: GQA group %d > 8", H_q / H_kv);
  PrefillUmmaParams p{};
  p.q = static_cast<const __half*>(Q); p.out = static_cast<__half*>(out); p.cu_q = cu_seqlens_q;
  p.cache = static_cast<const uint8_t*>(kv_cache); p.block_table = block_table; p.seq_lens = seq_lens;
  p.cb_k = cb_K; p.cb_v = cb_V; p.status = nullptr; p.block_size = block_size; p.bt_stride = block_table_stride;
  p.bs_shift = -1;
  for (int sft = 4; sft < 31; ++sft) if ((1 << sft) == block_size) p.bs_shift = sft;
  p.num_blocks = static_cast<int>(num_slots / block_size);
  p.H_q = H_q; p.H_kv = H_kv; p.group = H_q / H_kv; p.scale_log2 = scale * kLog2e;
  return dispatch_prefill_umma(p, k_bits, v_bits, max_query_len, B, static_cast<cudaStream_t>(stream));
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
  PrefillParams p{};
  p.q = static_cast<const __half*>(Q); p.out = static_cast<__half*>(out); p.cu_q = cu_seqlens_q;
  p.k_rot = static_cast<const __half*>(k_rot); p.v_rot = static_cast<const __half*>(v_rot);
  p.cu_k = cu_seqlens_k; p.seqused_k = seqused_k;
  p.H_q = H_q; p.H_kv = H_kv; p.group = H_q / H_kv; p.scale_log2 = scale * kLog2e;
  return launch_prefill<4, 4, false>(p, max_query_len, B, static_cast<cudaStream_t>(stream));
}
