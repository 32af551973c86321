// Single-query GQA decode over the paged codebook cache.
//
// Split kernel (decode_split_kernel).  Grid = (key-range splits, sequences, KV-head groups); a CTA has
// 8 warps and owns up to 8 KV heads of one key range of one sequence.  A warp owns ONE KV head (and the
// whole GQA group of query heads that reads it) and walks its share of the range 16 tokens at a time:
//
//   HBM -> shared   16-byte cp.async.cg copies of the 16 slots into a per-warp ring (no CTA barrier in the
//                   main loop); destinations are permuted so that later fragment reads are conflict free.
//   codes -> fp16   one shared-memory gather per code: a byte (two 4-bit indices) or nibble (two 2-bit
//                   indices) selects an fp16 pair from a lane-replicated table, which is exactly one
//                   32-bit operand register of mma.m16n8k16.
//   QK^T            tokens on the M axis, query heads on N: S[16 tok x 8 col] over 8 k-steps.  For a group
//                   of <= 4 query heads columns 4..7 repeat columns 0..3.
//   softmax         online, per 32-token tile, base-2 exponent; norms are applied to scores (K) and to
//                   the probabilities (V), never to the 128-wide vectors.
//   P V             computed transposed: A = decoded V codes (rows = byte position in the slot, k = (token,
//                   parity of the coordinate)), B = probabilities placed in the even or odd half of the
//                   register.  That keeps "one code -> one A register" without any data shuffling;
//                   movmatrix transposes the probability tile between the two products.
//
// Every warp writes an un-normalised partial (O[g][128], m, l) to the workspace; decode_merge_kernel
// combines them by log-sum-exp, rounds to fp16, applies the inverse Hadamard transform and stores fp16.
//
// HBM traffic per (token, KV head): one slot (144 B for k4v4; 136 B of it payload).
#include <cmath>

#include "common.cuh"

namespace cda {

constexpr int kDecWarps = 8;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kTileGroups = 2;     // 16-token groups per softmax tile
constexpr int kRing = 6;           // ring slots (groups) per warp

template <int KB, int VB>
struct Geom {
  static constexpr int kKBytes = 16 * KB;                      // index bytes of one row
  static constexpr int kVBytes = 16 * VB;
  static constexpr int kKChunks = kKBytes / 16;
  static constexpr int kVChunks = kVBytes / 16;
  static constexpr int kChunks = kKChunks + kVChunks + 1;      // 16-byte pieces per slot
  static constexpr int kSlotBytes = kChunks * 16;
  static constexpr int kGroupChunks = 16 * kChunks;
  static constexpr int kIssueIters = (kGroupChunks + 31) / 32;
  static constexpr int kKRegion = 16 * kKBytes;
  static constexpr int kVRegion = 16 * kVBytes;
  static constexpr int kNOffset = kKRegion + kVRegion;
  static constexpr int kStageBytes = kNOffset + 256;
  static constexpr int kLutKBytes = Lut<KB>::kBytes;
  static constexpr int kLutVBytes = Lut<VB>::kBytes;
  static constexpr int kQBytes = kDecWarps * 8 * kHeadDim * 2;
  static constexpr int kSmemBytes = kLutKBytes + kLutVBytes + kQBytes + kDecWarps * kRing * kStageBytes;
};

// Shared-memory placement of 16-byte piece `k` of row `rho` inside the V region of a stage.
template <int VB>
__device__ __forceinline__ int v_piece_offset(int rho, int k) {
  if (VB == 4) {   // 64-byte rows; rows {0,2,4,6} (and {1,3,5,7}) must land in four different 32-byte bank groups
    return ((rho & 3) | ((rho >> 3) << 2)) * 128 + ((rho >> 2) & 1) * 64 + ((k ^ (((rho >> 1) & 1) << 1)) * 16);
  } else {         // 32-byte rows
    return ((rho & 1) | ((rho >> 3) << 1)) * 128 + ((rho >> 1) & 3) * 32 + k * 16;
  }
}

struct DecodeParams {
  const __half* q;
  const uint8_t* cache;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const float* cb_k;
  const float* cb_v;
  float* part_ml;      // (P, B, H_q, 2): m (log2 domain, scale folded in), l
  float* part_o;       // (P, B, H_q, 128)
  int* status;         // device status word (bit 0: a block id was out of range)
  int B, H_q, H_kv, group;
  int heads_per_cta;   // power of two <= 8 dividing H_kv
  int block_size, bt_stride, num_blocks;
  int tokens_per_split;   // multiple of 16
  float scale_log2;       // softmax scale * log2(e)
};

template <int BITS, int POS>
__device__ __forceinline__ uint32_t code_hi(uint32_t w) {   // first code of byte POS of w
  if (BITS == 4) return __byte_perm(w, 0, 0x4440 | POS);
  return (w >> (8 * POS + 4)) & 0xf;
}
template <int BITS, int POS>
__device__ __forceinline__ uint32_t code_lo(uint32_t w) {   // second code (2-bit tables only)
  return (w >> (8 * POS)) & 0xf;
}

// Operand registers of k-step S for one K row held as packed words `w` (4-bit: 16 bytes, 2-bit: 8 bytes).
template <int KB, int S>
__device__ __forceinline__ void k_operands(const uint32_t* w, const uint32_t* lut, uint32_t& lo_k, uint32_t& hi_k) {
  if (KB == 4) {
    lo_k = lut[code_hi<4, (2 * S) & 3>(w[(2 * S) >> 2]) * 32];
    hi_k = lut[code_hi<4, (2 * S + 1) & 3>(w[(2 * S + 1) >> 2]) * 32];
  } else {
    lo_k = lut[code_hi<2, S & 3>(w[S >> 2]) * 32];
    hi_k = lut[code_lo<2, S & 3>(w[S >> 2]) * 32];
  }
}
// Operand registers of m-tile U for one V row: 4-bit rows give bytes 2U, 2U+1 of the lane's 8 bytes, 2-bit rows
// the two nibbles of byte U of the lane's 4 bytes.
template <int VB, int U>
__device__ __forceinline__ void v_operands(const uint32_t* w, const uint32_t* lut, uint32_t& first, uint32_t& second) {
  if (VB == 4) {
    first = lut[code_hi<4, (2 * U) & 3>(w[(2 * U) >> 2]) * 32];
    second = lut[code_hi<4, (2 * U + 1) & 3>(w[(2 * U + 1) >> 2]) * 32];
  } else {
    first = lut[code_hi<2, U>(w[0]) * 32];
    second = lut[code_lo<2, U>(w[0]) * 32];
  }
}

template <int KB, int S>
struct QkSteps {
  __device__ static __forceinline__ void run(float (&sc)[4], const uint32_t* ka, const uint32_t* kb, const uint32_t* lut,
                                             const uint32_t (&qf)[16]) {
    uint32_t a0, a1, a2, a3;
    k_operands<KB, S>(ka, lut, a0, a2);
    k_operands<KB, S>(kb, lut, a1, a3);
    mma_16816(sc, a0, a1, a2, a3, qf[2 * S], qf[2 * S + 1]);
    QkSteps<KB, S + 1>::run(sc, ka, kb, lut, qf);
  }
};
template <int KB>
struct QkSteps<KB, 8> {
  __device__ static __forceinline__ void run(float (&)[4], const uint32_t*, const uint32_t*, const uint32_t*,
                                             const uint32_t (&)[16]) {}
};

template <int VB, int NT, int U>
struct PvSteps {
  __device__ static __forceinline__ void run(float (&o)[4][NT][4], const uint32_t* va, const uint32_t* vb,
                                             const uint32_t* lut, const uint32_t (&bfrag)[NT][2]) {
    uint32_t a0, a1, a2, a3;
    v_operands<VB, U>(va, lut, a0, a1);
    v_operands<VB, U>(vb, lut, a2, a3);
#pragma unroll
    for (int t = 0; t < NT; ++t) mma_16816(o[U][t], a0, a1, a2, a3, bfrag[t][0], bfrag[t][1]);
    PvSteps<VB, NT, U + 1>::run(o, va, vb, lut, bfrag);
  }
};
template <int VB, int NT>
struct PvSteps<VB, NT, 4> {
  __device__ static __forceinline__ void run(float (&)[4][NT][4], const uint32_t*, const uint32_t*, const uint32_t*,
                                             const uint32_t (&)[NT][2]) {}
};

// G: padded GQA group (4 or 8).
template <int G, int KB, int VB>
__global__ void __launch_bounds__(kDecThreads, 1) decode_split_kernel(const DecodeParams p) {
  using Gm = Geom<KB, VB>;
  constexpr int NT = G / 4;   // n-tiles of the PV product
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* lut_k = reinterpret_cast<uint32_t*>(smem);
  uint32_t* lut_v = reinterpret_cast<uint32_t*>(smem + Gm::kLutKBytes);
  __half* q_all = reinterpret_cast<__half*>(smem + Gm::kLutKBytes + Gm::kLutVBytes);
  uint8_t* ring_all = smem + Gm::kLutKBytes + Gm::kLutVBytes + Gm::kQBytes;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int split = blockIdx.x, b = blockIdx.y, hg = blockIdx.z;
  const int hpc = p.heads_per_cta;
  const int R = kDecWarps / hpc;                 // warps sharing one head (each takes every R-th group)
  const int head = hg * hpc + (warp & (hpc - 1));
  const int sub = warp / hpc;
  const int g = p.group;

  const int seq_len = p.seq_lens[b];
  const int t_begin = split * p.tokens_per_split;
  const int t_end = min(seq_len, t_begin + p.tokens_per_split);
  const int cta_groups = t_end > t_begin ? (t_end - t_begin + 15) >> 4 : 0;
  const int g_begin = t_begin >> 4;
  const int ng = cta_groups > sub ? (cta_groups - sub + R - 1) / R : 0;   // groups of this warp

  const int part = split * R + sub;
  const int64_t prow0 = (static_cast<int64_t>(part) * p.B + b) * p.H_q + head * g;   // partial row of query 0

  if (cta_groups == 0) {   // nothing in range (short sequence): empty partials, no set-up
    if (lane < g) *reinterpret_cast<float2*>(p.part_ml + (prow0 + lane) * 2) = make_float2(-INFINITY, 0.f);
    return;
  }

  build_lut<KB>(lut_k, p.cb_k, tid, kDecThreads);
  build_lut<VB>(lut_v, p.cb_v, tid, kDecThreads);

  // ---- rotate this head's queries, stage them as fp16 rows, pick up the B fragments ------------------
  __half* q_rows = q_all + warp * 8 * kHeadDim;
  for (int qi = 0; qi < 8; ++qi) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (qi < g) {
      load_half4(p.q + (static_cast<int64_t>(b) * p.H_q + head * g + qi) * kHeadDim + 4 * lane, v);
      fht128_warp(v, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= kRsqrtD;
    }
    *reinterpret_cast<uint2*>(q_rows + qi * kHeadDim + 4 * lane) = pack_half4(v);
  }
  __syncthreads();   // tables + query rows visible (the only CTA-wide barrier)

  uint32_t qf[16];   // column r (query r, or r & 3 when the group is padded to 4), coordinates 32c .. 32c+31
  {
    const int qrow = G == 4 ? (r & 3) : r;
    const uint4* src = reinterpret_cast<const uint4*>(q_rows + qrow * kHeadDim + 32 * c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 t = src[i];
      qf[4 * i] = t.x; qf[4 * i + 1] = t.y; qf[4 * i + 2] = t.z; qf[4 * i + 3] = t.w;
    }
  }
  const uint32_t* lk = lut_k + lane;
  const uint32_t* lv = lut_v + lane;

  // ---- per-lane copy descriptors: which 16-byte pieces of a 16-slot group this lane moves -------------
  const int row_stride = p.H_kv * Gm::kSlotBytes;
  int src_off[Gm::kIssueIters], dst_off[Gm::kIssueIters];
#pragma unroll
  for (int it = 0; it < Gm::kIssueIters; ++it) {
    const int ch = it * 32 + lane;
    const int rho = ch / Gm::kChunks, piece = ch - rho * Gm::kChunks;
    src_off[it] = rho * row_stride + piece * 16;
    int d;
    if (piece < Gm::kKChunks) d = rho * Gm::kKBytes + piece * 16;
    else if (piece < Gm::kKChunks + Gm::kVChunks) d = Gm::kKRegion + v_piece_offset<VB>(rho, piece - Gm::kKChunks);
    else d = Gm::kNOffset + rho * 16;
    dst_off[it] = ch < Gm::kGroupChunks ? d : -1;
  }
  const uint32_t ring = smem_addr(ring_all + warp * kRing * Gm::kStageBytes);
  const uint8_t* ring_ptr = ring_all + warp * kRing * Gm::kStageBytes;

  // ---- block ids, fetched 32 groups at a time well ahead of use ------------------------------------------
  const int32_t* bt_row = p.block_table + static_cast<int64_t>(b) * p.bt_stride;
  auto load_block = [&](int j) -> int {
    if (j >= ng) return 0;
    const int tok0 = (g_begin + sub + R * j) << 4;
    int blk = __ldg(bt_row + tok0 / p.block_size);
    if (blk < 0 || blk >= p.num_blocks) { atomicOr(p.status, 1); blk = 0; }
    return blk;
  };
  int jb = 0;
  int bt_cur = load_block(lane), bt_nxt = load_block(32 + lane);

  int issue_slot = 0;
  auto issue = [&](int j) {
    if (j < ng) {
      if (j >= jb + 32) { jb += 32; bt_cur = bt_nxt; bt_nxt = load_block(jb + 32 + lane); }
      const int blk = __shfl_sync(0xffffffffu, bt_cur, j - jb);
      const int tok0 = (g_begin + sub + R * j) << 4;
      const int64_t slot0 = static_cast<int64_t>(blk) * p.block_size + (tok0 % p.block_size);
      const uint8_t* src = p.cache + (slot0 * p.H_kv + head) * Gm::kSlotBytes;
      const uint32_t dst = ring + issue_slot * Gm::kStageBytes;
#pragma unroll
      for (int it = 0; it < Gm::kIssueIters; ++it)
        if (dst_off[it] >= 0) cp_async16(dst + dst_off[it], src + src_off[it]);
    }
    cp_async_commit();
    issue_slot = issue_slot + 1 == kRing ? 0 : issue_slot + 1;
  };
#pragma unroll 1
  for (int j = 0; j < kRing; ++j) issue(j);

  // ---- running state ------------------------------------------------------------------------------------
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // columns 2c, 2c+1
  float oacc[4][NT][4];
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) oacc[u][t][i] = 0.f;

  const int my_end = t_end;   // tokens at or beyond this are masked
  int read_slot = 0;
#pragma unroll 1
  for (int j0 = 0; j0 < ng; j0 += kTileGroups) {
    cp_async_wait<kRing - kTileGroups>();
    __syncwarp();

    float sc[kTileGroups][4];
    float nvr[kTileGroups][2];
    int slot_of[kTileGroups];
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int gi = 0; gi < kTileGroups; ++gi) {
      slot_of[gi] = read_slot + gi >= kRing ? read_slot + gi - kRing : read_slot + gi;
      const uint8_t* st = ring_ptr + slot_of[gi] * Gm::kStageBytes;
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[gi][i] = 0.f;
      nvr[gi][0] = nvr[gi][1] = 0.f;
      if (j0 + gi < ng) {
        uint32_t ka[4], kb[4];
        if (KB == 4) {
          const uint4 t0 = *reinterpret_cast<const uint4*>(st + r * 64 + c * 16);
          const uint4 t1 = *reinterpret_cast<const uint4*>(st + (r + 8) * 64 + c * 16);
          ka[0] = t0.x; ka[1] = t0.y; ka[2] = t0.z; ka[3] = t0.w;
          kb[0] = t1.x; kb[1] = t1.y; kb[2] = t1.z; kb[3] = t1.w;
        } else {
          const uint2 t0 = *reinterpret_cast<const uint2*>(st + r * 32 + c * 8);
          const uint2 t1 = *reinterpret_cast<const uint2*>(st + (r + 8) * 32 + c * 8);
          ka[0] = t0.x; ka[1] = t0.y; kb[0] = t1.x; kb[1] = t1.y;
          ka[2] = ka[3] = kb[2] = kb[3] = 0;
        }
        QkSteps<KB, 0>::run(sc[gi], ka, kb, lk, qf);
        const float2 n0 = *reinterpret_cast<const float2*>(st + Gm::kNOffset + r * 16);
        const float2 n1 = *reinterpret_cast<const float2*>(st + Gm::kNOffset + (r + 8) * 16);
        const int tok0 = (g_begin + sub + R * (j0 + gi)) << 4;
        const bool ok0 = tok0 + r < my_end, ok1 = tok0 + r + 8 < my_end;
        const float f0 = n0.x * p.scale_log2, f1 = n1.x * p.scale_log2;
        sc[gi][0] = ok0 ? sc[gi][0] * f0 : -INFINITY;
        sc[gi][1] = ok0 ? sc[gi][1] * f0 : -INFINITY;
        sc[gi][2] = ok1 ? sc[gi][2] * f1 : -INFINITY;
        sc[gi][3] = ok1 ? sc[gi][3] * f1 : -INFINITY;
        nvr[gi][0] = ok0 ? n0.y : 0.f;
        nvr[gi][1] = ok1 ? n1.y : 0.f;
        mx0 = fmaxf(mx0, fmaxf(sc[gi][0], sc[gi][2]));
        mx1 = fmaxf(mx1, fmaxf(sc[gi][1], sc[gi][3]));
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[gi][i] = -INFINITY;
      }
    }
    // column maxima over the 32 tokens of the tile (rows live in the r dimension of the lane id)
#pragma unroll
    for (int mask = 4; mask < 32; mask <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, mask));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, mask));
    }
    const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    const float fs0 = fast_exp2(m_run[0] - ms0), fs1 = fast_exp2(m_run[1] - ms1);
    m_run[0] = mn0; m_run[1] = mn1;
    l_run[0] *= fs0; l_run[1] *= fs1;
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        oacc[u][t][0] *= fs0; oacc[u][t][1] *= fs1; oacc[u][t][2] *= fs0; oacc[u][t][3] *= fs1;
      }

#pragma unroll
    for (int gi = 0; gi < kTileGroups; ++gi) {
      if (j0 + gi < ng) {
        const uint8_t* st = ring_ptr + slot_of[gi] * Gm::kStageBytes;
        const float p0 = fast_exp2(sc[gi][0] - ms0), p1 = fast_exp2(sc[gi][1] - ms1);
        const float p2 = fast_exp2(sc[gi][2] - ms0), p3 = fast_exp2(sc[gi][3] - ms1);
        l_run[0] += p0 + p2;
        l_run[1] += p1 + p3;
        const uint32_t x0 = pack_half2(p0 * nvr[gi][0], p1 * nvr[gi][0]);   // row r,   columns 2c, 2c+1
        const uint32_t x1 = pack_half2(p2 * nvr[gi][1], p3 * nvr[gi][1]);   // row r+8
        const uint32_t y[2] = {movmatrix_trans(x0), movmatrix_trans(x1)};    // (P[2c][r], P[2c+1][r]) of rows 0-7 / 8-15
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int ra = 8 * hh + 2 * c, rb = ra + 1;
          uint32_t va[2], vb[2];
          if (VB == 4) {
            const uint2 t0 = *reinterpret_cast<const uint2*>(st + Gm::kKRegion + v_piece_offset<4>(ra, r >> 1) + 8 * (r & 1));
            const uint2 t1 = *reinterpret_cast<const uint2*>(st + Gm::kKRegion + v_piece_offset<4>(rb, r >> 1) + 8 * (r & 1));
            va[0] = t0.x; va[1] = t0.y; vb[0] = t1.x; vb[1] = t1.y;
          } else {
            va[0] = *reinterpret_cast<const uint32_t*>(st + Gm::kKRegion + v_piece_offset<2>(ra, r >> 2) + 4 * (r & 3));
            vb[0] = *reinterpret_cast<const uint32_t*>(st + Gm::kKRegion + v_piece_offset<2>(rb, r >> 2) + 4 * (r & 3));
            va[1] = vb[1] = 0;
          }
          uint32_t bfrag[NT][2];
          if (G == 4) {          // column r = (parity r >> 2, query r & 3)
            const bool odd = (r >> 2) != 0;
            bfrag[0][0] = odd ? (y[hh] << 16) : (y[hh] & 0xffffu);
            bfrag[0][1] = odd ? (y[hh] & 0xffff0000u) : (y[hh] >> 16);
          } else {               // tile 0: even coordinate of every pair, tile 1: odd
            bfrag[0][0] = y[hh] & 0xffffu;
            bfrag[0][1] = y[hh] >> 16;
            bfrag[NT - 1][0] = y[hh] << 16;
            bfrag[NT - 1][1] = y[hh] & 0xffff0000u;
          }
          PvSteps<VB, NT, 0>::run(oacc, va, vb, lv, bfrag);
        }
      }
    }
    __syncwarp();
    read_slot = read_slot + kTileGroups >= kRing ? read_slot + kTileGroups - kRing : read_slot + kTileGroups;
    issue(j0 + kRing);
    issue(j0 + kRing + 1);
  }
  cp_async_wait<0>();

  // ---- write this warp's partial ---------------------------------------------------------------------------
#pragma unroll
  for (int mask = 4; mask < 32; mask <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], mask);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], mask);
  }
  if (G == 4) {
    const int parity = c >> 1, q0 = 2 * (c & 1);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int d = 16 * r + 4 * u + parity;
      if (q0 < g) { p.part_o[(prow0 + q0) * kHeadDim + d] = oacc[u][0][0]; p.part_o[(prow0 + q0) * kHeadDim + d + 2] = oacc[u][0][2]; }
      if (q0 + 1 < g) { p.part_o[(prow0 + q0 + 1) * kHeadDim + d] = oacc[u][0][1]; p.part_o[(prow0 + q0 + 1) * kHeadDim + d + 2] = oacc[u][0][3]; }
    }
    if (r == 0 && c < 2) {
      if (q0 < g) *reinterpret_cast<float2*>(p.part_ml + (prow0 + q0) * 2) = make_float2(m_run[0], l_run[0]);
      if (q0 + 1 < g) *reinterpret_cast<float2*>(p.part_ml + (prow0 + q0 + 1) * 2) = make_float2(m_run[1], l_run[1]);
    }
  } else {
    const int q0 = 2 * c;
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int d = 16 * r + 4 * u + t;
        if (q0 < g) { p.part_o[(prow0 + q0) * kHeadDim + d] = oacc[u][t][0]; p.part_o[(prow0 + q0) * kHeadDim + d + 2] = oacc[u][t][2]; }
        if (q0 + 1 < g) { p.part_o[(prow0 + q0 + 1) * kHeadDim + d] = oacc[u][t][1]; p.part_o[(prow0 + q0 + 1) * kHeadDim + d + 2] = oacc[u][t][3]; }
      }
    if (r == 0) {
      if (q0 < g) *reinterpret_cast<float2*>(p.part_ml + (prow0 + q0) * 2) = make_float2(m_run[0], l_run[0]);
      if (q0 + 1 < g) *reinterpret_cast<float2*>(p.part_ml + (prow0 + q0 + 1) * 2) = make_float2(m_run[1], l_run[1]);
    }
  }
}

// ---- merge --------------------------------------------------------------------------------------------------
// One CTA (8 warps) per output row.  Warp w folds partials w, w+8, ... with a running maximum; the eight
// warp results are combined through shared memory.  m values are multiplied by `m_to_log2` on load (1 for the
// split kernel's own partials, log2(e) for natural-log partials supplied through the C ABI).
// mode 0: normalise, round to fp16, optional inverse Hadamard, store fp16.
// mode 1: store the merged un-normalised partial as fp32 (O, m in natural log, l).
__global__ void __launch_bounds__(256) decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                                                           const float* __restrict__ part_l, int ml_stride, int P,
                                                           int64_t rows, float m_to_log2, int mode, int unrotate,
                                                           __half* __restrict__ out, float* __restrict__ out_o,
                                                           float* __restrict__ out_m, float* __restrict__ out_l) {
  __shared__ float s_o[8][kHeadDim];
  __shared__ float s_m[8], s_l[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  float m = -INFINITY, l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  for (int pi = warp; pi < P; pi += 8) {
    const int64_t pr = static_cast<int64_t>(pi) * rows + row;
    const float mp = part_m[pr * ml_stride] * m_to_log2;
    if (mp == -INFINITY) continue;          // empty range: nothing was written to part_o
    const float lp = part_l[pr * ml_stride];
    const float4 op = *reinterpret_cast<const float4*>(part_o + pr * kHeadDim + 4 * lane);
    const float mn = fmaxf(m, mp);
    const float a = fast_exp2(m - mn), bw = fast_exp2(mp - mn);
    l = l * a + lp * bw;
    o[0] = o[0] * a + op.x * bw; o[1] = o[1] * a + op.y * bw; o[2] = o[2] * a + op.z * bw; o[3] = o[3] * a + op.w * bw;
    m = mn;
  }
  s_o[warp][4 * lane] = o[0]; s_o[warp][4 * lane + 1] = o[1]; s_o[warp][4 * lane + 2] = o[2]; s_o[warp][4 * lane + 3] = o[3];
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
  __syncthreads();
  if (warp != 0) return;
  float mt = -INFINITY;
#pragma unroll
  for (int w = 0; w < 8; ++w) mt = fmaxf(mt, s_m[w]);
  const float ms = mt == -INFINITY ? 0.f : mt;
  float lt = 0.f, ot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const float a = fast_exp2(s_m[w] - ms);   // exp2(-inf) = 0 for warps that saw nothing
    lt += s_l[w] * a;
#pragma unroll
    for (int i = 0; i < 4; ++i) ot[i] += s_o[w][4 * lane + i] * a;
  }
  if (mode == 1) {
    *reinterpret_cast<float4*>(out_o + row * kHeadDim + 4 * lane) = make_float4(ot[0], ot[1], ot[2], ot[3]);
    if (lane == 0) { out_m[row] = mt == -INFINITY ? -INFINITY : mt * kLn2; out_l[row] = lt; }
    return;
  }
  const float inv = 1.0f / fmaxf(lt, 1e-30f);   // merge_partials clamps the denominator (attention.py:271)
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = round_to_half(ot[i] * inv);   // the oracle rounds O_rot to fp16 before un-rotating
  if (unrotate) {
    fht128_warp(v, lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= kRsqrtD;
  }
  *reinterpret_cast<uint2*>(out + row * kHeadDim + 4 * lane) = pack_half4(v);
}

// ---- scalar cross-check kernel ----------------------------------------------------------------------------------
// One warp per (sequence, query head); lane l owns coordinates 4l..4l+3.  K and V are decoded the way
// Compressor.decode does (fp32 level * fp32 norm, rounded to fp16), scores and sums are fp32.
template <int KB, int VB>
__global__ void __launch_bounds__(32) decode_scalar_kernel(const __half* __restrict__ q, const uint8_t* __restrict__ cache,
                                                           const int32_t* __restrict__ block_table,
                                                           const int32_t* __restrict__ seq_lens, const float* __restrict__ cb_k,
                                                           const float* __restrict__ cb_v, __half* __restrict__ out, int H_q,
                                                           int H_kv, int group, int block_size, int bt_stride, int num_blocks,
                                                           int slot_bytes, float scale) {
  const int lane = threadIdx.x, hq = blockIdx.x, b = blockIdx.y;
  const int head = hq / group;
  __shared__ float s_cb[2][16];
  if (lane < 16) {
    s_cb[0][lane] = lane < (KB == 4 ? 16 : 4) ? cb_k[lane] : 0.f;
    s_cb[1][lane] = lane < (VB == 4 ? 16 : 4) ? cb_v[lane] : 0.f;
  }
  __syncwarp();
  float qv[4];
  load_half4(q + (static_cast<int64_t>(b) * H_q + hq) * kHeadDim + 4 * lane, qv);
  fht128_warp(qv, lane);
#pragma unroll
  for (int i = 0; i < 4; ++i) qv[i] = round_to_half(qv[i] * kRsqrtD);
  const int n = seq_lens[b];
  float m = -INFINITY, l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  for (int t = 0; t < n; ++t) {
    int blk = block_table[static_cast<int64_t>(b) * bt_stride + t / block_size];
    if (blk < 0 || blk >= num_blocks) blk = 0;
    const uint8_t* slot = cache + ((static_cast<int64_t>(blk) * block_size + t % block_size) * H_kv + head) * slot_bytes;
    const float nk = *reinterpret_cast<const float*>(slot + 16 * KB + 16 * VB);
    const float nv = *reinterpret_cast<const float*>(slot + 16 * KB + 16 * VB + 4);
    int ik[4], iv[4];
    if (KB == 4) { const uint8_t b0 = slot[2 * lane], b1 = slot[2 * lane + 1]; ik[0] = b0 >> 4; ik[1] = b0 & 15; ik[2] = b1 >> 4; ik[3] = b1 & 15; }
    else { const uint8_t b0 = slot[lane]; ik[0] = b0 >> 6; ik[1] = (b0 >> 4) & 3; ik[2] = (b0 >> 2) & 3; ik[3] = b0 & 3; }
    const uint8_t* vs = slot + 16 * KB;
    if (VB == 4) { const uint8_t b0 = vs[2 * lane], b1 = vs[2 * lane + 1]; iv[0] = b0 >> 4; iv[1] = b0 & 15; iv[2] = b1 >> 4; iv[3] = b1 & 15; }
    else { const uint8_t b0 = vs[lane]; iv[0] = b0 >> 6; iv[1] = (b0 >> 4) & 3; iv[2] = (b0 >> 2) & 3; iv[3] = b0 & 3; }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) dot = fmaf(qv[i], round_to_half(s_cb[0][ik[i]] * nk), dot);
    const float s = warp_sum(dot) * scale;
    const float mn = fmaxf(m, s);
    const float a = expf(m - mn), pw = expf(s - mn);
    l = l * a + pw;
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = o[i] * a + pw * round_to_half(s_cb[1][iv[i]] * nv);
    m = mn;
  }
  float v[4];
  const float inv = n > 0 ? 1.0f / fmaxf(l, 1e-30f) : 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = round_to_half(o[i] * inv);
  fht128_warp(v, lane);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= kRsqrtD;
  *reinterpret_cast<uint2*>(out + (static_cast<int64_t>(b) * H_q + hq) * kHeadDim + 4 * lane) = pack_half4(v);
}

// ---- host side --------------------------------------------------------------------------------------------------
struct Plan {
  int heads_per_cta, head_groups, warps_per_head, splits, tokens_per_split, parts;
};

static int pick_heads_per_cta(int H_kv) {
  int h = 8;
  while (h > 1 && (h > H_kv || H_kv % h)) h >>= 1;
  return h;
}

// Choose the number of key-range splits.  One CTA occupies one SM, so the grid should be a whole number of
// waves of the SM count: take the largest wave count (<= 8) whose splits still hold >= 256 tokens; if even one
// wave would cut the range finer than that, fall back to 128-token splits (a latency-bound launch anyway).
static Plan make_plan(int B, int H_kv, int max_seq_len, int num_splits, int sms) {
  constexpr int kMinTokens = 256, kFloorTokens = 128, kMaxWaves = 8;
  Plan pl;
  pl.heads_per_cta = pick_heads_per_cta(H_kv);
  pl.head_groups = H_kv / pl.heads_per_cta;
  pl.warps_per_head = kDecWarps / pl.heads_per_cta;
  const int n = max_seq_len > 0 ? max_seq_len : 1;
  int S = num_splits;
  if (S <= 0) {
    const int64_t other = static_cast<int64_t>(B) * pl.head_groups;
    S = 0;
    for (int w = kMaxWaves; w >= 1 && S == 0; --w) {
      const int64_t s_w = static_cast<int64_t>(w) * sms / other;
      if (s_w >= 1 && (n + s_w - 1) / s_w >= kMinTokens) S = static_cast<int>(s_w);
    }
    if (S == 0) {
      const int64_t one_wave = sms / other > 1 ? sms / other : 1;
      const int64_t by_work = (n + kFloorTokens - 1) / kFloorTokens;
      S = static_cast<int>(one_wave < by_work ? one_wave : by_work);
    }
  }
  int tps = ((n + S - 1) / S + 15) / 16 * 16;
  pl.tokens_per_split = tps;
  pl.splits = (n + tps - 1) / tps;
  pl.parts = pl.splits * pl.warps_per_head;
  return pl;
}

static size_t ws_bytes(const Plan& pl, int B, int H_q) {
  const size_t rows = static_cast<size_t>(pl.parts) * B * H_q;
  return 256 + rows * 2 * sizeof(float) + rows * kHeadDim * sizeof(float);
}

struct DecodeCommon {
  const void* Q; const void* cache; const int32_t* bt; const int32_t* sl; const float* cbk; const float* cbv;
  int B, H_q, H_kv, block_size, bt_stride, max_seq_len; int64_t num_slots; int slot_bytes, k_bits, v_bits; float scale;
};

static int validate(const char* who, const DecodeCommon& a) {
  if (a.B < 0 || a.H_q <= 0 || a.H_kv <= 0 || a.max_seq_len < 0 || a.num_slots < 0 || a.bt_stride < 0)
    return fail(CDA_ERR_BAD_ARG, "%s: negative or zero size", who);
  if (!bits_ok(a.k_bits) || !bits_ok(a.v_bits)) return fail(CDA_ERR_UNSUPPORTED, "%s: bits must be 2 or 4", who);
  if (a.slot_bytes != slot_bytes_for(a.k_bits, a.v_bits))
    return fail(CDA_ERR_BAD_SHAPE, "%s: slot width %d, expected %d for k%dv%d", who, a.slot_bytes,
                slot_bytes_for(a.k_bits, a.v_bits), a.k_bits, a.v_bits);
  if (a.H_q % a.H_kv) return fail(CDA_ERR_BAD_SHAPE, "%s: H_q=%d is not a multiple of H_kv=%d", who, a.H_q, a.H_kv);
  if (a.H_q / a.H_kv > 8) return fail(CDA_ERR_UNSUPPORTED, "%s: GQA group %d > 8", who, a.H_q / a.H_kv);
  if (a.block_size <= 0 || a.block_size % 16) return fail(CDA_ERR_BAD_SHAPE, "%s: block_size=%d is not a multiple of 16", who, a.block_size);
  if (a.max_seq_len > (1 << 30)) return fail(CDA_ERR_N_TOO_LARGE, "%s: max_seq_len too large", who);
  if (static_cast<int64_t>(a.bt_stride) * a.block_size < a.max_seq_len)
    return fail(CDA_ERR_BAD_SHAPE, "%s: block table row (%d blocks of %d) shorter than max_seq_len=%d", who, a.bt_stride,
                a.block_size, a.max_seq_len);
  if (a.B == 0) return CDA_OK;
  if (!a.Q || !a.cache || !a.bt || !a.sl || !a.cbk || !a.cbv) return fail(CDA_ERR_BAD_ARG, "%s: null pointer", who);
  if (!aligned16(a.Q) || !aligned16(a.cache)) return fail(CDA_ERR_BAD_ALIGN, "%s: Q and the cache must be 16-byte aligned", who);
  return CDA_OK;
}

template <int G, int KB, int VB>
static int launch_split(const DecodeParams& p, const Plan& pl, cudaStream_t st) {
  using Gm = Geom<KB, VB>;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(decode_split_kernel<G, KB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, Gm::kSmemBytes) != cudaSuccess)
      return check_launch("decode: shared memory opt-in");
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid(pl.splits, p.B, pl.head_groups);
  decode_split_kernel<G, KB, VB><<<grid, kDecThreads, Gm::kSmemBytes, st>>>(p);
  return check_launch("decode split kernel");
}

template <int G>
static int dispatch_bits(const DecodeParams& p, const Plan& pl, int kb, int vb, cudaStream_t st) {
  if (kb == 4 && vb == 4) return launch_split<G, 4, 4>(p, pl, st);
  if (kb == 4 && vb == 2) return launch_split<G, 4, 2>(p, pl, st);
  if (kb == 2 && vb == 2) return launch_split<G, 2, 2>(p, pl, st);
  return launch_split<G, 2, 4>(p, pl, st);
}

static int run_split(const char* who, const DecodeCommon& a, void* workspace, size_t workspace_bytes, int num_splits,
                     cudaStream_t st, Plan* plan_out, float** ml_out, float** o_out) {
  const Plan pl = make_plan(a.B, a.H_kv, a.max_seq_len, num_splits, device_sm_count(-1));
  const size_t need = ws_bytes(pl, a.B, a.H_q);
  if (!workspace || workspace_bytes < need)
    return fail(CDA_ERR_WORKSPACE, "%s: workspace of %zu bytes, need %zu", who, workspace_bytes, need);
  if (!aligned16(workspace)) return fail(CDA_ERR_BAD_ALIGN, "%s: workspace must be 16-byte aligned", who);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const size_t rows = static_cast<size_t>(pl.parts) * a.B * a.H_q;
  DecodeParams p;
  p.q = static_cast<const __half*>(a.Q);
  p.cache = static_cast<const uint8_t*>(a.cache);
  p.block_table = a.bt; p.seq_lens = a.sl; p.cb_k = a.cbk; p.cb_v = a.cbv;
  p.status = reinterpret_cast<int*>(ws);
  p.part_ml = reinterpret_cast<float*>(ws + 256);
  p.part_o = reinterpret_cast<float*>(ws + 256 + rows * 2 * sizeof(float));
  p.B = a.B; p.H_q = a.H_q; p.H_kv = a.H_kv; p.group = a.H_q / a.H_kv;
  p.heads_per_cta = pl.heads_per_cta;
  p.block_size = a.block_size; p.bt_stride = a.bt_stride;
  p.num_blocks = static_cast<int>(a.num_slots / a.block_size);
  p.tokens_per_split = pl.tokens_per_split;
  p.scale_log2 = a.scale * kLog2e;
  const int rc = p.group <= 4 ? dispatch_bits<4>(p, pl, a.k_bits, a.v_bits, st) : dispatch_bits<8>(p, pl, a.k_bits, a.v_bits, st);
  if (rc != CDA_OK) return rc;
  *plan_out = pl; *ml_out = p.part_ml; *o_out = p.part_o;
  return CDA_OK;
}

}  // namespace cda

using namespace cda;

extern "C" int cda_b200_decode_plan_splits(int B, int H_kv, int max_seq_len, int device) {
  if (B <= 0 || H_kv <= 0 || max_seq_len < 0) return fail(CDA_ERR_BAD_ARG, "decode_plan_splits: bad size");
  return make_plan(B, H_kv, max_seq_len, 0, device_sm_count(device)).splits;
}

extern "C" size_t cda_b200_decode_workspace_bytes(int B, int H_q, int H_kv, int max_seq_len, int num_splits, int device) {
  if (B <= 0 || H_q <= 0 || H_kv <= 0 || max_seq_len < 0) return 256;
  return ws_bytes(make_plan(B, H_kv, max_seq_len, num_splits, device_sm_count(device)), B, H_q);
}

extern "C" int cda_b200_decode(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                               const float* cb_K, const float* cb_V, void* out, void* workspace, size_t workspace_bytes, int B,
                               int H_q, int H_kv, int block_size, int block_table_stride, int max_seq_len, int64_t num_slots,
                               int slot_bytes, int k_bits, int v_bits, float scale, int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  int rc = validate("decode", a);
  if (rc != CDA_OK || B == 0) return rc;
  if (!out) return fail(CDA_ERR_BAD_ARG, "decode: null output");
  if (reinterpret_cast<uintptr_t>(out) & 7u) return fail(CDA_ERR_BAD_ALIGN, "decode: output must be 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Plan pl; float* ml; float* po;
  rc = run_split("decode", a, workspace, workspace_bytes, num_splits, st, &pl, &ml, &po);
  if (rc != CDA_OK) return rc;
  const int64_t rows = static_cast<int64_t>(B) * H_q;
  if (rows > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "decode: B*H_q too large");
  decode_merge_kernel<<<static_cast<unsigned>(rows), 256, 0, st>>>(po, ml, ml + 1, 2, pl.parts, rows, 1.0f, 0, 1,
                                                                  static_cast<__half*>(out), nullptr, nullptr, nullptr);
  return check_launch("decode merge kernel");
}

extern "C" int cda_b200_decode_partial(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                       const float* cb_K, const float* cb_V, float* O, float* m, float* l, void* workspace,
                                       size_t workspace_bytes, int B, int H_q, int H_kv, int block_size, int block_table_stride,
                                       int max_seq_len, int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale,
                                       int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  int rc = validate("decode_partial", a);
  if (rc != CDA_OK || B == 0) return rc;
  if (!O || !m || !l) return fail(CDA_ERR_BAD_ARG, "decode_partial: null output");
  if (!aligned16(O)) return fail(CDA_ERR_BAD_ALIGN, "decode_partial: O must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Plan pl; float* ml; float* po;
  rc = run_split("decode_partial", a, workspace, workspace_bytes, num_splits, st, &pl, &ml, &po);
  if (rc != CDA_OK) return rc;
  const int64_t rows = static_cast<int64_t>(B) * H_q;
  if (rows > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "decode_partial: B*H_q too large");
  decode_merge_kernel<<<static_cast<unsigned>(rows), 256, 0, st>>>(po, ml, ml + 1, 2, pl.parts, rows, 1.0f, 1, 0, nullptr, O, m, l);
  return check_launch("decode partial merge kernel");
}

extern "C" int cda_b200_merge_partials(const float* O, const float* m, const float* l, int S, int64_t R, void* out,
                                       int unrotate, void* stream) {
  if (S <= 0 || R < 0) return fail(CDA_ERR_BAD_ARG, "merge_partials: bad size");
  if (R == 0) return CDA_OK;
  if (!O || !m || !l || !out) return fail(CDA_ERR_BAD_ARG, "merge_partials: null pointer");
  if (!aligned16(O) || (reinterpret_cast<uintptr_t>(out) & 7u)) return fail(CDA_ERR_BAD_ALIGN, "merge_partials: misaligned buffer");
  if (R > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "merge_partials: too many rows");
  decode_merge_kernel<<<static_cast<unsigned>(R), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      O, m, l, 1, S, R, kLog2e, 0, unrotate ? 1 : 0, static_cast<__half*>(out), nullptr, nullptr, nullptr);
  return check_launch("merge_partials");
}

extern "C" int cda_b200_decode_scalar(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                      const float* cb_K, const float* cb_V, void* out, int B, int H_q, int H_kv, int block_size,
                                      int block_table_stride, int64_t num_slots, int slot_bytes, int k_bits, int v_bits,
                                      float scale, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       0, num_slots, slot_bytes, k_bits, v_bits, scale};
  int rc = validate("decode_scalar", a);
  if (rc != CDA_OK || B == 0) return rc;
  if (!out) return fail(CDA_ERR_BAD_ARG, "decode_scalar: null output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(H_q, B);
  const int nb = static_cast<int>(num_slots / block_size), grp = H_q / H_kv;
  const __half* q = static_cast<const __half*>(Q);
  const uint8_t* c = static_cast<const uint8_t*>(kv_cache);
  __half* o = static_cast<__half*>(out);
  if (k_bits == 4 && v_bits == 4)
    decode_scalar_kernel<4, 4><<<grid, 32, 0, st>>>(q, c, block_table, seq_lens, cb_K, cb_V, o, H_q, H_kv, grp, block_size, block_table_stride, nb, slot_bytes, scale);
  else if (k_bits == 4 && v_bits == 2)
    decode_scalar_kernel<4, 2><<<grid, 32, 0, st>>>(q, c, block_table, seq_lens, cb_K, cb_V, o, H_q, H_kv, grp, block_size, block_table_stride, nb, slot_bytes, scale);
  else if (k_bits == 2 && v_bits == 2)
    decode_scalar_kernel<2, 2><<<grid, 32, 0, st>>>(q, c, block_table, seq_lens, cb_K, cb_V, o, H_q, H_kv, grp, block_size, block_table_stride, nb, slot_bytes, scale);
  else
    decode_scalar_kernel<2, 4><<<grid, 32, 0, st>>>(q, c, block_table, seq_lens, cb_K, cb_V, o, H_q, H_kv, grp, block_size, block_table_stride, nb, slot_bytes, scale);
  return check_launch("decode_scalar");
}
