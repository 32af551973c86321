// Paged encode (Hadamard rotation -> L2 norm -> nearest codebook level -> packed slot), the index
// selection on its own, and the stand-alone 128-point Hadamard transform.
//
// Paged encode: one warp owns 16 vectors, rotated on the tensor cores (see rotate16).  The other kernels: one warp owns
// one 128-vector, lane l holds coordinates 4l..4l+3, the rotation is 2 in-register and 5 shuffle butterfly stages, the
// norm a shuffle reduction.  The kernels are HBM-bound on paper: 2 x 256 B read and one payload (136 B for k4v4)
// written per (token, KV head).
#include "common.cuh"

namespace cda {

// Index selection of Compressor.quantize_unit (cda/algorithm/compression.py:298-313): upper = number of levels
// strictly below x, clamped to L-1; lower = upper-1 clamped to 0; upper wins only if strictly closer
// (fabsf(cb[upper] - x) < fabsf(x - cb[lower])), ties go to lower.
// That rule is monotone in x, so it is the same as counting thresholds: index(x) = #{i : x > T[i]}, where T[i] is
// the largest float in [cb[i], cb[i+1]] for which the rule still answers i.  T[i] is found by bisection over the
// ordered integer image of the floats, evaluating the rule's own comparison fabsf(cb[i+1] - x) < fabsf(x - cb[i]) in
// fp32 exactly as the rule does, so the result is bit-identical, ties and rounding included.
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
// Threads 0 .. L-2 of the calling group each find one threshold; T gets 16 entries (unused ones = +inf).
template <int L>
__device__ __forceinline__ void build_thresholds(const float* cb, float* T, int t) {
  if (t >= 0 && t < 16) {
    float thr = INFINITY;
    if (t < L - 1) {
      const float lo = cb[t], hi = cb[t + 1];
      uint32_t a = float_key(lo), b = float_key(hi);        // rule says t at a; says t+1 at b (if hi > lo)
      thr = lo;
      if (b > a) {
        while (b - a > 1u) {
          const uint32_t mid = a + ((b - a) >> 1);
          const float x = key_float(mid);
          if (fabsf(hi - x) < fabsf(x - lo)) b = mid; else a = mid;
        }
        thr = key_float(a);
      }
    }
    T[t] = thr;
  }
}
template <int L>
__device__ __forceinline__ int count_thresholds(float x, const float* T) {
  int lo = 0;
  if (L == 16) {
    lo = x > T[7] ? 8 : 0;
    lo += x > T[lo + 3] ? 4 : 0;
  }
  lo += x > T[lo + 1] ? 2 : 0;
  lo += x > T[lo] ? 1 : 0;
  return lo;
}
// The same count times four: the running value is the byte offset of the next threshold to look at, so every step is
// one load at (offset + constant), one comparison and one conditional add.
template <int L>
__device__ __forceinline__ uint32_t count_thresholds_x4(float x, const float* T) {
  const char* base = reinterpret_cast<const char*>(T);
  auto at = [&](uint32_t off) { return *reinterpret_cast<const float*>(base + off); };
  uint32_t lo = 0;
  if (L == 16) {
    lo = x > at(28) ? 32u : 0u;
    lo += x > at(lo + 12) ? 16u : 0u;
  }
  lo += x > at(lo + 4) ? 8u : 0u;
  lo += x > at(lo) ? 4u : 0u;
  return lo;
}

// ---- one-look-up form of the same count -----------------------------------------------------------------------------------------
// [-1, 1] is cut into 128 cells of width 1/64.  For a cell the table holds how many thresholds lie in lower cells and the
// one threshold inside it (+inf if none): index(x) = below[cell(x)] + (x > inside[cell(x)]) -- one 64-bit load, one
// comparison, one add instead of four dependent load/compare steps.  cell() is monotone in x, so thresholds in lower
// cells are below x and thresholds in higher cells are not: the count is the rule's, bit for bit.  A codebook with two
// thresholds in one cell cannot use the table; the CTA then keeps the four-step search (build_cells reports it).
constexpr int kCells = 129;                       // x = +1 lands in cell 128
constexpr float kCellMagic = 1048576.0f + 64.0f;  // 2^20 + 64: the sum below has a unit in the last place of 1/8
// Byte offset (cell * 8) of x's table entry; x in [-1, 1].  One FMA (rounded once, hence monotone) and one mask.
__device__ __forceinline__ uint32_t cell_offset(float x) { return __float_as_uint(__fmaf_rn(x, 64.0f, kCellMagic)) & 0xff8u; }
struct CellEntry {
  float inside;      // the threshold in this cell, +inf if there is none
  uint32_t below;    // thresholds in lower cells
};
// Threads `t` = 0 .. kCells-1 of the calling group fill one cell each from the L-1 thresholds in T (ascending).  Returns
// true (to that thread) if its cell holds more than one threshold.
template <int L>
__device__ __forceinline__ bool cell_of(const float* T, int t, CellEntry& e) {
  uint32_t below = 0;
  int inside = 0;
  float thr = INFINITY;
#pragma unroll
  for (int i = 0; i < L - 1; ++i) {
    const int c = static_cast<int>(cell_offset(fminf(fmaxf(T[i], -1.0f), 1.0f)) >> 3);
    below += c < t ? 1u : 0u;
    if (c == t) { ++inside; thr = T[i]; }
  }
  e.inside = thr;
  e.below = below;
  return inside > 1;
}
template <int L>
__device__ __forceinline__ bool build_cell(const float* T, CellEntry* cells, int t) {
  if (t < 0 || t >= kCells) return false;
  CellEntry e;
  const bool crowded = cell_of<L>(T, t, e);
  cells[t] = e;
  return crowded;
}
// Where the code of the p-th (p = 0..7, in coordinate order) of a lane's eight coordinates of a quarter row sits in the piece of the index field the lane writes
// (32 bits of 4-bit codes, 16 bits of 2-bit codes): the first code of a byte on top.
template <int BITS>
__host__ __device__ constexpr int code_shift(int p) {
  return BITS == 4 ? 8 * (p >> 1) + 4 * (1 - (p & 1)) : 8 * (p >> 2) + 4 - 4 * ((p >> 1) & 1) + 2 * (1 - (p & 1));
}
// Eight copies of the cell table, one per coordinate position of a lane, with `below` already shifted to the place of
// that position's code: a lane's piece of the index field is then a plain sum of table words and compare results.
template <int BITS>
__device__ __forceinline__ bool build_cells_by_position(const float* T, CellEntry (*cells)[kCells + 1], int t) {
  if (t < 0 || t >= kCells) return false;
  CellEntry e;
  const bool crowded = cell_of<(BITS == 4 ? 16 : 4)>(T, t, e);
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    cells[p][t].inside = e.inside;
    cells[p][t].below = e.below << code_shift<BITS>(p);
  }
  return crowded;
}
__device__ __forceinline__ uint32_t count_by_cell(float x, const CellEntry* cells) {
  const uint2 e = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(cells) + cell_offset(x));
  return e.y + (x > __uint_as_float(e.x) ? 1u : 0u);
}

// v: this lane's four rotated fp32 coordinates.  Writes the packed indices of the row to `idx_dst`
// (16*BITS bytes per row) and returns the row norm (identical in every lane).  T: thresholds of the codebook.
template <int BITS, bool FAST>
__device__ __forceinline__ float quantize_row(const float (&v)[4], const float* T, const CellEntry* cells, uint8_t* idx_dst, int lane) {
  constexpr int L = BITS == 4 ? 16 : 4;
  float ss = v[0] * v[0];
  ss = fmaf(v[1], v[1], ss);
  ss = fmaf(v[2], v[2], ss);
  ss = fmaf(v[3], v[3], ss);
  ss = warp_sum(ss);
  const float norm = fmaxf(sqrtf(ss), kNormFloor);
  int idx[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float u = __fdiv_rn(v[i], norm);
    u = fminf(fmaxf(u, -1.0f), 1.0f);
    idx[i] = FAST ? static_cast<int>(count_by_cell(u, cells)) : count_thresholds<L>(u, T);
  }
  if (BITS == 4) {
    const uint16_t two = static_cast<uint16_t>(((idx[0] << 4) | idx[1]) | (((idx[2] << 4) | idx[3]) << 8));
    reinterpret_cast<uint16_t*>(idx_dst)[lane] = two;
  } else {
    idx_dst[lane] = static_cast<uint8_t>((idx[0] << 6) | (idx[1] << 4) | (idx[2] << 2) | idx[3]);
  }
  return norm;
}

// ---- tensor-core rotation of 16 rows at a time (RotFrag, make_rot_frag: common.cuh) --------------------------------------
// The 2 x 64 bytes of rows `row_lo` and `row_hi` that lane c of a quad contracts (A operands of rotate16).
struct RowFrags {
  uint4 lo[4], hi[4];
};
__device__ __forceinline__ void load_row_frags(const __half* __restrict__ x, int64_t row_lo, int64_t row_hi, int c, RowFrags& a) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    a.lo[j] = __ldg(reinterpret_cast<const uint4*>(x + row_lo * kHeadDim + 32 * j + 8 * c));
    a.hi[j] = __ldg(reinterpret_cast<const uint4*>(x + row_hi * kHeadDim + 32 * j + 8 * c));
  }
}
// The 16 rows of an MMA are fed with 8 tensor rows: MMA row r takes the coordinates 8c + {0,1,4,5} of a quarter of tensor
// row r, MMA row r + 8 the coordinates 8c + {2,3,6,7} of the SAME tensor row -- so the A operand of a product is exactly the
// four registers of one 16-byte load (x, y, z, w), in order, and needs no register moves.  The product contracts the bits
// {4,3,2,0} of the coordinate index; bit 1 (which of the two MMA rows) is one add/sub inside the accumulator quad, bits
// 6 and 5 (the quarter) two butterfly stages across quads.
// y[h][j][t][i]: rotated (unscaled) coordinate 32 j + 8c + 4t + i of row h (0: the lane's low row, 1: its high row).
__device__ __forceinline__ void rotate16(const RowFrags& a, const RotFrag& f, float (&y)[2][4][2][4]) {
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4& q = h ? a.hi[j] : a.lo[j];
#pragma unroll
      for (int t = 0; t < 2; ++t) mma_16816_zero(y[h][j][t], q.x, q.y, q.z, q.w, f.b0[t], f.b1[t]);
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int t = 0; t < 2; ++t) {                         // bit 1: the quad's halves came from inputs with bit 1 clear / set
        const uint64_t lo = f2_pack(y[h][j][t][0], y[h][j][t][1]), hi = f2_pack(y[h][j][t][2], y[h][j][t][3]);
        f2_unpack(f2_add(lo, hi), y[h][j][t][0], y[h][j][t][1]);
        f2_unpack(f2_sub(lo, hi), y[h][j][t][2], y[h][j][t][3]);
      }
#pragma unroll
    for (int bit = 1; bit < 4; bit <<= 1)                    // bits 5 and 6: across the quarters
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (!(j & bit)) {
#pragma unroll
          for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
              const uint64_t p = f2_pack(y[h][j][t][i], y[h][j][t][i + 1]), q = f2_pack(y[h][j | bit][t][i], y[h][j | bit][t][i + 1]);
              f2_unpack(f2_add(p, q), y[h][j][t][i], y[h][j][t][i + 1]);
              f2_unpack(f2_sub(p, q), y[h][j | bit][t][i], y[h][j | bit][t][i + 1]);
            }
        }
  }
}
// Scales the accumulators by 1/sqrt(128) and rounds them to fp16, as the rotation's output is: hp[h][j][t][k] = coordinates
// 32 j + 8c + 4t + 2k + {0, 1} of row h as an fp16 pair.  Half the registers of y, so that the next fragments can be in flight.
__device__ __forceinline__ void scale_and_pack(const float (&y)[2][4][2][4], uint32_t (&hp)[2][4][2][2]) {
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          float s0, s1;
          f2_unpack(f2_mul(f2_pack(y[h][j][t][2 * k], y[h][j][t][2 * k + 1]), f2_pack(kRsqrtD, kRsqrtD)), s0, s1);
          hp[h][j][t][k] = pack_half2(s0, s1);
        }
}
// Quantises the two rows held in hp and writes this lane's pieces of their index fields.  Returns the two norms (the same in the four lanes of a quad).
//
// x / norm: the rotated coordinates are fp16 values, so a non-zero one is at least 2^-24 in size and the norm at most
// 2^24; with y = RN(1/norm), q = RN(x y) and r = x - q norm (exact in one FMA: no intermediate leaves the normal
// range), RN(q + r y) is the correctly rounded quotient (Markstein's division step), i.e. the value of x / norm; only
// a zero loses its sign (-0 comes out as +0), which no comparison below can see.
// FAST: take the indices from the cell table; otherwise from the four-step search.
template <int BITS, bool FAST>
__device__ __forceinline__ float2 quantize_pair(const uint32_t (&hp)[2][4][2][2], const float* T, const CellEntry* cells,
                                                uint8_t* dst_lo, uint8_t* dst_hi, int c, bool ok_lo, bool ok_hi) {
  constexpr int L = BITS == 4 ? 16 : 4;
  float ss[2];
  {
    uint64_t acc[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};      // even and odd coordinates summed side by side
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&hp[h][j][t][k]));
            const uint64_t vv = f2_pack(v.x, v.y);
            acc[h] = f2_fma(vv, vv, acc[h]);
          }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float even, odd;
      f2_unpack(acc[h], even, odd);
      ss[h] = even + odd;
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 1);
    ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 2);
  }
  float norm[2], rcp[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    norm[h] = fmaxf(sqrtf(ss[h]), kNormFloor);
    rcp[h] = __frcp_rn(norm[h]);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint8_t* dst = h ? dst_hi : dst_lo;
    const bool ok = h ? ok_hi : ok_lo;
#pragma unroll
    for (int w = 0; w < 4; ++w) {                                    // quarter of the row
      uint32_t word = 0;
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int k = 0; k < 2; ++k) {                                // coordinates 8c + 4t + 2k + {0, 1} of the quarter
          const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&hp[h][w][t][k]));
          uint32_t ix[2];                                            // the indices of coordinates e = 0, 1
          // the division step and the cell index on both coordinates at once (each lane rounded as the scalar form;
          // q * (-norm) is the same product as (-q) * norm)
          float u2[2], cf2[2];
          {
            const uint64_t vv = f2_pack(v2.x, v2.y), rr = f2_pack(rcp[h], rcp[h]);
            const uint64_t q0 = f2_mul(vv, rr);
            const uint64_t rem = f2_fma(q0, f2_pack(-norm[h], -norm[h]), vv);
            const uint64_t uu = f2_fma(rem, rr, q0);
            f2_unpack(uu, u2[0], u2[1]);
            f2_unpack(f2_fma(uu, f2_pack(64.0f, 64.0f), f2_pack(kCellMagic, kCellMagic)), cf2[0], cf2[1]);
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float u = u2[e];
            const uint32_t cell_off = __float_as_uint(cf2[e]) & 0xff8u;
            if (FAST) {                                              // table word: the count of lower cells, already in place
              constexpr int kPosStride = (kCells + 1) * static_cast<int>(sizeof(CellEntry));
              const int pos = 4 * t + 2 * k + e;
              const uint2 ce = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(cells) + pos * kPosStride + cell_off);
              ix[e] = ce.y + (u > __uint_as_float(ce.x) ? (1u << code_shift<BITS>(pos)) : 0u);
            } else {
              ix[e] = (count_thresholds_x4<L>(u, T) >> 2) << code_shift<BITS>(4 * t + 2 * k + e);
            }
          }
          word += ix[0] + ix[1];
        }
      if (ok) {
        if (BITS == 4) *reinterpret_cast<uint32_t*>(dst + 16 * w + 4 * c) = word;
        else *reinterpret_cast<uint16_t*>(dst + 8 * w + 2 * c) = static_cast<uint16_t>(word);
      }
    }
  }
  return make_float2(norm[0], norm[1]);
}

// The tile loop of the paged encoder: one warp per 16 rows (row = token * H_kv + head); lane 4r + c works on rows r and
// r + 8 of the tile.  FAST: index selection by the cell tables, else by the four-step search.
template <int KB, int VB, bool FAST>
__device__ __forceinline__ void encode_tiles(const __half* __restrict__ K, const __half* __restrict__ V,
                                             const int32_t* __restrict__ slot_mapping, uint8_t* __restrict__ cache, int64_t rows,
                                             int H_kv, int64_t num_slots, int slot_bytes, const float (*thr)[16],
                                             const CellEntry* cells_k, const CellEntry* cells_v) {
  const int lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3;
  constexpr int kKBytes = 16 * KB, kVBytes = 16 * VB;
  const RotFrag frag = make_rot_frag(lane);
  const int64_t tiles = (rows + 15) >> 4;
  const bool small = rows < 0x7fffffffLL;                            // then token = row / H_kv is a 32-bit division
  const int64_t tile_step = static_cast<int64_t>(gridDim.x) * 8;
  RowFrags fr;
  bool first = true;
  for (int64_t tile = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); tile < tiles; tile += tile_step) {
    int64_t row[2] = {tile * 16 + r, tile * 16 + r + 8};
    uint8_t* dst[2];
    bool ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      ok[h] = row[h] < rows;
      if (!ok[h]) row[h] = rows - 1;                                 // read a valid row, write nothing
      int64_t t;
      int head;
      if (small) {
        const uint32_t t32 = static_cast<uint32_t>(row[h]) / static_cast<uint32_t>(H_kv);
        t = t32;
        head = static_cast<int>(static_cast<uint32_t>(row[h]) - t32 * static_cast<uint32_t>(H_kv));
      } else {
        t = row[h] / H_kv;
        head = static_cast<int>(row[h] - t * H_kv);
      }
      const int64_t slot = slot_mapping[t];
      ok[h] = ok[h] && slot >= 0 && slot < num_slots;
      dst[h] = cache + ((ok[h] ? slot : 0) * H_kv + head) * slot_bytes;
    }
    // K fragments were requested a turn ago; V's are requested before K is quantised, the next tile's K before V is
    if (first) { load_row_frags(K, row[0], row[1], c, fr); first = false; }
    float2 nk, nv;
    {
      float y[2][4][2][4];
      uint32_t hp[2][4][2][2];
      rotate16(fr, frag, y);
      load_row_frags(V, row[0], row[1], c, fr);
      scale_and_pack(y, hp);
      nk = quantize_pair<KB, FAST>(hp, thr[0], cells_k, dst[0], dst[1], c, ok[0], ok[1]);
      rotate16(fr, frag, y);
      {
        const int64_t next = tile + tile_step;
        if (next < tiles) {
          const int64_t n_lo = next * 16 + r, n_hi = n_lo + 8;
          load_row_frags(K, n_lo < rows ? n_lo : rows - 1, n_hi < rows ? n_hi : rows - 1, c, fr);
        }
      }
      scale_and_pack(y, hp);
      nv = quantize_pair<VB, FAST>(hp, thr[1], cells_v, dst[0] + kKBytes, dst[1] + kKBytes, c, ok[0], ok[1]);
    }
    if (c == 0) {
      if (ok[0]) *reinterpret_cast<float2*>(dst[0] + kKBytes + kVBytes) = make_float2(nk.x, nv.x);
      if (ok[1]) *reinterpret_cast<float2*>(dst[1] + kKBytes + kVBytes) = make_float2(nk.y, nv.y);
    }
  }
}

// One warp per 16 rows (row = token * H_kv + head); lane 4r + c works on rows r and r + 8 of the tile.
template <int KB, int VB>
__global__ void __launch_bounds__(256, 2) paged_encode_kernel(const __half* __restrict__ K, const __half* __restrict__ V,
                                                              const int32_t* __restrict__ slot_mapping,
                                                              uint8_t* __restrict__ cache, const float* __restrict__ cb_K,
                                                              const float* __restrict__ cb_V, int64_t rows, int H_kv,
                                                              int64_t num_slots, int slot_bytes) {
  __shared__ float s_cb[2][16], s_thr[2][16];
  __shared__ __align__(8) CellEntry s_cell[2][8][kCells + 1];
  if (threadIdx.x < 16) {
    s_cb[0][threadIdx.x] = threadIdx.x < (KB == 4 ? 16 : 4) ? cb_K[threadIdx.x] : 0.f;
    s_cb[1][threadIdx.x] = threadIdx.x < (VB == 4 ? 16 : 4) ? cb_V[threadIdx.x] : 0.f;
  }
  __syncthreads();
  build_thresholds<(KB == 4 ? 16 : 4)>(s_cb[0], s_thr[0], threadIdx.x);
  build_thresholds<(VB == 4 ? 16 : 4)>(s_cb[1], s_thr[1], static_cast<int>(threadIdx.x) - 32);
  __syncthreads();
  bool crowded = build_cells_by_position<KB>(s_thr[0], s_cell[0], threadIdx.x);
  crowded |= build_cells_by_position<VB>(s_thr[1], s_cell[1], static_cast<int>(threadIdx.x) - 127);   // threads 127 .. 255: cells 0 .. 128
  // a codebook with two thresholds in one cell keeps the four-step search (the same choice in every CTA)
  if (__syncthreads_or(crowded ? 1 : 0))
    encode_tiles<KB, VB, false>(K, V, slot_mapping, cache, rows, H_kv, num_slots, slot_bytes, s_thr, &s_cell[0][0][0], &s_cell[1][0][0]);
  else
    encode_tiles<KB, VB, true>(K, V, slot_mapping, cache, rows, H_kv, num_slots, slot_bytes, s_thr, &s_cell[0][0][0], &s_cell[1][0][0]);
}

template <int BITS>
__global__ void __launch_bounds__(256) quantize_rotated_kernel(const float* __restrict__ x, int64_t rows,
                                                               const float* __restrict__ cb, uint8_t* __restrict__ idx_out,
                                                               float* __restrict__ norm_out) {
  __shared__ float s_cb[16], s_thr[16];
  __shared__ __align__(8) CellEntry s_cell[kCells + 1];
  if (threadIdx.x < 16) s_cb[threadIdx.x] = threadIdx.x < (BITS == 4 ? 16 : 4) ? cb[threadIdx.x] : 0.f;
  __syncthreads();
  build_thresholds<(BITS == 4 ? 16 : 4)>(s_cb, s_thr, threadIdx.x);
  __syncthreads();
  // the same choice as the paged encoder makes: cell tables unless two thresholds share a cell
  const bool fast = !__syncthreads_or(build_cell<(BITS == 4 ? 16 : 4)>(s_thr, s_cell, threadIdx.x) ? 1 : 0);
  const int lane = threadIdx.x & 31;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += static_cast<int64_t>(gridDim.x) * 8) {
    const float4 raw = *reinterpret_cast<const float4*>(x + row * kHeadDim + 4 * lane);
    const float v[4] = {raw.x, raw.y, raw.z, raw.w};
    const float n = fast ? quantize_row<BITS, true>(v, s_thr, s_cell, idx_out + row * (16 * BITS), lane)
                         : quantize_row<BITS, false>(v, s_thr, s_cell, idx_out + row * (16 * BITS), lane);
    if (lane == 0) norm_out[row] = n;
  }
}

__global__ void __launch_bounds__(256) hadamard128_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                          int64_t rows, float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float v[4];
  load_half4(x + row * kHeadDim + 4 * lane, v);
  fht128_warp(v, lane);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= scale;
  *reinterpret_cast<uint2*>(y + row * kHeadDim + 4 * lane) = pack_half4(v);
}

static int64_t blocks_for_rows(int64_t rows) { return (rows + 7) / 8; }
// Grid of the row kernels that loop over rows: enough CTAs to fill every SM (8 CTAs of 256 threads each), no more.
static unsigned persistent_grid(int64_t rows) {
  const int64_t want = blocks_for_rows(rows), cap = static_cast<int64_t>(device_sm_count(-1)) * 8;
  return static_cast<unsigned>(want < cap ? want : cap);
}

}  // namespace cda

using namespace cda;

extern "C" int cda_b200_paged_encode(const void* K, const void* V, const int32_t* slot_mapping, void* flat_cache,
                                     const float* cb_K, const float* cb_V, int64_t T, int H_kv, int64_t num_slots,
                                     int slot_bytes, int k_bits, int v_bits, void* stream) {
  if (T < 0 || H_kv <= 0 || num_slots < 0) return fail(CDA_ERR_BAD_ARG, "paged_encode: negative size");
  if (!bits_ok(k_bits) || !bits_ok(v_bits)) return fail(CDA_ERR_UNSUPPORTED, "paged_encode: bits must be 2 or 4");
  if (slot_bytes != slot_bytes_for(k_bits, v_bits))
    return fail(CDA_ERR_BAD_SHAPE, "paged_encode: slot width %d, expected %d for k%dv%d", slot_bytes,
                slot_bytes_for(k_bits, v_bits), k_bits, v_bits);
  if (T == 0) return CDA_OK;
  if (!K || !V || !slot_mapping || !flat_cache || !cb_K || !cb_V) return fail(CDA_ERR_BAD_ARG, "paged_encode: null pointer");
  if (!aligned16(K) || !aligned16(V) || !aligned16(flat_cache))
    return fail(CDA_ERR_BAD_ALIGN, "paged_encode: K, V and the cache must be 16-byte aligned");
  const int64_t rows = T * H_kv;
  if (blocks_for_rows(rows) > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "paged_encode: T*H_kv too large");
  // a CTA of 8 warps takes 128 rows per turn; two CTAs fit on an SM
  const int64_t want = (rows + 127) / 128, cap = static_cast<int64_t>(device_sm_count(-1)) * 2;
  const dim3 grid(static_cast<unsigned>(want < cap ? want : cap)), block(256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* k = static_cast<const __half*>(K);
  const __half* v = static_cast<const __half*>(V);
  uint8_t* c = static_cast<uint8_t*>(flat_cache);
  if (k_bits == 4 && v_bits == 4)
    paged_encode_kernel<4, 4><<<grid, block, 0, st>>>(k, v, slot_mapping, c, cb_K, cb_V, rows, H_kv, num_slots, slot_bytes);
  else if (k_bits == 4 && v_bits == 2)
    paged_encode_kernel<4, 2><<<grid, block, 0, st>>>(k, v, slot_mapping, c, cb_K, cb_V, rows, H_kv, num_slots, slot_bytes);
  else if (k_bits == 2 && v_bits == 2)
    paged_encode_kernel<2, 2><<<grid, block, 0, st>>>(k, v, slot_mapping, c, cb_K, cb_V, rows, H_kv, num_slots, slot_bytes);
  else
    paged_encode_kernel<2, 4><<<grid, block, 0, st>>>(k, v, slot_mapping, c, cb_K, cb_V, rows, H_kv, num_slots, slot_bytes);
  return check_launch("paged_encode");
}

extern "C" int cda_b200_quantize_rotated(const float* x_rot, int64_t rows, const float* cb, int bits, uint8_t* idx_out,
                                         float* norm_out, void* stream) {
  if (rows < 0) return fail(CDA_ERR_BAD_ARG, "quantize_rotated: negative rows");
  if (!bits_ok(bits)) return fail(CDA_ERR_UNSUPPORTED, "quantize_rotated: bits must be 2 or 4");
  if (rows == 0) return CDA_OK;
  if (!x_rot || !cb || !idx_out || !norm_out) return fail(CDA_ERR_BAD_ARG, "quantize_rotated: null pointer");
  if (!aligned16(x_rot)) return fail(CDA_ERR_BAD_ALIGN, "quantize_rotated: x_rot must be 16-byte aligned");
  const int64_t blocks = blocks_for_rows(rows);
  if (blocks > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "quantize_rotated: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bits == 4)
    quantize_rotated_kernel<4><<<persistent_grid(rows), 256, 0, st>>>(x_rot, rows, cb, idx_out, norm_out);
  else
    quantize_rotated_kernel<2><<<persistent_grid(rows), 256, 0, st>>>(x_rot, rows, cb, idx_out, norm_out);
  return check_launch("quantize_rotated");
}

extern "C" int cda_b200_hadamard128(const void* x, void* y, int64_t rows, float scale, void* stream) {
  if (rows < 0) return fail(CDA_ERR_BAD_ARG, "hadamard128: negative rows");
  if (rows == 0) return CDA_OK;
  if (!x || !y) return fail(CDA_ERR_BAD_ARG, "hadamard128: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) & 7u) || (reinterpret_cast<uintptr_t>(y) & 7u))
    return fail(CDA_ERR_BAD_ALIGN, "hadamard128: rows must be 8-byte aligned");
  const int64_t blocks = blocks_for_rows(rows);
  if (blocks > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "hadamard128: too many rows");
  hadamard128_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(x), static_cast<__half*>(y), rows, scale);
  return check_launch("hadamard128");
}
