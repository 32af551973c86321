// Causal varlen prefill over the paged compressed cache on the sm_100a tensor-core path (tcgen05.mma, accumulators
// in tensor memory).  Same contract as the reference's fused prefill (cda/kernels_cuda/fa2_cda.py:98-230 with
// fuse_fa2_epilogue=True; oracle: attention_compressed(causal=True, q_offset=seq_len-q_len), cda/algorithm/attention.py:426-482):
// rotate Q, attend to the dequantised keys and values in the rotated domain with bottom-right aligned causal masking,
// round the normalised output to fp16, rotate back.
//
// One CTA per SM works on 256 rows = two blocks of 128 rows = (256 / G) consecutive query positions x the G query heads
// of one KV head, so that a dequantised key/value tile serves the whole GQA group and both blocks.  Keys are processed
// 128 at a time; the two blocks run half a step apart, so one block's softmax overlaps the other's matrix products:
//
//   producer warps (8)    cache slots -> registers (one tile ahead) -> fp16 tiles in shared memory (128-byte swizzled
//                         rows, the layout tcgen05.mma reads).  A tile row is the reference's decoded row, fp16(level x
//                         norm): each key's 16 (or 4) values are computed once and selected per code with byte permutes
//   MMA warp (1 thread)   per block: S = Q K^T (128x128x128, Q and K from shared memory) and O += P V (128x128x128, P from
//                         tensor memory, V from shared memory)
//   softmax warps (2 x 8) two threads per row (64 keys each): TMEM -> registers, softmax scale, mask, online
//                         maximum with lazy rescaling of O, exp2, fp16 P -> TMEM over the thread's own score columns
//
// Tensor memory (512 columns): S of block b at [128 b, 128 b + 128), O of block b at [256 + 128 b, ...).  P of the keys
// [64 h, 64 h + 64) lives in the first 32 columns of the same thread's scores, [128 b + 64 h, + 32).
// Shared memory (198 KB): Q 64 KB, K 2 x 32 KB, V 2 x 32 KB, exchange words, barriers.
//
// The roles hand tiles over through mbarriers; every wait is bounded (umma.cuh) and a wait that gives up sets a fault
// flag and ends the CTA cleanly (TMEM is released).
#include "common.cuh"
#include <type_traits>
#include "umma.cuh"
#include "prefill_umma.cuh"

namespace cda {

// Set when a CTA of the prefill kernel gave up on a wait: later CTAs and launches return at once instead of each
// running into its own time-out.  Read by cda_b200_prefill_fault(), cleared only by cda_b200_prefill_clear_status().
__device__ int g_prefill_fault = 0;
// Sticky per-device report of what the prefill kernel saw in its inputs (cda_b200_prefill_status()):
//   bit 0  a block-table entry was outside the cache (block 0 was read instead)
//   bit 2  a bounded wait gave up (same event as g_prefill_fault)
//   bit 3  a sequence had more new tokens than tokens (q_len > seq_len): its output rows were left unwritten
__device__ int g_prefill_status = 0;

// Diagnostic knobs of the next launches (host side, set by cda_b200_prefill_debug): the wait limit, and whether the
// producers keep back the "K tile 0 is full" arrive so that the waits behind it run out.
static unsigned long long g_wait_limit_ns = umma::kWaitLimitNs;
static int g_withhold_first_k = 0;

namespace pfu {

constexpr int kRows = 128;            // rows of one block (one tcgen05.mma M)
constexpr int kBlocks = 2;            // row blocks per CTA
constexpr int kKeys = 128;            // keys per tile
constexpr int kSoftmaxWarpsPerBlock = 8, kSoftmaxWarps = kBlocks * kSoftmaxWarpsPerBlock, kProducerWarps = 8;
constexpr int kMmaWarp = kSoftmaxWarps + kProducerWarps;
constexpr int kThreads = (kMmaWarp + 1) * 32;
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256;    // + 128 * block
constexpr float kLazy = 4.0f;         // O is rescaled only when the row maximum grew by more than 2^4

// shared memory map (bytes from the 1024-aligned base)
constexpr int kOffQ = 0;                       // 2 blocks x (2 column blocks x 128 rows x 128 B)
constexpr int kOffK = 65536;                   // 2 stages x (2 column blocks x 128 rows x 128 B); also stages the O rows
constexpr int kOffV = 131072;                  // 2 stages x (2 column blocks x 128 rows x 128 B)
constexpr int kTileBytes = 32768, kColBlockBytes = 16384;
constexpr int kOffXch = 196608;                // 2 blocks x 2 parities x 2 halves x 128 floats: row maxima / sums of the two threads of a row
constexpr int kOffBar = kOffXch + 4096;        // mbarriers, TMEM address, flags
constexpr int kSmemBytes = kOffBar + 256 + 1024;   // + slack for the 1024-byte alignment

// barrier slots (8 bytes each) inside kOffBar
constexpr int kBarKFull = 0, kBarKEmpty = 2, kBarVFull = 4, kBarVEmpty = 6, kBarSFull = 8, kBarPFull = 10, kBarPvDone = 12;   // 14 barriers
constexpr int kOffTmemAddr = 160, kOffOutcome = 168, kOffAbort = 192;   // outcome words: 2 per waiting group (3 groups); WaitState (16 B)

__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// A group of warps waits for an mbarrier phase: only lane 0 of the group's first warp polls, the others are parked on
// a named hardware barrier (a parked warp takes no issue slots from the warps that are working).  The poller always
// arrives at the named barrier -- its own wait is bounded -- and publishes its outcome in one of two words used
// alternately (it can be at most one call ahead of the slowest reader), so the result is the same for every thread
// of the group and nobody is left behind at a later barrier.
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
struct GroupWaiter {
  volatile int* outcome;     // two words in shared memory
  volatile umma::WaitState* abort_flag;
  int id, nthreads, turn;
  bool leader;               // lane 0 of the group's first warp
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity) {
    if (leader) outcome[turn] = umma::mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    named_barrier(id, nthreads);
    const bool ok = outcome[turn] != 0;
    turn ^= 1;
    return ok;
  }
};
constexpr int kBarIdSoftmax = 1, kBarIdProducer = 3;   // named barriers 1 and 2: the softmax groups of blocks 0 and 1

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) {   // byte offset inside a block of 128-byte rows
  return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

// ---- 4-bit codes: exact rows from a per-key table held in registers -----------------------------------------------------
// The reference decodes a row as fp16(level * norm) (fp32 product, one rounding; compression.py:337-361).  A key has only
// 16 such values, so the producer computes them once per key -- 16 fp32 products and roundings -- and keeps them as byte
// planes: lo[k] holds the low bytes of the values of levels 4k .. 4k + 3, hi[k] the high bytes.  A code then selects its
// value with byte permutes (the low three bits of the code pick one of eight bytes, its top bit picks the register pair),
// four codes per instruction, and the tile holds exactly the reference's fp16 rows: no table in shared memory, no gather,
// no per-level or per-norm rounding of its own.
struct LevelPlanes { uint32_t lo[4], hi[4]; };
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// cb_addr: shared address of the 16 fp32 levels (16-byte aligned; every thread reads the same words).
__device__ __forceinline__ LevelPlanes level_planes(uint32_t cb_addr, float norm) {
  LevelPlanes t;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint4 c = lds128(cb_addr + 16u * k);
    float p0, p1, p2, p3;                            // packed fp32 products: each half rounds as the scalar multiply does
    f2_unpack(f2_mul(f2_pack(c.x, c.y), f2_pack(norm, norm)), p0, p1);
    f2_unpack(f2_mul(f2_pack(c.z, c.w), f2_pack(norm, norm)), p2, p3);
    const uint32_t h0 = pack_half2(p0, p1), h1 = pack_half2(p2, p3);
    t.lo[k] = prmt(h0, h1, 0x6420u);
    t.hi[k] = prmt(h0, h1, 0x7531u);
  }
  return t;
}
// 16 bytes of 4-bit codes (32 coordinates of token row `nl`, piece `quad` of its 64 code bytes) into the tile.  A code byte
// holds coordinate 2j in its high nibble and 2j + 1 in its low nibble (compression.py:163-188), so the selector nibbles of
// two bytes pick (1, 0, 3, 2); the last two permutes put the bytes back in order while pairing low and high bytes.
__device__ __forceinline__ void expand_quad_exact(uint32_t tile, const LevelPlanes& t, const uint4& w, int nl, int quad) {
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    const uint32_t x = ws[wi];
    const uint32_t m = x & 0x77777777u;            // low three bits of every code: byte selectors
    const uint32_t y = x & 0x88888888u, a = y << 4;   // top bit of every code, as the sign bit of a byte of y or a
    uint32_t v[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {                  // two code bytes = four coordinates per turn
      const uint32_t sel = h ? m >> 16 : m;
      const uint32_t upper = prmt(a, y, h ? 0xFBEAu : 0xD9C8u);   // 0xFF in the bytes whose code is 8 .. 15
      const uint32_t la = prmt(t.lo[0], t.lo[1], sel), lb = prmt(t.lo[2], t.lo[3], sel);
      const uint32_t ha = prmt(t.hi[0], t.hi[1], sel), hb = prmt(t.hi[2], t.hi[3], sel);
      const uint32_t lo = (lb & upper) | (la & ~upper), hi = (hb & upper) | (ha & ~upper);
      v[2 * h] = prmt(lo, hi, 0x4051u);
      v[2 * h + 1] = prmt(lo, hi, 0x6273u);
    }
    const int c16 = quad * 4 + wi;                 // 16-byte chunk of the row: 8 coordinates
    sts128(tile + (c16 >> 3) * kColBlockBytes + sw128(nl, c16 & 7), v[0], v[1], v[2], v[3]);
  }
}

// 2-bit codes: a key has four values; their low bytes sit in one register, their high bytes in another.
struct LevelPlanes2 { uint32_t lo, hi; };
__device__ __forceinline__ LevelPlanes2 level_planes2(uint32_t cb_addr, float norm) {
  const uint4 c = lds128(cb_addr);
  float p0, p1, p2, p3;
  f2_unpack(f2_mul(f2_pack(c.x, c.y), f2_pack(norm, norm)), p0, p1);
  f2_unpack(f2_mul(f2_pack(c.z, c.w), f2_pack(norm, norm)), p2, p3);
  const uint32_t h0 = pack_half2(p0, p1), h1 = pack_half2(p2, p3);
  return LevelPlanes2{prmt(h0, h1, 0x6420u), prmt(h0, h1, 0x7531u)};
}
// 16 bytes of 2-bit codes (64 coordinates of token row `nl`, piece `quad` of its 32 code bytes) into the tile.  A code byte
// holds coordinates 4j .. 4j + 3 from its top bit pair down (compression.py:375-386).  Two bytes are spread to eight
// nibbles -- coordinates 3, 2, 1, 0 of the first byte, then of the second -- which select the value bytes four at a time.
__device__ __forceinline__ void expand_quad_exact2(uint32_t tile, const LevelPlanes2& t, const uint4& w, int nl, int quad) {
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {               // two code bytes = 8 coordinates = one 16-byte chunk
      uint32_t s = hb ? ws[wi] >> 16 : ws[wi] & 0xFFFFu;
      s = (s | (s << 8)) & 0x00FF00FFu;
      s = (s | (s << 4)) & 0x0F0F0F0Fu;
      s = (s | (s << 2)) & 0x33333333u;
      const uint32_t l0 = prmt(t.lo, t.lo, s), h0 = prmt(t.hi, t.hi, s);
      const uint32_t l1 = prmt(t.lo, t.lo, s >> 16), h1 = prmt(t.hi, t.hi, s >> 16);
      const int c16 = quad * 8 + wi * 2 + hb;
      sts128(tile + (c16 >> 3) * kColBlockBytes + sw128(nl, c16 & 7), prmt(l0, h0, 0x6273u), prmt(l0, h0, 0x4051u),
             prmt(l1, h1, 0x6273u), prmt(l1, h1, 0x4051u));
    }
  }
}

// One thread's 64 scores of a tile (columns s_col .. s_col + 63 of its TMEM lane), times the factor kf (softmax scale x log2 e)
// (16-byte aligned).  MASK: keys beyond q_pos (the row's diagonal) count as minus infinity.  The next 16 columns are
// requested before the current ones are worked on (tcgen05.wait::ld covers every load issued so far).
template <bool MASK>
__device__ __forceinline__ float row_max(uint32_t s_col, float kf, int key0, int q_pos) {
  float mx[2] = {-INFINITY, -INFINITY};
  const uint64_t ku = f2_pack(kf, kf);
  uint32_t s[2][16];
  umma::tmem_ld16(s_col, s[0]);
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    umma::tmem_wait_ld();
    if (ch < 3) umma::tmem_ld16(s_col + 16 * (ch + 1), s[(ch + 1) & 1]);
#pragma unroll
    for (int c = 0; c < 16; c += 4) {
      float x[4];
      f2_unpack(f2_mul(f2_pack(s[ch & 1][c], s[ch & 1][c + 1]), ku), x[0], x[1]);
      f2_unpack(f2_mul(f2_pack(s[ch & 1][c + 2], s[ch & 1][c + 3]), ku), x[2], x[3]);
      if (MASK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = key0 + 16 * ch + c + i > q_pos ? -INFINITY : x[i];
      }
      mx[0] = fmax3(mx[0], x[0], x[1]);
      mx[1] = fmax3(mx[1], x[2], x[3]);
    }
  }
  return fmaxf(mx[0], mx[1]);
}
// exp2(score * kn - m) for the same 64 scores; P as fp16 pairs into columns s_col .. s_col + 31 (the value norms are
// already inside the V tile).  Returns the sum of the probabilities.
template <bool MASK>
__device__ __forceinline__ float row_probabilities(uint32_t s_col, float kf, float m, int key0, int q_pos) {
  uint64_t sum = f2_pack(0.f, 0.f);
  const uint64_t neg_m = f2_pack(-m, -m);
  const uint64_t ku = f2_pack(kf, kf);
  uint32_t s[2][16];
  umma::tmem_ld16(s_col, s[0]);
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint32_t pk[8];
    umma::tmem_wait_ld();
    if (ch < 3) umma::tmem_ld16(s_col + 16 * (ch + 1), s[(ch + 1) & 1]);
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      float a0, a1;
      f2_unpack(f2_fma(f2_pack(s[ch & 1][c], s[ch & 1][c + 1]), ku, neg_m), a0, a1);
      if (MASK) {
        a0 = key0 + 16 * ch + c > q_pos ? -INFINITY : a0;
        a1 = key0 + 16 * ch + c + 1 > q_pos ? -INFINITY : a1;
      }
      const float e0 = fast_exp2(a0), e1 = fast_exp2(a1);
      sum = f2_add(sum, f2_pack(e0, e1));
      pk[c / 2] = pack_half2(e0, e1);
    }
    umma::tmem_st8(s_col + 8 * ch, pk);
  }
  float s0, s1;
  f2_unpack(sum, s0, s1);
  return s0 + s1;
}

// fp16 pairs times a common factor (a power of two here).
__device__ __forceinline__ uint32_t hmul2_scalar(uint32_t pair, float f) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&pair), __float2half2_rn(f));
  return *reinterpret_cast<const uint32_t*>(&r);
}
// Multiplies `chunks` 8-column pieces of fp16 pairs starting at column `col` of this thread's TMEM lane by f.
__device__ __forceinline__ void scale_p_chunks(uint32_t col, int chunks, float f) {
  umma::tmem_wait_st();
#pragma unroll 1
  for (int cc = 0; cc < chunks; ++cc) {
    uint32_t pp[8];
    umma::tmem_ld8(col + 8 * cc, pp);
    umma::tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 8; ++i) pp[i] = hmul2_scalar(pp[i], f);
    umma::tmem_st8(col + 8 * cc, pp);
  }
}
// The one-pass form of the two functions above for every tile but a row's first: the probabilities are taken against
// the reference m the row already has (its running maximum before this tile) instead of the tile's own maximum, which
// saves the first read of the scores and the wait for the other half of the row.  An fp16 probability can carry 2^15;
// whenever a chunk of 16 scores would pass 2^kSafe the thread moves its own reference up by a whole number d of
// binary orders first (its earlier probabilities of this tile and their sum are multiplied by 2^-d).  `shift` returns
// the total of those moves; the caller settles the two halves of a row on the larger shift before P is published.
constexpr float kSafe = 14.0f;
template <bool MASK>
__device__ __forceinline__ float row_probabilities_stale(uint32_t s_col, float kf, float m, int key0, int q_pos, float& shift) {
  uint64_t sum = f2_pack(0.f, 0.f);
  uint64_t neg_ref = f2_pack(-m, -m);
  const uint64_t ku = f2_pack(kf, kf);
  shift = 0.f;
  uint32_t s[2][16];
  umma::tmem_ld16(s_col, s[0]);
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint32_t pk[8];
    umma::tmem_wait_ld();
    if (ch < 3) umma::tmem_ld16(s_col + 16 * (ch + 1), s[(ch + 1) & 1]);
    float a[16];
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      f2_unpack(f2_fma(f2_pack(s[ch & 1][c], s[ch & 1][c + 1]), ku, neg_ref), a[c], a[c + 1]);
      if (MASK) {
        a[c] = key0 + 16 * ch + c > q_pos ? -INFINITY : a[c];
        a[c + 1] = key0 + 16 * ch + c + 1 > q_pos ? -INFINITY : a[c + 1];
      }
    }
    float cmax = fmax3(a[0], a[1], a[2]);
#pragma unroll
    for (int c = 3; c < 15; c += 2) cmax = fmax3(cmax, a[c], a[c + 1]);
    cmax = fmaxf(cmax, a[15]);
    if (__any_sync(0xffffffffu, cmax > kSafe)) {             // rare: a score far above everything the row has seen
      const float d = cmax > kSafe ? ceilf(fminf(cmax, 1.0e30f)) : 0.f;
      const float f = fast_exp2(-d);
      shift += d;
      neg_ref = f2_pack(-(m + shift), -(m + shift));
#pragma unroll
      for (int c = 0; c < 16; ++c) a[c] -= d;
      sum = f2_mul(sum, f2_pack(f, f));
      scale_p_chunks(s_col, ch, f);                          // every lane takes part (factor 1 where d = 0)
    }
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      const float e0 = fast_exp2(a[c]), e1 = fast_exp2(a[c + 1]);
      sum = f2_add(sum, f2_pack(e0, e1));
      pk[c / 2] = pack_half2(e0, e1);
    }
    umma::tmem_st8(s_col + 8 * ch, pk);
  }
  float s0, s1;
  f2_unpack(sum, s0, s1);
  return s0 + s1;
}

// This thread's 64 fp32 columns of O times `factor`.
__device__ __forceinline__ void rescale_o(uint32_t o_col, float factor) {
#pragma unroll 1
  for (int ch = 0; ch < 2; ++ch) {
    uint32_t o[32];
    umma::tmem_ld32(o_col + 32 * ch, o);
    umma::tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
      float o0, o1;
      f2_unpack(f2_mul(f2_pack(o[c], o[c + 1]), f2_pack(factor, factor)), o0, o1);
      o[c] = __float_as_uint(o0);
      o[c + 1] = __float_as_uint(o1);
    }
    umma::tmem_st32(o_col + 32 * ch, o);
  }
}
// Rows of 128 fp16 parked in shared memory: 256-byte rows, 16-byte chunk c of row r at chunk position c ^ (r & 15).
__device__ __forceinline__ uint32_t staged_chunk(uint32_t area, uint32_t row, uint32_t chunk) {
  return area + row * 256u + ((chunk ^ (row & 15u)) << 4);
}
// Hadamard rotation (times `scale`, rounded to fp16) of the 16 staged rows 16 * tile .. 16 * tile + 15 on the tensor
// cores (common.cuh: RotFrag).  Lane 4r + c ends up with coordinates 32 w + 8 c .. 32 w + 8 c + 7 (w = 0..3) of rows r and
// r + 8 and hands each such 16-byte piece to emit(row, w, piece).  Two passes, one per 8-column half of the MMA output,
// keep the accumulators at 32 registers; the first pass's results wait as fp16 pairs.
template <class Emit>
__device__ __forceinline__ void rotate_staged_rows(uint32_t area, int tile, int lane, float scale, Emit emit) {
  const int r = lane >> 2, c = lane & 3;
  const uint32_t row_lo = 16u * tile + r, row_hi = row_lo + 8u;
  const RotFrag f = make_rot_frag(lane);
  uint32_t first[8][2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    float y[8][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 lo = lds128(staged_chunk(area, row_lo, 4 * j + c)), hi = lds128(staged_chunk(area, row_hi, 4 * j + c));
#pragma unroll
      for (int i = 0; i < 4; ++i) y[2 * j][i] = y[2 * j + 1][i] = 0.f;
      mma_16816(y[2 * j], lo.x, hi.x, lo.y, hi.y, f.b0[t], f.b1[t]);
      mma_16816(y[2 * j + 1], lo.z, hi.z, lo.w, hi.w, f.b0[t], f.b1[t]);
    }
#pragma unroll
    for (int bit = 1; bit < 8; bit <<= 1)
#pragma unroll
      for (int g = 0; g < 8; ++g)
        if (!(g & bit)) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float a = y[g][i], b = y[g | bit][i];
            y[g][i] = a + b;
            y[g | bit][i] = a - b;
          }
        }
    if (t == 0) {
#pragma unroll
      for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int h = 0; h < 2; ++h) first[g][h] = pack_half2(y[g][2 * h] * scale, y[g][2 * h + 1] * scale);
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int w = 0; w < 4; ++w)   // coordinates 4 g0 + 2 t + e of the piece: g0 = 0 (t = 0, 1), then g0 = 1
          emit(h ? row_hi : row_lo, w, make_uint4(first[2 * w][h], pack_half2(y[2 * w][2 * h] * scale, y[2 * w][2 * h + 1] * scale),
                                                  first[2 * w + 1][h], pack_half2(y[2 * w + 1][2 * h] * scale, y[2 * w + 1][2 * h + 1] * scale)));
    }
  }
}

}  // namespace pfu

// KB == VB == 16 selects the dense source: keys and values are fp16 rows in the rotated frame (`k_dense`, `v_dense`,
// sequence b's rows start at cu_k[b]) instead of codes in the paged cache; the producers then copy rows into the tiles.
template <int G, int KB, int VB>
__global__ void __launch_bounds__(pfu::kThreads, 1) prefill_umma_kernel(const PrefillUmmaParams p) {
  using namespace pfu;
  using namespace umma;
  constexpr bool kDense = KB == 16;
  static_assert(!kDense || VB == 16, "dense source: both sides");
  constexpr int kPosPerTile = kBlocks * kRows / G;
  constexpr int kSlotBytes = 16 * KB + 16 * VB + 16;
  constexpr int kProducerThreads = kProducerWarps * 32;
  constexpr int kItK = kKeys * KB / kProducerThreads, kItV = kKeys * VB / kProducerThreads;   // 16-byte code pieces per producer thread and tile
  constexpr int kLevK = KB == 4 ? 16 : 4, kLevV = VB == 4 ? 16 : 4;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_addr(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Grid (sequence, KV head, tile rank): CTAs are handed out in x-fastest order, so every sequence's longest rows go first
  // and the last CTAs of the launch are the shortest rows of the longest sequence (close to longest-job-first).
  const int kvh = blockIdx.y, b = blockIdx.x;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int seq_len = p.seq_lens[b];
  const int n_qtiles = (q_len + kPosPerTile - 1) / kPosPerTile;
  const int qt = n_qtiles - 1 - static_cast<int>(blockIdx.z);   // longest rows first
  if (qt < 0 || seq_len <= 0) return;
  if (q_len > seq_len) {   // more new tokens than tokens: not a causal chunk; report it, write nothing
    if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) atomicOr(&g_prefill_status, 8);
    return;
  }
  if (*reinterpret_cast<volatile int*>(&g_prefill_fault)) return;
  const int p0 = qt * kPosPerTile;                               // first query position (within the new tokens) of this tile
  const int q_offset = seq_len - q_len;                          // bottom-right alignment
  const int pos_hi = min(p0 + kPosPerTile, q_len) - 1;
  const int n_tiles = (q_offset + pos_hi) / kKeys + 1;           // key tiles that hold an unmasked key
  const int g = p.group;

  volatile WaitState* abort_flag = reinterpret_cast<volatile WaitState*>(sm + kOffBar + kOffAbort);
  const uint32_t bar0 = base + kOffBar;
  auto bar = [&](int i) { return bar0 + 8u * i; };

  // The raw Q rows are requested first, one 16-byte chunk per thread and turn, so that their latency runs under the
  // table set-up; they are parked in the (still unused) K stages further down.
  constexpr int kQTurns = (kBlocks * kRows * 16 + kThreads - 1) / kThreads;
  uint4 q_raw[kQTurns];
#pragma unroll
  for (int k = 0; k < kQTurns; ++k) {
    const int i = tid + k * kThreads, r = i >> 4, chunk = i & 15;
    const int pos = p0 + r / G, hl = r % G;
    q_raw[k] = make_uint4(0u, 0u, 0u, 0u);
    if (i < kBlocks * kRows * 16 && pos < q_len && hl < g)
      q_raw[k] = __ldg(reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(q_begin + pos) * p.H_q + kvh * g + hl) * kHeadDim) + chunk);
  }

  // The fp32 code levels of both sides: the producers turn them into each key's exact fp16 values.
  __shared__ __align__(16) float s_levels[2][16];
  if constexpr (!kDense) {
    if (tid < kLevK) s_levels[0][tid] = __ldg(p.cb_k + tid);
    else if (tid >= 32 && tid < 32 + kLevV) s_levels[1][tid - 32] = __ldg(p.cb_v + tid - 32);
  }

  // ---- set-up: barriers, TMEM, tables, rotated queries -----------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(kBarKFull + i), kProducerWarps); mbar_init(bar(kBarKEmpty + i), 1);
      mbar_init(bar(kBarVFull + i), kProducerWarps); mbar_init(bar(kBarVEmpty + i), 1);
      mbar_init(bar(kBarSFull + i), 1); mbar_init(bar(kBarPFull + i), kSoftmaxWarpsPerBlock); mbar_init(bar(kBarPvDone + i), 1);
    }
    abort_flag->abort = 0;
    abort_flag->limit_ns = p.wait_limit_ns;
    mbar_init_fence();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(base + kOffBar + kOffTmemAddr, kTmemCols);
    tmem_relinquish();
  }
  // Q: park the raw rows; then warps 0..15 rotate 16 rows each and store them as the A operand of Q K^T (K-major,
  // 128-byte swizzle)
#pragma unroll
  for (int k = 0; k < kQTurns; ++k) {
    const int i = tid + k * kThreads;
    if (i < kBlocks * kRows * 16) sts128(staged_chunk(base + kOffK, i >> 4, i & 15), q_raw[k].x, q_raw[k].y, q_raw[k].z, q_raw[k].w);
  }
  __syncthreads();
  if (warp < kBlocks * kRows / 16) {
    rotate_staged_rows(base + kOffK, warp, lane, kRsqrtD, [&](uint32_t row, int w, const uint4& piece) {
      const uint32_t t = row & (kRows - 1);
      sts128(base + kOffQ + (row / kRows) * kTileBytes + (w >> 1) * kColBlockBytes + sw128(t, 4 * (w & 1) + (lane & 3)), piece.x, piece.y,
             piece.z, piece.w);
    });
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sm + kOffBar + kOffTmemAddr);

  if (warp < kSoftmaxWarps) {
    // ================= softmax: per block, two threads per row, 64 of the tile's 128 keys each ================================
    const int blk = warp / kSoftmaxWarpsPerBlock, w = warp % kSoftmaxWarpsPerBlock;
    const int quarter = w & 3, half = w >> 2;                // TMEM lane quarter of this warp; which 64 keys / 64 O columns
    const int t = quarter * 32 + lane;                       // row inside the block
    const int q_pos = q_offset + p0 + (blk * kRows + t) / G; // key index of the diagonal for this row
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_col = lane_base + kColS + 128 * blk + 64 * half;     // this thread's scores; P goes over the first 32 columns
    const uint32_t o_col = lane_base + kColO + 128 * blk + 64 * half;     // this thread's half of the O row
    float* xch = reinterpret_cast<float*>(sm + kOffXch) + blk * 4 * kRows;   // [2 parities][2 halves][128 rows]
    const int bar_id = kBarIdSoftmax + blk, group_threads = kSoftmaxWarpsPerBlock * 32;
    float m_used = -INFINITY, l_run = 0.f;
    const float kf = p.scale_log2;                         // the tiles hold whole rows (norm included): one factor for every key
    bool alive = true;
    GroupWaiter gw{reinterpret_cast<volatile int*>(sm + kOffBar + kOffOutcome + 8 * blk), abort_flag, bar_id, group_threads, 0, w == 0 && lane == 0};
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      // Q K^T of tile j was issued behind P V of tile j - 1 of this block, so its O is at rest as well
      alive = gw.wait(bar(kBarSFull + blk), j & 1);
      if (!alive) break;
      tc_fence_after_sync();
      const int key0 = j * kKeys + 64 * half;
      const bool diag = key0 + 63 > q_offset + p0;           // some row of the CTA masks some of these keys

      if (__any_sync(0xffffffffu, m_used == -INFINITY)) {
      // a row without a reference yet (tile 0: key 0 is never masked, so every row has one afterwards): two passes
      // pass 1: maximum of this thread's 64 scaled scores (diagonal tiles take the masking variant)
      const float mx_own = diag ? row_max<true>(s_col, kf, key0, q_pos) : row_max<false>(s_col, kf, key0, q_pos);
      float mx = mx_own;
      // the row maximum needs the other half's keys
      xch[((j & 1) * 2 + half) * kRows + t] = mx;
      named_barrier(bar_id, group_threads);
      mx = fmaxf(mx, xch[((j & 1) * 2 + (half ^ 1)) * kRows + t]);
      float factor = 1.0f;
      if (mx > m_used + kLazy || m_used == -INFINITY) {
        const float m_new = fmaxf(m_used, mx);
        factor = m_used == -INFINITY ? 0.0f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l_run *= factor;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, factor != 1.0f);
      if (rescale) rescale_o(o_col, factor);
      // pass 2: probabilities.  The scores are read again from TMEM, 16 columns at a time; the fp16 P of a chunk
      // (keys 2c, 2c+1 in column c) goes straight over score columns this thread has already consumed.
      l_run += diag ? row_probabilities<true>(s_col, kf, m_used, key0, q_pos) : row_probabilities<false>(s_col, kf, m_used, key0, q_pos);
      } else {
      // one pass against the reference the row already has; the halves of a row then settle on a common reference
      float shift;
      float sum = diag ? row_probabilities_stale<true>(s_col, kf, m_used, key0, q_pos, shift)
                       : row_probabilities_stale<false>(s_col, kf, m_used, key0, q_pos, shift);
      xch[((j & 1) * 2 + half) * kRows + t] = shift;
      named_barrier(bar_id, group_threads);
      const float common = fmaxf(shift, xch[((j & 1) * 2 + (half ^ 1)) * kRows + t]);
      if (__any_sync(0xffffffffu, common > 0.f)) {           // rare: some row of this warp moved its reference
        const float f_own = fast_exp2(shift - common);       // this half's probabilities against the common reference
        if (__any_sync(0xffffffffu, shift != common)) scale_p_chunks(s_col, 4, f_own);
        sum *= f_own;
        const float f_old = fast_exp2(-common);              // what the row had before this tile
        rescale_o(o_col, f_old);                             // O is at rest: P V of this tile waits for the arrive below
        l_run *= f_old;
        m_used += common;
      }
      l_run += sum;
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull + blk));
    }
    // ---- epilogue part 1: normalised fp16 row of O into the staging area (the K stages), 256-byte rows, chunk XOR (row & 15)
    if (alive) {   // the row sum needs the other half's keys
      const int j = n_tiles;
      xch[((j & 1) * 2 + half) * kRows + t] = l_run;
      named_barrier(bar_id, group_threads);
      l_run += xch[((j & 1) * 2 + (half ^ 1)) * kRows + t];
      alive = gw.wait(bar(kBarPvDone + blk), (n_tiles - 1) & 1);
    }
    if (alive) {
      tc_fence_after_sync();
      const float inv = 1.0f / fmaxf(l_run, 1e-30f);
      const uint32_t row = static_cast<uint32_t>(blk * kRows + t);
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t o[32];
        tmem_ld32(o_col + 32 * ch, o);
        tmem_wait_ld();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint32_t h[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float o0, o1;
            f2_unpack(f2_mul(f2_pack(o[8 * c8 + 2 * i], o[8 * c8 + 2 * i + 1]), f2_pack(inv, inv)), o0, o1);
            h[i] = pack_half2(o0, o1);
          }
          const uint32_t chunk = static_cast<uint32_t>(8 * half + ch * 4 + c8);
          sts128(base + kOffK + row * 256u + ((chunk ^ (row & 15u)) << 4), h[0], h[1], h[2], h[3]);
        }
      }
      // ---- epilogue part 2: once the block's 128 rows are parked, its eight warps rotate 16 of them each and store them; the
      // other block may still be in its last tile (`alive` is the same for every thread of the group)
      named_barrier(bar_id, group_threads);
      rotate_staged_rows(base + kOffK, warp, lane, kRsqrtD, [&](uint32_t row, int w, const uint4& piece) {
        const int pos = p0 + static_cast<int>(row) / G, hl = static_cast<int>(row) % G;
        if (pos < q_len && hl < g)
          *reinterpret_cast<uint4*>(p.out + (static_cast<int64_t>(q_begin + pos) * p.H_q + kvh * g + hl) * kHeadDim + 32 * w + 8 * (lane & 3)) = piece;
      });
    }
    tc_fence_before_sync();
  } else if (warp < kSoftmaxWarps + kProducerWarps) {
    // ================= producers: slots -> unit-level fp16 tiles ============================================================
    const int pt = tid - kSoftmaxWarps * 32;                 // 0..255
   if constexpr (kDense) {
    // Dense source: a tile is 128 rows of 256 bytes = 2048 16-byte chunks, eight per producer thread, copied with cp.async
    // straight into the swizzled tile; the copies of a tile start as soon as its stage is free (while the previous tile is
    // being consumed), and the thread publishes the tile when its own copies have landed.
    GroupWaiter gw{reinterpret_cast<volatile int*>(sm + kOffBar + kOffOutcome + 16), abort_flag, kBarIdProducer, kProducerThreads, 0, pt == 0};
    const int64_t row_halfs = static_cast<int64_t>(p.H_kv) * kHeadDim;
    const __half* k_src = p.k_dense + (static_cast<int64_t>(p.cu_k[b]) * p.H_kv + kvh) * kHeadDim;
    const __half* v_src = p.v_dense + (static_cast<int64_t>(p.cu_k[b]) * p.H_kv + kvh) * kHeadDim;
    auto copy_tile = [&](const __half* src, uint32_t tile, int j) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int x = pt + kProducerThreads * it, nl = x >> 4, c16 = x & 15;
        const int n = min(j * kKeys + nl, seq_len - 1);      // keys past the end are masked later; copy a valid row
        cp_async16(tile + (c16 >> 3) * kColBlockBytes + sw128(nl, c16 & 7), src + n * row_halfs + c16 * 8);
      }
      cp_async_commit();
    };
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
      if (i >= 2 && !gw.wait(bar(kBarKEmpty + (i & 1)), ((i - 2) >> 1) & 1)) break;
      copy_tile(k_src, base + kOffK + (i & 1) * kTileBytes, i);
      if (i >= 2 && !gw.wait(bar(kBarVEmpty + (i & 1)), ((i - 2) >> 1) & 1)) break;
      copy_tile(v_src, base + kOffV + (i & 1) * kTileBytes, i);
      cp_async_wait<1>();
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && !(p.withhold_first_k && i == 0)) mbar_arrive(bar(kBarKFull + (i & 1)));
      cp_async_wait<0>();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarVFull + (i & 1)));
    }
    cp_async_wait<0>();
   } else {
    const int nl = pt & (kKeys - 1);                         // this thread's key (row of the tile)
    const int32_t* bt_row = p.block_table + static_cast<int64_t>(b) * p.bt_stride;
    const int64_t row_stride = static_cast<int64_t>(p.H_kv) * kSlotBytes;
    bool bad_block = false;
    GroupWaiter gw{reinterpret_cast<volatile int*>(sm + kOffBar + kOffOutcome + 16), abort_flag, kBarIdProducer, kProducerThreads, 0, pt == 0};

    // Block ids are read one fetch ahead of the slots they address, slot words one tile ahead of their expansion:
    // neither global-memory latency sits on the tile-to-tile chain.
    auto block_id = [&](int tile) -> int {
      const int n = min(tile * kKeys + nl, seq_len - 1);     // keys past the end are masked later; read a valid slot
      const int bi = p.bs_shift >= 0 ? n >> p.bs_shift : n / p.block_size;
      return __ldg(bt_row + bi);
    };
    auto slot_ptr = [&](int blk, int tile) -> const uint8_t* {
      const int n = min(tile * kKeys + nl, seq_len - 1);
      const int in_block = p.bs_shift >= 0 ? n & (p.block_size - 1) : n % p.block_size;
      if (static_cast<unsigned>(blk) >= static_cast<unsigned>(p.num_blocks)) { bad_block = true; blk = 0; }
      return p.cache + (static_cast<int64_t>(blk) * p.block_size + in_block) * row_stride + kvh * kSlotBytes;
    };
    // Producer thread t works on key t mod 128 of every tile: it reads that key's slot (the 16-byte code pieces
    // (t / 128) kIt + it of either side, and its norm), builds the key's exact values once per side and expands its
    // pieces; the lanes of a warp store to 32 different rows of the swizzled tile (no bank conflicts).
    struct KRegs { uint4 w[kItK]; float n; };
    struct VRegs { uint4 w[kItV]; float n; };
    int blk_k = block_id(0), blk_v = blk_k;                   // block id of this key's row in the next tile to fetch
    auto load_k = [&](int j, KRegs& r) {
      if (j >= n_tiles) return;
      const uint8_t* src = slot_ptr(blk_k, j);
#pragma unroll
      for (int it = 0; it < kItK; ++it) r.w[it] = __ldg(reinterpret_cast<const uint4*>(src + 16 * ((pt >> 7) * kItK + it)));
      r.n = __ldg(reinterpret_cast<const float*>(src + 16 * KB + 16 * VB));
      blk_k = block_id(j + 1);
    };
    auto load_v = [&](int j, VRegs& r) {
      if (j >= n_tiles) return;
      const uint8_t* src = slot_ptr(blk_v, j);
#pragma unroll
      for (int it = 0; it < kItV; ++it) r.w[it] = __ldg(reinterpret_cast<const uint4*>(src + 16 * KB + 16 * ((pt >> 7) * kItV + it)));
      r.n = __ldg(reinterpret_cast<const float*>(src + 16 * KB + 16 * VB + 4));
      blk_v = block_id(j + 1);
    };
    auto expand_side = [&](auto bits_tag, uint32_t tile, uint32_t levels, const uint4* w, float norm) {
      constexpr int kBits = decltype(bits_tag)::value, kIt = kBits / 2;
      if constexpr (kBits == 4) {
        const LevelPlanes t = level_planes(levels, norm);
#pragma unroll
        for (int it = 0; it < kIt; ++it) expand_quad_exact(tile, t, w[it], nl, (pt >> 7) * kIt + it);
      } else {
        const LevelPlanes2 t = level_planes2(levels, norm);
#pragma unroll
        for (int it = 0; it < kIt; ++it) expand_quad_exact2(tile, t, w[it], nl, (pt >> 7) * kIt + it);
      }
      fence_async_smem();
      __syncwarp();
    };
    // Tile i is expanded from registers that were filled while tile i-1 was being expanded; its K stage is free once
    // Q K^T of tile i-2 is done for both blocks, its V stage once P V of tile i-2 is done for both blocks.
    KRegs kr;
    VRegs vr;
    load_k(0, kr);
    load_v(0, vr);
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
      if (i >= 2 && !gw.wait(bar(kBarKEmpty + (i & 1)), ((i - 2) >> 1) & 1)) break;
      expand_side(std::integral_constant<int, KB>{}, base + kOffK + (i & 1) * kTileBytes, smem_addr(s_levels[0]), kr.w, kr.n);
      if (lane == 0 && !(p.withhold_first_k && i == 0)) mbar_arrive(bar(kBarKFull + (i & 1)));
      load_k(i + 1, kr);
      if (i >= 2 && !gw.wait(bar(kBarVEmpty + (i & 1)), ((i - 2) >> 1) & 1)) break;
      expand_side(std::integral_constant<int, VB>{}, base + kOffV + (i & 1) * kTileBytes, smem_addr(s_levels[1]), vr.w, vr.n);
      if (lane == 0) mbar_arrive(bar(kBarVFull + (i & 1)));
      load_v(i + 1, vr);
    }
    if (bad_block) atomicOr(&g_prefill_status, 1);
   }
  } else {
    // ================= MMA issuer ==================================================================================================
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f16(kRows, 128, false, false);          // S = Q K^T: both operands K-major
      constexpr uint32_t idesc_pv = instr_desc_f16(kRows, kHeadDim, false, true);    // O += P V: V is MN-major
      bool alive = true;
      // P of keys [64 h, 64 h + 64) sits in columns [64 h, 64 h + 32) of the block's scores: contraction step ks (16 keys) reads
      // columns 64 (ks / 4) + 8 (ks % 4).
      auto issue_qk = [&](int blk, int j) {
        const uint32_t q = base + kOffQ + blk * kTileBytes, k = base + kOffK + (j & 1) * kTileBytes, s = tmem + kColS + 128 * blk;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kColBlockBytes + (ks & 3) * 32u;
          mma_ss(s, smem_desc_sw128(q + off, 16, 1024), smem_desc_sw128(k + off, 16, 1024), idesc, ks > 0 ? 1u : 0u);
        }
        mma_commit(bar(kBarSFull + blk));
        if (blk == kBlocks - 1) mma_commit(bar(kBarKEmpty + (j & 1)));
      };
      auto issue_pv = [&](int blk, int j) {
        const uint32_t v = base + kOffV + (j & 1) * kTileBytes, s = tmem + kColS + 128 * blk, o = tmem + kColO + 128 * blk;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t bd = smem_desc_sw128(v + ks * 2048u, kColBlockBytes, 1024);
          const uint32_t a = s + 64 * (ks >> 2) + 8 * (ks & 3);
          if (ks == 0 && j == 0) mma_ts<false>(o, a, bd, idesc_pv);
          else mma_ts<true>(o, a, bd, idesc_pv);
        }
        mma_commit(bar(kBarPvDone + blk));
        if (blk == kBlocks - 1) mma_commit(bar(kBarVEmpty + (j & 1)));
      };
      alive = mbar_wait(bar(kBarKFull), 0, abort_flag);
      if (alive) {
        tc_fence_after_sync();
        issue_qk(0, 0);
        issue_qk(1, 0);
      }
#pragma unroll 1
      for (int j = 0; j < n_tiles && alive; ++j) {
        alive = mbar_wait(bar(kBarVFull + (j & 1)), (j >> 1) & 1, abort_flag);
#pragma unroll 1
        for (int blk = 0; blk < kBlocks && alive; ++blk) {
          alive = mbar_wait(bar(kBarPFull + blk), j & 1, abort_flag);
          if (!alive) break;
          tc_fence_after_sync();
          issue_pv(blk, j);
          if (j + 1 < n_tiles) {   // the scores of the next tile overwrite P: issued behind P V, executed behind it
            if (blk == 0) alive = mbar_wait(bar(kBarKFull + ((j + 1) & 1)), ((j + 1) >> 1) & 1, abort_flag);
            if (!alive) break;
            tc_fence_after_sync();
            issue_qk(blk, j + 1);
          }
        }
      }
      for (int blk = 0; blk < kBlocks && alive; ++blk)        // nothing in flight when TMEM is released
        alive = mbar_wait(bar(kBarPvDone + blk), (n_tiles - 1) & 1, abort_flag);
    }
    __syncwarp();
    tc_fence_before_sync();
  }

  // ---- end: a CTA in which a wait gave up raises the device-wide flag; tensor memory is released either way ---------------
  __syncthreads();
  if (abort_flag->abort != 0 && tid == 0) {
    atomicOr(&g_prefill_fault, 1);
    atomicOr(&g_prefill_status, 4);
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int G, int KB, int VB>
static int launch_prefill_umma(const PrefillUmmaParams& p, int max_query_len, int B, cudaStream_t st) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(prefill_umma_kernel<G, KB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, pfu::kSmemBytes) != cudaSuccess)
      return check_launch("prefill: shared memory opt-in");
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int per_tile = pfu::kBlocks * pfu::kRows / G;
  const int q_tiles = (max_query_len + per_tile - 1) / per_tile;
  if (q_tiles > 65535 || p.H_kv > 65535) return fail(CDA_ERR_N_TOO_LARGE, "prefill: max_query_len %d or H_kv %d exceeds the grid limits", max_query_len, p.H_kv);
  const dim3 grid(B, p.H_kv, q_tiles);
  PrefillUmmaParams pp = p;
  pp.wait_limit_ns = g_wait_limit_ns;
  pp.withhold_first_k = g_withhold_first_k;
  prefill_umma_kernel<G, KB, VB><<<grid, pfu::kThreads, pfu::kSmemBytes, st>>>(pp);
  return check_launch("prefill kernel");
}

template <int KB, int VB>
static int dispatch_prefill_umma_group(const PrefillUmmaParams& p, int max_query_len, int B, cudaStream_t st) {
  return p.group <= 4 ? launch_prefill_umma<4, KB, VB>(p, max_query_len, B, st) : launch_prefill_umma<8, KB, VB>(p, max_query_len, B, st);
}

int dispatch_prefill_umma(const PrefillUmmaParams& p, int k_bits, int v_bits, int max_query_len, int B, cudaStream_t st) {
  if (k_bits == 16 && v_bits == 16) return dispatch_prefill_umma_group<16, 16>(p, max_query_len, B, st);
  if (k_bits == 4 && v_bits == 4) return dispatch_prefill_umma_group<4, 4>(p, max_query_len, B, st);
  if (k_bits == 4 && v_bits == 2) return dispatch_prefill_umma_group<4, 2>(p, max_query_len, B, st);
  if (k_bits == 2 && v_bits == 2) return dispatch_prefill_umma_group<2, 2>(p, max_query_len, B, st);
  return dispatch_prefill_umma_group<2, 4>(p, max_query_len, B, st);
}

}  // namespace cda

// 1 if a prefill CTA on the current device gave up on a wait since the last clear (synchronises the device), 0 if not,
// < 0 on error.
extern "C" int cda_b200_prefill_fault(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, cda::g_prefill_fault, sizeof(int)) != cudaSuccess) return cda::check_launch("prefill_fault");
  return v != 0 ? 1 : 0;
}

// Status bits the prefill kernel raised on the current device since the last clear (synchronises the device).
extern "C" int cda_b200_prefill_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, cda::g_prefill_status, sizeof(int)) != cudaSuccess) return cda::check_launch("prefill_status");
  return v & 0x7fffffff;
}

// Clears the status bits and the fault flag of the current device (synchronises the device).
extern "C" int cda_b200_prefill_clear_status(void) {
  const int zero = 0;
  if (cudaMemcpyToSymbol(cda::g_prefill_status, &zero, sizeof(int)) != cudaSuccess ||
      cudaMemcpyToSymbol(cda::g_prefill_fault, &zero, sizeof(int)) != cudaSuccess)
    return cda::check_launch("prefill_clear_status");
  return CDA_OK;
}

// Diagnostic knobs for the launches that follow on this process: wait_limit_us <= 0 restores the default limit.
extern "C" int cda_b200_prefill_debug(int wait_limit_us, int withhold_first_k_arrive) {
  cda::g_wait_limit_ns = wait_limit_us > 0 ? static_cast<unsigned long long>(wait_limit_us) * 1000ull : cda::umma::kWaitLimitNs;
  cda::g_withhold_first_k = withhold_first_k_arrive ? 1 : 0;
  return CDA_OK;
}
