// Single-query GQA decode over the paged codebook cache.
//
// Split kernel (decode_split_kernel).  Grid = (key-range splits, sequences, KV-head groups); a CTA has W warps
// and owns up to 8 KV heads of one key range of one sequence.  A warp owns ONE KV head (and the whole GQA group
// of query heads that reads it) and walks its share of the range 16 tokens at a time:
//
//   HBM -> shared     ONE tensor-map bulk copy (TMA, cp.async.bulk.tensor.2d) per group brings the 16 slots -- a box of
//                     16 rows x 160 bytes of the cache seen as (slot, bytes of all heads) -- into a per-warp ring of
//                     NS stages (NS-1 groups in flight per warp, one mbarrier per stage, no CTA barrier in the main
//                     loop).  The copy engine writes shared memory by itself: the load/store pipe, which the table
//                     gathers below keep busy, never sees the cache bytes on their way in.  (Issued by the load/store
//                     pipe as 16-byte cp.async copies, the same bytes cost that pipe about 45 cycles per group on top
//                     of the ~85 cycles of gathers and fragment reads -- a third of the kernel's time.)  Each slot
//                     lands in a 160-byte cell, which keeps the fragment reads free of bank conflicts.
//   codes -> fp16     one shared-memory gather per code: a byte (two 4-bit indices) or nibble (two 2-bit
//                     indices) selects an fp16 pair from a lane-replicated table, which is exactly one 32-bit
//                     operand register of mma.m16n8k16.  The table sits on a 64 KB boundary of the shared
//                     window with 256-byte rows (K entries in the low half, V entries in the high half), so the
//                     whole gather address is assembled by ONE byte-permute: [window hi | code | lane*4].
//   QK^T              tokens on the M axis, query heads on N: S[16 tok x 8 col] over 8 k-steps (two independent
//                     accumulator chains).  For a group of <= 4 query heads columns 4..7 repeat columns 0..3.
//   softmax           online, base-2 exponent; norms are applied to scores (K) and to probabilities (V), never
//                     to the 128-wide vectors.  The running maximum is only re-reduced across lanes when some
//                     lane saw a larger score (warp vote), which after the first groups is rare.
//   P V               computed transposed: A = decoded V codes (rows = byte position in the slot, k = (token,
//                     parity of the coordinate)), B = probabilities placed in the even or odd half of the
//                     register.  That keeps "one code -> one A register" without any data shuffling;
//                     movmatrix transposes the probability tile between the two products.
//
// Every warp writes an un-normalised partial (O[g][128], m, l) to the workspace; decode_merge_kernel
// combines them by log-sum-exp, rounds to fp16, applies the inverse Hadamard transform and stores fp16.
//
// HBM traffic per (token, KV head): one slot (144 B for k4v4; 136 B of it payload).
#include <cmath>
#include <cstdlib>

#include <cuda.h>   // CUtensorMap and the enums of cuTensorMapEncodeTiled (types only: the entry point is looked up at run time)

#include <cstring>
#include "common.cuh"

namespace cda {

constexpr int kLutWindow = 65536;   // a table window is one 64 KB-aligned block of the shared window
// Tables.  4-bit codes: entry = code byte -> fp16 pair, 4 bytes per lane, 128 bytes per row; when both sides are 4-bit the K
// and V tables share one window (K in the low, V in the high half of the 256-byte rows).  2-bit codes: entry = code byte
// (four codes) -> four fp16, 8 bytes per lane, 256 bytes per row: one 64-bit gather yields two operand registers.  A 2-bit
// side therefore fills a window of its own, and any kernel with a 2-bit side uses two windows.
template <int KB, int VB>
struct LutCfg {
  static constexpr int kWindows = (KB == 4 && VB == 4) ? 1 : 2;
  static constexpr int kBytes = kWindows * kLutWindow;
};
constexpr float kMinusBig = -1.0e30f;   // "no score yet": finite, so differences never produce NaN

struct DecodeParams {
  const __half* q;
  const uint8_t* cache;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const float* cb_k;
  const float* cb_v;
  float* part_ml;      // (P, B, H_q, 2): m (log2 domain, scale folded in), l
  float* part_o;       // (P, B, H_q, 128)
  int* status;         // device status word (bit 0: a block id was out of range, bit 1: shared window too small,
                       // bit 2: a wait for a cache copy ran out of time)
  int B, H_q, H_kv, group;
  int heads_per_cta;   // power of two <= 8 dividing H_kv
  int block_size, bt_stride, num_blocks;
  int gpb_shift;          // log2(block_size / 16), or -1 when block_size / 16 is not a power of two
  int chunk_groups;       // 16-token groups per chunk of the virtual line of groups (one CTA per chunk and head group)
  int groups_pad;         // positions of the line owned by each sequence (>= groups of the longest sequence)
  int smem_bytes;         // dynamic shared memory given to the kernel
  float scale_log2;       // softmax scale * log2(e)
};

template <int KB, int VB>
struct Geom {
  static constexpr int kKBytes = 16 * KB;                      // index bytes of one row
  static constexpr int kVBytes = 16 * VB;
  static constexpr int kSlotBytes = (KB + VB + 1) * 16;
  // A ring stage keeps every slot whole in a 160-byte cell, cells in token order (the copy box is 160 bytes wide: the
  // slot and the first bytes of the next head's slot, or zeros past the end of the row).
  // 160 = 32 (mod 128), and accumulator row r is fed by token perm(r) = 0,2,1,3,6,4,7,5: with that pairing the K
  // reads of two rows and the V reads of four rows always fall into different banks.
  static constexpr int kCell = 160;
  static constexpr int kStageBytes = 16 * kCell;
  static_assert(kSlotBytes <= kCell, "slot does not fit its cell");
};

__device__ __forceinline__ int stage_perm(int row) { return (0xBE6650u >> (3 * (row & 7))) & 7; }   // 0,2,1,3,6,4,7,5

// ---- shared-memory access by 32-bit window address ---------------------------------------------------------------
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {   // table reads: the table never changes after the barrier
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));   // volatile: keeps the gathers in program order, ahead of the mma block
  return v;
}
// Reads of staged cache bytes: ordered after the cp.async wait by the "memory" clobber.
template <int IMM>
__device__ __forceinline__ uint4 lds_stage16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(IMM) : "memory");
  return v;
}
template <int IMM>
__device__ __forceinline__ uint2 lds_stage8(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(IMM) : "memory");
  return v;
}
template <int IMM>
__device__ __forceinline__ uint32_t lds_stage4(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM) : "memory");
  return v;
}

// ---- tensor-map bulk copies and their mbarriers ------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Wait for the copy of a ring stage, for at most kCopyWaitNs (a copy takes microseconds).  False if the time ran out.
constexpr unsigned long long kCopyWaitNs = 100ull * 1000 * 1000;
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > kCopyWaitNs) return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}
// Box (x .. x+159 bytes of the row, rows y .. y+15) of the cache -> shared memory at dst; completion is counted in bytes
// on the mbarrier.  x must be a multiple of 16 (it is head * slot_bytes).  No multicast: the source is this GPU's memory
// and the destination this CTA's shared memory.
__device__ __forceinline__ void tma_load_group(uint32_t dst, const CUtensorMap* tmap, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
// Orders this thread's earlier ordinary shared-memory accesses before later writes of the copy engine to the same bytes.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Table entry for the code in byte POS of w: the address is [base.byte3 | base.byte2 | code | base.byte0].
template <int POS>
__device__ __forceinline__ uint32_t lut_byte(uint32_t w, uint32_t base) {
  return lds_u32(__byte_perm(w, base, 0x7604 | (POS << 4)));
}
// Table entry (four fp16 = two operand registers) for the four 2-bit codes in byte POS of w; same address trick, the
// lane's slot inside the 256-byte row is 8 bytes wide.
template <int POS>
__device__ __forceinline__ uint2 lut_byte4(uint32_t w, uint32_t base) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(__byte_perm(w, base, 0x7604 | (POS << 4))));
  return v;
}

// One 16-token group as the lane holds it: K index pieces of rows r and r+8, V index pieces of rows
// 2c, 2c+1, 8+2c, 9+2c, and the (K norm, V norm) pairs of rows r and r+8.
template <int KB, int VB>
struct GroupRegs {
  uint32_t k[2][KB];          // 4-bit: 16 bytes per row, 2-bit: 8 bytes
  uint32_t v[4][VB / 2];      // 4-bit: 8 bytes per row,  2-bit: 4 bytes
  float2 n[2];
};

// Gather phase / multiply phase are kept apart on purpose: all table reads of a product are issued back to back
// (32 for QK^T, 16 per half of P V) before the first mma that consumes them, so that the shared-memory pipe always
// has many independent gathers in flight.
template <int KB, int S>
struct QkGather {
  __device__ static __forceinline__ void run(uint32_t (&a)[8][4], const uint32_t (&k)[2][KB], uint32_t base) {
    if (KB == 4) {          // k-step S uses bytes 2S (coordinates 4S, 4S+1) and 2S+1 (4S+2, 4S+3) of the lane's 16
      a[S][0] = lut_byte<(2 * S) & 3>(k[0][(2 * S) >> 2], base);
      a[S][1] = lut_byte<(2 * S) & 3>(k[1][(2 * S) >> 2], base);
      a[S][2] = lut_byte<(2 * S + 1) & 3>(k[0][(2 * S + 1) >> 2], base);
      a[S][3] = lut_byte<(2 * S + 1) & 3>(k[1][(2 * S + 1) >> 2], base);
    } else {                // byte S of the lane's 8: coordinates 4S, 4S+1 (first register) and 4S+2, 4S+3 (second)
      const uint2 e0 = lut_byte4<S & 3>(k[0][S >> 2], base), e1 = lut_byte4<S & 3>(k[1][S >> 2], base);
      a[S][0] = e0.x; a[S][2] = e0.y;
      a[S][1] = e1.x; a[S][3] = e1.y;
    }
    QkGather<KB, S + 1>::run(a, k, base);
  }
};
template <int KB>
struct QkGather<KB, 8> {
  __device__ static __forceinline__ void run(uint32_t (&)[8][4], const uint32_t (&)[2][KB], uint32_t) {}
};

// m-tile U of the transposed PV product: rows = byte positions 8r+2U (accumulator rows r) and 8r+2U+1 (rows r+8)
// of the V index bytes, k = (token slot, parity).  va / vb are the lane's index pieces of the two token rows.
template <int VB, int U>
struct PvGather {
  __device__ static __forceinline__ void run(uint32_t (&a)[4][4], const uint32_t (&va)[VB / 2], const uint32_t (&vb)[VB / 2], uint32_t base) {
    if (VB == 4) {
      a[U][0] = lut_byte<(2 * U) & 3>(va[(2 * U) >> 2], base);
      a[U][1] = lut_byte<(2 * U + 1) & 3>(va[(2 * U + 1) >> 2], base);
      a[U][2] = lut_byte<(2 * U) & 3>(vb[(2 * U) >> 2], base);
      a[U][3] = lut_byte<(2 * U + 1) & 3>(vb[(2 * U + 1) >> 2], base);
    } else {
      const uint2 ea = lut_byte4<U>(va[0], base), eb = lut_byte4<U>(vb[0], base);
      a[U][0] = ea.x; a[U][1] = ea.y;
      a[U][2] = eb.x; a[U][3] = eb.y;
    }
    PvGather<VB, U + 1>::run(a, va, vb, base);
  }
};
template <int VB>
struct PvGather<VB, 4> {
  __device__ static __forceinline__ void run(uint32_t (&)[4][4], const uint32_t (&)[VB / 2], const uint32_t (&)[VB / 2], uint32_t) {}
};

template <int W, int NS, int KB, int VB>
struct DecCfg {
  static constexpr int kWarps = W;
  static constexpr int kThreads = W * 32;
  static constexpr int kRingBytes = NS * Geom<KB, VB>::kStageBytes;   // per warp, contiguous; also stages the query rows
  static_assert(kRingBytes >= 8 * kHeadDim * 2, "ring too small to stage the query rows");
};

// Everything one warp carries through the key loop.
template <int G, int KB, int VB, int NS>
struct WarpCtx {
  using Gm = Geom<KB, VB>;
  static constexpr int NT = G / 4;
  uint32_t qf[16];
  float oacc[4][NT][4];
  float m_run[2], l_run[2];
  uint32_t base_k, base_v, sel_b0, sel_b1;
  uint32_t ring;                          // window address of stage 0 of this warp's ring
  uint32_t bar;                           // window address of the mbarrier of stage 0 (stage S: + 8 S)
  uint32_t phases;                        // bit S: parity of the next completion of stage S's mbarrier
  const CUtensorMap* tmap;
  int x_bytes;                            // first byte of this warp's head inside a cache row
  bool leader, dead;                      // lane 0 issues the copies; dead: a wait ran out of time, stop waiting
  uint32_t k_addr, v_addr, v_addr_b, n_addr;   // window addresses of this lane's fragment pieces in stage 0 (V: rows 2c, 2c+1)
  const int32_t* bt_row;
  int block_size, num_blocks, gpb, gpb_shift;
  int g_begin_sub, R, ng, t_end, r;
  int tok_r;                              // position inside the group of the token that feeds accumulator row r
  int blk_q;                              // block id of the next group to be issued
  bool bad_block;                         // a block id was out of range (block 0 was read instead)
  float scale_log2;

  __device__ __forceinline__ int block_index(int gidx) const { return gpb_shift >= 0 ? gidx >> gpb_shift : gidx / gpb; }
  __device__ __forceinline__ int block_rem(int gidx) const { return gpb_shift >= 0 ? gidx & (gpb - 1) : gidx % gpb; }
  __device__ __forceinline__ void load_block_id(int j) {
    const int jj = j < ng ? j : ng - 1;
    blk_q = __ldg(bt_row + block_index(g_begin_sub + R * jj));
  }

  // Start the copy of group j into stage S (nothing if j is past the end).  Every lane is past its reads of the stage
  // (the callers put a __syncwarp() between the last read and this call).
  template <int S>
  __device__ __forceinline__ void issue(int j) {
    if (j < ng) {
      uint32_t blk = static_cast<uint32_t>(blk_q);
      const bool bad = blk >= static_cast<uint32_t>(num_blocks);   // reported once, when the warp is done
      bad_block |= bad;
      blk = bad ? 0u : blk;
      int y = static_cast<int>(blk) * block_size;                  // first slot of the group
      if (gpb > 1) y += block_rem(g_begin_sub + R * j) << 4;
      if (leader) {
        mbar_expect_tx(bar + 8 * S, Gm::kStageBytes);
        tma_load_group(ring + S * Gm::kStageBytes, tmap, x_bytes, y, bar + 8 * S);
      }
      load_block_id(j + 1);
    }
  }
  // Wait until the copy into stage S has landed.
  template <int S>
  __device__ __forceinline__ void wait_stage() {
    if (!dead && !mbar_wait(bar + 8 * S, (phases >> S) & 1u)) dead = true;
    phases ^= 1u << S;
  }

  template <int S, bool MASKED>
  __device__ __forceinline__ void consume(int j) {
    constexpr int O = S * Gm::kStageBytes, H = 8 * Gm::kCell;   // rows rho + 8 sit 8 cells further
    GroupRegs<KB, VB> gr;
    if (KB == 4) {
      const uint4 t0 = lds_stage16<O>(k_addr), t1 = lds_stage16<O + H>(k_addr);
      gr.k[0][0] = t0.x; gr.k[0][1] = t0.y; gr.k[0][KB - 2] = t0.z; gr.k[0][KB - 1] = t0.w;
      gr.k[1][0] = t1.x; gr.k[1][1] = t1.y; gr.k[1][KB - 2] = t1.z; gr.k[1][KB - 1] = t1.w;
    } else {
      const uint2 t0 = lds_stage8<O>(k_addr), t1 = lds_stage8<O + H>(k_addr);
      gr.k[0][0] = t0.x; gr.k[0][1] = t0.y; gr.k[1][0] = t1.x; gr.k[1][1] = t1.y;
    }
    const uint2 n0 = lds_stage8<O>(n_addr), n1 = lds_stage8<O + H>(n_addr);
    gr.n[0] = make_float2(__uint_as_float(n0.x), __uint_as_float(n0.y));
    gr.n[1] = make_float2(__uint_as_float(n1.x), __uint_as_float(n1.y));
    if (VB == 4) {
      const uint2 a = lds_stage8<O>(v_addr), b = lds_stage8<O>(v_addr_b);
      const uint2 c2 = lds_stage8<O + H>(v_addr), d = lds_stage8<O + H>(v_addr_b);
      gr.v[0][0] = a.x; gr.v[0][VB / 2 - 1] = a.y; gr.v[1][0] = b.x; gr.v[1][VB / 2 - 1] = b.y;
      gr.v[2][0] = c2.x; gr.v[2][VB / 2 - 1] = c2.y; gr.v[3][0] = d.x; gr.v[3][VB / 2 - 1] = d.y;
    } else {
      gr.v[0][0] = lds_stage4<O>(v_addr); gr.v[1][0] = lds_stage4<O>(v_addr_b);
      gr.v[2][0] = lds_stage4<O + H>(v_addr); gr.v[3][0] = lds_stage4<O + H>(v_addr_b);
    }

    attend<MASKED>(gr, j);
  }

  // Scores, online softmax and P V for one 16-token group held in registers.
  template <bool MASKED>
  __device__ __forceinline__ void attend(const GroupRegs<KB, VB>& gr, int j) {
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      uint32_t ka[8][4];
      QkGather<KB, 0>::run(ka, gr.k, base_k);
#pragma unroll
      for (int s = 0; s < 8; ++s)   // even / odd k-steps: two independent accumulator chains
        mma_16816(sc[s & 1], ka[s][0], ka[s][1], ka[s][2], ka[s][3], qf[2 * s], qf[2 * s + 1]);
    }
    const float f0 = gr.n[0].x * scale_log2, f1 = gr.n[1].x * scale_log2;
    float s0 = (sc[0][0] + sc[1][0]) * f0, s1 = (sc[0][1] + sc[1][1]) * f0;
    float s2 = (sc[0][2] + sc[1][2]) * f1, s3 = (sc[0][3] + sc[1][3]) * f1;
    float nv0 = gr.n[0].y, nv1 = gr.n[1].y;
    if (MASKED) {   // ragged tail: rows past the end contribute nothing, whatever bytes they hold
      const int tok0 = (g_begin_sub + R * j) << 4;
      const bool ok0 = tok0 + tok_r < t_end, ok1 = tok0 + tok_r + 8 < t_end;
      s0 = ok0 ? s0 : -INFINITY; s1 = ok0 ? s1 : -INFINITY; s2 = ok1 ? s2 : -INFINITY; s3 = ok1 ? s3 : -INFINITY;
      nv0 = ok0 ? nv0 : 0.f; nv1 = ok1 ? nv1 : 0.f;
    }
    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
    if (__any_sync(0xffffffffu, mx0 > m_run[0] || mx1 > m_run[1])) {   // a new maximum somewhere: reduce and rescale
#pragma unroll
      for (int mask = 4; mask < 32; mask <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, mask));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, mask));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const float fs0 = fast_exp2(m_run[0] - mn0), fs1 = fast_exp2(m_run[1] - mn1);
      m_run[0] = mn0; m_run[1] = mn1;
      l_run[0] *= fs0; l_run[1] *= fs1;
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          oacc[u][t][0] *= fs0; oacc[u][t][1] *= fs1; oacc[u][t][2] *= fs0; oacc[u][t][3] *= fs1;
        }
    }
    const float p0 = fast_exp2(s0 - m_run[0]), p1 = fast_exp2(s1 - m_run[1]);
    const float p2 = fast_exp2(s2 - m_run[0]), p3 = fast_exp2(s3 - m_run[1]);
    l_run[0] += p0 + p2;
    l_run[1] += p1 + p3;
    const uint32_t x0 = pack_half2(p0 * nv0, p1 * nv0);   // row r,   columns 2c, 2c+1
    const uint32_t x1 = pack_half2(p2 * nv1, p3 * nv1);   // row r+8
    const uint32_t y[2] = {movmatrix_trans(x0), movmatrix_trans(x1)};   // (P[2c][r], P[2c+1][r]) of rows 0-7 / 8-15
    uint32_t pa[2][4][4];
    PvGather<VB, 0>::run(pa[0], gr.v[0], gr.v[1], base_v);
    PvGather<VB, 0>::run(pa[1], gr.v[2], gr.v[3], base_v);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t bfrag[NT][2];
      if (G == 4) {            // column r = (parity r >> 2, query r & 3)
        bfrag[0][0] = __byte_perm(y[hh], 0, sel_b0);
        bfrag[0][1] = __byte_perm(y[hh], 0, sel_b1);
      } else {                 // tile 0: even coordinate of every pair, tile 1: odd
        bfrag[0][0] = y[hh] & 0xffffu;
        bfrag[0][1] = y[hh] >> 16;
        bfrag[NT - 1][0] = y[hh] << 16;
        bfrag[NT - 1][1] = y[hh] & 0xffff0000u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int t = 0; t < NT; ++t) mma_16816(oacc[u][t], pa[hh][u][0], pa[hh][u][1], pa[hh][u][2], pa[hh][u][3], bfrag[t][0], bfrag[t][1]);
    }
  }
};

// One turn of the ring: NS groups, stage S for group j0 + S.  STEADY turns are known to lie wholly inside the warp's
// range and to hold no ragged group, so they carry no range or mask tests.
template <int G, int KB, int VB, int NS, int S, bool STEADY>
struct RingSteps {
  __device__ static __forceinline__ void run(WarpCtx<G, KB, VB, NS>& cx, int j0, bool tail_masked) {
    const int j = j0 + S;
    if (STEADY || j < cx.ng) {
      cx.template issue<(S + NS - 1) % NS>(j + NS - 1);
      cx.template wait_stage<S>();
      if (!STEADY && tail_masked && j == cx.ng - 1) cx.template consume<S, true>(j);
      else cx.template consume<S, false>(j);
      __syncwarp();
    }
    RingSteps<G, KB, VB, NS, S + 1, STEADY>::run(cx, j0, tail_masked);
  }
};
template <int G, int KB, int VB, int NS, bool STEADY>
struct RingSteps<G, KB, VB, NS, NS, STEADY> {
  __device__ static __forceinline__ void run(WarpCtx<G, KB, VB, NS>&, int, bool) {}
};

template <int G, int KB, int VB, int NS, int S>
struct RingPrologue {
  __device__ static __forceinline__ void run(WarpCtx<G, KB, VB, NS>& cx) {
    cx.template issue<S>(S);
    RingPrologue<G, KB, VB, NS, S + 1>::run(cx);
  }
};
template <int G, int KB, int VB, int NS>
struct RingPrologue<G, KB, VB, NS, NS - 1> {
  __device__ static __forceinline__ void run(WarpCtx<G, KB, VB, NS>&) {}
};

// One piece of a CTA's chunk: groups [g_lo, g_hi) (16 tokens each) of sequence b, stored as partial `piece` of b.
struct ChunkItem {
  int b, g_lo, g_hi, piece;
};

// G: padded GQA group (4 or 8).  W: warps per CTA.  NS: ring stages per warp.
//
// Work decomposition.  Every sequence owns `groups_pad` consecutive positions of a virtual line of 16-token groups
// (sequence b: positions [b * groups_pad, (b + 1) * groups_pad)), and the line is cut into chunks of `chunk_groups`
// positions.  CTA (chunk, head group) walks the sequences its chunk touches, one item per sequence: with a chunk size of
// (all positions / SM count) every SM gets the same number of tokens whatever B and N are, and a chunk that straddles
// the end of one sequence simply continues with the next.  The partial of item (chunk, b) is row
// piece = chunk - first chunk of b; pieces a sequence does not reach hold m = -inf.
template <int G, int KB, int VB, int W, int NS>
__global__ void __launch_bounds__(W * 32, 1) decode_split_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap cache_map) {
  using Gm = Geom<KB, VB>;
  using Cfg = DecCfg<W, NS, KB, VB>;
  constexpr int NT = G / 4;
  extern __shared__ __align__(128) uint8_t smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int hpc = p.heads_per_cta;
  const int R = W / hpc;                 // warps sharing one head (each takes every R-th group)
  const int chunk = blockIdx.x, hg = blockIdx.y;
  const int head = hg * hpc + (warp & (hpc - 1));
  const int sub = warp / hpc;
  const int g = p.group;

  // ---- shared window layout: warp rings fill the space before the 64 KB-aligned table, the rest follow it -----------
  const uint32_t win0 = smem_addr(smem);
  const uint32_t lut_win = (win0 + kLutWindow - 1) & ~static_cast<uint32_t>(kLutWindow - 1);
  const int rings_before = static_cast<int>((lut_win - win0) / Cfg::kRingBytes);
  const int rings_after = W > rings_before ? W - rings_before : 0;
  constexpr uint32_t kLutBytes = LutCfg<KB, VB>::kBytes;
  const uint32_t win_end = lut_win + kLutBytes + rings_after * Cfg::kRingBytes;
  // (the copy engine wants 128-byte aligned destinations: every ring offset is a multiple of 128, so the window must be too)
  const bool fits = win_end - win0 <= static_cast<uint32_t>(p.smem_bytes) && (win0 & 127u) == 0u;
  const uint32_t ring = warp < rings_before ? win0 + warp * Cfg::kRingBytes
                                            : lut_win + kLutBytes + (warp - rings_before) * Cfg::kRingBytes;
  uint8_t* lut = smem + (lut_win - win0);

  // ---- the chunk's items -------------------------------------------------------------------------------------------------
  // The item of sequence b in this chunk, or false if the chunk ends before b.  Identical in every thread (depends on
  // the launch parameters only); everything is recomputed from b so that only b stays live across the key loop.
  auto item_of = [&](int b, ChunkItem& it) -> bool {
    const int64_t pos_lo = static_cast<int64_t>(blockIdx.x) * p.chunk_groups, pos_hi = pos_lo + p.chunk_groups;
    const int64_t base = static_cast<int64_t>(b) * p.groups_pad;
    if (b >= p.B || base >= pos_hi) return false;
    it.b = b;
    it.g_lo = static_cast<int>(pos_lo > base ? pos_lo - base : 0);
    const int64_t hi = pos_hi - base;
    it.g_hi = hi < p.groups_pad ? static_cast<int>(hi) : p.groups_pad;
    it.piece = static_cast<int>(blockIdx.x) - static_cast<int>(base / p.chunk_groups);
    return true;
  };
  // An item without tokens (short sequence) or a CTA without room: empty partial rows for every head of the CTA.
  auto write_empty = [&](const ChunkItem& it) {
    const int rows = hpc * g;
    const int64_t prow_cta = (static_cast<int64_t>(it.piece) * p.B + it.b) * p.H_q + hg * hpc * g;
    for (int i = tid; i < rows; i += W * 32) *reinterpret_cast<float2*>(p.part_ml + (prow_cta + i) * 2) = make_float2(-INFINITY, 0.f);
  };

  __shared__ __align__(8) unsigned long long s_bar[W * NS];   // one mbarrier per warp and ring stage
  WarpCtx<G, KB, VB, NS> cx;
  cx.ring = ring;
  cx.bar = smem_addr(s_bar) + warp * (8 * NS);
  cx.phases = 0u;
  cx.tmap = &cache_map;
  cx.x_bytes = head * Gm::kSlotBytes;
  cx.leader = lane == 0;
  cx.dead = false;
  if (cx.leader) {                       // only this warp ever touches its barriers: lane 0 arrives, all lanes wait
#pragma unroll
    for (int st = 0; st < NS; ++st) mbar_init(cx.bar + 8 * st, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncwarp();
  cx.k_addr = ring + stage_perm(r) * Gm::kCell + c * (4 * KB);
  cx.v_addr = ring + stage_perm(2 * c) * Gm::kCell + 16 * KB + r * (2 * VB);
  cx.v_addr_b = ring + stage_perm(2 * c + 1) * Gm::kCell + 16 * KB + r * (2 * VB);
  cx.n_addr = ring + stage_perm(r) * Gm::kCell + 16 * KB + 16 * VB;
  cx.block_size = p.block_size; cx.num_blocks = p.num_blocks;
  cx.gpb = p.block_size >> 4; cx.gpb_shift = p.gpb_shift;
  cx.R = R; cx.r = r; cx.tok_r = stage_perm(r);
  cx.bad_block = false;

  // Point the warp at an item and start its first copies (stages 0 .. NS-2; stage NS-1 stays free until the first turn
  // of the ring).  Returns the number of 16-token groups of the whole CTA in the item (0: nothing to read).
  int t_begin = 0, t_end = 0;
  auto begin_item = [&](const ChunkItem& it) -> int {
    const int seq_len = p.seq_lens[it.b];
    t_begin = it.g_lo << 4;
    t_end = min(seq_len, it.g_hi << 4);                           // tokens at or beyond this are masked
    const int cta_groups = t_end > t_begin ? (t_end - t_begin + 15) >> 4 : 0;
    cx.ng = cta_groups > sub ? (cta_groups - sub + R - 1) / R : 0;   // groups of this warp
    cx.bt_row = p.block_table + static_cast<int64_t>(it.b) * p.bt_stride;
    cx.g_begin_sub = it.g_lo + sub; cx.t_end = t_end;
    if (cx.ng > 0) {
      cx.load_block_id(0);
      RingPrologue<G, KB, VB, NS, 0>::run(cx);
    }
    return cta_groups;
  };

  int b_cur = static_cast<int>(static_cast<int64_t>(chunk) * p.chunk_groups / p.groups_pad);
  int cta_groups = 0;
  {
    ChunkItem item;
    bool have = item_of(b_cur, item);
    if (!fits) {                      // no room for the table and the rings: report it, leave well-formed empty partials
      if (tid == 0) atomicOr(p.status, 2);
      for (; have; have = item_of(++b_cur, item)) write_empty(item);
      return;
    }
    for (; have; have = item_of(++b_cur, item)) {   // leading items without tokens need no set-up at all
      cta_groups = begin_item(item);
      if (cta_groups > 0) break;
      write_empty(item);
    }
    if (!have) return;
  }

  __shared__ float s_err[64];
  __shared__ int s_idx[64];
  float alpha_k, alpha_v;
  find_table_scales<(KB == 4 ? 16 : 4), (VB == 4 ? 16 : 4)>(p.cb_k, p.cb_v, s_err, s_idx, alpha_k, alpha_v);
  {   // build the tables (levels divided by alpha); lane i keeps level i & (L - 1) of either codebook and the entries are
      // put together by shuffles.  Row e (one code byte) of a window is 256 bytes.
    constexpr int LK = KB == 4 ? 16 : 4, LV = VB == 4 ? 16 : 4;
    const float lev_k = __ldg(p.cb_k + (lane & (LK - 1))) * (1.0f / alpha_k);
    const float lev_v = __ldg(p.cb_v + (lane & (LV - 1))) * (1.0f / alpha_v);
    uint32_t* lw_k = reinterpret_cast<uint32_t*>(lut);
    uint32_t* lw_v = reinterpret_cast<uint32_t*>(lut + (LutCfg<KB, VB>::kWindows == 1 ? 128 : kLutWindow));
#pragma unroll 4
    for (int e = warp; e < 256; e += W) {
      if (KB == 4) {
        lw_k[e * 64 + lane] = pack_half2(__shfl_sync(0xffffffffu, lev_k, (e >> 4) & 15), __shfl_sync(0xffffffffu, lev_k, e & 15));
      } else {
        const uint32_t lo = pack_half2(__shfl_sync(0xffffffffu, lev_k, (e >> 6) & 3), __shfl_sync(0xffffffffu, lev_k, (e >> 4) & 3));
        const uint32_t hi = pack_half2(__shfl_sync(0xffffffffu, lev_k, (e >> 2) & 3), __shfl_sync(0xffffffffu, lev_k, e & 3));
        *reinterpret_cast<uint2*>(lw_k + e * 64 + 2 * lane) = make_uint2(lo, hi);
      }
      if (VB == 4) {
        lw_v[e * 64 + lane] = pack_half2(__shfl_sync(0xffffffffu, lev_v, (e >> 4) & 15), __shfl_sync(0xffffffffu, lev_v, e & 15));
      } else {
        const uint32_t lo = pack_half2(__shfl_sync(0xffffffffu, lev_v, (e >> 6) & 3), __shfl_sync(0xffffffffu, lev_v, (e >> 4) & 3));
        const uint32_t hi = pack_half2(__shfl_sync(0xffffffffu, lev_v, (e >> 2) & 3), __shfl_sync(0xffffffffu, lev_v, e & 3));
        *reinterpret_cast<uint2*>(lw_v + e * 64 + 2 * lane) = make_uint2(lo, hi);
      }
    }
  }
  cx.base_k = lut_win | (lane << (KB == 4 ? 2 : 3));
  cx.base_v = LutCfg<KB, VB>::kWindows == 1 ? (cx.base_k | 128u) : ((lut_win + kLutWindow) | (lane << (VB == 4 ? 2 : 3)));
  {   // operand placement of the probabilities: even columns take the low half, odd columns the high half
    const bool odd = G == 4 && (r >> 2) != 0;
    cx.sel_b0 = odd ? 0x1044u : 0x4410u;
    cx.sel_b1 = odd ? 0x3244u : 0x4432u;
  }
  cx.scale_log2 = p.scale_log2 * alpha_k;

  constexpr int kRowFloats = kHeadDim + 4;   // parked partial rows: 528 bytes keep the 16-byte reads aligned
  static_assert(G * kRowFloats * 4 <= Cfg::kRingBytes, "a warp's partial must fit its ring");
  auto ring_of = [&](int w) -> float* {
    const uint32_t a = w < rings_before ? win0 + w * Cfg::kRingBytes : lut_win + kLutBytes + (w - rings_before) * Cfg::kRingBytes;
    return reinterpret_cast<float*>(smem + (a - win0));
  };

  for (;;) {   // one turn per item with tokens; the copies of its first groups are already in flight
    // ---- rotate this head's queries, stage them as fp16 rows in the last stage of this warp's ring, pick up the B fragments --
    {
      const int b = b_cur;
      __half* q_rows = reinterpret_cast<__half*>(smem + (ring - win0) + (NS - 1) * Gm::kStageBytes);
      static_assert(8 * kHeadDim * 2 <= Gm::kStageBytes, "eight fp16 query rows must fit one ring stage");
      float qv[G][4];
#pragma unroll
      for (int qi = 0; qi < G; ++qi) {
        qv[qi][0] = qv[qi][1] = qv[qi][2] = qv[qi][3] = 0.f;
        if (qi < g) load_half4(p.q + (static_cast<int64_t>(b) * p.H_q + head * g + qi) * kHeadDim + 4 * lane, qv[qi]);
      }
#pragma unroll
      for (int qi = 0; qi < G; ++qi) {
        fht128_warp(qv[qi], lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[qi][i] *= kRsqrtD;
        *reinterpret_cast<uint2*>(q_rows + qi * kHeadDim + 4 * lane) = pack_half4(qv[qi]);
      }
      __syncwarp();
      const int qrow = G == 4 ? (r & 3) : r;   // column r: query r, or r & 3 when the group is padded to 4
      const uint4* src = reinterpret_cast<const uint4*>(q_rows + qrow * kHeadDim + 32 * c);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 t = src[i];
        cx.qf[4 * i] = t.x; cx.qf[4 * i + 1] = t.y; cx.qf[4 * i + 2] = t.z; cx.qf[4 * i + 3] = t.w;
      }
      fence_proxy_async();   // the stage that held the query rows is written by the copy engine next
    }
    __syncthreads();   // first turn: tables visible to every warp; every turn: every lane is done with its query rows

    cx.m_run[0] = cx.m_run[1] = kMinusBig;
    cx.l_run[0] = cx.l_run[1] = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) cx.oacc[u][t][i] = 0.f;

    const int ng = cx.ng;
    if (ng > 0) {
      const bool tail_masked = ((t_end - t_begin) & 15) != 0 && (cta_groups - 1) % R == sub;
      int j0 = 0;
      const int steady_end = ng - (tail_masked ? 1 : 0);
#pragma unroll 1
      for (; j0 + NS <= steady_end; j0 += NS) RingSteps<G, KB, VB, NS, 0, true>::run(cx, j0, false);
#pragma unroll 1
      for (; j0 < ng; j0 += NS) RingSteps<G, KB, VB, NS, 0, false>::run(cx, j0, tail_masked);
    }
    __syncwarp();         // every lane is done reading the ring before it is reused below (no copy is in flight: every
                          // group that was requested has been waited for and consumed)

    // ---- combine the partials of the warps that share a head, write one partial per (piece, head) ------------------------------
    float l0 = cx.l_run[0], l1 = cx.l_run[1];
#pragma unroll
    for (int mask = 4; mask < 32; mask <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, mask);
      l1 += __shfl_xor_sync(0xffffffffu, l1, mask);
    }
    const float m0 = l0 > 0.f ? cx.m_run[0] : -INFINITY, m1 = l1 > 0.f ? cx.m_run[1] : -INFINITY;
    // every warp parks (O[q][128], m[q], l[q]) for its G query rows in its own ring: rows of 132 floats
    {
      float* st = ring_of(warp);
      if (G == 4) {
        const int parity = c >> 1, q0 = 2 * (c & 1);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int d = 16 * r + 4 * u + parity;
          st[q0 * kRowFloats + d] = cx.oacc[u][0][0] * alpha_v; st[q0 * kRowFloats + d + 2] = cx.oacc[u][0][2] * alpha_v;
          st[(q0 + 1) * kRowFloats + d] = cx.oacc[u][0][1] * alpha_v; st[(q0 + 1) * kRowFloats + d + 2] = cx.oacc[u][0][3] * alpha_v;
        }
        if (r == 0 && c < 2) {
          st[q0 * kRowFloats + kHeadDim] = m0; st[q0 * kRowFloats + kHeadDim + 1] = l0;
          st[(q0 + 1) * kRowFloats + kHeadDim] = m1; st[(q0 + 1) * kRowFloats + kHeadDim + 1] = l1;
        }
      } else {
        const int q0 = 2 * c;
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const int d = 16 * r + 4 * u + t;
            st[q0 * kRowFloats + d] = cx.oacc[u][t][0] * alpha_v; st[q0 * kRowFloats + d + 2] = cx.oacc[u][t][2] * alpha_v;
            st[(q0 + 1) * kRowFloats + d] = cx.oacc[u][t][1] * alpha_v; st[(q0 + 1) * kRowFloats + d + 2] = cx.oacc[u][t][3] * alpha_v;
          }
        if (r == 0) {
          st[q0 * kRowFloats + kHeadDim] = m0; st[q0 * kRowFloats + kHeadDim + 1] = l0;
          st[(q0 + 1) * kRowFloats + kHeadDim] = m1; st[(q0 + 1) * kRowFloats + kHeadDim + 1] = l1;
        }
      }
    }
    __syncthreads();
    // (head, query row) pairs are dealt over all warps; lane s < R holds the (m, l) of the head's s-th warp, lane l adds
    // up coordinates 4l .. 4l+3 of the row
    const int items = hpc * g;
    ChunkItem item;
    item_of(b_cur, item);
    const int64_t prow_cta = (static_cast<int64_t>(item.piece) * p.B + item.b) * p.H_q + hg * hpc * g;
    for (int it = warp; it < items; it += W) {
      const int hh = it & (hpc - 1), q = it / hpc;
      float ms = -INFINITY, ls = 0.f;
      if (lane < R) {
        const float2 ml = *reinterpret_cast<const float2*>(ring_of(hh + lane * hpc) + q * kRowFloats + kHeadDim);
        ms = ml.x; ls = ml.y;
      }
      float mt = ms;
#pragma unroll
      for (int mask = 1; mask < 32; mask <<= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, mask));
      const float wgt = ms == -INFINITY ? 0.f : fast_exp2(ms - mt);
      const float lt = warp_sum(ls * wgt);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int s2 = 0; s2 < R; ++s2) {
        const float w2 = __shfl_sync(0xffffffffu, wgt, s2);
        const float4 o = *reinterpret_cast<const float4*>(ring_of(hh + s2 * hpc) + q * kRowFloats + 4 * lane);
        acc.x += o.x * w2; acc.y += o.y * w2; acc.z += o.z * w2; acc.w += o.w * w2;
      }
      const int64_t prow = prow_cta + hh * g + q;
      *reinterpret_cast<float4*>(p.part_o + prow * kHeadDim + 4 * lane) = acc;
      if (lane == 0) *reinterpret_cast<float2*>(p.part_ml + prow * 2) = make_float2(mt, lt);
    }

    // ---- next item with tokens of this chunk, if any ---------------------------------------------------------------------
    bool have = item_of(++b_cur, item);
    for (; have; have = item_of(++b_cur, item)) {
      if (p.seq_lens[item.b] > (item.g_lo << 4)) break;
      write_empty(item);
    }
    if (!have) break;
    fence_proxy_async();
    __syncthreads();   // the parked partials have been read: the rings are free again
    cta_groups = begin_item(item);
  }
  if (cx.bad_block) atomicOr(p.status, 1);
  if (cx.dead && lane == 0) atomicOr(p.status, 4);
}

// ---- merge --------------------------------------------------------------------------------------------------
// Inputs: P partial rows per output row, partial pi of row `row` at index pi * rows + row; O rows o_stride floats apart
// (128 for the split kernel's workspace, 130 for packed partials whose columns 128 / 129 hold m / l), m and l read at
// (index * ml_stride).  m values are multiplied by `m_to_log2` on load (1 for the split kernel's own partials, log2(e)
// for natural-log partials supplied through the C ABI).
// mode 0: normalise, round to fp16, optional inverse Hadamard, store fp16 (and log-sum-exp if asked).
// mode 1: store the merged un-normalised partial as fp32: O at out_o + row * out_o_stride, m (natural log) and l at
//         out_m / out_l + row * out_ml_stride.
// When chunk_groups > 0 the partials come from decode_split_kernel and row r (sequence r / rows_per_seq) owns only the
// pieces its sequence's positions touch; pieces beyond that were never written and are not read.
// Exchange of merged partials between the ranks of a sequence-sharded decode (mode 2 of the merge): every rank owns a
// buffer of [2 parities][world senders][rows] exchange rows and knows the address of every other rank's buffer (peer
// memory).  A row is 132 floats: O[128], m (log2 domain), l, the tag of the call that wrote it, one pad float.
constexpr int kXchRowFloats = kHeadDim + 4;
struct ExchangeParams {
  float* const* peers;            // device array of `world` pointers: peers[p] = rank p's exchange buffer
  unsigned long long* counters;   // this rank's [0] calls completed, [1] rows finished in the running call
  int* status;                    // bit 3: a wait for another rank's row ran out of time
  int rank, world;
  unsigned long long wait_ns;
};
struct MergeParams {
  ExchangeParams x;
  const float* part_o; const float* part_m; const float* part_l;
  int ml_stride, o_stride, P;
  int64_t rows;
  float m_to_log2;
  int mode, unrotate;
  __half* out; float* out_lse;
  float* out_o; float* out_m; float* out_l;
  int out_o_stride, out_ml_stride;
  int rows_per_seq, chunk_groups, groups_pad;
};

__device__ __forceinline__ int merge_valid_parts(const MergeParams& q, int64_t row) {
  if (q.chunk_groups <= 0) return q.P;
  const int64_t lo = (row / q.rows_per_seq) * q.groups_pad;
  const int n = static_cast<int>((lo + q.groups_pad - 1) / q.chunk_groups - lo / q.chunk_groups + 1);
  return n < q.P ? n : q.P;
}
__device__ __forceinline__ float4 merge_load4(const float* ptr, bool vec4) {
  if (vec4) return *reinterpret_cast<const float4*>(ptr);
  const float2 a = *reinterpret_cast<const float2*>(ptr), b = *reinterpret_cast<const float2*>(ptr + 2);
  return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ void st_release_sys(uint32_t* ptr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* ptr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// Mode 2: this rank's merged row (ot, mt, lt) goes to every rank's buffer with plain peer stores, followed by the call's
// tag with release semantics; then the warp waits -- lane s for sender s, for at most wait_ns -- until every sender's
// row of this call has arrived in its own buffer, and merges them.  Nothing here waits on another warp of this GPU: a
// warp first sends, then waits, so the ranks cannot block one another.  A sender that does not show up in time is left
// out and reported (status bit 3).  Two parities suffice: a rank can start call k+2 only after every rank has finished
// reading call k (its call k+1 needs every rank's k+1 rows, which are sent after their call k kernel has ended).
__device__ __forceinline__ void exchange_rows(const MergeParams& q, float (&ot)[4], float& lt, float& mt, int64_t row, int lane) {
  const ExchangeParams& x = q.x;
  const unsigned long long call = *reinterpret_cast<volatile unsigned long long*>(x.counters) + 1;   // bumped after the last row
  const uint32_t tag = static_cast<uint32_t>(call);
  const int64_t slot0 = static_cast<int64_t>(call & 1) * x.world;
  const int64_t my_off = ((slot0 + x.rank) * q.rows + row) * kXchRowFloats;
  for (int p = 0; p < x.world; ++p) {
    float* dst = x.peers[p] + my_off;
    *reinterpret_cast<float4*>(dst + 4 * lane) = make_float4(ot[0], ot[1], ot[2], ot[3]);
    if (lane == 0) *reinterpret_cast<float2*>(dst + kHeadDim) = make_float2(mt, lt);
  }
  __threadfence_system();
  __syncwarp();
  if (lane < x.world) st_release_sys(reinterpret_cast<uint32_t*>(x.peers[lane] + my_off + kHeadDim + 2), tag);

  const float* mine = x.peers[x.rank];
  const float* src_row = mine + ((slot0 + (lane < x.world ? lane : 0)) * q.rows + row) * kXchRowFloats;
  bool got = lane >= x.world;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t spin = 1;; ++spin) {
    if (!got) got = ld_acquire_sys(reinterpret_cast<const uint32_t*>(src_row + kHeadDim + 2)) == tag;
    if (__all_sync(0xffffffffu, got)) break;
    if ((spin & 31u) == 0u) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (__any_sync(0xffffffffu, t - t0 > x.wait_ns)) {
        if (lane == 0) atomicOr(x.status, 8);
        break;
      }
    }
  }
  __syncwarp();
  float ms = -INFINITY, ls = 0.f;
  if (lane < x.world && got) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(src_row + kHeadDim));
    ms = ml.x; ls = ml.y;
  }
  float mall = ms;
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) mall = fmaxf(mall, __shfl_xor_sync(0xffffffffu, mall, mask));
  const float bw = ms == -INFINITY ? 0.f : fast_exp2(ms - mall);
  lt = warp_sum(ls * bw);
  mt = mall;
  ot[0] = ot[1] = ot[2] = ot[3] = 0.f;
  for (int sdr = 0; sdr < x.world; ++sdr) {
    const float w = __shfl_sync(0xffffffffu, bw, sdr);
    if (w == 0.f) continue;
    const float4 o = __ldcg(reinterpret_cast<const float4*>(mine + ((slot0 + sdr) * q.rows + row) * kXchRowFloats + 4 * lane));
    ot[0] += o.x * w; ot[1] += o.y * w; ot[2] += o.z * w; ot[3] += o.w * w;
  }
  if (lane == 0) {   // the last row of the call closes it
    const unsigned long long done = atomicAdd(x.counters + 1, 1ull);
    if (done == static_cast<unsigned long long>(q.rows) - 1) {
      x.counters[1] = 0ull;
      __threadfence();
      *reinterpret_cast<volatile unsigned long long*>(x.counters) = call;
    }
  }
}

// Last step of a merge: lane l holds coordinates 4l .. 4l+3 of the summed row, every lane the row's l and maximum.
__device__ __forceinline__ void merge_finish(const MergeParams& q, const float (&ot_in)[4], float lt, float mt, int64_t row, int lane) {
  float ot[4] = {ot_in[0], ot_in[1], ot_in[2], ot_in[3]};
  if (q.mode == 2) exchange_rows(q, ot, lt, mt, row, lane);
  if (q.mode == 1) {
    float* dst = q.out_o + row * q.out_o_stride + 4 * lane;
    if ((q.out_o_stride & 3) == 0) *reinterpret_cast<float4*>(dst) = make_float4(ot[0], ot[1], ot[2], ot[3]);
    else { *reinterpret_cast<float2*>(dst) = make_float2(ot[0], ot[1]); *reinterpret_cast<float2*>(dst + 2) = make_float2(ot[2], ot[3]); }
    if (lane == 0) {
      q.out_m[row * q.out_ml_stride] = mt == -INFINITY ? -INFINITY : mt * kLn2;
      q.out_l[row * q.out_ml_stride] = lt;
    }
    return;
  }
  const float inv = 1.0f / fmaxf(lt, 1e-30f);   // merge_partials clamps the denominator (attention.py:271)
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = round_to_half(ot[i] * inv);   // the oracle rounds O_rot to fp16 before un-rotating
  if (q.unrotate) {
    fht128_warp(v, lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= kRsqrtD;
  }
  *reinterpret_cast<uint2*>(q.out + row * kHeadDim + 4 * lane) = pack_half4(v);
  if (q.out_lse != nullptr && lane == 0) q.out_lse[row] = (mt == -INFINITY || !(lt > 0.f)) ? -INFINITY : mt * kLn2 + logf(lt);
}

// One CTA (16 warps) per output row.  A first pass over the (m) column finds the row's maximum; then warp w sums
// partials w, w+16, ... weighted by exp2(m_p - max), four at a time so that their loads are in flight together,
// and the sixteen warp sums are added through shared memory.
constexpr int kMergeWarps = 16, kMergeUnroll = 4;
__global__ void __launch_bounds__(kMergeWarps * 32) decode_merge_kernel(const MergeParams q) {
  __shared__ float s_o[kMergeWarps][kHeadDim];
  __shared__ float s_l[kMergeWarps], s_max[kMergeWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x, rows = q.rows;
  const int P = merge_valid_parts(q, row);
  const bool vec4 = (q.o_stride & 3) == 0;
  float mx = -INFINITY;
  for (int pi = threadIdx.x; pi < P; pi += kMergeWarps * 32)
    mx = fmaxf(mx, q.part_m[(static_cast<int64_t>(pi) * rows + row) * q.ml_stride]);
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, mask));
  if (lane == 0) s_max[warp] = mx;
  __syncthreads();
  float mt = -INFINITY;
#pragma unroll
  for (int w = 0; w < kMergeWarps; ++w) mt = fmaxf(mt, s_max[w]);
  mt *= q.m_to_log2;                                 // the factor is positive: the maximum stays the maximum
  const float ms = mt == -INFINITY ? 0.f : mt;

  float l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  for (int base = warp; base < P; base += kMergeWarps * kMergeUnroll) {
    float mp[kMergeUnroll], lp[kMergeUnroll];
    float4 op[kMergeUnroll];
#pragma unroll
    for (int u = 0; u < kMergeUnroll; ++u) {
      const int pi = base + u * kMergeWarps;
      const bool valid = pi < P;
      const int64_t pr = static_cast<int64_t>(valid ? pi : base) * rows + row;
      mp[u] = valid ? q.part_m[pr * q.ml_stride] : -INFINITY;
      lp[u] = q.part_l[pr * q.ml_stride];
      op[u] = merge_load4(q.part_o + pr * q.o_stride + 4 * lane, vec4);
    }
#pragma unroll
    for (int u = 0; u < kMergeUnroll; ++u) {
      if (mp[u] == -INFINITY) continue;              // empty range: its O row was never written, do not touch it
      const float bw = fast_exp2(mp[u] * q.m_to_log2 - ms);
      l += lp[u] * bw;
      o[0] += op[u].x * bw; o[1] += op[u].y * bw; o[2] += op[u].z * bw; o[3] += op[u].w * bw;
    }
  }
  *reinterpret_cast<float4*>(&s_o[warp][4 * lane]) = make_float4(o[0], o[1], o[2], o[3]);
  if (lane == 0) s_l[warp] = l;
  __syncthreads();
  if (warp != 0) return;
  float lt = 0.f, ot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < kMergeWarps; ++w) {
    lt += s_l[w];
    const float4 t = *reinterpret_cast<const float4*>(&s_o[w][4 * lane]);
    ot[0] += t.x; ot[1] += t.y; ot[2] += t.z; ot[3] += t.w;
  }
  merge_finish(q, ot, lt, mt, row, lane);
}

// Merge of at most 32 partials per row: one warp per row, no shared memory.  Lane p holds (m, l) of partial p; the O
// rows are read eight at a time.
constexpr int kMergeSmallRows = 4, kMergeSmallMaxP = 32;
__global__ void __launch_bounds__(kMergeSmallRows * 32) decode_merge_small_kernel(const MergeParams q) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = q.rows, row = static_cast<int64_t>(blockIdx.x) * kMergeSmallRows + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int P = merge_valid_parts(q, row);
  const bool vec4 = (q.o_stride & 3) == 0;
  float mp = -INFINITY, lp = 0.f;
  if (lane < P) {
    const int64_t pr = static_cast<int64_t>(lane) * rows + row;
    mp = q.part_m[pr * q.ml_stride] * q.m_to_log2;
    lp = q.part_l[pr * q.ml_stride];
  }
  float mt = mp;
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, mask));
  const float bw = mp == -INFINITY ? 0.f : fast_exp2(mp - mt);   // an empty range weighs nothing
  const float lt = warp_sum(lp * bw);
  float ot[4] = {0.f, 0.f, 0.f, 0.f};
  for (int base = 0; base < P; base += 8) {
    float4 op[8];
    float w8[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int pi = base + u < P ? base + u : base;
      w8[u] = base + u < P ? __shfl_sync(0xffffffffu, bw, pi) : 0.f;
      op[u] = merge_load4(q.part_o + (static_cast<int64_t>(pi) * rows + row) * q.o_stride + 4 * lane, vec4);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (w8[u] == 0.f) continue;                                 // an empty range's O row may never have been written
      ot[0] += op[u].x * w8[u]; ot[1] += op[u].y * w8[u]; ot[2] += op[u].z * w8[u]; ot[3] += op[u].w * w8[u];
    }
  }
  merge_finish(q, ot, lt, mt, row, lane);
}

// Picks the merge kernel by the number of partials per row.
static void launch_merge(const MergeParams& q, cudaStream_t st) {
  if (q.P <= kMergeSmallMaxP) {
    const unsigned grid = static_cast<unsigned>((q.rows + kMergeSmallRows - 1) / kMergeSmallRows);
    decode_merge_small_kernel<<<grid, kMergeSmallRows * 32, 0, st>>>(q);
  } else {
    decode_merge_kernel<<<static_cast<unsigned>(q.rows), kMergeWarps * 32, 0, st>>>(q);
  }
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
  int warps, depth, heads_per_cta, head_groups, warps_per_head;
  int chunk_groups, groups_pad, chunks;   // work decomposition (see decode_split_kernel)
  int parts;                              // partial rows per output row = most chunks any sequence touches
};

// Warps per CTA and ring stages per warp of the split kernel: 16 warps (four per scheduler, 128 registers each)
// with three 2560-byte stages per warp leave room for the 64 KB table in the 227 KB of one SM.
#ifndef CDA_SPLIT_WARPS
#define CDA_SPLIT_WARPS 16
#endif
#ifndef CDA_SPLIT_STAGES
#define CDA_SPLIT_STAGES 3
#endif
constexpr int kSplitWarps = CDA_SPLIT_WARPS, kSplitStages = CDA_SPLIT_STAGES;

static int pick_heads_per_cta(int H_kv) {   // largest power of two <= 8 that divides both H_kv and the warp count
  int h = 8;
  while (h > 1 && (h > H_kv || H_kv % h || kSplitWarps % h)) h >>= 1;
  return h;
}

// Chunks touched by positions [lo, lo + len) of the line when it is cut every c positions.
static int chunks_touched(int64_t lo, int64_t len, int64_t c) { return static_cast<int>((lo + len - 1) / c - lo / c + 1); }

// Choose the chunk size.  One CTA occupies one SM and every chunk carries the same number of groups, so the launch runs
// in ceil(CTAs / SMs) rounds, each as long as one CTA: a fixed part (launch, table and query set-up, first copies,
// partial write and its share of the merge; measured at about the streaming time of 360 tokens when the CTA's warps
// cover eight heads, and proportionally more tokens when they share fewer heads and so pass over a token faster) plus
// the chunk's tokens.  Candidates are the chunk sizes that give 1, 2, ... CTAs per SM; the smallest estimate wins and a
// chunk never goes below 128 tokens.  num_splits > 0 instead cuts every sequence into that many equal key ranges of its
// own (chunks then never straddle two sequences).
static Plan make_plan(int B, int H_kv, int max_seq_len, int num_splits, int sms) {
  constexpr int kFloorGroups = 8, kFixedTokens = 360, kMaxParts = 4096, kMaxCtasPerSm = 8, kSwitchGroups = 116;
  Plan pl;
  pl.warps = kSplitWarps; pl.depth = kSplitStages;
  pl.heads_per_cta = pick_heads_per_cta(H_kv);
  pl.head_groups = H_kv / pl.heads_per_cta;
  pl.warps_per_head = pl.warps / pl.heads_per_cta;
  const int64_t batch = B > 0 ? B : 1;
  const int ng = max_seq_len > 0 ? (max_seq_len + 15) / 16 : 1;     // groups of the longest sequence
  if (num_splits > 0) {
    const int want = num_splits < kMaxParts ? num_splits : kMaxParts;
    pl.chunk_groups = (ng + want - 1) / want;
    pl.parts = (ng + pl.chunk_groups - 1) / pl.chunk_groups;
    pl.groups_pad = pl.chunk_groups * pl.parts;
    pl.chunks = static_cast<int>(batch * pl.parts);
    return pl;
  }
  const int64_t positions = batch * ng;
  const int fixed = kFixedTokens * 8 / pl.heads_per_cta / 16;     // per CTA, in groups
  const int fixed_item = fixed / 2 + 1;                           // a second item in a CTA: pipeline drained and refilled
  int64_t best = -1;
  int best_c = kFloorGroups, best_pad = ng;
  auto consider = [&](int64_t c, int pad, bool straddles) {
    const int64_t ctas = (batch * pad + c - 1) / c * pl.head_groups;
    const int64_t rounds = (ctas + sms - 1) / sms;
    const int64_t est = rounds * (fixed + c) + (straddles ? fixed_item : 0);
    if (best < 0 || est < best) { best = est; best_c = static_cast<int>(c); best_pad = pad; }
  };
  for (int k = 1; k <= kMaxCtasPerSm; ++k) {
    int64_t target = static_cast<int64_t>(sms) * k / pl.head_groups;
    if (target < 1) target = 1;
    // (a) equal key ranges inside every sequence: no chunk touches two sequences
    for (int64_t per_seq = target / batch; per_seq <= target / batch + 1; ++per_seq) {
      if (per_seq < 1) continue;
      int64_t c = (ng + per_seq - 1) / per_seq;
      if (c < kFloorGroups) c = kFloorGroups;
      const int64_t n = (ng + c - 1) / c;
      consider(c, static_cast<int>(c * n), false);
    }
    // (b) the whole line cut into `target` equal chunks, whatever the sequence boundaries
    int64_t c = (positions + target - 1) / target;
    if (c < kFloorGroups) c = kFloorGroups;
    consider(c, ng, ng % c != 0);
    // (c) the same with a stretch of empty positions behind every sequence, as long as a change of sequence costs a CTA
    // (measured: 6.5 us, the streaming time of ~116 groups of one head): a chunk that holds the end of one sequence
    // and the start of the next then carries that much less work, and all CTAs finish together
    if (ng % c != 0) {
      const int gap = kSwitchGroups / pl.heads_per_cta > 0 ? kSwitchGroups / pl.heads_per_cta : 1;
      int64_t cg = (batch * (ng + gap) + target - 1) / target;
      if (cg < kFloorGroups) cg = kFloorGroups;
      if (cg > gap) consider(cg, ng + gap, false);
    }
    if (c == kFloorGroups) break;
  }
  pl.chunk_groups = best_c;
  pl.groups_pad = best_pad;
  pl.chunks = static_cast<int>((batch * best_pad + best_c - 1) / best_c);
  int parts = 1;
  if (best_pad % best_c == 0) parts = best_pad / best_c;
  else if (batch <= 65536) {
    for (int64_t b = 0; b < batch; ++b) { const int t = chunks_touched(b * best_pad, best_pad, best_c); if (t > parts) parts = t; }
  } else {
    parts = (best_pad - 1) / best_c + 2;
  }
  pl.parts = parts;
  return pl;
}

// Workspace layout: 256-byte status block, the (m, l) pairs of every partial row, then the O rows.  The O rows are
// written and read 16 bytes at a time, so the (m, l) area is padded to a multiple of 16 (an odd number of rows --
// e.g. 13 sequences x 3 query heads x an odd number of parts -- would otherwise leave them 8 bytes off).
static size_t ws_ml_bytes(size_t rows) { return (rows * 2 * sizeof(float) + 15) & ~size_t(15); }
static size_t ws_bytes(const Plan& pl, int B, int H_q) {
  const size_t rows = static_cast<size_t>(pl.parts) * B * H_q;
  return 256 + ws_ml_bytes(rows) + rows * kHeadDim * sizeof(float);
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

constexpr int kMaxDynamicSmem = 232448 - 1024;   // the opt-in shared memory of one SM (227 KB) less the kernel's static arrays

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    cudaGetLastError();
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// The cache as a 2-D byte tensor: row = one slot position (all heads, H_kv * slot_bytes bytes), rows = slot positions.
// A copy box is 16 rows x 160 bytes starting at byte head * slot_bytes: one 16-token group of one head, each slot followed
// by the first bytes of the next head's slot (or zeros where the box leaves the row), so that a slot lands in a 160-byte
// cell of the ring stage.
static int make_cache_map(const char* who, const DecodeCommon& a, CUtensorMap* out) {
  const EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return fail(CDA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from this driver", who);
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(a.H_kv) * a.slot_bytes;
  const cuuint64_t dims[2] = {row_bytes, static_cast<cuuint64_t>(a.num_slots)};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {160u, 16u};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(a.cache), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(CDA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed (%d) for rows of %llu bytes x %lld slots", who,
                                      static_cast<int>(rc), static_cast<unsigned long long>(row_bytes), static_cast<long long>(a.num_slots));
  return CDA_OK;
}

template <int G, int KB, int VB, int W, int NS>
static int launch_split(const DecodeParams& p0, const Plan& pl, const CUtensorMap& cache_map, cudaStream_t st) {
  // Wherever the dynamic window starts relative to a 64 KB boundary, the rings packed around the aligned table need
  // at most one ring of slack (or, with few warps, the gap before the table itself).
  static_assert(LutCfg<KB, VB>::kBytes + (W + 1) * DecCfg<W, NS, KB, VB>::kRingBytes <= kMaxDynamicSmem &&
                    LutCfg<KB, VB>::kBytes + kLutWindow <= kMaxDynamicSmem,
                "warp rings and the lookup table do not fit the shared memory of one SM");
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(decode_split_kernel<G, KB, VB, W, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxDynamicSmem) != cudaSuccess)
      return check_launch("decode: shared memory opt-in");
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  DecodeParams p = p0;
  p.smem_bytes = kMaxDynamicSmem;
  const dim3 grid(pl.chunks, pl.head_groups);
  decode_split_kernel<G, KB, VB, W, NS><<<grid, W * 32, kMaxDynamicSmem, st>>>(p, cache_map);
  return check_launch("decode split kernel");
}

// Ring depth: three stages next to one table window, two next to two (both fit the 227 KB of an SM; the third stage
// buys nothing measurable -- the copy engine keeps two groups per warp in flight either way).
template <int G, int KB, int VB>
static int dispatch_shape(const DecodeParams& p, const Plan& pl, const CUtensorMap& cache_map, cudaStream_t st) {
  constexpr int NS = LutCfg<KB, VB>::kWindows == 1 ? kSplitStages : 2;
  return launch_split<G, KB, VB, kSplitWarps, NS>(p, pl, cache_map, st);
}

template <int G>
static int dispatch_bits(const DecodeParams& p, const Plan& pl, const CUtensorMap& cache_map, int kb, int vb, cudaStream_t st) {
  if (kb == 4 && vb == 4) return dispatch_shape<G, 4, 4>(p, pl, cache_map, st);
  if (kb == 4 && vb == 2) return dispatch_shape<G, 4, 2>(p, pl, cache_map, st);
  if (kb == 2 && vb == 2) return dispatch_shape<G, 2, 2>(p, pl, cache_map, st);
  return dispatch_shape<G, 2, 4>(p, pl, cache_map, st);
}

static int run_split(const char* who, const DecodeCommon& a, void* workspace, size_t workspace_bytes, const Plan& pl,
                     cudaStream_t st, float** ml_out, float** o_out) {
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
  p.part_o = reinterpret_cast<float*>(ws + 256 + ws_ml_bytes(rows));
  p.B = a.B; p.H_q = a.H_q; p.H_kv = a.H_kv; p.group = a.H_q / a.H_kv;
  p.heads_per_cta = pl.heads_per_cta;
  p.block_size = a.block_size; p.bt_stride = a.bt_stride;
  p.num_blocks = static_cast<int>(a.num_slots / a.block_size);
  p.chunk_groups = pl.chunk_groups; p.groups_pad = pl.groups_pad;
  p.scale_log2 = a.scale * kLog2e;
  const int gpb = a.block_size / 16;
  p.gpb_shift = -1;
  for (int sft = 0; sft < 16; ++sft) if ((1 << sft) == gpb) p.gpb_shift = sft;
  p.smem_bytes = 0;
  CUtensorMap cache_map;
  int rc = make_cache_map(who, a, &cache_map);
  if (rc != CDA_OK) return rc;
  rc = p.group <= 4 ? dispatch_bits<4>(p, pl, cache_map, a.k_bits, a.v_bits, st) : dispatch_bits<8>(p, pl, cache_map, a.k_bits, a.v_bits, st);
  if (rc != CDA_OK) return rc;
  *ml_out = p.part_ml; *o_out = p.part_o;
  return CDA_OK;
}

// ---- split-KV scratch that lives inside the library (for cda_b200_decode_static) ------------------------------------
// 8 MiB per GPU that loads the library, held until the process exits.  Same layout as the caller-owned workspace:
// a 256-byte status block, then the (m, l) rows and the un-normalised O rows of every partial.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the CURRENT device.  In host code the symbol's name is only a handle, so the
// address is asked from the runtime once per device (with that device current) and remembered.
static int static_scratch_address(uint8_t** out) {
  static uint8_t* cached[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_launch("decode_static: cudaGetDevice");
  if (dev >= 0 && dev < 64 && cached[dev]) { *out = cached[dev]; return CDA_OK; }
  void* ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (e != cudaSuccess || ptr == nullptr) {
    cudaGetLastError();
    return fail(CDA_ERR_LAUNCH, "decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
  }
  if (dev >= 0 && dev < 64) cached[dev] = static_cast<uint8_t*>(ptr);
  *out = static_cast<uint8_t*>(ptr);
  return CDA_OK;
}

// Where a decode call delivers its result.  mode 0: fp16 rows (and optionally the log-sum-exp); mode 1: the merged
// partial (O rows o_stride floats apart, m / l ml_stride floats apart).
struct DecodeSink {
  int mode;
  __half* out; float* lse;
  float* O; float* m; float* l;
  int o_stride, ml_stride;
  ExchangeParams x;
};

static int decode_run(const char* who, const DecodeCommon& a, const DecodeSink& sink, void* workspace, size_t workspace_bytes,
                      const Plan& pl, cudaStream_t st) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.H_q;
  if (rows > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "%s: B*H_q too large", who);
  float* ml; float* po;
  const int rc = run_split(who, a, workspace, workspace_bytes, pl, st, &ml, &po);
  if (rc != CDA_OK) return rc;
  MergeParams q{};
  q.part_o = po; q.part_m = ml; q.part_l = ml + 1; q.ml_stride = 2; q.o_stride = kHeadDim; q.P = pl.parts; q.rows = rows;
  q.m_to_log2 = 1.0f; q.mode = sink.mode; q.unrotate = 1; q.out = sink.out; q.out_lse = sink.lse;
  q.out_o = sink.O; q.out_m = sink.m; q.out_l = sink.l; q.out_o_stride = sink.o_stride; q.out_ml_stride = sink.ml_stride;
  q.rows_per_seq = a.H_q; q.chunk_groups = pl.chunk_groups; q.groups_pad = pl.groups_pad;
  q.x = sink.x;
  q.x.status = reinterpret_cast<int*>(workspace);
  launch_merge(q, st);
  return check_launch("decode merge kernel");
}

}  // namespace cda

using namespace cda;

extern "C" int cda_b200_decode_plan_splits(int B, int H_kv, int max_seq_len, int device) {
  if (B <= 0 || H_kv <= 0 || max_seq_len < 0) return fail(CDA_ERR_BAD_ARG, "decode_plan_splits: bad size");
  return make_plan(B, H_kv, max_seq_len, 0, device_sm_count(device)).parts;
}

extern "C" size_t cda_b200_decode_workspace_bytes(int B, int H_q, int H_kv, int max_seq_len, int num_splits, int device) {
  if (B <= 0 || H_q <= 0 || H_kv <= 0 || max_seq_len < 0) return 256;
  return ws_bytes(make_plan(B, H_kv, max_seq_len, num_splits, device_sm_count(device)), B, H_q);
}

static int decode_fp16(const char* who, const DecodeCommon& a, void* out, float* lse, void* workspace, size_t workspace_bytes,
                       int num_splits, void* stream) {
  const int rc = validate(who, a);
  if (rc != CDA_OK || a.B == 0) return rc;
  if (!out) return fail(CDA_ERR_BAD_ARG, "%s: null output", who);
  if (reinterpret_cast<uintptr_t>(out) & 7u) return fail(CDA_ERR_BAD_ALIGN, "%s: output must be 8-byte aligned", who);
  if (num_splits < 0) return fail(CDA_ERR_BAD_ARG, "%s: negative num_splits", who);
  const DecodeSink sink{0, static_cast<__half*>(out), lse, nullptr, nullptr, nullptr, 0, 0, {}};
  return decode_run(who, a, sink, workspace, workspace_bytes, make_plan(a.B, a.H_kv, a.max_seq_len, num_splits, device_sm_count(-1)),
                    static_cast<cudaStream_t>(stream));
}

extern "C" int cda_b200_decode(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                               const float* cb_K, const float* cb_V, void* out, void* workspace, size_t workspace_bytes, int B,
                               int H_q, int H_kv, int block_size, int block_table_stride, int max_seq_len, int64_t num_slots,
                               int slot_bytes, int k_bits, int v_bits, float scale, int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  return decode_fp16("decode", a, out, nullptr, workspace, workspace_bytes, num_splits, stream);
}

extern "C" int cda_b200_decode_lse(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                   const float* cb_K, const float* cb_V, void* out, float* lse, void* workspace,
                                   size_t workspace_bytes, int B, int H_q, int H_kv, int block_size, int block_table_stride,
                                   int max_seq_len, int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale,
                                   int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  if (B > 0 && !lse) return fail(CDA_ERR_BAD_ARG, "decode_lse: null lse");
  return decode_fp16("decode_lse", a, out, lse, workspace, workspace_bytes, num_splits, stream);
}

static int decode_partial_any(const char* who, const DecodeCommon& a, float* O, float* m, float* l, int o_stride, int ml_stride,
                              void* workspace, size_t workspace_bytes, int num_splits, void* stream) {
  const int rc = validate(who, a);
  if (rc != CDA_OK || a.B == 0) return rc;
  if (!O || !m || !l) return fail(CDA_ERR_BAD_ARG, "%s: null output", who);
  if (reinterpret_cast<uintptr_t>(O) & ((o_stride & 3) ? 7u : 15u)) return fail(CDA_ERR_BAD_ALIGN, "%s: O must be 16-byte aligned (packed rows: 8)", who);
  if (num_splits < 0) return fail(CDA_ERR_BAD_ARG, "%s: negative num_splits", who);
  const DecodeSink sink{1, nullptr, nullptr, O, m, l, o_stride, ml_stride, {}};
  return decode_run(who, a, sink, workspace, workspace_bytes, make_plan(a.B, a.H_kv, a.max_seq_len, num_splits, device_sm_count(-1)),
                    static_cast<cudaStream_t>(stream));
}

extern "C" int cda_b200_decode_partial(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                       const float* cb_K, const float* cb_V, float* O, float* m, float* l, void* workspace,
                                       size_t workspace_bytes, int B, int H_q, int H_kv, int block_size, int block_table_stride,
                                       int max_seq_len, int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale,
                                       int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  return decode_partial_any("decode_partial", a, O, m, l, kHeadDim, 1, workspace, workspace_bytes, num_splits, stream);
}

extern "C" int cda_b200_decode_partial_packed(const void* Q, const void* kv_cache, const int32_t* block_table,
                                              const int32_t* seq_lens, const float* cb_K, const float* cb_V, float* packed,
                                              void* workspace, size_t workspace_bytes, int B, int H_q, int H_kv, int block_size,
                                              int block_table_stride, int max_seq_len, int64_t num_slots, int slot_bytes,
                                              int k_bits, int v_bits, float scale, int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  constexpr int kPacked = kHeadDim + 2;
  return decode_partial_any("decode_partial_packed", a, packed, packed ? packed + kHeadDim : nullptr,
                            packed ? packed + kHeadDim + 1 : nullptr, kPacked, kPacked, workspace, workspace_bytes, num_splits, stream);
}

// ---- exchange buffers: plain device allocations, shared between the processes of a node by CUDA IPC handles -----------------
extern "C" int cda_b200_exchange_alloc(size_t nbytes, void** ptr) {
  if (!ptr || nbytes == 0) return fail(CDA_ERR_BAD_ARG, "exchange_alloc: bad argument");
  void* p = nullptr;
  if (cudaMalloc(&p, nbytes) != cudaSuccess || cudaMemset(p, 0, nbytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    if (p) cudaFree(p);
    return check_launch("exchange_alloc");
  }
  *ptr = p;
  return CDA_OK;
}
extern "C" int cda_b200_exchange_free(void* ptr) {
  if (ptr && cudaFree(ptr) != cudaSuccess) return check_launch("exchange_free");
  return CDA_OK;
}
extern "C" int cda_b200_exchange_export(const void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64) return fail(CDA_ERR_BAD_ARG, "exchange_export: null pointer");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)) != cudaSuccess) return check_launch("exchange_export");
  memcpy(handle64, &h, sizeof h);
  return CDA_OK;
}
extern "C" int cda_b200_exchange_import(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return fail(CDA_ERR_BAD_ARG, "exchange_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof h);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return check_launch("exchange_import");
  *ptr = p;
  return CDA_OK;
}
extern "C" int cda_b200_exchange_close(void* ptr) {
  if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) return check_launch("exchange_close");
  return CDA_OK;
}

extern "C" size_t cda_b200_decode_exchange_bytes(int B, int H_q, int world) {
  if (B <= 0 || H_q <= 0 || world <= 0) return 0;
  return static_cast<size_t>(2) * world * B * H_q * kXchRowFloats * sizeof(float);
}

extern "C" int cda_b200_decode_exchange(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                        const float* cb_K, const float* cb_V, void* out, void* workspace, size_t workspace_bytes,
                                        void* const* peer_buffers, unsigned long long* counters, int rank, int world, int wait_ms,
                                        int B, int H_q, int H_kv, int block_size, int block_table_stride, int max_seq_len,
                                        int64_t num_slots, int slot_bytes, int k_bits, int v_bits, float scale, int num_splits,
                                        void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  const int rc = validate("decode_exchange", a);
  if (rc != CDA_OK) return rc;
  if (B == 0) return fail(CDA_ERR_BAD_ARG, "decode_exchange: B = 0 (every rank must take part in every call)");
  if (world < 1 || world > 32 || rank < 0 || rank >= world) return fail(CDA_ERR_BAD_ARG, "decode_exchange: rank %d of %d (at most 32 ranks)", rank, world);
  if (!out || !peer_buffers || !counters) return fail(CDA_ERR_BAD_ARG, "decode_exchange: null pointer");
  if ((reinterpret_cast<uintptr_t>(out) & 7u) || (reinterpret_cast<uintptr_t>(counters) & 7u) || (reinterpret_cast<uintptr_t>(peer_buffers) & 7u))
    return fail(CDA_ERR_BAD_ALIGN, "decode_exchange: out, counters and the pointer array must be 8-byte aligned");
  if (wait_ms <= 0 || wait_ms > 10000) return fail(CDA_ERR_BAD_ARG, "decode_exchange: wait_ms must be in 1 .. 10000");
  if (num_splits < 0) return fail(CDA_ERR_BAD_ARG, "decode_exchange: negative num_splits");
  DecodeSink sink{2, static_cast<__half*>(out), nullptr, nullptr, nullptr, nullptr, 0, 0, {}};
  sink.x.peers = reinterpret_cast<float* const*>(peer_buffers);
  sink.x.counters = counters;
  sink.x.rank = rank; sink.x.world = world;
  sink.x.wait_ns = static_cast<unsigned long long>(wait_ms) * 1000000ull;
  return decode_run("decode_exchange", a, sink, workspace, workspace_bytes,
                    make_plan(a.B, a.H_kv, a.max_seq_len, num_splits, device_sm_count(-1)), static_cast<cudaStream_t>(stream));
}

static int merge_any(const char* who, const float* O, const float* m, const float* l, int o_stride, int ml_stride, int S, int64_t R,
                     void* out, int unrotate, void* stream) {
  if (S <= 0 || R < 0) return fail(CDA_ERR_BAD_ARG, "%s: bad size", who);
  if (R == 0) return CDA_OK;
  if (!O || !m || !l || !out) return fail(CDA_ERR_BAD_ARG, "%s: null pointer", who);
  if ((reinterpret_cast<uintptr_t>(O) & ((o_stride & 3) ? 7u : 15u)) || (reinterpret_cast<uintptr_t>(out) & 7u))
    return fail(CDA_ERR_BAD_ALIGN, "%s: misaligned buffer", who);
  if (R > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "%s: too many rows", who);
  MergeParams q{};
  q.part_o = O; q.part_m = m; q.part_l = l; q.ml_stride = ml_stride; q.o_stride = o_stride; q.P = S; q.rows = R;
  q.m_to_log2 = kLog2e; q.mode = 0; q.unrotate = unrotate ? 1 : 0; q.out = static_cast<__half*>(out);
  launch_merge(q, static_cast<cudaStream_t>(stream));
  return check_launch(who);
}

extern "C" int cda_b200_merge_partials(const float* O, const float* m, const float* l, int S, int64_t R, void* out,
                                       int unrotate, void* stream) {
  return merge_any("merge_partials", O, m, l, kHeadDim, 1, S, R, out, unrotate, stream);
}

extern "C" int cda_b200_merge_partials_packed(const float* packed, int S, int64_t R, void* out, int unrotate, void* stream) {
  constexpr int kPacked = kHeadDim + 2;
  return merge_any("merge_partials_packed", packed, packed ? packed + kHeadDim : nullptr, packed ? packed + kHeadDim + 1 : nullptr,
                   kPacked, kPacked, S, R, out, unrotate, stream);
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
  if (reinterpret_cast<uintptr_t>(out) & 7u) return fail(CDA_ERR_BAD_ALIGN, "decode_scalar: output must be 8-byte aligned");
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

extern "C" int cda_b200_decode_static(const void* Q, const void* kv_cache, const int32_t* block_table, const int32_t* seq_lens,
                                      const float* cb_K, const float* cb_V, void* out, int B, int H_q, int H_kv, int block_size,
                                      int block_table_stride, int max_seq_len, int64_t num_slots, int slot_bytes, int k_bits,
                                      int v_bits, float scale, int num_splits, void* stream) {
  const DecodeCommon a{Q, kv_cache, block_table, seq_lens, cb_K, cb_V, B, H_q, H_kv, block_size, block_table_stride,
                       max_seq_len, num_slots, slot_bytes, k_bits, v_bits, scale};
  int rc = validate("decode_static", a);
  if (rc != CDA_OK || B == 0) return rc;
  if (!out) return fail(CDA_ERR_BAD_ARG, "decode_static: null output");
  if (reinterpret_cast<uintptr_t>(out) & 7u) return fail(CDA_ERR_BAD_ALIGN, "decode_static: output must be 8-byte aligned");
  if (num_splits < 0) return fail(CDA_ERR_BAD_ARG, "decode_static: negative num_splits");
  // Pick the decomposition: the planned (or requested) one if its partials fit in the built-in scratch, otherwise equal
  // key ranges per sequence with the largest count that does.  If not even one range per sequence fits, the problem is
  // too large for this entry point.
  const int sms = device_sm_count(-1);
  Plan pl = make_plan(B, H_kv, max_seq_len, num_splits, sms);
  for (int s = pl.parts; ws_bytes(pl, B, H_q) > kStaticScratchBytes && s > 1;) pl = make_plan(B, H_kv, max_seq_len, --s, sms);
  const size_t need = ws_bytes(pl, B, H_q);
  if (need > kStaticScratchBytes)
    return fail(CDA_ERR_WORKSPACE, "decode_static: B=%d, H_q=%d needs %zu bytes of scratch even unsplit; the built-in scratch holds %zu "
                "(use cda_b200_decode with a caller-owned workspace)", B, H_q, need, kStaticScratchBytes);
  uint8_t* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != CDA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Only the status block has to start at zero; every (m, l) row and
  // every O row that the merge reads is rewritten by this call's split kernel first.
  if (cudaMemsetAsync(scratch, 0, 256, st) != cudaSuccess) return check_launch("decode_static: clearing the status block");
  const DecodeSink sink{0, static_cast<__half*>(out), nullptr, nullptr, nullptr, nullptr, 0, 0};
  return decode_run("decode_static", a, sink, scratch, kStaticScratchBytes, pl, st);
}

// Status word of the most recent cda_b200_decode_static call on the current device (the call clears it first): bit 0 a
// block id was out of range, bit 1 the shared-memory window did not fit, bit 2 a wait for a cache copy ran out of time.
// Synchronises the device.
extern "C" int cda_b200_decode_static_status(int* status) {
  if (!status) return fail(CDA_ERR_BAD_ARG, "decode_static_status: null pointer");
  uint8_t* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != CDA_OK) return rc;
  if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(status, scratch, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return check_launch("decode_static_status");
  return CDA_OK;
}
