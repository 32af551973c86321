// Causal varlen prefill over the paged compressed cache on the sm_100a tensor-core path (tcgen05.mma, accumulators
// in tensor memory).  Same contract as the reference's fused prefill (cda/kernels_cuda/fa2_cda.py:98-230 with
// fuse_fa2_epilogue=True; oracle: attention_compressed(causal=True, q_offset=seq_len-q_len), cda/algorithm/attention.py:426-482):
// rotate Q, attend to the dequantised keys and values in the rotated domain with bottom-right aligned causal masking,
// round the normalised output to fp16, rotate back.
//
// One CTA = 128 rows = (128 / G) consecutive query positions x the G query heads of one KV head, so that a
// dequantised key/value tile serves the whole GQA group.  Keys are processed 64 at a time:
//
//   producer warps (4)   cache slots -> unit-level fp16 tiles in shared memory (128-byte swizzled rows, the layout
//                        tcgen05.mma reads), norms to side arrays
//   MMA warp (1 thread)  S = Q K^T (128x64x128) into TMEM, O += P V (128x128x64) into TMEM
//   softmax warps (4)    thread t owns row t: TMEM -> registers, scale by the key norm, mask, online maximum with lazy
//                        rescaling of O, exp2, fold the value norm, fp16 P -> shared memory
//
// The roles hand tiles over through mbarriers; every wait is bounded (umma.cuh) and a wait that gives up sets bit 2 of
// the status word and ends the CTA cleanly (TMEM is released).  Two CTAs fit one SM (108 KB shared memory, 256 TMEM
// columns each), so one CTA's softmax overlaps the other's matrix products.
#include "common.cuh"
#include "umma.cuh"
#include "prefill_umma.cuh"

namespace cda {

// Set (and never cleared) when a CTA of the prefill kernel gave up on a wait: later CTAs and launches return at once
// instead of each running into its own time-out.  Read by cda_b200_prefill_fault().
__device__ int g_prefill_fault = 0;

namespace pfu {

constexpr int kRows = 128;            // rows of a CTA tile
constexpr int kKeys = 64;             // keys per tile
constexpr int kSoftmaxWarps = 4, kProducerWarps = 4;
constexpr int kThreads = (kSoftmaxWarps + kProducerWarps + 1) * 32;
constexpr int kTmemCols = 256;        // S0 [0,64)  S1 [64,128)  O [128,256)
constexpr float kLazy = 4.0f;         // O is rescaled only when the row maximum grew by more than 2^4

// shared memory map (bytes from the 1024-aligned base)
constexpr int kOffQ = 0;                       // 2 column blocks x 128 rows x 128 B
constexpr int kOffK = 32768;                   // 2 stages x (2 column blocks x 64 rows x 128 B)
constexpr int kOffV = 65536;                   // 2 column blocks x 64 rows x 128 B
constexpr int kOffP = 81920;                   // 128 rows x 128 B
constexpr int kOffKn = 98304;                  // 4 x 64 floats: key norm * softmax scale * log2(e) * alpha_k
constexpr int kOffVn = kOffKn + 1024;          // 4 x 64 floats: value norm
constexpr int kOffLutK = kOffVn + 1024;        // 4 KB
constexpr int kOffLutV = kOffLutK + 4096;      // 4 KB
constexpr int kOffBar = kOffLutV + 4096;       // mbarriers, TMEM address, flags
constexpr int kSmemBytes = kOffBar + 256 + 1024;   // + slack for the 1024-byte alignment

// barrier slots (8 bytes each) inside kOffBar
constexpr int kBarKFull = 0, kBarSFull = 2, kBarVFull = 4, kBarPFull = 5, kBarPvDone = 6, kBarNorms = 7;   // 11 barriers
constexpr int kOffTmemAddr = 96, kOffAbort = 100;

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void unpack_half4(const uint2& raw, float (&v)[4]) {
  const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  v[0] = fa.x; v[1] = fa.y; v[2] = fb.x; v[3] = fb.y;
}
// mbar_wait with a warp-uniform result (the callers go on to warp-synchronous instructions)
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = umma::mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) {   // byte offset inside a block of 128-byte rows
  return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

// Table entry for one code byte.  4-bit codes: 2 levels (4 bytes), four copies per entry (16-byte stride).  2-bit codes:
// 4 levels (8 bytes), two copies.
template <int BITS>
__device__ __forceinline__ void fill_code_table(uint8_t* lut, const float* __restrict__ cb, float inv_alpha, int tid, int nthreads) {
  for (int e = tid; e < 256; e += nthreads) {
    if (BITS == 4) {
      const uint32_t w = pack_half2(__ldg(cb + (e >> 4)) * inv_alpha, __ldg(cb + (e & 15)) * inv_alpha);
      *reinterpret_cast<uint4*>(lut + e * 16) = make_uint4(w, w, w, w);
    } else {
      const uint32_t w0 = pack_half2(__ldg(cb + ((e >> 6) & 3)) * inv_alpha, __ldg(cb + ((e >> 4) & 3)) * inv_alpha);
      const uint32_t w1 = pack_half2(__ldg(cb + ((e >> 2) & 3)) * inv_alpha, __ldg(cb + (e & 3)) * inv_alpha);
      *reinterpret_cast<uint4*>(lut + e * 16) = make_uint4(w0, w1, w0, w1);
    }
  }
}

// Expand 16 bytes of codes (one quad of a slot) of token row `nl` into fp16 chunks of a 64-row tile.
// tile: shared address of column block 0 (block 1 is 8192 bytes further).  quad: index of the 16 bytes in the row's codes.
template <int BITS>
__device__ __forceinline__ void expand_quad(uint32_t tile, uint32_t lut_lane, const uint4& w, int nl, int quad) {
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
  if (BITS == 4) {
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const uint32_t x = ws[wi];
      uint32_t v[4];
      v[0] = lds32(lut_lane + ((x << 4) & 0xff0u));
      v[1] = lds32(lut_lane + ((x >> 4) & 0xff0u));
      v[2] = lds32(lut_lane + ((x >> 12) & 0xff0u));
      v[3] = lds32(lut_lane + ((x >> 20) & 0xff0u));
      const int c16 = quad * 4 + wi;                       // 16-byte chunk of the row: 8 coordinates
      sts128(tile + (c16 >> 3) * 8192u + sw128(nl, c16 & 7), v[0], v[1], v[2], v[3]);
    }
  } else {
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const uint32_t x = ws[wi];
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {                     // two code bytes = 8 coordinates = one chunk
        const uint32_t b0 = (x >> (16 * hb)) & 0xffu, b1 = (x >> (16 * hb + 8)) & 0xffu;
        const uint2 lo = lds64(lut_lane + (b0 << 4)), hi = lds64(lut_lane + (b1 << 4));
        const int c16 = quad * 8 + wi * 2 + hb;
        sts128(tile + (c16 >> 3) * 8192u + sw128(nl, c16 & 7), lo.x, lo.y, hi.x, hi.y);
      }
    }
  }
}

}  // namespace pfu

template <int G, int KB, int VB>
__global__ void __launch_bounds__(pfu::kThreads, 2) prefill_umma_kernel(const PrefillUmmaParams p) {
  using namespace pfu;
  using namespace umma;
  constexpr int kPosPerTile = kRows / G;
  constexpr int kSlotBytes = 16 * KB + 16 * VB + 16;
  constexpr int kQuadsK = KB, kQuadsV = VB;                // 16-byte pieces of a row's codes (64 or 32 bytes)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_addr(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int seq_len = p.seq_lens[b];
  const int n_qtiles = (q_len + kPosPerTile - 1) / kPosPerTile;
  const int qt = n_qtiles - 1 - static_cast<int>(blockIdx.x);   // longest rows first
  if (qt < 0 || seq_len <= 0 || q_len > seq_len) return;
  if (*reinterpret_cast<volatile int*>(&g_prefill_fault)) return;
  const int p0 = qt * kPosPerTile;                               // first query position (within the new tokens) of this tile
  const int q_offset = seq_len - q_len;                          // bottom-right alignment
  const int pos_hi = min(p0 + kPosPerTile, q_len) - 1;
  const int n_tiles = (q_offset + pos_hi) / kKeys + 1;           // key tiles that hold an unmasked key
  const int g = p.group;

  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kOffBar + kOffAbort);
  const uint32_t bar0 = base + kOffBar;
  auto bar = [&](int i) { return bar0 + 8u * i; };

  __shared__ float s_err[64];
  __shared__ int s_idx[64];
  float alpha_k, alpha_v;
  find_table_scales<(KB == 4 ? 16 : 4), (VB == 4 ? 16 : 4)>(p.cb_k, p.cb_v, s_err, s_idx, alpha_k, alpha_v);

  // ---- set-up: barriers, TMEM, tables, rotated queries -----------------------------------------------------------------
  if (tid == 0) {
    mbar_init(bar(kBarKFull), kProducerWarps); mbar_init(bar(kBarKFull + 1), kProducerWarps);
    mbar_init(bar(kBarSFull), 1); mbar_init(bar(kBarSFull + 1), 1);
    mbar_init(bar(kBarVFull), kProducerWarps);
    mbar_init(bar(kBarPFull), kSoftmaxWarps);
    mbar_init(bar(kBarPvDone), 1);
    for (int i = 0; i < 4; ++i) mbar_init(bar(kBarNorms + i), kProducerWarps);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == kSoftmaxWarps + kProducerWarps) {
    tmem_alloc(base + kOffBar + kOffTmemAddr, kTmemCols);
    tmem_relinquish();
  }
  fill_code_table<KB>(sm + kOffLutK, p.cb_k, 1.0f / alpha_k, tid, kThreads);
  fill_code_table<VB>(sm + kOffLutV, p.cb_v, 1.0f / alpha_v, tid, kThreads);
  for (int t = warp; t < kRows; t += kThreads / 32) {   // one warp per row: load, rotate, store as the A operand of Q K^T
    const int pos = p0 + t / G, hl = t % G;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (pos < q_len && hl < g) {
      load_half4(p.q + (static_cast<int64_t>(q_begin + pos) * p.H_q + kvh * g + hl) * kHeadDim + 4 * lane, v);
      fht128_warp(v, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= kRsqrtD;
    }
    const uint32_t dst = base + kOffQ + (lane >> 4) * 16384u + sw128(t, (lane & 15) >> 1) + (lane & 1) * 8u;
    const uint2 h = pack_half4(v);
    sts64(dst, h.x, h.y);
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sm + kOffBar + kOffTmemAddr);

  if (warp < kSoftmaxWarps) {
    // ================= softmax: thread t owns row t =====================================================================
    const int t = tid;
    const int q_pos = q_offset + p0 + t / G;                 // key index of the diagonal for this row
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    float m_used = -INFINITY, l_run = 0.f;
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      const uint32_t s_tmem = lane_base + (j & 1) * kKeys;
      const float* kn = reinterpret_cast<const float*>(sm + kOffKn) + (j & 3) * kKeys;
      const float* vn = reinterpret_cast<const float*>(sm + kOffVn) + (j & 3) * kKeys;
      // the norms come straight from the producers (slot j & 3 is rewritten only for tile j + 4), the scores from the MMA
      alive = warp_wait(bar(kBarNorms + (j & 3)), (j >> 2) & 1, abort_flag) &&
              warp_wait(bar(kBarSFull + (j & 1)), (j >> 1) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after_sync();
      const int key0 = j * kKeys;
      const bool diag = key0 + kKeys - 1 > q_offset + p0;    // some row of the tile masks some key of this tile

      // pass 1: row maximum over the 64 scores (two 32-column reads; the second half stays in registers)
      uint32_t sa[32], sb[32];
      float mx = -INFINITY;
      tmem_ld32(s_tmem, sa);
      tmem_ld32(s_tmem + 32, sb);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float x = __uint_as_float(sa[c]) * kn[c];
        if (diag && key0 + c > q_pos) x = -INFINITY;
        mx = fmaxf(mx, x);
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float x = __uint_as_float(sb[c]) * kn[32 + c];
        if (diag && key0 + 32 + c > q_pos) x = -INFINITY;
        sb[c] = __float_as_uint(x);
        mx = fmaxf(mx, x);
      }
      float factor = 1.0f;
      if (mx > m_used + kLazy || m_used == -INFINITY) {      // tile 0 always lands here (key 0 is never masked)
        const float m_new = fmaxf(m_used, mx);
        factor = m_used == -INFINITY ? 0.0f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l_run *= factor;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, factor != 1.0f);

      // second half -> probabilities (registers), then the first half again from TMEM
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float e0 = fast_exp2(__uint_as_float(sb[c]) - m_used), e1 = fast_exp2(__uint_as_float(sb[c + 1]) - m_used);
        l_run += e0 + e1;
        pk[16 + c / 2] = pack_half2(e0 * vn[32 + c], e1 * vn[32 + c + 1]);
      }
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float x0 = __uint_as_float(sa[c]) * kn[c], x1 = __uint_as_float(sa[c + 1]) * kn[c + 1];
        if (diag && key0 + c > q_pos) x0 = -INFINITY;
        if (diag && key0 + c + 1 > q_pos) x1 = -INFINITY;
        const float e0 = fast_exp2(x0 - m_used), e1 = fast_exp2(x1 - m_used);
        l_run += e0 + e1;
        pk[c / 2] = pack_half2(e0 * vn[c], e1 * vn[c + 1]);
      }

      if (j > 0) {   // P and O belong to the previous P V product until it has completed
        alive = warp_wait(bar(kBarPvDone), (j - 1) & 1, abort_flag);
        if (!alive) break;
        tc_fence_after_sync();
      }
      if (rescale) {
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          tmem_ld32(lane_base + 128 + 32 * ch, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
          tmem_st32(lane_base + 128 + 32 * ch, o);
        }
        tmem_wait_st();
      }
      const uint32_t prow = base + kOffP;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) sts128(prow + sw128(t, ch), pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
      fence_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull));
    }
    // ---- epilogue part 1: normalised fp16 row of O into the (now unused) Q area, 256-byte rows, chunk XOR (t & 15) ------
    if (alive) alive = warp_wait(bar(kBarPvDone), (n_tiles - 1) & 1, abort_flag);
    if (alive) {
      tc_fence_after_sync();
      const float inv = alpha_v / fmaxf(l_run, 1e-30f);
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[32];
        tmem_ld32(lane_base + 128 + 32 * ch, o);
        tmem_wait_ld();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint32_t h[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            h[i] = pack_half2(__uint_as_float(o[8 * c8 + 2 * i]) * inv, __uint_as_float(o[8 * c8 + 2 * i + 1]) * inv);
          const uint32_t chunk = static_cast<uint32_t>(ch * 4 + c8);
          sts128(base + kOffQ + t * 256u + ((chunk ^ (t & 15u)) << 4), h[0], h[1], h[2], h[3]);
        }
      }
    }
    tc_fence_before_sync();
  } else if (warp < kSoftmaxWarps + kProducerWarps) {
    // ================= producers: slots -> unit-level fp16 tiles ============================================================
    const int pt = tid - kSoftmaxWarps * 32;                 // 0..127
    const uint32_t lutk_lane = base + kOffLutK + (KB == 4 ? (lane & 3) * 4u : (lane & 1) * 8u);
    const uint32_t lutv_lane = base + kOffLutV + (VB == 4 ? (lane & 3) * 4u : (lane & 1) * 8u);
    const int32_t* bt_row = p.block_table + static_cast<int64_t>(b) * p.bt_stride;
    const int64_t row_stride = static_cast<int64_t>(p.H_kv) * kSlotBytes;
    const float kscale = p.scale_log2 * alpha_k;
    bool alive = true, bad_block = false;

    auto slot_ptr = [&](int nl, int key0) -> const uint8_t* {
      const int n = min(key0 + nl, seq_len - 1);             // keys past the end are masked later; read a valid slot
      int blk = __ldg(bt_row + n / p.block_size);
      if (static_cast<unsigned>(blk) >= static_cast<unsigned>(p.num_blocks)) { bad_block = true; blk = 0; }
      return p.cache + (static_cast<int64_t>(blk) * p.block_size + n % p.block_size) * row_stride + kvh * kSlotBytes;
    };
    auto produce_k = [&](int j) {
      const uint32_t tile = base + kOffK + (j & 1) * 16384u;
      float* kn = reinterpret_cast<float*>(sm + kOffKn) + (j & 3) * kKeys;
      float* vn = reinterpret_cast<float*>(sm + kOffVn) + (j & 3) * kKeys;
#pragma unroll
      for (int it = 0; it < kKeys * kQuadsK / 128; ++it) {
        const int x = pt + 128 * it, nl = x / kQuadsK, quad = x % kQuadsK;
        const uint8_t* src = slot_ptr(nl, j * kKeys);
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(src + 16 * quad));
        if (quad == 0) {
          const float2 nrm = __ldg(reinterpret_cast<const float2*>(src + 16 * KB + 16 * VB));
          kn[nl] = nrm.x * kscale;
          vn[nl] = nrm.y;
        }
        expand_quad<KB>(tile, lutk_lane, w, nl, quad);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar(kBarNorms + (j & 3))); mbar_arrive(bar(kBarKFull + (j & 1))); }
    };
    auto produce_v = [&](int j) {
      const uint32_t tile = base + kOffV;
#pragma unroll
      for (int it = 0; it < kKeys * kQuadsV / 128; ++it) {
        const int x = pt + 128 * it, nl = x / kQuadsV, quad = x % kQuadsV;
        const uint8_t* src = slot_ptr(nl, j * kKeys);
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(src + 16 * KB + 16 * quad));
        expand_quad<VB>(tile, lutv_lane, w, nl, quad);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarVFull));
    };

    produce_k(0);
    if (n_tiles > 1) produce_k(1);
    produce_v(0);
    for (int j = 1; j < n_tiles && alive; ++j) {
      if (j + 1 < n_tiles) {                                 // stage (j+1)&1 is free once Q K^T of tile j-1 has completed
        alive = warp_wait(bar(kBarSFull + ((j + 1) & 1)), ((j - 1) >> 1) & 1, abort_flag);
        if (!alive) break;
        produce_k(j + 1);
      }
      alive = warp_wait(bar(kBarPvDone), (j - 1) & 1, abort_flag);   // the V tile is free once P V of tile j-1 has completed
      if (!alive) break;
      produce_v(j);
    }
    if (bad_block && p.status) atomicOr(p.status, 1);
  } else {
    // ================= MMA issuer ==================================================================================================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = instr_desc_f16(kRows, kKeys, false, false);
      constexpr uint32_t idesc_pv = instr_desc_f16(kRows, kHeadDim, false, true);
      const uint32_t o_tmem = tmem + 128;
      bool alive = true;
      auto issue_qk = [&](int j) {
        const uint32_t ktile = base + kOffK + (j & 1) * 16384u;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t a = smem_desc_sw128(base + kOffQ + (ks >> 2) * 16384u + (ks & 3) * 32u, 16, 1024);
          const uint64_t bd = smem_desc_sw128(ktile + (ks >> 2) * 8192u + (ks & 3) * 32u, 16, 1024);
          mma_ss(tmem + (j & 1) * kKeys, a, bd, idesc_qk, ks > 0 ? 1u : 0u);
        }
        mma_commit(bar(kBarSFull + (j & 1)));
      };
      alive = mbar_wait(bar(kBarKFull), 0, abort_flag);
      if (alive) {
        tc_fence_after_sync();
        issue_qk(0);
      }
      for (int j = 0; j < n_tiles && alive; ++j) {
        if (j + 1 < n_tiles) {
          alive = mbar_wait(bar(kBarKFull + ((j + 1) & 1)), ((j + 1) >> 1) & 1, abort_flag);
          if (!alive) break;
          tc_fence_after_sync();
          issue_qk(j + 1);
        }
        alive = mbar_wait(bar(kBarVFull), j & 1, abort_flag) && mbar_wait(bar(kBarPFull), j & 1, abort_flag);
        if (!alive) break;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t a = smem_desc_sw128(base + kOffP + ks * 32u, 16, 1024);
          const uint64_t bd = smem_desc_sw128(base + kOffV + ks * 2048u, 8192, 1024);
          mma_ss(o_tmem, a, bd, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        mma_commit(bar(kBarPvDone));
      }
      if (alive) mbar_wait(bar(kBarPvDone), (n_tiles - 1) & 1, abort_flag);   // nothing in flight when TMEM is released
    }
    __syncwarp();
    tc_fence_before_sync();
  }

  // ---- epilogue part 2: every warp rotates rows back and stores them ---------------------------------------------------------
  __syncthreads();
  const bool failed = *abort_flag != 0;
  if (!failed) {
    for (int t = warp; t < kRows; t += kThreads / 32) {
      const int pos = p0 + t / G, hl = t % G;
      if (pos >= q_len || hl >= g) continue;
      const uint32_t src = base + kOffQ + t * 256u + ((static_cast<uint32_t>(lane >> 1) ^ (t & 15u)) << 4) + (lane & 1) * 8u;
      const uint2 raw = lds64(src);
      float v[4];
      unpack_half4(raw, v);
      fht128_warp(v, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= kRsqrtD;
      *reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(q_begin + pos) * p.H_q + kvh * g + hl) * kHeadDim + 4 * lane) = pack_half4(v);
    }
  } else if (tid == 0) {
    atomicOr(&g_prefill_fault, 1);
    if (p.status) atomicOr(p.status, 4);
  }
  __syncthreads();
  if (warp == kSoftmaxWarps + kProducerWarps) {
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
  const int per_tile = pfu::kRows / G;
  const dim3 grid((max_query_len + per_tile - 1) / per_tile, p.H_kv, B);
  prefill_umma_kernel<G, KB, VB><<<grid, pfu::kThreads, pfu::kSmemBytes, st>>>(p);
  return check_launch("prefill kernel");
}

template <int KB, int VB>
static int dispatch_prefill_umma_group(const PrefillUmmaParams& p, int max_query_len, int B, cudaStream_t st) {
  return p.group <= 4 ? launch_prefill_umma<4, KB, VB>(p, max_query_len, B, st) : launch_prefill_umma<8, KB, VB>(p, max_query_len, B, st);
}

int dispatch_prefill_umma(const PrefillUmmaParams& p, int k_bits, int v_bits, int max_query_len, int B, cudaStream_t st) {
  if (k_bits == 4 && v_bits == 4) return dispatch_prefill_umma_group<4, 4>(p, max_query_len, B, st);
  if (k_bits == 4 && v_bits == 2) return dispatch_prefill_umma_group<4, 2>(p, max_query_len, B, st);
  if (k_bits == 2 && v_bits == 2) return dispatch_prefill_umma_group<2, 2>(p, max_query_len, B, st);
  return dispatch_prefill_umma_group<2, 4>(p, max_query_len, B, st);
}

}  // namespace cda

// 1 if a prefill CTA on the current device ever gave up on a wait (synchronises the device), 0 if not, < 0 on error.
extern "C" int cda_b200_prefill_fault(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, cda::g_prefill_fault, sizeof(int)) != cudaSuccess) return cda::check_launch("prefill_fault");
  return v != 0 ? 1 : 0;
}
