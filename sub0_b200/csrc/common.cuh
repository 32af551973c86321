// Shared device helpers for the sm_100a compressed-domain attention kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cda_b200.h"

namespace cda {

constexpr int kHeadDim = 128;
constexpr float kRsqrtD = 0.08838834764831845f;   // 1/sqrt(128)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNormFloor = 1e-12f;               // Compressor.encode, compression.py:328

// ---- host-side status plumbing -----------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
int device_sm_count(int device);   // cached cudaDevAttrMultiProcessorCount (device < 0: current)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int index_bytes(int bits) { return kHeadDim * bits / 8; }
inline int payload_bytes(int kb, int vb) { return index_bytes(kb) + index_bytes(vb) + 8; }
inline int slot_bytes_for(int kb, int vb) { return (payload_bytes(kb, vb) + 15) / 16 * 16; }
inline bool bits_ok(int b) { return b == 4 || b == 2; }

// ---- warp-level 128-point Walsh-Hadamard transform ---------------------------------------------
// Lane `lane` holds elements 4*lane .. 4*lane+3 of a 128-vector.  Natural (Sylvester) order,
// unnormalised: y[j] = sum_i x[i] * (-1)^popcount(i & j).
__device__ __forceinline__ void fht128_warp(float (&v)[4], int lane) {
  float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
  v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
#pragma unroll
  for (int mask = 1; mask < 32; mask <<= 1) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], mask);
      v[i] = upper ? other - v[i] : v[i] + other;
    }
  }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) x += __shfl_xor_sync(0xffffffffu, x, mask);
  return x;
}

// Four fp16 values <-> 8 bytes.
__device__ __forceinline__ void load_half4(const __half* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __half2 lo = *reinterpret_cast<const __half2*>(&raw.x);
  const __half2 hi = *reinterpret_cast<const __half2*>(&raw.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
__device__ __forceinline__ uint2 pack_half4(const float (&v)[4]) {
  const __half2 lo = __floats2half2_rn(v[0], v[1]);
  const __half2 hi = __floats2half2_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  return raw;
}
__device__ __forceinline__ float round_to_half(float x) { return __half2float(__float2half_rn(x)); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- asynchronous 16-byte copies global -> shared ------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tensor-core primitives ------------------------------------------------------------------------
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col).  Fragment ownership for lane = 4*r + c:
//   a0:(row r,   k 2c..2c+1)  a1:(row r+8, k 2c..2c+1)  a2:(row r,   k 2c+8..2c+9)  a3:(row r+8, k 2c+8..2c+9)
//   b0:(k 2c..2c+1, col r)    b1:(k 2c+8..2c+9, col r)
//   d0:(row r, col 2c) d1:(row r, col 2c+1) d2:(row r+8, col 2c) d3:(row r+8, col 2c+1)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same product with a zero accumulator: d = a * b.
__device__ __forceinline__ void mma_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// ---- packed fp32 pairs ----------------------------------------------------------------------------------------------------
// sm_100 executes mul / fma / add on two fp32 values per instruction, each lane rounded exactly as the scalar form, and a
// three-input maximum.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f2_pack(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_sub(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ---- tensor-core rotation of 16 rows at a time --------------------------------------------------------------------------
// The Sylvester matrix factors over the bits of the coordinate index: H128[i][j] = prod_b (-1)^(i_b j_b).  Four bits
// (16 values) are contracted by mma.m16n8k16 against a +-1 fp16 matrix (products exact, fp32 accumulation), the other
// three by in-register butterfly stages on the accumulators.  RotFrag is that 16 x 16 matrix as B fragments; it does
// not depend on WHICH four bits the caller maps to the 16 contraction slots (k slot 2c + e, and 8 + 2c + e for the
// fourth bit): the paged encoder contracts bits {4,3,2,0} (its A operand is one 16-byte load of one row), the staged
// rotation of the prefill kernel bits {4,3,1,0} (two rows per lane).  Either way lane c of a quad reads, for each of the
// four 64-byte quarters of a row, the 16 contiguous bytes 8c .. 8c+7 and ends up owning the same eight coordinates of
// the rotated row: what it packs is one contiguous 32-bit (4-bit codes) or 16-bit (2-bit codes) piece of the slot.
struct RotFrag {   // B operand: H16 restricted to this lane's contraction slots, for the two 8-column halves
  uint32_t b0[2], b1[2];
};
__device__ __forceinline__ RotFrag make_rot_frag(int lane) {
  const int n = lane >> 2, c = lane & 3;
  RotFrag f;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int out = 4 * (n >> 1) + 2 * t + (n & 1);                 // lo index of output column n of half t
    uint32_t h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = (__popc((4 * c + e) & out) & 1) ? 0xBC00u : 0x3C00u;   // -1 : +1
    f.b0[t] = h[0] | (h[1] << 16);
    f.b1[t] = h[2] | (h[3] << 16);
  }
  return f;
}

// Transpose an 8x8 matrix of 16-bit elements held one row-pair per lane: lane 4r+c holds (M[r][2c], M[r][2c+1])
// and receives (M[2c][r], M[2c+1][r]).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ---- codebook tables in fp16 with a compensating scale ---------------------------------------------------------
// The tensor-core operands are fp16, the codebook is fp32.  Rounding each level to fp16 puts the SAME relative error
// (up to 2^-12) on every occurrence of that level, which does not average out -- with only four levels it shifts all
// scores or all values together.  Instead the tables hold fp16(level / alpha) and the result is multiplied by alpha in
// fp32 (folded into the softmax scale for K, into the final normalisation for V).  This is done for 4-level tables
// only: with 16 levels the individual errors largely cancel and a common alpha cannot shrink all of them anyway, so
// those tables use alpha = 1 and pay no set-up time.  alpha is searched in
// [1, 1.0625) with step 2^-13 for the value whose worst-case |alpha * fp16(level / alpha) - level| is smallest; alpha = 1
// is a candidate, so the result is never worse than plain rounding.
constexpr int kScaleCandidates = 512;

__device__ __forceinline__ float table_value(float level, float inv_alpha) { return __half2float(__float2half_rn(level * inv_alpha)); }

// Call with all threads of the CTA (contains two barriers).  cb_a / cb_b: global codebooks of LA / LB levels.
// scratch: shared arrays of at least (blockDim.x / 32) entries each.
template <int LA, int LB>
__device__ __forceinline__ void find_table_scales(const float* __restrict__ cb_a, const float* __restrict__ cb_b, float* s_err, int* s_idx,
                                                  float& alpha_a, float& alpha_b) {
  if (LA != 4 && LB != 4) { alpha_a = 1.0f; alpha_b = 1.0f; return; }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  float la[LA], lb[LB];
#pragma unroll
  for (int i = 0; i < LA; ++i) la[i] = __ldg(cb_a + i);
#pragma unroll
  for (int i = 0; i < LB; ++i) lb[i] = __ldg(cb_b + i);
  float best[2] = {3.0e38f, 3.0e38f};
  int arg[2] = {0, 0};
  for (int cand = tid; cand < kScaleCandidates; cand += blockDim.x) {
    const float alpha = 1.0f + cand * (1.0f / 8192.0f), inv = 1.0f / alpha;
    float ea = 0.f, eb = 0.f;
    if (LA == 4) {
#pragma unroll
      for (int i = 0; i < LA; ++i) ea = fmaxf(ea, fabsf(fmaf(alpha, table_value(la[i], inv), -la[i])));
    }
    if (LB == 4) {
#pragma unroll
      for (int i = 0; i < LB; ++i) eb = fmaxf(eb, fabsf(fmaf(alpha, table_value(lb[i], inv), -lb[i])));
    }
    if (ea < best[0]) { best[0] = ea; arg[0] = cand; }
    if (eb < best[1]) { best[1] = eb; arg[1] = cand; }
  }
#pragma unroll
  for (int t = 0; t < 2; ++t) {
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) {
      const float oe = __shfl_xor_sync(0xffffffffu, best[t], mask);
      const int oi = __shfl_xor_sync(0xffffffffu, arg[t], mask);
      if (oe < best[t] || (oe == best[t] && oi < arg[t])) { best[t] = oe; arg[t] = oi; }
    }
    if (lane == 0) { s_err[t * 32 + warp] = best[t]; s_idx[t * 32 + warp] = arg[t]; }
  }
  __syncthreads();
  int win[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    float e = s_err[t * 32]; int i = s_idx[t * 32];
    for (int w = 1; w < nwarps; ++w) {
      const float oe = s_err[t * 32 + w]; const int oi = s_idx[t * 32 + w];
      if (oe < e || (oe == e && oi < i)) { e = oe; i = oi; }
    }
    win[t] = i;
  }
  __syncthreads();
  alpha_a = LA == 4 ? 1.0f + win[0] * (1.0f / 8192.0f) : 1.0f;
  alpha_b = LB == 4 ? 1.0f + win[1] * (1.0f / 8192.0f) : 1.0f;
}

}  // namespace cda
