// Paged encode (Hadamard rotation -> L2 norm -> nearest codebook level -> packed slot), the index
// selection on its own, and the stand-alone 128-point Hadamard transform.
//
// One warp owns one 128-vector: lane l holds coordinates 4l..4l+3, the rotation is 2 in-register and
// 5 shuffle butterfly stages, the norm a shuffle reduction.  The kernels are HBM-bound: 2 x 256 B
// read and one payload (136 B for k4v4) written per (token, KV head).
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

// v: this lane's four rotated fp32 coordinates.  Writes the packed indices of the row to `idx_dst`
// (16*BITS bytes per row) and returns the row norm (identical in every lane).  T: thresholds of the codebook.
template <int BITS>
__device__ __forceinline__ float quantize_row(const float (&v)[4], const float* T, uint8_t* idx_dst, int lane) {
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
    idx[i] = count_thresholds<L>(u, T);
  }
  if (BITS == 4) {
    const uint16_t two = static_cast<uint16_t>(((idx[0] << 4) | idx[1]) | (((idx[2] << 4) | idx[3]) << 8));
    reinterpret_cast<uint16_t*>(idx_dst)[lane] = two;
  } else {
    idx_dst[lane] = static_cast<uint8_t>((idx[0] << 6) | (idx[1] << 4) | (idx[2] << 2) | idx[3]);
  }
  return norm;
}

template <int KB, int VB>
__global__ void __launch_bounds__(256) paged_encode_kernel(const __half* __restrict__ K, const __half* __restrict__ V,
                                                           const int32_t* __restrict__ slot_mapping,
                                                           uint8_t* __restrict__ cache, const float* __restrict__ cb_K,
                                                           const float* __restrict__ cb_V, int64_t rows, int H_kv,
                                                           int64_t num_slots, int slot_bytes) {
  __shared__ float s_cb[2][16], s_thr[2][16];
  if (threadIdx.x < 16) {
    s_cb[0][threadIdx.x] = threadIdx.x < (KB == 4 ? 16 : 4) ? cb_K[threadIdx.x] : 0.f;
    s_cb[1][threadIdx.x] = threadIdx.x < (VB == 4 ? 16 : 4) ? cb_V[threadIdx.x] : 0.f;
  }
  __syncthreads();
  build_thresholds<(KB == 4 ? 16 : 4)>(s_cb[0], s_thr[0], threadIdx.x);
  build_thresholds<(VB == 4 ? 16 : 4)>(s_cb[1], s_thr[1], static_cast<int>(threadIdx.x) - 32);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  constexpr int kKBytes = 16 * KB, kVBytes = 16 * VB;
  // grid-stride over rows (row = t * H_kv + h): the threshold set-up is paid once per CTA
  // (token, head) of the row advance with the row, so the 64-bit division happens once per warp
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 8;
  const int64_t t_step = stride / H_kv;
  const int h_step = static_cast<int>(stride - t_step * H_kv);
  int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  int64_t t = row / H_kv;
  int h = static_cast<int>(row - t * H_kv);
  for (; row < rows; row += stride, t += t_step, h += h_step) {
    if (h >= H_kv) { h -= H_kv; ++t; }
    const int64_t slot = slot_mapping[t];
    if (slot < 0 || slot >= num_slots) continue;
    uint8_t* dst = cache + (slot * H_kv + h) * slot_bytes;

    float v[4], w[4];
    load_half4(K + row * kHeadDim + 4 * lane, v);
    load_half4(V + row * kHeadDim + 4 * lane, w);
    fht128_warp(v, lane);
    fht128_warp(w, lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) {                       // Compressor.rotate casts back to fp16
      v[i] = round_to_half(v[i] * kRsqrtD);
      w[i] = round_to_half(w[i] * kRsqrtD);
    }
    const float nk = quantize_row<KB>(v, s_thr[0], dst, lane);
    const float nv = quantize_row<VB>(w, s_thr[1], dst + kKBytes, lane);
    if (lane == 0) *reinterpret_cast<float2*>(dst + kKBytes + kVBytes) = make_float2(nk, nv);
  }
}

template <int BITS>
__global__ void __launch_bounds__(256) quantize_rotated_kernel(const float* __restrict__ x, int64_t rows,
                                                               const float* __restrict__ cb, uint8_t* __restrict__ idx_out,
                                                               float* __restrict__ norm_out) {
  __shared__ float s_cb[16], s_thr[16];
  if (threadIdx.x < 16) s_cb[threadIdx.x] = threadIdx.x < (BITS == 4 ? 16 : 4) ? cb[threadIdx.x] : 0.f;
  __syncthreads();
  build_thresholds<(BITS == 4 ? 16 : 4)>(s_cb, s_thr, threadIdx.x);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += static_cast<int64_t>(gridDim.x) * 8) {
    const float4 raw = *reinterpret_cast<const float4*>(x + row * kHeadDim + 4 * lane);
    const float v[4] = {raw.x, raw.y, raw.z, raw.w};
    const float n = quantize_row<BITS>(v, s_thr, idx_out + row * (16 * BITS), lane);
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
  const int64_t blocks = blocks_for_rows(rows);
  if (blocks > 0x7fffffffLL) return fail(CDA_ERR_N_TOO_LARGE, "paged_encode: T*H_kv too large");
  const dim3 grid(persistent_grid(rows)), block(256);
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
