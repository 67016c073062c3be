// Activation rows prepared for the W4A16 kernels: the k order 0,4,1,5,2,6,3,7 inside every 8 (the order in which
// one logic op per nibble pair unpacks a weight word) and the row's sums over every 128 k.
// Two formats.  bf16: the values as they are.  fp16: every row multiplied by a power of two 2^e that puts its
// largest magnitude into [2^14, 2^15), then converted to fp16.  A bf16 value has 8 significant bits and fp16
// holds 11, so the conversion is exact for every element within 2^-28 of the row's largest (smaller ones land
// on fp16 subnormals and may lose low bits: an error below 2^-39 of the largest element, far under the
// rounding of the fp32 sums they enter); products and sums then run on the scaled values and the result is
// multiplied by 2^-e, which the rows' sums table carries in its last slot.  fp16 weights can be unpacked with
// five instead of seven integer instructions per word, which is why the stream kernel prefers this format.
#pragma once

#include "common.cuh"

namespace mq {

constexpr int W4_XS_STRIDE = 32;            // floats per row in the sums table
constexpr int W4_XS_UNSCALE = 31;           // fp16 format: slot of 2^-e (so at most 31 groups, K <= 3968)

// e with amax * 2^e in [2^14, 2^15); 0 for a row of zeros or non-finite values.
__device__ __forceinline__ int w4_row_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  const int ex = (int)((bits >> 23) & 0xFFu);
  if (ex == 0 || ex == 0xFF) return 0;
  int e = 14 - (ex - 127);
  return e < -100 ? -100 : (e > 100 ? 100 : e);
}
__device__ __forceinline__ float w4_pow2(int e) { return __uint_as_float((uint32_t)(127 + e) << 23); }

// One 16-byte piece (8 consecutive k) of a row: returns it in the prepared order and format and adds the sum
// of its (prepared) values to `sum`, k ascending.
__device__ __forceinline__ uint4 w4_prepare_piece(const uint4& v, bool shuffle, bool f16, float scale, float& sum) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(&v);
  uint16_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float f = __bfloat162float(__ushort_as_bfloat16(h[j]));
    if (f16) {
      const __half hv = __float2half_rn(f * scale);
      o[j] = __half_as_ushort(hv);
      sum += __half2float(hv);
    } else {
      o[j] = h[j];
      sum += f;
    }
  }
  uint4 w;
  if (shuffle) {
    w.x = (uint32_t)o[0] | ((uint32_t)o[4] << 16);
    w.y = (uint32_t)o[1] | ((uint32_t)o[5] << 16);
    w.z = (uint32_t)o[2] | ((uint32_t)o[6] << 16);
    w.w = (uint32_t)o[3] | ((uint32_t)o[7] << 16);
  } else {
    w.x = (uint32_t)o[0] | ((uint32_t)o[1] << 16);
    w.y = (uint32_t)o[2] | ((uint32_t)o[3] << 16);
    w.z = (uint32_t)o[4] | ((uint32_t)o[5] << 16);
    w.w = (uint32_t)o[6] | ((uint32_t)o[7] << 16);
  }
  return w;
}

// largest magnitude of a 16-byte piece of bf16 values
__device__ __forceinline__ float w4_piece_amax(const uint4& v) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(&v);
  float m = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(__bfloat162float(__ushort_as_bfloat16(h[j]))));
  return m;
}

}  // namespace mq
