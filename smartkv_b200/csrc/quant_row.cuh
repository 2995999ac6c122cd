// Row-level helpers shared by the append and the repack kernels: one warp owns one row of
// head_dim values (EPL = head_dim / 32 consecutive elements per lane).
//
// Arithmetic follows the reference CPU quantiser (smartkv/core/_quant_cpu.py:20-34):
// scale = absmax / max(max_code, 1) with an IEEE fp32 divide, 0 -> 1,
// code = clamp(rint(x / scale)) with round-half-even.  No fast-math: codes and scales are
// bit-exact with the CPU path.  Packed format: smartkv/csrc/bit_packing.cu:20-43, 69-95, 128-151.
#pragma once

#include "common.cuh"

namespace skv {

template <int EPL>  // elements per lane: head_dim / 32
struct RowVals {
  float v[EPL];
};

template <int EPL>
__device__ __forceinline__ RowVals<EPL> load_row(const void* base, int dtype, long long row, int lane) {
  RowVals<EPL> r;
  constexpr int D = EPL * 32;
  if (dtype == SKV_DTYPE_F32) {
    const float* p = static_cast<const float*>(base) + row * D + lane * EPL;
    if constexpr (EPL == 4) {
      float4 f = *reinterpret_cast<const float4*>(p);
      r.v[0] = f.x; r.v[1] = f.y; r.v[2] = f.z; r.v[3] = f.w;
    } else {
      float2 f = *reinterpret_cast<const float2*>(p);
      r.v[0] = f.x; r.v[1] = f.y;
    }
  } else {
    const __half* p = static_cast<const __half*>(base) + row * D + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; i += 2) {
      __half2 h = *reinterpret_cast<const __half2*>(p + i);
      r.v[i] = __low2float(h);
      r.v[i + 1] = __high2float(h);
    }
  }
  return r;
}

// ---- the quantiser's arithmetic without a division or a conversion per element ----------------------------
// The reference computes scale = amax / levels and q = clamp(round_half_even(x / scale)) in IEEE single
// precision.  A division is a subroutine of tens of instructions and every int<->float conversion goes
// through the quarter-rate pipe, which made the kernels that quantise issue-bound; both are avoided here
// without changing a bit of the result.
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// amax / levels, correctly rounded (levels = 2^(bits-1) - 1, at least 1): the product with the rounded
// reciprocal, corrected once through the exact remainder (two fused multiply-adds), is the correctly rounded
// quotient for every normal amax (checked over all 2^23 significands for 3, 7 and 127).
__device__ __forceinline__ float scale_of(float amax, int levels) {
  const float d = levels >= 127 ? 127.f : levels >= 7 ? 7.f : levels >= 3 ? 3.f : 1.f;
  if (!(amax >= 1e-30f && amax <= 1e30f)) return __fdiv_rn(amax, d);
  const float y = levels >= 127 ? (1.f / 127.f) : levels >= 7 ? (1.f / 7.f) : levels >= 3 ? (1.f / 3.f) : 1.f;
  const float q0 = __fmul_rn(amax, y);
  const float r = __fmaf_rn(-q0, d, amax);
  return __fmaf_rn(r, y, q0);
}

// q_i = clamp(rint(x_i / s), lo, hi) for N values that are NaN or satisfy |x_i| <= levels * s with
// s = max|x| / levels, levels <= 127 (what both callers pass: s comes from the same values).
// t = x * (1/s approx) differs from the rounded quotient by less than 7e-5 for |t| <= 256, so rint(t) is
// rint(x / s) unless t lies within that distance of a half-integer; rint itself is the add of 1.5 * 2^23,
// whose significand then holds the integer.  A lane that meets a near-tie, a NaN or a scale outside the
// normal range redoes its values with the division.
template <int N>
__device__ __forceinline__ void quantize_vals(const float (&x)[N], float s, int lo, int hi, int (&q)[N]) {
  constexpr float kMagic = 12582912.f;  // 1.5 * 2^23 = 0x4B400000
  bool exact = !(s >= 1e-30f && s <= 1e30f);
  if (!exact) {
    const float r = rcp_approx(s);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float t = __fmul_rn(x[i], r);
      const float m = __fadd_rn(t, kMagic);
      const float d = __fsub_rn(t, __fsub_rn(m, kMagic));
      exact |= !(fabsf(d) < 0.5f - 1.25e-4f);  // also true for a NaN
      q[i] = __float_as_int(m) - 0x4B400000;   // |t| <= levels * (1 + 2^-22): already inside [lo, hi]
    }
  }
  if (exact) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float v = rintf(__fdiv_rn(x[i], s));
      v = fminf(fmaxf(v, (float)lo), (float)hi);
      q[i] = (int)v;
    }
  }
}

// Quantise one row held across a warp.  Returns this lane's EPL codes and the row scale.
template <int EPL>
__device__ __forceinline__ float quantize_row(const RowVals<EPL>& x, int bits, int (&code)[EPL]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) amax = fmaxf(amax, fabsf(x.v[i]));
  amax = warp_max(amax);
  const int hi = (1 << (bits - 1)) - 1, lo = -(1 << (bits - 1));
  float scale = scale_of(amax, hi);
  if (scale == 0.f) scale = 1.f;
  quantize_vals<EPL>(x.v, scale, lo, hi, code);
  return scale;
}

// Packs the warp's row (EPL codes per lane, element index = lane*EPL + i) and
// stores row_bytes = 32*EPL*bits/8 bytes at dst (4-byte aligned).
template <int EPL>
__device__ __forceinline__ void pack_store_row(const int (&code)[EPL], int bits, uint8_t* dst, int lane) {
  const int wbits = bits * EPL;  // bits this lane contributes
  uint32_t mine = 0;
  if (bits == 8) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) mine |= ((uint32_t)code[i] & 0xffu) << (8 * i);
  } else {
    const int off = 1 << (bits - 1);
    const uint32_t fm = (1u << bits) - 1u;
#pragma unroll
    for (int i = 0; i < EPL; ++i) mine |= (((uint32_t)(code[i] + off)) & fm) << (bits * i);
  }
  // Neighbouring lanes' fields are joined by doubling (shuffle down, shift, or) until the lanes that
  // lead a group hold whole words; no step depends on a division by the field width.
  uint32_t* out = reinterpret_cast<uint32_t*>(dst);
  if (bits == 3) {
    // 3*EPL-bit fields -> 24-bit fields in every S-th lane; four of those make three words
    constexpr int S = 8 / EPL;
    int w = 3 * EPL;
#pragma unroll
    for (int st = 1; st < S; st <<= 1) {
      mine |= __shfl_down_sync(0xffffffffu, mine, st) << w;
      w <<= 1;
    }
    const uint32_t n = __shfl_down_sync(0xffffffffu, mine, S);  // the next 24-bit field
    const int r = (lane / S) & 3;
    const uint32_t word = r == 0 ? (mine | (n << 24)) : r == 1 ? ((mine >> 8) | (n << 16)) : ((mine >> 16) | (n << 8));
    if ((lane & (S - 1)) == 0 && r < 3) out[3 * (lane / (4 * S)) + r] = word;
  } else {
    // field widths 4, 8, 16 or 32 bits: log2(32 / wbits) doubling steps (the width is the same for the whole warp)
    int w = wbits, lg = 0;
#pragma unroll
    for (int st = 1; st < 8; st <<= 1) {
      if (w < 32) {
        mine |= __shfl_down_sync(0xffffffffu, mine, st) << w;
        w <<= 1;
        ++lg;
      }
    }
    if ((lane & ((1 << lg) - 1)) == 0) out[lane >> lg] = mine;
  }
}

// Reads this lane's EPL codes (element index = lane*EPL + i) out of a packed row.
template <int EPL>
__device__ __forceinline__ void unpack_row(const uint8_t* src, int bits, int lane, int (&code)[EPL]) {
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane * EPL + i;
    if (bits == 8) {
      code[i] = (int)(int8_t)src[e];
    } else {
      const int bitpos = e * bits, byte = bitpos >> 3, sh = bitpos & 7;
      uint32_t win = src[byte];
      if (sh + bits > 8) win |= (uint32_t)src[byte + 1] << 8;
      code[i] = (int)((win >> sh) & ((1u << bits) - 1u)) - (1 << (bits - 1));
    }
  }
}

}  // namespace skv
