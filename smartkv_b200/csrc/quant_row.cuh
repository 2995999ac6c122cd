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

// Quantise one row held across a warp.  Returns this lane's EPL codes and the row scale.
template <int EPL>
__device__ __forceinline__ float quantize_row(const RowVals<EPL>& x, int bits, int (&code)[EPL]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) amax = fmaxf(amax, fabsf(x.v[i]));
  amax = warp_max(amax);
  const int hi = (1 << (bits - 1)) - 1, lo = -(1 << (bits - 1));
  float scale = __fdiv_rn(amax, (float)(hi > 1 ? hi : 1));
  if (scale == 0.f) scale = 1.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    float q = rintf(__fdiv_rn(x.v[i], scale));
    q = fminf(fmaxf(q, (float)lo), (float)hi);
    code[i] = (int)q;
  }
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
  // output word `lane` covers row bits [32*lane, 32*lane+32): gather the lanes that overlap it
  const int nwords = wbits;  // 32 lanes * wbits bits / 32
  const int first = (32 * lane) / wbits;
  uint32_t word = 0;
  const int max_src = 32 / wbits + 2;
  for (int j = 0; j < max_src; ++j) {
    int src = first + j;
    uint32_t v = __shfl_sync(0xffffffffu, mine, src & 31);
    int pos = src * wbits - 32 * lane;  // bit position of that lane's field inside my word
    if (src < 32 && pos < 32 && pos + wbits > 0) word |= (pos >= 0) ? (v << pos) : (v >> (-pos));
  }
  if (lane < nwords) reinterpret_cast<uint32_t*>(dst)[lane] = word;
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
