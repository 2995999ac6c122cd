// Register-level unpack of packed K/V rows straight into mma.sync m16n8k16
// fragments, for the fused decode-attention kernel.
//
// Layout of one 16-key tile (one KV head) in shared memory: 16 packed K rows,
// row_bytes apart; same for V.  lane = 4*g + t.
//
//  scores = Q (A operand, 16 x D, rows 0..7 = query heads of the group, rows
//           8..15 = their fp16 residuals or zero)  x  K^T (B operand).
//     For n-tile n (keys 8n..8n+7) lane (g,t) supplies key 8n+g, and of that
//     key the D/4 consecutive elements [t*D/4, (t+1)*D/4) -- its "K slice".
//     The order in which a slice's elements are fed to the k-steps is free as
//     long as Q uses the same order, so each bit-width uses whichever order
//     its cheapest bit extraction produces (kelem<BITS>() records it and the
//     Q fragments are gathered through it).
//
//  out = P (A operand, 16 x 16 keys)  x  V (B operand, 16 keys x D).
//     For n-tile j lane (g,t) supplies column d = g*D/8 + j for the key pairs
//     (2t,2t+1) and (2t+8,2t+9); a half2 therefore pairs the SAME element of
//     two different rows, which a byte permute of the two rows' words gives
//     for free, in natural element order.
//
// Sub-byte fields become fp16 through the 0x6400 trick: OR a field that sits
// at bit p (p+width <= 10) of a 16-bit lane into the mantissa of 1024.0, then
// one HFMA2 computes (1024 + f*2^p) * 2^-p - (1024*2^-p + 2^(w-1)) = f - 2^(w-1)
// exactly.  The two lanes of a register may use different p.
#pragma once

#include "common.cuh"

namespace skv {

__host__ __device__ constexpr uint16_t f2h_exact(double v) {
  uint16_t sign = 0;
  if (v < 0) {
    sign = 0x8000;
    v = -v;
  }
  if (v == 0) return sign;
  int e = 0;
  while (v >= 2.0) {
    v /= 2;
    ++e;
  }
  while (v < 1.0) {
    v *= 2;
    --e;
  }
  int m = (int)((v - 1.0) * 1024.0 + 0.5);
  return (uint16_t)(sign | ((e + 15) << 10) | m);
}
__host__ __device__ constexpr uint32_t h2c(double lo, double hi) { return (uint32_t)f2h_exact(lo) | ((uint32_t)f2h_exact(hi) << 16); }
__host__ __device__ constexpr uint32_t h2c(double v) { return h2c(v, v); }

constexpr uint32_t kMagic = 0x64006400u;  // (1024.0, 1024.0)

// field at lane-bit p with `w` bits: fp16 = 1024 + f*2^p  ->  f - off
__host__ __device__ constexpr double fmul(int p) { return 1.0 / (double)(1 << p); }
__host__ __device__ constexpr double fadd(int p, int off) { return -(1024.0 / (double)(1 << p) + off); }

template <int P_LO, int P_HI, int W>
__device__ __forceinline__ uint32_t extract2(uint32_t x) {
  constexpr uint32_t fm = (1u << W) - 1u;
  constexpr uint32_t mask = (fm << P_LO) | ((fm << P_HI) << 16);
  constexpr int off = 1 << (W - 1);
  constexpr uint32_t mul = h2c(fmul(P_LO), fmul(P_HI));
  constexpr uint32_t add = h2c(fadd(P_LO, off), fadd(P_HI, off));
  uint32_t y = lop_and_or(x, mask, kMagic);
  if constexpr (P_LO == 0 && P_HI == 0) {
    return hadd2_bits(y, add);
  } else {
    return hfma2_bits(y, mul, add);
  }
}

// ---------------------------------------------------------------------------
// Element order of the K-slice unpackers: half2 number `o`, half `hl` (0 = low)
// holds slice element kelem<BITS>(o, hl).
// ---------------------------------------------------------------------------
template <int BITS>
__host__ __device__ constexpr int kelem(int o, int hl) {
  if (BITS == 8) return 2 * o + hl;
  if (BITS == 4) return 8 * (o / 4) + (o % 4) + 4 * hl;
  if (BITS == 2) return 16 * (o / 8) + (o % 8) + 8 * hl;
  // 3-bit: groups of 16 elements (6 bytes)
  constexpr int lo3[8] = {0, 1, 2, 6, 8, 9, 10, 7};
  constexpr int hi3[8] = {3, 4, 5, 14, 11, 12, 13, 15};
  return 16 * (o / 8) + (hl ? hi3[o % 8] : lo3[o % 8]);
}

// 8-bit: one word = 4 two's-complement codes -> 2 half2 (natural order)
__device__ __forceinline__ void k8_word(uint32_t w, uint32_t* o) {
  w ^= 0x80808080u;  // code + 128
  constexpr uint32_t add = h2c(-1152.0);
  o[0] = hadd2_bits(prmt(w, 0x64646464u, 0x4140), add);
  o[1] = hadd2_bits(prmt(w, 0x64646464u, 0x4342), add);
}
// 4-bit: one word = 8 nibbles n0..n7 -> (n0,n4) (n1,n5) (n2,n6) (n3,n7)
__device__ __forceinline__ void k4_word(uint32_t w, uint32_t* o) {
  o[0] = extract2<0, 0, 4>(w);
  o[1] = extract2<4, 4, 4>(w);
  uint32_t w8 = w >> 8;
  o[2] = extract2<0, 0, 4>(w8);
  o[3] = extract2<4, 4, 4>(w8);
}
// 2-bit: one word = 16 crumbs c0..c15 -> (c_i, c_{i+8}), i = 0..7
__device__ __forceinline__ void k2_word(uint32_t w, uint32_t* o) {
  o[0] = extract2<0, 0, 2>(w);
  o[1] = extract2<2, 2, 2>(w);
  o[2] = extract2<4, 4, 2>(w);
  o[3] = extract2<6, 6, 2>(w);
  o[4] = extract2<8, 8, 2>(w);
  uint32_t s = w >> 10;
  o[5] = extract2<0, 0, 2>(s);
  o[6] = extract2<2, 2, 2>(s);
  o[7] = extract2<4, 4, 2>(s);
}
// 3-bit: a 6-byte group B0..B5 = 16 fields.  The three selectors pick
//   X0 = [B0,B1 | B1,B2]  X1 = [B3,B4 | B4,B5]  X2 = [B2,B3 | B5,--]  out of (a,b).
template <uint32_t S0, uint32_t S1, uint32_t S2>
__device__ __forceinline__ void k3_group(uint32_t a, uint32_t b, uint32_t* o) {
  uint32_t x0 = prmt(a, b, S0), x1 = prmt(a, b, S1), x2 = prmt(a, b, S2);
  o[0] = extract2<0, 1, 3>(x0);  // (f0 , f3 )
  o[1] = extract2<3, 4, 3>(x0);  // (f1 , f4 )
  o[2] = extract2<6, 7, 3>(x0);  // (f2 , f5 )
  o[3] = extract2<2, 2, 3>(x2);  // (f6 , f14)
  o[4] = extract2<0, 1, 3>(x1);  // (f8 , f11)
  o[5] = extract2<3, 4, 3>(x1);  // (f9 , f12)
  o[6] = extract2<6, 7, 3>(x1);  // (f10, f13)
  o[7] = extract2<5, 5, 3>(x2);  // (f7 , f15)
}

// Loads lane (g,t)'s K slice of `row` and unpacks it to D/8 half2 registers.
template <int D, int BITS>
__device__ __forceinline__ void load_unpack_kslice(const uint8_t* tile, int row, int t, uint32_t* o) {
  constexpr int PD = D * BITS / 8;      // row bytes
  constexpr int SB = PD / 4;            // slice bytes
  const uint8_t* p = tile + row * PD + t * SB;
  if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < SB / 16; ++i) {
      uint4 v = *reinterpret_cast<const uint4*>(p + 16 * i);
      k8_word(v.x, o + 8 * i + 0);
      k8_word(v.y, o + 8 * i + 2);
      k8_word(v.z, o + 8 * i + 4);
      k8_word(v.w, o + 8 * i + 6);
    }
  } else if constexpr (BITS == 4) {
    if constexpr (SB == 16) {
      uint4 v = *reinterpret_cast<const uint4*>(p);
      k4_word(v.x, o + 0);
      k4_word(v.y, o + 4);
      k4_word(v.z, o + 8);
      k4_word(v.w, o + 12);
    } else {
      uint2 v = *reinterpret_cast<const uint2*>(p);
      k4_word(v.x, o + 0);
      k4_word(v.y, o + 4);
    }
  } else if constexpr (BITS == 2) {
    if constexpr (SB == 8) {
      uint2 v = *reinterpret_cast<const uint2*>(p);
      k2_word(v.x, o + 0);
      k2_word(v.y, o + 8);
    } else {
      uint32_t v = *reinterpret_cast<const uint32_t*>(p);
      k2_word(v, o + 0);
    }
  } else {  // 3-bit
    if constexpr (SB == 12) {
      const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
      uint32_t w0 = q[0], w1 = q[1], w2 = q[2];
      k3_group<0x2110, 0x5443, 0x5532>(w0, w1, o + 0);   // bytes 0..5
      k3_group<0x4332, 0x7665, 0x7754>(w1, w2, o + 8);   // bytes 6..11
    } else {  // 6 bytes at offset 6t: 4-byte aligned only for even t
      const int sh = (t & 1) * 16;
      const uint32_t* q = reinterpret_cast<const uint32_t*>(p - (t & 1) * 2);
      uint32_t w0 = q[0], w1 = q[1];
      uint32_t lo = __funnelshift_r(w0, w1, sh), hi = w1 >> sh;
      k3_group<0x2110, 0x5443, 0x5532>(lo, hi, o + 0);
    }
  }
}

// ---------------------------------------------------------------------------
// V: pairs of rows (A, B) -> half2 (A.e_j, B.e_j), natural order j
// ---------------------------------------------------------------------------
__device__ __forceinline__ void v8_pair_word(uint32_t a, uint32_t b, uint32_t* o) {
  constexpr uint32_t add = h2c(-1152.0);
  // (x & 0x00ff00ff) ^ 0x64806480 : magic exponent in, sign bit of the code flipped
  o[0] = hadd2_bits(lop_and_xor(prmt(a, b, 0x0400), 0x00ff00ffu, 0x64806480u), add);
  o[1] = hadd2_bits(lop_and_xor(prmt(a, b, 0x0501), 0x00ff00ffu, 0x64806480u), add);
  o[2] = hadd2_bits(lop_and_xor(prmt(a, b, 0x0602), 0x00ff00ffu, 0x64806480u), add);
  o[3] = hadd2_bits(lop_and_xor(prmt(a, b, 0x0703), 0x00ff00ffu, 0x64806480u), add);
}
// x = [A.b0, A.b1 | B.b0, B.b1]: four nibbles per lane
__device__ __forceinline__ void v4_pair_x(uint32_t x, uint32_t* o) {
  o[0] = extract2<0, 0, 4>(x);
  o[1] = extract2<4, 4, 4>(x);
  uint32_t s = x >> 8;
  o[2] = extract2<0, 0, 4>(s);
  o[3] = extract2<4, 4, 4>(s);
}
// x = [A.b0, A.b1 | B.b0, B.b1]: eight crumbs per lane
__device__ __forceinline__ void v2_pair_x(uint32_t x, uint32_t* o) {
  o[0] = extract2<0, 0, 2>(x);
  o[1] = extract2<2, 2, 2>(x);
  o[2] = extract2<4, 4, 2>(x);
  o[3] = extract2<6, 6, 2>(x);
  o[4] = extract2<8, 8, 2>(x);
  uint32_t s = x >> 10;
  o[5] = extract2<0, 0, 2>(s);
  o[6] = extract2<2, 2, 2>(s);
  o[7] = extract2<4, 4, 2>(s);
}
// a, b = [B0,B1,B2,--] of each row: eight 3-bit fields per row
__device__ __forceinline__ void v3_pair_half(uint32_t a, uint32_t b, uint32_t* o) {
  uint32_t x0 = prmt(a, b, 0x5410), x1 = prmt(a, b, 0x6521), x2 = prmt(a, b, 0x7632);
  o[0] = extract2<0, 0, 3>(x0);
  o[1] = extract2<3, 3, 3>(x0);
  o[2] = extract2<6, 6, 3>(x0);
  o[3] = extract2<1, 1, 3>(x1);
  o[4] = extract2<4, 4, 3>(x1);
  o[5] = extract2<7, 7, 3>(x1);
  o[6] = extract2<2, 2, 3>(x2);
  o[7] = extract2<5, 5, 3>(x2);
}

// Loads lane (g,t)'s V slices of rows rowA, rowA+1 and unpacks to D/8 half2.
template <int D, int BITS>
__device__ __forceinline__ void load_unpack_vpair(const uint8_t* tile, int rowA, int g, uint32_t* o) {
  constexpr int PD = D * BITS / 8;
  constexpr int SB = PD / 8;  // slice bytes
  const uint8_t* pa = tile + rowA * PD + g * SB;
  const uint8_t* pb = pa + PD;
  if constexpr (BITS == 8) {
    if constexpr (SB == 16) {
      uint4 a = *reinterpret_cast<const uint4*>(pa), b = *reinterpret_cast<const uint4*>(pb);
      v8_pair_word(a.x, b.x, o + 0);
      v8_pair_word(a.y, b.y, o + 4);
      v8_pair_word(a.z, b.z, o + 8);
      v8_pair_word(a.w, b.w, o + 12);
    } else {
      uint2 a = *reinterpret_cast<const uint2*>(pa), b = *reinterpret_cast<const uint2*>(pb);
      v8_pair_word(a.x, b.x, o + 0);
      v8_pair_word(a.y, b.y, o + 4);
    }
  } else if constexpr (BITS == 4) {
    if constexpr (SB == 8) {
      uint2 a = *reinterpret_cast<const uint2*>(pa), b = *reinterpret_cast<const uint2*>(pb);
      v4_pair_x(prmt(a.x, b.x, 0x5410), o + 0);
      v4_pair_x(prmt(a.x, b.x, 0x7632), o + 4);
      v4_pair_x(prmt(a.y, b.y, 0x5410), o + 8);
      v4_pair_x(prmt(a.y, b.y, 0x7632), o + 12);
    } else {
      uint32_t a = *reinterpret_cast<const uint32_t*>(pa), b = *reinterpret_cast<const uint32_t*>(pb);
      v4_pair_x(prmt(a, b, 0x5410), o + 0);
      v4_pair_x(prmt(a, b, 0x7632), o + 4);
    }
  } else if constexpr (BITS == 2) {
    if constexpr (SB == 4) {
      uint32_t a = *reinterpret_cast<const uint32_t*>(pa), b = *reinterpret_cast<const uint32_t*>(pb);
      v2_pair_x(prmt(a, b, 0x5410), o + 0);
      v2_pair_x(prmt(a, b, 0x7632), o + 8);
    } else {
      uint32_t a = *reinterpret_cast<const uint16_t*>(pa), b = *reinterpret_cast<const uint16_t*>(pb);
      v2_pair_x(a | (b << 16), o + 0);
    }
  } else {  // 3-bit
    if constexpr (SB == 6) {  // 6 bytes at offset 6g: aligned for even g
      const int sh = (g & 1) * 16;
      const uint32_t* qa = reinterpret_cast<const uint32_t*>(pa - (g & 1) * 2);
      const uint32_t* qb = reinterpret_cast<const uint32_t*>(pb - (g & 1) * 2);
      uint32_t a0 = qa[0], a1 = qa[1], b0 = qb[0], b1 = qb[1];
      uint32_t alo = __funnelshift_r(a0, a1, sh), ahi = a1 >> sh;
      uint32_t blo = __funnelshift_r(b0, b1, sh), bhi = b1 >> sh;
      v3_pair_half(alo, blo, o + 0);
      v3_pair_half(__funnelshift_r(alo, ahi, 24), __funnelshift_r(blo, bhi, 24), o + 8);
    } else {  // 3 bytes at offset 3g
      const int mis = (g * 3) & 3;
      const uint32_t* qa = reinterpret_cast<const uint32_t*>(pa - mis);
      const uint32_t* qb = reinterpret_cast<const uint32_t*>(pb - mis);
      uint32_t a = __funnelshift_r(qa[0], qa[1], mis * 8);
      uint32_t b = __funnelshift_r(qb[0], qb[1], mis * 8);
      v3_pair_half(a, b, o + 0);
    }
  }
}

// ---------------------------------------------------------------------------
// Query fragments for one bit-width.  qs: shared fp16 [16][D + QPAD]
// ---------------------------------------------------------------------------
constexpr int kQPad = 8;

template <int D, int BITS>
__device__ __forceinline__ void gather_q_frags(const __half* qs, int lane, uint32_t (&qa)[D / 16][4]) {
  const int g = lane >> 2, t = lane & 3;
  const unsigned short* r0 = reinterpret_cast<const unsigned short*>(qs) + g * (D + kQPad) + t * (D / 4);
  const unsigned short* r1 = r0 + 8 * (D + kQPad);
#pragma unroll
  for (int s = 0; s < D / 16; ++s) {
    const int e00 = kelem<BITS>(2 * s, 0), e01 = kelem<BITS>(2 * s, 1);
    const int e10 = kelem<BITS>(2 * s + 1, 0), e11 = kelem<BITS>(2 * s + 1, 1);
    qa[s][0] = (uint32_t)r0[e00] | ((uint32_t)r0[e01] << 16);
    qa[s][1] = (uint32_t)r1[e00] | ((uint32_t)r1[e01] << 16);
    qa[s][2] = (uint32_t)r0[e10] | ((uint32_t)r0[e11] << 16);
    qa[s][3] = (uint32_t)r1[e10] | ((uint32_t)r1[e11] << 16);
  }
}

// scores for one 16-key tile: s[n][0..1] = rows g of keys 8n+2t, 8n+2t+1; s[n][2..3] = rows g+8
template <int D, int BITS>
__device__ __forceinline__ void qk_tile(const uint8_t* ktile, int lane, const uint32_t (&qa)[D / 16][4],
                                        float (&s)[2][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint32_t kb0[D / 8], kb1[D / 8];
  load_unpack_kslice<D, BITS>(ktile, g, t, kb0);
  load_unpack_kslice<D, BITS>(ktile, g + 8, t, kb1);
#pragma unroll
  for (int i = 0; i < 4; ++i) s[0][i] = s[1][i] = 0.f;
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    mma_16816(s[0], qa[k], kb0[2 * k], kb0[2 * k + 1]);
    mma_16816(s[1], qa[k], kb1[2 * k], kb1[2 * k + 1]);
  }
}

// o[j][0..1] += rows g, columns d = (D/8)*(2t) + j and (D/8)*(2t+1) + j ; o[j][2..3] rows g+8
template <int D, int BITS>
__device__ __forceinline__ void pv_tile(const uint8_t* vtile, int lane, const uint32_t (&pa)[4],
                                        float (&o)[D / 8][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint32_t v0[D / 8], v1[D / 8];
  load_unpack_vpair<D, BITS>(vtile, 2 * t, g, v0);
  load_unpack_vpair<D, BITS>(vtile, 2 * t + 8, g, v1);
#pragma unroll
  for (int j = 0; j < D / 8; ++j) mma_16816(o[j], pa, v0[j], v1[j]);
}

}  // namespace skv
