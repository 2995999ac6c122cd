// Register-level unpack of packed K/V rows straight into mma.sync fragments, for the fused
// decode-attention kernel.
//
// One 16-key tile (one KV head) sits in shared memory as 16 packed K rows, row_bytes apart, and
// 16 packed V rows.  lane = 4*g + t.
//
//  S[8 heads x 16 keys] = Q (A operand, rows = heads)  x  K^T (B operand, two n-tiles of 8 keys)
//     2-, 4-, 8-bit keys and (head_dim 128) 3-bit keys: integer product, mma.sync.m16n8k32.s8.(u8|s8) on the stored
//     (offset-binary) codes.  The query row of a head is split into two radix-128 int8 limbs; rows
//     0..7 of the A operand hold limb 0 of the 8 heads, rows 8..15 limb 1, so one MMA yields both
//     partial products and the score is 128 * c[row g] + c[row g+8].  The constant that the offset
//     of the stored codes adds (2^(w-1) * sum of the limb) is folded into the accumulator's initial
//     value.  3-bit keys at head_dim 64: fp16 product, m16n8k16, rows 8..15 carry the fp16
//     residual of the query in the precise mode.
//     Lane (g,t) supplies, for the B operand, key g (and g+8 for the second n-tile) and of it a
//     "K slice" of D/4 elements.  The order in which a slice's elements are fed to the k-steps is
//     free as long as Q uses the same order, so each bit-width uses whichever order its cheapest bit
//     extraction produces (kelem<BITS>() / kelem_i8<BITS>() record it and the Q fragments are
//     gathered through it).
//     The accumulator of lane (g,t) holds head g, keys 2t, 2t+1 (and 2t+8, 2t+9): exactly the
//     B-fragment layout of the next product, so nothing is transposed or shuffled in between.
//
//  O^T[D x 8 heads] = V^T (A operand, D x 16 keys)  x  P^T (B operand, 16 keys x 8 heads)
//     For m-tile j lane (g,t) supplies rows d = g*D/8 + 2j and d+1 for the key pairs (2t,2t+1) and
//     (2t+8,2t+9); a half2 therefore pairs the SAME element of two different rows, which a byte
//     permute of the two rows' words gives for free, in natural element order.
//
// Sub-byte fields become fp16 through the 0x6400 trick: OR a field that sits at bit p
// (p+width <= 10) of a 16-bit lane into the mantissa of 1024.0, then one HFMA2 computes
// (1024 + f*2^p) * 2^-p - (1024*2^-p + 2^(w-1)) = f - 2^(w-1) exactly.  The two lanes of a
// register may use different p.
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

// Words a lane loads for its K slice (D/4 elements) and for its V slice of one row (D/8 elements).
template <int D, int BITS>
struct SliceWords {
  static constexpr int K = (D * BITS / 32 + 3) / 4;   // 128: 8,4,3,2   64: 4,2,2,1
  static constexpr int V = (BITS == 3) ? 2 : (D * BITS / 64 + 3) / 4;   // 128: 4,2,2,1   64: 2,1,2,1
};

// Loads lane (g,t)'s K slice of `row` as raw words (unpacked later, so the loads of a whole
// tile can be issued before any arithmetic).
template <int D, int BITS>
__device__ __forceinline__ void load_kslice(const uint8_t* tile, int row, int t, uint32_t (&w)[SliceWords<D, BITS>::K]) {
  constexpr int PD = D * BITS / 8;  // row bytes
  constexpr int SB = PD / 4;        // slice bytes
  const uint8_t* p = tile + row * PD + t * SB;
  if constexpr (SB % 16 == 0) {
#pragma unroll
    for (int i = 0; i < SB / 16; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(p + 16 * i);
      w[4 * i + 0] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
  } else if constexpr (SB == 8) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    w[0] = v.x; w[1] = v.y;
  } else if constexpr (SB == 4) {
    w[0] = *reinterpret_cast<const uint32_t*>(p);
  } else if constexpr (SB == 12) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
    w[0] = q[0]; w[1] = q[1]; w[2] = q[2];
  } else {  // 6 bytes at offset 6t: 4-byte aligned only for even t -> load from the aligned word below
    static_assert(SB == 6, "unexpected K slice size");
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p - (t & 1) * 2);
    w[0] = q[0]; w[1] = q[1];
  }
}

// Unpacks a raw K slice to D/8 half2 registers in the order kelem<BITS> records.
template <int D, int BITS>
__device__ __forceinline__ void unpack_kslice(const uint32_t (&w)[SliceWords<D, BITS>::K], int t, uint32_t* o) {
  constexpr int NW = SliceWords<D, BITS>::K;
  if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < NW; ++i) k8_word(w[i], o + 2 * i);
  } else if constexpr (BITS == 4) {
#pragma unroll
    for (int i = 0; i < NW; ++i) k4_word(w[i], o + 4 * i);
  } else if constexpr (BITS == 2) {
#pragma unroll
    for (int i = 0; i < NW; ++i) k2_word(w[i], o + 8 * i);
  } else if constexpr (D == 128) {
    k3_group<0x2110, 0x5443, 0x5532>(w[0], w[1], o + 0);  // bytes 0..5
    k3_group<0x4332, 0x7665, 0x7754>(w[1], w[2], o + 8);  // bytes 6..11
  } else {
    const int sh = (t & 1) * 16;
    const uint32_t lo = __funnelshift_r(w[0], w[1], sh), hi = w[1] >> sh;
    k3_group<0x2110, 0x5443, 0x5532>(lo, hi, o + 0);
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

// Loads lane (g,t)'s V slice of one row as raw words.
template <int D, int BITS>
__device__ __forceinline__ void load_vrow(const uint8_t* tile, int row, int g, uint32_t (&w)[SliceWords<D, BITS>::V]) {
  constexpr int PD = D * BITS / 8;
  constexpr int SB = PD / 8;  // slice bytes
  const uint8_t* p = tile + row * PD + g * SB;
  if constexpr (SB == 16) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if constexpr (SB == 8) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    w[0] = v.x; w[1] = v.y;
  } else if constexpr (SB == 4) {
    w[0] = *reinterpret_cast<const uint32_t*>(p);
  } else if constexpr (SB == 2) {
    w[0] = *reinterpret_cast<const uint16_t*>(p);
  } else if constexpr (SB == 6) {  // 6 bytes at offset 6g: aligned for even g
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p - (g & 1) * 2);
    w[0] = q[0]; w[1] = q[1];
  } else {  // 3 bytes at offset 3g
    static_assert(SB == 3, "unexpected V slice size");
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p - ((g * 3) & 3));
    w[0] = q[0]; w[1] = q[1];
  }
}

// Unpacks the raw V slices of rows A (key 2t or 2t+8) and B (the next key) to D/8 half2
// registers (A.e_j, B.e_j), natural element order j.
template <int D, int BITS>
__device__ __forceinline__ void unpack_vpair(const uint32_t (&a)[SliceWords<D, BITS>::V],
                                             const uint32_t (&b)[SliceWords<D, BITS>::V], int g, uint32_t* o) {
  constexpr int NW = SliceWords<D, BITS>::V;
  if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < NW; ++i) v8_pair_word(a[i], b[i], o + 4 * i);
  } else if constexpr (BITS == 4) {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      v4_pair_x(prmt(a[i], b[i], 0x5410), o + 8 * i);
      v4_pair_x(prmt(a[i], b[i], 0x7632), o + 8 * i + 4);
    }
  } else if constexpr (BITS == 2) {
    if constexpr (D == 128) {
      v2_pair_x(prmt(a[0], b[0], 0x5410), o + 0);
      v2_pair_x(prmt(a[0], b[0], 0x7632), o + 8);
    } else {
      v2_pair_x(a[0] | (b[0] << 16), o + 0);
    }
  } else if constexpr (D == 128) {
    const int sh = (g & 1) * 16;
    const uint32_t alo = __funnelshift_r(a[0], a[1], sh), ahi = a[1] >> sh;
    const uint32_t blo = __funnelshift_r(b[0], b[1], sh), bhi = b[1] >> sh;
    v3_pair_half(alo, blo, o + 0);
    v3_pair_half(__funnelshift_r(alo, ahi, 24), __funnelshift_r(blo, bhi, 24), o + 8);
  } else {
    const int sh = ((g * 3) & 3) * 8;
    v3_pair_half(__funnelshift_r(a[0], a[1], sh), __funnelshift_r(b[0], b[1], sh), o + 0);
  }
}

// ---------------------------------------------------------------------------
// Tile-level products.  lane = 4*g + t.
//
// Scores S[heads x keys] = Q (A operand) x K^T (B operand):
//   * 2/4/8-bit keys: int8 MMA m16n8k32.  A rows 0..7 = most significant int8 limb of the 8
//     heads, rows 8..15 = next limb (the query is split into radix-128 limbs); the B fragment of
//     n-tile n is key 8n+g, and its two registers are two consecutive words of that key's slice,
//     so 8-bit rows feed the tensor core straight from the shared-memory load.
//   * 3-bit keys: fp16 MMA m16n8k16, A rows 0..7 = fp16 query, rows 8..15 = fp16 residual.
//   The accumulator layout -- lane (g,t) holds head g, keys 2t,2t+1 (+8) -- is exactly the B
//   fragment layout P^T needs below, so probabilities go from registers to registers.
// Output O^T[D x heads] = V^T (A operand) x P^T (B operand), fp16 MMA.
// ---------------------------------------------------------------------------
constexpr int kQPad = 0;  // query rows are dense in shared memory

// Element order of the int8 path: k-step s, register r (0/1), byte j holds slice element
// kelem_i8<BITS>(s, r, j).
template <int BITS>
__host__ __device__ constexpr int kelem_i8(int s, int r, int j) {
  if (BITS == 8) return 8 * s + 4 * r + j;
  if (BITS == 4) return 8 * s + 2 * j + r;          // word s: even nibbles -> r = 0, odd -> r = 1
  if (BITS == 3) return (2 * s + r) + 8 * j;        // register 2s+r: field 2s+r of each of the four 24-bit groups
  return 16 * (s / 2) + 4 * j + 2 * (s % 2) + r;    // 2-bit: word s/2, shift index 2*(s%2)+r
}

// D(16x8,s32) += A(16x32, s8, row) * B(32x8, u8 or s8, col)
template <bool B_UNSIGNED>
__device__ __forceinline__ void mma_i8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (B_UNSIGNED) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Raw K slice -> D/16 int8x4 registers (two per k-step).
template <int D, int BITS>
__device__ __forceinline__ void unpack_kslice_i8(const uint32_t (&w)[SliceWords<D, BITS>::K], uint32_t* o) {
  constexpr int NW = SliceWords<D, BITS>::K;
  static_assert(BITS != 3 || D == 128, "3-bit rows of head_dim 64 use the fp16 path");
  if constexpr (BITS == 3) {
    // 32 fields of 3 bits in 12 bytes (four 24-bit groups).  Field i0 of every group sits at the same
    // offset inside its byte, 3 bytes apart, so one byte gather + shift + mask yields the register of
    // a field class (bytes = groups).  Classes 2 and 5 straddle a byte boundary: they are taken from the
    // slice shifted right by 6 bits, where they do not.
    constexpr uint32_t m = 0x07070707u;
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    const uint32_t g0 = prmt(prmt(w0, w1, 0x0630), w2, 0x5210);  // bytes 0, 3, 6, 9
    const uint32_t g1 = prmt(prmt(w0, w1, 0x0741), w2, 0x6210);  // bytes 1, 4, 7, 10
    const uint32_t g2 = prmt(prmt(w0, w1, 0x0052), w2, 0x7410);  // bytes 2, 5, 8, 11
    const uint32_t s0 = __funnelshift_r(w0, w1, 6), s1 = __funnelshift_r(w1, w2, 6), s2 = w2 >> 6;
    const uint32_t h0 = prmt(prmt(s0, s1, 0x0630), s2, 0x5210);
    const uint32_t h1 = prmt(prmt(s0, s1, 0x0741), s2, 0x6210);
    o[0] = g0 & m;
    o[1] = (g0 >> 3) & m;
    o[2] = h0 & m;
    o[3] = (g1 >> 1) & m;
    o[4] = (g1 >> 4) & m;
    o[5] = (h1 >> 1) & m;
    o[6] = (g2 >> 2) & m;
    o[7] = (g2 >> 5) & m;
  } else if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < NW; ++i) o[i] = w[i];
  } else if constexpr (BITS == 4) {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      o[2 * i] = w[i] & 0x0f0f0f0fu;
      o[2 * i + 1] = (w[i] >> 4) & 0x0f0f0f0fu;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      o[4 * i] = w[i] & 0x03030303u;
      o[4 * i + 1] = (w[i] >> 2) & 0x03030303u;
      o[4 * i + 2] = (w[i] >> 4) & 0x03030303u;
      o[4 * i + 3] = (w[i] >> 6) & 0x03030303u;
    }
  }
}

// A fragments of the int8 query: rows g <- limb_hi[head g], rows g+8 <- limb_lo[head g]
// (limb_lo may be null: those rows are zero).  limbs int8 [8][D] in shared memory.
template <int D, int BITS>
__device__ __forceinline__ void gather_qa_i8(const int8_t* limb_hi, const int8_t* limb_lo, int lane,
                                             uint32_t (&qa)[D / 32][4]) {
  const int g = lane >> 2, t = lane & 3;
  const uint8_t* rh = reinterpret_cast<const uint8_t*>(limb_hi) + g * D + t * (D / 4);
  const uint8_t* rl = limb_lo ? reinterpret_cast<const uint8_t*>(limb_lo) + g * D + t * (D / 4) : nullptr;
#pragma unroll
  for (int s = 0; s < D / 32; ++s) {
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      uint32_t vh = 0, vl = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        vh |= (uint32_t)rh[kelem_i8<BITS>(s, rr, j)] << (8 * j);
        if (rl) vl |= (uint32_t)rl[kelem_i8<BITS>(s, rr, j)] << (8 * j);
      }
      qa[s][2 * rr] = vh;
      qa[s][2 * rr + 1] = vl;
    }
  }
}

// A fragments of the fp16 query (3-bit keys): rows g <- qs row g, rows g+8 <- qs row g+8 when
// `with_residual`, else zero.  qs fp16 [8 or 16][D] in shared memory.
template <int D, int BITS>
__device__ __forceinline__ void gather_qa_f16(const __half* qs, bool with_residual, int lane,
                                              uint32_t (&qa)[D / 16][4]) {
  const int g = lane >> 2, t = lane & 3;
  const unsigned short* r0 = reinterpret_cast<const unsigned short*>(qs) + g * D + t * (D / 4);
  const unsigned short* r1 = r0 + 8 * D;
#pragma unroll
  for (int s = 0; s < D / 16; ++s) {
    const int e00 = kelem<BITS>(2 * s, 0), e01 = kelem<BITS>(2 * s, 1);
    const int e10 = kelem<BITS>(2 * s + 1, 0), e11 = kelem<BITS>(2 * s + 1, 1);
    qa[s][0] = (uint32_t)r0[e00] | ((uint32_t)r0[e01] << 16);
    qa[s][2] = (uint32_t)r0[e10] | ((uint32_t)r0[e11] << 16);
    qa[s][1] = with_residual ? ((uint32_t)r1[e00] | ((uint32_t)r1[e01] << 16)) : 0u;
    qa[s][3] = with_residual ? ((uint32_t)r1[e10] | ((uint32_t)r1[e11] << 16)) : 0u;
  }
}

// Integer scores of one n-tile (8 keys; this lane supplies the raw slice `k` of key 8n+g):
//   acc[0] = (limb_hi of head g, key 2t)  acc[1] = (limb_hi, key 2t+1)  acc[2], acc[3] = limb_lo rows
// acc is initialised by the caller.
template <int D, int BITS>
__device__ __forceinline__ void qk_ntile_i8(const uint32_t (&k)[SliceWords<D, BITS>::K],
                                            const uint32_t (&qa)[D / 32][4], int (&acc)[4]) {
  uint32_t b[D / 16];
  unpack_kslice_i8<D, BITS>(k, b);
#pragma unroll
  for (int s = 0; s < D / 32; ++s) mma_i8_16832<BITS != 8>(acc, qa[s], b[2 * s], b[2 * s + 1]);
}

// fp16 scores of one n-tile: acc[0], acc[1] = (head g, keys 2t, 2t+1) from the query rows,
// acc[2], acc[3] = the same from the residual rows.  Even / odd k-steps use two accumulators.
template <int D, int BITS>
__device__ __forceinline__ void qk_ntile_f16(const uint32_t (&k)[SliceWords<D, BITS>::K], int t,
                                             const uint32_t (&qa)[D / 16][4], float (&acc)[4]) {
  uint32_t kb[D / 8];
  unpack_kslice<D, BITS>(k, t, kb);
  float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < D / 16; ++s) {
    if (s & 1) mma_16816(a1, qa[s], kb[2 * s], kb[2 * s + 1]);
    else mma_16816(a0, qa[s], kb[2 * s], kb[2 * s + 1]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = a0[i] + a1[i];
}

// o[j][0] = (d = g*D/8 + 2j, head 2t)   o[j][1] = (same d, head 2t+1)
// o[j][2] = (d + 1,          head 2t)   o[j][3] = (d + 1,  head 2t+1)
// v0 / v1: unpacked V fragments of the key pairs (2t,2t+1) / (2t+8,2t+9);
// pb0/pb1: P^T fragments for those pairs, head g; pl0/pl1 their fp16 residuals.
template <int D, bool PRECISE>
__device__ __forceinline__ void pv_tile(const uint32_t (&v0)[D / 8], const uint32_t (&v1)[D / 8], uint32_t pb0,
                                        uint32_t pb1, uint32_t pl0, uint32_t pl1, float (&o)[D / 16][4]) {
#pragma unroll
  for (int j = 0; j < D / 16; ++j) {
    const uint32_t a[4] = {v0[2 * j], v0[2 * j + 1], v1[2 * j], v1[2 * j + 1]};
    mma_16816(o[j], a, pb0, pb1);
    if (PRECISE) mma_16816(o[j], a, pl0, pl1);
  }
}

}  // namespace skv
