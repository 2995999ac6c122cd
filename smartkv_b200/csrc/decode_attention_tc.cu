// Fused packed-KV decode attention on the 5th-generation tensor cores (tcgen05) of sm_100a, for
// head_dim 128, fp16 queries and GQA groups of up to 8 query heads (q_len == 1).
//
// The keys are the M operand.  A block is 128 keys of one bucket of one (sequence, KV head):
//
//   S[128 keys x 16]  = K[128 x 128] . Qlimbs^T     tcgen05.mma kind::i8, accumulators in tensor memory.
//                       K is the int8 code matrix, K-major, 128-byte rows in the 128-byte swizzle.  Rows of
//                       the 8-bit bucket are exactly that, so a tiled TMA load (cp.async.bulk.tensor, 3-D map
//                       over the arena, SWIZZLE_128B, no multicast) lands them ready for the MMA and no CUDA core
//                       ever touches an 8-bit code.  2/3/4-bit rows arrive packed (1-D bulk copies) and a
//                       warpgroup spreads their fields to bytes into the same tile.  The query rows are two
//                       radix-128 int8 limbs per head, stored once per run in the element order each width's
//                       unpacker produces.
//   softmax           one thread per key: tcgen05.ld of its row of S, scale by the key's K scale, block
//                       maximum per head (redux.sync + one exchange through shared memory), probabilities
//                       relative to the block maximum times the key's V scale (relative to the block's largest)
//                       as 24-bit fixed point in three unsigned byte limbs -> P[128 keys x 16|32] in shared memory.
//   O^T[128 d x 16|32] = V^T[128 x 128 keys] . P     kind::i8, V^T is the same kind of tile read MN-major, P is
//                       MN-major without swizzle.  One thread per output row d folds the three limbs and the
//                       block's scale into fp32 registers (the rescale of an online softmax happens there, never in
//                       tensor memory).
//
// Persistent CTAs (one per SM) walk the runs of the step's plan (attn_sched.cuh, 128-key tiles).  Warp roles:
//   producer      streams blocks into a ring of shared-memory slots (and asks L2 for the blocks after them),
//                 prepares the query limbs of the next run
//   score issuer  one thread issues the K.Q MMAs as tiles become ready
//   PV issuer     one thread issues the V.P MMAs as probabilities become ready; its commit frees the slot
//   warpgroups    take the blocks round-robin; each unpacks its narrow blocks, turns scores into probabilities
//                 and drains the P.V accumulators, software-pipelined over its own blocks
// so a single thread's MMA issue time and every MMA latency stay off the warpgroups' critical path.  All
// hand-offs are mbarriers; every wait is bounded (attn_params.cuh).  At the end of a run each warpgroup writes
// one partial (max, sum, out[128]) per query head; the combine step (post_attention.cuh) folds a segment's partials.
//
// Replaces smartkv/csrc/quantized_attention.cu:460-828 (per-bucket kernel, one CTA per head) and the host LSE
// combine in smartkv/kernels/__init__.py:350-371; numerics follow the CPU streaming path
// smartkv/core/fused_cpu.py:70-113 (dequantise, q.k/sqrt(d), online softmax).
#include <cstdio>
#include <mutex>

#include "attn_frag.cuh"
#include "attn_params.cuh"
#include "post_attention.cuh"
#include "tc05.cuh"

namespace skv {

constexpr int kTcKeys = 128;                         // keys per block
constexpr int kTcTile = 16384;                       // one int8 tile: 128 rows x 128 B
constexpr int kTcSlotBytes = 2 * kTcTile + 1024;     // K tile | V tile | 128 x (K scale, V scale)
constexpr int kTcQBufs = 2;                          // query ring (runs in flight)
constexpr int kTcPartialsPerRun = 4;                 // partial slots per run (one per warpgroup; unused ones are marked empty)
// (No L2 prefetch ahead of the copies: measured, each bulk prefetch costs the producer about 200 cycles of issue time,
// three per block, and the copies did not land any sooner.)
// Fixed-point unit of P: the largest probability-times-V-scale of a block maps to 2^24 - 256, so that no
// rounding in the chain can reach 2^24 (whose three low bytes would read as zero).
constexpr float kTcPOne = 16776960.f;


template <int GP>
struct TcCfg {
  static constexpr int WGS = GP <= 4 ? 4 : 3;              // warpgroups that consume blocks
  static constexpr int NS = GP <= 4 ? 6 : 5;               // ring slots
  static constexpr int PN = GP <= 4 ? 16 : 32;             // bytes of one P row = N of the PV MMA (3 limbs x GP, padded)
  static constexpr int PBYTES = kTcKeys * PN;              // the P buffer of a warpgroup
  static constexpr int SCOLS = 16;                         // N of the score MMA (2 limbs x GP, padded)
  static constexpr int WG_COLS = 2 * SCOLS + PN;           // tensor-memory columns of one warpgroup: S twice, O once
  static constexpr int TMEM_COLS = 256;                    // power of two >= WGS * WG_COLS
  static constexpr int QROWS = GP <= 4 ? 8 : 16;           // limb rows of one element order: GP high limbs, GP low limbs
  static constexpr int QSTRIDE = QROWS * 128;              // bytes between two element orders
  static constexpr int QBUF = 4 * QSTRIDE + (16 - QROWS) * 128;  // the MMA reads 16 rows whatever QROWS is
  static constexpr int THREADS = (WGS * 4 + 3) * 32;       // + producer, PV issuer, query warp
  static_assert(WGS * WG_COLS <= TMEM_COLS, "tensor memory budget");
};

struct TcQMeta {
  float qs[8];   // limb step of head g times 1/sqrt(d) * log2(e)
  int sumA[8];   // 128 * sum(limb 0) + sum(limb 1): what the offset of unsigned codes adds per unit of offset
};

template <int GP>
struct TcMeta {
  uint64_t full[8], empty[8];
  uint64_t qfull[kTcQBufs], qempty[kTcQBufs];
  uint64_t sbar[4][2], ubar[4], pready[4], obar[4];
  uint64_t drain[2];
  uint64_t q0bar;                  // the first run's query heads, prepared by the consumer warps (one arrival per head)
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) uint32_t red[4][4][12];  // per warpgroup and warp: GP block maxima (order keys) + the largest V scale
  TcQMeta q[kTcQBufs];
};

template <int GP>
constexpr size_t tc_smem_bytes() {
  return (size_t)TcCfg<GP>::NS * kTcSlotBytes + (size_t)kTcQBufs * TcCfg<GP>::QBUF + (size_t)TcCfg<GP>::WGS * TcCfg<GP>::PBYTES +
         (size_t)TcCfg<GP>::WGS * GP * 128 * sizeof(float) + sizeof(TcMeta<GP>);
}

// ---- element order of the unpacked tiles ----------------------------------------------------------
// Byte position i of an unpacked row holds element tc_perm(bucket, i) of the stored row; the order is
// whatever the cheapest field extraction of that width yields.  The query limbs are stored in the same order
// (a dot product does not care) and the output rows are put back in order once per run.
__host__ __device__ constexpr int tc_perm(int bucket, int i) {
  return bucket == 0   ? (i & ~15) + 8 * ((i >> 3) & 1) + 2 * (i & 3) + ((i >> 2) & 1)  // 2-bit: word k of 4, byte b -> 8(k/2) + 2b + k%2
         : bucket == 1 ? (i & ~31) + 8 * (i & 3) + ((i >> 2) & 7)    // 3-bit: field class f, group g -> 8g + f
         : bucket == 2 ? (i & ~7) + 2 * (i & 3) + ((i >> 2) & 1)     // 4-bit: word s, low/high nibble e, byte j -> 8s + 2j + e
                       : i;                                          // 8-bit: as stored
}
__host__ __device__ constexpr int tc_perm_inv(int bucket, int d) {
  return bucket == 0   ? (d & ~15) + 8 * ((d >> 3) & 1) + 4 * (d & 1) + ((d >> 1) & 3)
         : bucket == 1 ? (d & ~31) + 4 * (d & 7) + ((d >> 3) & 3)
         : bucket == 2 ? (d & ~7) + 4 * (d & 1) + ((d >> 1) & 3)
                       : d;
}
// byte offset of (row, byte position) inside a 128-byte-swizzled tile whose base is 1024-byte aligned
__host__ __device__ constexpr int tc_swz(int row, int pos) { return row * 128 + ((((pos >> 4) ^ (row & 7))) << 4) + (pos & 15); }

// Which operands are signed bytes after the unpack.  V tiles always are (so that P.V needs no offset term);
// K tiles of the 3- and 4-bit buckets keep the stored offset-binary code, whose share of the score,
// offset * sum(query limbs), is a per-head constant.
__host__ __device__ constexpr int tc_k_signed(int bucket) { return bucket == 0 || bucket == 3; }
__host__ __device__ constexpr int tc_k_offset(int bucket) { return bucket == 1 ? 4 : bucket == 2 ? 8 : 0; }

// ---- unpack: packed rows of a narrow bucket -> int8 tile -------------------------------------------
// All loads of the warpgroup complete before the first store (the tiles overlay the packed bytes).
// `wt` = thread index inside the warpgroup, `bar` = the warpgroup's named barrier.
__device__ __forceinline__ void tc_store_chunk(uint8_t* tile, int row, int oc, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  *reinterpret_cast<uint4*>(tile + row * 128 + ((oc ^ (row & 7)) << 4)) = make_uint4(a, b, c, d);
}
// bytes u (0 <= u < 128) -> signed bytes u - off, four at a time
__device__ __forceinline__ uint32_t tc_sub4(uint32_t x_or_80, uint32_t off4) { return (x_or_80 - off4) ^ 0x80808080u; }

// The K tile is finished before the V rows are fetched (two barriers, half the registers): the K tile
// [0, 16 KB) never reaches the packed V rows, which start at 16 KB.

// 2-bit: 128 rows x 32 B = 256 chunks of 16 B per tile; thread wt takes chunks wt and wt + 128.
// Four crumbs at a time go through a byte permute used as a look-up table (0,1,2,3 -> -2,-1,0,1).
__device__ __forceinline__ void tc_unpack2(uint8_t* slot, int wt, int bar) {
  constexpr uint32_t lut = 0x0100fffeu;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    uint8_t* tile = slot + which * kTcTile;
    uint4 in[2];
#pragma unroll
    for (int n = 0; n < 2; ++n) in[n] = *reinterpret_cast<const uint4*>(tile + (wt + 128 * n) * 16);
    named_bar_sync(bar, 128);
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int c = wt + 128 * n, row = c >> 1, hf = c & 1;
      const uint32_t w[4] = {in[n].x, in[n].y, in[n].z, in[n].w};
#pragma unroll
      for (int s = 0; s < 4; ++s)
        tc_store_chunk(tile, row, 4 * hf + s, prmt(lut, 0u, w[s] & 0x3333u), prmt(lut, 0u, (w[s] >> 2) & 0x3333u),
                       prmt(lut, 0u, (w[s] >> 16) & 0x3333u), prmt(lut, 0u, (w[s] >> 18) & 0x3333u));
    }
  }
}

// 4-bit: 128 rows x 64 B = 512 chunks per tile; thread wt takes chunks wt + 128 n, n = 0..3.
__device__ __forceinline__ void tc_unpack4(uint8_t* slot, int wt, int bar) {
  constexpr uint32_t m = 0x0f0f0f0fu, hi = 0x80808080u, off = 0x08080808u;
  {
    uint4 in[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) in[n] = *reinterpret_cast<const uint4*>(slot + (wt + 128 * n) * 16);
    named_bar_sync(bar, 128);
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int c = wt + 128 * n, row = c >> 2, q = c & 3;
      tc_store_chunk(slot, row, 2 * q, in[n].x & m, (in[n].x >> 4) & m, in[n].y & m, (in[n].y >> 4) & m);
      tc_store_chunk(slot, row, 2 * q + 1, in[n].z & m, (in[n].z >> 4) & m, in[n].w & m, (in[n].w >> 4) & m);
    }
  }
  {
    uint8_t* tile = slot + kTcTile;
    uint4 in[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) in[n] = *reinterpret_cast<const uint4*>(tile + (wt + 128 * n) * 16);
    named_bar_sync(bar, 128);
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int c = wt + 128 * n, row = c >> 2, q = c & 3;
      tc_store_chunk(tile, row, 2 * q, tc_sub4(lop_and_or(in[n].x, m, hi), off), tc_sub4(lop_and_or(in[n].x >> 4, m, hi), off),
                     tc_sub4(lop_and_or(in[n].y, m, hi), off), tc_sub4(lop_and_or(in[n].y >> 4, m, hi), off));
      tc_store_chunk(tile, row, 2 * q + 1, tc_sub4(lop_and_or(in[n].z, m, hi), off), tc_sub4(lop_and_or(in[n].z >> 4, m, hi), off),
                     tc_sub4(lop_and_or(in[n].w, m, hi), off), tc_sub4(lop_and_or(in[n].w >> 4, m, hi), off));
    }
  }
}

// 3-bit: a row is 48 B = four 12-byte groups of 32 fields; thread wt takes row wt.
__device__ __forceinline__ void tc_unpack3(uint8_t* slot, int wt, int bar) {
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    uint8_t* tile = slot + which * kTcTile;
    uint32_t in[12];
#pragma unroll
    for (int n = 0; n < 3; ++n) {
      const uint4 a = *reinterpret_cast<const uint4*>(tile + wt * 48 + 16 * n);
      in[4 * n] = a.x; in[4 * n + 1] = a.y; in[4 * n + 2] = a.z; in[4 * n + 3] = a.w;
    }
    named_bar_sync(bar, 128);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const uint32_t w[3] = {in[3 * a], in[3 * a + 1], in[3 * a + 2]};
      uint32_t o[8];
      unpack_kslice_i8<128, 3>(w, o);
      if (which == 1) {  // V: signed codes
        constexpr uint32_t hi = 0x80808080u, off = 0x04040404u;
#pragma unroll
        for (int f = 0; f < 8; ++f) o[f] = tc_sub4(o[f] | hi, off);
      }
      tc_store_chunk(tile, wt, 2 * a, o[0], o[1], o[2], o[3]);
      tc_store_chunk(tile, wt, 2 * a + 1, o[4], o[5], o[6], o[7]);
    }
  }
}

// ---- block cursor: the blocks of a run in the order every role follows -------------------------------
// (element selection by compare chains: a dynamically indexed copy of the descriptor would live in local memory)
__device__ __forceinline__ int tc_sel4(const int (&a)[kNumBuckets], int i) {
  return i == 0 ? a[0] : i == 1 ? a[1] : i == 2 ? a[2] : a[3];
}
// The blocks of a run come in an order that interleaves the 8-bit bucket with the narrow ones in proportion to
// their block counts: 8-bit blocks cost the warpgroups little and the memory system a lot, narrow blocks the other
// way round, so mixing them keeps both busy all the time.  Block i of a run is an 8-bit block iff
// floor((i+1) * n8 / total) > floor(i * n8 / total); inside the narrow stream the buckets follow one another
// (2-, 3-, 4-bit).  A closed form, so that every role finds block i by itself with one integer division.
struct TcRun {
  int n0, n01, n8, total;   // narrow blocks of bucket 0, of buckets 0+1; 8-bit blocks; all blocks
  int ka0, ka1, ka2, ka3;   // first 128-key tile of every bucket in this run
  int c0, c1, c2, c3;       // live keys per bucket of the sequence
};
__device__ __forceinline__ TcRun tc_run(const RunDesc& d) {
  TcRun r;
  r.n0 = d.kb[0] - d.ka[0];
  r.n01 = r.n0 + (d.kb[1] - d.ka[1]);
  r.n8 = d.kb[3] - d.ka[3];
  r.total = r.n01 + (d.kb[2] - d.ka[2]) + r.n8;
  r.ka0 = d.ka[0]; r.ka1 = d.ka[1]; r.ka2 = d.ka[2]; r.ka3 = d.ka[3];
  r.c0 = d.cnt[0]; r.c1 = d.cnt[1]; r.c2 = d.cnt[2]; r.c3 = d.cnt[3];
  return r;
}
// block i of the run -> bucket, first key, number of keys
__device__ __forceinline__ void tc_block(const TcRun& r, int i, int& ci, int& key0, int& nkeys) {
  const unsigned prod = (unsigned)i * (unsigned)r.n8;
  const unsigned q = prod / (unsigned)r.total;          // 8-bit blocks before block i
  const unsigned rem = prod - q * (unsigned)r.total;
  int t, cnt;
  if (rem + (unsigned)r.n8 >= (unsigned)r.total) {
    ci = 3; t = r.ka3 + (int)q; cnt = r.c3;
  } else {
    const int n = i - (int)q;
    if (n < r.n0) { ci = 0; t = r.ka0 + n; cnt = r.c0; }
    else if (n < r.n01) { ci = 1; t = r.ka1 + (n - r.n0); cnt = r.c1; }
    else { ci = 2; t = r.ka2 + (n - r.n01); cnt = r.c2; }
  }
  key0 = t * kTcKeys;
  nkeys = (cnt - key0) < kTcKeys ? (cnt - key0) : kTcKeys;
}

// Bounded waits of the tensor-memory kernel.  tc_wait: the thread is suspended inside mbarrier.try_wait (a loop of
// test_wait polls by the sixteen consumer warps measured slower: it crowds the issue slots and the barrier words); the
// number of resumptions is limited, so the wait always ends.  tc_spin: back-to-back polls, for the single-thread roles
// whose reaction time every block waits for.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* err, unsigned polls) {
  const unsigned limit = (polls >> 4) + 16;  // a suspended try_wait lasts far longer than a 50 ns poll
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(err, 1);
  return false;
}

__device__ __forceinline__ bool tc_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* err, unsigned polls) {
  for (unsigned i = 0; i < polls; ++i) {  // a poll is a few tens of cycles: at least as long as `polls` sleeping polls
    if (mbar_test_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(err, 1);
  return false;
}

// ---- query limbs of a run, in the four element orders (one warp) ---------------------------------------------
// One warp, one query head: the two int8 limbs of every element, written in the four element orders.
template <int GP>
__device__ __forceinline__ void tc_prep_query_head(uint8_t* qbuf, TcQMeta& meta, const AttnParams& p, int seq, int head, int G,
                                                   int h, int lane) {
  constexpr int QSTRIDE = TcCfg<GP>::QSTRIDE;
  const long long q_off = ((long long)seq * p.num_q_heads + (long long)head * G + h) * 128;
  const __half2* src = reinterpret_cast<const __half2*>(static_cast<const __half*>(p.query) + q_off + lane * 4);
  const float2 a = __half22float2(src[0]), b = __half22float2(src[1]);
  const float q[4] = {a.x, a.y, b.x, b.y};
  float amax = fmaxf(fmaxf(fabsf(q[0]), fabsf(q[1])), fmaxf(fabsf(q[2]), fabsf(q[3])));
  amax = warp_max(amax);
  constexpr float range = 127.f * 128.f;
  const float step = amax > 0.f ? amax / range : 1.f;
  const float inv = 1.f / step;
  int s0 = 0, s1 = 0;
  uint8_t* row_hi = qbuf + h * 128;
  uint8_t* row_lo = qbuf + (GP + h) * 128;
  const int xh = h & 7, xl = (GP + h) & 7;  // swizzle of the two rows
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int d = lane * 4 + e;
    const float rem = fminf(fmaxf(rintf(q[e] * inv), -range), range);
    const float hi = rintf(rem * (1.f / 128.f));
    const int lo = (int)(rem - hi * 128.f);  // in [-64, 64]
    s0 += (int)hi;
    s1 += lo;
#pragma unroll
    for (int c = 0; c < kNumBuckets; ++c) {
      const int pos = tc_perm_inv(c, d);
      row_hi[c * QSTRIDE + ((((pos >> 4) ^ xh)) << 4) + (pos & 15)] = (uint8_t)(int8_t)(int)hi;
      row_lo[c * QSTRIDE + ((((pos >> 4) ^ xl)) << 4) + (pos & 15)] = (uint8_t)(int8_t)lo;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    s0 += __shfl_xor_sync(0xffffffffu, s0, off);
    s1 += __shfl_xor_sync(0xffffffffu, s1, off);
  }
  if (lane == 0) {
    meta.qs[h] = step * p.scale_log2;
    meta.sumA[h] = 128 * s0 + s1;
  }
}

template <int GP>
__global__ void __launch_bounds__(TcCfg<GP>::THREADS, 1)
    decode_attn_tc_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  using Cfg = TcCfg<GP>;
  constexpr int NS = Cfg::NS, PN = Cfg::PN, WGS = Cfg::WGS;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base (it is: the window starts at 0)
    if (threadIdx.x == 0) atomicExch(p.err, 5);
    return;
  }
  uint8_t* slots = smem;                                        // [NS][kTcSlotBytes]
  uint8_t* qbufs = slots + (size_t)NS * kTcSlotBytes;           // [kTcQBufs][QBUF]
  uint8_t* pbufs = qbufs + (size_t)kTcQBufs * Cfg::QBUF;        // [WGS][PBYTES]
  float* obufs = reinterpret_cast<float*>(pbufs + (size_t)WGS * Cfg::PBYTES);   // [WGS][GP][128] output accumulators
  TcMeta<GP>& mt = *reinterpret_cast<TcMeta<GP>*>(obufs + (size_t)WGS * GP * 128);
  const StoreGeom& g = p.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.group, Hkv = g.num_kv_heads;
  volatile int* abort_flag = &mt.abort_flag;

  {  // limb rows of heads that do not exist stay zero
    uint32_t* z = reinterpret_cast<uint32_t*>(qbufs);
    for (int i = tid; i < kTcQBufs * Cfg::QBUF / 4; i += Cfg::THREADS) z[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&mt.full[s], 1);
      mbar_init(&mt.empty[s], 1);
    }
    for (int s = 0; s < kTcQBufs; ++s) {
      mbar_init(&mt.qfull[s], 1);
      mbar_init(&mt.qempty[s], WGS);
    }
    for (int w = 0; w < WGS; ++w) {
      mbar_init(&mt.sbar[w][0], 1);
      mbar_init(&mt.sbar[w][1], 1);
      mbar_init(&mt.ubar[w], 4);    // one arrival per warp: the warpgroup's narrow tile is unpacked
      mbar_init(&mt.pready[w], 4);  // one arrival per warp: the warpgroup's P rows are written
      mbar_init(&mt.obar[w], 1);
    }
    mbar_init(&mt.drain[1], 1);
    mbar_init(&mt.q0bar, (uint32_t)G);
    mt.abort_flag = 0;
    for (int q = 0; q < kTcQBufs; ++q)
      for (int h = 0; h < 8; ++h) {
        mt.q[q].qs[h] = 0.f;
        mt.q[q].sumA[h] = 0;
      }
  }
  mbar_fence_init();
  if (warp == 0) tmem_alloc(&mt.tmem_base, Cfg::TMEM_COLS);
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = mt.tmem_base;

  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.num_ctas, g.num_seqs * Hkv);
  const int run_begin = pv.cta_begin[blockIdx.x], run_end = pv.cta_begin[blockIdx.x + 1];
  // never below 2^20 polls: a shorter limit could run out while this CTA's own copies and MMAs are still in flight
  const unsigned polls = p.wait_polls < (1u << 20) ? (1u << 20) : p.wait_polls;

  if (warp < G && run_begin < run_end) {  // warps 0..G-1 are consumer warps (G <= 8 < WGS * 4)
    const RunDesc d0 = pv.first[blockIdx.x];
    tc_prep_query_head<GP>(qbufs, mt.q[0], p, d0.seq, d0.head, G, warp, lane);
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(&mt.q0bar);
  }

  if (warp == WGS * 4) {
    // ================================ producer warp ================================
    int gi = 0;
    bool ok = run_begin < run_end;
    const uint64_t stream_policy = l2_evict_first_policy();  // the cache is read once per step
    for (int r = run_begin; ok && r < run_end; ++r) {
      const RunDesc d = r == run_begin ? pv.first[blockIdx.x] : pv.runs[r];
      const TcRun run = tc_run(d);
      const uint8_t* arena = arena_ptr(g, p.store, p.layer, d.seq);
      for (int i = 0; ok && i < run.total; ++i, ++gi) {
        const int slot = gi % NS;
        ok = tc_wait(&mt.empty[slot], ((gi / NS) & 1) ^ 1u, abort_flag, p.err, polls);
        if (!ok) break;
        if (lane == 0) {
          int ci, key0, nkeys;
          tc_block(run, i, ci, key0, nkeys);
          const int n16 = (nkeys + 15) & ~15;
          uint8_t* sb = slots + (size_t)slot * kTcSlotBytes;
          const long long row = (long long)d.head * g.cap[ci] + key0;
          const uint32_t sbytes = (uint32_t)(n16 * 8);
          // no proxy fence here: whoever touched the slot through the generic proxy fenced before the hand-off chain
          // (unpack -> score MMA, P -> PV MMA) whose completion freed the slot
          if (ci == 3) {
            mbar_expect_tx(&mt.full[slot], 2 * kTcTile + sbytes);
            tma_load_3d(sb, &kmap, 0, (int)row, p.layer * g.num_seqs + d.seq, &mt.full[slot], stream_policy);
            tma_load_3d(sb + kTcTile, &vmap, 0, (int)row, p.layer * g.num_seqs + d.seq, &mt.full[slot], stream_policy);
          } else {
            const int pd = g.row_bytes[ci];
            const uint32_t kbytes = (uint32_t)(n16 * pd);
            mbar_expect_tx(&mt.full[slot], 2 * kbytes + sbytes);
            bulk_g2s_hint(sb, arena + g.k_off[ci] + row * pd, kbytes, &mt.full[slot], stream_policy);
            bulk_g2s_hint(sb + kTcTile, arena + g.v_off[ci] + row * pd, kbytes, &mt.full[slot], stream_policy);
          }
          bulk_g2s_hint(sb + 2 * kTcTile, arena + g.sc_off[ci] + row * 8, sbytes, &mt.full[slot], stream_policy);
        }
      }
    }
  } else if (warp == WGS * 4 + 2) {
    // ================================ query warp ================================
    // Publishes the query limbs of every run one run ahead of its use.  The first run's heads were prepared by the
    // consumer warps, one head each (they have nothing else to do while the first bytes are in flight).
    int qi = 0;
    uint32_t qepar = 1;  // a fresh barrier passes a wait on parity 1: every slot starts empty
    bool ok = true;
    for (int r = run_begin; ok && r < run_end; ++r) {
      ok = tc_wait(&mt.qempty[qi], qepar, abort_flag, p.err, polls);
      if (!ok) break;
      if (r == run_begin) {
        ok = tc_wait(&mt.q0bar, 0, abort_flag, p.err, polls);
      } else {
        const RunDesc d = pv.runs[r];
#pragma unroll 1
        for (int h = 0; h < G; ++h) tc_prep_query_head<GP>(qbufs + (size_t)qi * Cfg::QBUF, mt.q[qi], p, d.seq, d.head, G, h, lane);
        fence_proxy_async();  // the MMA reads the limb rows through the async proxy
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&mt.qfull[qi]);
      if (++qi == kTcQBufs) {
        qi = 0;
        qepar ^= 1u;
      }
    }
  } else if (warp == WGS * 4 + 1) {
    // ================================ PV issuer ================================
    if (lane == 0) {
      int i = 0;
      bool ok = true;
      const uint32_t idesc = idesc_i8(1, 0, 1, 1, 128, PN);
      for (int r = run_begin; ok && r < run_end; ++r) {
        const RunDesc d = r == run_begin ? pv.first[blockIdx.x] : pv.runs[r];
        const int nblocks = tc_run(d).total;
        for (int bi = 0; ok && bi < nblocks; ++bi, ++i) {
          const int w = i % WGS, j = i / WGS, slot = i % NS;
          ok = tc_wait(&mt.pready[w], j & 1, abort_flag, p.err, polls);
          if (!ok) break;
          tc_fence_after();
          const uint32_t va = smem_u32(slots + (size_t)slot * kTcSlotBytes + kTcTile), pa = smem_u32(pbufs + (size_t)w * Cfg::PBYTES);
          const uint32_t dcol = tmem_base + (uint32_t)(w * Cfg::WG_COLS + 2 * Cfg::SCOLS);
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4)
            mma_i8_ss(dcol, smem_desc(va + 4096 * s4, 64, 64, 2), smem_desc(pa + 512 * s4, 8, kTcKeys, 0), idesc, s4 > 0);
          mma_commit(&mt.obar[w]);
          mma_commit(&mt.empty[slot]);  // the slot goes back to the producer when the tile has been read
        }
      }
      mma_commit(&mt.drain[1]);
      tc_wait(&mt.drain[1], 0, abort_flag, p.err, polls);
    }
    __syncwarp();
  } else {
    // ================================== consumer warpgroups ==================================
    const int wg = warp >> 2, wt = tid & 127, wq = warp & 3;  // wq: this warp's lane quarter of tensor memory
    const int bar = 1 + wg;
    const uint32_t tm_wg = tmem_base + (uint32_t)(wg * Cfg::WG_COLS) + ((uint32_t)(wq * 32) << 16);
    uint8_t* pbuf = pbufs + (size_t)wg * Cfg::PBYTES;
    int gi = 0, qi = 0;
    uint32_t qfpar = 0, unpacked = 0;  // unpacked: narrow blocks of this warpgroup so far (phase of its unpack barrier)
    bool aborted = false;

    struct Blk {
      int ci, key0, nkeys, slot, jj;
      uint32_t fpar;
      bool valid;
    };

    for (int r = run_begin; r < run_end; ++r) {
      const RunDesc d = r == run_begin ? pv.first[blockIdx.x] : pv.runs[r];
      if (!aborted && !tc_wait(&mt.qfull[qi], qfpar, abort_flag, p.err, polls)) aborted = true;
      const TcQMeta& qm = mt.q[qi];  // limb steps and limb sums of the run's query heads
      const int b = d.seq, hkv = d.head;
      // Online-softmax state.  The output accumulators live in shared memory, one row of 128 per head: thread wt
      // owns, for a block of bucket c, the output row tc_perm(c, wt) (the element order of that bucket's V tile), so
      // the rows of all buckets add up in natural order without a reshuffle, and no register holds them.
      float m_run[GP], l_run[GP];
      float* oacc = obufs + (size_t)wg * GP * 128;
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
        oacc[h * 128 + wt] = 0.f;
      }
      named_bar_sync(bar, 128);
      float* lbase = nullptr;  // logits row of head 0 of this group
      if (p.logits != nullptr) lbase = p.logits + ((long long)b * p.num_q_heads + hkv * G) * g.slots;

      const TcRun run = tc_run(d);
      const int gi_run = gi;                                   // global index of the run's first block
      int bi = (wg - gi_run % WGS + WGS) % WGS;                // this warpgroup's first block of the run
      auto next_mine = [&]() -> Blk {
        Blk k{};
        k.valid = bi < run.total;
        if (k.valid) {
          tc_block(run, bi, k.ci, k.key0, k.nkeys);
          const int gb = gi_run + bi;
          k.slot = gb % NS;
          k.fpar = (gb / NS) & 1;
          k.jj = gb / WGS;
          bi += WGS;
        }
        return k;
      };

      // ---- unpack: narrow rows spread to bytes, tile handed to the score issuer ----
      auto phase_u = [&](const Blk& k) {
        uint8_t* sb = slots + (size_t)k.slot * kTcSlotBytes;
        if (k.ci != 3) {  // 8-bit rows are MMA operands as they land
          if (!aborted && !tc_wait(&mt.full[k.slot], k.fpar, abort_flag, p.err, polls)) aborted = true;
          if (k.ci == 0) tc_unpack2(sb, wt, bar);
          else if (k.ci == 1) tc_unpack3(sb, wt, bar);
          else tc_unpack4(sb, wt, bar);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&mt.ubar[wg]);
        }
        // The warpgroup's first thread issues the score MMA of its own block (an issuer shared by the warpgroups
        // would have to take the blocks in order, and a block whose tile is ready would wait behind one whose unpack
        // is not); the other warps go on to the previous block's epilogue meanwhile.
        if (wt == 0) {
          if (k.ci == 3) {
            if (!aborted && !tc_wait(&mt.full[k.slot], k.fpar, abort_flag, p.err, polls)) aborted = true;
          } else {
            if (!aborted && !tc_wait(&mt.ubar[wg], unpacked & 1u, abort_flag, p.err, polls)) aborted = true;
          }
          tc_fence_after();
          const int sbuf = k.jj & 1;
          const uint32_t idesc = idesc_i8(tc_k_signed(k.ci), 1, 0, 0, 128, Cfg::SCOLS);
          const uint32_t ka = smem_u32(sb), qa = smem_u32(qbufs + (size_t)qi * Cfg::QBUF) + k.ci * Cfg::QSTRIDE;
          const uint32_t dcol = tmem_base + (uint32_t)(wg * Cfg::WG_COLS + sbuf * Cfg::SCOLS);
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4)
            mma_i8_ss(dcol, smem_desc(ka + 32 * s4, 1, 64, 2), smem_desc(qa + 32 * s4, 1, 64, 2), idesc, s4 > 0);
          mma_commit(&mt.sbar[wg][sbuf]);
        }
        if (k.ci != 3) ++unpacked;
      };

      // what the epilogue needs from the softmax of the same block
      struct Pend {
        float mb[GP];
        float vsmax;
        int ci, jj;
      };
      float x[GP], vs_cur = 0.f;  // scores of this thread's key (log2 units), its V scale

      // ---- scores: S out of tensor memory, scaled; block maxima exchanged ---------------------------
      auto phase_b1 = [&](const Blk& k, Pend& pe) {
        uint8_t* sb = slots + (size_t)k.slot * kTcSlotBytes;
        const int sbuf = k.jj & 1;
        if (!aborted && !tc_wait(&mt.sbar[wg][sbuf], (k.jj >> 1) & 1, abort_flag, p.err, polls)) aborted = true;
        tc_fence_after();
        uint32_t s[2 * GP];
        if constexpr (GP <= 4) {
          uint32_t t8[8];
          tmem_ld8(tm_wg + (uint32_t)(sbuf * Cfg::SCOLS), t8);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) s[i] = t8[i];
        } else {
          uint32_t t16[16];
          tmem_ld16(tm_wg + (uint32_t)(sbuf * Cfg::SCOLS), t16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) s[i] = t16[i];
        }
        tc_fence_before();  // the warpgroup's next score MMA into this buffer comes after a barrier all threads pass
        if (k.ci == 3 && !aborted && !tc_wait(&mt.full[k.slot], k.fpar, abort_flag, p.err, polls)) aborted = true;
        const float2 sc = *reinterpret_cast<const float2*>(sb + 2 * kTcTile + wt * 8);
        const bool valid = wt < k.nkeys;
        const float ks = valid ? sc.x : 0.f;
        vs_cur = valid ? sc.y : 0.f;
        const int off = tc_k_offset(k.ci);
        float madd = 0.f;
        if (p.mask != nullptr && valid) {
          const int tok = p.slot_token[(long long)b * g.slots + g.bucket_base[k.ci] + k.key0 + wt];
          madd = tok >= 0 ? p.mask[(long long)b * p.mask_stride + tok] * 1.4426950408889634f : 0.f;
        }
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const int si = (int)s[h] * 128 + (int)s[GP + h] - off * qm.sumA[h];
          x[h] = valid ? fmaf((float)si, ks * qm.qs[h], madd) : -INFINITY;
        }
        if (lbase != nullptr && valid) {
          float* lrow = lbase + g.bucket_base[k.ci] + k.key0 + wt;
#pragma unroll
          for (int h = 0; h < GP; ++h)
            if (h < G) lrow[(long long)h * g.slots] = x[h];
        }
        // block maxima: one redux per head and one for the V scale, then the four warps' values through shared memory
        uint32_t rk[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) rk[h] = redux_max_u32(float_order_key(x[h]));
        const uint32_t rv = redux_max_u32(__float_as_uint(vs_cur));
        if (lane == 0) {
#pragma unroll
          for (int h = 0; h < GP; h += 4)
            *reinterpret_cast<uint4*>(&mt.red[wg][wq][h]) = make_uint4(rk[h], rk[h + 1], rk[h + 2], rk[h + 3]);
          mt.red[wg][wq][GP] = rv;
        }
        named_bar_sync(bar, 128);
        {
          uint32_t a = mt.red[wg][0][GP], c2 = mt.red[wg][1][GP], c3 = mt.red[wg][2][GP], c4 = mt.red[wg][3][GP];
          a = a > c2 ? a : c2;
          c3 = c3 > c4 ? c3 : c4;
          pe.vsmax = __uint_as_float(a > c3 ? a : c3);
        }
#pragma unroll
        for (int h = 0; h < GP; h += 4) {
          const uint4 r0 = *reinterpret_cast<const uint4*>(&mt.red[wg][0][h]), r1 = *reinterpret_cast<const uint4*>(&mt.red[wg][1][h]);
          const uint4 r2 = *reinterpret_cast<const uint4*>(&mt.red[wg][2][h]), r3 = *reinterpret_cast<const uint4*>(&mt.red[wg][3][h]);
          pe.mb[h] = float_from_order_key(max(max(r0.x, r1.x), max(r2.x, r3.x)));
          pe.mb[h + 1] = float_from_order_key(max(max(r0.y, r1.y), max(r2.y, r3.y)));
          pe.mb[h + 2] = float_from_order_key(max(max(r0.z, r1.z), max(r2.z, r3.z)));
          pe.mb[h + 3] = float_from_order_key(max(max(r0.w, r1.w), max(r2.w, r3.w)));
        }
        pe.ci = k.ci;
        pe.jj = k.jj;
      };

      // ---- probabilities: running state updated, P row written, handed to the PV issuer --------------------
      auto phase_b2 = [&](const Blk& k, const Pend& pe) {
        const float vnorm = pe.vsmax > 0.f ? kTcPOne / pe.vsmax : 0.f;
        uint32_t wfix[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const float mb = pe.mb[h];
          const float mn = fmaxf(m_run[h], mb);
          if (mn != m_run[h]) {  // uniform over the warpgroup: every thread holds the same state
            const float alpha = ex2f(m_run[h] - mn);
            l_run[h] *= alpha;
            oacc[h * 128 + wt] *= alpha;  // every thread scales one element of the row; its owner adds to it only after a barrier
            m_run[h] = mn;
          }
          const float pb = ex2f(x[h] - mb);  // in [0, 1]; 0 for rows past the end
          l_run[h] = fmaf(pb, ex2f(mb - mn), l_run[h]);
          wfix[h] = __float2uint_rn(pb * (vs_cur * vnorm));
        }
        // P row of this key: byte h of limb word l = limb l of head h (most significant limb first)
        if constexpr (GP <= 4) {
          const uint32_t lo01 = prmt(wfix[0], wfix[1], 0x5410), lo23 = prmt(wfix[2], wfix[3], 0x5410);  // bytes 0,1 of each
          const uint32_t hi01 = prmt(wfix[0], wfix[1], 0x0062), hi23 = prmt(wfix[2], wfix[3], 0x0062);  // byte 2 of each
          const uint32_t l0 = prmt(lo01, lo23, 0x6420), l1 = prmt(lo01, lo23, 0x7531), l2 = prmt(hi01, hi23, 0x5410);
          *reinterpret_cast<uint4*>(pbuf + wt * 16) = make_uint4(l2, l1, l0, 0u);
        } else {
          uint32_t l0[2], l1[2], l2[2];
#pragma unroll
          for (int q4 = 0; q4 < 2; ++q4) {
            const uint32_t lo01 = prmt(wfix[4 * q4], wfix[4 * q4 + 1], 0x5410), lo23 = prmt(wfix[4 * q4 + 2], wfix[4 * q4 + 3], 0x5410);
            const uint32_t hi01 = prmt(wfix[4 * q4], wfix[4 * q4 + 1], 0x0062), hi23 = prmt(wfix[4 * q4 + 2], wfix[4 * q4 + 3], 0x0062);
            l0[q4] = prmt(lo01, lo23, 0x6420);
            l1[q4] = prmt(lo01, lo23, 0x7531);
            l2[q4] = prmt(hi01, hi23, 0x5410);
          }
          // columns 0..15 (limbs 2 and 1) form the first 16-byte panel, columns 16..31 (limb 0, zeros) the second
          *reinterpret_cast<uint4*>(pbuf + wt * 16) = make_uint4(l2[0], l2[1], l1[0], l1[1]);
          *reinterpret_cast<uint4*>(pbuf + kTcKeys * 16 + wt * 16) = make_uint4(l0[0], l0[1], 0u, 0u);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&mt.pready[wg]);
      };

      // ---- epilogue: the block's P.V out of tensor memory into the fp32 accumulators ---------------
      auto phase_c = [&](const Pend& pe) {
        if (!aborted && !tc_wait(&mt.obar[wg], pe.jj & 1, abort_flag, p.err, polls)) aborted = true;
        tc_fence_after();
        uint32_t acc[PN];
        if constexpr (GP <= 4) {
          uint32_t t16[16];
          tmem_ld16(tm_wg + (uint32_t)(2 * Cfg::SCOLS), t16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = t16[i];
        } else {
          uint32_t t16[16], u16[16];
          tmem_ld16(tm_wg + (uint32_t)(2 * Cfg::SCOLS), t16);
          tmem_ld16(tm_wg + (uint32_t)(2 * Cfg::SCOLS + 16), u16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            acc[i] = t16[i];
            acc[16 + i] = u16[i];
          }
        }
        tc_fence_before();
        const float unit = pe.vsmax * (1.f / kTcPOne);
        const int drow = tc_perm(pe.ci, wt);  // the output row this thread's lane of tensor memory holds for this bucket
        // a row of a narrow bucket is rescaled by one thread (the one with wt == row) and added to by another: the
        // rescale of the probabilities phase must have landed (8-bit rows: same thread, program order suffices)
        if (pe.ci != 3) named_bar_sync(bar, 128);
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const float v = fmaf((float)(int)acc[h], 65536.f, fmaf((float)(int)acc[GP + h], 256.f, (float)(int)acc[2 * GP + h]));
          const float f = unit * ex2f(pe.mb[h] - m_run[h]);
          oacc[h * 128 + drow] = fmaf(v, f, oacc[h * 128 + drow]);
        }
      };

      // ---- software pipeline over this warpgroup's blocks of the run: unpack of block j (its score MMA is then
      // issued), epilogue of block j-1, scores and probabilities of block j.  Every phase is instantiated once:
      // the loop body is the kernel's hot code and has to stay small. ------------------------------------------
      Pend pend;  // written by the scores phase of a block, read by that block's epilogue one iteration later
      bool have_prev = false;
      while (true) {
        const Blk cur = next_mine();
        if (cur.valid) phase_u(cur);             // its score MMA runs while the previous block's epilogue does
        if (have_prev) phase_c(pend);
        if (!cur.valid) break;
        phase_b1(cur, pend);
        phase_b2(cur, pend);
        have_prev = true;
      }

      // ---- end of the run: this warpgroup's partial (max, sum, out) ------------------------------------
      // every score MMA of this warpgroup's blocks has completed (the softmax waited for each), so the query slot
      // can go back once all warpgroups say so
      if (wt == 0) mbar_arrive(&mt.qempty[qi]);
      {
        float ltot[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const float s = warp_sum(l_run[h]);
          if (lane == 0) mt.red[wg][wq][h] = __float_as_uint(s);
        }
        named_bar_sync(bar, 128);
#pragma unroll
        for (int h = 0; h < GP; ++h)
          ltot[h] = (__uint_as_float(mt.red[wg][0][h]) + __uint_as_float(mt.red[wg][1][h])) +
                    (__uint_as_float(mt.red[wg][2][h]) + __uint_as_float(mt.red[wg][3][h]));
        // the barrier above also orders every thread's additions to the output rows before they are read here
        float accum[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) accum[h] = oacc[h * 128 + wt];
        float* out = p.partials + ((long long)r * kTcPartialsPerRun + wg) * partial_stride(G, 128);
        if (WGS < kTcPartialsPerRun && wg == 0 && wt < G) {  // partial slots no warpgroup owns read as empty
          for (int e = WGS; e < kTcPartialsPerRun; ++e) {
            float* eo = p.partials + ((long long)r * kTcPartialsPerRun + e) * partial_stride(G, 128);
            eo[wt * 130] = -INFINITY;
            eo[wt * 130 + 1] = 0.f;
          }
        }
        if (wt < G) {
          float mh = -INFINITY, lh = 0.f;
#pragma unroll
          for (int h = 0; h < GP; ++h)
            if (h == wt) {
              mh = m_run[h];
              lh = ltot[h];
            }
          out[wt * 130] = mh;
          out[wt * 130 + 1] = lh;
        }
        if (have_prev) {
#pragma unroll
          for (int h = 0; h < GP; ++h)
            if (h < G) out[h * 130 + 2 + wt] = accum[h];
        }
      }
      gi += run.total;
      if (++qi == kTcQBufs) {
        qi = 0;
        qfpar ^= 1u;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace skv

using namespace skv;

// ---- tensor maps of the 8-bit bucket (host) -------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// rows [num_kv_heads * cap][128 B] of every (layer, sequence) arena, box = 128 rows
bool encode_rows_map(CUtensorMap* map, const uint8_t* base, long long rows, long long arenas, long long arena_bytes) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t gdim[3] = {128, (cuuint64_t)(rows > 0 ? rows : 1), (cuuint64_t)arenas};
  const cuuint64_t gstr[2] = {128, (cuuint64_t)arena_bytes};
  const cuuint32_t box[3] = {128, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(base), gdim, gstr, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapCacheEntry {
  const uint8_t* store;
  long long rows, arenas, arena_bytes, k_off, v_off;
  CUtensorMap kmap, vmap;
  bool used;
};
constexpr int kMapCache = 8;
MapCacheEntry g_maps[kMapCache];
int g_maps_next = 0;
std::mutex g_maps_mutex;

bool get_maps(const AttnParams& p, const SkvStoreDesc& d, CUtensorMap* kmap, CUtensorMap* vmap) {
  const long long rows = (long long)d.num_kv_heads * d.cap[3], arenas = (long long)d.num_layers * d.num_seqs;
  std::lock_guard<std::mutex> guard(g_maps_mutex);
  for (int i = 0; i < kMapCache; ++i) {
    const MapCacheEntry& e = g_maps[i];
    if (e.used && e.store == p.store && e.rows == rows && e.arenas == arenas && e.arena_bytes == d.arena_bytes &&
        e.k_off == d.k_off[3] && e.v_off == d.v_off[3]) {
      *kmap = e.kmap;
      *vmap = e.vmap;
      return true;
    }
  }
  MapCacheEntry e;
  e.store = p.store;
  e.rows = rows;
  e.arenas = arenas;
  e.arena_bytes = d.arena_bytes;
  e.k_off = d.k_off[3];
  e.v_off = d.v_off[3];
  e.used = true;
  if (!encode_rows_map(&e.kmap, p.store + d.k_off[3], rows, arenas, d.arena_bytes)) return false;
  if (!encode_rows_map(&e.vmap, p.store + d.v_off[3], rows, arenas, d.arena_bytes)) return false;
  g_maps[g_maps_next] = e;
  g_maps_next = (g_maps_next + 1) % kMapCache;
  *kmap = e.kmap;
  *vmap = e.vmap;
  return true;
}

template <int GP>
int launch_tc(const AttnParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, cudaStream_t st) {
  static bool configured[64] = {};  // per template instance and device: the attribute belongs to the device's context
  const size_t smem = tc_smem_bytes<GP>();
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SKV_ERR_CUDA;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    const cudaError_t rc =
        cudaFuncSetAttribute(decode_attn_tc_kernel<GP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (rc != cudaSuccess) {
      fprintf(stderr, "skv_decode_attention: cannot reserve %zu bytes of shared memory: %s\n", smem, cudaGetErrorString(rc));
      return SKV_ERR_CUDA;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  decode_attn_tc_kernel<GP><<<p.num_ctas, TcCfg<GP>::THREADS, smem, st>>>(p, kmap, vmap);
  const cudaError_t rc = cudaGetLastError();
  if (rc != cudaSuccess) {
    fprintf(stderr, "skv_decode_attention: launch failed: %s\n", cudaGetErrorString(rc));
    return SKV_ERR_CUDA;
  }
  return SKV_OK;
}

}  // namespace


namespace skv {

int attn_tc_partials_per_run() { return kTcPartialsPerRun; }

int launch_attn_tc(const AttnParams& p, const SkvStoreDesc& desc, cudaStream_t stream) {
  if (desc.head_dim != 128 || !p.q_is_half || p.group < 1 || p.group > 8) return SKV_ERR_UNSUPPORTED;
  if (desc.arena_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(p.store) & 15) != 0) return SKV_ERR_INVALID;
  CUtensorMap kmap, vmap;
  if (!get_maps(p, desc, &kmap, &vmap)) {
    fprintf(stderr, "skv_decode_attention: cuTensorMapEncodeTiled failed\n");
    return SKV_ERR_CUDA;
  }
  return p.group <= 4 ? launch_tc<4>(p, kmap, vmap, stream) : launch_tc<8>(p, kmap, vmap, stream);
}

}  // namespace skv
