// Fused packed-KV decode attention on the 5th-generation tensor cores (tcgen05) of sm_100a, for
// head_dim 128, fp16 queries and GQA groups of up to 8 query heads (q_len == 1).
//
// The keys are the M operand.  A block is 128 keys of one bucket of one (sequence, KV head):
//
//   S[128 keys x 16]  = K[128 x 128] . Qlimbs^T     tcgen05.mma kind::i8, accumulators in tensor memory.
//                       K is the int8 code matrix, K-major, 128-byte rows in the 128-byte swizzle.  Rows of
//                       the 8-bit bucket are exactly that, so a tiled TMA load (cp.async.bulk.tensor, 3-D map
//                       over the arena, SWIZZLE_128B, no multicast) lands them ready for the MMA and no CUDA core
//                       ever touches an 8-bit code.  2/3/4-bit rows arrive packed (1-D bulk copies) and one
//                       warpgroup spreads their fields to bytes (offset-binary, unsigned operand) into the
//                       same tile.  The query rows are two radix-128 int8 limbs per head (columns h and
//                       GP + h), stored once per run in the element order each width's unpacker produces.
//   softmax           one thread per key: tcgen05.ld of its row of S, scale by the key's K scale, block
//                       maximum per head (redux.sync + one exchange through shared memory), probabilities
//                       relative to the block maximum times the key's V scale (relative to the block's largest)
//                       as 24-bit fixed point in three unsigned byte limbs -> P[128 keys x 16|32] in shared memory.
//   O^T[128 d x 16|32] = V^T[128 x 128 keys] . P     kind::i8, V^T is the same kind of tile read MN-major, P is
//                       MN-major without swizzle.  One thread per output row d folds the three limbs and the
//                       block's scale into fp32 registers (the rescale of an online softmax happens there, never in
//                       tensor memory).
//
// Persistent CTAs (one per SM) walk the runs of the step's plan (attn_sched.cuh, 128-key tiles): a producer
// warp streams blocks into a ring of shared-memory slots; two warpgroups take the blocks alternately,
// each software-pipelined over its own blocks (unpack + score MMA of block j+1, softmax + PV MMA of block j,
// epilogue of block j-1), so the MMA latencies hide behind the other phases.  Every wait is bounded (attn_params.cuh).
// At the end of a run each warpgroup writes one partial (max, sum, out[128]) per query head; the combine step
// (post_attention.cuh) folds the partials of a segment.
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
constexpr int kTcWgs = 2;                            // warpgroups that consume blocks
constexpr int kTcQBufs = 2;                          // query ring (runs in flight)
constexpr int kTcThreads = (kTcWgs * 4 + 1) * 32;    // + the producer warp
constexpr int kTcQTile = 16 * 128;                   // 16 limb rows x 128 B, swizzled like a K tile
// Fixed-point unit of P: the largest probability-times-V-scale of a block maps to 2^24 - 256, so that no
// rounding in the chain can reach 2^24 (whose three low bytes would read as zero).
constexpr float kTcPOne = 16776960.f;

template <int GP>
struct TcCfg {
  static constexpr int NS = GP <= 4 ? 6 : 5;               // ring slots
  static constexpr int PN = GP <= 4 ? 16 : 32;             // bytes of one P row = N of the PV MMA (3 limbs x GP, padded)
  static constexpr int PBYTES = kTcKeys * PN;              // one P buffer
  static constexpr int SCOLS = 16;                         // N of the score MMA (2 limbs x GP, padded)
  static constexpr int WG_COLS = 2 * SCOLS + 2 * PN;       // tensor-memory columns of one warpgroup (double buffered)
  static constexpr int TMEM_COLS = GP <= 4 ? 128 : 256;    // power of two >= kTcWgs * WG_COLS
  static_assert(kTcWgs * WG_COLS <= TMEM_COLS, "tensor memory budget");
};

struct TcQMeta {
  float qs[8];   // limb step of head g times 1/sqrt(d) * log2(e)
  int sumA[8];   // 128 * sum(limb 0) + sum(limb 1): what the offset of unsigned codes adds per unit of offset
  RunDesc desc;
};

template <int GP>
struct TcMeta {
  uint64_t full[8], empty[8];
  uint64_t qfull[kTcQBufs], qempty[kTcQBufs];
  uint64_t sbar[kTcWgs][2], obar[kTcWgs][2];
  uint64_t drain[kTcWgs];
  uint32_t tmem_base;
  int abort_flag;
  uint32_t red[kTcWgs][4][12];          // per warp: GP block maxima (order keys) + the largest V scale
  uint32_t wsum[kTcWgs][2][4][8];       // per warp: sum of the fixed-point P of every head (unsigned-code blocks)
  TcQMeta q[kTcQBufs];
};

template <int GP>
constexpr size_t tc_smem_bytes() {
  return (size_t)TcCfg<GP>::NS * kTcSlotBytes + (size_t)kTcQBufs * 4 * kTcQTile + (size_t)kTcWgs * 2 * TcCfg<GP>::PBYTES +
         sizeof(TcMeta<GP>) + 1024;  // + slack to align the base to 1024 B
}

// ---- element order of the unpacked tiles ----------------------------------------------------------
// Byte position i of an unpacked row holds element tc_perm(bucket, i) of the stored row; the order is
// whatever the cheapest field extraction of that width yields.  The query limbs are stored in the same order
// (a dot product does not care) and the output rows are put back in order once per run.
__host__ __device__ constexpr int tc_perm(int bucket, int i) {
  return bucket == 0   ? (i & ~15) + ((i >> 2) & 3) + 4 * (i & 3)    // 2-bit: word s, shift j, byte b -> 16s + j + 4b
         : bucket == 1 ? (i & ~31) + 8 * (i & 3) + ((i >> 2) & 7)    // 3-bit: field class f, group g -> 8g + f
         : bucket == 2 ? (i & ~7) + 2 * (i & 3) + ((i >> 2) & 1)     // 4-bit: word s, low/high nibble e, byte j -> 8s + 2j + e
                       : i;                                          // 8-bit: as stored
}
__host__ __device__ constexpr int tc_perm_inv(int bucket, int d) {
  return bucket == 0   ? (d & ~15) + 4 * (d & 3) + ((d >> 2) & 3)
         : bucket == 1 ? (d & ~31) + 4 * (d & 7) + ((d >> 3) & 3)
         : bucket == 2 ? (d & ~7) + 4 * (d & 1) + ((d >> 1) & 3)
                       : d;
}
// byte offset of (row, byte position) inside a 128-byte-swizzled tile whose base is 1024-byte aligned
__host__ __device__ constexpr int tc_swz(int row, int pos) { return row * 128 + ((((pos >> 4) ^ (row & 7))) << 4) + (pos & 15); }

// ---- unpack: packed rows of a narrow bucket -> int8 tile (unsigned codes) -------------------------------
// All loads of the warpgroup complete before the first store (the tiles overlay the packed bytes).
// `wt` = thread index inside the warpgroup, `bar` = the warpgroup's named barrier.
__device__ __forceinline__ void tc_store_chunk(uint8_t* tile, int row, int oc, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  *reinterpret_cast<uint4*>(tile + row * 128 + ((oc ^ (row & 7)) << 4)) = make_uint4(a, b, c, d);
}

// 2-bit: 128 rows x 32 B = 256 chunks of 16 B per tile; thread wt takes chunks wt and wt + 128 of K and of V.
__device__ __forceinline__ void tc_unpack2(uint8_t* slot, int wt, int bar) {
  uint4 kin[2], vin[2];
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    kin[n] = *reinterpret_cast<const uint4*>(slot + (wt + 128 * n) * 16);
    vin[n] = *reinterpret_cast<const uint4*>(slot + kTcTile + (wt + 128 * n) * 16);
  }
  named_bar_sync(bar, 128);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const uint4 in = which ? vin[n] : kin[n];
      const int c = wt + 128 * n, row = c >> 1, hf = c & 1;
      const uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
      for (int s = 0; s < 4; ++s)
        tc_store_chunk(slot + which * kTcTile, row, 4 * hf + s, w[s] & 0x03030303u, (w[s] >> 2) & 0x03030303u,
                       (w[s] >> 4) & 0x03030303u, (w[s] >> 6) & 0x03030303u);
    }
  }
}

// 4-bit: 128 rows x 64 B = 512 chunks per tile; thread wt takes chunks wt + 128 n, n = 0..3.
__device__ __forceinline__ void tc_unpack4(uint8_t* slot, int wt, int bar) {
  uint4 kin[4], vin[4];
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    kin[n] = *reinterpret_cast<const uint4*>(slot + (wt + 128 * n) * 16);
    vin[n] = *reinterpret_cast<const uint4*>(slot + kTcTile + (wt + 128 * n) * 16);
  }
  named_bar_sync(bar, 128);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const uint4 in = which ? vin[n] : kin[n];
      const int c = wt + 128 * n, row = c >> 2, q = c & 3;
      constexpr uint32_t m = 0x0f0f0f0fu;
      tc_store_chunk(slot + which * kTcTile, row, 2 * q, in.x & m, (in.x >> 4) & m, in.y & m, (in.y >> 4) & m);
      tc_store_chunk(slot + which * kTcTile, row, 2 * q + 1, in.z & m, (in.z >> 4) & m, in.w & m, (in.w >> 4) & m);
    }
  }
}

// 3-bit: a row is 48 B = four 12-byte groups of 32 fields; thread wt takes row wt of K and of V.
__device__ __forceinline__ void tc_unpack3(uint8_t* slot, int wt, int bar) {
  uint32_t kin[12], vin[12];
#pragma unroll
  for (int n = 0; n < 3; ++n) {
    const uint4 a = *reinterpret_cast<const uint4*>(slot + wt * 48 + 16 * n);
    const uint4 b = *reinterpret_cast<const uint4*>(slot + kTcTile + wt * 48 + 16 * n);
    kin[4 * n] = a.x; kin[4 * n + 1] = a.y; kin[4 * n + 2] = a.z; kin[4 * n + 3] = a.w;
    vin[4 * n] = b.x; vin[4 * n + 1] = b.y; vin[4 * n + 2] = b.z; vin[4 * n + 3] = b.w;
  }
  named_bar_sync(bar, 128);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const uint32_t* in = which ? vin : kin;
      const uint32_t w[3] = {in[3 * a], in[3 * a + 1], in[3 * a + 2]};
      uint32_t o[8];
      unpack_kslice_i8<128, 3>(w, o);
      tc_store_chunk(slot + which * kTcTile, wt, 2 * a, o[0], o[1], o[2], o[3]);
      tc_store_chunk(slot + which * kTcTile, wt, 2 * a + 1, o[4], o[5], o[6], o[7]);
    }
  }
}

// ---- block cursor: the blocks of a run in the order producer and consumers both follow ------------------
struct TcCursor {
  int ci, t;
};
__device__ __forceinline__ void tc_cursor_skip(const RunDesc& d, TcCursor& c) {
  while (c.ci < kNumBuckets && c.t >= d.kb[c.ci]) {
    ++c.ci;
    if (c.ci < kNumBuckets) c.t = d.ka[c.ci];
  }
}
__device__ __forceinline__ TcCursor tc_cursor_begin(const RunDesc& d) {
  TcCursor c{0, d.ka[0]};
  tc_cursor_skip(d, c);
  return c;
}

// ---- query limbs of a run, in the four element orders (one warp) ---------------------------------------------
template <int GP>
__device__ __forceinline__ void tc_prep_query(uint8_t* qtiles, TcQMeta& meta, const AttnParams& p, int seq, int head, int G,
                                              int lane) {
  const long long q_off = ((long long)seq * p.num_q_heads + (long long)head * G) * 128;
  float q[GP][4];
#pragma unroll
  for (int h = 0; h < GP; ++h) {
    if (h < G) {
      const __half2* src = reinterpret_cast<const __half2*>(static_cast<const __half*>(p.query) + q_off + h * 128 + lane * 4);
      const float2 a = __half22float2(src[0]), b = __half22float2(src[1]);
      q[h][0] = a.x; q[h][1] = a.y; q[h][2] = b.x; q[h][3] = b.y;
    }
  }
#pragma unroll
  for (int h = 0; h < GP; ++h) {
    if (h >= G) break;
    float amax = fmaxf(fmaxf(fabsf(q[h][0]), fabsf(q[h][1])), fmaxf(fabsf(q[h][2]), fabsf(q[h][3])));
    amax = warp_max(amax);
    constexpr float range = 127.f * 128.f;
    const float step = amax > 0.f ? amax / range : 1.f;
    const float inv = 1.f / step;
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = lane * 4 + e;
      const float rem = fminf(fmaxf(rintf(q[h][e] * inv), -range), range);
      const float hi = rintf(rem * (1.f / 128.f));
      const int lo = (int)(rem - hi * 128.f);  // in [-64, 64]
      s0 += (int)hi;
      s1 += lo;
#pragma unroll
      for (int c = 0; c < kNumBuckets; ++c) {
        const int pos = tc_perm_inv(c, d);
        qtiles[c * kTcQTile + tc_swz(h, pos)] = (uint8_t)(int8_t)(int)hi;
        qtiles[c * kTcQTile + tc_swz(GP + h, pos)] = (uint8_t)(int8_t)lo;
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
}

template <int GP>
__global__ void __launch_bounds__(kTcThreads, 1)
    decode_attn_tc_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  using Cfg = TcCfg<GP>;
  constexpr int NS = Cfg::NS, PN = Cfg::PN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* slots = smem;                                               // [NS][kTcSlotBytes]
  uint8_t* qtiles = slots + (size_t)NS * kTcSlotBytes;                 // [kTcQBufs][4][kTcQTile]
  uint8_t* pbufs = qtiles + (size_t)kTcQBufs * 4 * kTcQTile;           // [kTcWgs][2][PBYTES]
  TcMeta<GP>& mt = *reinterpret_cast<TcMeta<GP>*>(pbufs + (size_t)kTcWgs * 2 * Cfg::PBYTES);
  const StoreGeom& g = p.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.group, Hkv = g.num_kv_heads;
  volatile int* abort_flag = &mt.abort_flag;

  {  // limb rows of heads that do not exist stay zero
    uint32_t* z = reinterpret_cast<uint32_t*>(qtiles);
    for (int i = tid; i < kTcQBufs * 4 * kTcQTile / 4; i += kTcThreads) z[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&mt.full[s], 1);
      mbar_init(&mt.empty[s], 1);
    }
    for (int s = 0; s < kTcQBufs; ++s) {
      mbar_init(&mt.qfull[s], 1);
      mbar_init(&mt.qempty[s], kTcWgs);
    }
    for (int w = 0; w < kTcWgs; ++w) {
      mbar_init(&mt.sbar[w][0], 1);
      mbar_init(&mt.sbar[w][1], 1);
      mbar_init(&mt.obar[w][0], 1);
      mbar_init(&mt.obar[w][1], 1);
      mbar_init(&mt.drain[w], 1);
    }
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
  const unsigned polls = p.wait_polls;

  if (warp == kTcWgs * 4) {
    // ================================ producer warp ================================
    int gi = 0, qi = 0;
    uint32_t qepar = 1;  // a fresh barrier passes a wait on parity 1: every slot starts empty
    bool ok = run_begin < run_end;
    const uint64_t stream_policy = l2_evict_first_policy();  // the cache is read once per step
    // issues up to `limit` further blocks of run d, resuming at cursor c
    auto issue_blocks = [&](const RunDesc& d, TcCursor& c, int limit) -> bool {
      const uint8_t* arena = arena_ptr(g, p.store, p.layer, d.seq);
      while (c.ci < kNumBuckets) {
        if (limit-- <= 0) return true;
        const int slot = gi % NS;
        if (!wait_or_abort(&mt.empty[slot], ((gi / NS) & 1) ^ 1u, abort_flag, p.err, polls)) return false;
        if (lane == 0) {
          const int ci = c.ci, key0 = c.t * kTcKeys;
          const int nkeys = (d.cnt[ci] - key0) < kTcKeys ? (d.cnt[ci] - key0) : kTcKeys;
          const int n16 = (nkeys + 15) & ~15;
          uint8_t* sb = slots + (size_t)slot * kTcSlotBytes;
          const long long row = (long long)d.head * g.cap[ci] + key0;
          const uint32_t sbytes = (uint32_t)(n16 * 8);
          fence_proxy_async();
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
        ++gi;
        ++c.t;
        tc_cursor_skip(d, c);
      }
      return true;
    };
    auto publish_query = [&](const RunDesc& d) -> bool {
      if (!wait_or_abort(&mt.qempty[qi], qepar, abort_flag, p.err, polls)) return false;
      if (lane == 0) mt.q[qi].desc = d;
      tc_prep_query<GP>(qtiles + (size_t)qi * 4 * kTcQTile, mt.q[qi], p, d.seq, d.head, G, lane);
      fence_proxy_async();  // the MMA reads the limb rows through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&mt.qfull[qi]);
      if (++qi == kTcQBufs) {
        qi = 0;
        qepar ^= 1u;
      }
      return true;
    };
    RunDesc d = pv.first[blockIdx.x];  // meaningful when the CTA has a run
    for (int r = run_begin; ok && r < run_end; ++r) {
      TcCursor c = tc_cursor_begin(d);
      // the first blocks of a run go out first; while they are in flight the query of the NEXT run is
      // published, so that no consumer waits for query rows at a run boundary
      ok = issue_blocks(d, c, NS);
      if (r == run_begin) ok = ok && publish_query(d);
      RunDesc dn = d;
      if (ok && r + 1 < run_end) {
        dn = pv.runs[r + 1];
        ok = publish_query(dn);
      }
      ok = ok && issue_blocks(d, c, 1 << 30);
      d = dn;
    }
  } else {
    // ================================== consumer warpgroups ==================================
    const int wg = warp >> 2, wt = tid & 127, wq = warp & 3;  // wq: this warp's lane quarter of tensor memory
    const int bar = 1 + wg;
    const uint32_t tm_wg = tmem_base + (uint32_t)(wg * Cfg::WG_COLS) + ((uint32_t)(wq * 32) << 16);
    uint8_t* pbuf_wg = pbufs + (size_t)wg * 2 * Cfg::PBYTES;
    int gi = 0, j = 0, qi = 0;
    uint32_t qfpar = 0;
    bool aborted = false;

    struct Blk {
      int ci, key0, nkeys, slot, buf;
      uint32_t fpar, bpar;
      bool valid;
    };

    for (int r = run_begin; r < run_end; ++r) {
      if (!aborted && !wait_or_abort(&mt.qfull[qi], qfpar, abort_flag, p.err, polls)) aborted = true;
      const RunDesc d = mt.q[qi].desc;
      const uint8_t* qt = qtiles + (size_t)qi * 4 * kTcQTile;
      float qs[GP];
      int sumA[GP];
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        qs[h] = mt.q[qi].qs[h];
        sumA[h] = mt.q[qi].sumA[h];
      }
      const int b = d.seq, hkv = d.head;
      float m_run[GP], l_run[GP], o[kNumBuckets][GP];
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
#pragma unroll
        for (int c = 0; c < kNumBuckets; ++c) o[c][h] = 0.f;
      }
      float* lbase = nullptr;  // logits row of head 0 of this group
      if (p.logits != nullptr) lbase = p.logits + ((long long)b * p.num_q_heads + hkv * G) * g.slots;

      TcCursor cur_c = tc_cursor_begin(d);
      auto next_mine = [&]() -> Blk {
        Blk k{};
        k.valid = false;
        while (cur_c.ci < kNumBuckets) {
          const bool take = (gi % kTcWgs) == wg;
          if (take) {
            k.ci = cur_c.ci;
            k.key0 = cur_c.t * kTcKeys;
            k.nkeys = (d.cnt[k.ci] - k.key0) < kTcKeys ? (d.cnt[k.ci] - k.key0) : kTcKeys;
            k.slot = gi % NS;
            k.fpar = (gi / NS) & 1;
            k.buf = j & 1;
            k.bpar = (j >> 1) & 1;
            k.valid = true;
            ++j;
          }
          ++gi;
          ++cur_c.t;
          tc_cursor_skip(d, cur_c);
          if (take) break;
        }
        return k;
      };

      // ---- phase A: data of the block present, narrow rows spread to bytes, score MMA issued ----
      auto phase_a = [&](const Blk& k) {
        uint8_t* sb = slots + (size_t)k.slot * kTcSlotBytes;
        if (!aborted && !wait_or_abort(&mt.full[k.slot], k.fpar, abort_flag, p.err, polls)) aborted = true;
        if (k.ci != 3) {
          if (k.ci == 0) tc_unpack2(sb, wt, bar);
          else if (k.ci == 1) tc_unpack3(sb, wt, bar);
          else tc_unpack4(sb, wt, bar);
          fence_proxy_async();
          tc_fence_before();
          named_bar_sync(bar, 128);
        }
        if (wt == 0) {
          tc_fence_after();
          const uint32_t idesc = idesc_i8(k.ci == 3, 1, 0, 0, 128, Cfg::SCOLS);
          const uint32_t ka = smem_u32(sb), qa = smem_u32(qt + k.ci * kTcQTile);
#pragma unroll
          for (int s = 0; s < 4; ++s)
            mma_i8_ss(tmem_base + (uint32_t)(wg * Cfg::WG_COLS + k.buf * Cfg::SCOLS), smem_desc(ka + 32 * s, 1, 64, 2),
                      smem_desc(qa + 32 * s, 1, 64, 2), idesc, s > 0);
          mma_commit(&mt.sbar[wg][k.buf]);
        }
      };

      // what phase C needs from phase B of the same block
      struct Pend {
        float mb[GP];
        float vsmax;
        Blk k;
      };

      // ---- phase B: scores -> probabilities (24-bit fixed point), PV MMA issued -----------------------
      auto phase_b = [&](const Blk& k, Pend& pe) {
        uint8_t* sb = slots + (size_t)k.slot * kTcSlotBytes;
        if (!aborted && !wait_or_abort(&mt.sbar[wg][k.buf], k.bpar, abort_flag, p.err, polls)) aborted = true;
        tc_fence_after();
        uint32_t s[2 * GP];
        if constexpr (GP <= 4) {
          uint32_t t8[8];
          tmem_ld8(tm_wg + (uint32_t)(k.buf * Cfg::SCOLS), t8);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) s[i] = t8[i];
        } else {
          uint32_t t16[16];
          tmem_ld16(tm_wg + (uint32_t)(k.buf * Cfg::SCOLS), t16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) s[i] = t16[i];
        }
        const float2 sc = *reinterpret_cast<const float2*>(sb + 2 * kTcTile + wt * 8);
        const bool valid = wt < k.nkeys;
        const float ks = valid ? sc.x : 0.f, vs = valid ? sc.y : 0.f;
        const int off = k.ci == 3 ? 0 : (1 << (bucket_bits(k.ci) - 1));
        float x[GP];
        float madd = 0.f;
        if (p.mask != nullptr && valid) {
          const int tok = p.slot_token[(long long)b * g.slots + g.bucket_base[k.ci] + k.key0 + wt];
          madd = tok >= 0 ? p.mask[(long long)b * p.mask_stride + tok] * 1.4426950408889634f : 0.f;
        }
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const int si = (int)s[h] * 128 + (int)s[GP + h] - off * sumA[h];
          x[h] = valid ? fmaf((float)si, ks * qs[h], madd) : -INFINITY;
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
        const uint32_t rv = redux_max_u32(__float_as_uint(vs));
        if (lane == 0) {
#pragma unroll
          for (int h = 0; h < GP; ++h) mt.red[wg][wq][h] = rk[h];
          mt.red[wg][wq][GP] = rv;
        }
        named_bar_sync(bar, 128);
        float vsmax;
        {
          uint32_t a = mt.red[wg][0][GP], c2 = mt.red[wg][1][GP], c3 = mt.red[wg][2][GP], c4 = mt.red[wg][3][GP];
          a = a > c2 ? a : c2;
          c3 = c3 > c4 ? c3 : c4;
          vsmax = __uint_as_float(a > c3 ? a : c3);
        }
        const float vnorm = vsmax > 0.f ? kTcPOne / vsmax : 0.f;
        uint32_t wfix[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          uint32_t a = mt.red[wg][0][h], c2 = mt.red[wg][1][h], c3 = mt.red[wg][2][h], c4 = mt.red[wg][3][h];
          a = a > c2 ? a : c2;
          c3 = c3 > c4 ? c3 : c4;
          const float mb = float_from_order_key(a > c3 ? a : c3);
          pe.mb[h] = mb;
          const float mn = fmaxf(m_run[h], mb);
          if (mn != m_run[h]) {  // uniform over the warpgroup: every thread holds the same state
            const float alpha = ex2f(m_run[h] - mn);
            l_run[h] *= alpha;
#pragma unroll
            for (int c = 0; c < kNumBuckets; ++c) o[c][h] *= alpha;
            m_run[h] = mn;
          }
          const float pb = ex2f(x[h] - mb);  // in [0, 1]; 0 for rows past the end
          l_run[h] = fmaf(pb, ex2f(mb - mn), l_run[h]);
          wfix[h] = __float2uint_rn(pb * (vs * vnorm));
        }
        pe.vsmax = vsmax;
        pe.k = k;
        // P row of this key: byte h of limb word l = limb l of head h (most significant limb first)
        uint8_t* prow = pbuf_wg + (size_t)k.buf * Cfg::PBYTES;
        if constexpr (GP <= 4) {
          const uint32_t lo01 = prmt(wfix[0], wfix[1], 0x5410), lo23 = prmt(wfix[2], wfix[3], 0x5410);  // bytes 0,1 of each
          const uint32_t hi01 = prmt(wfix[0], wfix[1], 0x0062), hi23 = prmt(wfix[2], wfix[3], 0x0062);  // byte 2 of each
          const uint32_t l0 = prmt(lo01, lo23, 0x6420), l1 = prmt(lo01, lo23, 0x7531), l2 = prmt(hi01, hi23, 0x5410);
          *reinterpret_cast<uint4*>(prow + wt * 16) = make_uint4(l2, l1, l0, 0u);
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
          *reinterpret_cast<uint4*>(prow + wt * 16) = make_uint4(l2[0], l2[1], l1[0], l1[1]);
          *reinterpret_cast<uint4*>(prow + kTcKeys * 16 + wt * 16) = make_uint4(l0[0], l0[1], 0u, 0u);
        }
        if (k.ci != 3) {  // unsigned codes: the offset's share of the product is offset * sum of P
#pragma unroll
          for (int h = 0; h < GP; ++h) {
            const uint32_t sum = redux_add_u32(wfix[h]);
            if (lane == 0) mt.wsum[wg][k.buf][wq][h] = sum;
          }
        }
        fence_proxy_async();
        tc_fence_before();
        named_bar_sync(bar, 128);
        if (wt == 0) {
          tc_fence_after();
          const uint32_t idesc = idesc_i8(k.ci == 3, 0, 1, 1, 128, PN);
          const uint32_t va = smem_u32(sb + kTcTile), pa = smem_u32(prow);
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4)
            mma_i8_ss(tmem_base + (uint32_t)(wg * Cfg::WG_COLS + 2 * Cfg::SCOLS + k.buf * PN), smem_desc(va + 4096 * s4, 64, 64, 2),
                      smem_desc(pa + 512 * s4, 8, kTcKeys, 0), idesc, s4 > 0);
          mma_commit(&mt.obar[wg][k.buf]);
          mma_commit(&mt.empty[k.slot]);  // the slot goes back to the producer when the tile has been read
        }
      };

      // ---- phase C: the block's P.V out of tensor memory into the fp32 accumulators ---------------
      auto phase_c = [&](const Pend& pe) {
        const Blk& k = pe.k;
        if (!aborted && !wait_or_abort(&mt.obar[wg][k.buf], k.bpar, abort_flag, p.err, polls)) aborted = true;
        tc_fence_after();
        uint32_t acc[PN];
        if constexpr (GP <= 4) {
          uint32_t t16[16];
          tmem_ld16(tm_wg + (uint32_t)(2 * Cfg::SCOLS + k.buf * PN), t16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = t16[i];
        } else {
          uint32_t t16[16], u16[16];
          tmem_ld16(tm_wg + (uint32_t)(2 * Cfg::SCOLS + k.buf * PN), t16);
          tmem_ld16(tm_wg + (uint32_t)(2 * Cfg::SCOLS + k.buf * PN + 16), u16);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            acc[i] = t16[i];
            acc[16 + i] = u16[i];
          }
        }
        tc_fence_before();
        const float unit = pe.vsmax * (1.f / kTcPOne);
        const int off = k.ci == 3 ? 0 : (1 << (bucket_bits(k.ci) - 1));
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float v = fmaf((float)(int)acc[h], 65536.f, fmaf((float)(int)acc[GP + h], 256.f, (float)(int)acc[2 * GP + h]));
          if (k.ci != 3) {
            const uint32_t ws = mt.wsum[wg][k.buf][0][h] + mt.wsum[wg][k.buf][1][h] + mt.wsum[wg][k.buf][2][h] +
                                mt.wsum[wg][k.buf][3][h];
            v -= (float)off * (float)ws;
          }
          const float f = unit * ex2f(pe.mb[h] - m_run[h]);
          if (k.ci == 0) o[0][h] = fmaf(v, f, o[0][h]);
          else if (k.ci == 1) o[1][h] = fmaf(v, f, o[1][h]);
          else if (k.ci == 2) o[2][h] = fmaf(v, f, o[2][h]);
          else o[3][h] = fmaf(v, f, o[3][h]);
        }
      };

      // ---- software pipeline over this warpgroup's blocks of the run -----------------------------
      Pend pend_cur, pend_prev;
      bool have_prev = false;
      Blk cur = next_mine();
      const bool any = cur.valid;
      if (cur.valid) phase_a(cur);
      while (cur.valid) {
        const Blk nxt = next_mine();
        if (nxt.valid) phase_a(nxt);
        phase_b(cur, pend_cur);
        if (have_prev) phase_c(pend_prev);
        pend_prev = pend_cur;
        have_prev = true;
        cur = nxt;
      }
      if (have_prev) phase_c(pend_prev);

      // ---- end of the run: this warpgroup's partial (max, sum, out) ------------------------------------
      // every score MMA of the run has completed (phase B waited for each), so the query slot can go back
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
        // rows of the narrow buckets come out in their unpack order: put them back through shared memory
        float accum[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) accum[h] = o[3][h];
        float* stage = reinterpret_cast<float*>(pbuf_wg);  // [GP][128]; no MMA of this warpgroup is in flight
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          if (d.ka[c] >= d.kb[c]) continue;  // uniform: the run has no block of this bucket
          named_bar_sync(bar, 128);
          const int dpos = tc_perm(c, wt);
#pragma unroll
          for (int h = 0; h < GP; ++h) stage[h * 128 + dpos] = o[c][h];
          named_bar_sync(bar, 128);
#pragma unroll
          for (int h = 0; h < GP; ++h) accum[h] += stage[h * 128 + wt];
        }
        named_bar_sync(bar, 128);  // stage (a P buffer) and red are free again
        float* out = p.partials + ((long long)r * kTcWgs + wg) * partial_stride(G, 128);
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
        if (any) {
#pragma unroll
          for (int h = 0; h < GP; ++h)
            if (h < G) out[h * 130 + 2 + wt] = accum[h];
        }
      }
      if (++qi == kTcQBufs) {
        qi = 0;
        qfpar ^= 1u;
      }
    }
    // every MMA this warpgroup issued must have completed before tensor memory is freed
    if (wt == 0) {
      mma_commit(&mt.drain[wg]);
      wait_or_abort(&mt.drain[wg], 0, abort_flag, p.err, polls);
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
  decode_attn_tc_kernel<GP><<<p.num_ctas, kTcThreads, smem, st>>>(p, kmap, vmap);
  const cudaError_t rc = cudaGetLastError();
  if (rc != cudaSuccess) {
    fprintf(stderr, "skv_decode_attention: launch failed: %s\n", cudaGetErrorString(rc));
    return SKV_ERR_CUDA;
  }
  return SKV_OK;
}

}  // namespace

namespace skv {

int attn_tc_partials_per_run() { return kTcWgs; }

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
