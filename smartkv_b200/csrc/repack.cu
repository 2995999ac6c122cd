// Requantise / repack after a reallocation.
//
// Replaces SmartKVCache._requantize_tokens / _requantize_single / _write_quantized_slot
// (smartkv/core/cache.py:806-926) and the bucket bookkeeping around them (swap-with-last
// delete :1121-1161, append :1046-1083): a Python loop over every (layer, changed token).
//
// A token whose width changed is dequantised from its stored codes (code * scale, fp32),
// quantised again at the new width (cache.py:819-844: from the dequantised codes, not from
// the original values) and moved to the bucket of the new width.  Buckets stay dense: the
// positions a bucket loses are refilled first by its own rows that now lie beyond the new
// count, then by the arriving rows, so only changed rows and a few tail rows are touched.
// Which row of a bucket a token occupies is not observable (attention is a sum over keys).
//
// Three steps, every one stream-ordered:
//   skv_repack_plan     one block per sequence: the list of moves (source -> destination
//                       storage index), the same for every layer
//   skv_requant_repack  per layer range: all moved rows -> staging (requantised where the
//                       width changed), then staging -> destination.  Two kernels, so every
//                       read of the old layout precedes every write of the new one.
//   skv_repack_meta     the per-token arrays kept in storage order follow the same moves.
#include <cub/block/block_scan.cuh>

#include "quant_row.cuh"

namespace skv {

constexpr int kPlanThreads = 1024;
constexpr int kStageRowBytes = 136;  // 128 packed bytes at most, the fp32 scale at offset 128, padding
constexpr int kMaxSeqsRepack = 1024;

__device__ __forceinline__ int bucket_of_slot(const StoreGeom& g, int s) {
  int b = 0;
#pragma unroll
  for (int i = 1; i < kNumBuckets; ++i)
    if (s >= g.bucket_base[i]) b = i;
  return b;
}

// ---- the moves ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kPlanThreads)
    repack_plan_kernel(StoreGeom g, const int32_t* counts, const uint8_t* new_bits, int32_t* move_src,
                       int32_t* move_dst, int32_t* n_moves, int32_t* counts_new, int32_t* scratch, int32_t* err) {
  const int b = blockIdx.x, tid = threadIdx.x, T = g.slots;
  using Scan = cub::BlockScan<int, kPlanThreads>;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ int s_new[kNumBuckets], s_free[kNumBuckets], s_tail[kNumBuckets], s_off[kNumBuckets + 1];
  __shared__ int s_run[2];
  const uint8_t* nb = new_bits + (long long)b * T;
  int32_t* free_pos = scratch + (long long)b * 2 * T;  // [T], bucket w's list at [bucket_base[w] ...)
  int32_t* tail_src = free_pos + T;                     // [T]
  int32_t* msrc = move_src + (long long)b * T;
  int32_t* mdst = move_dst + (long long)b * T;
  int cnt[kNumBuckets];
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) cnt[i] = counts[b * kNumBuckets + i];
  if (tid < kNumBuckets) s_new[tid] = 0;
  __syncthreads();

  // new counts
  for (int w = 0; w < kNumBuckets; ++w) {
    for (int pos = tid; pos < cnt[w]; pos += kPlanThreads) {
      const int nbk = bits_bucket(nb[g.bucket_base[w] + pos]);
      if (nbk >= 0) atomicAdd(&s_new[nbk], 1);
      else if (err) atomicExch(err, 4);  // a live token without a width
    }
  }
  __syncthreads();
  bool over = false;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) over |= s_new[i] > g.cap[i];
  if (over) {
    if (tid == 0) {
      if (err) atomicExch(err, 3);  // a bucket would overflow: nothing moves
      n_moves[b] = 0;
      for (int i = 0; i < kNumBuckets; ++i) counts_new[b * kNumBuckets + i] = cnt[i];
    }
    return;
  }

  // per bucket: free positions (ascending) and own rows beyond the new count (ascending)
  for (int w = 0; w < kNumBuckets; ++w) {
    const int c_old = cnt[w], c_new = s_new[w], base = g.bucket_base[w], width = bucket_bits(w);
    const int span = c_old > c_new ? c_old : c_new;
    if (tid == 0) s_run[0] = s_run[1] = 0;
    __syncthreads();
    for (int p0 = 0; p0 < span; p0 += kPlanThreads) {
      const int pos = p0 + tid;
      const bool live = pos < c_old;
      const bool stays = live && nb[base + pos] == width;
      const int is_free = (pos < c_new && !stays) ? 1 : 0;
      const int is_tail = (stays && pos >= c_new) ? 1 : 0;
      int packed = is_free | (is_tail << 16), excl, total;
      Scan(tmp).ExclusiveSum(packed, excl, total);
      const int rf = s_run[0] + (excl & 0xffff), rt = s_run[1] + (excl >> 16);
      if (is_free) free_pos[base + rf] = pos;
      if (is_tail) tail_src[base + rt] = base + pos;
      __syncthreads();
      if (tid == 0) {
        s_run[0] += total & 0xffff;
        s_run[1] += total >> 16;
      }
      __syncthreads();
    }
    if (tid == 0) {
      s_free[w] = s_run[0];
      s_tail[w] = s_run[1];
    }
    __syncthreads();
  }
  if (tid == 0) {
    int off = 0;
    for (int w = 0; w < kNumBuckets; ++w) {
      s_off[w] = off;
      off += s_free[w];
    }
    s_off[kNumBuckets] = off;
    n_moves[b] = off;
    for (int i = 0; i < kNumBuckets; ++i) counts_new[b * kNumBuckets + i] = s_new[i];
  }
  __syncthreads();

  // arrivals of every bucket in ascending source storage index, after the bucket's tail rows
  __shared__ int s_arr[kNumBuckets];
  if (tid < kNumBuckets) s_arr[tid] = 0;
  __syncthreads();
  for (int ws = 0; ws < kNumBuckets; ++ws) {
    const int base = g.bucket_base[ws], width = bucket_bits(ws);
    for (int p0 = 0; p0 < cnt[ws]; p0 += kPlanThreads) {
      const int pos = p0 + tid;
      int to = -1;
      if (pos < cnt[ws]) {
        const int nw = nb[base + pos];
        if (nw != width) to = bits_bucket(nw);
      }
      // a chunk can send up to 1024 rows to one bucket: two scans of two 16-bit fields each
      int pa = (to == 0 ? 1 : 0) | ((to == 1 ? 1 : 0) << 16);
      int pb = (to == 2 ? 1 : 0) | ((to == 3 ? 1 : 0) << 16);
      int ea, ta, eb, tb;
      Scan(tmp).ExclusiveSum(pa, ea, ta);
      __syncthreads();
      Scan(tmp).ExclusiveSum(pb, eb, tb);
      if (to >= 0) {
        const int rank = to == 0 ? (ea & 0xffff) : to == 1 ? (ea >> 16) : to == 2 ? (eb & 0xffff) : (eb >> 16);
        msrc[s_off[to] + s_tail[to] + s_arr[to] + rank] = base + pos;
      }
      __syncthreads();
      if (tid == 0) {
        s_arr[0] += ta & 0xffff;
        s_arr[1] += ta >> 16;
        s_arr[2] += tb & 0xffff;
        s_arr[3] += tb >> 16;
      }
      __syncthreads();
    }
  }
  // destinations and the tail sources
  for (int w = 0; w < kNumBuckets; ++w) {
    const int base = g.bucket_base[w];
    if (tid == 0 && s_tail[w] + s_arr[w] != s_free[w] && err) atomicExch(err, 5);  // bookkeeping broken
    for (int k = tid; k < s_free[w]; k += kPlanThreads) mdst[s_off[w] + k] = base + free_pos[base + k];
    for (int k = tid; k < s_tail[w]; k += kPlanThreads) msrc[s_off[w] + k] = tail_src[base + k];
  }
}

// ---- moving the rows ------------------------------------------------------------------------------------
struct RowMoveParams {
  StoreGeom g;
  uint8_t* store;
  int layer_begin, layer_end;
  const int32_t* move_src;
  const int32_t* move_dst;
  const int32_t* n_moves;
  uint8_t* staging;
  long long staging_rows;
  int32_t* err;
};

// prefix of the per-sequence move counts into shared memory; returns the total
__device__ __forceinline__ int load_move_prefix(const int32_t* n_moves, int B, int* s_prefix) {
  // all counts are fetched at once (one round trip to memory), then one thread adds them up
  for (int b = threadIdx.x; b < B; b += blockDim.x) s_prefix[b + 1] = n_moves[b];
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    s_prefix[0] = 0;
    for (int b = 0; b < B; ++b) {
      acc += s_prefix[b + 1];
      s_prefix[b + 1] = acc;
    }
  }
  __syncthreads();
  return s_prefix[B];
}
__device__ __forceinline__ int find_seq(const int* s_prefix, int B, int m) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (s_prefix[mid] <= m) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ---- head_dim 128: half a warp per row, 8 consecutive elements per lane --------------------------------
// The K row and the V row of one (token, head) are handled by the two halves of a warp at once, which
// halves the per-row cost of everything that is not per element (reductions, address arithmetic, packing).

// this lane's 8 values code * scale (elements 8*l16 .. 8*l16+7) of a packed 128-element row, from the two
// aligned words (w0 at word bitpos/32, w1 the next one or 0 past the row's end) that hold the lane's field.
// The code goes into the significand of 2^23 and the offset comes off in the same subtraction, so no
// int->float conversion is needed; 8-bit rows hold two's complement, which flipping the top bit turns
// into the offset form of the other widths.
__device__ __forceinline__ void dequant8(uint32_t w0, uint32_t w1, int l16, int bits, float scale, float (&x)[8]) {
  const int sh = (l16 * 8 * bits) & 31;
  // a lane's field is 8 * bits wide: 64 bits = two aligned words at 8 bits (sh == 0), else at most 32 bits
  const uint32_t lo = __funnelshift_r(w0, w1, sh), hi = w1;
  const uint32_t fm = (1u << bits) - 1u, flip = bits == 8 ? 0x80u : 0u;
  const float bias = bits == 8 ? 8388736.f : bits == 4 ? 8388616.f : bits == 3 ? 8388612.f : 8388610.f;  // 2^23 + 2^(bits-1)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int at = bits * i;
    const uint32_t u = (((at >= 32 ? hi : lo) >> (at & 31)) ^ flip) & fm;
    x[i] = __fmul_rn(__fsub_rn(__uint_as_float(u | 0x4B000000u), bias), scale);  // codes.float() * scale
  }
}

// packs this lane's 8 codes and stores the half-warp's 128-element row at dst (4-byte aligned)
__device__ __forceinline__ void pack8_store(const int (&code)[8], int bits, uint8_t* dst, int l16) {
  uint32_t* out = reinterpret_cast<uint32_t*>(dst);
  if (bits == 8) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= ((uint32_t)code[i] & 0xffu) << (8 * i);
      hi |= ((uint32_t)code[4 + i] & 0xffu) << (8 * i);
    }
    out[2 * l16] = lo;
    out[2 * l16 + 1] = hi;
    return;
  }
  const int off = 1 << (bits - 1);
  const uint32_t fm = (1u << bits) - 1u;
  uint32_t f = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) f |= (((uint32_t)(code[i] + off)) & fm) << (bits * i);  // 16, 24 or 32 bits
  const uint32_t n = __shfl_down_sync(0xffffffffu, f, 1);  // the next lane's field (same half for the lanes that use it)
  if (bits == 4) {
    out[l16] = f;
  } else if (bits == 2) {
    if ((l16 & 1) == 0) out[l16 >> 1] = f | (n << 16);
  } else {  // 3 bits: four 24-bit fields make three words
    const int r = l16 & 3;
    const uint32_t word = r == 0 ? (f | (n << 24)) : r == 1 ? ((f >> 8) | (n << 16)) : ((f >> 16) | (n << 8));
    if (r < 3) out[3 * (l16 >> 2) + r] = word;
  }
}

// quantises the half-warp's row x again at `bits`; returns the new scale (all 16 lanes of the row)
__device__ __forceinline__ float requant8(const float (&x)[8], int bits, int (&q)[8]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // stays inside the half
  const int hi = (1 << (bits - 1)) - 1, lo = -(1 << (bits - 1));
  float ns = scale_of(amax, hi);
  if (ns == 0.f) ns = 1.f;
  quantize_vals<8>(x, ns, lo, hi, q);
  return ns;
}

// head_dim 64: the same with 4 consecutive elements per lane
__device__ __forceinline__ float requant4(const int (&code)[4], float scale, int bits, int (&q)[4]) {
  float x[4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i] = __fmul_rn((float)code[i], scale);
    amax = fmaxf(amax, fabsf(x[i]));
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const int hi = (1 << (bits - 1)) - 1, lo = -(1 << (bits - 1));
  float ns = scale_of(amax, hi);
  if (ns == 0.f) ns = 1.f;
  quantize_vals<4>(x, ns, lo, hi, q);
  return ns;
}

// packs the half-warp's 64-element row (4 codes per lane) and stores its 2 * bits words at dst
__device__ __forceinline__ void pack4_store(const int (&code)[4], int bits, uint8_t* dst, int l16) {
  const int wb = 4 * bits;  // bits this lane contributes: 8, 12, 16 or 32
  uint32_t mine = 0;
  if (bits == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) mine |= ((uint32_t)code[i] & 0xffu) << (8 * i);
  } else {
    const int off = 1 << (bits - 1);
    const uint32_t fm = (1u << bits) - 1u;
#pragma unroll
    for (int i = 0; i < 4; ++i) mine |= (((uint32_t)(code[i] + off)) & fm) << (bits * i);
  }
  // lane l16 assembles word l16 of the row from the (at most four) lanes whose fields overlap it
  const int base_lane = (threadIdx.x & 16), first = (32 * l16) / wb;
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int sl = first + i;
    const uint32_t f = __shfl_sync(0xffffffffu, mine, base_lane + (sl & 15));
    const int pos = sl * wb - 32 * l16;
    if (sl < 16 && pos < 32 && pos + wb > 0) word |= pos >= 0 ? (f << pos) : (f >> (-pos));
  }
  if (l16 < 2 * bits) reinterpret_cast<uint32_t*>(dst)[l16] = word;
}

// phase 0: source rows -> staging (requantised at the destination width); phase 1: staging -> destination.
// Staging holds one row per (layer, KV head, K|V, move), moves innermost.
//
// A row is a separate memory transaction of 32..128 bytes.  Two things keep the memory system busy with
// such small pieces: a warp takes kRowBatch consecutive moves of one (layer, KV head) and issues all their
// loads before it does anything with them; and because consecutive moves mostly have consecutive source
// and destination positions (the planner lists them in ascending order), the warps of a block touch
// neighbouring rows, scales and staging rows at about the same time, so that the 4- and 8-byte scale
// accesses and the short rows of neighbouring tokens share sectors and DRAM pages.
// Half a warp per row: the K row in lanes 0..15, the V row of the same (token, head) in lanes 16..31.
constexpr int kRowBatch = 4;

struct MoveInfo {
  int src, dst, seq;
};

template <int EPL, int PHASE>
__global__ void __launch_bounds__(256) repack_rows_kernel(const RowMoveParams p) {
  const StoreGeom& g = p.g;
  __shared__ int s_prefix[kMaxSeqsRepack + 1];
  const int total_moves = load_move_prefix(p.n_moves, g.num_seqs, s_prefix);
  const int Hkv = g.num_kv_heads, nl = p.layer_end - p.layer_begin;
  if ((long long)total_moves * nl * Hkv * 2 > p.staging_rows) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && p.err) atomicExch(p.err, 6);  // staging too small: nothing moves
    return;
  }
  const int lane = threadIdx.x & 31;
  const int which = lane >> 4, l16 = lane & 15;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const int groups = (total_moves + kRowBatch - 1) / kRowBatch;
  const long long items = (long long)groups * nl * Hkv;
  for (long long it = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += nwarps) {
    int lh, grp;
    if (items >> 31) {  // 64-bit division is a long subroutine: only where the item count needs it
      lh = (int)(it / groups);
      grp = (int)(it - (long long)lh * groups);
    } else {
      lh = (int)it / groups;
      grp = (int)it - lh * groups;
    }
    const int li = lh / Hkv, h = lh - li * Hkv;
    const int m0 = grp * kRowBatch;
    // lanes 0..kRowBatch-1 look one move up each
    MoveInfo mine{-1, -1, 0};
    if (lane < kRowBatch && m0 + lane < total_moves) {
      mine.seq = find_seq(s_prefix, g.num_seqs, m0 + lane);
      const long long at = (long long)mine.seq * g.slots + (m0 + lane - s_prefix[mine.seq]);
      mine.src = p.move_src[at];
      mine.dst = p.move_dst[at];
    }
    // rows of (layer li, head h, K|V): staging row index = ((lh * 2 + which) * total_moves + move)
    uint8_t* stage = p.staging + (((long long)lh * 2 + which) * total_moves + m0) * kStageRowBytes;
    uint32_t w0[kRowBatch], w1[kRowBatch];
    float sc[kRowBatch];
    if (PHASE == 0) {
#pragma unroll
      for (int u = 0; u < kRowBatch; ++u) {
        const int src = __shfl_sync(0xffffffffu, mine.src, u), seq = __shfl_sync(0xffffffffu, mine.seq, u);
        const int dst = __shfl_sync(0xffffffffu, mine.dst, u);
        w0[u] = w1[u] = 0u;
        sc[u] = 0.f;
        if (src < 0) continue;
        const int wb_s = bucket_of_slot(g, src), bits_s = bucket_bits(wb_s), rb_s = g.row_bytes[wb_s];
        const uint8_t* arena = arena_ptr(g, p.store, p.layer_begin + li, seq);
        const long long row = (long long)h * g.cap[wb_s] + (src - g.bucket_base[wb_s]);
        const uint32_t* rp =
            reinterpret_cast<const uint32_t*>(arena + (which ? g.v_off[wb_s] : g.k_off[wb_s]) + row * rb_s);
        const float2 t = reinterpret_cast<const float2*>(arena + g.sc_off[wb_s])[row];
        sc[u] = which ? t.y : t.x;
        if (bucket_of_slot(g, dst) == wb_s || EPL != 4) {
          // the row only changes place (up to 32 words, two per lane), or head_dim 64: whole-row words
          const int words = rb_s >> 2;
          if (l16 < words) w0[u] = rp[l16];
          if (l16 + 16 < words) w1[u] = rp[l16 + 16];
        } else {
          // head_dim 128: 8 consecutive elements per lane lie in at most two aligned words
          const int wi = (l16 * 8 * bits_s) >> 5;
          w0[u] = rp[wi];
          if (wi + 1 < 4 * bits_s) w1[u] = rp[wi + 1];
        }
      }
#pragma unroll
      for (int u = 0; u < kRowBatch; ++u) {
        const int src = __shfl_sync(0xffffffffu, mine.src, u), dst = __shfl_sync(0xffffffffu, mine.dst, u);
        if (src < 0) continue;  // the same for the whole warp: the shuffles below see every lane
        const int wb_s = bucket_of_slot(g, src), wb_d = bucket_of_slot(g, dst);
        const int bits_s = bucket_bits(wb_s), bits_d = bucket_bits(wb_d);
        uint8_t* st = stage + u * kStageRowBytes;
        if (wb_s == wb_d) {
          const int words = g.row_bytes[wb_s] >> 2;
          if (l16 < words) reinterpret_cast<uint32_t*>(st)[l16] = w0[u];
          if (l16 + 16 < words) reinterpret_cast<uint32_t*>(st)[l16 + 16] = w1[u];
          if (l16 == 0) *reinterpret_cast<float*>(st + 128) = sc[u];
        } else if constexpr (EPL == 4) {
          float x[8];
          int q[8];
          dequant8(w0[u], w1[u], l16, bits_s, sc[u], x);
          const float ns = requant8(x, bits_d, q);
          pack8_store(q, bits_d, st, l16);
          if (l16 == 0) *reinterpret_cast<float*>(st + 128) = ns;
        } else {
          // head_dim 64: 4 consecutive elements per lane, out of the row's words held by the half-warp
          const int bitpos = l16 * 4 * bits_s, wi = bitpos >> 5, sh = bitpos & 31;
          const int base_lane = lane & 16;
          const uint32_t lo = __shfl_sync(0xffffffffu, w0[u], base_lane + (wi & 15));
          const uint32_t hi = __shfl_sync(0xffffffffu, w0[u], base_lane + ((wi + 1) & 15));
          const uint32_t field = __funnelshift_r(lo, hi, sh);
          int code[4], q[4];
          if (bits_s == 8) {
#pragma unroll
            for (int i = 0; i < 4; ++i) code[i] = (int)(int8_t)((field >> (8 * i)) & 0xffu);
          } else {
            const uint32_t fm = (1u << bits_s) - 1u;
#pragma unroll
            for (int i = 0; i < 4; ++i) code[i] = (int)((field >> (bits_s * i)) & fm) - (1 << (bits_s - 1));
          }
          const float ns = requant4(code, sc[u], bits_d, q);
          pack4_store(q, bits_d, st, l16);
          if (l16 == 0) *reinterpret_cast<float*>(st + 128) = ns;
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < kRowBatch; ++u) {
        const int dst = __shfl_sync(0xffffffffu, mine.dst, u);
        w0[u] = w1[u] = 0u;
        sc[u] = 0.f;
        if (dst < 0) continue;
        const int words = g.row_bytes[bucket_of_slot(g, dst)] >> 2;
        const uint32_t* st = reinterpret_cast<const uint32_t*>(stage + u * kStageRowBytes);
        if (l16 < words) w0[u] = st[l16];
        if (l16 + 16 < words) w1[u] = st[l16 + 16];
        if (l16 == 0) sc[u] = reinterpret_cast<const float*>(st)[32];
      }
#pragma unroll
      for (int u = 0; u < kRowBatch; ++u) {
        const int dst = __shfl_sync(0xffffffffu, mine.dst, u), seq = __shfl_sync(0xffffffffu, mine.seq, u);
        if (dst < 0) continue;
        const int wb_d = bucket_of_slot(g, dst), rb_d = g.row_bytes[wb_d], words = rb_d >> 2;
        uint8_t* arena = arena_ptr(g, p.store, p.layer_begin + li, seq);
        const long long row = (long long)h * g.cap[wb_d] + (dst - g.bucket_base[wb_d]);
        uint32_t* rp = reinterpret_cast<uint32_t*>(arena + (which ? g.v_off[wb_d] : g.k_off[wb_d]) + row * rb_d);
        if (l16 < words) rp[l16] = w0[u];
        if (l16 + 16 < words) rp[l16 + 16] = w1[u];
        if (l16 == 0) {
          reinterpret_cast<float*>(arena + g.sc_off[wb_d])[2 * row + which] = sc[u];
          if (which) note_v_scale(g, arena, sc[u]);
        }
      }
    }
  }
}

// ---- per-token arrays -----------------------------------------------------------------------------------
struct MetaParams {
  StoreGeom g;
  const int32_t* move_src;
  const int32_t* move_dst;
  const int32_t* n_moves;
  int32_t* counts;
  const int32_t* counts_new;
  int32_t* slot_token;
  double* cumulative;
  double* rank_pct;
  int8_t* rank_streak;
  float* layer_ema;
  uint8_t* touched;
  uint8_t* staging;
  long long staging_moves;
  int32_t* err;
};

__host__ __device__ inline long long meta_move_bytes(int num_layers) { return 24 + 8LL * num_layers; }

template <int PHASE>
__global__ void repack_meta_kernel(const MetaParams p) {
  const StoreGeom& g = p.g;
  __shared__ int s_prefix[kMaxSeqsRepack + 1];
  const int total = load_move_prefix(p.n_moves, g.num_seqs, s_prefix);
  if (total > p.staging_moves) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && p.err) atomicExch(p.err, 6);
    return;
  }
  const int L = g.num_layers, T = g.slots, B = g.num_seqs;
  // staging arrays, one entry per move
  double* st_cum = reinterpret_cast<double*>(p.staging);
  double* st_pct = st_cum + p.staging_moves;
  int32_t* st_tok = reinterpret_cast<int32_t*>(st_pct + p.staging_moves);
  float* st_ema = reinterpret_cast<float*>(st_tok + p.staging_moves);             // [L][moves]
  uint8_t* st_tch = reinterpret_cast<uint8_t*>(st_ema + (long long)L * p.staging_moves);  // [L][moves]
  int8_t* st_str = reinterpret_cast<int8_t*>(st_tch + (long long)L * p.staging_moves);
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  for (long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x; m < total; m += nthreads) {
    const int b = find_seq(s_prefix, B, (int)m);
    const int k = (int)m - s_prefix[b];
    const long long si = (long long)b * T + p.move_src[(long long)b * T + k];
    const long long di = (long long)b * T + p.move_dst[(long long)b * T + k];
    if (PHASE == 0) {
      st_cum[m] = p.cumulative[si];
      st_pct[m] = p.rank_pct[si];
      st_tok[m] = p.slot_token[si];
      st_str[m] = p.rank_streak[si];
      for (int l = 0; l < L; ++l) {
        st_ema[(long long)l * p.staging_moves + m] = p.layer_ema[(long long)l * B * T + si];
        st_tch[(long long)l * p.staging_moves + m] = p.touched[(long long)l * B * T + si];
      }
    } else {
      p.cumulative[di] = st_cum[m];
      p.rank_pct[di] = st_pct[m];
      p.slot_token[di] = st_tok[m];
      p.rank_streak[di] = st_str[m];
      for (int l = 0; l < L; ++l) {
        p.layer_ema[(long long)l * B * T + di] = st_ema[(long long)l * p.staging_moves + m];
        p.touched[(long long)l * B * T + di] = st_tch[(long long)l * p.staging_moves + m];
      }
    }
  }
}

// indices a bucket gave up hold no token any more: a later append must find fresh state there
__global__ void repack_meta_clear_kernel(const MetaParams p) {
  const StoreGeom& g = p.g;
  const int b = blockIdx.y, L = g.num_layers, T = g.slots, B = g.num_seqs;
  for (int w = 0; w < kNumBuckets; ++w) {
    const int c_old = p.counts[b * kNumBuckets + w], c_new = p.counts_new[b * kNumBuckets + w];
    for (int pos = c_new + blockIdx.x * blockDim.x + threadIdx.x; pos < c_old; pos += gridDim.x * blockDim.x) {
      const long long i = (long long)b * T + g.bucket_base[w] + pos;
      p.cumulative[i] = 0.0;
      p.rank_pct[i] = 0.0;
      p.rank_streak[i] = -1;
      p.slot_token[i] = -1;
      for (int l = 0; l < L; ++l) {
        p.layer_ema[(long long)l * B * T + i] = 0.f;
        p.touched[(long long)l * B * T + i] = 0;
      }
    }
  }
}
__global__ void repack_commit_counts_kernel(int32_t* counts, const int32_t* counts_new, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) counts[i] = counts_new[i];
}

}  // namespace skv

using namespace skv;

extern "C" int64_t skv_repack_plan_workspace_bytes(const SkvStoreDesc* desc) {
  if (!desc || desc->num_seqs <= 0 || desc->slots <= 0) return SKV_ERR_INVALID;
  return (int64_t)desc->num_seqs * desc->slots * 2 * (int64_t)sizeof(int32_t);
}

extern "C" int skv_repack_plan(const SkvStoreDesc* desc, const int32_t* counts, const uint8_t* new_bits,
                               int32_t* move_src, int32_t* move_dst, int32_t* n_moves, int32_t* counts_new,
                               void* workspace, int32_t* err_flag, void* stream) {
  if (!desc || !counts || !new_bits || !move_src || !move_dst || !n_moves || !counts_new || !workspace)
    return SKV_ERR_INVALID;
  if (desc->num_seqs > kMaxSeqsRepack) return SKV_ERR_UNSUPPORTED;
  repack_plan_kernel<<<desc->num_seqs, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      make_geom(*desc), counts, new_bits, move_src, move_dst, n_moves, counts_new, static_cast<int32_t*>(workspace),
      err_flag);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

extern "C" int64_t skv_requant_staging_bytes(const SkvStoreDesc* desc, int64_t max_moves, int num_layers) {
  if (!desc || max_moves < 0 || num_layers <= 0) return SKV_ERR_INVALID;
  return max_moves * num_layers * desc->num_kv_heads * 2 * (int64_t)kStageRowBytes;
}

extern "C" int skv_requant_repack(const SkvStoreDesc* desc, void* store, int layer_begin, int layer_end,
                                  const int32_t* move_src, const int32_t* move_dst, const int32_t* n_moves,
                                  void* staging, int64_t staging_bytes, int32_t* err_flag, void* stream) {
  if (!desc || !store || !move_src || !move_dst || !n_moves || !staging) return SKV_ERR_INVALID;
  if (layer_begin < 0 || layer_end > desc->num_layers || layer_begin >= layer_end) return SKV_ERR_INVALID;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if (desc->num_seqs > kMaxSeqsRepack) return SKV_ERR_UNSUPPORTED;
  RowMoveParams p;
  p.g = make_geom(*desc);
  p.store = static_cast<uint8_t*>(store);
  p.layer_begin = layer_begin;
  p.layer_end = layer_end;
  p.move_src = move_src;
  p.move_dst = move_dst;
  p.n_moves = n_moves;
  p.staging = static_cast<uint8_t*>(staging);
  p.staging_rows = staging_bytes / kStageRowBytes;
  p.err = err_flag;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = sms * 8, threads = 256;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (desc->head_dim == 128) {
    repack_rows_kernel<4, 0><<<grid, threads, 0, st>>>(p);
    repack_rows_kernel<4, 1><<<grid, threads, 0, st>>>(p);
  } else {
    repack_rows_kernel<2, 0><<<grid, threads, 0, st>>>(p);
    repack_rows_kernel<2, 1><<<grid, threads, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

extern "C" int64_t skv_repack_meta_staging_bytes(const SkvStoreDesc* desc, int64_t max_moves) {
  if (!desc || max_moves < 0) return SKV_ERR_INVALID;
  return max_moves * meta_move_bytes(desc->num_layers) + 256;
}

extern "C" int skv_repack_meta(const SkvStoreDesc* desc, const int32_t* move_src, const int32_t* move_dst,
                               const int32_t* n_moves, int32_t* counts, const int32_t* counts_new,
                               int32_t* slot_token, double* cumulative, double* rank_pct, int8_t* rank_streak,
                               float* layer_ema, uint8_t* touched, void* staging, int64_t staging_bytes,
                               int32_t* err_flag, void* stream) {
  if (!desc || !move_src || !move_dst || !n_moves || !counts || !counts_new || !slot_token || !cumulative ||
      !rank_pct || !rank_streak || !layer_ema || !touched || !staging)
    return SKV_ERR_INVALID;
  if (desc->num_seqs > kMaxSeqsRepack) return SKV_ERR_UNSUPPORTED;
  MetaParams p;
  p.g = make_geom(*desc);
  p.move_src = move_src;
  p.move_dst = move_dst;
  p.n_moves = n_moves;
  p.counts = counts;
  p.counts_new = counts_new;
  p.slot_token = slot_token;
  p.cumulative = cumulative;
  p.rank_pct = rank_pct;
  p.rank_streak = rank_streak;
  p.layer_ema = layer_ema;
  p.touched = touched;
  p.staging = static_cast<uint8_t*>(staging);
  p.staging_moves = (staging_bytes - 256) / meta_move_bytes(desc->num_layers);
  p.staging_moves &= ~7LL;  // keeps every staging array 8-byte aligned
  p.err = err_flag;
  if (p.staging_moves <= 0) return SKV_ERR_CAPACITY;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  repack_meta_kernel<0><<<296, 256, 0, st>>>(p);
  repack_meta_kernel<1><<<296, 256, 0, st>>>(p);
  repack_meta_clear_kernel<<<dim3(8, desc->num_seqs), 256, 0, st>>>(p);
  repack_commit_counts_kernel<<<(desc->num_seqs * kNumBuckets + 255) / 256, 256, 0, st>>>(counts, counts_new,
                                                                                        desc->num_seqs * kNumBuckets);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
