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
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int b = 0; b < B; ++b) {
      s_prefix[b] = acc;
      acc += n_moves[b];
    }
    s_prefix[B] = acc;
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

// Reads this lane's EPL codes out of a packed row through aligned 32-bit loads (rows are at least
// 16 bytes and 4-byte aligned; a lane's field of EPL*bits <= 32 bits spans at most two words).
template <int EPL>
__device__ __forceinline__ void unpack_row_words(const uint8_t* src, int bits, int lane, int (&code)[EPL]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(src);
  const int bitpos = lane * EPL * bits, wi = bitpos >> 5, sh = bitpos & 31, nbits = EPL * bits;
  const int nwords = nbits;  // 32 lanes * nbits / 32
  uint32_t lo = w[wi];
  uint32_t hi = (sh + nbits > 32 && wi + 1 < nwords) ? w[wi + 1] : 0u;
  const uint32_t field = __funnelshift_r(lo, hi, sh);
  if (bits == 8) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) code[i] = (int)(int8_t)((field >> (8 * i)) & 0xffu);
  } else {
    const uint32_t fm = (1u << bits) - 1u;
    const int off = 1 << (bits - 1);
#pragma unroll
    for (int i = 0; i < EPL; ++i) code[i] = (int)((field >> (bits * i)) & fm) - off;
  }
}

// ---- head_dim 128: half a warp per row, 8 consecutive elements per lane --------------------------------
// The K row and the V row of one (token, head) are handled by the two halves of a warp at once, which
// halves the per-row cost of everything that is not per element (reductions, address arithmetic, packing).

// this lane's 8 codes (elements 8*l16 .. 8*l16+7) of a packed 128-element row
__device__ __forceinline__ void unpack8(const uint8_t* src, int bits, int l16, int (&code)[8]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(src);
  const int bitpos = l16 * 8 * bits, wi = bitpos >> 5, sh = bitpos & 31, nwords = 4 * bits;  // 128*bits/32
  const uint32_t w0 = w[wi];
  const uint32_t w1 = wi + 1 < nwords ? w[wi + 1] : 0u;
  // a lane's field is 8 * bits wide: 64 bits = two aligned words at 8 bits (sh == 0), else at most 32 bits
  const uint32_t lo = __funnelshift_r(w0, w1, sh), hi = w1;
  if (bits == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      code[i] = (int)(int8_t)((lo >> (8 * i)) & 0xffu);
      code[4 + i] = (int)(int8_t)((hi >> (8 * i)) & 0xffu);
    }
  } else {
    const uint32_t fm = (1u << bits) - 1u;
    const int off = 1 << (bits - 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) code[i] = (int)((lo >> (bits * i)) & fm) - off;  // 8 * bits <= 32
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

// dequantise (code * scale) and quantise again at `bits`; returns the new scale (all 16 lanes of the row)
__device__ __forceinline__ float requant8(const int (&code)[8], float scale, int bits, int (&q)[8]) {
  float x[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[i] = __fmul_rn((float)code[i], scale);  // codes.float() * scale
    amax = fmaxf(amax, fabsf(x[i]));
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // stays inside the half
  const int hi = (1 << (bits - 1)) - 1, lo = -(1 << (bits - 1));
  float ns = __fdiv_rn(amax, (float)(hi > 1 ? hi : 1));
  if (ns == 0.f) ns = 1.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v = rintf(__fdiv_rn(x[i], ns));
    v = fminf(fmaxf(v, (float)lo), (float)hi);
    q[i] = (int)v;
  }
  return ns;
}

// phase 0: source rows -> staging (requantised at the destination width); phase 1: staging -> destination.
// One warp takes one move and walks its rows (layers of the call x KV heads x {K, V}).
template <int EPL, int PHASE>
__global__ void repack_rows_kernel(const RowMoveParams p) {
  const StoreGeom& g = p.g;
  __shared__ int s_prefix[kMaxSeqsRepack + 1];
  const int total_moves = load_move_prefix(p.n_moves, g.num_seqs, s_prefix);
  const int Hkv = g.num_kv_heads, nl = p.layer_end - p.layer_begin;
  const int rows_per_move = nl * Hkv * 2;
  if ((long long)total_moves * rows_per_move > p.staging_rows) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && p.err) atomicExch(p.err, 6);  // staging too small: nothing moves
    return;
  }
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  for (int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); m < total_moves; m += nwarps) {
    const int b = find_seq(s_prefix, g.num_seqs, m);
    const int k = m - s_prefix[b];
    const int src = p.move_src[(long long)b * g.slots + k], dst = p.move_dst[(long long)b * g.slots + k];
    const int wb_s = bucket_of_slot(g, src), wb_d = bucket_of_slot(g, dst);
    const int bits_s = bucket_bits(wb_s), bits_d = bucket_bits(wb_d);
    const int rb_s = g.row_bytes[wb_s], rb_d = g.row_bytes[wb_d];
    const int pos_s = src - g.bucket_base[wb_s], pos_d = dst - g.bucket_base[wb_d];
    uint8_t* stage = p.staging + (long long)m * rows_per_move * kStageRowBytes;
    for (int li = 0; li < nl; ++li) {
      uint8_t* arena = arena_ptr(g, p.store, p.layer_begin + li, b);
      if (PHASE == 0) {
        const float* scales = reinterpret_cast<const float*>(arena + g.sc_off[wb_s]);
        if constexpr (EPL == 4) {
          // head_dim 128: lanes 0..15 take the K row, lanes 16..31 the V row of the same (token, head)
          const int which = lane >> 4, l16 = lane & 15;
          for (int h = 0; h < Hkv; ++h) {
            const long long row = (long long)h * g.cap[wb_s] + pos_s;
            const float2 sc = reinterpret_cast<const float2*>(scales)[row];
            const uint8_t* rp = arena + (which ? g.v_off[wb_s] : g.k_off[wb_s]) + row * rb_s;
            uint8_t* st = stage + ((li * Hkv + h) * 2 + which) * kStageRowBytes;
            const float scale = which ? sc.y : sc.x;
            if (bits_s == bits_d) {
              const int words = rb_s >> 2;  // 8, 12, 16 or 32
              if (l16 < words) reinterpret_cast<uint32_t*>(st)[l16] = reinterpret_cast<const uint32_t*>(rp)[l16];
              if (l16 + 16 < words) reinterpret_cast<uint32_t*>(st)[l16 + 16] = reinterpret_cast<const uint32_t*>(rp)[l16 + 16];
              if (l16 == 0) *reinterpret_cast<float*>(st + 128) = scale;
            } else {
              int code[8], q[8];
              unpack8(rp, bits_s, l16, code);
              const float ns = requant8(code, scale, bits_d, q);
              pack8_store(q, bits_d, st, l16);
              if (l16 == 0) *reinterpret_cast<float*>(st + 128) = ns;
            }
          }
        } else {
        for (int h = 0; h < Hkv; ++h) {
          const long long row = (long long)h * g.cap[wb_s] + pos_s;
          const float2 sc = reinterpret_cast<const float2*>(scales)[row];
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            const uint8_t* rp = arena + (which ? g.v_off[wb_s] : g.k_off[wb_s]) + row * rb_s;
            uint8_t* st = stage + ((li * Hkv + h) * 2 + which) * kStageRowBytes;
            const float scale = which ? sc.y : sc.x;
            if (bits_s == bits_d) {
              if (lane < (rb_s >> 2)) reinterpret_cast<uint32_t*>(st)[lane] = reinterpret_cast<const uint32_t*>(rp)[lane];
              if (lane == 0) *reinterpret_cast<float*>(st + 128) = scale;
            } else {
              int code[EPL];
              unpack_row_words<EPL>(rp, bits_s, lane, code);
              RowVals<EPL> x;
#pragma unroll
              for (int i = 0; i < EPL; ++i) x.v[i] = __fmul_rn((float)code[i], scale);  // codes.float() * scale
              int q[EPL];
              const float ns = quantize_row<EPL>(x, bits_d, q);
              pack_store_row<EPL>(q, bits_d, st, lane);
              if (lane == 0) *reinterpret_cast<float*>(st + 128) = ns;
            }
          }
        }
        }
      } else {
        float* scales = reinterpret_cast<float*>(arena + g.sc_off[wb_d]);
        for (int h = 0; h < Hkv; ++h) {
          const long long row = (long long)h * g.cap[wb_d] + pos_d;
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            uint8_t* rp = arena + (which ? g.v_off[wb_d] : g.k_off[wb_d]) + row * rb_d;
            const uint8_t* st = stage + ((li * Hkv + h) * 2 + which) * kStageRowBytes;
            if (lane < (rb_d >> 2)) reinterpret_cast<uint32_t*>(rp)[lane] = reinterpret_cast<const uint32_t*>(st)[lane];
            if (lane == 0) scales[2 * row + which] = *reinterpret_cast<const float*>(st + 128);
          }
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
