// Block-level bodies of the three steps that follow the streaming attention kernel of a layer:
//   combine     fold the split-KV partials of a (sequence, KV head), add the current token in full
//               precision, normalise (smartkv/core/fused_cpu.py:115-137)
//   importance  per-key attention mass -> cumulative importance + per-layer EMA
//               (smartkv/core/cache.py:232-264, smartkv/core/importance.py:44-101)
//   append      quantise + pack the step's new token into the store (smartkv/core/cache.py:1187-1355)
// The importance step of a layer needs what that layer's combine step produced, but nothing stops
// it from running one launch later: post_attention.cu runs the combine and the append of layer l
// side by side with the importance step of the layer before it.  The stand-alone entry points run
// the same bodies from their own kernels.
#pragma once

#include "attn_sched.cuh"
#include "quant_row.cuh"

namespace skv {

constexpr int kPostThreads = 256;
constexpr int kCombineChunk = 256;
constexpr int kMaxQHeads = 128;

__host__ __device__ inline int partial_stride(int group, int head_dim) { return group * (head_dim + 2); }

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- combine ----------------------------------------------------------------------------------------
struct CombineParams {
  StoreGeom g;
  const int* plan;
  const void* query;
  int q_is_half;
  int num_q_heads;
  int group;
  const float* partials;
  int per_run;  // partials per run = consumer warps of the attention launch
  int num_ctas;
  const void* cur_k;
  const void* cur_v;
  int kv_is_half;
  const float* cur_mask;  // additive mask of the current token per sequence, natural-log units (may be null)
  float* out;
  float* lse_max;
  float* lse_sum;
  float* cur_prob;
  float scale_log2;
};

__host__ __device__ inline int combine_heads_per_block(int head_dim) { return kPostThreads / head_dim; }
__host__ __device__ inline int combine_units(const StoreGeom& g, int group) {
  const int hpb = combine_heads_per_block(g.head_dim);
  return g.num_seqs * g.num_kv_heads * ((group + hpb - 1) / hpb);
}

struct CombineShared {
  float red[kPostThreads / 32][2];
  float f[kPostThreads / 64][kCombineChunk];   // per head of the block
  float lf[kPostThreads / 64][kCombineChunk];
};

// The scaled logit of the current token for one query head: q . k * scale, reduced over the D threads
// of the head in a fixed shape (warp tree, then the warps of the head in order).
// `sub` = head slot inside the block, `d` = thread's element.
__device__ __forceinline__ float head_dot(float prod, int sub, int d, int D, float (*red)[2], int slot) {
  const float s = warp_sum(prod);
  const int warp_in_head = d >> 5, lane = d & 31, wph = D >> 5;
  if (lane == 0) red[sub * wph + warp_in_head][slot] = s;
  __syncthreads();
  float acc = 0.f;
  for (int w = 0; w < wph; ++w) acc += red[sub * wph + w][slot];
  return acc;
}

// One unit = up to kPostThreads / D query heads of one (sequence, KV head); blockDim.x == kPostThreads.
__device__ __forceinline__ void combine_unit(const CombineParams& p, int unit, CombineShared& sh) {
  const StoreGeom& g = p.g;
  const int D = g.head_dim, G = p.group, Hkv = g.num_kv_heads;
  const int hpb = combine_heads_per_block(D), groups = (G + hpb - 1) / hpb;
  const int seg = unit / groups, hg = unit - seg * groups;
  const int b = seg / Hkv, h = seg - b * Hkv;
  const int tid = threadIdx.x, sub = tid / D, d = tid - sub * D;
  const int gq = hg * hpb + sub;
  const bool valid = gq < G;
  const int gqc = valid ? gq : G - 1;  // threads of a missing head go through the motions of the last one
  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.num_ctas, g.num_seqs * Hkv);
  const int nsplit = pv.seg_count[seg] * p.per_run;
  const int r0 = nsplit > 0 ? pv.seg_begin[seg] * p.per_run : 0;
  const int pstride = partial_stride(G, D);
  const float* base = p.partials + (long long)r0 * pstride + gqc * (D + 2);
  const bool has_cur = p.cur_k != nullptr && p.cur_v != nullptr;
  const long long hq = (long long)b * p.num_q_heads + h * G + gqc;
  const long long kv = ((long long)b * Hkv + h) * D + d;

  float prod = 0.f;
  if (has_cur) {
    const float q = p.q_is_half ? __half2float(static_cast<const __half*>(p.query)[hq * D + d])
                                : static_cast<const float*>(p.query)[hq * D + d];
    const float k = p.kv_is_half ? __half2float(static_cast<const __half*>(p.cur_k)[kv])
                                 : static_cast<const float*>(p.cur_k)[kv];
    prod = q * k;
  }
  // (max, sum) headers of this thread's share of the partials: one 8-byte load each, kept in registers
  // when the segment has at most kCombineChunk partials (the usual case), so that the chain of
  // dependent loads is plan -> headers -> rows and nothing more
  constexpr int kHdrRegs = kCombineChunk / 64;  // D >= 64
  const bool small = nsplit <= kCombineChunk;
  float2 hdr[kHdrRegs];
  float mloc = -INFINITY;
  if (small) {
#pragma unroll
    for (int j = 0; j < kHdrRegs; ++j) {
      const int k = d + j * D;
      hdr[j] = k < nsplit ? *reinterpret_cast<const float2*>(base + (long long)k * pstride) : make_float2(-INFINITY, 0.f);
      mloc = fmaxf(mloc, hdr[j].x);
    }
  } else {
    for (int k = d; k < nsplit; k += D) mloc = fmaxf(mloc, base[(long long)k * pstride]);
  }
  float s_cur = head_dot(prod, sub, d, D, sh.red, 0) * p.scale_log2;
  if (has_cur && p.cur_mask != nullptr) s_cur = fmaf(p.cur_mask[b], 1.4426950408889634f, s_cur);
  {
    const float m = warp_max(mloc);
    const int wph = D >> 5;
    if ((d & 31) == 0) sh.red[sub * wph + (d >> 5)][1] = m;
    __syncthreads();
    mloc = -INFINITY;
    for (int w = 0; w < wph; ++w) mloc = fmaxf(mloc, sh.red[sub * wph + w][1]);
  }
  float M = mloc;
  if (has_cur) M = fmaxf(M, s_cur);

  // fold the partials in a fixed order, kCombineChunk at a time; the weights of a chunk go through
  // shared memory so that the row loads do not depend on anything loaded in the same loop
  float acc = 0.f, L = 0.f;
  for (int c0 = 0; c0 < nsplit; c0 += kCombineChunk) {
    const int cn = (nsplit - c0) < kCombineChunk ? (nsplit - c0) : kCombineChunk;
    __syncthreads();
    if (small) {
#pragma unroll
      for (int j = 0; j < kHdrRegs; ++j) {
        const int k = d + j * D;
        if (k < cn) {
          const float f = hdr[j].x == -INFINITY ? 0.f : ex2f(hdr[j].x - M);
          sh.f[sub][k] = f;
          sh.lf[sub][k] = f == 0.f ? 0.f : hdr[j].y * f;
        }
      }
    } else {
      for (int k = d; k < cn; k += D) {
        const float* row = base + (long long)(c0 + k) * pstride;
        const float mw = row[0];
        const float f = mw == -INFINITY ? 0.f : ex2f(mw - M);
        sh.f[sub][k] = f;
        sh.lf[sub][k] = f == 0.f ? 0.f : row[1] * f;
      }
    }
    __syncthreads();
    const float* col = base + (long long)c0 * pstride + 2 + d;
#pragma unroll 16
    for (int k = 0; k < cn; ++k) {
      const float f = sh.f[sub][k];
      const float x = col[(long long)k * pstride];  // a partial without keys holds stale bytes: select, not multiply
      acc += f == 0.f ? 0.f : x * f;
      L += sh.lf[sub][k];
    }
  }
  float pc = 0.f;
  if (has_cur) {
    pc = ex2f(s_cur - M);
    const float v = p.kv_is_half ? __half2float(static_cast<const __half*>(p.cur_v)[kv])
                                 : static_cast<const float*>(p.cur_v)[kv];
    acc = fmaf(pc, v, acc);
    L += pc;
  }
  if (!valid) return;
  p.out[hq * D + d] = L > 0.f ? acc / L : 0.f;
  if (d == 0) {
    if (p.lse_max) p.lse_max[hq] = M;
    if (p.lse_sum) p.lse_sum[hq] = L;
    if (p.cur_prob) p.cur_prob[hq] = (has_cur && L > 0.f) ? pc / L : 0.f;
  }
}

// ---- importance ---------------------------------------------------------------------------------------
struct ImportanceParams {
  StoreGeom g;
  int layer;
  const int32_t* counts;
  int num_q_heads;
  const float* logits;
  const float* lse_max;
  const float* lse_sum;
  const float* cur_prob;
  const int32_t* cur_slot;
  float* head_state;
  int parity;
  double* cumulative;
  float* layer_ema;
  uint8_t* touched;
  float decay;
  float head_decay;
};

struct ImportanceShared {
  float w[kMaxQHeads];      // head weight / final sum
  float mx[kMaxQHeads];     // final max
  float cprob[kMaxQHeads];  // pc (unnormalised probability of the current token)
};

// Maps the j-th *live* chunk of sequence b (chunks of kPostThreads storage indices that hold a cached
// key or the slot the current token will take) to its chunk index; -1 when j is past the last one.
// Buckets lie at increasing storage indices, so their chunk ranges are increasing and only neighbours can
// share a chunk.  j == 0 always maps to a chunk (chunk 0 if nothing is live): that block publishes the
// head-importance EMA.
__device__ __forceinline__ int live_chunk(const StoreGeom& g, const int32_t* counts4, int j) {
  int prev_last = -1, seen = 0;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) {
    const int cnt = counts4[i] + 1;  // + the slot a token appended this step would take
    if (g.cap[i] == 0) continue;
    int first = g.bucket_base[i] / kPostThreads;
    const int last = (g.bucket_base[i] + cnt - 1) / kPostThreads;
    if (first <= prev_last) first = prev_last + 1;
    if (last >= first) {
      const int n = last - first + 1;
      if (j < seen + n) return first + (j - seen);
      seen += n;
      prev_last = last;
    }
  }
  return (j == 0 && seen == 0) ? 0 : -1;
}

// Bucket counts and the current token's slot of one sequence.
struct ImportanceSeq {
  int cnt[kNumBuckets];
  int cur_slot;
  bool has_cur;
};

__device__ __forceinline__ ImportanceSeq importance_seq(const ImportanceParams& p, int b) {
  ImportanceSeq q;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) q.cnt[i] = p.counts[b * kNumBuckets + i];
  q.cur_slot = (p.cur_prob != nullptr && p.cur_slot != nullptr) ? p.cur_slot[b] : -1;
  q.has_cur = q.cur_slot >= 0;
  return q;
}

// True if the 256 storage indices of `chunk` hold a cached key or the slot of the current token.
__device__ __forceinline__ bool importance_chunk_live(const StoreGeom& g, const ImportanceSeq& q, int chunk) {
  const int s_lo = chunk * kPostThreads, s_hi = s_lo + kPostThreads;
  bool live = q.has_cur && q.cur_slot >= s_lo && q.cur_slot < s_hi;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i)
    live |= q.cnt[i] > 0 && g.bucket_base[i] < s_hi && g.bucket_base[i] + q.cnt[i] > s_lo;
  return live;
}

// Head weights of sequence b into shared memory: w = weight / final sum, mx = final max, cprob = unnormalised
// probability of the current token (all threads of the block; ends with a barrier).  `publish` marks the one block
// per sequence that writes the new head-importance EMA.
__device__ __forceinline__ void importance_prologue(const ImportanceParams& p, int b, const ImportanceSeq& q, bool publish,
                                                    ImportanceShared& sh) {
  const int tid = threadIdx.x, Hq = p.num_q_heads;
  int nkeys = 0;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) nkeys += q.cnt[i];
  const int total_keys = nkeys + (q.has_cur ? 1 : 0);
  // final (max, sum) of every query head and the probability of the current token, as the combine
  // step of this layer left them (issued early: independent of the EMA chain below)
  float lse_l = 0.f, lse_m = 0.f, pcur = 0.f;
  if (tid < Hq) {
    lse_l = p.lse_sum[(long long)b * Hq + tid];
    lse_m = p.lse_max[(long long)b * Hq + tid];
    pcur = q.has_cur ? p.cur_prob[(long long)b * Hq + tid] * lse_l : 0.f;
  }
  // head-importance EMA (cache.py:242-248).  Every softmax row sums to one, so the
  // mean over keys of a head's probabilities is 1 / (number of keys).
  const float* hs_old = p.head_state + ((long long)b * 2 + p.parity) * Hq;
  float* hs_new = p.head_state + ((long long)b * 2 + (p.parity ^ 1)) * Hq;
  const float head_mean = total_keys > 0 ? 1.0f / (float)total_keys : 0.f;
  float hn = 0.f;
  if (tid < Hq) {
    hn = hs_old[tid] * p.head_decay + head_mean * (1.0f - p.head_decay);
    sh.mx[tid] = hn;  // staged, replaced below
    if (publish) hs_new[tid] = hn;
  }
  __syncthreads();
  float my_w = 0.f;
  if (tid < Hq) {
    float acc = 0.f;
    for (int h = 0; h < Hq; ++h) acc += sh.mx[h];  // same order in every thread: one mean per block
    my_w = hn / (acc / (float)Hq + 1e-6f);
  }
  __syncthreads();
  if (tid < Hq) {
    sh.w[tid] = lse_l > 0.f ? my_w / lse_l : 0.f;
    sh.mx[tid] = lse_m;
    sh.cprob[tid] = pcur;
  }
  __syncthreads();
}

// KPT chunks of 256 storage indices at once, one storage index of each per thread: the loads of all of them are in
// flight together (the update of one key is two dependent round trips to memory and a handful of bytes; a large
// batch is thousands of such blocks otherwise, each waiting out the same latencies).  chunks[k] < 0: nothing to do.
// Per key the sum over the heads runs in head order whatever KPT is, so the results do not depend on it.
template <int KPT>
__device__ __forceinline__ void importance_chunks(const ImportanceParams& p, const int (&chunks)[KPT], int b,
                                                  const ImportanceSeq& q, const ImportanceShared& sh) {
  const StoreGeom& g = p.g;
  const int Hq = p.num_q_heads;
  int s[KPT];
  bool valid[KPT], is_cur[KPT];
  double cum[KPT];
  float ema[KPT], mass[KPT];
  uint8_t seen[KPT];
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    s[k] = chunks[k] * kPostThreads + threadIdx.x;  // storage index
    valid[k] = false;
    if (chunks[k] >= 0 && s[k] < g.slots) {
#pragma unroll
      for (int i = 0; i < kNumBuckets; ++i) valid[k] |= (s[k] >= g.bucket_base[i] && s[k] < g.bucket_base[i] + q.cnt[i]);
    }
    is_cur[k] = chunks[k] >= 0 && !valid[k] && q.has_cur && s[k] == q.cur_slot;
    mass[k] = 0.f;
    cum[k] = 0.0;
    ema[k] = 0.f;
    seen[k] = 0;
  }
  const long long seq_base = (long long)b * g.slots;
  const long long lay_base = ((long long)p.layer * g.num_seqs + b) * g.slots;
  // the state these threads update is fetched before the logits so that the latencies overlap
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    if (valid[k] || is_cur[k]) {
      cum[k] = p.cumulative[seq_base + s[k]];
      ema[k] = p.layer_ema[lay_base + s[k]];
      seen[k] = p.touched[lay_base + s[k]];
    }
  }
  const float* lg = p.logits + (long long)b * Hq * g.slots;
  // The loads of the loop below carry no condition (a thread without a key reads index 0 and drops the result), so
  // that the compiler can put a batch of them in flight before the first use.
  int sv[KPT];
  bool any_valid = false;
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    sv[k] = valid[k] ? s[k] : 0;
    any_valid |= valid[k];
  }
  if (any_valid) {
    constexpr int kHeadsInFlight = 16 / KPT;  // 16 logit loads in flight per thread either way
#pragma unroll kHeadsInFlight
    for (int h = 0; h < Hq; ++h) {
      const float wv = sh.w[h], mv = sh.mx[h];
      const float* row = lg + (long long)h * g.slots;
#pragma unroll
      for (int k = 0; k < KPT; ++k) mass[k] += wv * ex2f(row[sv[k]] - mv);
    }
  }
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    if (!valid[k]) mass[k] = 0.f;
    if (is_cur[k]) {
      // the newest token: it is stored at this storage index when the step's append commits
      for (int h = 0; h < Hq; ++h) mass[k] += sh.w[h] * sh.cprob[h];
    }
  }
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    if (valid[k] || is_cur[k]) {
      p.cumulative[seq_base + s[k]] = cum[k] + (double)mass[k];
      if (seen[k]) {
        p.layer_ema[lay_base + s[k]] = p.decay * ema[k] + (1.0f - p.decay) * mass[k];
      } else {
        p.layer_ema[lay_base + s[k]] = mass[k];
        p.touched[lay_base + s[k]] = 1;
      }
    }
  }
}

// One unit = 256 consecutive storage indices of one sequence; blockDim.x == kPostThreads.  (The common case, kept as one
// straight-line function: the wide variant above costs this path a per cent when both go through the same code.)
// `publish` marks the one block per sequence that writes the new head-importance EMA.
__device__ __forceinline__ void importance_unit(const ImportanceParams& p, int chunk, int b, bool publish,
                                                ImportanceShared& sh) {
  const StoreGeom& g = p.g;
  const int tid = threadIdx.x, Hq = p.num_q_heads;
  int cnt[kNumBuckets];
  int nkeys = 0;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) {
    cnt[i] = p.counts[b * kNumBuckets + i];
    nkeys += cnt[i];
  }
  const int cur_slot = (p.cur_prob != nullptr && p.cur_slot != nullptr) ? p.cur_slot[b] : -1;
  const bool has_cur = cur_slot >= 0;
  const int total_keys = nkeys + (has_cur ? 1 : 0);

  // most storage indices of a sequence are unused capacity: a block without a live key leaves at once
  // (the publishing block of every sequence stays)
  const int s_lo = chunk * kPostThreads, s_hi = s_lo + kPostThreads;
  bool block_live = publish || (has_cur && cur_slot >= s_lo && cur_slot < s_hi);
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i)
    block_live |= cnt[i] > 0 && g.bucket_base[i] < s_hi && g.bucket_base[i] + cnt[i] > s_lo;
  if (!block_live) return;

  // final (max, sum) of every query head and the probability of the current token, as the combine
  // step of this layer left them (issued early: independent of the EMA chain below)
  float lse_l = 0.f, lse_m = 0.f, pcur = 0.f;
  if (tid < Hq) {
    lse_l = p.lse_sum[(long long)b * Hq + tid];
    lse_m = p.lse_max[(long long)b * Hq + tid];
    pcur = has_cur ? p.cur_prob[(long long)b * Hq + tid] * lse_l : 0.f;
  }

  // head-importance EMA (cache.py:242-248).  Every softmax row sums to one, so the
  // mean over keys of a head's probabilities is 1 / (number of keys).
  const float* hs_old = p.head_state + ((long long)b * 2 + p.parity) * Hq;
  float* hs_new = p.head_state + ((long long)b * 2 + (p.parity ^ 1)) * Hq;
  const float head_mean = total_keys > 0 ? 1.0f / (float)total_keys : 0.f;
  float hn = 0.f;
  if (tid < Hq) {
    hn = hs_old[tid] * p.head_decay + head_mean * (1.0f - p.head_decay);
    sh.mx[tid] = hn;  // staged, replaced below
    if (publish) hs_new[tid] = hn;
  }
  __syncthreads();
  float my_w = 0.f;
  if (tid < Hq) {
    float acc = 0.f;
    for (int h = 0; h < Hq; ++h) acc += sh.mx[h];  // same order in every thread: one mean per block
    my_w = hn / (acc / (float)Hq + 1e-6f);
  }
  __syncthreads();
  if (tid < Hq) {
    sh.w[tid] = lse_l > 0.f ? my_w / lse_l : 0.f;
    sh.mx[tid] = lse_m;
    sh.cprob[tid] = pcur;
  }
  __syncthreads();

  const int s = s_lo + tid;  // storage index
  bool valid = false;
  if (s < g.slots) {
#pragma unroll
    for (int i = 0; i < kNumBuckets; ++i) valid |= (s >= g.bucket_base[i] && s < g.bucket_base[i] + cnt[i]);
  }
  float mass = 0.f;
  const bool is_cur = !valid && has_cur && s == cur_slot;
  const bool write = valid || is_cur;
  const long long ci = (long long)b * g.slots + s;
  const long long li = ((long long)p.layer * g.num_seqs + b) * g.slots + s;
  // the state this thread updates is fetched before the logits so that the two latencies overlap
  double cum = 0.0;
  float ema = 0.f;
  uint8_t seen = 0;
  if (write) {
    cum = p.cumulative[ci];
    ema = p.layer_ema[li];
    seen = p.touched[li];
  }
  if (valid) {
    const float* lg = p.logits + (long long)b * Hq * g.slots + s;
#pragma unroll 16
    for (int h = 0; h < Hq; ++h) mass += sh.w[h] * ex2f(lg[(long long)h * g.slots] - sh.mx[h]);
  } else if (is_cur) {
    // the newest token: it is stored at this storage index when the step's append commits
    for (int h = 0; h < Hq; ++h) mass += sh.w[h] * sh.cprob[h];
  }
  if (write) {
    p.cumulative[ci] = cum + (double)mass;
    if (seen) {
      p.layer_ema[li] = p.decay * ema + (1.0f - p.decay) * mass;
    } else {
      p.layer_ema[li] = mass;
      p.touched[li] = 1;
    }
  }
}

// ---- append ---------------------------------------------------------------------------------------------
struct AppendParams {
  StoreGeom g;
  uint8_t* store;
  int layer;
  const void* k;
  const void* v;
  int dtype;
  int rows;
  const int32_t* dst_seq;
  const int32_t* dst_bucket;
  const int32_t* dst_pos;
  int32_t* err;
};

// One warp quantises and packs one row (one of K / V of one KV head of one new token).
template <int EPL>
__device__ __forceinline__ void append_row(const AppendParams& p, long long warp, int lane) {
  const StoreGeom& g = p.g;
  const int which = (int)(warp & 1);  // 0 = K, 1 = V
  const long long rh = warp >> 1;
  int h, r;
  if (rh >> 31) {  // 64-bit division is a long subroutine: only where the row count needs it
    h = (int)(rh % g.num_kv_heads);
    r = (int)(rh / g.num_kv_heads);
  } else {
    r = (int)rh / g.num_kv_heads;
    h = (int)rh - r * g.num_kv_heads;
  }
  // the row's values do not depend on where it goes: both loads are in flight together
  RowVals<EPL> x = load_row<EPL>(which ? p.v : p.k, p.dtype, rh, lane);
  const int seq = p.dst_seq[r], bucket = p.dst_bucket[r], pos = p.dst_pos[r];
  if (seq < 0 || seq >= g.num_seqs || bucket < 0 || bucket >= kNumBuckets || pos < 0 || pos >= g.cap[bucket]) {
    if (lane == 0 && p.err) atomicExch(p.err, 2);
    return;
  }
  const int bits = bucket_bits(bucket);
  int code[EPL];
  const float scale = quantize_row<EPL>(x, bits, code);
  uint8_t* arena = arena_ptr(g, p.store, p.layer, seq);
  const long long row_index = (long long)h * g.cap[bucket] + pos;
  uint8_t* dst = arena + (which ? g.v_off[bucket] : g.k_off[bucket]) + row_index * g.row_bytes[bucket];
  pack_store_row<EPL>(code, bits, dst, lane);
  if (lane == 0) {
    float* sc = reinterpret_cast<float*>(arena + g.sc_off[bucket]);
    sc[2 * row_index + which] = scale;
    if (which) note_v_scale(g, arena, scale);
  }
}

}  // namespace skv
