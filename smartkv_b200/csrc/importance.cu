// Fused importance update for the decode path.
//
// Replaces, for one (layer, decode step), the reference's
//   SmartKVCache.update_attention head weighting   (smartkv/core/cache.py:232-253)
//   ImportanceTracker.update_attention             (smartkv/core/importance.py:44-101)
// which copy the whole probability tensor to the host and loop over tokens in
// Python.  Here the probabilities are never materialised: the attention kernel
// left scaled logits per (query head, key) in storage order, the combine left the
// final max and sum per query head, and this kernel rebuilds
//   p = exp2(logit - max) / sum
// sums it over the query heads with the head weights and folds the per-key mass
// into the cumulative importance (fp64, what the allocator reads) and the
// per-layer EMA (decay 0.9 by default), both kept in storage order.
#include "common.cuh"

namespace skv {

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

constexpr int kImpThreads = 256;
constexpr int kMaxQHeads = 128;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// grid = (ceil(slots / 256), num_seqs)
__global__ void importance_update_kernel(const ImportanceParams p) {
  const StoreGeom& g = p.g;
  const int b = blockIdx.y, tid = threadIdx.x, Hq = p.num_q_heads;
  __shared__ float s_w[kMaxQHeads];    // head weight / final sum
  __shared__ float s_max[kMaxQHeads];

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
  // (block 0 of every sequence stays, it publishes the head-importance EMA)
  const int s_lo = blockIdx.x * kImpThreads, s_hi = s_lo + kImpThreads;
  bool block_live = blockIdx.x == 0 || (has_cur && cur_slot >= s_lo && cur_slot < s_hi);
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i)
    block_live |= cnt[i] > 0 && g.bucket_base[i] < s_hi && g.bucket_base[i] + cnt[i] > s_lo;
  if (!block_live) return;

  // head-importance EMA (cache.py:242-248).  Every softmax row sums to one, so the
  // mean over keys of a head's probabilities is 1 / (number of keys).
  const float* hs_old = p.head_state + ((long long)b * 2 + p.parity) * Hq;
  float* hs_new = p.head_state + ((long long)b * 2 + (p.parity ^ 1)) * Hq;
  const float head_mean = total_keys > 0 ? 1.0f / (float)total_keys : 0.f;
  float hn = 0.f, lse_l = 0.f, lse_m = 0.f;
  if (tid < Hq) {
    lse_l = p.lse_sum[(long long)b * Hq + tid];  // issued early: independent of the EMA chain below
    lse_m = p.lse_max[(long long)b * Hq + tid];
    hn = hs_old[tid] * p.head_decay + head_mean * (1.0f - p.head_decay);
    s_max[tid] = hn;  // staged, replaced below
    if (blockIdx.x == 0) hs_new[tid] = hn;
  }
  __syncthreads();
  float my_w = 0.f;
  if (tid < Hq) {
    float acc = 0.f;
    for (int h = 0; h < Hq; ++h) acc += s_max[h];  // same order in every thread: one mean per block
    my_w = hn / (acc / (float)Hq + 1e-6f);
  }
  __syncthreads();
  if (tid < Hq) {
    s_w[tid] = lse_l > 0.f ? my_w / lse_l : 0.f;
    s_max[tid] = lse_m;
  }
  __syncthreads();

  const int s = blockIdx.x * kImpThreads + tid;  // storage index
  bool valid = false;
  if (s < g.slots) {
#pragma unroll
    for (int i = 0; i < kNumBuckets; ++i) valid |= (s >= g.bucket_base[i] && s < g.bucket_base[i] + cnt[i]);
  }
  float mass = 0.f;
  bool write = false;
  if (valid) {
    const float* lg = p.logits + (long long)b * Hq * g.slots + s;
#pragma unroll 8
    for (int h = 0; h < Hq; ++h) mass += s_w[h] * ex2_approx(lg[(long long)h * g.slots] - s_max[h]);
    write = true;
  } else if (has_cur && s == cur_slot) {
    // the newest token: its probability came out of the combine; it is stored at
    // this storage index when the step's append commits
    for (int h = 0; h < Hq; ++h) {
      const float L = p.lse_sum[(long long)b * Hq + h];
      mass += (L > 0.f ? s_w[h] * L : 0.f) * p.cur_prob[(long long)b * Hq + h];
    }
    write = true;
  }
  if (write) {
    const long long ci = (long long)b * g.slots + s;
    p.cumulative[ci] += (double)mass;
    const long long li = ((long long)p.layer * g.num_seqs + b) * g.slots + s;
    if (p.touched[li]) {
      p.layer_ema[li] = p.decay * p.layer_ema[li] + (1.0f - p.decay) * mass;
    } else {
      p.layer_ema[li] = mass;
      p.touched[li] = 1;
    }
  }
}

}  // namespace skv

using namespace skv;

extern "C" int skv_importance_update(const SkvStoreDesc* desc, int layer, const int32_t* counts, int num_q_heads,
                                     const float* logits, const float* lse_max, const float* lse_sum,
                                     const float* cur_prob, const int32_t* cur_slot, float* head_state, int parity,
                                     double* cumulative, float* layer_ema, uint8_t* touched, float decay,
                                     float head_decay, void* stream) {
  if (!desc || !counts || !logits || !lse_max || !lse_sum || !head_state || !cumulative || !layer_ema || !touched)
    return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || num_q_heads <= 0 || num_q_heads > kMaxQHeads) return SKV_ERR_INVALID;
  if (parity != 0 && parity != 1) return SKV_ERR_INVALID;
  ImportanceParams p;
  p.g = make_geom(*desc);
  p.layer = layer;
  p.counts = counts;
  p.num_q_heads = num_q_heads;
  p.logits = logits;
  p.lse_max = lse_max;
  p.lse_sum = lse_sum;
  p.cur_prob = cur_prob;
  p.cur_slot = cur_slot;
  p.head_state = head_state;
  p.parity = parity;
  p.cumulative = cumulative;
  p.layer_ema = layer_ema;
  p.touched = touched;
  p.decay = decay;
  p.head_decay = head_decay;
  dim3 grid((desc->slots + kImpThreads - 1) / kImpThreads, desc->num_seqs);
  importance_update_kernel<<<grid, kImpThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
