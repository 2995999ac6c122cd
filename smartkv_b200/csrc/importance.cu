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
#include "post_attention.cuh"

namespace skv {

// grid = (ceil(slots / 256), num_seqs)
__global__ void __launch_bounds__(kPostThreads) importance_update_kernel(const ImportanceParams p) {
  __shared__ ImportanceShared sh;
  importance_unit(p, blockIdx.x, blockIdx.y, blockIdx.x == 0, sh);
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
  ImportanceParams p = {};
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
  dim3 grid((desc->slots + kPostThreads - 1) / kPostThreads, desc->num_seqs);
  importance_update_kernel<<<grid, kPostThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
