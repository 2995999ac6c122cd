// Everything between two streaming attention kernels in one launch: the LSE combine and the
// quantise-pack append of this layer, and the importance update of the layer before it (whose
// combine results are complete by now).  The three are independent, so their blocks run side by
// side and a decode step costs two launches per layer instead of four.
#include "post_attention.cuh"

#include <atomic>

extern std::atomic<int> g_dependent_launch;  // decode_attention.cu

namespace skv {

constexpr int kImpWide = 4;  // chunks per importance block once the grid would exceed two waves

struct PostParams {
  CombineParams c;
  ImportanceParams imp;
  AppendParams app;
  int combine_blocks;
  int imp_chunks;      // importance blocks = imp_chunks * num_seqs (0: no importance update)
  int imp_compact;     // 1: block j of a sequence takes that sequence's j-th live chunk
  int imp_kpt;         // chunks per importance block (1 or kImpWide): one storage index of each per thread
  int append_blocks;   // 8 rows-of-a-head per block (0: no append)
};

union PostShared {
  CombineShared c;
  ImportanceShared i;
};

// WIDE: importance blocks of kImpWide chunks (large batches); its own instantiation, so that the common kernel's
// register allocation is not touched by it
template <int EPL, bool WIDE>
__global__ void __launch_bounds__(kPostThreads) post_attention_kernel(const PostParams p) {
  __shared__ PostShared sh;
  // dependent launch: the next layer's attention kernel may be scheduled as soon as every block here has started (it
  // touches nothing this kernel uses until it has waited for this grid itself); this kernel needs the attention kernel
  // before it complete
  pdl_launch_dependents();
  pdl_wait();
  int blk = blockIdx.x;
  if (blk < p.combine_blocks) {
    combine_unit(p.c, blk, sh.c);
    return;
  }
  blk -= p.combine_blocks;
  const int per_seq = (p.imp_chunks + p.imp_kpt - 1) / p.imp_kpt;
  const int imp_blocks = per_seq * p.c.g.num_seqs;
  if (blk < imp_blocks) {
    const int b = blk / per_seq, j = blk - b * per_seq;
    if constexpr (!WIDE) {
      // a compact grid walks the live chunks only; the full grid visits every chunk
      const int chunk = p.imp_compact ? live_chunk(p.c.g, p.imp.counts + b * kNumBuckets, j) : j;
      if (chunk >= 0) importance_unit(p.imp, chunk, b, j == 0, sh.i);
      return;
    } else {
    // wide blocks (large batches): kImpWide chunks per block
    const ImportanceSeq q = importance_seq(p.imp, b);
    int chunks[kImpWide];
    bool any = j == 0;  // the first block of a sequence publishes the head-importance EMA whatever it holds
#pragma unroll
    for (int k = 0; k < kImpWide; ++k) {
      const int jj = j * kImpWide + k;
      int c = jj < p.imp_chunks ? (p.imp_compact ? live_chunk(p.c.g, p.imp.counts + b * kNumBuckets, jj) : jj) : -1;
      if (c >= 0 && !importance_chunk_live(p.c.g, q, c)) c = -1;
      chunks[k] = c;
      any |= c >= 0;
    }
    if (!any) return;
    importance_prologue(p.imp, b, q, j == 0, sh.i);
    importance_chunks<kImpWide>(p.imp, chunks, b, q, sh.i);
    return;
    }
  }
  blk -= imp_blocks;
  const long long warp = (long long)blk * (kPostThreads / 32) + (threadIdx.x >> 5);
  if (warp < (long long)p.app.rows * p.app.g.num_kv_heads * 2) append_row<EPL>(p.app, warp, threadIdx.x & 31);
}

}  // namespace skv

using namespace skv;

extern "C" int skv_post_attention(const SkvStoreDesc* desc, void* store, int layer, const void* plan,
                                  const void* query, int query_dtype, int num_q_heads, const void* partials,
                                  int num_ctas, const void* cur_k, const void* cur_v, int kv_dtype, float* out,
                                  float* lse_max, float* lse_sum, float* cur_prob, const int32_t* counts,
                                  int imp_layer, const float* imp_logits, const float* imp_lse_max,
                                  const float* imp_lse_sum, const float* imp_cur_prob, const int32_t* cur_slot,
                                  float* head_state, int parity,
                                  double* cumulative, float* layer_ema, uint8_t* touched, float decay,
                                  float head_decay, const int32_t* dst_seq, const int32_t* dst_bucket,
                                  const int32_t* dst_pos, int max_seq_tokens, int32_t* err_flag, void* stream) {
  if (!desc || !plan || !query || !partials || !out) return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || num_ctas <= 0) return SKV_ERR_INVALID;
  if (num_q_heads % desc->num_kv_heads != 0 || num_q_heads > kMaxQHeads) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  if (group < 1 || group > 8) return SKV_ERR_UNSUPPORTED;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if ((cur_k == nullptr) != (cur_v == nullptr)) return SKV_ERR_INVALID;
  const bool with_importance = imp_logits != nullptr;
  if (with_importance && (!counts || !head_state || !cumulative || !layer_ema || !touched || !imp_lse_max ||
                          !imp_lse_sum || imp_layer < 0 || imp_layer >= desc->num_layers))
    return SKV_ERR_INVALID;
  if (with_importance && (imp_lse_max == lse_max || imp_lse_sum == lse_sum || (imp_cur_prob && imp_cur_prob == cur_prob)))
    return SKV_ERR_INVALID;  // the importance step reads an earlier launch's results, not this launch's
  if (with_importance && parity != 0 && parity != 1) return SKV_ERR_INVALID;
  const bool with_append = dst_seq != nullptr;
  if (with_append && (!store || !dst_bucket || !dst_pos || !cur_k)) return SKV_ERR_INVALID;

  PostParams p = {};
  CombineParams& c = p.c;
  c.g = make_geom(*desc);
  c.plan = static_cast<const int*>(plan);
  c.query = query;
  c.q_is_half = query_dtype == SKV_DTYPE_F16;
  c.num_q_heads = num_q_heads;
  c.group = group;
  c.partials = static_cast<const float*>(partials);
  c.per_run = skv_attn_partials_per_run(desc, query_dtype);
  c.num_ctas = num_ctas;
  c.cur_k = cur_k;
  c.cur_v = cur_v;
  c.kv_is_half = kv_dtype == SKV_DTYPE_F16;
  c.out = out;
  c.lse_max = lse_max;
  c.lse_sum = lse_sum;
  c.cur_prob = cur_prob;
  c.scale_log2 = (float)(1.4426950408889634 / sqrt((double)desc->head_dim));
  p.combine_blocks = combine_units(c.g, group);
  if (with_importance) {
    ImportanceParams& i = p.imp;
    i.g = c.g;
    i.layer = imp_layer;
    i.counts = counts;
    i.num_q_heads = num_q_heads;
    i.logits = imp_logits;
    i.lse_max = imp_lse_max;
    i.lse_sum = imp_lse_sum;
    i.cur_prob = imp_cur_prob;
    i.cur_slot = cur_slot;
    i.head_state = head_state;
    i.parity = parity;
    i.cumulative = cumulative;
    i.layer_ema = layer_ema;
    i.touched = touched;
    i.decay = decay;
    i.head_decay = head_decay;
    p.imp_chunks = (desc->slots + kPostThreads - 1) / kPostThreads;
    if (max_seq_tokens > 0) {
      // live chunks of a sequence: its tokens spread over the buckets, every bucket may begin and end inside a chunk
      const int compact = (max_seq_tokens + 1 + kPostThreads - 1) / kPostThreads + 2 * kNumBuckets + 2;
      if (compact < p.imp_chunks) {
        p.imp_chunks = compact;
        p.imp_compact = 1;
      }
    }
  }
  if (with_append) {
    AppendParams& a = p.app;
    a.g = c.g;
    a.store = static_cast<uint8_t*>(store);
    a.layer = layer;
    a.k = cur_k;
    a.v = cur_v;
    a.dtype = kv_dtype;
    a.rows = desc->num_seqs;
    a.dst_seq = dst_seq;
    a.dst_bucket = dst_bucket;
    a.dst_pos = dst_pos;
    a.err = err_flag;
    const long long warps = (long long)a.rows * desc->num_kv_heads * 2;
    p.append_blocks = (int)((warps + kPostThreads / 32 - 1) / (kPostThreads / 32));
  }
  p.imp_kpt = 1;
  if (with_importance && (long long)p.imp_chunks * desc->num_seqs > 2LL * num_ctas * 4) p.imp_kpt = kImpWide;
  const int imp_grid = with_importance ? ((p.imp_chunks + p.imp_kpt - 1) / p.imp_kpt) * desc->num_seqs : 0;
  const int grid = p.combine_blocks + imp_grid + p.append_blocks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool dep = g_dependent_launch.load() == 1 || g_dependent_launch.load() == 3;
  const bool wide = p.imp_kpt != 1;
  if (desc->head_dim == 128)
    launch_maybe_dependent(wide ? post_attention_kernel<4, true> : post_attention_kernel<4, false>, dim3(grid),
                           dim3(kPostThreads), 0, st, p, dep);
  else
    launch_maybe_dependent(wide ? post_attention_kernel<2, true> : post_attention_kernel<2, false>, dim3(grid),
                           dim3(kPostThreads), 0, st, p, dep);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
