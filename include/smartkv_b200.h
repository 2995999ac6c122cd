/*
 * smartkv_b200 -- C ABI of the B200 (sm_100a) quantized-KV decode path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*; NULL = the legacy default stream), returns an int status
 * (0 = SKV_OK, negative = error, see skv_status_string) and never throws.
 * Unless stated otherwise an entry point allocates nothing, launches on the
 * given stream and returns without synchronising; inputs are borrowed and
 * outputs are caller-owned device buffers.
 *
 * The entry points replace the functions the reference exports from its
 * pybind11 module `smartkv_cuda` (smartkv/csrc/bindings.cpp:11-111) and the
 * Python hot loops around them; each declaration cites what it replaces.
 *
 * Storage model ("the store").  One byte arena per (layer, sequence).  Inside
 * an arena every bit-width w in {2,3,4,8} owns a *bucket*: three contiguous,
 * 256-byte aligned regions
 *     K rows   [num_kv_heads][cap_w][row_bytes_w]   packed codes
 *     V rows   [num_kv_heads][cap_w][row_bytes_w]
 *     scales   [num_kv_heads][cap_w][2]             fp32 (K scale, V scale) of the same row
 * row_bytes_w = head_dim*w/8.  Rows use the reference's packed format
 * (smartkv/csrc/bit_packing.cu:20-43,69-95,128-151: code + 2^(w-1), low bits
 * first, 8 three-bit codes per 24-bit little-endian group; 8-bit rows are the
 * raw int8 codes).  A token lives in exactly one bucket, at the same bucket
 * position in every layer.  The position of a token inside the store is its
 * *storage index*  s = bucket_base[w] + position,  bucket_base = prefix sum of
 * the capacities; per-token arrays (token ids, importance) are kept in storage
 * order so the kernels stream them.
 */
#ifndef SMARTKV_B200_H_
#define SMARTKV_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKV_NUM_BUCKETS 4 /* bucket index 0..3 <-> 2,3,4,8 bits */

enum {
  SKV_OK = 0,
  SKV_ERR_INVALID = -1,   /* bad argument (null pointer, unsupported shape, ...) */
  SKV_ERR_CUDA = -2,      /* a CUDA runtime call or launch failed */
  SKV_ERR_CAPACITY = -3,  /* a bucket / scratch capacity would be exceeded */
  SKV_ERR_TIMEOUT = -4,   /* a bounded device-side wait gave up (see skv_read_error_flag) */
  SKV_ERR_UNSUPPORTED = -5
};

enum { SKV_DTYPE_F32 = 0, SKV_DTYPE_F16 = 1 };

/* Geometry of the store.  Fill the first block, call skv_store_layout(). */
typedef struct SkvStoreDesc {
  int32_t num_layers;
  int32_t num_seqs;
  int32_t num_kv_heads;            /* KV heads resident on this GPU */
  int32_t head_dim;                /* 64 or 128 */
  int32_t cap[SKV_NUM_BUCKETS];    /* tokens per bucket, each a multiple of 128 */
  /* derived */
  int32_t row_bytes[SKV_NUM_BUCKETS];
  int32_t bucket_base[SKV_NUM_BUCKETS]; /* first storage index of each bucket */
  int32_t slots;                        /* sum of cap = storage indices per sequence */
  int32_t reserved_;
  int64_t k_off[SKV_NUM_BUCKETS];
  int64_t v_off[SKV_NUM_BUCKETS];
  int64_t sc_off[SKV_NUM_BUCKETS];
  int64_t arena_bytes;             /* one (layer, sequence) arena */
  int64_t total_bytes;             /* num_layers * num_seqs * arena_bytes */
} SkvStoreDesc;

const char* skv_status_string(int status);

/* Library build info: returns the SM architecture the kernels were built for (100). */
int skv_build_arch(void);

/* Host only.  Validates the geometry and fills the derived fields. */
int skv_store_layout(SkvStoreDesc* desc);

/* ---- parity helpers: same semantics as the reference's extension -------- */

/* Replaces quantize_per_head_forward (smartkv/csrc/quantized_attention.cu:402-454,
 * bound at bindings.cpp:25-31) with the CPU path's arithmetic
 * (smartkv/core/_quant_cpu.py:26-29): IEEE fp32 divide, round-half-even.
 * input [rows][head_dim] (fp32 or fp16) -> codes int8 [rows][head_dim], scales fp32 [rows]. */
int skv_quantize_per_head(const void* input, int input_dtype, int64_t rows, int head_dim, int bits,
                          int8_t* codes, float* scales, void* stream);

/* Replace pack_values / unpack_values (smartkv/csrc/bit_packing.cu:305-325,
 * bound at bindings.cpp:93-110).  Flat vectors; packed size as compute_packed_size
 * (smartkv/kernels/bit_packing.py:102-122). */
int skv_pack(const int8_t* codes, int64_t num_elements, int bits, uint8_t* packed, void* stream);
int skv_unpack(const uint8_t* packed, int64_t num_elements, int bits, int8_t* codes, void* stream);

/* ---- append: quantize + pack + write into the bucketed store ------------ */

/* Replaces SmartKVCache.quantize_and_store_batch's quantize / pack / slot-write
 * (smartkv/core/cache.py:1187-1355, per-token pack loop :1279-1310, bucket append
 * :1046-1083).  k,v: [rows][num_kv_heads][head_dim] fp32 or fp16.  Row r goes to
 * sequence dst_seq[r], bucket dst_bucket[r] (0..3), bucket position dst_pos[r];
 * the three index arrays are device int32.  Codes are produced with the fp32
 * scale (bit-exact with the reference CPU quantizer) and packed on the fly. */
int skv_quantize_pack_append(const SkvStoreDesc* desc, void* store, int layer, const void* k, const void* v,
                             int input_dtype, int rows, const int32_t* dst_seq, const int32_t* dst_bucket,
                             const int32_t* dst_pos, void* stream);

/* Bookkeeping of one decode step, the per-token part of quantize_and_store_batch
 * (smartkv/core/cache.py:1214, :1319-1339, :1355) for one new token per sequence.
 * skv_step_plan: where each sequence's token goes: bucket of bits[b] (uint8 [num_seqs]; NULL = the
 * default 4 bits), position = the bucket's live count.  Outputs int32 [num_seqs] each; dst_storage
 * is the storage index.  *err_flag = 3 if a bucket is full.
 * skv_step_commit: after every layer appended the token: records its id (next_token[b]) at that
 * storage index, counts[b][bucket] += 1, next_token[b] += 1. */
int skv_step_plan(const SkvStoreDesc* desc, const int32_t* counts, const uint8_t* bits, int32_t* dst_seq,
                  int32_t* dst_bucket, int32_t* dst_pos, int32_t* dst_storage, int32_t* err_flag, void* stream);
int skv_step_commit(const SkvStoreDesc* desc, int32_t* counts, int32_t* slot_token, int32_t* next_token,
                    const int32_t* dst_bucket, const int32_t* dst_storage, void* stream);

/* Reads rows back out of the store as int8 codes + fp32 scales (the dequantising
 * read side of cache.py:1493-1543 / get_bucket_views :671-744).  Row r is read
 * from (src_seq[r], src_bucket[r], src_pos[r]); outputs [rows][num_kv_heads][head_dim]
 * and [rows][num_kv_heads]. */
int skv_export_rows(const SkvStoreDesc* desc, const void* store, int layer, int rows, const int32_t* src_seq,
                    const int32_t* src_bucket, const int32_t* src_pos, int8_t* k_codes, int8_t* v_codes,
                    float* k_scale, float* v_scale, void* stream);

/* The dequantising read of SmartKVCache.retrieve / retrieve_all (smartkv/core/cache.py:1357-1439,
 * :1493-1543): rows of the store as values, code * scale in fp32, written as fp32 or fp16
 * [rows][num_kv_heads][head_dim]. */
int skv_dequant_rows(const SkvStoreDesc* desc, const void* store, int layer, int rows, const int32_t* src_seq,
                     const int32_t* src_bucket, const int32_t* src_pos, int out_dtype, void* k_out, void* v_out,
                     void* stream);

/* The inverse of skv_export_rows: writes already quantised rows (int8 codes + fp32 scales, the form
 * the reference's cache hands to its kernels, smartkv/core/cache.py:1441-1491) into the store,
 * packing them at the width of the destination bucket.  Codes outside that width's range are clamped. */
int skv_import_rows(const SkvStoreDesc* desc, void* store, int layer, int rows, const int32_t* dst_seq,
                    const int32_t* dst_bucket, const int32_t* dst_pos, const int8_t* k_codes, const int8_t* v_codes,
                    const float* k_scale, const float* v_scale, int32_t* err_flag, void* stream);

/* ---- fused packed decode attention --------------------------------------- */

/* Size queries (host only). */
int skv_attn_num_ctas(int device);                       /* persistent CTAs the kernel launches */
int64_t skv_attn_partials_bytes(const SkvStoreDesc* desc, int num_q_heads, int num_ctas);
int64_t skv_attn_plan_bytes(const SkvStoreDesc* desc, int num_ctas);
/* Partials every run writes (one per consumer warp of the attention launch for that query dtype);
 * skv_lse_combine folds runs * this many partials per (sequence, KV head). */
int skv_attn_partials_per_run(const SkvStoreDesc* desc, int query_dtype);

/* Builds the work partition of one decode step: which tiles of which (sequence, KV head) every
 * persistent CTA streams, balanced by estimated time (tiles of 128 keys where the tensor-memory
 * kernel serves the shape, of 16 keys otherwise).  It depends only on the bucket counts, which are
 * the same for every layer of the step, so one call serves all layers.  No counterpart in the
 * reference (its kernel walks one head per CTA, smartkv/csrc/quantized_attention.cu:679-777).
 *   counts int32 [num_seqs][4] live tokens per bucket (device); plan: device buffer
 *   of skv_attn_plan_bytes() bytes. */
int skv_attn_plan(const SkvStoreDesc* desc, const int32_t* counts, int num_ctas, void* plan, void* stream);

/* Replaces quantized_attention_bucket_forward + the host cross-bucket LSE combine
 * (smartkv/csrc/quantized_attention.cu:460-828, smartkv/kernels/__init__.py:269-386)
 * and the CPU streaming path (smartkv/core/fused_cpu.py:7-167) for q_len == 1.
 *
 * Streams the packed buckets of `layer` for every sequence, split-KV over
 * persistent CTAs as laid out by `plan`, and writes partial (max, sum, out) triples into
 * `partials`: skv_attn_partials_per_run() of them per run; if `logits`
 * is not NULL it also writes the scaled logit (log2 units) of every cached key,
 * logits[seq][q_head][storage index].
 *   query    [num_seqs][num_q_heads][head_dim] fp32 or fp16
 * num_q_heads must be a multiple of num_kv_heads with group size <= 8.
 * Two kernels can serve the call (skv_set_attention_path): the mma.sync fragment kernel (any shape) and,
 * for head_dim 128 with fp16 queries, a kernel on the tcgen05 tensor cores with the keys as the M operand,
 * accumulators in tensor memory and the 8-bit rows landed by tiled TMA loads.  Both read the same store.
 * err_flag: device int32, set non-zero if a bounded wait inside the kernel gave up. */
int skv_decode_attention(const SkvStoreDesc* desc, const void* store, int layer, const void* plan,
                         const void* query, int query_dtype, int num_q_heads, void* partials, int num_ctas,
                         float* logits, int32_t* err_flag, void* stream);

/* skv_decode_attention with the additive attention mask the reference's kernels take
 * (smartkv/csrc/quantized_attention.cu:213-216, 570-575: mask indexed by the key's global slot).
 *   mask fp32 [num_seqs][mask_stride], natural-log units, indexed by TOKEN ID (position in the
 *   sequence); slot_token int32 [num_seqs][slots] gives the token id of every storage index.
 *   mask == NULL: no mask (slot_token may then be NULL).  The mask value of the step's current token is
 *   an argument of the combine step (skv_lse_combine_masked).
 *   flags: SKV_ATTN_DEPENDENT_LAUNCH launches the kernel with the programmatic-serialization attribute: it may start
 *   (set up, put its first copies of this layer's rows in flight) while the kernel before it in the stream is still
 *   running, and waits for that kernel before it reads the query or writes anything.  The caller asserts that the
 *   plan and this layer's rows were NOT written by the kernel directly before this launch (in a decode step: the
 *   previous layer's skv_post_attention, or the model's own kernels between two layers).
 *   skv_set_dependent_launch(mode): 0 = never, 2 = the attention kernel when the flag is given (default), 1 = also
 *   skv_post_attention (it waits before it reads anything, so it needs no flag), 3 = skv_post_attention only.  Measured on
 *   the 8B shape: mode 2 takes 5 % off the step at batch 16 and 6 % at batch 1 x 131072; launching the post-attention
 *   kernel that way (its blocks become resident while the attention kernel still runs) costs 1 % and 10 %. */
#define SKV_ATTN_DEPENDENT_LAUNCH 1
int skv_decode_attention_masked(const SkvStoreDesc* desc, const void* store, int layer, const void* plan,
                                const void* query, int query_dtype, int num_q_heads, void* partials, int num_ctas,
                                float* logits, const float* mask, int64_t mask_stride, const int32_t* slot_token,
                                int flags, int32_t* err_flag, void* stream);
int skv_set_dependent_launch(int on);

/* Kernel selection for skv_decode_attention: 0 = default (the mma.sync fragment kernel), 1 = always the
 * fragment kernel, 2 = the tensor-memory (tcgen05) kernel wherever it applies (head_dim 128, fp16 queries).
 * The tensor-memory kernel streams 8-bit rows at about 0.85 of the HBM copy bandwidth but pays more per
 * narrow block, so it wins once most cached tokens are 8-bit; time both on the live cache to choose
 * (PackedKVStore.autotune_attention does).  Process-wide; plans and partials built under one setting must
 * be consumed under the same setting.  No counterpart in the reference. */
int skv_set_attention_path(int path);
int skv_get_attention_path(void);

/* Limit of every bounded device-side wait of the attention kernels, in polls of about 50 ns (default
 * 2^24, about one second).  When a wait runs out the kernel sets *err_flag, waits (bounded) for its own
 * copies still in flight and returns; nothing faults and the context stays usable.  The fragment kernel
 * honours any limit; the tensor-memory kernel never uses fewer than 2^20 polls.  No counterpart in the
 * reference. */
int skv_set_wait_limit(unsigned polls);

/* Combines the partials with the newest token, which takes part in full precision
 * (smartkv/core/fused_cpu.py:115-137; wrapper call smartkv/models/llama_smartkv.py:264-305),
 * and normalises.  cur_k/cur_v [num_seqs][num_kv_heads][head_dim] (may be NULL: no
 * current token).  out fp32 [num_seqs][num_q_heads][head_dim]; lse_max / lse_sum fp32
 * [num_seqs][num_q_heads]: the reference point m (log2 units; the kernels raise their running
 * maximum lazily, so m may lie below the true maximum) and the sum of 2^(logit - m), i.e.
 * lse_max + log2(lse_sum) is the log-sum-exp; cur_prob fp32
 * [num_seqs][num_q_heads] = probability of the current token (may be NULL). */
int skv_lse_combine(const SkvStoreDesc* desc, const void* plan, const void* query, int query_dtype,
                    int num_q_heads, const void* partials, int num_ctas, const void* cur_k, const void* cur_v,
                    int kv_dtype, float* out, float* lse_max, float* lse_sum, float* cur_prob, void* stream);

/* skv_lse_combine with the additive mask value of the current token: cur_mask fp32 [num_seqs],
 * natural-log units, NULL = none (the counterpart of the last column of the reference's mask,
 * smartkv/core/fused_cpu.py:121-126). */
int skv_lse_combine_masked(const SkvStoreDesc* desc, const void* plan, const void* query, int query_dtype,
                           int num_q_heads, const void* partials, int num_ctas, const void* cur_k, const void* cur_v,
                           int kv_dtype, const float* cur_mask, float* out, float* lse_max, float* lse_sum,
                           float* cur_prob, void* stream);

/* ---- attention without a caller-owned scratch buffer --------------------------- */

/* No counterpart in the reference.  Same launch as skv_decode_attention, but the partials go
 * into a fixed array that is part of the library's device code (16 MiB per device) instead of a
 * buffer the caller allocated.  It is meant for callers that cannot allocate device memory at
 * decode time -- a server that froze its memory pool after start-up, a runtime whose allocator
 * may not be entered from the decode thread.  The call itself allocates nothing and calls no
 * allocating library routine.
 *   *partials_out receives the device address of the array; pass it as `partials` to
 *   skv_lse_combine on the same stream.
 * Limits and rules:
 *   - skv_attn_partials_bytes(desc, num_q_heads, num_ctas) must not exceed 16 MiB, otherwise
 *     the call returns SKV_ERR_CAPACITY, prints the two sizes to stderr and launches nothing.
 *   - The first call on each device looks the array's address up (cudaGetSymbolAddress); make
 *     that first call before any stream capture begins.  Later calls only launch.
 *   - There is one array per device: two calls whose kernels can overlap on the GPU (different
 *     streams, or a second call issued before the first call's combine step was enqueued on the
 *     same stream) race on it.  Keep attention -> combine pairs in one stream order.
 *   - Nothing in the array needs clearing between calls. */
int skv_decode_attention_static(const SkvStoreDesc* desc, const void* store, int layer, const void* plan,
                                const void* query, int query_dtype, int num_q_heads, int num_ctas, float* logits,
                                int32_t* err_flag, void** partials_out, void* stream);

/* ---- everything between two attention kernels in one launch -------------------------------- */

/* skv_lse_combine and the skv_quantize_pack_append of the step's new token (one row per sequence:
 * cur_k / cur_v, the same tensors the combine step attends to) for `layer`, together with the
 * skv_importance_update of an EARLIER attention launch, as ONE kernel launch; the three are
 * independent, so their blocks run side by side.  Same results as the separate calls.
 *   imp_layer / imp_logits / imp_lse_max / imp_lse_sum / imp_cur_prob: the inputs of the importance
 *   update, i.e. the logits an earlier skv_decode_attention wrote and the (max, sum, current-token
 *   probability) an earlier combine wrote for layer imp_layer.  They must not alias this launch's
 *   lse_max / lse_sum / cur_prob outputs (callers double-buffer them).  imp_logits == NULL skips the
 *   importance update; dst_seq == NULL skips the append (store may then be NULL).
 *   max_seq_tokens: an upper bound of the cached tokens of any sequence if the caller knows one (the
 *   importance blocks are then launched for that many storage indices only), 0 otherwise.
 *   Under CUDA-graph capture both host scalars are frozen into the graph: pass max_seq_tokens = 0 (the
 *   cache grows between replays), and capture an even number of importance updates per graph, because
 *   `parity` must alternate from one update to the next and a replay repeats the captured values.
 * No counterpart in the reference, which runs these steps as host Python
 * (smartkv/core/fused_cpu.py:115-167, cache.py:216-279, :1187-1355). */
int skv_post_attention(const SkvStoreDesc* desc, void* store, int layer, const void* plan, const void* query,
                       int query_dtype, int num_q_heads, const void* partials, int num_ctas, const void* cur_k,
                       const void* cur_v, int kv_dtype, float* out, float* lse_max, float* lse_sum, float* cur_prob,
                       const int32_t* counts, int imp_layer, const float* imp_logits, const float* imp_lse_max,
                       const float* imp_lse_sum, const float* imp_cur_prob, const int32_t* cur_slot,
                       float* head_state, int parity, double* cumulative, float* layer_ema, uint8_t* touched,
                       float decay, float head_decay, const int32_t* dst_seq, const int32_t* dst_bucket,
                       const int32_t* dst_pos, int max_seq_tokens, int32_t* err_flag, void* stream);

/* ---- prompt pass -------------------------------------------------------------- */

/* Causal self-attention over the unquantised prompt plus the per-key attention mass of the
 * importance update, replacing the wrapper's dense path for more than one query token
 * (smartkv/models/llama_smartkv.py:392-415: matmul, causal mask, softmax, matmul) together with the
 * head weighting and the sum over batch, heads and queries of SmartKVCache.update_attention /
 * ImportanceTracker.update_attention (smartkv/core/cache.py:232-259, smartkv/core/importance.py:62-72) --
 * without writing the [batch, heads, queries, keys] probabilities to memory.
 *   q [batch][tokens][num_q_heads][head_dim], k, v [batch][tokens][num_kv_heads][head_dim], fp16, addressed
 *   through element strides {batch, token, head} (head_dim contiguous, strides multiples of 8, bases 16-byte
 *   aligned); dtype must be SKV_DTYPE_F16; head_dim 64 or 128.
 *   head_weights fp32 [batch][num_q_heads] (the normalised head importance) or NULL (= 1).
 *   out fp16 [batch][tokens][num_q_heads][head_dim]; lse fp32 [batch][num_q_heads][tokens] (base-2
 *   log-sum-exp of every query row, also the scratch of the second pass).
 *   key_mass fp32 [batch][num_kv_heads][tokens]: sum over the queries and the query heads of the KV head's
 *   group of weight * probability; adding the KV heads gives the reference's per-key importance.  NULL skips
 *   the second pass. */
int skv_prefill_attention(const void* q, const void* k, const void* v, int dtype, int batch, int tokens,
                          int num_q_heads, int num_kv_heads, int head_dim, const int64_t* q_strides,
                          const int64_t* k_strides, const int64_t* v_strides, const float* head_weights, void* out,
                          float* lse, float* key_mass, void* stream);

/* ---- importance ----------------------------------------------------------- */

/* Replaces SmartKVCache.update_attention's head weighting + ImportanceTracker.update_attention
 * (smartkv/core/cache.py:232-264, smartkv/core/importance.py:44-101) for the case the
 * decode path produces: every cached key (and the current token) is a key of this call.
 * Per key: mass = sum over query heads of w_h * exp2(logit - max_h) / sum_h, added to the
 * cumulative importance (fp64, storage order) and folded into the per-layer EMA
 * (first touch assigns; afterwards decay*old + (1-decay)*mass).
 *   head_state fp32 [num_seqs][2][num_q_heads]: the head-importance EMA, double buffered;
 *   `parity` (0/1) says which half is current, the other half receives the update.
 *   touched uint8 [num_layers][num_seqs][slots] first-touch flags of the EMA. */
int skv_importance_update(const SkvStoreDesc* desc, int layer, const int32_t* counts, int num_q_heads,
                          const float* logits, const float* lse_max, const float* lse_sum, const float* cur_prob,
                          const int32_t* cur_slot, float* head_state, int parity, double* cumulative,
                          float* layer_ema, uint8_t* touched, float decay, float head_decay, void* stream);

/* ---- reallocation: bit allocation ------------------------------------------- */

#define SKV_ALLOC_MAX_PROTECTED 16

/* Parameters of the allocator; the fields mirror SmartKVCache.__init__ (smartkv/core/cache.py:42-67)
 * after the clamping done there (:131-141). */
typedef struct SkvAllocConfig {
  int32_t num_heads;            /* KV heads of the whole model (accounting only) */
  int32_t head_dim;
  int32_t num_bits;             /* 1..4 widths */
  int32_t bits[4];              /* ascending, each in {2,3,4,8} */
  double util[4];               /* bits[i] ** utility_alpha, computed by the host (its libm is the reference's) */
  double memory_budget;
  double importance_floor;
  double rank_threshold;        /* hysteresis_rank_threshold */
  double high_fraction;         /* high_precision_fraction */
  double high_boost;            /* high_precision_boost */
  int32_t hysteresis_intervals;
  int32_t min_high_tokens;
  int32_t scale_bits;           /* 32 or 16: bits of one stored scale in the accounting */
  int32_t use_packing;          /* must be 1 */
  int32_t critical_window;      /* token ids below it are protected (cache.py:309) */
  int32_t num_protected;
  int32_t protected_ids[SKV_ALLOC_MAX_PROTECTED];
} SkvAllocConfig;

int64_t skv_alloc_workspace_bytes(const SkvStoreDesc* desc);

/* Replaces SmartKVCache.allocate_precision + _solve_allocation (smartkv/core/cache.py:281-351,
 * 353-601) for every sequence of the store at once: marginal-gain greedy under the memory
 * budget with the 0.85-budget gate, rank hysteresis and the high-priority pass, bit-exact with
 * the reference's heap loop (ties: lower token id first).
 *   counts int32 [num_seqs][4], slot_token int32 [num_seqs][slots] (token id of every storage
 *   index), scores fp64 [num_seqs][slots] (cumulative importance, storage order), recency fp64
 *   [num_seqs][slots] or NULL (factor exp(-age/512) of cache.py:304-306; NULL = 1).
 *   rank_pct fp64 / rank_streak int8 [num_seqs][slots]: the persistent hysteresis record
 *   (cache.py:423-450); streak -1 marks a token without a record.
 * Outputs: new_bits uint8 [num_seqs][slots] (0 on unused indices), new_counts int32
 * [num_seqs][4], changed int32 [num_seqs] (tokens whose width differs from their bucket's). */
int skv_alloc_bits(const SkvStoreDesc* desc, const SkvAllocConfig* cfg, const int32_t* counts,
                   const int32_t* slot_token, const double* scores, const double* recency, double* rank_pct,
                   int8_t* rank_streak, uint8_t* new_bits, int32_t* new_counts, int32_t* changed, void* workspace,
                   void* stream);

/* ---- reallocation: requantise + repack ------------------------------------------ */

/* The three calls below replace SmartKVCache._requantize_tokens / _requantize_single /
 * _write_quantized_slot (smartkv/core/cache.py:806-926) and the bucket delete / append around
 * them (:1046-1083, :1121-1161).  All are stream-ordered and allocate nothing.
 *
 * skv_repack_plan: from the new widths (skv_alloc_bits' new_bits) builds, per sequence, the list
 * of row moves that makes every bucket dense again: move k of sequence b takes the row at storage
 * index move_src[b][k] to move_dst[b][k] (both int32 [num_seqs][slots]; n_moves int32 [num_seqs]).
 * counts_new int32 [num_seqs][4].  workspace: skv_repack_plan_workspace_bytes().  If a bucket
 * would exceed its capacity nothing moves (n_moves = 0, counts_new = counts) and *err_flag = 3. */
int64_t skv_repack_plan_workspace_bytes(const SkvStoreDesc* desc);
int skv_repack_plan(const SkvStoreDesc* desc, const int32_t* counts, const uint8_t* new_bits, int32_t* move_src,
                    int32_t* move_dst, int32_t* n_moves, int32_t* counts_new, void* workspace, int32_t* err_flag,
                    void* stream);

/* skv_requant_repack: applies the moves to the packed rows of layers [layer_begin, layer_end).
 * A row whose destination bucket has another width is dequantised (code * scale, fp32) and
 * quantised again at the new width, from the stored codes as the reference does (cache.py:819-844);
 * other rows are copied.  Every moved row passes through `staging`
 * (skv_requant_staging_bytes(desc, upper bound of the moves of all sequences, layers per call));
 * if the staging buffer is too small for the moves found on the device nothing moves and
 * *err_flag = 6. */
int64_t skv_requant_staging_bytes(const SkvStoreDesc* desc, int64_t max_moves, int num_layers);
int skv_requant_repack(const SkvStoreDesc* desc, void* store, int layer_begin, int layer_end,
                       const int32_t* move_src, const int32_t* move_dst, const int32_t* n_moves, void* staging,
                       int64_t staging_bytes, int32_t* err_flag, void* stream);

/* skv_repack_meta: the per-token arrays kept in storage order (token ids, cumulative importance,
 * hysteresis record, per-layer EMA and its first-touch flags) follow the same moves; indices a
 * bucket gave up are reset; finally counts <- counts_new.  Call it after the rows of every layer
 * have moved. */
int64_t skv_repack_meta_staging_bytes(const SkvStoreDesc* desc, int64_t max_moves);
int skv_repack_meta(const SkvStoreDesc* desc, const int32_t* move_src, const int32_t* move_dst,
                    const int32_t* n_moves, int32_t* counts, const int32_t* counts_new, int32_t* slot_token,
                    double* cumulative, double* rank_pct, int8_t* rank_streak, float* layer_ema, uint8_t* touched,
                    void* staging, int64_t staging_bytes, int32_t* err_flag, void* stream);

/* ---- error flag ---------------------------------------------------------- */

/* Reads and clears a device error flag (synchronises the stream). */
int skv_read_error_flag(int32_t* err_flag, int32_t* host_value, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SMARTKV_B200_H_ */
