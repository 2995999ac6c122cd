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

/* Reads rows back out of the store as int8 codes + fp32 scales (the dequantising
 * read side of cache.py:1493-1543 / get_bucket_views :671-744).  Row r is read
 * from (src_seq[r], src_bucket[r], src_pos[r]); outputs [rows][num_kv_heads][head_dim]
 * and [rows][num_kv_heads]. */
int skv_export_rows(const SkvStoreDesc* desc, const void* store, int layer, int rows, const int32_t* src_seq,
                    const int32_t* src_bucket, const int32_t* src_pos, int8_t* k_codes, int8_t* v_codes,
                    float* k_scale, float* v_scale, void* stream);

/* ---- fused packed decode attention --------------------------------------- */

/* Size queries (host only). */
int skv_attn_num_ctas(int device);                       /* persistent CTAs the kernel launches */
int64_t skv_attn_partials_bytes(const SkvStoreDesc* desc, int num_q_heads, int num_ctas);
int64_t skv_attn_plan_bytes(const SkvStoreDesc* desc, int num_ctas);

/* Builds the work partition of one decode step: which 16-key tiles of which
 * (sequence, KV head) every persistent CTA streams, balanced by packed bytes.  It
 * depends only on the bucket counts, which are the same for every layer of the
 * step, so one call serves all layers.  No counterpart in the reference (its kernel
 * walks one head per CTA, smartkv/csrc/quantized_attention.cu:679-777).
 *   counts int32 [num_seqs][4] live tokens per bucket (device); plan: device buffer
 *   of skv_attn_plan_bytes() bytes. */
int skv_attn_plan(const SkvStoreDesc* desc, const int32_t* counts, int num_ctas, void* plan, void* stream);

/* Replaces quantized_attention_bucket_forward + the host cross-bucket LSE combine
 * (smartkv/csrc/quantized_attention.cu:460-828, smartkv/kernels/__init__.py:269-386)
 * and the CPU streaming path (smartkv/core/fused_cpu.py:7-167) for q_len == 1.
 *
 * Streams the packed buckets of `layer` for every sequence, split-KV over
 * persistent CTAs as laid out by `plan`, and writes one partial (max, sum, out)
 * triple per run into `partials`; if `logits` is not NULL it also writes the scaled
 * logit (log2 units) of every cached key, logits[seq][q_head][storage index].
 *   query    [num_seqs][num_q_heads][head_dim] fp32 or fp16
 * num_q_heads must be a multiple of num_kv_heads with group size <= 8.
 * err_flag: device int32, set non-zero if a bounded wait inside the kernel gave up. */
int skv_decode_attention(const SkvStoreDesc* desc, const void* store, int layer, const void* plan,
                         const void* query, int query_dtype, int num_q_heads, void* partials, int num_ctas,
                         float* logits, int32_t* err_flag, void* stream);

/* Combines the partials with the newest token, which takes part in full precision
 * (smartkv/core/fused_cpu.py:115-137; wrapper call smartkv/models/llama_smartkv.py:264-305),
 * and normalises.  cur_k/cur_v [num_seqs][num_kv_heads][head_dim] (may be NULL: no
 * current token).  out fp32 [num_seqs][num_q_heads][head_dim]; lse_max / lse_sum fp32
 * [num_seqs][num_q_heads] (final max in log2 units, final sum); cur_prob fp32
 * [num_seqs][num_q_heads] = probability of the current token (may be NULL). */
int skv_lse_combine(const SkvStoreDesc* desc, const void* plan, const void* query, int query_dtype,
                    int num_q_heads, const void* partials, int num_ctas, const void* cur_k, const void* cur_v,
                    int kv_dtype, float* out, float* lse_max, float* lse_sum, float* cur_prob, void* stream);

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

/* ---- debug / test hooks ---------------------------------------------------- */

/* Raw tensor-core tile products through the same fragment code as the attention
 * kernel, for one 16-key tile of packed rows (row_bytes apart):
 *   scores[8][16] = (Q[0..7] + Q[8..15]) . Kcodes^T      Q fp16 [16][head_dim]
 *   out[8][head_dim] = (P[0..7] + P[8..15]) . Vcodes      P fp16 [16][16] ([row][key])
 * Rows 0..7 are the query heads of a group, rows 8..15 the residual rows the
 * precise (fp32-query) mode adds. */
int skv_debug_tile_products(int head_dim, int bits, const uint8_t* k_rows, const uint8_t* v_rows,
                            const void* q_half, const void* p_half, float* scores, float* out, void* stream);

/* Integer scores of one 16-key tile through the int8 tensor-core path the attention kernel
 * uses for 2-, 4- and 8-bit rows: scores int32 [8][16] = sum_d q[h][d] * u[key][d], q int8
 * [8][head_dim], u = the stored code (offset-binary for 2/4-bit rows, two's complement for 8-bit). */
int skv_debug_tile_scores_i8(int head_dim, int bits, const uint8_t* k_rows, const int8_t* q_int8, int32_t* scores,
                             void* stream);

/* Reads and clears a device error flag (synchronises the stream). */
int skv_read_error_flag(int32_t* err_flag, int32_t* host_value, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SMARTKV_B200_H_ */
