// Per-(token, head) symmetric quantisation, bit packing, and the append into
// the bucketed store.  One warp owns one row of head_dim values.
//
// Arithmetic follows the reference CPU quantiser (smartkv/core/_quant_cpu.py:20-34):
// scale = absmax / max(max_code, 1) with an IEEE fp32 divide, 0 -> 1,
// code = clamp(rint(x / scale)) with round-half-even.  No fast-math anywhere in
// this file: codes and scales are bit-exact with the CPU path.
// Packed format: smartkv/csrc/bit_packing.cu:20-43, 69-95, 128-151.
#include "post_attention.cuh"

namespace skv {

// ---- append into the store ----------------------------------------------------
template <int EPL>
__global__ void quantize_pack_append_kernel(const AppendParams p) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= (long long)p.rows * p.g.num_kv_heads * 2) return;
  append_row<EPL>(p, warp, lane);
}

// ---- plain quantise (parity helper) --------------------------------------------
template <int EPL>
__global__ void quantize_rows_kernel(const void* in, int dtype, long long rows, int bits, int8_t* codes,
                                     float* scales) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= rows) return;
  RowVals<EPL> x = load_row<EPL>(in, dtype, warp, lane);
  int code[EPL];
  const float scale = quantize_row<EPL>(x, bits, code);
  constexpr int D = EPL * 32;
#pragma unroll
  for (int i = 0; i < EPL; ++i) codes[warp * D + lane * EPL + i] = (int8_t)code[i];
  if (lane == 0) scales[warp] = scale;
}

// Generic row quantiser for any head_dim (one warp per row, strided); used when
// head_dim is not 64 or 128.
__global__ void quantize_rows_generic_kernel(const void* in, int dtype, long long rows, int D, int bits,
                                             int8_t* codes, float* scales) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= rows) return;
  auto ld = [&](int d) -> float {
    return dtype == SKV_DTYPE_F32 ? static_cast<const float*>(in)[warp * D + d]
                                  : __half2float(static_cast<const __half*>(in)[warp * D + d]);
  };
  float amax = 0.f;
  for (int d = lane; d < D; d += 32) amax = fmaxf(amax, fabsf(ld(d)));
  amax = warp_max(amax);
  const int hi = (1 << (bits - 1)) - 1, lo = -(1 << (bits - 1));
  float scale = __fdiv_rn(amax, (float)(hi > 1 ? hi : 1));
  if (scale == 0.f) scale = 1.f;
  for (int d = lane; d < D; d += 32) {
    float q = rintf(__fdiv_rn(ld(d), scale));
    codes[warp * D + d] = (int8_t)(int)fminf(fmaxf(q, (float)lo), (float)hi);
  }
  if (lane == 0) scales[warp] = scale;
}

// ---- flat pack / unpack (parity helpers) ---------------------------------------
// One thread per output byte group; partial trailing groups are zero filled.
__global__ void pack_flat_kernel(const int8_t* codes, long long n, int bits, uint8_t* packed) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (bits == 8) {
    if (i < n) packed[i] = (uint8_t)codes[i];
    return;
  }
  const int per = bits == 2 ? 4 : bits == 4 ? 2 : 8;
  const long long groups = (n + per - 1) / per;
  if (i >= groups) return;
  const int off = 1 << (bits - 1);
  const uint32_t fm = (1u << bits) - 1u;
  uint32_t w = 0;
  for (int j = 0; j < per; ++j) {
    long long e = i * per + j;
    if (e < n) w |= (((uint32_t)(codes[e] + off)) & fm) << (bits * j);
  }
  if (bits == 3) {
    packed[3 * i + 0] = (uint8_t)(w & 0xff);
    packed[3 * i + 1] = (uint8_t)((w >> 8) & 0xff);
    packed[3 * i + 2] = (uint8_t)((w >> 16) & 0xff);
  } else {
    packed[i] = (uint8_t)w;
  }
}

__global__ void unpack_flat_kernel(const uint8_t* packed, long long n, int bits, int8_t* codes) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (bits == 8) {
    codes[i] = (int8_t)packed[i];
    return;
  }
  const long long bitpos = i * bits;
  const long long byte = bitpos >> 3;
  const int sh = (int)(bitpos & 7);
  uint32_t win = packed[byte];
  if (sh + bits > 8) win |= (uint32_t)packed[byte + 1] << 8;
  const uint32_t fm = (1u << bits) - 1u;
  codes[i] = (int8_t)((int)((win >> sh) & fm) - (1 << (bits - 1)));
}

// ---- export rows from the store as int8 codes + scales ---------------------------
__global__ void export_rows_kernel(StoreGeom g, const uint8_t* store, int layer, int rows, const int32_t* src_seq,
                                   const int32_t* src_bucket, const int32_t* src_pos, int8_t* k_codes,
                                   int8_t* v_codes, float* k_scale, float* v_scale) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)rows * g.num_kv_heads * 2;
  if (warp >= total) return;
  const int which = (int)(warp & 1);
  const long long rh = warp >> 1;
  const int h = (int)(rh % g.num_kv_heads);
  const int r = (int)(rh / g.num_kv_heads);
  const int seq = src_seq[r], bucket = src_bucket[r], pos = src_pos[r];
  if (seq < 0 || seq >= g.num_seqs || bucket < 0 || bucket >= kNumBuckets || pos < 0 || pos >= g.cap[bucket]) return;
  const int bits = bucket_bits(bucket);
  const uint8_t* arena = arena_ptr(g, store, layer, seq);
  const long long row_index = (long long)h * g.cap[bucket] + pos;
  const uint8_t* src = arena + (which ? g.v_off[bucket] : g.k_off[bucket]) + row_index * g.row_bytes[bucket];
  int8_t* out = (which ? v_codes : k_codes) + rh * g.head_dim;
  const uint32_t fm = (1u << bits) - 1u;
  for (int d = lane; d < g.head_dim; d += 32) {
    int c;
    if (bits == 8) {
      c = (int8_t)src[d];
    } else {
      const int bitpos = d * bits, byte = bitpos >> 3, sh = bitpos & 7;
      uint32_t win = src[byte];
      if (sh + bits > 8) win |= (uint32_t)src[byte + 1] << 8;
      c = (int)((win >> sh) & fm) - (1 << (bits - 1));
    }
    out[d] = (int8_t)c;
  }
  if (lane == 0) {
    const float* sc = reinterpret_cast<const float*>(arena + g.sc_off[bucket]);
    (which ? v_scale : k_scale)[rh] = sc[2 * row_index + which];
  }
}

// ---- dequantising read: rows of the store as fp32 / fp16 values ------------------------------
template <typename OutT>
__global__ void dequant_rows_kernel(StoreGeom g, const uint8_t* store, int layer, int rows, const int32_t* src_seq,
                                    const int32_t* src_bucket, const int32_t* src_pos, OutT* k_out, OutT* v_out) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)rows * g.num_kv_heads * 2;
  if (warp >= total) return;
  const int which = (int)(warp & 1);
  const long long rh = warp >> 1;
  const int h = (int)(rh % g.num_kv_heads);
  const int r = (int)(rh / g.num_kv_heads);
  const int seq = src_seq[r], bucket = src_bucket[r], pos = src_pos[r];
  if (seq < 0 || seq >= g.num_seqs || bucket < 0 || bucket >= kNumBuckets || pos < 0 || pos >= g.cap[bucket]) return;
  const int bits = bucket_bits(bucket);
  const uint8_t* arena = arena_ptr(g, store, layer, seq);
  const long long row_index = (long long)h * g.cap[bucket] + pos;
  const uint8_t* src = arena + (which ? g.v_off[bucket] : g.k_off[bucket]) + row_index * g.row_bytes[bucket];
  const float scale = reinterpret_cast<const float*>(arena + g.sc_off[bucket])[2 * row_index + which];
  OutT* out = (which ? v_out : k_out) + rh * g.head_dim;
  const uint32_t fm = (1u << bits) - 1u;
  for (int d = lane; d < g.head_dim; d += 32) {
    int c;
    if (bits == 8) {
      c = (int8_t)src[d];
    } else {
      const int bitpos = d * bits, byte = bitpos >> 3, sh = bitpos & 7;
      uint32_t win = src[byte];
      if (sh + bits > 8) win |= (uint32_t)src[byte + 1] << 8;
      c = (int)((win >> sh) & fm) - (1 << (bits - 1));
    }
    out[d] = (OutT)__fmul_rn((float)c, scale);  // code.float() * scale, as the reference dequantises (cache.py:1493-1543)
  }
}

// ---- import rows: int8 codes + scales -> packed rows of the store -----------------------
template <int EPL>
__global__ void import_rows_kernel(StoreGeom g, uint8_t* store, int layer, int rows, const int32_t* dst_seq,
                                   const int32_t* dst_bucket, const int32_t* dst_pos, const int8_t* k_codes,
                                   const int8_t* v_codes, const float* k_scale, const float* v_scale, int32_t* err) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)rows * g.num_kv_heads * 2;
  if (warp >= total) return;
  const int which = (int)(warp & 1);
  const long long rh = warp >> 1;
  const int h = (int)(rh % g.num_kv_heads);
  const int r = (int)(rh / g.num_kv_heads);
  const int seq = dst_seq[r], bucket = dst_bucket[r], pos = dst_pos[r];
  if (seq < 0 || seq >= g.num_seqs || bucket < 0 || bucket >= kNumBuckets || pos < 0 || pos >= g.cap[bucket]) {
    if (lane == 0 && err) atomicExch(err, 2);
    return;
  }
  const int bits = bucket_bits(bucket);
  const int8_t* in = (which ? v_codes : k_codes) + rh * g.head_dim + lane * EPL;
  const int lo = -(1 << (bits - 1)), hi = (1 << (bits - 1)) - 1;
  int code[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int c = in[i];
    code[i] = c < lo ? lo : (c > hi ? hi : c);  // codes outside the width's range are clamped
  }
  uint8_t* arena = arena_ptr(g, store, layer, seq);
  const long long row_index = (long long)h * g.cap[bucket] + pos;
  uint8_t* dst = arena + (which ? g.v_off[bucket] : g.k_off[bucket]) + row_index * g.row_bytes[bucket];
  pack_store_row<EPL>(code, bits, dst, lane);
  if (lane == 0) {
    float* sc = reinterpret_cast<float*>(arena + g.sc_off[bucket]);
    const float scale = (which ? v_scale : k_scale)[rh];
    sc[2 * row_index + which] = scale;
    if (which) note_v_scale(g, arena, scale);
  }
}

}  // namespace skv

using namespace skv;

static inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
static inline int launch_status() { return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA; }

extern "C" int skv_quantize_per_head(const void* input, int input_dtype, int64_t rows, int head_dim, int bits,
                                     int8_t* codes, float* scales, void* stream) {
  if (!input || !codes || !scales || rows < 0 || head_dim <= 0) return SKV_ERR_INVALID;
  if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return SKV_ERR_INVALID;
  if (input_dtype != SKV_DTYPE_F32 && input_dtype != SKV_DTYPE_F16) return SKV_ERR_INVALID;
  if (rows == 0) return SKV_OK;
  const int wpb = 8;
  const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
  if (head_dim == 128)
    quantize_rows_kernel<4><<<grid, wpb * 32, 0, as_stream(stream)>>>(input, input_dtype, rows, bits, codes, scales);
  else if (head_dim == 64)
    quantize_rows_kernel<2><<<grid, wpb * 32, 0, as_stream(stream)>>>(input, input_dtype, rows, bits, codes, scales);
  else
    quantize_rows_generic_kernel<<<grid, wpb * 32, 0, as_stream(stream)>>>(input, input_dtype, rows, head_dim, bits,
                                                                          codes, scales);
  return launch_status();
}

extern "C" int skv_pack(const int8_t* codes, int64_t n, int bits, uint8_t* packed, void* stream) {
  if (!codes || !packed || n < 0) return SKV_ERR_INVALID;
  if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return SKV_ERR_INVALID;
  if (n == 0) return SKV_OK;
  const int per = bits == 8 ? 1 : bits == 2 ? 4 : bits == 4 ? 2 : 8;
  const long long groups = (n + per - 1) / per;
  pack_flat_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, as_stream(stream)>>>(codes, n, bits, packed);
  return launch_status();
}

extern "C" int skv_unpack(const uint8_t* packed, int64_t n, int bits, int8_t* codes, void* stream) {
  if (!codes || !packed || n < 0) return SKV_ERR_INVALID;
  if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return SKV_ERR_INVALID;
  if (n == 0) return SKV_OK;
  unpack_flat_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(packed, n, bits, codes);
  return launch_status();
}

extern "C" int skv_quantize_pack_append(const SkvStoreDesc* desc, void* store, int layer, const void* k,
                                        const void* v, int input_dtype, int rows, const int32_t* dst_seq,
                                        const int32_t* dst_bucket, const int32_t* dst_pos, void* stream) {
  if (!desc || !store || !k || !v || !dst_seq || !dst_bucket || !dst_pos) return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || rows < 0) return SKV_ERR_INVALID;
  if (input_dtype != SKV_DTYPE_F32 && input_dtype != SKV_DTYPE_F16) return SKV_ERR_INVALID;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if (rows == 0) return SKV_OK;
  AppendParams p;
  p.g = make_geom(*desc);
  p.store = static_cast<uint8_t*>(store);
  p.layer = layer;
  p.k = k;
  p.v = v;
  p.dtype = input_dtype;
  p.rows = rows;
  p.dst_seq = dst_seq;
  p.dst_bucket = dst_bucket;
  p.dst_pos = dst_pos;
  p.err = nullptr;
  const int wpb = 8;
  const long long warps = (long long)rows * p.g.num_kv_heads * 2;
  const unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
  if (desc->head_dim == 128)
    quantize_pack_append_kernel<4><<<grid, wpb * 32, 0, as_stream(stream)>>>(p);
  else
    quantize_pack_append_kernel<2><<<grid, wpb * 32, 0, as_stream(stream)>>>(p);
  return launch_status();
}

extern "C" int skv_export_rows(const SkvStoreDesc* desc, const void* store, int layer, int rows,
                               const int32_t* src_seq, const int32_t* src_bucket, const int32_t* src_pos,
                               int8_t* k_codes, int8_t* v_codes, float* k_scale, float* v_scale, void* stream) {
  if (!desc || !store || !src_seq || !src_bucket || !src_pos || !k_codes || !v_codes || !k_scale || !v_scale)
    return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || rows < 0) return SKV_ERR_INVALID;
  if (rows == 0) return SKV_OK;
  StoreGeom g = make_geom(*desc);
  const int wpb = 8;
  const long long warps = (long long)rows * g.num_kv_heads * 2;
  export_rows_kernel<<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, as_stream(stream)>>>(
      g, static_cast<const uint8_t*>(store), layer, rows, src_seq, src_bucket, src_pos, k_codes, v_codes, k_scale,
      v_scale);
  return launch_status();
}

extern "C" int skv_import_rows(const SkvStoreDesc* desc, void* store, int layer, int rows, const int32_t* dst_seq,
                               const int32_t* dst_bucket, const int32_t* dst_pos, const int8_t* k_codes,
                               const int8_t* v_codes, const float* k_scale, const float* v_scale, int32_t* err_flag,
                               void* stream) {
  if (!desc || !store || !dst_seq || !dst_bucket || !dst_pos || !k_codes || !v_codes || !k_scale || !v_scale)
    return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || rows < 0) return SKV_ERR_INVALID;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if (rows == 0) return SKV_OK;
  const StoreGeom g = make_geom(*desc);
  const int wpb = 8;
  const long long warps = (long long)rows * g.num_kv_heads * 2;
  const unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
  if (desc->head_dim == 128)
    import_rows_kernel<4><<<grid, wpb * 32, 0, as_stream(stream)>>>(g, static_cast<uint8_t*>(store), layer, rows, dst_seq,
                                                                    dst_bucket, dst_pos, k_codes, v_codes, k_scale,
                                                                    v_scale, err_flag);
  else
    import_rows_kernel<2><<<grid, wpb * 32, 0, as_stream(stream)>>>(g, static_cast<uint8_t*>(store), layer, rows, dst_seq,
                                                                    dst_bucket, dst_pos, k_codes, v_codes, k_scale,
                                                                    v_scale, err_flag);
  return launch_status();
}

extern "C" int skv_dequant_rows(const SkvStoreDesc* desc, const void* store, int layer, int rows,
                                const int32_t* src_seq, const int32_t* src_bucket, const int32_t* src_pos,
                                int out_dtype, void* k_out, void* v_out, void* stream) {
  if (!desc || !store || !src_seq || !src_bucket || !src_pos || !k_out || !v_out) return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || rows < 0) return SKV_ERR_INVALID;
  if (out_dtype != SKV_DTYPE_F32 && out_dtype != SKV_DTYPE_F16) return SKV_ERR_INVALID;
  if (rows == 0) return SKV_OK;
  const StoreGeom g = make_geom(*desc);
  const int wpb = 8;
  const long long warps = (long long)rows * g.num_kv_heads * 2;
  const unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
  if (out_dtype == SKV_DTYPE_F32)
    dequant_rows_kernel<float><<<grid, wpb * 32, 0, as_stream(stream)>>>(
        g, static_cast<const uint8_t*>(store), layer, rows, src_seq, src_bucket, src_pos, static_cast<float*>(k_out),
        static_cast<float*>(v_out));
  else
    dequant_rows_kernel<__half><<<grid, wpb * 32, 0, as_stream(stream)>>>(
        g, static_cast<const uint8_t*>(store), layer, rows, src_seq, src_bucket, src_pos, static_cast<__half*>(k_out),
        static_cast<__half*>(v_out));
  return launch_status();
}
