// Host-side pieces of the C ABI that launch nothing heavy: geometry, status strings,
// the error-flag read.
#include "common.cuh"

extern "C" const char* skv_status_string(int status) {
  switch (status) {
    case SKV_OK: return "ok";
    case SKV_ERR_INVALID: return "invalid argument";
    case SKV_ERR_CUDA: return "CUDA runtime error";
    case SKV_ERR_CAPACITY: return "capacity exceeded";
    case SKV_ERR_TIMEOUT: return "device-side wait timed out";
    case SKV_ERR_UNSUPPORTED: return "unsupported configuration";
    default: return "unknown status";
  }
}

extern "C" int skv_build_arch(void) { return 100; }

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

extern "C" int skv_store_layout(SkvStoreDesc* d) {
  if (!d) return SKV_ERR_INVALID;
  if (d->num_layers <= 0 || d->num_seqs <= 0 || d->num_kv_heads <= 0) return SKV_ERR_INVALID;
  if (d->head_dim != 64 && d->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  int64_t off = 0;
  int base = 0;
  for (int i = 0; i < SKV_NUM_BUCKETS; ++i) {
    if (d->cap[i] < 0 || d->cap[i] % 128 != 0) return SKV_ERR_INVALID;
    const int bits = skv::bucket_bits(i);
    d->row_bytes[i] = skv::row_bytes_for(d->head_dim, bits);
    d->bucket_base[i] = base;
    base += d->cap[i];
    const int64_t rows = (int64_t)d->num_kv_heads * d->cap[i];
    d->k_off[i] = off;
    off = align_up(off + rows * d->row_bytes[i], 256);
    d->v_off[i] = off;
    off = align_up(off + rows * d->row_bytes[i], 256);
    d->sc_off[i] = off;
    off = align_up(off + rows * 8, 256);
  }
  d->slots = base;
  d->reserved_ = 0;
  // slack so that a 3-bit slice load that rounds its address down/up never leaves the arena, then the footer
  // (256 bytes; word 0 = "a V scale above 64 is stored here", see common.cuh)
  d->arena_bytes = align_up(off + 256, 256) + 256;
  d->total_bytes = d->arena_bytes * d->num_layers * d->num_seqs;
  return SKV_OK;
}

extern "C" int skv_read_error_flag(int32_t* err_flag, int32_t* host_value, void* stream) {
  if (!err_flag || !host_value) return SKV_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(host_value, err_flag, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return SKV_ERR_CUDA;
  if (cudaMemsetAsync(err_flag, 0, sizeof(int32_t), st) != cudaSuccess) return SKV_ERR_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return SKV_ERR_CUDA;
  // 1: a bounded wait ran out; 2, 3, 6: a bucket or a staging buffer was too small (the row was refused / nothing
  // moved); 4, 5: inconsistent widths or bookkeeping handed to a kernel
  switch (*host_value) {
    case 0: return SKV_OK;
    case 1: return SKV_ERR_TIMEOUT;
    case 2: case 3: case 6: return SKV_ERR_CAPACITY;
    default: return SKV_ERR_INVALID;
  }
}

// ---- placement of the token every sequence appends in a decode step ----------------------------
namespace skv {

__global__ void step_plan_kernel(StoreGeom g, const int32_t* counts, const uint8_t* bits, int32_t* dst_seq,
                                 int32_t* dst_bucket, int32_t* dst_pos, int32_t* dst_storage, int32_t* err) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= g.num_seqs) return;
  int bucket = bits ? bits_bucket(bits[b]) : bits_bucket(4);  // unseen tokens enter at 4 bits (cache.py:1214)
  if (bucket < 0) {
    if (err) atomicExch(err, 4);
    bucket = bits_bucket(4);
  }
  const int pos = counts[b * kNumBuckets + bucket];
  if (pos >= g.cap[bucket] && err) atomicExch(err, 3);  // the bucket is full: the append kernel will refuse the row
  dst_seq[b] = b;
  dst_bucket[b] = bucket;
  dst_pos[b] = pos;
  dst_storage[b] = g.bucket_base[bucket] + pos;
}

__global__ void step_commit_kernel(StoreGeom g, int32_t* counts, int32_t* slot_token, int32_t* next_token,
                                   const int32_t* dst_bucket, const int32_t* dst_storage) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= g.num_seqs) return;
  const int bucket = dst_bucket[b], s = dst_storage[b];
  if (bucket < 0 || bucket >= kNumBuckets || s < 0 || s >= g.slots) return;
  if (s - g.bucket_base[bucket] >= g.cap[bucket]) return;  // was refused
  slot_token[(long long)b * g.slots + s] = next_token[b];
  counts[b * kNumBuckets + bucket] += 1;
  next_token[b] += 1;
}

}  // namespace skv

extern "C" int skv_step_plan(const SkvStoreDesc* desc, const int32_t* counts, const uint8_t* bits, int32_t* dst_seq,
                             int32_t* dst_bucket, int32_t* dst_pos, int32_t* dst_storage, int32_t* err_flag,
                             void* stream) {
  if (!desc || !counts || !dst_seq || !dst_bucket || !dst_pos || !dst_storage) return SKV_ERR_INVALID;
  skv::step_plan_kernel<<<(desc->num_seqs + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      skv::make_geom(*desc), counts, bits, dst_seq, dst_bucket, dst_pos, dst_storage, err_flag);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

extern "C" int skv_step_commit(const SkvStoreDesc* desc, int32_t* counts, int32_t* slot_token, int32_t* next_token,
                               const int32_t* dst_bucket, const int32_t* dst_storage, void* stream) {
  if (!desc || !counts || !slot_token || !next_token || !dst_bucket || !dst_storage) return SKV_ERR_INVALID;
  skv::step_commit_kernel<<<(desc->num_seqs + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      skv::make_geom(*desc), counts, slot_token, next_token, dst_bucket, dst_storage);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
