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
  // slack so that a 3-bit slice load that rounds its address down/up never leaves the arena
  d->arena_bytes = align_up(off + 256, 256);
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
  return *host_value == 0 ? SKV_OK : SKV_ERR_TIMEOUT;
}
