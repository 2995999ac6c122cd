// Shared device helpers for the sm_100a SmartKV kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/smartkv_b200.h"

namespace skv {

constexpr int kNumBuckets = SKV_NUM_BUCKETS;

__host__ __device__ constexpr int bucket_bits(int bucket) {
  return bucket == 0 ? 2 : bucket == 1 ? 3 : bucket == 2 ? 4 : 8;
}
__host__ __device__ constexpr int bits_bucket(int bits) {
  return bits == 2 ? 0 : bits == 3 ? 1 : bits == 4 ? 2 : bits == 8 ? 3 : -1;
}
__host__ __device__ constexpr int row_bytes_for(int head_dim, int bits) { return head_dim * bits / 8; }

// Device-side copy of the store geometry (passed by value to kernels).
struct StoreGeom {
  int num_layers, num_seqs, num_kv_heads, head_dim;
  int cap[kNumBuckets];
  int row_bytes[kNumBuckets];
  int bucket_base[kNumBuckets];
  int slots;
  long long k_off[kNumBuckets], v_off[kNumBuckets], sc_off[kNumBuckets];
  long long arena_bytes;
};

inline StoreGeom make_geom(const SkvStoreDesc& d) {
  StoreGeom g;
  g.num_layers = d.num_layers;
  g.num_seqs = d.num_seqs;
  g.num_kv_heads = d.num_kv_heads;
  g.head_dim = d.head_dim;
  for (int i = 0; i < kNumBuckets; ++i) {
    g.cap[i] = d.cap[i];
    g.row_bytes[i] = d.row_bytes[i];
    g.bucket_base[i] = d.bucket_base[i];
    g.k_off[i] = d.k_off[i];
    g.v_off[i] = d.v_off[i];
    g.sc_off[i] = d.sc_off[i];
  }
  g.slots = d.slots;
  g.arena_bytes = d.arena_bytes;
  return g;
}

__device__ __forceinline__ const uint8_t* arena_ptr(const StoreGeom& g, const void* store, int layer, int seq) {
  return static_cast<const uint8_t*>(store) + ((long long)layer * g.num_seqs + seq) * g.arena_bytes;
}
__device__ __forceinline__ uint8_t* arena_ptr(const StoreGeom& g, void* store, int layer, int seq) {
  return static_cast<uint8_t*>(store) + ((long long)layer * g.num_seqs + seq) * g.arena_bytes;
}

// The last 256 bytes of every (layer, sequence) arena are a footer.  Word 0 becomes non-zero once a V scale above
// kVScaleGuard has been stored in that arena (it is never cleared): the attention kernel multiplies probabilities
// of up to 2^8 by the V scale in fp16, which is safe without a check only below that scale.
constexpr float kVScaleGuard = 64.0f;
__device__ __forceinline__ const int* arena_flags(const StoreGeom& g, const uint8_t* arena) {
  return reinterpret_cast<const int*>(arena + g.arena_bytes - 256);
}
__device__ __forceinline__ void note_v_scale(const StoreGeom& g, uint8_t* arena, float v_scale) {
  if (v_scale > kVScaleGuard) *reinterpret_cast<volatile int*>(arena + g.arena_bytes - 256) = 1;
}

// ---- programmatic dependent launch ----------------------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in the stream is
// still running: launch_dependents lets the successor's blocks be scheduled once every block of this grid has
// executed it (or exited); wait blocks until the predecessor grid has completed and its writes are visible.  Both are
// no-ops in a launch without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with (or, if `dependent` is false, without) the programmatic-serialization attribute.
template <class Params>
inline cudaError_t launch_maybe_dependent(void (*kernel)(Params), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                          const Params& p, bool dependent) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

// ---- small PTX wrappers -----------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// (a & b) | c
__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// (a & b) ^ c
__device__ __forceinline__ uint32_t lop_and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
// x * m + a on packed halves, operands given as raw 32-bit patterns
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t x, uint32_t m, uint32_t a) {
  return h2_bits(__hfma2(bits_h2(x), bits_h2(m), bits_h2(a)));
}
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t x, uint32_t a) {
  return h2_bits(__hadd2(bits_h2(x), bits_h2(a)));
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier + bulk async copy (TMA, 1-D, no multicast) ------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// non-blocking test of a phase
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the limit ran out (caller sets the error flag).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 17)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// global -> shared bulk copy; all three of dst, src, bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// L2 policy for data that is read once: its lines are the first to be evicted, so that what the kernel
// writes for its successor (partials, logits) stays resident
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// asks the memory system to bring [gsrc, gsrc+bytes) into L2 (no destination, no completion)
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace skv
