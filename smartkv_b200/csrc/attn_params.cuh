// Launch parameters and helpers shared by the two decode-attention kernels (the mma.sync fragment
// kernel in decode_attention.cu and the tensor-memory kernel in decode_attention_tc.cu).
#pragma once

#include "attn_sched.cuh"

namespace skv {

constexpr int kMaxSeqs = 1024;
constexpr int kMaxCtas = 1024;

struct AttnParams {
  StoreGeom g;
  const uint8_t* store;
  int layer;
  const int* plan;
  const void* query;
  int q_is_half;
  int num_q_heads;
  int group;
  float* partials;
  int num_ctas;
  float* logits;
  const float* mask;  // additive mask [num_seqs][mask_stride] indexed by token id, log-e units (may be null)
  const int32_t* slot_token;  // [num_seqs][slots] token id of every storage index (needed with a mask)
  long long mask_stride;
  int32_t* err;
  float scale_log2;
  unsigned wait_polls;  // limit of every bounded wait, in polls of about 50 ns
  int dependent;        // launch with the programmatic-serialization attribute (SKV_ATTN_DEPENDENT_LAUNCH)
};

// Bounded mbarrier wait that also gives up as soon as another thread of the CTA has given up.
// Polls the phase with a short sleep in between: a warp suspended inside mbarrier.try_wait resumed
// noticeably later after the phase completed, and the sleep keeps a waiting warp out of the issue
// slots.  `polls` polls of at least 50 ns bound the wait (2^24: about a second).  On expiry the CTA's
// abort flag and the global error flag are set and false is returned; the kernel then runs to its end
// without waiting for anything else, so a launch always returns.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* err,
                                              unsigned polls) {
  for (uint32_t i = 0; i < polls; ++i) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
    __nanosleep(50);
  }
  *abort_flag = 1;
  atomicExch(err, 1);
  return false;
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// The tensor-memory kernel (decode_attention_tc.cu): head_dim 128, fp16 queries, group <= 8.
int launch_attn_tc(const AttnParams& p, const SkvStoreDesc& desc, cudaStream_t stream);
int attn_tc_partials_per_run();

}  // namespace skv
