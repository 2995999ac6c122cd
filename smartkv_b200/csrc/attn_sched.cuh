// Work partition of the fused decode attention: which tiles of which (sequence, KV head) segment a
// persistent CTA owns.
//
// Two kernels consume a plan and each has its own cost model (`model`):
//   model 0  mma.sync fragment kernel: tiles of 16 keys; the cost of a tile is the time one CTA needs
//            for it (measured with every token at that width: narrow tiles are bound by their
//            arithmetic, 8-bit tiles by their bytes)
//   model 1  tensor-memory (tcgen05) kernel: tiles of 128 keys = one MMA block; the cost is the block's
//            bytes plus a fixed term for the per-block arithmetic and hand-offs
// Every segment is a string of cost units: for each bucket in turn, ceil(count / tile_keys) tiles of
// tile_cost(bucket).  All heads of a sequence have the same length W[b].
// The global string concatenates the segments in (sequence, head) order; CTA c
// owns the tiles whose first unit lies in [ceil(c*T/C), ceil((c+1)*T/C)), i.e. the
// CTAs are balanced by estimated time and never share a tile.  A maximal piece of one
// segment owned by one CTA is a *run*; runs are numbered in byte order, which is
// both (CTA, segment) order and (segment, CTA) order, so a CTA's runs and a
// segment's runs are each consecutive.  The partition depends only on the bucket
// counts, which are the same for every layer of a decode step, so it is built once
// per step into a small plan buffer and read by every layer's launches.
#pragma once

#include "common.cuh"

namespace skv {

__host__ __device__ constexpr int tile_bytes_for(int head_dim, int bits) {
  return 16 * (2 * row_bytes_for(head_dim, bits) + 8);
}

constexpr int kPlanModelFrag = 0;  // 16-key tiles, mma.sync fragment kernel
constexpr int kPlanModelTc = 1;    // 128-key tiles, tensor-memory kernel
__host__ __device__ constexpr int plan_tile_keys(int model) { return model == kPlanModelTc ? 128 : 16; }

// Relative cost of one tile.  Model 0: nanoseconds one CTA spends per 16-key tile of each width at
// head_dim 128 (B200, all tokens at one width: 46.5 / 51.6 / 48.9 / 63.3 us per launch of 65,536 tiles
// on 148 CTAs).  Model 1: the block's bytes in units of 256 B plus a fixed per-block term.  Only the
// ratios matter.
__host__ __device__ constexpr int tile_cost_for(int head_dim, int bits, int model) {
  if (model == kPlanModelTc) return 128 * (2 * row_bytes_for(head_dim, bits) + 8) / 256 + 24;
  return bits == 2 ? 105 : bits == 3 ? 116 : bits == 4 ? 110 : 143;
}

struct SegLayout {
  int cnt[kNumBuckets];          // live keys per bucket
  int nt[kNumBuckets];           // tiles per bucket
  long long start[kNumBuckets];  // first cost unit of the bucket inside the segment
  long long bytes;               // W: cost units of one segment of this sequence
};

__host__ __device__ inline SegLayout seg_layout(const int32_t* counts4, int head_dim, int model) {
  SegLayout s;
  long long off = 0;
  const int tk = plan_tile_keys(model);
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) {
    s.cnt[i] = counts4[i];
    s.nt[i] = (counts4[i] + tk - 1) / tk;
    s.start[i] = off;
    off += (long long)s.nt[i] * tile_cost_for(head_dim, bucket_bits(i), model);
  }
  s.bytes = off;
  return s;
}

__host__ __device__ inline long long cta_range_begin(long long total, int c, int num_ctas) {
  return (total * c + num_ctas - 1) / num_ctas;
}

// Tiles [ka, kb) of every bucket whose first unit lies in the segment-local range [lo, hi).
// Returns the number of tiles.
__host__ __device__ inline int seg_tiles_in_range(const SegLayout& s, int head_dim, long long lo, long long hi,
                                                  int (&ka)[kNumBuckets], int (&kb)[kNumBuckets], int model) {
  int total = 0;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) {
    const long long tb = tile_cost_for(head_dim, bucket_bits(i), model);
    long long a = lo - s.start[i], b = hi - s.start[i];
    a = a <= 0 ? 0 : (a + tb - 1) / tb;
    b = b <= 0 ? 0 : (b + tb - 1) / tb;
    if (a > s.nt[i]) a = s.nt[i];
    if (b > s.nt[i]) b = s.nt[i];
    ka[i] = (int)a;
    kb[i] = (int)b;
    total += (int)(b - a);
  }
  return total;
}

// One run: the tiles [ka, kb) of each bucket of segment (seq, head) that one CTA streams, in units of the
// plan's tile size (header word 3).
struct __align__(16) RunDesc {
  int seq, head;
  int ka[kNumBuckets];
  int kb[kNumBuckets];
  int cnt[kNumBuckets];  // live keys per bucket of the sequence
  int pad_[2];
};
static_assert(sizeof(RunDesc) == 64, "RunDesc is one 64-byte record");

// Plan buffer (int32 words):
//   [0] number of runs  [1] number of CTAs  [2] number of segments  [3] keys per tile (16 or 128)
//   cta_begin[C + 1]     first run of every CTA
//   seg_begin[nseg]      first run of every segment (undefined when seg_count is 0)
//   seg_count[nseg]      runs of every segment
//   (padding to 16 words)  RunDesc runs[C + nseg]
//   RunDesc first[C]     copy of every CTA's first run, so that a CTA reaches it with one load
//                        instead of two dependent ones (cta_begin, then runs[])
struct PlanView {
  int* header;
  int* cta_begin;
  int* seg_begin;
  int* seg_count;
  RunDesc* runs;
  RunDesc* first;
};
__host__ __device__ inline long long plan_words(int num_ctas, int nseg) {
  long long head = 4 + (num_ctas + 1) + 2LL * nseg;
  head = (head + 15) / 16 * 16;
  return head + 16LL * (num_ctas + nseg) + 16LL * num_ctas;
}
__host__ __device__ inline PlanView plan_view(int* base, int num_ctas, int nseg) {
  PlanView v;
  v.header = base;
  v.cta_begin = base + 4;
  v.seg_begin = v.cta_begin + (num_ctas + 1);
  v.seg_count = v.seg_begin + nseg;
  long long head = 4 + (num_ctas + 1) + 2LL * nseg;
  head = (head + 15) / 16 * 16;
  v.runs = reinterpret_cast<RunDesc*>(base + head);
  v.first = v.runs + (num_ctas + nseg);
  return v;
}

}  // namespace skv
