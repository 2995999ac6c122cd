// Fused packed-KV decode attention for sm_100a (q_len == 1, GQA group <= 8).
//
// Persistent CTAs (one per SM).  The packed buckets of every (sequence, KV head)
// segment form one string of 16-key tiles; the global string is split into ranges of
// equal estimated time over the CTAs (attn_sched.cuh) by a tiny plan kernel that runs
// once per decode step.  A CTA streams its runs through a ring of shared-memory
// stages: one producer warp issues bulk async copies (TMA 1-D, L2 evict-first: packed
// K rows, packed V rows, scales) and publishes the query rows of each run (fp16 copy
// and int8 limbs), the consumer warps take the tiles of a block round-robin, unpack
// the codes in registers straight into tensor-core fragments (attn_frag.cuh), keep an
// online softmax and accumulate P.V in registers.  Full/empty mbarriers order producer
// and consumers; every wait is bounded.  At the end of a run every consumer warp writes
// its own (max, sum, out) partial; the combine step (post_attention.cuh) folds the
// partials of a segment, adds the full-precision current token and normalises.
//
// Replaces smartkv/csrc/quantized_attention.cu:460-828 (per-bucket kernel, one
// CTA per head walking the whole context) and the host LSE combine in
// smartkv/kernels/__init__.py:350-371; numerics follow the CPU streaming path
// smartkv/core/fused_cpu.py:70-113 (dequantise, q.k/sqrt(d), online softmax).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "attn_frag.cuh"
#include "attn_params.cuh"
#include "post_attention.cuh"

namespace skv {

constexpr int kQBufs = 4;        // query / run-descriptor ring (the producer runs at most STAGES blocks ahead)

// Shape of the persistent CTA: NCONS consumer warps + 1 producer warp share STAGES stages.
template <int NCONS_, int STAGES_, int STAGE_BYTES_>
struct AttnCfg {
  static constexpr int NCONS = NCONS_, STAGES = STAGES_, STAGE_BYTES = STAGE_BYTES_;
};
constexpr int kMaxPartialsPerRun = 11;  // consumer warps of the widest configuration
using AttnCfgFast = AttnCfg<11, 3, 63360>;  // fp16 queries: 11 consumer warps x 145 registers (12 were no faster, 13 and 15 at 128 registers slower); 15 8-bit tiles per stage
using AttnCfgPrecise = AttnCfg<7, 3, 42240>;   // fp32 queries (hi/lo split): 8 warps, more registers per thread

// tiles per block for a bit-width: as many 16-key tiles as fit one stage
__host__ __device__ constexpr int block_tiles(int stage_bytes, int head_dim, int bits) {
  return stage_bytes / tile_bytes_for(head_dim, bits);
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return h2_bits(h);
}

// ---- plan: the byte-balanced partition, built once per decode step --------------------
__global__ void __launch_bounds__(1024) attn_plan_kernel(StoreGeom g, const int32_t* counts, int C, int* plan_base,
                                                         int model) {
  __shared__ long long cumw[kMaxSeqs + 1];
  __shared__ int nruns_of[kMaxCtas + 1];
  const int tid = threadIdx.x, NT = blockDim.x;
  const int B = g.num_seqs, Hkv = g.num_kv_heads, D = g.head_dim, nseg = B * Hkv;
  PlanView pv = plan_view(plan_base, C, nseg);
  for (int b = tid; b < B; b += NT) cumw[b + 1] = seg_layout(counts + b * kNumBuckets, D, model).bytes;
  for (int s = tid; s < nseg; s += NT) {
    pv.seg_begin[s] = 0x7fffffff;
    pv.seg_count[s] = 0;
  }
  __syncthreads();
  if (tid == 0) {
    long long acc = 0;
    cumw[0] = 0;
    for (int b = 0; b < B; ++b) {
      acc += cumw[b + 1];
      cumw[b + 1] = acc;
    }
  }
  __syncthreads();
  const long long total = cumw[B] * Hkv;
  // walks the segments CTA c overlaps; with `out` set, writes the runs starting at run index `first`
  auto walk = [&](int c, RunDesc* out, int first) {
    int n = 0;
    long long y = cta_range_begin(total, c, C);
    const long long y_end = cta_range_begin(total, c + 1, C);
    int b = 0;
    while (y < y_end) {
      int lo = b, hi = B;  // last b with Hkv*cumw[b] <= y
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cumw[mid] * Hkv <= y) lo = mid; else hi = mid;
      }
      b = lo;
      const SegLayout sl = seg_layout(counts + b * kNumBuckets, D, model);
      const long long seq_first = cumw[b] * Hkv;
      const int h = (int)((y - seq_first) / sl.bytes);
      const long long seg_off = seq_first + (long long)h * sl.bytes;
      const long long seg_end = seg_off + sl.bytes;
      const long long y_next = seg_end < y_end ? seg_end : y_end;
      int ka[kNumBuckets], kb[kNumBuckets];
      if (seg_tiles_in_range(sl, D, y - seg_off, y_next - seg_off, ka, kb, model) > 0) {
        if (out != nullptr) {
          RunDesc r;
          r.seq = b;
          r.head = h;
#pragma unroll
          for (int i = 0; i < kNumBuckets; ++i) {
            r.ka[i] = ka[i];
            r.kb[i] = kb[i];
            r.cnt[i] = sl.cnt[i];
          }
          r.pad_[0] = r.pad_[1] = 0;
          out[first + n] = r;
          const int seg = b * Hkv + h;
          atomicMin(&pv.seg_begin[seg], first + n);
          atomicAdd(&pv.seg_count[seg], 1);
        }
        ++n;
      }
      y = y_next;
    }
    return n;
  };
  for (int c = tid; c < C; c += NT) nruns_of[c + 1] = total > 0 ? walk(c, nullptr, 0) : 0;
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    nruns_of[0] = 0;
    for (int c = 0; c < C; ++c) {
      acc += nruns_of[c + 1];
      nruns_of[c + 1] = acc;
    }
    pv.header[0] = acc;
    pv.header[1] = C;
    pv.header[2] = nseg;
    pv.header[3] = plan_tile_keys(model);
  }
  __syncthreads();
  for (int c = tid; c <= C; c += NT) pv.cta_begin[c] = nruns_of[c];
  for (int c = tid; c < C; c += NT) {
    if (total > 0) walk(c, pv.runs, nruns_of[c]);
    if (nruns_of[c + 1] > nruns_of[c]) pv.first[c] = pv.runs[nruns_of[c]];  // written by this thread just above
  }
}

// Online-softmax state of one lane: query head g = lane >> 2 (the 4 lanes of a head share m).
struct LaneState {
  float m;  // running reference maximum (log2 units)
  float l;  // this lane's share of the running sum
};

// The running maximum is only raised when a score exceeds it by more than kLazyTau (log2
// units), so most tiles need no cross-lane reduction and no rescale of the accumulators;
// probabilities then reach at most 2^kLazyTau, well inside fp16 / fp32 range.
constexpr float kLazyTau = 8.0f;

// Per-run query data the producer warp prepares in shared memory.
template <int D, bool PRECISE>
struct QSlot {
  static constexpr int NLIMB = PRECISE ? 3 : 2;
  static constexpr int QROWS = PRECISE ? 16 : 8;
  __half qh[QROWS][D];       // fp16 rows (rows 8.. = fp16 residuals), for 3-bit keys
  int8_t limb[NLIMB][8][D];  // int8 limbs (radix 128), most significant first
  float sq[8];               // limb step per head: q = sq * sum_l limb_l * 128^(NLIMB-1-l)
  int sumA[8];               // 128*sum(limb0) + sum(limb1)
  int sumB[8];               // sum(limb2) (precise mode)
  RunDesc desc;
  int guard;                 // the run's arena holds a V scale above kVScaleGuard (see process_tile)
};

// Query of one run as a lane sees it, specialised per bit-width of the keys it meets.
template <int D, int BITS, bool PRECISE>
struct QFrags {
  static constexpr bool INT8 = BITS != 3 || D == 128;  // 3-bit rows of head_dim 64 keep the fp16 score path
  uint32_t qa[INT8 ? D / 32 : D / 16][4];   // A fragments: int8 limbs 0/1, or fp16 query/residual
  uint32_t qa2[(INT8 && PRECISE) ? D / 32 : 1][4];  // precise mode: limb 2
  float sq;     // limb step of head g
  int initA;    // -offset * (128*sum(limb0) + sum(limb1)) of head g (offset-binary codes)
  int initB;    // -offset * sum(limb2)
};

template <int D, int BITS, bool PRECISE>
__device__ __forceinline__ void load_qfrags(const QSlot<D, PRECISE>& q, int lane, QFrags<D, BITS, PRECISE>& f) {
  const int g = lane >> 2;
  constexpr int off = BITS == 8 ? 0 : (1 << (BITS - 1));  // 8-bit rows are two's complement
  if constexpr (QFrags<D, BITS, PRECISE>::INT8) {
    gather_qa_i8<D, BITS>(&q.limb[0][0][0], &q.limb[1][0][0], lane, f.qa);
    if constexpr (PRECISE) gather_qa_i8<D, BITS>(&q.limb[2][0][0], nullptr, lane, f.qa2);
    f.sq = q.sq[g];
    f.initA = -off * q.sumA[g];
    f.initB = -off * q.sumB[g];
  } else {
    gather_qa_f16<D, BITS>(&q.qh[0][0], PRECISE, lane, f.qa);
  }
}

// One 16-key tile.  Lane (g,t): supplies the K slices of keys g, g+8 and the V slices of the key
// pairs (2t,2t+1), (2t+8,2t+9); receives the scores of head g for keys 2t, 2t+1, 2t+8, 2t+9.
// WRITE_LOGITS: lrow = logits row of head g (first key of the tile), written as two float2.
// MASKED: the launch carries an additive mask (tok / mrow are only read then).  GUARD: the (layer, sequence) arena
// holds a V scale above kVScaleGuard somewhere, so p * v_scale has to be checked against the fp16 range.
template <int D, int BITS, bool PRECISE, bool WRITE_LOGITS, bool MASKED, bool GUARD>
__device__ __forceinline__ void process_tile(const uint8_t* ktile, const uint8_t* vtile, const float4* sc, int nvalid,
                                             int lane, const QFrags<D, BITS, PRECISE>& qf, LaneState& st,
                                             float (&o)[D / 16][4], float scale_log2, float* lrow,
                                             const int32_t* tok, const float* mrow) {
  const int g = lane >> 2, t = lane & 3;
  // ---- every shared-memory load of the tile up front ---------------------------------
  uint32_t kr0[SliceWords<D, BITS>::K], kr1[SliceWords<D, BITS>::K];
  uint32_t vr0[SliceWords<D, BITS>::V], vr1[SliceWords<D, BITS>::V], vr2[SliceWords<D, BITS>::V],
      vr3[SliceWords<D, BITS>::V];
  load_kslice<D, BITS>(ktile, g, t, kr0);
  load_kslice<D, BITS>(ktile, g + 8, t, kr1);
  load_vrow<D, BITS>(vtile, 2 * t, g, vr0);
  load_vrow<D, BITS>(vtile, 2 * t + 1, g, vr1);
  load_vrow<D, BITS>(vtile, 2 * t + 8, g, vr2);
  load_vrow<D, BITS>(vtile, 2 * t + 9, g, vr3);
  const float4 scA = sc[t], scB = sc[t + 4];  // (ks, vs) of keys 2t, 2t+1 and of keys 2t+8, 2t+9
  // ---- scores of head g (log2 units): x0, x1 = keys 2t, 2t+1; x2, x3 = keys 2t+8, 2t+9 ----
  float x0, x1, x2, x3;
  if constexpr (QFrags<D, BITS, PRECISE>::INT8) {
    int c0[4] = {0, 0, qf.initA, qf.initA}, c1[4] = {0, 0, qf.initA, qf.initA};
    qk_ntile_i8<D, BITS>(kr0, qf.qa, c0);
    qk_ntile_i8<D, BITS>(kr1, qf.qa, c1);
    float f0 = (float)(c0[0] * 128 + c0[2]), f1 = (float)(c0[1] * 128 + c0[3]);
    float f2 = (float)(c1[0] * 128 + c1[2]), f3 = (float)(c1[1] * 128 + c1[3]);
    if constexpr (PRECISE) {
      int e0[4] = {qf.initB, qf.initB, 0, 0}, e1[4] = {qf.initB, qf.initB, 0, 0};
      qk_ntile_i8<D, BITS>(kr0, qf.qa2, e0);
      qk_ntile_i8<D, BITS>(kr1, qf.qa2, e1);
      f0 = fmaf(f0, 128.f, (float)e0[0]);
      f1 = fmaf(f1, 128.f, (float)e0[1]);
      f2 = fmaf(f2, 128.f, (float)e1[0]);
      f3 = fmaf(f3, 128.f, (float)e1[1]);
    }
    const float qs = qf.sq * scale_log2;
    x0 = f0 * (scA.x * qs);
    x1 = f1 * (scA.z * qs);
    x2 = f2 * (scB.x * qs);
    x3 = f3 * (scB.z * qs);
  } else {
    float c0[4], c1[4];
    qk_ntile_f16<D, BITS>(kr0, t, qf.qa, c0);
    qk_ntile_f16<D, BITS>(kr1, t, qf.qa, c1);
    x0 = (c0[0] + c0[2]) * (scA.x * scale_log2);
    x1 = (c0[1] + c0[3]) * (scA.z * scale_log2);
    x2 = (c1[0] + c1[2]) * (scB.x * scale_log2);
    x3 = (c1[1] + c1[3]) * (scB.z * scale_log2);
  }
  float vs0 = scA.y, vs1 = scA.w, vs2 = scB.y, vs3 = scB.w;
  if constexpr (MASKED) {
    // additive mask, indexed by the key's token id as the reference indexes it by the key's global slot
    // (smartkv/csrc/quantized_attention.cu:570-575); natural-log units -> log2 units
    constexpr float kLog2e = 1.4426950408889634f;
    const int k0 = 2 * t, k2 = 2 * t + 8;
    if (k0 < nvalid) { const int id = tok[k0]; if (id >= 0) x0 = fmaf(mrow[id], kLog2e, x0); }
    if (k0 + 1 < nvalid) { const int id = tok[k0 + 1]; if (id >= 0) x1 = fmaf(mrow[id], kLog2e, x1); }
    if (k2 < nvalid) { const int id = tok[k2]; if (id >= 0) x2 = fmaf(mrow[id], kLog2e, x2); }
    if (k2 + 1 < nvalid) { const int id = tok[k2 + 1]; if (id >= 0) x3 = fmaf(mrow[id], kLog2e, x3); }
  }
  if (nvalid < 16) {  // last tile of a bucket: rows past its end may hold anything, scales included
    if (2 * t >= nvalid) { x0 = -INFINITY; vs0 = 0.f; }
    if (2 * t + 1 >= nvalid) { x1 = -INFINITY; vs1 = 0.f; }
    if (2 * t + 8 >= nvalid) { x2 = -INFINITY; vs2 = 0.f; }
    if (2 * t + 9 >= nvalid) { x3 = -INFINITY; vs3 = 0.f; }
  }
  if constexpr (WRITE_LOGITS) {
    if (lrow != nullptr) {
      *reinterpret_cast<float2*>(lrow + 2 * t) = make_float2(x0, x1);
      *reinterpret_cast<float2*>(lrow + 2 * t + 8) = make_float2(x2, x3);
    }
  }
  float mx = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
  // The P operand of the P.V product is p * v_scale in fp16.  With p <= 2^kLazyTau that product stays inside
  // the fp16 range as long as the V scale does not exceed kVScaleGuard; every kernel that writes a V scale
  // records in the arena's footer when one does, and only runs over such an arena pay for the test: a tile
  // with a large scale takes the slow path below, which raises the running maximum far enough for the
  // product to fit.
  bool slow = mx > st.m + kLazyTau;
  if constexpr (GUARD) slow = slow || fmaxf(fmaxf(vs0, vs1), fmaxf(vs2, vs3)) > kVScaleGuard;
  if (__any_sync(0xffffffffu, slow)) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float n = fmaxf(st.m, mx);
    if constexpr (GUARD) {
      const float mu2 = (n == -INFINITY) ? 0.f : n;
      float am = fmaxf(fmaxf(ex2f(x0 - mu2) * vs0, ex2f(x1 - mu2) * vs1), fmaxf(ex2f(x2 - mu2) * vs2, ex2f(x3 - mu2) * vs3));
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
      if (am > 16384.f) n += ceilf(log2f(am)) - 14.f;  // am > 0 needs a finite score, so n is finite here
    }
    const float alpha = (n == -INFINITY) ? 1.f : ex2f(st.m - n);
    st.l *= alpha;
    st.m = n;
    // the accumulators of this lane belong to heads 2t and 2t+1, whose lanes are 8t.. and 8t+4..
    const float a0 = __shfl_sync(0xffffffffu, alpha, 8 * t), a1 = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);
#pragma unroll
    for (int j = 0; j < D / 16; ++j) {
      o[j][0] *= a0;
      o[j][2] *= a0;
      o[j][1] *= a1;
      o[j][3] *= a1;
    }
  }
  const float mu = (st.m == -INFINITY) ? 0.f : st.m;
  const float p0 = ex2f(x0 - mu), p1 = ex2f(x1 - mu), p2 = ex2f(x2 - mu), p3 = ex2f(x3 - mu);
  st.l += (p0 + p1) + (p2 + p3);
  const float a0 = p0 * vs0, a1 = p1 * vs1, a2 = p2 * vs2, a3 = p3 * vs3;
  // P^T B fragments: (keys 2t, 2t+1 ; head g) and (keys 2t+8, 2t+9 ; head g) -- already in place
  const uint32_t pb0 = pack_h2(a0, a1), pb1 = pack_h2(a2, a3);
  uint32_t pl0 = 0u, pl1 = 0u;
  if (PRECISE) {
    const __half2 h0 = bits_h2(pb0), h1 = bits_h2(pb1);
    pl0 = pack_h2(a0 - __low2float(h0), a1 - __high2float(h0));
    pl1 = pack_h2(a2 - __low2float(h1), a3 - __high2float(h1));
  }
  uint32_t v0[D / 8], v1[D / 8];
  unpack_vpair<D, BITS>(vr0, vr1, g, v0);
  unpack_vpair<D, BITS>(vr2, vr3, g, v1);
  pv_tile<D, PRECISE>(v0, v1, pb0, pb1, pl0, pl1, o);
}

// One block = up to KBKEYS keys of one bucket, staged at `sb`: [K rows][V rows][float2 scales].
// This warp owns tiles first, first + NCONS, ... of it.  lrow: logits row of head g at the
// block's first key (null in lanes whose head does not exist).
template <int D, int BITS, bool PRECISE, int KBKEYS, int NCONS, bool MASKED>
__device__ __forceinline__ void process_block(const uint8_t* sb, int nkeys, int first, int lane,
                                              const QFrags<D, BITS, PRECISE>& qf, LaneState& st,
                                              float (&o)[D / 16][4], float scale_log2, bool write_logits, bool guard,
                                              float* lrow, const int32_t* tok, const float* mrow) {
  constexpr int PD = D * BITS / 8;
  const uint8_t* kbase = sb;
  const uint8_t* vbase = sb + KBKEYS * PD;
  const float4* sc = reinterpret_cast<const float4*>(sb + 2 * KBKEYS * PD);  // two keys per float4
  const int ntl = (nkeys + 15) >> 4;
  auto tiles = [&](auto wl_tag, auto gd_tag) {
    constexpr bool WL = decltype(wl_tag)::value, GD = decltype(gd_tag)::value;
    for (int tile = first; tile < ntl; tile += NCONS)
      process_tile<D, BITS, PRECISE, WL, MASKED, GD>(kbase + tile * 16 * PD, vbase + tile * 16 * PD, sc + tile * 8,
                                                     nkeys - tile * 16, lane, qf, st, o, scale_log2,
                                                     (WL && lrow) ? lrow + tile * 16 : nullptr,
                                                     MASKED ? tok + tile * 16 : nullptr, mrow);
  };
  // both flags are warp-uniform (lanes of heads >= G carry a null logits row)
  if (write_logits) {
    if (guard) tiles(std::true_type{}, std::true_type{}); else tiles(std::true_type{}, std::false_type{});
  } else {
    if (guard) tiles(std::false_type{}, std::true_type{}); else tiles(std::false_type{}, std::false_type{});
  }
}

// The query rows of a run: fp16 copy (plus a residual row in the precise mode) and radix-128 int8
// limbs with their row sums.  One warp per call, heads [gq0, gq1) (at most 8); every head's elements are
// fetched before any is processed, so the call costs one round trip to memory, not one per head.
template <int D, bool PRECISE>
__device__ __forceinline__ void prep_query_heads(QSlot<D, PRECISE>& slot, const AttnParams& p, int seq, int head,
                                                 int G, int gq0, int gq1, int lane) {
  constexpr int NL = QSlot<D, PRECISE>::NLIMB;
  constexpr int EPL = D / 32;  // query elements per lane and head
  const long long q_off = ((long long)seq * p.num_q_heads + (long long)head * G) * D;
  float q[8][EPL];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gq = gq0 + i;
    if (gq < gq1) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const long long idx = q_off + (long long)gq * D + lane * EPL + e;
        q[i][e] = p.q_is_half ? __half2float(static_cast<const __half*>(p.query)[idx])
                              : static_cast<const float*>(p.query)[idx];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gq = gq0 + i;
    if (gq >= gq1) break;
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(q[i][e]));
    amax = warp_max(amax);
    float range = 127.f;
#pragma unroll
    for (int l = 1; l < NL; ++l) range *= 128.f;
    const float step = amax > 0.f ? amax / range : 1.f;
    const float inv = 1.f / step;
    int sum[NL];
#pragma unroll
    for (int l = 0; l < NL; ++l) sum[l] = 0;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d_idx = lane * EPL + e;
      const __half qh = __float2half_rn(q[i][e]);
      slot.qh[gq][d_idx] = qh;
      if (PRECISE) slot.qh[gq + 8][d_idx] = __float2half_rn(q[i][e] - __half2float(qh));
      float rem = fminf(fmaxf(rintf(q[i][e] * inv), -range), range);  // integer in [-range, range]
#pragma unroll
      for (int l = NL - 1; l >= 1; --l) {
        const float hi = rintf(rem * (1.f / 128.f));
        const int low = (int)(rem - hi * 128.f);  // in [-64, 64]
        slot.limb[l][gq][d_idx] = (int8_t)low;
        sum[l] += low;
        rem = hi;
      }
      slot.limb[0][gq][d_idx] = (int8_t)(int)rem;
      sum[0] += (int)rem;
    }
#pragma unroll
    for (int l = 0; l < NL; ++l) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum[l] += __shfl_xor_sync(0xffffffffu, sum[l], off);
    }
    if (lane == 0) {
      slot.sq[gq] = step;
      slot.sumA[gq] = 128 * sum[0] + sum[1];
      slot.sumB[gq] = NL == 3 ? sum[NL - 1] : 0;
    }
  }
}

template <int D, bool PRECISE, class CFG, bool MASKED>
__global__ void __launch_bounds__((CFG::NCONS + 1) * 32, 1) decode_attn_kernel(const AttnParams p) {
  constexpr int NCONS = CFG::NCONS, STAGES = CFG::STAGES, STAGE_BYTES = CFG::STAGE_BYTES;
  constexpr int NTC = NCONS * 32;  // consumer threads
  constexpr int KBT0 = block_tiles(STAGE_BYTES, D, 2), KBT1 = block_tiles(STAGE_BYTES, D, 3),
                KBT2 = block_tiles(STAGE_BYTES, D, 4), KBT3 = block_tiles(STAGE_BYTES, D, 8);
  static_assert(KBT3 >= 1, "stage too small for one tile");
  using Slot = QSlot<D, PRECISE>;
  extern __shared__ __align__(128) uint8_t smem[];
  const StoreGeom& g = p.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.group, Hkv = g.num_kv_heads;

  uint8_t* stages = smem;                                                          // [STAGES][STAGE_BYTES]
  Slot* qslots = reinterpret_cast<Slot*>(smem + STAGES * STAGE_BYTES);             // [kQBufs]
  uint64_t* full = reinterpret_cast<uint64_t*>(qslots + kQBufs);                   // [STAGES]
  uint64_t* empty = full + STAGES;                                                 // [STAGES]
  uint64_t* qfull = empty + STAGES;                                                // [kQBufs]
  uint64_t* qempty = qfull + kQBufs;                                               // [kQBufs]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(qempty + kQBufs);

  {  // rows of heads >= G are never written again and must read as zero
    uint32_t* z = reinterpret_cast<uint32_t*>(qslots);
    for (int i = tid; i < (int)(kQBufs * sizeof(Slot) / 4); i += (NCONS + 1) * 32) z[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NCONS);
    }
    for (int s = 0; s < kQBufs; ++s) {
      mbar_init(&qfull[s], 1);
      mbar_init(&qempty[s], NCONS);
    }
    *abort_flag = 0;
  }
  mbar_fence_init();
  __syncthreads();
  // Dependent launch (layers after the first of a step): this grid may start while the previous layer's post-attention
  // kernel is still running.  What is read before pdl_wait() -- the plan and this layer's packed rows -- was written
  // by kernels that completed long before; the query and everything written here come after the wait.  The launch that
  // follows (combine + append + importance of this layer) waits for this grid itself; letting it be scheduled now only
  // hides its launch latency.
  pdl_launch_dependents();

  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.num_ctas, g.num_seqs * Hkv);
  const int run_begin = pv.cta_begin[blockIdx.x], run_end = pv.cta_begin[blockIdx.x + 1];
  if (run_begin >= run_end) {  // nothing to do here; still, no CTA of a dependent launch leaves before its predecessor ended
    pdl_wait();
    return;
  }

  if (warp == NCONS) {
    // ================================ producer warp ================================
    int stg = 0, qi = 0;
    uint32_t epar = 1, qepar = 1;  // a fresh barrier passes a wait on parity 1: every slot starts empty
    const int kbt[kNumBuckets] = {KBT0, KBT1, KBT2, KBT3};
    bool first_block = true;
    uint32_t armed = 0, armed_par = 0;  // stages with a copy issued, and the parity of their last full phase
    const uint64_t stream_policy = l2_evict_first_policy();  // the cache is read once per step
    constexpr int NL = Slot::NLIMB;
    constexpr int EPL = D / 32;  // query elements per lane and head
    // issues up to `limit` further blocks of run d, resuming at (bucket ci, tile ct0)
    auto issue_blocks = [&](const RunDesc& d, int& ci, int& ct0, int limit) -> bool {
      const uint8_t* arena = arena_ptr(g, p.store, p.layer, d.seq);
      for (; ci < kNumBuckets; ++ci, ct0 = -1) {
        if (ct0 < 0) ct0 = d.ka[ci];
        const int pd = g.row_bytes[ci], kbkeys = kbt[ci] * 16;
        for (int step = 0; ct0 < d.kb[ci]; ct0 += step) {
          if (limit-- <= 0) return true;
          // the CTA's very first block is short (one tile per consumer warp), so that it arrives early
          step = (first_block && kbt[ci] > NCONS) ? NCONS : kbt[ci];
          first_block = false;
          if (!wait_or_abort(&empty[stg], epar, abort_flag, p.err, p.wait_polls)) return false;
          armed |= 1u << stg;
          armed_par = (armed_par & ~(1u << stg)) | ((epar ^ 1u) << stg);
          if (lane == 0) {
            const int ntl = (d.kb[ci] - ct0) < step ? (d.kb[ci] - ct0) : step;
            const int key0 = ct0 * 16;
            const int nkeys = (d.cnt[ci] - key0) < ntl * 16 ? (d.cnt[ci] - key0) : ntl * 16;
            const int n16 = (nkeys + 15) & ~15;
            uint8_t* sb = stages + (long long)stg * STAGE_BYTES;
            const long long row = (long long)d.head * g.cap[ci] + key0;
            const uint32_t kbytes = (uint32_t)(n16 * pd), sbytes = (uint32_t)(n16 * 8);
            fence_proxy_async();
            mbar_expect_tx(&full[stg], 2 * kbytes + sbytes);
            bulk_g2s_hint(sb, arena + g.k_off[ci] + row * pd, kbytes, &full[stg], stream_policy);
            bulk_g2s_hint(sb + kbkeys * pd, arena + g.v_off[ci] + row * pd, kbytes, &full[stg], stream_policy);
            bulk_g2s_hint(sb + 2 * kbkeys * pd, arena + g.sc_off[ci] + row * 8, sbytes, &full[stg], stream_policy);
          }
          if (++stg == STAGES) {
            stg = 0;
            epar ^= 1u;
          }
        }
      }
      return true;
    };
    // Publishes the query slot of run r: its descriptor and, except for the CTA's first run (whose
    // rows the consumer warps prepare themselves, one head each, while the first copies are in
    // flight), the query rows.
    auto publish_query = [&](int r, const RunDesc& d) -> bool {
      if (!wait_or_abort(&qempty[qi], qepar, abort_flag, p.err, p.wait_polls)) return false;
      Slot& slot = qslots[qi];
      if (lane == 0) {
        slot.desc = d;
        slot.guard = *arena_flags(g, arena_ptr(g, p.store, p.layer, d.seq));
      }
      if (r != run_begin) {
        prep_query_heads<D, PRECISE>(slot, p, d.seq, d.head, G, 0, G, lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qfull[qi]);
      if (++qi == kQBufs) {
        qi = 0;
        qepar ^= 1u;
      }
      return true;
    };
    // a plan cut in 128-key tiles (built for the tensor-memory kernel) is read in 16-key tiles here
    const int tile_mul = pv.header[3] == 128 ? 8 : 1;
    auto in_16_key_tiles = [&](RunDesc x) {
      if (tile_mul != 1) {
#pragma unroll
        for (int i = 0; i < kNumBuckets; ++i) {
          const int nt = (x.cnt[i] + 15) >> 4;
          x.ka[i] = x.ka[i] * tile_mul < nt ? x.ka[i] * tile_mul : nt;
          x.kb[i] = x.kb[i] * tile_mul < nt ? x.kb[i] * tile_mul : nt;
        }
      }
      return x;
    };
    RunDesc d = in_16_key_tiles(pv.first[blockIdx.x]);  // meaningful when the CTA has a run
    bool ok = run_begin < run_end;
    for (int r = run_begin; ok && r < run_end; ++r) {
      int ci = 0, ct0 = -1;
      // the first blocks of a run go out first; then, while they are in flight, the query slot of
      // the NEXT run is published, so that no consumer ever waits for query rows at a run boundary
      ok = issue_blocks(d, ci, ct0, STAGES);
      if (r == run_begin) {
        pdl_wait();  // the first copies are in flight; query rows are read from here on
        ok = ok && publish_query(r, d);
      }
      RunDesc dn = d;
      if (ok && r + 1 < run_end) {
        dn = in_16_key_tiles(pv.runs[r + 1]);
        ok = publish_query(r + 1, dn);
      }
      ok = ok && issue_blocks(d, ci, ct0, 1 << 30);
      d = dn;
    }
    if (*abort_flag) {
      // A wait gave up somewhere in the CTA.  The shared memory must outlive the copies still in flight: wait
      // (bounded, about a fifth of a second) for the last phase armed on every stage; a full barrier completes
      // on bytes alone, whatever the consumers do.
      for (int s = 0; s < STAGES; ++s) {
        if (!((armed >> s) & 1u)) continue;
        for (uint32_t i = 0; i < (1u << 22); ++i) {
          if (mbar_test_wait(&full[s], (armed_par >> s) & 1u)) break;
          __nanosleep(50);
        }
      }
    }
    return;
  }

  // ================================== consumer warps ==================================
  int stg = 0, qi = 0;
  uint32_t fpar = 0, qfpar = 0;
  bool aborted = false;
  bool first_block = true;  // the CTA's first block holds one tile per consumer warp
  for (int r = run_begin; r < run_end; ++r) {
    if (!aborted && !wait_or_abort(&qfull[qi], qfpar, abort_flag, p.err, p.wait_polls)) aborted = true;
    // The run's descriptor steers every loop below and the address of the partials, so it may only be read if
    // it was published.  All consumer warps take that decision together: one thread samples the abort flag
    // between two barriers, and either every warp goes on or every warp leaves.
    named_bar_sync(2, NTC);
    if (tid == 0) abort_flag[1] = *abort_flag;
    named_bar_sync(2, NTC);
    if (abort_flag[1]) return;
    const Slot& slot = qslots[qi];  // stays valid until this warp arrives on qempty below
    const RunDesc& d = slot.desc;
    const bool guard = slot.guard != 0;
    if (r == run_begin) {
      pdl_wait();
      for (int gq = warp; gq < G; gq += NCONS) prep_query_heads<D, PRECISE>(qslots[qi], p, d.seq, d.head, G, gq, gq + 1, lane);
      named_bar_sync(1, NCONS * 32);
    }
    const int b = d.seq, h = d.head;

    LaneState st;
    st.m = -INFINITY;
    st.l = 0.f;
    float o[D / 16][4];
#pragma unroll
    for (int j = 0; j < D / 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const int gq = lane >> 2, t = lane & 3;  // scores: head gq; accumulators: heads 2t, 2t+1
    float* lbase = nullptr;  // logits row of head gq
    if (p.logits != nullptr && gq < G) lbase = p.logits + ((long long)b * p.num_q_heads + h * G + gq) * g.slots;
    const bool write_logits = p.logits != nullptr;
    int tile_base = 0;  // tile i of a block goes to warp (tile_base + i) % NCONS

    auto run_bucket = [&](auto bits_tag, auto kbt_tag, int bucket) {
      constexpr int BITS = decltype(bits_tag)::value;
      constexpr int KBT = decltype(kbt_tag)::value;
      if (d.ka[bucket] >= d.kb[bucket]) return;
      QFrags<D, BITS, PRECISE> qf;
      load_qfrags<D, BITS, PRECISE>(slot, lane, qf);
      for (int t0 = d.ka[bucket], step = 0; t0 < d.kb[bucket]; t0 += step) {
        step = (first_block && KBT > NCONS) ? NCONS : KBT;  // as the producer issued it
        first_block = false;
        const int ntl = (d.kb[bucket] - t0) < step ? (d.kb[bucket] - t0) : step;
        const int key0 = t0 * 16;
        const int nkeys = (d.cnt[bucket] - key0) < ntl * 16 ? (d.cnt[bucket] - key0) : ntl * 16;
        if (!aborted && !wait_or_abort(&full[stg], fpar, abort_flag, p.err, p.wait_polls)) aborted = true;
        int first = warp - tile_base;
        if (first < 0) first += NCONS;
        if (!aborted && first < ntl) {
          float* lrow = lbase != nullptr ? lbase + g.bucket_base[bucket] + key0 : nullptr;
          const int32_t* tok = MASKED ? p.slot_token + (long long)b * g.slots + g.bucket_base[bucket] + key0 : nullptr;
          process_block<D, BITS, PRECISE, KBT * 16, NCONS, MASKED>(
              stages + (long long)stg * STAGE_BYTES, nkeys, first, lane, qf, st, o, p.scale_log2, write_logits, guard,
              lrow, tok, MASKED ? p.mask + (long long)b * p.mask_stride : nullptr);
        }
        tile_base = (tile_base + ntl) % NCONS;
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stg]);
        if (++stg == STAGES) {
          stg = 0;
          fpar ^= 1u;
        }
      }
    };
    run_bucket(std::integral_constant<int, 2>{}, std::integral_constant<int, KBT0>{}, 0);
    run_bucket(std::integral_constant<int, 3>{}, std::integral_constant<int, KBT1>{}, 1);
    run_bucket(std::integral_constant<int, 4>{}, std::integral_constant<int, KBT2>{}, 2);
    run_bucket(std::integral_constant<int, 8>{}, std::integral_constant<int, KBT3>{}, 3);

    // ---- every consumer warp writes its own partial (max, sum, out) of this run -------------------
    // (no cross-warp merge: skv_lse_combine folds the NCONS partials of a run like any others)
    __syncwarp();
    if (lane == 0) mbar_arrive(&qempty[qi]);  // query rows and descriptor are no longer needed
    {
      float lsum = st.l;
      lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
      lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
      float* out = p.partials + ((long long)r * NCONS + warp) * partial_stride(G, D);
      if (t == 0 && gq < G) {
        out[gq * (D + 2)] = st.m;
        out[gq * (D + 2) + 1] = lsum;
      }
      if (__any_sync(0xffffffffu, st.m != -INFINITY)) {  // a warp without tiles in this run has nothing to add
        float* row0 = out + (2 * t) * (D + 2) + 2 + gq * (D / 8);
        float* row1 = row0 + (D + 2);
        const bool ok0 = 2 * t < G, ok1 = 2 * t + 1 < G;
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          if (ok0) *reinterpret_cast<float2*>(row0 + 2 * j) = make_float2(o[j][0], o[j][2]);
          if (ok1) *reinterpret_cast<float2*>(row1 + 2 * j) = make_float2(o[j][1], o[j][3]);
        }
      }
    }
    if (++qi == kQBufs) {
      qi = 0;
      qfpar ^= 1u;
    }
  }
}

// ---- combine ----------------------------------------------------------------------
__global__ void __launch_bounds__(kPostThreads) lse_combine_kernel(const CombineParams p) {
  __shared__ CombineShared sh;
  combine_unit(p, blockIdx.x, sh);
}

}  // namespace skv

using namespace skv;

static inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

template <int D, class CFG, bool PRECISE>
static size_t attn_smem_bytes() {
  return (size_t)CFG::STAGES * CFG::STAGE_BYTES + (size_t)kQBufs * sizeof(QSlot<D, PRECISE>) +
         (2 * CFG::STAGES + 2 * kQBufs) * sizeof(uint64_t) + 64;
}

// ---- which kernel serves a launch -----------------------------------------------------------------
// 0 = default: the mma.sync fragment kernel (measured faster on mixed-width caches: its narrow tiles cost less),
// 1 = always the fragment kernel, 2 = the tensor-memory kernel wherever it applies (head_dim 128, fp16 queries;
// measured faster once most cached tokens sit in the 8-bit bucket).  PackedKVStore.autotune_attention times both
// on the live cache and sets this.
static std::atomic<int> g_attn_path{0};

extern "C" int skv_set_attention_path(int path) {
  if (path < 0 || path > 2) return SKV_ERR_INVALID;
  g_attn_path.store(path);
  return SKV_OK;
}
extern "C" int skv_get_attention_path(void) { return g_attn_path.load(); }

static bool use_tc_path(const SkvStoreDesc* desc, int query_dtype) {
  return g_attn_path.load() == 2 && desc->head_dim == 128 && query_dtype == SKV_DTYPE_F16;
}
// The plan is shared by every launch of a step; its tile size follows the kernel that head_dim selects
// for fp16 queries (the fragment kernel reads either tile size).
static int plan_model_for(const SkvStoreDesc* desc) {
  return (g_attn_path.load() == 2 && desc->head_dim == 128) ? kPlanModelTc : kPlanModelFrag;
}

extern "C" int skv_attn_num_ctas(int device) {
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return SKV_ERR_CUDA;
  return sms < kMaxCtas ? sms : kMaxCtas;
}

extern "C" int64_t skv_attn_partials_bytes(const SkvStoreDesc* desc, int num_q_heads, int num_ctas) {
  if (!desc || num_ctas <= 0 || num_q_heads <= 0 || desc->num_kv_heads <= 0) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  const int64_t runs = (int64_t)num_ctas + (int64_t)desc->num_seqs * desc->num_kv_heads;
  return runs * kMaxPartialsPerRun * partial_stride(group, desc->head_dim) * (int64_t)sizeof(float);
}

extern "C" int skv_attn_partials_per_run(const SkvStoreDesc* desc, int query_dtype) {
  if (!desc) return SKV_ERR_INVALID;
  if (use_tc_path(desc, query_dtype)) return attn_tc_partials_per_run();
  int n = query_dtype == SKV_DTYPE_F16 ? AttnCfgFast::NCONS : AttnCfgPrecise::NCONS;
  return n;
}

extern "C" int64_t skv_attn_plan_bytes(const SkvStoreDesc* desc, int num_ctas) {
  if (!desc || num_ctas <= 0) return SKV_ERR_INVALID;
  return plan_words(num_ctas, desc->num_seqs * desc->num_kv_heads) * (int64_t)sizeof(int);
}

extern "C" int skv_attn_plan(const SkvStoreDesc* desc, const int32_t* counts, int num_ctas, void* plan,
                             void* stream) {
  if (!desc || !counts || !plan) return SKV_ERR_INVALID;
  if (num_ctas <= 0 || num_ctas > kMaxCtas || desc->num_seqs > kMaxSeqs) return SKV_ERR_UNSUPPORTED;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  attn_plan_kernel<<<1, 1024, 0, as_stream(stream)>>>(make_geom(*desc), counts, num_ctas, static_cast<int*>(plan),
                                                      plan_model_for(desc));
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

// Programmatic dependent launch of the attention and post-attention kernels (skv_set_dependent_launch).
std::atomic<int> g_dependent_launch{2};  // measured: the attention kernel gains from it, the post-attention kernel loses
extern "C" int skv_set_dependent_launch(int on) {
  // 0 = off, 1 = attention and post-attention kernels, 2 = attention kernel only, 3 = post-attention kernel only
  if (on < 0 || on > 3) return SKV_ERR_INVALID;
  g_dependent_launch.store(on);
  return SKV_OK;
}

template <int D, bool PRECISE, class CFG, bool MASKED>
static int launch_attn_inst(AttnParams& p, cudaStream_t st) {
  static bool configured[64] = {};  // per template instance and device: the attribute belongs to the device's context
  const size_t smem = attn_smem_bytes<D, CFG, PRECISE>();
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SKV_ERR_CUDA;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    const cudaError_t rc = cudaFuncSetAttribute(decode_attn_kernel<D, PRECISE, CFG, MASKED>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (rc != cudaSuccess) {
      fprintf(stderr, "skv_decode_attention: cannot reserve %zu bytes of shared memory: %s\n", smem, cudaGetErrorString(rc));
      return SKV_ERR_CUDA;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  launch_maybe_dependent(decode_attn_kernel<D, PRECISE, CFG, MASKED>, dim3(p.num_ctas), dim3((CFG::NCONS + 1) * 32), smem, st, p,
                         p.dependent != 0 && (g_dependent_launch.load() == 1 || g_dependent_launch.load() == 2));
  const cudaError_t rc = cudaGetLastError();
  if (rc != cudaSuccess) {
    fprintf(stderr, "skv_decode_attention: launch failed: %s\n", cudaGetErrorString(rc));
    return SKV_ERR_CUDA;
  }
  return SKV_OK;
}

// A launch with an additive mask runs its own instantiation, so that launches without one carry none of its cost.
template <int D, bool PRECISE, class CFG>
static int launch_attn(AttnParams& p, cudaStream_t st) {
  return p.mask != nullptr ? launch_attn_inst<D, PRECISE, CFG, true>(p, st) : launch_attn_inst<D, PRECISE, CFG, false>(p, st);
}

// Limit of every bounded device-side wait, in polls of about 50 ns (default 2^24, about a second).
static std::atomic<unsigned> g_wait_polls{1u << 24};
extern "C" int skv_set_wait_limit(unsigned polls) {
  if (polls == 0) return SKV_ERR_INVALID;
  g_wait_polls.store(polls);
  return SKV_OK;
}

extern "C" int skv_decode_attention_masked(const SkvStoreDesc* desc, const void* store, int layer, const void* plan,
                                           const void* query, int query_dtype, int num_q_heads, void* partials,
                                           int num_ctas, float* logits, const float* mask, int64_t mask_stride,
                                           const int32_t* slot_token, int flags, int32_t* err_flag, void* stream) {
  if (!desc || !store || !plan || !query || !partials || !err_flag) return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || num_ctas <= 0 || num_ctas > kMaxCtas) return SKV_ERR_INVALID;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if (desc->num_seqs > kMaxSeqs) return SKV_ERR_UNSUPPORTED;
  if (num_q_heads % desc->num_kv_heads != 0) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  if (group < 1 || group > 8) return SKV_ERR_UNSUPPORTED;
  if (query_dtype != SKV_DTYPE_F32 && query_dtype != SKV_DTYPE_F16) return SKV_ERR_INVALID;
  if (mask != nullptr && (slot_token == nullptr || mask_stride <= 0)) return SKV_ERR_INVALID;
  AttnParams p;
  p.g = make_geom(*desc);
  p.store = static_cast<const uint8_t*>(store);
  p.layer = layer;
  p.plan = static_cast<const int*>(plan);
  p.query = query;
  p.q_is_half = query_dtype == SKV_DTYPE_F16;
  p.num_q_heads = num_q_heads;
  p.group = group;
  p.partials = static_cast<float*>(partials);
  p.num_ctas = num_ctas;
  p.logits = logits;
  p.mask = mask;
  p.slot_token = slot_token;
  p.mask_stride = mask_stride;
  p.err = err_flag;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)desc->head_dim));
  p.wait_polls = g_wait_polls.load();
  p.dependent = (flags & SKV_ATTN_DEPENDENT_LAUNCH) ? 1 : 0;
  if (use_tc_path(desc, query_dtype)) return launch_attn_tc(p, *desc, as_stream(stream));
  const bool precise = !p.q_is_half;
  if (desc->head_dim == 128)
    return precise ? launch_attn<128, true, AttnCfgPrecise>(p, as_stream(stream))
                   : launch_attn<128, false, AttnCfgFast>(p, as_stream(stream));
  return precise ? launch_attn<64, true, AttnCfgPrecise>(p, as_stream(stream))
                 : launch_attn<64, false, AttnCfgFast>(p, as_stream(stream));
}

extern "C" int skv_decode_attention(const SkvStoreDesc* desc, const void* store, int layer, const void* plan,
                                    const void* query, int query_dtype, int num_q_heads, void* partials,
                                    int num_ctas, float* logits, int32_t* err_flag, void* stream) {
  return skv_decode_attention_masked(desc, store, layer, plan, query, query_dtype, num_q_heads, partials, num_ctas,
                                     logits, nullptr, 0, nullptr, 0, err_flag, stream);
}

extern "C" int skv_lse_combine_masked(const SkvStoreDesc* desc, const void* plan, const void* query, int query_dtype,
                                      int num_q_heads, const void* partials, int num_ctas, const void* cur_k,
                                      const void* cur_v, int kv_dtype, const float* cur_mask, float* out, float* lse_max,
                                      float* lse_sum, float* cur_prob, void* stream) {
  if (!desc || !plan || !query || !partials || !out) return SKV_ERR_INVALID;
  if (num_q_heads % desc->num_kv_heads != 0 || num_ctas <= 0) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  if (group < 1 || group > 8) return SKV_ERR_UNSUPPORTED;
  if ((cur_k == nullptr) != (cur_v == nullptr)) return SKV_ERR_INVALID;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  CombineParams p;
  p.g = make_geom(*desc);
  p.plan = static_cast<const int*>(plan);
  p.query = query;
  p.q_is_half = query_dtype == SKV_DTYPE_F16;
  p.num_q_heads = num_q_heads;
  p.group = group;
  p.partials = static_cast<const float*>(partials);
  p.num_ctas = num_ctas;
  p.cur_k = cur_k;
  p.cur_v = cur_v;
  p.kv_is_half = kv_dtype == SKV_DTYPE_F16;
  p.cur_mask = cur_mask;
  p.out = out;
  p.lse_max = lse_max;
  p.lse_sum = lse_sum;
  p.cur_prob = cur_prob;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)desc->head_dim));
  p.per_run = skv_attn_partials_per_run(desc, query_dtype);
  lse_combine_kernel<<<combine_units(p.g, group), kPostThreads, 0, as_stream(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

extern "C" int skv_lse_combine(const SkvStoreDesc* desc, const void* plan, const void* query, int query_dtype,
                               int num_q_heads, const void* partials, int num_ctas, const void* cur_k,
                               const void* cur_v, int kv_dtype, float* out, float* lse_max, float* lse_sum,
                               float* cur_prob, void* stream) {
  return skv_lse_combine_masked(desc, plan, query, query_dtype, num_q_heads, partials, num_ctas, cur_k, cur_v, kv_dtype,
                                nullptr, out, lse_max, lse_sum, cur_prob, stream);
}

// ---- attention with the partials in a fixed device array ------------------------------
// Some callers cannot hand the library a scratch buffer of their own: a serving loop that
// froze its device memory pool after start-up, or a host runtime whose allocator must not
// be entered from the decode thread.  For them the partials live in the array below, which
// is part of the loaded module, so using it never allocates.
constexpr long long kStaticPartialsBytes = 16ll << 20;  // the stated maximum: 16 MiB per device
static __device__ __align__(256) unsigned char g_static_partials[kStaticPartialsBytes];

static constexpr int kStaticMaxDevices = 64;
static void* g_static_partials_ptr[kStaticMaxDevices];  // address of the array on every device seen so far
static std::mutex g_static_mutex;

extern "C" int skv_decode_attention_static(const SkvStoreDesc* desc, const void* store, int layer,
                                           const void* plan, const void* query, int query_dtype,
                                           int num_q_heads, int num_ctas, float* logits, int32_t* err_flag,
                                           void** partials_out, void* stream) {
  if (!desc || !partials_out) return SKV_ERR_INVALID;
  *partials_out = nullptr;
  const int64_t need = skv_attn_partials_bytes(desc, num_q_heads, num_ctas);
  if (need < 0) return (int)need;
  if (need > kStaticPartialsBytes) {
    fprintf(stderr,
            "skv_decode_attention_static: this shape needs %lld bytes of partials, the fixed array holds %lld; "
            "use skv_decode_attention with a caller-owned buffer\n",
            (long long)need, kStaticPartialsBytes);
    return SKV_ERR_CAPACITY;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return SKV_ERR_CUDA;
  if (dev < 0 || dev >= kStaticMaxDevices) return SKV_ERR_UNSUPPORTED;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_static_mutex);
    if (g_static_partials_ptr[dev] == nullptr) {  // set-up, once per device: look the array up in the module
      void* sym = nullptr;
      const cudaError_t rc = cudaGetSymbolAddress(&sym, g_static_partials);
      if (rc != cudaSuccess || sym == nullptr) {
        fprintf(stderr, "skv_decode_attention_static: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(rc));
        return SKV_ERR_CUDA;
      }
      g_static_partials_ptr[dev] = sym;
    }
    scratch = g_static_partials_ptr[dev];
  }
  // Nothing in the array has to start at zero: the launch writes the (max, sum) header of every
  // partial the combine step reads before that step can run on the same stream.
  const int rc = skv_decode_attention(desc, store, layer, plan, query, query_dtype, num_q_heads, scratch, num_ctas,
                                      logits, err_flag, stream);
  if (rc == SKV_OK) *partials_out = scratch;
  return rc;
}
