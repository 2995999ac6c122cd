// Fused packed-KV decode attention for sm_100a (q_len == 1, GQA group <= 8).
//
// Persistent CTAs (one per SM).  The packed buckets of every (sequence, KV head)
// are cut into blocks of a few KB (uniform bit-width per block); the global
// block list is split evenly -- i.e. by bytes -- over the CTAs, so a CTA owns a
// contiguous run of blocks that may span several (sequence, head) segments.
// Inside a segment the CTA's warps take blocks round-robin.  Each warp runs its
// own bulk-async-copy (TMA 1-D) pipeline into private shared-memory stages,
// unpacks the codes in registers straight into tensor-core fragments
// (attn_frag.cuh), keeps an online softmax and accumulates P.V in registers.
// At the end of a segment the warps' (max, sum, out) are merged through shared
// memory and one partial per (CTA, segment) is written; skv_lse_combine merges
// partials, adds the full-precision current token and normalises.
//
// Replaces smartkv/csrc/quantized_attention.cu:460-828 (per-bucket kernel, one
// CTA per head walking the whole context) and the host LSE combine in
// smartkv/kernels/__init__.py:350-371; numerics follow the CPU streaming path
// smartkv/core/fused_cpu.py:70-113 (dequantise, q.k/sqrt(d), online softmax).
#include "attn_frag.cuh"

namespace skv {

constexpr int kAttnWarps = 8;
constexpr int kAttnStages = 3;
constexpr int kStageBytes = 8448;
constexpr int kMaxSeqs = 4096;

// keys per block for a bit-width: as many as fit one stage (K rows + V rows + 2 fp32 scales per key)
__host__ __device__ constexpr int block_keys(int head_dim, int bits) {
  return (kStageBytes / (2 * row_bytes_for(head_dim, bits) + 8)) / 16 * 16;
}

struct AttnParams {
  StoreGeom g;
  const uint8_t* store;
  int layer;
  const int32_t* counts;
  const void* query;
  int q_is_half;
  int num_q_heads;
  int group;
  float* partials;
  int num_ctas;
  float* logits;
  int32_t* err;
  float scale_log2;
};

__host__ __device__ inline int partial_stride(int group, int head_dim) { return group * (head_dim + 2); }

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return h2_bits(h);
}

struct WarpState {
  float m;  // running max (log2 units) of this lane's query row
  float l;  // this lane's share of the running sum
};

template <int D, int BITS, bool PRECISE>
__device__ __forceinline__ void process_block(const uint8_t* sb, int nkeys, int lane,
                                              const uint32_t (&qa)[D / 16][4], WarpState& st, float (&o)[D / 8][4],
                                              float scale_log2, float* logit_row) {
  constexpr int PD = D * BITS / 8;
  constexpr int KB = block_keys(D, BITS);
  const uint8_t* kbase = sb;
  const uint8_t* vbase = sb + KB * PD;
  const float* ks = reinterpret_cast<const float*>(sb + 2 * KB * PD);
  const float* vs = ks + KB;
  const int t = lane & 3;
  const int ntiles = (nkeys + 15) >> 4;
  const float ninf = -INFINITY;
  for (int tile = 0; tile < ntiles; ++tile) {
    float s[2][4];
    qk_tile<D, BITS>(kbase + tile * 16 * PD, lane, qa, s);
    const int kk = tile * 16 + 2 * t;
    const float2 ks01 = *reinterpret_cast<const float2*>(ks + kk);
    const float2 ks23 = *reinterpret_cast<const float2*>(ks + kk + 8);
    float sv0 = s[0][0], sv1 = s[0][1], sv2 = s[1][0], sv3 = s[1][1];
    if (PRECISE) {
      sv0 += s[0][2];
      sv1 += s[0][3];
      sv2 += s[1][2];
      sv3 += s[1][3];
    }
    const bool ok0 = kk < nkeys, ok1 = kk + 1 < nkeys, ok2 = kk + 8 < nkeys, ok3 = kk + 9 < nkeys;
    sv0 = ok0 ? sv0 * (ks01.x * scale_log2) : ninf;
    sv1 = ok1 ? sv1 * (ks01.y * scale_log2) : ninf;
    sv2 = ok2 ? sv2 * (ks23.x * scale_log2) : ninf;
    sv3 = ok3 ? sv3 * (ks23.y * scale_log2) : ninf;
    if (logit_row != nullptr) {
      *reinterpret_cast<float2*>(logit_row + kk) = make_float2(sv0, sv1);
      *reinterpret_cast<float2*>(logit_row + kk + 8) = make_float2(sv2, sv3);
    }
    float mt = fmaxf(fmaxf(sv0, sv1), fmaxf(sv2, sv3));
    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
    if (__any_sync(0xffffffffu, mt > st.m)) {
      const float m_new = fmaxf(st.m, mt);
      const float alpha = (m_new == ninf) ? 1.f : ex2f(st.m - m_new);
      st.l *= alpha;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[j][0] *= alpha;
        o[j][1] *= alpha;
        if (PRECISE) {
          o[j][2] *= alpha;
          o[j][3] *= alpha;
        }
      }
      st.m = m_new;
    }
    const float mu = (st.m == ninf) ? 0.f : st.m;
    const float p0 = ex2f(sv0 - mu), p1 = ex2f(sv1 - mu), p2 = ex2f(sv2 - mu), p3 = ex2f(sv3 - mu);
    st.l += (p0 + p1) + (p2 + p3);
    const float2 vs01 = *reinterpret_cast<const float2*>(vs + kk);
    const float2 vs23 = *reinterpret_cast<const float2*>(vs + kk + 8);
    const float a0 = ok0 ? p0 * vs01.x : 0.f, a1 = ok1 ? p1 * vs01.y : 0.f;
    const float a2 = ok2 ? p2 * vs23.x : 0.f, a3 = ok3 ? p3 * vs23.y : 0.f;
    uint32_t pa[4];
    pa[0] = pack_h2(a0, a1);
    pa[2] = pack_h2(a2, a3);
    if (PRECISE) {
      const __half2 h01 = bits_h2(pa[0]), h23 = bits_h2(pa[2]);
      pa[1] = pack_h2(a0 - __low2float(h01), a1 - __high2float(h01));
      pa[3] = pack_h2(a2 - __low2float(h23), a3 - __high2float(h23));
    } else {
      pa[1] = 0u;
      pa[3] = 0u;
    }
    pv_tile<D, BITS>(vbase + tile * 16 * PD, lane, pa, o);
  }
}

template <int D, bool PRECISE>
__global__ void __launch_bounds__(kAttnWarps * 32, 1) decode_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const StoreGeom& g = p.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.group, Hkv = g.num_kv_heads, B = g.num_seqs;
  constexpr int NT = kAttnWarps * 32;

  uint8_t* stages = smem;                                         // [warps][stages][kStageBytes]
  __half* qs = reinterpret_cast<__half*>(smem + kAttnWarps * kAttnStages * kStageBytes);  // [16][D+pad]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(qs) + 16 * (D + kQPad) * 2);
  int* prefix = reinterpret_cast<int*>(bars + kAttnWarps * kAttnStages);  // [B+1] blocks before sequence b (per head)

  // ---- block schedule --------------------------------------------------------
  int kb[kNumBuckets];
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) kb[i] = block_keys(D, bucket_bits(i));
  for (int b = tid; b < B; b += NT) {
    int n = 0;
#pragma unroll
    for (int i = 0; i < kNumBuckets; ++i) n += (p.counts[b * kNumBuckets + i] + kb[i] - 1) / kb[i];
    prefix[b + 1] = n;
  }
  for (int i = tid; i < 16 * (D + kQPad); i += NT) qs[i] = __float2half(0.f);
  if (tid < kAttnWarps * kAttnStages) mbar_init(&bars[tid], 1);
  mbar_fence_init();
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    prefix[0] = 0;
    for (int b = 0; b < B; ++b) {
      acc += prefix[b + 1];
      prefix[b + 1] = acc;
    }
  }
  __syncthreads();
  const long long total_blocks = (long long)prefix[B] * Hkv;
  const int C = p.num_ctas, c = blockIdx.x;
  const long long x_begin = (total_blocks * c + C - 1) / C;
  const long long x_end = (total_blocks * (c + 1) + C - 1) / C;

  uint8_t* my_stages = stages + warp * kAttnStages * kStageBytes;
  uint64_t* my_bars = bars + warp * kAttnStages;
  uint32_t issued = 0, waited = 0;  // per-warp running counters (identical in all lanes)
  bool failed = false;

  long long x = x_begin;
  while (x < x_end) {
    // ---- locate the segment (sequence b, KV head h) holding global block x ----
    int lo = 0, hi = B;  // last b with Hkv*prefix[b] <= x
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if ((long long)prefix[mid] * Hkv <= x) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int nblk = prefix[b + 1] - prefix[b];
    const long long seq_first = (long long)prefix[b] * Hkv;
    const int h = (int)((x - seq_first) / nblk);
    const int r0 = (int)((x - seq_first) - (long long)h * nblk);
    const long long seg_end = seq_first + (long long)(h + 1) * nblk;
    const long long e = seg_end < x_end ? seg_end : x_end;
    const int r1 = r0 + (int)(e - x);
    const int seg = b * Hkv + h;

    int cnt[kNumBuckets], nb[kNumBuckets];
#pragma unroll
    for (int i = 0; i < kNumBuckets; ++i) {
      cnt[i] = p.counts[b * kNumBuckets + i];
      nb[i] = (cnt[i] + kb[i] - 1) / kb[i];
    }

    __syncthreads();  // previous segment's merge has finished with qs and the stages
    // ---- query rows of this group -> shared fp16 (rows 0..G-1 hi, 8..8+G-1 residual)
    for (int i = tid; i < G * D; i += NT) {
      const int gq = i / D, d = i - gq * D;
      const long long qi = ((long long)b * p.num_q_heads + h * G + gq) * D + d;
      float q = p.q_is_half ? __half2float(static_cast<const __half*>(p.query)[qi])
                            : static_cast<const float*>(p.query)[qi];
      const __half qh = __float2half_rn(q);
      qs[gq * (D + kQPad) + d] = qh;
      if (PRECISE) qs[(gq + 8) * (D + kQPad) + d] = __float2half_rn(q - __half2float(qh));
    }
    __syncthreads();

    // ---- this warp's blocks: r0 + warp, r0 + warp + W, ... < r1 ----------------
    WarpState st;
    st.m = -INFINITY;
    st.l = 0.f;
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    uint32_t qa[D / 16][4];
    int cur_bucket = -1;
    const uint8_t* arena = arena_ptr(g, p.store, p.layer, b);
    const int nmine = (r1 - r0 - warp + kAttnWarps - 1) / kAttnWarps;  // may be <= 0

    auto locate = [&](int r, int& bucket, int& k0, int& nkeys) {
      bucket = 0;
      int rr = r;
#pragma unroll
      for (int i = 0; i < kNumBuckets - 1; ++i) {
        if (bucket == i && rr >= nb[i]) {
          rr -= nb[i];
          bucket = i + 1;
        }
      }
      k0 = rr * kb[bucket];
      nkeys = min(kb[bucket], cnt[bucket] - k0);
    };
    auto issue = [&](int i) {  // lane 0 only
      int bucket, k0, nkeys;
      locate(r0 + warp + i * kAttnWarps, bucket, k0, nkeys);
      const int n16 = (nkeys + 15) & ~15;
      const int pd = g.row_bytes[bucket];
      const uint32_t stg = issued % kAttnStages;
      uint8_t* sb = my_stages + stg * kStageBytes;
      const long long row = (long long)h * g.cap[bucket] + k0;
      const uint32_t kbytes = (uint32_t)(n16 * pd), sbytes = (uint32_t)(n16 * 4);
      fence_proxy_async();
      mbar_expect_tx(&my_bars[stg], 2 * kbytes + 2 * sbytes);
      bulk_g2s(sb, arena + g.k_off[bucket] + row * pd, kbytes, &my_bars[stg]);
      bulk_g2s(sb + kb[bucket] * pd, arena + g.v_off[bucket] + row * pd, kbytes, &my_bars[stg]);
      bulk_g2s(sb + 2 * kb[bucket] * pd, arena + g.ks_off[bucket] + row * 4, sbytes, &my_bars[stg]);
      bulk_g2s(sb + 2 * kb[bucket] * pd + kb[bucket] * 4, arena + g.vs_off[bucket] + row * 4, sbytes,
               &my_bars[stg]);
    };

    if (!failed) {
      for (int i = 0; i < kAttnStages - 1 && i < nmine; ++i) {
        if (lane == 0) issue(i);
        ++issued;
      }
      for (int i = 0; i < nmine; ++i) {
        __syncwarp();
        if (i + kAttnStages - 1 < nmine) {
          if (lane == 0) issue(i + kAttnStages - 1);
          ++issued;
        }
        const uint32_t stg = waited % kAttnStages, par = (waited / kAttnStages) & 1;
        if (!mbar_wait_bounded(&my_bars[stg], par)) {
          failed = true;
          if (lane == 0) atomicExch(p.err, 1);
          break;
        }
        ++waited;
        int bucket, k0, nkeys;
        locate(r0 + warp + i * kAttnWarps, bucket, k0, nkeys);
        const uint8_t* sb = my_stages + stg * kStageBytes;
        const int gq = lane >> 2;
        float* logit_row = nullptr;
        if (p.logits != nullptr && gq < G)
          logit_row = p.logits + ((long long)b * p.num_q_heads + h * G + gq) * g.slots + g.bucket_base[bucket] + k0;
        if (bucket != cur_bucket) {
          cur_bucket = bucket;
          switch (bucket) {
            case 0: gather_q_frags<D, 2>(qs, lane, qa); break;
            case 1: gather_q_frags<D, 3>(qs, lane, qa); break;
            case 2: gather_q_frags<D, 4>(qs, lane, qa); break;
            default: gather_q_frags<D, 8>(qs, lane, qa); break;
          }
        }
        switch (bucket) {
          case 0: process_block<D, 2, PRECISE>(sb, nkeys, lane, qa, st, o, p.scale_log2, logit_row); break;
          case 1: process_block<D, 3, PRECISE>(sb, nkeys, lane, qa, st, o, p.scale_log2, logit_row); break;
          case 2: process_block<D, 4, PRECISE>(sb, nkeys, lane, qa, st, o, p.scale_log2, logit_row); break;
          default: process_block<D, 8, PRECISE>(sb, nkeys, lane, qa, st, o, p.scale_log2, logit_row); break;
        }
      }
    }
    // drain anything still in flight (only after a failed wait)
    while (waited < issued) {
      const uint32_t stg = waited % kAttnStages, par = (waited / kAttnStages) & 1;
      mbar_wait_bounded(&my_bars[stg], par);
      ++waited;
    }
    __syncwarp();

    // ---- merge the warps of this CTA and write the partial -----------------------
    {
      float lsum = st.l;
      lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
      lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
      float* scratch = reinterpret_cast<float*>(my_stages);  // [G][D+2], this warp's stage 0
      const int gq = lane >> 2, t = lane & 3;
      if (gq < G) {
        float* row = scratch + gq * (D + 2);
        if (t == 0) {
          row[0] = st.m;
          row[1] = lsum;
        }
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          float v0 = o[j][0], v1 = o[j][1];
          if (PRECISE) {
            v0 += o[j][2];
            v1 += o[j][3];
          }
          row[2 + (D / 8) * (2 * t) + j] = v0;
          row[2 + (D / 8) * (2 * t + 1) + j] = v1;
        }
      }
    }
    __syncthreads();
    {
      float* out = p.partials + (long long)(c + seg) * partial_stride(G, D);
      for (int i = tid; i < G * D; i += NT) {
        const int gq = i / D, d = i - gq * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
          const float* row = reinterpret_cast<const float*>(stages + w * kAttnStages * kStageBytes) + gq * (D + 2);
          M = fmaxf(M, row[0]);
        }
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
          const float* row = reinterpret_cast<const float*>(stages + w * kAttnStages * kStageBytes) + gq * (D + 2);
          const float mw = row[0];
          if (mw != -INFINITY) {
            const float f = ex2f(mw - M);
            acc += row[2 + d] * f;
            L += row[1] * f;
          }
        }
        float* orow = out + gq * (D + 2);
        orow[2 + d] = acc;
        if (d == 0) {
          orow[0] = M;
          orow[1] = L;
        }
      }
    }
    x = e;
  }
}

// ---- combine ----------------------------------------------------------------------
struct CombineParams {
  StoreGeom g;
  const int32_t* counts;
  const void* query;
  int q_is_half;
  int num_q_heads;
  int group;
  const float* partials;
  int num_ctas;
  const void* cur_k;
  const void* cur_v;
  int kv_is_half;
  float* out;
  float* lse_max;
  float* lse_sum;
  float* cur_prob;
  float scale_log2;
};

// one block (128 threads) per (sequence, KV head) segment
__global__ void lse_combine_kernel(const CombineParams p) {
  const StoreGeom& g = p.g;
  const int D = g.head_dim, G = p.group, Hkv = g.num_kv_heads, B = g.num_seqs;
  const int seg = blockIdx.x, b = seg / Hkv, h = seg - b * Hkv;
  const int tid = threadIdx.x, NT = blockDim.x;
  __shared__ long long s_before;  // blocks (per head) of the sequences before b
  __shared__ long long s_total;   // blocks (per head) of all sequences
  __shared__ int s_nblk;
  __shared__ float s_cur[8];

  int kb[kNumBuckets];
  for (int i = 0; i < kNumBuckets; ++i) kb[i] = block_keys(D, bucket_bits(i));
  if (tid == 0) {
    long long before = 0, total = 0;
    int mine = 0;
    for (int bb = 0; bb < B; ++bb) {
      int n = 0;
      for (int i = 0; i < kNumBuckets; ++i) n += (p.counts[bb * kNumBuckets + i] + kb[i] - 1) / kb[i];
      if (bb < b) before += n;
      if (bb == b) mine = n;
      total += n;
    }
    s_before = before;
    s_total = total;
    s_nblk = mine;
  }
  __syncthreads();
  const long long total_blocks = s_total * Hkv;
  const int nblk = s_nblk;
  const long long S = s_before * Hkv + (long long)h * nblk, E = S + nblk;
  const int C = p.num_ctas;
  int c_first = 0, c_last = -1;
  if (nblk > 0) {
    c_first = (int)((S * C) / total_blocks);
    c_last = (int)(((E - 1) * C) / total_blocks);
  }
  // CTA c holds a partial of this segment iff its block range meets [S, E)
  auto cta_has = [&](int c) {
    const long long lo = (total_blocks * c + C - 1) / C, hi = (total_blocks * (c + 1) + C - 1) / C;
    return (lo > S ? lo : S) < (hi < E ? hi : E);
  };

  // ---- current-token logits (full precision), one warp per group row -------------
  const bool has_cur = p.cur_k != nullptr && p.cur_v != nullptr;
  const int warp = tid >> 5, lane = tid & 31, nwarps = NT >> 5;
  if (has_cur) {
    for (int gq = warp; gq < G; gq += nwarps) {
      const long long qi = ((long long)b * p.num_q_heads + h * G + gq) * D;
      const long long ki = ((long long)b * Hkv + h) * D;
      float acc = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float q = p.q_is_half ? __half2float(static_cast<const __half*>(p.query)[qi + d])
                                    : static_cast<const float*>(p.query)[qi + d];
        const float k = p.kv_is_half ? __half2float(static_cast<const __half*>(p.cur_k)[ki + d])
                                     : static_cast<const float*>(p.cur_k)[ki + d];
        acc = fmaf(q, k, acc);
      }
      acc = warp_sum(acc);
      if (lane == 0) s_cur[gq] = acc * p.scale_log2;
    }
  }
  __syncthreads();

  const int pstride = partial_stride(G, D);
  for (int i = tid; i < G * D; i += NT) {
    const int gq = i / D, d = i - gq * D;
    float M = has_cur ? s_cur[gq] : -INFINITY;
    for (int c = c_first; c <= c_last; ++c) {
      if (!cta_has(c)) continue;
      const float* row = p.partials + (long long)(c + seg) * pstride + gq * (D + 2);
      M = fmaxf(M, row[0]);
    }
    float acc = 0.f, L = 0.f;
    for (int c = c_first; c <= c_last; ++c) {
      if (!cta_has(c)) continue;
      const float* row = p.partials + (long long)(c + seg) * pstride + gq * (D + 2);
      const float mw = row[0];
      if (mw != -INFINITY) {
        const float f = ex2f(mw - M);
        acc += row[2 + d] * f;
        L += row[1] * f;
      }
    }
    float pc = 0.f;
    if (has_cur) {
      pc = ex2f(s_cur[gq] - M);
      const long long vi = ((long long)b * Hkv + h) * D + d;
      const float v = p.kv_is_half ? __half2float(static_cast<const __half*>(p.cur_v)[vi])
                                   : static_cast<const float*>(p.cur_v)[vi];
      acc += pc * v;
      L += pc;
    }
    const long long hq = (long long)b * p.num_q_heads + h * G + gq;
    p.out[hq * D + d] = L > 0.f ? acc / L : 0.f;
    if (d == 0) {
      if (p.lse_max) p.lse_max[hq] = M;
      if (p.lse_sum) p.lse_sum[hq] = L;
      if (p.cur_prob) p.cur_prob[hq] = (has_cur && L > 0.f) ? pc / L : 0.f;
    }
  }
}

}  // namespace skv

using namespace skv;

static inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

static size_t attn_smem_bytes(int head_dim, int num_seqs) {
  return (size_t)kAttnWarps * kAttnStages * kStageBytes + 16 * (head_dim + kQPad) * 2 +
         kAttnWarps * kAttnStages * sizeof(uint64_t) + (size_t)(num_seqs + 1) * sizeof(int) + 16;
}

extern "C" int skv_attn_num_ctas(int device) {
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return SKV_ERR_CUDA;
  return sms;
}

extern "C" int64_t skv_attn_partials_bytes(const SkvStoreDesc* desc, int num_q_heads, int num_ctas) {
  if (!desc || num_ctas <= 0 || num_q_heads <= 0 || desc->num_kv_heads <= 0) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  const int64_t slots = (int64_t)num_ctas + (int64_t)desc->num_seqs * desc->num_kv_heads;
  return slots * partial_stride(group, desc->head_dim) * (int64_t)sizeof(float);
}

template <int D, bool PRECISE>
static int launch_attn(const AttnParams& p, size_t smem, cudaStream_t st) {
  static bool configured = false;  // per template instance
  if (!configured) {
    if (cudaFuncSetAttribute(decode_attn_kernel<D, PRECISE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(kAttnWarps * kAttnStages * kStageBytes + 16 * (D + kQPad) * 2 +
                                   kAttnWarps * kAttnStages * 8 + (kMaxSeqs + 1) * 4 + 16)) != cudaSuccess)
      return SKV_ERR_CUDA;
    configured = true;
  }
  decode_attn_kernel<D, PRECISE><<<p.num_ctas, kAttnWarps * 32, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

extern "C" int skv_decode_attention(const SkvStoreDesc* desc, const void* store, int layer, const int32_t* counts,
                                    const void* query, int query_dtype, int num_q_heads, void* partials,
                                    int num_ctas, float* logits, int32_t* err_flag, void* stream) {
  if (!desc || !store || !counts || !query || !partials || !err_flag) return SKV_ERR_INVALID;
  if (layer < 0 || layer >= desc->num_layers || num_ctas <= 0) return SKV_ERR_INVALID;
  if (desc->head_dim != 64 && desc->head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if (desc->num_seqs > kMaxSeqs) return SKV_ERR_UNSUPPORTED;
  if (num_q_heads % desc->num_kv_heads != 0) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  if (group < 1 || group > 8) return SKV_ERR_UNSUPPORTED;
  if (query_dtype != SKV_DTYPE_F32 && query_dtype != SKV_DTYPE_F16) return SKV_ERR_INVALID;
  AttnParams p;
  p.g = make_geom(*desc);
  p.store = static_cast<const uint8_t*>(store);
  p.layer = layer;
  p.counts = counts;
  p.query = query;
  p.q_is_half = query_dtype == SKV_DTYPE_F16;
  p.num_q_heads = num_q_heads;
  p.group = group;
  p.partials = static_cast<float*>(partials);
  p.num_ctas = num_ctas;
  p.logits = logits;
  p.err = err_flag;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)desc->head_dim));
  const size_t smem = attn_smem_bytes(desc->head_dim, desc->num_seqs);
  const bool precise = !p.q_is_half;
  if (desc->head_dim == 128)
    return precise ? launch_attn<128, true>(p, smem, as_stream(stream))
                   : launch_attn<128, false>(p, smem, as_stream(stream));
  return precise ? launch_attn<64, true>(p, smem, as_stream(stream))
                 : launch_attn<64, false>(p, smem, as_stream(stream));
}

extern "C" int skv_lse_combine(const SkvStoreDesc* desc, const int32_t* counts, const void* query, int query_dtype,
                               int num_q_heads, const void* partials, int num_ctas, const void* cur_k,
                               const void* cur_v, int kv_dtype, float* out, float* lse_max, float* lse_sum,
                               float* cur_prob, void* stream) {
  if (!desc || !counts || !query || !partials || !out) return SKV_ERR_INVALID;
  if (num_q_heads % desc->num_kv_heads != 0 || num_ctas <= 0) return SKV_ERR_INVALID;
  const int group = num_q_heads / desc->num_kv_heads;
  if (group < 1 || group > 8) return SKV_ERR_UNSUPPORTED;
  if ((cur_k == nullptr) != (cur_v == nullptr)) return SKV_ERR_INVALID;
  CombineParams p;
  p.g = make_geom(*desc);
  p.counts = counts;
  p.query = query;
  p.q_is_half = query_dtype == SKV_DTYPE_F16;
  p.num_q_heads = num_q_heads;
  p.group = group;
  p.partials = static_cast<const float*>(partials);
  p.num_ctas = num_ctas;
  p.cur_k = cur_k;
  p.cur_v = cur_v;
  p.kv_is_half = kv_dtype == SKV_DTYPE_F16;
  p.out = out;
  p.lse_max = lse_max;
  p.lse_sum = lse_sum;
  p.cur_prob = cur_prob;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)desc->head_dim));
  lse_combine_kernel<<<desc->num_seqs * desc->num_kv_heads, 128, 0, as_stream(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

// ---- debug: raw tile products through the production fragment code ----------------
namespace skv {
template <int D, int BITS>
__global__ void debug_tile_kernel(const uint8_t* k_rows, const uint8_t* v_rows, const __half* q, const __half* pm,
                                  float* scores, float* out) {
  constexpr int PD = D * BITS / 8;
  __shared__ __align__(16) uint8_t ks[16 * PD + 16];
  __shared__ __align__(16) uint8_t vs[16 * PD + 16];
  __shared__ __align__(16) __half qs[16 * (D + kQPad)];
  const int lane = threadIdx.x;
  for (int i = lane; i < 16 * PD; i += 32) {
    ks[i] = k_rows[i];
    vs[i] = v_rows[i];
  }
  for (int i = lane; i < 16 * D; i += 32) qs[(i / D) * (D + kQPad) + (i % D)] = q[i];
  __syncwarp();
  uint32_t qa[D / 16][4];
  gather_q_frags<D, BITS>(qs, lane, qa);
  float s[2][4];
  qk_tile<D, BITS>(ks, lane, qa, s);
  const int g = lane >> 2, t = lane & 3;
  for (int n = 0; n < 2; ++n) {
    scores[g * 16 + 8 * n + 2 * t] = s[n][0];
    scores[g * 16 + 8 * n + 2 * t + 1] = s[n][1];
    scores[(g + 8) * 16 + 8 * n + 2 * t] = s[n][2];
    scores[(g + 8) * 16 + 8 * n + 2 * t + 1] = s[n][3];
  }
  uint32_t pa[4];
  auto ld2 = [&](int r, int cidx) {
    return (uint32_t)reinterpret_cast<const unsigned short*>(pm)[r * 16 + cidx] |
           ((uint32_t)reinterpret_cast<const unsigned short*>(pm)[r * 16 + cidx + 1] << 16);
  };
  pa[0] = ld2(g, 2 * t);
  pa[1] = ld2(g + 8, 2 * t);
  pa[2] = ld2(g, 2 * t + 8);
  pa[3] = ld2(g + 8, 2 * t + 8);
  float o[D / 8][4];
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  pv_tile<D, BITS>(vs, lane, pa, o);
  for (int j = 0; j < D / 8; ++j) {
    out[g * D + (D / 8) * (2 * t) + j] = o[j][0];
    out[g * D + (D / 8) * (2 * t + 1) + j] = o[j][1];
    out[(g + 8) * D + (D / 8) * (2 * t) + j] = o[j][2];
    out[(g + 8) * D + (D / 8) * (2 * t + 1) + j] = o[j][3];
  }
}
}  // namespace skv

template <int D>
static int launch_debug(int bits, const uint8_t* k, const uint8_t* v, const __half* q, const __half* pm, float* s,
                        float* o, cudaStream_t st) {
  switch (bits) {
    case 2: debug_tile_kernel<D, 2><<<1, 32, 0, st>>>(k, v, q, pm, s, o); break;
    case 3: debug_tile_kernel<D, 3><<<1, 32, 0, st>>>(k, v, q, pm, s, o); break;
    case 4: debug_tile_kernel<D, 4><<<1, 32, 0, st>>>(k, v, q, pm, s, o); break;
    case 8: debug_tile_kernel<D, 8><<<1, 32, 0, st>>>(k, v, q, pm, s, o); break;
    default: return SKV_ERR_INVALID;
  }
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

extern "C" int skv_debug_tile_products(int head_dim, int bits, const uint8_t* k_rows, const uint8_t* v_rows,
                                       const void* q_half, const void* p_half, float* scores, float* out,
                                       void* stream) {
  if (!k_rows || !v_rows || !q_half || !p_half || !scores || !out) return SKV_ERR_INVALID;
  if (head_dim == 128)
    return launch_debug<128>(bits, k_rows, v_rows, static_cast<const __half*>(q_half),
                             static_cast<const __half*>(p_half), scores, out, as_stream(stream));
  if (head_dim == 64)
    return launch_debug<64>(bits, k_rows, v_rows, static_cast<const __half*>(q_half),
                            static_cast<const __half*>(p_half), scores, out, as_stream(stream));
  return SKV_ERR_UNSUPPORTED;
}
