// Budgeted bit allocation on the device.
//
// Replaces SmartKVCache.allocate_precision / _solve_allocation
// (smartkv/core/cache.py:281-351, 353-601), a Python heap loop over every cached
// token, for all sequences of the batch at once.
//
// The heap pops (token, step) items by (gain-per-bit desc, token id asc); an item is
// pushed only after the token's previous step was accepted.  Give every item the
// *effective key* min(own score, effective key of the token's previous step): sorted
// by (effective key desc, token id asc, step asc) the items come out in exactly the
// heap's pop order.  The walk over the sorted items then has two phases:
//   1. while the memory ratio is below 0.85 * budget nothing is gated and (for all but
//      tiny caches) every step is affordable, so everything is accepted: the payload
//      is a prefix sum and the phase ends at the first position c1 whose prefix
//      reaches 0.85 * budget (cache.py:468-472: a token accepted past the gate is not
//      pushed again);
//   2. after c1 a token can be accepted once more, and only if its previous step lies
//      before c1; those items are accepted greedily while they fit, skipping items that
//      do not (cache.py:502-505).  Step costs take at most three values, and once an
//      item of some cost fails every later item of that or a larger cost fails too, so
//      the walk is a few prefix sums with cut points instead of a serial loop.
// Caches so small that a single step can jump from below the gate to above the budget
// are walked serially by one thread with the same rules.
// The rank-percentile / streak state of the hysteresis (cache.py:423-450) is kept per
// token in storage order, and the high-priority post-pass (cache.py:522-591) runs as a
// serial kernel that returns at once when it has nothing to do (the usual case).
//
// All score arithmetic is fp64 in the reference's operation order; the powers
// bits^alpha come from the host so that they are the host libm's values.
#include <cub/block/block_reduce.cuh>
#include <cub/block/block_scan.cuh>
#include <cub/device/device_radix_sort.cuh>

#include <cmath>

#include "common.cuh"

namespace skv {

constexpr int kAllocThreads = 256;
constexpr int kScanThreads = 1024;
constexpr uint32_t kPadFlag = 0x80000000u;
constexpr int kStepsMax = 3;  // steps between the (up to) four widths

struct AllocCfgDev {
  int num_heads, head_dim;
  int nb;            // number of available widths
  int bits[4];       // ascending
  double util[4];    // bits^alpha
  double budget, floor_, rank_thr, high_frac, high_boost;
  int intervals, min_high, scale_bits, critical_window;
  int nprot;
  int prot[SKV_ALLOC_MAX_PROTECTED];
};

struct SeqInfo {
  int n;              // live tokens
  int n_prot;         // protected tokens (max bits, not ranked)
  int n_scored;       // unprotected tokens with a finite positive score
  int want;           // size of the high-priority set
  int gated0;         // baseline ratio already past the gate
  int serial;         // walk serially (tiny cache)
  long long payload;  // payload bits after the walk
  int changed;        // tokens whose width differs from their current bucket
  int pad_;
};

// Workspace carved out of one caller buffer.
struct AllocWs {
  uint64_t *k64a, *k64b;
  uint32_t *v32a, *v32b, *v32c;
  uint32_t *k32a, *k32b;
  uint32_t* tok_gslot;   // [NT] id order -> global slot (b*T + s), pad flagged
  uint32_t* rank_src;    // [NT] rank order -> id-order index
  uint32_t* item_src;    // [3NT] walk order -> item index
  int32_t* posof;        // [3NT] item index -> walk position
  double* tok_score;     // [NT]
  uint8_t* tok_flags;    // [NT] bit0 protected, bit1 high, bit2 blocked (serial walk), bit3 reset streak
  int32_t* tok_acc;      // [NT] accepted steps
  uint8_t* item_valid;   // [3NT]
  SeqInfo* info;         // [B]
  void* cub_temp;
  size_t cub_bytes;
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct AllocParams {
  StoreGeom g;
  AllocCfgDev c;
  int T;  // slots
  const int32_t* counts;
  const int32_t* slot_token;
  const double* scores;
  const double* recency;
  double* rank_pct;
  int8_t* rank_streak;
  uint8_t* new_bits;
  int32_t* new_counts;
  int32_t* changed;
  AllocWs w;
};

__device__ __forceinline__ uint64_t desc_key(double x) {
  uint64_t u = (uint64_t)__double_as_longlong(x);
  u = (u >> 63) ? ~u : (u | 0x8000000000000000ull);  // ascending-sortable
  return ~u;                                         // descending
}

__device__ __forceinline__ bool is_protected(const AllocCfgDev& c, int id) {
  if (id < c.critical_window) return true;
  for (int i = 0; i < c.nprot; ++i)
    if (c.prot[i] == id) return true;
  return false;
}
__device__ __forceinline__ bool in_protected_list(const AllocCfgDev& c, int id) {
  for (int i = 0; i < c.nprot; ++i)
    if (c.prot[i] == id) return true;
  return false;
}

// ratio(payload) of cache.py:374-388 for n tokens
__device__ __forceinline__ double mem_ratio(const AllocCfgDev& c, int n, long long payload_bits) {
  const double elements = (double)(2 * c.num_heads * c.head_dim);
  const double scale_total = (double)((long long)n * 2 * c.num_heads * c.scale_bits);
  const double fp16_total = (double)n * elements * 16.0;
  return fp16_total > 0.0 ? ((double)payload_bits + scale_total) / fp16_total : 0.0;
}

__device__ __forceinline__ int slot_bucket(const StoreGeom& g, int s) {
  int b = 0;
#pragma unroll
  for (int i = 1; i < kNumBuckets; ++i)
    if (s >= g.bucket_base[i]) b = i;
  return b;
}

// ---- 1. live tokens of every sequence, keyed by token id ----------------------------------
__global__ void alloc_gather_kernel(const AllocParams p) {
  const int b = blockIdx.y, j = blockIdx.x * kAllocThreads + threadIdx.x, T = p.T;
  if (j >= T) return;
  int cnt[kNumBuckets], n = 0;
#pragma unroll
  for (int i = 0; i < kNumBuckets; ++i) {
    cnt[i] = p.counts[b * kNumBuckets + i];
    n += cnt[i];
  }
  const long long gi = (long long)b * T + j;
  if (j == 0) {
    SeqInfo si = {};
    si.n = n;
    p.w.info[b] = si;
  }
  if (j < n) {
    int rem = j, s = 0;
#pragma unroll
    for (int i = 0; i < kNumBuckets; ++i) {
      if (rem >= 0 && rem < cnt[i]) s = p.g.bucket_base[i] + rem;
      rem -= cnt[i];
      if (rem < 0) rem = -(1 << 30);
    }
    p.w.k64a[gi] = (uint64_t)(uint32_t)p.slot_token[(long long)b * T + s];
    p.w.v32a[gi] = (uint32_t)(b * T + s);
  } else {
    p.w.k64a[gi] = ~0ull;
    p.w.v32a[gi] = (uint32_t)gi | kPadFlag;
  }
}

// sequence of every payload, as the key of the second (stable) pass that brings each
// sequence's entries back together
__global__ void alloc_seqkey_kernel(const uint32_t* payload, uint32_t* key, long long n, int per_seq) {
  const long long i = (long long)blockIdx.x * kAllocThreads + threadIdx.x;
  if (i < n) key[i] = (payload[i] & ~kPadFlag) / (uint32_t)per_seq;
}

// ---- 2. scores -> descending sort keys -------------------------------------------------------
__global__ void alloc_score_kernel(const AllocParams p) {
  const int b = blockIdx.y, j = blockIdx.x * kAllocThreads + threadIdx.x, T = p.T;
  if (j >= T) return;
  const long long gi = (long long)b * T + j;
  const uint32_t gs = p.w.tok_gslot[gi];
  p.w.tok_acc[gi] = 0;
  if (gs & kPadFlag) {
    p.w.k64a[gi] = ~0ull;
    p.w.v32a[gi] = (uint32_t)gi | kPadFlag;
    p.w.tok_flags[gi] = 0;
    return;
  }
  const int id = p.slot_token[gs];
  double score = p.scores[gs];
  if (p.recency) score *= p.recency[gs];
  const bool prot = is_protected(p.c, id);
  if (prot) score = INFINITY;
  p.w.tok_score[gi] = score;
  p.w.tok_flags[gi] = prot ? 1 : 0;
  if (prot) p.w.tok_acc[gi] = p.c.nb - 1;  // protected tokens sit at the widest width (cache.py:364-368)
  p.w.k64a[gi] = prot ? ~0ull : desc_key(score);
  p.w.v32a[gi] = (uint32_t)gi;
  if (prot) {
    atomicAdd(&p.w.info[b].n_prot, 1);
  } else if (isfinite(score) && score > 0.0) {
    atomicAdd(&p.w.info[b].n_scored, 1);
  }
}

// ---- 3. ranks, hysteresis state, high-priority set, item keys -------------------------------
__global__ void alloc_items_kernel(const AllocParams p) {
  const int b = blockIdx.y, r = blockIdx.x * kAllocThreads + threadIdx.x, T = p.T;
  if (r >= T) return;
  const AllocCfgDev& c = p.c;
  const long long gr = (long long)b * T + r;
  const uint32_t src = p.w.rank_src[gr];
  const long long gp = (long long)(src & ~kPadFlag);  // id-order index (global)
  uint64_t* ikey = p.w.k64a + 3 * gp;
  uint32_t* ival = p.w.v32a + 3 * gp;
  uint8_t* ivalid = p.w.item_valid + 3 * gp;
  const SeqInfo si = p.w.info[b];
  const bool pad = (src & kPadFlag) != 0;
#pragma unroll
  for (int i = 0; i < kStepsMax; ++i) {
    ikey[i] = ~0ull;
    ival[i] = (uint32_t)(3 * gp + i) | (pad ? kPadFlag : 0u);
    ivalid[i] = 0;
  }
  if (pad) return;

  const int n = si.n, n_ranked = n - si.n_prot;
  const int lo = c.bits[0], hi = c.bits[c.nb - 1];
  // sequence-wide facts (every thread of the sequence computes the same values)
  int want = 0;
  if (c.high_frac > 0.0 || c.min_high > 0) {
    if (si.n_scored > 0) {
      const int byfrac = (int)ceil((double)si.n_scored * c.high_frac);
      want = c.min_high > byfrac ? c.min_high : byfrac;
      if (want > si.n_scored) want = si.n_scored;
    }
  }
  const long long payload0 = (long long)(n - si.n_prot) * lo * (2 * c.num_heads * c.head_dim) +
                             (long long)si.n_prot * hi * (2 * c.num_heads * c.head_dim);
  const bool gated0 = mem_ratio(c, n, payload0) >= c.budget * 0.85;
  const int max_cost = [&] {
    int m = 0;
    for (int i = 0; i + 1 < c.nb; ++i) m = (c.bits[i + 1] - c.bits[i]) > m ? (c.bits[i + 1] - c.bits[i]) : m;
    return m;
  }();
  // a single step may carry the ratio from below the gate past the budget: walk serially
  const double step_ratio = (double)max_cost / ((double)n * 16.0);
  const bool serial = !(step_ratio * 1.0000001 + 1e-9 < 0.15 * c.budget - 1e-6);
  if (r == 0) {
    SeqInfo* o = &p.w.info[b];
    o->want = want;
    o->gated0 = gated0 ? 1 : 0;
    o->serial = serial ? 1 : 0;
    o->payload = payload0;
  }

  const uint32_t gs = p.w.tok_gslot[gp];
  uint8_t flags = p.w.tok_flags[gp];
  const bool prot = flags & 1;
  int8_t streak = p.rank_streak[gs];
  if (prot) {
    // cache.py:448-450: an unranked token without state gets the neutral record
    if (streak < 0) {
      p.rank_pct[gs] = 1.0;
      p.rank_streak[gs] = (int8_t)c.intervals;
    }
    return;
  }
  // rank percentile and streak (cache.py:423-446)
  const int den = (n_ranked - 1) > 1 ? (n_ranked - 1) : 1;
  const double pct = n_ranked == 1 ? 0.0 : (double)r / (double)den;
  if (streak < 0) {
    streak = (int8_t)c.intervals;
  } else {
    const bool moved = fabs(pct - p.rank_pct[gs]) >= c.rank_thr;
    streak = moved ? (int8_t)((streak + 1) < c.intervals ? (streak + 1) : c.intervals) : (int8_t)0;
  }
  p.rank_pct[gs] = pct;
  p.rank_streak[gs] = streak;
  const bool high = r < want;  // positive finite scores sort first, so rank < want implies both
  if (high) flags |= 2;
  p.w.tok_flags[gp] = flags;

  // items (cache.py:455-482)
  double imp = p.w.tok_score[gp];
  if (!isfinite(imp)) imp = c.floor_ > 0.0 ? c.floor_ : 0.0;
  if (imp <= 0.0) {
    if (c.floor_ <= 0.0) return;
    imp = c.floor_;
  }
  if (gated0 && streak < c.intervals) return;  // not even the first step is pushed
  double eff = INFINITY;
  for (int i = 0; i + 1 < c.nb; ++i) {
    const int cur = c.bits[i], nxt = c.bits[i + 1];
    double v = imp;
    if (high && nxt >= hi) v *= c.high_boost;
    const double gain = c.util[i + 1] - c.util[i];
    if (gain <= 0.0 || nxt - cur <= 0) break;
    const double own = (v * gain) / (double)(nxt - cur);
    eff = own < eff ? own : eff;
    ikey[i] = desc_key(eff);
    ivalid[i] = 1;
  }
}

// ---- 4. the walk ---------------------------------------------------------------------------------
struct WalkShared {
  long long payload;
  int phase;      // 1 = before the gate, 2 = after it
  int c1;         // position of the accept that reached the gate (-1: gated from the start)
  int dead_cost;  // steps of this cost or more no longer fit
  int start;      // next position to look at
  int event;      // local index of the first event of the chunk, or kScanThreads
  int done;
};

__global__ void __launch_bounds__(kScanThreads) alloc_walk_kernel(const AllocParams p) {
  const int b = blockIdx.x, tid = threadIdx.x, T = p.T;
  const AllocCfgDev& c = p.c;
  const SeqInfo si = p.w.info[b];
  const int n = si.n, n_items = 3 * n;
  const uint32_t* order = p.w.item_src + (long long)b * 3 * T;
  int32_t* posof = p.w.posof;  // indexed by global item index
  const long long elements = 2LL * c.num_heads * c.head_dim;
  using Scan = cub::BlockScan<int, kScanThreads>;
  using MinReduce = cub::BlockReduce<int, kScanThreads>;
  __shared__ typename Scan::TempStorage scan_tmp;
  __shared__ typename MinReduce::TempStorage red_tmp;
  __shared__ WalkShared ws;
  if (n == 0) return;

  for (int pos = tid; pos < n_items; pos += kScanThreads) posof[order[pos] & ~kPadFlag] = pos;
  if (tid == 0) {
    ws.payload = si.payload;
    ws.phase = si.gated0 ? 2 : 1;
    ws.c1 = -1;
    ws.dead_cost = 1 << 30;
    ws.start = 0;
    ws.done = 0;
  }
  __syncthreads();

  if (si.serial) {
    // tiny cache: the literal walk (accept iff the token sits at the step's width, is not
    // gate-blocked and the step fits)
    if (tid == 0) {
      long long P = si.payload;
      const double gate = c.budget * 0.85, limit = c.budget + 1e-6;
      for (int pos = 0; pos < n_items; ++pos) {
        const uint32_t it = order[pos] & ~kPadFlag;
        if (!p.w.item_valid[it]) continue;
        const long long gp = it / 3;
        const int step = (int)(it - 3 * gp);
        if (p.w.tok_acc[gp] != step || (p.w.tok_flags[gp] & 4)) continue;
        const long long delta = (long long)(c.bits[step + 1] - c.bits[step]) * elements;
        if (mem_ratio(c, n, P + delta) > limit) continue;
        p.w.tok_acc[gp] = step + 1;
        P += delta;
        p.w.tok_flags[gp] |= 8;
        if (mem_ratio(c, n, P) >= gate) p.w.tok_flags[gp] |= 4;
      }
      p.w.info[b].payload = P;
    }
    return;
  }

  const double gate = c.budget * 0.85, limit = c.budget + 1e-6;
  int min_cost = 1 << 30;
  for (int i = 0; i + 1 < c.nb; ++i) min_cost = min(min_cost, c.bits[i + 1] - c.bits[i]);

  while (true) {
    __syncthreads();
    const int start = ws.start, phase = ws.phase, c1 = ws.c1, dead = ws.dead_cost;
    const long long P = ws.payload;
    if (ws.done || start >= n_items) break;
    const int pos = start + tid;
    int cost = 0;
    long long gp = 0;
    int step = 0;
    bool elig = false;
    if (pos < n_items) {
      const uint32_t it = order[pos] & ~kPadFlag;
      if (p.w.item_valid[it]) {
        gp = it / 3;
        step = (int)(it - 3 * gp);
        cost = c.bits[step + 1] - c.bits[step];
        elig = phase == 1 || (cost < dead && (step == 0 || posof[it - 1] < c1));
      }
    }
    const int w = elig ? cost : 0;
    int incl;
    Scan(scan_tmp).InclusiveSum(w, incl);
    // first event of the chunk
    int ev = kScanThreads;
    if (elig) {
      const double ratio = mem_ratio(c, n, P + (long long)incl * elements);
      if (phase == 1 ? (ratio >= gate) : (ratio > limit)) ev = tid;
    }
    ev = MinReduce(red_tmp).Reduce(ev, cub::Min());
    if (tid == 0) ws.event = ev;
    __syncthreads();
    ev = ws.event;
    // phase 1: the item that reaches the gate is itself accepted; phase 2: the failing item is not
    const bool accept = elig && (phase == 1 ? tid <= ev : tid < ev);
    if (accept) {
      atomicMax(&p.w.tok_acc[gp], step + 1);
      p.w.tok_flags[gp] |= 8;  // two steps of one token may set the same bit at once: same value either way
    }
    if (ev < kScanThreads) {
      if (tid == ev) {
        if (phase == 1) {
          ws.payload = P + (long long)incl * elements;
          ws.phase = 2;
          ws.c1 = pos;
        } else {
          ws.payload = P + (long long)(incl - cost) * elements;
          ws.dead_cost = cost;
          if (cost <= min_cost) ws.done = 1;
        }
        ws.start = pos + 1;
      }
    } else if (tid == kScanThreads - 1) {
      ws.payload = P + (long long)incl * elements;
      ws.start = start + kScanThreads;
    }
  }
  __syncthreads();
  if (tid == 0) p.w.info[b].payload = ws.payload;
}

// ---- 5. high-priority post-pass (cache.py:522-591) ------------------------------------------------
// Usually nothing to do: the top-ranked tokens reach the widest width in phase 1.  When one of
// them did not, one thread replays the reference's loop literally.
__global__ void alloc_highpass_kernel(const AllocParams p) {
  const int b = blockIdx.x, tid = threadIdx.x, T = p.T;
  const AllocCfgDev& c = p.c;
  const SeqInfo si = p.w.info[b];
  const int want = si.want, nb = c.nb, hi = c.bits[nb - 1];
  const uint32_t* rank = p.w.rank_src + (long long)b * T;
  __shared__ int s_need;
  if (tid == 0) s_need = 0;
  __syncthreads();
  for (int r = tid; r < want; r += blockDim.x) {
    const long long gp = rank[r] & ~kPadFlag;
    if ((p.w.tok_flags[gp] & 2) && c.bits[p.w.tok_acc[gp]] < hi) s_need = 1;
  }
  __syncthreads();
  if (!s_need || tid != 0) return;

  const int n = si.n, n_ranked = n - si.n_prot;
  const long long elements = 2LL * c.num_heads * c.head_dim;
  const double limit = c.budget + 1e-6;
  long long P = si.payload;
  int32_t* undo = reinterpret_cast<int32_t*>(p.w.v32b) + (long long)b * 3 * T;  // free after the sorts
  for (int r = 0; r < want; ++r) {
    const long long gt = rank[r] & ~kPadFlag;
    if (!(p.w.tok_flags[gt] & 2)) continue;
    const int cur = c.bits[p.w.tok_acc[gt]];
    if (cur >= hi) continue;
    const long long delta = (long long)(hi - cur) * elements;
    double cand = mem_ratio(c, n, P + delta);
    if (cand > limit) {
      int n_undo = 0;
      bool fits = false;
      // victims in ascending score, equal scores in ascending id: walk the ranking from its tail,
      // each run of equal scores front to back; then the window-protected tokens (score +inf)
      auto try_victim = [&](long long gc) -> bool {
        const uint8_t f = p.w.tok_flags[gc];
        if ((f & 2) || gc == gt) return false;
        // tokens on the protected list are never victims; a token protected only by the
        // critical window can be (cache.py:541-546 filters on the list alone)
        if ((f & 1) && in_protected_list(c, p.slot_token[p.w.tok_gslot[gc]])) return false;
        const int acc = p.w.tok_acc[gc];
        if (acc <= 0) return false;
        const long long give = (long long)(c.bits[acc] - c.bits[acc - 1]) * elements;
        p.w.tok_acc[gc] = acc - 1;
        P -= give;
        undo[n_undo++] = (int32_t)(gc - (long long)b * T);
        cand = mem_ratio(c, n, P + delta);
        return cand <= limit;
      };
      int r2 = n_ranked - 1;
      while (r2 >= 0 && !fits) {
        int g0 = r2;
        const double sc = p.w.tok_score[rank[r2] & ~kPadFlag];
        while (g0 > 0 && p.w.tok_score[rank[g0 - 1] & ~kPadFlag] == sc) --g0;
        for (int q = g0; q <= r2 && !fits; ++q) fits = try_victim((long long)(rank[q] & ~kPadFlag));
        r2 = g0 - 1;
      }
      for (int q = n_ranked; q < n && !fits; ++q) fits = try_victim((long long)(rank[q] & ~kPadFlag));
      if (!fits) {
        for (int u = n_undo - 1; u >= 0; --u) {
          const long long gc = (long long)b * T + undo[u];
          const int acc = p.w.tok_acc[gc];
          P += (long long)(c.bits[acc + 1] - c.bits[acc]) * elements;
          p.w.tok_acc[gc] = acc + 1;
        }
        continue;
      }
      for (int u = 0; u < n_undo; ++u) p.w.tok_flags[(long long)b * T + undo[u]] |= 8;
    }
    p.w.tok_acc[gt] = nb - 1;
    P += delta;
    p.w.tok_flags[gt] |= 8;
  }
  p.w.info[b].payload = P;
}

// ---- 6. results in storage order -----------------------------------------------------------------
__global__ void alloc_finish_kernel(const AllocParams p) {
  const int b = blockIdx.y, j = blockIdx.x * kAllocThreads + threadIdx.x, T = p.T;
  const AllocCfgDev& c = p.c;
  __shared__ int s_hist[kNumBuckets];
  __shared__ int s_changed;
  if (threadIdx.x < kNumBuckets) s_hist[threadIdx.x] = 0;
  if (threadIdx.x == 0) s_changed = 0;
  __syncthreads();
  if (j < T) {
    const long long gp = (long long)b * T + j;
    const uint32_t gs = p.w.tok_gslot[gp];
    if (!(gs & kPadFlag)) {
      const uint8_t f = p.w.tok_flags[gp];
      const int bits = c.bits[p.w.tok_acc[gp]];
      p.new_bits[gs] = (uint8_t)bits;
      if (f & 8) p.rank_streak[gs] = 0;  // accepted or touched by the post-pass (cache.py:511-514)
      atomicAdd(&s_hist[bits_bucket(bits)], 1);
      if (bucket_bits(slot_bucket(p.g, (int)(gs - (uint32_t)(b * T)))) != bits) atomicAdd(&s_changed, 1);
    }
  }
  __syncthreads();
  if (threadIdx.x < kNumBuckets && s_hist[threadIdx.x]) atomicAdd(&p.new_counts[b * kNumBuckets + threadIdx.x], s_hist[threadIdx.x]);
  if (threadIdx.x == 0 && s_changed) atomicAdd(&p.changed[b], s_changed);
}

__global__ void alloc_clear_kernel(uint8_t* new_bits, long long n, int32_t* new_counts, int32_t* changed, int B) {
  const long long i = (long long)blockIdx.x * kAllocThreads + threadIdx.x;
  if (i < n) new_bits[i] = 0;
  if (i < B * kNumBuckets) new_counts[i] = 0;
  if (i < B) changed[i] = 0;
}

}  // namespace skv

using namespace skv;

namespace {

size_t cub_temp_bytes(long long items) {
  size_t a = 0, b = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, (const uint64_t*)nullptr, (uint64_t*)nullptr, (const uint32_t*)nullptr,
                                  (uint32_t*)nullptr, items);
  cub::DeviceRadixSort::SortPairs(nullptr, b, (const uint32_t*)nullptr, (uint32_t*)nullptr, (const uint32_t*)nullptr,
                                  (uint32_t*)nullptr, items);
  return a > b ? a : b;
}

// lays the workspace out inside `base` (nullptr: size query); returns the bytes needed
size_t carve(AllocWs& w, void* base, long long NT) {
  size_t off = 0;
  auto take = [&](size_t bytes) -> void* {
    void* ptr = base ? static_cast<uint8_t*>(base) + off : nullptr;
    off += align_up(bytes, 256);
    return ptr;
  };
  w.k64a = (uint64_t*)take(3 * NT * 8);
  w.k64b = (uint64_t*)take(3 * NT * 8);
  w.v32a = (uint32_t*)take(3 * NT * 4);
  w.v32b = (uint32_t*)take(3 * NT * 4);
  w.v32c = (uint32_t*)take(3 * NT * 4);
  w.k32a = (uint32_t*)take(3 * NT * 4);
  w.k32b = (uint32_t*)take(3 * NT * 4);
  w.tok_gslot = (uint32_t*)take(NT * 4);
  w.rank_src = (uint32_t*)take(NT * 4);
  w.item_src = (uint32_t*)take(3 * NT * 4);
  w.posof = (int32_t*)take(3 * NT * 4);
  w.tok_score = (double*)take(NT * 8);
  w.tok_flags = (uint8_t*)take(NT);
  w.tok_acc = (int32_t*)take(NT * 4);
  w.item_valid = (uint8_t*)take(3 * NT);
  w.info = (SeqInfo*)take(1024 * sizeof(SeqInfo));
  w.cub_bytes = cub_temp_bytes(3 * NT);
  w.cub_temp = take(w.cub_bytes);
  return off;
}

int seq_bits(int B) {
  int b = 1;
  while ((1 << b) < B) ++b;
  return b;
}

// (key64, payload) -> payload order by (sequence, key64 asc, original order): a stable sort by the
// key followed by a stable sort by the sequence the payload belongs to
int sort_by_key_then_seq(AllocWs& w, long long items, int per_seq, int B, int key_bits, uint32_t* out,
                         cudaStream_t st) {
  size_t tb = w.cub_bytes;
  if (B == 1) {
    if (cub::DeviceRadixSort::SortPairs(w.cub_temp, tb, w.k64a, w.k64b, w.v32a, out, items, 0, key_bits, st) !=
        cudaSuccess)
      return SKV_ERR_CUDA;
    return SKV_OK;
  }
  if (cub::DeviceRadixSort::SortPairs(w.cub_temp, tb, w.k64a, w.k64b, w.v32a, w.v32b, items, 0, key_bits, st) !=
      cudaSuccess)
    return SKV_ERR_CUDA;
  alloc_seqkey_kernel<<<(unsigned)((items + kAllocThreads - 1) / kAllocThreads), kAllocThreads, 0, st>>>(
      w.v32b, w.k32a, items, per_seq);
  tb = w.cub_bytes;
  if (cub::DeviceRadixSort::SortPairs(w.cub_temp, tb, w.k32a, w.k32b, w.v32b, out, items, 0, seq_bits(B), st) !=
      cudaSuccess)
    return SKV_ERR_CUDA;
  return SKV_OK;
}

}  // namespace

extern "C" int64_t skv_alloc_workspace_bytes(const SkvStoreDesc* desc) {
  if (!desc || desc->num_seqs <= 0 || desc->slots <= 0) return SKV_ERR_INVALID;
  AllocWs w;
  return (int64_t)carve(w, nullptr, (long long)desc->num_seqs * desc->slots);
}

extern "C" int skv_alloc_bits(const SkvStoreDesc* desc, const SkvAllocConfig* cfg, const int32_t* counts,
                              const int32_t* slot_token, const double* scores, const double* recency,
                              double* rank_pct, int8_t* rank_streak, uint8_t* new_bits, int32_t* new_counts,
                              int32_t* changed, void* workspace, void* stream) {
  if (!desc || !cfg || !counts || !slot_token || !scores || !rank_pct || !rank_streak || !new_bits || !new_counts ||
      !changed || !workspace)
    return SKV_ERR_INVALID;
  if (cfg->num_bits < 1 || cfg->num_bits > 4 || cfg->num_protected < 0 || cfg->num_protected > SKV_ALLOC_MAX_PROTECTED)
    return SKV_ERR_INVALID;
  if (!cfg->use_packing) return SKV_ERR_UNSUPPORTED;  // the store is always packed
  if (desc->num_seqs > 1024) return SKV_ERR_UNSUPPORTED;
  for (int i = 0; i < cfg->num_bits; ++i) {
    if (bits_bucket(cfg->bits[i]) < 0) return SKV_ERR_INVALID;
    if (i > 0 && cfg->bits[i] <= cfg->bits[i - 1]) return SKV_ERR_INVALID;
  }
  const int B = desc->num_seqs, T = desc->slots;
  const long long NT = (long long)B * T;
  if (3 * NT >= (1ll << 31)) return SKV_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AllocParams p;
  p.g = make_geom(*desc);
  p.T = T;
  p.c.num_heads = cfg->num_heads;
  p.c.head_dim = cfg->head_dim;
  p.c.nb = cfg->num_bits;
  for (int i = 0; i < 4; ++i) {
    p.c.bits[i] = i < cfg->num_bits ? cfg->bits[i] : 0;
    p.c.util[i] = i < cfg->num_bits ? cfg->util[i] : 0.0;
  }
  p.c.budget = cfg->memory_budget;
  p.c.floor_ = cfg->importance_floor > 0.0 ? cfg->importance_floor : 0.0;
  p.c.rank_thr = cfg->rank_threshold > 0.0 ? cfg->rank_threshold : 0.0;
  p.c.high_frac = cfg->high_fraction < 0.0 ? 0.0 : (cfg->high_fraction > 0.5 ? 0.5 : cfg->high_fraction);
  p.c.high_boost = cfg->high_boost < 1.0 ? 1.0 : cfg->high_boost;
  p.c.intervals = cfg->hysteresis_intervals < 1 ? 1 : cfg->hysteresis_intervals;
  p.c.min_high = cfg->min_high_tokens < 0 ? 0 : cfg->min_high_tokens;
  p.c.scale_bits = cfg->scale_bits == 16 ? 16 : 32;
  p.c.critical_window = cfg->critical_window;
  p.c.nprot = cfg->num_protected;
  for (int i = 0; i < SKV_ALLOC_MAX_PROTECTED; ++i) p.c.prot[i] = i < cfg->num_protected ? cfg->protected_ids[i] : -1;
  p.counts = counts;
  p.slot_token = slot_token;
  p.scores = scores;
  p.recency = recency;
  p.rank_pct = rank_pct;
  p.rank_streak = rank_streak;
  p.new_bits = new_bits;
  p.new_counts = new_counts;
  p.changed = changed;
  carve(p.w, workspace, NT);

  const dim3 tgrid((T + kAllocThreads - 1) / kAllocThreads, B);
  alloc_clear_kernel<<<(unsigned)((NT + kAllocThreads - 1) / kAllocThreads), kAllocThreads, 0, st>>>(new_bits, NT,
                                                                                                     new_counts, changed, B);
  alloc_gather_kernel<<<tgrid, kAllocThreads, 0, st>>>(p);
  int rc = sort_by_key_then_seq(p.w, NT, T, B, 33, p.w.tok_gslot, st);  // token ids (pads carry bit 63..: all ones)
  if (rc != SKV_OK) return rc;
  alloc_score_kernel<<<tgrid, kAllocThreads, 0, st>>>(p);
  rc = sort_by_key_then_seq(p.w, NT, T, B, 64, p.w.rank_src, st);
  if (rc != SKV_OK) return rc;
  alloc_items_kernel<<<tgrid, kAllocThreads, 0, st>>>(p);
  rc = sort_by_key_then_seq(p.w, 3 * NT, 3 * T, B, 64, p.w.item_src, st);
  if (rc != SKV_OK) return rc;
  alloc_walk_kernel<<<B, kScanThreads, 0, st>>>(p);
  alloc_highpass_kernel<<<B, 256, 0, st>>>(p);
  alloc_finish_kernel<<<tgrid, kAllocThreads, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
