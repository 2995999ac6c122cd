// Causal self-attention over the unquantised prompt (more than one query token against an empty
// cache), with the per-key attention mass the importance tracker needs -- without ever writing the
// [batch, heads, queries, keys] probability tensor to memory.
//
//   pass 1 (prefill_fwd_kernel):  per (64-query tile, query head, sequence) the usual streaming
//       softmax: S = Q K^T, running max / sum, O += P V; writes O (fp16) and, per query row, the
//       log-sum-exp in base-2 units.
//   pass 2 (prefill_mass_kernel): per (64-key tile, KV head, sequence) the transposed product
//       S^T = K Q^T over every query tile at or after the key tile and every query head of the group;
//       with the row normalisers of pass 1, p = exp2(s - lse[q]) is final, and its sum over the
//       queries, weighted by the head weight, is the key's mass.  One value per (sequence, KV head,
//       key) is written; the caller adds the KV heads (a fixed order, so the result is reproducible).
//
// Both products are GEMM tiles on mma.sync m16n8k16 (fp16 in, fp32 accumulate): the prompt pass runs
// once per sequence, reads O(n) bytes for O(n^2) arithmetic, and is a small part of a generation.
#include <cuda_fp16.h>

#include "common.cuh"

namespace skv {

constexpr int kPfTile = 64;     // queries per CTA tile and keys per streamed tile
constexpr int kPfThreads = 128;  // 4 warps x 16 rows

struct PrefillParams {
  const __half* q;
  const __half* k;
  const __half* v;
  long long q_sb, q_st, q_sh;  // element strides of batch, token, head (head_dim is contiguous)
  long long k_sb, k_st, k_sh;
  long long v_sb, v_st, v_sh;
  __half* out;                 // [batch][tokens][q heads][head_dim]
  float* lse;                  // [batch][q heads][tokens], base-2
  const float* head_w;         // [batch][q heads] or null
  float* mass;                 // [batch][kv heads][tokens]
  int batch, tokens, num_q_heads, num_kv_heads;
  float scale_log2;
};

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem_row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Copies rows [row0, row0 + 64) x D halves of a strided [tokens][D] matrix into shared memory with row
// stride LD; rows at or beyond `tokens` are zero.
template <int D, int LD>
__device__ __forceinline__ void load_tile(__half* dst, const __half* src, long long token_stride, int row0, int tokens) {
  constexpr int CH = D / 8;  // 16-byte chunks per row
  for (int i = threadIdx.x; i < kPfTile * CH; i += kPfThreads) {
    const int r = i / CH, c = i % CH;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + r < tokens) val = *reinterpret_cast<const uint4*>(src + (long long)(row0 + r) * token_stride + c * 8);
    *reinterpret_cast<uint4*>(dst + r * LD + c * 8) = val;
  }
}

// A fragments (16 rows x D) of this warp's rows out of a shared tile [64][LD]
template <int D, int LD>
__device__ __forceinline__ void load_a_frags(const __half* tile, int warp, int lane, uint32_t (&a)[D / 16][4]) {
  const int g = lane >> 2, t = lane & 3;
  const __half* r0 = tile + (warp * 16 + g) * LD;
  const __half* r1 = r0 + 8 * LD;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    a[kk][0] = *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + 2 * t);
    a[kk][1] = *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + 2 * t);
    a[kk][2] = *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + 2 * t + 8);
    a[kk][3] = *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + 2 * t + 8);
  }
}

// c[j] (j = 0..7: eight 8-column tiles) = A (16 x D, registers) times the transpose of the shared tile [64][LD]
template <int D, int LD>
__device__ __forceinline__ void gemm_a_bt(const uint32_t (&a)[D / 16][4], const __half* tile, int lane, float (&c)[8][4]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
    const __half* row = tile + (j * 8 + g) * LD + 2 * t;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(row + kk * 16);
      const uint32_t b1 = *reinterpret_cast<const uint32_t*>(row + kk * 16 + 8);
      mma_f16(c[j], a[kk], b0, b1);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kPfThreads) prefill_fwd_kernel(const PrefillParams p) {
  constexpr int LD = D + 8;
  extern __shared__ __align__(16) uint8_t pf_smem[];
  __half* ks = reinterpret_cast<__half*>(pf_smem);  // [64][LD], first used for the query tile
  __half* vs = ks + kPfTile * LD;                   // [64][LD]
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // the longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.num_q_heads / p.num_kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n = p.tokens, q0 = qt * kPfTile;

  load_tile<D, LD>(ks, p.q + b * p.q_sb + h * p.q_sh, p.q_st, q0, n);
  __syncthreads();
  uint32_t qa[D / 16][4];
  load_a_frags<D, LD>(ks, warp, lane, qa);
  __syncthreads();

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8 of this warp
  const int row0 = q0 + warp * 16 + g, row1 = row0 + 8;

  const __half* kbase = p.k + b * p.k_sb + hk * p.k_sh;
  const __half* vbase = p.v + b * p.v_sb + hk * p.v_sh;
  for (int kt = 0; kt <= qt; ++kt) {
    const int k0 = kt * kPfTile;
    load_tile<D, LD>(ks, kbase, p.k_st, k0, n);
    load_tile<D, LD>(vs, vbase, p.v_st, k0, n);
    __syncthreads();
    float s[8][4];
    gemm_a_bt<D, LD>(qa, ks, lane, s);
    // scale, causal mask (only the diagonal tile and the ragged end need it)
    const bool edge = kt == qt || k0 + kPfTile > n;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[j][e] * p.scale_log2;
        if (edge) {
          const int key = k0 + j * 8 + 2 * t + (e & 1);
          const int row = (e < 2) ? row0 : row1;
          if (key > row || key >= n) x = -INFINITY;
        }
        s[j][e] = x;
      }
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float a0 = (n0 == -INFINITY) ? 1.f : fast_exp2(m0 - n0), a1 = (n1 == -INFINITY) ? 1.f : fast_exp2(m1 - n1);
    const float u0 = (n0 == -INFINITY) ? 0.f : n0, u1 = (n1 == -INFINITY) ? 0.f : n1;
    m0 = n0;
    m1 = n1;
    l0 *= a0;
    l1 *= a1;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= a0;
      o[j][1] *= a0;
      o[j][2] *= a1;
      o[j][3] *= a1;
    }
    uint32_t pa[4][4];  // P as A fragments: four 16-key steps
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = fast_exp2(s[j][0] - u0), p1 = fast_exp2(s[j][1] - u0);
      const float p2 = fast_exp2(s[j][2] - u1), p3 = fast_exp2(s[j][3] - u1);
      l0 += p0 + p1;
      l1 += p2 + p3;
      pa[j >> 1][(j & 1) * 2] = pack_half2(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_half2(p2, p3);
    }
    // O += P V : B fragments of V (keys x dims) through transposing matrix loads
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const __half* vrow = vs + (kk * 16 + (lane & 15)) * LD;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        uint32_t b0, b1;
        ldmatrix_x2_trans(b0, b1, vrow + j * 8);
        mma_f16(o[j], pa[kk], b0, b1);
      }
    }
    __syncthreads();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  if (t == 0) {
    float* lse = p.lse + ((long long)b * p.num_q_heads + h) * n;
    if (row0 < n) lse[row0] = m0 + log2f(l0);
    if (row1 < n) lse[row1] = m1 + log2f(l1);
  }
  __half* ob = p.out + ((long long)b * n * p.num_q_heads + h) * D;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    if (row0 < n)
      *reinterpret_cast<__half2*>(ob + (long long)row0 * p.num_q_heads * D + j * 8 + 2 * t) =
          __floats2half2_rn(o[j][0] * i0, o[j][1] * i0);
    if (row1 < n)
      *reinterpret_cast<__half2*>(ob + (long long)row1 * p.num_q_heads * D + j * 8 + 2 * t) =
          __floats2half2_rn(o[j][2] * i1, o[j][3] * i1);
  }
}

template <int D>
__global__ void __launch_bounds__(kPfThreads) prefill_mass_kernel(const PrefillParams p) {
  constexpr int LD = D + 8;
  extern __shared__ __align__(16) uint8_t pf_smem[];
  __half* qs = reinterpret_cast<__half*>(pf_smem);                  // [64][LD]: key tile first, then query tiles
  float* lse_s = reinterpret_cast<float*>(qs + kPfTile * LD);       // [64]
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.num_q_heads / p.num_kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n = p.tokens, k0 = kt * kPfTile;
  const int nqt = (n + kPfTile - 1) / kPfTile;

  load_tile<D, LD>(qs, p.k + b * p.k_sb + hk * p.k_sh, p.k_st, k0, n);
  __syncthreads();
  uint32_t ka[D / 16][4];
  load_a_frags<D, LD>(qs, warp, lane, ka);
  __syncthreads();

  const int key0 = k0 + warp * 16 + g, key1 = key0 + 8;
  float acc0 = 0.f, acc1 = 0.f;
  for (int hh = 0; hh < G; ++hh) {
    const int h = hk * G + hh;
    const float w = p.head_w != nullptr ? p.head_w[(long long)b * p.num_q_heads + h] : 1.f;
    const float* lse = p.lse + ((long long)b * p.num_q_heads + h) * n;
    float h0 = 0.f, h1 = 0.f;
    for (int qt = kt; qt < nqt; ++qt) {
      const int q0 = qt * kPfTile;
      load_tile<D, LD>(qs, p.q + b * p.q_sb + h * p.q_sh, p.q_st, q0, n);
      if (threadIdx.x < kPfTile) lse_s[threadIdx.x] = (q0 + threadIdx.x < n) ? lse[q0 + threadIdx.x] : INFINITY;
      __syncthreads();
      float s[8][4];
      gemm_a_bt<D, LD>(ka, qs, lane, s);
      const bool edge = qt == kt;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qi = j * 8 + 2 * t + (e & 1);
          // a query beyond the prompt carries lse = +inf, which makes its probability zero
          float pr = fast_exp2(s[j][e] * p.scale_log2 - lse_s[qi]);
          if (edge && q0 + qi < ((e < 2) ? key0 : key1)) pr = 0.f;  // causal: the query precedes the key
          if (e < 2) h0 += pr; else h1 += pr;
        }
      }
      __syncthreads();
    }
    acc0 = fmaf(w, h0, acc0);
    acc1 = fmaf(w, h1, acc1);
  }
  acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
  acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
  acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
  acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
  if (t == 0) {
    float* m = p.mass + ((long long)b * p.num_kv_heads + hk) * n;
    if (key0 < n) m[key0] = acc0;
    if (key1 < n) m[key1] = acc1;
  }
}

template <int D>
static int launch_prefill(const PrefillParams& p, bool want_mass, cudaStream_t st) {
  constexpr int LD = D + 8;
  const int tiles = (p.tokens + kPfTile - 1) / kPfTile;
  const size_t smem_fwd = 2 * (size_t)kPfTile * LD * sizeof(__half);
  const size_t smem_mass = (size_t)kPfTile * LD * sizeof(__half) + kPfTile * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fwd) != cudaSuccess)
      return SKV_ERR_CUDA;
    configured = true;
  }
  prefill_fwd_kernel<D><<<dim3(tiles, p.num_q_heads, p.batch), kPfThreads, smem_fwd, st>>>(p);
  if (want_mass)
    prefill_mass_kernel<D><<<dim3(tiles, p.num_kv_heads, p.batch), kPfThreads, smem_mass, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

}  // namespace skv

using namespace skv;

extern "C" int skv_prefill_attention(const void* q, const void* k, const void* v, int dtype, int batch, int tokens,
                                     int num_q_heads, int num_kv_heads, int head_dim, const int64_t* q_strides,
                                     const int64_t* k_strides, const int64_t* v_strides, const float* head_weights,
                                     void* out, float* lse, float* key_mass, void* stream) {
  if (!q || !k || !v || !out || !lse || !q_strides || !k_strides || !v_strides) return SKV_ERR_INVALID;
  if (dtype != SKV_DTYPE_F16) return SKV_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128) return SKV_ERR_UNSUPPORTED;
  if (batch <= 0 || tokens <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return SKV_ERR_INVALID;
  if (batch > 65535 || num_q_heads > 65535) return SKV_ERR_UNSUPPORTED;
  for (int i = 0; i < 3; ++i)  // 16-byte vector loads of every row
    if (q_strides[i] % 8 || k_strides[i] % 8 || v_strides[i] % 8) return SKV_ERR_INVALID;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) return SKV_ERR_INVALID;
  PrefillParams p;
  p.q = static_cast<const __half*>(q);
  p.k = static_cast<const __half*>(k);
  p.v = static_cast<const __half*>(v);
  p.q_sb = q_strides[0]; p.q_st = q_strides[1]; p.q_sh = q_strides[2];
  p.k_sb = k_strides[0]; p.k_st = k_strides[1]; p.k_sh = k_strides[2];
  p.v_sb = v_strides[0]; p.v_st = v_strides[1]; p.v_sh = v_strides[2];
  p.out = static_cast<__half*>(out);
  p.lse = lse;
  p.head_w = head_weights;
  p.mass = key_mass;
  p.batch = batch;
  p.tokens = tokens;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)head_dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return head_dim == 64 ? launch_prefill<64>(p, key_mass != nullptr, st) : launch_prefill<128>(p, key_mass != nullptr, st);
}
