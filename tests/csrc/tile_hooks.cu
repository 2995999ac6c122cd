// Test-only hooks (never part of libsmartkv_b200.so): raw tensor-core tile products through the same fragment
// code as the mma.sync decode-attention kernel, for one 16-key tile of packed rows (row_bytes apart).
// Built by tests/test_gpu_tile_products.py into tests/_build/libskv_tile_hooks.so.
#include "../../smartkv_b200/csrc/attn_frag.cuh"

using namespace skv;
static inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

namespace skv {
// q [16][D] fp16 (rows 0..7 heads, rows 8..15 residual rows), pm [16][16] fp16 laid out
// [row][key] (rows 0..7 heads, 8..15 residual rows); scores [8][16], out [8][D] (hi + residual).
template <int D, int BITS>
__global__ void debug_tile_kernel(const uint8_t* k_rows, const uint8_t* v_rows, const __half* q, const __half* pm,
                                  float* scores, float* out) {
  constexpr int PD = D * BITS / 8;
  __shared__ __align__(16) uint8_t ks[16 * PD + 16];
  __shared__ __align__(16) uint8_t vs[16 * PD + 16];
  __shared__ __align__(16) __half qs[16 * D];
  const int lane = threadIdx.x;
  for (int i = lane; i < 16 * PD; i += 32) {
    ks[i] = k_rows[i];
    vs[i] = v_rows[i];
  }
  for (int i = lane; i < 16 * D; i += 32) qs[i] = q[i];
  __syncwarp();
  const int g = lane >> 2, t = lane & 3;
  uint32_t qa[D / 16][4];
  gather_qa_f16<D, BITS>(qs, true, lane, qa);
  uint32_t kr0[SliceWords<D, BITS>::K], kr1[SliceWords<D, BITS>::K];
  load_kslice<D, BITS>(ks, g, t, kr0);
  load_kslice<D, BITS>(ks, g + 8, t, kr1);
  float c0[4], c1[4];
  qk_ntile_f16<D, BITS>(kr0, t, qa, c0);
  qk_ntile_f16<D, BITS>(kr1, t, qa, c1);
  scores[g * 16 + 2 * t] = c0[0] + c0[2];
  scores[g * 16 + 2 * t + 1] = c0[1] + c0[3];
  scores[g * 16 + 2 * t + 8] = c1[0] + c1[2];
  scores[g * 16 + 2 * t + 9] = c1[1] + c1[3];
  auto ld2 = [&](int r, int cidx) {
    return (uint32_t)reinterpret_cast<const unsigned short*>(pm)[r * 16 + cidx] |
           ((uint32_t)reinterpret_cast<const unsigned short*>(pm)[r * 16 + cidx + 1] << 16);
  };
  // P^T fragments: keys (2t, 2t+1) and (2t+8, 2t+9) of head g
  const uint32_t pb0 = ld2(g, 2 * t), pb1 = ld2(g, 2 * t + 8);
  const uint32_t pl0 = ld2(g + 8, 2 * t), pl1 = ld2(g + 8, 2 * t + 8);
  float o[D / 16][4];
  for (int j = 0; j < D / 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  uint32_t vr0[SliceWords<D, BITS>::V], vr1[SliceWords<D, BITS>::V], vr2[SliceWords<D, BITS>::V],
      vr3[SliceWords<D, BITS>::V];
  load_vrow<D, BITS>(vs, 2 * t, g, vr0);
  load_vrow<D, BITS>(vs, 2 * t + 1, g, vr1);
  load_vrow<D, BITS>(vs, 2 * t + 8, g, vr2);
  load_vrow<D, BITS>(vs, 2 * t + 9, g, vr3);
  uint32_t v0[D / 8], v1[D / 8];
  unpack_vpair<D, BITS>(vr0, vr1, g, v0);
  unpack_vpair<D, BITS>(vr2, vr3, g, v1);
  pv_tile<D, true>(v0, v1, pb0, pb1, pl0, pl1, o);
  for (int j = 0; j < D / 16; ++j) {
    const int d = g * (D / 8) + 2 * j;
    out[(2 * t) * D + d] = o[j][0];
    out[(2 * t + 1) * D + d] = o[j][1];
    out[(2 * t) * D + d + 1] = o[j][2];
    out[(2 * t + 1) * D + d + 1] = o[j][3];
  }
}

// q int8 [8][D]; scores int32 [8][16] = sum_d q[h][d] * u[key][d], u = stored code (offset-binary
// for 2/4-bit rows, two's complement for 8-bit rows).
template <int D, int BITS>
__global__ void debug_tile_i8_kernel(const uint8_t* k_rows, const int8_t* q, int* scores) {
  constexpr int PD = D * BITS / 8;
  __shared__ __align__(16) uint8_t ks[16 * PD + 16];
  __shared__ __align__(16) int8_t qs[8 * D];
  const int lane = threadIdx.x;
  for (int i = lane; i < 16 * PD; i += 32) ks[i] = k_rows[i];
  for (int i = lane; i < 8 * D; i += 32) qs[i] = q[i];
  __syncwarp();
  const int g = lane >> 2, t = lane & 3;
  uint32_t qa[D / 32][4];
  gather_qa_i8<D, BITS>(qs, nullptr, lane, qa);
  uint32_t kr0[SliceWords<D, BITS>::K], kr1[SliceWords<D, BITS>::K];
  load_kslice<D, BITS>(ks, g, t, kr0);
  load_kslice<D, BITS>(ks, g + 8, t, kr1);
  int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
  qk_ntile_i8<D, BITS>(kr0, qa, c0);
  qk_ntile_i8<D, BITS>(kr1, qa, c1);
  scores[g * 16 + 2 * t] = c0[0];
  scores[g * 16 + 2 * t + 1] = c0[1];
  scores[g * 16 + 2 * t + 8] = c1[0];
  scores[g * 16 + 2 * t + 9] = c1[1];
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

extern "C" int skv_test_tile_products(int head_dim, int bits, const uint8_t* k_rows, const uint8_t* v_rows,
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

extern "C" int skv_test_tile_scores_i8(int head_dim, int bits, const uint8_t* k_rows, const int8_t* q_int8,
                                        int32_t* scores, void* stream) {
  if (!k_rows || !q_int8 || !scores) return SKV_ERR_INVALID;
  cudaStream_t st = as_stream(stream);
  if (head_dim == 128) {
    if (bits == 2) debug_tile_i8_kernel<128, 2><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else if (bits == 3) debug_tile_i8_kernel<128, 3><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else if (bits == 4) debug_tile_i8_kernel<128, 4><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else if (bits == 8) debug_tile_i8_kernel<128, 8><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else return SKV_ERR_INVALID;
  } else if (head_dim == 64) {
    if (bits == 2) debug_tile_i8_kernel<64, 2><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else if (bits == 4) debug_tile_i8_kernel<64, 4><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else if (bits == 8) debug_tile_i8_kernel<64, 8><<<1, 32, 0, st>>>(k_rows, q_int8, scores);
    else return SKV_ERR_INVALID;
  } else {
    return SKV_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
