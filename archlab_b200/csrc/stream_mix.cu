// Per-token mixing of a few wide rows: out[t, o, :] = sum_j W[t, o, j] * in[t, j, :].
// The inputs may come from two tensors (in_a: na rows per token, in_b: nb rows), which covers both
// halves of a hyper-connection without concatenating: the read (1 x n weights over the n residual
// streams) and the write-back (n x (n + 1) weights over the streams and the sublayer output), as well
// as the 4-stream gated residual.  Weights are fp32 and differ per token; rows are bf16.
// The weight gradient dW[t, o, j] = <dout[t, o, :], in[t, j, :]> is a second kernel; the input gradient
// is the first kernel again with W transposed.  One warp per token, 16-byte accesses.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"
#include "misc_kernels.h"

namespace nga {
namespace {

constexpr int MIX_MAX = 8;      // rows in (na + nb) and rows out

__device__ __forceinline__ void mix_ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint32_t mix_pk(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int NO>
__global__ void __launch_bounds__(256)
token_mix_kernel(const __nv_bfloat16* __restrict__ in_a, const __nv_bfloat16* __restrict__ in_b, const float* __restrict__ W,
                 __nv_bfloat16* __restrict__ out, long long tokens, int na, int nb, int C, int transpose_w, int ldw) {
  const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int lane = threadIdx.x & 31, ni = na + nb;
  // weights of this token: w[o][j]; with transpose_w the stored matrix is [ni][NO']
  float w[NO][MIX_MAX];
#pragma unroll
  for (int o = 0; o < NO; ++o)
#pragma unroll
    for (int j = 0; j < MIX_MAX; ++j)
      w[o][j] = j < ni ? (transpose_w ? W[t * ldw + (long long)j * NO + o] : W[t * ldw + (long long)o * ni + j]) : 0.f;
  for (int c = lane * 8; c < C; c += 256) {
    float acc[NO][8];
#pragma unroll
    for (int o = 0; o < NO; ++o)
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[o][k] = 0.f;
#pragma unroll
    for (int j = 0; j < MIX_MAX; ++j) {
      if (j < ni) {
        float x[8];
        mix_ld8(j < na ? in_a + (t * na + j) * C + c : in_b + (t * nb + (j - na)) * C + c, x);
#pragma unroll
        for (int o = 0; o < NO; ++o)
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[o][k] = fmaf(w[o][j], x[k], acc[o][k]);
      }
    }
#pragma unroll
    for (int o = 0; o < NO; ++o) {
      uint4 u;
      u.x = mix_pk(acc[o][0], acc[o][1]);
      u.y = mix_pk(acc[o][2], acc[o][3]);
      u.z = mix_pk(acc[o][4], acc[o][5]);
      u.w = mix_pk(acc[o][6], acc[o][7]);
      *reinterpret_cast<uint4*>(out + (t * NO + o) * C + c) = u;
    }
  }
}

// dW[t, o, j] = sum_c dout[t, o, c] * in[t, j, c]
template <int NO>
__global__ void __launch_bounds__(256)
token_mix_dw_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ in_a,
                    const __nv_bfloat16* __restrict__ in_b, float* __restrict__ dW, long long tokens, int na, int nb, int C) {
  const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int lane = threadIdx.x & 31, ni = na + nb;
  float acc[NO][MIX_MAX];
#pragma unroll
  for (int o = 0; o < NO; ++o)
#pragma unroll
    for (int j = 0; j < MIX_MAX; ++j) acc[o][j] = 0.f;
  for (int c = lane * 8; c < C; c += 256) {
    float g[NO][8];
#pragma unroll
    for (int o = 0; o < NO; ++o) mix_ld8(dout + (t * NO + o) * C + c, g[o]);
#pragma unroll
    for (int j = 0; j < MIX_MAX; ++j) {
      if (j < ni) {
        float x[8];
        mix_ld8(j < na ? in_a + (t * na + j) * C + c : in_b + (t * nb + (j - na)) * C + c, x);
#pragma unroll
        for (int o = 0; o < NO; ++o)
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[o][j] = fmaf(g[o][k], x[k], acc[o][j]);
      }
    }
  }
#pragma unroll
  for (int o = 0; o < NO; ++o)
#pragma unroll
    for (int j = 0; j < MIX_MAX; ++j) {
      if (j < ni) {
        float v = acc[o][j];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0) dW[(t * NO + o) * ni + j] = v;
      }
    }
}

}  // namespace
}  // namespace nga

using namespace nga;
#define MIX_DISPATCH(NOUT, CALL)              \
  switch (NOUT) {                             \
    case 1: { constexpr int NO = 1; CALL; break; } \
    case 2: { constexpr int NO = 2; CALL; break; } \
    case 3: { constexpr int NO = 3; CALL; break; } \
    case 4: { constexpr int NO = 4; CALL; break; } \
    case 5: { constexpr int NO = 5; CALL; break; } \
    case 8: { constexpr int NO = 8; CALL; break; } \
    default: return -2;                       \
  }

// out [tokens, n_out, C]; W [tokens, n_out, na + nb] (or its transpose [tokens, na + nb, n_out] when transpose_w).
extern "C" int nga_token_mix(const void* in_a, const void* in_b, const float* W, void* out, long long tokens, int na, int nb,
                             int n_out, int C, int transpose_w, void* stream) {
  if (tokens <= 0 || na < 0 || nb < 0 || na + nb < 1 || na + nb > MIX_MAX || n_out < 1 || C <= 0 || (C & 7)) return -1;
  const unsigned blocks = (unsigned)((tokens + 7) / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int ldw = n_out * (na + nb);
  MIX_DISPATCH(n_out, (token_mix_kernel<NO><<<blocks, 256, 0, st>>>(
                          reinterpret_cast<const __nv_bfloat16*>(in_a), reinterpret_cast<const __nv_bfloat16*>(in_b), W,
                          reinterpret_cast<__nv_bfloat16*>(out), tokens, na, nb, C, transpose_w, ldw)));
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_token_mix_dw(const void* dout, const void* in_a, const void* in_b, float* dW, long long tokens, int na, int nb,
                                int n_out, int C, void* stream) {
  if (tokens <= 0 || na < 0 || nb < 0 || na + nb < 1 || na + nb > MIX_MAX || n_out < 1 || C <= 0 || (C & 7)) return -1;
  const unsigned blocks = (unsigned)((tokens + 7) / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  MIX_DISPATCH(n_out, (token_mix_dw_kernel<NO><<<blocks, 256, 0, st>>>(
                          reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(in_a),
                          reinterpret_cast<const __nv_bfloat16*>(in_b), dW, tokens, na, nb, C)));
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
