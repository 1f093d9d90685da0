// Hyper-connection coefficients for n = 4 streams, one thread per token, forward and backward.
//   logits = mixes * scale[group] + base                       (groups: pre [4], post [4], comb [16])
//   pre  = sigmoid(logits[0:4]) + eps
//   post = 2 sigmoid(logits[4:8])
//   comb = softmax over each row of logits[8:24] viewed [4][4], + eps; one column normalisation
//          c / (colsum + eps); then (iters - 1) x { row normalisation, column normalisation } (each + eps)
// (the arithmetic of hc_split_sinkhorn in src/archlab/architectures/deepseek_v41_math.py:14-33).
// In PyTorch this is ~45 tiny kernels forward and twice that backward per call; here one launch each.  The backward
// re-runs the forward keeping every iterate in thread-local memory and walks the steps in reverse.
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"
#include "misc_kernels.h"

namespace nga {
namespace {

constexpr int HC_N = 4;
constexpr int HC_W = (HC_N + 2) * HC_N;   // 24
constexpr int HC_MAX_ITERS = 32;

__device__ __forceinline__ void row_norm(const float* in, float* out, float eps) {
#pragma unroll
  for (int r = 0; r < HC_N; ++r) {
    float s = eps;
#pragma unroll
    for (int c = 0; c < HC_N; ++c) s += in[r * HC_N + c];
    const float inv = 1.f / s;
#pragma unroll
    for (int c = 0; c < HC_N; ++c) out[r * HC_N + c] = in[r * HC_N + c] * inv;
  }
}
__device__ __forceinline__ void col_norm(const float* in, float* out, float eps) {
#pragma unroll
  for (int c = 0; c < HC_N; ++c) {
    float s = eps;
#pragma unroll
    for (int r = 0; r < HC_N; ++r) s += in[r * HC_N + c];
    const float inv = 1.f / s;
#pragma unroll
    for (int r = 0; r < HC_N; ++r) out[r * HC_N + c] = in[r * HC_N + c] * inv;
  }
}
// y = x / (sum_group(x) + eps): dx_i = (dy_i - sum_group(dy * y)) / (sum + eps); `x` is the input iterate
__device__ __forceinline__ void row_norm_bwd(const float* x, const float* dy, float* dx, float eps) {
#pragma unroll
  for (int r = 0; r < HC_N; ++r) {
    float s = eps, dot = 0.f;
#pragma unroll
    for (int c = 0; c < HC_N; ++c) s += x[r * HC_N + c];
    const float inv = 1.f / s;
#pragma unroll
    for (int c = 0; c < HC_N; ++c) dot += dy[r * HC_N + c] * x[r * HC_N + c] * inv;
#pragma unroll
    for (int c = 0; c < HC_N; ++c) dx[r * HC_N + c] = (dy[r * HC_N + c] - dot) * inv;
  }
}
__device__ __forceinline__ void col_norm_bwd(const float* x, const float* dy, float* dx, float eps) {
#pragma unroll
  for (int c = 0; c < HC_N; ++c) {
    float s = eps, dot = 0.f;
#pragma unroll
    for (int r = 0; r < HC_N; ++r) s += x[r * HC_N + c];
    const float inv = 1.f / s;
#pragma unroll
    for (int r = 0; r < HC_N; ++r) dot += dy[r * HC_N + c] * x[r * HC_N + c] * inv;
#pragma unroll
    for (int r = 0; r < HC_N; ++r) dx[r * HC_N + c] = (dy[r * HC_N + c] - dot) * inv;
  }
}

__global__ void hc_coeff_fwd_kernel(const float* __restrict__ mixes, const float* __restrict__ scale, const float* __restrict__ base,
                                    float* __restrict__ pre, float* __restrict__ post, float* __restrict__ comb, long long T,
                                    int iters, float eps) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* m = mixes + t * HC_W;
  float a[16], b[16];
#pragma unroll
  for (int i = 0; i < HC_N; ++i) {
    pre[t * HC_N + i] = 1.f / (1.f + __expf(-(m[i] * scale[0] + base[i]))) + eps;
    post[t * HC_N + i] = 2.f / (1.f + __expf(-(m[HC_N + i] * scale[1] + base[HC_N + i])));
  }
#pragma unroll
  for (int r = 0; r < HC_N; ++r) {
    float l[HC_N], mx = -INFINITY, s = 0.f;
#pragma unroll
    for (int c = 0; c < HC_N; ++c) {
      l[c] = m[2 * HC_N + r * HC_N + c] * scale[2] + base[2 * HC_N + r * HC_N + c];
      mx = fmaxf(mx, l[c]);
    }
#pragma unroll
    for (int c = 0; c < HC_N; ++c) {
      l[c] = __expf(l[c] - mx);
      s += l[c];
    }
#pragma unroll
    for (int c = 0; c < HC_N; ++c) a[r * HC_N + c] = l[c] / s + eps;
  }
  col_norm(a, b, eps);
  for (int it = 1; it < iters; ++it) {
    row_norm(b, a, eps);
    col_norm(a, b, eps);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) comb[t * 16 + i] = b[i];
}

__global__ void __launch_bounds__(128)
hc_coeff_bwd_kernel(const float* __restrict__ mixes, const float* __restrict__ scale, const float* __restrict__ base,
                    const float* __restrict__ dpre, const float* __restrict__ dpost, const float* __restrict__ dcomb,
                    float* __restrict__ dmixes, float* __restrict__ dscale, float* __restrict__ dbase, long long T, int iters,
                    float eps) {
  __shared__ float red[HC_W + 3];
  if (threadIdx.x < HC_W + 3) red[threadIdx.x] = 0.f;
  __syncthreads();
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float dl[HC_W];                                     // gradient w.r.t. the 24 logits of this token
#pragma unroll
  for (int i = 0; i < HC_W; ++i) dl[i] = 0.f;
  float mloc[HC_W];
  if (t < T) {
    const float* m = mixes + t * HC_W;
#pragma unroll
    for (int i = 0; i < HC_W; ++i) mloc[i] = m[i];
#pragma unroll
    for (int i = 0; i < HC_N; ++i) {
      const float s0 = 1.f / (1.f + __expf(-(mloc[i] * scale[0] + base[i])));
      dl[i] = dpre[t * HC_N + i] * s0 * (1.f - s0);
      const float s1 = 1.f / (1.f + __expf(-(mloc[HC_N + i] * scale[1] + base[HC_N + i])));
      dl[HC_N + i] = dpost[t * HC_N + i] * 2.f * s1 * (1.f - s1);
    }
    // forward again, keeping the input of every normalisation step
    float hist[2 * HC_MAX_ITERS][16];                 // [step][16]: step 0 = softmax + eps, then alternating col / row inputs
    float p[16];
#pragma unroll
    for (int r = 0; r < HC_N; ++r) {
      float l[HC_N], mx = -INFINITY, s = 0.f;
#pragma unroll
      for (int c = 0; c < HC_N; ++c) {
        l[c] = mloc[2 * HC_N + r * HC_N + c] * scale[2] + base[2 * HC_N + r * HC_N + c];
        mx = fmaxf(mx, l[c]);
      }
#pragma unroll
      for (int c = 0; c < HC_N; ++c) {
        l[c] = __expf(l[c] - mx);
        s += l[c];
      }
#pragma unroll
      for (int c = 0; c < HC_N; ++c) {
        p[r * HC_N + c] = l[c] / s;
        hist[0][r * HC_N + c] = p[r * HC_N + c] + eps;
      }
    }
    int steps = 0;                                     // hist[steps] is the input of step `steps` (even: col, odd: row)
    {
      float cur[16];
      col_norm(hist[0], cur, eps);
      steps = 1;
      for (int it = 1; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 16; ++i) hist[steps][i] = cur[i];
        row_norm(hist[steps], cur, eps);
        ++steps;
#pragma unroll
        for (int i = 0; i < 16; ++i) hist[steps][i] = cur[i];
        col_norm(hist[steps], cur, eps);
        ++steps;
      }
    }
    float g[16], gn[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) g[i] = dcomb[t * 16 + i];
    for (int s = steps - 1; s >= 0; --s) {             // step s: even = column normalisation, odd = row normalisation
      if (s & 1) row_norm_bwd(hist[s], g, gn, eps);
      else col_norm_bwd(hist[s], g, gn, eps);
#pragma unroll
      for (int i = 0; i < 16; ++i) g[i] = gn[i];
    }
    // softmax rows: d logits = p * (g - sum(g * p))
#pragma unroll
    for (int r = 0; r < HC_N; ++r) {
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < HC_N; ++c) dot += g[r * HC_N + c] * p[r * HC_N + c];
#pragma unroll
      for (int c = 0; c < HC_N; ++c) dl[2 * HC_N + r * HC_N + c] = p[r * HC_N + c] * (g[r * HC_N + c] - dot);
    }
#pragma unroll
    for (int i = 0; i < HC_W; ++i) dmixes[t * HC_W + i] = dl[i] * scale[i < HC_N ? 0 : (i < 2 * HC_N ? 1 : 2)];
  } else {
#pragma unroll
    for (int i = 0; i < HC_W; ++i) mloc[i] = 0.f;
  }
  // d base[i] = sum_t dl[i];  d scale[k] = sum_t sum_{i in group k} dl[i] * m[i]
  float ds[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < HC_W; ++i) ds[i < HC_N ? 0 : (i < 2 * HC_N ? 1 : 2)] += dl[i] * mloc[i];
#pragma unroll
  for (int i = 0; i < HC_W; ++i) {
    float v = dl[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&red[i], v);
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    float v = ds[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&red[HC_W + k], v);
  }
  __syncthreads();
  if (threadIdx.x < HC_W) atomicAdd(dbase + threadIdx.x, red[threadIdx.x]);
  else if (threadIdx.x < HC_W + 3) atomicAdd(dscale + (threadIdx.x - HC_W), red[threadIdx.x]);
}

}  // namespace
}  // namespace nga

extern "C" int nga_hc_coeff_fwd(const float* mixes, const float* scale, const float* base, float* pre, float* post, float* comb,
                                long long T, int streams, int iters, float eps, void* stream) {
  using namespace nga;
  if (T <= 0 || streams != HC_N || iters < 1 || iters > HC_MAX_ITERS) return -1;
  hc_coeff_fwd_kernel<<<(unsigned)((T + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(mixes, scale, base, pre, post,
                                                                                                       comb, T, iters, eps);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

// dscale [3] and dbase [24] must be zeroed by the caller (they are accumulated with atomics).
extern "C" int nga_hc_coeff_bwd(const float* mixes, const float* scale, const float* base, const float* dpre, const float* dpost,
                                const float* dcomb, float* dmixes, float* dscale, float* dbase, long long T, int streams, int iters,
                                float eps, void* stream) {
  using namespace nga;
  if (T <= 0 || streams != HC_N || iters < 1 || iters > HC_MAX_ITERS) return -1;
  hc_coeff_bwd_kernel<<<(unsigned)((T + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      mixes, scale, base, dpre, dpost, dcomb, dmixes, dscale, dbase, T, iters, eps);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
