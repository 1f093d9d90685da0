// Fused optimizer kernels: one pass per tensor instead of the ~15 elementwise passes of the
// reference's compiled step functions (src/archlab/optimizers/speedrun.py:31-72 AdamW, :147-231
// Muon).  The Newton-Schulz products themselves run on the tcgen05 GEMM (gemm.cu).
//
// All master weights, gradients and moments are fp32; every kernel that changes a weight also
// writes its bf16 shadow, so no separate cast pass is needed after the step.
#include "ptx.cuh"
#include "host_util.h"
#include "optim.h"

namespace nga {

// ------------------------------------------------------------------------------------------------
// AdamW: m, v lerp -> bias correction -> (cautious) decoupled weight decay -> update -> bf16 shadow
// ------------------------------------------------------------------------------------------------
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n,
                             float lr, float beta1, float beta2, float eps, float wd, float inv_bias1,
                             float inv_bias2, int cautious) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 pv = *reinterpret_cast<float4*>(p + i);
  const float4 gv = *reinterpret_cast<const float4*>(g + i);
  float4 mv = *reinterpret_cast<float4*>(m + i);
  float4 vv = *reinterpret_cast<float4*>(v + i);
  float* pp = reinterpret_cast<float*>(&pv);
  const float* gp = reinterpret_cast<const float*>(&gv);
  float* mp = reinterpret_cast<float*>(&mv);
  float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    mp[k] += (1.f - beta1) * (gp[k] - mp[k]);
    vp[k] += (1.f - beta2) * (gp[k] * gp[k] - vp[k]);
    const float upd = mp[k] / (sqrtf(vp[k] * inv_bias2) + eps);
    if (cautious) {
      if (upd * pp[k] >= 0.f) pp[k] -= lr * wd * pp[k];
    } else {
      pp[k] *= 1.f - lr * wd;
    }
    pp[k] -= lr * inv_bias1 * upd;
  }
  *reinterpret_cast<float4*>(p + i) = pv;
  *reinterpret_cast<float4*>(m + i) = mv;
  *reinterpret_cast<float4*>(v + i) = vv;
  if (shadow) {
    uint2 u;
    u.x = pack_bf16(pp[0], pp[1]);
    u.y = pack_bf16(pp[2], pp[3]);
    *reinterpret_cast<uint2*>(shadow + i) = u;
  }
}

// ------------------------------------------------------------------------------------------------
// Muon, step 1: Nesterov momentum in place and the squared Frobenius norm of each stacked matrix.
//   m = lerp(m, g, 1 - mu) ; g = lerp(g, m, mu) ; norm2[k] += sum g^2
// grid.y = matrix index k, grid.x covers `per` elements of that matrix.
// ------------------------------------------------------------------------------------------------
__global__ void muon_momentum_kernel(float* __restrict__ g, float* __restrict__ m,
                                     float* __restrict__ norm2, long long per, float mu) {
  __shared__ float red[8];
  const long long base = (long long)blockIdx.y * per;
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  float acc = 0.f;
  if (i < per) {
    float4 gv = *reinterpret_cast<float4*>(g + base + i);
    float4 mv = *reinterpret_cast<float4*>(m + base + i);
    float* gp = reinterpret_cast<float*>(&gv);
    float* mp = reinterpret_cast<float*>(&mv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mp[k] += (1.f - mu) * (gp[k] - mp[k]);
      gp[k] += mu * (mp[k] - gp[k]);
      acc += gp[k] * gp[k];
    }
    *reinterpret_cast<float4*>(g + base + i) = gv;
    *reinterpret_cast<float4*>(m + base + i) = mv;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    atomicAdd(norm2 + blockIdx.y, t);
  }
}

// Muon, step 2: X = bf16(g / (1.01 * ||g|| + 1e-6))
__global__ void muon_normalize_kernel(const float* __restrict__ g, const float* __restrict__ norm2,
                                      __nv_bfloat16* __restrict__ x, long long per) {
  const long long base = (long long)blockIdx.y * per;
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= per) return;
  const float s = 1.f / (sqrtf(norm2[blockIdx.y]) * 1.01f + 1e-6f);
  const float4 gv = *reinterpret_cast<const float4*>(g + base + i);
  uint2 u;
  u.x = pack_bf16(gv.x * s, gv.y * s);
  u.y = pack_bf16(gv.z * s, gv.w * s);
  *reinterpret_cast<uint2*>(x + base + i) = u;
}

// Mean of squares along rows (one warp per row): out[k, r] = mean_c x[k, r, c]^2
__global__ void rowsq_mean_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                                  long long rows, int n) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * n;
  float acc = 0.f;
  for (int c = lane * 2; c < n; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    acc += v.x * v.x + v.y * v.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] = acc / n;
}

// Mean of squares along columns: out[k, c] = mean_r x[k, r, c]^2.  grid.y = k; each thread owns two
// adjacent columns and walks the rows (coalesced across the warp).
__global__ void colsq_mean_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int m,
                                  int n) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= n) return;
  const __nv_bfloat16* xk = x + (long long)blockIdx.y * m * n;
  float a0 = 0.f, a1 = 0.f;
  for (int r = 0; r < m; ++r) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xk + (long long)r * n + c));
    a0 += v.x * v.x;
    a1 += v.y * v.y;
  }
  out[(long long)blockIdx.y * n + c] = a0 / m;
  out[(long long)blockIdx.y * n + c + 1] = a1 / m;
}

// Muon, final step: u = x * scale (per row or per column); cautious decay; p -= lr*u + lr*wd*p*[u*p>=0]
__global__ void muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ x,
                                  const float* __restrict__ scale, __nv_bfloat16* __restrict__ shadow,
                                  int m, int n, int per_row, float lr, float wd) {
  const long long per = (long long)m * n;
  const long long base = (long long)blockIdx.y * per;
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= per) return;
  const int r = int(i / n), c = int(i % n);
  float4 pv = *reinterpret_cast<float4*>(p + base + i);
  const uint2 xv = *reinterpret_cast<const uint2*>(x + base + i);
  const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.x));
  const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.y));
  const float xs[4] = {x01.x, x01.y, x23.x, x23.y};
  float* pp = reinterpret_cast<float*>(&pv);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float sc = per_row ? scale[(long long)blockIdx.y * m + r] : scale[(long long)blockIdx.y * n + c + k];
    // the reference rounds the scaled update to bf16 before applying it
    const float u = __bfloat162float(__float2bfloat16(xs[k] * sc));
    const float decay = (u * pp[k] >= 0.f) ? lr * wd * pp[k] : 0.f;
    pp[k] -= lr * u + decay;
  }
  *reinterpret_cast<float4*>(p + base + i) = pv;
  uint2 u2;
  u2.x = pack_bf16(pp[0], pp[1]);
  u2.y = pack_bf16(pp[2], pp[3]);
  *reinterpret_cast<uint2*>(shadow + base + i) = u2;
}

}  // namespace nga

using namespace nga;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int nga_adamw(float* p, const float* g, float* m, float* v, void* shadow, long long n, float lr,
                         float beta1, float beta2, float eps, float wd, int step, int cautious,
                         void* stream) {
  if (n <= 0 || (n % 4) || step < 1) return -1;
  const float inv_b1 = 1.f / (1.f - powf(beta1, (float)step));
  const float inv_b2 = 1.f / (1.f - powf(beta2, (float)step));
  adamw_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, ST(stream)>>>(
      p, g, m, v, reinterpret_cast<__nv_bfloat16*>(shadow), n, lr, beta1, beta2, eps, wd, inv_b1, inv_b2,
      cautious);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_muon_momentum(float* g, float* m, float* norm2, int K, long long per, float mu,
                                 void* stream) {
  if (K <= 0 || per <= 0 || (per % 4)) return -1;
  cudaMemsetAsync(norm2, 0, sizeof(float) * K, ST(stream));
  dim3 grid((unsigned)((per / 4 + 255) / 256), K);
  muon_momentum_kernel<<<grid, 256, 0, ST(stream)>>>(g, m, norm2, per, mu);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_muon_normalize(const float* g, const float* norm2, void* x, int K, long long per,
                                  void* stream) {
  if (K <= 0 || per <= 0 || (per % 4)) return -1;
  dim3 grid((unsigned)((per / 4 + 255) / 256), K);
  muon_normalize_kernel<<<grid, 256, 0, ST(stream)>>>(g, norm2, reinterpret_cast<__nv_bfloat16*>(x), per);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_sq_mean(const void* x, float* out, int K, int m, int n, int along_rows, void* stream) {
  if (K <= 0 || m <= 0 || n <= 0 || (n % 2)) return -1;
  if (along_rows) {
    const long long rows = (long long)K * m;
    rowsq_mean_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ST(stream)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), out, rows, n);
  } else {
    dim3 grid((unsigned)((n / 2 + 127) / 128), K);
    colsq_mean_kernel<<<grid, 128, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, m, n);
  }
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_muon_apply(float* p, const void* x, const float* scale, void* shadow, int K, int m, int n,
                              int per_row, float lr, float wd, void* stream) {
  if (K <= 0 || m <= 0 || n <= 0 || (n % 4)) return -1;
  const long long per = (long long)m * n;
  dim3 grid((unsigned)((per / 4 + 255) / 256), K);
  muon_apply_kernel<<<grid, 256, 0, ST(stream)>>>(p, reinterpret_cast<const __nv_bfloat16*>(x), scale,
                                                  reinterpret_cast<__nv_bfloat16*>(shadow), m, n, per_row,
                                                  lr, wd);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
