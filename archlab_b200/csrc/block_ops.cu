// Backward / fused forms of the small per-block operators of the PyTorch-level model families:
// RMSNorm backward (with gain gradient), SwiGLU forward and backward on a packed [gate | up] tensor,
// and cross-entropy over bf16 logits that writes the logit gradient in place.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"
#include "misc_kernels.h"

namespace nga {
namespace {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint32_t pk(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pk(f[0], f[1]);
  u.y = pk(f[2], f[3]);
  u.z = pk(f[4], f[5]);
  u.w = pk(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward.  y = x * rstd * w  (w = 1 + weight when zero-centred, 1 when there is no gain).
//   dx = rstd * (dy*w - xhat * mean(dy*w*xhat)),   dw[c] += sum_rows dy * xhat
// One warp per normalised slice (row x group); a lane owns columns lane*8 + 256*j.  Each warp walks
// slices with a grid stride and keeps its gain-gradient partials in registers; one atomicAdd per
// owned column at the end.  WIDTH / 256 register tiles, so WIDTH <= 256 * MAXT.
// ------------------------------------------------------------------------------------------------
template <int MAXT>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, long long slices, int groups, int width,
                   float eps, int zero_centered) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * 8;
  const int tiles = (width + 255) / 256;
  // all slices of one warp must share the group (so that dw partials stay per column): stride by a
  // multiple of `groups`
  const long long stride = nwarps / groups * groups;           // host guarantees nwarps >= groups
  if (warp0 >= stride) return;
  float acc[MAXT][8];
#pragma unroll
  for (int t = 0; t < MAXT; ++t)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[t][i] = 0.f;
  const int g = int(warp0 % groups);
  for (long long s = warp0; s < slices; s += stride) {
    const __nv_bfloat16* xr = x + s * width;
    const __nv_bfloat16* dr = dy + s * width;
    float xv[MAXT][8], gv[MAXT][8];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      const int c = t * 256 + lane * 8;
      if (t < tiles && c < width) {
        ld8(xr + c, xv[t]);
        ld8(dr + c, gv[t]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float wi = w ? (zero_centered ? 1.f + w[g * width + c + i] : w[g * width + c + i]) : 1.f;
          ss += xv[t][i] * xv[t][i];
          dot += gv[t][i] * wi * xv[t][i];
        }
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rstd = rsqrtf(ss / float(width) + eps);
    const float coef = dot * rstd * rstd / float(width);     // mean(dy*w*xhat) * rstd, in units of x
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      const int c = t * 256 + lane * 8;
      if (t < tiles && c < width) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float wi = w ? (zero_centered ? 1.f + w[g * width + c + i] : w[g * width + c + i]) : 1.f;
          o[i] = rstd * (gv[t][i] * wi - xv[t][i] * coef);
          acc[t][i] += gv[t][i] * xv[t][i] * rstd;
        }
        st8(dx + s * width + c, o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      const int c = t * 256 + lane * 8;
      if (t < tiles && c < width) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(dw + g * width + c + i, acc[t][i]);
      }
    }
  }
}

// Wide rows (width > 1024): one block of 256 threads per slice, a thread owns columns tid*8 + 2048*j.
template <int MAXT>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_wide_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, long long slices, int groups, int width,
                        float eps, int zero_centered) {
  __shared__ float red[2][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long stride = (long long)gridDim.x / groups * groups;   // host guarantees gridDim.x >= groups
  if (blockIdx.x >= stride) return;
  const int g = int(blockIdx.x % groups);
  float acc[MAXT][8];
#pragma unroll
  for (int t = 0; t < MAXT; ++t)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[t][i] = 0.f;
  for (long long s = blockIdx.x; s < slices; s += stride) {
    float xv[MAXT][8], gv[MAXT][8];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      const int c = t * 2048 + threadIdx.x * 8;
      if (c < width) {
        ld8(x + s * width + c, xv[t]);
        ld8(dy + s * width + c, gv[t]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float wi = w ? (zero_centered ? 1.f + w[g * width + c + i] : w[g * width + c + i]) : 1.f;
          ss += xv[t][i] * xv[t][i];
          dot += gv[t][i] * wi * xv[t][i];
        }
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    __syncthreads();                              // previous iteration's readers are done
    if (lane == 0) {
      red[0][warp] = ss;
      red[1][warp] = dot;
    }
    __syncthreads();
    ss = dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ss += red[0][i];
      dot += red[1][i];
    }
    const float rstd = rsqrtf(ss / float(width) + eps);
    const float coef = dot * rstd * rstd / float(width);
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      const int c = t * 2048 + threadIdx.x * 8;
      if (c < width) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float wi = w ? (zero_centered ? 1.f + w[g * width + c + i] : w[g * width + c + i]) : 1.f;
          o[i] = rstd * (gv[t][i] * wi - xv[t][i] * coef);
          acc[t][i] += gv[t][i] * xv[t][i] * rstd;
        }
        st8(dx + s * width + c, o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      const int c = t * 2048 + threadIdx.x * 8;
      if (c < width) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(dw + g * width + c + i, acc[t][i]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU on a packed [rows, 2*inter] tensor ([gate | up]); optional clamp (gate <= limit, |up| <= limit).
// ------------------------------------------------------------------------------------------------
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dh, long long rows, int inter, float limit) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= rows * inter) return;
  const long long m = i / inter;
  const int c = int(i - m * inter);
  float g[8], u[8], d[8], dg[8], du[8];
  ld8(h + m * 2 * inter + c, g);
  ld8(h + m * 2 * inter + inter + c, u);
  ld8(dout + m * inter + c, d);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float gk = g[k], uk = u[k];
    bool g_open = true, u_open = true;
    if (limit > 0.f) {
      g_open = gk <= limit;
      u_open = uk >= -limit && uk <= limit;
      gk = fminf(gk, limit);
      uk = fminf(fmaxf(uk, -limit), limit);
    }
    const float sg = 1.f / (1.f + __expf(-gk));
    const float silu = gk * sg;
    du[k] = u_open ? d[k] * silu : 0.f;
    dg[k] = g_open ? d[k] * uk * sg * (1.f + gk * (1.f - sg)) : 0.f;
  }
  st8(dh + m * 2 * inter + c, dg);
  st8(dh + m * 2 * inter + inter + c, du);
}

// ------------------------------------------------------------------------------------------------
// Cross-entropy of one row of bf16 logits per block; the logits are overwritten by
// gscale * (softmax - onehot) (zero for ignored rows).  Online max/sum, then the gradient pass.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
ce_inplace_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss_rows,
                  float gscale, long long ld, int V, long long ignore_index) {
  __shared__ float red_m[16], red_s[16];
  __shared__ float row_m, row_inv;
  const long long row = blockIdx.x;
  __nv_bfloat16* l = logits + row * ld;
  const long long tgt = targets[row];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float kLog2e = 1.4426950408889634f;
  float m = -INFINITY, s = 0.f;
  const int V8 = V & ~7;
  for (int c = threadIdx.x * 8; c < V8; c += 512 * 8) {
    float v[8];
    ld8(l + c, v);
    float mx = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, v[i]);
    if (mx > m) {
      s *= exp2f((m - mx) * kLog2e);
      m = mx;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += exp2f((v[i] - m) * kLog2e);
  }
  for (int c = V8 + threadIdx.x; c < V; c += 512) {
    const float v = __bfloat162float(l[c]);
    if (v > m) {
      s *= exp2f((m - v) * kLog2e);
      m = v;
    }
    s += exp2f((v - m) * kLog2e);
  }
  const float wm = warp_max(m);
  s *= (m == -INFINITY) ? 0.f : exp2f((m - wm) * kLog2e);
  s = warp_sum(s);
  if (lane == 0) {
    red_m[warp] = wm;
    red_s[warp] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = red_m[0];
    for (int i = 1; i < 16; ++i) bm = fmaxf(bm, red_m[i]);
    float bs = 0.f;
    for (int i = 0; i < 16; ++i) bs += red_s[i] * exp2f((red_m[i] - bm) * kLog2e);
    row_m = bm;
    row_inv = 1.f / bs;
    const bool live = tgt != ignore_index && tgt >= 0 && tgt < V;
    loss_rows[row] = live ? (logf(bs) + bm - __bfloat162float(l[tgt])) : 0.f;
  }
  __syncthreads();
  const float bm = row_m, inv = row_inv;
  const bool live = tgt != ignore_index && tgt >= 0 && tgt < V;
  const float gs = live ? gscale : 0.f;
  for (int c = threadIdx.x * 8; c < V8; c += 512 * 8) {
    float v[8];
    ld8(l + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = gs * (exp2f((v[i] - bm) * kLog2e) * inv - ((long long)(c + i) == tgt ? 1.f : 0.f));
    st8(l + c, v);
  }
  for (int c = V8 + threadIdx.x; c < V; c += 512) {
    const float v = __bfloat162float(l[c]);
    l[c] = __float2bfloat16(gs * (exp2f((v - bm) * kLog2e) * inv - ((long long)c == tgt ? 1.f : 0.f)));
  }
}

}  // namespace
}  // namespace nga

using namespace nga;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFW(p) reinterpret_cast<__nv_bfloat16*>(p)

extern "C" int nga_rmsnorm_bwd(const void* x, const float* weight, const void* dy, void* dx, float* dw, long long rows,
                               int groups, int width, float eps, int zero_centered, void* stream) {
  if (rows <= 0 || groups <= 0 || width <= 0 || (width & 7) || width > 8192) return -1;
  const long long slices = rows * groups;
  long long blocks = (slices + 7) / 8;
  const long long cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  if (blocks * 8 < groups) blocks = (groups + 7) / 8;
  if (width <= 256)
    rmsnorm_bwd_kernel<1><<<(unsigned)blocks, 256, 0, STREAM(stream)>>>(BF(x), weight, BF(dy), BFW(dx), dw, slices, groups,
                                                                        width, eps, zero_centered);
  else if (width <= 1024)
    rmsnorm_bwd_kernel<4><<<(unsigned)blocks, 256, 0, STREAM(stream)>>>(BF(x), weight, BF(dy), BFW(dx), dw, slices, groups,
                                                                        width, eps, zero_centered);
  else {
    long long wb = slices < 148 * 4 ? slices : 148 * 4;
    if (wb < groups) wb = groups;
    if (width <= 4096)
      rmsnorm_bwd_wide_kernel<2><<<(unsigned)wb, 256, 0, STREAM(stream)>>>(BF(x), weight, BF(dy), BFW(dx), dw, slices, groups,
                                                                          width, eps, zero_centered);
    else
      rmsnorm_bwd_wide_kernel<4><<<(unsigned)wb, 256, 0, STREAM(stream)>>>(BF(x), weight, BF(dy), BFW(dx), dw, slices, groups,
                                                                          width, eps, zero_centered);
  }
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_swiglu_bwd(const void* h, const void* dout, void* dh, long long rows, int inter, float limit,
                              void* stream) {
  if (rows <= 0 || inter <= 0 || (inter & 7)) return -1;
  const long long n = rows * inter / 8;
  swiglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>(BF(h), BF(dout), BFW(dh), rows, inter, limit);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_ce_inplace(void* logits, const long long* targets, float* loss_rows, float gscale, long long rows,
                              long long ld, int V, long long ignore_index, void* stream) {
  if (rows <= 0 || V <= 0 || (ld & 7)) return -1;
  ce_inplace_kernel<<<(unsigned)rows, 512, 0, STREAM(stream)>>>(BFW(logits), targets, loss_rows, gscale, ld, V, ignore_index);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
