// Memory-bound building blocks of the model zoo as single-pass sm_100a kernels (fp32 statistics, bf16 or
// fp32 I/O, 16-byte vector accesses): RMSNorm (plain / zero-centred / per-stream groups), rotary
// embedding (half-split or interleaved, partial), router scoring + top-k, causal depthwise conv + SiLU,
// hashed n-gram ids, block FP8 (1 x 128, power-of-two scales) and NVFP4 quantisers, stochastic bf16.
#include "ptx.cuh"
#include "host_util.h"
#include "misc_kernels.h"
#include <cuda_fp8.h>

namespace nga {

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

// ---------------------------------------------------------------------------------------------- RMSNorm
// One warp per (row, group).  x, y: [rows, groups * width] bf16; weight: [groups * width] fp32 or null.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ weight,
                               __nv_bfloat16* __restrict__ y, long long rows, int groups, int width, float eps,
                               int zero_centered) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= rows * groups) return;
  const long long row = w / groups;
  const int g = int(w - row * groups);
  const __nv_bfloat16* xr = x + (row * groups + g) * (long long)width;
  __nv_bfloat16* yr = y + (row * groups + g) * (long long)width;
  float ss = 0.f;
  for (int c = lane * 8; c < width; c += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  const float inv = rsqrtf(warp_sum(ss) / width + eps);
  for (int c = lane * 8; c < width; c += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x * inv;
      o[2 * i + 1] = f.y * inv;
    }
    if (weight != nullptr) {
      const float* wr = weight + (long long)g * width + c;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] *= zero_centered ? (1.f + wr[i]) : wr[i];
    }
    uint4 u;
    u.x = pack_bf16(o[0], o[1]);
    u.y = pack_bf16(o[2], o[3]);
    u.z = pack_bf16(o[4], o[5]);
    u.w = pack_bf16(o[6], o[7]);
    *reinterpret_cast<uint4*>(yr + c) = u;
  }
}

// ---------------------------------------------------------------------------------------------- RoPE
// x: [B*T, H, D] bf16 in place; cos/sin: [T, rot/2] fp32; one thread per rotated pair.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            long long rows, int T, int H, int D, int rot, int interleaved) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int half = rot / 2;
  if (i >= rows * H * half) return;
  const int p = int(i % half);
  const long long rh = i / half;
  const long long row = rh / H;
  const int t = int(row % T);
  __nv_bfloat16* v = x + rh * D;
  const int ia = interleaved ? 2 * p : p, ib = interleaved ? 2 * p + 1 : p + half;
  const float a = __bfloat162float(v[ia]), b = __bfloat162float(v[ib]);
  const float c = cs[(long long)t * half + p], s = sn[(long long)t * half + p];
  v[ia] = __float2bfloat16(a * c - b * s);
  v[ib] = __float2bfloat16(a * s + b * c);
}

// ---------------------------------------------------------------------------------------------- router
// One warp per token.  logits = x . W^T (E <= 512, computed here in fp32), score in {softmax 0, sigmoid 1,
// sqrt-softplus 2}, selection on score + bias, top-k by repeated warp arg-max (ties to the lower index),
// weights = scores of the selected experts, renormalised, times route_scale.
__global__ void router_topk_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   const float* __restrict__ bias, float* __restrict__ out_w, int* __restrict__ out_idx,
                                   float* __restrict__ out_scores, int T, int C, int E, int k, int score_fn,
                                   float route_scale, int renorm) {
  extern __shared__ float sh[];                          // [warps per block][E]
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp_in_block;
  if (t >= T) return;
  float* sc = sh + warp_in_block * E;
  const __nv_bfloat16* xr = x + (long long)t * C;
  for (int e = 0; e < E; ++e) {
    const __nv_bfloat16* wr = w + (long long)e * C;
    float acc = 0.f;
    for (int c = lane * 8; c < C; c += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(xr + c);
      const uint4 b = *reinterpret_cast<const uint4*>(wr + c);
      const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(ah[i]), g = __bfloat1622float2(bh[i]);
        acc += f.x * g.x + f.y * g.y;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) sc[e] = acc;
  }
  __syncwarp();
  if (score_fn == 0) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
    m = warp_max(m);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) s += __expf(sc[e] - m);
    s = warp_sum(s);
    for (int e = lane; e < E; e += 32) sc[e] = __expf(sc[e] - m) / s;
  } else {
    for (int e = lane; e < E; e += 32) {
      const float z = sc[e];
      sc[e] = (score_fn == 1) ? 1.f / (1.f + __expf(-z)) : sqrtf(z > 20.f ? z : log1pf(__expf(z)));
    }
  }
  __syncwarp();
  if (out_scores != nullptr)
    for (int e = lane; e < E; e += 32) out_scores[(long long)t * E + e] = sc[e];
  float total = 0.f;
  unsigned long long taken_lo = 0ull;                     // per-lane bitmap over the lane's experts (E <= 512 -> 16 each)
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane, q = 0; e < E; e += 32, ++q) {
      if (taken_lo >> q & 1ull) continue;
      const float v = sc[e] + (bias ? bias[e] : 0.f);
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((bi & 31) == lane) taken_lo |= 1ull << (bi >> 5);
    if (lane == 0) {
      out_idx[t * k + j] = bi;
      out_w[t * k + j] = sc[bi];
    }
    total += sc[bi];
  }
  __syncwarp();
  if (lane < k) {
    float v = out_w[t * k + lane];
    if (renorm && k > 1) v = v / (total + 1e-20f);
    out_w[t * k + lane] = v * route_scale;
  }
}

// ---------------------------------------------------------------------------------------------- conv
// y[b, t, c] = act(sum_j w[c, j] * x[b, t - (K-1-j) * dil, c] + bias[c]); x, y: [B, T, Cc] bf16; w: [Cc, K] fp32.
__global__ void causal_conv1d_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                     const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int B, int T, int Cc,
                                     int K, int dil, int silu) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * T * Cc) return;
  const int c = int(i % Cc);
  const long long bt = i / Cc;
  const int t = int(bt % T);
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int ts = t - (K - 1 - j) * dil;
    if (ts >= 0) acc += w[c * K + j] * __bfloat162float(x[i - (long long)(t - ts) * Cc]);
  }
  if (silu) acc = acc / (1.f + __expf(-acc));
  y[i] = __float2bfloat16(acc);
}

// ---------------------------------------------------------------------------------------------- hashing
// ids[b, t, h] for n-gram heads: for order o in 2..n and head j: (xor_{p<o} tok[t-p] * mult[p]) mod size[h] + offset[h];
// tok[t-p] is the EOS id when t-p falls before the start of the EOS-delimited segment of t (seg_start[b, t]).
__global__ void ngram_hash_kernel(const long long* __restrict__ tok, const int* __restrict__ seg_start,
                                  const long long* __restrict__ mult, const long long* __restrict__ sizes,
                                  const long long* __restrict__ offsets, long long* __restrict__ ids, int B, int T, int n,
                                  int heads_per_order, long long eos) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * T) return;
  const int t = int(i % T);
  const int s0 = seg_start[i];
  const int H = (n - 1) * heads_per_order;
  long long mixed = tok[i] * mult[0];
  for (int order = 2; order <= n; ++order) {
    const int p = order - 1;
    const long long tk = (t - p >= s0) ? tok[i - p] : eos;
    mixed ^= tk * mult[p];
    for (int j = 0; j < heads_per_order; ++j) {
      const int h = (order - 2) * heads_per_order + j;
      long long r = mixed % sizes[h];
      if (r < 0) r += sizes[h];
      ids[i * H + h] = r + offsets[h];
    }
  }
}

// ---------------------------------------------------------------------------------------------- quantisers
// FP8 e4m3 with one power-of-two scale per 128 (or 32) consecutive elements; one warp per block.
__global__ void fp8_block_quant_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_storage_t* __restrict__ q,
                                       float* __restrict__ scales, long long nblocks, int block, int pow2) {
  const long long b = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  const __nv_bfloat16* xb = x + b * block;
  const int per = block / 32;                              // 4 for 128, 1 for 32
  float v[4];
  float amax = 0.f;
  for (int i = 0; i < per; ++i) {
    v[i] = __bfloat162float(xb[lane * per + i]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  float s = fmaxf(amax, 1e-4f) * (1.f / 448.f);
  if (pow2) {
    const unsigned bits = __float_as_uint(s);
    const unsigned ex = ((bits >> 23) & 255u) + ((bits & 0x7fffffu) != 0u);
    s = __uint_as_float(ex << 23);
  }
  if (lane == 0) scales[b] = s;
  for (int i = 0; i < per; ++i) {
    const float z = fminf(fmaxf(v[i] / s, -448.f), 448.f);
    q[b * block + lane * per + i] = __nv_cvt_float_to_fp8(z, __NV_SATFINITE, __NV_E4M3);
  }
}

__device__ __forceinline__ float e2m1_rne(float a) {       // |value| <= 6 onto {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to even code
  if (a < 0.25f) return 0.f;
  if (a == 0.25f) return 0.f;
  if (a < 0.75f) return 0.5f;
  if (a == 0.75f) return 1.f;
  if (a < 1.25f) return 1.f;
  if (a == 1.25f) return 1.f;
  if (a < 1.75f) return 1.5f;
  if (a == 1.75f) return 2.f;
  if (a < 2.5f) return 2.f;
  if (a == 2.5f) return 2.f;
  if (a < 3.5f) return 3.f;
  if (a == 3.5f) return 4.f;
  if (a < 5.f) return 4.f;
  if (a == 5.f) return 4.f;
  return 6.f;
}

// NVFP4: 16-element blocks, e4m3 block scale, fp32 tensor scale (given); values returned dequantisable on
// the e2m1 grid (as bf16) plus the e4m3 block scales.  One thread per block.
__global__ void nvfp4_quant_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ vals,
                                   __nv_fp8_storage_t* __restrict__ bscale, float tensor_scale, long long nblocks) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  float v[16];
  float amax = 0.f;
  for (int i = 0; i < 16; ++i) {
    v[i] = __bfloat162float(x[b * 16 + i]) / tensor_scale;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  const __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(fmaxf(amax / 6.f, 0.001953125f), __NV_SATFINITE, __NV_E4M3);
  bscale[b] = s8;
  const float s = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3)));
  for (int i = 0; i < 16; ++i) {
    const float z = fminf(fabsf(v[i] / s), 6.f);
    vals[b * 16 + i] = __float2bfloat16(copysignf(e2m1_rne(z), v[i]));
  }
}

// Unbiased fp32 -> bf16: add 16 uniform random bits below the kept mantissa, truncate.  Counter-based RNG.
__global__ void stochastic_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                                       unsigned long long seed) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(i + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  const unsigned bits = __float_as_uint(x[i]) + unsigned(z & 0xffffu);
  y[i] = __ushort_as_bfloat16((unsigned short)(bits >> 16));
}

}  // namespace nga

using namespace nga;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int nga_rmsnorm(const void* x, const float* weight, void* y, long long rows, int groups, int width, float eps,
                           int zero_centered, void* stream) {
  if (rows <= 0 || groups <= 0 || width <= 0 || (width & 7)) return -1;
  const long long warps = rows * groups;
  rmsnorm_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), weight, reinterpret_cast<__nv_bfloat16*>(y), rows, groups, width, eps,
      zero_centered);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_rope(void* x, const float* cos_t, const float* sin_t, long long rows, int T, int H, int D, int rot,
                        int interleaved, void* stream) {
  if (rows <= 0 || T <= 0 || H <= 0 || D <= 0 || rot <= 0 || rot > D || (rot & 1)) return -1;
  const long long n = rows * H * (rot / 2);
  rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>(reinterpret_cast<__nv_bfloat16*>(x), cos_t, sin_t, rows,
                                                                      T, H, D, rot, interleaved);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_router_topk(const void* x, const void* w, const float* bias, float* out_w, int* out_idx,
                               float* out_scores, int T, int C, int E, int k, int score_fn, float route_scale, int renorm,
                               void* stream) {
  if (T <= 0 || C <= 0 || (C & 7) || E <= 0 || E > 512 || k <= 0 || k > 32 || k > E || score_fn < 0 || score_fn > 2) return -1;
  const int warps = 4;
  router_topk_kernel<<<(T + warps - 1) / warps, warps * 32, warps * E * sizeof(float), STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w), bias, out_w, out_idx, out_scores,
      T, C, E, k, score_fn, route_scale, renorm);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_causal_conv1d(const void* x, const float* w, const float* bias, void* y, int B, int T, int Cc, int K,
                                 int dil, int silu, void* stream) {
  if (B <= 0 || T <= 0 || Cc <= 0 || K <= 0 || dil <= 0) return -1;
  const long long n = (long long)B * T * Cc;
  causal_conv1d_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), w, bias, reinterpret_cast<__nv_bfloat16*>(y), B, T, Cc, K, dil, silu);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_ngram_hash(const long long* tok, const int* seg_start, const long long* mult, const long long* sizes,
                              const long long* offsets, long long* ids, int B, int T, int n, int heads_per_order,
                              long long eos, void* stream) {
  if (B <= 0 || T <= 0 || n < 2 || heads_per_order <= 0) return -1;
  const long long m = (long long)B * T;
  ngram_hash_kernel<<<(unsigned)((m + 255) / 256), 256, 0, STREAM(stream)>>>(tok, seg_start, mult, sizes, offsets, ids, B, T, n,
                                                                            heads_per_order, eos);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_fp8_block_quant(const void* x, void* q, float* scales, long long n, int block, int pow2, void* stream) {
  if (n <= 0 || (block != 128 && block != 32) || n % block) return -1;
  const long long nb = n / block;
  fp8_block_quant_kernel<<<(unsigned)((nb * 32 + 255) / 256), 256, 0, STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_fp8_storage_t*>(q), scales, nb, block, pow2);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_nvfp4_quant(const void* x, void* vals, void* bscale, float tensor_scale, long long n, void* stream) {
  if (n <= 0 || n % 16 || !(tensor_scale > 0.f)) return -1;
  const long long nb = n / 16;
  nvfp4_quant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(vals),
      reinterpret_cast<__nv_fp8_storage_t*>(bscale), tensor_scale, nb);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_stochastic_bf16(const float* x, void* y, long long n, unsigned long long seed, void* stream) {
  if (n <= 0) return -1;
  stochastic_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>(x, reinterpret_cast<__nv_bfloat16*>(y), n, seed);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
