// Quantisers for the block-scaled GEMM operand format (see gemm_bs.h): bf16 -> fp8 + ue8m0 scales and
// bf16 -> e2m1 + ue4m3 scales, written straight in the 512-byte chunk layout the tensor core's scale copy
// expects.  Memory-bound elementwise kernels: every input byte is read once.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "gemm_bs.h"
#include "host_util.h"

namespace nga {

__device__ __forceinline__ long long sf_offset(long long r, long long sfi, long long chunks_k) {
  const long long tile = r >> 7, chunk = sfi >> 2;
  const int rr = int(r & 127);
  return (tile * chunks_k + chunk) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + int(sfi & 3);
}

// power-of-two scale: smallest 2^e with max(amax, 1e-4) / 2^e <= fmax (the floor keeps all-zero blocks at a
// finite scale, as the DeepSeek-V4.1 quantiser does); returns the biased ue8m0 byte and 2^-e
__device__ __forceinline__ uint8_t pow2_scale(float amax, float fmax, float& inv) {
  amax = fmaxf(amax, 1e-4f);
  int e = int(ceilf(log2f(amax / fmax)));
  // log2f may be off by an ulp at exact powers of two: make sure the block fits, and fits tightly
  if (ldexpf(fmax, e) < amax) ++e;
  else if (ldexpf(fmax, e - 1) >= amax) --e;
  e = max(-127, min(127, e));
  inv = ldexpf(1.f, -e);
  return uint8_t(e + 127);
}

// One warp per (row, 256-element span); a lane holds 8 consecutive elements (16-byte load, 8-byte store), so a
// 32-element scale block is 4 lanes and a 128-element one 16 lanes.
template <int BLOCK>
__global__ void quant_mxfp8_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                        long long rows, long long K, long long ldx, long long ldq, int e5m2) {
  const long long segs = (K + 127) / 128, spans = (K + 255) / 256;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= rows * spans) return;                                   // warp-uniform
  const int lane = threadIdx.x & 31;
  const long long r = w / spans, sp = w - r * spans;
  const long long k0 = sp * 256 + lane * 8;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  const __nv_bfloat16* src = x + r * ldx + k0;
  if (k0 + 8 <= K && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  } else {
    for (int i = 0; i < 8; ++i)
      if (k0 + i < K) v[i] = __bfloat162float(src[i]);
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 1; o < BLOCK / 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float inv;
  const uint8_t sb = pow2_scale(amax, e5m2 ? 57344.f : 448.f, inv);
  const __nv_fp8_interpretation_t kind = e5m2 ? __NV_E5M2 : __NV_E4M3;
  uint32_t pk[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h] * inv, v[4 * h + 1] * inv), __NV_SATFINITE, kind);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h + 2] * inv, v[4 * h + 3] * inv), __NV_SATFINITE, kind);
    pk[h] = lo | (hi << 16);
  }
  uint8_t* dst = q + r * ldq + k0;
  if (k0 + 8 <= K && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(pk[0], pk[1]);
  } else {
    for (int i = 0; i < 8; ++i)
      if (k0 + i < K) dst[i] = uint8_t(pk[i >> 2] >> (8 * (i & 3)));
  }
  if ((lane & 3) == 0 && k0 < segs * 128) sf[sf_offset(r, k0 >> 5, segs)] = sb;
}

// One CTA (256 threads) per 128 x 128 block: block maximum, one power-of-two scale for the whole block.
__global__ void quant_mxfp8_block128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                            long long rows, long long K, long long ldx, long long ldq, int e5m2) {
  __shared__ float red[8];
  const long long segs = (K + 127) / 128;
  const long long r0 = (long long)blockIdx.y * 128, k0 = (long long)blockIdx.x * 128;
  const int tr = threadIdx.x >> 3, tc = (threadIdx.x & 7) * 16;      // 32 rows x 8 column groups per pass
  float v[4][16];
  float amax = 0.f;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const long long r = r0 + pass * 32 + tr;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const long long k = k0 + tc + i;
      v[pass][i] = (r < rows && k < K) ? __bfloat162float(x[r * ldx + k]) : 0.f;
      amax = fmaxf(amax, fabsf(v[pass][i]));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  float inv;
  const uint8_t sb = pow2_scale(amax, e5m2 ? 57344.f : 448.f, inv);
  const __nv_fp8_interpretation_t kind = e5m2 ? __NV_E5M2 : __NV_E4M3;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const long long r = r0 + pass * 32 + tr;
    if (r >= rows) continue;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const long long k = k0 + tc + i;
      if (k < K) q[r * ldq + k] = uint8_t(__nv_cvt_float_to_fp8(v[pass][i] * inv, __NV_SATFINITE, kind));
    }
  }
  // the chunk of this (row tile, k segment): all 512 bytes carry the block's scale
  uint8_t* chunk = sf + ((long long)blockIdx.y * segs + blockIdx.x) * 512;
  const uint32_t rep = 0x01010101u * sb;
  if (threadIdx.x < 128) reinterpret_cast<uint32_t*>(chunk)[threadIdx.x] = rep;
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t a, uint32_t b) {
  uint32_t h = a * 0x9E3779B1u ^ (b + 0x7F4A7C15u + (a << 6) + (a >> 2));
  h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
  return h;
}

// Two scaled values -> one byte of e2m1 codes (first value in the low nibble), round to nearest even in hardware.
__device__ __forceinline__ uint32_t e2m1_pair(float a, float b) {
  return uint32_t(__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest)) & 0xFFu;
}
// Stochastic rounding onto the e2m1 grid {0, .5, 1, 1.5, 2, 3, 4, 6}: the grid step is .5 below 2, 1 below 4, 2
// above; floor(|a| / step + u) * step with u uniform in [0, 1) lands on a grid point and is unbiased.
__device__ __forceinline__ float e2m1_stochastic(float a, float u) {
  const float m = fminf(fabsf(a), 6.f);
  const float step = m < 2.f ? 0.5f : (m < 4.f ? 1.f : 2.f);
  const float qv = fminf(floorf(__fmaf_rn(m, 1.f / step, u)) * step, 6.f);
  return copysignf(qv, a);
}

// Thread = one 16-element block of one row.  Row mode: consecutive lanes take consecutive blocks of a row (coalesced).
// 16 x 16 mode: the 16 lanes of a half-warp hold 16 consecutive rows of one block column and share their maximum
// through shuffles.
template <int TWO_D>
__global__ void quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                   const float* __restrict__ amax_ptr, long long rows, long long K, long long ldx,
                                   long long ldq, uint32_t hseed, uint32_t sr_seed) {
  const long long nblk = (K + 15) / 16;
  const long long chunks_k = ((K + 255) / 256) * 4;      // whole k-blocks of four chunks, as the GEMM loads them
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long r, kb;
  bool live;
  if (TWO_D) {
    const long long rgroups = (rows + 15) / 16;
    long long grp = t >> 4;
    // threads past the end stay for the warp shuffles below (full mask) and store nothing
    const bool in_range = grp < rgroups * nblk;
    if (!in_range) grp = rgroups * nblk - 1;
    const long long rg = grp / nblk;
    kb = grp - rg * nblk;
    r = rg * 16 + (t & 15);
    live = in_range && r < rows;
  } else {
    r = t / nblk;
    kb = t - r * nblk;
    live = r < rows;
    if (!live) return;
  }
  const long long k0 = kb * 16;
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = 0.f;
  if (live) {
    const __nv_bfloat16* src = x + r * ldx + k0;
    if (k0 + 16 <= K && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(src)), b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(ha[i]), fb = __bfloat1622float2(hb[i]);
        v[2 * i] = fa.x; v[2 * i + 1] = fa.y; v[8 + 2 * i] = fb.x; v[8 + 2 * i + 1] = fb.y;
      }
    } else {
      for (int i = 0; i < 16; ++i)
        if (k0 + i < K) v[i] = __bfloat162float(src[i]);
    }
  }
  if (hseed != 0u) {
    // y = H (d * v) / 4 with d a fixed random sign vector: orthogonal, so applying it to both operands of a
    // product over K leaves the product unchanged while spreading outliers over the block
    const uint32_t signs = hash_u32(hseed, 0x5EEDu);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (signs >> i) & 1u ? -v[i] : v[i];
#pragma unroll
    for (int s = 1; s < 16; s <<= 1)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if ((i & s) == 0) {
          const float a = v[i], b = v[i | s];
          v[i] = a + b;
          v[i | s] = a - b;
        }
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= 0.25f;
  }
  float bmax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
  if (TWO_D) {
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
  }
  const float tmax = *amax_ptr;
  const float s_enc = tmax > 0.f ? 2688.f / tmax : 1.f;               // 448 * 6 / amax
  // block decode scale in e4m3 (round to nearest, saturating), then the encode factor that matches it exactly
  const __nv_fp8_storage_t sbyte = __nv_cvt_float_to_fp8(bmax / 6.f * s_enc, __NV_SATFINITE, __NV_E4M3);
  const float sdec = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbyte, __NV_E4M3)));
  const float enc = sdec > 0.f ? s_enc / sdec : 0.f;
  if (!live) return;
  uint32_t words[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    float a = __fmul_rn(v[i], enc), b = __fmul_rn(v[i + 1], enc);
    if (sr_seed != 0u) {
      const uint32_t h = hash_u32(sr_seed, uint32_t(r * K + k0 + i));
      a = e2m1_stochastic(a, float(h >> 16) * (1.f / 65536.f));
      b = e2m1_stochastic(b, float(h & 0xFFFFu) * (1.f / 65536.f));
    }
    words[i >> 3] |= e2m1_pair(a, b) << (4 * (i & 7));
  }
  uint8_t* dst = q + r * ldq + k0 / 2;
  if (k0 + 16 <= K && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(words[0], words[1]);
  } else {
    for (int i = 0; i < 16 && k0 + i < K; i += 2) dst[i / 2] = uint8_t((words[i >> 3] >> (4 * (i & 7))) & 0xFFu);
  }
  sf[sf_offset(r, kb, chunks_k)] = sbyte;
}

}  // namespace nga

extern "C" long long nga_sf_bytes(int kind, long long rows, long long K) {
  const long long per_chunk = kind == 1 ? 128 : 64;
  const long long kblock = kind == 1 ? 128 : 256;               // the GEMM loads whole k-blocks of chunks
  const long long chunks_k = ((K + kblock - 1) / kblock) * (kblock / per_chunk);
  return ((rows + 127) / 128) * chunks_k * 512;
}

extern "C" int nga_quant_mxfp8(const void* x, void* q, void* sf, long long rows, long long K, long long ldx, long long ldq_bytes,
                               int block, int e5m2, void* stream) {
  using namespace nga;
  if (rows <= 0 || K <= 0 || x == nullptr || q == nullptr || sf == nullptr) return -1;
  if (ldx < K || ldq_bytes < K) return -5;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long segs = (K + 127) / 128;
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto qb = reinterpret_cast<uint8_t*>(q);
  auto sb = reinterpret_cast<uint8_t*>(sf);
  if (block == -128) {
    dim3 grid((unsigned)segs, (unsigned)((rows + 127) / 128));
    quant_mxfp8_block128_kernel<<<grid, 256, 0, st>>>(xb, qb, sb, rows, K, ldx, ldq_bytes, e5m2);
  } else if (block == 32 || block == 128) {
    const long long warps = rows * ((K + 255) / 256);
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    if (block == 32) quant_mxfp8_rows_kernel<32><<<blocks, 256, 0, st>>>(xb, qb, sb, rows, K, ldx, ldq_bytes, e5m2);
    else quant_mxfp8_rows_kernel<128><<<blocks, 256, 0, st>>>(xb, qb, sb, rows, K, ldx, ldq_bytes, e5m2);
  } else {
    return -2;
  }
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_quant_nvfp4(const void* x, void* q, void* sf, const float* amax, long long rows, long long K, long long ldx,
                               long long ldq_bytes, int two_d, unsigned hadamard_seed, unsigned sr_seed, void* stream) {
  using namespace nga;
  if (rows <= 0 || K <= 0 || x == nullptr || q == nullptr || sf == nullptr || amax == nullptr) return -1;
  if ((K & 1) || ldx < K || ldq_bytes * 2 < K) return -5;
  if (two_d && (rows & 15)) return -2;
  const long long nblk = (K + 15) / 16, rgroups = (rows + 15) / 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto qb = reinterpret_cast<uint8_t*>(q);
  auto sb = reinterpret_cast<uint8_t*>(sf);
  if (two_d) {
    const long long threads = rgroups * nblk * 16;
    quant_nvfp4_kernel<1><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(xb, qb, sb, amax, rows, K, ldx, ldq_bytes,
                                                                             hadamard_seed, sr_seed);
  } else {
    const long long threads = rows * nblk;
    quant_nvfp4_kernel<0><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(xb, qb, sb, amax, rows, K, ldx, ldq_bytes,
                                                                             hadamard_seed, sr_seed);
  }
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

// Row gather with de-quantisation for frozen fp8 tables with one ue8m0 scale per 32 columns (row-sharded Engram
// memories): out[i, :] = e4m3(weight[idx[i], :]) * 2^(scale[idx[i], c / 32] - 127) in bf16.  One warp per output row;
// a lane converts 8 columns per step (8-byte load, 16-byte store).
namespace nga {
__global__ void gather_dequant_fp8_kernel(const uint8_t* __restrict__ weight, const uint8_t* __restrict__ scale,
                                          const long long* __restrict__ idx, __nv_bfloat16* __restrict__ out, long long n,
                                          long long rows, int dim) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n) return;
  const int lane = threadIdx.x & 31;
  long long r = idx[w];
  r = r < 0 ? 0 : (r >= rows ? rows - 1 : r);             // ids are validated on the host; never read outside the shard
  const uint8_t* src = weight + r * dim;
  const uint8_t* sc = scale + r * (dim / 32);
  for (int c = lane * 8; c < dim; c += 256) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + c);
    const float s = ldexpf(1.f, int(sc[c >> 5]) - 127);
    const uint32_t words[2] = {raw.x, raw.y};
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const __half2_raw pr = __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t((words[h] >> (16 * j)) & 0xFFFFu), __NV_E4M3);
        const float2 f = __half22float2(__half2(pr));
        const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * s, f.y * s);
        o[h * 2 + j] = *reinterpret_cast<const uint32_t*>(&b);
      }
    *reinterpret_cast<uint4*>(out + w * dim + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}
}  // namespace nga

extern "C" int nga_gather_dequant_fp8(const void* weight, const void* scale, const void* idx, void* out, long long n,
                                      long long rows, int dim, void* stream) {
  using namespace nga;
  if (n <= 0 || rows <= 0 || dim <= 0 || (dim % 32)) return -1;
  if ((reinterpret_cast<uintptr_t>(weight) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return -5;
  gather_dequant_fp8_kernel<<<(unsigned)((n + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(weight), reinterpret_cast<const uint8_t*>(scale), reinterpret_cast<const long long*>(idx),
      reinterpret_cast<__nv_bfloat16*>(out), n, rows, dim);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
