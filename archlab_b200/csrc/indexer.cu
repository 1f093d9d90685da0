// Lightning-indexer key selection: for every query row, scores s[j] = scale * sum_h w[h] * relu(q[h] . k[j]) over the
// causal keys j <= i, the top-k threshold by radix select in shared memory, and one bit per key (bit j % 32 of word
// j / 32) for the keys whose score reaches the threshold.  Replaces materialising the [S, S] fp32 score matrix, a
// full-row sort and an index scatter per layer.  Rows with at most k candidates select all of them.
// One CTA per (batch, query row); scores live in shared memory (S <= 8192).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"
#include "misc_kernels.h"

namespace nga {
namespace {

constexpr int IX_THREADS = 256;
constexpr int IX_MAX_S = 8192;

__device__ __forceinline__ uint32_t sortable(float f) {          // monotone map float -> uint32
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <int HI, int DI>
__global__ void __launch_bounds__(IX_THREADS, 4)
indexer_select_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const float* __restrict__ w,
                      uint32_t* __restrict__ bits, int S, int top_k, float scale) {
  extern __shared__ uint32_t sh[];
  uint32_t* key = sh;                                   // [S] sortable scores of the causal keys
  __shared__ float sq[HI * DI];
  __shared__ float sw[HI];
  __shared__ unsigned int hist[256];
  __shared__ uint32_t sel_prefix, sel_remaining;
  const int i = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int n = i + 1;                                  // causal candidates
  const long long row = (long long)b * S + i;
  for (int x = tid; x < HI * DI; x += IX_THREADS) sq[x] = __bfloat162float(q[row * HI * DI + x]);
  if (tid < HI) sw[tid] = w[row * HI + tid] * scale;
  __syncthreads();
  const __nv_bfloat16* kb = k + (long long)b * S * DI;
  for (int j = tid; j < n; j += IX_THREADS) {
    float dot[HI];
#pragma unroll
    for (int h = 0; h < HI; ++h) dot[h] = 0.f;
    const uint4* kr = reinterpret_cast<const uint4*>(kb + (long long)j * DI);
#pragma unroll 2
    for (int c = 0; c < DI / 8; ++c) {
      const uint4 u = kr[c];
      const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 kv = __bfloat1622float2(hp[e]);
#pragma unroll
        for (int h = 0; h < HI; ++h) dot[h] = fmaf(sq[h * DI + c * 8 + 2 * e], kv.x, fmaf(sq[h * DI + c * 8 + 2 * e + 1], kv.y, dot[h]));
      }
    }
    float s = 0.f;
#pragma unroll
    for (int h = 0; h < HI; ++h) s = fmaf(sw[h], fmaxf(dot[h], 0.f), s);
    key[j] = sortable(s);
  }
  __syncthreads();
  uint32_t thr = 0u;                                    // select everything unless more than top_k candidates
  if (n > top_k) {
    // radix select of the top_k-th largest key: 4 passes of 8 bits from the top
    if (tid == 0) { sel_prefix = 0u; sel_remaining = (uint32_t)top_k; }
    uint32_t mask = 0u;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      hist[tid] = 0u;                                   // IX_THREADS == 256 bins
      __syncthreads();
      const uint32_t prefix = sel_prefix;
      for (int j = tid; j < n; j += IX_THREADS) {
        const uint32_t v = key[j];
        if ((v & mask) == prefix) atomicAdd(&hist[(v >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        uint32_t need = sel_remaining, bin = 255u;
        for (int x = 255; x >= 0; --x) {                // walk bins from the largest digit
          if (hist[x] >= need) { bin = (uint32_t)x; break; }
          need -= hist[x];
        }
        sel_prefix = prefix | (bin << shift);
        sel_remaining = need;
      }
      mask |= 255u << shift;
      __syncthreads();
    }
    thr = sel_prefix;
  }
  // one word per 32 keys
  const int words = S >> 5;
  uint32_t* out = bits + row * words;
  const int lane = tid & 31, warp = tid >> 5;
  for (int wd = warp; wd < words; wd += IX_THREADS / 32) {
    const int j = wd * 32 + lane;
    const bool on = j < n && key[j < n ? j : 0] >= thr;
    const uint32_t word = __ballot_sync(0xffffffffu, on);
    if (lane == 0) out[wd] = word;
  }
}

}  // namespace
}  // namespace nga

// q [B, S, 4, 64] bf16, k [B, S, 64] bf16, w [B, S, 4] fp32 -> bits [B, S, S / 32] (S a multiple of 32, <= 8192).
extern "C" int nga_indexer_select(const void* q, const void* k, const float* w, void* bits, int B, int S, int heads, int dim,
                                  int top_k, float scale, void* stream) {
  using namespace nga;
  if (B <= 0 || S <= 0 || (S & 31) || S > IX_MAX_S || top_k <= 0) return -1;
  if (heads != 4 || dim != 64) return -2;
  indexer_select_kernel<4, 64><<<dim3(S, B), IX_THREADS, S * sizeof(uint32_t), reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k), w, reinterpret_cast<uint32_t*>(bits), S,
      top_k, scale);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
