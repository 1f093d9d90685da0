// Expert-parallel MoE token exchange over NVLink peer memory, fused with the permutation.
//
//   push_rows  (dispatch): every (token, slot) row of this rank is written straight into the receive
//              buffer of the rank that owns its expert, at the row the routing prefix sums assigned
//              (all-to-all + permute in one pass; one warp per row, 16-byte lanes, full 128-byte lines
//              on the link).  Optional per-row scale (used by the backward of the combine).
//   pull_combine (combine): every token of this rank reads its k expert outputs back from the owners'
//              buffers and sums them, weighted, in the slot order given (ascending expert id, so the
//              fp32 sum is deterministic) - all-to-all + un-permute + weighted reduction in one pass.
//              Optionally also returns d(weight) = <grad_out, expert_row> for the backward pass.
// Both are the adjoint of each other, which is how the autograd wrappers use them.
// (Replaces the counts / tokens / weights all-to-all sequence of
// src/archlab/automodel/deepseek_v41_parallel.py:16-111 and DeepEP in the reference's stack.)
#include "ptx.cuh"
#include "host_util.h"
#include "moe.h"

namespace nga {

constexpr int kMoeMaxWorld = 16;
struct MoePeers {
  void* p[kMoeMaxWorld];
};

// rows: [n, C] bf16 local.  dst_rank / dst_row: [n] int32.  scale: optional [n] fp32.
__global__ void moe_push_rows_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ src_row,
                                     const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                                     const float* __restrict__ scale, MoePeers dst, int n, int C) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n) return;
  const int r = dst_rank[warp];
  if (r < 0) return;                                    // dropped slot
  const __nv_bfloat16* s = rows + (long long)(src_row ? src_row[warp] : warp) * C;
  __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst.p[r]) + (long long)dst_row[warp] * C;
  const float sc = scale ? scale[warp] : 1.f;
  for (int c = lane * 8; c < C; c += 256) {
    uint4 v = *reinterpret_cast<const uint4*>(s + c);
    if (scale) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        h[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
      }
    }
    *reinterpret_cast<uint4*>(d + c) = v;
  }
}

// out[t] = sum_j w[t, j] * peer[rank[t, j]][row[t, j]]   (j in the order given), fp32 accumulation.
// dweight[t, j] = <gout[t], peer row> when gout != nullptr.
__global__ void moe_pull_combine_kernel(MoePeers src, const int* __restrict__ rank, const int* __restrict__ row,
                                        const float* __restrict__ weight, const __nv_bfloat16* __restrict__ gout,
                                        __nv_bfloat16* __restrict__ out, float* __restrict__ out_f32,
                                        float* __restrict__ dweight, int T, int k, int C) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c0 = 0; c0 < C; c0 += 256) {
    const int c = c0 + lane * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float g[8];
    if (gout != nullptr && c < C) {
      const uint4 gv = *reinterpret_cast<const uint4*>(gout + (long long)t * C + c);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(gh[i]);
        g[2 * i] = f.x;
        g[2 * i + 1] = f.y;
      }
    }
    for (int j = 0; j < k; ++j) {
      const int r = rank[t * k + j];
      float dot = 0.f;
      if (r >= 0 && c < C) {
        const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[r]) +
                                                        (long long)row[t * k + j] * C + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float w = weight ? weight[t * k + j] : 1.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += w * f.x;
          acc[2 * i + 1] += w * f.y;
          if (gout != nullptr) dot += g[2 * i] * f.x + g[2 * i + 1] * f.y;
        }
      }
      if (dweight != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) {
          if (c0 == 0) dweight[t * k + j] = dot; else dweight[t * k + j] += dot;
        }
      }
    }
    if (c < C) {
      if (out != nullptr) {
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]);
        o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]);
        o.w = pack_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(out + (long long)t * C + c) = o;
      }
      if (out_f32 != nullptr) {
        float4* of = reinterpret_cast<float4*>(out_f32 + (long long)t * C + c);
        of[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        of[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  }
}

// SwiGLU with clamp: out[m, i] = silu(min(g, limit)) * clamp(u, -limit, limit) * (prob ? prob[m] : 1), h = [g | u].
__global__ void swiglu_clamped_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ prob,
                                      __nv_bfloat16* __restrict__ out, long long rows, int inter, float limit) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= rows * inter) return;
  const long long m = i / inter;
  const int c = int(i - m * inter);
  const uint4 gv = *reinterpret_cast<const uint4*>(h + m * 2 * inter + c);
  const uint4 uv = *reinterpret_cast<const uint4*>(h + m * 2 * inter + inter + c);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
  const float p = prob ? prob[m] : 1.f;
  float r[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 g = __bfloat1622float2(gh[q]), u = __bfloat1622float2(uh[q]);
    if (limit > 0.f) {
      g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
      u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
    }
    r[2 * q] = g.x / (1.f + __expf(-g.x)) * u.x * p;
    r[2 * q + 1] = g.y / (1.f + __expf(-g.y)) * u.y * p;
  }
  uint4 o;
  o.x = pack_bf16(r[0], r[1]);
  o.y = pack_bf16(r[2], r[3]);
  o.z = pack_bf16(r[4], r[5]);
  o.w = pack_bf16(r[6], r[7]);
  *reinterpret_cast<uint4*>(out + m * inter + c) = o;
}

static MoePeers moe_ptrs(const long long* host, int world) {
  MoePeers p;
  for (int i = 0; i < kMoeMaxWorld; ++i) p.p[i] = i < world ? reinterpret_cast<void*>(host[i]) : nullptr;
  return p;
}

}  // namespace nga

using namespace nga;

extern "C" int nga_moe_push_rows(const void* rows, const int* src_row, const int* dst_rank, const int* dst_row,
                                 const float* scale, const long long* dst_ptrs, int world, int n, int C, void* stream) {
  if (world < 1 || world > kMoeMaxWorld || n < 0 || C <= 0 || (C & 7)) return -1;
  if (n == 0) return 0;
  moe_push_rows_kernel<<<(n * 32 + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(rows), src_row, dst_rank, dst_row, scale, moe_ptrs(dst_ptrs, world), n, C);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_moe_pull_combine(const long long* src_ptrs, int world, const int* rank, const int* row,
                                    const float* weight, const void* gout, void* out, float* out_f32, float* dweight,
                                    int T, int k, int C, void* stream) {
  if (world < 1 || world > kMoeMaxWorld || T < 0 || k <= 0 || C <= 0 || (C & 7)) return -1;
  if (T == 0) return 0;
  moe_pull_combine_kernel<<<(T * 32 + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      moe_ptrs(src_ptrs, world), rank, row, weight, reinterpret_cast<const __nv_bfloat16*>(gout),
      reinterpret_cast<__nv_bfloat16*>(out), out_f32, dweight, T, k, C);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_swiglu_clamped(const void* h, const float* prob, void* out, long long rows, int inter, float limit,
                                  void* stream) {
  if (rows < 0 || inter <= 0 || (inter & 7)) return -1;
  if (rows == 0) return 0;
  const long long n8 = rows * inter / 8;
  swiglu_clamped_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(h), prob, reinterpret_cast<__nv_bfloat16*>(out), rows, inter, limit);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
