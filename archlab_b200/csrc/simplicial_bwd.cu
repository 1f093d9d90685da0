// 2-simplicial (trilinear) windowed attention, backward, on tcgen05 + TMEM.  head_dim 128,
// w1 in {8, 16, 32}.  With rows r = (query i, short key j), A_r = q_i * k1_j, G_r = dO_i * v1_j:
//     S  = A K2^T                 P  = exp2(S * scale*log2e - lse2[i])          (joint softmax)
//     dP = G V2^T                 dS = P * (dP - delta[i]) * scale,   delta[i] = dO_i . O_i
//     dA = dS K2   -> dq_i = sum_j dA_(i,j) * k1_j ,  dk1_j += sum_i dA_(i,j) * q_i
//     Op = P  V2   -> dv1_j += sum_i Op_(i,j) * dO_i
//     dK2 = dS^T A ,  dV2 = P^T G
// (oracle: autograd through src/archlab/architectures/simplicial_attention.py:49-74; incumbents:
// Triton simplicial_kernels.py:56-177, TileLang tilelang_attention.py:143-378.)
//
// Two kernels, each keeping its accumulators in TMEM for the CTA lifetime:
//   * query-owned (this file, part 1): CTA = 128 rows (128 / w1 queries), walks 64-key tiles of the
//     long window; dA and Op accumulate in TMEM; dq is written directly, dk1 / dv1 are added to fp32
//     buffers with vector atomics (rows of neighbouring CTAs and of the query heads of a KV group
//     overlap).
//   * key-owned (part 2): CTA = 128 long keys, walks the 64-row groups that can see them in the
//     transposed frame (thread = key); dK2 / dV2 accumulate in TMEM and are added once per CTA.
#include "ptx.cuh"
#include "host_util.h"
#include "simplicial.h"
#include <cuda.h>

namespace nga {

constexpr int SB_D = 128;
constexpr int SB_BK = 64;            // long keys per tile (query-owned kernel)
constexpr int SB_THREADS = 192;

struct SimpBwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k1;
  const __nv_bfloat16* v1;
  const __nv_bfloat16* dout;   // [B*N, lddo]
  const float* lse2;           // [B, Hq, N]
  const float* delta;          // [B, Hq, N]
  __nv_bfloat16* dq;           // [B*N, lddq]
  float* dk1;                  // [B*N, Hkv*D] fp32, zeroed by the launcher
  float* dv1;                  // [B*N, Hkv*D] fp32, zeroed by the launcher
  float* dk2;                  // [B*N, Hkv*D] fp32, zeroed by the launcher
  float* dv2;
  // Deterministic mode (null otherwise): every (query, short key, query head) row stores its dk1 / dv1 contribution
  // at [(query row * w1 + short-key slot) * Hq + head][D] instead of adding it atomically; a second kernel sums the
  // contributions of a key in a fixed order.
  float* dk1_part;
  float* dv1_part;
  long long ldq, ldk1, ldv1, lddo, lddq;
  int B, N, Hq, Hkv, w1, w2;
  float scale, scale_log2;
  int* status;
};

// delta[b, h, i] = sum_d out * dout   (one warp per (token, head)); strided rows.
__global__ void simp_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, long long ldo, long long lddo, int B, int N, int Hq) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)B * N * Hq) return;
  const long long row = w / Hq;
  const int h = int(w % Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(out + row * ldo + h * SB_D + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(dout + row * lddo + h * SB_D + lane * 4);
  const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(gh[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[((row / N) * Hq + h) * N + (row % N)] = s;
}

// out[row, c] = bf16(acc[row, c]) for an fp32 [rows, cols] buffer into a strided bf16 destination.
__global__ void simp_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dst, long long rows,
                                 int cols, long long ld) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= rows * cols) return;
  const long long row = i / cols;
  const int c = int(i % cols);
  const float4 v = *reinterpret_cast<const float4*>(acc + i);
  uint2 u;
  u.x = pack_bf16(v.x, v.y);
  u.y = pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(dst + row * ld + c) = u;
}

// Deterministic reductions.  dk1[b, j, hk, :] = sum over short-key slots jj (ascending) and the query heads of the
// group (ascending) of the contribution stored by query i = j + w1 - 1 - jj; one thread per 4 channels.
__global__ void simp_reduce_short_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dst, int B, int N, int Hq,
                                         int Hkv, int w1, long long ld) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cols4 = Hkv * SB_D / 4;
  if (t >= (long long)B * N * cols4) return;
  const long long row = t / cols4;
  const int c4 = int(t - row * cols4);
  const int hk = (c4 * 4) / SB_D, d = (c4 * 4) % SB_D;
  const int b = int(row / N), j = int(row - (long long)b * N);
  const int group = Hq / Hkv;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int jj = 0; jj < w1; ++jj) {
    const int i = j + w1 - 1 - jj;
    if (i >= N) continue;
    const long long qrow = (long long)b * N + i;
    for (int g = 0; g < group; ++g) {
      const float4 v = *reinterpret_cast<const float4*>(part + ((qrow * w1 + jj) * Hq + hk * group + g) * (long long)SB_D + d);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  }
  uint2 u;
  u.x = pack_bf16(acc.x, acc.y);
  u.y = pack_bf16(acc.z, acc.w);
  *reinterpret_cast<uint2*>(dst + row * ld + c4 * 4) = u;
}

// dst[row, c] = bf16(sum over planes g = 0 .. group-1, ascending, of part[g][row, c]).
__global__ void simp_reduce_planes_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dst, long long rows, int cols,
                                          int group, long long ld) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= rows * cols) return;
  const long long row = i / cols;
  const int c = int(i % cols);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = 0; g < group; ++g) {
    const float4 v = *reinterpret_cast<const float4*>(part + (long long)g * rows * cols + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  uint2 u;
  u.x = pack_bf16(acc.x, acc.y);
  u.y = pack_bf16(acc.z, acc.w);
  *reinterpret_cast<uint2*>(dst + row * ld + c) = u;
}

// Row r of a [128 x 128] K-major operand tile (two 64-column halves of 16 KB, 128-byte swizzle):
// element-wise product of two bf16 rows, zero when the row is masked.
// bf16 x bf16 rounded to bf16 equals the fp32 product rounded once, so the packed multiply is exact enough
// and five times cheaper than unpack / multiply / repack.
__device__ __forceinline__ uint4 mul_bf16x8(const uint4& a, const uint4& b) {
  uint4 o;
  const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&b);
  __nv_bfloat162* z = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) z[e] = __hmul2(x[e], y[e]);
  return o;
}

// All sixteen chunks of both rows are loaded before any product is stored: a store through a generic
// pointer between two global loads keeps the compiler from hoisting the loads, which serialises every
// chunk on the L2 latency.
__device__ __forceinline__ void build_product_row(uint8_t* tile, int r, const __nv_bfloat16* x, const __nv_bfloat16* y,
                                                  bool valid) {
#pragma unroll
  for (int hb = 0; hb < 2; ++hb) {
    uint4 xa[8], ya[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      xa[c] = valid ? *reinterpret_cast<const uint4*>(x + (hb * 8 + c) * 8) : make_uint4(0u, 0u, 0u, 0u);
      ya[c] = valid ? *reinterpret_cast<const uint4*>(y + (hb * 8 + c) * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int chunk = c ^ (r & 7);
      *reinterpret_cast<uint4*>(tile + hb * 16384 + r * 128 + chunk * 16) = mul_bf16x8(xa[c], ya[c]);
    }
  }
}

__device__ __forceinline__ float ex2_approx(float x) {   // one MUFU op; exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float segsum(float v, int w1) {
  for (int o = 1; o < w1; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Barrier of the 128 compute threads of the query-owned kernel that ANDs a predicate.
__device__ __forceinline__ bool sb_bar_and(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

struct SimpBwdQSmem {
  static constexpr int kA = 0;                    // 32 KB  q * k1 rows
  static constexpr int kG = 32768;                // 32 KB  dO * v1 rows
  static constexpr int kK = 65536;                // 2 x 16 KB  K2 tiles [64 keys][128 d]
  static constexpr int kV = kK + 2 * 16384;       // 2 x 16 KB  V2 tiles
  static constexpr int kP = kV + 2 * 16384;       // 16 KB  P  [128 rows][64 keys]
  static constexpr int kDS = kP + 16384;          // 16 KB  dS
  static constexpr int kBar = kDS + 16384;
  static constexpr int kTotal = kBar + 16 * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(SB_THREADS, 1)
simplicial_bwd_q_kernel(const __grid_constant__ CUtensorMap tm_k2, const __grid_constant__ CUtensorMap tm_v2,
                        const SimpBwdParams p) {
  using S = SimpBwdQSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* ag_full = bars + 0;
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* kv_empty = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;      // [2]
  uint64_t* s_free = bars + 7;      // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* p_empty = bars + 10;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BQ = 128 / p.w1;
  const int i0 = blockIdx.x * BQ;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int row_base = b * p.N;
  const int i_last = min(i0 + BQ - 1, p.N - 1);
  const int t_lo = max(0, i0 - p.w2 + 1) / SB_BK;
  const int t_hi = i_last / SB_BK;
  const int ntiles = t_hi - t_lo + 1;
  const int kv_col = hk * SB_D;

  if (threadIdx.x == 0) {
    mbar_init(ag_full, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;            // 2 x 64 columns
  const uint32_t tmem_dP = tmem_base + 128;     // 2 x 64 columns
  const uint32_t tmem_dA = tmem_base + 256;     // 128 columns
  const uint32_t tmem_Op = tmem_base + 384;     // 128 columns

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k2);
      tma_prefetch_desc(&tm_v2);
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j & 1;
        ok = mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1u, abort_word);
        if (!ok) break;
        const int krow = row_base + (t_lo + j) * SB_BK;
        uint8_t* sK = smem + S::kK + st * 16384;
        uint8_t* sV = smem + S::kV + st * 16384;
        mbar_expect_tx(&kv_full[st], 2 * 16384);
        tma_load_3d(sK, &tm_k2, &kv_full[st], kv_col, krow, 0);
        tma_load_3d(sK + 8192, &tm_k2, &kv_full[st], kv_col + 64, krow, 0);
        tma_load_3d(sV, &tm_v2, &kv_full[st], kv_col, krow, 0);
        tma_load_3d(sV + 8192, &tm_v2, &kv_full[st], kv_col + 64, krow, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);      // [128 rows] x [64 keys], K = d
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, 0, 1);   // [128 rows] x [128 d],   K = keys
      const uint32_t sA = smem_u32(smem + S::kA);
      const uint32_t sG = smem_u32(smem + S::kG);
      const uint32_t sP = smem_u32(smem + S::kP);
      const uint32_t sDS = smem_u32(smem + S::kDS);
      bool ok = mbar_wait(ag_full, 0, abort_word);
      auto issue_scores = [&](int j) {
        const uint32_t sK = smem_u32(smem + S::kK + (j & 1) * 16384);
        const uint32_t sV = smem_u32(smem + S::kV + (j & 1) * 16384);
        const uint32_t dS_ = tmem_S + uint32_t((j & 1) * 64);
        const uint32_t dP_ = tmem_dP + uint32_t((j & 1) * 64);
#pragma unroll
        for (int k = 0; k < SB_D / 16; ++k) {
          const uint32_t offa = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * 8192 + (k & 3) * 32;
          umma_bf16_ss(dS_, umma_smem_desc(sA + offa, 16, 1024), umma_smem_desc(sK + offb, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < SB_D / 16; ++k) {
          const uint32_t offa = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * 8192 + (k & 3) * 32;
          umma_bf16_ss(dP_, umma_smem_desc(sG + offa, 16, 1024), umma_smem_desc(sV + offb, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          const int jn = j + 1;
          ok = mbar_wait(&kv_full[jn & 1], (jn >> 1) & 1, abort_word);
          if (ok) ok = mbar_wait(&s_free[jn & 1], ((jn >> 1) & 1) ^ 1u, abort_word);
          if (!ok) break;
          tc_fence_after();
          issue_scores(jn);
        }
        ok = mbar_wait(p_full, j & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + S::kK + (j & 1) * 16384);
        const uint32_t sV = smem_u32(smem + S::kV + (j & 1) * 16384);
#pragma unroll
        for (int k = 0; k < SB_BK / 16; ++k) {
          umma_bf16_ss(tmem_dA, umma_smem_desc(sDS + k * 32, 16, 1024), umma_smem_desc(sK + k * 2048, 8192, 1024),
                       idesc_acc, (j | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < SB_BK / 16; ++k) {
          umma_bf16_ss(tmem_Op, umma_smem_desc(sP + k * 32, 16, 1024), umma_smem_desc(sV + k * 2048, 8192, 1024),
                       idesc_acc, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[j & 1]);
        umma_commit(p_empty);
      }
    }
  } else {
    // ---------------------------------------------------------------- compute warps: row = (query, short key)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qi = r / p.w1, jj = r % p.w1;
    const int i = i0 + qi;
    const int p1 = i - p.w1 + 1 + jj;
    const bool row_valid = (i < p.N) && (p1 >= 0);
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const long long qrow_idx = row_base + min(i, p.N - 1);
    const long long krow_idx = row_base + max(p1, 0);
    const __nv_bfloat16* qrow = p.q + qrow_idx * p.ldq + h * SB_D;
    const __nv_bfloat16* k1row = p.k1 + krow_idx * p.ldk1 + hk * SB_D;
    const __nv_bfloat16* v1row = p.v1 + krow_idx * p.ldv1 + hk * SB_D;
    const __nv_bfloat16* dorow = p.dout + qrow_idx * p.lddo + h * SB_D;
    build_product_row(smem + S::kA, r, qrow, k1row, row_valid);
    build_product_row(smem + S::kG, r, dorow, v1row, row_valid);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(ag_full);
    const long long stat = ((long long)b * p.Hq + h) * p.N + min(i, p.N - 1);
    const float lse = p.lse2[stat];
    const float dlt = p.delta[stat];
    bool ok = true;
    uint8_t* sP = smem + S::kP;
    uint8_t* sDS = smem + S::kDS;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int k0 = (t_lo + j) * SB_BK;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[2][32], dv[2][32];
      const uint32_t tS = tmem_S + uint32_t((j & 1) * 64) + lane_off;
      const uint32_t tP = tmem_dP + uint32_t((j & 1) * 64) + lane_off;
      tmem_ld_32x32(tS, sv[0]);
      tmem_ld_32x32(tS + 32, sv[1]);
      tmem_ld_32x32(tP, dv[0]);
      tmem_ld_32x32(tP + 32, dv[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[j & 1]);          // the score buffers can be overwritten
      const int lo = i - p.w2 + 1 - k0, hi = i - k0;      // valid columns are [lo, hi]
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (j - 1) & 1, abort_word));
        if (!ok) break;
      }
      // rows whose whole 64-key tile is visible skip the per-element window test
      const bool full = row_valid && lo <= 0 && hi >= SB_BK - 1;
      const float lse_row = row_valid ? lse : INFINITY;          // exp2(-inf) = 0 for padded rows
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float pr[8], ds[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = c * 32 + g * 8 + e;
            const float l = (full || (col >= lo && col <= hi)) ? lse_row : INFINITY;
            const float pv = ex2_approx(fmaf(__uint_as_float(sv[c][g * 8 + e]), p.scale_log2, -l));
            pr[e] = pv;
            ds[e] = (pv * p.scale) * (__uint_as_float(dv[c][g * 8 + e]) - dlt);
          }
          const int chunk = (c * 4 + g) ^ (r & 7);
          uint4 u, w;
          u.x = pack_bf16(pr[0], pr[1]);
          u.y = pack_bf16(pr[2], pr[3]);
          u.z = pack_bf16(pr[4], pr[5]);
          u.w = pack_bf16(pr[6], pr[7]);
          w.x = pack_bf16(ds[0], ds[1]);
          w.y = pack_bf16(ds[2], ds[3]);
          w.z = pack_bf16(ds[4], ds[5]);
          w.w = pack_bf16(ds[6], ds[7]);
          *reinterpret_cast<uint4*>(sP + r * 128 + chunk * 16) = u;
          *reinterpret_cast<uint4*>(sDS + r * 128 + chunk * 16) = w;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (ntiles - 1) & 1, abort_word));
    if (ok) {
      tc_fence_after();
      float* red = reinterpret_cast<float*>(smem + S::kK);
      float* dk1row = p.dk1 + krow_idx * ((long long)p.Hkv * SB_D) + hk * SB_D;
      float* dv1row = p.dv1 + krow_idx * ((long long)p.Hkv * SB_D) + hk * SB_D;
      const long long part_off = ((qrow_idx * p.w1 + jj) * p.Hq + h) * (long long)SB_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint4 kk[4], qq[4], gg[4];                         // loads first: the atomics below would pin them in place
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          kk[g] = *reinterpret_cast<const uint4*>(k1row + c * 32 + g * 8);
          qq[g] = *reinterpret_cast<const uint4*>(qrow + c * 32 + g * 8);
          gg[g] = *reinterpret_cast<const uint4*>(dorow + c * 32 + g * 8);
        }
        uint32_t da[32], op[32];
        tmem_ld_32x32(tmem_dA + lane_off + c * 32, da);
        tmem_ld_32x32(tmem_Op + lane_off + c * 32, op);
        tmem_ld_wait();
        float dqv[32];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kk[g]);
          const __nv_bfloat162* qh = reinterpret_cast<const __nv_bfloat162*>(&qq[g]);
          const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gg[g]);
          float dk[8], dvv[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 kf = __bfloat1622float2(kh[e]), qf = __bfloat1622float2(qh[e]), gf = __bfloat1622float2(gh[e]);
            const float a0 = __uint_as_float(da[g * 8 + 2 * e]), a1 = __uint_as_float(da[g * 8 + 2 * e + 1]);
            const float o0 = __uint_as_float(op[g * 8 + 2 * e]), o1 = __uint_as_float(op[g * 8 + 2 * e + 1]);
            dqv[g * 8 + 2 * e] = row_valid ? a0 * kf.x : 0.f;
            dqv[g * 8 + 2 * e + 1] = row_valid ? a1 * kf.y : 0.f;
            dk[2 * e] = a0 * qf.x;
            dk[2 * e + 1] = a1 * qf.y;
            dvv[2 * e] = o0 * gf.x;
            dvv[2 * e + 1] = o1 * gf.y;
          }
          if (row_valid && p.dk1_part != nullptr) {
            float* pk1 = p.dk1_part + part_off + c * 32 + g * 8;
            float* pv1 = p.dv1_part + part_off + c * 32 + g * 8;
            *reinterpret_cast<float4*>(pk1) = make_float4(dk[0], dk[1], dk[2], dk[3]);
            *reinterpret_cast<float4*>(pk1 + 4) = make_float4(dk[4], dk[5], dk[6], dk[7]);
            *reinterpret_cast<float4*>(pv1) = make_float4(dvv[0], dvv[1], dvv[2], dvv[3]);
            *reinterpret_cast<float4*>(pv1 + 4) = make_float4(dvv[4], dvv[5], dvv[6], dvv[7]);
          } else if (row_valid) {
            atomicAdd(reinterpret_cast<float4*>(dk1row + c * 32 + g * 8), make_float4(dk[0], dk[1], dk[2], dk[3]));
            atomicAdd(reinterpret_cast<float4*>(dk1row + c * 32 + g * 8 + 4), make_float4(dk[4], dk[5], dk[6], dk[7]));
            atomicAdd(reinterpret_cast<float4*>(dv1row + c * 32 + g * 8), make_float4(dvv[0], dvv[1], dvv[2], dvv[3]));
            atomicAdd(reinterpret_cast<float4*>(dv1row + c * 32 + g * 8 + 4), make_float4(dvv[4], dvv[5], dvv[6], dvv[7]));
          }
        }
        // dq partials of this row go to shared memory (the K2 / V2 / P / dS buffers are idle now); the
        // sum over a query's w1 rows is done per column below instead of by 160 dependent shuffles
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<float4*>(red + r * 132 + c * 32 + g * 4) =
              make_float4(dqv[4 * g], dqv[4 * g + 1], dqv[4 * g + 2], dqv[4 * g + 3]);
      }
    }
    ok = sb_bar_and(ok);                            // all four compute warps, whatever happened above
    if (ok) {
      const float* red = reinterpret_cast<const float*>(smem + S::kK);
      for (int qq = 0; qq < BQ; ++qq) {
        const int iq = i0 + qq;
        if (iq >= p.N) break;
        float a0 = 0.f, a1 = 0.f;
        const float* col = red + (qq * p.w1) * 132 + r;
        for (int x = 0; x < p.w1; x += 2) {
          a0 += col[x * 132];
          a1 += col[(x + 1) * 132];
        }
        p.dq[(long long)(row_base + iq) * p.lddq + h * SB_D + r] = __float2bfloat16(a0 + a1);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}


// ================================================================================================
// Part 2: key-owned kernel.  CTA = 128 long keys of one (batch, kv head); thread t of the compute
// warps owns key k0 + t.  Walks, for every query head of the group, the 64-row groups (64 / w1
// queries x w1 short keys) whose long window reaches these keys, in the transposed frame:
//     S^T = K2 A^T    dP^T = V2 G^T    dK2 += dS^T A    dV2 += P^T G
// The A / G row groups are rebuilt by two builder warps (double-buffered) while the tensor core and
// the compute warps work on the previous group.  dK2 / dV2 never leave TMEM until the end: plain
// stores, no atomics, bit-reproducible.
// ================================================================================================
constexpr int SK_BK = 128;           // keys per CTA
constexpr int SK_ROWS = 64;          // rows (query, short key) per inner step
constexpr int SK_THREADS = 448;      // TMA warp, MMA warp, 8 compute warps (two per scheduler), 4 builder warps

struct SimpBwdKParams {
  SimpBwdParams c;
  long long* prof;             // optional phase cycle counters
  __nv_bfloat16* dk2;          // [B*N, lddk2] bf16 (written directly when every KV head has one query head)
  __nv_bfloat16* dv2;
  long long lddk2, lddv2;
  float* dk2_acc;              // [B*N, Hkv*D] fp32, zeroed by the launcher: target of the per-query-head CTAs'
  float* dv2_acc;              //   vector atomics when a KV head serves several query heads
  float* dk2_part;             // deterministic mode: [group][B*N, Hkv*D] fp32, one plane per query head of a KV group
  float* dv2_part;             //   (plain stores; summed in head order afterwards)
};

// Optional phase cycle counters (16 slots), written by CTA (0,0,0) of the key-owned kernel.
static long long* g_simp_prof = nullptr;

struct SimpBwdKSmem {
  static constexpr int kK = 0;                    // 32 KB K2 [128 keys][128 d]
  static constexpr int kV = 32768;                // 32 KB V2
  static constexpr int kA = 65536;                // 2 x 16 KB A row groups [64 rows][128 d]
  static constexpr int kG = kA + 2 * 16384;       // 2 x 16 KB G row groups
  static constexpr int kPT = kG + 2 * 16384;      // 16 KB P^T  [128 keys][64 rows]
  static constexpr int kDST = kPT + 16384;        // 16 KB dS^T
  static constexpr int kVec = kDST + 16384;       // [2 buffers][lse 64 | delta 64] floats
  static constexpr int kBar = kVec + 2 * 128 * 4;
  static constexpr int kTotal = kBar + 16 * 8 + 16 + 1024;
};

template <int W1>
__global__ void __launch_bounds__(SK_THREADS, 1)
simplicial_bwd_k_kernel(const __grid_constant__ CUtensorMap tm_k2, const __grid_constant__ CUtensorMap tm_v2,
                        const SimpBwdKParams pk) {
  using S = SimpBwdKSmem;
  const SimpBwdParams& p = pk.c;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* kv_full = bars + 0;
  uint64_t* ag_full = bars + 1;     // [2] builders -> MMA / compute
  uint64_t* ag_empty = bars + 3;    // [2] accumulation MMAs done with the row group
  uint64_t* st_full = bars + 5;     // [2] S^T / dP^T ready in TMEM
  uint64_t* st_free = bars + 7;     // [2] compute warps have read them
  uint64_t* pds_full = bars + 9;    // P^T / dS^T written to shared memory
  uint64_t* pds_empty = bars + 10;  // accumulation MMAs have consumed them
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* s_vec = reinterpret_cast<float*>(smem + S::kVec);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;     // one CTA per (key tile, QUERY head)
  const int group = p.Hq / p.Hkv;
  const int hk = hq / group;
  const int k0 = kt * SK_BK;
  const int row_base = b * p.N;
  constexpr int sh = (W1 == 8) ? 3 : (W1 == 16 ? 4 : 5);
  constexpr int QS = SK_ROWS >> sh;                           // queries per row group
  const int q_lo = (k0 / QS) * QS;
  const int q_last = min(p.N - 1, k0 + SK_BK - 1 + p.w2 - 1);
  const int nsub = (q_last - q_lo) / QS + 1;
  const int total = nsub;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ag_full[i], 4);
      mbar_init(&ag_empty[i], 1);
      mbar_init(&st_full[i], 1);
      mbar_init(&st_free[i], 8);
    }
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_ST = tmem_base;            // 2 x 64 columns
  const uint32_t tmem_dPT = tmem_base + 128;     // 2 x 64 columns
  const uint32_t tmem_dK = tmem_base + 256;      // 128 columns
  const uint32_t tmem_dV = tmem_base + 384;      // 128 columns

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k2);
      tma_prefetch_desc(&tm_v2);
      mbar_expect_tx(kv_full, 2 * 32768);
      const int kv_col = hk * SB_D;
      tma_load_3d(smem + S::kK, &tm_k2, kv_full, kv_col, row_base + k0, 0);
      tma_load_3d(smem + S::kK + 16384, &tm_k2, kv_full, kv_col + 64, row_base + k0, 0);
      tma_load_3d(smem + S::kV, &tm_v2, kv_full, kv_col, row_base + k0, 0);
      tma_load_3d(smem + S::kV + 16384, &tm_v2, kv_full, kv_col + 64, row_base + k0, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);      // [128 keys] x [64 rows], K = d
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, 0, 1);   // [128 keys] x [128 d],   K = rows
      const uint32_t sK = smem_u32(smem + S::kK);
      const uint32_t sV = smem_u32(smem + S::kV);
      const uint32_t sPT = smem_u32(smem + S::kPT);
      const uint32_t sDST = smem_u32(smem + S::kDST);
      bool ok = mbar_wait(kv_full, 0, abort_word);
      auto issue_scores = [&](int it) {
        const uint32_t sA = smem_u32(smem + S::kA + (it & 1) * 16384);
        const uint32_t sG = smem_u32(smem + S::kG + (it & 1) * 16384);
        const uint32_t dS_ = tmem_ST + uint32_t((it & 1) * 64);
        const uint32_t dP_ = tmem_dPT + uint32_t((it & 1) * 64);
#pragma unroll
        for (int k = 0; k < SB_D / 16; ++k) {
          const uint32_t offa = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * 8192 + (k & 3) * 32;
          umma_bf16_ss(dS_, umma_smem_desc(sK + offa, 16, 1024), umma_smem_desc(sA + offb, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < SB_D / 16; ++k) {
          const uint32_t offa = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * 8192 + (k & 3) * 32;
          umma_bf16_ss(dP_, umma_smem_desc(sV + offa, 16, 1024), umma_smem_desc(sG + offb, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
        umma_commit(&st_full[it & 1]);
      };
      if (ok) ok = mbar_wait(&ag_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int it = 0; it < total && ok; ++it) {
        if (it + 1 < total) {
          const int n = it + 1;
          ok = mbar_wait(&ag_full[n & 1], (n >> 1) & 1, abort_word);
          if (ok) ok = mbar_wait(&st_free[n & 1], ((n >> 1) & 1) ^ 1u, abort_word);
          if (!ok) break;
          tc_fence_after();
          issue_scores(n);
        }
        ok = mbar_wait(pds_full, it & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sA = smem_u32(smem + S::kA + (it & 1) * 16384);
        const uint32_t sG = smem_u32(smem + S::kG + (it & 1) * 16384);
#pragma unroll
        for (int k = 0; k < SK_ROWS / 16; ++k)
          umma_bf16_ss(tmem_dK, umma_smem_desc(sDST + k * 32, 16, 1024), umma_smem_desc(sA + k * 2048, 8192, 1024),
                       idesc_acc, (it | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < SK_ROWS / 16; ++k)
          umma_bf16_ss(tmem_dV, umma_smem_desc(sPT + k * 32, 16, 1024), umma_smem_desc(sG + k * 2048, 8192, 1024),
                       idesc_acc, (it | k) != 0 ? 1u : 0u);
        umma_commit(&ag_empty[it & 1]);
        umma_commit(pds_empty);
      }
    }
  } else if (warp >= 10) {
    // ---------------------------------------------------------------- builder warps: half a row each
    const int tid = (warp - 10) * 32 + lane;              // 0..127
    const int c = tid >> 1, half = tid & 1;               // row of the group, 64-column half
    const int qi = c >> sh, jj = c & (W1 - 1);
    bool ok = true;
    const bool prof = pk.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 10 && lane == 0;
    long long bw = 0, bb = 0;
    // The rows of step it + 1 are fetched into registers BEFORE waiting for their buffer: the L2 latency of
    // the 32 loads per thread overlaps the wait instead of following it.
    // (k1 / v1 rows only: the q / dO rows are shared by the w1 rows of a query and hit in L1, they are read after
    // the wait so that 64 instead of 128 registers stay live across it)
    uint4 kv[8], vv[8];
    const __nv_bfloat16* n_qrow = p.q;
    const __nv_bfloat16* n_dorow = p.dout;
    bool n_valid = false;
    float n_lse = INFINITY, n_del = 0.f;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    auto fetch = [&](int it) {
      const int i = q_lo + it * QS + qi;
      const int p1 = i - W1 + 1 + jj;
      const bool valid = (i <= q_last) && (p1 >= 0);
      const long long qrow_idx = row_base + min(i, p.N - 1);
      const long long krow_idx = row_base + max(p1, 0);
      n_qrow = p.q + qrow_idx * p.ldq + hq * SB_D + half * 64;
      n_dorow = p.dout + qrow_idx * p.lddo + hq * SB_D + half * 64;
      n_valid = valid;
      const __nv_bfloat16* k1row = p.k1 + krow_idx * p.ldk1 + hk * SB_D + half * 64;
      const __nv_bfloat16* v1row = p.v1 + krow_idx * p.ldv1 + hk * SB_D + half * 64;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        kv[ch] = valid ? *reinterpret_cast<const uint4*>(k1row + ch * 8) : zero4;
        vv[ch] = valid ? *reinterpret_cast<const uint4*>(v1row + ch * 8) : zero4;
      }
      if (half == 0) {
        const long long stat = ((long long)b * p.Hq + hq) * p.N + min(i, p.N - 1);
        n_lse = valid ? p.lse2[stat] : INFINITY;
        n_del = valid ? p.delta[stat] : 0.f;
      }
    };
    if (total > 0) fetch(0);
    for (int it = 0; it < total && ok; ++it) {
      const int buf = it & 1;
      const long long b0 = clock64();
      ok = __all_sync(0xffffffffu, mbar_wait(&ag_empty[buf], ((it >> 1) & 1) ^ 1u, abort_word));
      if (!ok) break;
      const long long b1 = clock64();
      uint8_t* tA = smem + S::kA + buf * 16384 + half * 8192 + c * 128;     // a [64 x 128] group: two 8 KB halves
      uint8_t* tG = smem + S::kG + buf * 16384 + half * 8192 + c * 128;
      {
        uint4 qv[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) qv[ch] = n_valid ? *reinterpret_cast<const uint4*>(n_qrow + ch * 8) : zero4;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(tA + (ch ^ (c & 7)) * 16) = mul_bf16x8(qv[ch], kv[ch]);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) qv[ch] = n_valid ? *reinterpret_cast<const uint4*>(n_dorow + ch * 8) : zero4;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(tG + (ch ^ (c & 7)) * 16) = mul_bf16x8(qv[ch], vv[ch]);
      }
      if (half == 0) {
        s_vec[buf * 128 + c] = n_lse;
        s_vec[buf * 128 + 64 + c] = n_del;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ag_full[buf]);
      if (it + 1 < total) fetch(it + 1);
      if (prof) { bw += b1 - b0; bb += clock64() - b1; }
    }
    if (prof) { pk.prof[8] = bw; pk.prof[9] = bb; }
  } else {
    // ---------------------------------------------------------------- compute warps: thread = key; warps 2..5 own
    // columns 0..31 of the 64-row step, warps 6..9 columns 32..63, so that every scheduler has two of them
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int t = quarter * 32 + lane;
    const int kp = k0 + t;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    uint8_t* sPT = smem + S::kPT;
    uint8_t* sDST = smem + S::kDST;
    bool ok = true;
    const bool prof = pk.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 2 && lane == 0;
    long long pc[5] = {0, 0, 0, 0, 0};
    for (int it = 0; it < total && ok; ++it) {
      const int buf = it & 1;
      const int i_start = q_lo + it * QS;
      const long long c0 = clock64();
      ok = __all_sync(0xffffffffu, mbar_wait(&ag_full[buf], (it >> 1) & 1, abort_word));   // stats visible
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&st_full[buf], (it >> 1) & 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      const long long c1 = clock64();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem_ST + uint32_t(buf * 64 + chalf * 32) + lane_off, sv);
      tmem_ld_32x32(tmem_dPT + uint32_t(buf * 64 + chalf * 32) + lane_off, dv);
      tmem_ld_wait();
      const long long c2 = clock64();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&st_free[buf]);
      if (it > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(pds_empty, (it - 1) & 1, abort_word));
        if (!ok) break;
      }
      const long long c3 = clock64();
      const float4* lse4 = reinterpret_cast<const float4*>(s_vec + buf * 128);
      const float4* dlt4 = lse4 + 16;
      bool qmask[QS];                                      // this key is inside query qq's long window
#pragma unroll
      for (int qq = 0; qq < QS; ++qq) {
        const int i = i_start + qq;
        qmask[qq] = (kp <= i) && (kp > i - p.w2);
      }
      {
        const int c2 = chalf;
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          float ls[8], dl[8];
          *reinterpret_cast<float4*>(&ls[0]) = lse4[c2 * 8 + gq * 2];
          *reinterpret_cast<float4*>(&ls[4]) = lse4[c2 * 8 + gq * 2 + 1];
          *reinterpret_cast<float4*>(&dl[0]) = dlt4[c2 * 8 + gq * 2];
          *reinterpret_cast<float4*>(&dl[4]) = dlt4[c2 * 8 + gq * 2 + 1];
          float pr[8], ds[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = c2 * 32 + gq * 8 + e;
            const float l = qmask[col >> sh] ? ls[e] : INFINITY;        // masked or padded row: exp2(-inf) = 0
            const float pv = ex2_approx(fmaf(__uint_as_float(sv[gq * 8 + e]), p.scale_log2, -l));
            pr[e] = pv;
            ds[e] = (pv * p.scale) * (__uint_as_float(dv[gq * 8 + e]) - dl[e]);
          }
          const int chunk = (c2 * 4 + gq) ^ (t & 7);
          uint4 u, w;
          u.x = pack_bf16(pr[0], pr[1]);
          u.y = pack_bf16(pr[2], pr[3]);
          u.z = pack_bf16(pr[4], pr[5]);
          u.w = pack_bf16(pr[6], pr[7]);
          w.x = pack_bf16(ds[0], ds[1]);
          w.y = pack_bf16(ds[2], ds[3]);
          w.z = pack_bf16(ds[4], ds[5]);
          w.w = pack_bf16(ds[6], ds[7]);
          *reinterpret_cast<uint4*>(sPT + t * 128 + chunk * 16) = u;
          *reinterpret_cast<uint4*>(sDST + t * 128 + chunk * 16) = w;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (prof) {
        const long long c4 = clock64();
        pc[0] += c1 - c0; pc[1] += c2 - c1; pc[2] += c3 - c2; pc[3] += c4 - c3; pc[4] += 1;
      }
    }
    if (prof) {
      for (int i = 0; i < 5; ++i) pk.prof[i] = pc[i];
    }
    // ---------------------------------------------------------------- epilogue: plain stores
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(pds_empty, (total - 1) & 1, abort_word));
    if (ok) {
      tc_fence_after();
      const long long krow = row_base + min(kp, p.N - 1);
      __nv_bfloat16* dkrow = pk.dk2 + krow * pk.lddk2 + hk * SB_D;
      __nv_bfloat16* dvrow = pk.dv2 + krow * pk.lddv2 + hk * SB_D;
      float* dkacc = pk.dk2_acc + krow * ((long long)p.Hkv * SB_D) + hk * SB_D;
      float* dvacc = pk.dv2_acc + krow * ((long long)p.Hkv * SB_D) + hk * SB_D;
#pragma unroll 1
      for (int c = chalf * 2; c < chalf * 2 + 2; ++c) {          // each warp of a lane quarter stores half the channels
        uint32_t a[32], v[32];
        tmem_ld_32x32(tmem_dK + lane_off + c * 32, a);
        tmem_ld_32x32(tmem_dV + lane_off + c * 32, v);
        tmem_ld_wait();
        if (kp < p.N) {
          if (group == 1) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              uint4 u, w;
              u.x = pack_bf16(__uint_as_float(a[8 * gq + 0]), __uint_as_float(a[8 * gq + 1]));
              u.y = pack_bf16(__uint_as_float(a[8 * gq + 2]), __uint_as_float(a[8 * gq + 3]));
              u.z = pack_bf16(__uint_as_float(a[8 * gq + 4]), __uint_as_float(a[8 * gq + 5]));
              u.w = pack_bf16(__uint_as_float(a[8 * gq + 6]), __uint_as_float(a[8 * gq + 7]));
              w.x = pack_bf16(__uint_as_float(v[8 * gq + 0]), __uint_as_float(v[8 * gq + 1]));
              w.y = pack_bf16(__uint_as_float(v[8 * gq + 2]), __uint_as_float(v[8 * gq + 3]));
              w.z = pack_bf16(__uint_as_float(v[8 * gq + 4]), __uint_as_float(v[8 * gq + 5]));
              w.w = pack_bf16(__uint_as_float(v[8 * gq + 6]), __uint_as_float(v[8 * gq + 7]));
              *reinterpret_cast<uint4*>(dkrow + c * 32 + gq * 8) = u;
              *reinterpret_cast<uint4*>(dvrow + c * 32 + gq * 8) = w;
            }
          } else if (pk.dk2_part != nullptr) {
            const long long plane = (long long)(hq % group) * p.B * p.N * ((long long)p.Hkv * SB_D);
            float* pkd = pk.dk2_part + plane + krow * ((long long)p.Hkv * SB_D) + hk * SB_D + c * 32;
            float* pvd = pk.dv2_part + plane + krow * ((long long)p.Hkv * SB_D) + hk * SB_D + c * 32;
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              *reinterpret_cast<float4*>(pkd + q4 * 4) = make_float4(__uint_as_float(a[4 * q4]), __uint_as_float(a[4 * q4 + 1]),
                                                                     __uint_as_float(a[4 * q4 + 2]), __uint_as_float(a[4 * q4 + 3]));
              *reinterpret_cast<float4*>(pvd + q4 * 4) = make_float4(__uint_as_float(v[4 * q4]), __uint_as_float(v[4 * q4 + 1]),
                                                                     __uint_as_float(v[4 * q4 + 2]), __uint_as_float(v[4 * q4 + 3]));
            }
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              atomicAdd(reinterpret_cast<float4*>(dkacc + c * 32 + q4 * 4),
                        make_float4(__uint_as_float(a[4 * q4]), __uint_as_float(a[4 * q4 + 1]), __uint_as_float(a[4 * q4 + 2]),
                                    __uint_as_float(a[4 * q4 + 3])));
              atomicAdd(reinterpret_cast<float4*>(dvacc + c * 32 + q4 * 4),
                        make_float4(__uint_as_float(v[4 * q4]), __uint_as_float(v[4 * q4 + 1]), __uint_as_float(v[4 * q4 + 2]),
                                    __uint_as_float(v[4 * q4 + 3])));
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

}  // namespace nga

extern "C" void nga_simplicial_bwd_set_prof(long long* device_ptr) { nga::g_simp_prof = device_ptr; }

// Deterministic (atomic-free, bit-reproducible) mode for the NEXT call of nga_simplicial_bwd on this thread: scratch for
// the per-row short-key contributions, [B*N * w1 * Hq, 128] fp32 each, and (only when Hq > Hkv, else null) the per-head
// planes of the long-key gradients, [Hq / Hkv][B*N, Hkv*128] fp32 each.  The pointers are consumed by that call.
static thread_local float* g_det[4] = {nullptr, nullptr, nullptr, nullptr};
extern "C" void nga_simplicial_bwd_set_deterministic(float* dk1_part, float* dv1_part, float* dk2_part, float* dv2_part) {
  g_det[0] = dk1_part; g_det[1] = dv1_part; g_det[2] = dk2_part; g_det[3] = dv2_part;
}

// Backward of nga_simplicial_fwd.  `out`, `lse2` come from the forward pass.  dq / dk2 / dv2 are
// written as bf16 (strided like their inputs); dk1 / dv1 are accumulated in the fp32 scratch
// buffers `dk1_acc` / `dv1_acc` ([B*N, Hkv*128], zeroed here) and cast into dk1 / dv1; `dk2_acc` /
// `dv2_acc` (same shape) are needed only when Hq > Hkv (may be null otherwise); `delta` is fp32
// scratch [B, Hq, N].
extern "C" int nga_simplicial_bwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                                  const void* out, const void* dout, const float* lse2, void* dq, void* dk1,
                                  void* dk2, void* dv1, void* dv2, float* dk1_acc, float* dv1_acc, float* dk2_acc,
                                  float* dv2_acc, float* delta,
                                  long long ldq, long long ldk1, long long ldk2, long long ldv1, long long ldv2,
                                  long long ldo, long long lddo, long long lddq, long long lddk1, long long lddk2,
                                  long long lddv1, long long lddv2, int B, int N, int Hq, int Hkv, int D, int w1,
                                  int w2, float scale, int* status, void* stream) {
  using namespace nga;
  if (D != SB_D || B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  if (!(w1 == 8 || w1 == 16 || w1 == 32) || w2 < w1) return -6;
  if ((ldq | ldk1 | ldk2 | ldv1 | ldv2 | ldo | lddo | lddq | lddk1 | lddk2 | lddv1 | lddv2) & 7) return -5;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * N;
  const long long kvcols = (long long)Hkv * D;
  float* det[4] = {g_det[0], g_det[1], g_det[2], g_det[3]};
  g_det[0] = g_det[1] = g_det[2] = g_det[3] = nullptr;
  const bool deterministic = det[0] != nullptr && det[1] != nullptr;
  if (deterministic && Hq != Hkv && (det[2] == nullptr || det[3] == nullptr)) return -7;
  CUtensorMap tk64, tv64, tk128, tv128;
  int rc = make_tmap_3d(&tk64, k2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kvcols, rows, 1, ldk2 * 2, rows * ldk2 * 2, 64, 64, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tv64, v2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kvcols, rows, 1, ldv2 * 2, rows * ldv2 * 2, 64, 64, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tk128, k2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kvcols, rows, 1, ldk2 * 2, rows * ldk2 * 2, 64, 128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tv128, v2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kvcols, rows, 1, ldv2 * 2, rows * ldv2 * 2, 64, 128, true);
  if (rc) return rc;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(simplicial_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SimpBwdQSmem::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    for (auto kern : {simplicial_bwd_k_kernel<8>, simplicial_bwd_k_kernel<16>, simplicial_bwd_k_kernel<32>}) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SimpBwdKSmem::kTotal);
      if (e != cudaSuccess) return -1000 - (int)e;
    }
    attr_done = true;
  }
  {
    const long long warps = rows * Hq;
    simp_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, ldo, lddo, B,
        N, Hq);
    count_launch();
  }
  if (!deterministic) {
    cudaMemsetAsync(dk1_acc, 0, sizeof(float) * rows * kvcols, st);
    cudaMemsetAsync(dv1_acc, 0, sizeof(float) * rows * kvcols, st);
  }
  SimpBwdParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k1 = reinterpret_cast<const __nv_bfloat16*>(k1);
  p.v1 = reinterpret_cast<const __nv_bfloat16*>(v1);
  p.dout = reinterpret_cast<const __nv_bfloat16*>(dout);
  p.lse2 = lse2;
  p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk1 = dk1_acc;
  p.dv1 = dv1_acc;
  p.dk2 = nullptr;
  p.dv2 = nullptr;
  p.dk1_part = deterministic ? det[0] : nullptr;
  p.dv1_part = deterministic ? det[1] : nullptr;
  p.ldq = ldq; p.ldk1 = ldk1; p.ldv1 = ldv1; p.lddo = lddo; p.lddq = lddq;
  p.B = B; p.N = N; p.Hq = Hq; p.Hkv = Hkv; p.w1 = w1; p.w2 = w2;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  {
    const int BQ = 128 / w1;
    dim3 grid((N + BQ - 1) / BQ, Hq, B);
    simplicial_bwd_q_kernel<<<grid, SB_THREADS, SimpBwdQSmem::kTotal, st>>>(tk64, tv64, p);
    count_launch();
  }
  {
    SimpBwdKParams pk;
    pk.c = p;
    pk.dk2 = reinterpret_cast<__nv_bfloat16*>(dk2);
    pk.dv2 = reinterpret_cast<__nv_bfloat16*>(dv2);
    pk.lddk2 = lddk2; pk.lddv2 = lddv2;
    pk.dk2_acc = dk2_acc; pk.dv2_acc = dv2_acc;
    pk.prof = g_simp_prof;
    pk.dk2_part = (deterministic && Hq != Hkv) ? det[2] : nullptr;
    pk.dv2_part = (deterministic && Hq != Hkv) ? det[3] : nullptr;
    if (Hq != Hkv && pk.dk2_part == nullptr) {
      if (dk2_acc == nullptr || dv2_acc == nullptr) return -7;
      cudaMemsetAsync(dk2_acc, 0, sizeof(float) * rows * kvcols, st);
      cudaMemsetAsync(dv2_acc, 0, sizeof(float) * rows * kvcols, st);
    }
    dim3 grid((N + SK_BK - 1) / SK_BK, Hq, B);
    auto kern = w1 == 8 ? simplicial_bwd_k_kernel<8> : (w1 == 16 ? simplicial_bwd_k_kernel<16> : simplicial_bwd_k_kernel<32>);
    kern<<<grid, SK_THREADS, SimpBwdKSmem::kTotal, st>>>(tk128, tv128, pk);
    count_launch();
    if (Hq != Hkv && pk.dk2_part != nullptr) {
      const long long n4 = rows * kvcols / 4;
      simp_reduce_planes_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(pk.dk2_part, reinterpret_cast<__nv_bfloat16*>(dk2), rows,
                                                                             (int)kvcols, Hq / Hkv, lddk2);
      count_launch();
      simp_reduce_planes_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(pk.dv2_part, reinterpret_cast<__nv_bfloat16*>(dv2), rows,
                                                                             (int)kvcols, Hq / Hkv, lddv2);
      count_launch();
    } else if (Hq != Hkv) {
      const long long n4 = rows * kvcols / 4;
      simp_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dk2_acc, reinterpret_cast<__nv_bfloat16*>(dk2), rows,
                                                                    (int)kvcols, lddk2);
      count_launch();
      simp_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dv2_acc, reinterpret_cast<__nv_bfloat16*>(dv2), rows,
                                                                    (int)kvcols, lddv2);
      count_launch();
    }
  }
  if (deterministic) {
    const long long n4 = rows * kvcols / 4;
    simp_reduce_short_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(det[0], reinterpret_cast<__nv_bfloat16*>(dk1), B, N, Hq, Hkv,
                                                                          w1, lddk1);
    count_launch();
    simp_reduce_short_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(det[1], reinterpret_cast<__nv_bfloat16*>(dv1), B, N, Hq, Hkv,
                                                                          w1, lddv1);
    count_launch();
  } else {
    const long long n4 = rows * kvcols / 4;
    simp_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dk1_acc, reinterpret_cast<__nv_bfloat16*>(dk1), rows,
                                                                  (int)kvcols, lddk1);
    count_launch();
    simp_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dv1_acc, reinterpret_cast<__nv_bfloat16*>(dv1), rows,
                                                                  (int)kvcols, lddv1);
    count_launch();
  }
  NGA_CHECK_LAUNCH();
  return 0;
}
