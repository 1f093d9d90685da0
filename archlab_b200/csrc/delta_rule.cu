// Gated delta rule (scalar log-decay per token and head), chunk 64, key/value width 128, forward,
// on tcgen05 + TMEM.
//
//   S_t = e^{g_t} S_{t-1} + k_t (beta_t (v_t - k_t^T e^{g_t} S_{t-1}))^T ,   o_t = S_t^T q_t
//
// with q, k L2-normalised per row and q scaled by 1/sqrt(128) (the statement of
// src/archlab/architectures/qwen38_flash_next_full.py:535-554, whose fast path is fla-core's Triton
// chunk_gated_delta_rule).  Two kernels:
//
// 1. prep (one CTA per chunk x head x batch, fully parallel): normalise q and k, cumulative decay
//    G, the gram blocks [K; Q] K^T on the tensor core, the unit-lower-triangular inverse
//    T = (I + tril(beta P, -1))^-1 by forward substitution, then W = T (beta k e^G) and
//    U = T (beta v) on the tensor core.  Everything the recurrence needs for the chunk is written
//    as ONE 72 KB record that already has the shared-memory operand layout (128-byte swizzle), so
//    the second kernel fetches it with a single bulk copy and no tensor map.
// 2. scan (one CTA per head x batch, sequential over chunks): the state lives transposed in TMEM
//    (lane = value channel, column = key channel, fp32).  Per chunk: the state is copied to shared
//    memory as a bf16 operand and scaled in TMEM by e^{G_C}; u^T = U^T - S^T W^T; o^T = S^T qd^T
//    + u^T Aq^T; S^T += u^T kend.  All products have M = 128 (the value channels), so the chunk
//    length 64 only ever appears as N or as the reduction length.
#include "ptx.cuh"
#include "host_util.h"
#include "misc_kernels.h"
#include <cuda.h>

namespace nga {

constexpr int DR_C = 64;
constexpr int DR_D = 128;
// record layout (bytes)
constexpr int DR_W = 0;        // W   [c][k]  K-major image: two 64-wide k blocks of 64 rows x 128 B
constexpr int DR_QD = 16384;   // q e^{G}    same image
constexpr int DR_KE = 32768;   // k e^{G_C - G}  same bytes, read as an MN-major operand
constexpr int DR_U = 49152;    // U   [c][v]  plain row-major bf16
constexpr int DR_AQ = 65536;   // Aq  [t][s]  K-major image, 64 rows x 128 B
constexpr int DR_REC = 73728;

__device__ __forceinline__ uint32_t off64(int r, int k) {   // 64-row blocks
  return uint32_t((k >> 6) * 8192 + r * 128 + ((((k & 63) >> 3) ^ (r & 7)) << 4) + (k & 7) * 2);
}
__device__ __forceinline__ uint32_t off128(int r, int k) {  // 128-row blocks
  return uint32_t((k >> 6) * 16384 + r * 128 + ((((k & 63) >> 3) ^ (r & 7)) << 4) + (k & 7) * 2);
}
__device__ __forceinline__ void dr_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void dr_bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
// Barrier over `n` threads that also ANDs a predicate: every participant learns whether all waits
// before it succeeded, so that the whole group leaves a loop together.
__device__ __forceinline__ bool bar_and(int id, int n, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %3, 0;\n\t"
      "barrier.cta.red.and.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(n), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8], float s) {
  uint4 u;
  u.x = pack_bf16(f[0] * s, f[1] * s);
  u.y = pack_bf16(f[2] * s, f[3] * s);
  u.z = pack_bf16(f[4] * s, f[5] * s);
  u.w = pack_bf16(f[6] * s, f[7] * s);
  return u;
}

struct DeltaPrepParams {
  const __nv_bfloat16 *q, *k, *v;   // [B, T, H, 128]
  const float *g, *beta;            // [B, T, H]
  uint8_t* rec;                     // [B, H, chunks, DR_REC]
  float* eg;                        // [B, H, chunks]  e^{G_C}
  int B, T, H, chunks;
  float qscale;
  int* status;
};

struct DeltaPrepSmem {
  static constexpr int kKQ = 0;                       // 32 KB: [k rows 0..63; q rows 64..127] K-major, 128-row blocks
  static constexpr int kKB = 32768;                   // 16 KB: beta k e^G, [s][k] (MN-major A operand)
  static constexpr int kVB = kKB + 16384;             // 16 KB: beta v,    [s][v]
  static constexpr int kT = kVB + 16384;              // 8 KB : T [t][s] K-major
  static constexpr int kRec = kT + 8192;              // 72 KB record
  static constexpr int kA = kRec + DR_REC;            // 64 x 68 fp32
  static constexpr int kG = kA + 64 * 68 * 4;         // 64 G + 64 beta + 2 warp totals
  static constexpr int kBar = kG + 1024;
  static constexpr int kTotal = kBar + 64 + 1024;
};

__global__ void __launch_bounds__(128, 1)
delta_prep_kernel(const DeltaPrepParams p) {
  using S = DeltaPrepSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sA = reinterpret_cast<float*>(smem + S::kA);
  float* sG = reinterpret_cast<float*>(smem + S::kG);
  float* sBeta = sG + 64;
  float* sTot = sG + 128;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  uint8_t* sRec = smem + S::kRec;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = chunk * DR_C;

  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  float gsum = 0.f;
  if (tid < 64) {
    gsum = p.g[((long long)b * p.T + t0 + tid) * p.H + h];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, gsum, o);
      if (lane >= o) gsum += y;
    }
    if (lane == 31) sTot[warp] = gsum;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (tid < 64) {
    if (warp == 1) gsum += sTot[0];
    sG[tid] = gsum;
    sBeta[tid] = p.beta[((long long)b * p.T + t0 + tid) * p.H + h];
  }
  __syncthreads();
  const float kLog2e = 1.4426950408889634f;
  const float g_end = sG[63];

  // ---- rows: thread r < 64 owns k row r and v row r, thread 64 + t owns q row t
  {
    const int t = tid & 63;
    const bool is_q = tid >= 64;
    const long long row = (((long long)b * p.T + t0 + t) * p.H + h) * DR_D;
    const uint4* src = reinterpret_cast<const uint4*>((is_q ? p.q : p.k) + row);
    uint4 raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) raw[i] = src[i];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float f[8];
      unpack8(raw[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    const float rn = (is_q ? p.qscale : 1.f) / fmaxf(sqrtf(ss), 1e-12f);
    const float G = sG[t], be = sBeta[t];
    const float eG = ex2_fast(G * kLog2e);
    const float eEnd = ex2_fast((g_end - G) * kLog2e);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float f[8];
      unpack8(raw[i], f);
      *reinterpret_cast<uint4*>(smem + S::kKQ + off128(tid, i * 8)) = pack8(f, rn);
      if (is_q) {
        *reinterpret_cast<uint4*>(sRec + DR_QD + off64(t, i * 8)) = pack8(f, rn * eG);
      } else {
        *reinterpret_cast<uint4*>(smem + S::kKB + off64(t, i * 8)) = pack8(f, rn * be * eG);
        *reinterpret_cast<uint4*>(sRec + DR_KE + off64(t, i * 8)) = pack8(f, rn * eEnd);
      }
    }
    if (!is_q) {
      const uint4* vs = reinterpret_cast<const uint4*>(p.v + row);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float f[8];
        unpack8(vs[i], f);
        *reinterpret_cast<uint4*>(smem + S::kVB + off64(t, i * 8)) = pack8(f, be);
      }
    }
  }
  fence_proxy_async_smem();
  __syncthreads();

  // ---- gram blocks: D[128 x 64] = [K; Q] K^T
  if (tid == 0) {
    tc_fence_after();
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 0);
    const uint32_t sKQ = smem_u32(smem + S::kKQ);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t d = umma_smem_desc(sKQ + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
      umma_bf16_ss(tmem_base, d, d, idesc, kk != 0);
    }
    umma_commit(bar);
  }
  bool ok = mbar_wait(bar, 0, abort_word);
  ok = __syncthreads_and(ok);
  tc_fence_after();
  const uint32_t lane_off = uint32_t(warp * 32) << 16;
  if (ok) {
    uint32_t d[2][32];
    tmem_ld_32x32(tmem_base + lane_off, d[0]);
    tmem_ld_32x32(tmem_base + lane_off + 32, d[1]);
    tmem_ld_wait();
    if (tid < 64) {
      const float Gr = sG[tid], be = sBeta[tid];
#pragma unroll
      for (int s = 0; s < 64; ++s) {
        const float val = be * __uint_as_float(d[s >> 5][s & 31]) * ex2_fast((Gr - sG[s]) * kLog2e);
        sA[tid * 68 + s] = s < tid ? val : 0.f;
      }
    } else {
      const int t = tid - 64;
      const float Gt = sG[t];
#pragma unroll
      for (int gq = 0; gq < 8; ++gq) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int s = gq * 8 + j;
          f[j] = s <= t ? __uint_as_float(d[s >> 5][s & 31]) * ex2_fast((Gt - sG[s]) * kLog2e) : 0.f;
        }
        *reinterpret_cast<uint4*>(sRec + DR_AQ + t * 128 + ((gq ^ (t & 7)) << 4)) = pack8(f, 1.f);
      }
    }
  }
  __syncthreads();

  // ---- T = (I + A)^-1 : thread c < 64 solves column c by forward substitution
  if (ok && tid < 64) {
    float x[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      float a0 = (i == tid) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float* arow = sA + i * 68;
#pragma unroll
      for (int j = 0; j + 3 < i; j += 4) {
        const float4 a = *reinterpret_cast<const float4*>(arow + j);
        a0 -= a.x * x[j];
        a1 -= a.y * x[j + 1];
        a2 -= a.z * x[j + 2];
        a3 -= a.w * x[j + 3];
      }
#pragma unroll
      for (int j = i & ~3; j < i; ++j) a0 -= arow[j] * x[j];
      x[i] = (a0 + a1) + (a2 + a3);
    }
    uint8_t* sT = smem + S::kT;
#pragma unroll
    for (int i = 0; i < 64; ++i)
      *reinterpret_cast<__nv_bfloat16*>(sT + i * 128 + ((((tid >> 3) ^ (i & 7))) << 4) + (tid & 7) * 2) =
          __float2bfloat16(x[i]);
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- W^T = (beta k e^G)^T T^T and U^T = (beta v)^T T^T, both [128 x 64]
  if (ok && tid == 0) {
    tc_fence_after();
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 1, 0);
    const uint32_t sT = smem_u32(smem + S::kT), sKB = smem_u32(smem + S::kKB), sVB = smem_u32(smem + S::kVB);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma_bf16_ss(tmem_base + 64, umma_smem_desc(sKB + kk * 2048, 8192, 1024), umma_smem_desc(sT + kk * 32, 16, 1024),
                   idesc, kk != 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma_bf16_ss(tmem_base + 128, umma_smem_desc(sVB + kk * 2048, 8192, 1024), umma_smem_desc(sT + kk * 32, 16, 1024),
                   idesc, kk != 0);
    umma_commit(bar);
  }
  if (ok) ok = mbar_wait(bar, 1, abort_word);
  ok = __syncthreads_and(ok);
  tc_fence_after();
  if (ok) {
    uint32_t d[2][32];
    tmem_ld_32x32(tmem_base + lane_off + 64, d[0]);
    tmem_ld_32x32(tmem_base + lane_off + 96, d[1]);
    tmem_ld_wait();
#pragma unroll
    for (int t = 0; t < 64; ++t)
      *reinterpret_cast<__nv_bfloat16*>(sRec + DR_W + off64(t, tid)) = __float2bfloat16(__uint_as_float(d[t >> 5][t & 31]));
    tmem_ld_32x32(tmem_base + lane_off + 128, d[0]);
    tmem_ld_32x32(tmem_base + lane_off + 160, d[1]);
    tmem_ld_wait();
#pragma unroll
    for (int t = 0; t < 64; ++t)
      *reinterpret_cast<__nv_bfloat16*>(sRec + DR_U + t * 256 + tid * 2) = __float2bfloat16(__uint_as_float(d[t >> 5][t & 31]));
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && ok) {
    const long long idx = ((long long)b * p.H + h) * p.chunks + chunk;
    dr_bulk_store(p.rec + idx * DR_REC, sRec, DR_REC);
    tma_store_commit();
    p.eg[idx] = ex2_fast(g_end * kLog2e);
    tma_store_wait0();
  }
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (tid == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

struct DeltaScanParams {
  const uint8_t* rec;     // [B, H, chunks, DR_REC]
  const float* eg;        // [B, H, chunks]
  __nv_bfloat16* o;       // [B, T, H, 128]
  const float* s0;        // optional initial state [B, H, 128(k), 128(v)]
  float* s_out;           // optional final state, same layout
  int B, T, H, chunks;
  int* status;
};

struct DeltaScanSmem {
  static constexpr int kStage = 0;                     // 2 x 72 KB
  static constexpr int kS = 2 * DR_REC;                // 32 KB: S^T bf16 [v][k], K-major, 128-row blocks
  static constexpr int kU = kS + 32768;                // 16 KB: u^T bf16 [v][c], K-major
  static constexpr int kBar = kU + 16384;
  static constexpr int kTotal = kBar + 128 + 1024;
};

constexpr int DS_THREADS = 160;   // warps 0..3: value rows (TMEM lanes); warp 4: record loader

__global__ void __launch_bounds__(DS_THREADS, 1)
delta_scan_kernel(const DeltaScanParams p) {
  using S = DeltaScanSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* full = bars;          // [2]
  uint64_t* empty = bars + 2;     // [2]
  uint64_t* mma_bar = bars + 4;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const long long bh = (long long)b * p.H + h;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(mma_bar, 1);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tS = tmem_base, tUT = tmem_base + 128, tOT = tmem_base + 192;

  if (warp == 4) {
    if (lane == 0) {
      for (int c = 0; c < p.chunks; ++c) {
        const int st = c & 1;
        if (!mbar_wait(&empty[st], ((c >> 1) & 1) ^ 1u, abort_word)) break;
        mbar_expect_tx(&full[st], DR_REC);
        dr_bulk_load(smem + S::kStage + st * DR_REC, p.rec + (bh * p.chunks + c) * DR_REC, DR_REC, &full[st]);
      }
    }
  } else {
    const int v = tid;                                  // value channel = TMEM lane
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    // initial state
    {
      uint32_t z[32];
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          z[i] = p.s0 ? __float_as_uint(p.s0[(bh * DR_D + qd * 32 + i) * DR_D + v]) : 0u;
        tmem_st_32x32(tS + lane_off + qd * 32, z);
      }
      tmem_st_wait();
    }
    uint8_t* sS = smem + S::kS;
    uint8_t* sU = smem + S::kU;
    bool ok = true;
#pragma unroll 1
    for (int c = 0; c < p.chunks; ++c) {
      const int st = c & 1;
      uint8_t* rec = smem + S::kStage + st * DR_REC;
      ok = bar_and(1, 128, mbar_wait(&full[st], (c >> 1) & 1, abort_word));
      if (!ok) break;
      const float e = p.eg[bh * p.chunks + c];
      // (a) state -> bf16 operand in shared memory; TMEM copy decays by e^{G_C}
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t s[32];
        tmem_ld_32x32(tS + lane_off + qd * 32, s);
        tmem_ld_wait();
        uint8_t* line = sS + (qd >> 1) * 16384 + v * 128;
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          uint4 u;
          u.x = pack_bf16(__uint_as_float(s[8 * gq + 0]), __uint_as_float(s[8 * gq + 1]));
          u.y = pack_bf16(__uint_as_float(s[8 * gq + 2]), __uint_as_float(s[8 * gq + 3]));
          u.z = pack_bf16(__uint_as_float(s[8 * gq + 4]), __uint_as_float(s[8 * gq + 5]));
          u.w = pack_bf16(__uint_as_float(s[8 * gq + 6]), __uint_as_float(s[8 * gq + 7]));
          *reinterpret_cast<uint4*>(line + ((((qd & 1) * 4 + gq) ^ (v & 7)) << 4)) = u;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = __float_as_uint(__uint_as_float(s[i]) * e);
        tmem_st_32x32(tS + lane_off + qd * 32, s);
      }
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      bar_and(1, 128, true);
      // (b) u^T = -S^T W^T (the sign is applied when U is added) and o^T = S^T qd^T
      if (tid == 0) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 0);
        const uint32_t aS = smem_u32(sS), bW = smem_u32(rec + DR_W), bQ = smem_u32(rec + DR_QD);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ss(tUT, umma_smem_desc(aS + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                       umma_smem_desc(bW + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc, kk != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ss(tOT, umma_smem_desc(aS + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                       umma_smem_desc(bQ + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc, kk != 0);
        umma_commit(mma_bar);
      }
      ok = bar_and(1, 128, mbar_wait(mma_bar, 0, abort_word));
      if (!ok) break;
      tc_fence_after();
      // (c) u = U - W S, as a bf16 operand [v][c]
      {
        uint32_t d[2][32];
        tmem_ld_32x32(tUT + lane_off, d[0]);
        tmem_ld_32x32(tUT + lane_off + 32, d[1]);
        tmem_ld_wait();
        const __nv_bfloat16* U = reinterpret_cast<const __nv_bfloat16*>(rec + DR_U);
#pragma unroll
        for (int gq = 0; gq < 8; ++gq) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int cc = gq * 8 + j;
            f[j] = __bfloat162float(U[cc * DR_D + v]) - __uint_as_float(d[cc >> 5][cc & 31]);
          }
          *reinterpret_cast<uint4*>(sU + v * 128 + ((gq ^ (v & 7)) << 4)) = pack8(f, 1.f);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      bar_and(1, 128, true);
      // (d) o^T += u^T Aq^T ;  S^T += u^T kend
      if (tid == 0) {
        tc_fence_after();
        constexpr uint32_t idesc_o = umma_idesc_bf16(128, 64, 0, 0);
        constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 1);
        const uint32_t aU = smem_u32(sU), bA = smem_u32(rec + DR_AQ), bK = smem_u32(rec + DR_KE);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ss(tOT, umma_smem_desc(aU + kk * 32, 16, 1024), umma_smem_desc(bA + kk * 32, 16, 1024), idesc_o, 1u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ss(tS, umma_smem_desc(aU + kk * 32, 16, 1024), umma_smem_desc(bK + kk * 2048, 8192, 1024), idesc_s, 1u);
        umma_commit(mma_bar);
        umma_commit(&empty[st]);
      }
      ok = bar_and(1, 128, mbar_wait(mma_bar, 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      // (e) o[t][v]
      {
        uint32_t d[2][32];
        tmem_ld_32x32(tOT + lane_off, d[0]);
        tmem_ld_32x32(tOT + lane_off + 32, d[1]);
        tmem_ld_wait();
        __nv_bfloat16* orow = p.o + (((long long)b * p.T + (long long)c * DR_C) * p.H + h) * DR_D + v;
#pragma unroll
        for (int t = 0; t < 64; ++t)
          orow[(long long)t * p.H * DR_D] = __float2bfloat16(__uint_as_float(d[t >> 5][t & 31]));
      }
      tc_fence_before();
    }
    if (ok && p.s_out) {
      tc_fence_after();
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t s[32];
        tmem_ld_32x32(tS + lane_off + qd * 32, s);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) p.s_out[(bh * DR_D + qd * 32 + i) * DR_D + v] = __uint_as_float(s[i]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (tid == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

}  // namespace nga

extern "C" long long nga_gdn_workspace_bytes(int B, int T, int H) {
  const long long chunks = T / nga::DR_C;
  return (long long)B * H * chunks * nga::DR_REC + (long long)B * H * chunks * 4 + 256;
}

// q, k, v: [B, T, H, 128] bf16 (q, k not yet normalised); g (log-decay <= 0), beta: [B, T, H] fp32;
// o: [B, T, H, 128] bf16; s0 / s_out: optional [B, H, 128, 128] fp32 states; T a multiple of 64.
extern "C" int nga_gdn_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o,
                           const float* s0, float* s_out, void* workspace, int B, int T, int H, int D, int* status,
                           void* stream) {
  using namespace nga;
  if (D != DR_D || B <= 0 || H <= 0 || T <= 0 || (T % DR_C)) return -1;
  const int chunks = T / DR_C;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DeltaPrepSmem::kTotal);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DeltaScanSmem::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    attr_done = true;
  }
  uint8_t* rec = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  float* eg = reinterpret_cast<float*>(rec + (long long)B * H * chunks * DR_REC);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DeltaPrepParams pp;
  pp.q = reinterpret_cast<const __nv_bfloat16*>(q);
  pp.k = reinterpret_cast<const __nv_bfloat16*>(k);
  pp.v = reinterpret_cast<const __nv_bfloat16*>(v);
  pp.g = g; pp.beta = beta; pp.rec = rec; pp.eg = eg;
  pp.B = B; pp.T = T; pp.H = H; pp.chunks = chunks;
  pp.qscale = 0.08838834764831845f;                    // 128^-0.5
  pp.status = status;
  delta_prep_kernel<<<dim3(chunks, H, B), 128, DeltaPrepSmem::kTotal, st>>>(pp);
  count_launch();
  NGA_CHECK_LAUNCH();
  DeltaScanParams sp;
  sp.rec = rec; sp.eg = eg; sp.o = reinterpret_cast<__nv_bfloat16*>(o); sp.s0 = s0; sp.s_out = s_out;
  sp.B = B; sp.T = T; sp.H = H; sp.chunks = chunks; sp.status = status;
  delta_scan_kernel<<<dim3(H, B), DS_THREADS, DeltaScanSmem::kTotal, st>>>(sp);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
