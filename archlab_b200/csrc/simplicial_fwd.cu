// 2-simplicial (trilinear) windowed attention, forward, on tcgen05 + TMEM.  head_dim 128,
// short window w1 in {8, 16, 32}, long window w2 >= w1.
//
//   s[i; j, k] = scale * sum_d q[i,d] k1[j,d] k2[k,d],   j in (i-w1, i], k in (i-w2, i]
//   p = softmax over ALL valid (j, k) pairs;   out[i] = sum_{j,k} p[j,k] * (v1[j] * v2[k])
// (src/archlab/architectures/simplicial_attention.py:49-74; incumbents: Triton
// simplicial_kernels.py:16-52, TileLang tilelang_attention.py:25-129.)
//
// The short axis is folded into the GEMM M dimension: a CTA owns BQ = 128 / w1 consecutive queries
// and its 128 rows are the (query, short key) pairs.  Row (i, j) of the A operand is q[i] * k1[j]
// (built once by the CUDA cores into a 128B-swizzled tile), so per 128-key tile of the long window
//   S = A K2^T   and   O_pair += P V2
// are plain 128x128x128 tensor-core products; the joint softmax only needs the row statistics to be
// combined across the w1 lanes of a query (warp shuffles), and the output is
//   out[i] = (1 / l_i) * sum_j v1[j] * O_pair[(i, j)].
// Roles: warp 0 TMA producer (K2 / V2 ring), warp 1 MMA issuer, warps 2..5 softmax + epilogue.
#include "ptx.cuh"
#include "host_util.h"
#include "simplicial.h"
#include <cuda.h>
#include <cstdlib>

namespace nga {

constexpr int SX_D = 128;
constexpr int SX_BK = 128;
constexpr int SX_TILE = 128 * 128 * 2;
constexpr int SX_THREADS = 192;

struct SimpFwdParams {
  const __nv_bfloat16* q;    // [B*N, ldq] rows, head h at column h*D
  const __nv_bfloat16* k1;
  const __nv_bfloat16* v1;
  __nv_bfloat16* out;        // [B*N, ldo]
  float* lse2;               // [B, Hq, N]
  long long ldq, ldk1, ldv1, ldo;
  int B, N, Hq, Hkv, w1, w2;
  float scale_log2;
  int* status;
  long long* prof;           // optional phase cycle counters written by one mid-grid CTA (tuning aid)
  // decode mode: one new token per sequence against paged caches (page = 128 positions = one key tile)
  const int* block_table;    // [B, max_pages] physical page of every logical page
  const int* seq_lens;       // [B] tokens in the cache including the new one
  int max_pages;
  int p_tmem;                // 1: P returns to the tensor core through TMEM (A operand of P V2)
};

struct SimpFwdSmem {
  static constexpr int kA = 0;
  static constexpr int kK = SX_TILE;
  static constexpr int kV = kK + 2 * SX_TILE;
  static constexpr int kP = kV + 2 * SX_TILE;
  static constexpr int kBar = kP + SX_TILE;
  static constexpr int kTotal = kBar + 16 * 8 + 16 + 1024;
};

// Barrier of the 128 softmax threads that ANDs a predicate.
__device__ __forceinline__ bool sx_bar_and(bool pred) {
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
__device__ __forceinline__ float seg_max(float v, int w1) {
  for (int o = 1; o < w1; o <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float seg_sum(float v, int w1) {
  for (int o = 1; o < w1; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// DECODE = false: a CTA owns 128 / w1 consecutive queries of one head (prefill / training forward).
// DECODE = true : a CTA owns the newest token of one sequence for the Hq / Hkv query heads that share a
//                 KV head; its rows are (query head, short key), keys come from paged caches.
template <bool DECODE>
__global__ void __launch_bounds__(SX_THREADS, 1)
simplicial_fwd_kernel(const __grid_constant__ CUtensorMap tm_k2, const __grid_constant__ CUtensorMap tm_v2,
                      const SimpFwdParams p) {
  using S = SimpFwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* a_full = bars + 0;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* s_full = bars + 5;
  uint64_t* s_free = bars + 7;
  uint64_t* p_full = bars + 9;
  uint64_t* p_empty = bars + 10;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool prof = p.prof != nullptr && blockIdx.x == gridDim.x / 2 && blockIdx.y == 0 && blockIdx.z == 0 &&
                    warp == 2 && lane == 0;
  long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long pt0 = prof ? clock64() : 0;
  const int G = p.Hq / p.Hkv;
  const int BQ = DECODE ? G : 128 / p.w1;
  const int b = blockIdx.z;
  const int pos_last = DECODE ? p.seq_lens[b] - 1 : 0;
  const int i0 = DECODE ? pos_last : blockIdx.x * BQ;
  const int h = blockIdx.y;                       // query head (prefill) or KV head (decode)
  const int hk = DECODE ? h : h / G;
  const int row_base = DECODE ? 0 : b * p.N;
  const int i_last = DECODE ? pos_last : min(i0 + BQ - 1, p.N - 1);
  const int* pages = DECODE ? p.block_table + (long long)b * p.max_pages : nullptr;
  const int t_lo = max(0, i0 - p.w2 + 1) / SX_BK;
  const int t_hi = i_last / SX_BK;
  const int ntiles = t_hi - t_lo + 1;
  const int kv_col = hk * SX_D;

  if (threadIdx.x == 0) {
    mbar_init(a_full, 4);
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
  const uint32_t tmem_S0 = tmem_base;
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k2);
      tma_prefetch_desc(&tm_v2);
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j & 1;
        ok = mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1u, abort_word);
        if (!ok) break;
        const int krow = DECODE ? pages[t_lo + j] * SX_BK : row_base + (t_lo + j) * SX_BK;
        uint8_t* sK = smem + S::kK + st * SX_TILE;
        uint8_t* sV = smem + S::kV + st * SX_TILE;
        mbar_expect_tx(&kv_full[st], 2 * SX_TILE);
        tma_load_3d(sK, &tm_k2, &kv_full[st], kv_col, krow, 0);
        tma_load_3d(sK + 16384, &tm_k2, &kv_full[st], kv_col + 64, krow, 0);
        tma_load_3d(sV, &tm_v2, &kv_full[st], kv_col, krow, 0);
        tma_load_3d(sV + 16384, &tm_v2, &kv_full[st], kv_col + 64, krow, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t sA = smem_u32(smem + S::kA);
      const uint32_t sP = smem_u32(smem + S::kP);
      bool ok = mbar_wait(a_full, 0, abort_word);
      auto issue_s = [&](int j) {
        const uint32_t sK = smem_u32(smem + S::kK + (j & 1) * SX_TILE);
        const uint32_t d = tmem_S0 + uint32_t((j & 1) * 128);
#pragma unroll
        for (int k = 0; k < SX_D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16_ss(d, umma_smem_desc(sA + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          const int jn = j + 1;
          ok = mbar_wait(&kv_full[jn & 1], (jn >> 1) & 1, abort_word);
          if (ok) ok = mbar_wait(&s_free[jn & 1], ((jn >> 1) & 1) ^ 1u, abort_word);
          if (!ok) break;
          tc_fence_after();
          issue_s(jn);
        }
        ok = mbar_wait(p_full, j & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sV = smem_u32(smem + S::kV + (j & 1) * SX_TILE);
#pragma unroll
        for (int k = 0; k < SX_BK / 16; ++k) {
          const uint64_t db = umma_smem_desc(sV + k * 2048, 16384, 1024);
          if (p.p_tmem) {
            umma_bf16_ts(tmem_O, tmem_S0 + uint32_t((j & 1) * 128 + k * 8), db, idesc_pv, (j | k) != 0 ? 1u : 0u);
          } else {
            const uint64_t da = umma_smem_desc(sP + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
            umma_bf16_ss(tmem_O, da, db, idesc_pv, (j | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&kv_empty[j & 1]);
        umma_commit(p_empty);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: row = (query, short key)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qi = r / p.w1, jj = r % p.w1;
    const int i = DECODE ? pos_last : i0 + qi;   // query position
    const int head = DECODE ? hk * G + qi : h;   // query head of this row
    const int p1 = i - p.w1 + 1 + jj;            // short-key position of this row
    const bool row_valid = DECODE ? (qi < G && p1 >= 0) : ((i < p.N) && (p1 >= 0));
    // row of the short key / value in its tensor (paged in decode mode)
    const long long short_row = DECODE ? (long long)pages[max(p1, 0) >> 7] * SX_BK + (max(p1, 0) & 127)
                                       : (long long)(row_base + max(p1, 0));
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    if (prof) pc[0] = clock64() - pt0;             // setup (barriers, TMEM allocation)
    long long pt = prof ? clock64() : 0;
    // ---- build this row of A = q[i] * k1[p1] into the swizzled tile
    {
      const __nv_bfloat16* qrow = DECODE ? p.q + (long long)b * p.ldq + min(head, p.Hq - 1) * SX_D
                                         : p.q + (long long)(row_base + min(i, p.N - 1)) * p.ldq + h * SX_D;
      const __nv_bfloat16* krow = p.k1 + short_row * p.ldk1 + hk * SX_D;
      uint8_t* sA = smem + S::kA;
      // loads of a half row first, then the packed products (bf16 x bf16 rounded to bf16 equals the fp32
      // product rounded once): a generic shared store between two global loads would serialise every
      // chunk on the L2 latency
      uint4 qa[16], ka[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        qa[c] = row_valid ? *reinterpret_cast<const uint4*>(qrow + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        ka[c] = row_valid ? *reinterpret_cast<const uint4*>(krow + c * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 o;
        const __nv_bfloat162* qh = reinterpret_cast<const __nv_bfloat162*>(&qa[c]);
        const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&ka[c]);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __hmul2(qh[e], kh[e]);
        *reinterpret_cast<uint4*>(sA + (c >> 3) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) * 16)) = o;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_full);
    }
    if (prof) { const long long n = clock64(); pc[1] = n - pt; pt = n; }   // A build
    float m_ref = -INFINITY, l_row = 0.f;
    bool ok = true;
    uint8_t* sP = smem + S::kP;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int k0 = (t_lo + j) * SX_BK;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      if (prof) { const long long n = clock64(); pc[2] += n - pt; pt = n; }   // wait for S
      const uint32_t tS = tmem_S0 + uint32_t((j & 1) * 128) + lane_off;
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + c * 32, sv[c]);
      tmem_ld_wait();
      if (prof) { const long long n = clock64(); pc[3] += n - pt; pt = n; }   // TMEM load
      // visibility of long key pos2 = k0 + col for this row: i - w2 < pos2 <= i
      const int lo = i - p.w2 + 1 - k0, hi = i - k0;      // valid columns are [lo, hi]
      const bool full = row_valid && lo <= 0 && hi >= SX_BK - 1;
      if (!full) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            if (!row_valid || col < lo || col > hi) sv[c][e] = 0xff800000u;
          }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 32; ++e) mx4[c] = fmaxf(mx4[c], __uint_as_float(sv[c][e]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      mx = seg_max(mx, p.w1);                    // joint over the query's short keys
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (j - 1) & 1, abort_word));
        if (!ok) break;
        tc_fence_after();
      }
      if (prof) { const long long n = clock64(); pc[4] += n - pt; pt = n; }   // mask + max + wait for the P buffer
      const float m_new = fmaxf(m_ref, mx);
      const bool grow = (m_new > m_ref + 8.f) || (m_ref == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_use = grow ? m_new : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_use);
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_O + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x32(tmem_O + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
        l_row *= alpha;
        m_ref = m_use;
      }
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pr[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pr[e]) : "f"(fmaf(__uint_as_float(sv[c][e]), p.scale_log2, -m_sub)));
          ps4[e & 3] += pr[e];
        }
        if (p.p_tmem) {
          uint32_t pk[16];
#pragma unroll
          for (int g = 0; g < 16; ++g) pk[g] = pack_bf16(pr[2 * g], pr[2 * g + 1]);
          tmem_st_32x16(tS + c * 16, pk);
        } else {
          uint8_t* line = sP + (c >> 1) * 16384 + r * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = ((c & 1) * 4 + g) ^ (r & 7);
            uint4 u;
            u.x = pack_bf16(pr[8 * g + 0], pr[8 * g + 1]);
            u.y = pack_bf16(pr[8 * g + 2], pr[8 * g + 3]);
            u.z = pack_bf16(pr[8 * g + 4], pr[8 * g + 5]);
            u.w = pack_bf16(pr[8 * g + 6], pr[8 * g + 7]);
            *reinterpret_cast<uint4*>(line + chunk * 16) = u;
          }
        }
      }
      if (p.p_tmem) tmem_st_wait();
      l_row += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_free[j & 1]);
        mbar_arrive(p_full);
      }
      if (prof) { const long long n = clock64(); pc[5] += n - pt; pt = n; }   // rescale + exp + P store
    }
    // ---------------------------------------------------------------- epilogue
    // this row's v1 values are fetched while the last P V2 product is still running
    const __nv_bfloat16* v1row = p.v1 + short_row * p.ldv1 + hk * SX_D;
    uint4 vv[16];
#pragma unroll
    for (int g = 0; g < 16; ++g)
      vv[g] = row_valid ? *reinterpret_cast<const uint4*>(v1row + g * 8) : make_uint4(0u, 0u, 0u, 0u);
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (ntiles - 1) & 1, abort_word));
    ok = sx_bar_and(ok);                        // the four softmax warps agree before sharing a barrier
    if (ok) {
      tc_fence_after();
      const float l_q = seg_sum(l_row, p.w1);
      const float inv = l_q > 0.f ? 1.f / l_q : 0.f;
      // The K2 / V2 / P buffers are idle now: each row leaves inv * O_pair[row] * v1[row] there in fp32
      // (row stride 132 floats keeps the 16-byte stores of a quarter warp on distinct banks), then thread t
      // adds the w1 rows of every query for column t.  (A shuffle reduction would serialise 640 dependent
      // shuffles per thread.)
      float* red = reinterpret_cast<float*>(smem + S::kK);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vv[c * 4 + g]);
          float4 lo, hi;
          float2 f = __bfloat1622float2(vh[0]);
          lo.x = __uint_as_float(v[g * 8 + 0]) * f.x * inv;
          lo.y = __uint_as_float(v[g * 8 + 1]) * f.y * inv;
          f = __bfloat1622float2(vh[1]);
          lo.z = __uint_as_float(v[g * 8 + 2]) * f.x * inv;
          lo.w = __uint_as_float(v[g * 8 + 3]) * f.y * inv;
          f = __bfloat1622float2(vh[2]);
          hi.x = __uint_as_float(v[g * 8 + 4]) * f.x * inv;
          hi.y = __uint_as_float(v[g * 8 + 5]) * f.y * inv;
          f = __bfloat1622float2(vh[3]);
          hi.z = __uint_as_float(v[g * 8 + 6]) * f.x * inv;
          hi.w = __uint_as_float(v[g * 8 + 7]) * f.y * inv;
          *reinterpret_cast<float4*>(red + r * 132 + c * 32 + g * 8) = lo;
          *reinterpret_cast<float4*>(red + r * 132 + c * 32 + g * 8 + 4) = hi;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int qq = 0; qq < BQ && (qq + 1) * p.w1 <= 128; ++qq) {
        const int iq = i0 + qq;
        if (!DECODE && iq >= p.N) break;
        float a0 = 0.f, a1 = 0.f;
        const float* col = red + (qq * p.w1) * 132 + r;
        for (int x = 0; x < p.w1; x += 2) {
          a0 += col[x * 132];
          a1 += col[(x + 1) * 132];
        }
        const long long o = DECODE ? (long long)b * p.ldo + (hk * G + qq) * SX_D + r
                                   : (long long)(row_base + iq) * p.ldo + h * SX_D + r;
        p.out[o] = __float2bfloat16(a0 + a1);
      }
      if (DECODE) {
        if (jj == 0 && qi < G) p.lse2[(long long)b * p.Hq + head] = m_ref + log2f(l_q);
      } else if (jj == 0 && i < p.N) {
        p.lse2[((long long)b * p.Hq + h) * p.N + i] = m_ref + log2f(l_q);
      }
    }
    if (prof) {
      pc[6] = clock64() - pt;                      // last PV wait + epilogue
      pc[7] = ntiles;
      for (int x = 0; x < 8; ++x) p.prof[x] = pc[x];
      p.prof[8] = clock64() - pt0;
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

static int simp_p_tmem() {                         // NGA_SIMP_P_TMEM=1 selects the TMEM route for P
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("NGA_SIMP_P_TMEM");
    v = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return v;
}
static long long* g_simp_fwd_prof = nullptr;
extern "C" void nga_simplicial_fwd_set_prof(long long* device_ptr) { g_simp_fwd_prof = device_ptr; }

extern "C" int nga_simplicial_fwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                                  void* out, float* lse2, long long ldq, long long ldk1, long long ldk2,
                                  long long ldv1, long long ldv2, long long ldo, int B, int N, int Hq, int Hkv,
                                  int D, int w1, int w2, float scale, int* status, void* stream) {
  using namespace nga;
  if (D != SX_D || B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  if (!(w1 == 8 || w1 == 16 || w1 == 32) || w2 < w1) return -6;
  if ((ldq | ldk1 | ldk2 | ldv1 | ldv2 | ldo) & 7) return -5;
  const long long rows = (long long)B * N;
  CUtensorMap tk, tv;
  int rc = make_tmap_3d(&tk, k2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)Hkv * D, rows, 1, ldk2 * 2,
                        rows * ldk2 * 2, 64, 128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tv, v2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)Hkv * D, rows, 1, ldv2 * 2,
                    rows * ldv2 * 2, 64, 128, true);
  if (rc) return rc;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(simplicial_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SimpFwdSmem::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    attr_done = true;
  }
  SimpFwdParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k1 = reinterpret_cast<const __nv_bfloat16*>(k1);
  p.v1 = reinterpret_cast<const __nv_bfloat16*>(v1);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse2 = lse2;
  p.ldq = ldq; p.ldk1 = ldk1; p.ldv1 = ldv1; p.ldo = ldo;
  p.B = B; p.N = N; p.Hq = Hq; p.Hkv = Hkv; p.w1 = w1; p.w2 = w2;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.prof = g_simp_fwd_prof;
  p.block_table = nullptr; p.seq_lens = nullptr; p.max_pages = 0;
  p.p_tmem = simp_p_tmem();
  const int BQ = 128 / w1;
  dim3 grid((N + BQ - 1) / BQ, Hq, B);
  simplicial_fwd_kernel<false><<<grid, SX_THREADS, SimpFwdSmem::kTotal, reinterpret_cast<cudaStream_t>(stream)>>>(tk, tv, p);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

// One new token per sequence against paged caches.  q: [B, Hq*D]; caches: [num_pages * 128, Hkv*D] bf16 (page p
// holds rows p*128 .. p*128+127); block_table [B, max_pages] int32; seq_lens [B] int32 (cache length including
// the new token, whose k1/k2/v1/v2 are already written); out [B, Hq*D]; lse2 [B, Hq].
// Requires (Hq / Hkv) * w1 <= 128.
extern "C" int nga_simplicial_decode(const void* q, const void* k1c, const void* k2c, const void* v1c, const void* v2c,
                                     void* out, float* lse2, const int* block_table, const int* seq_lens, long long ldq,
                                     long long ldc, long long ldo, int B, int Hq, int Hkv, int D, int w1, int w2,
                                     int max_pages, int num_pages, float scale, int* status, void* stream) {
  using namespace nga;
  if (D != SX_D || B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || num_pages <= 0 || max_pages <= 0) return -1;
  if (!(w1 == 8 || w1 == 16 || w1 == 32) || w2 < w1 || (Hq / Hkv) * w1 > 128) return -6;
  if ((ldq | ldc | ldo) & 7) return -5;
  const long long rows = (long long)num_pages * SX_BK;
  CUtensorMap tk, tv;
  int rc = make_tmap_3d(&tk, k2c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)Hkv * D, rows, 1, ldc * 2, rows * ldc * 2,
                        64, 128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tv, v2c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)Hkv * D, rows, 1, ldc * 2, rows * ldc * 2, 64, 128,
                    true);
  if (rc) return rc;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(simplicial_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SimpFwdSmem::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    attr_done = true;
  }
  SimpFwdParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k1 = reinterpret_cast<const __nv_bfloat16*>(k1c);
  p.v1 = reinterpret_cast<const __nv_bfloat16*>(v1c);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse2 = lse2;
  p.ldq = ldq; p.ldk1 = ldc; p.ldv1 = ldc; p.ldo = ldo;
  p.B = B; p.N = 1; p.Hq = Hq; p.Hkv = Hkv; p.w1 = w1; p.w2 = w2;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.prof = nullptr;
  p.block_table = block_table; p.seq_lens = seq_lens; p.max_pages = max_pages;
  p.p_tmem = simp_p_tmem();
  simplicial_fwd_kernel<true><<<dim3(1, Hkv, B), SX_THREADS, SimpFwdSmem::kTotal, reinterpret_cast<cudaStream_t>(stream)>>>(tk, tv, p);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
