// Causal / sliding-window GQA attention forward on tcgen05 + TMEM, head_dim 128.
//
// Semantics are those of flash_attn_func(q, k, v, causal=True, window_size=(left, 0)) as used by
// the reference trunk (src/archlab/architectures/base.py:325-333; mask rule in
// src/archlab/speedrun/attention.py:175-181): key j is visible to query i iff j <= i and
// (left < 0 or i - j <= left).  Softmax scale is 1/sqrt(D).
//
// One CTA owns a 128-query tile of one (batch, head).  Roles: warp 0 TMA producer (Q once, then a
// two-stage K/V ring), warp 1 MMA issuer, warps 2..5 softmax (thread = query row = TMEM lane).
// S = Q K^T is double-buffered in TMEM so the next tile's QK^T overlaps this tile's softmax; P goes
// back to the tensor core through shared memory in the canonical 128-byte-swizzled K-major layout;
// O accumulates in TMEM and is rescaled only when a row maximum grows by more than 2^8.
#include "ptx.cuh"
#include "host_util.h"
#include "attention.h"
#include <cuda.h>
#include <cstdlib>
#include <cstdio>

namespace nga {

constexpr int AT_D = 128;
constexpr int AT_BQ = 128;
constexpr int AT_BK = 128;
constexpr int AT_TILE_BYTES = 128 * 128 * 2;  // 32 KB: one 128 x 128 bf16 tile (two 64-wide blocks)
constexpr int AT_THREADS = 192;

struct AttnFwdParams {
  __nv_bfloat16* out;   // [B*T, Hq*D]
  float* lse2;          // [B, Hq, T]  log2-domain log-sum-exp of the scaled scores
  int B, T, Hq, Hkv, window;
  float scale_log2;
  int* status;
  long long* prof;      // optional: 16 cycle counters written by CTA (0,0,0) (phase timing for tuning)
  const uint32_t* sel;  // optional key-selection bits [B, T, T/32] (bit k of row q: query q may see key k)
  const float* sink;    // optional per-head sink logit: adds exp(sink) to every row's softmax denominator
  int p_tmem;           // 1: P goes back to the tensor core through TMEM (A operand of P V), not shared memory
};

struct AttnFwdSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = AT_TILE_BYTES;                 // 2 stages
  static constexpr int kV = kK + 2 * AT_TILE_BYTES;        // 2 stages
  static constexpr int kP = kV + 2 * AT_TILE_BYTES;
  static constexpr int kBar = kP + AT_TILE_BYTES;
  static constexpr int kTotal = kBar + 16 * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnFwdParams p) {
  using S = AttnFwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* s_free = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* p_empty = bars + 10;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qt = (p.T + AT_BQ - 1) / AT_BQ;
  const int qt = num_qt - 1 - blockIdx.x;   // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * AT_BQ;
  const int k_lo = (p.window < 0) ? 0 : max(0, q0 - p.window) / AT_BK;
  const int k_hi = min(q0 + AT_BQ - 1, p.T - 1) / AT_BK;
  const int ntiles = k_hi - k_lo + 1;
  const int row_base = b * p.T;
  const int q_col = h * AT_D;
  const int k_col = (p.Hq + hk) * AT_D;
  const int v_col = (p.Hq + p.Hkv + hk) * AT_D;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
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
  const uint32_t tmem_S0 = tmem_base;            // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 256;       // 128 columns

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm);
      mbar_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_3d(smem + S::kQ, &tm, q_full, q_col, row_base + q0, 0);
      tma_load_3d(smem + S::kQ + 16384, &tm, q_full, q_col + 64, row_base + q0, 0);
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j & 1;
        ok = mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1u, abort_word);
        if (!ok) break;
        const int krow = row_base + (k_lo + j) * AT_BK;
        uint8_t* sK = smem + S::kK + st * AT_TILE_BYTES;
        uint8_t* sV = smem + S::kV + st * AT_TILE_BYTES;
        mbar_expect_tx(&kv_full[st], 2 * AT_TILE_BYTES);
        tma_load_3d(sK, &tm, &kv_full[st], k_col, krow, 0);
        tma_load_3d(sK + 16384, &tm, &kv_full[st], k_col + 64, krow, 0);
        tma_load_3d(sV, &tm, &kv_full[st], v_col, krow, 0);
        tma_load_3d(sV + 16384, &tm, &kv_full[st], v_col + 64, krow, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t sQ = smem_u32(smem + S::kQ);
      const uint32_t sP = smem_u32(smem + S::kP);
      bool ok = mbar_wait(q_full, 0, abort_word);
      auto issue_qk = [&](int j) {
        const uint32_t sK = smem_u32(smem + S::kK + (j & 1) * AT_TILE_BYTES);
        const uint32_t d = tmem_S0 + uint32_t((j & 1) * 128);
#pragma unroll
        for (int k = 0; k < AT_D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16_ss(d, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024),
                       idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          const int jn = j + 1;
          ok = mbar_wait(&kv_full[jn & 1], (jn >> 1) & 1, abort_word);
          if (ok) ok = mbar_wait(&s_free[jn & 1], ((jn >> 1) & 1) ^ 1u, abort_word);
          if (!ok) break;
          tc_fence_after();
          issue_qk(jn);
        }
        ok = mbar_wait(p_full, j & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sV = smem_u32(smem + S::kV + (j & 1) * AT_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < AT_BK / 16; ++k) {
          // A = P: K-major, keys contiguous, two 64-key blocks of 16 KB (or, in TMEM, 8 columns of bf16 pairs
          // per 16 keys inside the S buffer of this tile).
          // B = V: MN-major, rows are keys (128 B = 64 d), the two 64-wide d blocks 16 KB apart.
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
    // ---------------------------------------------------------------- softmax warps
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;           // query row inside the tile
    const int q = q0 + r;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    uint8_t* sP = smem + S::kP;
    const bool prof_on = p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 64;
    long long pc[6] = {0, 0, 0, 0, 0, 0};
    long long tp = clock64();
#define NGA_PROF(i) do { if (prof_on) { long long tn = clock64(); pc[i] += tn - tp; tp = tn; } } while (0)
    for (int j = 0; j < ntiles && ok; ++j) {
      const int k0 = (k_lo + j) * AT_BK;
      const bool need_mask = (k0 + AT_BK - 1 > q0) || (p.window >= 0 && q0 + AT_BQ - 1 - k0 > p.window);
      uint4 selw = make_uint4(~0u, ~0u, ~0u, ~0u);            // fetched before the wait for S
      if (p.sel != nullptr && q < p.T)
        selw = *reinterpret_cast<const uint4*>(p.sel + ((long long)b * p.T + q) * (p.T >> 5) + (k0 >> 5));
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_word));
      if (!ok) break;
      NGA_PROF(0);
      tc_fence_after();
      const uint32_t tS = tmem_S0 + uint32_t((j & 1) * 128) + lane_off;
      // The whole 128-column row goes to registers with four back-to-back loads and ONE wait, so
      // the TMEM read latency is paid once per tile instead of once per 32 columns.
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + c * 32, sv[c]);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = k0 + c * 32 + i;
            if (key > q || (p.window >= 0 && q - key > p.window)) sv[c][i] = 0xff800000u;  // -inf
          }
      }
      if (p.sel != nullptr) {
        const uint32_t w4[4] = {selw.x, selw.y, selw.z, selw.w};
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!((w4[c] >> i) & 1u)) sv[c][i] = 0xff800000u;
      }
      // row maximum with four independent chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[c] = fmaxf(mx4[c], __uint_as_float(sv[c][i]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      NGA_PROF(1);
      // P buffer and O are free once the previous PV has completed
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (j - 1) & 1, abort_word));
        if (!ok) break;
        tc_fence_after();
      }
      NGA_PROF(2);
      const float m_new = fmaxf(m_ref, mx);
      const bool grow = (m_new > m_ref + 8.f) || (m_ref == -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        // rows of this warp rescale together (the TMEM accesses are warp-collective)
        const float m_use = grow ? m_new : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_use);
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_O + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_O + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_ref = m_use;
      }
      NGA_PROF(3);
      // probabilities -> bf16 -> swizzled shared memory (masked entries are exp2(-inf) = 0)
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          pr[i] = ex2_fast(fmaf(__uint_as_float(sv[c][i]), p.scale_log2, -m_sub));
          ps4[i & 3] += pr[i];
        }
        if (p.p_tmem) {
          // 32 keys = 16 columns of packed pairs, written over the (already consumed) scores of this tile
          uint32_t pk[16];
#pragma unroll
          for (int g = 0; g < 16; ++g) pk[g] = pack_bf16(pr[2 * g], pr[2 * g + 1]);
          tmem_st_32x16(tS + c * 16, pk);
        } else {
          // 32 keys = 64 B = four 16-byte chunks of this row's 128-byte line in key block (c >> 1)
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
      const float psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      l_sum += psum;
      NGA_PROF(4);
      // S buffer consumed; P written
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_free[j & 1]);
        mbar_arrive(p_full);
      }
      NGA_PROF(5);
    }
    if (prof_on) { for (int i = 0; i < 6; ++i) p.prof[i] = pc[i]; p.prof[6] = ntiles; }
    // ---------------------------------------------------------------- epilogue
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (ntiles - 1) & 1, abort_word));
    if (ok) {
      tc_fence_after();
      if (p.sink != nullptr) {                       // the sink takes probability mass but carries no value
        const float s2 = p.sink[h] * 1.4426950408889634f;
        if (m_ref == -INFINITY) {
          m_ref = s2;
          l_sum = 1.f;
        } else {
          l_sum += exp2f(s2 - m_ref);
        }
      }
      const float inv = 1.f / l_sum;
      const bool q_ok = q < p.T;
      __nv_bfloat16* orow = p.out + (long long)(row_base + q) * (p.Hq * AT_D) + q_col;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_off + c * 32, v);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
            u.y = pack_bf16(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
            u.z = pack_bf16(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
            u.w = pack_bf16(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = u;
          }
        }
      }
      if (q_ok) p.lse2[((long long)b * p.Hq + h) * p.T + q] = m_ref + log2f(l_sum);
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


// ---------------------------------------------------------------------------------------------------------------
// Two-CTAs-per-SM form.  Inside a CTA the chain S = Q K^T -> softmax -> O += P V is strictly serial, so one CTA
// leaves the tensor pipe idle while its softmax warps work and the issue slots idle while its MMAs run.  This form
// makes a CTA small enough for two to be resident on an SM (96 KB of shared memory: Q and one stage each of K and V;
// 256 TMEM columns: one S buffer whose consumed scores are overwritten by the packed probabilities, and O), so the
// hardware interleaves two independent chains: one CTA's MMAs run under the other's softmax.  K(j+1) is fetched
// while softmax(j) runs (its buffer is free once Q K^T(j) has completed), V(j+1) after P V(j).  The scores are read
// from TMEM twice (row maximum, then probabilities 32 columns at a time) to stay under 168 registers per thread.
struct AttnFwd2Smem {
  static constexpr int kQ = 0;
  static constexpr int kK = AT_TILE_BYTES;
  static constexpr int kV = 2 * AT_TILE_BYTES;
  static constexpr int kBar = 3 * AT_TILE_BYTES;
  static constexpr int kTotal = kBar + 16 * 8 + 32;       // no alignment slack: two CTAs must fit in 196 KB
};

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm, const AttnFwdParams p) {
  using S = AttnFwd2Smem;
  extern __shared__ __align__(1024) uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn;
  if ((smem_u32(smem) & 1023u) != 0u) {                   // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, 3);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* p_empty = bars + 7;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qt = (p.T + AT_BQ - 1) / AT_BQ;
  const int qt = num_qt - 1 - blockIdx.x;   // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * AT_BQ;
  const int k_lo = (p.window < 0) ? 0 : max(0, q0 - p.window) / AT_BK;
  const int k_hi = min(q0 + AT_BQ - 1, p.T - 1) / AT_BK;
  const int ntiles = k_hi - k_lo + 1;
  const int row_base = b * p.T;
  const int q_col = h * AT_D;
  const int k_col = (p.Hq + hk) * AT_D;
  const int v_col = (p.Hq + p.Hkv + hk) * AT_D;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;             // 128 columns: scores, then packed probabilities in the first 64
  const uint32_t tmem_O = tmem_base + 128;       // 128 columns

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm);
      mbar_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_3d(smem + S::kQ, &tm, q_full, q_col, row_base + q0, 0);
      tma_load_3d(smem + S::kQ + 16384, &tm, q_full, q_col + 64, row_base + q0, 0);
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int krow = row_base + (k_lo + j) * AT_BK;
        ok = mbar_wait(k_empty, (j & 1) ^ 1u, abort_word);
        if (!ok) break;
        mbar_expect_tx(k_full, AT_TILE_BYTES);
        tma_load_3d(smem + S::kK, &tm, k_full, k_col, krow, 0);
        tma_load_3d(smem + S::kK + 16384, &tm, k_full, k_col + 64, krow, 0);
        ok = mbar_wait(v_empty, (j & 1) ^ 1u, abort_word);
        if (!ok) break;
        mbar_expect_tx(v_full, AT_TILE_BYTES);
        tma_load_3d(smem + S::kV, &tm, v_full, v_col, krow, 0);
        tma_load_3d(smem + S::kV + 16384, &tm, v_full, v_col + 64, krow, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t sQ = smem_u32(smem + S::kQ);
      const uint32_t sK = smem_u32(smem + S::kK);
      const uint32_t sV = smem_u32(smem + S::kV);
      bool ok = mbar_wait(q_full, 0, abort_word);
      for (int j = 0; j < ntiles && ok; ++j) {
        ok = mbar_wait(k_full, j & 1, abort_word);
        // P V of the previous tile has read the probabilities that alias S, and O is at rest for a rescale
        if (ok && j > 0) ok = mbar_wait(p_empty, (j - 1) & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT_D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16_ss(tmem_S, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024), idesc_qk,
                       k != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        umma_commit(k_empty);
        ok = mbar_wait(p_full, j & 1, abort_word);
        if (ok) ok = mbar_wait(v_full, j & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT_BK / 16; ++k)
          umma_bf16_ts(tmem_O, tmem_S + uint32_t(k * 8), umma_smem_desc(sV + k * 2048, 16384, 1024), idesc_pv,
                       (j | k) != 0 ? 1u : 0u);
        umma_commit(v_empty);
        umma_commit(p_empty);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int q = q0 + r;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const uint32_t tS = tmem_S + lane_off;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int k0 = (k_lo + j) * AT_BK;
      const bool need_mask = (k0 + AT_BK - 1 > q0) || (p.window >= 0 && q0 + AT_BQ - 1 - k0 > p.window);
      uint4 selw = make_uint4(~0u, ~0u, ~0u, ~0u);
      if (p.sel != nullptr && q < p.T)
        selw = *reinterpret_cast<const uint4*>(p.sel + ((long long)b * p.T + q) * (p.T >> 5) + (k0 >> 5));
      const uint32_t w4[4] = {selw.x, selw.y, selw.z, selw.w};
      // visible keys of this row inside the tile form the range [lo, hi] (causal upper end, window lower end)
      const int hi = min(AT_BK - 1, q - k0);
      const int lo = (p.window >= 0) ? max(0, q - p.window - k0) : 0;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      // pass 1: row maximum
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(tS + c * 32, sv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kk = c * 32 + i;
          const bool vis = (!need_mask || (kk <= hi && kk >= lo)) && ((w4[c] >> i) & 1u);
          mx4[i & 3] = fmaxf(mx4[i & 3], vis ? __uint_as_float(sv[i]) : -INFINITY);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const float m_new = fmaxf(m_ref, mx);
      const bool grow = (m_new > m_ref + 8.f) || (m_ref == -INFINITY);
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
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_O + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_ref = m_use;
      }
      // pass 2: probabilities, 32 keys at a time, packed over the scores already read
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(tS + c * 32, sv);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int g = 0; g < 16; ++g) {
          float e[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int i = 2 * g + u, kk = c * 32 + i;
            const bool vis = (!need_mask || (kk <= hi && kk >= lo)) && ((w4[c] >> i) & 1u);
            e[u] = vis ? ex2_fast(fmaf(__uint_as_float(sv[i]), p.scale_log2, -m_sub)) : 0.f;
            ps4[i & 3] += e[u];
          }
          pk[g] = pack_bf16(e[0], e[1]);
        }
        tmem_st_32x16(tS + c * 16, pk);
      }
      tmem_st_wait();
      l_sum += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (ntiles - 1) & 1, abort_word));
    if (ok) {
      tc_fence_after();
      if (p.sink != nullptr) {
        const float s2 = p.sink[h] * 1.4426950408889634f;
        if (m_ref == -INFINITY) {
          m_ref = s2;
          l_sum = 1.f;
        } else {
          l_sum += exp2f(s2 - m_ref);
        }
      }
      const float inv = 1.f / l_sum;
      const bool q_ok = q < p.T;
      __nv_bfloat16* orow = p.out + (long long)(row_base + q) * (p.Hq * AT_D) + q_col;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_off + c * 32, v);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
            u.y = pack_bf16(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
            u.z = pack_bf16(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
            u.w = pack_bf16(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = u;
          }
        }
      }
      if (q_ok) p.lse2[((long long)b * p.Hq + h) * p.T + q] = m_ref + log2f(l_sum);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}


// ---------------------------------------------------------------------------------------------------------------
// Two-query-tile form (ping-pong).  A CTA owns two consecutive 128-query tiles A and B of one (batch, head); each has
// its own softmax warpgroup (four warps, thread = query row), score buffer and output accumulator in TMEM
// (S_A | S_B | O_A | O_B = 512 columns), and both read the same K / V stages.  The MMA warp alternates
//     P_A V (t), Q_A K^T (t+1), P_B V (t), Q_B K^T (t+1), ...
// so the tensor pipe works on one tile while the other tile's warpgroup is in its softmax.  Probabilities go back as
// the TMEM A operand, packed over the scores they came from (S is single-buffered per tile: tcgen05.mma operations of
// one thread execute in issue order, so Q K^T (t+1) cannot overtake the P V (t) that reads the same columns, and a
// completed Q K^T (t+1) implies that P V (t) is complete, which is what an O rescale needs).  Tile A never needs the
// key tiles past its diagonal and tile B never needs the earliest window tile; both skip them.
constexpr int AT3_THREADS = 320;

struct AttnFwd3Smem {
  static constexpr int kQ = 0;                              // 2 tiles
  static constexpr int kK = 2 * AT_TILE_BYTES;              // 2 stages
  static constexpr int kV = 4 * AT_TILE_BYTES;              // 2 stages
  static constexpr int kBar = 6 * AT_TILE_BYTES;
  static constexpr int kTotal = kBar + 16 * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(AT3_THREADS, 1)
attn_fwd3_kernel(const __grid_constant__ CUtensorMap tm, const AttnFwdParams p) {
  using S = AttnFwd3Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2] per query tile
  uint64_t* p_full = bars + 7;     // [2] per query tile
  uint64_t* o_done = bars + 9;     // [2] per query tile
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qt = (p.T + AT_BQ - 1) / AT_BQ;
  const int num_pairs = (num_qt + 1) / 2;
  const int pair = num_pairs - 1 - blockIdx.x;               // heavy (late) pairs first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int row_base = b * p.T;
  const int q_col = h * AT_D;
  const int k_col = (p.Hq + hk) * AT_D;
  const int v_col = (p.Hq + p.Hkv + hk) * AT_D;
  // per query tile X: first / last key tile; B may be absent (odd tile count)
  auto q0_of = [&](int x) { return (2 * pair + x) * AT_BQ; };
  auto klo_of = [&](int x) { return (p.window < 0) ? 0 : max(0, q0_of(x) - p.window) / AT_BK; };
  auto khi_of = [&](int x) { return min(q0_of(x) + AT_BQ - 1, p.T - 1) / AT_BK; };
  const bool hasB = q0_of(1) < p.T;
  const int k_lo = klo_of(0);
  const int k_hi = hasB ? khi_of(1) : khi_of(0);
  const int n = k_hi - k_lo + 1;                              // key tiles the CTA walks
  const int nA = khi_of(0) - k_lo + 1;                           // A takes tiles [0, nA)
  const int offB = hasB ? klo_of(1) - k_lo : n;                  // B takes tiles [offB, n)

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
    }
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

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm);
      mbar_expect_tx(q_full, (hasB ? 2 : 1) * AT_TILE_BYTES);
      for (int x = 0; x < (hasB ? 2 : 1); ++x) {
        tma_load_3d(smem + S::kQ + x * AT_TILE_BYTES, &tm, q_full, q_col, row_base + q0_of(x), 0);
        tma_load_3d(smem + S::kQ + x * AT_TILE_BYTES + 16384, &tm, q_full, q_col + 64, row_base + q0_of(x), 0);
      }
      bool ok = true;
      for (int t = 0; t < n && ok; ++t) {
        const int st = t & 1;
        ok = mbar_wait(&kv_empty[st], ((t >> 1) & 1) ^ 1u, abort_word);
        if (!ok) break;
        const int krow = row_base + (k_lo + t) * AT_BK;
        uint8_t* sK = smem + S::kK + st * AT_TILE_BYTES;
        uint8_t* sV = smem + S::kV + st * AT_TILE_BYTES;
        mbar_expect_tx(&kv_full[st], 2 * AT_TILE_BYTES);
        tma_load_3d(sK, &tm, &kv_full[st], k_col, krow, 0);
        tma_load_3d(sK + 16384, &tm, &kv_full[st], k_col + 64, krow, 0);
        tma_load_3d(sV, &tm, &kv_full[st], v_col, krow, 0);
        tma_load_3d(sV + 16384, &tm, &kv_full[st], v_col + 64, krow, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      auto takes = [&](int x, int t) { return x == 0 ? (t < nA) : (t >= offB && t < n); };
      auto issue_qk = [&](int x, int t) {
        const uint32_t sQ = smem_u32(smem + S::kQ + x * AT_TILE_BYTES);
        const uint32_t sK = smem_u32(smem + S::kK + (t & 1) * AT_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < AT_D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16_ss(tmem_base + uint32_t(x * 128), umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024),
                       idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[x]);
      };
      bool ok = mbar_wait(q_full, 0, abort_word);
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        for (int x = 0; x < 2; ++x)
          if (takes(x, 0)) issue_qk(x, 0);
      }
      for (int t = 0; t < n && ok; ++t) {
        bool next_ready = false;
        for (int x = 0; x < 2 && ok; ++x) {
          if (takes(x, t)) {
            const int i = t - (x == 0 ? 0 : offB);             // this tile's index in X's own sequence
            ok = mbar_wait(&p_full[x], i & 1, abort_word);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sV = smem_u32(smem + S::kV + (t & 1) * AT_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < AT_BK / 16; ++k)
              umma_bf16_ts(tmem_base + uint32_t(256 + x * 128), tmem_base + uint32_t(x * 128 + k * 8),
                           umma_smem_desc(sV + k * 2048, 16384, 1024), idesc_pv, (i | k) != 0 ? 1u : 0u);
            if (!takes(x, t + 1)) umma_commit(&o_done[x]);    // X's last key tile
          }
          if (t + 1 < n && takes(x, t + 1)) {
            if (!next_ready) {
              ok = mbar_wait(&kv_full[(t + 1) & 1], ((t + 1) >> 1) & 1, abort_word);
              if (!ok) break;
              tc_fence_after();
              next_ready = true;
            }
            issue_qk(x, t + 1);
          }
        }
        umma_commit(&kv_empty[t & 1]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups: warps 2..5 -> A, 6..9 -> B
    const int x = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int q0 = q0_of(x);
    const int q = q0 + r;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const uint32_t tS = tmem_base + uint32_t(x * 128) + lane_off;
    const uint32_t tO = tmem_base + uint32_t(256 + x * 128) + lane_off;
    const int first = (x == 0) ? 0 : offB;
    const int count = (x == 0) ? nA : (hasB ? n - offB : 0);
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int i = 0; i < count && ok; ++i) {
      const int k0 = (k_lo + first + i) * AT_BK;
      const bool need_mask = (k0 + AT_BK - 1 > q0) || (p.window >= 0 && q0 + AT_BQ - 1 - k0 > p.window);
      uint4 selw = make_uint4(~0u, ~0u, ~0u, ~0u);
      if (p.sel != nullptr && q < p.T)
        selw = *reinterpret_cast<const uint4*>(p.sel + ((long long)b * p.T + q) * (p.T >> 5) + (k0 >> 5));
      const uint32_t w4[4] = {selw.x, selw.y, selw.z, selw.w};
      const bool use_sel = p.sel != nullptr;
      // the keys of this tile that the row may see form the range [lo, hi]
      const int hi = need_mask ? min(AT_BK - 1, q - k0) : AT_BK - 1;
      const int lo = (need_mask && p.window >= 0) ? max(0, q - p.window - k0) : 0;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[x], i & 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      // visibility bits of the four 32-key chunks (all ones on tiles that need no mask)
      uint32_t vb[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int l = max(lo - c * 32, 0), hcl = min(hi - c * 32, 31);
        const uint32_t range = (hcl < l) ? 0u : ((hcl >= 31 ? ~0u : ((1u << (hcl + 1)) - 1u)) & ~((1u << l) - 1u));
        vb[c] = range & w4[c];
      }
      const bool masked = need_mask || use_sel;
      // pass 1: row maximum, 64 columns per TMEM round trip
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        uint32_t sv[2][32];
        tmem_ld_32x32(tS + hc * 64, sv[0]);
        tmem_ld_32x32(tS + hc * 64 + 32, sv[1]);
        tmem_ld_wait();
        if (masked) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e)
              mx4[e & 3] = fmaxf(mx4[e & 3], ((vb[hc * 2 + c] >> e) & 1u) ? __uint_as_float(sv[c][e]) : -INFINITY);
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[c][e]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const float m_new = fmaxf(m_ref, mx);
      const bool grow = (m_new > m_ref + 8.f) || (m_ref == -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_use = grow ? m_new : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_use);
        if (i > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x32(tO + c * 32, o);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_ref = m_use;
      }
      // pass 2: probabilities, packed over the scores they came from (32 keys -> 16 columns)
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        uint32_t sv[2][32];
        tmem_ld_32x32(tS + hc * 64, sv[0]);
        tmem_ld_32x32(tS + hc * 64 + 32, sv[1]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float ev[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) ev[e] = ex2_fast(fmaf(__uint_as_float(sv[c][e]), p.scale_log2, -m_sub));
          if (masked) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (!((vb[hc * 2 + c] >> e) & 1u)) ev[e] = 0.f;
          }
          uint32_t pk[16];
#pragma unroll
          for (int g = 0; g < 16; ++g) {
            ps4[g & 3] += ev[2 * g] + ev[2 * g + 1];
            pk[g] = pack_bf16(ev[2 * g], ev[2 * g + 1]);
          }
          tmem_st_32x16(tS + (hc * 2 + c) * 16, pk);
        }
      }
      tmem_st_wait();
      l_sum += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }
    if (count > 0 && ok) ok = __all_sync(0xffffffffu, mbar_wait(&o_done[x], 0, abort_word));
    if (count > 0 && ok) {
      tc_fence_after();
      if (p.sink != nullptr) {
        const float s2 = p.sink[h] * 1.4426950408889634f;
        if (m_ref == -INFINITY) {
          m_ref = s2;
          l_sum = 1.f;
        } else {
          l_sum += exp2f(s2 - m_ref);
        }
      }
      const float inv = 1.f / l_sum;
      const bool q_ok = q < p.T;
      __nv_bfloat16* orow = p.out + (long long)(row_base + q) * (p.Hq * AT_D) + q_col;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tO + c * 32, v);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
            u.y = pack_bf16(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
            u.z = pack_bf16(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
            u.w = pack_bf16(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = u;
          }
        }
      }
      if (q_ok) p.lse2[((long long)b * p.Hq + h) * p.T + q] = m_ref + log2f(l_sum);
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

static long long* g_attn_prof = nullptr;
static const uint32_t* g_attn_sel = nullptr;
static const float* g_attn_sink = nullptr;
// Key-selection bits and sink logits for the NEXT forward launch only (consumed by it).
extern "C" void nga_attn_fwd_set_extras(const uint32_t* sel_bits, const float* sink) {
  g_attn_sel = sel_bits;
  g_attn_sink = sink;
}
// Tuning aid: when set, CTA (0,0,0) of the next forward launches writes per-phase cycle counts there.
extern "C" void nga_attn_set_prof(long long* device_ptr) { g_attn_prof = device_ptr; }

extern "C" int nga_attn_fwd(const void* qkv, void* out, float* lse2, int B, int T, int Hq, int Hkv,
                            int D, int window, float scale, int* status, void* stream) {
  using namespace nga;
  if (D != AT_D || B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  const long long cols = (long long)(Hq + 2 * Hkv) * D;
  CUtensorMap tm;
  int rc = make_tmap_3d(&tm, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cols, (long long)B * T, 1,
                        cols * 2, (long long)B * T * cols * 2, 64, 128, true);
  if (rc) return rc;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         AttnFwdSmem::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    attr_done = true;
  }
  AttnFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse2 = lse2;
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.prof = g_attn_prof;
  p.sel = g_attn_sel;
  p.sink = g_attn_sink;
  {
    static int p_tmem = -1;                        // NGA_ATTN_P_TMEM=1 selects the TMEM route for P
    if (p_tmem < 0) {
      const char* e = getenv("NGA_ATTN_P_TMEM");
      p_tmem = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    p.p_tmem = p_tmem;
  }
  g_attn_sel = nullptr;
  g_attn_sink = nullptr;
  if (p.sel != nullptr && (T % 128)) return -7;     // rows of selection words are read 16 bytes at a time
  dim3 grid((T + AT_BQ - 1) / AT_BQ, Hq, B);
  static int impl = -1;                            // NGA_ATTN_FWD_IMPL=1 selects the one-CTA-per-SM kernel with the K/V ring
  if (impl < 0) {
    const char* e = getenv("NGA_ATTN_FWD_IMPL");
    impl = (e != nullptr && e[0] >= '1' && e[0] <= '3') ? (e[0] - '0') : 3;
  }
  if (impl == 3 && p.prof == nullptr) {
    static nga::PerDevice<bool> attr3_flags;
    bool& attr3_done = attr3_flags.here();
    if (!attr3_done) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnFwd3Smem::kTotal);
      if (e != cudaSuccess) return -1000 - (int)e;
      attr3_done = true;
    }
    const int num_qt = (T + AT_BQ - 1) / AT_BQ;
    dim3 grid3((num_qt + 1) / 2, Hq, B);
    attn_fwd3_kernel<<<grid3, AT3_THREADS, AttnFwd3Smem::kTotal, reinterpret_cast<cudaStream_t>(stream)>>>(tm, p);
    count_launch();
    NGA_CHECK_LAUNCH();
    return 0;
  }
  if (impl == 2 && p.prof == nullptr) {
    static nga::PerDevice<bool> attr2_flags;
    bool& attr2_done = attr2_flags.here();
    if (!attr2_done) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnFwd2Smem::kTotal);
      if (e != cudaSuccess) return -1000 - (int)e;
      // two CTAs of 97 KB each must fit: ask for the largest shared-memory carve-out
      e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      if (e != cudaSuccess) return -1000 - (int)e;
      if (getenv("NGA_ATTN_DEBUG") != nullptr) {
        int nb = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, attn_fwd2_kernel, AT_THREADS, AttnFwd2Smem::kTotal);
        fprintf(stderr, "attn_fwd2: %d CTAs per SM\n", nb);
      }
      attr2_done = true;
    }
    attn_fwd2_kernel<<<grid, AT_THREADS, AttnFwd2Smem::kTotal, reinterpret_cast<cudaStream_t>(stream)>>>(tm, p);
    count_launch();
    NGA_CHECK_LAUNCH();
    return 0;
  }
  attn_fwd_kernel<<<grid, AT_THREADS, AttnFwdSmem::kTotal, reinterpret_cast<cudaStream_t>(stream)>>>(tm, p);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
