// Causal / sliding-window GQA attention backward on tcgen05 + TMEM, head_dim 128, key-owned.
//
// One CTA owns 128 keys of one (batch, kv head) and walks the 64-query tiles (of every query head
// in the group) that can see them.  Everything is computed in the transposed frame so that the
// thread <-> TMEM-lane mapping is "one key per thread":
//     S^T  = K Q^T            P^T  = exp2(S^T * scale*log2e - lse2[q])
//     dP^T = V dO^T           dS^T = P^T * (dP^T - delta[q]) * scale
//     dV  += P^T dO           dK  += dS^T Q           dQ^T = K^T dS^T   (-> fp32 atomics)
// Warps: TMA producer, MMA issuer, eight compute warps (P^T / dS^T of a step), four dQ warps that carry dQ^T of the
// previous step from TMEM through a shared staging tile into the fp32 accumulator with one bulk tensor reduction, so
// that the compute warps go straight to the next step (a completed S^T of step i+1 implies that the products of step
// i have finished reading P^T / dS^T, because one thread's tcgen05.mma operations complete in issue order).
// dK / dV stay in TMEM for the whole CTA lifetime and are written once: no atomics on them and a
// bit-reproducible result; only dQ uses floating-point atomics (the reference's key-owned TileLang
// backward, src/archlab/architectures/tilelang_gqa.py:64-152, makes the same choice).
#include "ptx.cuh"
#include "host_util.h"
#include "attention.h"
#include <cuda.h>
#include <mutex>
#include <cstdlib>

namespace nga {

constexpr int AB_D = 128;
constexpr int AB_BK = 128;   // keys per CTA
constexpr int AB_BQ = 64;    // queries per inner step
constexpr int AB_THREADS = 448;   // TMA warp, MMA warp, 8 compute warps, 4 dQ warps

struct AttnBwdParams {
  __nv_bfloat16* dqkv;   // [B*T, (Hq+2Hkv)*D]
  float* dq_acc;         // [B*T, Hq*D] fp32, zeroed by the launcher
  const float* lse2;     // [B, Hq, T]
  const float* delta;    // [B, Hq, T]
  int B, T, Hq, Hkv, window;
  float scale, scale_log2;
  int* status;
  long long* prof;       // optional phase cycle counters written by CTA (0,0,0)
  int debug_skip_dq;     // measurement aid: leave the dQ reduction out
  int pt_tmem;           // 1: P^T and dS^T reach the dV / dK products as TMEM A operands instead of shared tiles
  const uint32_t* selT;  // optional key-major selection bits [B, T(key), T/32] (bit q of row k)
};

struct AttnBwdSmem {
  static constexpr int kK = 0;                      // 32 KB
  static constexpr int kV = 32768;                  // 32 KB
  static constexpr int kQ = 65536;                  // 2 x 16 KB
  static constexpr int kDO = kQ + 2 * 16384;        // 2 x 16 KB
  static constexpr int kPT = kDO + 2 * 16384;       // 16 KB
  static constexpr int kDST = kPT + 16384;          // 16 KB
  static constexpr int kDQ = kDST + 16384;          // 32 KB: fp32 dQ staging tile [64 q][128 d]
  static constexpr int kVec = kDQ + 32768;          // per compute warp: [2][lse 32 | delta 32]
  static constexpr int kBar = kVec + 8 * 128 * 4;
  static constexpr int kTotal = kBar + 16 * 8 + 16 + 1024;
};

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// delta[b, h, t] = sum_d O * dO   (16 lanes per (token, head), 16 bytes per lane and tensor)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out,
                                  const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                  int B, int T, int Hq) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int sub = int(gid & 15);
  const long long item = gid >> 4;
  const bool active = item < (long long)B * T * Hq;
  const long long row = active ? item / Hq : 0;
  const int h = active ? int(item % Hq) : 0;
  float s = 0.f;
  if (active) {
    const long long off = row * (long long)(Hq * AB_D) + h * AB_D + sub * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(out + off);
    const uint4 g = *reinterpret_cast<const uint4*>(dout + off);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(gh[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (active && sub == 0) delta[((long long)(row / T) * Hq + h) * T + (row % T)] = s;
}

// dqkv[:, q columns] = bf16(dq_acc)
__global__ void attn_dq_cast_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv,
                                    long long rows, int qcols, int allcols) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;      // qcols is a multiple of 128
  if (i >= rows * qcols) return;
  const long long row = i / qcols;
  const int c = int(i % qcols);
  const float4 v = *reinterpret_cast<const float4*>(dq_acc + i);
  const float4 w = *reinterpret_cast<const float4*>(dq_acc + i + 4);
  uint4 u;
  u.x = pack_bf16(v.x, v.y);
  u.y = pack_bf16(v.z, v.w);
  u.z = pack_bf16(w.x, w.y);
  u.w = pack_bf16(w.z, w.w);
  *reinterpret_cast<uint4*>(dqkv + row * allcols + c) = u;
}

__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_kv,   // qkv, box {64, 128}
                const __grid_constant__ CUtensorMap tm_q,    // qkv, box {64, 64}
                const __grid_constant__ CUtensorMap tm_do,   // dout, box {64, 64}
                const __grid_constant__ CUtensorMap tm_dq,   // dq_acc fp32, box {128, 64}, no swizzle
                const AttnBwdParams p) {
  using S = AttnBwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* st_full = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* mma2_done = bars + 7;
  uint64_t* dq_free = bars + 8;
  uint64_t* all_done = bars + 9;    // every product of the CTA has completed (dK / dV are final)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* s_vec = reinterpret_cast<float*>(smem + S::kVec);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int k0 = kt * AB_BK;
  const int row_base = b * p.T;
  const int qt_lo = k0 / AB_BQ;
  const int q_last = (p.window < 0) ? (p.T - 1) : min(p.T - 1, k0 + AB_BK - 1 + p.window);
  const int qt_hi = q_last / AB_BQ;
  const int nq = qt_hi - qt_lo + 1;
  const int niter = nq * group;
  const int k_col = (p.Hq + hk) * AB_D;
  const int v_col = (p.Hq + p.Hkv + hk) * AB_D;
  // full 64-query steps everywhere: the per-query vectors can come in by bulk copy (16-byte aligned, in bounds)
  const bool fast_vec = (p.T % AB_BQ) == 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(mma2_done, 1);
    mbar_init(dq_free, 4);
    mbar_init(all_done, 1);
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
  const uint32_t t_ST = tmem_base;          // 64 cols
  const uint32_t t_DPT = tmem_base + 64;    // 64 cols
  const uint32_t t_DQT = tmem_base + 128;   // 64 cols
  const uint32_t t_PT = tmem_base + 192;    // 32 cols: P^T as packed bf16 pairs (TMEM A operand of dV)
  const uint32_t t_DS = tmem_base + 224;    // 32 cols: dS^T as packed bf16 pairs (TMEM A operand of dK)
  const uint32_t t_DV = tmem_base + 256;    // 128 cols
  const uint32_t t_DK = tmem_base + 384;    // 128 cols

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_kv);
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      mbar_expect_tx(kv_full, 65536);
      tma_load_3d(smem + S::kK, &tm_kv, kv_full, k_col, row_base + k0, 0);
      tma_load_3d(smem + S::kK + 16384, &tm_kv, kv_full, k_col + 64, row_base + k0, 0);
      tma_load_3d(smem + S::kV, &tm_kv, kv_full, v_col, row_base + k0, 0);
      tma_load_3d(smem + S::kV + 16384, &tm_kv, kv_full, v_col + 64, row_base + k0, 0);
      bool ok = true;
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it & 1;
        ok = mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1u, abort_word);
        if (!ok) break;
        const int h = hk * group + it / nq;
        const int qrow = row_base + (qt_lo + it % nq) * AB_BQ;
        uint8_t* sQ = smem + S::kQ + st * 16384;
        uint8_t* sDO = smem + S::kDO + st * 16384;
        mbar_expect_tx(&qdo_full[st], 32768 + (fast_vec ? 512 : 0));
        if (fast_vec) {
          // log-sum-exp and delta of the step's 64 queries ride on the same barrier (256 contiguous bytes each)
          const long long vi = ((long long)b * p.Hq + h) * p.T + (qt_lo + it % nq) * AB_BQ;
          bulk_load_1d(s_vec + st * 128, p.lse2 + vi, 256, &qdo_full[st]);
          bulk_load_1d(s_vec + st * 128 + 64, p.delta + vi, 256, &qdo_full[st]);
        }
        tma_load_3d(sQ, &tm_q, &qdo_full[st], h * AB_D, qrow, 0);
        tma_load_3d(sQ + 8192, &tm_q, &qdo_full[st], h * AB_D + 64, qrow, 0);
        tma_load_3d(sDO, &tm_do, &qdo_full[st], h * AB_D, qrow, 0);
        tma_load_3d(sDO + 8192, &tm_do, &qdo_full[st], h * AB_D + 64, qrow, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_st = umma_idesc_bf16(128, 64, 0, 0);    // K Q^T, V dO^T
      constexpr uint32_t id_dv = umma_idesc_bf16(128, 128, 0, 1);   // P^T dO, dS^T Q
      constexpr uint32_t id_dq = umma_idesc_bf16(128, 64, 1, 1);    // K^T dS^T
      const uint32_t sK = smem_u32(smem + S::kK), sV = smem_u32(smem + S::kV);
      const uint32_t sPT = smem_u32(smem + S::kPT), sDST = smem_u32(smem + S::kDST);
      auto issue_mma1 = [&](int it) {
        const uint32_t sQ = smem_u32(smem + S::kQ + (it & 1) * 16384);
        const uint32_t sDO = smem_u32(smem + S::kDO + (it & 1) * 16384);
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // contraction over d
          const uint32_t offA = (k >> 2) * 16384 + (k & 3) * 32;   // K / V: 128-row blocks
          const uint32_t offB = (k >> 2) * 8192 + (k & 3) * 32;    // Q / dO: 64-row blocks
          umma_bf16_ss(t_ST, umma_smem_desc(sK + offA, 16, 1024), umma_smem_desc(sQ + offB, 16, 1024),
                       id_st, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t offA = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t offB = (k >> 2) * 8192 + (k & 3) * 32;
          umma_bf16_ss(t_DPT, umma_smem_desc(sV + offA, 16, 1024), umma_smem_desc(sDO + offB, 16, 1024),
                       id_st, k != 0 ? 1u : 0u);
        }
        umma_commit(st_full);
      };
      bool ok = mbar_wait(kv_full, 0, abort_word);
      if (ok) ok = mbar_wait(&qdo_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        issue_mma1(0);
      }
      for (int it = 0; it < niter && ok; ++it) {
        ok = mbar_wait(pds_full, it & 1, abort_word);
        if (ok && it > 0) ok = mbar_wait(dq_free, (it - 1) & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + S::kQ + (it & 1) * 16384);
        const uint32_t sDO = smem_u32(smem + S::kDO + (it & 1) * 16384);
#pragma unroll
        for (int k = 0; k < 4; ++k) {   // contraction over the 64 queries
          // A: P^T / dS^T, K-major (q contiguous), one 64-wide block.  B: dO / Q, MN-major:
          // rows are queries, d blocks 8 KB apart, 16 queries = 2048 B.
          if (p.pt_tmem)
            umma_bf16_ts(t_DV, t_PT + uint32_t(k * 8), umma_smem_desc(sDO + k * 2048, 8192, 1024), id_dv, (it | k) != 0 ? 1u : 0u);
          else
            umma_bf16_ss(t_DV, umma_smem_desc(sPT + k * 32, 16, 1024),
                         umma_smem_desc(sDO + k * 2048, 8192, 1024), id_dv, (it | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (p.pt_tmem)
            umma_bf16_ts(t_DK, t_DS + uint32_t(k * 8), umma_smem_desc(sQ + k * 2048, 8192, 1024), id_dv, (it | k) != 0 ? 1u : 0u);
          else
            umma_bf16_ss(t_DK, umma_smem_desc(sDST + k * 32, 16, 1024),
                         umma_smem_desc(sQ + k * 2048, 8192, 1024), id_dv, (it | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // contraction over the 128 keys
          // A: K^T, MN-major (rows are keys, d blocks 16 KB apart).  B: dS^T, MN-major (rows are
          // keys, one 64-wide q block).
          umma_bf16_ss(t_DQT, umma_smem_desc(sK + k * 2048, 16384, 1024),
                       umma_smem_desc(sDST + k * 2048, 8192, 1024), id_dq, k != 0 ? 1u : 0u);
        }
        umma_commit(mma2_done);
        umma_commit(&qdo_empty[it & 1]);
        if (it + 1 == niter) umma_commit(all_done);
        if (it + 1 < niter) {
          ok = mbar_wait(&qdo_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_word);
          if (!ok) break;
          tc_fence_after();
          issue_mma1(it + 1);
        }
      }
    }
  } else if (warp >= 10) {
    // ---------------------------------------------------------------- dQ warps 10..13: thread = d (TMEM lane)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    float* sDQ = reinterpret_cast<float*>(smem + S::kDQ);          // [64 q][128 d] fp32
    const bool tma_thread = (warp == 10 && lane == 0);
    bool ok = true;
    for (int it = 0; it < niter && ok; ++it) {
      const int h = hk * group + it / nq;
      const int q0 = (qt_lo + it % nq) * AB_BQ;
      ok = __all_sync(0xffffffffu, mbar_wait(mma2_done, it & 1, abort_word));
      if (!ok) break;
      tc_fence_after();
      uint32_t qv[2][32];
      tmem_ld_32x32(t_DQT + lane_off, qv[0]);
      tmem_ld_32x32(t_DQT + lane_off + 32, qv[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);
      // the staging tile is free once the previous bulk reduction has read it (its issuer waited for that before
      // it came to this barrier).  (Reducing straight from registers with scalar red.global was measured slower:
      // 1.23 against 1.11 ms at B16 T2048 H10.)
      asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) sDQ[(c * 32 + i) * AB_D + r] = __uint_as_float(qv[c][i]);
      fence_proxy_async_smem();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (tma_thread && !p.debug_skip_dq) {
        // one bulk tensor reduction adds the 64 x 128 fp32 tile into dq_acc (rows past the sequence end carry exact
        // zeros, rows past the tensor end are clipped by the copy engine)
        tma_reduce_add_3d(&tm_dq, sDQ, h * AB_D, row_base + q0, 0);
        tma_store_commit();
        tma_store_wait_read0();
      }
    }
    if (tma_thread) tma_store_wait0();
  } else {
    // ---------------------------------------------------------------- compute warps 2..9
    // thread = key row (TMEM lane); warps 2..5 own query columns 0..31 of the step, warps 6..9 own
    // columns 32..63, so every scheduler has two warps to hide TMEM / MUFU latency behind.
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int chalf = cw >> 2;
    const int r = quarter * 32 + lane;
    const int key = k0 + r;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const uint32_t col_off = uint32_t(chalf * 32);
    uint8_t* rowPT = smem + S::kPT + r * 128;
    uint8_t* rowDST = smem + S::kDST + r * 128;
    float* my_vec = s_vec + cw * 128;                              // [2][lse 32 | delta 32]
    bool ok = true;
    const bool prof_on = p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 64;
    long long pc[6] = {0, 0, 0, 0, 0, 0};
    long long tp = clock64();
#define NGA_PROFB(i) do { if (prof_on) { long long tn = clock64(); pc[i] += tn - tp; tp = tn; } } while (0)
    // per-query vectors of the first step; later steps are prefetched one step ahead
    float nxt_l = INFINITY, nxt_d = 0.f;
    uint32_t nxt_sel = ~0u;
    auto fetch_vec = [&](int it) {
      const int h = hk * group + it / nq;
      const int q = (qt_lo + it % nq) * AB_BQ + chalf * 32 + lane;
      if (p.selT != nullptr && key < p.T)
        nxt_sel = p.selT[((long long)b * p.T + key) * (p.T >> 5) + (((qt_lo + it % nq) * AB_BQ + chalf * 32) >> 5)];
      const long long vi = ((long long)b * p.Hq + h) * p.T + q;
      nxt_l = q < p.T ? p.lse2[vi] : INFINITY;
      nxt_d = q < p.T ? p.delta[vi] : 0.f;
    };
    if (niter > 0 && (!fast_vec || p.selT != nullptr)) fetch_vec(0);
    for (int it = 0; it < niter && ok; ++it) {
      const int h = hk * group + it / nq;
      const int q0 = (qt_lo + it % nq) * AB_BQ;
      const bool need_mask = (q0 < k0 + AB_BK - 1) || (p.window >= 0 && q0 + AB_BQ - 1 - k0 > p.window) ||
                             (q0 + AB_BQ > p.T);
      float* lse_b = fast_vec ? s_vec + (it & 1) * 128 + chalf * 32 : my_vec + (it & 1) * 64;
      float* del_b = fast_vec ? lse_b + 64 : lse_b + 32;
      if (!fast_vec) {
        lse_b[lane] = nxt_l;
        del_b[lane] = nxt_d;
      }
      // queries of this warp's 32 columns that the key row may pair with: q in [key, min(T - 1, key + window)]
      uint32_t vis = nxt_sel;
      if (need_mask) {
        const int qb = q0 + chalf * 32;
        const int i_lo = max(key - qb, 0);
        const int i_hi = min(min(p.T - 1, p.window >= 0 ? key + p.window : p.T - 1) - qb, 31);
        vis &= (i_hi < i_lo) ? 0u : ((i_hi >= 31 ? ~0u : ((1u << (i_hi + 1)) - 1u)) & ~((1u << i_lo) - 1u));
      }
      __syncwarp();
      if (it + 1 < niter && (!fast_vec || p.selT != nullptr)) fetch_vec(it + 1);     // global loads in flight during this step
      NGA_PROFB(0);
      if (fast_vec) ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full[it & 1], (it >> 1) & 1, abort_word));   // vectors landed
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(st_full, it & 1, abort_word));
      if (!ok) break;
      NGA_PROFB(1);
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(t_ST + lane_off + col_off, sv);
      tmem_ld_32x32(t_DPT + lane_off + col_off, dv);
      tmem_ld_wait();
      {
        float pr[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = ex2_fast(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse_b[i]));
          if (!((vis >> i) & 1u)) e = 0.f;
          pr[i] = e;
          ds[i] = e * (__uint_as_float(dv[i]) - del_b[i]) * p.scale;
        }
        if (p.pt_tmem) {
          // P^T and dS^T: 32 queries = 16 columns of packed pairs each, this warp's half of the 32-column operands
          uint32_t pk[16], dk[16];
#pragma unroll
          for (int g = 0; g < 16; ++g) {
            pk[g] = pack_bf16(pr[2 * g], pr[2 * g + 1]);
            dk[g] = pack_bf16(ds[2 * g], ds[2 * g + 1]);
          }
          tmem_st_32x16(t_PT + lane_off + uint32_t(chalf * 16), pk);
          tmem_st_32x16(t_DS + lane_off + uint32_t(chalf * 16), dk);
          // dS^T is also the shared B operand of dQ^T = K^T dS^T
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = (chalf * 4 + g) ^ (r & 7);
            *reinterpret_cast<uint4*>(rowDST + chunk * 16) = make_uint4(dk[4 * g], dk[4 * g + 1], dk[4 * g + 2], dk[4 * g + 3]);
          }
          tmem_st_wait();
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = (chalf * 4 + g) ^ (r & 7);
            uint4 u, w;
            u.x = pack_bf16(pr[8 * g + 0], pr[8 * g + 1]);
            u.y = pack_bf16(pr[8 * g + 2], pr[8 * g + 3]);
            u.z = pack_bf16(pr[8 * g + 4], pr[8 * g + 5]);
            u.w = pack_bf16(pr[8 * g + 6], pr[8 * g + 7]);
            w.x = pack_bf16(ds[8 * g + 0], ds[8 * g + 1]);
            w.y = pack_bf16(ds[8 * g + 2], ds[8 * g + 3]);
            w.z = pack_bf16(ds[8 * g + 4], ds[8 * g + 5]);
            w.w = pack_bf16(ds[8 * g + 6], ds[8 * g + 7]);
            *reinterpret_cast<uint4*>(rowPT + chunk * 16) = u;
            *reinterpret_cast<uint4*>(rowDST + chunk * 16) = w;
          }
        }
      }
      NGA_PROFB(2);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    if (prof_on) { for (int i = 0; i < 6; ++i) p.prof[i] = pc[i]; p.prof[6] = niter; }
    if (ok && niter > 0) ok = __all_sync(0xffffffffu, mbar_wait(all_done, 0, abort_word));
    // ---------------------------------------------------------------- dK / dV write-out
    // warps 2..5 write dK, warps 6..9 write dV (each thread: its key row, 128 columns)
    if (ok && niter > 0) {
      tc_fence_after();
      const bool key_ok = key < p.T;
      const long long cols = (long long)(p.Hq + 2 * p.Hkv) * AB_D;
      __nv_bfloat16* dst_row = p.dqkv + (long long)(row_base + key) * cols + (chalf == 0 ? k_col : v_col);
      const uint32_t src = (chalf == 0 ? t_DK : t_DV) + lane_off;
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t v2[2][32];
        tmem_ld_32x32(src + c2 * 64, v2[0]);
        tmem_ld_32x32(src + c2 * 64 + 32, v2[1]);
        tmem_ld_wait();
        if (key_ok) {
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            __nv_bfloat16* dst = dst_row + c2 * 64 + hc * 32;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 u;
              u.x = pack_bf16(__uint_as_float(v2[hc][8 * g + 0]), __uint_as_float(v2[hc][8 * g + 1]));
              u.y = pack_bf16(__uint_as_float(v2[hc][8 * g + 2]), __uint_as_float(v2[hc][8 * g + 3]));
              u.z = pack_bf16(__uint_as_float(v2[hc][8 * g + 4]), __uint_as_float(v2[hc][8 * g + 5]));
              u.w = pack_bf16(__uint_as_float(v2[hc][8 * g + 6]), __uint_as_float(v2[hc][8 * g + 7]));
              *reinterpret_cast<uint4*>(dst + g * 8) = u;
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

static long long* g_attn_bwd_prof = nullptr;
static const uint32_t* g_attn_bwd_selT = nullptr;
// Key-major selection bits for the NEXT backward launch only (consumed by it).
extern "C" void nga_attn_bwd_set_extras(const uint32_t* sel_bits_key_major) { g_attn_bwd_selT = sel_bits_key_major; }
extern "C" void nga_attn_bwd_set_prof(long long* device_ptr) { g_attn_bwd_prof = device_ptr; }

extern "C" int nga_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse2,
                            void* dqkv, float* dq_acc, float* delta, int B, int T, int Hq, int Hkv,
                            int D, int window, float scale, int* status, void* stream) {
  using namespace nga;
  if (D != AB_D || B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * T;
  const long long cols = (long long)(Hq + 2 * Hkv) * D;
  const long long ocols = (long long)Hq * D;
  CUtensorMap tm_kv, tm_q, tm_do;
  int rc = make_tmap_3d(&tm_kv, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cols, rows, 1, cols * 2,
                        rows * cols * 2, 64, 128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tm_q, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cols, rows, 1, cols * 2,
                    rows * cols * 2, 64, 64, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tm_do, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ocols, rows, 1, ocols * 2,
                    rows * ocols * 2, 64, 64, true);
  if (rc) return rc;
  CUtensorMap tm_dq;
  rc = make_tmap_3d(&tm_dq, dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ocols, rows, 1, ocols * 4,
                    rows * ocols * 4, 128, 64, false);
  if (rc) return rc;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         AttnBwdSmem::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    attr_done = true;
  }
  {
    const long long threads = rows * Hq * 16;
    attn_delta_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout),
        delta, B, T, Hq);
    count_launch();
  }
  cudaMemsetAsync(dq_acc, 0, sizeof(float) * rows * ocols, st);
  AttnBwdParams p;
  p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.dq_acc = dq_acc;
  p.lse2 = lse2;
  p.delta = delta;
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.prof = g_attn_bwd_prof;
  p.debug_skip_dq = getenv("NGA_ATTN_BWD_SKIP_DQ") != nullptr;
  {
    const char* e = getenv("NGA_ATTN_BWD_PT_TMEM");          // 0: P^T / dS^T as shared A operands of the dV / dK products
    p.pt_tmem = (e != nullptr && e[0] == '0') ? 0 : 1;       // TMEM operands: 1.105 against 1.125 ms (B16 T2048 H10)
  }
  p.selT = g_attn_bwd_selT;
  g_attn_bwd_selT = nullptr;
  if (p.selT != nullptr && (T % 64)) return -7;
  dim3 grid((T + AB_BK - 1) / AB_BK, Hkv, B);
  attn_bwd_kernel<<<grid, AB_THREADS, AttnBwdSmem::kTotal, st>>>(tm_kv, tm_q, tm_do, tm_dq, p);
  count_launch();
  {
    const long long n8 = rows * ocols / 8;
    attn_dq_cast_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(
        dq_acc, reinterpret_cast<__nv_bfloat16*>(dqkv), rows, (int)ocols, (int)cols);
    count_launch();
  }
  NGA_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free attention backward.
//
// Some callers cannot hand over scratch buffers: a host runtime that drives the kernels straight
// through the C ABI with no tensor library behind it, a serving loop that has frozen its memory
// pool, or code that runs where a device allocation would synchronise the whole GPU.  For them the
// fp32 dQ accumulator and the delta rows live in the two fixed device arrays below, which are part
// of the loaded module, so no cudaMalloc / cudaFree / allocator call happens on any call.
//
// Limits (rejected with -20 beyond them):  B*T*Hq*128 <= kStaticDqElems (16 MiB of fp32) and
// B*Hq*T <= kStaticDeltaElems.  The arrays are shared by every call on a device: two calls whose
// execution can overlap (different streams, or different host threads on different streams) race
// on them and must be ordered by the caller.  The accumulator is cleared by the launcher on each
// call, so nothing has to be zeroed by the caller.
//
// The first call on each device looks the arrays' addresses up (cudaGetSymbolAddress, with that
// device current) and caches them; make that first call outside of any stream capture.
namespace nga {
constexpr long long kStaticDqElems = 4ll * 1024 * 1024;
constexpr long long kStaticDeltaElems = kStaticDqElems / AB_D;
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) float g_static_dq_acc[kStaticDqElems];
static __device__ __align__(256) float g_static_delta[kStaticDeltaElems];
static float* g_static_dq_ptr[kStaticMaxDevices] = {};
static float* g_static_delta_ptr[kStaticMaxDevices] = {};
static std::mutex g_static_mu;
}  // namespace nga

extern "C" long long nga_attn_bwd_static_max_elems(void) { return nga::kStaticDqElems; }

extern "C" int nga_attn_bwd_static(const void* qkv, const void* out, const void* dout, const float* lse2,
                                   void* dqkv, int B, int T, int Hq, int Hkv, int D, int window,
                                   float scale, int* status, void* stream) {
  using namespace nga;
  if (D != AB_D || B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  if ((long long)B * T * Hq * D > kStaticDqElems || (long long)B * Hq * T > kStaticDeltaElems) return -20;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return -21;
  // The scratch handed to the kernel is the CURRENT device's copy of the arrays: the caller's
  // buffers (and hence its stream) must live on that device, or another GPU's scratch would be
  // paired with them.  A query of the output pointer catches the mismatch (no allocation).
  cudaPointerAttributes where = {};
  if (cudaPointerGetAttributes(&where, dqkv) != cudaSuccess) { cudaGetLastError(); return -22; }
  if (where.type == cudaMemoryTypeDevice && where.device != dev) return -22;
  float *dq = nullptr, *dl = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_dq_ptr[dev] == nullptr) {
      float *a = nullptr, *b = nullptr;
      cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&a), g_static_dq_acc);
      if (e != cudaSuccess || a == nullptr) return -1000 - (int)e;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&b), g_static_delta);
      if (e != cudaSuccess || b == nullptr) return -1000 - (int)e;
      g_static_delta_ptr[dev] = b;
      g_static_dq_ptr[dev] = a;
    }
    dq = g_static_dq_ptr[dev];
    dl = g_static_delta_ptr[dev];
  }
  return nga_attn_bwd(qkv, out, dout, lse2, dqkv, dq, dl, B, T, Hq, Hkv, D, window, scale, status, stream);
}
