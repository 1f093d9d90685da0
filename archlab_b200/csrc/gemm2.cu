// CTA-pair bf16 GEMM for sm_100a: two CTAs of a cluster (two SMs) issue ONE tcgen05.mma with
// cta_group::2 on a 256 x 256 output tile.  Each CTA stages its own 128 rows of A and its own half
// (128 of 256 N-rows) of B, so shared-memory traffic per SM drops from 96 to 64 bytes per tensor
// cycle for reads and from 48 to 32 KB per k-block for TMA writes: the single-CTA 128 x 256 kernel
// in gemm.cu is bound by exactly that traffic.  Same operand orientations and epilogues as gemm.cu.
//
// Protocol (per CTA: warp 0 TMA producer, warp 1 MMA issuer in the leader, warps 2..5 epilogue):
//   * every TMA load of either CTA completes its bytes on the LEADER's full[stage] barrier
//     (cp.async.bulk.tensor with .cta_group::2; each CTA loads its own tiles);
//   * the leader's MMA thread waits on full[stage], issues the pair MMA, and releases the stage with
//     a tcgen05.commit multicast to empty[stage] of BOTH CTAs;
//   * accumulator hand-off uses tmem_full[acc] (commit multicast, one arrival per CTA) and the
//     leader's tmem_empty[acc] (8 arrivals: 4 epilogue warps of each CTA, the peer's via remote
//     mbarrier arrive).
// All waits are bounded; the two CTAs rendezvous on the hardware cluster barrier at start and end.
#include <cmath>
#include <cstdlib>
#include "gemm_common.cuh"
#include "pair_ptx.cuh"
#include "host_util.h"
#include <cuda.h>
#include <cudaTypedefs.h>

namespace nga {

constexpr int G2_BN = 256;                  // pair tile: 256 (M) x 256 (N)
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = BM * BK * 2;     // 16 KB: this CTA's 128 rows of A
constexpr int G2_B_BYTES = 128 * BK * 2;    // 16 KB: this CTA's half of B
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_OUT_OFFSET = G2_STAGES * G2_STAGE_BYTES;      // 4 warps x 2 staging tiles of 32 rows x 128 B
constexpr int G2_OUT_BYTES = 8 * 4096;    // 8 epilogue warps x one 32 x 64 staging tile (see below)
constexpr int G2_BAR_OFFSET = G2_OUT_OFFSET + G2_OUT_BYTES;
constexpr int G2_SMEM = G2_BAR_OFFSET + (2 * G2_STAGES + 4) * 8 + 16 + 1024;
constexpr int G2_THREADS = 320;          // TMA warp, MMA warp, 8 epilogue warps

// Untiled bulk copies (TMA engine) used by the all-gather clusters: peer global -> shared -> local global.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void st_release_gpu(int* addr, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// Bounded wait for a gathered 128-row block; false (and the abort word set) when the budget runs out.
// `sys`: the flag is written by another GPU (owner-push), so the acquire has system scope.
__device__ __forceinline__ bool wait_block_ready(const int* flag, int epoch, volatile int* abort_word, bool sys = false) {
  if ((sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag)) >= epoch) return true;
  const long long t0 = clock64();
  while ((sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag)) < epoch) {
    if (*abort_word != 0) return false;
    if (clock64() - t0 > kPeerWaitBudgetCycles) {
      *abort_word = kErrPeerTimeout;
      return false;
    }
  }
  return true;
}


// All-gather role of one CTA: pulls its share of the 128-row blocks into `tp.gathered` (remote shards in
// ring order, this rank's own rows last so that the gathered matrix is complete for the weight-gradient
// GEMM).  One thread drives a ring of G2_STAGES bulk copies of up to G2_STAGE_BYTES each.
__device__ __forceinline__ void tp_copy_role(const TpParams& tp, int K, uint8_t* smem, uint64_t* full_bar,
                                             int copy_cta, int num_copy_ctas, volatile int* abort_word) {
  const int blocks_per_rank = tp.rows_per_rank / BM;
  const int items = tp.world * blocks_per_rank;
  const long long block_bytes = (long long)BM * K * 2;
  const int chunks = int((block_bytes + G2_STAGE_BYTES - 1) / G2_STAGE_BYTES);
  uint32_t use = 0;                                   // global chunk counter -> slot and parity
  for (int it = copy_cta; it < items; it += num_copy_ctas) {
    const int src_rank = (tp.rank + 1 + it / blocks_per_rank) % tp.world;
    const int blk = it % blocks_per_rank;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(tp.peer_src[src_rank]) + (long long)blk * block_bytes;
    const long long grow = (long long)src_rank * tp.rows_per_rank + (long long)blk * BM;
    uint8_t* dst = reinterpret_cast<uint8_t*>(tp.gathered) + grow * K * 2;
    const int ahead = chunks < G2_STAGES ? chunks : G2_STAGES;
    for (int c = 0; c < ahead; ++c) {
      const uint32_t slot = (use + c) % G2_STAGES;
      const uint32_t bytes = uint32_t(min((long long)G2_STAGE_BYTES, block_bytes - (long long)c * G2_STAGE_BYTES));
      mbar_expect_tx(&full_bar[slot], bytes);
      bulk_load(smem + slot * G2_STAGE_BYTES, src + (long long)c * G2_STAGE_BYTES, bytes, &full_bar[slot]);
    }
    for (int c = 0; c < chunks; ++c) {
      const uint32_t u = use + c;
      const uint32_t slot = u % G2_STAGES;
      const uint32_t bytes = uint32_t(min((long long)G2_STAGE_BYTES, block_bytes - (long long)c * G2_STAGE_BYTES));
      if (!mbar_wait(&full_bar[slot], (u / G2_STAGES) & 1u, abort_word)) return;
      bulk_store(dst + (long long)c * G2_STAGE_BYTES, smem + slot * G2_STAGE_BYTES, bytes);
      tma_store_commit();
      const int nx = c + G2_STAGES;
      if (nx < chunks) {
        tma_store_wait_read0();                         // the slot's bytes have left shared memory
        const uint32_t nb = uint32_t(min((long long)G2_STAGE_BYTES, block_bytes - (long long)nx * G2_STAGE_BYTES));
        mbar_expect_tx(&full_bar[slot], nb);
        bulk_load(smem + slot * G2_STAGE_BYTES, src + (long long)nx * G2_STAGE_BYTES, nb, &full_bar[slot]);
      }
    }
    use += chunks;
    tma_store_wait0();                                  // the block is written
    fence_proxy_async_all();
    __threadfence();
    st_release_gpu(tp.flags + grow / BM, tp.epoch);
  }
}

__device__ __forceinline__ void red_release_sys_add(int* addr, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
// Owner-push all-gather, run by the 256 epilogue threads of a CTA (`tid` 0..255) before their tile loop.  Work item =
// (destination rank, 128-row block, one of `tp.push_parts` row slices of it); remote ranks first.  Every finished
// slice adds one to the destination's counter of that block, which therefore reads epoch * push_parts when the
// block of this call is complete.
__device__ __forceinline__ void tp_push_role(const TpParams& tp, int tid, int cta, int num_ctas) {
  const int bpr = tp.rows_per_rank / BM;
  const int parts = tp.push_parts;
  const int items = tp.world * bpr * parts;
  const long long part_bytes = (long long)(BM / parts) * tp.row_elems * 2;
  const int n16 = int(part_bytes >> 4);
  for (int it = cta; it < items; it += num_ctas) {
    const int peer = (tp.rank + 1 + it / (bpr * parts)) % tp.world;
    const int sub = it % (bpr * parts);                     // slice index inside this rank's shard
    const int blk = sub / parts;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(tp.push_src) + sub * part_bytes);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(tp.peer_dst[peer]) +
                                          (long long)tp.rank * tp.rows_per_rank * tp.row_elems * 2 + sub * part_bytes);
    int i = tid;
    for (; i + 768 < n16; i += 1024) {                       // four loads in flight per thread
      const uint4 a = __ldg(src + i), b = __ldg(src + i + 256), c = __ldg(src + i + 512), d = __ldg(src + i + 768);
      dst[i] = a; dst[i + 256] = b; dst[i + 512] = c; dst[i + 768] = d;
    }
    for (; i < n16; i += 256) dst[i] = __ldg(src + i);
    __threadfence_system();                                   // this thread's stores before the counter, at system scope
    asm volatile("bar.sync 1, 256;" ::: "memory");           // all 256 pushing threads have fenced
    if (tid == 0) red_release_sys_add(tp.peer_flags[peer] + tp.rank * bpr + blk, 1);
  }
}
// F8: 0 = bf16 operands; 1 + 2 * (A is e5m2) + 4 * (B is e5m2) = 8-bit operands (K-major only, 128 per k-block).
template <int A_MN, int B_MN, int TP, int F8 = 0>
__global__ void __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const GemmParams p, const __grid_constant__ CUtensorMap tmA2, const TpParams tp,
                  const __grid_constant__ TpMaps tpm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + G2_BAR_OFFSET);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tfull_bar = empty_bar + G2_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  // With the all-gather fused in, the first `copy_clusters` clusters only move data.
  const int copy_clusters = (TP && (tp.mode & kTpGatherAny) && !(tp.mode & kTpPush)) ? tp.copy_clusters : 0;
  const bool copy_role = TP && int(blockIdx.x >> 1) < copy_clusters;
  const int cluster_id = int(blockIdx.x >> 1) - copy_clusters;
  const int num_clusters = int(gridDim.x >> 1) - copy_clusters;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);   // 256-row tiles
  const int num_n = (p.N + G2_BN - 1) / G2_BN;
  constexpr int BKE = F8 ? 2 * BK : BK;             // elements per 128-byte k-block row
  const int num_kb = (p.K + BKE - 1) / BKE;
  const int num_tiles = num_m * num_n * p.batch * p.splits;   // work items (tile x k-split)

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 16);
    }
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_holder, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // barriers of both CTAs are initialised and visible
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  TileSeq seq = {cluster_id, 0x3fffffff, num_clusters, 0, 1};
  if (TP && copy_clusters > 0) {
    if (tp.early_rounds < 0) {
      if (copy_role) seq = {0, 0, 1, num_tiles, 1};                    // copy only
    } else {
      const int t1 = tp.early_rounds * num_clusters;
      if (copy_role) seq = {0, 0, 1, t1 + num_clusters + int(blockIdx.x >> 1), num_clusters + copy_clusters};
      else seq = {cluster_id, tp.early_rounds, num_clusters, t1 + cluster_id, num_clusters + copy_clusters};
    }
  }
  if (copy_role) {
    if (threadIdx.x == 0)
      tp_copy_role(tp, tp.row_elems, smem, full_bar, int(blockIdx.x), 2 * copy_clusters, abort_word);
    __syncthreads();
    if (threadIdx.x == 0) {            // the copies used the load barriers with their own phases: start them afresh
      for (int s = 0; s < G2_STAGES; ++s) {
        mbar_inval(&full_bar[s]);
        mbar_init(&full_bar[s], 1);
      }
      fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();                // both CTAs of the pair are done copying before either loads a GEMM stage
    if (*abort_word != 0) seq = {0, 0, 1, num_tiles, 1};   // a copy gave up: no tiles for this CTA (its pair times out)
  }
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (TP) tma_prefetch_desc(&tmA2);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool gathered_seen = false;                          // every block of the gathered B has been waited for once
      for (int it = 0, tile = seq.at(0); tile < num_tiles && ok; tile = seq.at(++it)) {
        int b, mb, nb, otile, kb0, kb1;
        split_range(tile, p.splits, num_kb, otile, kb0, kb1);
        tile_coords(otile, num_m, num_n, b, mb, nb);
        if (TP) { mb = tp_remap_mb(tp, mb, num_m); nb = tp_remap_nb(tp, nb, num_n); }
        if (!tile_has_work(p, b, mb, kb0, kb1)) continue;
        int m0 = mb * 2 * BM + int(rank) * BM;             // this CTA's 128 rows of A
        int n0 = nb * G2_BN + int(rank) * 128;             // this CTA's 128 N-rows of B
        const int grp_off = p.group_of_mtile ? p.group_of_mtile[mb] * p.group_rows : 0;   // rows of B before this tile's group
        const CUtensorMap* mapA = &tmA;
        if (TP && (tp.mode & kTpGather)) {
          const int owner = m0 / tp.rows_per_rank;
          if (owner == tp.rank) {                          // own rows: straight from the local shard
            mapA = &tmA2;
            m0 -= owner * tp.rows_per_rank;
          } else {
            ok = (tp.mode & kTpPush) ? wait_block_ready(tp.flags + m0 / BM, tp.epoch * tp.push_parts, abort_word, true)
                                     : wait_block_ready(tp.flags + m0 / BM, tp.epoch, abort_word);
            if (!ok) break;
            fence_proxy_async_all();
          }
        }
        const CUtensorMap* mapB = &tmB;
        if (TP && (tp.mode & kTpGatherB)) {
          const int owner = n0 / tp.rows_per_rank;
          if (owner == tp.rank) {                          // own weight rows: straight from the local shard
            mapB = &tmA2;
            n0 -= owner * tp.rows_per_rank;
          } else {
            ok = wait_block_ready(tp.flags + n0 / 128, tp.epoch, abort_word);
            if (!ok) break;
            fence_proxy_async_all();
          }
        }
        for (int kbi = kb0; kbi < kb1; ++kbi) {
          int kb = kbi;
          int brow = kb * BK;                              // first reduction row of an MN-major B block
          const CUtensorMap* mapBk = mapB;
          if (TP && B_MN && (tp.mode & kTpGatherBk)) {
            kb = kbi + tp.rank * (tp.rows_per_rank / BK);  // start at this rank's own rows
            if (kb >= num_kb) kb -= num_kb;
            brow = kb * BK;
            if (brow / tp.rows_per_rank == tp.rank) {
              mapBk = &tmA2;
              brow -= tp.rank * tp.rows_per_rank;
            } else if (!gathered_seen) {
              ok = wait_block_ready(tp.flags + brow / 128, tp.epoch, abort_word);
              if (!ok) break;
              fence_proxy_async_all();
            }
          }
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word);
          if (!ok) break;
          uint8_t* sA = smem + stage * G2_STAGE_BYTES;
          uint8_t* sB = sA + G2_A_BYTES;
          const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * G2_STAGE_BYTES);
          const int bl = p.kb_range != nullptr ? 0 : b;    // variable-length reductions share one A / B row range
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(sA + j * 8192, mapA, leader_full, m0 + j * 64, kb * BK, bl);
          } else {
            tma_load_3d_pair(sA, mapA, leader_full, kb * BKE, m0, bl);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(sB + j * 8192, mapBk, leader_full, n0 + j * 64, brow + grp_off, bl);
          } else {
            tma_load_3d_pair(sB, mapB, leader_full, kb * BKE, n0 + grp_off, bl);
          }
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (TP && (tp.mode & kTpGatherBk) && ok) gathered_seen = true;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = F8 ? umma_idesc_f8(2 * BM, G2_BN, (F8 >> 1) & 1, (F8 >> 2) & 1)
                                    : umma_idesc_bf16(2 * BM, G2_BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int it = 0, tile = seq.at(0); tile < num_tiles && ok; tile = seq.at(++it)) {
        int otile, kb0, kb1;
        split_range(tile, p.splits, num_kb, otile, kb0, kb1);
        if (p.group_of_mtile != nullptr || p.kb_range != nullptr) {
          int b, mb, nb;
          tile_coords(otile, num_m, num_n, b, mb, nb);
          if (!tile_has_work(p, b, mb, kb0, kb1)) continue;
        }
        ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + uint32_t(acc * G2_BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_word);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * G2_STAGE_BYTES);
          const uint32_t sB = sA + G2_A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc(sA + k * (UMMA_K * 128), 8192, 1024)
                                     : umma_smem_desc(sA + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sB + k * (UMMA_K * 128), 8192, 1024)
                                     : umma_smem_desc(sB + k * (UMMA_K * 2), 16, 1024);
            if (F8) umma2_f8_ss(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
            else umma2_bf16_ss(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma2_commit_multicast(&empty_bar[stage], 3);
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma2_commit_multicast(&tfull_bar[acc], 3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    // eight epilogue warps: TMEM lane quarter = warp % 4 (hardware rule), and the two warps of a quarter
    // split the 256 accumulator columns (the aux epilogues were issue-bound with four warps)
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = epilogue_vec_ok(p);
    const bool need_aux = (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2);
    const bool aux_fast = aux_prefetchable(p);
    uint32_t out_cnt = 0;
    if (TP && (tp.mode & kTpPush)) tp_push_role(tp, int(threadIdx.x) - 64, int(blockIdx.x), int(gridDim.x));
    const bool reduce_mode = TP && (tp.mode & kTpScatter) && (tp.mode & kTpReduce);
    for (int it = 0, tile = seq.at(0); tile < num_tiles && ok; tile = seq.at(++it)) {
      int b, mb, nb, otile, kb0, kb1;
      split_range(tile, p.splits, num_kb, otile, kb0, kb1);
      tile_coords(otile, num_m, num_n, b, mb, nb);
      if (TP) { mb = tp_remap_mb(tp, mb, num_m); nb = tp_remap_nb(tp, nb, num_n); }
      if (!tile_has_work(p, b, mb, kb0, kb1)) continue;
      const int row = mb * 2 * BM + int(rank) * BM + quarter * 32 + lane;
      GemmParams pt = p;
      if (TP && (tp.mode & kTpScatter)) {                   // this tile's rows live on rank `owner`
        const int owner = (mb * 2 * BM) / tp.rows_per_rank;
        pt.D = tp.peer_dst[owner];
        pt.row_shift = (long long)(tp.rank - owner) * tp.rows_per_rank;
      }
      AuxPre nxt;
      aux_prefetch(p, nxt, row, nb * G2_BN + chalf * 128, b, aux_fast);   // in flight while the main loop finishes
      ok = __all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, abort_word));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + uint32_t(acc * G2_BN) + (uint32_t(quarter * 32) << 16);
      const bool scatter = TP && (tp.mode & kTpScatter);
      int signal_owner = -1;
      if (reduce_mode && (mb * 2 * BM) / tp.rows_per_rank == tp.rank) {
        // a tile this rank owns: wait for the partial tiles of the other ranks, then sum and write the final rows
        const int per = tp.rows_per_rank / (2 * BM);
        const int* counter = tp.flags + (mb - tp.rank * per) * num_n + nb;
        bool arrived = true;
        if (lane == 0) arrived = wait_block_ready(counter, tp.arrivals, abort_word, true);
        ok = __all_sync(0xffffffffu, arrived);
        if (!ok) break;
        const int lrow = row - tp.rank * tp.rows_per_rank;               // row inside this rank's slice
        const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(tp.peer_dst[tp.rank]);
        const __nv_bfloat16* resid = reinterpret_cast<const __nv_bfloat16*>(tp.resid);
        __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(tp.reduce_out);
#pragma unroll 1
        for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {                 // 32-column chunks of this warp's half
          const int col0 = nb * G2_BN + c * 32;
          if (col0 >= p.N) break;   // warp-uniform
          uint32_t r[32];
          tmem_ld_32x32(taddr + uint32_t(c * 32), r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = p.alpha * __uint_as_float(r[i]);
          auto add_row = [&](const __nv_bfloat16* src) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 pk = *reinterpret_cast<const uint4*>(src + q * 8);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                v[q * 8 + 2 * e] += f.x;
                v[q * 8 + 2 * e + 1] += f.y;
              }
            }
          };
          for (int s = 0; s < tp.world; ++s)                                 // ascending source rank: a fixed order
            if (s != tp.rank) add_row(slots + ((long long)s * tp.rows_per_rank + lrow) * tp.ld_slot + col0);
          if (resid != nullptr) add_row(resid + (long long)lrow * tp.ld_resid + col0);
          __nv_bfloat16* d = outp + (long long)lrow * tp.ld_out + col0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16(v[8 * q], v[8 * q + 1]);
            o.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
            o.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]);
            o.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
            *reinterpret_cast<uint4*>(d + q * 8) = o;
          }
        }
      } else if (scatter || p.tma_store) {
        // bf16 tile -> swizzled staging tile -> one TMA store: into the owner's slot (reduce-scatter) or into D
        const int owner = scatter ? (mb * 2 * BM) / tp.rows_per_rank : 0;
        const int row0 = mb * 2 * BM + int(rank) * BM + quarter * 32 + int(pt.row_shift);
#pragma unroll 1
        for (int c2 = chalf * 2; c2 < chalf * 2 + 2; ++c2) {
          const int col0 = nb * G2_BN + c2 * 64;
          if (col0 >= p.N) break;   // warp-uniform
          const AuxPre cur = nxt;
          if (c2 + 1 < chalf * 2 + 2) aux_prefetch(p, nxt, row, nb * G2_BN + (c2 + 1) * 64, b, aux_fast);
          uint32_t r2[2][32];
          tmem_ld_32x32(taddr + uint32_t(c2 * 64), r2[0]);
          tmem_ld_32x32(taddr + uint32_t(c2 * 64 + 32), r2[1]);
          tmem_ld_wait();
          uint8_t* buf = smem + G2_OUT_OFFSET + (chalf * 4 + quarter) * 4096;      // one staging tile per warp
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (int hc = 0; hc < 2; ++hc)
            epilogue_stage_chunk(p, r2[hc], cur.valid[hc] ? cur.v[hc] : nullptr, buf, lane, hc);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tpm.d[owner], buf, col0, row0, scatter ? 0 : b);
            tma_store_commit();
          }
          ++out_cnt;
        }
        if (reduce_mode) signal_owner = owner;
      } else
#pragma unroll 1
      for (int c2 = chalf * 2; c2 < chalf * 2 + 2; ++c2) {
        if (nb * G2_BN + c2 * 64 >= p.N) break;   // warp-uniform
        const AuxPre cur = nxt;
        if (c2 + 1 < chalf * 2 + 2) aux_prefetch(p, nxt, row, nb * G2_BN + (c2 + 1) * 64, b, aux_fast);
        uint32_t r2[2][32];
        tmem_ld_32x32(taddr + uint32_t(c2 * 64), r2[0]);
        tmem_ld_32x32(taddr + uint32_t(c2 * 64 + 32), r2[1]);
        tmem_ld_wait();
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          const int col0 = nb * G2_BN + (c2 * 2 + hc) * 32;
          if (col0 >= p.N) break;   // warp-uniform
          epilogue_store_chunk(pt, r2[hc], row, col0, b, vec_ok, need_aux, cur.valid[hc] ? cur.v[hc] : nullptr);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      if (signal_owner >= 0) {
        // this warp's part of a remote owner's tile has been handed to the TMA engine and TMEM is released: once the
        // writes are complete, count one arrival on the owner's tile counter (16 warps of the pair make a tile)
        if (lane == 0) {
          tma_store_wait0();
          fence_proxy_async_all();                         // the engine's writes before the generic-proxy release below
          const int per = tp.rows_per_rank / (2 * BM);
          red_release_sys_add(tp.peer_flags[signal_owner] + (mb - signal_owner * per) * num_n + nb, 1);
        }
        __syncwarp();
      }
    }
    if (((TP && (tp.mode & kTpScatter)) || p.tma_store) && lane == 0) tma_store_wait0();   // every tile has landed
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();                  // neither CTA leaves while the pair may still touch its memory
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

template <int A_MN, int B_MN, int TP, int F8 = 0>
static int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream,
                        const CUtensorMap& ta2, const TpParams& tp, const TpMaps& tpm) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, TP, F8>;
  static nga::PerDevice<int> max_clusters_by_device;
  int& max_clusters = max_clusters_by_device.here();
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(G2_THREADS);
  cfg.dynamicSmemBytes = G2_SMEM;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM);
    if (e != cudaSuccess) return -1000 - (int)e;
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) return -1000 - (int)e;
    max_clusters = n;
  }
  // plain bf16 output: hand the tiles to the TMA engine (full 128-byte lines) instead of per-thread row stores
  GemmParams pp = p;
  TpMaps maps = tpm;
  pp.tma_store = 0;
  static int tma_store_on = -1;
  if (tma_store_on < 0) {
    const char* e = getenv("NGA_GEMM_TMA_STORE");
    tma_store_on = e ? atoi(e) : 1;              // 0: off; 1: every bf16 epilogue; 2: only those without aux
  }
  const bool aux_epi = (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2);
  // aux epilogues take the row's aux values from the register prefetch, which covers whole 32-column chunks only
  const bool epi_ok = p.epi == kEpiScale || p.epi == kEpiRelu2 ||
                      (aux_epi && !p.aux_fp32 && p.aux != nullptr && (p.N & 31) == 0 && (p.ldaux & 7) == 0 &&
                       (p.sAux & 7) == 0 && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0);
  if (tma_store_on && !(tma_store_on == 2 && aux_epi) && !(TP && (tp.mode & kTpScatter)) && epi_ok && !p.out_fp32 && p.splits == 1 &&
      p.row_shift == 0 && p.D != nullptr && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 && (p.ldd & 7) == 0 &&
      (p.batch == 1 || (p.sD & 7) == 0)) {
    const long long bstride = p.batch > 1 ? p.sD : (long long)p.M * p.ldd;
    if (make_tmap_3d(&maps.d[0], p.D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.M, p.batch, p.ldd * 2, bstride * 2, 64, 32,
                     true) == 0)
      pp.tma_store = 1;
  }
  const int num_tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256) * p.batch * p.splits;
  int clusters = num_tiles < max_clusters ? num_tiles : max_clusters;
  if (TP && (tp.mode & kTpGatherAny) && !(tp.mode & kTpPush)) {
    // every cluster must be resident at once: the GEMM clusters wait for the copy clusters
    if (tp.copy_clusters < 1 || tp.copy_clusters >= max_clusters) return -9;
    const int gemm_clusters = num_tiles < max_clusters - tp.copy_clusters ? num_tiles : max_clusters - tp.copy_clusters;
    clusters = gemm_clusters + tp.copy_clusters;
  }
  cfg.gridDim = dim3(2 * clusters);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, pp, ta2, tp, maps);
  count_launch();
  if (e != cudaSuccess) return -1000 - (int)e;
  return 0;
}

// out[r, c] = (resid ? resid[r, c] : 0) + sum_s stage[s * rows + r, c]   (fp32 accumulation, bf16 in/out)
__global__ void tp_reduce_slots_kernel(const __nv_bfloat16* __restrict__ stage, const __nv_bfloat16* __restrict__ resid,
                                       __nv_bfloat16* __restrict__ out, int world, long long rows, int N,
                                       long long ld_stage, long long ld_resid, long long ld_out) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= rows * N) return;
  const long long r = i / N;
  const int c = int(i - r * N);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  auto add = [&](const __nv_bfloat16* src) {
    const uint4 v = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      acc[2 * k] += f.x;
      acc[2 * k + 1] += f.y;
    }
  };
  if (resid != nullptr) add(resid + r * ld_resid + c);
  for (int s = 0; s < world; ++s) add(stage + ((long long)s * rows + r) * ld_stage + c);
  uint4 o;
  o.x = pack_bf16(acc[0], acc[1]);
  o.y = pack_bf16(acc[2], acc[3]);
  o.z = pack_bf16(acc[4], acc[5]);
  o.w = pack_bf16(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + r * ld_out + c) = o;
}

}  // namespace nga

// Same contract as nga_gemm_bf16 (gemm.h); returns -7 when the shape is better served by the
// single-CTA kernel (the caller then uses that one).
extern "C" int nga_gemm2_bf16(const void* A, const void* B, void* D, const void* aux, int M, int N, int K,
                              int batch, long long lda, long long ldb, long long ldd, long long ldaux,
                              long long sA, long long sB, long long sD, long long sAux, int a_mn, int b_mn,
                              int epi, int out_fp32, int aux_fp32, float alpha, float beta, int splits,
                              int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -1;
  if ((lda & 7) || (ldb & 7) || (sA & 7) || (sB & 7)) return -5;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn)
    rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, batch, lda * 2,
                      (batch > 1 ? sA : (long long)K * lda) * 2, 64, 64, true);
  else
    rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, batch, lda * 2,
                      (batch > 1 ? sA : (long long)M * lda) * 2, 64, 128, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, batch, ldb * 2,
                      (batch > 1 ? sB : (long long)K * ldb) * 2, 64, 64, true);
  else
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, batch, ldb * 2,
                      (batch > 1 ? sB : (long long)N * ldb) * 2, 64, 128, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.D = D; p.aux = aux; p.ldd = ldd; p.ldaux = ldaux; p.sD = sD; p.sAux = sAux;
  p.epi = epi; p.out_fp32 = out_fp32; p.aux_fp32 = aux_fp32; p.alpha = alpha; p.beta = beta;
  {
    const int num_kb = (K + BK - 1) / BK;
    int sp = (epi == kEpiAtomicAdd && splits > 1) ? (splits < num_kb ? splits : num_kb) : 1;
    const int per = (num_kb + sp - 1) / sp;
    p.splits = (num_kb + per - 1) / per;
  }
  if (epi == kEpiAtomicAdd && !out_fp32) return -8;
  p.status = status;
  p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TpParams tp = {};
  static const TpMaps no_maps = {};
  if (a_mn && b_mn) return launch_gemm2<1, 1, 0>(ta, tb, p, st, ta, tp, no_maps);
  if (a_mn && !b_mn) return launch_gemm2<1, 0, 0>(ta, tb, p, st, ta, tp, no_maps);
  if (!a_mn && b_mn) return launch_gemm2<0, 1, 0>(ta, tb, p, st, ta, tp, no_maps);
  return launch_gemm2<0, 0, 0>(ta, tb, p, st, ta, tp, no_maps);
}

// Grouped GEMM for expert layers: D[M, N] = A[M, K] . B_g^T (b_mn = 0: B is the stack [G * N, K] of K-major matrices)
// or A[M, K] . B_g (b_mn = 1: B is the stack [G * K, N] of MN-major matrices), where g = group_of_mtile[m / 256] for
// every 256-row tile (device int array of ceil(M / 256) entries; segments are padded to multiples of 256 rows).
extern "C" int nga_gemm2_grouped_bf16(const void* A, const void* B, void* D, const int* group_of_mtile, int groups, int M, int N,
                                      int K, long long lda, long long ldb, long long ldd, int b_mn, int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0 || group_of_mtile == nullptr) return -1;
  if ((lda & 7) || (ldb & 7)) return -5;
  if (b_mn && (K % BK)) return -6;                 // a k-block must not straddle two groups' matrices
  CUtensorMap ta, tb;
  int rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, 1, lda * 2, (long long)M * lda * 2, 64, 128, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, (long long)groups * K, 1, ldb * 2,
                      (long long)groups * K * ldb * 2, 64, 64, true);
  else
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, (long long)groups * N, 1, ldb * 2,
                      (long long)groups * N * ldb * 2, 64, 128, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = D; p.aux = nullptr; p.ldd = ldd; p.ldaux = 0; p.sD = 0; p.sAux = 0;
  p.epi = kEpiScale; p.out_fp32 = 0; p.aux_fp32 = 0; p.alpha = 1.f; p.beta = 0.f;
  p.splits = 1;
  p.status = status;
  p.row_shift = 0;
  p.group_of_mtile = group_of_mtile; p.kb_range = nullptr;
  p.group_rows = b_mn ? K : N;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TpParams tp = {};
  static const TpMaps no_maps = {};
  if (b_mn) return launch_gemm2<0, 1, 0>(ta, tb, p, st, ta, tp, no_maps);
  return launch_gemm2<0, 0, 0>(ta, tb, p, st, ta, tp, no_maps);
}

// Grouped weight gradient in one launch: dW[g] ([N_out, K_in] bf16, `groups` of them, contiguous) = dY_g^T X_g, where
// group g owns the 64-row blocks [kb_range[2g], kb_range[2g + 1]) of dY [rows, N_out] and X [rows, K_in] (device int
// array; rows are sorted by group and padded to 256 per group, rows of the padding must be zero in dY or X).  Groups
// without rows are skipped: dW[g] keeps what the caller put there (zeros).
extern "C" int nga_gemm2_grouped_wgrad_bf16(const void* dY, const void* X, void* dW, const int* kb_range, int groups, int rows,
                                            int n_out, int k_in, long long ldy, long long ldx, int* status, void* stream) {
  using namespace nga;
  if (rows <= 0 || n_out <= 0 || k_in <= 0 || groups <= 0 || kb_range == nullptr) return -1;
  if ((ldy & 7) || (ldx & 7) || (rows % BK)) return -5;
  CUtensorMap ta, tb;
  int rc = make_tmap_3d(&ta, dY, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n_out, rows, 1, ldy * 2, (long long)rows * ldy * 2, 64, 64, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tb, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_in, rows, 1, ldx * 2, (long long)rows * ldx * 2, 64, 64, true);
  if (rc) return rc;
  GemmParams p;
  p.M = n_out; p.N = k_in; p.K = rows; p.batch = groups;
  p.D = dW; p.aux = nullptr; p.ldd = k_in; p.ldaux = 0; p.sD = (long long)n_out * k_in; p.sAux = 0;
  p.epi = kEpiScale; p.out_fp32 = 0; p.aux_fp32 = 0; p.alpha = 1.f; p.beta = 0.f;
  p.splits = 1;
  p.status = status;
  p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = kb_range;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TpParams tp = {};
  static const TpMaps no_maps = {};
  return launch_gemm2<1, 1, 0>(ta, tb, p, st, ta, tp, no_maps);
}

// D[M, N] (bf16 or fp32) = alpha * A[M, K] B[N, K]^T with 8-bit floating-point operands (row-major, K contiguous,
// K a multiple of 16 bytes); a_e5m2 / b_e5m2 select e5m2 instead of e4m3.  `alpha` carries the product of the two
// tensor scales; epilogues as in nga_gemm2_bf16 (aux in bf16 / fp32).
extern "C" int nga_gemm2_fp8(const void* A, const void* B, void* D, const void* aux, int M, int N, int K, long long lda,
                             long long ldb, long long ldd, long long ldaux, int a_e5m2, int b_e5m2, int epi, int out_fp32,
                             int aux_fp32, float alpha, float beta, int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((lda & 15) || (ldb & 15)) return -5;
  CUtensorMap ta, tb;
  int rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, 1, lda, (long long)M * lda, 128, 128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, 1, ldb, (long long)N * ldb, 128, 128, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = D; p.aux = aux; p.ldd = ldd; p.ldaux = ldaux; p.sD = 0; p.sAux = 0;
  p.epi = epi; p.out_fp32 = out_fp32; p.aux_fp32 = aux_fp32; p.alpha = alpha; p.beta = beta;
  p.splits = 1;
  if (epi == kEpiAtomicAdd) return -8;
  p.status = status;
  p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TpParams tp = {};
  static const TpMaps no_maps = {};
  const int f = 1 + 2 * (a_e5m2 ? 1 : 0) + 4 * (b_e5m2 ? 1 : 0);
  switch (f) {
    case 1: return launch_gemm2<0, 0, 0, 1>(ta, tb, p, st, ta, tp, no_maps);
    case 3: return launch_gemm2<0, 0, 0, 3>(ta, tb, p, st, ta, tp, no_maps);
    case 5: return launch_gemm2<0, 0, 0, 5>(ta, tb, p, st, ta, tp, no_maps);
    default: return launch_gemm2<0, 0, 0, 7>(ta, tb, p, st, ta, tp, no_maps);
  }
}

// Whether the copy clusters also compute tiles once their copies are done (TpParams::early_rounds).  Measured on
// 2 x B200 (8192 x 9728 x 2560): when tiles follow the arrival order (kTpGather, kTpGatherB) a handful of copy
// clusters is enough and dedicated ones are faster (0.302 ms with 6 static clusters against 0.31-0.35 ms with any
// late-joining count); when every tile needs the whole gather (kTpGatherBk) the first round waits for the copies
// anyway and the copy clusters should take a share of the later rounds (0.45 against 0.51 ms at 12 clusters).
// NGA_TP_EARLY_ROUNDS overrides the choice (-1: copy only; r >= 0: join after r rounds).
static int tp_early_rounds(int copy_ctas, bool whole_k_per_tile) {
  static int forced = -2;
  if (forced == -2) {
    const char* e = getenv("NGA_TP_EARLY_ROUNDS");
    forced = e ? atoi(e) : -3;
  }
  if (copy_ctas <= 0) return 0;
  if (forced >= -1) return forced;
  return whole_k_per_tile ? 1 : -1;
}

// Tensor-parallel GEMM fused with its collective (see TpParams).  A is K-major; B is K-major (b_mn = 0)
// or MN-major (b_mn = 1); D is bf16.
//   mode = 1 (all-gather -> GEMM): `src_ptrs[r]` is rank r's row shard [rows_per_rank, K] (contiguous,
//     symmetric memory), `gathered` a local [world * rows_per_rank, K] buffer, `flags` a local int array
//     with one entry per 128 gathered rows (zero-initialised once; `epoch` must grow by one per call).
//     D [M = world * rows_per_rank, N] is local.
//   mode = 2 (GEMM -> reduce-scatter): A [M, K] is local; `dst_ptrs[r]` is rank r's staging buffer
//     [world, rows_per_rank, ldd]; this rank's partial sums for rank r's rows land in slot `rank` there.
//     The owner sums the slots with nga_tp_reduce_slots after a cross-rank barrier.
extern "C" int nga_tp_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long ldb,
                                long long ldd, int b_mn, int mode, int rank, int world, int rows_per_rank,
                                const long long* src_ptrs, void* gathered, int* flags, int epoch,
                                int copy_clusters, const long long* dst_ptrs, int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank % 256 || M != world * rows_per_rank) return -2;
  if ((K & 63) || (ldb & 7) || (ldd & 7)) return -5;
  if (mode != kTpGather && mode != kTpScatter) return -3;
  TpParams tp = {};
  tp.mode = mode; tp.rank = rank; tp.world = world; tp.rows_per_rank = rows_per_rank;
  tp.copy_clusters = copy_clusters; tp.epoch = epoch; tp.flags = flags; tp.gathered = gathered;
  tp.row_elems = K;
  tp.early_rounds = tp_early_rounds(2 * copy_clusters, false);
  for (int r = 0; r < world; ++r) {
    tp.peer_src[r] = (mode == kTpGather) ? reinterpret_cast<const void*>(src_ptrs[r]) : nullptr;
    tp.peer_dst[r] = (mode == kTpScatter) ? reinterpret_cast<void*>(dst_ptrs[r]) : nullptr;
  }
  const void* a_full = (mode == kTpGather) ? gathered : A;
  const void* a_own = (mode == kTpGather) ? tp.peer_src[rank] : A;
  if (a_full == nullptr || a_own == nullptr) return -4;
  CUtensorMap ta, ta2, tb;
  int rc = make_tmap_3d(&ta, a_full, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, 1, (long long)K * 2,
                        (long long)M * K * 2, 64, 128, true);
  if (rc) return rc;
  const long long own_rows = (mode == kTpGather) ? rows_per_rank : M;
  rc = make_tmap_3d(&ta2, a_own, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, own_rows, 1, (long long)K * 2,
                    own_rows * K * 2, 64, 128, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, 1, ldb * 2, (long long)K * ldb * 2, 64, 64, true);
  else
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, 1, ldb * 2, (long long)N * ldb * 2, 64, 128, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = D; p.aux = nullptr; p.ldd = ldd; p.ldaux = 0; p.sD = 0; p.sAux = 0;
  p.epi = kEpiScale; p.out_fp32 = 0; p.aux_fp32 = 0; p.alpha = 1.f; p.beta = 0.f; p.splits = 1;
  p.status = status; p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  TpMaps tpm = {};
  if (mode == kTpScatter) {
    for (int r = 0; r < world; ++r) {
      rc = make_tmap_3d(&tpm.d[r], tp.peer_dst[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, (long long)world * rows_per_rank,
                        1, ldd * 2, (long long)world * rows_per_rank * ldd * 2, 64, 32, true);
      if (rc) return rc;
    }
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (b_mn) return launch_gemm2<0, 1, 1>(ta, tb, p, st, ta2, tp, tpm);
  return launch_gemm2<0, 0, 1>(ta, tb, p, st, ta2, tp, tpm);
}

// Owner-push all-gather -> GEMM (kTpGather | kTpPush): D [M = world * rows_per_rank, N] = gather(X) . B^T (or . B with b_mn).
//   x_local         this rank's row shard [rows_per_rank, K] (any local memory; read directly for this rank's tiles)
//   gathered_ptrs   HOST array: the [M, K] gathered buffer of every rank for this call (symmetric memory; callers alternate
//                   between two buffers from call to call, which is all the ordering two consecutive calls need)
//   flag_ptrs       HOST array: every rank's flag array (symmetric, one int per 128 gathered rows, zero-initialised once);
//                   `epoch` grows by one per call
// No barrier precedes the call: a rank can run ahead by at most one call, because finishing a call needs every
// peer's shard of that call.
extern "C" int nga_tp_gemm_push_bf16(const void* x_local, const void* B, void* D, int M, int N, int K, long long ldb,
                                     long long ldd, int b_mn, int rank, int world, int rows_per_rank,
                                     const long long* gathered_ptrs, const long long* flag_ptrs, int epoch, int* status,
                                     void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank % 256 || M != world * rows_per_rank) return -2;
  if ((K & 63) || (ldb & 7) || (ldd & 7)) return -5;
  if (x_local == nullptr || gathered_ptrs == nullptr || flag_ptrs == nullptr) return -4;
  TpParams tp = {};
  tp.mode = kTpGather | kTpPush;
  tp.rank = rank; tp.world = world; tp.rows_per_rank = rows_per_rank;
  tp.copy_clusters = 0; tp.epoch = epoch; tp.row_elems = K; tp.early_rounds = 0;
  tp.push_src = x_local;
  // slices per 128-row block: enough work items for about two per CTA, so that every SM stores for a few microseconds only
  // One 128-row block per push item measured fastest at two ranks (0.133 ms against 0.138 / 0.147 ms with the block cut
  // in two / four slices): more pushing CTAs put peer stores on more SMs and slow every main loop.
  tp.push_parts = 1;
  {
    static int forced = -1;                                  // NGA_TP_PUSH_PARTS = 1 | 2 | 4 for measurements
    if (forced < 0) {
      const char* e = getenv("NGA_TP_PUSH_PARTS");
      forced = e ? atoi(e) : 0;
    }
    if (forced == 1 || forced == 2 || forced == 4) tp.push_parts = forced;
  }
  for (int r = 0; r < world; ++r) {
    tp.peer_dst[r] = reinterpret_cast<void*>(gathered_ptrs[r]);
    tp.peer_flags[r] = reinterpret_cast<int*>(flag_ptrs[r]);
    if (tp.peer_dst[r] == nullptr || tp.peer_flags[r] == nullptr) return -4;
  }
  tp.flags = tp.peer_flags[rank];
  tp.gathered = tp.peer_dst[rank];
  CUtensorMap ta, ta2, tb;
  int rc = make_tmap_3d(&ta, tp.gathered, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, 1, (long long)K * 2, (long long)M * K * 2, 64,
                        128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&ta2, x_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, rows_per_rank, 1, (long long)K * 2,
                    (long long)rows_per_rank * K * 2, 64, 128, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, 1, ldb * 2, (long long)K * ldb * 2, 64, 64, true);
  else
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, 1, ldb * 2, (long long)N * ldb * 2, 64, 128, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = D; p.aux = nullptr; p.ldd = ldd; p.ldaux = 0; p.sD = 0; p.sAux = 0;
  p.epi = kEpiScale; p.out_fp32 = 0; p.aux_fp32 = 0; p.alpha = 1.f; p.beta = 0.f; p.splits = 1;
  p.status = status; p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  TpMaps tpm = {};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (b_mn) return launch_gemm2<0, 1, 1>(ta, tb, p, st, ta2, tp, tpm);
  return launch_gemm2<0, 0, 1>(ta, tb, p, st, ta2, tp, tpm);
}

// GEMM -> reduce-scatter finished in the kernel (kTpScatter | kTpReduce): out [rows_per_rank, N] = this rank's rows of
// sum over ranks (A . B^T) (+ resid).  A [M, K] local.
//   slot_ptrs     HOST array: every rank's staging buffer [world][rows_per_rank, N] bf16 for this call (symmetric; callers
//                 alternate between two buffers from call to call)
//   counter_ptrs  HOST array: every rank's arrival counters (symmetric int array, one per owned 256 x 256 tile,
//                 zero-initialised once; never reset) and `call_index` = number of calls made on them so far + 1
// No barrier and no separate reduction kernel: see kTpReduce.
extern "C" int nga_tp_gemm_rs_reduce_bf16(const void* A, const void* B, void* out, const void* resid, int M, int N, int K,
                                          long long ldb, long long ld_out, long long ld_resid, int b_mn, int rank, int world,
                                          int rows_per_rank, const long long* slot_ptrs, const long long* counter_ptrs,
                                          int call_index, int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank % 256 || M != world * rows_per_rank) return -2;
  if ((K & 63) || (ldb & 7) || (N & 31) || (ld_out & 7) || (ld_resid & 7)) return -5;
  if (A == nullptr || out == nullptr || slot_ptrs == nullptr || counter_ptrs == nullptr || call_index < 1) return -4;
  TpParams tp = {};
  tp.mode = kTpScatter | kTpReduce;
  tp.rank = rank; tp.world = world; tp.rows_per_rank = rows_per_rank;
  tp.row_elems = K;
  tp.resid = resid; tp.reduce_out = out; tp.ld_resid = ld_resid; tp.ld_out = ld_out; tp.ld_slot = N;
  tp.arrivals = call_index * 16 * (world - 1);
  for (int r = 0; r < world; ++r) {
    tp.peer_dst[r] = reinterpret_cast<void*>(slot_ptrs[r]);
    tp.peer_flags[r] = reinterpret_cast<int*>(counter_ptrs[r]);
    if (tp.peer_dst[r] == nullptr || tp.peer_flags[r] == nullptr) return -4;
  }
  tp.flags = tp.peer_flags[rank];
  CUtensorMap ta, tb;
  int rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, 1, (long long)K * 2, (long long)M * K * 2, 64, 128, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, 1, ldb * 2, (long long)K * ldb * 2, 64, 64, true);
  else
    rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, 1, ldb * 2, (long long)N * ldb * 2, 64, 128, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = nullptr; p.aux = nullptr; p.ldd = N; p.ldaux = 0; p.sD = 0; p.sAux = 0;
  p.epi = kEpiScale; p.out_fp32 = 0; p.aux_fp32 = 0; p.alpha = 1.f; p.beta = 0.f; p.splits = 1;
  p.status = status; p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  TpMaps tpm = {};
  for (int r = 0; r < world; ++r) {
    rc = make_tmap_3d(&tpm.d[r], tp.peer_dst[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, (long long)world * rows_per_rank, 1,
                      (long long)N * 2, (long long)world * rows_per_rank * N * 2, 64, 32, true);
    if (rc) return rc;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (b_mn) return launch_gemm2<0, 1, 1>(ta, tb, p, st, ta, tp, tpm);
  return launch_gemm2<0, 0, 1>(ta, tb, p, st, ta, tp, tpm);
}

// GEMMs against a fully-sharded weight W [w_rows = world * rows_per_rank, w_cols] that lives as row shards on the
// ranks of a data-parallel group: `src_ptrs[r]` is rank r's shard [rows_per_rank, w_cols] (contiguous, symmetric
// memory), `gathered` a local [w_rows, w_cols] buffer that holds the whole weight afterwards, `flags` a local int
// array with one entry per 128 weight rows (zero-initialised once; `epoch` grows by one per call on the same
// flags).  A and D are local bf16 with row pitches lda, ldd.
//   transposed = 0 (forward):        D [M, w_rows] = A [M, w_cols] . W^T
//   transposed = 1 (data gradient):  D [M, w_cols] = A [M, w_rows] . W
extern "C" int nga_fsdp_gemm_bf16(const void* A, void* D, int M, int w_rows, int w_cols, long long lda, long long ldd,
                                  int transposed, int rank, int world, int rows_per_rank, const long long* src_ptrs,
                                  void* gathered, int* flags, int epoch, int copy_clusters, int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || w_rows <= 0 || w_cols <= 0 || world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank % 256 || w_rows != world * rows_per_rank) return -2;
  if ((w_cols & 63) || (lda & 7) || (ldd & 7)) return -5;
  if (A == nullptr || D == nullptr || gathered == nullptr || flags == nullptr || src_ptrs == nullptr) return -4;
  TpParams tp = {};
  tp.mode = transposed ? kTpGatherBk : kTpGatherB;
  tp.rank = rank; tp.world = world; tp.rows_per_rank = rows_per_rank;
  tp.copy_clusters = copy_clusters; tp.epoch = epoch; tp.flags = flags; tp.gathered = gathered;
  tp.row_elems = w_cols;
  tp.early_rounds = tp_early_rounds(2 * copy_clusters, transposed != 0);
  for (int r = 0; r < world; ++r) {
    tp.peer_src[r] = reinterpret_cast<const void*>(src_ptrs[r]);
    tp.peer_dst[r] = nullptr;
    if (tp.peer_src[r] == nullptr) return -4;
  }
  const int N = transposed ? w_cols : w_rows;
  const int K = transposed ? w_rows : w_cols;
  CUtensorMap ta, tb, tb_own;
  int rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, 1, lda * 2, (long long)M * lda * 2, 64, 128, true);
  if (rc) return rc;
  const int box_rows = transposed ? 64 : 128;     // MN-major B: 64 output columns x 64 reduction rows per load
  rc = make_tmap_3d(&tb, gathered, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_cols, w_rows, 1, (long long)w_cols * 2,
                    (long long)w_rows * w_cols * 2, 64, box_rows, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tb_own, tp.peer_src[rank], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_cols, rows_per_rank, 1,
                    (long long)w_cols * 2, (long long)rows_per_rank * w_cols * 2, 64, box_rows, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = D; p.aux = nullptr; p.ldd = ldd; p.ldaux = 0; p.sD = 0; p.sAux = 0;
  p.epi = kEpiScale; p.out_fp32 = 0; p.aux_fp32 = 0; p.alpha = 1.f; p.beta = 0.f; p.splits = 1;
  p.status = status; p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  TpMaps tpm = {};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (transposed) return launch_gemm2<0, 1, 1>(ta, tb, p, st, tb_own, tp, tpm);
  return launch_gemm2<0, 0, 1>(ta, tb, p, st, tb_own, tp, tpm);
}

extern "C" int nga_tp_reduce_slots(const void* stage, const void* resid, void* out, int world, long long rows, int N,
                                   long long ld_stage, long long ld_resid, long long ld_out, void* stream) {
  using namespace nga;
  if (world < 1 || rows <= 0 || N <= 0 || (N & 7) || (ld_stage & 7) || (ld_resid & 7) || (ld_out & 7)) return -1;
  const long long n8 = rows * N / 8;
  tp_reduce_slots_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(stage), reinterpret_cast<const __nv_bfloat16*>(resid),
      reinterpret_cast<__nv_bfloat16*>(out), world, rows, N, ld_stage, ld_resid, ld_out);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
