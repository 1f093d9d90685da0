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
#include "gemm_common.cuh"
#include "host_util.h"
#include <cuda.h>
#include <cudaTypedefs.h>

namespace nga {

constexpr int G2_BN = 256;                  // pair tile: 256 (M) x 256 (N)
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = BM * BK * 2;     // 16 KB: this CTA's 128 rows of A
constexpr int G2_B_BYTES = 128 * BK * 2;    // 16 KB: this CTA's half of B
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_BAR_OFFSET = G2_STAGES * G2_STAGE_BYTES;
constexpr int G2_SMEM = G2_BAR_OFFSET + (2 * G2_STAGES + 4) * 8 + 16 + 1024;
constexpr int G2_THREADS = 192;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_smem_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes go to a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in every CTA of `mask`, when all MMAs
// issued so far have completed.
__device__ __forceinline__ void umma2_commit_multicast(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const GemmParams p) {
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
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);   // 256-row tiles
  const int num_n = (p.N + G2_BN - 1) / G2_BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = num_m * num_n * p.batch * p.splits;   // work items (tile x k-split)

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int b, mb, nb, otile, kb0, kb1;
        split_range(tile, p.splits, num_kb, otile, kb0, kb1);
        tile_coords(otile, num_m, num_n, b, mb, nb);
        const int m0 = mb * 2 * BM + int(rank) * BM;       // this CTA's 128 rows of A
        const int n0 = nb * G2_BN + int(rank) * 128;       // this CTA's 128 N-rows of B
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word);
          if (!ok) break;
          uint8_t* sA = smem + stage * G2_STAGE_BYTES;
          uint8_t* sB = sA + G2_A_BYTES;
          const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * G2_STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(sA + j * 8192, &tmA, leader_full, m0 + j * 64, kb * BK, b);
          } else {
            tma_load_3d_pair(sA, &tmA, leader_full, kb * BK, m0, b);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(sB + j * 8192, &tmB, leader_full, n0 + j * 64, kb * BK, b);
          } else {
            tma_load_3d_pair(sB, &tmB, leader_full, kb * BK, n0, b);
          }
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, G2_BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + uint32_t(acc * G2_BN);
        int otile, kb0, kb1;
        split_range(tile, p.splits, num_kb, otile, kb0, kb1);
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
            umma2_bf16_ss(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
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
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = epilogue_vec_ok(p);
    const bool need_aux = (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2);
    const bool aux_fast = aux_prefetchable(p);
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int b, mb, nb, otile, kb0, kb1;
      split_range(tile, p.splits, num_kb, otile, kb0, kb1);
      tile_coords(otile, num_m, num_n, b, mb, nb);
      const int row = mb * 2 * BM + int(rank) * BM + quarter * 32 + lane;
      AuxPre nxt;
      aux_prefetch(p, nxt, row, nb * G2_BN, b, aux_fast);   // in flight while the main loop finishes
      ok = __all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, abort_word));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + uint32_t(acc * G2_BN) + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
      for (int c2 = 0; c2 < G2_BN / 64; ++c2) {
        if (nb * G2_BN + c2 * 64 >= p.N) break;   // warp-uniform
        const AuxPre cur = nxt;
        if (c2 + 1 < G2_BN / 64) aux_prefetch(p, nxt, row, nb * G2_BN + (c2 + 1) * 64, b, aux_fast);
        uint32_t r2[2][32];
        tmem_ld_32x32(taddr + uint32_t(c2 * 64), r2[0]);
        tmem_ld_32x32(taddr + uint32_t(c2 * 64 + 32), r2[1]);
        tmem_ld_wait();
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          const int col0 = nb * G2_BN + (c2 * 2 + hc) * 32;
          if (col0 >= p.N) break;   // warp-uniform
          epilogue_store_chunk(p, r2[hc], row, col0, b, vec_ok, need_aux, cur.valid[hc] ? cur.v[hc] : nullptr);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
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

template <int A_MN, int B_MN>
static int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN>;
  static int max_clusters = 0;
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
  const int num_tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256) * p.batch * p.splits;
  const int clusters = num_tiles < max_clusters ? num_tiles : max_clusters;
  cfg.gridDim = dim3(2 * clusters);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, p);
  count_launch();
  if (e != cudaSuccess) return -1000 - (int)e;
  return 0;
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
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch_gemm2<1, 1>(ta, tb, p, st);
  if (a_mn && !b_mn) return launch_gemm2<1, 0>(ta, tb, p, st);
  if (!a_mn && b_mn) return launch_gemm2<0, 1>(ta, tb, p, st);
  return launch_gemm2<0, 0>(ta, tb, p, st);
}
