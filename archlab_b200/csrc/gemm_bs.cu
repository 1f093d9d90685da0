// Block-scaled CTA-pair GEMMs for sm_100a: D[M, N] = alpha * (A . B^T) where A [M, K] and B [N, K] are
// narrow-float matrices (K contiguous) with one scale factor per block of consecutive K elements,
// multiplied in by the tensor core itself (tcgen05.mma ... .block_scale, scale factors in TMEM).
//
//   KIND 1 (kind::mxf8f6f4): e4m3 / e5m2 operands, one ue8m0 (power of two) scale per 32 elements.
//          DeepSeek-style 1 x 128 activation scales and 128 x 128 weight-block scales are this format with the
//          scale replicated over the four 32-element sub-blocks (and, for weights, over the 128 rows).
//   KIND 2 (kind::mxf4nvf4, scale_vec::4X): e2m1 operands packed two per byte, one ue4m3 scale per 16
//          elements; the fp32 per-tensor scales of NVFP4 go into `alpha`.
//
// Scale-factor layout in global memory (what the quantisers in quant_bs.cu write): for every 128 rows and
// every group of 4 scale factors along K one 512-byte chunk; byte (r % 32) * 16 + (r / 32) * 4 + j holds
// scale j of row r.  Chunks are ordered [row tile][chunk along K].  That is the image tcgen05.cp
// (32x128b.warpx4) moves into 4 TMEM columns, so a chunk travels global -> shared (TMA) -> TMEM untouched.
//
// Tile and pipeline follow the bf16 pair kernel (gemm2.cu): 256 x 256 per cluster of two CTAs, 128-byte
// k-blocks (128 fp8 or 256 fp4 elements), each CTA stages its 128 rows of A, its half of B, the scale
// chunks of its A rows and those of all 256 B rows; every load completes on the leader's barrier.  TMEM
// holds ONE 256-column accumulator plus the scale columns (512 columns cannot hold two accumulators and
// scales).  The plain epilogues (scale, ReLU^2 to bf16) therefore pull the accumulator into registers as
// packed bf16, hand TMEM back to the MMA warp at once and only then stage and store the tile, so that
// all but the TMEM reads overlaps the next tile's main loop; epilogues with an aux operand release TMEM
// after their stores.  The TMA producer prefetches throughout.  All waits are bounded.
#include <cstdlib>
#include "gemm_common.cuh"
#include "pair_ptx.cuh"
#include "host_util.h"
#include "gemm_bs.h"
#include <cuda.h>

namespace nga {

constexpr int BS_BN = 256;
constexpr int BS_STAGES = 4;
constexpr int BS_TILE_BYTES = 16384;                       // 128 rows x 128 bytes
constexpr int BS_SFA_OFF = 2 * BS_TILE_BYTES;              // scale chunks of this CTA's A rows (up to 4)
constexpr int BS_SFB_OFF = BS_SFA_OFF + 2048;              // scale chunks of the 256 B rows ([half][chunk])
constexpr int BS_STAGE_BYTES = BS_SFB_OFF + 4096;          // 38912 = 38 KB
constexpr int BS_OUT_OFFSET = BS_STAGES * BS_STAGE_BYTES;
constexpr int BS_OUT_BYTES = 16 * 4096;                    // 8 epilogue warps x two 32 x 64 bf16 staging tiles
constexpr int BS_BAR_OFFSET = BS_OUT_OFFSET + BS_OUT_BYTES;
constexpr int BS_SMEM = BS_BAR_OFFSET + (2 * BS_STAGES + 2) * 8 + 16 + 1024;
constexpr int BS_THREADS = 320;                            // TMA warp, MMA warp, 8 epilogue warps
constexpr uint32_t BS_SFA_COL = 256;                       // TMEM columns: accumulator 0..255, then scales
constexpr uint32_t BS_SFB_COL = 272;
static_assert(BS_STAGE_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
static_assert(BS_SMEM <= 232448, "shared memory per CTA");

// Shared-memory descriptor of one 512-byte scale chunk: 32 rows of 16 bytes, no swizzle (8-row core
// matrices 128 bytes apart).
__device__ __forceinline__ uint64_t sf_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFFu) >> 4);
  d |= uint64_t(128 >> 4) << 32;      // stride between 8-row groups
  d |= uint64_t(1) << 46;             // descriptor version for sm_100
  return d;
}
// shared -> TMEM in both CTAs of the pair (each from its own shared memory at the same offset): 32 rows x
// 128 bits, replicated to the four 32-lane quarters.
__device__ __forceinline__ void sf_copy_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma2_mxf8_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                              uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
__device__ __forceinline__ void umma2_nvf4_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                              uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// Instruction descriptor of the block-scaled kinds (fp32 accumulator, K-major operands): operand formats,
// N / 8, scale format (0 = ue4m3, 1 = ue8m0), M / 16 and which byte of the 32-bit scale column each
// operand uses (a_sf, b_sf; only with one scale per MMA).
__device__ __forceinline__ uint32_t umma_idesc_bs(int m, int n, int a_fmt, int b_fmt, int ue8m0, int a_sf, int b_sf) {
  return (uint32_t(b_sf & 3) << 4) | (uint32_t(a_fmt & 7) << 7) | (uint32_t(b_fmt & 7) << 10) |
         (uint32_t(n >> 3) << 17) | (uint32_t(ue8m0 & 1) << 23) | (uint32_t(m >> 4) << 24) | (uint32_t(a_sf & 3) << 29);
}

// Epilogue arithmetic on one 64-column piece of an accumulator row, packed to bf16 pairs (register i = columns 2i, 2i+1).
template <int EPI>
__device__ __forceinline__ void pack_piece(const uint32_t (&r)[2][32], uint32_t (&pk)[32], float alpha) {
#pragma unroll
  for (int hc = 0; hc < 2; ++hc)
#pragma unroll
    for (int i = 0; i < 16; ++i)
      pk[hc * 16 + i] = pack_bf16(epi_apply<EPI>(__uint_as_float(r[hc][2 * i]), 0.f, alpha, 0.f),
                                  epi_apply<EPI>(__uint_as_float(r[hc][2 * i + 1]), 0.f, alpha, 0.f));
}

struct BsExtra {
  int a_fmt, b_fmt;          // KIND 1: 0 = e4m3, 1 = e5m2
  int sfb_group_tiles;       // grouped form: 128-row scale tiles per group of B (group_rows / 128)
  // KIND 2: device pointers to the tensors' absolute maxima (may be null); alpha is multiplied by the two
  // decode scales amax / 2688 that undo the quantisers' encode scales, without a host read of the maxima
  const float* amax_a;
  const float* amax_b;
};

template <int KIND>
__global__ void __launch_bounds__(BS_THREADS, 1)
gemm_bs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
               const __grid_constant__ CUtensorMap tmD, const GemmParams p, const BsExtra x) {
  constexpr int CPK = KIND == 1 ? 1 : 4;                   // scale chunks per k-block and 128 rows
  constexpr int BKE = KIND == 1 ? 128 : 256;               // elements per k-block
  constexpr uint32_t kStageTx = 2u * (2u * BS_TILE_BYTES + 3u * 512u * CPK);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + BS_BAR_OFFSET);
  uint64_t* empty_bar = full_bar + BS_STAGES;
  uint64_t* tfull_bar = empty_bar + BS_STAGES;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = int(blockIdx.x >> 1);
  const int num_clusters = int(gridDim.x >> 1);
  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + BS_BN - 1) / BS_BN;
  const int num_kb = (p.K + BKE - 1) / BKE;
  const int num_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < BS_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_holder, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      tma_prefetch_desc(&tmSFA);
      tma_prefetch_desc(&tmSFB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int b, mb, nb;
        tile_coords(tile, num_m, num_n, b, mb, nb);
        if (p.group_of_mtile != nullptr && p.group_of_mtile[mb] < 0) continue;      // a tile of the row bound without rows
        const int m0 = mb * 2 * BM + int(rank) * BM;
        const int group = p.group_of_mtile ? p.group_of_mtile[mb] : 0;
        const int n0 = nb * BS_BN + int(rank) * 128 + group * p.group_rows;
        const int sfb_tile0 = nb * 2 + group * x.sfb_group_tiles;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word);
          if (!ok) break;
          uint8_t* st = smem + stage * BS_STAGE_BYTES;
          const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], kStageTx);
          tma_load_3d_pair(st, &tmA, leader_full, kb * 128, m0, 0);
          tma_load_3d_pair(st + BS_TILE_BYTES, &tmB, leader_full, kb * 128, n0, 0);
          tma_load_3d_pair(st + BS_SFA_OFF, &tmSFA, leader_full, 0, kb * CPK, m0 / 128);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_3d_pair(st + BS_SFB_OFF + h * CPK * 512, &tmSFB, leader_full, 0, kb * CPK, sfb_tile0 + h);
          if (++stage == BS_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ scale copies + MMA (leader only)
    if (rank == 0 && lane == 0) {
      const int a_fmt = KIND == 1 ? x.a_fmt : 1, b_fmt = KIND == 1 ? x.b_fmt : 1;
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (p.group_of_mtile != nullptr) {
          int b, mb, nb;
          tile_coords(tile, num_m, num_n, b, mb, nb);
          if (p.group_of_mtile[mb] < 0) continue;
        }
        ok = mbar_wait(tempty_bar, acc_phase ^ 1u, abort_word);      // the epilogue has drained the accumulator
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_word);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * BS_STAGE_BYTES);
          const uint32_t sB = sA + BS_TILE_BYTES;
#pragma unroll
          for (int c = 0; c < CPK; ++c) sf_copy_pair(tmem_base + BS_SFA_COL + 4 * c, sf_smem_desc(sA + BS_SFA_OFF + c * 512));
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < CPK; ++c)
              sf_copy_pair(tmem_base + BS_SFB_COL + (KIND == 1 ? 4 * h : 8 * c + 4 * h),
                           sf_smem_desc(sA + BS_SFB_OFF + (h * CPK + c) * 512));
#pragma unroll
          for (int k = 0; k < 4; ++k) {                              // 4 x 32 bytes of K per 128-byte row
            const uint64_t da = umma_smem_desc(sA + k * 32, 16, 1024);
            const uint64_t db = umma_smem_desc(sB + k * 32, 16, 1024);
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (KIND == 1) {
              const uint32_t idesc = umma_idesc_bs(2 * BM, BS_BN, a_fmt, b_fmt, 1, k, k);
              umma2_mxf8_ss(tmem_base, da, db, idesc, tmem_base + BS_SFA_COL, tmem_base + BS_SFB_COL, accum);
            } else {
              const uint32_t idesc = umma_idesc_bs(2 * BM, BS_BN, a_fmt, b_fmt, 0, 0, 0);
              umma2_nvf4_ss(tmem_base, da, db, idesc, tmem_base + BS_SFA_COL + 4 * k, tmem_base + BS_SFB_COL + 8 * k, accum);
            }
          }
          umma2_commit_multicast(&empty_bar[stage], 3);
          if (++stage == BS_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma2_commit_multicast(tfull_bar, 3);
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = epilogue_vec_ok(p);
    const bool need_aux = (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2);
    const bool aux_fast = aux_prefetchable(p);
    const bool fast_epi = p.tma_store && (p.epi == kEpiScale || p.epi == kEpiRelu2);
    GemmParams pe = p;
    if (x.amax_a != nullptr) { const float a = *x.amax_a; pe.alpha *= a > 0.f ? a * (1.f / 2688.f) : 1.f; }
    if (x.amax_b != nullptr) { const float a = *x.amax_b; pe.alpha *= a > 0.f ? a * (1.f / 2688.f) : 1.f; }
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int b, mb, nb;
      tile_coords(tile, num_m, num_n, b, mb, nb);
      if (p.group_of_mtile != nullptr && p.group_of_mtile[mb] < 0) continue;
      const int row = mb * 2 * BM + int(rank) * BM + quarter * 32 + lane;
      AuxPre nxt;
      aux_prefetch(p, nxt, row, nb * BS_BN + chalf * 128, 0, aux_fast);
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar, acc_phase, abort_word));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
      if (fast_epi) {
        // accumulator -> packed bf16 in registers, TMEM handed back, then staging + TMA stores
        uint32_t pk[2][32];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t r2[2][32];
          tmem_ld_32x32(taddr + uint32_t((chalf * 2 + j) * 64), r2[0]);
          tmem_ld_32x32(taddr + uint32_t((chalf * 2 + j) * 64 + 32), r2[1]);
          tmem_ld_wait();
          if (pe.epi == kEpiRelu2) pack_piece<kEpiRelu2>(r2, pk[j], pe.alpha);
          else pack_piece<kEpiScale>(r2, pk[j], pe.alpha);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(tempty_bar), 0));
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col0 = nb * BS_BN + (chalf * 2 + j) * 64;
          if (col0 >= p.N) {        // warp-uniform; an empty group keeps the two-groups-per-tile cadence the wait counts on
            if (lane == 0) tma_store_commit();
            continue;
          }
          uint8_t* buf = smem + BS_OUT_OFFSET + ((chalf * 4 + quarter) * 2 + j) * 4096;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the store that last read this tile
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((q ^ (lane & 7)) * 16)) =
                make_uint4(pk[j][4 * q], pk[j][4 * q + 1], pk[j][4 * q + 2], pk[j][4 * q + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmD, buf, col0, mb * 2 * BM + int(rank) * BM + quarter * 32, 0);
            tma_store_commit();
          }
        }
        acc_phase ^= 1u;
        continue;
      }
#pragma unroll 1
      for (int c2 = chalf * 2; c2 < chalf * 2 + 2; ++c2) {
        const int col0 = nb * BS_BN + c2 * 64;
        if (col0 >= p.N) break;   // warp-uniform
        const AuxPre cur = nxt;
        if (c2 + 1 < chalf * 2 + 2) aux_prefetch(p, nxt, row, nb * BS_BN + (c2 + 1) * 64, 0, aux_fast);
        uint32_t r2[2][32];
        tmem_ld_32x32(taddr + uint32_t(c2 * 64), r2[0]);
        tmem_ld_32x32(taddr + uint32_t(c2 * 64 + 32), r2[1]);
        tmem_ld_wait();
        if (p.tma_store) {
          uint8_t* buf = smem + BS_OUT_OFFSET + (chalf * 4 + quarter) * 4096;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (int hc = 0; hc < 2; ++hc)
            epilogue_stage_chunk(pe, r2[hc], cur.valid[hc] ? cur.v[hc] : nullptr, buf, lane, hc);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmD, buf, col0, mb * 2 * BM + int(rank) * BM + quarter * 32, 0);
            tma_store_commit();
          }
        } else {
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            const int c0 = col0 + hc * 32;
            if (c0 >= p.N) break;   // warp-uniform
            epilogue_store_chunk(pe, r2[hc], row, c0, 0, vec_ok, need_aux, cur.valid[hc] ? cur.v[hc] : nullptr);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(tempty_bar), 0));
      acc_phase ^= 1u;
    }
    if (p.tma_store && lane == 0) tma_store_wait0();
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

template <int KIND>
static int launch_gemm_bs(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                          GemmParams p, const BsExtra& x, cudaStream_t stream) {
  auto kern = gemm_bs_kernel<KIND>;
  static PerDevice<int> max_clusters_by_device;
  int& max_clusters = max_clusters_by_device.here();
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(BS_THREADS);
  cfg.dynamicSmemBytes = BS_SMEM;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BS_SMEM);
    if (e != cudaSuccess) return -1000 - (int)e;
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) return -1000 - (int)e;
    max_clusters = n;
  }
  CUtensorMap td = {};
  p.tma_store = 0;
  const bool aux_epi = (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2);
  const bool epi_ok = p.epi == kEpiScale || p.epi == kEpiRelu2 ||
                      (aux_epi && !p.aux_fp32 && p.aux != nullptr && (p.N & 31) == 0 && (p.ldaux & 7) == 0 &&
                       (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0);
  if (epi_ok && !p.out_fp32 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 && (p.ldd & 7) == 0 &&
      make_tmap_3d(&td, p.D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.M, 1, p.ldd * 2, (long long)p.M * p.ldd * 2, 64, 32,
                   true) == 0)
    p.tma_store = 1;
  if (!p.tma_store) td = ta;    // never used by the kernel, but the parameter must be a valid map
  const int num_tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  const int clusters = num_tiles < max_clusters ? num_tiles : max_clusters;
  cfg.gridDim = dim3(2 * clusters);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tsa, tsb, td, p, x);
  count_launch();
  if (e != cudaSuccess) return -1000 - (int)e;
  return 0;
}

// Tensor map over the chunked scale array of a matrix with `rows` rows and `chunks_k` chunks along K:
// [ceil(rows / 128)][chunks_k][128 x uint32]; one box = the `cpk` chunks of one k-block.
static int make_sf_map(CUtensorMap* out, const void* sf, long long rows, long long chunks_k, int cpk) {
  const long long tiles = (rows + 127) / 128;
  return make_tmap_3d(out, sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, 128, chunks_k, tiles, 512, chunks_k * 512, 128, cpk, false);
}

static int gemm_bs_common(int kind, const void* A, const void* sfa, const void* B, const void* sfb, void* D, const void* aux,
                          int M, int N, int K, long long lda_bytes, long long ldb_bytes, long long ldd, long long ldaux,
                          int a_fmt, int b_fmt, int epi, int out_fp32, int aux_fp32, float alpha, float beta,
                          const int* group_of_mtile, int groups, const float* amax_a, const float* amax_b, int* status,
                          void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || A == nullptr || B == nullptr || sfa == nullptr || sfb == nullptr || D == nullptr) return -1;
  const int bke = kind == 1 ? 128 : 256, cpk = kind == 1 ? 1 : 4;
  const int epb = kind == 1 ? 1 : 2;                               // elements per byte
  if (K % (kind == 1 ? 32 : 64)) return -6;                        // whole MMA steps only
  if ((lda_bytes & 15) || (ldb_bytes & 15)) return -5;
  if (epi == kEpiAtomicAdd) return -8;
  if (group_of_mtile != nullptr && (groups <= 0 || N % 128)) return -2;
  const long long num_kb = (K + bke - 1) / bke;
  const long long brows = (long long)(group_of_mtile ? groups : 1) * N;
  CUtensorMap ta, tb, tsa, tsb;
  int rc = make_tmap_3d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / epb, M, 1, lda_bytes, (long long)M * lda_bytes, 128, 128, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / epb, brows, 1, ldb_bytes, brows * ldb_bytes, 128, 128, true);
  if (rc) return rc;
  rc = make_sf_map(&tsa, sfa, M, num_kb * cpk, cpk);
  if (rc) return rc;
  rc = make_sf_map(&tsb, sfb, brows, num_kb * cpk, cpk);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.D = D; p.aux = aux; p.ldd = ldd; p.ldaux = ldaux; p.sD = 0; p.sAux = 0;
  p.epi = epi; p.out_fp32 = out_fp32; p.aux_fp32 = aux_fp32; p.alpha = alpha; p.beta = beta;
  p.splits = 1; p.status = status; p.row_shift = 0;
  p.group_of_mtile = group_of_mtile; p.group_rows = group_of_mtile ? N : 0; p.kb_range = nullptr;
  p.tma_store = 0;
  BsExtra x = {a_fmt, b_fmt, group_of_mtile ? N / 128 : 0, amax_a, amax_b};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return kind == 1 ? launch_gemm_bs<1>(ta, tb, tsa, tsb, p, x, st) : launch_gemm_bs<2>(ta, tb, tsa, tsb, p, x, st);
}

}  // namespace nga

extern "C" int nga_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* D, const void* aux, int M,
                              int N, int K, long long lda, long long ldb, long long ldd, long long ldaux, int a_e5m2, int b_e5m2,
                              int epi, int out_fp32, int aux_fp32, float alpha, float beta, int* status, void* stream) {
  return nga::gemm_bs_common(1, A, sfa, B, sfb, D, aux, M, N, K, lda, ldb, ldd, ldaux, a_e5m2 ? 1 : 0, b_e5m2 ? 1 : 0, epi,
                             out_fp32, aux_fp32, alpha, beta, nullptr, 0, nullptr, nullptr, status, stream);
}

extern "C" int nga_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, void* D, const void* aux, int M,
                              int N, int K, long long lda_bytes, long long ldb_bytes, long long ldd, long long ldaux, int epi,
                              int out_fp32, int aux_fp32, float alpha, float beta, const float* amax_a, const float* amax_b,
                              int* status, void* stream) {
  return nga::gemm_bs_common(2, A, sfa, B, sfb, D, aux, M, N, K, lda_bytes, ldb_bytes, ldd, ldaux, 1, 1, epi, out_fp32,
                             aux_fp32, alpha, beta, nullptr, 0, amax_a, amax_b, status, stream);
}

extern "C" int nga_gemm_grouped_bs(int kind, const void* A, const void* sfa, const void* B, const void* sfb, void* D,
                                   const int* group_of_mtile, int groups, int M, int N, int K, long long lda_bytes,
                                   long long ldb_bytes, long long ldd, float alpha, const float* amax_a, const float* amax_b,
                                   int* status, void* stream) {
  if (kind != 1 && kind != 2) return -1;
  return nga::gemm_bs_common(kind, A, sfa, B, sfb, D, nullptr, M, N, K, lda_bytes, ldb_bytes, ldd, 0, 0, 0, kEpiScale, 0, 0,
                             alpha, 0.f, group_of_mtile, groups, amax_a, amax_b, status, stream);
}
