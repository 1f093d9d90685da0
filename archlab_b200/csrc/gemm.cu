// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma with
// the accumulator double-buffered in TMEM, and a register epilogue that fuses the elementwise tail
// (scale, residual/accumulate, ReLU^2, ReLU^2 backward) into the store.
//
//   D[b] = epi(alpha * A[b] * B[b]^T, Aux[b])        A: M x K, B: N x K  (logical shapes)
//
// Either operand may be stored K-major (K contiguous) or MN-major (its M/N index contiguous); the
// three orientations of a linear layer (forward, dgrad, wgrad) are therefore all served without a
// transposed copy.  This replaces the cuBLAS calls behind F.linear in the reference
// (src/archlab/architectures/base.py:182-190) and the batched Newton-Schulz matmuls of
// src/archlab/optimizers/speedrun.py:199-208.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (one 32-lane TMEM quarter each).
#include "gemm_common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>
#include <atomic>

namespace nga {

constexpr int kGemmThreads = 192;

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  // full[S], empty[S], tmem_full[2], tmem_empty[2], then holder + abort word
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 16 + 1024;
};

template <int BN, int A_MN, int B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + S::kStages;
  uint64_t* tfull_bar = empty_bar + S::kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = num_m * num_n * p.batch * p.splits;   // work items (tile x k-split)

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, mb, nb, otile, kb0, kb1;
        split_range(tile, p.splits, num_kb, otile, kb0, kb1);
        tile_coords(otile, num_m, num_n, b, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word);
          if (!ok) break;
          uint8_t* sA = smem + stage * S::kStageBytes;
          uint8_t* sB = sA + S::kABytes;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sA + j * 8192, &tmA, &full_bar[stage], m0 + j * 64, kb * BK, b);
          } else {
            tma_load_3d(sA, &tmA, &full_bar[stage], kb * BK, m0, b);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * 8192, &tmB, &full_bar[stage], n0 + j * 64, kb * BK, b);
          } else {
            tma_load_3d(sB, &tmB, &full_bar[stage], kb * BK, n0, b);
          }
          if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + uint32_t(acc * BN);
        int otile, kb0, kb1;
        split_range(tile, p.splits, num_kb, otile, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_word);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sB = sA + S::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc(sA + k * (UMMA_K * 128), 8192, 1024)
                                     : umma_smem_desc(sA + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sB + k * (UMMA_K * 128), 8192, 1024)
                                     : umma_smem_desc(sB + k * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = epilogue_vec_ok(p);
    const bool need_aux = (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2);
    const bool aux_fast = aux_prefetchable(p);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int b, mb, nb, otile, kb0, kb1;
      split_range(tile, p.splits, num_kb, otile, kb0, kb1);
      tile_coords(otile, num_m, num_n, b, mb, nb);
      const int row = mb * BM + quarter * 32 + lane;
      AuxPre nxt;
      aux_prefetch(p, nxt, row, nb * BN, b, aux_fast);      // in flight while the main loop finishes
      ok = __all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, abort_word));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + uint32_t(acc * BN) + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
      for (int c2 = 0; c2 < BN / 64; ++c2) {
        if (nb * BN + c2 * 64 >= p.N) break;   // warp-uniform
        const AuxPre cur = nxt;
        if (c2 + 1 < BN / 64) aux_prefetch(p, nxt, row, nb * BN + (c2 + 1) * 64, b, aux_fast);
        // two 32-column chunks per TMEM round trip
        uint32_t r2[2][32];
        tmem_ld_32x32(taddr + uint32_t(c2 * 64), r2[0]);
        tmem_ld_32x32(taddr + uint32_t(c2 * 64 + 32), r2[1]);
        tmem_ld_wait();
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          const int col0 = nb * BN + (c2 * 2 + hc) * 32;
          if (col0 >= p.N) break;   // warp-uniform
          epilogue_store_chunk(p, r2[hc], row, col0, b, vec_ok, need_aux, cur.valid[hc] ? cur.v[hc] : nullptr);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

}  // namespace nga

// ------------------------------------------------------------------------------------------------
// Host launcher
// ------------------------------------------------------------------------------------------------
#include "host_util.h"

namespace nga {

template <int BN, int A_MN, int B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                       cudaStream_t stream) {
  using S = GemmSmem<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static nga::PerDevice<bool> attr_flags;
  bool& attr_done = attr_flags.here();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -1000 - (int)e;
    attr_done = true;
  }
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch * p.splits;
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  kern<<<grid, kGemmThreads, S::kTotal, stream>>>(ta, tb, p);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

}  // namespace nga

extern "C" int nga_gemm_bf16(const void* A, const void* B, void* D, const void* aux, int M, int N,
                             int K, int batch, long long lda, long long ldb, long long ldd,
                             long long ldaux, long long sA, long long sB, long long sD,
                             long long sAux, int a_mn, int b_mn, int epi, int out_fp32,
                             int aux_fp32, float alpha, float beta, int splits, int* status, void* stream) {
  using namespace nga;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -1;
  if ((lda & 7) || (ldb & 7) || (sA & 7) || (sB & 7)) return -5;
  // Tile width: 256 when that still fills the machine, else 128 (more, smaller tiles).
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256) * batch;
  const bool bn256 = (N > 128) && tiles256 >= sm_count();
  const int BNsel = bn256 ? 256 : 128;
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
                      (batch > 1 ? sB : (long long)N * ldb) * 2, 64, BNsel, true);
  if (rc) return rc;
  GemmParams p;
  p.row_shift = 0;
  p.group_of_mtile = nullptr; p.group_rows = 0; p.kb_range = nullptr;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.D = D; p.aux = aux; p.ldd = ldd; p.ldaux = ldaux; p.sD = sD; p.sAux = sAux;
  p.epi = epi; p.out_fp32 = out_fp32; p.aux_fp32 = aux_fp32; p.alpha = alpha; p.beta = beta;
  {
    const int num_kb = (K + BK - 1) / BK;
    int sp = (epi == kEpiAtomicAdd && splits > 1) ? (splits < num_kb ? splits : num_kb) : 1;
    const int per = (num_kb + sp - 1) / sp;
    p.splits = (num_kb + per - 1) / per;       // every split is non-empty
  }
  if (epi == kEpiAtomicAdd && !out_fp32) return -8;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NGA_DISPATCH(BNV)                                                    \
  if (a_mn && b_mn) return launch_gemm<BNV, 1, 1>(ta, tb, p, st);            \
  if (a_mn && !b_mn) return launch_gemm<BNV, 1, 0>(ta, tb, p, st);           \
  if (!a_mn && b_mn) return launch_gemm<BNV, 0, 1>(ta, tb, p, st);           \
  return launch_gemm<BNV, 0, 0>(ta, tb, p, st);
  if (bn256) { NGA_DISPATCH(256) }
  NGA_DISPATCH(128)
#undef NGA_DISPATCH
}
