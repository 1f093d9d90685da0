// Pieces shared by the single-CTA and the CTA-pair GEMM kernels: parameter block, tile order and the
// register epilogue (scale / axpby / ReLU^2 / ReLU^2-backward, bf16 or fp32 output).
#pragma once
#include <cuda.h>
#include "ptx.cuh"
#include "gemm.h"

namespace nga {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

struct GemmParams {
  int M, N, K, batch;
  void* D;
  const void* aux;
  long long ldd, ldaux;          // row strides (elements)
  long long sD, sAux;            // batch strides (elements)
  int epi, out_fp32, aux_fp32;
  float alpha, beta;
  int splits;                    // split-K factor (> 1 only with kEpiAtomicAdd)
  int* status;
  long long row_shift;           // added to the row index when addressing D (tensor-parallel staging slots)
  // grouped form (expert GEMMs in one launch): rows are sorted by group and every 256-row tile belongs to one
  // group; `group_of_mtile[mb]` names it and B is the stack of the groups' matrices, `group_rows` rows each
  // A negative entry marks a tile of the (fixed, upper-bound) row range that holds no rows: every role skips it.
  const int* group_of_mtile;
  int group_rows;
  // variable-length reductions (grouped weight gradients): batch element b reduces over the 64-row blocks
  // [kb_range[2b], kb_range[2b + 1]) of the shared A / B row range; an empty range skips the tile (its output keeps
  // what the caller put there)
  const int* kb_range;
  int tma_store;                 // pair kernel, plain bf16 output: tiles leave through swizzled staging + TMA stores
};

// Tensor-parallel fusion of the CTA-pair GEMM with its collective over NVLink peer memory.
//   kTpGather : A = concatenation over ranks of row shards [rows_per_rank, K].  `copy_clusters`
//               clusters pull the remote shards into the local `gathered` buffer with bulk copies (each
//               remote byte crosses NVLink once; one SM sustains ~17 GB/s of such copies, so about two
//               dozen CTAs are needed to keep a link busy) and publish 128-row blocks through `flags`;
//               the GEMM clusters start on this rank's own rows (read straight from the shard) and wait
//               (bounded) for a block before loading it.
//   kTpScatter: D row blocks belong to the rank that owns those rows; tiles are stored straight into
//               that rank's staging buffer at slot `rank` ([world][rows_per_rank, ldd]), remote owners
//               first, so the reduce-scatter traffic overlaps the remaining tiles.
constexpr int kTpMaxWorld = 8;
constexpr int kTpGather = 1;
constexpr int kTpScatter = 2;
// kTpGatherB: the B operand (a weight [N, K] whose row shards live on the ranks of a data-parallel group)
//               is gathered by the copy clusters exactly as kTpGather gathers A; the GEMM clusters start on
//               the output columns of this rank's own shard (read straight from it) and wait (bounded) for
//               the 128-row blocks of the other shards.  A [M, K] and D [M, N] are local.
constexpr int kTpGatherB = 4;
// kTpGatherBk: the same gather for an MN-major B whose rows are the reduction dimension (the data gradient
//               dX = dY . W of a fully-sharded weight): every tile walks the k-blocks starting at this rank's
//               own shard and waits (bounded) for each block of the others the first time it needs it.
constexpr int kTpGatherBk = 8;
constexpr int kTpGatherAny = kTpGather | kTpGatherB | kTpGatherBk;
// kTpPush (with kTpGather): owner-push all-gather.  No copy clusters: at kernel start the epilogue warps of every CTA
//               STORE this rank's row shard, 128-row block by block, into every rank's gathered buffer (`peer_dst`,
//               remote ranks first) and publish each block with a release store to that rank's flag array
//               (`peer_flags`).  Posted stores need no round trip, so a few dozen SMs fill the link, and they run under
//               the main loops of the first tiles, which are this rank's own rows (read straight from the shard).
constexpr int kTpPush = 16;
// kTpReduce (with kTpScatter): the reduce-scatter is finished inside the GEMM kernel.  Tiles of remote owners come
//               first: stored into the owner's slot as before, then every epilogue warp adds one to the owner's
//               arrival counter of that tile (`peer_flags`, release at system scope, after its bulk stores have
//               completed).  Tiles this rank owns come last: their epilogue waits (bounded) until the counter shows all
//               remote partial tiles, then adds them (and the residual) to the accumulator and writes the final rows -
//               no barrier kernels and no separate reduction pass.
constexpr int kTpReduce = 32;
struct TpParams {
  int mode, rank, world, rows_per_rank;
  int copy_clusters, epoch;
  int row_elems;                       // elements per row of the gathered matrix
  int early_rounds;                    // >= 0: the copy clusters compute tiles too once their copies are done; the first
                                       // early_rounds rounds of tiles belong to the GEMM clusters alone.  < 0: copy only
  int* flags;                          // one per 128-row block of the gathered matrix; value = epoch when ready
  const void* peer_src[kTpMaxWorld];   // row shard of every rank (bf16, contiguous rows of K elements, symmetric)
  void* gathered;                      // local [world * rows_per_rank, K] bf16
  void* peer_dst[kTpMaxWorld];         // reduce-scatter staging buffer of every rank; kTpPush: gathered buffer of every rank
  int* peer_flags[kTpMaxWorld];        // kTpPush: block flags of every rank; kTpReduce: tile arrival counters of every rank
  const void* push_src;                // kTpPush: this rank's row shard [rows_per_rank, row_elems]
  int push_parts;                      // kTpPush: row slices per 128-row block (1, 2 or 4); a block counter reads epoch * parts
  const void* resid;                   // kTpReduce: optional residual [rows_per_rank, ld_resid] added to the owned rows
  void* reduce_out;                    // kTpReduce: final [rows_per_rank, ld_out] bf16 rows of this rank
  long long ld_resid, ld_out, ld_slot; // row pitches (elements) of residual, output and staging slots
  int arrivals;                        // kTpReduce: counter value at which a tile of this call is complete
};

// Tensor maps of the reduce-scatter staging buffer on every rank ([world * rows_per_rank, ldd] bf16,
// box 64 columns x 32 rows, 128-byte swizzle): output tiles leave through TMA stores, so the NVLink
// write stream consists of full 128-byte lines.
struct TpMaps {
  CUtensorMap d[kTpMaxWorld];
};

// The tiles of one cluster in launch order.  Without a gather every cluster strides through the tile list.  With
// copy clusters that join late, the first `early_n` rounds are dealt to the GEMM clusters only and the rest to all
// clusters, so that the copy clusters (which start on tiles when their copies are done) finish with the others.
struct TileSeq {
  int first, early_n, early_step, late_first, late_step;
  __device__ __forceinline__ int at(int i) const {
    return i < early_n ? first + i * early_step : late_first + (i - early_n) * late_step;
  }
};

__device__ __forceinline__ int tp_remap_mb(const TpParams& tp, int mb, int num_m) {
  if (tp.mode == 0 || (tp.mode & (kTpGatherB | kTpGatherBk))) return mb;
  const int per = tp.rows_per_rank / (2 * BM);
  const int first = (tp.mode & kTpGather) ? tp.rank * per : ((tp.rank + 1) % tp.world) * per;
  int r = mb + first;
  return r >= num_m ? r - num_m : r;
}

// Column-tile order under kTpGatherB: this rank's own shard first, then the shards in the order the copy
// clusters fetch them (rank + 1, rank + 2, ...).
__device__ __forceinline__ int tp_remap_nb(const TpParams& tp, int nb, int num_n) {
  if (!(tp.mode & kTpGatherB)) return nb;
  const int r = nb + tp.rank * (tp.rows_per_rank / 256);
  return r >= num_n ? r - num_n : r;
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& b, int& mb, int& nb) {
  const int per_batch = num_m * num_n;
  b = tile / per_batch;
  int r = tile - b * per_batch;
  constexpr int kGroup = 16;
  const int per_group = kGroup * num_n;
  const int g = r / per_group;
  r -= g * per_group;
  const int first_m = g * kGroup;
  const int gm = min(kGroup, num_m - first_m);
  mb = first_m + r % gm;
  nb = r / gm;
}

// Work item -> (output tile index, k-block range) under split-K.
// Grouped forms: whether this tile has anything to do, and (variable-length reductions) its range of 64-row blocks.
// Every role of the kernel asks the same question of the same device tables, so they skip the same tiles.
__device__ __forceinline__ bool tile_has_work(const GemmParams& p, int b, int mb, int& kb0, int& kb1) {
  if (p.group_of_mtile != nullptr && p.group_of_mtile[mb] < 0) return false;
  if (p.kb_range != nullptr) {
    kb0 = p.kb_range[2 * b];
    kb1 = p.kb_range[2 * b + 1];
    return kb1 > kb0;
  }
  return true;
}

__device__ __forceinline__ void split_range(int item, int splits, int num_kb, int& tile, int& kb0, int& kb1) {
  const int sidx = item % splits;
  tile = item / splits;
  const int per = (num_kb + splits - 1) / splits;
  kb0 = sidx * per;
  kb1 = min(num_kb, kb0 + per);
}

template <int EPI>
__device__ __forceinline__ float epi_apply(float acc, float aux, float alpha, float beta) {
  if constexpr (EPI == kEpiAxpby) return alpha * acc + beta * aux;
  if constexpr (EPI == kEpiRelu2) { float r = fmaxf(alpha * acc, 0.f); return r * r; }
  if constexpr (EPI == kEpiMulDRelu2) {
    // d/dh relu(h)^2 = 2 relu(h) = 2 sqrt(aux); one MUFU op (the IEEE sqrt sequence costs ~30
    // instructions per element and made this epilogue issue-bound), bf16 output hides the 1-ulp error
    float rt;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(rt) : "f"(fmaxf(aux, 0.f)));
    return alpha * acc * 2.f * rt;
  }
  return alpha * acc;   // kEpiScale, kEpiAtomicAdd
}

// Applies the epilogue to one 32-column chunk of one accumulator row and stores it.
// r: the 32 fp32 accumulator values of (row, col0 .. col0+31); b: batch index.
// Register prefetch of the bf16 aux operand for two adjacent 32-column chunks of one row.  Issued
// before the accumulator is read, so the global-load latency overlaps the main loop / TMEM reads
// instead of serialising the epilogue (which made K <= 1280 GEMMs with an aux epilogue-bound).
struct AuxPre {
  uint4 v[2][4];
  bool valid[2];
};
__device__ __forceinline__ void aux_prefetch(const GemmParams& p, AuxPre& a, int row, int col_pair0, int b,
                                             bool fast) {
#pragma unroll
  for (int hc = 0; hc < 2; ++hc) {
    const int col0 = col_pair0 + hc * 32;
    a.valid[hc] = fast && row < p.M && col0 + 32 <= p.N;
    if (a.valid[hc]) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.aux) +
                                                        (long long)b * p.sAux + (long long)row * p.ldaux + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) a.v[hc][q] = src[q];
    }
  }
}
__device__ __forceinline__ bool aux_prefetchable(const GemmParams& p) {
  return (p.epi == kEpiAxpby || p.epi == kEpiMulDRelu2) && !p.aux_fp32 && (p.ldaux & 7) == 0 &&
         (p.sAux & 7) == 0 && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0;
}

// The epilogue mode is a template parameter: the per-element arithmetic must not branch on it (a
// run-time switch per element made every K <= 1280 GEMM epilogue-bound).
template <int EPI>
__device__ __forceinline__ void epilogue_chunk_t(const GemmParams& p, const uint32_t (&r)[32], int row, int col0,
                                                 int b, bool vec_ok, const uint4* pre) {
  constexpr bool kNeedAux = (EPI == kEpiAxpby || EPI == kEpiMulDRelu2);
  if (row >= p.M) return;
  const long long doff = (long long)b * p.sD + ((long long)row + p.row_shift) * p.ldd + col0;
  const int ncol = min(32, p.N - col0);
  const float alpha = p.alpha, beta = p.beta;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  if constexpr (kNeedAux) {
    const long long aoff = (long long)b * p.sAux + (long long)row * p.ldaux + col0;
    if (p.aux_fp32) {
      const float* ax = reinterpret_cast<const float*>(p.aux) + aoff;
      if (ncol == 32 && (p.ldaux & 3) == 0 && (p.sAux & 3) == 0 && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 f = reinterpret_cast<const float4*>(ax)[q];
          v[4 * q] = epi_apply<EPI>(v[4 * q], f.x, alpha, beta);
          v[4 * q + 1] = epi_apply<EPI>(v[4 * q + 1], f.y, alpha, beta);
          v[4 * q + 2] = epi_apply<EPI>(v[4 * q + 2], f.z, alpha, beta);
          v[4 * q + 3] = epi_apply<EPI>(v[4 * q + 3], f.w, alpha, beta);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = epi_apply<EPI>(v[i], i < ncol ? ax[i] : 0.f, alpha, beta);
      }
    } else {
      const __nv_bfloat16* ax = reinterpret_cast<const __nv_bfloat16*>(p.aux) + aoff;
      if (pre != nullptr || (ncol == 32 && (p.ldaux & 7) == 0 && (p.sAux & 7) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0)) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 pk = pre ? pre[q] : reinterpret_cast<const uint4*>(ax)[q];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[q * 8 + 2 * i] = epi_apply<EPI>(v[q * 8 + 2 * i], f.x, alpha, beta);
            v[q * 8 + 2 * i + 1] = epi_apply<EPI>(v[q * 8 + 2 * i + 1], f.y, alpha, beta);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          v[i] = epi_apply<EPI>(v[i], i < ncol ? __bfloat162float(ax[i]) : 0.f, alpha, beta);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = epi_apply<EPI>(v[i], 0.f, alpha, beta);
  }
  if constexpr (EPI == kEpiAtomicAdd) {
    // split-K partial sums: fp32 vector reductions into the (pre-existing) output
    float* d = reinterpret_cast<float*>(p.D) + doff;
    if (ncol == 32 && vec_ok) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        atomicAdd(reinterpret_cast<float4*>(d) + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncol) atomicAdd(d + i, v[i]);
    }
  } else if (p.out_fp32) {
    float* d = reinterpret_cast<float*>(p.D) + doff;
    if (ncol == 32 && vec_ok) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        reinterpret_cast<float4*>(d)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncol) d[i] = v[i];
    }
  } else {
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + doff;
    if (ncol == 32 && vec_ok) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 pk;
        pk.x = pack_bf16(v[8 * q], v[8 * q + 1]);
        pk.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
        pk.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]);
        pk.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
        reinterpret_cast<uint4*>(d)[q] = pk;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncol) d[i] = __float2bfloat16(v[i]);
    }
  }
}

// Staging form of the epilogue for TMA stores: applies the epilogue to one 32-column chunk of one accumulator row
// and writes the bf16 result into this lane's 128-byte row of a 32 x 64 staging tile (128-byte swizzle; `half`
// selects columns 0..31 or 32..63 of the tile).  `pre` holds the row's 32 bf16 aux values (nullptr: zeros; the
// caller only uses this form when every chunk inside the matrix has them).
template <int EPI>
__device__ __forceinline__ void epilogue_stage_t(const GemmParams& p, const uint32_t (&r)[32], const uint4* pre,
                                                 uint8_t* buf, int lane, int half) {
  constexpr bool kNeedAux = (EPI == kEpiAxpby || EPI == kEpiMulDRelu2);
  const float alpha = p.alpha, beta = p.beta;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
    if constexpr (kNeedAux) {
      if (pre != nullptr) {
        const uint4 pk = pre[q];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          a[2 * i] = f.x;
          a[2 * i + 1] = f.y;
        }
      }
    }
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = epi_apply<EPI>(__uint_as_float(r[q * 8 + i]), a[i], alpha, beta);
    uint4 o;
    o.x = pack_bf16(v[0], v[1]);
    o.y = pack_bf16(v[2], v[3]);
    o.z = pack_bf16(v[4], v[5]);
    o.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4*>(buf + lane * 128 + (((half * 4 + q) ^ (lane & 7)) * 16)) = o;
  }
}
__device__ __forceinline__ void epilogue_stage_chunk(const GemmParams& p, const uint32_t (&r)[32], const uint4* pre,
                                                     uint8_t* buf, int lane, int half) {
  switch (p.epi) {
    case kEpiAxpby: epilogue_stage_t<kEpiAxpby>(p, r, pre, buf, lane, half); break;
    case kEpiRelu2: epilogue_stage_t<kEpiRelu2>(p, r, pre, buf, lane, half); break;
    case kEpiMulDRelu2: epilogue_stage_t<kEpiMulDRelu2>(p, r, pre, buf, lane, half); break;
    default: epilogue_stage_t<kEpiScale>(p, r, pre, buf, lane, half); break;
  }
}

__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, const uint32_t (&r)[32], int row,
                                                     int col0, int b, bool vec_ok, bool /*need_aux*/,
                                                     const uint4* pre = nullptr) {
  switch (p.epi) {
    case kEpiAxpby: epilogue_chunk_t<kEpiAxpby>(p, r, row, col0, b, vec_ok, pre); break;
    case kEpiRelu2: epilogue_chunk_t<kEpiRelu2>(p, r, row, col0, b, vec_ok, pre); break;
    case kEpiMulDRelu2: epilogue_chunk_t<kEpiMulDRelu2>(p, r, row, col0, b, vec_ok, pre); break;
    case kEpiAtomicAdd: epilogue_chunk_t<kEpiAtomicAdd>(p, r, row, col0, b, vec_ok, pre); break;
    default: epilogue_chunk_t<kEpiScale>(p, r, row, col0, b, vec_ok, pre); break;
  }
}

__device__ __forceinline__ bool epilogue_vec_ok(const GemmParams& p) {
  return p.out_fp32 ? ((p.ldd & 3) == 0 && (p.sD & 3) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0)
                    : ((p.ldd & 7) == 0 && (p.sD & 7) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0);
}

}  // namespace nga
