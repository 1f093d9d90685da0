// C ABI of the native library (loaded with ctypes).  All pointers are device pointers unless a
// comment says otherwise; `stream` is a cudaStream_t passed as void*.  Functions return 0 on
// success or a negative number for a host-side error (bad shape / alignment / CUDA launch error).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Epilogue selector of nga_gemm_bf16.
enum {
  kEpiScale = 0,      // D = alpha * acc
  kEpiAxpby = 1,      // D = alpha * acc + beta * aux        (aux may alias D)
  kEpiRelu2 = 2,      // D = relu(alpha * acc)^2
  kEpiMulDRelu2 = 3,  // D = alpha * acc * 2 * sqrt(aux)     (aux = relu(h)^2 saved by kEpiRelu2)
  kEpiAtomicAdd = 4,  // D(fp32) += alpha * acc with vector atomics; allows split-K (splits > 1)
};

// D[b] = epi(alpha * A[b] * B[b]^T).  A is M x K, B is N x K (logical).  a_mn / b_mn = 1 when the
// operand is stored with its M (resp. N) index contiguous, i.e. as a K x M (K x N) row-major
// array; lda / ldb are then the strides between consecutive K rows.  Strides are in elements;
// lda, ldb and the batch strides must be multiples of 8 and the base pointers 16-byte aligned.
int nga_gemm_bf16(const void* A, const void* B, void* D, const void* aux, int M, int N, int K,
                  int batch, long long lda, long long ldb, long long ldd, long long ldaux,
                  long long sA, long long sB, long long sD, long long sAux, int a_mn, int b_mn,
                  int epi, int out_fp32, int aux_fp32, float alpha, float beta, int splits,
                  int* status, void* stream);

// CTA-pair (cta_group::2, 256 x 256 tile) variant with the same contract; best for large problems.
int nga_gemm2_bf16(const void* A, const void* B, void* D, const void* aux, int M, int N, int K,
                   int batch, long long lda, long long ldb, long long ldd, long long ldaux,
                   long long sA, long long sB, long long sD, long long sAux, int a_mn, int b_mn,
                   int epi, int out_fp32, int aux_fp32, float alpha, float beta, int splits,
                   int* status, void* stream);

// Owner-push all-gather -> GEMM and GEMM -> reduce-scatter finished in the kernel (gemm2.cu; no barrier kernels, no copy
// clusters, no separate reduction pass).  `*_ptrs` are HOST arrays of `world` device addresses of symmetric buffers.
int nga_tp_gemm_push_bf16(const void* x_local, const void* B, void* D, int M, int N, int K, long long ldb, long long ldd,
                          int b_mn, int rank, int world, int rows_per_rank, const long long* gathered_ptrs,
                          const long long* flag_ptrs, int epoch, int* status, void* stream);
int nga_tp_gemm_rs_reduce_bf16(const void* A, const void* B, void* out, const void* resid, int M, int N, int K, long long ldb,
                               long long ld_out, long long ld_resid, int b_mn, int rank, int world, int rows_per_rank,
                               const long long* slot_ptrs, const long long* counter_ptrs, int call_index, int* status,
                               void* stream);

// Tensor-parallel GEMM fused with its collective over NVLink peer memory (CTA-pair kernel).
// mode 1: all-gather of A row shards -> GEMM; mode 2: GEMM -> reduce-scatter of D row blocks into the
// owners' staging slots, summed by nga_tp_reduce_slots after a cross-rank barrier.  See gemm2.cu.
int nga_tp_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long ldb, long long ldd,
                     int b_mn, int mode, int rank, int world, int rows_per_rank, const long long* src_ptrs,
                     void* gathered, int* flags, int epoch, int copy_clusters, const long long* dst_ptrs,
                     int* status, void* stream);
// Fully-sharded weight [w_rows, w_cols] in row shards on the ranks of a group: D = A . W^T (transposed = 0) or
// D = A . W (transposed = 1), with the gather done by copy clusters of the same kernel (see gemm2.cu).
int nga_fsdp_gemm_bf16(const void* A, void* D, int M, int w_rows, int w_cols, long long lda, long long ldd, int transposed,
                       int rank, int world, int rows_per_rank, const long long* src_ptrs, void* gathered, int* flags,
                       int epoch, int copy_clusters, int* status, void* stream);
int nga_tp_reduce_slots(const void* stage, const void* resid, void* out, int world, long long rows, int N,
                        long long ld_stage, long long ld_resid, long long ld_out, void* stream);

// Number of kernels this library has launched since load (every launcher increments it).
long long nga_launch_count(void);
void nga_launch_count_reset(void);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
int nga_gemm2_fp8(const void* A, const void* B, void* D, const void* aux, int M, int N, int K, long long lda, long long ldb,
                  long long ldd, long long ldaux, int a_e5m2, int b_e5m2, int epi, int out_fp32, int aux_fp32, float alpha,
                  float beta, int* status, void* stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
int nga_gemm2_grouped_bf16(const void* A, const void* B, void* D, const int* group_of_mtile, int groups, int M, int N, int K,
                           long long lda, long long ldb, long long ldd, int b_mn, int* status, void* stream);
#ifdef __cplusplus
}
#endif
