// C ABI of the block-scaled GEMMs (gemm_bs.cu) and of the quantisers that write their operand format
// (quant_bs.cu).
//
// Operand format.  Data: row-major, K contiguous; fp8 = one byte per element, fp4 (e2m1) = two elements per byte
// (element 2i in the low nibble).  Scales: for every 128 rows and every 4 consecutive scale factors along K one
// 512-byte chunk, byte (r % 32) * 16 + (r / 32) * 4 + j = scale j of row r of the tile; chunks ordered
// [row tile][chunk along K], nga_sf_bytes() bytes in total (rows and K padded up).  fp8 scales are ue8m0 per 32
// elements (a chunk spans 128 elements), fp4 scales ue4m3 per 16 elements (a chunk spans 64).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// Bytes of the chunked scale array of a [rows, K] matrix: kind 1 = fp8 / ue8m0 / 32, kind 2 = fp4 / ue4m3 / 16.
long long nga_sf_bytes(int kind, long long rows, long long K);

// D [M, N] (bf16, or fp32 with out_fp32) = epilogue(alpha * A . B^T); epilogues and aux as in nga_gemm2_bf16.
// lda / ldb are row pitches in BYTES (multiples of 16).  fp8: K a multiple of 32; fp4: of 64.
int nga_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* D, const void* aux, int M,
                   int N, int K, long long lda, long long ldb, long long ldd, long long ldaux, int a_e5m2, int b_e5m2,
                   int epi, int out_fp32, int aux_fp32, float alpha, float beta, int* status, void* stream);
int nga_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, void* D, const void* aux, int M,
                   int N, int K, long long lda_bytes, long long ldb_bytes, long long ldd, long long ldaux, int epi,
                   int out_fp32, int aux_fp32, float alpha, float beta, const float* amax_a, const float* amax_b,
                   int* status, void* stream);
// (amax_a / amax_b: device pointers to the tensors' absolute maxima as given to nga_quant_nvfp4, or null; alpha is
// multiplied by amax / 2688 for each, which undoes the quantisers' encode scales without a host read.)
// Expert form: B is the stack [groups * N, K] (scales likewise, N a multiple of 128) and every 256-row tile of A
// multiplies the matrix of group_of_mtile[m / 256] (device array; row segments padded to multiples of 256).
int nga_gemm_grouped_bs(int kind, const void* A, const void* sfa, const void* B, const void* sfb, void* D,
                        const int* group_of_mtile, int groups, int M, int N, int K, long long lda_bytes,
                        long long ldb_bytes, long long ldd, float alpha, const float* amax_a, const float* amax_b,
                        int* status, void* stream);

// bf16 [rows, K] (row pitch ldx elements) -> fp8 + ue8m0 scales.  block = 32 (MX) or 128 (one scale per row and
// 128 elements, replicated over its four sub-blocks); block = -128: one scale per 128 x 128 block (weights).
// Scales are powers of two: 2^ceil(log2(amax / max_normal)).  Elements past K in the last chunk count as zero.
int nga_quant_mxfp8(const void* x, void* q, void* sf, long long rows, long long K, long long ldx, long long ldq_bytes,
                    int block, int e5m2, void* stream);
// bf16 -> e2m1 pairs + ue4m3 scales per 16 elements.  `amax` (device fp32) is the absolute maximum of the tensor;
// the encode scale is 2688 / amax and the matching decode scale amax / 2688 belongs into the GEMM's alpha.
// two_d: 16 x 16 blocks share a scale (weights; rows a multiple of 16).  hadamard_seed != 0: every 16-block is
// multiplied by a sign-randomised 16 x 16 Hadamard matrix first (the same seed on both operands of a GEMM cancels
// out).  sr_seed != 0: stochastic rounding.
int nga_quant_nvfp4(const void* x, void* q, void* sf, const float* amax, long long rows, long long K, long long ldx,
                    long long ldq_bytes, int two_d, unsigned hadamard_seed, unsigned sr_seed, void* stream);
// out [n, dim] bf16 = rows idx[i] (int64, inside [0, rows)) of a frozen e4m3 table [rows, dim] times its ue8m0 scales
// [rows, dim / 32] (one per 32 columns); dim a multiple of 32.
int nga_gather_dequant_fp8(const void* weight, const void* scale, const void* idx, void* out, long long n, long long rows,
                           int dim, void* stream);
#ifdef __cplusplus
}
#endif
