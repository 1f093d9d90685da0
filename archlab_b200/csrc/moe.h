// C ABI of the expert-parallel MoE exchange kernels over peer memory (see moe.cu).  `*_ptrs` are host
// arrays of `world` device addresses of the same symmetric buffer on every rank.  Index arrays are
// int32 on the device; a negative rank marks a dropped slot.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_moe_push_rows(const void* rows, const int* src_row, const int* dst_rank, const int* dst_row, const float* scale,
                      const long long* dst_ptrs, int world, int n, int C, void* stream);
int nga_moe_pull_combine(const long long* src_ptrs, int world, const int* rank, const int* row, const float* weight,
                         const void* gout, void* out, float* out_f32, float* dweight, int T, int k, int C, void* stream);
int nga_swiglu_clamped(const void* h, const float* prob, void* out, long long rows, int inter, float limit, void* stream);
#ifdef __cplusplus
}
#endif
