// C ABI of the 2-simplicial attention kernels.  All tensors are bf16 with head_dim 128, laid out as
// [B*N rows, heads*128 columns] with explicit row strides (elements), so they may be column slices
// of one fused projection output.  lse2 is [B, Hq, N] fp32 (log2 domain).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_simplicial_fwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* out,
                       float* lse2, long long ldq, long long ldk1, long long ldk2, long long ldv1, long long ldv2,
                       long long ldo, int B, int N, int Hq, int Hkv, int D, int w1, int w2, float scale,
                       int* status, void* stream);
#ifdef __cplusplus
}
#endif
