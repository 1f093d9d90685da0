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
// Backward.  `out` / `lse2` are the forward results, `dout` the incoming gradient [B*N, Hq*128].
// dq, dk1, dk2, dv1, dv2 receive bf16 gradients with the given row strides.  Scratch (fp32):
// dk1_acc, dv1_acc [B*N, Hkv*128] (zeroed inside), dk2_acc, dv2_acc (same shape; needed only when
// Hq > Hkv, may be null otherwise) and delta [B, Hq, N].
int nga_simplicial_bwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                       const void* out, const void* dout, const float* lse2, void* dq, void* dk1, void* dk2,
                       void* dv1, void* dv2, float* dk1_acc, float* dv1_acc, float* dk2_acc, float* dv2_acc, float* delta,
                       long long ldq,
                       long long ldk1, long long ldk2, long long ldv1, long long ldv2, long long ldo, long long lddo,
                       long long lddq, long long lddk1, long long lddk2, long long lddv1, long long lddv2, int B,
                       int N, int Hq, int Hkv, int D, int w1, int w2, float scale, int* status, void* stream);
// Atomic-free, bit-reproducible mode for the next nga_simplicial_bwd call of the calling thread: fp32 scratch for the
// per-row short-key contributions ([B*N * w1 * Hq, 128] each) and, when Hq > Hkv, for the per-head planes of the long-key
// gradients ([Hq / Hkv][B*N, Hkv*128] each; null otherwise).  Without this call dk1 / dv1 (and dk2 / dv2 under GQA)
// are accumulated with fp32 vector atomics, whose order varies from run to run.
void nga_simplicial_bwd_set_deterministic(float* dk1_part, float* dv1_part, float* dk2_part, float* dv2_part);
#ifdef __cplusplus
}
#endif
