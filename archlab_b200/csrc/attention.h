// C ABI of the attention kernels.  qkv is the fused projection output [B*T, (Hq + 2*Hkv) * 128]
// bf16 (q heads, then k heads, then v heads); out is [B*T, Hq*128] bf16; lse2 is [B, Hq, T] fp32
// holding log2(sum exp) of the scaled scores.  window < 0 means unlimited left context.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_attn_fwd(const void* qkv, void* out, float* lse2, int B, int T, int Hq, int Hkv, int D,
                 int window, float scale, int* status, void* stream);
void nga_attn_set_prof(long long* device_ptr);
void nga_attn_bwd_set_prof(long long* device_ptr);
// dqkv receives the gradient in the same fused layout.  `dq_acc` is fp32 scratch
// [B*T, Hq*128] that the kernel accumulates dQ into (it is zeroed by the launcher) and `delta`
// is fp32 scratch [B, Hq, T].
int nga_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse2,
                 void* dqkv, float* dq_acc, float* delta, int B, int T, int Hq, int Hkv, int D,
                 int window, float scale, int* status, void* stream);
#ifdef __cplusplus
}
#endif
