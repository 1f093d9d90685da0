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
// Allocation-free form of nga_attn_bwd: same inputs and outputs, but the two scratch buffers are
// fixed arrays inside the loaded module instead of caller memory, so the call performs no device
// allocation at all.  For hosts that drive the C ABI without a tensor allocator or that must not
// allocate once running.  Accepts B*T*Hq*128 <= nga_attn_bwd_static_max_elems() (4 Mi fp32 elements,
// 16 MiB); returns -20 beyond that.  Calls that may overlap on one device race on the shared
// scratch; order them.  The first call per device resolves the arrays' addresses and should be made
// outside stream capture.  The current device must be the one that owns the buffers and the stream
// (the scratch used is the current device's; a dqkv that lives on another device returns -22).
// This entry point has no counterpart in the reference project.
int nga_attn_bwd_static(const void* qkv, const void* out, const void* dout, const float* lse2,
                        void* dqkv, int B, int T, int Hq, int Hkv, int D, int window, float scale,
                        int* status, void* stream);
long long nga_attn_bwd_static_max_elems(void);
#ifdef __cplusplus
}
#endif
