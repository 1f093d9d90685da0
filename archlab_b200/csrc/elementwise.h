// C ABI of the memory-bound trunk kernels (see elementwise.cu for the arithmetic).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_mix_norm_fwd(const void* x, const void* x0, const float* a, const float* b, float a_scale,
                     float b_scale, void* x1, void* n, long long rows, int C, void* stream);
int nga_norm_bwd(const void* x, const void* dn, const void* dres, void* dx, int mode, const float* a,
                 const float* b, float a_scale, float b_scale, const void* xprev, const void* x0,
                 void* dx0, int dx0_init, float* da, float* db, long long rows, int C, void* stream);
int nga_embed_fwd(const long long* idx, const void* wte, const float* gate_w, const float* lam,
                  void* x0, float* gate_pre, long long rows, int T, int C, int G, void* stream);
int nga_embed_bwd(const long long* idx, const void* wte, const float* gate_w, const float* lam,
                  const float* gate_pre, const void* g, float* dwte, float* dgate_w, float* dlam,
                  long long rows, int T, int C, int G, void* stream);
int nga_qkv_post_fwd(void* qkv, const float* cosT, const float* sinT, float gain,
                     const long long* idx, const void* ve_table, const float* gate_w, const void* n,
                     int GC, int C, float* rstd, float* gate_pre, long long rows, int T, int Hq,
                     int Hkv, int D, void* stream);
int nga_qkv_post_bwd(void* dqkv, const void* qkv, const float* cosT, const float* sinT, float gain,
                     const long long* idx, const void* ve_table, const float* rstd,
                     const float* gate_pre, float* dgp, float* dve_table, long long rows, int T,
                     int Hq, int Hkv, int D, void* stream);
int nga_gate_bwd(void* dn, const void* n, const float* dgp, const float* gate_w, float* dgate_w,
                 long long rows, int C, int GC, int H, void* stream);
int nga_softcap_ce(void* logits, const long long* targets, float* loss_rows, float cap,
                   float gscale, long long rows, long long ld, int V, void* stream);
int nga_axpby_bf16(const void* x, void* y, float a, float b, long long n, void* stream);
int nga_cast_f32_bf16(const float* src, void* dst, long long n, void* stream);
#ifdef __cplusplus
}
#endif
