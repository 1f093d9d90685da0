// C ABI of the fused optimizer kernels (see optim.cu).  fp32 master / gradient / moment buffers,
// bf16 shadows; element counts must be multiples of 4.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_adamw(float* p, const float* g, float* m, float* v, void* shadow, long long n, float lr, float beta1,
              float beta2, float eps, float wd, int step, int cautious, void* stream);
int nga_muon_momentum(float* g, float* m, float* norm2, int K, long long per, float mu, void* stream);
int nga_muon_normalize(const float* g, const float* norm2, void* x, int K, long long per, void* stream);
int nga_sq_mean(const void* x, float* out, int K, int m, int n, int along_rows, void* stream);
int nga_muon_apply(float* p, const void* x, const float* scale, void* shadow, int K, int m, int n, int per_row,
                   float lr, float wd, void* stream);
#ifdef __cplusplus
}
#endif
