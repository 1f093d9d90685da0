// C ABI of the peer-memory (NVLink) fused collective + optimizer kernels (see peer.cu).
// `*_ptrs` are HOST arrays of `world` device addresses: the same symmetric buffer on every rank.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_peer_barrier(const long long* flag_ptrs, int rank, int world, int epoch, int* status, void* stream);
// Budget of the barrier's wait for the other ranks' flags (nanoseconds; 0 restores the 2 s default).  When it runs
// out the kernel returns and the status word reads 2; nothing hangs and the context stays usable.
void nga_set_peer_wait_budget_ns(unsigned long long ns);
unsigned long long nga_peer_wait_budget_ns(void);
int nga_peer_adamw(const long long* grad_ptrs, const long long* shadow_ptrs, float* p, float* m, float* v,
                   long long e0, long long n, int world, float lr, float beta1, float beta2, float eps, float wd,
                   int step, int cautious, void* stream);
int nga_peer_muon_momentum(const long long* grad_ptrs, float* g_out, float* m, float* norm2, long long e0, int K,
                           long long per, int world, float mu, void* stream);
int nga_peer_muon_apply(float* p, const void* x, const float* scale, const long long* shadow_ptrs, long long e0,
                        int K, int m, int n, int per_row, int world, float lr, float wd, void* stream);
#ifdef __cplusplus
}
#endif
