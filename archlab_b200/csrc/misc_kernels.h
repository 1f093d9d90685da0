// C ABI of the single-pass model-zoo kernels (see misc_kernels.cu).  bf16 tensors unless noted.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int nga_rmsnorm(const void* x, const float* weight, void* y, long long rows, int groups, int width, float eps,
                int zero_centered, void* stream);
int nga_rope(void* x, const float* cos_t, const float* sin_t, long long rows, int T, int H, int D, int rot, int interleaved,
             void* stream);
int nga_router_topk(const void* x, const void* w, const float* bias, float* out_w, int* out_idx, float* out_scores, int T,
                    int C, int E, int k, int score_fn, float route_scale, int renorm, void* stream);
int nga_causal_conv1d(const void* x, const float* w, const float* bias, void* y, int B, int T, int Cc, int K, int dil,
                      int silu, void* stream);
int nga_ngram_hash(const long long* tok, const int* seg_start, const long long* mult, const long long* sizes,
                   const long long* offsets, long long* ids, int B, int T, int n, int heads_per_order, long long eos,
                   void* stream);
int nga_fp8_block_quant(const void* x, void* q, float* scales, long long n, int block, int pow2, void* stream);
int nga_nvfp4_quant(const void* x, void* vals, void* bscale, float tensor_scale, long long n, void* stream);
int nga_stochastic_bf16(const float* x, void* y, long long n, unsigned long long seed, void* stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
int nga_rmsnorm_bwd(const void* x, const float* weight, const void* dy, void* dx, float* dw, long long rows, int groups,
                    int width, float eps, int zero_centered, void* stream);
int nga_swiglu_bwd(const void* h, const void* dout, void* dh, long long rows, int inter, float limit, void* stream);
int nga_ce_inplace(void* logits, const long long* targets, float* loss_rows, float gscale, long long rows, long long ld,
                   int V, long long ignore_index, void* stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
long long nga_gdn_workspace_bytes(int B, int T, int H);
int nga_gdn_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o, const float* s0,
                float* s_out, void* workspace, int B, int T, int H, int D, int* status, void* stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
int nga_token_mix(const void* in_a, const void* in_b, const float* W, void* out, long long tokens, int na, int nb, int n_out, int C,
                  int transpose_w, void* stream);
int nga_token_mix_dw(const void* dout, const void* in_a, const void* in_b, float* dW, long long tokens, int na, int nb, int n_out,
                     int C, void* stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
int nga_indexer_select(const void* q, const void* k, const float* w, void* bits, int B, int S, int heads, int dim, int top_k,
                       float scale, void* stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
int nga_hc_coeff_fwd(const float* mixes, const float* scale, const float* base, float* pre, float* post, float* comb, long long T,
                     int streams, int iters, float eps, void* stream);
int nga_hc_coeff_bwd(const float* mixes, const float* scale, const float* base, const float* dpre, const float* dpost,
                     const float* dcomb, float* dmixes, float* dscale, float* dbase, long long T, int streams, int iters, float eps,
                     void* stream);
#ifdef __cplusplus
}
#endif
