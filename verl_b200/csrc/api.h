// C entry points of the sm_100a kernel library (no libtorch dependency). All functions return 0 on success and a
// negative code for rejected arguments; kernels with device-side waits report run-time failures through `err_word`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int vb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
                 int a_mn, int b_mn, int out_f32, int accumulate, int bn, int* err_word, cudaStream_t stream);

int vb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd, int T, int H,
                   float eps, cudaStream_t st);
int vb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx, float* dw,
                   int T, int H, cudaStream_t st);
int vb_rope(void* x, const int* pos, const float* cs, const float* sn, int T, int nheads, int D, long ld, float sign,
            cudaStream_t st);
int vb_swiglu_fwd(const void* gu, void* out, long T, int I, cudaStream_t st);
int vb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long T, int I, cudaStream_t st);
int vb_adamw(float* p32, float* m, float* v, const void* g, int g_is_bf16, void* p16, long n, float lr, float b1, float b2,
             float eps, float wd, int step, const float* scalars, cudaStream_t st);
int vb_sqnorm(const void* g, int is_bf16, long n, float* out, cudaStream_t st);
int vb_clip_coef(const float* sumsq, float max_norm, float* scalars, cudaStream_t st);

#ifdef __cplusplus
}
#endif
