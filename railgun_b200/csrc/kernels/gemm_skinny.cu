// The plain entry point of the weight-streaming decode product (gemm_skinny.cuh has the kernel).
#include "gemm_skinny.cuh"

// out_dtype: RG_DTYPE_BF16 or RG_DTYPE_F32.  epilogue: 0 plain (out [M, N]); 1 SiLU-mul over interleaved gate|up rows
// (out [M, N / 2]).  Refuses M > 64, K % 8 != 0 and, for the SiLU-mul epilogue, N % 16 != 0.
extern "C" int rg_skinny_gemm(const void* W, const void* x, int ldx, void* out, int ldo, int out_dtype, int epilogue,
                              int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K % 8 || K <= 0 || ldx % 8) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const bf16* w = (const bf16*)W;
    const bf16* xx = (const bf16*)x;
    const SkinnyFusion none = {};
    if (epilogue == EPI_SILU_MUL) {
        if (N % 16 || out_dtype != RG_DTYPE_BF16) return RG_ERR_UNSUPPORTED;
        return dispatch_skinny<EPI_SILU_MUL, PRO_PLAIN, bf16>(w, xx, ldx, (bf16*)out, ldo, M, N, K, none, nullptr, s);
    }
    if (epilogue != EPI_NONE) return RG_ERR_UNSUPPORTED;
    if (out_dtype == RG_DTYPE_BF16) return dispatch_skinny<EPI_NONE, PRO_PLAIN, bf16>(w, xx, ldx, (bf16*)out, ldo, M, N, K, none, nullptr, s);
    if (out_dtype == RG_DTYPE_F32) return dispatch_skinny<EPI_NONE, PRO_PLAIN, float>(w, xx, ldx, (float*)out, ldo, M, N, K, none, nullptr, s);
    return RG_ERR_UNSUPPORTED;
}
