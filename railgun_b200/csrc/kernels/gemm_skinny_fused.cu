// The weight-streaming decode product with the neighbouring residual addition and RMSNorm folded in
// (gemm_skinny.cuh has the kernel and the arithmetic):
//
//   rg_skinny_gemm_residual   resid[M, N] (32-bit) += x[M, K] W[N, K]^T; scaled[M, N] = bf16(resid * norm_w), the
//                             next norm's output but for the factor 1 / rms; and for every block of W's rows the
//                             sum over its columns of resid[m, n]^2, the partial sums that factor is made of.
//   rg_skinny_gemm_scaled     y = (scaled[M, K] W[N, K]^T) / rms: the product over the rows above, every sum
//                             multiplied by 1 / rms (from the partial sums) before the plain or SiLU-mul epilogue.
//
//   rg_skinny_gemm_rope_cache the q|k|v projection of single tokens with the rotary encoding and the cache write in its
//                             epilogue (EPI_ROPE_CACHE in gemm_skinny.cuh), reading plain rows or rows whose norm is
//                             finished here, as above.
//
// All take up to 16 batch rows (the sizes at which this product is used).  Together they take the two norm
// launches out of a decoder layer at small batch: the residual additions and the norms
// (crates/vllm-models/src/llama/architecture.rs:47-58) run inside the four products.
#include "gemm_skinny.cuh"

// norm_w: the following norm's weight [N], 32-bit.  scaled: bfloat16 [M, N], rows ld_resid apart like resid's.
// ss_out: [>= *row_blocks rows][ss_ld] floats, ss_ld >= 8 * ceil(M / 8); (N + 15) / 16 rows always suffice.
// *row_blocks receives how many rows of ss_out the kernel writes.
extern "C" int rg_skinny_gemm_residual(const void* W, const void* x, int ldx, float* resid, int ld_resid,
                                       const float* norm_w, void* scaled, int M, int N, int K, float* ss_out,
                                       int ss_ld, int* row_blocks, void* stream) {
    if (row_blocks) *row_blocks = 0;
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K % 8 || K <= 0 || ldx % 8 || ss_ld < 8 * ((M + 7) / 8) || !ss_out || !norm_w || !scaled)
        return RG_ERR_UNSUPPORTED;
    SkinnyFusion fu = {};
    fu.norm_w = norm_w;
    fu.scaled_out = (bf16*)scaled;
    fu.ss_out = ss_out;
    fu.ss_ld = ss_ld;
    return dispatch_skinny<EPI_RESIDUAL, PRO_PLAIN, float, 2>((const bf16*)W, (const bf16*)x, ldx, resid, ld_resid, M, N, K,
                                                              fu, row_blocks, (cudaStream_t)stream);
}

// scaled rows are ldx elements apart (a multiple of 8); K % 8 == 0.
// epilogue: 0 plain, 1 SiLU-mul over interleaved gate|up rows; out is bfloat16.
extern "C" int rg_skinny_gemm_scaled(const void* W, const void* scaled, int ldx, float eps, const float* ss_in, int ss_ld,
                                     int ss_blocks, void* out, int ldo, int epilogue, int M, int N, int K,
                                     void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K % 8 || K <= 0 || ldx % 8 || ss_blocks <= 0 || ss_ld < 8 * ((M + 7) / 8) || !ss_in)
        return RG_ERR_UNSUPPORTED;
    SkinnyFusion fu = {};
    fu.ss_in = ss_in;
    fu.ss_in_blocks = ss_blocks;
    fu.ss_ld = ss_ld;
    fu.eps = eps;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == EPI_SILU_MUL) {
        if (N % 16) return RG_ERR_UNSUPPORTED;
        return dispatch_skinny<EPI_SILU_MUL, PRO_SCALED, bf16, 2>((const bf16*)W, (const bf16*)scaled, ldx, (bf16*)out, ldo, M,
                                                                  N, K, fu, nullptr, s);
    }
    if (epilogue != EPI_NONE) return RG_ERR_UNSUPPORTED;
    return dispatch_skinny<EPI_NONE, PRO_SCALED, bf16, 2>((const bf16*)W, (const bf16*)scaled, ldx, (bf16*)out, ldo, M, N, K,
                                                          fu, nullptr, s);
}

// x: bfloat16 rows (ss_in == nullptr) or the scaled rows of rg_skinny_gemm_residual with their partial sums.
// W [(nh + 2 nkv) d, K] with q and k rows in the paired8 order; out [M, ldo] receives the rotated q heads;
// table [max_pos, d]; positions, slots [M] (slots nullptr or < 0: no cache write); d % 16 == 0.
extern "C" int rg_skinny_gemm_rope_cache(const void* W, const void* x, int ldx, float eps, const float* ss_in, int ss_ld,
                                         int ss_blocks, void* out, int ldo, int M, int N, int K, const float* table,
                                         const int* positions, const int* slots, void* kv_cache, int nh, int nkv, int d,
                                         int page_size, int max_pos, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K % 8 || K <= 0 || ldx % 8 || d <= 0 || d % 16 || nh <= 0 || nkv <= 0 || N != (nh + 2 * nkv) * d ||
        !table || !positions || (slots && (!kv_cache || page_size <= 0)) ||
        (ss_in && (ss_blocks <= 0 || ss_ld < 8 * ((M + 7) / 8))))
        return RG_ERR_UNSUPPORTED;
    SkinnyFusion fu = {};
    fu.ss_in = ss_in;
    fu.ss_in_blocks = ss_blocks;
    fu.ss_ld = ss_ld;
    fu.eps = eps;
    fu.rope_table = table;
    fu.positions = positions;
    fu.slots = slots;
    fu.kv_cache = (bf16*)kv_cache;
    fu.nh = nh; fu.nkv = nkv; fu.d = d; fu.page_size = page_size; fu.max_pos = max_pos;
    fu.err = err;
    cudaStream_t s = (cudaStream_t)stream;
    if (ss_in)
        return dispatch_skinny<EPI_ROPE_CACHE, PRO_SCALED, bf16, 2>((const bf16*)W, (const bf16*)x, ldx, (bf16*)out, ldo, M, N,
                                                                    K, fu, nullptr, s);
    return dispatch_skinny<EPI_ROPE_CACHE, PRO_PLAIN, bf16, 2>((const bf16*)W, (const bf16*)x, ldx, (bf16*)out, ldo, M, N, K,
                                                               fu, nullptr, s);
}
