// SiLU-mul of the fused gate|up projection: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(z) = z / (1 + exp(-z)) in 32-bit
// (crates/vllm-models/src/llama/architecture.rs:81-85 computes silu(gate) * up
// with two library ops).
#include "common.cuh"

template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ out, int I, size_t total) {
    pdl_wait();
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * I + i]);
    const float u = to_f32(gu[t * 2 * I + I + i]);
    out[idx] = from_f32<A>(g / (1.f + expf(-g)) * u);
}

// The same over the interleaved storage of gate|up (rows 16t..16t+7 gate, 16t+8..16t+15 the matching up
// rows), as the decode GEMM's fused epilogue reads it: out[t, 8b + j] = silu(gu[t, 16b + j]) * gu[t, 16b + 8 + j].
template <typename A>
__global__ void silu_mul_interleaved_kernel(const A* __restrict__ gu, A* __restrict__ out, int I, size_t total) {
    pdl_wait();
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const int src = (i >> 3) * 16 + (i & 7);
    const float g = to_f32(gu[t * 2 * I + src]);
    const float u = to_f32(gu[t * 2 * I + src + 8]);
    out[idx] = from_f32<A>(g / (1.f + expf(-g)) * u);
}

extern "C" int rg_silu_mul_interleaved(const void* gu, void* out, int dtype, int T, int I, void* stream) {
    if (T <= 0) return 0;
    if (I % 8) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(silu_mul_interleaved_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)gu,
                         (bf16*)out, I, total);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(silu_mul_interleaved_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)gu,
                         (float*)out, I, total);
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_silu_mul(const void* gu, void* out, int dtype, int T, int I, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)gu, (bf16*)out, I,
                         total);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)gu, (float*)out, I,
                         total);
    return RG_ERR_UNSUPPORTED;
}
