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

// Eight outputs per thread with 16-byte loads and stores (bfloat16, I % 8 == 0): the plain storage reads
// gate[i..i+7] and up[i..i+7], the interleaved one reads one 16-column block [8 gate | 8 up].
template <bool INTERLEAVED>
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, size_t groups) {
    pdl_wait();
    pdl_trigger();
    const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gidx >= groups) return;
    const int per_row = I >> 3;
    const size_t t = gidx / per_row;
    const int b = (int)(gidx - t * per_row);
    const bf16* row = gu + t * 2 * (size_t)I;
    const uint4 gv = *reinterpret_cast<const uint4*>(row + (INTERLEAVED ? b * 16 : b * 8));
    const uint4 uv = *reinterpret_cast<const uint4*>(row + (INTERLEAVED ? b * 16 + 8 : I + b * 8));
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        o2[i] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)I + b * 8) = ov;
}

static bool vec8_ok(const void* gu, const void* out, int I) {
    return I % 8 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0;
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
    if (dtype == RG_DTYPE_BF16 && vec8_ok(gu, out, I)) {
        const size_t groups = total / 8;
        return rg_launch(silu_mul_vec8_kernel<true>, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads),
                         0, s, 1, (const bf16*)gu, (bf16*)out, I, groups);
    }
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
    if (dtype == RG_DTYPE_BF16 && vec8_ok(gu, out, I)) {
        const size_t groups = total / 8;
        return rg_launch(silu_mul_vec8_kernel<false>, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads),
                         0, s, 1, (const bf16*)gu, (bf16*)out, I, groups);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)gu, (bf16*)out, I,
                         total);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)gu, (float*)out, I,
                         total);
    return RG_ERR_UNSUPPORTED;
}
