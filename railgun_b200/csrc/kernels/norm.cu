// Fused residual-add + RMSNorm.
//
//   r = residual[row] (+ pending[row])        32-bit sum, written back
//   out[i] = w * r / sqrt(mean(r^2) + eps)     sum of squares, rsqrt and the
//                                              product in 32-bit, one rounding
// The reference builds the norm from its tensor library
// (crates/vllm-models/src/llama/architecture.rs:27-28,48,56,154) and adds the
// residual as a separate op (:53,58); here both are one pass over the row.
// With `rows` given, output row i is computed from residual row rows[i] and the
// residual is not written back (the final norm runs only where logits are wanted).
#include "common.cuh"

template <typename P, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const P* __restrict__ pending,
                                   const float* __restrict__ w, float eps, O* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const P* p = pending ? pending + (size_t)srow * H : nullptr;
    const bool write_back = (rows == nullptr) && (p != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (p) v += to_f32(p[i]);
        if (write_back) r[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    O* o = out + (size_t)orow * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (p && !write_back) v += to_f32(p[i]);
        o[i] = from_f32<O>(v * inv * w[i]);
    }
}

// The same with 4 elements per access for H % 4 == 0 (16-byte residual accesses).  The order of the sum of
// squares inside a thread differs from the scalar kernel's, the block reduction is the same.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}

template <typename P, typename O>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ resid, const P* __restrict__ pending,
                                        const float* __restrict__ w, float eps, O* __restrict__ out,
                                        const int* __restrict__ rows, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const P* p = pending ? pending + (size_t)srow * H : nullptr;
    const bool write_back = (rows == nullptr) && (p != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        float4 v = load4(r + i);
        if (p) {
            const float4 q = load4(p + i);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
            if (write_back) store4(r + i, v);
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    O* o = out + (size_t)orow * H;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        float4 v = load4(r + i);
        if (p && !write_back) {
            const float4 q = load4(p + i);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        }
        const float4 g = load4(w + i);
        store4(o + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
    }
}

// residual[row] += pending[row] only (a block arrangement that ends without a norm).
template <typename P>
__global__ void residual_add_kernel(float* __restrict__ resid, const P* __restrict__ pending, size_t n) {
    pdl_wait();
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += to_f32(pending[i]);
}

extern "C" int rg_add_rmsnorm(float* resid, const void* pending, int pending_dtype, const float* w,
                              float eps, void* out, int out_dtype, const int* rows, int n_out_rows,
                              int H, void* stream) {
    if (n_out_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (uintptr_t)pending % 16 == 0 && (uintptr_t)w % 16 == 0;
    const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define RG_NORM(P, O) return vec ? rg_launch(add_rmsnorm_vec4_kernel<P, O>, dim3(n_out_rows), dim3(threads), 0, s, 1, \
        resid, (const P*)pending, w, eps, (O*)out, rows, H) \
      : rg_launch(add_rmsnorm_kernel<P, O>, dim3(n_out_rows), dim3(threads), 0, s, 1, \
        resid, (const P*)pending, w, eps, (O*)out, rows, H)
    if (pending == nullptr) pending_dtype = out_dtype;
    if (pending_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) RG_NORM(bf16, bf16);
    if (pending_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) RG_NORM(float, float);
    if (pending_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) RG_NORM(float, bf16);
    if (pending_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_F32) RG_NORM(bf16, float);
#undef RG_NORM
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_residual_add(float* resid, const void* pending, int pending_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (pending_dtype == RG_DTYPE_BF16)
        return rg_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, resid, (const bf16*)pending,
                         (size_t)n);
    if (pending_dtype == RG_DTYPE_F32)
        return rg_launch(residual_add_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, resid, (const float*)pending,
                         (size_t)n);
    return RG_ERR_UNSUPPORTED;
}
