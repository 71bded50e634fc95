// Token embedding: residual[t, :] = table[ids[t], :], written in 32-bit, no
// scaling (crates/vllm-models/src/llama/architecture.rs:150 does the same
// gather through the tensor library).
#include "common.cuh"

template <typename W>
__global__ void embed_kernel(const int* __restrict__ ids, const W* __restrict__ table,
                             float* __restrict__ out, int H, int V) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {                 // the host validates ids; never read outside the table
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const W* row = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int rg_embedding(const int* ids, const void* table, int table_dtype, float* out,
                            int T, int H, int V, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == RG_DTYPE_BF16)
        return rg_launch(embed_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, ids, (const bf16*)table, out, H, V);
    if (table_dtype == RG_DTYPE_F32)
        return rg_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, s, 1, ids, (const float*)table, out, H, V);
    return RG_ERR_UNSUPPORTED;
}
