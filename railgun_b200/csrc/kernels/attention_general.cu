// General paged attention: one thread block per (query token, head), any head
// size up to 256, any page size, 32-bit or bfloat16 storage, all arithmetic in
// 32-bit.  It serves the true 32-bit path and every shape the fast kernels
// refuse.  A query at absolute position p of request r attends the keys of r
// at positions [max(0, p - window + 1), p], read from the paged cache through
// r's block table (the step's own keys are written before it runs).
//
// Formulas: kv_head = head / (nh / nkv); s_j = scale * q.k_j; running max m,
// p_j = exp(s_j - m), out = sum p_j v_j / sum p_j
// (crates/vllm-cuda/src/kernels/paged_attention.cu:40,66-69,103-107;
// single-pass online form crates/vllm-cuda/src/kernels/paged_attention_v1_plus.cu:56-100).
// The reference masks only j < context_len; the mask by the query's own
// position (causal inside a portion of a prompt) is added here.
#include "common.cuh"

#define ATT_THREADS 128

// q: rows of stride q_stride elements, head h at offset h*d.  out: [T, nh*d].
// kv_cache: [NP, 2, nkv, ps, d].  block_table: [R, max_blocks].
template <typename A>
__global__ void paged_attention_general_kernel(
        const A* __restrict__ q, int q_stride, A* __restrict__ out, const A* __restrict__ kv_cache,
        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ req_of_token,
        const int* __restrict__ positions, int nh, int nkv, int d, int page_size, int window, float scale) {
    extern __shared__ float smem[];
    float* qs = smem;                    // [d]
    float* ps = qs + d;                  // [ATT_THREADS]
    float* scratch = ps + ATT_THREADS;   // [33]
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (nh / nkv);
    const int r = req_of_token[t];
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)r * max_blocks;
    const A* qrow = q + (size_t)t * q_stride + (size_t)h * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) qs[i] = to_f32(qrow[i]) * scale;
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;        // output dims threadIdx.x and threadIdx.x + 128
    const size_t page_elems = (size_t)2 * nkv * page_size * d;
    for (int base = lo; base <= pos; base += ATT_THREADS) {
        const int j = base + threadIdx.x;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = bt[j / page_size], off = j % page_size;
            const A* krow = kv_cache + (size_t)page * page_elems + ((size_t)kvh * page_size + off) * d;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot += qs[i] * to_f32(krow[i]);
            s = dot;
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);           // 0 when m = -inf
        const float csum = block_sum(p, scratch);
        l = l * alpha + csum;
        m = m_new;
        ps[threadIdx.x] = p;
        __syncthreads();
        acc0 *= alpha;
        acc1 *= alpha;
        const int n = min(ATT_THREADS, pos - base + 1);
        for (int k = 0; k < n; ++k) {
            const int jj = base + k;
            const int page = bt[jj / page_size], off = jj % page_size;
            const A* vrow = kv_cache + (size_t)page * page_elems
                            + ((size_t)(nkv + kvh) * page_size + off) * d;
            const float pk = ps[k];
            if (threadIdx.x < d) acc0 += pk * to_f32(vrow[threadIdx.x]);
            if (threadIdx.x + ATT_THREADS < d) acc1 += pk * to_f32(vrow[threadIdx.x + ATT_THREADS]);
        }
        __syncthreads();
    }
    A* orow = out + ((size_t)t * nh + h) * d;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (threadIdx.x < d) orow[threadIdx.x] = from_f32<A>(acc0 * inv);
    if (threadIdx.x + ATT_THREADS < d) orow[threadIdx.x + ATT_THREADS] = from_f32<A>(acc1 * inv);
}

extern "C" int rg_paged_attention_general(
        const void* q, int q_stride, void* out, const void* kv_cache, int dtype,
        const int* block_table, int max_blocks, const int* req_of_token, const int* positions,
        int T, int nh, int nkv, int d, int page_size, int window, float scale, void* stream) {
    if (T <= 0) return 0;
    if (d > 2 * ATT_THREADS || d < 1 || nkv < 1 || nh < nkv || nh % nkv) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh);
    const size_t smem = (size_t)(d + ATT_THREADS + 33) * sizeof(float);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(paged_attention_general_kernel<bf16>, grid, dim3(ATT_THREADS), smem, s, 1,
                         (const bf16*)q, q_stride, (bf16*)out, (const bf16*)kv_cache, block_table, max_blocks,
                         req_of_token, positions, nh, nkv, d, page_size, window, scale);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(paged_attention_general_kernel<float>, grid, dim3(ATT_THREADS), smem, s, 1,
                         (const float*)q, q_stride, (float*)out, (const float*)kv_cache, block_table, max_blocks,
                         req_of_token, positions, nh, nkv, d, page_size, window, scale);
    return RG_ERR_UNSUPPORTED;
}
