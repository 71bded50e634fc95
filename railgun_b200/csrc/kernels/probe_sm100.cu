// Cycle counts of the building blocks of the tcgen05 kernels, measured on the GPU at hand: how long a special-
// function exponential, a packed FMA, a small tcgen05.mma, a tcgen05.commit, a wait on an mbarrier whose phase has
// completed, a proxy fence and a store to tensor memory take.  The attention kernel's design rests on these figures
// (attention_tcgen05.cu); `bench.py --mode kernels --cases primitives` prints them.  Not on any product path.
//
// Every kernel here is one CTA per SM, times itself with clock64 in CTA 0 and writes cycles to `out`; every wait
// is bounded as in the product kernels.  There is no counterpart in the reference.
#include "tcgen05.cuh"

#define PROBE_RESULTS 16

// ---- instruction rates: 8 independent chains per thread, 16 warps per SM (4 per scheduler) -----------------------
template <int OP>
__global__ void __launch_bounds__(512) probe_rate_kernel(float* sink, long long* cyc, int iters) {
    float a[8];
    uint32_t u[8];
    uint64_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a[i] = (float)(threadIdx.x + i) * 1e-3f;
        u[i] = threadIdx.x + i;
        w[i] = ((uint64_t)__float_as_uint(a[i]) << 32) | __float_as_uint(a[i]);
    }
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (OP == 0) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a[i]));
            if (OP == 1) { asm volatile("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(u[i]) : "f"(a[i])); a[i] = __uint_as_float(u[i]); }
            if (OP == 2) asm volatile("fma.rn.f32x2 %0, %0, %0, %0;" : "+l"(w[i]));
            if (OP == 3) asm volatile("fma.rn.f32 %0, %0, %0, %0;" : "+f"(a[i]));
            if (OP == 4) asm volatile("max.f32 %0, %0, %1;" : "+f"(a[i]) : "f"(a[(i + 1) & 7]));
        }
    }
    const long long t1 = clock64();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += a[i] + (float)u[i] + (float)(w[i] & 0xffffu);
    sink[blockIdx.x * blockDim.x + threadIdx.x] = s;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}

// ---- tcgen05.mma (M 128, K 16, bfloat16 operands of zeros in shared memory) ------------------------------------
// mode 0: n_mma instructions back to back into one accumulator; mode 1: groups of four with two commits after each
__global__ void __launch_bounds__(128) probe_mma_kernel(long long* cyc, int* err, int n_mma, int N, int mode) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = base, sB = base + 16384u, bar = sB + 32768u;
    __shared__ uint32_t slot;
    __shared__ int abort_flag;
    uint32_t* words = reinterpret_cast<uint32_t*>(smem_raw + (base - smem_addr(smem_raw)));
    for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) words[i] = 0u;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < 4; ++i) mbar_init(bar + 8 * i, 1);
        fence_barrier_init();
    }
    if (threadIdx.x < 32) tmem_alloc(&slot, 256u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc(128, N, false);
        const uint64_t ad = desc_k_major(sA), bd = desc_k_major(sB);
        const long long t0 = clock64();
        if (mode == 0) {
            for (int i = 0; i < n_mma; ++i) tc_mma(tm, ad + 2u * (i & 3), bd + 2u * (i & 3), idesc, 1u);
        } else {
            for (int g = 0; g < n_mma / 4; ++g) {
                for (int i = 0; i < 4; ++i) tc_mma(tm + (uint32_t)((g & 1) * 64), ad + 2u * i, bd + 2u * i, idesc, i > 0);
                tc_commit(bar + 8 * (1 + (g & 1)));
                tc_commit(bar + 24);
            }
        }
        tc_commit(bar);
        const bool ok = mbar_wait(bar, 0, err, 1, &abort_flag);
        const long long t1 = clock64();
        if (blockIdx.x == 0) *cyc = ok ? t1 - t0 : -1;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_free(tm, 256u);
    }
}

// ---- synchronisation with nothing to wait for: the fixed cost of each step of a hand-over -------------------------
// out[0..5]: mbarrier wait with every lane polling; with lane 0 polling and a shuffle; fence.proxy.async;
// mbarrier.arrive; tcgen05.st of 8 columns + wait::st; tcgen05.ld of 32 columns + wait::ld.  Cycles for 64 of each.
__global__ void __launch_bounds__(128) probe_sync_kernel(long long* cyc, int* err) {
    __shared__ __align__(8) unsigned long long bar_mem[2];
    __shared__ int abort_flag;
    __shared__ uint32_t slot;
    const uint32_t bar = smem_addr(&bar_mem[0]), bar_many = smem_addr(&bar_mem[1]);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(bar, 1);
        mbar_init(bar_many, 128);
        fence_barrier_init();
    }
    if (threadIdx.x < 32) tmem_alloc(&slot, 32u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) mbar_arrive(bar);                                   // phase 0 of `bar` completes
    __syncthreads();
    const uint32_t taddr = slot + ((uint32_t)((threadIdx.x >> 5) * 32) << 16);
    constexpr int R = 64;
    long long t[7];
    bool ok = true;
    uint32_t v[32], w[8] = {1, 2, 3, 4, 5, 6, 7, 8};
    t[0] = clock64();
    for (int i = 0; i < R; ++i) ok &= mbar_wait_all(bar, 0, err, 1, &abort_flag);
    t[1] = clock64();
    for (int i = 0; i < R; ++i) ok &= mbar_wait_warp(bar, 0, err, 1, &abort_flag);
    t[2] = clock64();
    for (int i = 0; i < R; ++i) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    t[3] = clock64();
    for (int i = 0; i < R; ++i) mbar_arrive(bar_many);
    t[4] = clock64();
    for (int i = 0; i < R; ++i) { tc_st8(taddr, w); tc_st_wait(); }
    t[5] = clock64();
    for (int i = 0; i < R; ++i) { tc_ld32(taddr, v); w[i & 7] += v[i & 31]; }
    t[6] = clock64();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        for (int i = 0; i < 6; ++i) cyc[i] = t[i + 1] - t[i];
        cyc[6] = ok ? (long long)(w[0] & 1u) : -1;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_free(slot, 32u);
    }
}

// ---- the attention kernel's pass over a row of 64 scores, alone: scale, 2^x, sum, conversion, store -------------
__global__ void __launch_bounds__(256) probe_softmax_pass_kernel(const float* in, float* sink, long long* cyc, int iters) {
    extern __shared__ unsigned char smem_raw[];
    const int row = threadIdx.x & 127;
    const uint32_t sP = smem_addr(smem_raw) + (uint32_t)(threadIdx.x >> 7) * 16384u + (uint32_t)row * 128u;
    float s[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) s[i] = in[(size_t)(blockIdx.x * blockDim.x + threadIdx.x) * 64 + i];
    float total = 0.f;
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        const float ms = 1.f + (float)it * 1e-3f;
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                float p0, p1;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(s[c * 8 + i], 0.18f, -ms)));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(s[c * 8 + i + 1], 0.18f, -ms)));
                sum[(i >> 1) & 3] += p0 + p1;
                const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&hh);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sP + (uint32_t)((c ^ (row & 7)) * 16)),
                         "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
        }
        total += (sum[0] + sum[1]) + (sum[2] + sum[3]);
    }
    const long long t1 = clock64();
    sink[blockIdx.x * blockDim.x + threadIdx.x] = total;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}

// out[PROBE_RESULTS] (cycles; device pointers are the caller's scratch: floats >= 148 * 512 * 64, long long >= 16):
//  0 ex2.approx.ftz.f32   1 cvt.rn.bf16x2.f32   2 fma.rn.f32x2   3 fma.rn.f32   4 max.f32      per warp instruction and scheduler
//  5 6 7  tcgen05.mma M 128 K 16, N 64 / 128 / 256, back to back                               per instruction
//  8 four N 64 MMAs and two commits                                                            per group
//  9 mbarrier wait, every lane   10 lane 0 + shuffle   11 fence.proxy.async   12 mbarrier.arrive
//  13 tcgen05.st x8 + wait       14 softmax pass, 2 warps per scheduler   15 the same, 1 warp per scheduler
extern "C" int rg_probe_sm100(double* out, float* scratch, long long* cyc, int* err, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    long long h[8];
    auto fetch = [&](int n) -> int {
        cudaError_t e = cudaMemcpyAsync(h, cyc, n * sizeof(long long), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        return (int)e;
    };
    const int iters = 1024, sms = 148;
    int e;
#define RATE(OP, SLOT)                                                                                   \
    for (int r = 0; r < 2; ++r) probe_rate_kernel<OP><<<sms, 512, 0, stream>>>(scratch, cyc, iters);       \
    if ((e = fetch(1))) return e;                                                                         \
    out[SLOT] = (double)h[0] / (iters * 8.0 * 16 / 4);
    RATE(0, 0) RATE(1, 1) RATE(2, 2) RATE(3, 3) RATE(4, 4)
#undef RATE
    const size_t mma_smem = 16384 + 32768 + 64 + 1024;
    if ((e = (int)cudaFuncSetAttribute(probe_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_smem))) return e;
    const int n_mma = 256;
    const int widths[3] = {64, 128, 256};
    for (int i = 0; i < 4; ++i) {
        for (int r = 0; r < 2; ++r) probe_mma_kernel<<<sms, 128, mma_smem, stream>>>(cyc, err, n_mma, i < 3 ? widths[i] : 64, i < 3 ? 0 : 1);
        if ((e = fetch(1))) return e;
        out[5 + i] = h[0] < 0 ? -1.0 : (double)h[0] / (i < 3 ? n_mma : n_mma / 4);
    }
    for (int r = 0; r < 2; ++r) probe_sync_kernel<<<sms, 128, 0, stream>>>(cyc, err);
    if ((e = fetch(7))) return e;
    out[9] = h[0] / 64.0; out[10] = h[1] / 64.0; out[11] = h[2] / 64.0; out[12] = h[3] / 64.0; out[13] = h[4] / 64.0;
    if (h[6] < 0) out[9] = -1.0;
    if ((e = (int)cudaFuncSetAttribute(probe_softmax_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768))) return e;
    for (int t = 0; t < 2; ++t) {
        for (int r = 0; r < 2; ++r) probe_softmax_pass_kernel<<<sms, t == 0 ? 256 : 128, 32768, stream>>>(scratch, scratch + (size_t)sms * 256 * 64, cyc, 256);
        if ((e = fetch(1))) return e;
        out[14 + t] = h[0] / 256.0;
    }
    return RG_LAUNCH_RESULT();
}
