// Matrix product on the 5th-generation tensor cores: C[M, N] = A[M, K] B[N, K]^T, bfloat16 operands, 32-bit
// accumulation in tensor memory.
//
// One CTA computes 128 x BN tiles of C, one after the other (persistent, one CTA per SM).  A thread of the producer warp moves 128 x 64 tiles of A and
// BN x 64 tiles of B into a ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle, each
// CTA its own copies); one thread of the MMA warp issues tcgen05.mma (M 128, N BN, K 16) on shared-memory
// descriptors, accumulating in TMEM, and hands stages back with tcgen05.commit; four epilogue warps read the
// accumulator with tcgen05.ld and write C, plain or through SiLU-mul over the interleaved gate|up columns
// (crates/vllm-models/src/llama/architecture.rs:81-85).  The reference runs these products through cuBLAS
// (crates/vllm-models/src/llama/attention.rs:94-96,133).
//
// Every wait on an mbarrier is bounded: after RG_SPIN_LIMIT tries the waiter records where it gave up in *err,
// every role stops, the CTA waits for copies that may still be in flight, frees its TMEM and returns; the
// host reads *err and raises.
#include "common.cuh"
#include <cuda.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192            // warps 0-3: epilogue; warp 4: TMA producer; warp 5: MMA issue and TMEM owner
#define RG_SPIN_LIMIT 1000000u
#define EPI_NONE 0
#define EPI_SILU_MUL 1

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with this parity.  false: gave up (the code is left in *err).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code, volatile int* abort_flag) {
    for (uint32_t i = 0; i < RG_SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    atomicCAS(err, 0, code);
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes (64 bfloat16), 128-byte swizzle,
// groups of 8 rows 1024 bytes apart.  Fields: start address >> 4 in bits [0,14), leading byte offset >> 4 in
// [16,30) (1: unused for swizzled K-major), stride byte offset >> 4 in [32,46) (1024 >> 4), version 1 in
// [46,48), layout type SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Persistent: CTA b works on tiles b, b + gridDim.x, ... (rows of C fastest, so that CTAs running at the same
// time share a tile of B in L2).  Two accumulators in TMEM: while the epilogue warps drain one, the MMA warp
// fills the other.
template <int BN, int STAGES, int EPI, typename OUT>
__global__ void __launch_bounds__(TC_THREADS)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               OUT* __restrict__ out, int ldo, int M, int N, int K, int* err) {
    extern __shared__ unsigned char smem_raw[];
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
    const uint32_t bars = base + STAGES * STAGE_BYTES;  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    constexpr uint32_t TMEM_COLS = 2 * BN;                                  // 256 or 512: a power of two

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {                                                        // this warp owns the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();                                                             // A is the previous kernel's output
    pdl_trigger();

    if (warp == 4 && lane == 0) {
        // ---- producer: TMA loads into the ring, running ahead across tiles
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            const int m0 = (t % m_tiles) * TC_BM, n0 = (t / m_tiles) * BN;
            for (int kt = 0; kt < KT; ++kt, ++it) {
                const int s = it % STAGES, r = it / STAGES;
                if (r > 0 && !mbar_wait(empty_bar(s), (r & 1) ^ 1, err, 1, &abort_flag)) { ok = false; break; }
                mbar_expect_tx(full_bar(s), STAGE_BYTES);
                const uint32_t sa = base + s * STAGE_BYTES;
                tma_load_2d(sa, &map_a, full_bar(s), kt * TC_BK, m0);
                tma_load_2d(sa + A_BYTES, &map_b, full_bar(s), kt * TC_BK, n0);
            }
        }
    } else if (warp == 5 && lane == 0) {
        // ---- MMA issue: D[128 x BN] (+)= A[128 x 16] B[BN x 16]^T, four K steps per stage
        // instruction descriptor: D F32 (bits 4-5 = 1), A and B BF16 (bits 7-9, 10-12 = 1), both K-major,
        // N >> 3 in bits 17-22, M >> 4 in bits 24-28
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)(TC_BM >> 4) << 24);
        int it = 0, local = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
            const int b = local & 1, u = local >> 1;
            if (u > 0 && !mbar_wait(acc_empty(b), (u & 1) ^ 1, err, 4, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
            for (int kt = 0; kt < KT; ++kt, ++it) {
                const int s = it % STAGES, r = it / STAGES;
                if (!mbar_wait(full_bar(s), r & 1, err, 2, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sa = base + s * STAGE_BYTES;
                const uint64_t adesc = make_desc(sa), bdesc = make_desc(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)                        // 16 elements = 32 bytes = 2 descriptor units
                    tc_mma(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty_bar(s));                                    // the stage is free once these MMAs have read it
            }
            if (ok) tc_commit(acc_full(b));                                 // this tile's accumulator is complete
        }
    } else if (warp < 4) {
        // ---- epilogue: each warp reads its 32 lanes (rows) of the accumulator, 32 columns at a time
        int local = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
            const int b = local & 1, u = local >> 1;
            if (!mbar_wait(acc_full(b), u & 1, err, 3, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int m0 = (t % m_tiles) * TC_BM, n0 = (t / m_tiles) * BN;
            const int row = m0 + warp * 32 + lane;
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN) + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tc_ld32(tmem_d + (uint32_t)(c * 32), v);
                const int col0 = n0 + c * 32;
                if (row < M && col0 < N) {
                    if (EPI == EPI_NONE) {
                        OUT* o = out + (size_t)row * ldo + col0;
                        if (col0 + 32 <= N && sizeof(OUT) == 2 && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 pk;
                                uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[i * 8 + 2 * j]),
                                                                             __uint_as_float(v[i * 8 + 2 * j + 1]));
                                    w[j] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(o) + i * 8) = pk;
                            }
                        } else if (col0 + 32 <= N && sizeof(OUT) == 4 && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                *reinterpret_cast<uint4*>(reinterpret_cast<float*>(o) + i * 4) =
                                    make_uint4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
                        } else {
                            for (int i = 0; i < 32; ++i)
                                if (col0 + i < N) o[i] = from_f32<OUT>(__uint_as_float(v[i]));
                        }
                    } else {
                        // columns come as blocks of 16 = 8 gate | 8 up; two blocks per 32 columns -> 16 outputs
                        bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * ldo + (col0 >> 1);
#pragma unroll
                        for (int bk = 0; bk < 2; ++bk) {
                            if (col0 + bk * 16 + 16 <= N) {
                                uint4 pk;
                                uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float g0 = __uint_as_float(v[bk * 16 + 2 * j]), u0 = __uint_as_float(v[bk * 16 + 8 + 2 * j]);
                                    const float g1 = __uint_as_float(v[bk * 16 + 2 * j + 1]), u1 = __uint_as_float(v[bk * 16 + 9 + 2 * j]);
                                    __nv_bfloat162 h = __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * u0,
                                                                             g1 / (1.f + expf(-g1)) * u1);
                                    w[j] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                if ((((uintptr_t)(o + bk * 8)) & 15) == 0) {
                                    *reinterpret_cast<uint4*>(o + bk * 8) = pk;
                                } else {
                                    const bf16* src = reinterpret_cast<const bf16*>(&pk);
                                    for (int j = 0; j < 8; ++j) o[bk * 8 + j] = src[j];
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));                       // this warp has drained its rows
        }
    }
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {                                                       // give copies in flight time to land
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side: tensor maps through the driver entry point (no link-time dependency on libcuda) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// rows x cols bfloat16, row pitch ld elements; box = box_rows x 64 columns, 128-byte swizzle, zeros out of bounds
static int make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RG_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

template <int BN, int STAGES, int EPI, typename OUT>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, OUT* out, int ldo, int M, int N, int K, int* err,
                     cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 8 * (2 * STAGES + 4) + 1024;
    auto kernel = tc_gemm_kernel<BN, STAGES, EPI, OUT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
            num_sms = 148;
    }
    const int tiles = ((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
    dim3 grid(tiles < num_sms ? tiles : num_sms);                          // persistent: one CTA per SM at most
    return rg_launch(kernel, grid, dim3(TC_THREADS), smem, s, 1, ma, mb, out, ldo, M, N, K, err);
}

// out_dtype: RG_DTYPE_BF16 or RG_DTYPE_F32; epilogue 0 plain (out [M, N]) or 1 SiLU-mul over interleaved gate|up
// columns (out [M, N / 2], bfloat16).  K % 8 == 0, lda % 8 == 0, 16-byte aligned A and B; err: device int, 0 before
// the call, non-zero afterwards if a wait gave up (1 producer, 2 and 4 MMA, 3 epilogue).
extern "C" int rg_tc_gemm(const void* A, int lda, const void* B, void* out, int ldo, int out_dtype, int epilogue,
                          int M, int N, int K, int wide, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return RG_ERR_UNSUPPORTED;
    if (epilogue == EPI_SILU_MUL && (N % 16 || out_dtype != RG_DTYPE_BF16)) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int BN = wide ? 256 : 128;
    CUtensorMap ma, mb;
    int e = make_map(&ma, A, M, K, lda, TC_BM);
    if (e) return e;
    e = make_map(&mb, B, N, K, K, BN);
    if (e) return e;
    if (epilogue == EPI_SILU_MUL)
        return wide ? launch_tc<256, 4, EPI_SILU_MUL, bf16>(ma, mb, (bf16*)out, ldo, M, N, K, err, s)
                    : launch_tc<128, 6, EPI_SILU_MUL, bf16>(ma, mb, (bf16*)out, ldo, M, N, K, err, s);
    if (epilogue != EPI_NONE) return RG_ERR_UNSUPPORTED;
    if (out_dtype == RG_DTYPE_BF16)
        return wide ? launch_tc<256, 4, EPI_NONE, bf16>(ma, mb, (bf16*)out, ldo, M, N, K, err, s)
                    : launch_tc<128, 6, EPI_NONE, bf16>(ma, mb, (bf16*)out, ldo, M, N, K, err, s);
    if (out_dtype == RG_DTYPE_F32)
        return wide ? launch_tc<256, 4, EPI_NONE, float>(ma, mb, (float*)out, ldo, M, N, K, err, s)
                    : launch_tc<128, 6, EPI_NONE, float>(ma, mb, (float*)out, ldo, M, N, K, err, s);
    return RG_ERR_UNSUPPORTED;
}
