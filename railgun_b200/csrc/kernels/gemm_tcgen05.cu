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
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192            // warps 0-3: epilogue; warp 4: TMA producer; warp 5: MMA issue and TMEM owner
#define EPI_NONE 0
#define EPI_SILU_MUL 1

// 32 accumulator columns of one row -> C: plain (bf16 or fp32), or SiLU-mul over the interleaved gate|up columns.
template <int EPI, typename OUT>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], OUT* __restrict__ out, int ldo, int row, int col0,
                                            int N) {
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
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc(&tmem_base_slot, TMEM_COLS);                  // this warp owns the tensor memory
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
        constexpr uint32_t idesc = make_idesc(TC_BM, BN, false);
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
                const uint64_t adesc = desc_k_major(sa), bdesc = desc_k_major(sa + A_BYTES);
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
                if (row < M && col0 < N) store_chunk<EPI, OUT>(v, out, ldo, row, col0, N);
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
        tmem_free(tmem_base, TMEM_COLS);
    }
}

static int rg_num_sms() {
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
            num_sms = 148;
    }
    return num_sms;
}

template <int BN, int STAGES, int EPI, typename OUT>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, OUT* out, int ldo, int M, int N, int K, int* err,
                     cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 8 * (2 * STAGES + 4) + 1024;
    auto kernel = tc_gemm_kernel<BN, STAGES, EPI, OUT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int num_sms = rg_num_sms();
    const int tiles = ((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
    dim3 grid(tiles < num_sms ? tiles : num_sms);                          // persistent: one CTA per SM at most
    return rg_launch(kernel, grid, dim3(TC_THREADS), smem, s, 1, ma, mb, out, ldo, M, N, K, err);
}

// ---- the same product on CTA pairs: tiles of 256 x BN, one pair per two SMs (cta_group::2) ----------------
// Each CTA of the pair keeps its own 128 rows of A and its own BN / 2 rows of B per stage, so that a stage of
// shared memory feeds twice the arithmetic of the single-CTA kernel and every tile of B crosses L2 -> SM once per
// 256 rows of C.  The first CTA's MMA thread issues for both; its commits arrive on the barriers of both CTAs.
//   full[s]       first CTA only: its producer announces the bytes of both CTAs, both producers' copies count there
//   empty[s]      in each CTA, for its own producer
//   acc_full[b]   in each CTA, for its own epilogue warps
//   acc_empty[b]  first CTA only: the 2 x 4 epilogue warps of the pair arrive there
template <int BN, int STAGES, int EPI, typename OUT>
__global__ void __launch_bounds__(TC_THREADS)
tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OUT* __restrict__ out, int ldo, int M, int N, int K, int* err) {
    extern __shared__ unsigned char smem_raw[];
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = (BN / 2) * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int KT = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (M + 2 * TC_BM - 1) / (2 * TC_BM), n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    constexpr uint32_t TMEM_COLS = 2 * BN;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 8); }
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc_pair(&tmem_base_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                                     // both CTAs' barriers exist before either is used
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();
    pdl_trigger();

    if (warp == 4 && lane == 0) {
        // ---- producer (both CTAs): this CTA's rows of A and of B, counted on the first CTA's barrier
        int it = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += n_pairs) {
            const int m0 = (t % m_tiles) * 2 * TC_BM + (int)rank * TC_BM, n0 = (t / m_tiles) * BN + (int)rank * (BN / 2);
            for (int kt = 0; kt < KT; ++kt, ++it) {
                const int s = it % STAGES, r = it / STAGES;
                if (r > 0 && !mbar_wait(empty_bar(s), (r & 1) ^ 1, err, 1, &abort_flag)) { ok = false; break; }
                if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
                const uint32_t sa = base + s * STAGE_BYTES, full0 = mapa_shared(full_bar(s), 0);
                tma_load_2d_pair(sa, &map_a, full0, kt * TC_BK, m0);
                tma_load_2d_pair(sa + A_BYTES, &map_b, full0, kt * TC_BK, n0);
            }
        }
    } else if (warp == 5 && lane == 0 && rank == 0) {
        // ---- MMA issue for the pair: D[256 x BN] (+)= A[256 x 16] B[BN x 16]^T
        constexpr uint32_t idesc = make_idesc(2 * TC_BM, BN, false);
        int it = 0, local = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += n_pairs, ++local) {
            const int b = local & 1, u = local >> 1;
            if (u > 0 && !mbar_wait(acc_empty(b), (u & 1) ^ 1, err, 4, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
            for (int kt = 0; kt < KT; ++kt, ++it) {
                const int s = it % STAGES, r = it / STAGES;
                if (!mbar_wait(full_bar(s), r & 1, err, 2, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sa = base + s * STAGE_BYTES;
                const uint64_t adesc = desc_k_major(sa), bdesc = desc_k_major(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    tc_mma_pair(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                tc_commit_pair(empty_bar(s), 3);                            // both producers may refill the stage
            }
            if (ok) tc_commit_pair(acc_full(b), 3);                         // both CTAs' epilogues may read
        }
    } else if (warp < 4) {
        // ---- epilogue (both CTAs): this CTA's 128 rows of the accumulator
        int local = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += n_pairs, ++local) {
            const int b = local & 1, u = local >> 1;
            if (!mbar_wait(acc_full(b), u & 1, err, 3, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int m0 = (t % m_tiles) * 2 * TC_BM + (int)rank * TC_BM, n0 = (t / m_tiles) * BN;
            const int row = m0 + warp * 32 + lane;
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN) + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tc_ld32(tmem_d + (uint32_t)(c * 32), v);
                const int col0 = n0 + c * 32;
                if (row < M && col0 < N) store_chunk<EPI, OUT>(v, out, ldo, row, col0, N);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(acc_empty(b));
                else mbar_arrive_cluster(mapa_shared(acc_empty(b), 0));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();                                                     // the other CTA's MMAs and arrivals are done with this one
    if (warp == 5) {
        tc_fence_after();
        tmem_free_pair(tmem_base, TMEM_COLS);
    }
}

template <int BN, int STAGES, int EPI, typename OUT>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, OUT* out, int ldo, int M, int N, int K, int* err,
                          cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + (BN / 2) * TC_BK * 2) + 8 * (2 * STAGES + 4) + 1024;
    auto kernel = tc_gemm_pair_kernel<BN, STAGES, EPI, OUT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int num_sms = rg_num_sms();
    const int tiles = ((N + BN - 1) / BN) * ((M + 2 * TC_BM - 1) / (2 * TC_BM));
    const int pairs = tiles < num_sms / 2 ? tiles : num_sms / 2;
    return rg_launch(kernel, dim3(2 * pairs), dim3(TC_THREADS), smem, s, 2, ma, mb, out, ldo, M, N, K, err);
}

// out_dtype: RG_DTYPE_BF16 or RG_DTYPE_F32; epilogue 0 plain (out [M, N]) or 1 SiLU-mul over interleaved gate|up
// columns (out [M, N / 2], bfloat16).  K % 8 == 0, lda % 8 == 0, 16-byte aligned A and B; err: device int, 0 before
// the call, non-zero afterwards if a wait gave up (1 producer, 2 and 4 MMA, 3 epilogue).
extern "C" int rg_tc_gemm(const void* A, int lda, const void* B, void* out, int ldo, int out_dtype, int epilogue,
                          int M, int N, int K, int wide, int* err, void* stream) {
    // wide: 0 one CTA per 128 x 128 tile, 1 per 128 x 256; 2 a CTA pair per 256 x 256 tile, 3 per 256 x 128
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return RG_ERR_UNSUPPORTED;
    if (epilogue == EPI_SILU_MUL && (N % 16 || out_dtype != RG_DTYPE_BF16)) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int BN = (wide == 1 || wide == 2) ? 256 : 128;
    CUtensorMap ma, mb;
    int e = rg_make_map(&ma, A, M, K, lda, TC_BM);
    if (e) return e;
    e = rg_make_map(&mb, B, N, K, K, wide >= 2 ? BN / 2 : BN);              // a pair's CTAs fetch half of B's rows each
    if (e) return e;
    if (wide >= 2) {
#define RG_PAIR(EPI_, OUT_) (wide == 2 ? launch_tc_pair<256, 6, EPI_, OUT_>(ma, mb, (OUT_*)out, ldo, M, N, K, err, s) \
                                       : launch_tc_pair<128, 8, EPI_, OUT_>(ma, mb, (OUT_*)out, ldo, M, N, K, err, s))
        if (wide > 3) return RG_ERR_UNSUPPORTED;
        if (epilogue == EPI_SILU_MUL) return RG_PAIR(EPI_SILU_MUL, bf16);
        if (epilogue != EPI_NONE) return RG_ERR_UNSUPPORTED;
        if (out_dtype == RG_DTYPE_BF16) return RG_PAIR(EPI_NONE, bf16);
        if (out_dtype == RG_DTYPE_F32) return RG_PAIR(EPI_NONE, float);
#undef RG_PAIR
        return RG_ERR_UNSUPPORTED;
    }
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
