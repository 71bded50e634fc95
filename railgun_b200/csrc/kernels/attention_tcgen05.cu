// Flash attention for portions of prompts on the 5th-generation tensor cores (bfloat16, head size 64).
//
// One CTA takes 128 consecutive positions of one request and one head.  For every tile of 128 keys:
//   S = Q K^T            tcgen05.mma, M 128 (queries) x N 128 (keys) x K 64 (head), accumulator in TMEM
//   softmax              128 threads, one per query row: the row is read from TMEM with tcgen05.ld, masked by
//                        absolute position, and max / exp2 / sum run inside the thread (no shuffles); P goes to
//                        shared memory as bfloat16 in the swizzled layout the tensor core reads
//   O_tile = P V         tcgen05.mma, M 128 x N 64 x K 128 (keys), V read as it lies in the cache ([key][dim],
//                        an MN-major operand)
//   O = alpha O + O_tile in registers (64 per thread), alpha from the running max
// K and V pages are fetched by TMA (one box per page, 128-byte swizzle) through the request's block table, Q by
// one TMA box.  Two such CTAs fit an SM, so one CTA's softmax overlaps the other's tensor-core work.
//
// Same formulas and masks as attention_mma.cu's prefill kernel (s = scale q.k, keys [max(0, p - w + 1), p],
// crates/vllm-cuda/src/kernels/paged_attention.cu:40,66-69,103-107); the reference has no prefill attention.
// Every mbarrier wait is bounded and reports through *err (see gemm_tcgen05.cu).
#include "tcgen05.cuh"

#define FA_BM 128
#define FA_BN 128
#define FA_D 64
#define FA_THREADS 192            // warps 0-3: softmax / output rows; warp 4: TMA producer; warp 5: MMA issue, TMEM owner

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// tiles: [NT][3] = first token row, rows (<= 128), request.  q_map: the fused qkv buffer [T, (nh + 2 nkv) d];
// kv_map: the cache as rows of d, [pages * 2 * nkv * page_size, d], box = one page of one head.
__global__ void __launch_bounds__(FA_THREADS)
fa_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
             bf16* __restrict__ out, const int* __restrict__ block_table, int max_blocks,
             const int* __restrict__ tiles, const int* __restrict__ positions, int nh, int nkv, int page_size,
             int window, float scale_log2, int* err) {
    extern __shared__ unsigned char smem_raw[];
    constexpr uint32_t TILE_BYTES = 128 * 128;                               // 128 rows x 64 bfloat16
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK0 = base + TILE_BYTES, sV = base + 3 * TILE_BYTES, sP = base + 4 * TILE_BYTES;
    const uint32_t bars = base + 6 * TILE_BYTES;
    const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = bars + 24, v_full = bars + 40, v_empty = bars + 48,
                   s_full = bars + 56, p_full = bars + 64, o_full = bars + 72;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // later tiles of a prompt attend more keys: start them first
    const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
    const int row0 = tiles[tile * 3 + 0], nrows = tiles[tile * 3 + 1], r = tiles[tile * 3 + 2];
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)r * max_blocks;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(q_full, 1);
        mbar_init(k_full0, 1); mbar_init(k_full0 + 8, 1);
        mbar_init(k_empty0, 1); mbar_init(k_empty0 + 8, 1);
        mbar_init(v_full, 1); mbar_init(v_empty, 1);
        mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_full, 1);
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc(&tmem_base_slot, 256u);                        // S: columns [0,128), O_tile: [128,192)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_base_slot, tmem_o = tmem_base_slot + 128u;
    pdl_wait();
    pdl_trigger();

    const int p0 = positions[row0];
    const int hi = p0 + nrows - 1;
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int kt0 = lo / FA_BN, kt1 = hi / FA_BN, n_kt = kt1 - kt0 + 1;
    const int pages_per_tile = FA_BN / page_size;
    const uint32_t page_bytes = (uint32_t)page_size * 128u;

    if (warp == 4) {
        // ---- producer: the whole warp.  Lane l fetches the id of page l of the next tile (one tile ahead, so
        // that the table read is not on the critical path) and issues that page's K and V boxes.
        if (lane == 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_2d(sQ, &q_map, q_full, h * FA_D, row0);
        }
        auto page_of = [&](int kt) -> int {                                  // beyond the context: any page (masked)
            return lane < pages_per_tile ? bt[min(kt * pages_per_tile + lane, max_blocks - 1)] : 0;
        };
        int page_next = page_of(kt0);
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int s = j & 1;
            const int page = page_next;
            if (j + 1 < n_kt) page_next = page_of(kt0 + j + 1);
            if (lane == 0) {
                if (j >= 2) ok = mbar_wait(k_empty0 + 8 * s, ((j >> 1) & 1) ^ 1, err, 11, &abort_flag);
                if (ok) mbar_expect_tx(k_full0 + 8 * s, TILE_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile)
                tma_load_2d(sK0 + s * TILE_BYTES + lane * page_bytes, &kv_map, k_full0 + 8 * s, 0,
                            ((page * 2 + 0) * nkv + kvh) * page_size);
            if (lane == 0) {
                if (j >= 1) ok = mbar_wait(v_empty, (j & 1) ^ 1, err, 12, &abort_flag);
                if (ok) mbar_expect_tx(v_full, TILE_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile)
                tma_load_2d(sV + lane * page_bytes, &kv_map, v_full, 0, ((page * 2 + 1) * nkv + kvh) * page_size);
        }
    } else if (warp == 5 && lane == 0) {
        // ---- MMA issue
        // S: D F32, A/B BF16 K-major, N 128, M 128.  PV: the same with B MN-major (bit 16) and N 64.
        constexpr uint32_t idesc_s = make_idesc(FA_BM, FA_BN, false);
        constexpr uint32_t idesc_o = make_idesc(FA_BM, FA_D, true);
        bool ok = mbar_wait(q_full, 0, err, 21, &abort_flag);
        if (ok) ok = mbar_wait(k_full0, 0, err, 22, &abort_flag);
        if (ok) {
            tc_fence_after();
            const uint64_t qd = desc_k_major(sQ), kd = desc_k_major(sK0);
#pragma unroll
            for (int k = 0; k < FA_D / 16; ++k) tc_mma(tmem_s, qd + 2u * k, kd + 2u * k, idesc_s, k > 0 ? 1u : 0u);
            tc_commit(s_full);
            tc_commit(k_empty0);
        }
        for (int j = 0; j < n_kt && ok; ++j) {
            // O_tile(j) = P(j) V(j)
            ok = mbar_wait(p_full, j & 1, err, 23, &abort_flag);
            if (ok) ok = mbar_wait(v_full, j & 1, err, 24, &abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < FA_BN / 16; ++k) {
                // P: two 64-key halves of [128 rows x 128 bytes]; inside a half, 16 keys = 32 bytes
                const uint64_t pd = desc_k_major(sP + (uint32_t)(k >> 2) * TILE_BYTES) + 2u * (k & 3);
                // V: 16 keys further down = 16 rows of 128 bytes
                const uint64_t vd = desc_mn_major(sV + (uint32_t)k * 2048u, 16384u);
                tc_mma(tmem_o, pd, vd, idesc_o, k > 0 ? 1u : 0u);
            }
            tc_commit(o_full);
            tc_commit(v_empty);
            if (j + 1 < n_kt) {
                // S(j+1): the S columns are free (P(j) was written after S(j) was read)
                const int s = (j + 1) & 1;
                ok = mbar_wait(k_full0 + 8 * s, ((j + 1) >> 1) & 1, err, 25, &abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t qd = desc_k_major(sQ), kd = desc_k_major(sK0 + s * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < FA_D / 16; ++k) tc_mma(tmem_s, qd + 2u * k, kd + 2u * k, idesc_s, k > 0 ? 1u : 0u);
                tc_commit(s_full);
                tc_commit(k_empty0 + 8 * s);
            }
        }
    } else if (warp < 4) {
        // ---- softmax and output: thread = query row
        const int row = warp * 32 + lane;
        const int prow = p0 + row;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        float o[FA_D];
#pragma unroll
        for (int i = 0; i < FA_D; ++i) o[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int key_base = (kt0 + j) * FA_BN;
            ok = mbar_wait(s_full, j & 1, err, 31, &abort_flag);
            if (!ok) break;
            tc_fence_after();
            // Interior tiles (every key attended by every row of the CTA) take the short path; the tile on the
            // diagonal and tiles at a window's edge mask by absolute position.  One uniform branch per tile.
            const bool edge = key_base + FA_BN - 1 > p0 || (window > 0 && key_base < p0 + FA_BM - window);
            const int k_hi = prow - key_base;                                 // columns <= k_hi are not in the future
            const int k_lo = window > 0 ? prow - window + 1 - key_base : -1;  // columns >= k_lo are inside the window
            // pass 1: the row's maximum, on the raw scores (scale > 0, so the maximum commutes with it); two
            // chunks of 32 columns in flight per wait, four independent running maxima
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
            for (int c = 0; c < FA_BN / 32; c += 2) {
                uint32_t v[32], w[32];
                tc_ld32_nowait(tmem_s + lane_off + (uint32_t)(c * 32), v);
                tc_ld32_nowait(tmem_s + lane_off + (uint32_t)(c * 32 + 32), w);
                tc_ld_wait();
                if (!edge) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(v[i]), __uint_as_float(w[i])));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = c * 32 + i;
                        if (col <= k_hi && col >= k_lo) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
                        if (col + 32 <= k_hi && col + 32 >= k_lo) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(w[i]));
                    }
                }
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            mx *= scale_log2;
            const float mn = fmaxf(m_run, mx);
            const float ms = mn == -INFINITY ? 0.f : mn;
            const float alpha = ex2(m_run - ms);
            m_run = mn;
            // pass 2: p = 2^(s scale - m), row sum, P -> shared memory (bfloat16, 16-byte pieces XOR-swizzled by row)
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int c = 0; c < FA_BN / 32; ++c) {
                uint32_t v[32];
                tc_ld32(tmem_s + lane_off + (uint32_t)(c * 32), v);
                uint32_t pk[16];
                if (!edge) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0v = ex2(fmaf(__uint_as_float(v[i]), scale_log2, -ms));
                        const float p1v = ex2(fmaf(__uint_as_float(v[i + 1]), scale_log2, -ms));
                        rs4[(i >> 1) & 3] += p0v + p1v;
                        __nv_bfloat162 hh = __floats2bfloat162_rn(p0v, p1v);
                        pk[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int col = c * 32 + i;
                        const float p0v = (col <= k_hi && col >= k_lo)
                                              ? ex2(fmaf(__uint_as_float(v[i]), scale_log2, -ms)) : 0.f;
                        const float p1v = (col + 1 <= k_hi && col + 1 >= k_lo)
                                              ? ex2(fmaf(__uint_as_float(v[i + 1]), scale_log2, -ms)) : 0.f;
                        rs4[(i >> 1) & 3] += p0v + p1v;
                        __nv_bfloat162 hh = __floats2bfloat162_rn(p0v, p1v);
                        pk[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
                    }
                }
                // columns c*32 .. c*32+31 of this row: half (c >> 1), 16-byte pieces (c & 1) * 4 .. + 3
                const uint32_t half_base = sP + (uint32_t)(c >> 1) * TILE_BYTES + (uint32_t)row * 128u;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint32_t piece = (uint32_t)((c & 1) * 4 + q4) ^ (uint32_t)(row & 7);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(half_base + piece * 16u),
                                 "r"(pk[q4 * 4]), "r"(pk[q4 * 4 + 1]), "r"(pk[q4 * 4 + 2]), "r"(pk[q4 * 4 + 3]) : "memory");
                }
            }
            l_run = l_run * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // P must be visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            // O = alpha O + O_tile
            ok = mbar_wait(o_full, j & 1, err, 32, &abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < FA_D / 32; ++c) {
                uint32_t v[32];
                tc_ld32(tmem_o + lane_off + (uint32_t)(c * 32), v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
            }
        }
        if (ok && row < nrows) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* dst = out + ((size_t)(row0 + row) * nh + h) * FA_D;
#pragma unroll
            for (int i = 0; i < FA_D; i += 8) {
                uint4 pk;
                uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                for (int j2 = 0; j2 < 4; ++j2) {
                    __nv_bfloat162 hh = __floats2bfloat162_rn(o[i + 2 * j2] * inv, o[i + 2 * j2 + 1] * inv);
                    w[j2] = *reinterpret_cast<uint32_t*>(&hh);
                }
                *reinterpret_cast<uint4*>(dst + i) = pk;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_free(tmem_base_slot, 256u);
    }
}

// q: the fused qkv buffer [n_rows_total, q_stride] (head h of q at column h * 64); out [n_rows_total, nh * 64];
// kv_cache [num_pages, 2, nkv, page_size, 64]; tiles [n_tiles][3] with at most 128 rows each.
// Takes head size 64 and page sizes that are multiples of 8 and divide 128; refuses everything else.
extern "C" int rg_prefill_attention_tc(const void* q, int q_stride, int n_rows_total, void* out, const void* kv_cache,
                                       int num_pages, const int* block_table, int max_blocks, const int* tiles,
                                       int n_tiles, const int* positions, int nh, int nkv, int d, int page_size,
                                       int window, float scale, int* err, void* stream) {
    if (n_tiles <= 0) return 0;
    if (d != FA_D || nh % nkv || page_size % 8 || page_size > FA_BN || FA_BN % page_size || q_stride % 8 ||
        ((uintptr_t)q & 15) || ((uintptr_t)kv_cache & 15) || nh > 65535)
        return RG_ERR_UNSUPPORTED;
    CUtensorMap qm, kvm;
    int e = rg_make_map(&qm, q, (unsigned long long)n_rows_total, (unsigned long long)q_stride, (unsigned long long)q_stride, FA_BM);
    if (e) return e;
    e = rg_make_map(&kvm, kv_cache, (unsigned long long)num_pages * 2ull * nkv * page_size, FA_D, FA_D, page_size);
    if (e) return e;
    const size_t smem = 6 * 128 * 128 + 128 + 1024;
    cudaError_t ce = cudaFuncSetAttribute(fa_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    return rg_launch(fa_tc_kernel, dim3(n_tiles, nh), dim3(FA_THREADS), smem, (cudaStream_t)stream, 1, qm, kvm,
                     (bf16*)out, block_table, max_blocks, tiles, positions, nh, nkv, page_size, window,
                     scale * 1.4426950408889634f, err);
}
