// Weight-streaming matrix product for decode batches of 17 to 64 rows on the 5th-generation tensor cores:
// y[M, N] = x[M, K] W[N, K]^T with the operands swapped, so that 128 rows of W fill the M side of tcgen05.mma
// and the batch (padded to 64) its N side: D[128 weight rows, 64 tokens] accumulates in tensor memory while W
// streams through a ring of TMA stages exactly once.  At these sizes the product is bound by reading W, and a
// product with few rows of W (q|k|v, O, down) has too few 128-row tiles to occupy the GPU, so K is split over the
// CTAs of a thread-block cluster: every CTA accumulates its K range of the cluster's tile, leaves the partial sums
// in its shared memory, and the cluster's CTAs add them, each for its share of the tokens, reading the others'
// through distributed shared memory in rank order: one fixed order, no atomics, a token's result does not depend on
// the batch.  Products with many tiles (gate|up, the head) run unsplit and persistent: a CTA takes tile after tile
// with two accumulators in tensor memory, so that a tile's epilogue overlaps the next tile's loads.
//
// Roles as in gemm_tcgen05.cu: warps 0-3 epilogue (one lane of tensor memory = one row of W each), warp 4 the TMA
// producer, warp 5 issues the MMAs and owns the tensor memory.  Epilogues: plain (bfloat16 or 32-bit out) and
// SiLU-mul over interleaved gate|up rows (crates/vllm-models/src/llama/architecture.rs:81-85).  The reference runs
// these products through cuBLAS (crates/vllm-models/src/llama/attention.rs:94-96,133).
//
// Every wait on an mbarrier is bounded (tcgen05.cuh): a waiter that gives up records where in *err, every role
// stops, the CTA waits for copies in flight, frees its tensor memory and returns; the host reads *err and raises.
#include "tcgen05.cuh"

#define TS_ROWS 128               // rows of W per tile (the MMA's M)
#define TS_TOK 64                 // tokens per tile (the MMA's N); fewer tokens are padded with zeros by TMA
#define TS_BK 64
#define TS_THREADS 192
#define TS_STAGES 6
#define TS_EPI_NONE 0
#define TS_EPI_SILU_MUL 1
#define TS_EPI_RESIDUAL 2         // out (32-bit) += product; also the next norm's input and sums of squares
#define TS_EPI_ROPE_CACHE 3       // the q|k|v projection: rotate q and k, write q out and k, v into the paged cache
#define TS_PRO_PLAIN 0
#define TS_PRO_SCALED 1           // x is a residual row times the norm's weight; 1 / rms is applied to the sums

// RMSNorm around the product without a kernel of its own, as in gemm_skinny.cuh: y = W (w . r) / rms(r) is linear
// in 1 / rms, so the producer of the residual r leaves bf16(r * norm weight) and partial sums of squares, and the
// product that reads them multiplies its 32-bit sums by 1 / rms.
//   TS_EPI_RESIDUAL:  r = out[m, n] += product;  scaled_out[m, n] = bf16(r * norm_w[n]);
//                     ss_out[tile, m] = sum over the tile's 128 columns of r^2.
//   TS_PRO_SCALED:    every sum is multiplied by rsqrt(sum_p ss_in[p, m] / K + eps) before the epilogue.
// TS_EPI_ROPE_CACHE: N = (nh + 2 nkv) d, d % 16 == 0, the rows of every q and k head in the order that puts rotation
// pair i at (16 (i / 8) + i % 8, + 8) (rope_cache.cu's paired8 layout, as gemm_skinny.cuh's fused projection): rows
// (r, r + 8) of a group of 16 are a pair, rotated in 32-bit by the angles of the token's position (table
// [max_pos, d] = cos | sin); q goes to out, k and v to the token's slot of the cache [pages, 2, nkv, page_size, d].
struct StreamFusion {
    const float* norm_w;
    bf16* scaled_out;             // [M, N], rows ldo apart like out
    float* ss_out;                // [tiles, ss_ld]
    const float* ss_in;           // [ss_in_blocks, ss_ld]
    int ss_in_blocks;
    int ss_ld;
    float eps;
    const float* rope_table;      // TS_EPI_ROPE_CACHE from here
    const int* positions;
    const int* slots;             // nullptr: nothing is written to the cache
    bf16* kv_cache;
    int nh, nkv, d, page_size, max_pos;
    int* pos_err;                 // set to 1 when a position is outside the table (never read outside it)
};

__device__ __forceinline__ float4 ts_ld_remote4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// A tile's sums -> the output, for the tokens m_lo .. m_hi - 1, by `nthreads` threads (a multiple of 32) of which
// this is thread `tid`.  load4(r, i) gives partial sums i .. i + 3 of CTA r's [token][row] array; they are added in
// rank order.  inv: 1 / rms per token (TS_PRO_SCALED).
template <int SPLITS, int EPI, int PRO, typename OUT, typename Load>
__device__ __forceinline__ void ts_write_out(Load load4, OUT* __restrict__ out, int ldo, int N, int n0, int tile,
                                             int m_lo, int m_hi, int tid, int nthreads, const float* inv,
                                             const StreamFusion& fu) {
    if constexpr (EPI == TS_EPI_ROPE_CACHE) {
        // rows 16 t .. + 7 and their partners + 8: four rotation pairs at a time
        const int half = fu.d >> 1;
        for (int idx = tid; idx < (m_hi - m_lo) * (TS_ROWS / 8); idx += nthreads) {
            const int m = m_lo + idx / (TS_ROWS / 8), q = idx % (TS_ROWS / 8);
            const int row = (q >> 1) * 16 + (q & 1) * 4;
            float4 a[SPLITS], b[SPLITS];
#pragma unroll
            for (int r = 0; r < SPLITS; ++r) { a[r] = load4(r, m * TS_ROWS + row); b[r] = load4(r, m * TS_ROWS + row + 8); }
            float4 as = a[0], bs = b[0];
#pragma unroll
            for (int r = 1; r < SPLITS; ++r) {
                as.x += a[r].x; as.y += a[r].y; as.z += a[r].z; as.w += a[r].w;
                bs.x += b[r].x; bs.y += b[r].y; bs.z += b[r].z; bs.w += b[r].w;
            }
            const float sc = PRO == TS_PRO_SCALED ? inv[m] : 1.f;
            const float x0[4] = {as.x * sc, as.y * sc, as.z * sc, as.w * sc}, x1[4] = {bs.x * sc, bs.y * sc, bs.z * sc, bs.w * sc};
            const int f = n0 + row;                                          // output feature of the first pair's first element
            if (f + 8 >= N) continue;
            const int head = f / fu.d, e = f - head * fu.d;                  // e: storage index inside the head (a multiple of 4)
            float y0[4], y1[4];
            if (head < fu.nh + fu.nkv) {
                int pos = fu.positions[m];
                if (pos < 0 || pos >= fu.max_pos) {
                    if (fu.pos_err) atomicExch(fu.pos_err, 1);
                    pos = 0;
                }
                const int i0 = ((e >> 4) << 3) + (e & 7);                    // the first pair's number = its angle's index
                const float4 cs = __ldg(reinterpret_cast<const float4*>(fu.rope_table + (size_t)pos * fu.d + i0));
                const float4 sn = __ldg(reinterpret_cast<const float4*>(fu.rope_table + (size_t)pos * fu.d + half + i0));
                const float c[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) { y0[i] = x0[i] * c[i] - x1[i] * sv[i]; y1[i] = x1[i] * c[i] + x0[i] * sv[i]; }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) { y0[i] = x0[i]; y1[i] = x1[i]; }
            }
            bf16* dst = nullptr;
            if (head < fu.nh) {
                dst = reinterpret_cast<bf16*>(out) + (size_t)m * ldo + f;
            } else if (fu.slots) {
                const int slot = fu.slots[m];
                if (slot >= 0) {
                    const int kind = head < fu.nh + fu.nkv ? 0 : 1, kvh = head - fu.nh - kind * fu.nkv;
                    const int page = slot / fu.page_size, off = slot - page * fu.page_size;
                    dst = fu.kv_cache + ((((size_t)page * 2 + kind) * fu.nkv + kvh) * fu.page_size + off) * fu.d + e;
                }
            }
            if (dst) {
#pragma unroll
                for (int i = 0; i < 4; ++i) { dst[i] = __float2bfloat16_rn(y0[i]); dst[8 + i] = __float2bfloat16_rn(y1[i]); }
            }
        }
    } else if constexpr (EPI == TS_EPI_SILU_MUL) {
        // gate rows 16 t .. + 7 and their up rows + 8: four gate values and their four up values at a time
        for (int idx = tid; idx < (m_hi - m_lo) * (TS_ROWS / 8); idx += nthreads) {
            const int m = m_lo + idx / (TS_ROWS / 8), q = idx % (TS_ROWS / 8);
            const int row = (q >> 1) * 16 + (q & 1) * 4;
            float4 g[SPLITS], u[SPLITS];
#pragma unroll
            for (int r = 0; r < SPLITS; ++r) { g[r] = load4(r, m * TS_ROWS + row); u[r] = load4(r, m * TS_ROWS + row + 8); }
            float4 gs = g[0], us = u[0];
#pragma unroll
            for (int r = 1; r < SPLITS; ++r) {
                gs.x += g[r].x; gs.y += g[r].y; gs.z += g[r].z; gs.w += g[r].w;
                us.x += u[r].x; us.y += u[r].y; us.z += u[r].z; us.w += u[r].w;
            }
            const float sc = PRO == TS_PRO_SCALED ? inv[m] : 1.f;
            const float gv[4] = {gs.x * sc, gs.y * sc, gs.z * sc, gs.w * sc}, uv[4] = {us.x * sc, us.y * sc, us.z * sc, us.w * sc};
            OUT* o = out + (size_t)m * ldo + (n0 >> 1) + (q >> 1) * 8 + (q & 1) * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n0 + row + i + 8 < N) o[i] = from_f32<OUT>(gv[i] / (1.f + expf(-gv[i])) * uv[i]);
        }
    } else {
    // four consecutive rows of one token at a time; the 32 pieces of a token's 128 rows are one warp's
    for (int idx = tid; idx < (m_hi - m_lo) * (TS_ROWS / 4); idx += nthreads) {
        const int m = m_lo + idx / (TS_ROWS / 4), row = (idx % (TS_ROWS / 4)) * 4;
        float4 p[SPLITS];
#pragma unroll
        for (int r = 0; r < SPLITS; ++r) p[r] = load4(r, m * TS_ROWS + row);
        float4 v = p[0];
#pragma unroll
        for (int r = 1; r < SPLITS; ++r) { v.x += p[r].x; v.y += p[r].y; v.z += p[r].z; v.w += p[r].w; }
        float vv[4] = {v.x, v.y, v.z, v.w};
        const int n = n0 + row;
        if (EPI == TS_EPI_RESIDUAL) {
            float ssq = 0.f;
            float* o = reinterpret_cast<float*>(out) + (size_t)m * ldo + n;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (n + i < N) {
                    const float r = o[i] + vv[i];
                    o[i] = r;
                    ssq += r * r;
                    if (fu.scaled_out) fu.scaled_out[(size_t)m * ldo + n + i] = __float2bfloat16_rn(r * __ldg(fu.norm_w + n + i));
                }
            }
            ssq = warp_sum(ssq);
            if ((idx & 31) == 0) fu.ss_out[(size_t)tile * fu.ss_ld + m] = ssq;
        } else {
            const float sc = PRO == TS_PRO_SCALED ? inv[m] : 1.f;
            OUT* o = out + (size_t)m * ldo + n;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n + i < N) o[i] = from_f32<OUT>(vv[i] * sc);
        }
    }
    }
}

template <int SPLITS, int EPI, int PRO, typename OUT>
__global__ void __launch_bounds__(TS_THREADS)
tc_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 OUT* __restrict__ out, int ldo, int M, int N, int K, int* err, const StreamFusion fu) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ float inv_rms[TS_TOK];
    constexpr uint32_t W_BYTES = TS_ROWS * TS_BK * 2, X_BYTES = TS_TOK * TS_BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
    unsigned char* base_ptr = smem_raw + (base - smem_addr(smem_raw));
    float* part = reinterpret_cast<float*>(base_ptr + TS_STAGES * STAGE_BYTES);          // [TS_TOK][TS_ROWS]
    const uint32_t bars = base + TS_STAGES * STAGE_BYTES + TS_TOK * TS_ROWS * 4;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (TS_STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * TS_STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * TS_STAGES + 2 + b); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = SPLITS > 1 ? (int)cluster_ctarank() : 0;
    const int n_tiles = (N + TS_ROWS - 1) / TS_ROWS;
    const int KT_all = (K + TS_BK - 1) / TS_BK;
    const int kt_lo = KT_all * rank / SPLITS, kt_hi = KT_all * (rank + 1) / SPLITS;       // this CTA's K range, in boxes
    const int KT = kt_hi - kt_lo;
    // split products: one tile per cluster; unsplit ones: tile after tile
    const int first_tile = SPLITS > 1 ? (int)(blockIdx.x / SPLITS) : (int)blockIdx.x;
    const int tile_step = SPLITS > 1 ? n_tiles : (int)gridDim.x;
    constexpr uint32_t TMEM_COLS = 2 * TS_TOK;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < TS_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 4); }
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 4 && lane == 0) {
        // ---- producer: W does not depend on the kernel before this one, x does: the first stages' W boxes are
        // requested before the wait, their x boxes after it (both count on the stage's barrier)
        int it = 0;
        bool ok = true, waited = false;
        int early = 0;
        if (first_tile < n_tiles) {
            for (; early < KT && early < TS_STAGES; ++early) {
                mbar_expect_tx(full_bar(early), STAGE_BYTES);
                tma_load_2d(base + early * STAGE_BYTES, &map_w, full_bar(early), (kt_lo + early) * TS_BK, first_tile * TS_ROWS);
            }
        }
        pdl_wait();
        pdl_trigger();
        waited = true;
        for (int e = 0; e < early; ++e)
            tma_load_2d(base + e * STAGE_BYTES + W_BYTES, &map_x, full_bar(e), (kt_lo + e) * TS_BK, 0);
        for (int t = first_tile; t < n_tiles && ok; t += tile_step) {
            for (int kt = 0; kt < KT; ++kt, ++it) {
                if (it < early) continue;                                    // requested above
                const int s = it % TS_STAGES, r = it / TS_STAGES;
                if (r > 0 && !mbar_wait(empty_bar(s), (r & 1) ^ 1, err, 1, &abort_flag)) { ok = false; break; }
                mbar_expect_tx(full_bar(s), STAGE_BYTES);
                const uint32_t sa = base + s * STAGE_BYTES;
                tma_load_2d(sa, &map_w, full_bar(s), (kt_lo + kt) * TS_BK, t * TS_ROWS);
                tma_load_2d(sa + W_BYTES, &map_x, full_bar(s), (kt_lo + kt) * TS_BK, 0);
            }
        }
        (void)waited;
    } else {
        pdl_wait();
        pdl_trigger();
    }
    if (warp == 5 && lane == 0) {
        // ---- MMA issue: D[128 x 64] (+)= W[128 x 16] x[64 x 16]^T, four K steps per stage
        constexpr uint32_t idesc = make_idesc(TS_ROWS, TS_TOK, false);
        int it = 0, local = 0;
        bool ok = true;
        for (int t = first_tile; t < n_tiles && ok; t += tile_step, ++local) {
            const int b = local & 1, u = local >> 1;
            if (u > 0 && !mbar_wait(acc_empty(b), (u & 1) ^ 1, err, 4, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * TS_TOK);
            for (int kt = 0; kt < KT; ++kt, ++it) {
                const int s = it % TS_STAGES, r = it / TS_STAGES;
                if (!mbar_wait(full_bar(s), r & 1, err, 2, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sa = base + s * STAGE_BYTES;
                const uint64_t adesc = desc_k_major(sa), bdesc = desc_k_major(sa + W_BYTES);
#pragma unroll
                for (int k = 0; k < TS_BK / 16; ++k)
                    tc_mma(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty_bar(s));
            }
            if (ok) tc_commit(acc_full(b));
        }
    } else if (warp < 4) {
        // ---- epilogue, first half: this warp's 32 rows of the accumulator into shared memory, token-major, so
        // that what follows reads and writes along rows of W
        int local = 0;
        bool ok = true;
        if (PRO == TS_PRO_SCALED && threadIdx.x < TS_TOK) {
            // 1 / rms of every token from the producer's partial sums of squares, added in their order
            float ssq = 0.f;
            for (int p = 0; p < fu.ss_in_blocks; ++p) ssq += fu.ss_in[(size_t)p * fu.ss_ld + threadIdx.x];
            inv_rms[threadIdx.x] = rsqrtf(ssq / (float)K + fu.eps);
        }
        for (int t = first_tile; t < n_tiles && ok; t += tile_step, ++local) {
            const int b = local & 1, u = local >> 1;
            if (!mbar_wait(acc_full(b), u & 1, err, 3, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * TS_TOK) + ((uint32_t)(warp * 32) << 16);
            if (SPLITS == 1 && local > 0) asm volatile("bar.sync 1, 128;" ::: "memory");   // the tile before has been written out
#pragma unroll
            for (int c = 0; c < TS_TOK / 32; ++c) {
                uint32_t v[32];
                tc_ld32(tmem_d + (uint32_t)(c * 32), v);
#pragma unroll
                for (int i = 0; i < 32; ++i) part[(c * 32 + i) * TS_ROWS + warp * 32 + lane] = __uint_as_float(v[i]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));
            if (SPLITS == 1) {
                // ---- second half, unsplit: the four epilogue warps write the tile out
                asm volatile("bar.sync 1, 128;" ::: "memory");
                auto load4 = [&](int, int i) { return *reinterpret_cast<const float4*>(part + i); };
                ts_write_out<1, EPI, PRO, OUT>(load4, out, ldo, N, t * TS_ROWS, t, 0, M, (int)threadIdx.x, 128, inv_rms, fu);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (SPLITS > 1) {
        // ---- second half, split over the cluster: CTA `rank` adds the partial sums of its share of the tokens
        cluster_sync_all();                                                 // every CTA's partial sums are in its shared memory
        if (first_tile < n_tiles && !abort_flag) {
            const int n0 = first_tile * TS_ROWS;
            const int m_lo = M * rank / SPLITS, m_hi = M * (rank + 1) / SPLITS;
            const uint32_t mine = smem_addr(part);
            uint32_t peer[SPLITS];
#pragma unroll
            for (int r = 0; r < SPLITS; ++r) peer[r] = mapa_shared(mine, (uint32_t)r);
            auto load4 = [&](int r, int i) { return ts_ld_remote4(peer[r] + (uint32_t)i * 4u); };
            ts_write_out<SPLITS, EPI, PRO, OUT>(load4, out, ldo, N, n0, first_tile, m_lo, m_hi, (int)threadIdx.x, TS_THREADS,
                                                inv_rms, fu);
        }
        cluster_sync_all();                                                 // nobody leaves while its partial sums are being read
    }
    if (abort_flag) {                                                       // give copies in flight time to land
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_free(tmem_base, TMEM_COLS);
    }
}

static int ts_num_sms() {
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
            num_sms = 148;
    }
    return num_sms;
}

template <int SPLITS, int EPI, int PRO, typename OUT>
static int launch_ts(const CUtensorMap& mw, const CUtensorMap& mx, OUT* out, int ldo, int M, int N, int K, int* err,
                     const StreamFusion& fu, cudaStream_t s) {
    const size_t smem = (size_t)TS_STAGES * (TS_ROWS * TS_BK * 2 + TS_TOK * TS_BK * 2) + TS_TOK * TS_ROWS * 4 +
                        8 * (2 * TS_STAGES + 4) + 1024;
    auto kernel = tc_stream_kernel<SPLITS, EPI, PRO, OUT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int n_tiles = (N + TS_ROWS - 1) / TS_ROWS;
    const int sms = ts_num_sms();
    const unsigned grid = SPLITS > 1 ? (unsigned)(n_tiles * SPLITS) : (unsigned)(n_tiles < sms ? n_tiles : sms);
    return rg_launch(kernel, dim3(grid), dim3(TS_THREADS), smem, s, SPLITS, mw, mx, out, ldo, M, N, K, err, fu);
}

static int ts_pick_splits(int splits, int N, int K) {
    const int n_tiles = (N + TS_ROWS - 1) / TS_ROWS, kt = (K + TS_BK - 1) / TS_BK;
    if (splits == 0) {
        // as many CTAs per tile as keep the whole product in one wave (clusters of 8 start slowly: 4 at most)
        splits = 1;
        while (splits < 4 && n_tiles * splits * 2 <= ts_num_sms() && kt >= splits * 2 * 2) splits *= 2;
    }
    if ((splits != 1 && splits != 2 && splits != 4 && splits != 8) || kt < splits) return -1;
    return splits;
}

template <int EPI, int PRO, typename OUT>
static int dispatch_ts(const void* x, int ldx, const void* W, OUT* out, int ldo, int M, int N, int K, int splits,
                       int* err, const StreamFusion& fu, cudaStream_t s) {
    CUtensorMap mw, mx;
    int e = rg_make_map(&mw, W, N, K, K, TS_ROWS);
    if (e) return e;
    e = rg_make_map(&mx, x, M, K, ldx, TS_TOK);
    if (e) return e;
    return splits == 1 ? launch_ts<1, EPI, PRO, OUT>(mw, mx, out, ldo, M, N, K, err, fu, s)
         : splits == 2 ? launch_ts<2, EPI, PRO, OUT>(mw, mx, out, ldo, M, N, K, err, fu, s)
         : splits == 4 ? launch_ts<4, EPI, PRO, OUT>(mw, mx, out, ldo, M, N, K, err, fu, s)
                       : launch_ts<8, EPI, PRO, OUT>(mw, mx, out, ldo, M, N, K, err, fu, s);
}

static bool ts_operands_ok(const void* x, int ldx, const void* W, int M, int K) {
    return M <= TS_TOK && K > 0 && K % 8 == 0 && ldx % 8 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)W & 15);
}

// y = x W^T for 1 <= M <= 64 rows of x (bfloat16, rows ldx elements apart), W [N, K] bfloat16 contiguous.
// out_dtype: RG_DTYPE_BF16 or RG_DTYPE_F32; epilogue 0 plain (out [M, N]) or 1 SiLU-mul over interleaved gate|up
// rows (out [M, N / 2], bfloat16).  splits: 1, 2, 4 or 8 CTAs share a tile's K (K >= 64 x splits); 0 picks.
// ss_in (may be null): x holds residual rows times a norm's weight and ss_in [ss_in_blocks, ss_ld] their partial
// sums of squares; the sums are multiplied by 1 / rms (eps inside the root).  err: device int, non-zero afterwards
// if a wait gave up.
extern "C" int rg_tc_stream_gemm(const void* x, int ldx, const void* W, void* out, int ldo, int out_dtype, int epilogue,
                                 int M, int N, int K, int splits, const float* ss_in, int ss_in_blocks, int ss_ld,
                                 float eps, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!ts_operands_ok(x, ldx, W, M, K)) return RG_ERR_UNSUPPORTED;
    if (epilogue == TS_EPI_SILU_MUL && (N % 16 || out_dtype != RG_DTYPE_BF16)) return RG_ERR_UNSUPPORTED;
    if (ss_in && (ss_in_blocks < 1 || ss_ld < M)) return RG_ERR_UNSUPPORTED;
    splits = ts_pick_splits(splits, N, K);
    if (splits < 0) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    StreamFusion fu = {};
    fu.ss_in = ss_in; fu.ss_in_blocks = ss_in_blocks; fu.ss_ld = ss_ld; fu.eps = eps;
#define RG_TS(EPI_, OUT_) (ss_in ? dispatch_ts<EPI_, TS_PRO_SCALED, OUT_>(x, ldx, W, (OUT_*)out, ldo, M, N, K, splits, err, fu, s) \
                                 : dispatch_ts<EPI_, TS_PRO_PLAIN, OUT_>(x, ldx, W, (OUT_*)out, ldo, M, N, K, splits, err, fu, s))
    if (epilogue == TS_EPI_SILU_MUL) return RG_TS(TS_EPI_SILU_MUL, bf16);
    if (epilogue != TS_EPI_NONE) return RG_ERR_UNSUPPORTED;
    if (out_dtype == RG_DTYPE_BF16) return RG_TS(TS_EPI_NONE, bf16);
    if (out_dtype == RG_DTYPE_F32) return RG_TS(TS_EPI_NONE, float);
#undef RG_TS
    return RG_ERR_UNSUPPORTED;
}

// The q|k|v projection of M single tokens with the rotary encoding and the cache write in the product's epilogue:
// out [M, N] (bfloat16) receives the rotated q heads (its k and v columns are not written), k (rotated) and v go to
// kv_cache at slots (null: no write).  W's q and k rows are in the paired8 order.  ss_in as in rg_tc_stream_gemm.
extern "C" int rg_tc_stream_gemm_rope_cache(const void* x, int ldx, const void* W, void* out, int ldo, int M, int N, int K,
                                            int splits, const float* ss_in, int ss_in_blocks, int ss_ld, float eps,
                                            const float* rope_table, const int* positions, const int* slots,
                                            void* kv_cache, int nh, int nkv, int d, int page_size, int max_pos,
                                            int* pos_err, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!ts_operands_ok(x, ldx, W, M, K) || d < 16 || d % 16 || nkv < 1 || nh < nkv || N != (nh + 2 * nkv) * d ||
        !rope_table || !positions || max_pos < 1 || (slots && (!kv_cache || page_size < 1)) ||
        (ss_in && (ss_in_blocks < 1 || ss_ld < M)))
        return RG_ERR_UNSUPPORTED;
    splits = ts_pick_splits(splits, N, K);
    if (splits < 0) return RG_ERR_UNSUPPORTED;
    StreamFusion fu = {};
    fu.ss_in = ss_in; fu.ss_in_blocks = ss_in_blocks; fu.ss_ld = ss_ld; fu.eps = eps;
    fu.rope_table = rope_table; fu.positions = positions; fu.slots = slots; fu.kv_cache = (bf16*)kv_cache;
    fu.nh = nh; fu.nkv = nkv; fu.d = d; fu.page_size = page_size; fu.max_pos = max_pos; fu.pos_err = pos_err;
    cudaStream_t s = (cudaStream_t)stream;
    return ss_in ? dispatch_ts<TS_EPI_ROPE_CACHE, TS_PRO_SCALED, bf16>(x, ldx, W, (bf16*)out, ldo, M, N, K, splits, err, fu, s)
                 : dispatch_ts<TS_EPI_ROPE_CACHE, TS_PRO_PLAIN, bf16>(x, ldx, W, (bf16*)out, ldo, M, N, K, splits, err, fu, s);
}

// resid [M, N] (32-bit, rows ldr apart) += x W^T, and the next RMSNorm prepared: scaled_out [M, N] (bfloat16, rows
// ldr apart) = bf16(resid * norm_w), ss_out [tiles of 128 columns, ss_ld >= M] = sums of squares of the new residual
// over each tile's columns.  *tiles_out receives the number of tiles.
extern "C" int rg_tc_stream_gemm_residual(const void* x, int ldx, const void* W, float* resid, int ldr,
                                          const float* norm_w, void* scaled_out, float* ss_out, int ss_ld, int M, int N,
                                          int K, int splits, int* tiles_out, int* err, void* stream) {
    if (tiles_out) *tiles_out = (N + TS_ROWS - 1) / TS_ROWS;
    if (M <= 0 || N <= 0) return 0;
    if (!ts_operands_ok(x, ldx, W, M, K) || ss_ld < M || !ss_out || !norm_w) return RG_ERR_UNSUPPORTED;
    splits = ts_pick_splits(splits, N, K);
    if (splits < 0) return RG_ERR_UNSUPPORTED;
    StreamFusion fu = {};
    fu.norm_w = norm_w; fu.scaled_out = (bf16*)scaled_out; fu.ss_out = ss_out; fu.ss_ld = ss_ld;
    return dispatch_ts<TS_EPI_RESIDUAL, TS_PRO_PLAIN, float>(x, ldx, W, resid, ldr, M, N, K, splits, err, fu,
                                                             (cudaStream_t)stream);
}
