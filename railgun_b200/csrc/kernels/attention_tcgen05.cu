// Flash attention for portions of prompts on the 5th-generation tensor cores (bfloat16, head size 64).
//
// One CTA takes 128 consecutive positions of one request and one head.  For every tile of 64 keys:
//   S = Q K^T            tcgen05.mma, M 128 (queries) x N 64 (keys) x K 64 (head), accumulator in TMEM
//   softmax              128 threads, one per query row: the row is read from TMEM with tcgen05.ld, masked by
//                        absolute position, p = 2^(s scale - reference) and the row sum run inside the thread
//                        (no shuffles); P goes back to TMEM as bfloat16, two keys per 32-bit cell (tcgen05.st)
//   O += P V             tcgen05.mma, M 128 x N 64 x K 64 (keys), P read from TMEM as the A operand, V read as it
//                        lies in the cache ([key][dim], an MN-major operand), accumulated in TMEM over the key tiles
// The three are a software pipeline: S and P have two buffers each in TMEM, so while the threads work on tile j the
// tensor core computes S(j+1) and O += P(j-1) V(j-1); K and V tiles come through rings of three, fetched by TMA
// (one box per page, or 64 rows of a larger page, 128-byte swizzle) through the request's block table two tiles
// ahead.  Two such CTAs fit an SM (256 of its 512 TMEM columns each).
//
// Hand-overs are kept cheap, because a tile's fixed costs weigh as much as its exponentials (measured, see
// probe_sm100.cu): the threads wait once per tile (S(j) is issued after O += P(j-2) V(j-2), so its completion also
// says that P's buffer is free); every wait is made by all lanes of its warp with a vote at the end (76 cycles
// when the phase is done, against 270 for one polling lane and a shuffle); every softmax thread arrives on P's
// barrier itself; the MMA warp waits for the next K before it waits for P.
//
// The exponentials use a reference maximum that is set from the first tile and raised only when a later tile's
// p summed to more than 2^8 in some row (then that tile's row maximum is taken, O and the row sum are rescaled, O
// by a read-modify-write of TMEM, and the tile is done again); otherwise a tile is one pass over its scores.
// Below 2^8, p is far inside bfloat16's range, and O / l is the same quotient whatever the reference.
//
// Same formulas and masks as attention_mma.cu's prefill kernel (s = scale q.k, keys [max(0, p - w + 1), p],
// crates/vllm-cuda/src/kernels/paged_attention.cu:40,66-69,103-107); the reference has no prefill attention.
// Every mbarrier wait is bounded and reports through *err (see gemm_tcgen05.cu).
#include "tcgen05.cuh"
#include <type_traits>

#define FA_BM 128
#define FA_BN 64
#define FA_D 64
#define FA_KV_STAGES 3
#define FA_S_BUFFERS 2
#define FA_THREADS 192            // warps 0-3: softmax / output rows; warp 4: TMA producer; warp 5: MMA issue, TMEM owner

// Two 32-bit operations in one instruction (packed f32x2 arithmetic): the same roundings as two scalar
// instructions, half the issue slots.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// The same three with their order fixed against one another and against the stores (volatile).
__device__ __forceinline__ float ex2_in_order(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint64_t add2_in_order(uint64_t a, uint64_t b) {
    uint64_t r;
    asm volatile("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_in_order(float lo, float hi) {      // lo in the low half
    uint32_t r;
    asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// tiles: [NT][3] = first token row, rows (<= 128), request.  q_map: the fused qkv buffer [T, (nh + 2 nkv) d];
// kv_map: the cache as rows of d, [pages * 2 * nkv * page_size, d], box = min(page, 64) rows of one head.
__global__ void __launch_bounds__(FA_THREADS, 2)
fa_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
             bf16* __restrict__ out, const int* __restrict__ block_table, int max_blocks,
             const int* __restrict__ tiles, const int* __restrict__ positions, int nh, int nkv, int page_size,
             int window, float scale_log2, int* err) {
    extern __shared__ unsigned char smem_raw[];
    constexpr uint32_t Q_BYTES = FA_BM * 128, KV_BYTES = FA_BN * 128;                          // rows of 64 bfloat16
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;            // swizzled tiles need 1024-byte alignment
    const uint32_t sQ = base, sK0 = sQ + Q_BYTES, sV0 = sK0 + FA_KV_STAGES * KV_BYTES;
    const uint32_t bars = sV0 + FA_KV_STAGES * KV_BYTES;
    // q_full | k_full[] k_empty[] v_full[] v_empty[] (one per stage) | s_full[2] p_full[2] p_free[2]
    const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = k_full0 + 8 * FA_KV_STAGES, v_full0 = k_empty0 + 8 * FA_KV_STAGES,
                   v_empty0 = v_full0 + 8 * FA_KV_STAGES, s_full0 = v_empty0 + 8 * FA_KV_STAGES,
                   p_full0 = s_full0 + 8 * FA_S_BUFFERS, p_free0 = p_full0 + 16;
    static_assert(8 + 32 * FA_KV_STAGES + 8 * FA_S_BUFFERS + 32 <= 256, "the barriers have 256 bytes");
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // later tiles of a prompt attend more keys: blocks are handed out in index order, so every head's
    // last tile starts first and the shortest tiles fill the gaps at the end
    const int tile = gridDim.x / nh - 1 - blockIdx.x / nh, h = blockIdx.x % nh;
    const int row0 = tiles[tile * 3 + 0], nrows = tiles[tile * 3 + 1], r = tiles[tile * 3 + 2];
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)r * max_blocks;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < FA_KV_STAGES; ++s) {
            mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1);
        }
        for (int b = 0; b < FA_S_BUFFERS; ++b) mbar_init(s_full0 + 8 * b, 1);
        for (int b = 0; b < 2; ++b) { mbar_init(p_full0 + 8 * b, FA_BM); mbar_init(p_free0 + 8 * b, 1); }   // p_full: every softmax thread
        fence_barrier_init();
    }
    // S: columns [0,64) and [64,128); O: [128,192); P (bfloat16, two keys per cell): [192,224) and [224,256)
    if (warp == 5) tmem_alloc(&tmem_base_slot, 256u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s0 = tmem_base_slot, tmem_o = tmem_base_slot + (uint32_t)(FA_S_BUFFERS * FA_BN);
    const uint32_t tmem_p0 = tmem_o + (uint32_t)FA_D;
    // Tiles, positions and block tables were written before the step's first kernel started: they are read, and the
    // first pages looked up, before the wait for the kernel before this one (which rotates q and writes this
    // portion's keys and values); only what moves q, K, V or the output comes after it.
    const int p0 = positions[row0];
    const int hi = p0 + nrows - 1;
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int kt0 = lo / FA_BN, kt1 = hi / FA_BN, n_kt = kt1 - kt0 + 1;

    if (warp == 4) {
        // ---- producer: the whole warp.  A tile of 64 keys is 64 / rows_per_box boxes (a page, or 64 rows of a
        // larger page); lane l fetches the page id of box l of the next tile (one tile ahead, so that the table
        // read is not on the critical path) and issues that box of K and of V.
        const int rows_per_box = min(page_size, FA_BN), boxes = FA_BN / rows_per_box;
        const uint32_t box_bytes = (uint32_t)rows_per_box * 128u;
        auto page_of = [&](int kt) -> int {                                  // beyond the context: any page (masked)
            const int key = kt * FA_BN + lane * rows_per_box;
            return lane < boxes ? bt[min(key / page_size, max_blocks - 1)] : 0;
        };
        int page_next = page_of(kt0);
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&q_map)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&kv_map)) : "memory");
        }
        pdl_wait();
        pdl_trigger();
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(sQ, &q_map, q_full, h * FA_D, row0);
        }
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int s = j % FA_KV_STAGES, u = j / FA_KV_STAGES;
            const int page = page_next;
            const int in_page = ((kt0 + j) * FA_BN + lane * rows_per_box) % page_size;
            if (j + 1 < n_kt) page_next = page_of(kt0 + j + 1);
            // every lane polls (a wait by one lane and a shuffle costs four times as much when the phase is done)
            if (u > 0) ok = mbar_wait_all(k_empty0 + 8 * s, (u & 1) ^ 1, err, 11, &abort_flag);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(k_full0 + 8 * s, KV_BYTES);
            __syncwarp();
            if (lane < boxes)
                tma_load_2d(sK0 + s * KV_BYTES + lane * box_bytes, &kv_map, k_full0 + 8 * s, 0,
                            ((page * 2 + 0) * nkv + kvh) * page_size + in_page);
            if (u > 0) ok = mbar_wait_all(v_empty0 + 8 * s, (u & 1) ^ 1, err, 12, &abort_flag);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(v_full0 + 8 * s, KV_BYTES);
            __syncwarp();
            if (lane < boxes)
                tma_load_2d(sV0 + s * KV_BYTES + lane * box_bytes, &kv_map, v_full0 + 8 * s, 0,
                            ((page * 2 + 1) * nkv + kvh) * page_size + in_page);
        }
    } else if (warp == 5) {
        pdl_wait();
        // ---- MMA issue.  The whole warp walks the loop and waits (so that tile indices, descriptors and
        // addresses are uniform values of the warp); one elected lane issues.
        // S: D F32, A/B BF16 K-major, N 64, M 128.  PV: the same with B MN-major (bit 16).
        constexpr uint32_t idesc_s = make_idesc(FA_BM, FA_BN, false);
        constexpr uint32_t idesc_o = make_idesc(FA_BM, FA_D, true);
        const bool issuer = elect_one();
        auto wait_k = [&](int j) -> bool {
            return mbar_wait_all(k_full0 + 8 * (j % FA_KV_STAGES), (j / FA_KV_STAGES) & 1, err, 22, &abort_flag);
        };
        auto issue_s = [&](int j) {                                           // S(j) = Q K(j)^T into buffer j & 1; K(j) is there
            const int s = j % FA_KV_STAGES, sb = j % FA_S_BUFFERS;
            if (issuer) {
                const uint64_t qd = desc_k_major(sQ), kd = desc_k_major(sK0 + s * KV_BYTES);
#pragma unroll
                for (int k = 0; k < FA_D / 16; ++k)
                    tc_mma(tmem_s0 + (uint32_t)(sb * FA_BN), qd + 2u * k, kd + 2u * k, idesc_s, k > 0 ? 1u : 0u);
                tc_commit(s_full0 + 8 * sb);
                tc_commit(k_empty0 + 8 * s);
            }
            __syncwarp();
        };
        bool ok = mbar_wait_all(q_full, 0, err, 21, &abort_flag);
        if (ok) ok = wait_k(0);
        if (ok) { tc_fence_after(); issue_s(0); }
        if (ok && n_kt > 1) ok = wait_k(1);
        if (ok && n_kt > 1) { tc_fence_after(); issue_s(1); }
        for (int j = 0; j < n_kt && ok; ++j) {
            // O += P(j) V(j): the threads have read S(j) and written P(j).  What else the tensor core will need is
            // waited for first, while the threads are in their pass.
            const int s = j % FA_KV_STAGES, u = j / FA_KV_STAGES, b = j & 1;
            ok = mbar_wait_all(v_full0 + 8 * s, u & 1, err, 24, &abort_flag);
            if (ok && j + 2 < n_kt) ok = wait_k(j + 2);
            if (ok) ok = mbar_wait_all(p_full0 + 8 * b, (j >> 1) & 1, err, 23, &abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (issuer) {
#pragma unroll
                for (int k = 0; k < FA_BN / 16; ++k) {
                    const uint64_t vd = desc_mn_major(sV0 + s * KV_BYTES + (uint32_t)k * 2048u, KV_BYTES);  // 16 keys = 16 rows
                    tc_mma_a_tmem(tmem_o, tmem_p0 + (uint32_t)(b * (FA_BN / 2) + k * 8), vd, idesc_o,    // 16 keys = 8 cells
                                  (j > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(p_free0 + 8 * b);                                   // P(j) consumed, O complete through tile j
                tc_commit(v_empty0 + 8 * s);
            }
            __syncwarp();
            // S(j+2) into the buffer the threads have just finished with.  It is issued after O += P(j) V(j), so
            // its completion (s_full) also tells the threads that P's buffer j & 1 has been read.
            if (j + 2 < n_kt) issue_s(j + 2);
        }
    } else if (warp < 4) {
        pdl_wait();
        // ---- softmax and output: thread = query row
        const int row = warp * 32 + lane;
        const int prow = p0 + row;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        float m_ref = -INFINITY, l_run = 0.f;                                 // reference maximum (log2 domain), row sum
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int b = j & 1, sb = j % FA_S_BUFFERS;
            const int key_base = (kt0 + j) * FA_BN;
            const uint32_t tmem_s = tmem_s0 + (uint32_t)(sb * FA_BN) + lane_off;
            const uint32_t tmem_p = tmem_p0 + (uint32_t)(b * (FA_BN / 2)) + lane_off;
            ok = mbar_wait_all(s_full0 + 8 * sb, (j / FA_S_BUFFERS) & 1, err, 31, &abort_flag);     // every lane polls: no exchange
            if (!ok) break;
            tc_fence_after();
            // Interior tiles (every key attended by every row of the CTA) take the short path; the tile on the
            // diagonal and tiles at a window's edge mask by absolute position.  One uniform branch per tile.
            const bool edge = key_base + FA_BN - 1 > p0 || (window > 0 && key_base < p0 + FA_BM - window);
            const int k_hi = prow - key_base;                                 // columns <= k_hi are not in the future
            const int k_lo = window > 0 ? prow - window + 1 - key_base : -1;  // columns >= k_lo are inside the window
            // P's buffer j & 1 is free: S(j) was issued after O += P(j-2) V(j-2), and the tensor core completes in order

            // One pass over the row: p = 2^(s scale - reference) -> P in shared memory (bfloat16, 16-byte pieces
            // XOR-swizzled by row), the row sum, and the largest p as packed bfloat16.  EDGE is a compile-time
            // constant so that interior tiles carry no masking code.
            auto exp_pass = [&](auto edge_c, float ms) -> float {
                constexpr bool EDGE = decltype(edge_c)::value;
                uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};                   // packed pairs of partial row sums
                const uint64_t scale2 = pack2(scale_log2, scale_log2), nms2 = pack2(-ms, -ms);
                uint32_t v[2][32];
                tc_ld32_nowait(tmem_s, v[0]);
                tc_ld32_nowait(tmem_s + 32u, v[1]);
                tc_ld_wait();
                // Four groups of 16 columns.  The exponentials of a group are issued back to back, and their
                // consumers (row sum, conversion, the store of P) only after the next group's exponentials: a
                // thread waits for no exponential it has just issued.  The order is pinned with volatile asm.
                float p[2][16];
                auto exps = [&](int g) {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const int col = g * 16 + i;
                        float s0 = __uint_as_float(v[col >> 5][col & 31]), s1 = __uint_as_float(v[col >> 5][(col & 31) + 1]);
                        if (EDGE) {
                            if (col > k_hi || col < k_lo) s0 = -INFINITY;
                            if (col + 1 > k_hi || col + 1 < k_lo) s1 = -INFINITY;
                        }
                        float t0, t1;
                        unpack2(fma2(pack2(s0, s1), scale2, nms2), t0, t1);
                        p[g & 1][i] = ex2_in_order(t0);
                        p[g & 1][i + 1] = ex2_in_order(t1);
                    }
                };
                auto consume = [&](int g) {
                    uint32_t pk[8];
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        rs2[(i >> 1) & 3] = add2_in_order(rs2[(i >> 1) & 3], pack2(p[g & 1][i], p[g & 1][i + 1]));
                        pk[i >> 1] = bf16x2_in_order(p[g & 1][i], p[g & 1][i + 1]);
                    }
                    tc_st8(tmem_p + (uint32_t)(g * 8), pk);                  // keys g*16 .. g*16+15 of this row
                };
                exps(0);
                exps(1);
                consume(0);
                exps(2);
                consume(1);
                exps(3);
                consume(2);
                consume(3);
                float lo, hi;
                unpack2(add2(add2(rs2[0], rs2[1]), add2(rs2[2], rs2[3])), lo, hi);
                return lo + hi;
            };
            auto pass = [&](float ms) -> float {
                return edge ? exp_pass(std::true_type{}, ms) : exp_pass(std::false_type{}, ms);
            };

            // The first tile sets the reference from the row's maximum; later tiles try the reference they have
            // and fall back to that path when some row of the warp summed to more than 2^8 (no p of the tile can
            // then be above 2^8 either: they are not negative).
            bool redo = j == 0;
            float row_sum = 0.f;
            if (!redo) {
                row_sum = pass(m_ref == -INFINITY ? 0.f : m_ref);
                redo = __any_sync(0xffffffffu, !(row_sum <= 256.f));          // also catches inf and NaN
            }
            if (redo && ok) {
                // the row's maximum on the raw scores (scale > 0, so the maximum commutes with it)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                {
                    uint32_t v[32], w[32];
                    tc_ld32_nowait(tmem_s, v);
                    tc_ld32_nowait(tmem_s + 32u, w);
                    tc_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (!edge || (i <= k_hi && i >= k_lo)) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
                        if (!edge || (i + 32 <= k_hi && i + 32 >= k_lo)) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(w[i]));
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
                const float m_new = fmaxf(m_ref, mx);
                if (j > 0) {
                    // rescale this warp's rows of O and the row sums: O must be complete through tile j - 1 (the
                    // product of tile j waits for this tile's P, so nothing else writes O meanwhile)
                    ok = mbar_wait_all(p_free0 + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, err, 33, &abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const float alpha = ex2(m_ref - (m_new == -INFINITY ? 0.f : m_new));
#pragma unroll
                    for (int c = 0; c < FA_D / 32; ++c) {
                        uint32_t o[32];
                        tc_ld32(tmem_o + lane_off + (uint32_t)(c * 32), o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tc_st32(tmem_o + lane_off + (uint32_t)(c * 32), o);
                    }
                    tc_st_wait();
                    l_run *= alpha;
                }
                m_ref = m_new;
                row_sum = pass(m_ref == -INFINITY ? 0.f : m_ref);
            }
            if (!ok) break;
            l_run += row_sum;
            tc_st_wait();                                                     // P is in tensor memory
            tc_fence_before();
            mbar_arrive(p_full0 + 8 * b);                                     // this row of S(j) has been read, of P(j) written
        }
        if (ok) ok = mbar_wait_all(p_free0 + 8 * ((n_kt - 1) & 1), ((n_kt - 1) >> 1) & 1, err, 34, &abort_flag);
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* dst = out + ((size_t)(row0 + row) * nh + h) * FA_D;
#pragma unroll
            for (int c = 0; c < FA_D / 32; ++c) {
                uint32_t o[32];
                tc_ld32(tmem_o + lane_off + (uint32_t)(c * 32), o);           // every lane takes part in the load
                if (row < nrows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 pk;
                        uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                        for (int j2 = 0; j2 < 4; ++j2) {
                            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * j2]) * inv,
                                                                      __uint_as_float(o[i + 2 * j2 + 1]) * inv);
                            w[j2] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = pk;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {                                                         // give copies in flight time to land
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_free(tmem_base_slot, 256u);
    }
}

static const size_t FA_SMEM_BYTES = (size_t)FA_BM * 128 + 2 * FA_KV_STAGES * FA_BN * 128 + 256 + 1024;

// q: the fused qkv buffer [n_rows_total, q_stride] (head h of q at column h * 64); out [n_rows_total, nh * 64];
// kv_cache [num_pages, 2, nkv, page_size, 64]; tiles [n_tiles][3] with at most 128 rows each.
// Takes head size 64 and page sizes 8, 16, 32, 64 and 128; refuses everything else.
extern "C" int rg_prefill_attention_tc(const void* q, int q_stride, int n_rows_total, void* out, const void* kv_cache,
                                       int num_pages, const int* block_table, int max_blocks, const int* tiles,
                                       int n_tiles, const int* positions, int nh, int nkv, int d, int page_size,
                                       int window, float scale, int* err, void* stream) {
    if (n_tiles <= 0) return 0;
    if (d != FA_D || nkv < 1 || nh < nkv || nh % nkv || page_size % 8 || page_size > 128 || 128 % page_size || q_stride % 8 ||
        ((uintptr_t)q & 15) || ((uintptr_t)kv_cache & 15) || (long long)n_tiles * nh > 0x7fffffffll)
        return RG_ERR_UNSUPPORTED;
    CUtensorMap qm, kvm;
    int e = rg_make_map(&qm, q, (unsigned long long)n_rows_total, (unsigned long long)q_stride, (unsigned long long)q_stride, FA_BM);
    if (e) return e;
    e = rg_make_map(&kvm, kv_cache, (unsigned long long)num_pages * 2ull * nkv * page_size, FA_D, FA_D,
                    page_size < FA_BN ? page_size : FA_BN);
    if (e) return e;
    static unsigned long long smem_allowed = 0;                              // one bit per device: set once, not per call
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev > 63) dev = 63;
    if (dev == 63 || !(smem_allowed >> dev & 1ull)) {
        cudaError_t ce = cudaFuncSetAttribute(fa_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_SMEM_BYTES);
        if (ce != cudaSuccess) return (int)ce;
        smem_allowed |= 1ull << dev;
    }
    return rg_launch(fa_tc_kernel, dim3(n_tiles * nh), dim3(FA_THREADS), FA_SMEM_BYTES, (cudaStream_t)stream, 1, qm, kvm,
                     (bf16*)out, block_table, max_blocks, tiles, positions, nh, nkv, page_size, window,
                     scale * 1.4426950408889634f, err);
}
