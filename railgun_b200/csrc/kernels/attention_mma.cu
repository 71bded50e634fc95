// Tensor-core attention over the paged cache, bfloat16 storage, 32-bit softmax
// and accumulation: a flash-style kernel for portions of prompts and a split
// kernel with its reduction for single decoded tokens.
//
// Both read K and V only through block tables (the step's own keys are
// written before they run) and mask by absolute position, so the result for a
// position does not depend on how the tokens were cut into steps.
//
//   s_j = scale * q.k_j ; m = max_j s_j ; p_j = exp(s_j - m) ; out = sum p_j v_j / sum p_j
//   kv_head = head / (nh / nkv)
// (crates/vllm-cuda/src/kernels/paged_attention.cu:40,66-69,103-107).  The
// split kernel is the counterpart of the reference's partition + reduce pair:
// per partition an unnormalised output with its max and sum, then
// out = sum_p e^{m_p - M} o_p / sum_p e^{m_p - M} l_p
// (crates/vllm-cuda/src/kernels/paged_attention_v2_partition.cu:60-107,
// crates/vllm-cuda/src/kernels/paged_attention_v2_reduce.cu:50-90); the
// reference's fixed 256-token partitions and 512-partition cap become a split
// count chosen by the caller.  The prefill kernel has no counterpart: the
// reference has no causal mask inside a portion of a prompt.
//
// Head sizes: any multiple of 16 up to 256, compiled in three register-size
// classes (<= 64, <= 128, <= 256).  Any page size.  K/V tiles are gathered
// row by row with cp.async (each key's page is looked up in the block table).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define BN 64              // keys per tile
#define NTHREADS 128       // 4 warps
#define PAD 8              // bf16 elements of padding per shared-memory row: conflict-free ldmatrix for any d % 16 == 0

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = smem_u32(dst);
    const int n = valid ? 16 : 0;          // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// D[16x8] += A[16x16] B[16x8], bf16 operands, fp32 accumulators
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x for x <= 0 (or -inf -> 0): the hardware approximation (2 ulp), in 32-bit
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gathering BN keys (rows key0 .. key0+BN-1 of a request) of K and V for one kv head into shared memory
// is done in 16-byte pieces.  The page of a piece's row is looked up one tile ahead so that the table read
// is off the critical path when the copies are issued.  Rows at or beyond key_end have page -1 and are
// zero-filled.  sK, sV: [BN][d + PAD].
// The same rule for the 64-row tiles all four warps of the prefill kernel share: piece idx = threadIdx.x +
// 128 j over 64 rows x d/8 pieces, consecutive threads on consecutive 16-byte pieces of a row.
template <int KD>
struct TileGather {
    int row[KD], dst[KD], src[KD];       // row in the tile; shared-memory offset; offset inside a page's K block
    int page_shift, page_size, d;
    __device__ __forceinline__ void init(int d_, int page_size_, int page_shift_, int kvh) {
        d = d_; page_size = page_size_; page_shift = page_shift_;
        const int d8 = d >> 3, stride = d + PAD;
#pragma unroll
        for (int j = 0; j < KD; ++j) {
            const int idx = threadIdx.x + NTHREADS * j;            // 64 d/8 = 8 d pieces
            row[j] = idx < 8 * d ? idx / d8 : -1;
            const int col = (idx % d8) * 8;
            dst[j] = row[j] * stride + col;
            src[j] = kvh * page_size * d + col;
        }
    }
    __device__ __forceinline__ void pages(const int* __restrict__ bt, int key0, int key_end, int (&pg)[KD]) const {
#pragma unroll
        for (int j = 0; j < KD; ++j) {
            const int key = key0 + row[j];
            pg[j] = (row[j] >= 0 && key < key_end) ? bt[page_shift >= 0 ? key >> page_shift : key / page_size] : -1;
        }
    }
    __device__ __forceinline__ void issue(bf16* sK, bf16* sV, const bf16* __restrict__ kv_cache, const int (&pg)[KD],
                                          int key0, size_t page_elems, int v_off) const {
#pragma unroll
        for (int j = 0; j < KD; ++j) {
            if (row[j] >= 0) {
                const bool valid = pg[j] >= 0;
                const bf16* ksrc = kv_cache;
                if (valid) {
                    const int key = key0 + row[j];
                    const int off = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
                    ksrc = kv_cache + (size_t)pg[j] * page_elems + (src[j] + off * d);
                }
                cp_async16(sK + dst[j], ksrc, valid);
                cp_async16(sV + dst[j], ksrc + (valid ? v_off : 0), valid);
            }
        }
    }
};

// ---------------------------------------------------------------------------------------------------
// Prefill: one CTA per (query tile of up to 64 consecutive positions of one request, head).
// tiles: [NT][3] = first token row, number of rows, request index.
// ---------------------------------------------------------------------------------------------------
// EXACT: the head size is DMAX itself, known at compile time (loops unroll without guards and shared-memory
// addresses fold into the instructions); otherwise any multiple of 16 up to DMAX, passed at run time.
template <int DMAX, bool EXACT>
__global__ void __launch_bounds__(NTHREADS, DMAX <= 64 ? 4 : (DMAX <= 128 ? 2 : 1))
prefill_attention_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                         const bf16* __restrict__ kv_cache, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ tiles, const int* __restrict__ positions, int nh, int nkv, int d_arg,
                         int page_size, int page_shift, int window, float scale_log2) {
    const int d = EXACT ? DMAX : d_arg;
    constexpr int KD = DMAX / 16;          // k-steps over the head dimension
    constexpr int ND = DMAX / 8;           // n-tiles of the output
    constexpr bool Q_IN_REGS = DMAX <= 128;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int stride = d + PAD;
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                 // [64][stride]
    bf16* sKV = sQ + 64 * stride;                                 // 2 stages x (K [BN][stride], V [BN][stride])
    const int stage_elems = 2 * BN * stride;

    pdl_wait();
    pdl_trigger();
    // later tiles of a prompt attend more keys: blocks are handed out in index order, so every head's
    // last tile starts first and the short ones fill the tail
    const int tile = gridDim.x / nh - 1 - blockIdx.x / nh, h = blockIdx.x % nh;
    const int row0 = tiles[tile * 3 + 0], nrows = tiles[tile * 3 + 1], r = tiles[tile * 3 + 2];
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)r * max_blocks;
    const int p0 = positions[row0];
    const int hi = p0 + nrows - 1;                                 // last key any row of the tile attends
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int kt0 = lo / BN, kt1 = hi / BN;
    const int d16 = d >> 4, d8 = d >> 3;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Q tile -> shared memory (rows beyond nrows are zeros)
    {
        const int chunks = d8;
        for (int idx = threadIdx.x; idx < 64 * chunks; idx += NTHREADS) {
            const int row = idx / chunks, c = idx - row * chunks;
            const bool valid = row < nrows;
            const bf16* src = valid ? q + (size_t)(row0 + row) * q_stride + (size_t)h * d + c * 8 : q;
            cp_async16(sQ + row * stride + c * 8, src, valid);
        }
    }
    TileGather<KD> tg;
    tg.init(d, page_size, page_shift, kvh);
    const size_t page_elems = (size_t)2 * nkv * page_size * d;
    const int v_off = nkv * page_size * d;
    int page_next[KD];
    tg.pages(bt, kt0 * BN, hi + 1, page_next);
    tg.issue(sKV, sKV + BN * stride, kv_cache, page_next, kt0 * BN, page_elems, v_off);
    cp_async_commit();
    tg.pages(bt, (kt0 + 1) * BN, hi + 1, page_next);               // beyond the last key: all -1

    uint32_t qf[Q_IN_REGS ? KD : 1][4];
    float o[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8 of this warp's 16
    const int g = lane >> 2, tq = lane & 3;
    const int prow0 = p0 + warp * 16 + g, prow1 = prow0 + 8;       // absolute positions of the two rows
    // ldmatrix source coordinates
    const int a_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_key = (lane & 7) + (lane >> 4) * 8, b_dim = ((lane >> 3) & 1) * 8;          // K as B operand
    const int v_key = (lane & 7) + ((lane >> 3) & 1) * 8, v_dim = (lane >> 4) * 8;          // V as B operand (.trans)

    for (int kt = kt0; kt <= kt1; ++kt) {
        const int stage = (kt - kt0) & 1;
        bf16* sK = sKV + stage * stage_elems;
        bf16* sV = sK + BN * stride;
        if (kt + 1 <= kt1) {
            bf16* nK = sKV + (stage ^ 1) * stage_elems;
            tg.issue(nK, nK + BN * stride, kv_cache, page_next, (kt + 1) * BN, page_elems, v_off);
            cp_async_commit();
            tg.pages(bt, (kt + 2) * BN, hi + 1, page_next);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (Q_IN_REGS && kt == kt0) {
#pragma unroll
            for (int kd = 0; kd < KD; ++kd)
                if (kd < d16) ldmatrix_x4(qf[kd], sQ + a_row * stride + kd * 16 + a_col);
        }
        // this warp's rows attend nothing in this tile?  (all keys after its last row, or before its first row's window)
        const int key_base = kt * BN;
        const int wfirst = p0 + warp * 16, wlast = wfirst + 15;      // warp-uniform: every lane takes the same branch
        const bool skip = key_base > wlast || (window > 0 && key_base + BN - 1 < wfirst - window + 1);
        if (!skip) {
            float s[BN / 8][4];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                if (kd < d16) {
                    uint32_t a[4];
                    if (Q_IN_REGS) { a[0] = qf[kd][0]; a[1] = qf[kd][1]; a[2] = qf[kd][2]; a[3] = qf[kd][3]; }
                    else ldmatrix_x4(a, sQ + a_row * stride + kd * 16 + a_col);
#pragma unroll
                    for (int j2 = 0; j2 < BN / 16; ++j2) {
                        uint32_t b[4];
                        ldmatrix_x4(b, sK + (j2 * 16 + b_key) * stride + kd * 16 + b_dim);
                        mma_bf16(s[2 * j2], a, b[0], b[1]);
                        mma_bf16(s[2 * j2 + 1], a, b[2], b[3]);
                    }
                }
            }
            // scale into the log2 domain; mask by absolute position where the tile is not wholly attended
            const bool edge = key_base + BN - 1 > wfirst || (window > 0 && key_base < wlast - window + 1);
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[j][e] * scale_log2;
                    if (edge) {
                        const int key = key_base + j * 8 + tq * 2 + (e & 1);
                        const int prow = (e < 2) ? prow0 : prow1;
                        if (!(key <= prow && (window <= 0 || key > prow - window))) v = -INFINITY;
                    }
                    s[j][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = ex2(m0 - ms0), al1 = ex2(m1 - ms1);
            m0 = mn0; m1 = mn1;
            float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
                s[j][0] = ex2(s[j][0] - ms0); s[j][1] = ex2(s[j][1] - ms0);
                s[j][2] = ex2(s[j][2] - ms1); s[j][3] = ex2(s[j][3] - ms1);
                rs0 += s[j][0] + s[j][1];
                rs1 += s[j][2] + s[j][3];
            }
            l0 = l0 * al0 + rs0;                                   // per-thread partial sums; reduced at the end
            l1 = l1 * al1 + rs1;
            if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {   // some row's max moved: rescale
#pragma unroll
                for (int i = 0; i < ND; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                uint32_t a[4];
                a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < ND / 2; ++n2) {
                    if (n2 < d16) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, sV + (kk * 16 + v_key) * stride + n2 * 16 + v_dim);
                        mma_bf16(o[2 * n2], a, b[0], b[1]);
                        mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                            // the stage may be overwritten next iteration
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int lr0 = warp * 16 + g, lr1 = lr0 + 8;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
        if (i < d8) {
            const int col = i * 8 + tq * 2;
            if (lr0 < nrows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + lr0) * nh + h) * d + col) =
                    pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
            if (lr1 < nrows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + lr1) * nh + h) * d + col) =
                    pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Decode: one CTA per (token, kv head x tile of up to 8 query heads of its group, split of the context).
// The four warps take 16 keys each of every 64-key tile, each warp gathering and consuming its own rows
// (no block-wide barrier in the loop), and are combined at the end; the CTA writes an unnormalised
// partial output with its max (log2 domain) and sum into the scratch arrays
//   part_o [n_tokens][nh][num_splits][d] (float), part_ml [n_tokens][nh][num_splits][2] (float).
// Scores are S[head, key] = Q K^T (heads padded to the 16 rows of the tensor-core tile); the output is
// accumulated transposed, O^T[dim, head] += V^T[dim, key] P^T[key, head], so that the softmax and the
// rescaling only cost work for 8 head columns and P feeds the second product straight from registers.
// ---------------------------------------------------------------------------------------------------
#ifndef DEC_STAGES
#define DEC_STAGES 3
#endif
#define DEC_HEADS 8        // query heads per CTA

template <int DMAX, bool EXACT>
__global__ void __launch_bounds__(NTHREADS)
decode_attention_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kv_cache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ rows,
                        const int* __restrict__ req_of_token, const int* __restrict__ positions,
                        float* __restrict__ part_o, float* __restrict__ part_ml, bf16* __restrict__ out,
                        int* __restrict__ counters, int nh, int nkv, int d_arg,
                        int page_size, int page_shift, int window, float scale_log2, int num_splits,
                        int head_tiles, int cluster_merge) {
    const int d = EXACT ? DMAX : d_arg;
    __shared__ int is_last;
    constexpr int KD = DMAX / 16;
    constexpr bool Q_IN_REGS = DMAX <= 128;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int stride = d + PAD;
    const int stage_elems = 2 * BN * stride;
    bf16* sKV = reinterpret_cast<bf16*>(smem_raw);                 // DEC_STAGES x (K [BN][stride], V [BN][stride])
    // Q [16][stride]: once its fragments are in registers it is not read again, so it may sit in the
    // last stage, which is first filled inside the loop
    bf16* sQ = Q_IN_REGS ? sKV + (DEC_STAGES - 1) * stage_elems : sKV + DEC_STAGES * stage_elems;

    // Positions, tables and every key but the token's own were written before the kernel that runs just before
    // this one started (its blocks all passed their own wait before this kernel could launch), so the first
    // tiles of K and V are requested ahead of the wait; q and the token's own key come from that kernel.
    // cluster_merge: the splits of a (token, head tile) are the blocks of one cluster (along x); they leave their
    // partial results in their own shared memory and add them up through distributed shared memory
    const int split = cluster_merge ? blockIdx.x : blockIdx.z;
    const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y - kvh * head_tiles;
    const int ti = cluster_merge ? blockIdx.z : blockIdx.x;
    const int t = rows ? rows[ti] : ti;
    const int group = nh / nkv;
    const int h0 = kvh * group + ht * DEC_HEADS;
    const int nheads = min(DEC_HEADS, group - ht * DEC_HEADS);
    const int r = req_of_token[t];
    const int pos = positions[t];
    const int* bt = block_table + (size_t)r * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int lo_al = (lo / BN) * BN;
    const int n_keys = pos + 1 - lo_al;
    const int per_split = ((n_keys + num_splits - 1) / num_splits + BN - 1) / BN * BN;
    const int k_begin = lo_al + split * per_split;
    const int k_end = min(pos + 1, k_begin + per_split);
    const int d16 = d >> 4, d8 = d >> 3;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;

    // With `counters` the block that finishes last for its (token, head tile) adds the splits' partial
    // results, always in split order, and writes the output; the counter is left at zero for the next launch.
    auto reduce_if_last = [&]() {
        if (counters == nullptr) return;                            // a separate kernel reduces
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            int* c = counters + (size_t)ti * gridDim.y + blockIdx.y;
            const int prev = atomicAdd(c, 1);
            is_last = prev == num_splits - 1;
            if (is_last) *c = 0;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        for (int idx = threadIdx.x; idx < nheads * d; idx += NTHREADS) {
            const int row = idx / d, col = idx - row * d;
            const size_t base = ((size_t)ti * nh + h0 + row) * num_splits;
            float M = -INFINITY;
            for (int s2 = 0; s2 < num_splits; ++s2) M = fmaxf(M, __ldcg(part_ml + (base + s2) * 2));
            const float Ms = M == -INFINITY ? 0.f : M;
            float L = 0.f, acc = 0.f;
            for (int s2 = 0; s2 < num_splits; ++s2) {
                const float w = exp2f(__ldcg(part_ml + (base + s2) * 2) - Ms);
                L += w * __ldcg(part_ml + (base + s2) * 2 + 1);
                if (w > 0.f) acc += w * __ldcg(part_o + (base + s2) * d + col);
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            out[((size_t)t * nh + h0 + row) * d + col] = __float2bfloat16_rn(acc * inv);
        }
    };
    // The splits' partial results in a cluster: fin_o [8 heads][d] unnormalised, fin_ml [8][2] = max (log2 domain) and
    // sum, behind the space of the four warps' results.  Every block of the cluster adds up its share of the
    // outputs, every one in split order: the same sums in the same order as decode_reduce_kernel.
    float* fin_o = reinterpret_cast<float*>(smem_raw) + 4 * DEC_HEADS * d + 4 * DEC_HEADS * 2;
    float* fin_ml = fin_o + DEC_HEADS * d;
    auto reduce_in_cluster = [&]() {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                             // every block's partial result is in place
        for (int idx = split * NTHREADS + threadIdx.x; idx < nheads * d; idx += num_splits * NTHREADS) {
            const int row = idx / d, col = idx - row * d;
            float M = -INFINITY;
            for (int s2 = 0; s2 < num_splits; ++s2) M = fmaxf(M, cluster.map_shared_rank(fin_ml, s2)[row * 2]);
            const float Ms = M == -INFINITY ? 0.f : M;
            float L = 0.f, acc = 0.f;
            for (int s2 = 0; s2 < num_splits; ++s2) {
                const float* ml = cluster.map_shared_rank(fin_ml, s2);
                const float w = exp2f(ml[row * 2] - Ms);
                L += w * ml[row * 2 + 1];
                if (w > 0.f) acc += w * cluster.map_shared_rank(fin_o, s2)[row * d + col];
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            out[((size_t)t * nh + h0 + row) * d + col] = __float2bfloat16_rn(acc * inv);
        }
        cluster.sync();                                             // nobody leaves while its results are being read
    };
    if (k_begin >= k_end) {                                         // an empty split: zero weight in the reduction
        pdl_wait();
        pdl_trigger();
        if (cluster_merge) {
            for (int i = threadIdx.x; i < nheads; i += NTHREADS) { fin_ml[i * 2] = -INFINITY; fin_ml[i * 2 + 1] = 0.f; }
            reduce_in_cluster();
            return;
        }
        for (int i = threadIdx.x; i < nheads; i += NTHREADS) {
            float* ml = part_ml + (((size_t)ti * nh + h0 + i) * num_splits + split) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        reduce_if_last();
        return;
    }
    const int n_tiles = (k_end - k_begin + BN - 1) / BN;

    // This warp gathers its own 16 rows of every tile.  Consecutive lanes take consecutive 16-byte pieces
    // of a row, so one instruction covers whole 128-byte lines (few, wide requests to L2).
    const size_t page_elems = (size_t)2 * nkv * page_size * d;
    const size_t v_off = (size_t)nkv * page_size * d;
    int g_row[KD], g_col[KD];                                      // piece j of this lane: row in the warp's 16, column
#pragma unroll
    for (int j = 0; j < KD; ++j) {
        const int idx = lane + 32 * j;                             // over 16 rows x d/8 pieces = 2 d pieces
        g_row[j] = idx < 2 * d ? idx / d8 : -1;
        g_col[j] = (idx % d8) * 8;
    }
    // When a page holds a multiple of 16 tokens, the warp's 16 rows of a tile are one contiguous run of the
    // cache (tiles start at multiples of 16): one table entry, pieces at consecutive addresses.
    const bool one_page = page_shift >= 4;
    int g_dst[KD];                                                 // shared-memory offset of piece j within the warp's rows
#pragma unroll
    for (int j = 0; j < KD; ++j) g_dst[j] = g_row[j] * stride + g_col[j];
    auto pages_of = [&](int key0, int (&pg)[KD]) {                 // page of every piece's row (-1: no such key)
        if (one_page) {
            const int key = key0 + warp * 16;                      // the same page for the whole warp
            pg[0] = key < k_end ? bt[key >> page_shift] : -1;
            return;
        }
#pragma unroll
        for (int j = 0; j < KD; ++j) {
            const int key = key0 + warp * 16 + g_row[j];
            pg[j] = (g_row[j] >= 0 && key < k_end) ? bt[page_shift >= 0 ? key >> page_shift : key / page_size] : -1;
        }
    };
    auto gather = [&](int stage, const int (&pg)[KD], int key0) {
        bf16* sK = sKV + stage * stage_elems + warp * 16 * stride;
        bf16* sV = sK + BN * stride;
        if (one_page) {
            const int key = key0 + warp * 16;
            const bool page_ok = pg[0] >= 0;
            const bf16* base = kv_cache;
            if (page_ok)
                base = kv_cache + (size_t)pg[0] * page_elems + ((size_t)kvh * page_size + (key & (page_size - 1))) * d;
            const int rows_ok = k_end - key;                        // rows at or beyond it are zero-filled
#pragma unroll
            for (int j = 0; j < KD; ++j) {
                if (g_row[j] >= 0) {
                    const bool valid = page_ok && g_row[j] < rows_ok;
                    const bf16* ksrc = valid ? base + (lane + 32 * j) * 8 : kv_cache;
                    cp_async16(sK + g_dst[j], ksrc, valid);
                    cp_async16(sV + g_dst[j], ksrc + (valid ? v_off : 0), valid);
                }
            }
            return;
        }
#pragma unroll
        for (int j = 0; j < KD; ++j) {
            if (g_row[j] >= 0) {
                const bool valid = pg[j] >= 0;
                const bf16* ksrc = kv_cache;
                if (valid) {
                    const int key = key0 + warp * 16 + g_row[j];
                    const int off = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
                    ksrc = kv_cache + (size_t)pg[j] * page_elems + ((size_t)kvh * page_size + off) * d + g_col[j];
                }
                cp_async16(sK + g_dst[j], ksrc, valid);
                cp_async16(sV + g_dst[j], ksrc + (valid ? v_off : 0), valid);
            }
        }
    };

    int page_next[KD];
    // a tile that holds the token's own position waits for the kernel before this one
    auto early = [&](int st) { return st < n_tiles && k_begin + (st + 1) * BN <= pos; };
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
        if (early(st)) {
            pages_of(k_begin + st * BN, page_next);
            gather(st, page_next, k_begin + st * BN);
        }
        cp_async_commit();
    }
    pdl_wait();
    pdl_trigger();
    for (int idx = threadIdx.x; idx < 16 * d8; idx += NTHREADS) {
        const int row = idx / d8, c = idx - row * d8;
        const bool valid = row < nheads;
        const bf16* src = valid ? q + (size_t)t * q_stride + (size_t)(h0 + row) * d + c * 8 : q;
        cp_async16(sQ + row * stride + c * 8, src, valid);
    }
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
        if (st < n_tiles && !early(st)) {
            pages_of(k_begin + st * BN, page_next);
            gather(st, page_next, k_begin + st * BN);
        }
    }
    cp_async_commit();                                               // Q and the tiles that had to wait: the newest group
    pages_of(k_begin + (DEC_STAGES - 1) * BN, page_next);            // beyond the split: all -1

    float oT[KD][4];                                                // O^T: dims (16 kd + g, + 8) x heads (2 tq, 2 tq + 1)
#pragma unroll
    for (int i = 0; i < KD; ++i) { oT[i][0] = oT[i][1] = oT[i][2] = oT[i][3] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;                           // of head g (lanes with g >= nheads carry padding)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_key = (lane & 7) + (lane >> 4) * 8, b_dim = ((lane >> 3) & 1) * 8;     // K as B operand
    const int vt_key = (lane & 7) + (lane >> 4) * 8, vt_dim = ((lane >> 3) & 1) * 8;   // V^T as A operand (.trans)

    uint32_t qf[Q_IN_REGS ? KD : 1][4];
    cp_async_wait<0>();                                              // Q (and the first tiles) have landed
    __syncthreads();                                                 // Q was gathered by all threads
    if (Q_IN_REGS) {
#pragma unroll
        for (int kd = 0; kd < KD; ++kd)
            if (kd < d16) ldmatrix_x4(qf[kd], sQ + a_row * stride + kd * 16 + a_col);
        __syncthreads();                                             // before the last stage is overwritten
    }

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it % DEC_STAGES;
        bf16* sK = sKV + stage * stage_elems;
        bf16* sV = sK + BN * stride;
        {
            const int nt = it + DEC_STAGES - 1;
            if (nt < n_tiles) gather(nt % DEC_STAGES, page_next, k_begin + nt * BN);
            cp_async_commit();
            pages_of(k_begin + (nt + 1) * BN, page_next);
            cp_async_wait<DEC_STAGES - 1>();
        }
        __syncwarp();
        const int key_base = k_begin + it * BN + warp * 16;          // this warp's 16 keys
        if (key_base < k_end && key_base + 15 >= lo) {
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                if (kd < d16) {
                    uint32_t a[4], b[4];
                    if (Q_IN_REGS) { a[0] = qf[kd][0]; a[1] = qf[kd][1]; a[2] = qf[kd][2]; a[3] = qf[kd][3]; }
                    else ldmatrix_x4(a, sQ + a_row * stride + kd * 16 + a_col);
                    ldmatrix_x4(b, sK + (warp * 16 + b_key) * stride + kd * 16 + b_dim);
                    mma_bf16(s0, a, b[0], b[1]);
                    mma_bf16(s1, a, b[2], b[3]);
                }
            }
            // head g, keys key_base + 2 tq + {0, 1} (s0) and + 8 (s1); rows 8..15 of the tile are padding
            float v00 = s0[0] * scale_log2, v01 = s0[1] * scale_log2, v10 = s1[0] * scale_log2, v11 = s1[1] * scale_log2;
            if (key_base + 16 > k_end || key_base < lo) {            // an edge tile: some of its keys are not attended
                const int k0 = key_base + tq * 2;
                if (!(k0 < k_end && k0 >= lo)) v00 = -INFINITY;
                if (!(k0 + 1 < k_end && k0 + 1 >= lo)) v01 = -INFINITY;
                if (!(k0 + 8 < k_end && k0 + 8 >= lo)) v10 = -INFINITY;
                if (!(k0 + 9 < k_end && k0 + 9 >= lo)) v11 = -INFINITY;
            }
            float mx = fmaxf(fmaxf(v00, v01), fmaxf(v10, v11));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m_run, mx);
            const float ms = mn == -INFINITY ? 0.f : mn;
            const float alpha = ex2(m_run - ms);
            m_run = mn;
            const float p00 = ex2(v00 - ms), p01 = ex2(v01 - ms), p10 = ex2(v10 - ms), p11 = ex2(v11 - ms);
            l_run = l_run * alpha + (p00 + p01) + (p10 + p11);       // per-thread partial; summed over tq at the end
            const uint32_t pb0 = pack_bf16(p00, p01), pb1 = pack_bf16(p10, p11);
            if (__any_sync(0xffffffffu, alpha != 1.f)) {             // some head's max moved: rescale
                const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * tq) * 4);
                const float al1 = __shfl_sync(0xffffffffu, alpha, (2 * tq + 1) * 4);
#pragma unroll
                for (int kd = 0; kd < KD; ++kd) { oT[kd][0] *= al0; oT[kd][1] *= al1; oT[kd][2] *= al0; oT[kd][3] *= al1; }
            }
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                if (kd < d16) {
                    uint32_t a[4];
                    ldmatrix_x4_trans(a, sV + (warp * 16 + vt_key) * stride + kd * 16 + vt_dim);
                    mma_bf16(oT[kd], a, pb0, pb1);
                }
            }
        }
        __syncwarp();                                                // this warp's rows of the stage are free again
    }
    cp_async_wait<0>();
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    // combine the four warps through shared memory (the K/V stages are free now)
    float* cO = reinterpret_cast<float*>(smem_raw);                  // [4 warps][8 heads][d]
    float* cML = cO + 4 * DEC_HEADS * d;                             // [4][8][2]
    __syncthreads();
#pragma unroll
    for (int kd = 0; kd < KD; ++kd) {
        if (kd < d16) {
            const int dim = kd * 16 + g;
            float* base = cO + (size_t)warp * DEC_HEADS * d;
            base[(2 * tq) * d + dim] = oT[kd][0];
            base[(2 * tq + 1) * d + dim] = oT[kd][1];
            base[(2 * tq) * d + dim + 8] = oT[kd][2];
            base[(2 * tq + 1) * d + dim + 8] = oT[kd][3];
        }
    }
    if (tq == 0) {
        cML[(warp * DEC_HEADS + g) * 2] = m_run;
        cML[(warp * DEC_HEADS + g) * 2 + 1] = l_run;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nheads * d; idx += NTHREADS) {
        const int row = idx / d, col = idx - row * d;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, cML[(w * DEC_HEADS + row) * 2]);
        const float Ms = M == -INFINITY ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float sc = exp2f(cML[(w * DEC_HEADS + row) * 2] - Ms);
            acc += sc * cO[((size_t)w * DEC_HEADS + row) * d + col];
            L += sc * cML[(w * DEC_HEADS + row) * 2 + 1];
        }
        if (num_splits == 1 && counters != nullptr) {               // the only split: this is the result
            const float inv = L > 0.f ? 1.f / L : 0.f;
            out[((size_t)t * nh + h0 + row) * d + col] = __float2bfloat16_rn(acc * inv);
        } else if (cluster_merge) {
            fin_o[row * d + col] = acc;
            if (col == 0) { fin_ml[row * 2] = M; fin_ml[row * 2 + 1] = L; }
        } else {
            const size_t base = ((size_t)ti * nh + h0 + row) * num_splits + split;
            part_o[base * d + col] = acc;
            if (col == 0) { part_ml[base * 2] = M; part_ml[base * 2 + 1] = L; }
        }
    }
    if (cluster_merge) reduce_in_cluster();
    else if (num_splits > 1) reduce_if_last();
}

// out[t, h, :] = sum_s 2^{m_s - M} o_s / sum_s 2^{m_s - M} l_s
__global__ void decode_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     bf16* __restrict__ out, const int* __restrict__ rows, int nh, int d,
                                     int num_splits) {
    pdl_wait();
    pdl_trigger();
    const int ti = blockIdx.x, h = blockIdx.y;
    const int t = rows ? rows[ti] : ti;
    const size_t base = ((size_t)ti * nh + h) * num_splits;
    float M = -INFINITY;
    for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f;
    for (int s = 0; s < num_splits; ++s) L += exp2f(part_ml[(base + s) * 2] - Ms) * part_ml[(base + s) * 2 + 1];
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < num_splits; ++s) {
            const float w = exp2f(part_ml[(base + s) * 2] - Ms);
            if (w > 0.f) acc += w * part_o[(base + s) * d + c];
        }
        out[((size_t)t * nh + h) * d + c] = __float2bfloat16_rn(acc * inv);
    }
}

static size_t prefill_smem(int d) { return (size_t)(64 + 2 * 2 * BN) * (d + PAD) * sizeof(bf16); }
static size_t decode_smem(int d) {
    // stages (+ a separate Q tile for the largest head-size class); the end-of-kernel combine reuses them
    const size_t stages = (size_t)((d > 128 ? 16 : 0) + DEC_STAGES * 2 * BN) * (d + PAD) * sizeof(bf16);
    const size_t combine = (size_t)(4 * DEC_HEADS * d + 4 * DEC_HEADS * 2 + DEC_HEADS * d + DEC_HEADS * 2) * sizeof(float);
    return stages > combine ? stages : combine;
}

template <typename K> static int allow_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

extern "C" int rg_prefill_attention(const void* q, int q_stride, void* out, const void* kv_cache,
                                    const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                                    const int* positions, int nh, int nkv, int d, int page_size, int window,
                                    float scale, void* stream) {
    if (n_tiles <= 0) return 0;
    if (d % 16 || d < 16 || d > 256 || nkv < 1 || nh < nkv || nh % nkv || (long long)n_tiles * nh > 0x7fffffffll)
        return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = prefill_smem(d);
    int page_shift = -1;                                            // log2 of the page size when it is a power of two
    for (int b = 0; b < 31; ++b) if (page_size == (1 << b)) page_shift = b;
    dim3 grid(n_tiles * nh);
#define RG_PREFILL(DM, EX) { int e = allow_smem(prefill_attention_kernel<DM, EX>, smem); if (e) return e; \
    return rg_launch(prefill_attention_kernel<DM, EX>, grid, dim3(NTHREADS), smem, s, 1, (const bf16*)q, q_stride, \
        (bf16*)out, (const bf16*)kv_cache, block_table, max_blocks, tiles, positions, nh, nkv, d, page_size, page_shift, \
        window, scale_log2); }
    if (d == 64) RG_PREFILL(64, true) else if (d == 128) RG_PREFILL(128, true)
    else if (d < 64) RG_PREFILL(64, false) else if (d < 128) RG_PREFILL(128, false) else RG_PREFILL(256, false)
#undef RG_PREFILL
}

static int rg_decode_attention_any(const void* q, int q_stride, void* out, const void* kv_cache,
                                   const int* block_table, int max_blocks, const int* rows, int n_tokens,
                                   const int* req_of_token, const int* positions, float* part_o, float* part_ml,
                                   int* counters, int nh, int nkv, int d, int page_size, int window, float scale,
                                   int num_splits, int cluster_merge, void* stream);

// Scratch the caller provides: part_o floats = n_tokens * nh * num_splits * d; part_ml = n_tokens * nh * num_splits * 2.
// counters: NULL (a second kernel reduces the splits), or n_tokens * nkv * ceil(group / 8) ints that are zero on
// entry and are left zero (the last block of each token and head tile reduces and resets its counter).
extern "C" int rg_decode_attention(const void* q, int q_stride, void* out, const void* kv_cache,
                                   const int* block_table, int max_blocks, const int* rows, int n_tokens,
                                   const int* req_of_token, const int* positions, float* part_o, float* part_ml,
                                   int* counters, int nh, int nkv, int d, int page_size, int window, float scale,
                                   int num_splits, void* stream) {
    return rg_decode_attention_any(q, q_stride, out, kv_cache, block_table, max_blocks, rows, n_tokens, req_of_token,
                                   positions, part_o, part_ml, counters, nh, nkv, d, page_size, window, scale, num_splits,
                                   0, stream);
}

// The same with the splits of every (token, head tile) as one thread-block cluster (2 to 8 splits): no scratch, no
// counters, no second kernel; the blocks add their partial results through distributed shared memory, in split
// order like the other two ways (the same bits).  Alone it is the fastest of the three (8 tokens, 1,024 keys, 4
// splits: 6.8 us against 10.1 with the second kernel), but inside a decode step, between the projection kernels
// that start early beside it, a batch-8 step took 0.87 ms with it against 0.76 ms (clusters of 4; of 8: 0.90), so
// the engine does not use it.
extern "C" int rg_decode_attention_cluster(const void* q, int q_stride, void* out, const void* kv_cache,
                                           const int* block_table, int max_blocks, const int* rows, int n_tokens,
                                           const int* req_of_token, const int* positions, int nh, int nkv, int d,
                                           int page_size, int window, float scale, int num_splits, void* stream) {
    if (num_splits < 2 || num_splits > 8 || n_tokens > 65535) return RG_ERR_UNSUPPORTED;
    return rg_decode_attention_any(q, q_stride, out, kv_cache, block_table, max_blocks, rows, n_tokens, req_of_token,
                                   positions, nullptr, nullptr, nullptr, nh, nkv, d, page_size, window, scale, num_splits,
                                   1, stream);
}

static int rg_decode_attention_any(const void* q, int q_stride, void* out, const void* kv_cache,
                                   const int* block_table, int max_blocks, const int* rows, int n_tokens,
                                   const int* req_of_token, const int* positions, float* part_o, float* part_ml,
                                   int* counters, int nh, int nkv, int d, int page_size, int window, float scale,
                                   int num_splits, int cluster_merge, void* stream) {
    if (n_tokens <= 0) return 0;
    if (d % 16 || d < 16 || d > 256 || nkv < 1 || nh < nkv || nh % nkv || num_splits < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = decode_smem(d);
    const int group = nh / nkv;
    const int head_tiles = (group + DEC_HEADS - 1) / DEC_HEADS;
    int page_shift = -1;                                            // log2 of the page size when it is a power of two
    for (int b = 0; b < 31; ++b) if (page_size == (1 << b)) page_shift = b;
    if (num_splits > 65535 || nkv * head_tiles > 65535) return RG_ERR_UNSUPPORTED;
    dim3 grid(n_tokens, nkv * head_tiles, num_splits);
    if (cluster_merge) grid = dim3(num_splits, nkv * head_tiles, n_tokens);
    int e = 0;
#define RG_DECODE(DM, EX) { e = allow_smem(decode_attention_kernel<DM, EX>, smem); if (e) return e; \
    e = rg_launch(decode_attention_kernel<DM, EX>, grid, dim3(NTHREADS), smem, s, cluster_merge ? num_splits : 1, \
        (const bf16*)q, q_stride, \
        (const bf16*)kv_cache, block_table, max_blocks, rows, req_of_token, positions, part_o, part_ml, (bf16*)out, \
        counters, nh, nkv, d, page_size, page_shift, window, scale_log2, num_splits, head_tiles, cluster_merge); }
    if (d == 64) RG_DECODE(64, true) else if (d == 128) RG_DECODE(128, true)
    else if (d < 64) RG_DECODE(64, false) else if (d < 128) RG_DECODE(128, false) else RG_DECODE(256, false)
#undef RG_DECODE
    if (e || counters != nullptr || cluster_merge) return e;
    dim3 rgrid(n_tokens, nh);
    RgStreamOrder in_order(true);       // measured: the merge starting early, beside the splits, costs a batch-8 step 4 %
    return rg_launch(decode_reduce_kernel, rgrid, dim3(d >= 128 ? 128 : 64), 0, s, 1, (const float*)part_o,
                     (const float*)part_ml, (bf16*)out, rows, nh, d, num_splits);
}

// ---------------------------------------------------------------------------------------------------
// The same split decode attention for callers that cannot allocate: scratch in a fixed device array.
// Declaration, limits and rules of use: attention_static_scratch.h.
// ---------------------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>
#include "attention_static_scratch.h"

// In host code this name is a stand-in for the symbol, not a device address; kernels get the address that
// cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char rg_static_scratch[RG_STATIC_SCRATCH_BYTES];

#define RG_MAX_DEVICES 64
static float* rg_static_scratch_ptr[RG_MAX_DEVICES];
static std::mutex rg_static_scratch_mutex;

static void rg_set_error(char* text, int cap, const char* msg) {
    if (text && cap > 0) snprintf(text, (size_t)cap, "%s", msg);
}

extern "C" int rg_decode_attention_static_scratch(
        const void* q, int q_stride, void* out, const void* kv_cache, const int* block_table, int max_blocks,
        const int* rows, int n_tokens, const int* req_of_token, const int* positions,
        int num_heads, int num_kv_heads, int head_dim, int page_size, int window, float scale, int num_splits,
        void* stream, char* error_text, int error_cap) {
    if (n_tokens <= 0) return 0;
    if (num_splits < 1 || num_heads < 1 || num_kv_heads < 1 || head_dim < 1) {
        rg_set_error(error_text, error_cap, "num_splits, num_heads, num_kv_heads and head_dim must be positive");
        return RG_ERR_UNSUPPORTED;
    }
    // part_o floats, rounded up to 64 floats (256 bytes), then part_ml likewise, then the counters
    const unsigned long long slots = (unsigned long long)n_tokens * num_heads * num_splits;
    const unsigned long long o_floats = (slots * head_dim + 63ull) / 64ull * 64ull;
    const unsigned long long ml_floats = (slots * 2ull + 63ull) / 64ull * 64ull;
    const unsigned long long n_counters = (unsigned long long)n_tokens * num_kv_heads *
                                          ((num_heads / num_kv_heads + 7) / 8);
    const unsigned long long need = (o_floats + ml_floats + n_counters) * sizeof(float);
    if (need > RG_STATIC_SCRATCH_BYTES) {
        char msg[320];
        snprintf(msg, sizeof msg,
                 "scratch of %llu bytes needed (n_tokens %d x heads %d x splits %d x (head_dim %d + 2) floats, each "
                 "part rounded up to 256 bytes, and %llu counters) but the fixed array holds %u: use fewer splits "
                 "or tokens per call",
                 need, n_tokens, num_heads, num_splits, head_dim, n_counters, (unsigned)RG_STATIC_SCRATCH_BYTES);
        rg_set_error(error_text, error_cap, msg);
        return RG_ERR_SCRATCH_TOO_LARGE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= RG_MAX_DEVICES) {
        rg_set_error(error_text, error_cap, "cannot tell the current device");
        return e != cudaSuccess ? (int)e : RG_ERR_UNSUPPORTED;
    }
    float* base;
    {
        std::lock_guard<std::mutex> lock(rg_static_scratch_mutex);
        if (rg_static_scratch_ptr[dev] == nullptr) {              // first call on this device: look the address up
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, rg_static_scratch);
            if (e != cudaSuccess || p == nullptr) {
                rg_set_error(error_text, error_cap, "cudaGetSymbolAddress failed for the scratch array");
                return e != cudaSuccess ? (int)e : RG_ERR_UNSUPPORTED;
            }
            rg_static_scratch_ptr[dev] = (float*)p;
        }
        base = rg_static_scratch_ptr[dev];
    }
    // The counters sit behind this call's partial results, at a place that depends on the sizes, and an earlier
    // call of other sizes may have left partial results there: every call clears its own counters first, on the
    // caller's stream (a memset node, no allocation).  That is also why calls must not overlap on the GPU.
    int* counters = reinterpret_cast<int*>(base + o_floats + ml_floats);
    cudaError_t ce = cudaMemsetAsync(counters, 0, n_counters * sizeof(int), (cudaStream_t)stream);
    if (ce != cudaSuccess) { rg_set_error(error_text, error_cap, cudaGetErrorString(ce)); return (int)ce; }
    const int code = rg_decode_attention(q, q_stride, out, kv_cache, block_table, max_blocks, rows, n_tokens,
                                         req_of_token, positions, base, base + o_floats, counters, num_heads,
                                         num_kv_heads, head_dim, page_size, window, scale, num_splits, stream);
    if (code == RG_ERR_UNSUPPORTED)
        rg_set_error(error_text, error_cap, "the kernels refuse these sizes (head_dim 16..256 in steps of 16, "
                                            "num_heads a multiple of num_kv_heads)");
    else if (code != 0)
        rg_set_error(error_text, error_cap, cudaGetErrorString((cudaError_t)code));
    return code;
}
