// Weight-streaming matrix product for decode: y[M, N] = x[M, K] W[N, K]^T with M <= 64.
//
// At these sizes the product is bound by reading W once from HBM, so the
// kernel is built around keeping many 16-byte loads of W in flight and nothing
// else: the weight rows take the tensor core's M side (swap-AB: 16 rows of W
// per mma, the batch on the 8-wide N side), both operand fragments come
// straight from 16-byte global loads (the k index is permuted the same way in
// both operands, which a dot product does not notice), W never touches shared
// memory and bypasses L1.  The warps of a block split K and are summed through
// shared memory in a fixed order, so a row's result depends neither on the
// batch it is in nor on anything but its own inputs.
//
// Epilogues: plain (bf16 or fp32 out), and SiLU-mul for the gate|up
// projection stored interleaved (rows 16t..16t+7 gate, 16t+8..16t+15 the
// matching up rows), out[m, 8t + j] = silu(gate) * up in 32-bit
// (crates/vllm-models/src/llama/architecture.rs:81-85).  The reference runs
// these products through cuBLAS (crates/vllm-models/src/llama/attention.rs:94-96,133).
#pragma once
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define EPI_NONE 0
#define EPI_SILU_MUL 1
#define EPI_RESIDUAL 2            // out (32-bit) += product; also the next norm's input and sums of squares
#define EPI_ROPE_CACHE 3          // the fused q|k|v projection: rotate q and k, write q out and k, v into the paged cache
#define PRO_PLAIN 0
#define PRO_SCALED 1              // x is a residual row times the norm's weight; 1 / rms is applied to the sums

// RMSNorm around the product without a kernel of its own.  y = W (w . r) / rms(r) is linear in 1 / rms, so the
// norm splits into a part the producer of r can do and a factor the consumer applies to its 32-bit sums:
//   EPI_RESIDUAL (producer):  r = out[m, n] += product;  scaled_out[m, n] = bf16(r * norm_w[n]);
//                             ss_out[block, m] = sum over the block's columns of r^2 (0 for m >= M).
//   PRO_SCALED (consumer):    x = scaled_out; every sum is multiplied by inv[m] = rsqrt(sum_p ss_in[p, m] / K + eps)
//                             before the epilogue (and before SiLU-mul).
// Sums of squares, 1 / rms and both products are 32-bit; the one rounding to bfloat16 is the one every
// product's input has.  ss rows are ss_ld floats apart; partial sums are added in a fixed order.
//
// EPI_ROPE_CACHE: the product is the q|k|v projection of single tokens, N = (nh + 2 nkv) d with d % 16 == 0 and the
// rows of every q and k head reordered so that rotation pair i sits at (16 (i / 8) + i % 8, + 8) (rope_cache.cu's
// `paired8` layout): every 16-row tile of W holds 8 whole pairs, so the block that owns the rows rotates them
// (32-bit sums, angles from the table [max_pos, d] = cos | sin at the token's position, one rounding), writes q
// to out and k and v straight into the token's slot of the paged cache [pages, 2, nkv, page_size, d]; the k and v
// columns of out are not written.  One kernel instead of the product followed by rope_cache.cu's.
struct SkinnyFusion {
    const float* norm_w;
    bf16* scaled_out;             // [M, N], rows ldo apart like out
    float* ss_out;
    const float* ss_in;
    int ss_in_blocks;
    int ss_ld;
    float eps;
    const float* rope_table;      // EPI_ROPE_CACHE from here
    const int* positions;
    const int* slots;             // nullptr: nothing is written to the cache
    bf16* kv_cache;
    int nh, nkv, d, page_size, max_pos;
    int* err;                     // set to 1 when a position is outside the table (never read outside it)
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One block: RT x 16 rows of W (from n0) and one slice of K, split over NW warps in interleaved 128-wide
// pieces; every warp multiplies all RT row tiles by the same fragments of x.  CS blocks of a cluster share the
// rows and take one K slice each; block 0 of the cluster adds the slices' sums, read from the other blocks'
// shared memory, in rank order (the same order every time).
// MT: batch rows / 8 (rounded up).  x rows are ldx elements apart.  K % 8 == 0.
template <int MT, int NW, int CS, int RT, int EPI, int PRO, typename OUT>
__global__ void __launch_bounds__(NW * 32)
skinny_gemm_kernel(const bf16* __restrict__ W, const bf16* __restrict__ x, int ldx, OUT* __restrict__ out, int ldo,
                   int M, int N, int K, SkinnyFusion fu) {
    extern __shared__ float red[];                     // [NW][RT * 16][8 * MT], then the block's sum [RT * 16][8 * MT]
    constexpr int COLS = 8 * MT, ROWS = RT * 16;
    __shared__ float ss_warp[PRO == PRO_SCALED ? NW * COLS : 1];   // per warp: its share of every row's sum of squares
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int rank = CS > 1 ? (int)(blockIdx.x % CS) : 0;
    const int n0 = (int)(blockIdx.x / CS) * ROWS;
    const int slice = ((K + CS * 128 - 1) / (CS * 128)) * 128;     // K slice of one block, a multiple of 128
    const int k_lo = rank * slice, k_hi = min(K, k_lo + slice);
    const bf16* w0[RT];
    const bf16* w1[RT];
    bool v0[RT], v1[RT];
#pragma unroll
    for (int t = 0; t < RT; ++t) {
        const int r0 = n0 + t * 16 + g, r1 = r0 + 8;
        v0[t] = r0 < N; v1[t] = r1 < N;
        w0[t] = W + (size_t)(v0[t] ? r0 : 0) * K + tq * 8;
        w1[t] = W + (size_t)(v1[t] ? r1 : 0) * K + tq * 8;
    }
    const bf16* xr[MT];
    bool xv[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        const int m = j * 8 + g;
        xv[j] = m < M;
        xr[j] = x + (size_t)(xv[j] ? m : 0) * ldx + tq * 8;
    }
    float acc[RT][MT][4];
#pragma unroll
    for (int t = 0; t < RT; ++t)
#pragma unroll
        for (int j = 0; j < MT; ++j) { acc[t][j][0] = acc[t][j][1] = acc[t][j][2] = acc[t][j][3] = 0.f; }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // W does not depend on the kernel before this one: its first piece is requested before the wait.
    // (Requesting every piece one iteration ahead was measured slower: the extra registers cost residency.)
    uint4 a[RT][4], b[RT][4];
    int kb = k_lo + warp * 128;
    auto load_w = [&]() {
#pragma unroll
        for (int t = 0; t < RT; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) {              // 8 RT loads of W in flight per thread
                const int k = kb + c * 32;
                const bool kin = k + tq * 8 < k_hi;
                a[t][c] = (kin && v0[t]) ? ld_stream16(w0[t] + k) : zero;
                b[t][c] = (kin && v1[t]) ? ld_stream16(w1[t] + k) : zero;
            }
    };
    load_w();
    pdl_wait();
    pdl_trigger();
    // Loads that the epilogue needs are requested now, so that they arrive while W streams.
    // EPI_RESIDUAL: the residual value and norm weight of the first element this thread will write
    float pre_r = 0.f, pre_w = 0.f;
    if (EPI == EPI_RESIDUAL && rank == 0 && threadIdx.x < ROWS * COLS) {
        const int m = threadIdx.x / ROWS, row = threadIdx.x - m * ROWS;
        if (m < M && n0 + row < N) {
            pre_r = reinterpret_cast<const float*>(out)[(size_t)m * ldo + n0 + row];
            pre_w = __ldg(fu.norm_w + n0 + row);
        }
    }
    bool first = true;
    for (; kb < k_hi; kb += NW * 128) {
        uint4 xq[MT][4];
        if (!first) load_w();
        first = false;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int k = kb + c * 32;
            const bool kin = k + tq * 8 < k_hi;
#pragma unroll
            for (int j = 0; j < MT; ++j) xq[j][c] = (kin && xv[j]) ? ld_cached16(xr[j] + k) : zero;
        }
#pragma unroll
        for (int t = 0; t < RT; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    mma16816(acc[t][j], a[t][c].x, b[t][c].x, a[t][c].y, b[t][c].y, xq[j][c].x, xq[j][c].y);
                    mma16816(acc[t][j], a[t][c].z, b[t][c].z, a[t][c].w, b[t][c].w, xq[j][c].z, xq[j][c].w);
                }
            }
    }
    if (PRO == PRO_SCALED) {
        // This thread's share of the producer's partial sums of squares (block p = 32 warp + lane, then every
        // NW * 32 further), all COLS batch rows of it; fetched here, not before the loop, where holding them would
        // cost the registers that decide how many blocks start early beside the kernel before (measured: a
        // batch-8 decode step 3 % faster; staging them in shared memory with cp.async was slower than either).
        float ssq[COLS];
#pragma unroll
        for (int m = 0; m < COLS; ++m) ssq[m] = 0.f;
        for (int p = warp * 32 + lane; p < fu.ss_in_blocks; p += NW * 32) {
            const float4* row = reinterpret_cast<const float4*>(fu.ss_in + (size_t)p * fu.ss_ld);
#pragma unroll
            for (int q = 0; q < COLS / 4; ++q) {
                const float4 v = __ldg(row + q);
                ssq[q * 4] += v.x; ssq[q * 4 + 1] += v.y; ssq[q * 4 + 2] += v.z; ssq[q * 4 + 3] += v.w;
            }
        }
#pragma unroll
        for (int m = 0; m < COLS; ++m) {
            const float t = warp_sum(ssq[m]);
            if (lane == 0) ss_warp[warp * COLS + m] = t;
        }
    }
    // the warps' partial sums -> shared memory, summed in warp order
    float* mine = red + (size_t)warp * ROWS * COLS;
#pragma unroll
    for (int t = 0; t < RT; ++t)
#pragma unroll
        for (int j = 0; j < MT; ++j) {
            const int col = j * 8 + tq * 2, row = t * 16 + g;
            mine[row * COLS + col] = acc[t][j][0];
            mine[row * COLS + col + 1] = acc[t][j][1];
            mine[(row + 8) * COLS + col] = acc[t][j][2];
            mine[(row + 8) * COLS + col + 1] = acc[t][j][3];
        }
    __syncthreads();
    float* fin = red + (size_t)NW * ROWS * COLS;        // [ROWS][COLS]
    for (int idx = threadIdx.x; idx < ROWS * COLS; idx += NW * 32) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) s += red[(size_t)w * ROWS * COLS + idx];
        fin[idx] = s;
    }
    // (with PRO_SCALED, 1 / rms multiplies the complete sums below: after the cluster's addition)
    if (CS > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                 // every block's sum is in its shared memory
        if (rank == 0) {
            for (int idx = threadIdx.x; idx < ROWS * COLS; idx += NW * 32) {
                float s = fin[idx];
#pragma unroll
                for (int r = 1; r < CS; ++r) s += cluster.map_shared_rank(fin, r)[idx];
                fin[idx] = s;
            }
        }
        cluster.sync();                                 // nobody leaves while its shared memory is being read
        if (rank != 0) return;
    }
    __syncthreads();
    auto inv_rms = [&](int m) {                          // 1 / rms of batch row m, the warps' shares added in warp order
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) t += ss_warp[w * COLS + m];
        return rsqrtf(t / (float)K + fu.eps);
    };
    if (EPI == EPI_RESIDUAL) {
        // consecutive threads, consecutive n of one batch row: ROWS (16 or 32) lanes share m and add their squares
        const int block_row = (int)(blockIdx.x / CS);
        for (int idx = threadIdx.x; idx < ROWS * COLS; idx += NW * 32) {
            const int m = idx / ROWS, row = idx - m * ROWS;
            float v = 0.f;
            if (m < M && n0 + row < N) {
                float* o = reinterpret_cast<float*>(out) + (size_t)m * ldo + n0 + row;
                const bool pre = idx < NW * 32;             // the first round's values were requested before the loop
                v = (pre ? pre_r : *o) + fin[row * COLS + m];
                *o = v;
                if (fu.scaled_out)
                    fu.scaled_out[(size_t)m * ldo + n0 + row] =
                        __float2bfloat16_rn(v * (pre ? pre_w : __ldg(fu.norm_w + n0 + row)));
            }
            float s = v * v;
#pragma unroll
            for (int off = ROWS / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (row == 0) fu.ss_out[(size_t)block_row * fu.ss_ld + m] = s;
        }
    } else if (EPI == EPI_ROPE_CACHE) {
        const int half = fu.d >> 1;
        for (int idx = threadIdx.x; idx < (ROWS / 2) * COLS; idx += NW * 32) {
            const int m = idx / (ROWS / 2), pr = idx - m * (ROWS / 2);        // pair pr of the block: tile pr / 8, row pr % 8
            const int row = (pr >> 3) * 16 + (pr & 7);
            const int f = n0 + row;                                           // output feature of the pair's first element
            if (m < M && f + 8 < N) {
                const float sc = PRO == PRO_SCALED ? inv_rms(m) : 1.f;
                const float x0 = fin[row * COLS + m] * sc, x1 = fin[(row + 8) * COLS + m] * sc;
                const int head = f / fu.d, e = f - head * fu.d;               // e: storage index inside the head
                float y0 = x0, y1 = x1;
                if (head < fu.nh + fu.nkv) {
                    int pos = fu.positions[m];
                    if (pos < 0 || pos >= fu.max_pos) {
                        if (fu.err) atomicExch(fu.err, 1);
                        pos = 0;
                    }
                    const int i = ((e >> 4) << 3) + (e & 7);                  // the pair's number = its angle's index
                    const float c = __ldg(fu.rope_table + (size_t)pos * fu.d + i);
                    const float sn = __ldg(fu.rope_table + (size_t)pos * fu.d + half + i);
                    y0 = x0 * c - x1 * sn;
                    y1 = x1 * c + x0 * sn;
                }
                if (head < fu.nh) {
                    bf16* o = reinterpret_cast<bf16*>(out) + (size_t)m * ldo + f;
                    o[0] = __float2bfloat16_rn(y0);
                    o[8] = __float2bfloat16_rn(y1);
                } else if (fu.slots) {
                    const int slot = fu.slots[m];
                    if (slot >= 0) {
                        const int kind = head < fu.nh + fu.nkv ? 0 : 1, kvh = head - fu.nh - kind * fu.nkv;
                        const int page = slot / fu.page_size, off = slot - page * fu.page_size;
                        bf16* dst = fu.kv_cache + ((((size_t)page * 2 + kind) * fu.nkv + kvh) * fu.page_size + off) * fu.d + e;
                        dst[0] = __float2bfloat16_rn(y0);
                        dst[8] = __float2bfloat16_rn(y1);
                    }
                }
            }
        }
    } else if (EPI == EPI_NONE) {
        for (int idx = threadIdx.x; idx < ROWS * COLS; idx += NW * 32) {
            const int m = idx / ROWS, row = idx - m * ROWS;   // consecutive threads -> consecutive n: coalesced stores
            if (m < M && n0 + row < N)
                out[(size_t)m * ldo + n0 + row] = from_f32<OUT>(fin[row * COLS + m] * (PRO == PRO_SCALED ? inv_rms(m) : 1.f));
        }
    } else {
        for (int idx = threadIdx.x; idx < (ROWS / 2) * COLS; idx += NW * 32) {
            const int m = idx / (ROWS / 2), o = idx - m * (ROWS / 2);  // output o of this block: tile o / 8, element o % 8
            const int row = (o >> 3) * 16 + (o & 7);
            if (m < M && n0 + row + 8 < N) {
                const float sc = PRO == PRO_SCALED ? inv_rms(m) : 1.f;
                const float gate = fin[row * COLS + m] * sc, up = fin[(row + 8) * COLS + m] * sc;
                out[(size_t)m * ldo + (n0 >> 1) + o] = from_f32<OUT>(gate / (1.f + expf(-gate)) * up);
            }
        }
    }
}

template <int MT, int NW, int CS, int RT, int EPI, int PRO, typename OUT>
static int launch_skinny(const bf16* W, const bf16* x, int ldx, OUT* out, int ldo, int M, int N, int K,
                         SkinnyFusion fu, int* row_blocks, cudaStream_t s) {
    const size_t smem = (size_t)(NW + 1) * RT * 16 * 8 * MT * sizeof(float);
    auto kernel = skinny_gemm_kernel<MT, NW, CS, RT, EPI, PRO, OUT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const unsigned blocks = (unsigned)(((N + RT * 16 - 1) / (RT * 16)) * CS);
    if (row_blocks) *row_blocks = (int)(blocks / CS);
    return rg_launch(kernel, dim3(blocks), dim3(NW * 32), smem, s, CS, W, x, ldx, out, ldo, M, N, K, fu);
}

// MAX_MT: the largest batch tile count (8 batch rows each) that is compiled; more rows are refused.
template <int EPI, int PRO, typename OUT, int MAX_MT = 8>
static int dispatch_skinny(const bf16* W, const bf16* x, int ldx, OUT* out, int ldo, int M, int N, int K,
                           SkinnyFusion fu, int* row_blocks, cudaStream_t s) {
    // Shapes from measurements on B200 at M = 8 (Llama 1B sizes): a block should stream enough of W to pay
    // for its start and its reduction (two row tiles per warp wherever there are enough rows), every warp should
    // have one or two 128-wide pieces of K, and all blocks should be resident at once.
    //   very many rows (head: 128256)            8 warps, 2 row tiles          6.75 TB/s
    //   many rows (gate|up: 16384)                4 warps, 2 row tiles          5.3 TB/s with SiLU-mul
    //   few rows, long K (down: 2048 x 8192)      8 warps, 2 row tiles, K over a cluster of 4
    //   few rows (QKV: 3072 / O: 2048)            16 warps, 2 / 1 row tiles
    const long long tiles = (N + 15) / 16;
    const int shape = tiles >= 16 * 148 ? 0 : tiles >= 4 * 148 ? 1 : (K >= 4096 && tiles < 2 * 148) ? 2
                    : tiles >= 160 ? 3 : 4;
#define RG_SK(MT_) (shape == 0 ? launch_skinny<MT_, 8, 1, 2, EPI, PRO, OUT>(W, x, ldx, out, ldo, M, N, K, fu, row_blocks, s) \
                  : shape == 1 ? launch_skinny<MT_, 4, 1, 2, EPI, PRO, OUT>(W, x, ldx, out, ldo, M, N, K, fu, row_blocks, s) \
                  : shape == 2 ? launch_skinny<MT_, 8, 4, 2, EPI, PRO, OUT>(W, x, ldx, out, ldo, M, N, K, fu, row_blocks, s) \
                  : shape == 3 ? launch_skinny<MT_, 16, 1, 2, EPI, PRO, OUT>(W, x, ldx, out, ldo, M, N, K, fu, row_blocks, s) \
                               : launch_skinny<MT_, 16, 1, 1, EPI, PRO, OUT>(W, x, ldx, out, ldo, M, N, K, fu, row_blocks, s))
    if (M <= 8) return RG_SK(1);
    if (M <= 16) return RG_SK(2);
    if constexpr (MAX_MT >= 4) {
        if (M <= 32) return RG_SK(4);
        if (M <= 64) return RG_SK(8);
    }
    return RG_ERR_UNSUPPORTED;
#undef RG_SK
}

