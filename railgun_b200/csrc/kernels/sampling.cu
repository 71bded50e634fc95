// Sampling over 32-bit logits: one thread block per row for short rows and for the greedy kernels, a cluster of
// eight blocks per row when a token is drawn from a long row.
//
// Greedy: argmax, ties to the lowest index (crates/vllm-models/src/llama/model.rs:210-218).
// Temperature: p = softmax(logits / T); top-k keeps logits >= the k-th largest,
// ties kept, k >= V or k = 0 no filter (crates/vllm-engine/src/sampling.rs:50-62);
// top-p keeps the probabilities >= t, t the largest value whose kept mass
// reaches top_p (crates/vllm-scheduler/src/request.rs:49-53); the token is the
// first index whose cumulative kept probability exceeds u * (kept mass).
// u comes from a counter-based generator (seed, counter), so a request's draws
// do not depend on the batch it is in or on when it runs; the reference seeds
// a new sampler from the wall clock every step (crates/vllm-engine/src/sampling.rs:19-30).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// order-preserving map float -> unsigned
__device__ __forceinline__ unsigned f2ord(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f(unsigned u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarp ? sv[lane] : -INFINITY;
        idx = lane < nwarp ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) { sv[0] = v; si[0] = idx; }
    }
    __syncthreads();
    v = sv[0];
    idx = si[0];
}

__global__ void argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_wait();
    pdl_trigger();
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    block_argmax(best, bi, sv, si);
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// ---------------------------------------------------------------------------------------------------
// Drawing a token.  A thread-block cluster of C blocks works on one row, each block on a contiguous part
// of it; what the blocks find is exchanged through distributed shared memory and added in rank order, so every
// block holds the same totals and takes the same decisions.
// Both filters are selections of a threshold: top-k wants the largest value u with count(logit >= u) >= k,
// top-p the largest e with mass(exp >= e) >= top_p * total.  Each is found by a radix search over the bit
// pattern, four bits a pass from the top (the patterns of floats order as the floats do): a pass counts, for
// the 16 values of the next four bits, the elements that agree with the bits chosen so far, in registers (no
// floating-point atomics: sums are added in a fixed order, so the same row gives the same token on every run),
// and picks the bucket in which the running count or mass crosses the target.  As soon as the elements at or
// above the chosen bucket are few (<= LIST_CAP), they are copied to the first block's shared memory, put
// into index order, and everything left is done there, one element per thread; kept sets that stay large (no
// filter, or a flat distribution) finish over the whole row.
// ---------------------------------------------------------------------------------------------------
#define LIST_CAP 1024
#define SAMPLE_MAX_CLUSTER 8

struct SampleShared {
    unsigned red_u[32][16];
    float red_f[32][16];
    unsigned tot_u[2][16];          // this block's totals, two buffers: the other blocks read one while the
    float tot_f[2][16];             // next exchange already fills the other
    float xv[2];                    // one value to exchange (a maximum, a sum)
    int xi[2];
    unsigned all_u[16];             // the cluster's totals
    float all_f[16];
    float sv[33];
    int si[32];
    float lv[2][LIST_CAP];          // candidates: logits (unordered, then by index); later their weights
    int li[2][LIST_CAP];
    int n_list;
    float seg[SAMPLE_THREADS];
    float wseg[32];
    int owner;
    float before;
};

// 16 packed counters of 16 bits each (a thread sees fewer than 65,536 elements a pass) in 8 registers
__device__ __forceinline__ void count_bucket(unsigned (&cp)[8], unsigned b, bool on) {
    const unsigned inc = on ? (1u << ((b & 1u) << 4)) : 0u;
    const unsigned w = b >> 1;
#pragma unroll
    for (int j = 0; j < 8; ++j) cp[j] += (w == (unsigned)j) ? inc : 0u;
}
__device__ __forceinline__ bool agrees_above(unsigned bits, unsigned prefix, int shift) {   // bits above shift + 3
    return shift >= 28 || ((bits ^ prefix) >> (shift + 4)) == 0u;
}

// What the blocks of a row's cluster exchange.  Every method is called by all threads of all blocks.
template <int C>
struct RowCluster {
    SampleShared& S;
    cg::cluster_group cl;
    int parity;
    __device__ RowCluster(SampleShared& s) : S(s), cl(cg::this_cluster()), parity(0) {}
    __device__ int rank() const { return C > 1 ? (int)cl.block_rank() : 0; }
    __device__ void sync() { if (C > 1) cl.sync(); else __syncthreads(); }

    // 16 counters -> S.all_u
    __device__ void totals_u(const unsigned (&cp)[8]) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, p = parity;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned lo = __reduce_add_sync(0xffffffffu, cp[j] & 0xffffu);
            const unsigned hi = __reduce_add_sync(0xffffffffu, cp[j] >> 16);
            if (lane == 0) { S.red_u[warp][2 * j] = lo; S.red_u[warp][2 * j + 1] = hi; }
        }
        __syncthreads();
        if (threadIdx.x < 16) {
            unsigned t = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += S.red_u[w][threadIdx.x];
            S.tot_u[p][threadIdx.x] = t;
        }
        sync();
        if (threadIdx.x < 16) {
            unsigned t = 0;
            for (int r = 0; r < C; ++r) t += C > 1 ? cl.map_shared_rank(&S.tot_u[p][0], r)[threadIdx.x] : S.tot_u[p][threadIdx.x];
            S.all_u[threadIdx.x] = t;
        }
        __syncthreads();
        parity ^= 1;
    }
    // 16 counters and 16 sums of weights (added in a fixed order) -> S.all_u, S.all_f
    __device__ void totals_uf(const unsigned (&cp)[8], float (&m)[16]) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, p = parity;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned lo = __reduce_add_sync(0xffffffffu, cp[j] & 0xffffu);
            const unsigned hi = __reduce_add_sync(0xffffffffu, cp[j] >> 16);
            if (lane == 0) { S.red_u[warp][2 * j] = lo; S.red_u[warp][2 * j + 1] = hi; }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            m[j] = warp_sum(m[j]);
            if (lane == 0) S.red_f[warp][j] = m[j];
        }
        __syncthreads();
        if (threadIdx.x < 16) {
            unsigned t = 0;
            float f = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { t += S.red_u[w][threadIdx.x]; f += S.red_f[w][threadIdx.x]; }
            S.tot_u[p][threadIdx.x] = t;
            S.tot_f[p][threadIdx.x] = f;
        }
        sync();
        if (threadIdx.x < 16) {
            unsigned t = 0;
            float f = 0.f;
            for (int r = 0; r < C; ++r) {
                t += C > 1 ? cl.map_shared_rank(&S.tot_u[p][0], r)[threadIdx.x] : S.tot_u[p][threadIdx.x];
                f += C > 1 ? cl.map_shared_rank(&S.tot_f[p][0], r)[threadIdx.x] : S.tot_f[p][threadIdx.x];
            }
            S.all_u[threadIdx.x] = t;
            S.all_f[threadIdx.x] = f;
        }
        __syncthreads();
        parity ^= 1;
    }
    // the sum of one value per thread over the whole cluster; `mine` gets this block's share, `before` the
    // shares of the blocks of lower rank
    __device__ float sum(float v, float* mine = nullptr, float* before = nullptr) {
        const int p = parity;
        const float b = block_sum(v, S.sv);
        if (threadIdx.x == 0) S.xv[p] = b;
        sync();
        float t = 0.f, bef = 0.f;
        for (int r = 0; r < C; ++r) {
            const float x = C > 1 ? *cl.map_shared_rank(&S.xv[p], r) : S.xv[p];
            if (r < rank()) bef += x;
            t += x;
        }
        if (mine) *mine = b;
        if (before) *before = bef;
        parity ^= 1;
        return t;
    }
    // the largest value and, among equals, the lowest index
    __device__ void argmax(float& v, int& idx) {
        const int p = parity;
        block_argmax(v, idx, S.sv, S.si);
        if (threadIdx.x == 0) { S.xv[p] = v; S.xi[p] = idx; }
        sync();
        for (int r = 0; r < C; ++r) {
            const float ov = C > 1 ? *cl.map_shared_rank(&S.xv[p], r) : S.xv[p];
            const int oi = C > 1 ? *cl.map_shared_rank(&S.xi[p], r) : S.xi[p];
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        parity ^= 1;
    }
    // append to the list in the first block's shared memory
    __device__ void list_push(float v, int i) {
        SampleShared* S0 = C > 1 ? cl.map_shared_rank(&S, 0) : &S;
        const int at = atomicAdd(&S0->n_list, 1);
        if (at < LIST_CAP) { S0->lv[0][at] = v; S0->li[0][at] = i; }
    }
};

__device__ __forceinline__ int block_min_int(int v, SampleShared& S) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = __reduce_min_sync(0xffffffffu, v);
    __syncthreads();
    if (lane == 0) S.si[warp] = v;
    __syncthreads();
    int t = S.si[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) t = min(t, S.si[w]);
    return t;
}

// Every thread's share of elements [first, first + n) of a row, f(value, index): 16-byte loads, two in
// flight, when the part allows it (its length a multiple of four and its start aligned); the order in which a
// thread sees its elements is fixed.
template <typename F>
__device__ __forceinline__ void for_part(const float* __restrict__ row, int first, int n, bool vec, F f) {
    if (vec) {
        const float4* r4 = reinterpret_cast<const float4*>(row + first);
        const int n4 = n >> 2, nthr = blockDim.x;
        int i = threadIdx.x;
        for (; i + nthr < n4; i += 2 * nthr) {
            const float4 a = __ldg(r4 + i), b = __ldg(r4 + i + nthr);
            const int ia = first + 4 * i, ib = first + 4 * (i + nthr);
            f(a.x, ia); f(a.y, ia + 1); f(a.z, ia + 2); f(a.w, ia + 3);
            f(b.x, ib); f(b.y, ib + 1); f(b.z, ib + 2); f(b.w, ib + 3);
        }
        if (i < n4) {
            const float4 a = __ldg(r4 + i);
            const int ia = first + 4 * i;
            f(a.x, ia); f(a.y, ia + 1); f(a.z, ia + 2); f(a.w, ia + 3);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) f(row[first + i], first + i);
    }
}

// Per-row parameters; temperature <= 0 means greedy.  Grid: rows * C blocks in clusters of C.
template <int C>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
              const unsigned long long* __restrict__ counter, int* __restrict__ out) {
    __shared__ SampleShared S;
    RowCluster<C> R(S);
    pdl_wait();
    pdl_trigger();
    const int row_i = blockIdx.x / C, rank = R.rank();
    const float* row = logits + (size_t)row_i * V;
    const float T = temperature[row_i];
    const int tid = threadIdx.x, nthr = blockDim.x;
    // this block's part of the row: a multiple of four elements, so that parts start aligned
    const int part = ((V + C - 1) / C + 3) & ~3;
    const int first = min(V, rank * part), count = min(V, first + part) - first;
    const bool vec = (count & 3) == 0 && (reinterpret_cast<uintptr_t>(row + first) & 15) == 0;
    if (tid == 0) S.n_list = 0;

    float best = -INFINITY;
    int bi = 0x7fffffff;
    for_part(row, first, count, vec, [&](float v, int i) {
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    });
    R.argmax(best, bi);
    if (bi == 0x7fffffff) bi = 0;                                   // a row without a largest value (all NaN)
    if (!(T > 0.f)) {
        if (tid == 0 && rank == 0) out[row_i] = bi;
        R.sync();                                                   // nobody leaves while its shared memory is read
        return;
    }
    const float inv_t = 1.f / T;
    const float zmax = best * inv_t;
    const int k = top_k ? top_k[row_i] : 0;
    const bool use_k = k > 0 && k < V;
    const float pp = top_p ? top_p[row_i] : 1.f;
    const bool use_p = pp < 1.f;
    const float u = uniform_from_counter(seed[row_i], counter[row_i]);

    float logit_thr = -INFINITY;        // top-k: logits below it are dropped
    float e_thr = 0.f;                  // top-p: weights exp(z - zmax) below it are dropped
    float total = 0.f;                  // the weight of everything top-k keeps
    bool listed = false;                // the candidates are in the first block's shared memory
    bool k_done = !use_k;               // logit_thr is final

    if (use_k) {
        unsigned prefix = 0u, above = 0u;
        for (int shift = 28; shift >= 0 && !listed; shift -= 4) {
            unsigned cp[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
            for_part(row, first, count, vec, [&](float v, int) {
                const unsigned o = f2ord(v);
                count_bucket(cp, (o >> shift) & 15u, agrees_above(o, prefix, shift));
            });
            R.totals_u(cp);
            unsigned run = above;
            int j = 15;
            for (; j > 0; --j) {                                    // the bucket in which the count reaches k
                if (run + S.all_u[j] >= (unsigned)k) break;
                run += S.all_u[j];
            }
            above = run;
            prefix |= (unsigned)j << shift;
            if (above + S.all_u[j] <= LIST_CAP) {                   // few enough: everything at or above this bucket
                for_part(row, first, count, vec, [&](float v, int i) {
                    if (f2ord(v) >= prefix) R.list_push(v, i);
                });
                listed = true;
            }
        }
        if (!listed) { logit_thr = ord2f(prefix); k_done = true; }
    }

    if (!listed && use_p) {
        float local = 0.f;
        for_part(row, first, count, vec, [&](float v, int) {
            if (v >= logit_thr) local += expf(v * inv_t - zmax);
        });
        total = R.sum(local);
        const float need = pp * total;
        unsigned prefix = 0u, above_c = 0u;
        float above_m = 0.f;
        for (int shift = 28; shift >= 0 && !listed; shift -= 4) {
            unsigned cp[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
            float m[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) m[j] = 0.f;
            for_part(row, first, count, vec, [&](float v, int) {
                const float ex = expf(v * inv_t - zmax);
                const unsigned eb = __float_as_uint(ex);
                const bool on = v >= logit_thr && agrees_above(eb, prefix, shift);
                const unsigned b = (eb >> shift) & 15u;
                count_bucket(cp, b, on);
#pragma unroll
                for (int j = 0; j < 16; ++j) m[j] += (on && b == (unsigned)j) ? ex : 0.f;
            });
            R.totals_uf(cp, m);
            float run_m = above_m;
            unsigned run_c = above_c;
            int j = 15;
            for (; j > 0; --j) {                                    // the bucket in which the weight reaches need
                if (run_m + S.all_f[j] >= need) break;
                run_m += S.all_f[j];
                run_c += S.all_u[j];
            }
            above_m = run_m;
            above_c = run_c;
            prefix |= (unsigned)j << shift;
            if (above_c + S.all_u[j] <= LIST_CAP) {
                for_part(row, first, count, vec, [&](float v, int i) {
                    if (v >= logit_thr && __float_as_uint(expf(v * inv_t - zmax)) >= prefix) R.list_push(v, i);
                });
                listed = true;
            }
        }
        if (!listed) e_thr = __uint_as_float(prefix);
    }

    if (listed) {
        R.sync();                                                   // the list is complete
        if (rank != 0) return;
        // ---- the candidates, one per thread: into index order first (the order of the cumulative sum)
        const int n = min(S.n_list, LIST_CAP);
        float v = -INFINITY;
        int idx = 0x7fffffff;
        if (tid < n) {
            v = S.lv[0][tid];
            idx = S.li[0][tid];
            int r = 0;
            for (int j = 0; j < n; ++j) r += S.li[0][j] < idx;
            S.lv[1][r] = v;
            S.li[1][r] = idx;
        }
        __syncthreads();
        if (tid < n) { v = S.lv[1][tid]; idx = S.li[1][tid]; }
        if (!k_done) {                                              // the k-th largest among them
            int cnt = 0;
            for (int j = 0; j < n; ++j) cnt += S.lv[1][j] >= v;
            logit_thr = block_max((tid < n && cnt >= k) ? v : -INFINITY, S.sv);
        }
        bool kept = tid < n && v >= logit_thr;
        float e = kept ? expf(v * inv_t - zmax) : 0.f;
        S.lv[0][tid] = e;
        __syncthreads();
        if (!k_done || !use_p) total = block_sum(e, S.sv);          // otherwise the whole row's total is known
        if (use_p) {
            const float need = pp * total;
            float mass = 0.f;
            for (int j = 0; j < n; ++j) { const float ej = S.lv[0][j]; mass += ej >= e ? ej : 0.f; }
            e_thr = block_max((kept && mass >= need) ? e : 0.f, S.sv);
            kept = kept && e >= e_thr;
            e = kept ? e : 0.f;
            __syncthreads();
            S.lv[0][tid] = e;
            __syncthreads();
            total = block_sum(e, S.sv);
        }
        const float target = u * total;
        float c = 0.f;
        for (int j = 0; j <= tid && j < n; ++j) c += S.lv[0][j];    // the cumulative weight up to this candidate
        const int hit = block_min_int((kept && c > target) ? tid : 0x7fffffff, S);
        const int last = -block_min_int(kept ? -tid : 1, S);         // rounding may leave the target at the very end
        if (tid == 0) out[row_i] = hit != 0x7fffffff ? S.li[1][hit] : (last >= 0 ? S.li[1][last] : bi);
        return;
    }

    // ---- a large kept set: each thread owns a contiguous segment of its block's part, so that the cumulative
    // sum runs in index order
    const int per = (count + nthr - 1) / nthr;
    const int b = first + min(count, tid * per), e_end = first + min(count, (tid + 1) * per);
    float local = 0.f;
    for (int i = b; i < e_end; ++i) {
        const float v = row[i];
        if (v >= logit_thr) {
            const float ex = expf(v * inv_t - zmax);
            if (ex >= e_thr) local += ex;
        }
    }
    float mine = 0.f, before_me = 0.f;
    total = R.sum(local, &mine, &before_me);
    const float target = u * total;
    R.sync();                                                       // the last exchange: blocks may leave after it
    if (!(before_me + mine > target)) {
        // the token lies in a later block's part, or in an earlier one's, or rounding left the target at the
        // very end: then the first block looks for the last kept token of the row
        if (rank == 0 && !(total > target) && tid == 0) {
            int last = bi;
            for (int i = V - 1; i >= 0; --i) {
                const float v = row[i];
                if (v >= logit_thr && expf(v * inv_t - zmax) >= e_thr) { last = i; break; }
            }
            out[row_i] = last;
        }
        return;
    }
    if (before_me > target) return;                                 // an earlier block's
    S.seg[tid] = local;
    __syncthreads();
    if (tid < 32) {                                                 // sums of 32 segments each, for a two-level walk
        float w = 0.f;
        for (int j = tid * (nthr / 32); j < (tid + 1) * (nthr / 32); ++j) w += S.seg[j];
        S.wseg[tid] = w;
    }
    __syncthreads();
    if (tid == 0) {
        float c = before_me;
        int o = -1, w = 0;
        for (; w < 32; ++w) {
            if (c + S.wseg[w] > target) break;
            c += S.wseg[w];
        }
        if (w < 32) {
            for (int tt = w * (nthr / 32); tt < (w + 1) * (nthr / 32); ++tt) {
                if (c + S.seg[tt] > target) { o = tt; break; }
                c += S.seg[tt];
            }
        }
        S.owner = o;
        S.before = c;
    }
    __syncthreads();
    const int owner = S.owner;
    if (owner < 0) {                                   // rounding inside the block: its last kept token
        if (tid == 0) {
            int last = bi;
            for (int i = first + count - 1; i >= first; --i) {
                const float v = row[i];
                if (v >= logit_thr && expf(v * inv_t - zmax) >= e_thr) { last = i; break; }
            }
            out[row_i] = last;
        }
        return;
    }
    if (tid == owner) {
        float c = S.before;
        int pick = -1, last_kept = -1;
        for (int i = b; i < e_end; ++i) {
            const float v = row[i];
            if (v >= logit_thr) {
                const float ex = expf(v * inv_t - zmax);
                if (ex >= e_thr) {
                    last_kept = i;
                    c += ex;
                    if (c > target) { pick = i; break; }
                }
            }
        }
        out[row_i] = pick >= 0 ? pick : (last_kept >= 0 ? last_kept : bi);
    }
}

// Two stages for wide rows: each block takes one piece of a row, then one block per row takes the best piece.
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int V, int chunk,
                                      float* __restrict__ pv, int* __restrict__ pi) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_wait();
    pdl_trigger();
    const float* row = logits + (size_t)blockIdx.y * V;
    const int b = blockIdx.x * chunk, e = min(V, b + chunk);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    block_argmax(best, bi, sv, si);
    if (threadIdx.x == 0) {
        pv[blockIdx.y * gridDim.x + blockIdx.x] = best;
        pi[blockIdx.y * gridDim.x + blockIdx.x] = bi;
    }
}
__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int n,
                                    int* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_wait();
    pdl_trigger();
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = pv[blockIdx.x * n + i];
        const int idx = pi[blockIdx.x * n + i];
        if (v > best || (v == best && idx < bi)) { best = v; bi = idx; }
    }
    block_argmax(best, bi, sv, si);
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// pieces > 1: pv/pi are scratch of rows * pieces entries each.
extern "C" int rg_argmax(const float* logits, int rows, int V, int* out, float* pv, int* pi, int pieces,
                         void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (pieces <= 1 || pv == nullptr || pi == nullptr) {
        return rg_launch(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, s, 1, logits, V, out);
    }
    const int chunk = (V + pieces - 1) / pieces;
    dim3 grid(pieces, rows);
    int e = rg_launch(argmax_partial_kernel, grid, dim3(256), 0, s, 1, logits, V, chunk, pv, pi);
    if (e) return e;
    return rg_launch(argmax_final_kernel, dim3(rows), dim3(64), 0, s, 1, (const float*)pv, (const int*)pi, pieces, out);
}

extern "C" int rg_sample(const float* logits, int rows, int V, const float* temperature, const int* top_k,
                         const float* top_p, const unsigned long long* seed,
                         const unsigned long long* counter, int* out, void* stream) {
    if (rows <= 0) return 0;
    // a cluster of blocks per row when the row is long enough to share
    if (V >= 16384)
        return rg_launch(sample_kernel<SAMPLE_MAX_CLUSTER>, dim3(rows * SAMPLE_MAX_CLUSTER), dim3(SAMPLE_THREADS), 0,
                         (cudaStream_t)stream, SAMPLE_MAX_CLUSTER, logits, V, temperature, top_k, top_p, seed, counter, out);
    return rg_launch(sample_kernel<1>, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 1, logits, V, temperature,
                     top_k, top_p, seed, counter, out);
}
