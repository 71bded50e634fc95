// Sampling over 32-bit logits, one thread block per row.
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

// Per-row parameters; temperature <= 0 means greedy.
__global__ void sample_kernel(const float* __restrict__ logits, int V,
                              const float* __restrict__ temperature, const int* __restrict__ top_k,
                              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                              const unsigned long long* __restrict__ counter, int* __restrict__ out) {
    __shared__ float sv[33];
    __shared__ int si[32];
    __shared__ float seg[SAMPLE_THREADS];
    pdl_wait();
    pdl_trigger();
    const int row_i = blockIdx.x;
    const float* row = logits + (size_t)row_i * V;
    const float T = temperature[row_i];

    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    block_argmax(best, bi, sv, si);
    if (!(T > 0.f)) {
        if (threadIdx.x == 0) out[row_i] = bi == 0x7fffffff ? 0 : bi;
        return;
    }
    const float inv_t = 1.f / T;
    const float zmax = best * inv_t;

    // top-k: the k-th largest logit by bisection over the ordered bit patterns
    float logit_thr = -INFINITY;
    const int k = top_k ? top_k[row_i] : 0;
    if (k > 0 && k < V) {
        unsigned lo = 0u, hi = 0xffffffffu;          // largest u with count(ord >= u) >= k
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            float cnt = 0.f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += (f2ord(row[i]) >= mid) ? 1.f : 0.f;
            cnt = block_sum(cnt, sv);
            if (cnt >= (float)k) lo = mid; else hi = mid - 1u;
        }
        logit_thr = ord2f(lo);
    }

    // each thread owns a contiguous segment so that the cumulative sum runs in index order
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int b = threadIdx.x * per, e = min(V, b + per);
    float local = 0.f;
    for (int i = b; i < e; ++i) {
        const float v = row[i];
        if (v >= logit_thr) local += expf(v * inv_t - zmax);
    }
    float total = block_sum(local, sv);

    // top-p: largest probability threshold whose kept mass reaches top_p * total
    float e_thr = 0.f;                                 // on exp(z - zmax), in (0, 1]
    const float pp = top_p ? top_p[row_i] : 1.f;
    if (pp < 1.f) {
        const float need = pp * total;
        unsigned lo = 0u, hi = __float_as_uint(1.0f);  // non-negative floats order as their bits
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo + 1u) >> 1);
            const float thr = __uint_as_float(mid);
            float mass = 0.f;
            for (int i = b; i < e; ++i) {
                const float v = row[i];
                if (v >= logit_thr) {
                    const float ex = expf(v * inv_t - zmax);
                    if (ex >= thr) mass += ex;
                }
            }
            mass = block_sum(mass, sv);
            if (mass >= need) lo = mid; else hi = mid - 1u;
        }
        e_thr = __uint_as_float(lo);
        local = 0.f;
        for (int i = b; i < e; ++i) {
            const float v = row[i];
            if (v >= logit_thr) {
                const float ex = expf(v * inv_t - zmax);
                if (ex >= e_thr) local += ex;
            }
        }
        total = block_sum(local, sv);
    }

    seg[threadIdx.x] = local;
    __syncthreads();
    const float u = uniform_from_counter(seed[row_i], counter[row_i]);
    const float target = u * total;
    // thread 0 walks the 1024 segment sums, then the owner walks its segment
    __shared__ int owner;
    __shared__ float before;
    if (threadIdx.x == 0) {
        float c = 0.f;
        int o = -1;
        for (int tt = 0; tt < (int)blockDim.x; ++tt) {
            if (c + seg[tt] > target) { o = tt; break; }
            c += seg[tt];
        }
        owner = o;
        before = c;
    }
    __syncthreads();
    if (owner < 0) {                                   // rounding left target at the very end
        if (threadIdx.x == 0) {
            int last = bi;
            for (int i = V - 1; i >= 0; --i) {
                const float v = row[i];
                if (v >= logit_thr && expf(v * inv_t - zmax) >= e_thr) { last = i; break; }
            }
            out[row_i] = last;
        }
        return;
    }
    if ((int)threadIdx.x == owner) {
        float c = before;
        int pick = -1, last_kept = -1;
        for (int i = b; i < e; ++i) {
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
    return rg_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 1, logits, V, temperature,
                     top_k, top_p, seed, counter, out);
}
