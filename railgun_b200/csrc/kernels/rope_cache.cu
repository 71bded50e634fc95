// Rotary position encoding of Q and K fused with the write of K and V into the
// paged cache.
//
// Rotation (pairs (i, i + d/2), 32-bit):  x'[i] = x[i] c - x[i+d/2] s,
// x'[i+d/2] = x[i+d/2] c + x[i] s, with c, s = table[pos][i], table[pos][d/2+i]
// (crates/vllm-cuda/src/kernels/rope.cu:30-41; the table layout [max_pos, d] =
// cos | sin is that kernel's).  Cache write: token slot = page * page_size +
// offset, cache[page][0|1][kv_head][offset][:] = k | v, slot < 0 skipped
// (crates/vllm-cuda/src/kernels/paged_attention.cu:111-138).  The reference
// never calls its rope kernel; here rotation happens once, before the write,
// so cached keys are rotated by their absolute position.
//
// Row layout `paired8` (head sizes that are multiples of 16): the projection's rows of every q and k head were
// reordered at load so that pair i = (i, i + d/2) sits at storage indices (16 (i / 8) + i % 8, + 8): every 16
// consecutive features hold 8 whole pairs, which lets the decode product rotate in its own epilogue
// (gemm_skinny.cuh).  q.k is unchanged by a reordering that q and k share; the cache then holds k in that order.
#include "common.cuh"

// storage index of the first element of pair i
__device__ __forceinline__ int rope_lo_index(int i, bool paired8) { return paired8 ? ((i >> 3) << 4) + (i & 7) : i; }

// qkv: [T, (nh + 2 nkv) d], q rotated in place.  kv_cache: [NP, 2, nkv, ps, d].
template <typename A>
__global__ void rope_cache_kernel(A* __restrict__ qkv, const float* __restrict__ table,
                                  const int* __restrict__ positions, const int* __restrict__ slots,
                                  A* __restrict__ kv_cache, int nh, int nkv, int d, int page_size,
                                  int max_pos, int* __restrict__ err, int paired8) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = d >> 1;
    const int apart = paired8 ? 8 : half;            // distance between the two elements of a pair
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {          // host-validated; never read outside the table
        if (threadIdx.x == 0 && err) atomicExch(err, 1);
        pos = 0;
    }
    A* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const float* cs = table ? table + (size_t)pos * d : nullptr;
    const int slot = slots ? slots[t] : -1;
    A* kdst = nullptr;
    A* vdst = nullptr;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        kdst = kv_cache + (((size_t)page * 2 + 0) * nkv * page_size + off) * d;
        vdst = kv_cache + (((size_t)page * 2 + 1) * nkv * page_size + off) * d;
    }
    const size_t head_stride = (size_t)page_size * d;   // between kv heads inside a page
    // q heads: rotate in place; k heads: rotate into the cache (and in place)
    const int n_rot = (nh + nkv) * half;
    for (int w = threadIdx.x; w < n_rot; w += blockDim.x) {
        const int h = w / half, i = w - h * half;
        const int e = rope_lo_index(i, paired8);
        A* x = row + (size_t)h * d;
        const float lo = to_f32(x[e]), hi = to_f32(x[e + apart]);
        float nlo = lo, nhi = hi;
        if (cs) {
            const float c = cs[i], s = cs[half + i];
            nlo = lo * c - hi * s;
            nhi = hi * c + lo * s;
        }
        const A olo = from_f32<A>(nlo), ohi = from_f32<A>(nhi);
        x[e] = olo;
        x[e + apart] = ohi;
        if (h >= nh && kdst) {
            A* kd = kdst + (size_t)(h - nh) * head_stride;
            kd[e] = olo;
            kd[e + apart] = ohi;
        }
    }
    if (vdst) {
        const A* v = row + (size_t)(nh + nkv) * d;
        for (int w = threadIdx.x; w < nkv * d; w += blockDim.x) {
            const int h = w / d, i = w - h * d;
            vdst[(size_t)h * head_stride + i] = v[w];
        }
    }
}

// Two neighbouring pairs per thread (4-byte accesses for bfloat16): d % 4 == 0.
template <typename A> struct Pair;
template <> struct Pair<bf16> {
    typedef __nv_bfloat162 T;
    static __device__ __forceinline__ float2 load(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const T*>(p)); }
    static __device__ __forceinline__ void store(bf16* p, float2 v) { *reinterpret_cast<T*>(p) = __floats2bfloat162_rn(v.x, v.y); }
};
template <> struct Pair<float> {
    typedef float2 T;
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};

template <typename A>
__global__ void rope_cache_vec2_kernel(A* __restrict__ qkv, const float* __restrict__ table,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       A* __restrict__ kv_cache, int nh, int nkv, int d, int page_size,
                                       int max_pos, int* __restrict__ err, int paired8) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = d >> 1, hq = half >> 1;          // hq: element pairs per half head
    const int apart = paired8 ? 8 : half;
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0 && err) atomicExch(err, 1);
        pos = 0;
    }
    A* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const float* cs = table ? table + (size_t)pos * d : nullptr;
    const int slot = slots ? slots[t] : -1;
    A* kdst = nullptr;
    A* vdst = nullptr;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        kdst = kv_cache + (((size_t)page * 2 + 0) * nkv * page_size + off) * d;
        vdst = kv_cache + (((size_t)page * 2 + 1) * nkv * page_size + off) * d;
    }
    const size_t head_stride = (size_t)page_size * d;
    const int n_rot = (nh + nkv) * hq;
    for (int w = threadIdx.x; w < n_rot; w += blockDim.x) {
        const int h = w / hq, i = (w - h * hq) * 2;   // pairs i and i + 1: neighbours in storage in both layouts
        const int e = rope_lo_index(i, paired8);
        A* x = row + (size_t)h * d;
        const float2 lo = Pair<A>::load(x + e), hi = Pair<A>::load(x + e + apart);
        float2 nlo = lo, nhi = hi;
        if (cs) {
            const float2 c = *reinterpret_cast<const float2*>(cs + i), s = *reinterpret_cast<const float2*>(cs + half + i);
            nlo = make_float2(lo.x * c.x - hi.x * s.x, lo.y * c.y - hi.y * s.y);
            nhi = make_float2(hi.x * c.x + lo.x * s.x, hi.y * c.y + lo.y * s.y);
        }
        Pair<A>::store(x + e, nlo);
        Pair<A>::store(x + e + apart, nhi);
        if (h >= nh && kdst) {
            A* kd = kdst + (size_t)(h - nh) * head_stride;
            Pair<A>::store(kd + e, nlo);
            Pair<A>::store(kd + e + apart, nhi);
        }
    }
    if (vdst) {
        const A* v = row + (size_t)(nh + nkv) * d;
        const int n_v = nkv * (d >> 1);
        for (int w = threadIdx.x; w < n_v; w += blockDim.x) {
            const int h = (w * 2) / d, i = w * 2 - h * d;
            Pair<A>::store(vdst + (size_t)h * head_stride + i, Pair<A>::load(v + w * 2));
        }
    }
}

// Eight neighbouring pairs per thread, 16-byte accesses: bfloat16 with d % 16 == 0 (both layouts: the first
// elements of pairs 8 b .. 8 b + 7 are 8 consecutive features, and so are their partners).  One thread block per
// token, as above; this is the kernel that long prompts go through.
__global__ void rope_cache_vec8_kernel(bf16* __restrict__ qkv, const float* __restrict__ table,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       bf16* __restrict__ kv_cache, int nh, int nkv, int d, int page_size,
                                       int max_pos, int* __restrict__ err, int paired8) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = d >> 1, groups = half >> 3;       // groups of 8 pairs per head
    const int apart = paired8 ? 8 : half;
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0 && err) atomicExch(err, 1);
        pos = 0;
    }
    bf16* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const float* cs = table ? table + (size_t)pos * d : nullptr;
    const int slot = slots ? slots[t] : -1;
    bf16* kdst = nullptr;
    bf16* vdst = nullptr;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        kdst = kv_cache + (((size_t)page * 2 + 0) * nkv * page_size + off) * d;
        vdst = kv_cache + (((size_t)page * 2 + 1) * nkv * page_size + off) * d;
    }
    const size_t head_stride = (size_t)page_size * d;
    for (int w = threadIdx.x; w < (nh + nkv) * groups; w += blockDim.x) {
        const int h = w / groups, i = (w - h * groups) * 8;          // pairs i .. i + 7
        const int e = rope_lo_index(i, paired8);
        bf16* x = row + (size_t)h * d;
        uint4 lo = *reinterpret_cast<const uint4*>(x + e), hi = *reinterpret_cast<const uint4*>(x + e + apart);
        if (cs) {
            const float4 c0 = *reinterpret_cast<const float4*>(cs + i), c1 = *reinterpret_cast<const float4*>(cs + i + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(cs + half + i), s1 = *reinterpret_cast<const float4*>(cs + half + i + 4);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 a = __bfloat1622float2(l2[k]), b = __bfloat1622float2(h2[k]);
                l2[k] = __floats2bfloat162_rn(a.x * c[2 * k] - b.x * sn[2 * k], a.y * c[2 * k + 1] - b.y * sn[2 * k + 1]);
                h2[k] = __floats2bfloat162_rn(b.x * c[2 * k] + a.x * sn[2 * k], b.y * c[2 * k + 1] + a.y * sn[2 * k + 1]);
            }
            *reinterpret_cast<uint4*>(x + e) = lo;
            *reinterpret_cast<uint4*>(x + e + apart) = hi;
        }
        if (h >= nh && kdst) {
            bf16* kd = kdst + (size_t)(h - nh) * head_stride;
            *reinterpret_cast<uint4*>(kd + e) = lo;
            *reinterpret_cast<uint4*>(kd + e + apart) = hi;
        }
    }
    if (vdst) {
        const bf16* v = row + (size_t)(nh + nkv) * d;
        for (int w = threadIdx.x; w < nkv * (d >> 3); w += blockDim.x) {
            const int h = (w * 8) / d, i = w * 8 - h * d;
            *reinterpret_cast<uint4*>(vdst + (size_t)h * head_stride + i) = *reinterpret_cast<const uint4*>(v + w * 8);
        }
    }
}

// paired8: 0 pairs (i, i + d/2) as stored by the model; 1 the reordered layout above (d % 16 == 0).
extern "C" int rg_rope_cache(void* qkv, int dtype, const float* table, const int* positions,
                             const int* slots, void* kv_cache, int T, int nh, int nkv, int d,
                             int page_size, int max_pos, int* err, int paired8, void* stream) {
    if (T <= 0) return 0;
    if (d % 2 || (paired8 && d % 16)) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    if (dtype == RG_DTYPE_BF16 && d % 16 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)kv_cache % 16 == 0 &&
        (uintptr_t)table % 16 == 0 && ((size_t)(nh + 2 * nkv) * d) % 8 == 0)
        return rg_launch(rope_cache_vec8_kernel, dim3(T), dim3(threads), 0, s, 1, (bf16*)qkv, table, positions, slots,
                         (bf16*)kv_cache, nh, nkv, d, page_size, max_pos, err, paired8);
    if (d % 4 == 0 && (uintptr_t)qkv % 8 == 0 && (uintptr_t)kv_cache % 8 == 0 && (uintptr_t)table % 8 == 0) {
        if (dtype == RG_DTYPE_BF16)
            return rg_launch(rope_cache_vec2_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, (bf16*)qkv, table, positions,
                             slots, (bf16*)kv_cache, nh, nkv, d, page_size, max_pos, err, paired8);
        if (dtype == RG_DTYPE_F32)
            return rg_launch(rope_cache_vec2_kernel<float>, dim3(T), dim3(threads), 0, s, 1, (float*)qkv, table,
                             positions, slots, (float*)kv_cache, nh, nkv, d, page_size, max_pos, err, paired8);
        return RG_ERR_UNSUPPORTED;
    }
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(rope_cache_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, (bf16*)qkv, table, positions, slots,
                         (bf16*)kv_cache, nh, nkv, d, page_size, max_pos, err, paired8);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(rope_cache_kernel<float>, dim3(T), dim3(threads), 0, s, 1, (float*)qkv, table, positions,
                         slots, (float*)kv_cache, nh, nkv, d, page_size, max_pos, err, paired8);
    return RG_ERR_UNSUPPORTED;
}
