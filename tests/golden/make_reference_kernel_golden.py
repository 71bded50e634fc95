#!/usr/bin/env python3
"""Makes ``reference_kernels.json``: outputs of the reference's own CUDA kernels, run on the CPU.

The reference's model code is Rust on the candle crates and cannot be compiled
where this repository is built, so the plain implementation (``tests/plain_llama.py``)
rests on the formulas.  Three of the reference's kernels, though, are plain
scalar CUDA C and compile as host C++ through a small stand-in for
``cuda_runtime.h`` (``__global__`` and friends made empty, ``threadIdx`` /
``blockIdx`` / ``gridDim`` as globals, ``float4``): ``paged_attention_v1`` and
``reshape_and_cache`` (crates/vllm-cuda/src/kernels/paged_attention.cu:19-138)
and ``rotary_embedding_kernel`` (crates/vllm-cuda/src/kernels/rope.cu:11-42).
This script includes those two files unchanged from a checkout of the
reference, runs them over a small seeded case (keys written through
``reshape_and_cache`` into shuffled pages, grouped-query attention over them;
rotation at several positions) and stores inputs and outputs.
``tests/test_golden.py`` holds the plain implementation against them.

    python tests/golden/make_reference_kernel_golden.py --reference <checkout of Atari-Katana/railgun>

What this anchors: the cache layout [block, kv_head, offset, dim] with
slot = block * block_size + offset, kv_head = head / (heads / kv_heads),
softmax(scale q.k) weighted values for a single query, and the rotation of
pairs (i, i + d/2) by a [position][cos | sin] table.  Norms, SwiGLU, llama3
frequency scaling, causal masking inside a prompt and the whole model are not
in the reference's kernels and stay anchored on the formulas.
"""
import argparse
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

SHIM = r"""
#pragma once
#include <math.h>
#include <stdint.h>
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __restrict__
struct dim3 { int x = 1, y = 1, z = 1; };
struct float4 { float x, y, z, w; };
static inline float4 make_float4(float x, float y, float z, float w) { float4 f; f.x = x; f.y = y; f.z = z; f.w = w; return f; }
extern dim3 threadIdx, blockIdx, gridDim, blockDim;
"""

DRIVER = r"""
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "cuda_runtime.h"
dim3 threadIdx, blockIdx, gridDim, blockDim;
#include "paged_attention.cu"
#include "rope.cu"

static std::vector<float> read_f(FILE* f, size_t n) { std::vector<float> v(n); if (fread(v.data(), 4, n, f) != n) exit(3); return v; }
static std::vector<int> read_i(FILE* f, size_t n) { std::vector<int> v(n); if (fread(v.data(), 4, n, f) != n) exit(3); return v; }

int main(int argc, char** argv) {
    FILE* f = fopen(argv[1], "rb");
    FILE* o = fopen(argv[2], "wb");
    int hdr[10];
    if (fread(hdr, 4, 10, f) != 10) return 2;
    const int T = hdr[0], nh = hdr[1], nkv = hdr[2], d = hdr[3], bs = hdr[4], nb = hdr[5], B = hdr[6], mb = hdr[7],
              n_rope = hdr[8], max_pos = hdr[9];
    auto k = read_f(f, (size_t)T * nkv * d), v = read_f(f, (size_t)T * nkv * d);
    auto slots = read_i(f, T);
    auto q = read_f(f, (size_t)B * nh * d);
    auto bt = read_i(f, (size_t)B * mb), lens = read_i(f, B);
    auto rope_x = read_f(f, (size_t)n_rope * nh * d);
    auto table = read_f(f, (size_t)max_pos * d);
    auto rope_pos = read_i(f, n_rope);
    float scale; if (fread(&scale, 4, 1, f) != 1) return 2;

    std::vector<float> kc((size_t)nb * nkv * bs * d, 0.f), vc((size_t)nb * nkv * bs * d, 0.f);
    // reshape_and_cache: grid (tokens), block (head_dim, kv_heads) as the kernel reads its indices
    gridDim.x = T;
    for (int t = 0; t < T; ++t) for (int h = 0; h < nkv; ++h) for (int i = 0; i < d; ++i) {
        blockIdx.x = t; threadIdx.y = h; threadIdx.x = i;
        reshape_and_cache(k.data(), v.data(), kc.data(), vc.data(), slots.data(), nkv, d, bs);
    }
    // paged_attention_v1: grid (batch), block (1, heads)
    std::vector<float> out((size_t)B * nh * d, 0.f);
    gridDim.x = B;
    for (int b = 0; b < B; ++b) for (int h = 0; h < nh; ++h) {
        blockIdx.x = b; threadIdx.y = h; threadIdx.x = 0;
        paged_attention_v1(q.data(), kc.data(), vc.data(), bt.data(), lens.data(), out.data(), scale, nh, nkv, d, bs, mb);
    }
    // rotary_embedding_kernel: grid (tokens, heads), block (d / 2)
    for (int t = 0; t < n_rope; ++t) for (int h = 0; h < nh; ++h) for (int i = 0; i < d / 2; ++i) {
        blockIdx.x = t; blockIdx.y = h; threadIdx.x = i;
        rotary_embedding_kernel(rope_x.data(), table.data(), rope_pos.data(), nh, d);
    }
    fwrite(kc.data(), 4, kc.size(), o);
    fwrite(vc.data(), 4, vc.size(), o);
    fwrite(out.data(), 4, out.size(), o);
    fwrite(rope_x.data(), 4, rope_x.size(), o);
    fclose(o);
    return 0;
}
"""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of Atari-Katana/railgun")
    ap.add_argument("--out", default=str(Path(__file__).with_name("reference_kernels.json")))
    args = ap.parse_args()
    kdir = Path(args.reference) / "crates" / "vllm-cuda" / "src" / "kernels"
    rng = np.random.default_rng(20240917)
    nh, nkv, d, bs = 4, 2, 8, 4
    lens = [9, 5]
    B = len(lens)
    nb, mb = 6, 3
    pages = rng.permutation(nb).tolist()
    tables = [pages[:3], pages[3:5] + [0]]
    T = sum(lens)
    k = rng.normal(size=(T, nkv, d)).astype(np.float32)
    v = rng.normal(size=(T, nkv, d)).astype(np.float32)
    slots, row = [], 0
    for b, n in enumerate(lens):
        for p in range(n):
            slots.append(tables[b][p // bs] * bs + p % bs)
    q = rng.normal(size=(B, nh, d)).astype(np.float32)
    scale = np.float32(d ** -0.5)
    n_rope, max_pos = 3, 16
    rope_x = rng.normal(size=(n_rope, nh, d)).astype(np.float32)
    rope_pos = [0, 5, 11]
    inv = 1.0 / (10000.0 ** (np.arange(0, d, 2) / d))
    ang = np.arange(max_pos)[:, None] * inv[None, :]
    table = np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)

    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "cuda_runtime.h").write_text(SHIM)
        (tmp / "driver.cpp").write_text(DRIVER)
        exe = tmp / "driver"
        subprocess.run(["g++", "-O1", "-std=c++17", "-I", str(tmp), "-I", str(kdir), "-o", str(exe),
                        str(tmp / "driver.cpp")], check=True)
        with open(tmp / "in.bin", "wb") as f:
            np.array([T, nh, nkv, d, bs, nb, B, mb, n_rope, max_pos], dtype=np.int32).tofile(f)
            k.tofile(f); v.tofile(f)
            np.array(slots, dtype=np.int32).tofile(f)
            q.tofile(f)
            np.array(tables, dtype=np.int32).tofile(f)
            np.array(lens, dtype=np.int32).tofile(f)
            rope_x.tofile(f); table.tofile(f)
            np.array(rope_pos, dtype=np.int32).tofile(f)
            np.array([scale], dtype=np.float32).tofile(f)
        subprocess.run([str(exe), str(tmp / "in.bin"), str(tmp / "out.bin")], check=True)
        raw = np.fromfile(tmp / "out.bin", dtype=np.float32)
    n_cache = nb * nkv * bs * d
    kc, vc = raw[:n_cache], raw[n_cache:2 * n_cache]
    out = raw[2 * n_cache:2 * n_cache + B * nh * d]
    roped = raw[2 * n_cache + B * nh * d:]
    doc = dict(
        made_by="tests/golden/make_reference_kernel_golden.py",
        kernels=["paged_attention_v1", "reshape_and_cache", "rotary_embedding_kernel"],
        sizes=dict(num_heads=nh, num_kv_heads=nkv, head_dim=d, block_size=bs, num_blocks=nb, max_blocks=mb),
        context_lens=lens, block_tables=tables, slot_mapping=slots, scale=float(scale),
        k=k.reshape(-1).tolist(), v=v.reshape(-1).tolist(), q=q.reshape(-1).tolist(),
        k_cache=kc.tolist(), v_cache=vc.tolist(), attention_out=out.tolist(),
        rope_theta=10000.0, rope_positions=rope_pos, rope_in=rope_x.reshape(-1).tolist(), rope_out=roped.tolist())
    Path(args.out).write_text(json.dumps(doc))
    print(f"wrote {args.out}: {len(json.dumps(doc))} bytes")


if __name__ == "__main__":
    sys.exit(main())
