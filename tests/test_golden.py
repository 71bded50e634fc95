"""The plain implementation against the reference's own kernels, run once on
the CPU by ``tests/golden/make_reference_kernel_golden.py`` (stored outputs:
``tests/golden/reference_kernels.json``)."""
import json
from pathlib import Path

import numpy as np

import plain_llama as P

GOLD = json.loads((Path(__file__).parent / "golden" / "reference_kernels.json").read_text())


def test_cache_layout_and_single_query_attention_match_the_reference_kernels():
    s = GOLD["sizes"]
    nh, nkv, d, bs, nb = s["num_heads"], s["num_kv_heads"], s["head_dim"], s["block_size"], s["num_blocks"]
    lens, tables = GOLD["context_lens"], GOLD["block_tables"]
    T = sum(lens)
    k = np.array(GOLD["k"]).reshape(T, nkv, d)
    v = np.array(GOLD["v"]).reshape(T, nkv, d)
    q = np.array(GOLD["q"]).reshape(len(lens), nh, d)
    kc = np.array(GOLD["k_cache"]).reshape(nb, nkv, bs, d)
    vc = np.array(GOLD["v_cache"]).reshape(nb, nkv, bs, d)
    out = np.array(GOLD["attention_out"]).reshape(len(lens), nh, d)
    row = 0
    for b, n in enumerate(lens):
        # slot = block * block_size + offset; cache[block][kv_head][offset][:]
        for p in range(n):
            slot = GOLD["slot_mapping"][row + p]
            assert slot == tables[b][p // bs] * bs + p % bs
            assert np.array_equal(kc[slot // bs, :, slot % bs], k[row + p].astype(np.float32))
            assert np.array_equal(vc[slot // bs, :, slot % bs], v[row + p].astype(np.float32))
        # the last position of a whole sequence attends every key: the reference's decode attention
        # (mask j < context_len) is the last row of the plain causal attention with a zero query before it
        qs = np.zeros((n, nh, d))
        qs[-1] = q[b]
        plain = P.attention(qs, k[row:row + n], v[row:row + n], np.arange(n), scale=GOLD["scale"])[-1]
        assert np.abs(plain - out[b]).max() < 2e-6
        row += n


def test_rotation_matches_the_reference_kernel():
    s = GOLD["sizes"]
    nh, d = s["num_heads"], s["head_dim"]
    pos = GOLD["rope_positions"]
    x = np.array(GOLD["rope_in"]).reshape(len(pos), nh, d)
    want = np.array(GOLD["rope_out"]).reshape(len(pos), nh, d)
    got = P.rope(x, pos, P.rope_inv_freq(d, GOLD["rope_theta"], None))
    assert np.abs(got - want).max() < 2e-6
    assert np.abs(want - x)[1:].max() > 0.1                  # positions > 0 really rotate
