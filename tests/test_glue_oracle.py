"""The numpy restatement of the reference's glue ops: properties that pin its conventions
(half-split RoPE pairs, position-major caches, grouped kv heads, first-largest argmax)."""
import numpy as np

from oracle import glue_oracle as GO


def test_rope_pairs_are_j_and_j_plus_half():
    d = 8
    v = np.zeros((1, d), dtype=np.float16)
    v[0, 1] = 1.0                                   # element j = 1 of the first half
    out = GO.rope(v, position=3, base=10000.0).astype(np.float64)
    ang = 3 * 10000.0 ** (-2 / d)
    expect = np.zeros(d)
    expect[1], expect[1 + d // 2] = np.cos(ang), np.sin(ang)
    assert np.allclose(out[0], expect, atol=1e-3)
    # position 0 is the identity, and the rotation keeps each pair's length
    x = np.random.default_rng(0).standard_normal((4, 128)).astype(np.float16)
    assert np.array_equal(GO.rope(x, 0, 5e5), x)
    y = GO.rope(x, 77, 5e5).astype(np.float64)
    xf = x.astype(np.float64)
    assert np.allclose(xf[:, :64] ** 2 + xf[:, 64:] ** 2, y[:, :64] ** 2 + y[:, 64:] ** 2, atol=2e-2)


def test_attention_single_token_and_head_grouping():
    rng = np.random.default_rng(1)
    hq, hkv, d, ctx = 4, 2, 16, 8
    kc = rng.standard_normal((ctx, hkv, d)).astype(np.float16)
    vc = rng.standard_normal((ctx, hkv, d)).astype(np.float16)
    q = rng.standard_normal((hq, d)).astype(np.float16)
    one = GO.attention_single(q, kc, vc, 1, 0.25)
    for h in range(hq):                              # one cached token: the output is its v
        assert np.array_equal(one[h], vc[0, h * hkv // hq])
    # heads 0,1 read kv head 0 and heads 2,3 kv head 1: equal queries give equal outputs
    q[1] = q[0]
    q[3] = q[2]
    out = GO.attention_single(q, kc, vc, ctx, 0.25)
    assert np.array_equal(out[0], out[1]) and np.array_equal(out[2], out[3])
    assert not np.array_equal(out[0], out[2])


def test_cache_append_is_position_major():
    kc = np.zeros((4, 2, 8), dtype=np.float16)
    vc = np.zeros_like(kc)
    k = np.ones((2, 8), dtype=np.float16)
    GO.cache_append(kc, vc, k, 2 * k, 3)
    assert kc[3].sum() == 16 and vc[3].sum() == 32 and kc[:3].sum() == 0


def test_rmsnorm_rounds_the_residual_sum_before_normalizing():
    x = np.full((1, 8), 1.0, dtype=np.float16)
    r = np.full((1, 8), 2.0 ** -11, dtype=np.float16)     # 1 + 2^-11 rounds back to 1 in fp16
    out, res = GO.rmsnorm(x, np.ones(8, dtype=np.float16), 0.0, r)
    assert np.array_equal(res, x)
    assert np.allclose(out.astype(np.float64), 1.0 / (1 + 2.0 ** -11), atol=1e-3)
    plain, none = GO.rmsnorm(3 * x, np.ones(8, dtype=np.float16), 0.0)
    assert none is None and np.array_equal(plain, x)


def test_gated_silu_and_argmax():
    g = np.array([[0.0, 20.0, -20.0, 1.0]], dtype=np.float16)
    u = np.array([[5.0, 2.0, 3.0, 1.0]], dtype=np.float16)
    out = GO.gated_silu(g, u).astype(np.float64)
    assert np.allclose(out, [[0.0, 40.0, 0.0, 1 / (1 + np.exp(-1.0))]], atol=1e-3)
    assert GO.argmax_first(np.array([1.0, 7.0, 7.0, 3.0])) == 1
