"""CPU tests of the pooling oracle: the reference's sub-bucket invariants (tests/test_subbuck_reduce.py:413-632)
and its reduce / unpool expectations restated with plain loops."""
import numpy as np
import pytest

from oracle import pool_oracle as pl
from flash3dtransformer_b200 import synthetic


def _scene(sizes, seed=0):
    c32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=seed)
    return c32.astype(np.float16), seps


@pytest.mark.parametrize("S", [2, 3, 4])
def test_subbuck_invariants(S):
    c, seps = _scene([3000, 1, 1025, 2048, 777], seed=1)
    sid, soff, unpool, rcoord, red_sep = pl.subbuck_build(c, seps, S)
    pl.subbuck_invariants(sid, soff, unpool, rcoord, c, seps, S)
    if S == 2:   # equals the reference's ceil(n/S) sizing (flash3dxfmr/psh/subbuck.py:40-53)
        sizes = np.diff(np.concatenate([[0], seps]))
        assert np.array_equal(np.diff(np.concatenate([[0], red_sep])), -(-sizes // 2))


@pytest.mark.parametrize("op", [0, 1, 2, 3])
def test_reduce_and_backward_against_loops(op):
    rng = np.random.default_rng(op)
    c, seps = _scene([700, 300], seed=2)
    S = 3
    _, _, unpool, _, _ = pl.subbuck_build(c, seps, S)
    n = c.shape[0]
    feat = pl._round(rng.normal(size=(n, 8)).astype(np.float32), "bf16")
    out = pl.pool_reduce(feat, unpool, n, op, unpool.shape[0] + 5, "fp32")
    g = rng.normal(size=(unpool.shape[0], 8)).astype(np.float32)
    gin = pl.pool_reduce_bwd(g, feat, unpool, n, op, "fp32")
    exp_gin = np.zeros_like(feat)
    for i in range(unpool.shape[0]):
        rows = [int(r) for r in unpool[i] if r < n]
        m = feat[rows]
        exp = {0: m.mean(0), 1: m.sum(0), 2: m.min(0), 3: m.max(0)}[op]
        assert np.allclose(out[i], exp, rtol=1e-6, atol=1e-6)
        if op == 1:
            exp_gin[rows] = g[i]
        elif op == 0:
            exp_gin[rows] = g[i] / len(rows)
        else:
            w = m.argmax(0) if op == 3 else m.argmin(0)
            for ch in range(8):
                exp_gin[rows[w[ch]], ch] = g[i, ch]
    assert np.all(out[unpool.shape[0]:] == 0)
    assert np.allclose(gin, exp_gin, rtol=1e-6, atol=1e-7)


def test_unpool_roundtrip_and_linearity():
    rng = np.random.default_rng(5)
    c, seps = _scene([1500], seed=3)
    _, _, unpool, _, _ = pl.subbuck_build(c, seps, 2)
    n = c.shape[0]
    res = rng.normal(size=(n + 36, 4)).astype(np.float32)
    down = rng.normal(size=(unpool.shape[0], 4)).astype(np.float32)
    up = pl.unpool_add(res, down, unpool, "fp32")
    for i in range(unpool.shape[0]):
        for r in unpool[i]:
            if r < res.shape[0]:
                assert np.allclose(up[r], res[r] + down[i])
    assert np.all(up[n:] == 0)
    g = rng.normal(size=res.shape).astype(np.float32)
    g_res, g_down = pl.unpool_add_bwd(g, unpool, unpool.shape[0], "fp32")
    assert np.array_equal(g_res[:n], g[:n]) and np.all(g_res[n:] == 0)
    # <up, g> is linear in down with gradient g_down
    assert np.isclose((pl.unpool_add(0 * res, down, unpool, "fp32") * g).sum(), (down * g_down).sum(), rtol=1e-4)
