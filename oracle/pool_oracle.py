"""CPU oracle of sub-bucket construction, feature pooling and additive unpooling (forward and backward).
TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg; never by the
product path.

Parity status: the reduce / unpool arithmetic is pinned by the expectations the reference's own tests compute
(tests/test_subbuck_reduce.py:46-410, tests/test_subbuck_bwd.py:49-429, tests/test_unpooling.py:46-246: a torch
recompute through unpool_ind), which `pool_reduce*` and `unpool_add*` restate.  The sub-bucket partition is
PARITY UNPINNED beyond invariants: the reference's partition depends on a random rotation, a thread-0-only
bounding box and atomic arrival order (src/psh/batch_psh_subbuck_reduce.cuh:193-200,217-238), so its tests
(tests/test_subbuck_reduce.py:413-632) check invariants only; `subbuck_invariants` restates those.

Restated from the reference:
  local_subbuck_ker          src/psh/batch_psh_subbuck_reduce.cuh:104-298
  reduce_feat_ker            src/psh/batch_psh_subbuck_reduce.cuh:300-359
  reduce_feat_backward_ker   src/psh/batch_psh_subbuck_reduce_bwd.cuh:38-126
  additive_unpool_{fwd,bwd}  src/psh/additive_unpool.cuh:42-136
  calc_red_sep_sizes         flash3dxfmr/psh/subbuck.py:40-53
"""
from __future__ import annotations

import numpy as np

from . import psh_oracle as po

BLOCK = 1024
BINS = 8192
F32 = np.float32


def calc_red_sep_sizes(seps, S: int):
    """Rows each scene gets after pooling.  For S dividing 1024 this equals the reference's ceil(n/S)
    (flash3dxfmr/psh/subbuck.py:40-53); otherwise every full 1024-point block contributes ceil(1024/S) rows, which
    is what the per-block construction actually needs."""
    seps = np.asarray(seps, dtype=np.int64)
    sizes = np.diff(np.concatenate([[0], seps]))
    per_block = -(-BLOCK // S)
    red = (sizes // BLOCK) * per_block + -(-(sizes % BLOCK) // S)
    return int(red.sum()), red, np.cumsum(red)


def subbuck_build(coord_f16: np.ndarray, seps, S: int, num_vox: int = 0xFFFF, hash_type: int = 1, fill=None,
                  red_rows_aligned=None):
    """Deterministic sub-bucket partition: per 1024-point block, key = 16-bit hash of the block-normalised voxel
    divided by 8 (13 bits), points ordered by (key, index), runs of S points share a reduced row; block k of a
    scene starts at row k*ceil(1024/S).  Returns subbuck_id, subbuck_off, unpool_ind, reduced_coord, red_sep."""
    seps = np.asarray(seps, dtype=np.int64)
    n_total = coord_f16.shape[0]
    red_len, _, red_sep = calc_red_sep_sizes(seps, S)
    rows_al = red_len if red_rows_aligned is None else red_rows_aligned
    fill = n_total + 3 if fill is None else fill
    sid = np.zeros(n_total, dtype=np.uint32)
    soff = np.zeros(n_total, dtype=np.uint16)
    unpool = np.full((red_len, S), fill, dtype=np.uint32)
    rcoord = np.zeros((rows_al, 3), dtype=np.float16)
    per_block = -(-BLOCK // S)
    start = 0
    for s in range(seps.shape[0]):
        end = int(min(seps[s], n_total))
        red_start = int(red_sep[s - 1]) if s else 0
        for k, b0 in enumerate(range(start, end, BLOCK)):
            b1 = min(b0 + BLOCK, end)
            c = coord_f16[b0:b1]
            vox = po.vox_coords(c, c.min(0), c.max(0), num_vox)
            if hash_type == po.H_ZORDER_DIV:
                key = po.zorder16(vox[:, 0], vox[:, 1], vox[:, 2]) // 8
            elif hash_type == po.H_XORSUM_DIV:
                key = ((vox[:, 0] ^ vox[:, 1] ^ vox[:, 2]) & 0xFFFF) // 8
            elif hash_type == po.H_ZORDER_MOD:
                key = po.zorder16(vox[:, 0], vox[:, 1], vox[:, 2]) % BINS
            else:
                key = ((vox[:, 0] ^ vox[:, 1] ^ vox[:, 2]) & 0xFFFF) % BINS
            order = np.argsort(key, kind="stable")
            pt_ind = np.empty(b1 - b0, dtype=np.int64)
            pt_ind[order] = np.arange(b1 - b0)
            local_row = k * per_block + pt_ind // S
            off = pt_ind % S
            sid[b0:b1] = local_row
            soff[b0:b1] = off
            rows = red_start + local_row
            unpool[rows, off] = np.arange(b0, b1)
            cs = c[order].astype(F32)
            nrow = -(-(b1 - b0) // S)
            pad = np.zeros((nrow * S, 3), dtype=F32)
            pad[: b1 - b0] = cs
            members = np.minimum(S, (b1 - b0) - np.arange(nrow) * S)
            acc = pad[0::S].copy()
            for j in range(1, S):          # sequential fp32 adds in sub-bucket order
                acc = np.where((members > j)[:, None], acc + pad[j::S], acc)
            r0 = red_start + k * per_block
            rcoord[r0:r0 + nrow] = (acc / members[:, None].astype(F32)).astype(np.float16)
        start = max(start, end)
    return sid, soff, unpool, rcoord, red_sep


def subbuck_invariants(sid, soff, unpool, rcoord, coord_f16, seps, S: int) -> None:
    """tests/test_subbuck_reduce.py:413-632: ids per scene are exactly 0..rows-1, offsets are dense 0..c-1 inside
    every sub-bucket, unpool_ind[row, off] is the point's global row, and reduced_coord is the member mean."""
    seps = np.asarray(seps, dtype=np.int64)
    _, red, red_sep = calc_red_sep_sizes(seps, S)
    n = coord_f16.shape[0]
    start = 0
    for s in range(seps.shape[0]):
        end = int(seps[s])
        ids = sid[start:end].astype(np.int64)
        if end > start:
            uniq = np.unique(ids)
            assert uniq.size == red[s] and uniq[0] == 0 and uniq[-1] == red[s] - 1
            rs = int(red_sep[s - 1]) if s else 0
            assert np.array_equal(unpool[rs + ids, soff[start:end]], np.arange(start, end))
            cnt = np.bincount(ids, minlength=int(red[s]))
            assert cnt.max() <= S and cnt.min() >= 1
            key = ids * S + soff[start:end]
            assert np.unique(key).size == key.size
            assert np.all(soff[start:end] < cnt[ids])
        start = end
    valid = unpool < n
    safe = np.where(valid, unpool, 0)
    mean = (coord_f16.astype(F32)[safe] * valid[..., None]).sum(1) / np.maximum(valid.sum(1), 1)[:, None]
    assert np.allclose(rcoord[: unpool.shape[0]].astype(F32), mean, atol=0.2)


# ---------------------------------------------------------------------------------------------- feature ops
def _round(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round fp32 to the feature dtype and back (bf16: round-to-nearest-even on the upper 16 bits)."""
    if dtype == "fp32":
        return x.astype(F32)
    if dtype == "fp16":
        return x.astype(np.float16).astype(F32)
    u = x.astype(F32).view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = r.astype(np.uint32).view(F32)
    return np.where(nan, np.float32(np.nan), out)


def pool_reduce(feat: np.ndarray, unpool: np.ndarray, n_valid: int, op: int, out_rows: int, dtype: str) -> np.ndarray:
    """reduce_feat_ker: fp32 accumulation in slot order; mean divides by the member count; empty rows are 0."""
    rows, S = unpool.shape
    C = feat.shape[1]
    out = np.zeros((out_rows, C), dtype=F32)
    init = {0: 0.0, 1: 0.0, 2: np.inf, 3: -np.inf}[op]
    acc = np.full((rows, C), init, dtype=F32)
    cnt = np.zeros(rows, dtype=np.int64)
    for s in range(S):
        idx = unpool[:, s]
        ok = idx < n_valid
        v = feat[np.where(ok, idx, 0)].astype(F32)
        if op in (0, 1):
            acc = np.where(ok[:, None], acc + v, acc)
        elif op == 2:
            acc = np.where(ok[:, None], np.minimum(acc, v), acc)
        else:
            acc = np.where(ok[:, None], np.maximum(acc, v), acc)
        cnt += ok
    if op == 0:
        acc = acc / np.maximum(cnt, 1)[:, None].astype(F32)
    acc = np.where((cnt == 0)[:, None], F32(0), acc)
    out[:rows] = acc
    return _round(out, dtype)


def pool_reduce_bwd(grad_red: np.ndarray, feat: np.ndarray, unpool: np.ndarray, n_valid: int, op: int,
                    dtype: str) -> np.ndarray:
    """reduce_feat_backward_ker into a zero-initialised gradient (flash3dxfmr/layers/pooling.py:102)."""
    rows, S = unpool.shape
    g_in = np.zeros_like(feat, dtype=F32)
    ok = unpool < n_valid
    cnt = ok.sum(1)
    g = grad_red[:rows].astype(F32)
    if op in (0, 1):
        if op == 0:
            g = _round(g / np.maximum(cnt, 1)[:, None].astype(F32), dtype)
        for s in range(S):
            m = ok[:, s]
            g_in[unpool[m, s]] = g[m]
        return g_in
    best = np.full(g.shape, np.inf if op == 2 else -np.inf, dtype=F32)
    win = np.zeros(g.shape, dtype=np.int64)
    for s in range(S):
        m = ok[:, s]
        v = feat[np.where(m, unpool[:, s], 0)].astype(F32)
        w = ((v > best) if op == 3 else (v < best)) & m[:, None]
        best = np.where(w, v, best)
        win = np.where(w, s, win)
    for s in range(S):
        m = ok[:, s]
        g_in[unpool[m, s]] = np.where(win[m] == s, g[m], F32(0))
    return g_in


def unpool_add(res: np.ndarray, down: np.ndarray, unpool: np.ndarray, dtype: str, covered_rows=None) -> np.ndarray:
    """additive_unpool_fwd_ker: up[r] = round(down[i] + res[r]); rows behind covered_rows are zero."""
    up_rows = res.shape[0]
    up = np.zeros_like(res, dtype=F32)
    ok = unpool < up_rows
    for s in range(unpool.shape[1]):
        m = ok[:, s]
        r = unpool[m, s]
        up[r] = _round(down[: unpool.shape[0]][m].astype(F32) + res[r].astype(F32), dtype)
    return up


def unpool_add_bwd(grad_up: np.ndarray, unpool: np.ndarray, down_rows: int, dtype: str):
    """additive_unpool_bwd_ker into zero-initialised outputs (flash3dxfmr/psh/subbuck.py:128-130)."""
    up_rows, C = grad_up.shape
    g_res = np.zeros((up_rows, C), dtype=F32)
    acc = np.zeros((unpool.shape[0], C), dtype=F32)
    ok = unpool < up_rows
    for s in range(unpool.shape[1]):
        m = ok[:, s]
        r = unpool[m, s]
        g_res[r] = grad_up[r].astype(F32)
        acc[m] = acc[m] + grad_up[r].astype(F32)
    g_down = np.zeros((down_rows, C), dtype=F32)
    g_down[: unpool.shape[0]] = _round(acc, dtype)
    return g_res, g_down
