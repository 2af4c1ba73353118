"""CPU oracle of the PSH bucketing + scatter path.  TEST INFRASTRUCTURE ONLY: nothing in the product path may
import this module; it is the checker that tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg
compare the CUDA kernels against.

Parity status: PARITY UNPINNED for the hash values themselves.  The reference's tests for this path hold no
numeric golden vectors (tests/test_psh.py:117-129 checks "no NaN", "cumsum(counter) == cumsum buffer" and the
scoreboard only, on KITTI scans that are not available), and the reference cannot be compiled here (its
ThunderKittens submodule is empty).  What pins this oracle: (1) the Philox4x32-10 known-answer vectors of the
published algorithm, (2) the reference's own invariants, restated in `scoreboard_check`, (3) the probe table
and num_buck arithmetic, checked against the reference's pure-Python helpers (tests/golden/).

Restated from the reference (file:line within the reference project):
  vox_coord                src/psh/hash_fns.cuh:23-33
  space_out_bit_3d, h1_zorder_{div,mod}_3d   src/psh/hash_fns.cuh:79-86,113-135
  h1_xorsum_{div,mod}      src/psh/hash_fns.cuh:48-68
  perturb_vox              src/common/rand.cuh:95-115 (draws: Philox-seeded linear congruential streams, see psh_scene)
  first hash + in-bucket offsets   src/psh/batch_psh_bucket.cuh:42-139, src/psh/two_stage_counter.cuh:23-143
  overflow rebalance       src/psh/batch_psh_bucket.cuh:157-246
  recycle redistribution   src/psh/batch_psh_bucket.cuh:259-382
  cumsum + scatter + pad   src/psh/batch_psh_bucket.cuh:493-614
  scoreboard               src/psh/bucket_sanitizer_cpu.cpp:92-176
  host parameters          flash3dxfmr/psh/psh_main.py:97-123, flash3dxfmr/psh/bucket.py:19-40

Where the reference is race- or RNG-defined the oracle fixes one deterministic outcome (see `psh_scatter`).
"""
from __future__ import annotations

import math
import numpy as np

H_ZORDER_DIV, H_XORSUM_DIV, H_ZORDER_MOD, H_XORSUM_MOD = 1, 2, 3, 4
NUM_PROBES = 128
RECYCLE = 0
PENDING = 0xFFFFFFFF
U32 = np.uint32
F32 = np.float32


# ----------------------------------------------------------------------------------------------- host params
def round_next_two_power(v: int) -> int:
    """flash3dxfmr/psh/arithmatic.py:12-20"""
    v -= 1
    for s in (1, 2, 4, 8, 16):
        v |= v >> s
    return v + 1


def probe_table() -> np.ndarray:
    """The 124 offsets of {-2..2}^3 without the origin plus four (+-3) corners, in generation order
    (flash3dxfmr/psh/bucket.py:19-33).  The reference shuffles this list with Python's global RNG on every call
    (bucket.py:35); the fixed order is the deterministic choice of this build."""
    rows = []
    for i in (-2, -1, 0, 1, 2):
        for j in (-2, -1, 0, 1, 2):
            for k in (-2, -1, 0, 1, 2):
                if (i, j, k) != (0, 0, 0):
                    rows.append((i, j, k))
    rows += [(3, 3, 3), (3, -3, 3), (-3, 3, -3), (-3, -3, -3)]
    return np.asarray(rows, dtype=np.int16)


def psh_params(sizes, bucket_size: int, num_vox: int = 0xFFFF):
    """num_buck and divisor heuristics of flash3dxfmr/psh/psh_main.py:100-104 (num_buck clamped to >= 1 so
    that scenes smaller than one bucket do not divide by zero)."""
    mean_n = float(np.mean(np.asarray(sizes, dtype=np.float32)))
    nb = max(1, round_next_two_power(int(mean_n / bucket_size)))
    div = int(math.ceil(num_vox / nb))
    return nb, div


# ------------------------------------------------------------------------------------------------- arithmetic
def vox_coords(coord_f16: np.ndarray, bbox_min_f16, bbox_max_f16, num_vox: int) -> np.ndarray:
    """src/psh/hash_fns.cuh:23-33 in IEEE fp32: floor((c - min) * num_vox / (max - min)) clamped to
    [0, num_vox-1] by max(0, min(x, num_vox-1)) (src/common/arithmetic.cuh:26-29).  Device min / max drop a NaN
    operand, so the 0/0 of an axis on which every point has the same coordinate becomes num_vox-1 (np.fmin / np.fmax
    have the same rule; oracle/_ref holds the reference's own lines compiled for the host, which agree)."""
    c = coord_f16.astype(F32)
    lo = np.asarray(bbox_min_f16, dtype=np.float16).astype(F32)
    hi = np.asarray(bbox_max_f16, dtype=np.float16).astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        t = ((c - lo[None, :]) * F32(num_vox)) / (hi - lo)[None, :]
        v = np.fmax(F32(0), np.fmin(np.floor(t), F32(num_vox - 1)))
    return v.astype(np.uint32)


def morton48(vx, vy, vz) -> np.ndarray:
    """48-bit Morton code, x in bit 3i, y in 3i+1, z in 3i+2 (src/psh/hash_fns.cuh:79-86,116-119)."""
    vx = vx.astype(np.uint64); vy = vy.astype(np.uint64); vz = vz.astype(np.uint64)
    code = np.zeros_like(vx)
    for i in range(16):
        code |= ((vx >> np.uint64(i)) & np.uint64(1)) << np.uint64(3 * i)
        code |= ((vy >> np.uint64(i)) & np.uint64(1)) << np.uint64(3 * i + 1)
        code |= ((vz >> np.uint64(i)) & np.uint64(1)) << np.uint64(3 * i + 2)
    return code


def zorder16(vx, vy, vz) -> np.ndarray:
    """(morton >> 31) stored into a 16-bit register (src/psh/hash_fns.cuh:120)."""
    return ((morton48(vx, vy, vz) >> np.uint64(31)) & np.uint64(0xFFFF)).astype(np.uint32)


def first_hash(hash_type: int, vox: np.ndarray, divisor: int, num_bucket: int) -> np.ndarray:
    vx, vy, vz = vox[:, 0], vox[:, 1], vox[:, 2]
    if hash_type == H_ZORDER_DIV:
        h = zorder16(vx, vy, vz) // U32(divisor)
    elif hash_type == H_XORSUM_DIV:
        h = ((vx ^ vy ^ vz) & U32(0xFFFF)) // U32(divisor)
    elif hash_type == H_ZORDER_MOD:
        h = zorder16(vx, vy, vz) % U32(num_bucket)
    elif hash_type == H_XORSUM_MOD:
        h = ((vx ^ vy ^ vz) & U32(0xFFFF)) % U32(num_bucket)
    else:
        raise ValueError(f"hash_type={hash_type} is unsupported")
    return np.minimum(h, U32(num_bucket - 1)).astype(np.uint32)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11)."""
    c0 = np.asarray(c0, dtype=np.uint64); c1 = np.asarray(c1, dtype=np.uint64)
    c2 = np.asarray(c2, dtype=np.uint64); c3 = np.asarray(c3, dtype=np.uint64)
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    m32 = np.uint64(0xFFFFFFFF)
    k0 = np.uint64(k0 & 0xFFFFFFFF); k1 = np.uint64(k1 & 0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & m32
        hi1, lo1 = p1 >> np.uint64(32), p1 & m32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & m32, lo1, (hi0 ^ c3 ^ k1) & m32, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & m32
        k1 = (k1 + np.uint64(0xBB67AE85)) & m32
    return [x.astype(np.uint32) for x in (c0, c1, c2, c3)]


def psh_rand(seed: int, scene, point, tag):
    """Counter layout of the kernels: counter = (point-in-scene, scene, tag, 0), key = seed (lo, hi)."""
    return philox4x32_10(point, scene, tag, 0, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)


def perturb_vox(r, num_vox: int, divisor: int, probe_row: np.ndarray, vox: np.ndarray) -> np.ndarray:
    """src/common/rand.cuh:95-115 with four 32-bit draws per probe.  probe_row is [M,3] (one row per point) and vox
    is [M,3].  segment = floor(U(2.56,5.12) * (fp32(num_vox) / fp32(divisor)) + 0.5); jitter = mulhi(draw, span) - half."""
    ratio = F32(num_vox) / F32(divisor)
    u = (r[0] >> U32(8)).astype(F32) * F32(1.0 / 16777216.0)
    scaling = F32(2.56) + u * F32(2.56)
    seg = np.floor(scaling * ratio + F32(0.5)).astype(np.int64)
    half = seg // 2
    span = (2 * half + 1)
    out = np.empty_like(vox)
    for d in range(3):
        jitter = ((r[1 + d].astype(np.uint64) * span.astype(np.uint64)) >> np.uint64(32)).astype(np.int64) - half
        shifted = vox[:, d].astype(np.int64) + probe_row[:, d].astype(np.int64) * seg + jitter
        out[:, d] = (np.abs(shifted) % num_vox).astype(np.uint32)
    return out


def stable_rank(keys: np.ndarray, num_keys: int):
    """rank[i] = number of j < i with keys[j] == keys[i]; counts[k] = occurrences of k."""
    order = np.argsort(keys, kind="stable")
    counts = np.bincount(keys, minlength=num_keys).astype(np.int64)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    rank = np.empty(keys.shape[0], dtype=np.int64)
    rank[order] = np.arange(keys.shape[0], dtype=np.int64) - starts[keys[order]]
    return rank, counts


# --------------------------------------------------------------------------------------------------- the path
def psh_scene(coord_f16, bbox_min, bbox_max, probe, scene: int, num_bucket: int, divisor: int, cap: int,
              num_vox: int, hash_type: int, seed: int):
    """Bucket ids and offsets of one scene.  Three deterministic rounds:

    A  stable rank (by input index) inside the first-hash bucket; a point keeps its slot when the bucket is the
       recycle bucket 0 or rank < cap (batch_psh_bucket.cuh:124-166).
    B  each remaining point makes one attempt (batch_psh_bucket.cuh:184-236 commits only after the last probe):
       first probe, in table order, whose perturbed hash is neither the own bucket nor bucket 0 and whose bucket
       had kept < cap; attempts are accepted in input order while capacity lasts; the rest go to bucket 0 after
       its own points, ordered by (attempted bucket, index), points without a probe last (:242-246).
    C  bucket-0 points at offset >= cap move to a perturbed-hash bucket chosen with one random probe, or to a
       random non-zero bucket when that hashes to 0, without capacity check (:259-382); arrivals are ranked by
       input index behind the bucket's round-B content.
    """
    n = coord_f16.shape[0]
    nb = num_bucket
    vox = vox_coords(coord_f16, bbox_min, bbox_max, num_vox)
    b0 = first_hash(hash_type, vox, divisor, nb).astype(np.int64)
    rank_a, count0 = stable_rank(b0, nb)
    kept = np.where(np.arange(nb) == RECYCLE, count0, np.minimum(count0, cap))
    bid = b0.copy()
    off = rank_a.copy()
    over = (b0 != RECYCLE) & (rank_a >= cap)
    cnt_b = kept.copy()
    idx_over = np.nonzero(over)[0]
    if idx_over.size:
        target = np.full(idx_over.size, nb, dtype=np.int64)          # nb = "no admissible probe"
        todo = np.arange(idx_over.size)
        # one Philox call (tag 200) seeds four linear congruential streams per point; every probe advances them once
        state = [w.astype(np.uint64) for w in psh_rand(seed, scene, idx_over, 200)]
        for p in range(NUM_PROBES):
            state = [(w * np.uint64(1664525) + np.uint64(1013904223)) & np.uint64(0xFFFFFFFF) for w in state]
            if todo.size == 0:
                break
            pts = idx_over[todo]
            r = [((w[todo] ^ (w[todo] >> np.uint64(15))) & np.uint64(0xFFFFFFFF)).astype(np.uint32) for w in state]
            nv = perturb_vox(r, num_vox, divisor, np.broadcast_to(probe[p], (pts.size, 3)), vox[pts])
            c = first_hash(hash_type, nv, divisor, nb).astype(np.int64)
            ok = (c != b0[pts]) & (c != RECYCLE) & (kept[c] < cap)
            target[todo[ok]] = c[ok]
            todo = todo[~ok]
        q, attempts = stable_rank(target, nb + 1)
        free = np.zeros(nb + 1, dtype=np.int64)
        free[1:nb] = np.maximum(cap - kept[1:nb], 0)
        acc = np.minimum(attempts, free)
        rej = attempts - acc
        rejpre = np.concatenate([[0], np.cumsum(rej)[:-1]])
        accepted = q < free[target]
        ia = idx_over[accepted]
        bid[ia] = target[accepted]
        off[ia] = kept[target[accepted]] + q[accepted]
        ir = idx_over[~accepted]
        tr = target[~accepted]
        bid[ir] = RECYCLE
        off[ir] = count0[RECYCLE] + rejpre[tr] + (q[~accepted] - free[tr])
        cnt_b[1:nb] = kept[1:nb] + acc[1:nb]
        cnt_b[RECYCLE] = count0[RECYCLE] + rej.sum()
    final = cnt_b.copy()
    if nb > 1:
        movers = np.nonzero((bid == RECYCLE) & (off >= cap))[0]
        if movers.size:
            r = psh_rand(seed, scene, movers, 128)
            p = (r[0] % U32(NUM_PROBES)).astype(np.int64)
            r = psh_rand(seed, scene, movers, 129)
            nv = perturb_vox(r, num_vox, divisor, probe[p], vox[movers])
            c = first_hash(hash_type, nv, divisor, nb).astype(np.int64)
            r = psh_rand(seed, scene, movers, 130)
            c = np.where(c == RECYCLE, 1 + (r[0].astype(np.int64) % (nb - 1)), c)
            qc, mv = stable_rank(c, nb)
            bid[movers] = c
            off[movers] = cnt_b[c] + qc
            final = cnt_b + mv
            final[RECYCLE] = min(cnt_b[RECYCLE], cap)
    return bid, off, final


def psh_scatter(coord_f16: np.ndarray, seps, num_bucket: int, divisor: int, cap: int, num_vox: int,
                bbox_min, bbox_max, probe: np.ndarray, pad_to: int, pad_num: float, hash_type: int,
                seed: int = 3407, scene_base: int = 0):
    """Whole operator (scene_base: global index of the first scene, for scene-sharded runs): returns dict(bucket_id u16 [N], bucket_offs u32 [N], bucket_cntr u32 [B,NB],
    bucket_cumsum u32 [B,NB], scattered_coord f16 [pad_to,3]) as batch_psh_scatter_pad_hash fills them
    (src/psh/batch_psh_bucket_dispatcher.cu:221-326)."""
    seps = np.asarray(seps, dtype=np.int64)
    n_total = coord_f16.shape[0]
    if pad_to < n_total:
        raise ValueError("Output coord buffer length is smaller than the input length")
    if num_vox // divisor > num_bucket:
        raise ValueError("bucket divisor too small")
    bsz = seps.shape[0]
    bucket_id = np.zeros(n_total, dtype=np.uint16)
    bucket_offs = np.zeros(n_total, dtype=np.uint32)
    cntr = np.zeros((bsz, num_bucket), dtype=np.uint32)
    scattered = np.full((pad_to, 3), np.float16(pad_num), dtype=np.float16)
    start = 0
    for s in range(bsz):
        end = int(min(seps[s], n_total))
        if end > start:
            bid, off, final = psh_scene(coord_f16[start:end], bbox_min, bbox_max, probe, s + scene_base, num_bucket, divisor,
                                        cap, num_vox, hash_type, seed)
            bucket_id[start:end] = bid
            bucket_offs[start:end] = off
            cntr[s] = final
            excl = np.concatenate([[0], np.cumsum(final)[:-1]])
            dst = start + excl[bid] + off
            scattered[dst] = coord_f16[start:end]
        start = max(start, end)
    cumsum = np.cumsum(cntr.astype(np.int64), axis=1).astype(np.uint32)
    return dict(bucket_id=bucket_id, bucket_offs=bucket_offs, bucket_cntr=cntr, bucket_cumsum=cumsum,
                scattered_coord=scattered)


def scatter_index(bucket_id, bucket_offs, bucket_cumsum, seps, pad_to: int):
    """(out2in [pad_to], in2out [N]): out2in[row in bucket order] = input row with total_N + 3 on the padding rows, as
    batch_psh_cumsum_scatter_feat_index_postpad_ker writes it (src/psh/batch_psh_bucket.cuh:667, 722-735: destination =
    scene start + exclusive cumsum of the scene's bucket counters at the point's bucket + its offset in the bucket);
    in2out is the inverse on the input rows."""
    n = len(bucket_id)
    out2in = np.full(pad_to, n + 3, dtype=np.uint32)
    in2out = np.zeros(n, dtype=np.uint32)
    start = 0
    for s, end in enumerate(int(e) for e in seps):
        if end > start:
            bid = np.asarray(bucket_id[start:end]).astype(np.int64)
            incl = np.asarray(bucket_cumsum[s]).astype(np.int64)
            excl = np.concatenate([[0], incl[:-1]])
            dst = start + excl[bid] + np.asarray(bucket_offs[start:end]).astype(np.int64)
            in2out[start:end] = dst
            out2in[dst] = np.arange(start, end)
        start = max(start, end)
    return out2in, in2out


def gather_rows(src: np.ndarray, index: np.ndarray) -> np.ndarray:
    """out[i] = src[index[i]], zero rows where the index is the padding mark (not a row of src)."""
    out = np.zeros((len(index),) + src.shape[1:], dtype=src.dtype)
    ok = index < len(src)
    out[ok] = src[index[ok]]
    return out


def collate_points(records: np.ndarray, sizes):
    """(coords fp16 [N, 3], extra fp32 [N, dim - 3], seps uint32 [B]) from fp32 point records: the cast, slice and
    cumulative sizes of collate_coords_flat_sep (flash3dxfmr/psh/batching.py:13-28; numpy's float16 cast rounds to
    nearest even like torch's)."""
    records = np.asarray(records, dtype=np.float32)
    with np.errstate(over="ignore"):
        coords = records[:, :3].astype(np.float16)
    return coords, np.ascontiguousarray(records[:, 3:]), np.cumsum(np.asarray(sizes, dtype=np.int64)).astype(np.uint32)


def scoreboard_check(bucket_id, bucket_cntr, bucket_offs, seps, num_bucket: int) -> None:
    """src/psh/bucket_sanitizer_cpu.cpp:92-176: every (bucket, offset) slot below the bucket's counter is hit
    exactly once, no id or offset is out of range, and the residual counters return to zero."""
    seps = np.asarray(seps, dtype=np.int64)
    start = 0
    for s in range(seps.shape[0]):
        end = int(seps[s])
        ids = bucket_id[start:end].astype(np.int64)
        offs = bucket_offs[start:end].astype(np.int64)
        cnt = bucket_cntr[s].astype(np.int64)
        if ids.size:
            if ids.max() >= num_bucket:
                raise AssertionError(f"scene {s}: bucket id {ids.max()} >= num_bucket {num_bucket}")
            if np.any(offs >= cnt[ids]):
                j = int(np.nonzero(offs >= cnt[ids])[0][0])
                raise AssertionError(f"scene {s}: col {start + j} offset {offs[j]} >= counter {cnt[ids[j]]}")
        slot = ids * (int(cnt.max()) if cnt.size else 0) + offs
        if np.unique(slot).size != slot.size:
            raise AssertionError(f"scene {s}: a (bucket, offset) slot is hit more than once")
        if np.any(np.bincount(ids, minlength=num_bucket) != cnt):
            raise AssertionError(f"scene {s}: residual counters are not zero")
        start = end
