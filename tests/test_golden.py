"""Pins the oracles and the host-side mirror on fixtures produced by the reference's own Python code
(tests/golden/make_golden.py lists what each file captures and how it was generated)."""
import json
import os

import numpy as np
import torch

from oracle import attn_oracle as ao
from oracle import pool_oracle as pl
from oracle import psh_oracle as po
from flash3dtransformer_b200.psh import arithmatic, batching, bucket, bucket_scope, subbuck

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_attention_oracle_matches_reference_naive_attention():
    z = np.load(os.path.join(G, "attn_naive.npz"))
    for name in ("a", "b"):
        q, k, v, o = (torch.from_numpy(z[f"{name}_{n}"]) for n in ("q", "k", "v", "o"))
        # [B,T,H,D] -> [B,H,T,D]
        got, _ = ao.naive_attn(*(t.permute(0, 2, 1, 3) for t in (q, k, v)))
        assert torch.allclose(got.permute(0, 2, 1, 3), o, atol=2e-4, rtol=1e-4)
        # and through the bucketed entry point with one all-bucket scope
        t = q.shape[1]
        got2, lse = ao.buck_swin_fwd(q, k, v, torch.tensor([[0, 1]]), t // 2)
        assert torch.allclose(got2, o, atol=2e-4, rtol=1e-4)
        s = torch.einsum("bthd,bshd->bhts", q, k) / q.shape[-1] ** 0.5
        assert torch.allclose(lse, torch.logsumexp(s, -1).permute(0, 2, 1), atol=1e-4)


def test_scope_tables_match_reference():
    ref = json.load(open(os.path.join(G, "scopes.json")))
    for e in ref["plans"]:
        plan = bucket_scope.SwinPlan(e["plan"], e["buck"], e["k"], 0)
        assert plan.scope_list(e["total"]) == e["scopes"]
        t = plan.gen_scopes_from_plan(e["total"], "cpu")
        assert t.dtype == torch.uint32 and t.to(torch.int64).tolist() == e["scopes"]
    for e in ref["swin"]:
        assert bucket_scope.generate_swin_scopes(e["total"], e["buck"], e["k"], e["offset"]) == e["scopes"]
    for e in ref["stride"]:
        assert bucket_scope.generate_stride_scopes(e["total"], e["buck"], e["k"], e["stride"]) == e["scopes"]


def test_scope_gather_matches_reference():
    z = np.load(os.path.join(G, "scope_gather.npz"))
    feat = torch.from_numpy(z["feat"])
    scopes = [[2, 0], [3, 1]]
    g = bucket_scope.construct_bucket_scopes(feat, 8, scopes)
    assert np.array_equal(g.numpy(), z["gathered"])
    assert np.array_equal(bucket_scope.revert_bucket_scopes(g, 8, scopes).numpy(), z["reverted"])
    assert np.array_equal(bucket_scope.reassign_bucket_scopes(g, 8, scopes, [[0, 1], [2, 3]]).numpy(), z["regroup"])
    # the oracle's token gather is the same operation
    idx = ao.scope_tokens(scopes[0], 8)
    assert np.array_equal(feat[:, idx].numpy(), z["gathered"][0])


def test_host_planning_matches_reference():
    ref = json.load(open(os.path.join(G, "host_plan.json")))
    for v, exp in ref["round_next_two_power"].items():
        assert arithmatic.round_next_two_power(int(v)) == exp == po.round_next_two_power(int(v))
    for a, b, exp in ref["cdiv"]:
        assert arithmatic.cdiv(a, b) == exp
    for v, b, exp in ref["round_next_multiply"]:
        assert arithmatic.round_next_multiply(v, b) == exp
    for e in ref["red_sep"]:
        red_len, red_sizes, red_sep = subbuck.calc_red_sep_sizes(torch.tensor(e["seps"], dtype=torch.int32), e["S"])
        assert (red_len, red_sizes.tolist(), red_sep.tolist()) == (e["red_len"], e["red_sizes"], e["red_sep"])
        o_len, o_sizes, o_sep = pl.calc_red_sep_sizes(e["seps"], e["S"])
        assert (o_len, o_sizes.tolist(), o_sep.tolist()) == (e["red_len"], e["red_sizes"], e["red_sep"])
    for e in ref["sep2sizes"]:
        t = torch.tensor(e["seps"], dtype=torch.int32)
        assert batching.sep2sizes(t).tolist() == e["sizes"] and batching.max_inslen_from_seps(t) == e["max"]
    rows = bucket.probe_offset_rows()
    assert sorted(map(tuple, rows)) == [tuple(r) for r in ref["probe_set"]]
    assert list(bucket.generate_probe_offsets("cpu").shape) == ref["probe_shape"]
    assert sorted(map(tuple, po.probe_table().tolist())) == [tuple(r) for r in ref["probe_set"]]
    assert [list(r) for r in rows] == po.probe_table().tolist()
    coords = [torch.arange(12, dtype=torch.float32).reshape(4, 3), torch.ones(2, 3)]
    flat, seps = batching.collate_coords_flat_sep(coords, coord_dtype=torch.float16, sep_dtype=torch.int32)
    assert flat.float().tolist() == ref["collate"]["flat"] and seps.tolist() == ref["collate"]["seps"]
    # num_buck / divisor heuristics of psh_main.py:100-104 on the benchmark configurations
    assert po.psh_params([20000], 256) == (128, 512)
    assert po.psh_params([120000] * 8, 512) == (256, 256)
    assert po.psh_params([200000] * 4, 512) == (512, 128)
