"""Generates the golden fixtures in this folder from the reference's own pure-Python code.

Run where the reference checkout is available, giving its path as the first argument or in $F3D_REFERENCE:
    python tests/golden/make_golden.py <path to the reference checkout>
The reference's compiled extension (flash3dxfmr.lib.pshattn), TransformerEngine and flash_attn are not needed:
stub modules stand in for them, and only functions that never touch them are called.  The outputs are small
.npz / .json files that the tests read; nothing at test time reads the reference checkout.

What is captured
  attn_naive.npz    naive_attn_fwd of the reference's tests (tests/test_lib.py:24-38) on seeded inputs
  scopes.json       SwinPlan.gen_scopes_from_plan, generate_*_scopes (flash3dxfmr/psh/bucket_scope.py:58-140)
  scope_gather.npz  construct_bucket_scopes / revert_bucket_scopes (bucket_scope.py:143-181) on an index pattern
  host_plan.json    round_next_two_power, cdiv, round_next_multiply (psh/arithmatic.py), calc_red_sep_sizes
                    (psh/subbuck.py:40-53), sep2sizes / collate (psh/batching.py), the probe-offset set
                    (psh/bucket.py:19-40, order-free because the reference shuffles it)
  call_sites.json   every call `pshattn.<operator>(...)` in the reference's Python package and tests (file, line, number
                    of positional arguments, keyword names), read from the syntax tree: the argument lists the drop-in
                    operator module has to accept
"""
import ast
import glob
import importlib
import json
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("F3D_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "flash3dxfmr")):
    raise SystemExit("usage: make_golden.py <path to the reference checkout> (or set F3D_REFERENCE)")
HERE = os.path.dirname(os.path.abspath(__file__))


def _install_stubs():
    pkg = types.ModuleType("flash3dxfmr")
    pkg.__path__ = [os.path.join(REF, "flash3dxfmr")]
    sys.modules["flash3dxfmr"] = pkg
    lib = types.ModuleType("flash3dxfmr.lib")
    lib.__path__ = []
    psh = types.ModuleType("flash3dxfmr.lib.pshattn")

    class _Mgr:
        @staticmethod
        def instance():
            return _Mgr()

        def init_dev_info(self, *_):
            pass

        def set_sync_stream(self, f):
            return f

        def get_sync_stream(self):
            return False

    psh.DeviceManagerSingleton = _Mgr
    lib.pshattn = psh
    sys.modules["flash3dxfmr.lib"] = lib
    sys.modules["flash3dxfmr.lib.pshattn"] = psh
    fa = types.ModuleType("flash_attn")
    fai = types.ModuleType("flash_attn.flash_attn_interface")
    fai.flash_attn_varlen_qkvpacked_func = None
    sys.modules["flash_attn"] = fa
    sys.modules["flash_attn.flash_attn_interface"] = fai


def main():
    _install_stubs()
    scope = importlib.import_module("flash3dxfmr.psh.bucket_scope")
    arith = importlib.import_module("flash3dxfmr.psh.arithmatic")
    subbuck = importlib.import_module("flash3dxfmr.psh.subbuck")
    batching = importlib.import_module("flash3dxfmr.psh.batching")
    bucket = importlib.import_module("flash3dxfmr.psh.bucket")
    spec = importlib.util.spec_from_file_location("ref_test_lib", os.path.join(REF, "tests", "test_lib.py"))
    test_lib = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(test_lib)

    # ---- naive attention
    torch.manual_seed(2)
    cases = {}
    for name, (b, t, h, d), mul in [("a", (2, 64, 2, 16), 1.0), ("b", (1, 96, 3, 32), 4.0)]:
        q, k, v = (torch.randn(b, t, h, d).bfloat16() * mul for _ in range(3))
        o = test_lib.naive_attn_fwd(q, k, v)
        for n, x in (("q", q), ("k", k), ("v", v)):
            cases[f"{name}_{n}"] = x.float().numpy()
        cases[f"{name}_o"] = o.float().numpy()
    np.savez_compressed(os.path.join(HERE, "attn_naive.npz"), **cases)

    # ---- scopes
    out = {"plans": [], "swin": [], "stride": []}
    for plan in ("swin", "stride"):
        for total, buck, k in [(4096, 512, 8), (8192, 512, 8), (24576, 512, 8), (3072, 512, 2), (1536, 256, 3),
                               (1280, 256, 5), (2048, 128, 4), (512, 512, 1)]:
            p = scope.SwinPlan(plan, buck, k, 0)
            t = p.gen_scopes_from_plan(total, "cpu")
            out["plans"].append({"plan": plan, "total": total, "buck": buck, "k": k,
                                 "scopes": t.to(torch.int64).tolist()})
    for total, buck, k, off in [(4096, 512, 4, 0), (4096, 512, 4, 1), (2048, 256, 2, 3)]:
        out["swin"].append({"total": total, "buck": buck, "k": k, "offset": off,
                            "scopes": scope.generate_swin_scopes(total, buck, k, off)})
    for total, buck, k, stride in [(6144, 512, 2, 1), (6144, 512, 2, 2), (6144, 512, 2, 3)]:
        out["stride"].append({"total": total, "buck": buck, "k": k, "stride": stride,
                              "scopes": scope.generate_stride_scopes(total, buck, k, stride)})
    json.dump(out, open(os.path.join(HERE, "scopes.json"), "w"))

    # ---- scope gather / revert on an index pattern
    feat = torch.arange(2 * 32, dtype=torch.float32).reshape(2, 32)
    scopes = [[2, 0], [3, 1]]
    gathered = scope.construct_bucket_scopes(feat, 8, scopes)
    reverted = scope.revert_bucket_scopes(gathered, 8, scopes)
    regroup = scope.reassign_bucket_scopes(gathered, 8, scopes, [[0, 1], [2, 3]])
    np.savez(os.path.join(HERE, "scope_gather.npz"), feat=feat.numpy(), gathered=gathered.numpy(),
             reverted=reverted.numpy(), regroup=regroup.numpy())

    # ---- host planning arithmetic
    plan = {"round_next_two_power": {str(v): arith.round_next_two_power(v) for v in [1, 2, 3, 78, 234, 256, 390, 1000]},
            "cdiv": [[a, b, arith.cdiv(a, b)] for a, b in [(10, 3), (12, 4), (120000, 512), (1, 7)]],
            "round_next_multiply": [[v, b, arith.round_next_multiply(v, b)] for v, b in [(10, 4), (12, 4), (20000, 256)]],
            "red_sep": [], "sep2sizes": [], "probe_set": None}
    for seps, s in [([7, 20, 21], 2), ([120000, 240001, 360001], 2), ([1024, 4096], 4), ([5, 5, 9], 2)]:
        red_len, red_sizes, red_sep = subbuck.calc_red_sep_sizes(torch.tensor(seps, dtype=torch.int32), s)
        plan["red_sep"].append({"seps": seps, "S": s, "red_len": red_len, "red_sizes": red_sizes.tolist(),
                                "red_sep": red_sep.tolist()})
    for seps in ([7, 20, 21], [100], [3, 3, 10]):
        t = torch.tensor(seps, dtype=torch.int32)
        plan["sep2sizes"].append({"seps": seps, "sizes": batching.sep2sizes(t).tolist(),
                                  "max": batching.max_inslen_from_seps(t)})
    probes = bucket.generate_probe_offsets("cpu")
    plan["probe_set"] = sorted(map(tuple, probes.tolist()))
    plan["probe_shape"] = list(probes.shape)
    coords = [torch.arange(12, dtype=torch.float32).reshape(4, 3), torch.ones(2, 3)]
    flat, seps = batching.collate_coords_flat_sep(coords, coord_dtype=torch.float16, sep_dtype=torch.int32)
    plan["collate"] = {"flat": flat.float().tolist(), "seps": seps.tolist()}
    json.dump(plan, open(os.path.join(HERE, "host_plan.json"), "w"))

    # ---- operator call sites of the reference's host code and tests
    sites = []
    for path in sorted(glob.glob(os.path.join(REF, "flash3dxfmr", "**", "*.py"), recursive=True)
                       + glob.glob(os.path.join(REF, "tests", "*.py"))):
        tree = ast.parse(open(path).read())
        for node in ast.walk(tree):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)):
                continue
            chain, cur = [node.func.attr], node.func.value
            while isinstance(cur, ast.Attribute):
                chain.append(cur.attr)
                cur = cur.value
            if isinstance(cur, ast.Call):          # pshattn.DeviceManagerSingleton.instance().method(...)
                inner = cur.func
                if isinstance(inner, ast.Attribute) and inner.attr == "instance":
                    chain.append("instance()")
                    cur = inner.value
                    while isinstance(cur, ast.Attribute):
                        chain.append(cur.attr)
                        cur = cur.value
            if not (isinstance(cur, ast.Name) and cur.id == "pshattn"):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args):
                continue
            sites.append({"file": os.path.relpath(path, REF), "line": node.lineno, "name": ".".join(reversed(chain)),
                          "nargs": len(node.args), "keywords": [k.arg for k in node.keywords]})
    json.dump(sites, open(os.path.join(HERE, "call_sites.json"), "w"), indent=0)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
