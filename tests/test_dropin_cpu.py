"""CPU checks of the drop-in boundary against the reference's own host code.

  * every `pshattn.<operator>(...)` call of the reference's Python package and tests (captured from its syntax trees into
    tests/golden/call_sites.json by tests/golden/make_golden.py) binds against the signature of the operator module
    that replaces the compiled extension;
  * the scoreboard operator `batch_bucket_sanitizer_cpu` (src/psh/bucket_sanitizer_cpu.cpp:92-176) accepts a correct
    bucketing, updates its two in/out tensors in place and raises on each kind of violation;
  * where a reference checkout is present ($F3D_REFERENCE, default /root/reference), its unmodified `flash3dxfmr`
    package imports over this library (`flash3dtransformer_b200.compat.install`) and the capture is still current.
No kernel is launched here.
"""
import inspect
import json
import os

import numpy as np
import pytest
import torch

from flash3dtransformer_b200 import compat, synthetic
from flash3dtransformer_b200.lib import pshattn
from oracle import psh_oracle as po

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF = os.environ.get("F3D_REFERENCE", "/root/reference")


def _sites():
    return json.load(open(os.path.join(G, "call_sites.json")))


def test_every_reference_call_site_binds():
    sites = _sites()
    names = {s["name"] for s in sites}
    # the surface the reference binds (src/f3d_frontend.cu:112-138) plus the two attention operators its layers call
    for must in ["batch_psh_scatter_pad_hash", "batch_subbuck_reduce", "batch_subbuck_reduce_backward",
                 "additive_unpool_fwd", "additive_unpool_bwd", "batch_bucket_sanitizer_cpu", "gemm_sm_bf16",
                 "buck_swin_fwd", "buck_swin_bwd", "DeviceManagerSingleton.instance"]:
        assert must in names, must
    for s in sites:
        obj = pshattn
        for part in s["name"].split("."):
            obj = getattr(obj, part)            # AttributeError = the drop-in lacks an operator the reference calls
        sig = inspect.signature(obj)
        try:
            sig.bind(*range(s["nargs"]), **{k: 0 for k in s["keywords"]})
        except TypeError as e:
            raise AssertionError(f"{s['file']}:{s['line']} {s['name']}: {e}") from None


def test_device_manager_methods_of_the_reference_exist():
    # flash3dxfmr/psh/dev_context.py:11-27 calls these on the singleton
    mgr = pshattn.DeviceManagerSingleton.instance()
    for m in ["init_dev_info", "init_dispatchers", "set_sync_stream", "get_sync_stream"]:
        assert callable(getattr(mgr, m)), m


def _bucketing(sizes=(3000, 2100, 2600), bucket_size=128, hash_type=2):
    c32, seps = synthetic.batch(synthetic.lidar_scan, list(sizes), seed=4)
    c16 = c32.astype(np.float16)
    nb, div = po.psh_params(list(sizes), bucket_size)
    out = po.psh_scatter(c16, seps, nb, div, bucket_size, 0xFFFF, c16.min(0), c16.max(0), po.probe_table(), len(c16), 0.0,
                         hash_type)
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).astype(dt.replace("u", "")).copy()).view(getattr(torch, dt))
    bid = t(out["bucket_id"], "uint16")
    cnt = t(out["bucket_cntr"], "uint32")
    off = t(out["bucket_offs"], "uint32")
    sp = t(seps, "uint32")
    return bid, cnt, off, sp, nb, len(sizes)


def _sanitize(bid, cnt, off, sp, nb, batch, table=None, res=None):
    """The argument preparation of the reference's own test, tests/test_psh.py:109-129."""
    maxcnt, _ = torch.max(cnt.to(torch.int32), dim=-1)
    maxcnt = maxcnt.to(torch.uint32)
    slots = int(torch.max(cnt.to(torch.int32)))
    table = torch.zeros((batch, nb, slots), dtype=torch.int8) if table is None else table
    res = cnt.detach().clone() if res is None else res
    pshattn.batch_bucket_sanitizer_cpu(bid, cnt, off, table, res, sp, maxcnt, batch, nb)
    return table, res


def test_sanitizer_accepts_a_correct_bucketing_and_updates_in_place():
    bid, cnt, off, sp, nb, batch = _bucketing()
    table, res = _sanitize(bid, cnt, off, sp, nb, batch)
    assert int(res.to(torch.int64).sum()) == 0                     # every unit of every bucket was taken
    c = cnt.to(torch.int64)
    assert int(table.to(torch.int64).sum()) == int(c.sum()) == bid.numel()
    slots = torch.arange(table.shape[2]).view(1, 1, -1)
    assert torch.equal(table.to(torch.int64), (slots < c.unsqueeze(-1)).to(torch.int64))
    po.scoreboard_check(bid.view(torch.int16).numpy().view(np.uint16), cnt.view(torch.int32).numpy().view(np.uint32),
                        off.view(torch.int32).numpy().view(np.uint32), sp.view(torch.int32).numpy().view(np.uint32), nb)


def _poke(t, index, value):
    a = t.view(torch.int16 if t.dtype == torch.uint16 else torch.int32).clone()
    a[index] = value
    return a.view(t.dtype)


def test_sanitizer_raises_on_each_violation_and_leaves_outputs_alone():
    bid, cnt, off, sp, nb, batch = _bucketing()
    n = bid.numel()
    # two points in one slot
    j = int((bid.view(torch.int16)[:3000] == bid.view(torch.int16)[0]).nonzero()[1])
    dup = _poke(off, j, int(off.view(torch.int32)[0]))
    table = torch.zeros((batch, nb, int(torch.max(cnt.to(torch.int32)))), dtype=torch.int8)
    res = cnt.detach().clone()
    with pytest.raises(RuntimeError, match="Wrong scoreboard"):
        _sanitize(bid, cnt, dup, sp, nb, batch, table, res)
    assert int(table.abs().sum()) == 0 and torch.equal(res.view(torch.int32), cnt.view(torch.int32))
    # bucket id out of range; offset beyond the scene's largest bucket
    with pytest.raises(RuntimeError, match="overflow"):
        _sanitize(_poke(bid, n - 1, nb), cnt, off, sp, nb, batch)
    with pytest.raises(RuntimeError, match="overflow"):
        _sanitize(bid, cnt, _poke(off, 5, 1 << 20), sp, nb, batch)
    # wrong dtype is an argument error like assert_dtype (src/common/runtime.h:72-86)
    with pytest.raises(RuntimeError, match="dtype"):
        pshattn.batch_bucket_sanitizer_cpu(bid.view(torch.int16), cnt, off, table, res, sp, sp, batch, nb)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "flash3dxfmr")), reason="no reference checkout")
def test_reference_package_imports_over_this_library_and_capture_is_current():
    import ast
    import glob
    try:
        pkg = compat.install(REF)
        from flash3dxfmr.lib import pshattn as shim          # noqa: the reference's own import path
        from flash3dxfmr.psh import psh_main, dev_context
        from flash3dxfmr.layers import pooling, unpool, buck_swin
        assert psh_main.pshattn is shim and pooling.pshattn is shim and unpool.pshattn is shim and buck_swin.pshattn is shim
        assert shim.batch_psh_scatter_pad_hash is pshattn.batch_psh_scatter_pad_hash
        assert os.path.dirname(psh_main.__file__) == os.path.join(REF, "flash3dxfmr", "psh")
        assert dev_context.DEV_MGR is pshattn.DeviceManagerSingleton.instance()
        assert pkg.Flash3D.__module__ == "flash3dxfmr.layers.flash3d"
    finally:
        compat.uninstall()
    # the committed capture lists the same call sites as the checkout
    count = 0
    for path in glob.glob(os.path.join(REF, "flash3dxfmr", "**", "*.py"), recursive=True) + glob.glob(os.path.join(REF, "tests", "*.py")):
        src = open(path).read()
        for node in ast.walk(ast.parse(src)):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and isinstance(node.func.value, ast.Name) \
                    and node.func.value.id == "pshattn":
                count += 1
    assert count == sum(1 for s in _sites() if "." not in s["name"])
