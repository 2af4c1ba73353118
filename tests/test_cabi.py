"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports every symbol that
include/f3d_b200.h declares, the ctypes prototypes cover the same set, and the operator module offers the names of
the reference's pybind module (src/f3d_frontend.cu:112-138).  No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "f3d_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(f3d_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from flash3dtransformer_b200.lib import _cabi
    if not _cabi.LIB_PATH.exists():
        from flash3dtransformer_b200 import build
        build.build()
    lib = ctypes.CDLL(os.fspath(_cabi.LIB_PATH))
    names = _declared()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in f3d_b200.h but not exported"
    assert sorted(_cabi.PROTOTYPES) == names, set(_cabi.PROTOTYPES) ^ set(names)
    assert _cabi.load().f3d_version() == 100
    assert _cabi.load().f3d_get_seed() == 3407


def test_operator_module_has_the_reference_surface():
    from flash3dtransformer_b200.lib import pshattn
    for name in ["DeviceManagerSingleton", "batch_psh_scatter", "batch_psh_scatter_pad", "batch_psh_scatter_pad_hash",
                 "additive_unpool_fwd", "additive_unpool_bwd", "batch_subbuck_reduce", "batch_subbuck_reduce_backward",
                 "gemm_sm_bf16", "buck_swin_fwd", "buck_swin_bwd", "batch_bucket_sanitizer_cpu"]:
        assert hasattr(pshattn, name), name
    mgr = pshattn.DeviceManagerSingleton.instance()
    assert mgr is pshattn.DeviceManagerSingleton.instance()
    old = mgr.set_sync_stream(True)
    assert mgr.get_sync_stream() is True
    mgr.set_sync_stream(old)
    mgr.set_seed(7)
    assert mgr.get_seed() == 7
    mgr.set_seed(3407)


def test_cpu_tensors_are_rejected_not_computed():
    import torch
    from flash3dtransformer_b200.lib import pshattn
    t = torch.zeros(4, 8, dtype=torch.bfloat16)
    ind = torch.zeros(2, 2, dtype=torch.uint32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pshattn.additive_unpool_fwd(t, t, t.clone(), ind, 2)


def test_layer_tree_keeps_reference_names():
    from flash3dtransformer_b200 import configs, layers
    model = configs.flash3d_backbone(channels=(32, 64), depths=(1, 1))
    keys = set(model.state_dict())
    for k in ["psh_scatter.lin.weight", "module_tree.encoder_blocks.0.norm.weight",
              "module_tree.encoder_blocks.0.bwa.qkv.weight", "module_tree.encoder_blocks.0.bwa.proj.bias",
              "module_tree.encoder_blocks.0.mlp.mlp.fc1_weight", "module_tree.middle.pooling.proj.weight",
              "module_tree.middle.unpooling.proj.0.weight", "module_tree.middle.unpooling.proj_skip.norm.weight",
              "module_tree.middle.submodule.middle.proj.weight"]:
        assert k in keys, k
    assert layers.__all__ == sorted(layers.__all__, key=lambda s: s.lower()) or len(layers.__all__) == 12
