"""Drop-in for the reference's compiled operator module `flash3dxfmr.lib.pshattn` (bindings src/f3d_frontend.cu:112-138).

Copy this file (and the `__init__.py` beside it) into the reference checkout's `flash3dxfmr/lib/`, or call
`flash3dtransformer_b200.compat.install(<reference checkout>)`: every `from ..lib import pshattn` of the reference's
host code (psh/psh_main.py:18, psh/dev_context.py:9, psh/bucket.py:13, layers/pooling.py:15, layers/unpool.py:15,
layers/buck_swin.py:17, layers/stage.py:18, layers/hourglass.py:18) then reaches libf3d_b200.so with the reference's own
argument lists.
"""
from flash3dtransformer_b200.lib.pshattn import *  # noqa: F401,F403
from flash3dtransformer_b200.lib.pshattn import (  # noqa: F401  (the bound surface, spelled out)
    DeviceManagerSingleton, additive_unpool_bwd, additive_unpool_fwd, batch_bucket_sanitizer_cpu, batch_psh_scatter,
    batch_psh_scatter_pad, batch_psh_scatter_pad_hash, batch_subbuck_reduce, batch_subbuck_reduce_backward, buck_swin_bwd,
    buck_swin_fwd, gemm_sm_bf16)
