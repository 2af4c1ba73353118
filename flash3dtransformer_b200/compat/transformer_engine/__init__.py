"""Stand-in for the `transformer_engine` package on hosts that do not have it: only the three modules the Flash3D
layers take from it (`transformer_engine.pytorch.Linear`, `.LayerNorm`, `.LayerNormMLP`), backed by this library's
kernels.  Used only when `flash3dtransformer_b200.compat.install(..., transformer_engine=True)` asks for it."""
from . import pytorch  # noqa: F401
