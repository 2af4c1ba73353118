"""Layer modules with the names the reference exports from flash3dxfmr.layers (layers/__init__.py:1-27)."""
from .buck_swin import BucketSwinAttentionModule
from .elem_wise import MLP
from .flash3d import Flash3D, F3DLevelSpecs
from .hourglass import PoolingWrapper, AdditiveUnpoolingWrapper, HourglassModule
from .psh_ops import PSHScatterLayer, PSH3DCoordEmbedding
from .stage import XFMRSpecs, XFMR, Stage

__all__ = [
    "AdditiveUnpoolingWrapper", "BucketSwinAttentionModule", "F3DLevelSpecs", "Flash3D", "HourglassModule", "MLP",
    "PoolingWrapper", "PSH3DCoordEmbedding", "PSHScatterLayer", "Stage", "XFMR", "XFMRSpecs",
]
