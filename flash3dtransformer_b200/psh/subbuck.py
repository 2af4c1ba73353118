"""Host side of pooling / unpooling: row planning and buffer allocation.

Mirror of the reference's flash3dxfmr/psh/subbuck.py:40-132 (`calc_red_sep_sizes`, `SubbuckBuffers`,
`UnpoolBuffers`, `UnpoolGradients`).  Differences: alignment rows of reduced_coord / reduced_feat and the tail rows
of the unpooled output are zero-filled by the kernels instead of being left uninitialised (they flow into the next
attention layer), and for sub-bucket sizes that do not divide 1024 each full block of 1024 points is given
ceil(1024/S) rows, which is what the per-block construction needs (the reference sizes ceil(n/S) and can write
past its buffer, src/psh/batch_psh_subbuck_reduce.cuh:254-255).
"""
from __future__ import annotations

import dataclasses as dcls

import torch

from . import batching as f3dbatch
from . import plan as f3dplan
from .arithmatic import cdiv

BLOCK_POINTS = 1024


def calc_red_sep_sizes(seps: torch.Tensor, subbuck_size: int):
    """(total reduced rows, rows per scene, inclusive row separators) for a flat batch."""
    assert seps.dim() == 1, f"Seps dimension is expected to be 1, got {seps.dim()} instead"
    wide = f3dbatch.host_seps(seps)                      # scene sizes are planned on the host
    sizes = torch.diff(wide, prepend=wide.new_zeros(1))
    per_block = -(-BLOCK_POINTS // subbuck_size)
    red_sizes = (sizes // BLOCK_POINTS) * per_block + ((sizes % BLOCK_POINTS) + subbuck_size - 1) // subbuck_size
    red_sep_cpu = torch.cumsum(red_sizes, dim=0)
    red_sep = f3dbatch.attach_host_seps(red_sep_cpu.to(seps.dtype).to(seps.device), red_sep_cpu)
    return int(red_sizes.sum()), red_sizes.to(seps.dtype).to(seps.device), red_sep


@dcls.dataclass(slots=True)
class SubbuckBuffers:
    bbox_min: torch.Tensor
    bbox_max: torch.Tensor
    expect_sep: torch.Tensor
    subbuck_id: torch.Tensor
    subbuck_off: torch.Tensor
    reduced_sep: torch.Tensor
    reduced_coord: torch.Tensor
    reduced_feat: torch.Tensor
    unpool_ind: torch.Tensor
    pooled_rows: int = 0          # leading rows of the input that belong to a scene (= last separator)
    shared: bool = False          # handed out by plan.level_buffers(): reused by the next call, nothing may be dropped

    @staticmethod
    def create_subbuck_buff(coords: torch.Tensor, input_feat: torch.Tensor, seps: torch.Tensor,
                            subbuck_size=2, out_alignment=1):
        """out_alignment: reduced row count is rounded up to a multiple of it so the next bucketed attention
        sees whole buckets."""
        total_n, d = coords.shape
        feat_dim = input_feat.shape[1]
        dev = coords.device
        if f3dplan.enabled():
            # inference inside plan.level_buffers(): one plan per batch signature (scene sizes, widths), reused and not
            # filled.  The bounding box is not computed: the sub-bucket hash normalises with each block's own box, the
            # two fields only keep the reference's argument list
            sizes = tuple(f3dbatch.host_seps(seps).tolist())
            key = ("subbuck", sizes, total_n, d, feat_dim, str(input_feat.dtype), subbuck_size, out_alignment, str(dev))

            def build():
                red_len, _, red_sep = calc_red_sep_sizes(seps, subbuck_size)
                aligned = cdiv(red_len, out_alignment) * out_alignment
                box = torch.zeros(d, dtype=torch.float16, device=dev)
                return SubbuckBuffers(
                    bbox_min=box, bbox_max=box, expect_sep=red_sep,
                    subbuck_id=torch.empty(total_n, dtype=torch.uint32, device=dev),
                    subbuck_off=torch.empty(total_n, dtype=torch.uint16, device=dev),
                    reduced_sep=red_sep,
                    reduced_coord=torch.empty(aligned, d, dtype=torch.float16, device=dev),
                    reduced_feat=torch.empty(aligned, feat_dim, dtype=input_feat.dtype, device=dev),
                    unpool_ind=torch.empty((red_len, subbuck_size), dtype=torch.uint32, device=dev),
                    pooled_rows=min(total_n, int(sizes[-1])) if sizes else 0, shared=True)

            return f3dplan.pooled(key, build)
        bbox_min, bbox_max = torch.aminmax(coords, dim=0)
        assert bbox_min.dtype == torch.float16
        red_len, _, red_sep = calc_red_sep_sizes(seps, subbuck_size)
        aligned = cdiv(red_len, out_alignment) * out_alignment
        return SubbuckBuffers(
            bbox_min=bbox_min, bbox_max=bbox_max, expect_sep=red_sep,
            subbuck_id=torch.zeros(total_n, dtype=torch.uint32, device=dev),
            subbuck_off=torch.empty(total_n, dtype=torch.uint16, device=dev),
            reduced_sep=red_sep,
            reduced_coord=torch.empty(aligned, d, dtype=torch.float16, device=dev),
            reduced_feat=torch.empty(aligned, feat_dim, dtype=input_feat.dtype, device=dev),
            # out-of-range default marks an unfilled sub-bucket slot
            unpool_ind=torch.full((red_len, subbuck_size), total_n + 3, dtype=torch.uint32, device=dev),
            pooled_rows=min(total_n, int(f3dbatch.host_seps(seps)[-1])) if seps.numel() else 0,
        )

    def remove_unused_buffers(self):
        if self.shared:
            return
        self.subbuck_id = None
        self.subbuck_off = None


@dcls.dataclass(slots=True)
class UnpoolBuffers:
    up_add_feat: torch.Tensor

    @staticmethod
    def create_unpool_buff(residual_feat: torch.Tensor):
        return UnpoolBuffers(torch.empty_like(residual_feat))


@dcls.dataclass(slots=True)
class UnpoolGradients:
    grad_res: torch.Tensor
    grad_down: torch.Tensor

    @staticmethod
    def create_unpool_grad(grad_up_added: torch.Tensor, sb: SubbuckBuffers):
        down_len = sb.reduced_feat.shape[0]
        return UnpoolGradients(
            torch.zeros_like(grad_up_added),
            torch.zeros(down_len, grad_up_added.shape[-1], dtype=grad_up_added.dtype, device=grad_up_added.device))
