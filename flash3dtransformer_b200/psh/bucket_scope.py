"""Attention scopes: which buckets attend to each other (reference: flash3dxfmr/psh/bucket_scope.py:14-209).

A scope is a list of bucket indices; `SwinPlan.gen_scopes_from_plan` returns the [num_scopes, scope_size] uint32
table the attention kernels take.  As in the reference, both plan names yield contiguous, disjoint runs of
`scope_size_in_buck` buckets when the length allows it and one all-bucket scope otherwise
(bucket_scope.py:58-78; `offset_or_stride` is carried but never used there either).  The table is cached per
(length, plan, device) instead of being rebuilt and copied to the device on every layer call.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List

import torch


def minimal_alignment(buck_size: int, scope_size_in_buck: int) -> int:
    return buck_size


def swinable_alignment(buck_size: int, scope_size_in_buck: int) -> int:
    return buck_size * scope_size_in_buck


def stridable_alignment(buck_size: int, scope_size_in_buck: int) -> int:
    """6 = lcm(1, 2, 3) times the swin alignment, so strides 1..3 divide the bucket count."""
    return buck_size * scope_size_in_buck * 6


def generate_single_scope(total_N: int, buck_size: int, scope_size: int) -> List[List[int]]:
    return [list(range(total_N // buck_size))]


def generate_stride_scopes(total_N: int, buck_size: int, scope_size: int, stride: int = 1) -> List[List[int]]:
    n = int(math.ceil(total_N / buck_size))
    assert n % stride == 0, f"num_bucket={n} must be divisible by stride={stride}"
    scopes = []
    chunk = scope_size * stride
    for start in range(0, n, chunk):
        for s in range(stride):
            idx = [start + s + stride * j for j in range(scope_size)]
            if all(i <= n for i in idx):
                scopes.append(idx)
    return scopes


def generate_swin_scopes(total_N: int, buck_size: int, scope_size: int, offset: int = 0) -> List[List[int]]:
    """Disjoint runs of `scope_size` buckets starting at `offset`, wrapping around the end."""
    n = int(math.ceil(total_N / buck_size))
    assert scope_size <= n, "scope_size must be less than or equal to the number of buckets (N)"
    assert n % scope_size == 0, "For non-overlapping scopes, the number of buckets N must be divisible by scope_size"
    return [[(offset + i * scope_size + j) % n for j in range(scope_size)] for i in range(n // scope_size)]


_SCOPE_CACHE = {}


@dataclass
class SwinPlan:
    plan_name: str
    buck_size: int
    scope_size_in_buck: int
    offset_or_stride: int

    def scope_list(self, total_N: int) -> List[List[int]]:
        assert self.plan_name in ["swin", "stride"], f"Unsupported scoping plan name: {self.plan_name}"
        min_align = minimal_alignment(self.buck_size, self.scope_size_in_buck)
        assert total_N % min_align == 0, \
            f"Input buffer length must be divisible by minimal alignment = {min_align}, but got {total_N}"
        if self.plan_name == "stride":
            if total_N % stridable_alignment(self.buck_size, self.scope_size_in_buck) == 0:
                return generate_stride_scopes(total_N, self.buck_size, self.scope_size_in_buck)
            return generate_single_scope(total_N, self.buck_size, self.scope_size_in_buck)
        if total_N % swinable_alignment(self.buck_size, self.scope_size_in_buck) == 0:
            return generate_swin_scopes(total_N, self.buck_size, self.scope_size_in_buck)
        return generate_single_scope(total_N, self.buck_size, self.scope_size_in_buck)

    def gen_scopes_from_plan(self, total_N: int, device) -> torch.Tensor:
        key = (total_N, self.plan_name, self.buck_size, self.scope_size_in_buck, str(device))
        if key not in _SCOPE_CACHE:
            scopes = self.scope_list(total_N)
            t = torch.tensor(scopes, dtype=torch.uint32).to(device)
            # every bucket in exactly one scope: the attention backward then writes every gradient row itself
            flat = sorted(b for sc in scopes for b in sc)
            t._f3d_partition_of = total_N if flat == list(range(total_N // self.buck_size)) else -1
            _SCOPE_CACHE[key] = t
        return _SCOPE_CACHE[key]


def construct_bucket_scopes(I: torch.Tensor, buck_size: int, attn_scopes: List[List[int]]) -> torch.Tensor:
    """[D, L] features -> [num_scopes, D, scope_len]: the buckets of each scope side by side."""
    return torch.stack([torch.cat([I[:, b * buck_size:(b + 1) * buck_size] for b in scope], dim=-1)
                        for scope in attn_scopes], dim=0)


def revert_bucket_scopes(I: torch.Tensor, bucket_size: int, attn_scopes: List[List[int]]) -> torch.Tensor:
    """Inverse of construct_bucket_scopes: [num_scopes, D, scope_len] -> [D, L]."""
    seg = {}
    for si, scope in enumerate(attn_scopes):
        for bi, b in enumerate(scope):
            seg[b] = I[si, :, bi * bucket_size:(bi + 1) * bucket_size]
    return torch.cat([seg[i] for i in range(max(seg) + 1)], dim=-1)


def reassign_bucket_scopes(I: torch.Tensor, bucket_size: int, old_scopes: List[List[int]],
                           new_scopes: List[List[int]]) -> torch.Tensor:
    """Regroup a scoped tensor from one scope assignment to another."""
    seg = {}
    for si, scope in enumerate(old_scopes):
        for bi, b in enumerate(scope):
            seg[b] = I[si, :, bi * bucket_size:(bi + 1) * bucket_size]
    return torch.stack([torch.cat([seg[b] for b in scope], dim=-1) for scope in new_scopes], dim=0)
