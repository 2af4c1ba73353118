"""CPU oracle of bucketed self-attention (forward, backward) and of the projection GEMMs, in fp32 with torch.
TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg; never by the
product path.

Parity status: pinned on the reference's own fixture.  `naive_attn` restates naive_attn_fwd of the reference's
tests (tests/test_lib.py:24-38), and tests/golden/attn_naive_*.npz holds outputs of that function, produced by
importing the reference's tests/test_lib.py in the build container (tests/golden/make_golden.py);
tests/test_attn_oracle.py checks this oracle against them.  The scope gather follows construct_bucket_scopes /
revert_bucket_scopes (flash3dxfmr/psh/bucket_scope.py:143-181), also pinned by a golden file.

Restated from the reference:
  naive attention            tests/test_lib.py:24-38
  scope construction         flash3dxfmr/psh/bucket_scope.py:143-181
  Delta                      tests/test_attn_bwd.py:24-27  (Delta = sum_d dO * O)
  backward formulas          tests/test_attn_bwd.py:54-62, autograd of the naive forward
"""
from __future__ import annotations

import math

import torch


def naive_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """q, k, v: [..., T, D] fp32 -> (o [..., T, D], lse [..., T]) with softmax(q k^T / sqrt(D)) v."""
    d = q.shape[-1]
    s = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(d)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    return torch.matmul(p, v), lse


def scope_tokens(scope_row, bucket_size: int) -> torch.Tensor:
    """Token indices of one scope: its buckets' ranges concatenated in listed order."""
    return torch.cat([torch.arange(int(b) * bucket_size, (int(b) + 1) * bucket_size) for b in scope_row])


def buck_swin_fwd(Q, K, V, scopes, bucket_size: int, O_init=None):
    """Q, K, V [B,L,H,D] (any float dtype) -> O [B,L,H,D] fp32, LSE [B,L,H] fp32.  Tokens of buckets not listed in
    `scopes` keep O_init (zeros by default) and LSE 0, like a caller-provided zero buffer
    (flash3dxfmr/psh/swin_attn.py:18-23)."""
    q, k, v = Q.float(), K.float(), V.float()
    b, l, h, d = q.shape
    o = torch.zeros_like(q) if O_init is None else O_init.float().clone()
    lse = torch.zeros(b, l, h)
    for row in scopes.tolist():
        idx = scope_tokens(row, bucket_size)
        qs, ks, vs = (t[:, idx].permute(0, 2, 1, 3) for t in (q, k, v))     # [B,H,T,D]
        os_, ls = naive_attn(qs, ks, vs)
        o[:, idx] = os_.permute(0, 2, 1, 3)
        lse[:, idx] = ls.permute(0, 2, 1)
    return o, lse


def buck_swin_bwd(Q, K, V, dO, scopes, bucket_size: int):
    """Gradients by autograd of the fp32 forward: (dQ, dK, dV, Delta) with Delta[b,t,h] = sum_d dO*O."""
    q, k, v = (t.float().detach().requires_grad_(True) for t in (Q, K, V))
    o, _ = _fwd_autograd(q, k, v, scopes, bucket_size)
    o.backward(dO.float())
    delta = (dO.float() * o.detach()).sum(-1)
    return q.grad, k.grad, v.grad, delta


def _fwd_autograd(q, k, v, scopes, bucket_size):
    b, l, h, d = q.shape
    pieces, order = [], []
    for row in scopes.tolist():
        idx = scope_tokens(row, bucket_size)
        qs, ks, vs = (t[:, idx].permute(0, 2, 1, 3) for t in (q, k, v))
        os_, _ = naive_attn(qs, ks, vs)
        pieces.append(os_.permute(0, 2, 1, 3))
        order.append(idx)
    o = torch.zeros(b, l, h, d)
    o = o.index_copy(1, torch.cat(order), torch.cat(pieces, dim=1))
    return o, None


def linear(x, w, b=None):
    """fp32 reference of the projection GEMMs (nn.Linear, flash3dxfmr/layers/buck_swin.py:159,163)."""
    y = x.float() @ w.float().t()
    return y if b is None else y + b.float()
