"""Multi-head self attention with a fused forward-Laplacian rule.

Counterpart of ``folx.experimental.pallas.attention.multi_head_self_attention``
(folx/experimental/pallas/attention/__init__.py:83-154): the function a model calls; when its
arguments carry triplets the registered rule ``'_multi_head_self_attention'`` (the fused sm_100a
kernel) runs, otherwise plain softmax attention.
"""

from __future__ import annotations

import torch

from .interpreter import LaplTensor, apply_rule


def multi_head_self_attention(q, k, v, mask=None, input_mask=None):
    """``softmax(q k^T) v`` per head; ``q, k, v``: ``(n, H, d)`` per walker (``(B, n, H, d)`` plain).

    ``mask``: ``(n,)`` / ``(B, n)`` bool, padded electrons; ``input_mask``: ``(R,)`` / ``(R, B)`` bool,
    padded input coordinates.  No ``1/sqrt(d)`` scaling is applied (scale ``q``), as in the
    reference kernel.
    """
    if not any(isinstance(t, LaplTensor) for t in (q, k, v)):
        s = torch.einsum('...ihd,...jhd->...hij', q, k)
        if mask is not None:
            sq = mask[..., :, None] & mask[..., None, :]
            s = torch.where(sq[..., None, :, :], s, torch.full_like(s, -1e20))
        return torch.einsum('...hij,...jhd->...ihd', torch.softmax(s, -1), v)
    t0 = next(t for t in (q, k, v) if isinstance(t, LaplTensor))
    if t0.nb == 0:
        # a single walker: the kernel wants a walker axis
        add = lambda t: t.unsqueeze(0) if t is not None else None
        q, k, v = add(q), add(k), add(v)
        mask = mask[None] if mask is not None else None
        input_mask = input_mask[:, None] if input_mask is not None else None
        t1 = next(t for t in (q, k, v) if isinstance(t, LaplTensor))
        out = apply_rule('_multi_head_self_attention', q, k, v, mask, input_mask)
        return out.squeeze(0) if t1 is not None else out
    return apply_rule('_multi_head_self_attention', q, k, v, mask, input_mask)


def multi_head_self_edge_attention(q, k, e, v, mask=None, input_mask=None):
    """``softmax(q k^T + e) v`` per head with an edge bias ``e``: ``(n, H, n)`` per walker
    (``(B, n, H, n)`` plain), indexed (query electron, head, key electron).

    Counterpart of the reference's ``multi_head_self_edge_attention``
    (folx/experimental/pallas/attention/__init__.py:50-79, 157-230); with triplet arguments the
    registered rule ``'_multi_head_self_edge_attention'`` runs.
    """
    args = (q, k, e, v)
    if not any(isinstance(t, LaplTensor) for t in args):
        s = torch.einsum('...ihd,...jhd->...hij', q, k) + e.transpose(-3, -2)
        if mask is not None:
            sq = mask[..., :, None] & mask[..., None, :]
            s = torch.where(sq[..., None, :, :], s, torch.full_like(s, -1e20))
        return torch.einsum('...hij,...jhd->...ihd', torch.softmax(s, -1), v)
    t0 = next(t for t in args if isinstance(t, LaplTensor))
    if t0.nb == 0:
        q, k, e, v = (t.unsqueeze(0) for t in args)
        mask = mask[None] if mask is not None else None
        input_mask = input_mask[:, None] if input_mask is not None else None
        return apply_rule('_multi_head_self_edge_attention', q, k, e, v, mask, input_mask).squeeze(0)
    return apply_rule('_multi_head_self_edge_attention', q, k, e, v, mask, input_mask)
