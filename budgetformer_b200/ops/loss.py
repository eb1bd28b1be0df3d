"""Readout loss: mean negative log-likelihood of ``softmax(logits)`` over a fixed set of rows.

On GPUs one kernel computes the loss and the full ``d loss / d logits`` (zeros outside the selected rows) in the
forward pass; backward just scales it.  Equivalent to ``F.nll_loss(F.log_softmax(logits)[idx], y[idx])``
(main_node_fullgraph_sp.py:1234-1237 in the reference)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _ext


class _MaskedNLL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, y, mask, count):
        need = logits.requires_grad
        loss_sum, d = _ext.load().nll_fwd_bwd(logits, y, mask, bool(need), 1.0 / max(float(count), 1.0))
        _ext.count_launches(1)
        ctx.save_for_backward(d)
        return (loss_sum / max(float(count), 1.0)).reshape(())

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g.to(d.dtype), None, None, None


def masked_nll(logits: torch.Tensor, y: torch.Tensor, idx: torch.Tensor, mask: torch.Tensor = None) -> torch.Tensor:
    """``logits`` ``[n, C]``, ``y`` ``[n]`` int64 (entries outside ``idx`` are ignored), ``idx`` the selected rows."""
    if logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1 and idx.numel() > 0:
        if mask is None:
            mask = torch.zeros(logits.size(0), dtype=torch.uint8, device=logits.device)
            mask[idx] = 1
        return _MaskedNLL.apply(logits, y.contiguous(), mask, int(idx.numel()))
    if idx.numel() == 0:
        return logits.sum() * 0
    return F.nll_loss(F.log_softmax(logits[idx].float(), dim=1), y[idx])
