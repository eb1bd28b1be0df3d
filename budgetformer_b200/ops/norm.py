"""LayerNorm and counter-based dropout on the row kernels of ``csrc/norm_fused.cu``.

``layer_norm`` keeps fp32 statistics per row and recomputes the normalised input in backward from
the saved input; ``hash_dropout`` derives its keep mask from ``(seed, row, col)`` exactly like the
GEMM epilogue does, so nothing but the seed is saved.  CPU tensors (and widths above 512) use the
PyTorch implementations."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _ext
from .gemm import hash_keep_mask


class ColsumSlot:
    """Hand-over of ``colsum(dx)`` from a LayerNorm backward to the backward of the linear layer that produced the
    normalised tensor (its bias gradient).  The consumer presents the gradient tensor it received; the value is only
    released when that is the very tensor the LayerNorm backward wrote (no other consumer added to it)."""

    __slots__ = ("ptr", "shape", "value")

    def __init__(self):
        self.ptr, self.shape, self.value = 0, None, None

    def put(self, dx: torch.Tensor, value: torch.Tensor) -> None:
        self.ptr, self.shape, self.value = dx.data_ptr(), tuple(dx.shape), value

    def take(self, dy: torch.Tensor):
        v = self.value
        self.value = None
        if v is not None and dy.data_ptr() == self.ptr and tuple(dy.shape) == self.shape:
            return v
        return None


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, slot=None):
        ext = _ext.load()
        g32, b32 = gamma.float().contiguous(), beta.float().contiguous()
        y, stats = ext.layernorm_fwd(x, g32, b32, float(eps))
        _ext.count_launches(1)
        ctx.save_for_backward(x, stats, g32)
        ctx.pdtype = gamma.dtype
        ctx.slot = slot
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.load()
        x, stats, g32 = ctx.saved_tensors
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        if ctx.slot is not None:
            dx, dg, db, dxsum = ext.layernorm_bwd(dy.to(x.dtype), x, stats, g32, True)
            ctx.slot.put(dx, dxsum)
        else:
            dx, dg, db = ext.layernorm_bwd(dy.to(x.dtype), x, stats, g32, False)
        _ext.count_launches(1)
        return dx, dg.to(ctx.pdtype), db.to(ctx.pdtype), None, None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5,
               dx_colsum: "ColsumSlot | None" = None) -> torch.Tensor:
    """2-D ``x`` ``[rows, h]``.  ``dx_colsum`` (optional) receives the column sums of the input gradient in backward."""
    if x.is_cuda and x.dim() == 2 and x.size(1) <= 512 and x.stride(1) == 1 and \
            x.dtype in (torch.bfloat16, torch.float16, torch.float32):
        return _LayerNorm.apply(x, weight, bias, eps, dx_colsum)
    return F.layer_norm(x.float(), (x.size(-1),), weight.float(), bias.float(), eps).to(x.dtype)


class _HashDropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seed, p):
        ctx.seed, ctx.p = int(seed), float(p)
        _ext.count_launches(1)
        return _ext.load().hash_dropout(x, int(seed), float(p))

    @staticmethod
    def backward(ctx, dy):
        _ext.count_launches(1)
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        return _ext.load().hash_dropout(dy, ctx.seed, ctx.p), None, None


def hash_dropout(x: torch.Tensor, seed: int, p: float) -> torch.Tensor:
    if p <= 0.0:
        return x
    if x.is_cuda and x.dim() == 2 and x.stride(1) == 1:
        return _HashDropout.apply(x, seed, p)
    keep = hash_keep_mask(seed, x.size(0), x.size(1), p, x.device)
    return torch.where(keep, x / (1.0 - p), torch.zeros_like(x))


def new_seed() -> int:
    """31-bit seed from torch's CPU generator (reproducible under ``torch.manual_seed``, no device sync)."""
    return int(torch.randint(0, 2 ** 31 - 1, (1,)).item())


def column_sum(x: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a 2-D tensor (bias gradients) without materialising an fp32 copy."""
    if x.is_cuda and x.dim() == 2 and x.stride(1) == 1 and x.size(1) % 8 == 0 and 8 <= x.size(1) <= 2048 \
            and x.data_ptr() % 16 == 0 and (x.stride(0) * x.element_size()) % 16 == 0 \
            and x.dtype in (torch.bfloat16, torch.float16, torch.float32):
        _ext.count_launches(1)
        return _ext.load().colsum(x)
    return torch.sum(x, dim=0, dtype=torch.float32)
