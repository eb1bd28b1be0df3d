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


def gelu_dropout(x: torch.Tensor, seed: int, p: float) -> torch.Tensor:
    """``dropout(gelu(x), p)`` in one pass over ``x`` with the hash keep mask of ``hash_dropout`` (no autograd: the caller
    differentiates it, see ``ops.ffn._FusedFFNGelu``)."""
    if x.is_cuda and x.dim() == 2 and x.stride(1) == 1:
        _ext.count_launches(1)
        return _ext.load().gelu_dropout(x, int(seed), float(p))
    y = torch.nn.functional.gelu(x.float()).to(x.dtype)
    if p <= 0.0:
        return y
    keep = hash_keep_mask(seed, x.size(0), x.size(1), p, x.device)
    return torch.where(keep, y / (1.0 - p), torch.zeros_like(y))


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


# ---------------------------------------------------------------------------------------------------
# BatchNorm over rows (GraphGPS / Exphormer post-norm, models/graphgps_dist_node_level.py:276-280 in the reference)
# ---------------------------------------------------------------------------------------------------
def _bn_kernel_ok(x: torch.Tensor) -> bool:
    return (x.is_cuda and x.dim() == 2 and x.stride(1) == 1 and x.size(1) % 8 == 0 and 8 <= x.size(1) <= 2048
            and x.data_ptr() % 16 == 0 and (x.stride(0) * x.element_size()) % 16 == 0
            and x.dtype in (torch.bfloat16, torch.float16, torch.float32))


def _bn_stats(x, shift):
    if _bn_kernel_ok(x):
        _ext.count_launches(1)
        return _ext.load().bn_stats(x, shift)
    d = x.float() - (shift if shift is not None else 0.0)
    return d.sum(0), (d * d).sum(0)


def _bn_bwd_reduce(dy, x, mean, rstd):
    if _bn_kernel_ok(x) and _bn_kernel_ok(dy):
        _ext.count_launches(1)
        return _ext.load().bn_bwd_reduce(dy, x, mean, rstd)
    dyf = dy.float()
    return dyf.sum(0), (dyf * (x.float() - mean) * rstd).sum(0)


def _col_affine(x, in2, a, b, c0):
    if _bn_kernel_ok(x) and (in2 is None or _bn_kernel_ok(in2)):
        _ext.count_launches(1)
        return _ext.load().col_affine(x, in2, a.contiguous(), b.contiguous(), None if c0 is None else c0.contiguous())
    if in2 is None:
        return (x.float() * a + b).to(x.dtype)
    return (in2.float() * a + x.float() * b + c0).to(x.dtype)


class _BatchNormTrain(torch.autograd.Function):
    """Training-mode BatchNorm on ``[rows, h]`` in the activation dtype with fp32 statistics.

    Two passes per direction: shifted one-pass column statistics (the shift is the running mean, which keeps
    ``E[(x-s)^2] - E[x-s]^2`` well conditioned), then one fused multiply-add per element.  With ``group`` the
    statistics and the backward reductions are summed over the ranks of the group, i.e. SyncBatchNorm over the
    sequence-parallel node shards; without it every rank normalises with its own rows like the reference.  CUDA
    tensors run on the row kernels of ``csrc/norm_fused.cu``, anything else on the same arithmetic in PyTorch."""

    @staticmethod
    def forward(ctx, x, weight, bias, shift, eps, group):
        s1, s2 = _bn_stats(x, shift)
        count = torch.tensor([float(x.size(0))], device=x.device)
        if group is not None:
            import torch.distributed as dist
            packed = torch.cat([s1, s2, count])
            dist.all_reduce(packed, group=group)
            h = x.size(1)
            s1, s2, count = packed[:h], packed[h:2 * h], packed[2 * h:]
        m1 = s1 / count
        var = (s2 / count - m1 * m1).clamp_min_(0.0)                # biased variance
        mean = m1 + (shift if shift is not None else 0.0)
        rstd = torch.rsqrt(var + eps)
        g32 = weight.float() if weight is not None else torch.ones_like(mean)
        b32 = bias.float() if bias is not None else torch.zeros_like(mean)
        a = g32 * rstd
        y = _col_affine(x, None, a, b32 - mean * a, None)
        ctx.save_for_backward(x, mean, rstd, g32)
        ctx.group, ctx.count = group, count
        ctx.pdtype = weight.dtype if weight is not None else torch.float32
        ctx.has_affine = (weight is not None, bias is not None)
        ctx.mark_non_differentiable(mean, var, count)
        return y, mean, var, count

    @staticmethod
    def backward(ctx, dy, _dmean, _dvar, _dcount):
        x, mean, rstd, g32 = ctx.saved_tensors
        dy = dy.to(x.dtype)
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        dbeta, dgamma = _bn_bwd_reduce(dy, x, mean, rstd)
        sb, sg = dbeta, dgamma
        if ctx.group is not None:
            import torch.distributed as dist
            packed = torch.cat([dbeta, dgamma])
            dist.all_reduce(packed, group=ctx.group)
            sb, sg = packed[:dbeta.numel()], packed[dbeta.numel():]
        n = ctx.count
        # dx = g*rstd * (dy - mean(dy) - xhat * mean(dy*xhat)),  xhat = (x - mean) * rstd
        a = g32 * rstd
        b = -a * rstd * (sg / n)
        c0 = a * (-(sb / n) + mean * rstd * (sg / n))
        dx = _col_affine(x, dy, a, b, c0)
        has_w, has_b = ctx.has_affine
        return dx, (dgamma.to(ctx.pdtype) if has_w else None), (dbeta.to(ctx.pdtype) if has_b else None), None, None, None


def batch_norm(x: torch.Tensor, bn: torch.nn.BatchNorm1d, group=None) -> torch.Tensor:
    """``bn(x)`` for 2-D ``x`` with the module's parameters and running statistics; ``group`` synchronises the batch
    statistics over a process group (``--sync_batchnorm``).  CUDA tensors use the row kernels in the activation
    dtype; CPU tensors without a group go through PyTorch in fp32."""
    training = bn.training or not bn.track_running_stats
    synced = group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1
    if training and (_bn_kernel_ok(x) or synced):
        shift = bn.running_mean.float().contiguous() if bn.running_mean is not None else None
        y, mean, var, count = _BatchNormTrain.apply(x, bn.weight, bn.bias, shift, float(bn.eps), group if synced else None)
        if bn.track_running_stats and bn.running_mean is not None:
            with torch.no_grad():
                bn.num_batches_tracked += 1
                mom = bn.momentum if bn.momentum is not None else 1.0 / float(bn.num_batches_tracked)
                unbias = count / torch.clamp(count - 1.0, min=1.0)
                bn.running_mean.mul_(1 - mom).add_(mean.to(bn.running_mean.dtype), alpha=mom)
                bn.running_var.mul_(1 - mom).add_((var * unbias).to(bn.running_var.dtype), alpha=mom)
        return y
    if _bn_kernel_ok(x) and not training:
        rstd = torch.rsqrt(bn.running_var.float() + bn.eps)
        a = (bn.weight.float() if bn.weight is not None else torch.ones_like(rstd)) * rstd
        b = (bn.bias.float() if bn.bias is not None else torch.zeros_like(rstd)) - bn.running_mean.float() * a
        return _col_affine(x, None, a, b, None)
    return bn(x.float()).to(x.dtype)
