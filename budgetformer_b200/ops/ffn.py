"""Feed-forward block on the tcgen05 GEMM: ``y = residual + drop2(W2 drop1(act(W1 x + b1)) + b2)``.

Forward is two kernels (activation + dropout in the first epilogue, bias + dropout + residual in the
second); forward passes without a backward (evaluation) run as one kernel with the hidden tile kept on chip
(``ffn_onchip``).  Backward for ReLU uses the mask epilogue: ``dh = (g W2) * [h > 0] / (1 - p1)`` comes out of
the GEMM directly, so the hidden gradient is never touched by a separate elementwise pass.  GELU keeps
the pre-activation and the same GEMM's epilogue multiplies by ``gelu'(z)`` (``_FusedFFNGelu``).  Replaces Linear -> act -> Dropout -> Linear ->
Dropout -> add of the reference layers (e.g. models/gt_dist_node_level.py:655-660)."""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import gemm
from .norm import hash_dropout, new_seed


# the ReLU mask travels from forward to backward as one bit per hidden element (off: the backward re-reads h)
USE_RELU_BITS = True
# Forward passes that no backward will follow run the whole block in one kernel with the hidden tile kept on chip
# (csrc/ffn_fused_tcgen05.cu; model width 128, hidden width 256).  "all" (default): evaluation passes and the first
# forward of recomputed layers (recompute / keep_mha tiers; its hash dropout masks are reproduced by the recomputation,
# which runs the two-GEMM form because the backward needs the hidden matrix); "1": evaluation passes only; "0": off.
ONCHIP_FFN = os.environ.get("BF_FFN_ONCHIP", "all")
# training forward of the ReLU block on the same kernel with the hidden matrix and the ReLU bits as side outputs
# (1.05 against 1.42 ms per layer at 2.9 M rows); "0": two GEMMs
ONCHIP_FFN_TRAIN = os.environ.get("BF_FFN_ONCHIP_TRAIN", "1") == "1"


def ffn_onchip(x: torch.Tensor, w1, b1, w2, b2, *, act: str, residual: bool, p1: float = 0.0, seed1: int = 0,
               p2: float = 0.0, seed2: int = 0, h_out: Optional[torch.Tensor] = None,
               relu_bits_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[x +] drop2(act(x W1^T + b1) W2^T + b2)`` in one kernel; the ``[rows, ffn]`` hidden matrix never reaches HBM
    unless ``h_out`` asks for it as a side output (then it is written once and not read back; ``relu_bits_out`` receives
    one bit per hidden element, value > 0).  No autograd.  Shapes: see ``onchip_supported``."""
    from . import _ext
    ext = _ext.load()

    def f32(b):
        if b is None:
            return None
        b = b.detach().float().contiguous()
        return b.clone() if b.data_ptr() % 16 else b
    y = ext.ffn_fused_fwd(x, gemm.operand_copy(w1, x.dtype), f32(b1), gemm.operand_copy(w2, x.dtype), f32(b2),
                          gemm.ACT[act], bool(residual), float(p1), int(seed1), float(p2), int(seed2),
                          gemm.status_tensor(x.device), h_out, relu_bits_out)
    _ext.count_launches(1)
    return y


def onchip_supported(x: torch.Tensor, w1, w2) -> bool:
    # bf16 only: the fp16 instantiation of the kernel exists but is not covered by the GPU tests
    if not (x.is_cuda and x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
            and (x.stride(0) * 2) % 16 == 0 and x.data_ptr() % 16 == 0 and x.size(0) > 0):
        return False
    from . import _ext
    return bool(_ext.load().ffn_fused_supported(x.size(0), x.size(1), w1.size(0))) and tuple(w2.shape) == (x.size(1), w1.size(0))


class _FusedFFNRelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, p1, p2, seed1, seed2, slot=None):
        w1h, w2h = gemm.operand_copy(w1, x.dtype), gemm.operand_copy(w2, x.dtype)
        # one bit per hidden element (h > 0, after dropout): the backward masks with it instead of re-reading h
        bits = torch.empty((w1.size(0) // 16, x.size(0)), dtype=torch.int16, device=x.device) if (USE_RELU_BITS and w1.size(0) % 16 == 0) else None
        # residual FFN (the residual is the input itself): backward adds the pass-through gradient in the epilogue of
        # the input-gradient GEMM instead of leaving a separate full-size addition to autograd
        res_is_x = residual is not None and residual.data_ptr() == x.data_ptr() and residual.shape == x.shape \
            and residual.stride() == x.stride()
        if ONCHIP_FFN_TRAIN and bits is not None and (residual is None or res_is_x) and onchip_supported(x, w1, w2):
            # one kernel: the hidden matrix is written once as a side output and never read back by the forward pass
            h = torch.empty((x.size(0), w1.size(0)), dtype=x.dtype, device=x.device)
            y = ffn_onchip(x, w1, b1, w2, b2, act="relu", residual=res_is_x, p1=p1, seed1=seed1, p2=p2, seed2=seed2,
                           h_out=h, relu_bits_out=bits)
        else:
            h = gemm.gemm_tn(x, w1h, b1, "relu", dropout_p=p1, dropout_seed=seed1, relu_bits_out=bits)
            y = gemm.gemm_tn(h, w2h, b2, None, dropout_p=p2, dropout_seed=seed2, residual=residual)
        ctx.weights = (w1, w2)
        ctx.save_for_backward(x, h, bits if bits is not None else x.new_empty(0))
        ctx.cfg = (float(p1), float(p2), int(seed1), int(seed2), residual is not None, w1.dtype,
                   b1 is not None, b2 is not None, res_is_x)
        ctx.slot = slot
        return y

    @staticmethod
    def backward(ctx, dy):
        x, h, bits = ctx.saved_tensors
        w1t = gemm.operand_copy(ctx.weights[0], x.dtype, transpose=True)
        w2t = gemm.operand_copy(ctx.weights[1], x.dtype, transpose=True)
        p1, p2, seed1, seed2, has_res, wdtype, has_b1, has_b2, res_is_x = ctx.cfg
        handed = ctx.slot.take(dy) if ctx.slot is not None else None
        dy = dy.contiguous()
        g2 = hash_dropout(dy, seed2, p2) if p2 > 0 else dy
        scale = 1.0 / (1.0 - p1) if p1 > 0 else 1.0
        if bits.numel():
            dh = gemm.gemm_tn(g2, w2t, relu_bits_in=bits, out_scale=scale)
        else:
            dh = gemm.gemm_tn(g2, w2t, relu_mask=h, out_scale=scale)
        dx = gemm.gemm_tn(dh, w1t, residual=dy if res_is_x else None)
        # weight gradients on the tcgen05 reduction kernel; a bias gradient rides along as one more accumulator column
        # unless the LayerNorm behind this block already produced it (handed) or the kernel has no column to spare
        need_db2 = has_b2 and not (handed is not None and p2 == 0)
        dw2, db2 = gemm.weight_grad(g2, h, need_db2)
        dw1, db1 = gemm.weight_grad(dh, x, has_b1)
        dw2, dw1 = dw2.to(wdtype), dw1.to(wdtype)
        if has_b2:
            db2 = (db2 if need_db2 else handed).to(wdtype)
        db1 = db1.to(wdtype) if has_b1 else None
        dres = dy if (has_res and not res_is_x) else None
        return dx, dw1, db1, dw2, db2, dres, None, None, None, None, None


class _FusedFFNGelu(torch.autograd.Function):
    """GELU form (Graphormer).  Forward: GEMM (bias) -> z, one pass ``h = dropout(gelu(z))``, GEMM (bias, dropout,
    residual).  Backward: the hidden gradient ``dz = (g W2) * keep / (1 - p1) * gelu'(z)`` comes out of the GEMM's
    epilogue (dropout mask regenerated from its seed, derivative evaluated on the saved pre-activation), so neither the
    GELU derivative nor the dropout mask is a separate pass over the ``[rows, ffn]`` gradient."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, p1, p2, seed1, seed2, slot=None):
        from .norm import gelu_dropout
        w1h, w2h = gemm.operand_copy(w1, x.dtype), gemm.operand_copy(w2, x.dtype)
        z = gemm.gemm_tn(x, w1h, b1)
        h = gelu_dropout(z, seed1, p1)
        y = gemm.gemm_tn(h, w2h, b2, None, dropout_p=p2, dropout_seed=seed2, residual=residual)
        ctx.weights = (w1, w2)
        ctx.save_for_backward(x, z, h)
        res_is_x = residual is not None and residual.data_ptr() == x.data_ptr() and residual.shape == x.shape \
            and residual.stride() == x.stride()
        ctx.cfg = (float(p1), float(p2), int(seed1), int(seed2), residual is not None, w1.dtype,
                   b1 is not None, b2 is not None, res_is_x)
        ctx.slot = slot
        return y

    @staticmethod
    def backward(ctx, dy):
        x, z, h = ctx.saved_tensors
        w1t = gemm.operand_copy(ctx.weights[0], x.dtype, transpose=True)
        w2t = gemm.operand_copy(ctx.weights[1], x.dtype, transpose=True)
        p1, p2, seed1, seed2, has_res, wdtype, has_b1, has_b2, res_is_x = ctx.cfg
        handed = ctx.slot.take(dy) if ctx.slot is not None else None
        dy = dy.contiguous()
        g2 = hash_dropout(dy, seed2, p2) if p2 > 0 else dy
        dz = gemm.gemm_tn(g2, w2t, dropout_p=p1, dropout_seed=seed1, gelu_grad_of=z)
        dx = gemm.gemm_tn(dz, w1t, residual=dy if res_is_x else None) if ctx.needs_input_grad[0] else None
        need_db2 = has_b2 and not (handed is not None and p2 == 0)
        dw2, db2 = gemm.weight_grad(g2, h, need_db2)
        dw1, db1 = gemm.weight_grad(dz, x, has_b1)
        dw2, dw1 = dw2.to(wdtype), dw1.to(wdtype)
        if has_b2:
            db2 = (db2 if need_db2 else handed).to(wdtype)
        db1 = db1.to(wdtype) if has_b1 else None
        dres = dy if (has_res and not res_is_x) else None
        return dx, dw1, db1, dw2, db2, dres, None, None, None, None, None


def fused_ffn(x: torch.Tensor, w1, b1, w2, b2, *, act: str = "relu", residual: Optional[torch.Tensor] = None,
              p1: float = 0.0, p2: float = 0.0, training: bool = True, out_grad_colsum=None) -> torch.Tensor:
    """2-D ``x`` ``[rows, h]``; ``residual`` is added last (pass ``x`` for a residual FFN).  ``out_grad_colsum`` is an
    optional ``ops.norm.ColsumSlot`` filled by the LayerNorm that consumes the result (bias gradient for free)."""
    if not training:
        p1 = p2 = 0.0
    n1, k1 = w1.shape
    ok = x.is_cuda and x.stride(1) == 1 and gemm.supported(x.size(0), n1, k1, x.dtype) \
        and gemm.supported(x.size(0), w2.size(0), w2.size(1), x.dtype)
    res_is_x = residual is not None and residual.data_ptr() == x.data_ptr() and residual.shape == x.shape \
        and residual.stride() == x.stride()
    forward_only = not torch.is_grad_enabled() and (not training or ONCHIP_FFN == "all")
    if ok and forward_only and ONCHIP_FFN != "0" and act in ("relu", "gelu") and (residual is None or res_is_x) \
            and onchip_supported(x, w1, w2):
        # same order of seed draws as the two-GEMM forms below, so that a recomputation reproduces the masks
        s1 = new_seed() if p1 > 0 else 0
        s2 = new_seed() if p2 > 0 else 0
        return ffn_onchip(x, w1, b1, w2, b2, act=act, residual=res_is_x, p1=p1, seed1=s1, p2=p2, seed2=s2)
    if ok and act == "relu":
        return _FusedFFNRelu.apply(x, w1, b1, w2, b2, residual, p1, p2, new_seed() if p1 > 0 else 0,
                                   new_seed() if p2 > 0 else 0, out_grad_colsum)
    if ok and act == "gelu":
        return _FusedFFNGelu.apply(x, w1, b1, w2, b2, residual, p1, p2, new_seed() if p1 > 0 else 0,
                                   new_seed() if p2 > 0 else 0, out_grad_colsum)
    hdn = F.linear(x, w1.to(x.dtype), None if b1 is None else b1.to(x.dtype))
    hdn = F.relu(hdn) if act == "relu" else F.gelu(hdn)
    hdn = F.dropout(hdn, p1, training and p1 > 0)
    y = F.dropout(F.linear(hdn, w2.to(x.dtype), None if b2 is None else b2.to(x.dtype)), p2, training and p2 > 0)
    return y if residual is None else residual + y
