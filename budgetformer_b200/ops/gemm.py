"""Linear layers on the tcgen05 GEMMs (``csrc/gemm_tcgen05.cu``, ``csrc/gemm_dw_tcgen05.cu``).

``gemm_tn`` is the raw call ``C = A @ W.T`` with the fused epilogue; ``weight_grad`` is ``dW = dY^T X`` together
with the bias gradient (column sums of ``dY``) from one pass over the operands; ``fused_linear`` is the autograd
function used by the models on B200: forward, input gradient and weight gradient all run on the tcgen05 kernels.
Shapes the kernels do not cover (features not a multiple of 8 / 16, fp32 operands) fall back to PyTorch."""
from __future__ import annotations

from typing import Optional

import torch

from . import _ext

ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2}
_STATUS = {}

# ---- operand copies of the weights ------------------------------------------------------------------------
# The kernels take weights in the activation dtype (and the input-gradient GEMM takes them transposed).  Those copies
# only change when the weights do: they are kept per parameter and rebuilt when the parameter's version counter moves
# (in-place updates by PyTorch optimizers, ``load_state_dict``) or when an optimizer that writes the storage directly
# announces a step through ``weights_changed()`` (``ops.optim.FlatAdamW``).
_WEIGHT_GEN = 0
_WEIGHT_COPIES = {}


def weights_changed() -> None:
    global _WEIGHT_GEN
    _WEIGHT_GEN += 1


def operand_copy(weight: torch.Tensor, dtype, transpose: bool = False, index: Optional[torch.Tensor] = None,
                 tag: str = "") -> torch.Tensor:
    """``weight[index].to(dtype)`` (``.t()`` when ``transpose``), contiguous, cached until the weight changes."""
    key = (id(weight), dtype, bool(transpose), tag)
    stamp = (_WEIGHT_GEN, weight._version, weight.data_ptr())
    hit = _WEIGHT_COPIES.get(key)
    if hit is not None and hit[0] == stamp and hit[2]() is weight:
        return hit[1]
    import weakref
    w = weight.detach()
    if index is not None:
        w = w[index]
    w = w.to(dtype)
    w = w.t().contiguous() if transpose else w.contiguous()
    _WEIGHT_COPIES[key] = (stamp, w, weakref.ref(weight))
    if len(_WEIGHT_COPIES) > 4096:                     # parameters of discarded models: drop what is dead
        for k in [k for k, v in _WEIGHT_COPIES.items() if v[2]() is None]:
            del _WEIGHT_COPIES[k]
    return w


def status_tensor(device) -> torch.Tensor:
    """Per-device int32[4] written by kernels whose bounded waits expired (0 = healthy)."""
    key = torch.device(device).index or 0
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _STATUS[key] = t
    return t


def check_status(device) -> None:
    """Host read of the status word; raises if any kernel gave up waiting."""
    t = _STATUS.get(torch.device(device).index or 0)
    if t is not None:
        code = int(t[0].item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"a device-side bounded wait expired (status {code}); results of that launch are invalid")


def supported(m: int, n: int, k: int, dtype) -> bool:
    return dtype in (torch.bfloat16, torch.float16) and m > 0 and k % 8 == 0 and k >= 16 and n % 16 == 0 and n >= 16


def gemm_tn(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None,
            dropout_p: float = 0.0, dropout_seed: int = 0, residual: Optional[torch.Tensor] = None,
            relu_mask: Optional[torch.Tensor] = None, out_scale: float = 1.0, out: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None, relu_bits_out: Optional[torch.Tensor] = None,
            relu_bits_in: Optional[torch.Tensor] = None, gelu_grad_of: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(dropout(a @ w.T * out_scale + bias)) [masked] + residual`` in one kernel.  ``relu_bits_out`` (int16
    ``[N / 16, M]``) receives one bit per element (result > 0); ``relu_bits_in`` zeroes the result where its bit is clear;
    ``gelu_grad_of`` (``[M, N]`` pre-activations) multiplies the result by ``gelu'(z)`` after the dropout mask - the
    hidden gradient of a GELU feed-forward block straight out of the GEMM."""
    if gelu_grad_of is not None:
        assert relu_mask is None, "one mask operand per call"
        relu_mask = gelu_grad_of
    ext = _ext.load()
    m, n = a.size(0), w.size(0)
    fp32_out = (out_dtype or (out.dtype if out is not None else a.dtype)) == torch.float32
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32 if fp32_out else a.dtype, device=a.device)
    if m == 0:
        return out
    if bias is not None:
        bias = bias.float().contiguous()
        if bias.data_ptr() % 16:                      # the epilogue reads the bias with 16-byte loads
            bias = bias.clone()
    ext.gemm_tn(a, w, bias, ACT[act], float(dropout_p), int(dropout_seed),
                residual, relu_mask, float(out_scale), bool(fp32_out), [out.data_ptr()], 0, out.stride(0),
                status_tensor(a.device), relu_bits_out, relu_bits_in, 1 if gelu_grad_of is not None else 0)
    _ext.count_launches(1)
    return out


def weight_grad(dy: torch.Tensor, x: torch.Tensor, want_bias: bool = False):
    """``(dy.T @ x, dy.sum(0) or None)`` in fp32.  One tcgen05 kernel reads both operands once (MN-major tiles straight
    from the row-major matrices) and leaves per-row-slice partial tiles that a second kernel adds in a fixed order; the
    bias gradient is one more accumulator column of the same kernel.  Falls back to PyTorch for shapes outside the
    kernel's reach (features not a multiple of 8, operands that are not 16-bit)."""
    ext = _ext.load()
    m, n, k = dy.size(0), dy.size(1), x.size(1)
    ok = (dy.is_cuda and dy.dtype in (torch.bfloat16, torch.float16) and x.dtype == dy.dtype and m > 0
          and dy.stride(1) == 1 and x.stride(1) == 1 and (dy.stride(0) * 2) % 16 == 0 and (x.stride(0) * 2) % 16 == 0
          and dy.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0 and ext.gemm_dw_supported(m, n, k, False))
    if not ok:
        dw = torch.matmul(dy.t(), x).float()
        return dw, (dy.float().sum(0) if want_bias else None)
    fused_bias = bool(want_bias and ext.gemm_dw_supported(m, n, k, True))
    out = ext.gemm_dw(dy, x, fused_bias, status_tensor(dy.device))
    _ext.count_launches(3 if fused_bias else 2)
    db = out[1] if fused_bias else None
    if want_bias and db is None:
        from .norm import column_sum
        db = column_sum(dy)
    return out[0], db


def hash_keep_mask(seed: int, rows: int, cols: int, p: float, device) -> torch.Tensor:
    """The epilogue's dropout keep mask, restated in PyTorch (tests and the fallback path)."""
    r = torch.arange(rows, device=device, dtype=torch.int64)[:, None]
    c = torch.arange(cols, device=device, dtype=torch.int64)[None, :]
    x = (r * 0x9E3779B1 + c * 0x85EBCA77 + (int(seed) & 0xFFFFFFFF)) & 0xFFFFFFFF
    x = ((x ^ (x >> 16)) * 0x7FEB352D) & 0xFFFFFFFF
    x = ((x ^ (x >> 15)) * 0x846CA68B) & 0xFFFFFFFF
    x = x ^ (x >> 16)
    return x >= int(p * 4294967296.0)


class _FusedLinear(torch.autograd.Function):
    """y = residual + dropout(x W^T + b): one GEMM forward; input-gradient GEMM + weight-gradient GEMM backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, dropout_p, dropout_seed):
        w16 = operand_copy(weight, x.dtype)
        y = gemm_tn(x, w16, bias, None, dropout_p=dropout_p, dropout_seed=dropout_seed, residual=residual)
        ctx.cfg = (residual is not None, float(dropout_p), int(dropout_seed), weight.dtype, bias is not None)
        ctx.weight = weight
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .norm import hash_dropout
        (x,) = ctx.saved_tensors
        has_res, p, seed, wdtype, has_bias = ctx.cfg
        dy = dy.contiguous()
        g = hash_dropout(dy, seed, p) if p > 0 else dy
        # dx = g @ W, expressed as g @ (W^T)^T; skipped for leaf inputs such as the feature matrix
        dx = None
        if ctx.needs_input_grad[0]:
            if supported(g.size(0), x.size(1), g.size(1), g.dtype):
                dx = gemm_tn(g, operand_copy(ctx.weight, x.dtype, transpose=True))
            else:                                      # fewer than 16 outputs (never through readout_linear, which pads)
                dx = torch.matmul(g, operand_copy(ctx.weight, x.dtype))
        dw, db = weight_grad(g, x, has_bias)
        return dx, dw.to(wdtype), (db.to(wdtype) if has_bias else None), (dy if has_res else None), None, None


def fused_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, dropout_p: float = 0.0, dropout_seed: int = 0) -> torch.Tensor:
    """2-D ``x``: ``residual + dropout(x @ weight.T + bias)``.  tcgen05 kernel when shape/dtype allow, else PyTorch."""
    if x.is_cuda and supported(x.size(0), weight.size(0), x.size(1), x.dtype) and x.stride(1) == 1 \
            and (x.stride(0) * 2) % 16 == 0 and x.data_ptr() % 16 == 0:
        return _FusedLinear.apply(x, weight, bias, residual, dropout_p, dropout_seed)
    y = torch.nn.functional.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    if dropout_p > 0:
        keep = hash_keep_mask(dropout_seed, y.size(0), y.size(1), dropout_p, y.device)
        y = torch.where(keep, y / (1.0 - dropout_p), torch.zeros_like(y))
    return y if residual is None else y + residual


def readout_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight.T + bias`` for the small output layers (h -> classes).  The tcgen05 kernels want the output width
    to be a multiple of 16: a narrower layer is run with zero rows appended to the weight (and zeros to the bias) and
    the extra columns are cut off again, so its forward, input gradient and weight gradient stay off the library GEMM
    (the kernels reduce over as few as 16 features: a narrower operand is one mostly zero-filled 64-wide panel).
    Inputs the kernels cannot take (fp32 activations, fewer than 16 input features) use ``torch.nn.functional.linear``."""
    n, k = weight.shape
    usable = (x.is_cuda and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and k >= 16 and k % 8 == 0
              and x.stride(1) == 1 and (x.stride(0) * 2) % 16 == 0 and x.data_ptr() % 16 == 0)
    if not usable:
        return torch.nn.functional.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    pad = (-n) % 16
    if pad == 0:
        return fused_linear(x, weight, bias)
    w = torch.cat([weight, weight.new_zeros(pad, k)], 0)
    b = None if bias is None else torch.cat([bias, bias.new_zeros(pad)], 0)
    return fused_linear(x, w, b)[:, :n]
