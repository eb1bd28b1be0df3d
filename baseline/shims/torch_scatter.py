"""Minimal pure-PyTorch stand-in for the ``torch_scatter`` wheel (not installable offline for this torch
build).  Used only by the baseline harness to run the reference; never imported by the product."""
import torch


def scatter(src, index, dim=0, out=None, dim_size=None, reduce="add"):
    assert dim == 0 and reduce in ("add", "sum"), "shim covers the reference's call sites only"
    index = index.to(torch.long)
    if out is None:
        size = int(dim_size if dim_size is not None else (int(index.max()) + 1 if index.numel() else 0))
        out = src.new_zeros((size,) + tuple(src.shape[1:]))
    return out.index_add_(0, index, src.to(out.dtype))
