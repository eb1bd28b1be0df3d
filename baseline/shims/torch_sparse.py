"""Minimal pure-PyTorch stand-in for ``torch_sparse.SparseTensor`` (coalesce + csr) used by the reference's
random-walk CSR builder (gt_sp/utils.py:926-931)."""
import torch


class SparseTensor:
    def __init__(self, row=None, col=None, value=None, sparse_sizes=None, **kw):
        self.row, self.col, self.sizes = row.to(torch.long), col.to(torch.long), sparse_sizes

    def coalesce(self):
        n = int(self.sizes[1])
        key = torch.unique(self.row * n + self.col)
        out = SparseTensor(torch.div(key, n, rounding_mode="floor"), key % n, sparse_sizes=self.sizes)
        return out

    def csr(self):
        n = int(self.sizes[0])
        order = torch.argsort(self.row * int(self.sizes[1]) + self.col)
        row, col = self.row[order], self.col[order]
        rowptr = torch.zeros(n + 1, dtype=torch.long, device=row.device)
        rowptr[1:] = torch.cumsum(torch.bincount(row, minlength=n), 0)
        return rowptr, col, None


def matmul(*a, **k):
    raise NotImplementedError("torch_sparse.matmul is not used on the benchmarked path")
