"""AdamW with global-norm clipping on the gradient reducer's flat buckets.

Parameters are re-pointed into one flat fp32 buffer per bucket (their ``.grad`` already lives in the matching
flat gradient bucket), so a whole optimizer step is: one sum-of-squares kernel and one AdamW kernel per bucket.
The clip coefficient ``min(1, max_norm / (||g|| + 1e-6))`` is evaluated inside the AdamW kernel from the
device-resident norm, so the step never synchronises with the host.  Same update rule as
``torch.optim.AdamW`` preceded by ``clip_grad_norm_`` (main_node_fullgraph_sp.py:1284-1293 in the reference)."""
from __future__ import annotations

from typing import List

import torch

from . import _ext


class FlatAdamW(torch.optim.Optimizer):
    def __init__(self, buckets, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, max_grad_norm: float = 1.0,
                 cuda_graph: bool = False):
        params = [p for b in buckets for p in b.params]
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.buckets = buckets
        self.max_grad_norm = float(max_grad_norm)
        self._step = 0
        self._flat_p: List[torch.Tensor] = []
        self._m: List[torch.Tensor] = []
        self._v: List[torch.Tensor] = []
        for b in buckets:
            flat = torch.zeros_like(b.flat)
            for p, off in zip(b.params, b.offsets):
                n = p.numel()
                flat[off:off + n].copy_(p.data.reshape(-1))
                p.data = flat[off:off + n].view_as(p)
            self._flat_p.append(flat)
            self._m.append(torch.zeros_like(flat))
            self._v.append(torch.zeros_like(flat))
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=buckets[0].flat.device)
        # --cuda_graph: the whole step (zero, sum of squares, AdamW per bucket) is captured once and replayed; the
        # step-dependent scalars travel through a 3-float device buffer refreshed from pinned memory before each replay
        self._use_graph = bool(cuda_graph) and buckets[0].flat.is_cuda
        self._graph = None
        if self._use_graph:
            self._hyper = torch.zeros(4, dtype=torch.float32, device=buckets[0].flat.device)
            self._hyper_host = torch.zeros(8, 4, dtype=torch.float32).pin_memory()   # ring: a slot is rewritten 8 steps later

    @torch.no_grad()
    def step(self, closure=None):
        ext = _ext.load()
        self._step += 1
        from .gemm import weights_changed
        weights_changed()                              # the kernels below rewrite the parameters' storage directly
        g0 = self.param_groups[0]
        lr, (b1, b2), eps, wd = g0["lr"], g0["betas"], g0["eps"], g0["weight_decay"]
        clip = self.max_grad_norm > 0
        if self._use_graph:
            slot = self._hyper_host[self._step % self._hyper_host.size(0)]
            slot[0] = float(lr)
            slot[1] = 1.0 - float(b1) ** self._step
            slot[2] = (1.0 - float(b2) ** self._step) ** 0.5
            self._hyper.copy_(slot, non_blocking=True)
            if self._graph is None:
                self._capture(ext, b1, b2, eps, wd, clip)
            self._graph.replay()
            _ext.count_launches(len(self.buckets) * (2 if clip else 1))
            return
        sumsq = self._fused_norm_parts() if clip else None
        fused = sumsq is not None
        if clip and not fused:
            self._sumsq.zero_()
            for b in self.buckets:
                ext.grad_sumsq(b.flat, self._sumsq)
            sumsq = self._sumsq
        self._last_sumsq = sumsq
        for b, p, m, v in zip(self.buckets, self._flat_p, self._m, self._v):
            ext.adamw_flat(p, b.flat, m, v, int(b.n_valid), float(lr), float(b1), float(b2), float(eps), float(wd),
                           int(self._step), sumsq, self.max_grad_norm)
        _ext.count_launches(len(self.buckets) * (2 if (clip and not fused) else 1))

    def _fused_norm_parts(self):
        """The gradient all-reduce of this step left the squared norm of every reduced slice with every rank
        (``parallel.symm.bucket_all_reduce_mean``): clip on their sum, no further pass over the gradients."""
        norms = [getattr(b, "norm", None) for b in self.buckets]
        if norms and all(n is not None and n["ready"] for n in norms):
            return norms[0]["all"]
        return None

    def _launch_dev(self, ext, b1, b2, eps, wd, clip) -> None:
        if clip:
            self._sumsq.zero_()
            for b in self.buckets:
                ext.grad_sumsq(b.flat, self._sumsq)
        for b, p, m, v in zip(self.buckets, self._flat_p, self._m, self._v):
            ext.adamw_flat_dev(p, b.flat, m, v, int(b.n_valid), float(b1), float(b2), float(eps), float(wd), self._hyper,
                               self._sumsq if clip else None, self.max_grad_norm)

    def _capture(self, ext, b1, b2, eps, wd, clip) -> None:
        """Record the step's launches into a CUDA graph (betas, eps, weight decay and the clip threshold are baked in;
        lr and the bias corrections come from ``self._hyper``).  Capture does not execute, so nothing is applied twice."""
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(self._hyper.device)
        side.wait_stream(torch.cuda.current_stream(self._hyper.device))
        with torch.cuda.stream(side):
            # thread-local capture mode: the look-ahead graph builder may allocate on its own thread meanwhile
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                self._launch_dev(ext, b1, b2, eps, wd, clip)
        torch.cuda.current_stream(self._hyper.device).wait_stream(side)
        self._graph = graph

    def grad_norm(self) -> torch.Tensor:
        """Device tensor holding the global gradient norm of the last step."""
        src = getattr(self, "_last_sumsq", None)
        return (self._sumsq if src is None else src.sum().reshape(1)).sqrt()

    def state_dict(self):
        return {"step": self._step, "m": [t.cpu() for t in self._m], "v": [t.cpu() for t in self._v],
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd):
        self._step = int(sd["step"])
        for dst, src in zip(self._m, sd["m"]):
            dst.copy_(src)
        for dst, src in zip(self._v, sd["v"]):
            dst.copy_(src)
        for g, s in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(s)
