"""Fused sequence-parallel attention block for B200.

Per encoder layer the portable path runs 3 projection GEMMs, 3 all-to-alls (each with two staging
copies), the edge attention, a fourth all-to-all and the output projection
(gt_sp/layer.py:264-280, models/gt_dist_node_level.py:558-560,650-653).  Here:

``QKV push``    one tcgen05 GEMM over the packed ``[Wq;Wk;Wv]`` (rows permuted so that the columns of one
                destination rank are contiguous) whose epilogue stores every tile straight into the owning
                rank's packed ``[N, 3*h/P]`` buffer over NVLink — the nodes->heads all-to-all *is* the epilogue;
``attention``   the edge-attention kernels read q|k|v from that packed buffer and write the context into a
                second symmetric buffer;
``ctx``         heads->nodes, two forms.  *Routed stores* (default where a rank's slice of a row is at least 128 bytes
                and the model has no virtual-node rows): the
                attention kernels store every context row a second time, straight into the buffer of the rank that
                owns the node (one slab per source rank), so the all-to-all rides on the attention kernel's stores
                and is hidden behind its gathers; the output-projection GEMM then gathers its A operand from the
                local slabs.  *Pull*: the GEMM's loader warps fetch this rank's rows of every peer's context from the
                peers' memory while the previous tile is multiplied.  Either way bias, dropout and residual are fused
                in the GEMM's epilogue and a local copy of the gathered rows is written from the same shared-memory
                stages only when the backward pass will need it;
backward        mirrors it: the d(context) GEMM pushes to the head owners, the attention backward writes
                dq|dk|dv packed - routed to the row owners' slabs, or locally for the pull form - and the
                input-gradient GEMM gathers its rows of every source's dq|dk|dv the same way (keeping the local copy
                that the weight-gradient GEMM reads).

Device-side barriers (bounded spins) order producers and consumers; no host synchronisation and no NCCL
call happens inside a layer.
"""
from __future__ import annotations

import os
import types
from typing import List, Optional

import torch
from torch.utils.checkpoint import checkpoint

from ..graph.attn_graph import AttnGraph, as_attn_graph
from ..parallel import symm
from . import _ext, gemm
from ..utils import debug
from .edge_attention import _VARIANTS
from .ffn import fused_ffn
from .norm import ColsumSlot, batch_norm, hash_dropout, layer_norm, new_seed


# context dropout inside the attention kernel's store (off: a separate hash_dropout pass over the pulled context)
FUSE_CONTEXT_DROPOUT = True
# heads->nodes by routed stores of the attention kernels (off, narrow row slices, or a model with virtual-node rows:
# the GEMMs pull); BF_ROUTE_ATTENTION_ROWS=0 switches the form off, =force takes it whatever the row width
ROUTE_ATTENTION_ROWS = os.environ.get("BF_ROUTE_ATTENTION_ROWS", "1") != "0"


class SPContext:
    """Symmetric buffers and geometry shared by all layers of one model."""

    def __init__(self, group, device, world: int, rows_local: int, hidden: int, heads: int, n_layers: int, dtype,
                 token_rows: Optional[List[int]] = None, routed: Optional[bool] = None):
        self.sw = symm.get_world(group, device)
        # seed shared by all ranks for masks that one rank generates and another regenerates (set by the trainer every
        # step from the run seed and the epoch; None = not set)
        self.step_seed: Optional[int] = None
        self._packs = {}                                  # layer -> (stamp, packed W, packed bias, packed W transposed)
        self.P, self.rank = self.sw.world, self.sw.rank
        assert self.P == world
        self.rows_local, self.total_rows = int(rows_local), int(rows_local) * self.P
        self.h, self.H = int(hidden), int(heads)
        self.hl_heads = self.H // self.P
        self.hn = self.h // self.H
        self.hl = self.hl_heads * self.hn                 # columns of one head slice
        self.dtype = dtype
        self.token_rows = token_rows
        # A node's packed row is k | v | q: the attention kernels gather k and v of a key together, so the pair comes
        # first, and the row pitch is padded to a multiple of 128 bytes so that a narrow pair (64 bytes with one head of
        # 16 per rank) never straddles two DRAM bursts.
        self.qkv_ld = (3 * self.hl + 63) // 64 * 64
        self.qkv = [self.sw.alloc((self.total_rows, self.qkv_ld), dtype) for _ in range(n_layers)]
        self.ctx = [self.sw.alloc((self.total_rows, self.hl), dtype) for _ in range(n_layers)]
        self.dqkv = self.sw.alloc((self.total_rows, self.qkv_ld), dtype)
        self.dctx = self.sw.alloc((self.total_rows, self.hl), dtype)
        # Routed form: ``ctx[l]`` and ``dqkv`` are indexed (source rank, row of this rank) - P slabs of rows_local rows
        # that the peers' attention kernels fill - instead of (global row); the head owner keeps its own context of all
        # rows in a plain local tensor for its backward pass.
        # Measured on the 2.9 M-node benchmark (GT, h = 128): with 128-byte rows per rank (2 ranks) the routed form is
        # 0.9 ms per step faster than the pull form (43.5 against 44.5 ms); with 64-byte rows (4 ranks) the attention
        # kernels' scattered remote stores cost more than the pulls they replace (31.1 against 29.4 ms).  Default: routed
        # when a rank's slice of a row is at least one 128-byte line.
        wide = self.hl * torch.empty((), dtype=dtype).element_size() >= 128
        if os.environ.get("BF_ROUTE_ATTENTION_ROWS", "") == "force":
            wide = True
        want = (ROUTE_ATTENTION_ROWS and wide) if routed is None else bool(routed)
        self.routed = bool(want and self.P > 1 and token_rows is None and self.hl % 8 == 0)
        self.ctx_local = ([torch.empty((self.total_rows, self.hl), dtype=dtype, device=device) for _ in range(n_layers)]
                          if self.routed else None)
        # row permutation of the packed [Wq;Wk;Wv]: destination-rank major, then k|v|q, then head columns
        idx = []
        for r in range(self.P):
            for part in (1, 2, 0):
                base = part * self.h + r * self.hl
                idx.extend(range(base, base + self.hl))
        self.perm = torch.tensor(idx, dtype=torch.long, device=device)
        self.inv_perm = torch.empty_like(self.perm)
        self.inv_perm[self.perm] = torch.arange(3 * self.h, device=device)

    @property
    def row0(self) -> int:
        return self.rank * self.rows_local

    def slab_ptrs(self, buf, row_bytes: int) -> List[int]:
        """Base address of every source rank's slab inside this rank's own copy of a routed buffer."""
        base = buf.tensor.data_ptr()
        return [base + s * self.rows_local * row_bytes for s in range(self.P)]

    def route(self, buf, ld: int, extra=()) -> List[int]:
        """Route descriptor of the attention bindings: rows per destination, this rank's slab, row stride, ``extra``
        header fields, then every destination's buffer base."""
        return [self.rows_local, self.rank * self.rows_local, int(ld)] + [int(v) for v in extra] + [int(p) for p in buf.ptrs]

    def packed_projection(self, layer: int, wq, wk, wv, bq, bk, bv, dtype):
        """``[Wq; Wk; Wv]`` with its rows in the order of ``perm`` (and the bias likewise), in the activation dtype.  The
        pack is rebuilt only when one of the six tensors changed since it was made."""
        parts = [t for t in (wq, wk, wv, bq, bk, bv) if t is not None]
        stamp = (gemm._WEIGHT_GEN, dtype) + tuple((t._version, t.data_ptr()) for t in parts)
        hit = self._packs.get(layer)
        if hit is None or hit[0] != stamp:
            w = torch.cat([wq, wk, wv], 0).detach().to(dtype)[self.perm].contiguous()
            b = None if bq is None else torch.cat([bq, bk, bv], 0).detach().float()[self.perm].contiguous()
            hit = self._packs[layer] = (stamp, w, b, w.t().contiguous())
        return hit[1], hit[2]

    def transposed_projection(self, layer: int, w: torch.Tensor) -> torch.Tensor:
        hit = self._packs.get(layer)
        return hit[3] if (hit is not None and hit[1] is w) else w.t().contiguous()

    def split_packed(self, t: torch.Tensor):
        """(q, k, v) views ``[rows, heads, hn]`` of a packed ``[rows, qkv_ld]`` buffer (column order k | v | q)."""
        r, hl = t.size(0), self.hl
        part = lambda i: t[:, i * hl:(i + 1) * hl].view(r, self.hl_heads, self.hn)
        return part(2), part(0), part(1)

    def shared_seed(self, layer: int, tag: int) -> Optional[int]:
        """31-bit seed every rank derives identically for (step, layer, purpose), or None when no step seed is set.
        A mask written on one rank and regenerated on another must not depend on each rank's private RNG state."""
        if self.step_seed is None:
            return None
        x = (int(self.step_seed) * 0x9E3779B1 + (int(layer) + 1) * 0x85EBCA77 + (int(tag) + 1) * 0xC2B2AE3D) & 0xFFFFFFFF
        x = ((x ^ (x >> 16)) * 0x7FEB352D) & 0xFFFFFFFF
        x = ((x ^ (x >> 15)) * 0x846CA68B) & 0xFFFFFFFF
        return (x ^ (x >> 16)) & 0x7FFFFFFF


# the pulled operand is fetched inside the GEMM (off: a separate peer-load gather kernel into a local matrix first)
FUSE_PULL = True


def _pull_gemm(src_ptrs, row0, src_ld, cols_per_src, rows, w, *, bias=None, residual=None, dropout_p=0.0, seed=0,
               keep_copy=False):
    """``y = drop(gathered @ w.T + bias) + residual`` where ``gathered[r, s*c:(s+1)*c] = src_s[row0 + r, :c]`` is pulled
    from the sources inside the kernel.  Returns ``(y, gathered or None)``."""
    ext = _ext.load()
    k = len(src_ptrs) * cols_per_src
    y = torch.empty((rows, w.size(0)), dtype=w.dtype, device=w.device)
    copy = torch.empty((rows, k), dtype=w.dtype, device=w.device) if keep_copy else None
    if bias is not None:
        bias = bias.float().contiguous()
        if bias.data_ptr() % 16:
            bias = bias.clone()
    ext.gemm_tn_pull(list(src_ptrs), int(row0), int(src_ld), int(cols_per_src), int(rows), w, copy, bias, float(dropout_p),
                     int(seed), residual, 1.0, y, gemm.status_tensor(w.device))
    _ext.count_launches(1)
    return y, copy


def _can_pull(sp, cols_per_src: int, rows: int, k: int, n: int, dtype) -> bool:
    return (FUSE_PULL and sp.P > 1 and cols_per_src % 16 == 0 and gemm.supported(rows, n, k, dtype)
            and _ext.load().gemm_supported(rows, n, k))


def _push_gemm(x, w, bias, dst_ptrs, row0, ldc, dropout_p=0.0, seed=0):
    ext = _ext.load()
    if bias is not None:
        bias = bias.float().contiguous()
        if bias.data_ptr() % 16:
            bias = bias.clone()
    ext.gemm_tn(x, w, bias, 0, float(dropout_p), int(seed), None, None,
                1.0, False, dst_ptrs, int(row0), int(ldc), gemm.status_tensor(x.device), None, None, 0)
    _ext.count_launches(1)


class _QKVPush(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wq, wk, wv, bq, bk, bv, sp: SPContext, layer: int, passthrough: bool = False):
        w, b = sp.packed_projection(layer, wq, wk, wv, bq, bk, bv, x.dtype)
        buf = sp.qkv[layer]
        _push_gemm(x, w, b, buf.ptrs, sp.row0, sp.qkv_ld)
        sp.sw.barrier(0)
        ctx.sp, ctx.has_bias, ctx.wdtype, ctx.layer = sp, bq is not None, wq.dtype, layer
        ctx.save_for_backward(x, w)
        if passthrough:
            # the input doubles as the residual of the output projection: handing it through this function routes the
            # residual's gradient back here, where the input-gradient GEMM adds it in its epilogue
            return buf.tensor.detach(), x
        return buf.tensor.detach()

    @staticmethod
    def backward(ctx, dqkv, dres=None):
        sp: SPContext = ctx.sp
        x, w = ctx.saved_tensors
        buf = sp.dqkv
        if dqkv.data_ptr() != buf.tensor.data_ptr():
            buf.tensor.copy_(dqkv)
        if dres is not None:
            dres = dres.to(x.dtype).contiguous()
        wt = sp.transposed_projection(ctx.layer, w)
        dx = None
        if _can_pull(sp, 3 * sp.hl, sp.rows_local, 3 * sp.h, sp.h, x.dtype):
            # dX = pulled(dq|dk|dv) W: the rows arrive inside the GEMM; the local copy feeds the weight gradient.
            # No barrier after the reads: the next writer of this buffer is the attention backward of the layer
            # below, and every rank reaches the barrier that follows that layer's d(context) push (or scatter) only
            # after this GEMM, so no peer can overwrite rows that are still being fetched.
            sp.sw.barrier(0)                                         # every rank's dq|dk|dv is complete
            # routed: the peers' attention kernels have delivered this rank's rows into its own slabs
            src = sp.slab_ptrs(buf, sp.qkv_ld * x.element_size()) if sp.routed else buf.ptrs
            dx, dloc = _pull_gemm(src, 0 if sp.routed else sp.row0, sp.qkv_ld, 3 * sp.hl, sp.rows_local, wt, residual=dres,
                                  keep_copy=True)
            if debug.enabled():
                sp.sw.barrier(0)                                     # poisoning below must wait for the peers' reads
        elif sp.P > 1:
            sp.sw.barrier(0)                                         # every rank's dq|dk|dv is complete
            dloc = torch.empty((sp.rows_local, 3 * sp.h), dtype=x.dtype, device=x.device)
            src = sp.slab_ptrs(buf, sp.qkv_ld * x.element_size()) if sp.routed else buf.ptrs
            _ext.load().peer_gather_cols(src, 0 if sp.routed else sp.row0, sp.rows_local, 3 * sp.hl * x.element_size(),
                                         sp.qkv_ld * x.element_size(), dloc)
            _ext.count_launches(1)
            sp.sw.barrier(0)                                         # all reads done before the buffer is reused
        else:
            dloc = buf.tensor[:, :3 * sp.h]
        if dx is None:
            dx = gemm.gemm_tn(dloc, wt, residual=dres)
        dw, db_src = gemm.weight_grad(dloc, x, ctx.has_bias)
        dw = dw[sp.inv_perm]
        if debug.enabled():
            debug.poison(buf.tensor)                  # consumed: whoever reads it before the next producer sees NaN
        dwq, dwk, dwv = (t.to(ctx.wdtype) for t in dw.split(sp.h, 0))
        if ctx.has_bias:
            db = db_src[sp.inv_perm]
            dbq, dbk, dbv = (t.to(ctx.wdtype) for t in db.split(sp.h, 0))
        else:
            dbq = dbk = dbv = None
        return dx, dwq, dwk, dwv, dbq, dbk, dbv, None, None, None


class _PackedEdgeAttention(torch.autograd.Function):
    """Edge attention on the packed q|k|v buffer; context and gradients live in symmetric buffers."""

    @staticmethod
    def forward(ctx, qkv, etable, graph: AttnGraph, sp: SPContext, layer: int, variant_id, dropout_p, seed,
                out_p=0.0, out_seed=0):
        ext = _ext.load()
        r, hlh, hn, hl = sp.total_rows, sp.hl_heads, sp.hn, sp.hl
        q, k, v = sp.split_packed(qkv)
        # routed: the kernel keeps this rank's copy of all rows in a local tensor (its backward reads it) and stores
        # every row a second time into the owner's slab of the symmetric buffer
        out = sp.ctx_local[layer] if sp.routed else sp.ctx[layer].tensor
        route = sp.route(sp.ctx[layer], hl) if sp.routed else []
        z = torch.empty((r, hlh), dtype=torch.float32, device=qkv.device)
        kmax = -1 if graph.max_degree is None else int(graph.max_degree)
        # dropout on the context (GT applies it before the output projection) is fused into the store: the mask of
        # element (row, c) is the one the owner of that row regenerates for (row - its first row, this rank's column)
        out_drop = [float(out_p), int(out_seed), int(sp.rows_local), int(sp.rank * hl)] if out_p > 0 else []
        ext.edge_attn_fwd(q, k, v, out.view(r, hlh, hn), z, graph.rowptr, graph.col, graph.etype, etable,
                          int(variant_id), float(dropout_p), int(seed), kmax, out_drop, route)
        _ext.count_launches(1)
        if sp.token_rows is not None and len(sp.token_rows) > 1:
            out[sp.token_rows[1:]] = out[sp.token_rows[0]].clone()  # copy_global_token0 (gt_sp/utils.py:2365-2386)
        ctx.sp, ctx.graph, ctx.layer = sp, graph, layer
        ctx.cfg = (int(variant_id), float(dropout_p), int(seed), etable is not None, kmax)
        ctx.out_drop = out_drop
        ctx.save_for_backward(qkv, z, etable if etable is not None else qkv.new_empty(0))
        return out.detach()

    @staticmethod
    def backward(ctx, dout):
        ext = _ext.load()
        sp: SPContext = ctx.sp
        qkv, z, etable = ctx.saved_tensors
        variant_id, dropout_p, seed, has_tab, kmax = ctx.cfg
        graph = ctx.graph.ensure_transpose()
        r, hlh, hn, hl = sp.total_rows, sp.hl_heads, sp.hn, sp.hl
        dout = dout.contiguous()
        if sp.token_rows is not None and len(sp.token_rows) > 1:
            dout = dout.clone()
            dout[sp.token_rows[0]] += dout[sp.token_rows[1:]].sum(0)
            dout[sp.token_rows[1:]] = 0
        out = sp.ctx_local[ctx.layer] if sp.routed else sp.ctx[ctx.layer].tensor
        q, k, v = sp.split_packed(qkv)
        # gradients land packed in the symmetric buffer: in this rank's copy so that peers can pull their rows, or
        # (routed) straight in the row owners' slabs at the k | v | q column offsets of a packed row
        dbuf = sp.dqkv.tensor
        dq, dk, dv = sp.split_packed(dbuf)
        route = sp.route(sp.dqkv, sp.qkv_ld, extra=(2 * hl, 0, hl)) if sp.routed else []
        zd = torch.empty((r, hlh, 2), dtype=torch.float32, device=qkv.device)
        detab = torch.zeros(etable.shape, dtype=torch.float32, device=qkv.device) if has_tab else None
        ext.edge_attn_bwd(q, k, v, out.view(r, hlh, hn), z, dout.view(r, hlh, hn), dq, dk, dv, zd, graph.rowptr, graph.col,
                          graph.etype, graph.t_rowptr, graph.t_row, graph.t_eid, etable if has_tab else None, detab,
                          variant_id, dropout_p, seed, kmax, graph.t_task, graph.t_split, int(graph.kv_slots), ctx.out_drop,
                          route)
        _ext.count_launches(3)
        if debug.enabled() and dout.data_ptr() == sp.dctx.tensor.data_ptr():
            debug.poison(sp.dctx.tensor)              # d(context) consumed; the next push must overwrite all of it
        return dbuf, (detab.to(etable.dtype) if has_tab else None), None, None, None, None, None, None, None, None


class _CtxPullOutProj(torch.autograd.Function):
    """heads->nodes pull + (optional) output projection with fused bias / dropout / residual.

    ``y = residual + drop_post(W_o drop_pre(a) + b_o)`` where ``a`` is this rank's rows of the context gathered from
    all head owners.  Without a projection (Exphormer) ``y = residual + drop_post(a)``."""

    @staticmethod
    def forward(ctx, ctx_full, wo, bo, residual, sp: SPContext, p_pre, p_post, seed_pre, seed_post, slot=None,
                pre_applied: bool = False):
        dt = ctx_full.dtype
        pre_pending = p_pre > 0 and not pre_applied   # pre_applied: the attention kernel already stored the dropped context
        if wo is not None and not pre_pending and _can_pull(sp, sp.hl, sp.rows_local, sp.h, wo.size(0), dt):
            # the projection GEMM pulls its operand itself; a local copy is written only when a backward pass will
            # read it (weight gradient)
            w = gemm.operand_copy(wo, dt)
            sp.sw.barrier(0)                                         # every head owner has written its context
            y, a = _pull_gemm(sp.ctx_ptrs_for(ctx_full), 0 if sp.routed else sp.row0, sp.hl, sp.hl, sp.rows_local, w, bias=bo,
                              residual=residual, dropout_p=p_post, seed=seed_post, keep_copy=any(ctx.needs_input_grad[:3]))
            ctx.save_for_backward(a if a is not None else ctx_full.new_empty(0), w)
        else:
            if sp.P > 1:
                sp.sw.barrier(0)                                     # every head owner has written its context
                a = torch.empty((sp.rows_local, sp.h), dtype=dt, device=ctx_full.device)
                esz = ctx_full.element_size()
                _ext.load().peer_gather_cols(sp.ctx_ptrs_for(ctx_full), 0 if sp.routed else sp.row0, sp.rows_local, sp.hl * esz,
                                             sp.hl * esz, a)
                _ext.count_launches(1)
            else:
                a = ctx_full
            if pre_pending:
                a = hash_dropout(a, seed_pre, p_pre)
            if wo is not None:
                w = gemm.operand_copy(wo, dt)
                y = gemm.gemm_tn(a, w, bo, None, dropout_p=p_post, dropout_seed=seed_post, residual=residual)
                ctx.save_for_backward(a, w)
            else:
                y = hash_dropout(a, seed_post, p_post) if p_post > 0 else a
                if residual is not None:
                    y = y + residual
                ctx.save_for_backward()
        ctx.sp, ctx.slot, ctx.wo = sp, slot, wo
        ctx.cfg = (float(p_pre), float(p_post), int(seed_pre), int(seed_post), residual is not None, wo is not None,
                   bo is not None, wo.dtype if wo is not None else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        sp: SPContext = ctx.sp
        p_pre, p_post, seed_pre, seed_post, has_res, has_w, has_b, wdtype = ctx.cfg
        handed = ctx.slot.take(dy) if ctx.slot is not None else None
        dy = dy.contiguous()
        g = hash_dropout(dy, seed_post, p_post) if p_post > 0 else dy
        dbuf = sp.dctx
        dw = db = None
        if has_w:
            a, w = ctx.saved_tensors
            # d(context) = (g W_o) [* pre-dropout mask], pushed to the head owners by the GEMM epilogue
            _push_gemm(g, gemm.operand_copy(ctx.wo, w.dtype, transpose=True), None, dbuf.ptrs, sp.row0, sp.hl,
                       dropout_p=p_pre, seed=seed_pre)
            need_db = has_b and not (handed is not None and p_post == 0)
            dw, db = gemm.weight_grad(g, a, need_db)
            dw = dw.to(wdtype)
            if has_b:
                db = (db if need_db else handed).to(wdtype)
        else:
            da = hash_dropout(g, seed_pre, p_pre) if p_pre > 0 else g
            esz = da.element_size()
            _ext.load().peer_scatter_cols(dbuf.ptrs, sp.row0, sp.rows_local, sp.hl * esz, sp.hl * esz, da.contiguous())
            _ext.count_launches(1)
        sp.sw.barrier(0)                                             # all d(context) rows have landed
        return dbuf.tensor, dw, db, (dy if has_res else None), None, None, None, None, None, None, None


def _ctx_ptrs_for(self, t):
    """Source pointers of the heads->nodes gather for the context tensor an attention call returned: the peers' buffers
    (pull form), or the slabs of this rank's own buffer that the peers' attention kernels have filled (routed form)."""
    if self.routed:
        for i, loc in enumerate(self.ctx_local):
            if loc.data_ptr() == t.data_ptr():
                return self.slab_ptrs(self.ctx[i], self.hl * t.element_size())
    else:
        for b in self.ctx:
            if b.tensor.data_ptr() == t.data_ptr():
                return b.ptrs
    raise RuntimeError("context tensor is not one of the context buffers")


SPContext.ctx_ptrs_for = _ctx_ptrs_for


# ---------------------------------------------------------------------------------------------------
# per-model fused layers
# ---------------------------------------------------------------------------------------------------
def _core(layer):
    d = layer.self_attention.dist_attn
    return getattr(d, "local_attn", d)


def _attention(layer, x2d, graph: AttnGraph, sp: SPContext, idx: int, passthrough: bool = False,
               out_p: float = 0.0, out_seed: int = 0):
    """Context of the layer's attention; with ``passthrough`` also the input routed through the projection function
    (use it as the residual so that its gradient is added inside the input-gradient GEMM)."""
    mha = layer.self_attention
    core = _core(layer)
    qkv = _QKVPush.apply(x2d, mha.linear_q.weight, mha.linear_k.weight, mha.linear_v.weight, mha.linear_q.bias,
                         mha.linear_k.bias, mha.linear_v.bias, sp, idx, passthrough)
    xr = None
    if passthrough:
        qkv, xr = qkv
    variant = core.variant
    etab = core.edge_table() if variant == "exphormer" else None
    if variant == "exphormer" and (etab is None or graph.etype is None):
        variant, etab = "plain", None
    p_att = core.attention_dropout_rate if (variant == "gps" and layer.training) else 0.0
    tab = etab.to(torch.float32).contiguous() if etab is not None else None
    out = _PackedEdgeAttention.apply(qkv, tab, graph, sp, idx, _VARIANTS[variant], p_att, new_seed() if p_att > 0 else 0,
                                     float(out_p), int(out_seed))
    return (out, xr) if passthrough else out


def _p(module, training) -> float:
    return float(module.p) if (training and module is not None) else 0.0


def _gt_attn(layer, x, graph, sp, idx):
    p = _p(layer.self_attention_dropout, layer.training)
    shared = sp.shared_seed(idx, 0) if p > 0 else None
    seed = (shared if shared is not None else new_seed()) if p > 0 else 0
    # The dropout before the output projection is applied by the attention kernel when it stores the context.  With
    # several ranks the head owner writes the mask and the row owner regenerates it in backward, so the seed has to be
    # the shared per-step one; without it the separate (rank-local) dropout pass is used.
    fuse = p > 0 and sp.token_rows is None and FUSE_CONTEXT_DROPOUT and (sp.P == 1 or shared is not None)
    ctx, xr = _attention(layer, x, graph, sp, idx, passthrough=True, out_p=p if fuse else 0.0, out_seed=seed)
    slot = ColsumSlot()                                   # LayerNorm backward -> bias gradient of the projection
    s = _CtxPullOutProj.apply(ctx, layer.O.weight, layer.O.bias, xr, sp, p, 0.0, seed, 0, slot, fuse)
    return layer_norm(s, layer.layer_norm1.weight, layer.layer_norm1.bias, layer.layer_norm1.eps, slot)


def _gt_ffn(layer, x1):
    p = _p(layer.self_attention_dropout, layer.training)
    slot = ColsumSlot()
    s = fused_ffn(x1, layer.FFN_layer1.weight, layer.FFN_layer1.bias, layer.FFN_layer2.weight, layer.FFN_layer2.bias,
                  act="relu", residual=x1, p1=p, p2=0.0, training=layer.training, out_grad_colsum=slot)
    return layer_norm(s, layer.layer_norm2.weight, layer.layer_norm2.bias, layer.layer_norm2.eps, slot)


def _graphormer_attn(layer, x, graph, sp, idx):
    n = layer.self_attention_norm
    y = layer_norm(x, n.weight, n.bias, n.eps)
    ctx = _attention(layer, y, graph, sp, idx)
    p = _p(layer.self_attention_dropout, layer.training)
    o = layer.self_attention.output_layer
    return _CtxPullOutProj.apply(ctx, o.weight, o.bias, x, sp, 0.0, p, 0, new_seed() if p > 0 else 0)


def _graphormer_ffn(layer, x):
    n = layer.ffn_norm
    y = layer_norm(x, n.weight, n.bias, n.eps)
    p = _p(layer.ffn_dropout, layer.training)
    return fused_ffn(y, layer.ffn.layer1.weight, layer.ffn.layer1.bias, layer.ffn.layer2.weight, layer.ffn.layer2.bias,
                     act="gelu", residual=x, p1=0.0, p2=p, training=layer.training)


def _bn(norm, x):
    return batch_norm(x, norm, getattr(norm, "_bf_sync_group", None))


def _gps_attn(layer, x, graph, sp, idx):
    ctx, xr = _attention(layer, x, graph, sp, idx, passthrough=True)
    p = _p(layer.dropout1, layer.training)
    o = getattr(layer.self_attention, "out_proj", None)
    s = _CtxPullOutProj.apply(ctx, None if o is None else o.weight, None if o is None else o.bias, xr, sp, 0.0, p, 0,
                              new_seed() if p > 0 else 0)
    return _bn(layer.norm1, s)


def _gps_ffn(layer, x1):
    s = fused_ffn(x1, layer.ffn1.weight, layer.ffn1.bias, layer.ffn2.weight, layer.ffn2.bias, act="relu", residual=x1,
                  p1=_p(layer.ff_dropout1, layer.training), p2=_p(layer.ff_dropout2, layer.training),
                  training=layer.training)
    return _bn(layer.norm2, s)


_LAYER_IMPL = {"gt": (_gt_attn, _gt_ffn), "graphormer": (_graphormer_attn, _graphormer_ffn),
               "graphgps": (_gps_attn, _gps_ffn), "exphormer": (_gps_attn, _gps_ffn)}


def _install(layer, idx: int, sp: SPContext, attn_fn, ffn_fn):
    portable_forward = layer.forward
    portable_attn_only = layer.forward_attn_only
    portable_ffn_ckpt = layer.forward_ffn_checkpointed

    def usable(x, edge_index, attn_type, attn_bias):
        return (x.is_cuda and x.dtype == sp.dtype and x.dim() == 3 and x.size(0) == 1 and x.size(1) == sp.rows_local
                and attn_bias is None and str(attn_type or "sparse").lower() == "sparse" and edge_index is not None)

    def forward_attn_only(self, x, attn_bias=None, edge_index=None, attn_type=None, **kw):
        if not usable(x, edge_index, attn_type, attn_bias):
            return portable_attn_only(x, attn_bias, edge_index, attn_type, **kw)
        graph = as_attn_graph(edge_index, sp.total_rows)
        return attn_fn(self, x.squeeze(0), graph, sp, idx).unsqueeze(0)

    def forward_ffn_checkpointed(self, x):
        if not (x.is_cuda and x.dtype == sp.dtype):
            return portable_ffn_ckpt(x)
        return checkpoint(lambda t: ffn_fn(self, t.squeeze(0)).unsqueeze(0), x, use_reentrant=False)

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None, **kw):
        if not usable(x, edge_index, attn_type, attn_bias):
            return portable_forward(x, attn_bias, edge_index, attn_type, **kw)
        graph = as_attn_graph(edge_index, sp.total_rows)
        # squeeze/unsqueeze are views in both directions (indexing would zero-fill and copy a full activation in backward)
        return ffn_fn(self, attn_fn(self, x.squeeze(0), graph, sp, idx)).unsqueeze(0)

    layer.forward = types.MethodType(forward, layer)
    layer.forward_attn_only = types.MethodType(forward_attn_only, layer)
    layer.forward_ffn_checkpointed = types.MethodType(forward_ffn_checkpointed, layer)


def enable_for_model(model, args, group, world: int, nodes_per_rank: int, amp_dtype) -> bool:
    """Install the fused layer path on ``model`` when the configuration allows it; returns whether it did."""
    name = str(args.model).lower()
    if name not in _LAYER_IMPL or amp_dtype not in (torch.bfloat16, torch.float16):
        return False
    h, heads = int(args.hidden_dim), int(args.num_heads)
    hl = (heads // world) * (h // heads)
    if h % 64 != 0 or hl % 16 != 0 or (3 * hl) % 16 != 0 or (h // heads) not in (8, 16, 32, 64, 128):
        return False
    if name == "graphgps" and str(getattr(args, "attn_type", "sparse")).lower() != "sparse":
        return False
    dev = next(model.parameters()).device
    rows_local = nodes_per_rank + (1 if (name == "graphormer" and int(args.num_global_node) > 0) else 0)
    token_rows = [r * rows_local for r in range(world)] if rows_local != nodes_per_rank else None
    sp = SPContext(group, dev, world, rows_local, h, heads, len(model.layers), amp_dtype, token_rows)
    attn_fn, ffn_fn = _LAYER_IMPL[name]
    for i, layer in enumerate(model.layers):
        _install(layer, i, sp, attn_fn, ffn_fn)
    model._fused_sp_context = sp
    return True
