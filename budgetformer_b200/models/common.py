"""Pieces shared by every node-level model: initialisation, the sparse core attention, the
activation-tier plumbing and the encoder loop."""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from ..graph.attn_graph import AttnGraph, as_attn_graph
from ..ops.edge_attention import edge_attention
from ..parallel.initialize import get_sequence_parallel_world_size


def init_params(module: nn.Module, n_layers: int) -> None:
    """Linear ~ N(0, 0.02/sqrt(n_layers)) with zero bias, Embedding ~ N(0, 0.02)
    (models/graphormer_dist_node_level.py:39-45)."""
    if isinstance(module, nn.Linear):
        module.weight.data.normal_(mean=0.0, std=0.02 / math.sqrt(n_layers))
        if module.bias is not None:
            module.bias.data.zero_()
    if isinstance(module, nn.Embedding):
        module.weight.data.normal_(mean=0.0, std=0.02)


class SparseCoreAttention(nn.Module):
    """Local attention over this rank's ``H/P`` heads and all nodes.

    ``variant`` selects the per-model numerics (see ``ops/edge_attention.py``).  Dense ``full`` attention
    is kept as a plain-PyTorch option for small graphs, as in the reference
    (models/graphormer_dist_node_level.py:267-337)."""

    variant = "plain"

    def __init__(self, hidden_size: int, attention_dropout_rate: float, num_heads: int):
        super().__init__()
        p = get_sequence_parallel_world_size()
        self.hidden_size_per_attention_head = hidden_size // num_heads
        self.num_attention_heads_per_partition = num_heads // p
        self.num_heads = num_heads
        self.scale = math.sqrt(self.hidden_size_per_attention_head)
        self.att_dropout = nn.Dropout(attention_dropout_rate)
        self.attention_dropout_rate = attention_dropout_rate
        self._dropout_calls = 0

    def _next_dropout_seed(self) -> int:
        # drawn from torch's generator so that runs are reproducible under torch.manual_seed
        return int(torch.randint(0, 2**31 - 1, (1,)).item())

    def edge_table(self) -> Optional[torch.Tensor]:
        return None

    # ---- research analytics (models/gt_dist_node_level.py:75-139 in the reference); off unless enabled ----------
    def enable_hop_mass_tracking(self, mass: float = 0.95, max_queries: int = 64, query_sampling: str = "random",
                                 max_batches: int = 1, max_hop: int = 15) -> None:
        from ..utils.analytics import HeadMassStats, HopMassTracker
        self.hop_tracker = HopMassTracker(mass, max_hop, max_batches)
        self.head_mass = HeadMassStats(self.num_attention_heads_per_partition)
        self.hop_mass_max_queries, self.hop_mass_query_sampling = int(max_queries), str(query_sampling)
        self.track_hop_mass = True

    def disable_hop_mass_tracking(self) -> None:
        self.track_hop_mass = False

    def reset_hop_mass_stats(self) -> None:
        if getattr(self, "hop_tracker", None) is not None:
            self.hop_tracker.reset()

    def reset_head_mass_stats(self) -> None:
        if getattr(self, "head_mass", None) is not None:
            self.head_mass.reset()

    def get_hop_mass_stats(self):
        t = getattr(self, "hop_tracker", None)
        return t.summary() if (t is not None and getattr(self, "track_hop_mass", False)) else None

    def get_head_mass_stats(self):
        h = getattr(self, "head_mass", None)
        return h.mean() if h is not None else None

    def _track_sparse(self, q, k, graph: AttnGraph, edge_hops) -> None:
        """Normalised edge weights of this call, restated in PyTorch (analytics only; the kernels do not store them)."""
        import math
        with torch.no_grad():
            src, dst = graph.col.to(torch.int64), graph.row_ids()
            s = (k[0].float()[src] * q[0].float()[dst]).sum(-1) / math.sqrt(q.size(-1))
            w = torch.exp(s.clamp(-5.0, 5.0))
            z = torch.zeros(q.size(1), q.size(2), device=q.device).index_add_(0, dst, w)
            a = w / (z[dst] + 1e-6)
            self.head_mass.add(a)
            if edge_hops is not None:
                self.hop_tracker.add_sparse(dst, edge_hops, a)

    # ---- dense-attention research hooks (models/graphormer_dist_node_level.py:121-130,296-304 in the reference) ----
    def set_full_attention_capture(self, enabled: bool = True) -> None:
        """Keep the head-averaged probabilities ``[b, q, k]`` of the next dense call on the CPU."""
        self.capture_full_attn = bool(enabled)
        if not self.capture_full_attn:
            self.last_full_attn_mean = None

    def get_last_full_attention_mean(self):
        return getattr(self, "last_full_attn_mean", None)

    def set_full_attention_extra_bias(self, extra_bias) -> None:
        """A tensor broadcastable to ``[b, heads, q, k]`` added to the dense scores before the softmax (``None`` = off)."""
        self.full_attention_extra_bias = extra_bias

    def full_attention(self, q, k, v, attn_bias=None):
        q = q.transpose(1, 2)
        k = k.transpose(1, 2).transpose(2, 3)
        v = v.transpose(1, 2)
        x = torch.matmul(q / self.scale, k)
        if attn_bias is not None:
            x = x + attn_bias
        extra = getattr(self, "full_attention_extra_bias", None)
        if extra is not None:
            x = x + extra.to(device=x.device, dtype=x.dtype)
        probs = torch.softmax(x, dim=3)
        if getattr(self, "capture_full_attn", False):
            self.last_full_attn_mean = probs.mean(dim=1).detach().cpu()
        if getattr(self, "track_hop_mass", False) and getattr(self, "hop_matrix", None) is not None:
            # hop_matrix [Q, K] holds the hop distance from the sampled queries hop_queries [Q] to every key
            with torch.no_grad():
                rows = probs.mean(dim=1)[0].index_select(0, self.hop_queries.to(probs.device)).float()
                self.hop_tracker.add_dense(rows, self.hop_matrix.to(probs.device))
                self.head_mass.add(probs[0].permute(1, 2, 0).reshape(-1, probs.size(1)))
        x = self.att_dropout(probs)
        return x.matmul(v).transpose(1, 2).contiguous()

    def sparse(self, q, k, v, graph: AttnGraph, edge_bias=None):
        b, s, hl, hn = q.shape
        assert b == 1, "full-graph attention runs with a single sequence"
        p_drop = self.attention_dropout_rate if (self.variant == "gps" and self.training) else 0.0
        seed = self._next_dropout_seed() if p_drop > 0 else 0
        out = edge_attention(q[0], k[0], v[0], graph, variant=self.variant, etable=self.edge_table(),
                             edge_bias=edge_bias, dropout_p=p_drop, dropout_seed=seed)
        if getattr(self, "track_hop_mass", False):
            self._track_sparse(q, k, graph, getattr(self, "edge_hops", None))
        return out.unsqueeze(0)

    # ---- two-phase form of the sparse path (models/graphormer_dist_node_level.py:515-587): the edge weights need only
    # q and k, so a caller can compute them while v is still in flight, then aggregate.  Plain PyTorch; the fused
    # kernels keep both phases in one pass because their v arrives with q and k in one packed transfer.
    def sparse_score_phase(self, q, k, edge_index, edge_bias=None):
        """``exp(clamp(q.k / sqrt(hn), -5, 5) [+ bias])`` per edge and head, with what the second phase needs."""
        graph = as_attn_graph(edge_index, q.size(1)).to(q.device)
        src, dst = graph.col.to(torch.int64), graph.row_ids()
        s = (k[0].float()[src] * q[0].float()[dst]).sum(-1) / self.scale
        s = s.clamp(-5.0, 5.0)
        if edge_bias is not None:
            s = s + edge_bias.float()
        return {"score": torch.exp(s), "src": src, "dst": dst, "num_nodes": q.size(1), "dtype": q.dtype}

    def sparse_aggregate_phase(self, score_ctx, v):
        """``sum_e w_e v_src(e) / (sum_e w_e + 1e-6)`` per query; returns ``[1, n, Hl, hn]``."""
        w, src, dst, n = score_ctx["score"], score_ctx["src"], score_ctx["dst"], score_ctx["num_nodes"]
        vv = v[0].float()
        wv = torch.zeros(n, vv.size(1), vv.size(2), device=vv.device).index_add_(0, dst, vv[src] * w.unsqueeze(-1))
        z = torch.zeros(n, vv.size(1), device=vv.device).index_add_(0, dst, w)
        return (wv / (z.unsqueeze(-1) + 1e-6)).to(score_ctx["dtype"]).unsqueeze(0)

    def sparse_head_groups(self, q, k, v, edge_sets, edge_bias=None):
        """One edge set per head group (models/graphormer_dist_node_level.py:175-214, models/gt_dist_node_level.py:195-221):
        with G sets, consecutive blocks of ceil(Hl / G) local heads attend over set g; the heads of a missing or empty
        set output zero.  ``edge_bias``, when given, is a list with one ``[E_g, heads of the group]`` tensor per set.
        Every group uses the score rule of the single-set path."""
        b, s, hl, hn = q.shape
        groups = max(1, len(edge_sets))
        per = -(-hl // groups)
        out = q.new_zeros(b, s, hl, hn)
        for g, edges in enumerate(edge_sets):
            h0, h1 = g * per, min((g + 1) * per, hl)
            if h0 >= h1 or edges is None or (isinstance(edges, torch.Tensor) and edges.numel() == 0):
                continue
            graph = as_attn_graph(edges, s)
            if graph.num_edges == 0:
                continue
            sl = lambda t: t[:, :, h0:h1].contiguous()
            out[:, :, h0:h1] = self.sparse(sl(q), sl(k), sl(v), graph.to(q.device),
                                           edge_bias=None if edge_bias is None else edge_bias[g])
        return out

    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None, **kw):
        b, s = q.size(0), q.size(1)
        attn_type = "sparse" if attn_type is None else str(attn_type).lower()
        if attn_type == "full":
            x = self.full_attention(q, k, v, attn_bias)
        elif attn_type == "sparse" and isinstance(edge_index, (list, tuple)):
            x = self.sparse_head_groups(q, k, v, edge_index, edge_bias=kw.get("edge_bias"))
        elif attn_type == "sparse":
            graph = as_attn_graph(edge_index, s)
            x = self.sparse(q, k, v, graph, edge_bias=kw.get("edge_bias"))
        else:
            raise ValueError(f"unsupported attn_type {attn_type!r}")
        return x.reshape(b, s, -1)


def apply_tier(layer, mode: str, x, **kwargs):
    """Run one encoder layer under an activation tier (gt_sp/multi_tier.py:31-53):
    ``retain`` keeps everything, ``keep_mha``/``ffn_only`` keeps the attention half and recomputes
    the FFN, anything else recomputes the whole layer (including its two all-to-alls)."""
    if mode == "retain" or mode == "none":
        return layer(x, **kwargs)
    if mode in ("keep_mha", "ffn_only"):
        x = layer.forward_attn_only(x, **kwargs)
        return layer.forward_ffn_checkpointed(x)

    def _full(h):
        return layer(h, **kwargs)

    return checkpoint(_full, x, use_reentrant=False)


def encode_features(encoder: nn.Linear, x: torch.Tensor, dropout: Optional[nn.Dropout] = None) -> torch.Tensor:
    """``dropout(encoder(x))`` for a 2-D feature matrix whose columns may have been zero-padded by the caller.

    Feature widths such as 269 leave rows unaligned, which sends the library GEMM to slow legacy kernels; the
    trainer therefore pads the feature matrix once to a multiple of 8 columns and the weight is padded to match
    here (the gradient of the padding is dropped by autograd).  16-bit CUDA inputs take the tcgen05 GEMM."""
    w = encoder.weight
    extra = x.size(-1) - w.size(1)
    if extra < 0:
        raise ValueError(f"feature matrix has {x.size(-1)} columns, encoder expects {w.size(1)}")
    if extra:
        w = F.pad(w, (0, extra))
    p = float(dropout.p) if (dropout is not None and dropout.training) else 0.0
    if x.is_cuda and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16):
        # input dropout runs in the GEMM epilogue (counter-based mask, regenerated in backward: no mask tensor)
        from ..ops.gemm import fused_linear
        from ..ops.norm import new_seed
        return fused_linear(x, w, encoder.bias, dropout_p=p, dropout_seed=new_seed() if p > 0 else 0)
    y = F.linear(x, w, encoder.bias)
    return dropout(y) if dropout is not None else y


class NodeModelBase(nn.Module):
    """Activation-checkpoint control shared by all models
    (e.g. models/gt_dist_node_level.py:741-775)."""

    def _init_ckpt_state(self):
        self.activation_checkpoint = False
        self.activation_checkpoint_mode = "none"
        self._comm_ckpt = None

    def set_activation_checkpoint(self, enabled: bool = True, mode: Optional[str] = None, deferred: bool = False) -> None:
        aliases = {None: "none", "none": "none", "all": "layer", "layer": "layer", "ffn_only": "ffn_only",
                   "multi_tier": "multi_tier", "adaptive": "comm_aware", "comm_aware": "comm_aware"}
        if mode not in aliases:
            raise ValueError(f"activation_checkpoint_mode must be one of all/ffn_only/adaptive/multi_tier, got {mode!r}")
        resolved = aliases[mode]
        enabled = bool(enabled) and resolved != "none"
        self.activation_checkpoint = enabled
        self.activation_checkpoint_mode = resolved if enabled else "none"
        if self.activation_checkpoint_mode == "multi_tier":
            from ..control.multi_tier import ExecutionPlanner
            self._comm_ckpt = ExecutionPlanner(len(self.layers), deferred=deferred)
        elif self.activation_checkpoint_mode == "comm_aware":
            from ..control.multi_tier import CommAwareCheckpointer
            self._comm_ckpt = CommAwareCheckpointer(len(self.layers))
        else:
            self._comm_ckpt = None

    def comm_aware_notify_budget_frozen(self, reuse_deferred_baseline: bool = False) -> None:
        if self._comm_ckpt is not None and hasattr(self._comm_ckpt, "notify_budget_frozen"):
            self._comm_ckpt.notify_budget_frozen(reuse_deferred_baseline=reuse_deferred_baseline)

    def comm_aware_notify_step_end(self, device, t_bwd: float = None, t_fwd: float = None) -> None:
        if self._comm_ckpt is not None:
            self._comm_ckpt.notify_step_end(device, t_bwd=t_bwd, t_fwd=t_fwd)

    def _run_layers(self, x, **kwargs):
        use_ckpt = self.activation_checkpoint and self.training and torch.is_grad_enabled()
        mode = self.activation_checkpoint_mode
        managed = use_ckpt and mode in ("multi_tier", "comm_aware") and self._comm_ckpt is not None
        if managed:
            self._comm_ckpt.plan(x.device)
        for i, layer in enumerate(self.layers):
            if not use_ckpt:
                x = layer(x, **kwargs)
                continue
            layer_mode = self._comm_ckpt.mode(i) if managed else mode
            x = apply_tier(layer, layer_mode, x, **kwargs)
        if managed:
            self._comm_ckpt.record_post_forward_memory(x.device)
        return x

    def core_attention_modules(self):
        for layer in self.layers:
            d = layer.self_attention.dist_attn
            yield getattr(d, "local_attn", d)

    # ---- per-layer switches of the dense-attention hooks (models/graphormer_dist_node_level.py:1178-1228) --------
    def _full_attention_layers(self, layer_mode: str = "all"):
        n = len(self.layers)
        mode = str(layer_mode).lower()
        if mode not in ("all", "last"):
            raise ValueError(f"unsupported full-attention layer mode: {layer_mode}")
        return list(range(n)) if mode == "all" else ([n - 1] if n else [])

    def set_full_attention_capture_layers(self, enabled: bool = True, layer_mode: str = "all") -> None:
        chosen = set(self._full_attention_layers(layer_mode)) if enabled else set()
        for i, core in enumerate(self.core_attention_modules()):
            core.set_full_attention_capture(i in chosen)

    def get_full_attention_means_per_layer(self, layer_mode: str = "all"):
        cores = list(self.core_attention_modules())
        return [cores[i].get_last_full_attention_mean() for i in self._full_attention_layers(layer_mode)]

    def set_full_attention_extra_biases(self, extra_biases, layer_mode: str = "all") -> None:
        chosen = self._full_attention_layers(layer_mode)
        if extra_biases is not None and len(extra_biases) != len(chosen):
            raise ValueError(f"expected {len(chosen)} extra bias tensors for layer_mode={layer_mode}, got {len(extra_biases)}")
        by_layer = dict(zip(chosen, extra_biases)) if extra_biases is not None else {}
        for i, core in enumerate(self.core_attention_modules()):
            core.set_full_attention_extra_bias(by_layer.get(i))

    def set_last_layer_full_attention_capture(self, enabled: bool = True) -> None:
        self.set_full_attention_capture_layers(enabled, layer_mode="last")

    def get_last_layer_full_attention_mean(self):
        means = self.get_full_attention_means_per_layer(layer_mode="last")
        return means[0] if means else None

    def set_last_layer_full_attention_extra_bias(self, extra_bias) -> None:
        self.set_full_attention_extra_biases([extra_bias], layer_mode="last")

    def enable_hop_mass_tracking(self, mass: float = 0.95, max_queries: int = 64, query_sampling: str = "random",
                                 max_batches: int = 1, max_hop: int = 15) -> None:
        for core in self.core_attention_modules():
            core.enable_hop_mass_tracking(mass, max_queries, query_sampling, max_batches, max_hop)

    def disable_hop_mass_tracking(self) -> None:
        for core in self.core_attention_modules():
            core.disable_hop_mass_tracking()

    def get_hop_mass_stats_per_layer(self):
        return [core.get_hop_mass_stats() for core in self.core_attention_modules()]
