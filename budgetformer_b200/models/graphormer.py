"""Graphormer, node level, with one virtual (global) node, sequence parallel.

Follows models/graphormer_dist_node_level.py: pre-LN encoder layer with GELU FFN of width
``ffn_dim`` (:674-740), q/k/v/output projections with bias (:616-671), each rank prepends its own
copy of the virtual node to its local slice (:1324-1328), ``final_ln`` + ``downstream_out_proj``
readout with the virtual-node row dropped (:1394-1399).  ``attn_bias`` (only used by the legacy
mini-batch driver) is projected to per-head scalars by ``attn_bias_proj`` (:1334-1360)."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from ..parallel.initialize import get_sequence_parallel_group
from ..parallel.sp_ops import DistributedAttentionNoMerge
from .common import NodeModelBase, SparseCoreAttention, encode_features, init_params


class FeedForwardNetwork(nn.Module):
    def __init__(self, hidden_size, ffn_size, dropout_rate):
        super().__init__()
        self.layer1 = nn.Linear(hidden_size, ffn_size)
        self.gelu = nn.GELU()
        self.layer2 = nn.Linear(ffn_size, hidden_size)

    def forward(self, x):
        return self.layer2(self.gelu(self.layer1(x)))


class CoreAttention(SparseCoreAttention):
    """Sparse path adds ``attn_bias[src, dst, head]`` after the clamp when a dense bias tensor is
    given (:216-229); the full-graph driver never passes one."""

    def __init__(self, hidden_size, attention_dropout_rate, num_heads, attn_bias_dim=1):
        super().__init__(hidden_size, attention_dropout_rate, num_heads)

    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None, **kw):
        attn_type = "sparse" if attn_type is None else str(attn_type).lower()
        if attn_type == "flash":
            from flash_attn import flash_attn_func
            return flash_attn_func(q, k, v, self.attention_dropout_rate if self.training else 0.0).reshape(
                q.size(0), q.size(1), -1)
        if attn_type == "sparse" and attn_bias is not None and isinstance(edge_index, (list, tuple)):
            # one edge set per head group: the bias of set g is read at its own edges for the heads of the group
            from ..graph.attn_graph import as_attn_graph
            hl, groups = q.size(2), max(1, len(edge_index))
            per = -(-hl // groups)
            graphs = [None if (e is None or (isinstance(e, torch.Tensor) and e.numel() == 0)) else as_attn_graph(e, q.size(1))
                      for e in edge_index]
            eb = [None if g is None else
                  attn_bias[0][i * per:min((i + 1) * per, hl)][:, g.row_ids(), g.col.long()].transpose(0, 1)
                  for i, g in enumerate(graphs)]
            return super().forward(q, k, v, None, graphs, "sparse", edge_bias=eb)
        if attn_type == "sparse" and attn_bias is not None:
            from ..graph.attn_graph import as_attn_graph
            g = as_attn_graph(edge_index, q.size(1))
            # attn_bias: [b, Hl, S_q, S_k] -> per-edge [E, Hl]
            eb = attn_bias[0][:, g.row_ids(), g.col.long()].transpose(0, 1)
            return super().forward(q, k, v, None, g, "sparse", edge_bias=eb)
        return super().forward(q, k, v, attn_bias, edge_index, attn_type, **kw)


class MultiHeadAttention(nn.Module):
    def __init__(self, hidden_size, attention_dropout_rate, num_heads, attn_bias_dim):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        self.linear_q = nn.Linear(hidden_size, num_heads * self.att_size)
        self.linear_k = nn.Linear(hidden_size, num_heads * self.att_size)
        self.linear_v = nn.Linear(hidden_size, num_heads * self.att_size)
        self.dist_attn = DistributedAttentionNoMerge(
            CoreAttention(hidden_size, attention_dropout_rate, num_heads, attn_bias_dim), get_sequence_parallel_group())
        self.output_layer = nn.Linear(num_heads * self.att_size, hidden_size)

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        b = x.size(0)
        q = self.linear_q(x).view(b, -1, self.num_heads, self.att_size)
        k = self.linear_k(x).view(b, -1, self.num_heads, self.att_size)
        v = self.linear_v(x).view(b, -1, self.num_heads, self.att_size)
        return self.output_layer(self.dist_attn(q, k, v, attn_bias, edge_index, attn_type))


class EncoderLayer(nn.Module):
    def __init__(self, hidden_size, ffn_size, dropout_rate, attention_dropout_rate, num_heads, attn_bias_dim):
        super().__init__()
        self.self_attention_norm = nn.LayerNorm(hidden_size)
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads, attn_bias_dim)
        self.self_attention_dropout = nn.Dropout(dropout_rate)
        self.ffn_norm = nn.LayerNorm(hidden_size)
        self.ffn = FeedForwardNetwork(hidden_size, ffn_size, dropout_rate)
        self.ffn_dropout = nn.Dropout(dropout_rate)

    def _ffn(self, h):
        return h + self.ffn_dropout(self.ffn(self.ffn_norm(h)))

    def forward_attn_only(self, x, attn_bias=None, edge_index=None, attn_type=None, **kwargs):
        y = self.self_attention(self.self_attention_norm(x), attn_bias, edge_index, attn_type=attn_type)
        return x + self.self_attention_dropout(y)

    def forward_ffn_checkpointed(self, x):
        return checkpoint(self._ffn, x, use_reentrant=False)

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        return self._ffn(self.forward_attn_only(x, attn_bias, edge_index, attn_type))


class Graphormer(NodeModelBase):
    def __init__(self, n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
                 input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node, **kwargs):
        super().__init__()
        self.num_heads = num_heads
        self.node_encoder = nn.Linear(input_dim, hidden_dim)
        self.input_dropout = nn.Dropout(input_dropout_rate)
        self.layers = nn.ModuleList([
            EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads, attn_bias_dim)
            for _ in range(n_layers)])
        self.n_layers = n_layers
        self.final_ln = nn.LayerNorm(hidden_dim)
        self.downstream_out_proj = nn.Linear(hidden_dim, output_dim)
        self.hidden_dim = hidden_dim
        self.num_global_node = num_global_node
        self.graph_token = nn.Embedding(self.num_global_node, hidden_dim)
        self.graph_token_virtual_distance = nn.Embedding(self.num_global_node, attn_bias_dim)
        self.attn_bias_proj = nn.Linear(attn_bias_dim, num_heads, bias=False)
        self._init_ckpt_state()
        self.apply(lambda m: init_params(m, n_layers=n_layers))

    def _graph_attn_bias(self, attn_bias, device):
        if attn_bias is None:
            return None
        proj = self.attn_bias_proj(attn_bias.to(device))                     # [sub_s, full_s, H]
        if self.num_global_node > 0:
            g = self.num_global_node
            vd = self.attn_bias_proj(self.graph_token_virtual_distance.weight)  # [g, H]
            sub_s, full_s = proj.size(0), proj.size(1)
            row = vd.unsqueeze(1).expand(g, full_s + g, self.num_heads)
            colb = vd.unsqueeze(0).expand(sub_s, g, self.num_heads)
            proj = torch.cat([row, torch.cat([colb, proj], dim=1)], dim=0)
        return proj.permute(2, 0, 1).unsqueeze(0)                               # [1, H, S_q, S_k]

    def forward_logits(self, x, attn_bias, edge_index, perturb=None, attn_type=None):
        x = encode_features(self.node_encoder, x).unsqueeze(0)
        if perturb is not None:
            x = x + perturb
        if self.num_global_node > 0:
            tok = self.graph_token.weight.unsqueeze(0).expand(x.size(0), -1, -1).to(x.dtype)
            x = torch.cat([tok, x], dim=1)
        x = self.input_dropout(x)
        bias = self._graph_attn_bias(attn_bias, x.device)
        x = self._run_layers(x, attn_bias=bias, edge_index=edge_index, attn_type=attn_type)
        x = self.final_ln(x)
        from ..ops.gemm import readout_linear
        return readout_linear(x[0, int(self.num_global_node):, :], self.downstream_out_proj.weight, self.downstream_out_proj.bias)

    def forward(self, x, attn_bias, edge_index, perturb=None, attn_type=None):
        return F.log_softmax(self.forward_logits(x, attn_bias, edge_index, perturb, attn_type), dim=1)
