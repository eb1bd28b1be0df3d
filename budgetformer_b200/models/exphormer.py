"""Exphormer, node level, sequence parallel.

Follows models/exphormer_dist_node_level.py: the score is modulated by a per-edge-type vector
``E = edge_proj(edge_type_emb(type))`` sliced to the rank's heads (:92-121); q/k/v without bias and
no output projection (:128-153); post-norm BatchNorm1d layers with ReLU FFN of width 2h (:160-202).
The reference evaluates ``edge_proj`` on an ``[E_m, h]`` matrix that has only two distinct rows; here
the two rows are projected once and the kernels look them up by edge type."""
from __future__ import annotations

from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from ..parallel.initialize import get_sequence_parallel_group, get_sequence_parallel_rank
from ..parallel.sp_ops import DistributedAttentionNodeLevel
from .common import NodeModelBase, SparseCoreAttention, encode_features, init_params


class ExphormerCoreAttention(SparseCoreAttention):
    variant = "exphormer"
    N_EDGE_TYPES = 2

    def __init__(self, hidden_size, attention_dropout_rate, num_heads):
        super().__init__(hidden_size, attention_dropout_rate, num_heads)
        hidden = num_heads * self.hidden_size_per_attention_head
        self.edge_type_emb = nn.Embedding(self.N_EDGE_TYPES, hidden)
        self.edge_proj = nn.Linear(hidden, hidden, bias=False)

    def edge_table(self):
        hl = self.num_attention_heads_per_partition
        tab = self.edge_proj(self.edge_type_emb.weight).view(self.N_EDGE_TYPES, self.num_heads,
                                                             self.hidden_size_per_attention_head)
        if hl != self.num_heads:
            r = get_sequence_parallel_rank()
            tab = tab[:, r * hl:(r + 1) * hl, :]
        return tab

    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None, **kw):
        return super().forward(q, k, v, None, edge_index, "sparse")


class MultiHeadAttention(nn.Module):
    def __init__(self, hidden_size, attention_dropout_rate, num_heads):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        self.linear_q = nn.Linear(hidden_size, num_heads * self.att_size, bias=False)
        self.linear_k = nn.Linear(hidden_size, num_heads * self.att_size, bias=False)
        self.linear_v = nn.Linear(hidden_size, num_heads * self.att_size, bias=False)
        self.dist_attn = DistributedAttentionNodeLevel(
            ExphormerCoreAttention(hidden_size, attention_dropout_rate, num_heads), get_sequence_parallel_group())

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        b = x.size(0)
        q = self.linear_q(x).view(b, -1, self.num_heads, self.att_size)
        k = self.linear_k(x).view(b, -1, self.num_heads, self.att_size)
        v = self.linear_v(x).view(b, -1, self.num_heads, self.att_size)
        return self.dist_attn(q, k, v, attn_bias, edge_index, attn_type)


class EncoderLayer(nn.Module):
    def __init__(self, hidden_size, dropout_rate, attention_dropout_rate, num_heads):
        super().__init__()
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads)
        self.dropout1 = nn.Dropout(dropout_rate)
        self.norm1 = nn.BatchNorm1d(hidden_size)
        self.ffn1 = nn.Linear(hidden_size, hidden_size * 2)
        self.ffn2 = nn.Linear(hidden_size * 2, hidden_size)
        self.ff_dropout1 = nn.Dropout(dropout_rate)
        self.ff_dropout2 = nn.Dropout(dropout_rate)
        self.norm2 = nn.BatchNorm1d(hidden_size)

    @staticmethod
    def _bn(norm, x):
        b, n, c = x.shape
        group = getattr(norm, "_bf_sync_group", None)
        if group is not None:
            from ..ops.norm import batch_norm
            return batch_norm(x.reshape(b * n, c), norm, group).view(b, n, c)
        return norm(x.reshape(b * n, c)).view(b, n, c)

    def _ffn(self, h):
        out = self.ff_dropout1(F.relu(self.ffn1(h)))
        out = self.ff_dropout2(self.ffn2(out))
        return self._bn(self.norm2, h + out)

    def forward_attn_only(self, x, attn_bias=None, edge_index=None, attn_type=None, **kwargs):
        h = self.dropout1(self.self_attention(x, attn_bias, edge_index=edge_index, attn_type=attn_type))
        return self._bn(self.norm1, x + h)

    def forward_ffn_checkpointed(self, x):
        return checkpoint(self._ffn, x, use_reentrant=False)

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        return self._ffn(self.forward_attn_only(x, attn_bias, edge_index, attn_type))


class Exphormer(NodeModelBase):
    def __init__(self, n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
                 input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node, **kwargs):
        super().__init__()
        self.node_encoder = nn.Linear(input_dim, hidden_dim)
        self.input_dropout = nn.Dropout(input_dropout_rate)
        self.layers = nn.ModuleList([
            EncoderLayer(hidden_dim, dropout_rate, attention_dropout_rate, num_heads) for _ in range(n_layers)])
        self.output_proj = nn.Linear(hidden_dim, output_dim)
        self.apply(lambda m: init_params(m, n_layers=n_layers))
        self._init_ckpt_state()

    def forward_logits(self, x, attn_bias, edge_index, attn_type=None):
        x = encode_features(self.node_encoder, x, self.input_dropout).unsqueeze(0)
        x = self._run_layers(x, attn_bias=attn_bias, edge_index=edge_index, attn_type=attn_type)
        from ..ops.gemm import readout_linear
        return readout_linear(x.squeeze(0), self.output_proj.weight, self.output_proj.bias)

    def forward(self, x, attn_bias, edge_index, attn_type=None):
        return F.log_softmax(self.forward_logits(x, attn_bias, edge_index, attn_type), dim=1)
