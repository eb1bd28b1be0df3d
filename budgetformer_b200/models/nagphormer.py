"""NAGphormer (Hop2Token), node level.

A transformer over each node's ``hops + 1`` pre-aggregated neighbourhood tokens followed by an
attention readout over hops (models/nagphormer_dist_node_level.py:148-236).  There is no
communication in this model: every rank processes its own ``N/P`` nodes.  The reference leaves it
unwired (not in ``--model`` choices); here ``--model nagphormer`` is accepted and uses the same
multi-hop feature preprocessing as ``--hops`` does for Graphormer/GT."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from .common import NodeModelBase, init_params


class FeedForwardNetwork(nn.Module):
    def __init__(self, hidden_size, ffn_size):
        super().__init__()
        self.layer1 = nn.Linear(hidden_size, ffn_size)
        self.gelu = nn.GELU()
        self.layer2 = nn.Linear(ffn_size, hidden_size)

    def forward(self, x):
        return self.layer2(self.gelu(self.layer1(x)))


class MultiHeadAttention(nn.Module):
    def __init__(self, hidden_size, attention_dropout_rate, num_heads):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        self.scale = self.att_size ** -0.5
        self.linear_q = nn.Linear(hidden_size, num_heads * self.att_size)
        self.linear_k = nn.Linear(hidden_size, num_heads * self.att_size)
        self.linear_v = nn.Linear(hidden_size, num_heads * self.att_size)
        self.att_dropout = nn.Dropout(attention_dropout_rate)
        self.output_layer = nn.Linear(num_heads * self.att_size, hidden_size)

    def forward(self, q, k, v):
        bsz, seq_len, _ = q.size()
        d = self.att_size
        q = self.linear_q(q).view(bsz, seq_len, self.num_heads, d).transpose(1, 2)
        k = self.linear_k(k).view(bsz, seq_len, self.num_heads, d).transpose(1, 2)
        v = self.linear_v(v).view(bsz, seq_len, self.num_heads, d).transpose(1, 2)
        attn = self.att_dropout(torch.softmax(torch.matmul(q * self.scale, k.transpose(2, 3)), dim=-1))
        x = attn.matmul(v).transpose(1, 2).contiguous().view(bsz, seq_len, -1)
        return self.output_layer(x)


class EncoderLayer(nn.Module):
    def __init__(self, hidden_size, ffn_size, dropout_rate, attention_dropout_rate, num_heads):
        super().__init__()
        self.self_attention_norm = nn.LayerNorm(hidden_size)
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads)
        self.self_attention_dropout = nn.Dropout(dropout_rate)
        self.ffn_norm = nn.LayerNorm(hidden_size)
        self.ffn = FeedForwardNetwork(hidden_size, ffn_size)
        self.ffn_dropout = nn.Dropout(dropout_rate)

    def _ffn(self, h):
        return h + self.ffn_dropout(self.ffn(self.ffn_norm(h)))

    def forward_attn_only(self, x, **kwargs):
        y = self.self_attention_norm(x)
        return x + self.self_attention_dropout(self.self_attention(y, y, y))

    def forward_ffn_checkpointed(self, x):
        return checkpoint(self._ffn, x, use_reentrant=False)

    def forward(self, x, **kwargs):
        return self._ffn(self.forward_attn_only(x))


class NAGphormer(NodeModelBase):
    def __init__(self, hops, n_class, input_dim, n_layers=1, num_heads=8, hidden_dim=512, ffn_dim=None,
                 dropout_rate=0.1, attention_dropout_rate=0.1, **kwargs):
        super().__init__()
        self.seq_len = hops + 1
        self.hidden_dim = hidden_dim
        self.n_layers = n_layers
        if ffn_dim is None or ffn_dim <= 0:
            ffn_dim = 2 * hidden_dim
        self.att_embeddings_nope = nn.Linear(input_dim, hidden_dim)
        self.layers = nn.ModuleList([
            EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads) for _ in range(n_layers)])
        self.final_ln = nn.LayerNorm(hidden_dim)
        self.out_proj = nn.Linear(hidden_dim, hidden_dim // 2)
        self.attn_layer = nn.Linear(2 * hidden_dim, 1)
        self.Linear1 = nn.Linear(hidden_dim // 2, n_class)
        self.scaling = nn.Parameter(torch.ones(1) * 0.5)
        self.apply(lambda m: init_params(m, n_layers=n_layers))
        self._init_ckpt_state()

    def core_attention_modules(self):
        return iter(())

    def forward_logits(self, x_local, attn_bias=None, edge_index=None, attn_type=None):
        if x_local.dim() == 2:                       # flattened (hops+1)*d features
            x_local = x_local.view(x_local.size(0), self.seq_len, -1)
        t = self.att_embeddings_nope(x_local)
        t = self._run_layers(t)
        out = self.final_ln(t)
        node, neigh = out[:, :1, :], out[:, 1:, :]
        target = node.expand(-1, self.seq_len - 1, -1)
        att = F.softmax(self.attn_layer(torch.cat([target, neigh], dim=2)), dim=1)
        out = (node + (neigh * att).sum(dim=1, keepdim=True)).squeeze(1)
        return self.Linear1(F.relu(self.out_proj(out)))

    def forward(self, x_local, attn_bias=None, edge_index=None, attn_type=None):
        return F.log_softmax(self.forward_logits(x_local, attn_bias, edge_index, attn_type), dim=1)
