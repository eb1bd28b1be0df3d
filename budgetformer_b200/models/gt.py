"""GT (Dwivedi-Bresson style graph transformer), node level, sequence parallel.

Structure and parameter names follow models/gt_dist_node_level.py: sparse-only attention
(:505-522), no projection inside the attention module (:525-577), post-LN encoder layer with the
output projection ``O``, ReLU FFN of width 2h and one dropout module reused in both halves
(:631-684), ``MLPReadout`` h -> h/2 -> h/4 -> C (:687-702)."""
from __future__ import annotations

from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from ..parallel.initialize import get_sequence_parallel_group
from ..parallel.sp_ops import DistributedAttentionNodeLevel
from .common import NodeModelBase, SparseCoreAttention, encode_features, init_params


class CoreAttention(SparseCoreAttention):
    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None, **kw):
        attn_type = "sparse" if attn_type is None else str(attn_type).lower()
        if attn_type != "sparse":
            raise ValueError(f"GT is restricted to graph-neighbourhood sparse attention; got attn_type={attn_type!r}.")
        return super().forward(q, k, v, attn_bias, edge_index, "sparse", **kw)


class MultiHeadAttention(nn.Module):
    def __init__(self, hidden_size, attention_dropout_rate, num_heads):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        self.linear_q = nn.Linear(hidden_size, num_heads * self.att_size)
        self.linear_k = nn.Linear(hidden_size, num_heads * self.att_size)
        self.linear_v = nn.Linear(hidden_size, num_heads * self.att_size)
        self.dist_attn = DistributedAttentionNodeLevel(
            CoreAttention(hidden_size, attention_dropout_rate, num_heads), get_sequence_parallel_group())

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        b = x.size(0)
        q = self.linear_q(x).view(b, -1, self.num_heads, self.att_size)
        k = self.linear_k(x).view(b, -1, self.num_heads, self.att_size)
        v = self.linear_v(x).view(b, -1, self.num_heads, self.att_size)
        out = self.dist_attn(q, k, v, attn_bias, edge_index, attn_type)
        assert out.size() == x.size()
        return out


class EncoderLayer(nn.Module):
    def __init__(self, hidden_size, ffn_size, dropout_rate, attention_dropout_rate, num_heads):
        super().__init__()
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads)
        self.self_attention_dropout = nn.Dropout(dropout_rate)
        self.O = nn.Linear(hidden_size, hidden_size)
        self.layer_norm1 = nn.LayerNorm(hidden_size)
        self.FFN_layer1 = nn.Linear(hidden_size, hidden_size * 2)
        self.FFN_layer2 = nn.Linear(hidden_size * 2, hidden_size)
        self.layer_norm2 = nn.LayerNorm(hidden_size)

    def _ffn(self, h):
        y = self.FFN_layer1(h)
        y = F.relu(y)
        y = self.self_attention_dropout(y)
        y = self.FFN_layer2(y)
        return self.layer_norm2(h + y)

    def forward_attn_only(self, x, attn_bias=None, edge_index=None, attn_type=None, **kwargs):
        y = self.self_attention(x, attn_bias, edge_index=edge_index, attn_type=attn_type)
        y = self.self_attention_dropout(y)
        y = self.O(y)
        return self.layer_norm1(x + y)

    def forward_ffn_checkpointed(self, x_ln):
        return checkpoint(self._ffn, x_ln, use_reentrant=False)

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        return self._ffn(self.forward_attn_only(x, attn_bias, edge_index, attn_type))


class MLPReadout(nn.Module):
    def __init__(self, input_dim, output_dim, L=2):
        super().__init__()
        layers = [nn.Linear(input_dim // 2 ** l, input_dim // 2 ** (l + 1), bias=True) for l in range(L)]
        layers.append(nn.Linear(input_dim // 2 ** L, output_dim, bias=True))
        self.FC_layers = nn.ModuleList(layers)
        self.L = L

    def forward(self, x):
        from ..ops.gemm import readout_linear
        y = x
        for l in range(self.L):
            y = F.relu(readout_linear(y, self.FC_layers[l].weight, self.FC_layers[l].bias))
        return readout_linear(y, self.FC_layers[self.L].weight, self.FC_layers[self.L].bias)


class GT(NodeModelBase):
    def __init__(self, n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
                 input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node, **kwargs):
        super().__init__()
        self.node_encoder = nn.Linear(input_dim, hidden_dim)
        self.input_dropout = nn.Dropout(input_dropout_rate)
        self.layers = nn.ModuleList([
            EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads) for _ in range(n_layers)])
        self.n_layers = n_layers
        self.MLP_layer = MLPReadout(hidden_dim, output_dim)
        self.apply(lambda m: init_params(m, n_layers=n_layers))
        self._init_ckpt_state()

    def forward_logits(self, x, attn_bias, edge_index, perturb=None, attn_type=None):
        if perturb is None:
            x = encode_features(self.node_encoder, x, self.input_dropout).unsqueeze(0)
        else:
            x = self.input_dropout(encode_features(self.node_encoder, x).unsqueeze(0) - perturb)
        x = self._run_layers(x, edge_index=edge_index, attn_type=attn_type)
        return self.MLP_layer(x.squeeze(0))

    def forward(self, x, attn_bias, edge_index, perturb=None, attn_type=None):
        return F.log_softmax(self.forward_logits(x, attn_bias, edge_index, perturb, attn_type), dim=1)
