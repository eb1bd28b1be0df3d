"""GraphGPS (transformer part only), node level, sequence parallel.

Follows models/graphgps_dist_node_level.py: sparse attention normalises per edge and applies
attention dropout to the normalised weights (:151-177); dense ``full`` (:179-188) and FAVOR+
``performer`` (:53-128, :190-198) variants kept in plain PyTorch; q/k/v bias only for ``full``,
``out_proj`` always with bias (:216-248); post-norm BatchNorm1d over the rank's local rows, ReLU FFN of
width 2h, two FFN dropouts (:255-293); default PyTorch initialisation and no input dropout (:316,333)."""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from ..parallel.initialize import get_sequence_parallel_group
from ..parallel.sp_ops import DistributedAttentionNodeLevel
from .common import NodeModelBase, SparseCoreAttention, encode_features


def _gaussian_orthogonal_random_matrix(nb_rows, nb_columns, device=None):
    blocks = []
    for _ in range(nb_rows // nb_columns):
        q, _ = torch.linalg.qr(torch.randn(nb_columns, nb_columns), mode="reduced")
        blocks.append(q.t())
    rem = nb_rows - (nb_rows // nb_columns) * nb_columns
    if rem > 0:
        q, _ = torch.linalg.qr(torch.randn(nb_columns, nb_columns), mode="reduced")
        blocks.append(q.t()[:rem])
    mat = torch.cat(blocks, dim=0)
    mult = torch.randn(nb_rows, nb_columns).norm(dim=1)
    out = torch.diag(mult) @ mat
    return out.to(device) if device is not None else out


def _softmax_kernel(data, *, projection_matrix, is_query, eps=1e-4):
    d = data.shape[-1]
    norm = d ** -0.25
    ratio = projection_matrix.shape[0] ** -0.5
    proj = projection_matrix.type_as(data)
    dash = torch.einsum("...nd,rd->...nr", norm * data, proj)
    diag = (data ** 2).sum(-1, keepdim=True) * 0.5 * (norm ** 2)
    if is_query:
        dash = ratio * torch.exp(dash - diag - dash.amax(dim=-1, keepdim=True)).clamp(min=eps)
    else:
        dash = ratio * torch.exp(dash - diag - dash.amax(dim=(-1, -2), keepdim=True)).clamp(min=eps)
    return dash.type_as(data)


def _linear_attention(q, k, v):
    k_sum = k.sum(dim=-2)
    d_inv = 1.0 / torch.einsum("...nd,...d->...n", q, k_sum)
    context = torch.einsum("...nd,...ne->...de", k, v)
    return torch.einsum("...de,...nd,...n->...ne", context, q, d_inv)


class PerformerFastAttention(nn.Module):
    def __init__(self, dim_heads, nb_features=None):
        super().__init__()
        nb_features = nb_features or max(1, int(dim_heads * math.log(dim_heads)))
        self.register_buffer("projection_matrix", _gaussian_orthogonal_random_matrix(nb_features, dim_heads))

    def redraw_projection_matrix(self, device=None):
        r, c = self.projection_matrix.shape
        self.projection_matrix.copy_(_gaussian_orthogonal_random_matrix(r, c, device=device or self.projection_matrix.device))

    def forward(self, q, k, v):
        qp = _softmax_kernel(q, projection_matrix=self.projection_matrix, is_query=True)
        kp = _softmax_kernel(k, projection_matrix=self.projection_matrix, is_query=False)
        return _linear_attention(qp, kp, v)


class GPSCoreAttention(SparseCoreAttention):
    variant = "gps"

    def __init__(self, hidden_size, attention_dropout_rate, num_heads):
        super().__init__(hidden_size, attention_dropout_rate, num_heads)
        self.performer = PerformerFastAttention(self.hidden_size_per_attention_head)

    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None, **kw):
        attn_type = "sparse" if attn_type is None else str(attn_type).lower()
        if attn_type == "performer":
            b, s = q.size(0), q.size(1)
            x = self.performer(q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2).float())
            x = self.att_dropout(x).to(q.dtype)
            return x.transpose(1, 2).contiguous().view(b, s, -1)
        if attn_type == "full":
            return super().forward(q, k, v, None, edge_index, "full")
        return super().forward(q, k, v, None, edge_index, "sparse")


class MultiHeadAttention(nn.Module):
    def __init__(self, hidden_size, attention_dropout_rate, num_heads, attn_type="sparse"):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        qkv_bias = str(attn_type).lower() == "full"
        self.linear_q = nn.Linear(hidden_size, num_heads * self.att_size, bias=qkv_bias)
        self.linear_k = nn.Linear(hidden_size, num_heads * self.att_size, bias=qkv_bias)
        self.linear_v = nn.Linear(hidden_size, num_heads * self.att_size, bias=qkv_bias)
        self.out_proj = nn.Linear(hidden_size, hidden_size)
        self.dist_attn = DistributedAttentionNodeLevel(
            GPSCoreAttention(hidden_size, attention_dropout_rate, num_heads), get_sequence_parallel_group())

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None):
        b = x.size(0)
        q = self.linear_q(x).view(b, -1, self.num_heads, self.att_size)
        k = self.linear_k(x).view(b, -1, self.num_heads, self.att_size)
        v = self.linear_v(x).view(b, -1, self.num_heads, self.att_size)
        return self.out_proj(self.dist_attn(q, k, v, attn_bias, edge_index, attn_type))


class EncoderLayer(nn.Module):
    def __init__(self, hidden_size, dropout_rate, attention_dropout_rate, num_heads, attn_type="sparse"):
        super().__init__()
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads, attn_type=attn_type)
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


class GraphGPS(NodeModelBase):
    def __init__(self, n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
                 input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node, attn_type="sparse", **kwargs):
        super().__init__()
        self.node_encoder = nn.Linear(input_dim, hidden_dim)
        self.layers = nn.ModuleList([
            EncoderLayer(hidden_dim, dropout_rate, attention_dropout_rate, num_heads, attn_type=attn_type)
            for _ in range(n_layers)])
        self.output_proj = nn.Linear(hidden_dim, output_dim)
        self._init_ckpt_state()

    def redraw_performer_projections(self, device=None):
        for core in self.core_attention_modules():
            if hasattr(core, "performer"):
                core.performer.redraw_projection_matrix(device=device)

    def forward_logits(self, x, attn_bias, edge_index, attn_type=None):
        x = encode_features(self.node_encoder, x).unsqueeze(0)
        x = self._run_layers(x, attn_bias=attn_bias, edge_index=edge_index, attn_type=attn_type)
        from ..ops.gemm import readout_linear
        return readout_linear(x.squeeze(0), self.output_proj.weight, self.output_proj.bias)

    def forward(self, x, attn_bias, edge_index, attn_type=None):
        return F.log_softmax(self.forward_logits(x, attn_bias, edge_index, attn_type), dim=1)
