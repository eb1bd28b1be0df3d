"""One encoder layer of each model family in float32, from a plain ``{name: tensor}`` dict of that layer's weights
(the names are the layer's ``state_dict`` keys).  Dropout is off (evaluation numerics); BatchNorm uses the statistics
of the rows it is given, as a training step does on a rank's local rows (models/graphgps_dist_node_level.py:270-272).

``x`` is ``[n, h]``; ``edge_index`` the int64 COO of the attention graph over those ``n`` rows."""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F

from . import attention


def _lin(x, w: Dict[str, torch.Tensor], name: str):
    b = w.get(name + ".bias")
    return F.linear(x, w[name + ".weight"].float(), None if b is None else b.float())


def _ln(x, w, name: str, eps: float = 1e-5):
    return F.layer_norm(x, (x.size(-1),), w[name + ".weight"].float(), w[name + ".bias"].float(), eps)


def _bn_train(x, w, name: str, eps: float = 1e-5):
    mean = x.mean(0)
    var = x.var(0, unbiased=False)
    return (x - mean) / torch.sqrt(var + eps) * w[name + ".weight"].float() + w[name + ".bias"].float()


def _heads(t, num_heads: int):
    return t.view(t.size(0), num_heads, -1)


def _qkv(x, w, num_heads, prefix="self_attention."):
    return tuple(_heads(_lin(x, w, prefix + f"linear_{c}"), num_heads) for c in "qkv")


def gt_layer(x, w, edge_index, num_heads: int):
    """Post-LN: ``h = LN1(x + O(attn(x)))``, ``LN2(h + FFN2(relu(FFN1(h))))`` (models/gt_dist_node_level.py:631-684)."""
    x = x.float()
    q, k, v = _qkv(x, w, num_heads)
    a = attention.sparse_attention(q, k, v, edge_index).reshape(x.size(0), -1)
    h = _ln(x + _lin(a, w, "O"), w, "layer_norm1")
    y = _lin(F.relu(_lin(h, w, "FFN_layer1")), w, "FFN_layer2")
    return _ln(h + y, w, "layer_norm2")


def graphormer_layer(x, w, edge_index, num_heads: int):
    """Pre-LN with a GELU FFN: ``x += out(attn(LN(x)))``, ``x += FFN(LN(x))``
    (models/graphormer_dist_node_level.py:705-724)."""
    x = x.float()
    y = _ln(x, w, "self_attention_norm")
    q, k, v = _qkv(y, w, num_heads)
    a = attention.sparse_attention(q, k, v, edge_index).reshape(x.size(0), -1)
    x = x + _lin(a, w, "self_attention.output_layer")
    y = _ln(x, w, "ffn_norm")
    return x + _lin(F.gelu(_lin(y, w, "ffn.layer1")), w, "ffn.layer2")


def graphgps_layer(x, w, edge_index, num_heads: int):
    """Post-norm BatchNorm over the given rows, ReLU FFN of width 2h (models/graphgps_dist_node_level.py:255-293)."""
    x = x.float()
    q, k, v = _qkv(x, w, num_heads)
    a = attention.gps_attention(q, k, v, edge_index).reshape(x.size(0), -1)
    h = _bn_train(x + _lin(a, w, "self_attention.out_proj"), w, "norm1")
    y = _lin(F.relu(_lin(h, w, "ffn1")), w, "ffn2")
    return _bn_train(h + y, w, "norm2")


def exphormer_layer(x, w, edge_index, num_heads: int):
    """No output projection; the edge-type table modulates the scores (models/exphormer_dist_node_level.py:160-202)."""
    x = x.float()
    q, k, v = _qkv(x, w, num_heads)
    core = "self_attention.dist_attn.local_attn."
    if core + "edge_type_emb.weight" not in w:
        core = "self_attention.dist_attn."
    if edge_index.size(0) >= 3:
        a = attention.exphormer_attention(q, k, v, edge_index, w[core + "edge_type_emb.weight"], w[core + "edge_proj.weight"])
    else:
        a = attention.sparse_attention(q, k, v, edge_index)
    h = _bn_train(x + a.reshape(x.size(0), -1), w, "norm1")
    y = _lin(F.relu(_lin(h, w, "ffn1")), w, "ffn2")
    return _bn_train(h + y, w, "norm2")


LAYERS = {"gt": gt_layer, "graphormer": graphormer_layer, "graphgps": graphgps_layer, "exphormer": exphormer_layer}
