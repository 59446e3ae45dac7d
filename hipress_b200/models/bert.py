"""BERT for masked-LM pre-training.  ``bert_large`` = 24 layers, hidden 1024, 16 heads,
FFN 4096, vocabulary 30522 (~340 M parameters with tied output embedding)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import FusedAddLayerNorm, FusedLinear


class BertLayer(nn.Module):
    """Post-LN transformer layer.  Separate query / key / value projections give the attention
    kernel three dense [batch, seq, heads, head_dim] operands and its output the same layout, so
    neither forward nor backward needs a permute copy or a concatenation of the three gradients;
    residual add + LayerNorm run fused on a bf16 residual stream (``layers.FusedAddLayerNorm``)."""

    def __init__(self, hidden: int, heads: int, ffn: int, dropout: float):
        super().__init__()
        self.heads = heads
        self.q = FusedLinear(hidden, hidden)
        self.k = FusedLinear(hidden, hidden)
        self.v = FusedLinear(hidden, hidden)
        self.out = FusedLinear(hidden, hidden)
        self.ln1 = FusedAddLayerNorm(hidden, eps=1e-12)
        self.fc1 = FusedLinear(hidden, ffn)
        self.fc2 = FusedLinear(ffn, hidden)
        self.ln2 = FusedAddLayerNorm(hidden, eps=1e-12)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        b, s, h = x.shape
        shape = (b, s, self.heads, h // self.heads)
        q = self.q(x).view(shape).transpose(1, 2)
        k = self.k(x).view(shape).transpose(1, 2)
        v = self.v(x).view(shape).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v)
        a = a.transpose(1, 2).reshape(b, s, h)
        x = self.ln1(x, self.drop(self.out(a)))
        return self.ln2(x, self.drop(self.fc2(F.gelu(self.fc1(x)))))


class BertForMaskedLM(nn.Module):
    def __init__(self, vocab: int = 30522, hidden: int = 1024, layers: int = 24, heads: int = 16,
                 ffn: int = 4096, max_pos: int = 512, dropout: float = 0.1):
        super().__init__()
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.typ = nn.Embedding(2, hidden)
        self.ln = FusedAddLayerNorm(hidden, eps=1e-12)
        self.drop = nn.Dropout(dropout)
        self.layers = nn.ModuleList(BertLayer(hidden, heads, ffn, dropout) for _ in range(layers))
        self.head_dense = FusedLinear(hidden, hidden)
        self.head_ln = FusedAddLayerNorm(hidden, eps=1e-12)
        self.head_bias = nn.Parameter(torch.zeros(vocab))
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, 0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, ids: torch.Tensor, labels: torch.Tensor | None = None):
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device)
        emb = self.tok(ids) + self.pos(pos)[None] + self.typ.weight[0]
        if emb.is_cuda and torch.is_autocast_enabled():
            emb = emb.to(torch.get_autocast_dtype("cuda"))   # the residual stream runs in the compute dtype
        x = self.drop(self.ln(emb))
        for layer in self.layers:
            x = layer(x)
        if labels is None:
            h = self.head_ln(F.gelu(self.head_dense(x)))
            return F.linear(h, self.tok.weight, self.head_bias)
        # score only the masked positions (labels == -100 elsewhere)
        flat = labels.view(-1)
        cap = getattr(self, "masked_capacity", None)
        if cap:
            # fixed-shape selection (no host round trip, so the step can be captured in a CUDA
            # graph): the `cap` positions picked contain every masked one as long as
            # cap >= their count; the rest carry label -100 and are ignored by the loss
            idx = torch.topk((flat >= 0).to(torch.float32), min(int(cap), flat.numel()), sorted=False).indices
            h = x.view(b * s, -1).index_select(0, idx)
            target = flat.index_select(0, idx)
        else:
            sel = flat >= 0
            h = x.view(b * s, -1)[sel]
            target = flat[sel]
        h = self.head_ln(F.gelu(self.head_dense(h)))
        logits = F.linear(h, self.tok.weight, self.head_bias)
        return F.cross_entropy(logits.float(), target, ignore_index=-100)


def bert_large() -> BertForMaskedLM:
    return BertForMaskedLM()


def bert_tiny() -> BertForMaskedLM:
    return BertForMaskedLM(vocab=1000, hidden=64, layers=2, heads=4, ffn=128, max_pos=64, dropout=0.0)
