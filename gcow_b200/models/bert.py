"""BERT encoder with the masked-LM + next-sentence pre-training heads.

BERT-large = 24 layers, hidden 1024, 16 heads, FFN 4096, vocabulary 30522,
sequence 512. The reference contains CNNs only; this family is part of the
training configurations this framework is measured on. Layers come from
gcow_b200.ops.nn (Linear / LayerNorm / attention / GELU / embedding /
cross-entropy) so the sm_100a kernels are used where they exist.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import nn as gnn


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    ffn: int = 4096
    max_pos: int = 512
    type_vocab: int = 2
    eps: float = 1e-12


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.heads = c.heads
        self.qkv = gnn.Linear(c.hidden, 3 * c.hidden)
        self.proj = gnn.Linear(c.hidden, c.hidden)
        self.ln1 = gnn.LayerNorm(c.hidden, eps=c.eps)
        self.fc1 = gnn.Linear(c.hidden, c.ffn)
        self.fc2 = gnn.Linear(c.ffn, c.hidden)
        self.ln2 = gnn.LayerNorm(c.hidden, eps=c.eps)

    def forward(self, x):                      # x: [B, S, H]
        B, S, H = x.shape
        qkv = self.qkv(x).view(B, S, 3, self.heads, H // self.heads)
        ctx = gnn.attention(qkv)               # [B, S, H]
        x = self.ln1(gnn.linear_residual(ctx, self.proj, x))
        return self.ln2(gnn.ffn_residual(x, self.fc1, self.fc2))


class BertForPreTraining(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.cfg = c
        self.tok = gnn.Embedding(c.vocab_size, c.hidden)
        self.pos = gnn.Embedding(c.max_pos, c.hidden)
        self.typ = gnn.Embedding(c.type_vocab, c.hidden)
        self.ln = gnn.LayerNorm(c.hidden, eps=c.eps)
        self.layers = nn.ModuleList([BertLayer(c) for _ in range(c.layers)])
        self.mlm_dense = gnn.Linear(c.hidden, c.hidden)
        self.mlm_ln = gnn.LayerNorm(c.hidden, eps=c.eps)
        self.mlm_bias = nn.Parameter(torch.zeros(c.vocab_size))
        self.pooler = gnn.Linear(c.hidden, c.hidden)
        self.nsp = gnn.Linear(c.hidden, 2)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, ids, type_ids=None, mlm_labels=None, nsp_labels=None):
        B, S = ids.shape
        if type_ids is None:                      # single-segment input: every token is type 0
            type_ids = torch.zeros_like(ids)
        x = self.ln(gnn.embed_sum3(ids, type_ids, self.tok, self.pos, self.typ))
        for layer in self.layers:
            x = layer(x)
        h = self.mlm_ln(gnn.gelu(self.mlm_dense(x)))
        logits = gnn.linear(h, self.tok.weight, self.mlm_bias)      # tied decoder [B, S, V]
        if mlm_labels is None:
            return logits
        loss = gnn.cross_entropy(logits.view(B * S, -1), mlm_labels.view(-1), ignore_index=-100)
        if nsp_labels is not None:
            pooled = torch.tanh(self.pooler(x[:, 0]))
            loss = loss + gnn.cross_entropy(self.nsp(pooled), nsp_labels)
        return loss


def bert_large(**kw): return BertForPreTraining(BertConfig(**kw))
def bert_base(**kw): return BertForPreTraining(BertConfig(hidden=768, layers=12, heads=12, ffn=3072, **kw))
def bert_tiny(**kw): return BertForPreTraining(BertConfig(vocab_size=1024, hidden=128, layers=2, heads=2, ffn=512, max_pos=128, **kw))
