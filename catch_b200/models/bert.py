"""BERT encoder with a sequence-classification head (BERT-base by default:
12 layers, hidden 768, 12 heads, FFN 3072, vocabulary 30522).

The reference lists BERT among the networks it trains
(docs/user_guide/source/pytorch_8_training/Pytorch_training.rst:10-18) with plain
matmul / bmm / softmax eager ops; this definition uses exactly those ops (embedding,
LayerNorm, linear, bmm, softmax, GELU, dropout), all of which have kernels in this
backend.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-12
    num_labels: int = 2


class BertEmbeddings(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embeddings = nn.Embedding(c.max_position_embeddings, c.hidden_size)
        self.token_type_embeddings = nn.Embedding(c.type_vocab_size, c.hidden_size)
        self.LayerNorm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)
        self.dropout = nn.Dropout(c.hidden_dropout_prob)
        self.register_buffer("position_ids", torch.arange(c.max_position_embeddings).unsqueeze(0), persistent=False)

    def forward(self, input_ids, token_type_ids=None):
        L = input_ids.shape[1]
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        x = (self.word_embeddings(input_ids) + self.position_embeddings(self.position_ids[:, :L]) +
             self.token_type_embeddings(token_type_ids))
        return self.dropout(self.LayerNorm(x))


class BertSelfAttention(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.h, self.d = c.num_attention_heads, c.hidden_size // c.num_attention_heads
        self.query = nn.Linear(c.hidden_size, c.hidden_size)
        self.key = nn.Linear(c.hidden_size, c.hidden_size)
        self.value = nn.Linear(c.hidden_size, c.hidden_size)
        self.dropout = nn.Dropout(c.attention_probs_dropout_prob)

    def forward(self, x, mask=None):
        B, L, H = x.shape

        def split(t):  # [B, L, H] -> [B*h, L, d]
            return t.view(B, L, self.h, self.d).permute(0, 2, 1, 3).reshape(B * self.h, L, self.d)

        q, k, v = split(self.query(x)), split(self.key(x)), split(self.value(x))
        scores = torch.bmm(q, k.transpose(1, 2)) * (1.0 / math.sqrt(self.d))
        if mask is not None:
            scores = scores.view(B, self.h, L, L) + mask
            scores = scores.view(B * self.h, L, L)
        probs = self.dropout(torch.softmax(scores, dim=-1))
        ctx = torch.bmm(probs, v).view(B, self.h, L, self.d).permute(0, 2, 1, 3).reshape(B, L, H)
        return ctx


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.attention = BertSelfAttention(c)
        self.attn_out = nn.Linear(c.hidden_size, c.hidden_size)
        self.attn_norm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)
        self.intermediate = nn.Linear(c.hidden_size, c.intermediate_size)
        self.output = nn.Linear(c.intermediate_size, c.hidden_size)
        self.out_norm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)
        self.dropout = nn.Dropout(c.hidden_dropout_prob)
        self.act = nn.GELU()

    def forward(self, x, mask=None):
        x = self.attn_norm(x + self.dropout(self.attn_out(self.attention(x, mask))))
        return self.out_norm(x + self.dropout(self.output(self.act(self.intermediate(x)))))


class FusedBertSelfAttention(BertSelfAttention):
    """Same parameters; the head split is a view and the two batched products read / write those views directly
    (``catch_b200.fusion.matmul_nd``), so no [batch * heads, seq, dim] copies are made in either direction."""

    def forward(self, x, mask=None):
        from catch_b200.fusion import matmul_nd

        if x.device.type != "blackwell" or not torch.is_autocast_enabled("blackwell"):
            return super().forward(x, mask)
        B, L, H = x.shape
        cd = torch.get_autocast_dtype("blackwell")

        def heads(t):  # [B, L, H] -> [B, h, L, d] view
            return t.to(cd).view(B, L, self.h, self.d).permute(0, 2, 1, 3)

        q, k, v = heads(self.query(x)), heads(self.key(x)), heads(self.value(x))
        scores = matmul_nd(q, k.transpose(-1, -2), 1.0 / math.sqrt(self.d))
        if mask is not None:
            scores = scores + mask.to(scores.dtype)
        with torch.autocast("blackwell", enabled=False):  # the softmax kernel computes in fp32 whatever the storage type
            probs = torch.softmax(scores, dim=-1)
        probs = self.dropout(probs)
        # the context is produced straight in [B, L, h, d] memory, seen as [B, h, L, d] by the product
        ctx = matmul_nd(probs, v, 1.0, (L * H, self.d, H, 1))
        return ctx.permute(0, 2, 1, 3).reshape(B, L, H)


class FusedBertLayer(BertLayer):
    """Same parameters; ``norm(x + dropout(h))`` runs as one fused kernel per direction."""

    def forward(self, x, mask=None):
        from catch_b200.fusion import dropout_add_layer_norm

        if x.device.type != "blackwell":
            return super().forward(x, mask)
        h = self.attn_out(self.attention(x, mask))
        x = dropout_add_layer_norm(h, x.to(h.dtype), self.attn_norm, self.dropout.p, self.training)
        h = self.output(self.act(self.intermediate(x)))
        return dropout_add_layer_norm(h, x.to(h.dtype), self.out_norm, self.dropout.p, self.training)


def fuse_bert(model: nn.Module) -> nn.Module:
    """Switch the layers of a BERT model to their fused forms and its linears to ``FusedLinear`` (in place; the
    parameters and the state dict are unchanged)."""
    from catch_b200.fusion import fuse_linear

    for m in model.modules():
        if type(m) is BertLayer:
            m.__class__ = FusedBertLayer
        elif type(m) is BertSelfAttention:
            m.__class__ = FusedBertSelfAttention
    return fuse_linear(model)


class BertForSequenceClassification(nn.Module):
    def __init__(self, config: BertConfig = None):
        super().__init__()
        c = self.config = config or BertConfig()
        self.embeddings = BertEmbeddings(c)
        self.layers = nn.ModuleList(BertLayer(c) for _ in range(c.num_hidden_layers))
        self.pooler = nn.Linear(c.hidden_size, c.hidden_size)
        self.dropout = nn.Dropout(c.hidden_dropout_prob)
        self.classifier = nn.Linear(c.hidden_size, c.num_labels)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None):
        mask = None
        if attention_mask is not None:
            mask = (1.0 - attention_mask[:, None, None, :].to(torch.float32)) * -10000.0
        x = self.embeddings(input_ids, token_type_ids)
        for layer in self.layers:
            x = layer(x, mask)
        pooled = torch.tanh(self.pooler(x[:, 0]))
        return self.classifier(self.dropout(pooled))
