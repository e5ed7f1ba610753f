"""BERT-large encoder (24 layers, hidden 1024, 16 heads, ~335 M parameters) with a masked-LM
head, for the bf16 benchmark with server-side Adam.

The reference has no model code.  The first GEMM that consumes pulled weights -- the fused
QKV projection of layer 0, X[tokens,1024] * W[3072,1024]^T -- can run as the kernel that also
pulls W (``ps_lite_b200.ops.gemm.pull_linear_bf16``); everything else is plain PyTorch.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class Layer(nn.Module):
    def __init__(self, hidden: int, heads: int, ffn: int):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(hidden, 3 * hidden)
        self.proj = nn.Linear(hidden, hidden)
        self.ln1 = nn.LayerNorm(hidden)
        self.fc1 = nn.Linear(hidden, ffn)
        self.fc2 = nn.Linear(ffn, hidden)
        self.ln2 = nn.LayerNorm(hidden)
        self.qkv_fn: Optional[Callable] = None  # replacement for the QKV matmul (fused pull)

    def forward(self, x):
        B, S, H = x.shape
        if self.qkv_fn is not None:
            qkv = self.qkv_fn(x) + self.qkv.bias
        else:
            qkv = self.qkv(x)
        q, k, v = qkv.view(B, S, 3, self.heads, H // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v)
        a = a.transpose(1, 2).reshape(B, S, H)
        x = self.ln1(x + self.proj(a))
        return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))


class BertLarge(nn.Module):
    def __init__(self, vocab: int = 30522, hidden: int = 1024, layers: int = 24, heads: int = 16,
                 ffn: int = 4096, max_seq: int = 512):
        super().__init__()
        # layer 0 first, so that its QKV weight is the first parameter of the model
        self.layers = nn.ModuleList([Layer(hidden, heads, ffn) for _ in range(layers)])
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_seq, hidden)
        self.ln = nn.LayerNorm(hidden)
        self.head = nn.Linear(hidden, hidden)
        self.head_ln = nn.LayerNorm(hidden)
        self.decoder_bias = nn.Parameter(torch.zeros(vocab))
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, ids, labels=None):
        B, S = ids.shape
        x = self.ln(self.tok(ids) + self.pos(torch.arange(S, device=ids.device))[None])
        for layer in self.layers:
            x = layer(x)
        h = self.head_ln(F.gelu(self.head(x)))
        logits = h @ self.tok.weight.t() + self.decoder_bias
        if labels is None:
            return logits
        return F.cross_entropy(logits.view(B * S, -1).float(), labels.view(-1))
