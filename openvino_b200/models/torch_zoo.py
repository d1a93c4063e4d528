"""Plain PyTorch definitions of the benchmark architectures (random weights; no downloads).

ResNet-18 (He et al. 2015, ImageNet layout), a BERT encoder (Devlin et al. 2018; ``bert_large`` = 24 layers,
hidden 1024, 16 heads) and a Llama-style decoder block stack. They are inputs for ``convert_model`` in tests
and benchmarks, and the numerical oracle the converted models are compared against.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.downsample = None
        if stride != 1 or cin != cout:
            self.downsample = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return F.relu(y + idt)


class ResNet18(nn.Module):
    def __init__(self, num_classes: int = 1000, width: int = 64):
        super().__init__()
        w = width
        self.conv1 = nn.Conv2d(3, w, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(w)
        self.layer1 = nn.Sequential(BasicBlock(w, w, 1), BasicBlock(w, w, 1))
        self.layer2 = nn.Sequential(BasicBlock(w, 2 * w, 2), BasicBlock(2 * w, 2 * w, 1))
        self.layer3 = nn.Sequential(BasicBlock(2 * w, 4 * w, 2), BasicBlock(4 * w, 4 * w, 1))
        self.layer4 = nn.Sequential(BasicBlock(4 * w, 8 * w, 2), BasicBlock(8 * w, 8 * w, 1))
        self.fc = nn.Linear(8 * w, num_classes)
        for m in self.modules():
            if isinstance(m, nn.BatchNorm2d):   # non-trivial statistics so that BN folding is really exercised
                nn.init.uniform_(m.weight, 0.5, 1.5)
                nn.init.uniform_(m.bias, -0.2, 0.2)
                m.running_mean.uniform_(-0.2, 0.2)
                m.running_var.uniform_(0.5, 1.5)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.bn1(self.conv1(x))), 3, 2, 1)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = F.adaptive_avg_pool2d(x, 1).flatten(1)
        return self.fc(x)


class BertLayer(nn.Module):
    def __init__(self, hidden, heads, inter):
        super().__init__()
        self.heads = heads
        self.q, self.k, self.v, self.o = (nn.Linear(hidden, hidden) for _ in range(4))
        self.ln1 = nn.LayerNorm(hidden, eps=1e-12)
        self.up = nn.Linear(hidden, inter)
        self.down = nn.Linear(inter, hidden)
        self.ln2 = nn.LayerNorm(hidden, eps=1e-12)

    def forward(self, x, mask):
        b, s, h = x.shape
        d = h // self.heads
        q = self.q(x).view(b, s, self.heads, d).transpose(1, 2)
        k = self.k(x).view(b, s, self.heads, d).transpose(1, 2)
        v = self.v(x).view(b, s, self.heads, d).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        a = a.transpose(1, 2).reshape(b, s, h)
        x = self.ln1(x + self.o(a))
        return self.ln2(x + self.down(F.gelu(self.up(x))))


class Bert(nn.Module):
    def __init__(self, vocab=30522, hidden=1024, layers=24, heads=16, inter=4096, max_pos=512):
        super().__init__()
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.typ = nn.Embedding(2, hidden)
        self.ln = nn.LayerNorm(hidden, eps=1e-12)
        self.layers = nn.ModuleList(BertLayer(hidden, heads, inter) for _ in range(layers))

    def forward(self, input_ids, attention_mask, token_type_ids):
        s = input_ids.shape[1]
        pos = torch.arange(s, device=input_ids.device).unsqueeze(0)
        x = self.ln(self.tok(input_ids) + self.pos(pos) + self.typ(token_type_ids))
        mask = (1.0 - attention_mask[:, None, None, :].to(x.dtype)) * -10000.0
        for layer in self.layers:
            x = layer(x, mask)
        return x


def bert_large(**kw) -> Bert:
    return Bert(hidden=1024, layers=24, heads=16, inter=4096, **kw)


def bert_tiny(**kw) -> Bert:
    return Bert(vocab=100, hidden=32, layers=2, heads=4, inter=64, max_pos=64, **kw)
