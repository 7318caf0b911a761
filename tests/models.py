"""nn.Modules of the benchmark configurations, as a user of ``DaceModule`` would write them (shared by the importer
tests on CPU and GPU).  ``efficientnet_pytorch`` is not installed, so the MBConv block is restated with plain
``nn.Conv2d`` modules and folded BatchNorm, like the hand-built graph."""
import warnings

import torch
import torch.nn as nn
import torch.nn.functional as F


class MLP(nn.Module):
    """The README network of the reference (``README.md:48-76``): 784 -> 120 -> 32 -> 10, LogSoftmax."""

    def __init__(self):
        super().__init__()
        self.fc1, self.fc2, self.fc3 = nn.Linear(784, 120), nn.Linear(120, 32), nn.Linear(32, 10)
        self.ls = nn.LogSoftmax(dim=-1)

    def forward(self, x):
        return self.ls(self.fc3(F.relu(self.fc2(F.relu(self.fc1(x))))))


class Swish(nn.Module):
    def forward(self, x):
        return x * torch.sigmoid(x)


class MBConv(nn.Module):
    def __init__(self, cin=24, mid=144, red=6):
        super().__init__()
        self.expand = nn.Conv2d(cin, mid, 1)
        self.depthwise = nn.Conv2d(mid, mid, 3, padding=1, groups=mid)
        self.se_reduce, self.se_expand = nn.Conv2d(mid, red, 1), nn.Conv2d(red, mid, 1)
        self.project = nn.Conv2d(mid, cin, 1)
        self.swish = Swish()

    def forward(self, x):
        y = self.swish(self.expand(x))
        y = self.swish(self.depthwise(y))
        s = F.adaptive_avg_pool2d(y, 1)
        s = self.se_expand(self.swish(self.se_reduce(s)))
        y = torch.sigmoid(s) * y
        return self.project(y) + x


def bert_layer(hidden, heads, ffn, seed=0):
    """HF ``BertLayer`` with eager attention, eval mode, as ``tests/torch/test_bert_encoder.py:11-33`` builds it."""
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from transformers import BertConfig
        from transformers.models.bert.modeling_bert import BertLayer
    torch.manual_seed(seed)
    cfg = BertConfig(hidden_size=hidden, num_attention_heads=heads, intermediate_size=ffn)
    cfg._attn_implementation = "eager"
    return BertLayer(cfg).eval()
