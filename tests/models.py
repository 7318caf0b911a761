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


class TinyBert(nn.Module):
    """Embeddings + HF encoder layers + pooler, with the additive attention mask computed inside the graph the way
    BERT implementations do (``(1 - mask) * -10000`` broadcast over heads and queries).  The whole-model class of
    ``transformers`` does not survive TorchScript tracing in this version, so the pieces are assembled here."""

    def __init__(self, vocab=1000, hidden=128, heads=2, ffn=256, layers=2, max_pos=64, seed=0):
        super().__init__()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            from transformers import BertConfig
            from transformers.models.bert.modeling_bert import BertLayer
        torch.manual_seed(seed)
        cfg = BertConfig(hidden_size=hidden, num_attention_heads=heads, intermediate_size=ffn)
        cfg._attn_implementation = "eager"
        self.tok, self.pos = nn.Embedding(vocab, hidden), nn.Embedding(max_pos, hidden)
        self.norm = nn.LayerNorm(hidden, eps=1e-12)
        self.layers = nn.ModuleList([BertLayer(cfg) for _ in range(layers)])
        self.pooler = nn.Linear(hidden, hidden)

    def forward(self, ids, mask):
        h = self.norm(self.tok(ids) + self.pos.weight[:ids.shape[1]])
        ext = (1.0 - mask[:, None, None, :].to(h.dtype)) * -10000.0
        for layer in self.layers:
            out = layer(h, attention_mask=ext)
            h = out[0] if isinstance(out, tuple) else out
        return h, torch.tanh(self.pooler(h[:, 0]))


class LeNet(nn.Module):
    """The classic 32x32 LeNet (two 3x3 convolutions with ReLU and 2x2 max pooling, three linear layers, log-softmax):
    the network of the reference's ``tests/torch/test_lenet.py``."""

    def __init__(self):
        super().__init__()
        self.conv1, self.conv2 = nn.Conv2d(1, 6, 3), nn.Conv2d(6, 16, 3)
        self.fc1, self.fc2, self.fc3 = nn.Linear(16 * 6 * 6, 120), nn.Linear(120, 84), nn.Linear(84, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = x.view(-1, 16 * 6 * 6)
        x = F.relu(self.fc2(F.relu(self.fc1(x))))
        return F.log_softmax(self.fc3(x), dim=1)
