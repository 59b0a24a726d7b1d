"""Same-box library baseline: the benchmark models written with stock PyTorch modules only.

Nothing here touches the framework's kernels or engines: BERT-large pre-training runs on ``F.linear`` (cuBLAS),
``F.scaled_dot_product_attention``, ``F.layer_norm`` and ``torch.optim.Adam(fused=True)``; ResNet-101 / VGG-16 on
``nn.Conv2d`` / ``nn.BatchNorm2d`` (cuDNN) in channels-last with ``torch.optim.SGD``; both under bf16 autocast with fp32
master weights and ``DistributedDataParallel`` (NCCL) when there is more than one rank. ``bench.py --impl library`` times
them with the harness of the main arm (same config, batch, steps, warm-up and end-to-end definition).

Model definitions follow the reference's benchmark drivers: ``examples/benchmark/bert.py:54-74`` (BERT-large, sequence
length 128, 20 masked positions) and ``examples/benchmark/imagenet.py:232-249`` (Keras application CNNs).
"""
import torch
from torch import nn
import torch.nn.functional as F


class LibraryBert(nn.Module):
    """BERT pre-training (MLM + NSP heads, untied MLM decoder like the framework's model) on library ops."""

    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        H, Fd, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
        self.word = nn.Embedding(V, H)
        self.pos = nn.Embedding(cfg.max_position_embeddings, H)
        self.tok = nn.Embedding(cfg.type_vocab_size, H)
        self.emb_ln = nn.LayerNorm(H, eps=cfg.layer_norm_eps)
        self.layers = nn.ModuleList()
        for _ in range(cfg.num_hidden_layers):
            self.layers.append(nn.ModuleDict({
                "qkv": nn.Linear(H, 3 * H), "out": nn.Linear(H, H), "ln1": nn.LayerNorm(H, eps=cfg.layer_norm_eps),
                "w1": nn.Linear(H, Fd), "w2": nn.Linear(Fd, H), "ln2": nn.LayerNorm(H, eps=cfg.layer_norm_eps)}))
        self.pooler = nn.Linear(H, H)
        self.nsp = nn.Linear(H, 2)
        self.mlm_dense = nn.Linear(H, H)
        self.mlm_ln = nn.LayerNorm(H, eps=cfg.layer_norm_eps)
        self.decoder = nn.Linear(H, V)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=cfg.initializer_range)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, input_ids, input_mask, segment_ids, mlm_positions, mlm_ids, mlm_weights, nsp_labels):
        c = self.cfg
        B, S = input_ids.shape
        H, nh = c.hidden_size, c.num_attention_heads
        D = H // nh
        pos = torch.arange(S, device=input_ids.device)
        x = self.emb_ln(self.word(input_ids) + self.pos(pos)[None] + self.tok(segment_ids))
        mask = ((1.0 - input_mask.to(torch.float32)) * -10000.0)[:, None, None, :].to(torch.bfloat16)
        pd_h, pd_a = c.hidden_dropout_prob, c.attention_probs_dropout_prob
        for L in self.layers:
            qkv = L["qkv"](x).view(B, S, 3, nh, D)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
            ctx = F.scaled_dot_product_attention(q, k, v, attn_mask=mask.to(q.dtype), dropout_p=pd_a if self.training else 0.0)
            ctx = ctx.transpose(1, 2).reshape(B, S, H)
            x = L["ln1"](F.dropout(L["out"](ctx), pd_h, self.training) + x)
            x = L["ln2"](F.dropout(L["w2"](F.gelu(L["w1"](x), approximate="tanh")), pd_h, self.training) + x)
        pooled = torch.tanh(self.pooler(x[:, 0]))
        nsp_loss = F.cross_entropy(self.nsp(pooled).float(), nsp_labels.view(-1))
        flat_pos = (mlm_positions + torch.arange(B, device=x.device)[:, None] * S).view(-1)
        hm = self.mlm_ln(F.gelu(self.mlm_dense(x.reshape(B * S, H)[flat_pos]), approximate="tanh"))
        per = F.cross_entropy(self.decoder(hm).float(), mlm_ids.view(-1), reduction="none")
        w = mlm_weights.view(-1).float()
        return (per * w).sum() / (w.sum() + 1e-5) + nsp_loss


class _Bottleneck(nn.Module):
    def __init__(self, cin, width, stride):
        super().__init__()
        cout = width * 4
        self.c1, self.b1 = nn.Conv2d(cin, width, 1, bias=False), nn.BatchNorm2d(width)
        self.c2, self.b2 = nn.Conv2d(width, width, 3, stride, 1, bias=False), nn.BatchNorm2d(width)
        self.c3, self.b3 = nn.Conv2d(width, cout, 1, bias=False), nn.BatchNorm2d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        idn = x if self.down is None else self.down(x)
        y = F.relu(self.b1(self.c1(x)), inplace=True)
        y = F.relu(self.b2(self.c2(y)), inplace=True)
        return F.relu(self.b3(self.c3(y)) + idn, inplace=True)


class LibraryResNet(nn.Module):
    def __init__(self, blocks=(3, 4, 23, 3), num_classes=1000):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64), nn.ReLU(inplace=True), nn.MaxPool2d(3, 2, 1))
        layers, cin = [], 64
        for i, n in enumerate(blocks):
            for j in range(n):
                layers.append(_Bottleneck(cin, 64 * 2 ** i, 2 if (j == 0 and i > 0) else 1))
                cin = 256 * 2 ** i
        self.layers = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, num_classes)

    def forward(self, x):
        x = self.layers(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


class LibraryVGG16(nn.Module):
    CFG = (64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M")

    def __init__(self, num_classes=1000):
        super().__init__()
        layers, cin = [], 3
        for v in self.CFG:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(cin, v, 3, 1, 1), nn.ReLU(inplace=True)]
                cin = v
        self.features = nn.Sequential(*layers)
        self.classifier = nn.Sequential(nn.Linear(512 * 7 * 7, 4096), nn.ReLU(inplace=True), nn.Linear(4096, 4096), nn.ReLU(inplace=True),
                                        nn.Linear(4096, num_classes))

    def forward(self, x):
        return self.classifier(torch.flatten(self.features(x), 1))


class LibraryImageClassifier(nn.Module):
    def __init__(self, backbone):
        super().__init__()
        self.net = {"resnet101": lambda: LibraryResNet((3, 4, 23, 3)), "resnet50": lambda: LibraryResNet((3, 4, 6, 3)),
                    "vgg16": LibraryVGG16}[backbone]()

    def forward(self, images, labels):
        return F.cross_entropy(self.net(images).float(), labels)


def build(model_name, device):
    """(module on ``device`` in training mode, optimizer, is_bert)."""
    if model_name.startswith("bert"):
        from autodist_b200.models.bert import BertConfig            # the configuration record only: no kernels involved
        cfg = {"bert-large": BertConfig.large, "bert-base": BertConfig.base, "bert-tiny": BertConfig.tiny}[model_name]()
        model = LibraryBert(cfg).to(device)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, fused=True)
        return model.train(), opt, cfg
    model = LibraryImageClassifier(model_name).to(device).to(memory_format=torch.channels_last)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9, foreach=True)
    return model.train(), opt, None


def param_count(model):
    return sum(p.numel() for p in model.parameters())
