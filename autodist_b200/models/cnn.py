"""ImageNet-shape CNNs of the reference's benchmark driver (``examples/benchmark/imagenet.py:232-249`` builds
``tf.keras.applications.{ResNet101, VGG16, InceptionV3, DenseNet121}`` with random weights).

ResNet-101 (v1.5 bottlenecks), VGG-16, DenseNet-121 and a small Inception-style network are defined here from
scratch. On a GPU every convolution (forward, input gradient, weight gradient) is the tcgen05 implicit GEMM of
``csrc/conv_tcgen05.cu`` over channels-last bf16 activations, with bias / ReLU and the batch-norm statistics in its
epilogue; batch-norm (+ residual add + ReLU) and max-pooling are hand-written kernels too, and the fully connected
layers - 25088x4096, 4096x4096, 4096x1000 for VGG-16 - run on the tcgen05 GEMM. ``AUTODIST_CONV=library`` switches the
convolutions to the library (the comparison baseline). ``ImageClassifier`` wraps a backbone and the loss into one leaf
module.
"""
import math
import os

import torch
from torch import nn
import torch.nn.functional as F

from autodist_b200.ops.functional import Linear, batch_norm, conv2d, fork, max_pool2d

CONV_MODE = os.environ.get("AUTODIST_CONV", "own")                      # own | library


class Conv2d(nn.Module):
    """Square-filter convolution whose weight is stored channels-last, ``[Cout, KH, KW, Cin]`` - the layout the implicit
    GEMM reads with one TMA box per filter tap and writes its gradient in. Initialised like ``nn.Conv2d``."""

    def __init__(self, cin, cout, k, stride=1, padding=0, bias=False, relu=False):
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size, self.stride, self.padding, self.relu = cin, cout, k, stride, padding, relu
        self.weight = nn.Parameter(torch.empty(cout, k, k, cin))
        self.bias = nn.Parameter(torch.empty(cout)) if bias else None
        bound = 1.0 / math.sqrt(cin * k * k)
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)            # kaiming_uniform(a=sqrt(5)) reduces to U(-1/sqrt(fan_in), 1/sqrt(fan_in))
            if bias:
                self.bias.uniform_(-bound, bound)

    def forward(self, x, stats=None, fork=None):
        if x.is_cuda and CONV_MODE != "library":
            return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.relu, stats, fork)
        y = F.conv2d(x, self.weight.permute(0, 3, 1, 2).to(x.dtype), None if self.bias is None else self.bias.to(x.dtype), self.stride,
                     self.padding)
        return F.relu(y) if self.relu else y

    def extra_repr(self):
        return f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, padding={self.padding}"


def _conv(cin, cout, k, stride=1, padding=0, bias=False, relu=False):
    return Conv2d(cin, cout, k, stride, padding, bias=bias, relu=relu)


class BatchNormAct(nn.BatchNorm2d):
    """Batch-norm with an optional fused residual add and ReLU. For bf16 activations on a GPU (the autocast training path)
    the training-mode statistics, the normalisation (+ add + ReLU), the running-statistics update and both backward passes
    run on the hand-written kernels; fp32 activations, evaluation mode and channel counts that are not a multiple of 8 use
    the library. ``AUTODIST_NORM_POOL=library`` forces the library everywhere, ``=own`` the kernels for fp32 inputs too."""

    def __init__(self, channels, relu=False):
        super().__init__(channels)
        self.relu = relu

    def forward(self, x, residual=None, sums=None, fork=None):
        if _own_norm_pool(x) and self.training and self.momentum is not None:
            return batch_norm(x, self.weight, self.bias, self.running_mean, self.running_var, True, self.momentum, self.eps, self.relu,
                              residual, sums, self.num_batches_tracked, fork)
        y = super().forward(x)
        if residual is not None:
            y = y + residual
        return F.relu(y, inplace=True) if self.relu else y


class _StatsArena:
    """One zeroed fp32 buffer per forward pass from which every ``ConvBN`` takes its ``[2, C]`` slice for the batch-norm
    sums: one memset per step instead of one per layer."""

    def __init__(self):
        self.buf, self.off = None, 0

    def begin(self, numel, device):
        self.buf, self.off = torch.zeros(numel, dtype=torch.float32, device=device), 0

    def take(self, channels, device):
        n = 2 * channels
        if self.buf is None or self.buf.device != device or self.off + n > self.buf.numel():
            return torch.zeros(2, channels, dtype=torch.float32, device=device)
        t = self.buf[self.off:self.off + n].view(2, channels)
        self.off += n
        return t

    def end(self):
        self.buf = None


_ARENA = _StatsArena()


class ConvBN(nn.Module):
    """Convolution followed by batch-norm (+ residual add, + ReLU). On the kernel path the convolution's epilogue already
    accumulates the per-channel sums the batch-norm needs, so the normalisation reads the activation once."""

    def __init__(self, cin, cout, k, stride=1, padding=0, relu=True):
        super().__init__()
        self.conv = _conv(cin, cout, k, stride, padding)
        self.bn = BatchNormAct(cout, relu=relu)

    def forward(self, x, residual=None, in_fork=None, res_fork=None):
        """``in_fork`` / ``res_fork``: the ``GradFork`` of ``x`` / of ``residual`` when that tensor has a second consumer."""
        cout = self.conv.out_channels
        fused = x.is_cuda and x.dim() == 4 and CONV_MODE != "library" and NORM_POOL_MODE != "library" and FUSE_BN_STATS and self.training \
            and self.bn.momentum is not None and cout % 8 == 0 and cout <= 2048 and (x.dtype == torch.bfloat16 or torch.is_autocast_enabled())
        if fused:
            sums = _ARENA.take(cout, x.device)
            return self.bn(self.conv(x, sums, in_fork), residual, sums, res_fork)
        return self.bn(self.conv(x, None, in_fork), residual, None, res_fork)


FUSE_BN_STATS = os.environ.get("AUTODIST_FUSE_BN_STATS", "1") == "1"
FORK_FUSION = os.environ.get("AUTODIST_FORK_FUSION", "1") == "1"


class MaxPool(nn.MaxPool2d):
    def forward(self, x):
        if _own_norm_pool(x) and not self.ceil_mode and self.dilation == 1 and isinstance(self.kernel_size, int):
            return max_pool2d(x, self.kernel_size, self.stride, self.padding)
        return super().forward(x)


NORM_POOL_MODE = os.environ.get("AUTODIST_NORM_POOL", "auto")          # auto | own | library


def _own_norm_pool(x):
    if not x.is_cuda or x.dim() != 4 or x.shape[1] % 8 or NORM_POOL_MODE == "library":
        return False
    return NORM_POOL_MODE == "own" or x.dtype == torch.bfloat16


def _conv_bn(cin, cout, k, stride=1, padding=0, relu=True):
    return ConvBN(cin, cout, k, stride, padding, relu=relu)


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, width, stride):
        super().__init__()
        cout = width * self.expansion
        self.a = _conv_bn(cin, width, 1)
        self.b = _conv_bn(width, width, 3, stride, 1)
        self.c = _conv_bn(width, cout, 1, relu=True)           # its ReLU comes after the residual add, inside the batch-norm kernel
        self.down = None
        if stride != 1 or cin != cout:
            self.down = _conv_bn(cin, cout, 1, stride, relu=False)

    def forward(self, x):
        # the block's input feeds the first convolution and the skip path: whichever gradient comes second is added inside
        # the kernel that produces it (the skip convolution is evaluated after the main path so that its backward runs first)
        xa, xr, box = fork(x) if FORK_FUSION else (x, x, None)
        if self.down is None:
            return self.c(self.b(self.a(xa, in_fork=box)), residual=xr, res_fork=box)
        h = self.b(self.a(xa, in_fork=box))
        return self.c(h, residual=self.down(xr, in_fork=box))


class ResNet(nn.Module):
    def __init__(self, blocks=(3, 4, 23, 3), num_classes=1000, width=64):
        super().__init__()
        self.stem = nn.Sequential(_conv_bn(3, width, 7, 2, 3), MaxPool(3, 2, 1))
        layers, cin = [], width
        for i, n in enumerate(blocks):
            w = width * 2 ** i
            for j in range(n):
                layers.append(Bottleneck(cin, w, 2 if (j == 0 and i > 0) else 1))
                cin = w * Bottleneck.expansion
        self.layers = nn.Sequential(*layers)
        self.fc = Linear(cin, num_classes)

    def forward(self, x):
        x = self.layers(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def resnet101(num_classes=1000):
    return ResNet((3, 4, 23, 3), num_classes)


def resnet50(num_classes=1000):
    return ResNet((3, 4, 6, 3), num_classes)


class VGG16(nn.Module):
    CFG = (64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M")

    def __init__(self, num_classes=1000, image_size=224):
        super().__init__()
        layers, cin = [], 3
        for v in self.CFG:
            if v == "M":
                layers.append(MaxPool(2, 2))
            else:
                layers.append(_conv(cin, v, 3, 1, 1, bias=True, relu=True))
                cin = v
        self.features = nn.Sequential(*layers)
        side = image_size // 32
        self.fc1 = Linear(512 * side * side, 4096)
        self.fc2 = Linear(4096, 4096)
        self.fc3 = Linear(4096, num_classes)

    def forward(self, x):
        x = torch.flatten(self.features(x), 1)
        return self.fc3(F.relu(self.fc2(F.relu(self.fc1(x)))))


class _DenseLayer(nn.Module):
    def __init__(self, cin, growth):
        super().__init__()
        self.f = nn.Sequential(BatchNormAct(cin, relu=True), _conv(cin, 4 * growth, 1),
                               BatchNormAct(4 * growth, relu=True), _conv(4 * growth, growth, 3, 1, 1))

    def forward(self, x):
        return torch.cat([x, self.f(x)], 1)


class DenseNet121(nn.Module):
    def __init__(self, num_classes=1000, growth=32, blocks=(6, 12, 24, 16)):
        super().__init__()
        c = 2 * growth
        mods = [_conv_bn(3, c, 7, 2, 3), MaxPool(3, 2, 1)]
        for i, n in enumerate(blocks):
            for _ in range(n):
                mods.append(_DenseLayer(c, growth))
                c += growth
            if i + 1 < len(blocks):
                mods += [BatchNormAct(c, relu=True), _conv(c, c // 2, 1), nn.AvgPool2d(2, 2)]
                c //= 2
        mods += [BatchNormAct(c, relu=True)]
        self.features = nn.Sequential(*mods)
        self.fc = Linear(c, num_classes)

    def forward(self, x):
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(self.features(x), 1), 1))


class _InceptionBlock(nn.Module):
    def __init__(self, cin, c1, c3r, c3, c5r, c5, cp):
        super().__init__()
        self.b1 = _conv_bn(cin, c1, 1)
        self.b3 = nn.Sequential(_conv_bn(cin, c3r, 1), _conv_bn(c3r, c3, 3, 1, 1))
        self.b5 = nn.Sequential(_conv_bn(cin, c5r, 1), _conv_bn(c5r, c5, 3, 1, 1), _conv_bn(c5, c5, 3, 1, 1))
        self.bp = nn.Sequential(nn.AvgPool2d(3, 1, 1), _conv_bn(cin, cp, 1))

    def forward(self, x):
        return torch.cat([self.b1(x), self.b3(x), self.b5(x), self.bp(x)], 1)


class InceptionNet(nn.Module):
    """Inception-style network (factorised 5x5 branches, batch-norm everywhere) at Inception-V3's depth class."""

    def __init__(self, num_classes=1000):
        super().__init__()
        self.stem = nn.Sequential(_conv_bn(3, 32, 3, 2), _conv_bn(32, 32, 3), _conv_bn(32, 64, 3, 1, 1), MaxPool(3, 2),
                                  _conv_bn(64, 80, 1), _conv_bn(80, 192, 3), MaxPool(3, 2))
        blocks, cin = [], 192
        for spec in [(64, 48, 64, 64, 96, 32), (64, 48, 64, 64, 96, 64), (64, 48, 64, 64, 96, 64)]:
            blocks.append(_InceptionBlock(cin, *spec))
            cin = spec[0] + spec[2] + spec[4] + spec[5]
        blocks.append(MaxPool(3, 2))
        for spec in [(192, 128, 192, 128, 192, 192)] * 4:
            blocks.append(_InceptionBlock(cin, *spec))
            cin = spec[0] + spec[2] + spec[4] + spec[5]
        blocks.append(MaxPool(3, 2))
        for spec in [(320, 384, 768, 448, 384, 192)] * 2:
            blocks.append(_InceptionBlock(cin, *spec))
            cin = spec[0] + spec[2] + spec[4] + spec[5]
        self.blocks = nn.Sequential(*blocks)
        self.fc = Linear(cin, num_classes)

    def forward(self, x):
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(self.blocks(self.stem(x)), 1), 1))


BACKBONES = {"resnet101": resnet101, "resnet50": resnet50, "vgg16": VGG16, "densenet121": DenseNet121,
             "inceptionv3": InceptionNet}


class ImageClassifier(nn.Module):
    """Backbone + softmax cross-entropy as one leaf module: ``loss = model(images[N,3,H,W], labels[N])``."""
    _autodist_leaf = True

    def __init__(self, backbone="resnet101", num_classes=1000, compute_dtype=torch.bfloat16, **kw):
        super().__init__()
        self.net = BACKBONES[backbone](num_classes=num_classes, **kw) if isinstance(backbone, str) else backbone
        self.compute_dtype = compute_dtype
        self._stat_floats = None

    def forward(self, images, labels):
        if images.is_cuda:
            images = images.contiguous(memory_format=torch.channels_last)
            if self._stat_floats is None:
                self._stat_floats = sum(2 * m.conv.out_channels for m in self.net.modules() if isinstance(m, ConvBN))
            _ARENA.begin(self._stat_floats, images.device)
            try:
                with torch.autocast("cuda", dtype=self.compute_dtype):
                    logits = self.net(images)
            finally:
                _ARENA.end()
        else:
            logits = self.net(images)
        return F.cross_entropy(logits.float(), labels)


def synthetic_images(batch, image_size=224, num_classes=1000, seed=0):
    """Images ~ N(0, 1) and uniform labels (the benchmark's synthetic input)."""
    g = torch.Generator().manual_seed(seed)
    return {"images": torch.randn(batch, 3, image_size, image_size, generator=g),
            "labels": torch.randint(0, num_classes, (batch,), generator=g)}
