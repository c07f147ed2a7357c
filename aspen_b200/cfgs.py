"""Darknet-style .cfg text for the benchmark networks, generated from their architecture.

The ASPEN cfg dialect is the one `parse_section` reads (reference src/darknet_parser.c:455-552):
`[net]`, `[convolutional]`, `[maxpool]`, `[avgpool]`, `[shortcut]`, `[connected]`, `[matmul]`,
`[attention_k]`, `[attention_v]`, `[layernorm]` with keys size/stride/pad/filters/output/parent/from/
M/K/n_head/n_embd/masked/activation.  Each builder returns `(cfg_text, weighted_layers)` where
`weighted_layers` lists, in file order, the layers that own weights -- the order the `LAYER:n`
counter of the weight file follows (reference src/apu_file_io.c:85-100).

Every entry of `weighted_layers` is `(kind, weight_shape, fan_in)`; weight_shape is the on-disk
shape: conv OIHW, connected [O][C][H][W], matmul [M][K], layernorm [M].
"""
from __future__ import annotations


class _Cfg:
    def __init__(self):
        self.lines: list[str] = []
        self.weighted: list[tuple[str, tuple[int, ...], int]] = []

    def sec(self, name: str, **kv):
        self.lines.append(f"[{name}]")
        for k, v in kv.items():
            if v is not None:
                self.lines.append(f"{k}={v}")
        self.lines.append("")

    def text(self) -> str:
        return "\n".join(self.lines) + "\n"


def _conv(c: _Cfg, cin: int, cout: int, size: int, stride: int, pad: int, act: str, parent=None, bn=True):
    c.sec("convolutional", parent=parent, batch_normalize=1 if bn else None, filters=cout, size=size,
          stride=stride, pad=pad, activation=act)
    c.weighted.append(("conv", (cout, cin, size, size), cin * size * size))
    return cout


def resnet50():
    """ResNet-50 v1.5 (stride on the 3x3), BN folded, 1000-way classifier as a 1x1 conv:
    73 sections like the reference's files/resnet50/resnet50_aspen.cfg."""
    c = _Cfg()
    c.sec("net", height=224, width=224, channels=3)
    ch = _conv(c, 3, 64, 7, 2, 3, "relu")
    c.sec("maxpool", size=3, stride=2, pad=1)
    for width, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        for b in range(blocks):
            cin = ch
            s = stride if b == 0 else 1
            _conv(c, cin, width, 1, 1, 0, "relu")
            _conv(c, width, width, 3, s, 1, "relu")
            ch = _conv(c, width, width * 4, 1, 1, 0, "linear")
            if b == 0:
                _conv(c, cin, width * 4, 1, s, 0, "linear", parent=-4)
                c.sec("shortcut", **{"from": -2}, activation="relu")
            else:
                c.sec("shortcut", **{"from": -4}, activation="relu")
    c.sec("avgpool", size=7, stride=1)
    _conv(c, ch, 1000, 1, 1, 0, "linear", bn=False)
    return c.text(), c.weighted


def vgg16():
    """VGG-16: conv blocks [2,2,3,3,3] x (64,128,256,512,512), 2x2 maxpools, FC 25088-4096-4096-1000."""
    c = _Cfg()
    c.sec("net", height=224, width=224, channels=3)
    ch, hw = 3, 224
    for n, width in ((2, 64), (2, 128), (3, 256), (3, 512), (3, 512)):
        for _ in range(n):
            ch = _conv(c, ch, width, 3, 1, 1, "relu", bn=False)
        c.sec("maxpool", size=2, stride=2)
        hw //= 2
    feat = (ch, hw, hw)
    for out, act in ((4096, "relu"), (4096, "relu"), (1000, "linear")):
        c.sec("connected", output=out, activation=act)
        c.weighted.append(("fc", (out,) + feat, feat[0] * feat[1] * feat[2]))
        feat = (out, 1, 1)
    return c.text(), c.weighted


def custom_cifar():
    """The small CIFAR-10 net of the reference's third example (files/custom.cfg)."""
    c = _Cfg()
    c.sec("net", height=32, width=32, channels=3)
    _conv(c, 3, 32, 5, 1, 2, "relu", bn=False)
    c.sec("maxpool", size=2, stride=2)
    _conv(c, 32, 64, 3, 1, 1, "relu", bn=False)
    c.sec("maxpool", size=2, stride=2)
    feat = (64, 8, 8)
    for out, act in ((256, "relu"), (128, "relu"), (10, "linear")):
        c.sec("connected", output=out, activation=act)
        c.weighted.append(("fc", (out,) + feat, feat[0] * feat[1] * feat[2]))
        feat = (out, 1, 1)
    return c.text(), c.weighted


def _matmul(c: _Cfg, m: int, k: int, parent=None, heads=None, embd=None, act=None):
    c.sec("matmul", parent=parent, M=m, n_head=heads, n_embd=embd, activation=act)
    c.weighted.append(("matmul", (m, k), k))


def _layernorm(c: _Cfg, m: int):
    c.sec("layernorm", M=m)
    c.weighted.append(("layernorm", (m,), m))


def transformer(layers: int, d: int, heads: int, ffn: int, pre_ln: bool, masked: bool, act: str,
                final_ln: bool = False, lm_head: int = 0):
    """Encoder/decoder stack in the reference's layer vocabulary.  post-LN + `gelu` is
    files/bert_base/bert_base_aspen.cfg; pre-LN + `masked=1` + `gelu_acc` is
    files/gpt2_124M/gpt2_124M_aspen.cfg.  `final_ln`/`lm_head` append the GPT-2 tail the
    reference cfg leaves out (same layer types, nothing new for the runtime)."""
    c = _Cfg()
    c.sec("net", M=d, height=1, filters=d)
    hd = d // heads
    for _ in range(layers):
        if pre_ln:
            _layernorm(c, d)
        _matmul(c, d, d, heads=heads, embd=d)                 # keys   (PARENT_1 of attention_k)
        _matmul(c, d, d, parent=-2, heads=heads, embd=d)      # queries (PARENT_0 of attention_k)
        _matmul(c, d, d, parent=-3, heads=heads, embd=d)      # values
        c.sec("attention_k", parent=-2, **{"from": -3}, M=1, K=hd, n_head=heads, n_embd=d,
              masked=1 if masked else None)
        c.sec("attention_v", **{"from": -2}, M=d, n_head=heads, n_embd=d)
        _matmul(c, d, d)
        c.sec("shortcut", **{"from": -8 if pre_ln else -7}, M=d)
        _layernorm(c, d)
        _matmul(c, ffn, d, act=act)
        _matmul(c, d, ffn)
        c.sec("shortcut", **{"from": -4 if pre_ln else -3}, M=d)
        if not pre_ln:
            _layernorm(c, d)
    if final_ln:
        _layernorm(c, d)
    if lm_head:
        _matmul(c, lm_head, d)
    return c.text(), c.weighted


def bert_base():
    return transformer(12, 768, 12, 3072, pre_ln=False, masked=False, act="gelu")


def gpt2_124m(with_lm_head: bool = False):
    return transformer(12, 768, 12, 3072, pre_ln=True, masked=True, act="gelu_acc",
                       final_ln=with_lm_head, lm_head=50257 if with_lm_head else 0)


def tiny_cnn():
    """A few-layer CNN that touches conv 3x3/1x1/strided, both pools, residual and connected;
    small enough for pure-CPU checks."""
    c = _Cfg()
    c.sec("net", height=20, width=20, channels=3)
    _conv(c, 3, 16, 3, 1, 1, "relu", bn=False)
    c.sec("maxpool", size=3, stride=2, pad=1)
    _conv(c, 16, 24, 1, 1, 0, "leaky", bn=False)
    _conv(c, 24, 24, 3, 1, 1, "relu", bn=False)
    _conv(c, 24, 24, 1, 1, 0, "linear", bn=False)
    c.sec("shortcut", **{"from": -3}, activation="relu")
    _conv(c, 24, 64, 3, 2, 1, "relu", bn=False)   # 64 rows: a connected layer needs an unpadded parent
    c.sec("avgpool", size=5, stride=1)
    c.sec("connected", output=10, activation="linear")
    c.weighted.append(("fc", (10, 64, 1, 1), 64))
    c.sec("softmax", output=10)
    return c.text(), c.weighted


YOLO_ANCHORS = "10,13,  16,30,  33,23,  30,61,  62,45,  59,119,  116,90,  156,198,  373,326"


def tiny_yolo(classes: int = 3):
    """Two detection heads joined by an upsample-and-concatenate layer, in the vocabulary of the
    reference's files/yolov3/yolov3_aspen.cfg: `[yolo]` (mask / anchors / classes / stride),
    `[convolutional] parent=-4` branching off before the first head, `[append] stride=2 parent=-1 from=-7`."""
    c = _Cfg()
    c.sec("net", height=32, width=32, channels=3)
    head = 3 * (5 + classes)
    _conv(c, 3, 16, 3, 1, 1, "leaky", bn=False)          # 1  32 x 32
    _conv(c, 16, 32, 3, 2, 1, "leaky", bn=False)         # 2  16 x 16
    _conv(c, 32, 32, 1, 1, 0, "leaky", bn=False)         # 3  16 x 16, joined again by the append layer
    _conv(c, 32, 64, 3, 2, 1, "leaky", bn=False)         # 4  8 x 8
    _conv(c, 64, 32, 1, 1, 0, "leaky", bn=False)         # 5
    _conv(c, 32, 64, 3, 1, 1, "leaky", bn=False)         # 6
    _conv(c, 64, head, 1, 1, 0, "linear", bn=False)      # 7
    c.sec("yolo", mask="6,7,8", stride=4, anchors=YOLO_ANCHORS, classes=classes, num=9)     # 8
    _conv(c, 32, 16, 1, 1, 0, "leaky", parent=-4, bn=False)                                 # 9  from layer 5
    c.sec("append", stride=2, parent=-1, **{"from": -7})                                    # 10 16 x 16, 16 + 32 channels
    _conv(c, 48, 32, 3, 1, 1, "leaky", bn=False)         # 11
    _conv(c, 32, head, 1, 1, 0, "linear", bn=False)      # 12
    c.sec("yolo", mask="3,4,5", stride=2, anchors=YOLO_ANCHORS, classes=classes, num=9)     # 13
    return c.text(), c.weighted


def tiny_acts():
    """Every activation of the cfg dialect that the benchmark networks do not use -- `logistic`, `tanh`, `elu`,
    `selu` (reference src/naive_kernels.c:11-57) -- once on a convolution / connected epilogue and once on a
    residual or pooling tile."""
    c = _Cfg()
    c.sec("net", height=12, width=12, channels=4)
    _conv(c, 4, 32, 3, 1, 1, "logistic", bn=False)       # 1
    _conv(c, 32, 32, 1, 1, 0, "tanh", bn=False)          # 2
    _conv(c, 32, 32, 3, 1, 1, "elu", bn=False)           # 3
    c.sec("shortcut", **{"from": -3}, activation="selu") # 4
    _conv(c, 32, 64, 3, 2, 1, "selu", bn=False)          # 5  6 x 6
    c.sec("maxpool", size=2, stride=2, activation="tanh")# 6  3 x 3
    c.sec("avgpool", size=3, stride=1, activation="elu") # 7  1 x 1
    c.sec("connected", output=16, activation="logistic") # 8
    c.weighted.append(("fc", (16, 64, 1, 1), 64))
    return c.text(), c.weighted


def tiny_transformer(masked: bool = False, pre_ln: bool = False, heads: int = 4):
    return transformer(2, 64, heads, 128, pre_ln=pre_ln, masked=masked, act="gelu_acc" if masked else "gelu")


def single_layer(kind: str):
    """One-layer (or one layer plus the producer it needs) networks for profiler captures of a single tile kernel:
    the shapes are the ones ResNet-50 / BERT-base spend their time in."""
    c = _Cfg()
    if kind == "conv3x3":            # stage-2 3x3 convolution: K = 1152
        c.sec("net", height=28, width=28, channels=128)
        _conv(c, 128, 128, 3, 1, 1, "relu", bn=False)
    elif kind == "conv1x1":          # stage-4 reduce convolution: K = 2048
        c.sec("net", height=7, width=7, channels=2048)
        _conv(c, 2048, 512, 1, 1, 0, "relu", bn=False)
    elif kind == "matmul_up":        # FFN up-projection with GELU: K = 768, 3072 rows
        c.sec("net", M=768, height=1, filters=768)
        _matmul(c, 3072, 768, act="gelu")
    elif kind == "matmul_down":      # FFN down-projection: K = 3072
        c.sec("net", M=3072, height=1, filters=3072)
        _matmul(c, 768, 3072)
    elif kind == "residual":         # stage-1 shortcut add behind its 1x1 expand convolution
        c.sec("net", height=56, width=56, channels=256)
        _conv(c, 256, 256, 1, 1, 0, "linear", bn=False)
        c.sec("shortcut", **{"from": -2}, activation="relu")
    elif kind == "layernorm":
        c.sec("net", M=768, height=1, filters=768)
        _layernorm(c, 768)
    elif kind == "maxpool":          # the 3x3 / 2 pool behind the stem
        c.sec("net", height=112, width=112, channels=64)
        c.sec("maxpool", size=3, stride=2, pad=1)
    else:
        raise ValueError(kind)
    return c.text(), c.weighted


BUILDERS = {
    "resnet50": resnet50,
    "vgg16": vgg16,
    "custom": custom_cifar,
    "bert_base": bert_base,
    "gpt2_124M": gpt2_124m,
    "tiny_cnn": tiny_cnn,
    "tiny_transformer": tiny_transformer,
    "tiny_yolo": tiny_yolo,
    "tiny_acts": tiny_acts,
    **{f"layer_{k}": (lambda k=k: single_layer(k)) for k in ("conv3x3", "conv1x1", "matmul_up", "matmul_down", "residual", "layernorm", "maxpool")},
}


def write_cfg(name: str, path: str, **kw):
    text, weighted = BUILDERS[name](**kw)
    with open(path, "w") as f:
        f.write(text)
    return weighted
