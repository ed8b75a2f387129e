"""Synthetic workloads of the benchmark: the five configurations of the task's baseline
file (plus the OHEM relabelling in front of a loss), with their seeded generators, algorithmic byte counts and CPU-sample sizes.
No dataset is involved: shapes and value distributions only.

Draw order per configuration (one `torch.Generator().manual_seed(1234 + cfg)` on the CPU):
logits, then labels (or the label cell grid), then the ignore mask.  "N(0, v)" is read as
mean 0, variance v.
"""
import math
import os

import torch


class Workload:
    def __init__(self, name, cfg, shape, dtype, desc, cpu_sample_items, kind=None, upstream=1.0, reduction='mean',
                 layout='nchw'):
        self.name, self.cfg, self.shape, self.dtype, self.desc = name, cfg, shape, dtype, desc
        self.cpu_sample_items = cpu_sample_items     # batch items timed on the CPU baseline
        self.kind = kind or name                     # which loss / kernel family (variants share one)
        self.upstream = upstream                     # d(objective)/d(loss) handed to backward
        self.reduction = reduction                   # 'none': per-pixel losses out, a per-pixel upstream tensor in
        self.layout = layout                         # 'nhwc': channels-last logits (torch.channels_last), consumed in place

    def with_items(self, items, note=None):
        """The same workload with another batch size (reduced cases for profiler captures, and a
        rank's shard of the global batch in multi-GPU runs)."""
        return Workload(self.name, self.cfg, (items,) + tuple(self.shape[1:]), self.dtype,
                        self.desc + (note or " [batch %d]" % items), min(self.cpu_sample_items, items),
                        self.kind, self.upstream, self.reduction, self.layout)

    @property
    def elems(self):
        return math.prod(self.shape)

    @property
    def pixels(self):
        return self.elems // self.shape[1]

    def esize(self):
        return 2 if self.dtype == torch.float16 else 4

    # algorithmic bytes per entry point (inputs once per pass, gradient once, no per-pixel
    # loss tensor, softmax recomputed in backward)
    def bytes_forward(self):
        e, p, s = self.elems, self.pixels, self.esize()
        if self.kind == "focal":
            return 12 * e                    # fused step: logits and labels read once, gradient written once
        if self.kind == "ohem":
            # relabelling: logits and labels read, labels written (4E + 16P; scores and the select
            # passes over them, <= 16P more, not counted) + label count 8P + fused cross entropy
            # step (logits read, gradient written, labels read) 8E + 8P
            return 12 * e + 32 * p
        if self.kind == "lovasz":
            # the passes over ALL elements: keys (read logits, write keys) 8E, prune count 4E,
            # compaction (read keys, write dJ = 0) 8E.  The sort of the kept elements (~7% of E
            # on this workload's random logits: two 16-byte scatter passes, three histogram reads,
            # the 12-byte Jaccard pass) is data dependent and not counted.
            return 20 * e + 8 * p
        if self.kind == "taylor":
            return 2 * s * e                 # input read, output written
        if self.kind == "pc_softmax":
            # label count (8P), then the fused step: logits read, gradient written, labels read
            return 2 * s * e + 16 * p
        if self.fused_softmax():
            # label count (8P), then the fused step: logits read, gradient written, labels read
            return 2 * s * e + 16 * p
        return s * e + 8 * p + (s * p if self.reduction == 'none' else 0)

    def bytes_backward(self):
        # (with many classes backward also reads 16 bytes of saved statistics per pixel: 0.1 byte per
        # element at 150 classes, not counted)
        e, p, s = self.elems, self.pixels, self.esize()
        if self.kind == "focal":
            # upstream gradient 1: the rescale kernel has nothing to do; otherwise it reads and
            # rewrites the gradient
            return 0 if self.upstream == 1.0 else 2 * s * e
        if self.kind == "lovasz":
            return 12 * e + 8 * p
        if self.kind == "taylor":
            return 3 * s * e                 # upstream gradient and input read, gradient written
        if self.kind in ("ohem", "pc_softmax") or self.fused_softmax():
            return 0                         # upstream gradient 1: the rescale kernel has nothing to do
        return 2 * s * e + 8 * p + (s * p if self.reduction == 'none' else 0)

    def fused_softmax(self):
        """The softmax workloads run the fused training step unless B200_SOFTMAX_FUSED=0."""
        return self.kind in ("lsr", "lsr_rows", "lmargin") and self.reduction != 'none' and \
            os.environ.get("B200_SOFTMAX_FUSED", "1") != "0"

    def bytes_step(self):
        return self.bytes_forward() + self.bytes_backward()

    def entries(self):
        if self.kind == "focal":
            return "b200_focal_forward_backward_reduced", "b200_rescale_gradient"
        if self.kind == "ohem":
            return "b200_ohem_label+b200_count_valid+b200_lsr_forward_backward_reduced", "b200_rescale_gradient"
        if self.kind == "taylor":
            return "b200_taylor_softmax_forward", "b200_taylor_softmax_backward"
        if self.kind == "pc_softmax":
            return "b200_count_valid+b200_pc_softmax_step", "b200_rescale_gradient"
        if self.fused_softmax():
            stem = "lmargin" if self.kind == "lmargin" else "lsr"
            return "b200_count_valid+b200_%s_forward_backward_reduced" % stem, "b200_rescale_gradient"
        stem = {"lsr": "lsr", "lsr_rows": "lsr", "focal": "focal", "lmargin": "lmargin", "lovasz": "lovasz"}[self.kind]
        return "b200_%s_forward" % stem, "b200_%s_backward" % stem

    # ---- data
    def make(self, seed_offset=0, device="cpu", items=None):
        """(logits, labels) for `items` batch items (default: all).  device='cpu' gives the
        canonical seeded tensors; a CUDA device draws the same distributions there."""
        logits, labels = self._make(seed_offset, device, items)
        if self.layout == 'nhwc':
            logits = logits.contiguous(memory_format=torch.channels_last)
        return logits, labels

    def _make(self, seed_offset, device, items):
        shape = list(self.shape)
        if items is not None:
            shape[0] = items
        g = torch.Generator(device=device).manual_seed(1234 + self.cfg + seed_offset)
        kw = dict(generator=g, device=device)
        n = shape[0]
        if self.kind == "focal":
            logits = torch.randn(shape, **kw) * math.sqrt(3.0)
            labels = (torch.rand(shape, **kw) < 0.1).float()
            return logits, labels
        if self.kind == "taylor":
            return torch.randn(shape, **kw) * math.sqrt(2.0), torch.randn(shape, **kw)     # input, upstream gradient
        if self.kind in ("lsr", "pc_softmax"):
            logits = torch.randn(shape, **kw) * math.sqrt(2.0)
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            labels[torch.rand([n] + shape[2:], **kw) < 0.05] = 255
            return logits, labels
        if self.kind == "lmargin":
            logits = torch.randn(shape, **kw)
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            labels[torch.rand([n] + shape[2:], **kw) < 0.10] = 255
            return logits, labels
        if self.kind == "ohem":
            # a mostly trained network: 97% of the pixels score well above the threshold, so the
            # n_min = P/16 hardest reach into the easy ones and the selection runs in full
            logits = torch.randn(shape, **kw) * math.sqrt(2.0)
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            easy = (torch.rand([n] + shape[2:], **kw) < 0.97).to(logits.dtype) * 9.0
            logits.scatter_add_(1, labels.unsqueeze(1), easy.unsqueeze(1))
            labels[torch.rand([n] + shape[2:], **kw) < 0.05] = 255
            return logits, labels
        if self.kind == "lovasz":
            logits = torch.randn(shape, **kw)
            h, w = shape[2], shape[3]
            cells = torch.randint(0, shape[1], (n, h // 32, w // 32), **kw)
            for i in range(n):                     # every image must contain every class
                cells[i].view(-1)[:shape[1]] = torch.arange(shape[1], device=device)
            labels = cells.repeat_interleave(32, 1).repeat_interleave(32, 2).contiguous()
            labels[torch.rand((n, h, w), **kw) < 0.03] = 255
            if self.name == "lovasz_full":
                # what a trained network gives: in every image one pixel of every class is predicted
                # with probability 1 (error exactly 0), so no element lies past the last foreground
                # element of its class and the sort has to rank every valid element
                for c in range(shape[1]):
                    labels[:, 0, c] = c            # cell (0, c//32) may hold another class: claim the pixel
                    logits[:, :, 0, c] = -40.0
                    logits[:, c, 0, c] = 40.0
            return logits, labels
        if self.kind == "lsr_rows":
            logits = torch.randn(shape, **kw).half()
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            return logits, labels
        raise KeyError(self.kind)

    def criterion(self, package, process_group=None):
        """The module under test from `package` (the CUDA package)."""
        if self.kind == "focal":
            return package.FocalLossV3(0.25, 2, 'mean', process_group=process_group)
        if self.kind == "lsr":
            return package.LabelSmoothSoftmaxCEV3(0.1, self.reduction, 255, process_group=process_group)
        if self.kind == "lmargin":
            return package.LargeMarginSoftmaxV3(0.3, self.reduction, 255, process_group=process_group)
        if self.kind == "taylor":
            return package.LogTaylorSoftmaxV3(dim=1, n=2)
        if self.kind == "pc_softmax":
            return package.PCSoftmaxCrossEntropyV2(self.proportions(), 'mean', 255)
        if self.kind == "lovasz":
            return package.LovaszSoftmaxV3('mean', 255, per_image=True, process_group=process_group)
        if self.kind == "ohem":
            return package.OhemCELoss(0.7, None, 255)
        return package.LabelSmoothSoftmaxCEV3(0.1, 'mean', -100, process_group=process_group)

    def upstream_tensor(self, device):
        """What backward() is given: None (autograd's 1), a scalar, or with reduction 'none' a tensor
        over the pixels."""
        if self.reduction == 'none':
            return torch.full((self.shape[0],) + tuple(self.shape[2:]), self.upstream / self.pixels, device=device)
        return None if self.upstream == 1.0 else torch.tensor(float(self.upstream), device=device)

    def proportions(self):
        """Class proportions of the PC-softmax workload: a long-tailed training set."""
        w = torch.arange(1, self.shape[1] + 1, dtype=torch.float64).reciprocal()
        return (w / w.sum()).tolist()

    def oracle(self, oracle_module):
        """The CPU port's function for this workload: f(logits, labels) -> (loss, grad)."""
        O = oracle_module
        if self.kind == "focal":
            return lambda x, y: O.focal_loss(x, y, 0.25, 2.0, 'mean')
        if self.kind == "lsr":
            return lambda x, y: O.label_smooth_ce(x, y, 0.1, 255, self.reduction)
        if self.kind == "lmargin":
            return lambda x, y: O.large_margin_softmax(x, y, 0.3, 255, self.reduction)
        if self.kind == "taylor":
            from oracle import taylor as OT
            return lambda x, g: OT.taylor_softmax(x, 1, 2, True, upstream=g)
        if self.kind == "pc_softmax":
            from oracle import pc_softmax as OP
            return lambda x, y: OP.pc_softmax_ce(x, y, self.proportions(), 255, 'mean')
        if self.kind == "lovasz":
            return lambda x, y: O.lovasz_softmax(x, y, 255, 'mean', per_image=True)
        if self.kind == "ohem":
            from oracle import ohem as OH
            return lambda x, y: OH.ohem_ce_loss(x, y, 0.7, None, 255)
        return lambda x, y: O.label_smooth_ce(x, y, 0.1, -100, 'mean')


WORKLOADS = {
    "lsr": Workload("lsr", 1, (16, 19, 512, 512), torch.float32,
                    "LabelSmoothSoftmaxCEV3 fp32 [16,19,512,512], 5% ignored, mean", 16),
    "focal": Workload("focal", 2, (16, 1, 1024, 1024), torch.float32,
                      "FocalLossV3 fp32 [16,1,1024,1024], alpha 0.25 gamma 2, mean", 16),
    "lmargin": Workload("lmargin", 3, (8, 150, 512, 512), torch.float32,
                        "LargeMarginSoftmaxV3 fp32 [8,150,512,512], 10% ignored, mean", 1),
    "lovasz": Workload("lovasz", 4, (8, 19, 1024, 1024), torch.float32,
                       "LovaszSoftmaxV3 per image fp32 [8,19,1024,1024], 3% ignored, mean", 1),
    "lsr_rows": Workload("lsr_rows", 5, (16384, 32768, 1, 1), torch.float16,
                         "LabelSmoothSoftmaxCEV3 fp16 [16384,32768,1,1], mean", 1024),
    # variants of the configurations above that put data-dependent or optional passes on record
    "lovasz_full": Workload("lovasz_full", 4, (8, 19, 1024, 1024), torch.float32,
                            "LovaszSoftmaxV3 per image fp32 [8,19,1024,1024], 3% ignored, mean, one saturated "
                            "foreground pixel per class and image (nothing can be pruned from the sort)", 1,
                            kind="lovasz"),
    "focal_up2": Workload("focal_up2", 2, (16, 1, 1024, 1024), torch.float32,
                          "FocalLossV3 fp32 [16,1,1024,1024], alpha 0.25 gamma 2, mean, upstream gradient 2.0 "
                          "(the gradient rescale pass runs in full)", 16, kind="focal", upstream=2.0),
    "lmargin_none": Workload("lmargin_none", 3, (8, 150, 512, 512), torch.float32,
                             "LargeMarginSoftmaxV3 fp32 [8,150,512,512], 10% ignored, reduction 'none', per-pixel "
                             "upstream gradient (the separate forward and backward kernels)", 1, kind="lmargin",
                             reduction='none'),
    "lsr_none": Workload("lsr_none", 1, (16, 19, 512, 512), torch.float32,
                         "LabelSmoothSoftmaxCEV3 fp32 [16,19,512,512], 5% ignored, reduction 'none', per-pixel "
                         "upstream gradient (the separate forward and backward kernels)", 16, kind="lsr",
                         reduction='none'),
    # configurations 1 and 3 with channels-last logits (what a network in torch.channels_last hands over)
    "lsr_nhwc": Workload("lsr_nhwc", 1, (16, 19, 512, 512), torch.float32,
                         "LabelSmoothSoftmaxCEV3 fp32 [16,19,512,512] channels-last, 5% ignored, mean", 16,
                         kind="lsr", layout='nhwc'),
    "lmargin_nhwc": Workload("lmargin_nhwc", 3, (8, 150, 512, 512), torch.float32,
                             "LargeMarginSoftmaxV3 fp32 [8,150,512,512] channels-last, 10% ignored, mean", 1,
                             kind="lmargin", layout='nhwc'),
    # a crop size that is not a multiple of 4 pixels (769 x 769): channel rows start on no 16-byte boundary
    "lsr_769": Workload("lsr_769", 11, (8, 19, 769, 769), torch.float32,
                        "LabelSmoothSoftmaxCEV3 fp32 [8,19,769,769] (odd image size), 5% ignored, mean", 4,
                        kind="lsr"),
    # label smoothing where it is used most: classification logits [batch, classes]
    "lsr_cls": Workload("lsr_cls", 10, (65536, 1000), torch.float32,
                        "LabelSmoothSoftmaxCEV3 fp32 [65536,1000] (classification rows), 5% ignored, mean", 8192,
                        kind="lsr"),
    # not baseline configurations: the relabelling step in front of the loss, and the two other
    # softmax variants of the reference on the shape of configuration 1
    "ohem": Workload("ohem", 6, (16, 19, 512, 512), torch.float32,
                     "OhemCELoss fp32 [16,19,512,512], thresh 0.7, n_min P/16, 97% easy pixels, 5% ignored", 4),
    "taylor": Workload("taylor", 7, (16, 19, 512, 512), torch.float32,
                       "LogTaylorSoftmaxV3 fp32 [16,19,512,512], dim 1, n 2, dense upstream gradient", 2),
    "taylor_c150": Workload("taylor_c150", 9, (8, 150, 512, 512), torch.float32,
                            "LogTaylorSoftmaxV3 fp32 [8,150,512,512], dim 1, n 2, dense upstream gradient", 1,
                            kind="taylor"),
    "pc_softmax": Workload("pc_softmax", 8, (16, 19, 512, 512), torch.float32,
                           "PCSoftmaxCrossEntropyV2 fp32 [16,19,512,512], 1/k class proportions, 5% ignored, mean", 2),
}
HEADLINE = "lmargin"        # the largest configuration that the baseline file shards over GPUs
# multi-GPU runs: these split their one global batch over the ranks (strong scaling) ...
SHARDED = ("lmargin", "lsr", "lovasz", "lsr_rows")
# ... and this one runs whole on every rank (weak scaling; its global batch is 64 MB)
WEAK = "focal"
