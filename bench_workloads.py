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
    def __init__(self, name, cfg, shape, dtype, desc, cpu_sample_items):
        self.name, self.cfg, self.shape, self.dtype, self.desc = name, cfg, shape, dtype, desc
        self.cpu_sample_items = cpu_sample_items     # batch items timed on the CPU baseline

    def with_items(self, items):
        """The same workload with another batch size (reduced cases for profiler captures)."""
        return Workload(self.name, self.cfg, (items,) + tuple(self.shape[1:]), self.dtype,
                        self.desc + " [batch %d]" % items, min(self.cpu_sample_items, items))

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
        if self.name == "focal":
            return 12 * e                    # fused step: logits and labels read once, gradient written once
        if self.name == "ohem":
            # relabelling: logits and labels read, labels written (4E + 16P; scores and the select
            # passes over them, <= 16P more, not counted) + label count 8P + fused cross entropy
            # step (logits read, gradient written, labels read) 8E + 8P
            return 12 * e + 32 * p
        if self.name == "lovasz":
            # the passes over ALL elements: keys (read logits, write keys) 8E, prune count 4E,
            # compaction (read keys, write dJ = 0) 8E.  The sort of the kept elements (~7% of E
            # on this workload's random logits: two 16-byte scatter passes, three histogram reads,
            # the 12-byte Jaccard pass) is data dependent and not counted.
            return 20 * e + 8 * p
        if self.fused_softmax():
            # label count (8P), then the fused step: logits read, gradient written, labels read
            return 2 * s * e + 16 * p
        return s * e + 8 * p

    def bytes_backward(self):
        # (with many classes backward also reads 16 bytes of saved statistics per pixel: 0.1 byte per
        # element at 150 classes, not counted)
        e, p, s = self.elems, self.pixels, self.esize()
        if self.name == "focal":
            return 0                         # upstream gradient 1: the rescale kernel has nothing to do
        if self.name == "lovasz":
            return 12 * e + 8 * p
        if self.name == "ohem" or self.fused_softmax():
            return 0                         # upstream gradient 1: the rescale kernel has nothing to do
        return 2 * s * e + 8 * p

    def fused_softmax(self):
        """The softmax workloads run the fused training step unless B200_SOFTMAX_FUSED=0."""
        return self.name in ("lsr", "lsr_rows", "lmargin") and os.environ.get("B200_SOFTMAX_FUSED", "1") != "0"

    def bytes_step(self):
        return self.bytes_forward() + self.bytes_backward()

    # DRAM traffic per logit element (dram__bytes_read.sum + dram__bytes_write.sum of every kernel
    # behind the entry point) from the ncu captures summarised under profiles/, taken on reduced
    # batches and scaled by the element count (traffic grows in proportion).  Written gradients
    # that are still in the 126 MB L2 when the kernel ends are not counted by those counters.
    MEASURED_TRAFFIC = {                     # fused training steps (forward entry = the whole step)
        "focal": (9.92, 0.0), "lsr": (6.16, 0.0), "lmargin": (7.44, 0.0),
        "lovasz": (22.3, 11.5), "lsr_rows": (3.23, 0.0), "ohem": (11.67, 0.0),
    }
    MEASURED_TRAFFIC_SEPARATE = {            # separate forward and backward kernels (B200_SOFTMAX_FUSED=0)
        "lsr": (4.45, 5.72), "lmargin": (4.15, 7.49), "lsr_rows": (2.01, 3.15),
    }

    def _traffic(self):
        if self.name in self.MEASURED_TRAFFIC_SEPARATE and not self.fused_softmax():
            return self.MEASURED_TRAFFIC_SEPARATE[self.name]
        return self.MEASURED_TRAFFIC[self.name]

    def traffic_forward(self):
        return self._traffic()[0] * self.elems

    def traffic_backward(self):
        return self._traffic()[1] * self.elems

    def entries(self):
        if self.name == "focal":
            return "b200_focal_forward_backward_reduced", "b200_rescale_gradient"
        if self.name == "ohem":
            return "b200_ohem_label+b200_count_valid+b200_lsr_forward_backward_reduced", "b200_rescale_gradient"
        if self.fused_softmax():
            stem = "lmargin" if self.name == "lmargin" else "lsr"
            return "b200_count_valid+b200_%s_forward_backward_reduced" % stem, "b200_rescale_gradient"
        stem = {"lsr": "lsr", "lsr_rows": "lsr", "focal": "focal", "lmargin": "lmargin", "lovasz": "lovasz"}[self.name]
        return "b200_%s_forward" % stem, "b200_%s_backward" % stem

    # ---- data
    def make(self, seed_offset=0, device="cpu", items=None):
        """(logits, labels) for `items` batch items (default: all).  device='cpu' gives the
        canonical seeded tensors; a CUDA device draws the same distributions there."""
        shape = list(self.shape)
        if items is not None:
            shape[0] = items
        g = torch.Generator(device=device).manual_seed(1234 + self.cfg + seed_offset)
        kw = dict(generator=g, device=device)
        n = shape[0]
        if self.name == "focal":
            logits = torch.randn(shape, **kw) * math.sqrt(3.0)
            labels = (torch.rand(shape, **kw) < 0.1).float()
            return logits, labels
        if self.name == "lsr":
            logits = torch.randn(shape, **kw) * math.sqrt(2.0)
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            labels[torch.rand([n] + shape[2:], **kw) < 0.05] = 255
            return logits, labels
        if self.name == "lmargin":
            logits = torch.randn(shape, **kw)
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            labels[torch.rand([n] + shape[2:], **kw) < 0.10] = 255
            return logits, labels
        if self.name == "ohem":
            # a mostly trained network: 97% of the pixels score well above the threshold, so the
            # n_min = P/16 hardest reach into the easy ones and the selection runs in full
            logits = torch.randn(shape, **kw) * math.sqrt(2.0)
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            easy = (torch.rand([n] + shape[2:], **kw) < 0.97).to(logits.dtype) * 9.0
            logits.scatter_add_(1, labels.unsqueeze(1), easy.unsqueeze(1))
            labels[torch.rand([n] + shape[2:], **kw) < 0.05] = 255
            return logits, labels
        if self.name == "lovasz":
            logits = torch.randn(shape, **kw)
            h, w = shape[2], shape[3]
            cells = torch.randint(0, shape[1], (n, h // 32, w // 32), **kw)
            for i in range(n):                     # every image must contain every class
                cells[i].view(-1)[:shape[1]] = torch.arange(shape[1], device=device)
            labels = cells.repeat_interleave(32, 1).repeat_interleave(32, 2).contiguous()
            labels[torch.rand((n, h, w), **kw) < 0.03] = 255
            return logits, labels
        if self.name == "lsr_rows":
            logits = torch.randn(shape, **kw).half()
            labels = torch.randint(0, shape[1], [n] + shape[2:], **kw)
            return logits, labels
        raise KeyError(self.name)

    def criterion(self, package, process_group=None):
        """The module under test from `package` (the CUDA package)."""
        if self.name == "focal":
            return package.FocalLossV3(0.25, 2, 'mean', process_group=process_group)
        if self.name == "lsr":
            return package.LabelSmoothSoftmaxCEV3(0.1, 'mean', 255, process_group=process_group)
        if self.name == "lmargin":
            return package.LargeMarginSoftmaxV3(0.3, 'mean', 255, process_group=process_group)
        if self.name == "lovasz":
            return package.LovaszSoftmaxV3('mean', 255, per_image=True, process_group=process_group)
        if self.name == "ohem":
            return package.OhemCELoss(0.7, None, 255)
        return package.LabelSmoothSoftmaxCEV3(0.1, 'mean', -100, process_group=process_group)

    def oracle(self, oracle_module):
        """The CPU port's function for this workload: f(logits, labels) -> (loss, grad)."""
        O = oracle_module
        if self.name == "focal":
            return lambda x, y: O.focal_loss(x, y, 0.25, 2.0, 'mean')
        if self.name == "lsr":
            return lambda x, y: O.label_smooth_ce(x, y, 0.1, 255, 'mean')
        if self.name == "lmargin":
            return lambda x, y: O.large_margin_softmax(x, y, 0.3, 255, 'mean')
        if self.name == "lovasz":
            return lambda x, y: O.lovasz_softmax(x, y, 255, 'mean', per_image=True)
        if self.name == "ohem":
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
    # not one of the five baseline configurations: the relabelling step in front of the loss
    "ohem": Workload("ohem", 6, (16, 19, 512, 512), torch.float32,
                     "OhemCELoss fp32 [16,19,512,512], thresh 0.7, n_min P/16, 97% easy pixels, 5% ignored", 4),
}
HEADLINE = "focal"
