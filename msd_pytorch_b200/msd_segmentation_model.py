"""MSD network for segmentation (API of the reference's msd_pytorch/msd_segmentation_model.py:11-119)."""
import numpy as np
import torch.nn as nn

from .msd_model import MSDModel, NormalizedNet, scaling_module_set_bias, scaling_module_set_scale
from .msd_module import DEFAULT_DILATIONS


class MSDSegmentationModel(MSDModel):
    def __init__(self, c_in, num_labels, depth, width, *, dilations=DEFAULT_DILATIONS, parallel=False, ndim=2):
        self.num_labels = num_labels
        super().__init__(c_in, num_labels, depth, width, dilations, ndim=ndim)
        self.criterion = nn.NLLLoss()
        net_trained = nn.Sequential(self.msd, nn.LogSoftmax(dim=1))
        self.net = NormalizedNet(self.scale_in, net_trained)
        self.net.cuda()
        if parallel:
            self.net = nn.DataParallel(self.net)
        # Everything but scale_in is trained.
        self.init_optimizer(net_trained)

    def set_normalization(self, dataloader):
        """Input normalisation only (targets are labels)."""
        mean = square = 0
        for (data_in, _) in dataloader:
            mean += data_in.mean()
            square += data_in.pow(2).mean()
        mean /= len(dataloader)
        square /= len(dataloader)
        std = np.sqrt(square - mean ** 2)
        scaling_module_set_scale(self.scale_in, 1 / std)
        scaling_module_set_bias(self.scale_in, -mean / std)

    def set_target(self, target):
        # Labels: long, in [0, num_labels), without the channel axis, on the GPU.
        target = target.long()
        lo, hi = target.min(), target.max()
        if lo < 0 or self.num_labels <= hi:
            raise ValueError(f"Target invalid: expected values in range {[0, self.num_labels - 1]}, but got {[lo, hi]}")
        self.target = target.squeeze(1).cuda()
