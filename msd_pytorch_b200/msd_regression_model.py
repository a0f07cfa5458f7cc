"""MSD network for regression (API of the reference's msd_pytorch/msd_regression_model.py:8-82)."""
import torch.nn as nn

from .msd_model import MSDModel, NormalizedNet
from .msd_module import DEFAULT_DILATIONS

loss_functions = {"L1": nn.L1Loss(), "L2": nn.MSELoss()}


class MSDRegressionModel(MSDModel):
    def __init__(self, c_in, c_out, depth, width, *, dilations=DEFAULT_DILATIONS, loss="L2", parallel=False, ndim=2):
        super().__init__(c_in, c_out, depth, width, dilations, ndim=ndim)
        self.criterion = loss_functions.get(loss)
        if self.criterion is None:
            raise ValueError(f"The loss must be one of {list(loss_functions.keys())}. Supplied {loss}. ")
        self.net = NormalizedNet(self.scale_in, self.msd, self.scale_out)
        self.net.cuda()
        if parallel:
            self.net = nn.DataParallel(self.net)
        # Only the MSD parameters are trained.
        self.init_optimizer(self.msd)
