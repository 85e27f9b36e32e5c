"""nn.Module wrapper of libs/MemorySaver/modules/MemorySaver.py."""
import torch

from .functions import ComputeMaxAvgFunction


class ComputeMaxAvgModule(torch.nn.Module):
    def forward(self, img1_features_l0, img2_features_lk):
        return ComputeMaxAvgFunction.apply(img1_features_l0, img2_features_lk)
