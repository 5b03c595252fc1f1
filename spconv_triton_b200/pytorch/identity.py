from torch import nn


class Identity(nn.Module):
    """Returns its input (kept for API compatibility)."""

    def __init__(self, *args, **kwargs):
        super().__init__()

    def forward(self, input):
        return input

    def input_spatial_size(self, out_size):
        return out_size
