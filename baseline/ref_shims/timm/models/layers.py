"""Stand-in for ``timm.models.layers`` (only ``DropPath`` is imported by the reference)."""
import torch


class DropPath(torch.nn.Module):
    """Stochastic depth per sample; the identity when ``drop_prob`` is 0 or in eval mode."""

    def __init__(self, drop_prob: float = 0.0, scale_by_keep: bool = True):
        super().__init__()
        self.drop_prob = drop_prob
        self.scale_by_keep = scale_by_keep

    def forward(self, x):
        if self.drop_prob == 0.0 or not self.training:
            return x
        keep = 1.0 - self.drop_prob
        mask = x.new_empty((x.shape[0],) + (1,) * (x.ndim - 1)).bernoulli_(keep)
        if keep > 0.0 and self.scale_by_keep:
            mask.div_(keep)
        return x * mask
