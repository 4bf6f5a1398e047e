"""The benchmark workload: a particle-domain U-Net assembled from the aprnet operator modules.

Structure follows the reference's `APRUNet` (apr_models/apr_models/unet/unet_model.py:7-94 with the
blocks of unet_parts.py:6-83): every stage is `n_conv` x [APRConv 3x3x3 (no bias) -> GroupNorm ->
ReLU]; going down a stage starts with MaxPool; going up, a 1x1x1 conv block halves the channels,
UpSampleConst restores the finer level, the skip tensor is concatenated in front, and a stage of conv
blocks follows; a biased 1x1x1 conv maps to the output classes.  Channel widths double per level.
GroupNorm / ReLU / cat are ordinary torch operators, as in the reference.

`ops` is any namespace providing `APRConv`, `MaxPool` and `UpSampleConst` with the reference's
constructor and call signatures: `pyapr.aprnet.cuda` for the GPU path, or the CPU reference modules
used for the timed CPU baseline.  The reference's own `apr_models` package runs unchanged on
`pyapr.aprnet.cuda` as well; this copy exists so the benchmark does not need that checkout.
"""
import torch
from torch import nn


class ConvNormAct(nn.Module):
    """conv -> GroupNorm -> ReLU.  When the operator namespace offers a fused `GroupNormReLU` (same
    function and parameters as nn.GroupNorm followed by nn.ReLU) and `fused_norm` is set, it is used."""

    def __init__(self, ops, cin, cout, nstencils, kernel_size, num_groups, fused_norm=True):
        super().__init__()
        self.conv = ops.APRConv(cin, cout, nstencils=nstencils, kernel_size=kernel_size, bias=False)
        groups = min(num_groups, cout) if num_groups else cout
        if fused_norm and hasattr(ops, "GroupNormReLU"):
            self.norm = ops.GroupNormReLU(groups, cout)
            self.act = nn.Identity()
        else:
            self.norm = nn.GroupNorm(groups, cout)
            self.act = nn.ReLU()

    def forward(self, x, aprs, level_deltas):
        return self.act(self.norm(self.conv(x, aprs, level_deltas)))


class Stage(nn.Module):
    def __init__(self, ops, cin, cout, nstencils, n_conv, num_groups, fused_norm=True):
        super().__init__()
        widths = [cin] + [cout] * n_conv
        self.blocks = nn.ModuleList(ConvNormAct(ops, widths[i], widths[i + 1], nstencils, (3, 3, 3), num_groups, fused_norm)
                                    for i in range(n_conv))

    def forward(self, x, aprs, level_deltas):
        for b in self.blocks:
            x = b(x, aprs, level_deltas)
        return x


class APRUNet(nn.Module):
    def __init__(self, ops, in_channels, out_channels, depth=3, n_filters_base=32, n_conv_per_block=2, n_stencils=2, fused_norm=True):
        super().__init__()
        widths = [n_filters_base * 2 ** i for i in range(depth + 1)]
        groups = n_filters_base
        self.depth = depth
        self.enc = nn.ModuleList([Stage(ops, in_channels, widths[0], n_stencils, n_conv_per_block, groups, fused_norm)])
        self.pools = nn.ModuleList()
        for i in range(depth):
            self.pools.append(ops.MaxPool())
            self.enc.append(Stage(ops, widths[i], widths[i + 1], n_stencils, n_conv_per_block, groups, fused_norm))
        self.reduce = nn.ModuleList()
        self.ups = nn.ModuleList()
        self.dec = nn.ModuleList()
        for i in reversed(range(depth)):
            self.reduce.append(ConvNormAct(ops, widths[i + 1], widths[i + 1] // 2, n_stencils, (1, 1, 1), None, fused_norm))
            self.ups.append(ops.UpSampleConst())
            self.dec.append(Stage(ops, widths[i + 1], widths[i], n_stencils, n_conv_per_block, groups, fused_norm))
        self.head = ops.APRConv(widths[0], out_channels, nstencils=n_stencils, kernel_size=(1, 1, 1))

    def forward(self, x, aprs, level_deltas=None):
        if level_deltas is None:
            level_deltas = torch.zeros(len(aprs), dtype=torch.int32)
        skips = [self.enc[0](x, aprs, level_deltas)]
        for i in range(self.depth):
            skips.append(self.enc[i + 1](self.pools[i](skips[-1], aprs, level_deltas), aprs, level_deltas))
        y = skips[-1]
        for k in range(self.depth):
            y = self.reduce[k](y, aprs, level_deltas)
            y = self.ups[k](y, aprs, level_deltas)
            y = torch.cat([skips[self.depth - 1 - k], y], dim=1)
            y = self.dec[k](y, aprs, level_deltas)
        return self.head(y, aprs, level_deltas)
