"""Sparse 3-D U-Net built only from the mirrored layer surface (the benchmark network).

Encoder: stages of 32 / 64 / 128 / 256 channels, each two SubMConv3D(k3) + SparseBatchNorm + ReLU,
joined by SparseConv3D(k2, s2).  Decoder: SparseConvTransposed3D(k2, s2) back up, the encoder
features of the same level concatenated as skip, two SubMConv3D(k3) + BN + ReLU per level, ending at
32 channels; a SparseLinear head gives 20 classes.

Even kernels follow the reference's rule (kmap.py:135-180): the k2 s2 down-conv maps inputs
{2o-1, 2o} to output o and the k2 s2 transposed conv emits {2i-1, 2i}, so the decoder's coordinate
set at a level is a superset of the encoder's.  The skip is therefore a lookup: every decoder
coordinate takes the encoder row with the same coordinate, or zeros.

Precision: parameters stay fp32 (master weights); features run in `feature_dtype` (bf16 in the
benchmarks); the conv Functions cast the weights per call and return fp32 weight gradients;
batch norm computes in fp32 per sample and casts back.
"""
import torch
from torch import nn

from sparsetriton_b200.nn.modules import ReLU, SparseBatchNorm, SparseConv3D, SparseConvTransposed3D, SparseLinear, SubMConv3D
from sparsetriton_b200.tensor import SparseTensor
from sparsetriton_b200.utils.hash import HashTable, round_up_capacity

__all__ = ["SparseUNet", "skip_concat"]


def skip_concat(decoder: SparseTensor, encoder: SparseTensor) -> SparseTensor:
    """Features of `decoder` with the `encoder` row of the same coordinate (or zeros) appended."""
    table = encoder._cache.hashtable
    if table is None:
        table = HashTable(round_up_capacity(encoder.C.shape[0], 2.0), device=encoder.C.device)
        table.insert(encoder.C)
        encoder._cache.hashtable = table
    idx = table.query(decoder.C).long()
    found = (idx >= 0).unsqueeze(1)
    rows = encoder.F.index_select(0, idx.clamp(min=0)) * found.to(encoder.F.dtype)
    return decoder.replace(torch.cat([decoder.F, rows], dim=1))


class _Block(nn.Module):
    """Two SubMConv3D(k3) + BN + ReLU."""

    def __init__(self, c_in, c_out):
        super().__init__()
        self.conv1, self.bn1 = SubMConv3D(c_in, c_out, 3, bias=False), SparseBatchNorm(c_out)
        self.conv2, self.bn2 = SubMConv3D(c_out, c_out, 3, bias=False), SparseBatchNorm(c_out)
        self.act = ReLU()

    def forward(self, x):
        x = self.act(self.bn1(self.conv1(x)))
        return self.act(self.bn2(self.conv2(x)))


class SparseUNet(nn.Module):
    def __init__(self, in_channels=4, widths=(32, 64, 128, 256), num_classes=20):
        super().__init__()
        self.enc = nn.ModuleList()
        self.down = nn.ModuleList()
        c = in_channels
        for i, w in enumerate(widths):
            if i > 0:
                self.down.append(SparseConv3D(widths[i - 1], w, 2, stride=2, bias=False))
                c = w
            self.enc.append(_Block(c, w))
        self.up = nn.ModuleList()
        self.dec = nn.ModuleList()
        for i in range(len(widths) - 1, 0, -1):
            self.up.append(SparseConvTransposed3D(widths[i], widths[i - 1], 2, stride=2, bias=False))
            self.dec.append(_Block(2 * widths[i - 1], widths[i - 1]))
        self.head = SparseLinear(widths[0], num_classes)

    def forward(self, x: SparseTensor) -> SparseTensor:
        skips = []
        for i, block in enumerate(self.enc):
            if i > 0:
                x = self.down[i - 1](x)
            x = block(x)
            skips.append(x)
        for j, (up, block) in enumerate(zip(self.up, self.dec)):
            x = up(x)
            x = skip_concat(x, skips[len(skips) - 2 - j])
            x = block(x)
        return x.replace(self.head(x.F.float()))
