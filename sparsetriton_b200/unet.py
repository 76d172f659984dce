"""Sparse 3-D U-Net built only from the mirrored layer surface (the benchmark network).

Encoder: stages of 32 / 64 / 128 / 256 channels, each two SubMConv3D(k3) + SparseBatchNorm + ReLU,
joined by SparseConv3D(k2, s2).  Decoder: SparseConvTransposed3D(k2, s2) back up, the encoder
features of the same level concatenated as skip, two SubMConv3D(k3) + BN + ReLU per level, ending at
32 channels; a SparseLinear head gives 20 classes.

Even kernels follow the reference's rule (kmap.py:135-180): the k2 s2 down-conv maps inputs
{2o-1, 2o} to output o and the k2 s2 transposed conv emits {2i-1, 2i}, so what a transposed conv
produces at a level is a superset of the encoder's coordinates of that level (up to 8 children per
voxel, of which the encoder had only some).  Two decoder modes:

  prune=True (default, the usual U-Net)  the up-conv is evaluated only at the encoder's coordinates
      of the level, so decoder and encoder tensors share coordinates, hash table and neighbour maps
      and the skip is a plain channel concatenation.  Evaluating a transposed convolution at the
      children the down-conv came from needs no new map: child = parent*s + off_t[k] is the very
      relation the down-conv's map stores, so the up-conv is a gather over that map's inverse.
  prune=False (the literal composition of the reference's layers)  every child is materialised and
      the skip is a lookup (encoder row of the same coordinate, or zeros).  The active set then grows
      up to 8x per level: on the 1440x1440x41 benchmark scenes a batch-16 training step does not fit
      180 GB, which is why the benchmarks run the pruned form.

Precision: parameters stay fp32 (master weights); features run in `feature_dtype` (bf16 in the
benchmarks); the conv Functions cast the weights per call and return fp32 weight gradients;
batch norm computes in fp32 per sample and casts back.
"""
import torch
from torch import nn

from sparsetriton_b200.config import ConvAlgo, get_conv_algo
from sparsetriton_b200.nn.functional.conv.funcs import ConvPrecomputedNeighborGEMM
from sparsetriton_b200.nn.functional.conv.conv import ConvPreparation
from sparsetriton_b200.nn.functional.conv.funcs.implicit_precomputed_gemm import inverse_map, prepare_plans
from sparsetriton_b200.nn.functional.norm import _batch_info
from sparsetriton_b200.nn.modules import ReLU, SparseBatchNorm, SparseConv3D, SparseConvTransposed3D, SparseLinear, SubMConv3D
from sparsetriton_b200.tensor import SparseTensor, TensorCache
from sparsetriton_b200.utils.concat import concat_features
from sparsetriton_b200.utils.hash import HashTable, round_up_capacity

__all__ = ["SparseUNet", "skip_concat", "up_conv_onto"]


def up_conv_onto(x: SparseTensor, up: SparseConvTransposed3D, target: SparseTensor) -> SparseTensor:
    """`up(x)` evaluated only at the coordinates of `target`, the tensor that `x`'s coordinates were
    downsampled from by a SparseConv3D with the same kernel size / stride / padding / dilation.

    With the stored-map algorithm and the down-conv's map still cached on `target`, this is one gather
    GEMM over the inverse of that map (no coordinate or map building).  Otherwise it falls back to the
    full transposed convolution followed by a lookup of the target's coordinates in its output."""
    k, s, p, d = up.kernel_size[0], up.stride[0], up.padding[0], up.dilation[0]
    cached = target._cache.neighbor_indices.get((k, s, p, d, False, False))
    if get_conv_algo() == ConvAlgo.PrecomputedNeighborGEMM and cached is not None and cached[1].shape[0] == x.F.shape[0]:
        inv = inverse_map(cached[1], target.C.shape[0])         # (N_target, K): parent row per child and offset
        feats = ConvPrecomputedNeighborGEMM.apply(x.F, up.weight, inv)
        if up.bias is not None:
            feats = feats + up.bias.to(feats.dtype)
        return target.replace(feats)
    full = up(x)
    table = HashTable(round_up_capacity(full.C.shape[0], 2.0), device=full.C.device)
    table.insert(full.C)
    idx = table.query(target.C).long()
    found = (idx >= 0).unsqueeze(1)
    rows = full.F.index_select(0, idx.clamp(min=0)) * found.to(full.F.dtype)
    if up.bias is not None:                                   # a child without any parent gets the bias alone
        rows = rows + up.bias.to(rows.dtype) * (~found).to(rows.dtype)
    return target.replace(rows)


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
        # the activation is folded into the normalisation kernels; self.act stays for state_dict / module parity
        x = self.bn1(self.conv1(x), relu=True)
        return self.bn2(self.conv2(x), relu=True)


class SparseUNet(nn.Module):
    def __init__(self, in_channels=4, widths=(32, 64, 128, 256), num_classes=20, prune=True):
        super().__init__()
        self.prune = prune
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

    def prepare(self, coords, spatial_shape, batch_size, backward=True, consumer_stream=None) -> TensorCache:
        """Everything this network derives from the input coordinates alone, ahead of the features: per level the
        submanifold map, the down-convolution's output coordinates and map, the inverse map the pruned up-convolution
        gathers over, their tile plans and the per-sample row counts of the normalisation layers.  Returns the
        TensorCache for `SparseTensor(feats, coords, spatial_shape, batch_size, cache=...)`; the forward and backward
        passes then launch no coordinate work and read nothing back from the device.

        Stored-map algorithm and prune=True only.  Runs on the current stream: under a side stream it overlaps the
        previous step (pass the training stream as `consumer_stream` and make it wait for an event recorded after
        this call).  The waits for the three output counts are waits for that side stream alone."""
        assert self.prune and get_conv_algo() == ConvAlgo.PrecomputedNeighborGEMM, \
            "prepare() serves the pruned decoder under the stored-map algorithm"
        root = cache = TensorCache()
        shape = tuple(spatial_shape)
        made = []
        for level in range(len(self.enc)):
            ConvPreparation(coords, shape, 3, submanifold=True, backward=backward, cache=cache,
                            consumer_stream=consumer_stream).finish()
            made += [t for t in _batch_info(SparseTensor._trusted(None, coords, shape, batch_size, cache))]
            if level + 1 == len(self.enc):
                break
            down = self.down[level]
            k, s, p, d = down.kernel_size[0], down.stride[0], down.padding[0], down.dilation[0]
            prep = ConvPreparation(coords, shape, k, stride=s, dilation=d, padding=p, submanifold=False, backward=backward,
                                   cache=cache, consumer_stream=consumer_stream, batch_size=batch_size)
            prep.finish()
            if prep.neighbor_indices.shape[0] > 0:
                # the pruned up-convolution of this level is a gather over the inverse of the down-convolution's map
                inv = inverse_map(prep.neighbor_indices, coords.shape[0])
                made += [inv] + prepare_plans(inv, prep.out_coords.shape[0], backward)
            cache = cache.child((k, s, p, d, False, False))
            coords, shape = prep.out_coords, prep.new_shape
        if consumer_stream is not None:
            for t in made:
                if t is not None and t.is_cuda and t.numel() > 0:
                    t.record_stream(consumer_stream)
        return root

    def forward(self, x: SparseTensor) -> SparseTensor:
        skips = []
        for i, block in enumerate(self.enc):
            if i > 0:
                x = self.down[i - 1](x)
            x = block(x)
            skips.append(x)
        for j, (up, block) in enumerate(zip(self.up, self.dec)):
            skip = skips[len(skips) - 2 - j]
            if self.prune:
                x = up_conv_onto(x, up, skip)
                x = x.replace(concat_features(x.F, skip.F))
            else:
                x = skip_concat(up(x), skip)
            x = block(x)
        return x.replace(self.head(x.F.float()))
