from .implicit_hashfly_gemm import ConvHashOnTheFlyImplicitGEMM
from .implicit_precomputed_gemm import ConvPrecomputedNeighborGEMM

__all__ = ["ConvHashOnTheFlyImplicitGEMM", "ConvPrecomputedNeighborGEMM"]
