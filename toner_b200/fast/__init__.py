"""Layer-sharded CUDA Toner optimizers for uniform transformer blocks, and the plain Muon baseline."""

from .adapter import FastAdamT, FastMuonT, NanoGPTBlock, ProjectionBlock
from .muon import Muon

__all__ = ["FastMuonT", "FastAdamT", "ProjectionBlock", "NanoGPTBlock", "Muon"]
