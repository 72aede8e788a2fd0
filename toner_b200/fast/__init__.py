"""Layer-sharded CUDA Toner optimizers for uniform transformer blocks."""

from .adapter import FastAdamT, FastMuonT, NanoGPTBlock, ProjectionBlock

__all__ = ["FastMuonT", "FastAdamT", "ProjectionBlock", "NanoGPTBlock"]
