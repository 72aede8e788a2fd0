"""toner_b200: the Toner optimizer step (input-statistic preconditioning for Muon and AdamW) on
hand-written sm_100a CUDA, behind the reference's Python interface.

    from toner_b200 import MuonT, AdamT, ActivationStatistics
    from toner_b200.fast import FastMuonT, FastAdamT, NanoGPTBlock, ProjectionBlock

The CUDA library (``toner_b200/csrc/libtoner_b200.so``, C ABI in ``include/toner_b200.h``) is loaded
on first use; there is no CPU or PyTorch fallback.
"""

from .general import AdamT, MuonT
from .statistics import ActivationStatistics

__all__ = ["MuonT", "AdamT", "ActivationStatistics"]
__version__ = "0.1.0"
