"""snntc_2023_b200 -- B200 (sm_100a) implementation of the SNN-TC operators SnnFc, SnnFcGrad, SnnCv,
SnnCvGrad behind the reference's Python layer API (SNN_dense, SNN_conv)."""
from . import _lib, ops  # noqa: F401
from .SNN_TC_Modules import (SNN_dense, SNN_conv, SNN_maxpool2d, SNN_avgpool2d, SNN_LRN, loss_func,  # noqa: F401
                             init_weight)

__version__ = "0.1"
