"""Drop-in module name of the reference (`import SNN_TC_Modules as SNN`): re-exports the B200 layers."""
from snntc_2023_b200.SNN_TC_Modules import *  # noqa: F401,F403
from snntc_2023_b200.SNN_TC_Modules import (SNN_dense, SNN_conv, SNN_maxpool2d, SNN_avgpool2d, SNN_LRN,  # noqa: F401
                                            loss_func, init_weight, snnfc, snnfc_grad, snncv, snncv_grad)
