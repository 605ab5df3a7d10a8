"""actnn_b200: ActNN's activation-compression path on B200 (sm_100a).

Public names follow the reference package (actnn/actnn/__init__.py:1-10).  Importing this
package loads ``csrc/libactnn_b200.so``; without it nothing works and the import fails
loudly (there is no CPU or pure-PyTorch substitute for the kernels)."""
from . import _lib

_lib.load()

from . import ops                                                         # noqa: E402
from .conf import config, set_optimization_level                          # noqa: E402
from .layers import (QAvgPool2d, QBatchNorm1d, QBatchNorm2d, QBatchNorm3d, QConv1d, QConv2d, QConv3d,   # noqa: E402
                     QConvTranspose1d, QConvTranspose2d, QConvTranspose3d, QDropout, QLinear, QMaxPool2d,
                     QReLU, QSyncBatchNorm)
from .module import QModule                                               # noqa: E402
from .qbnscheme import QBNScheme                                          # noqa: E402
from .qscheme import QScheme                                              # noqa: E402
from .utils import compute_tensor_bytes, exp_recorder, get_memory_usage   # noqa: E402

__all__ = ["config", "set_optimization_level", "QModule", "QScheme", "QBNScheme", "ops",
           "QConv1d", "QConv2d", "QConv3d", "QConvTranspose1d", "QConvTranspose2d", "QConvTranspose3d",
           "QBatchNorm1d", "QBatchNorm2d", "QBatchNorm3d", "QSyncBatchNorm", "QLinear", "QReLU", "QDropout",
           "QMaxPool2d", "QAvgPool2d", "get_memory_usage", "compute_tensor_bytes", "exp_recorder"]
