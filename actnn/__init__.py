"""``import actnn`` for programs written against the reference package.

The reference's drivers do ``import actnn``, ``from actnn import config, QScheme, QModule``,
``from actnn.layers import QConv2d`` and ``import actnn.cpp_extension.quantization as
ext_quantization`` (mem_speed_benchmark/train.py:29-31,292; actnn/actnn/ops.py:15-17).  This
package makes those statements resolve to ``actnn_b200``: every public name is re-exported and
every submodule is registered under the reference's module path, so both spellings name the
very same module objects (one ``config``, one list of ``QScheme.layers``).

The reference's ``actnn.dataloader`` (a fork of torch's DataLoader that also yields sample
indices, only needed for ``config.use_gradient``) is not part of this path and is not provided.
"""
import importlib
import sys

import actnn_b200 as _impl
from actnn_b200 import *            # noqa: F401,F403
from actnn_b200 import __all__      # noqa: F401

_SUBMODULES = ("ops", "conf", "layers", "module", "qscheme", "qbnscheme", "utils", "cpp_extension",
               "cpp_extension.minimax", "cpp_extension.quantization", "cpp_extension.calc_precision",
               "cpp_extension.backward_func")
for _name in _SUBMODULES:
    _mod = importlib.import_module("actnn_b200." + _name)
    sys.modules[__name__ + "." + _name] = _mod
    if "." not in _name:
        globals()[_name] = _mod
del _name, _mod
