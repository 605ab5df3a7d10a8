"""``minimax(data) -> (min, max)`` per row of a ``[rows, cols]`` tensor.

Mirror of actnn/actnn/cpp_extension/minimax.cc:7-16."""
import torch

from .. import _lib
from ._checks import check_cuda_tensor


def minimax(data: torch.Tensor):
    check_cuda_tensor(data, "data")
    if data.dim() != 2:
        raise RuntimeError("The dimension of data is not correct!")
    rows, cols = data.shape
    if cols % 32 != 0 or cols <= 32:          # TORCH_CHECK(D % 32 == 0 && D > 32)
        raise RuntimeError("Expected D % 32 == 0 && D > 32 to be true, but got false.")
    mn = torch.empty(rows, dtype=data.dtype, device=data.device)
    mx = torch.empty(rows, dtype=data.dtype, device=data.device)
    _lib.call("actnn_minimax", data, data.data_ptr(), mn.data_ptr(), mx.data_ptr(), rows, cols,
              _lib.dtype_id(data.dtype), _lib.stream_of(data))
    return mn, mx
