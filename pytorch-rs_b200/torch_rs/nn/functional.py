"""`torch_rs.nn.functional` for the hot path: relu routes to `torch.relu`
(python/torch_rs/nn/functional.py:108-118 in the reference)."""
from ..tensor import Tensor


def relu(input, inplace=False):
    if not isinstance(input, Tensor):
        raise TypeError(f"relu(): argument 'input' (position 1) must be Tensor, not {type(input).__name__}")
    if inplace:
        raise RuntimeError("relu(): in-place operation is not supported")
    return input.relu()
