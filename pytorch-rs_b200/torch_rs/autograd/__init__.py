"""`torch_rs.autograd.backward` with default options: a single scalar root
(python/torch_rs/autograd/__init__.py:44-127 in the reference)."""
from ..tensor import Tensor


def backward(tensors, grad_tensors=None, retain_graph=None, create_graph=False, inputs=None):
    if isinstance(tensors, (list, tuple)):
        if len(tensors) != 1:
            raise RuntimeError("backward(): only a single root tensor is supported")
        tensors = tensors[0]
    if not isinstance(tensors, Tensor):
        raise TypeError("backward(): expected a Tensor root")
    if grad_tensors is not None or retain_graph or create_graph or inputs is not None:
        raise RuntimeError("backward(): only default options are supported")
    tensors.backward()
