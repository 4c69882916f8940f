"""The slice of the reference's ``Tensor`` (tensorax/tensor.py) that the SDPA
forward path touches: construction, device moves, ``tolist``, ``numpy``,
``repeat_interleave``.  Arithmetic, autograd and the rest of the reference class
are outside this package's scope.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import numpy as np

from . import _C

_VALID_DTYPES = ("float32", "float16")
_DEVICES = ("cpu", "cuda")


class Tensor:
    """Python-side mirror (shape / dtype / device) of one backend tensor, as in
    the reference (tensorax/tensor.py:26-88): ``_c_tensor`` is the backend handle."""

    def __init__(self, data, shape: Optional[Sequence[int]] = None, dtype: Optional[str] = None,
                 device: str = "cpu", requires_grad: bool = False) -> None:
        if device not in _DEVICES:
            raise ValueError(f"Unknown device: {device}")
        if dtype is not None and dtype not in _VALID_DTYPES:
            raise ValueError(f"Invalid dtype: {dtype}. Must be one of {_VALID_DTYPES}")
        self.requires_grad = requires_grad
        self.grad = None
        self._grad_fn = None
        if isinstance(data, Tensor):
            self._shape, self._size = data._shape, data._size
            self.dtype, self.device = data.dtype, data.device
            self._c_tensor = _C.copy_tensor(data._c_tensor)
            return
        try:
            arr = np.asarray(data, dtype=np.float16 if dtype == "float16" else np.float32)
        except ValueError as exc:
            raise ValueError("Cannot infer shape from data: inconsistent nested list lengths.") from exc
        if shape is not None:
            shape = tuple(int(s) for s in shape)
            if int(np.prod(shape, dtype=np.int64)) != arr.size:
                raise ValueError(f"Data size {arr.size} does not match provided shape {shape}")
            arr = arr.reshape(shape)
        self.dtype = dtype or "float32"
        self.device = device
        self._shape = tuple(arr.shape)
        self._size = int(arr.size)
        self._c_tensor = _C.from_numpy(arr, device, self.dtype)

    # ------------------------------------------------------------ construction helpers
    @classmethod
    def _wrap(cls, c_tensor, requires_grad: bool = False) -> "Tensor":
        t = cls.__new__(cls)
        t._c_tensor = c_tensor
        t._shape = tuple(c_tensor.shape)
        t._size = c_tensor.size
        t.dtype = c_tensor.dtype
        t.device = c_tensor.device
        t.requires_grad = requires_grad
        t.grad = None
        t._grad_fn = None
        return t

    @staticmethod
    def cuda_is_available() -> bool:
        return _C.cuda_is_available()

    @classmethod
    def randn(cls, shape, dtype: str = "float32", device: str = "cpu", seed=None) -> "Tensor":
        if isinstance(shape, int):
            shape = (shape,)
        rng = np.random.default_rng(seed)
        return cls(rng.standard_normal(tuple(shape), dtype=np.float32), dtype=dtype, device=device)

    @classmethod
    def zeros(cls, shape, dtype: str = "float32", device: str = "cpu", requires_grad=False) -> "Tensor":
        return cls(np.zeros(tuple(shape), dtype=np.float32), dtype=dtype, device=device,
                   requires_grad=requires_grad)

    # ------------------------------------------------------------ properties
    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self._shape)

    @property
    def size(self) -> int:
        return self._size

    @property
    def ndim(self) -> int:
        return len(self._shape)

    # ------------------------------------------------------------ movement / export
    def cuda(self) -> "Tensor":
        if self.device == "cuda":
            return self
        return Tensor._wrap(_C.tensor_cpu_to_cuda(self._c_tensor), self.requires_grad)

    def cpu(self) -> "Tensor":
        if self.device == "cpu":
            return self
        return Tensor._wrap(_C.tensor_cuda_to_cpu(self._c_tensor), self.requires_grad)

    def to(self, device: str) -> "Tensor":
        if device not in _DEVICES:
            raise ValueError(f"Unknown device: {device}")
        return self.cuda() if device == "cuda" else self.cpu()

    def numpy(self):
        return _C.to_numpy(self._c_tensor)

    def tolist(self):
        return self.numpy().astype(np.float64).tolist()

    def reshape(self, shape) -> "Tensor":
        return Tensor._wrap(_C.reshape(self._c_tensor, list(shape)), self.requires_grad)

    def repeat_interleave(self, repeats: int, dim: int = 0) -> "Tensor":
        """tensorax/tensor.py:933-959."""
        return Tensor._wrap(_C.repeat_interleave(self._c_tensor, int(repeats), int(dim)))

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, device={self.device})"
