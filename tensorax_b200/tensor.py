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

    def backward(self, grad: Optional["Tensor"] = None) -> None:
        """Backpropagation entry of the reference (tensorax/tensor.py:604-620) for the one
        operation this package records: 'scaled_dot_product_attention' (tensorax/tensor.py:806-827),
        evaluated by the flash backward kernels instead of dense [Sq,Sk] temporaries.  A tensor that
        already holds a gradient would need tensor addition to accumulate, which is outside this
        package: that raises instead of silently overwriting."""
        if not self.requires_grad:
            return
        if grad is None:
            if self.size != 1:
                raise RuntimeError("grad must be specified for non-scalar tensors")
            grad = Tensor(np.ones(self._shape, dtype=np.float32), device=self.device)
        if self.grad is not None:
            raise RuntimeError("gradient accumulation is not available in tensorax_b200: clear .grad first")
        self.grad = grad
        if self._grad_fn is None:
            return
        op, *inputs = self._grad_fn
        if op != "scaled_dot_product_attention":
            raise RuntimeError(f"backward of {op!r} is outside tensorax_b200")
        query, key, value = inputs[0], inputs[1], inputs[2]
        saved = getattr(self, "_saved", None)
        if saved is None:
            raise RuntimeError("SDPA backward: built for float16 CUDA tensors with d_k == d_v in {64, 128, 256} and "
                               "implicit (causal / kv_lens) masks; this forward kept no row statistics")
        g = grad if grad.dtype == "float32" else None
        if g is None or g.device != "cuda":
            raise RuntimeError("SDPA backward: grad must be a float32 CUDA tensor")
        # Checked before any kernel runs or any .grad is touched: the same tensor passed twice (q is k, k is v)
        # would need its two gradients added, and an input that already holds a gradient would need accumulation.
        wanted = [t for t in (query, key, value) if t.requires_grad]
        if len({id(t) for t in wanted}) != len(wanted):
            self.grad = None
            raise RuntimeError("SDPA backward: the same tensor was passed as more than one of query/key/value; "
                               "summing its gradients is outside tensorax_b200 -- pass copies")
        if any(t.grad is not None for t in wanted):
            self.grad = None
            raise RuntimeError("gradient accumulation is not available in tensorax_b200: clear .grad of the inputs first")
        dq, dk, dv = _C.scaled_dot_product_attention_backward(
            query._c_tensor, key._c_tensor, value._c_tensor, self._c_tensor, saved["lse"], g._c_tensor,
            causal=saved["causal"], kv_lens=saved["kv_lens"])
        for t, c in ((query, dq), (key, dk), (value, dv)):
            if t.requires_grad:
                t.backward(Tensor._wrap(c))

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, device={self.device})"
