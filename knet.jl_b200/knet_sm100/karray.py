"""KnetArray: a dense column-major device array, the host-side mirror of
`KnetArray{T,N}` = (ptr, dims) (src/knetarrays/karray.jl:53-56).

The memory is a 1-D torch tensor (torch is used for device memory and streams only); the
Julia shape lives beside it, so `reshape` aliases the memory and `vec`-style views carry
element offsets exactly like KnetArray views do (src/knetarrays/getindex.jl:153-159).
"""
import numpy as np
import torch


def _prod(t):
    p = 1
    for v in t:
        p *= int(v)
    return p


class KnetArray:
    __array_priority__ = 1000

    def __init__(self, data, shape=None):
        if isinstance(data, KnetArray):
            data, shape = data.data, (shape if shape is not None else data.shape)
        if isinstance(data, np.ndarray):
            shape = data.shape if shape is None else tuple(shape)
            flat = np.ascontiguousarray(np.asfortranarray(data).reshape(-1, order="F"))
            data = torch.from_numpy(flat).cuda()
        if not (isinstance(data, torch.Tensor) and data.dim() == 1 and data.is_contiguous()):
            raise TypeError("KnetArray needs a contiguous 1-D tensor or a NumPy array")
        if not data.is_cuda:
            raise TypeError("KnetArray memory must live on the GPU")
        self.data = data
        self.shape = tuple(int(s) for s in (shape if shape is not None else (data.numel(),)))
        if _prod(self.shape) != data.numel():
            raise ValueError(f"shape {self.shape} does not match {data.numel()} elements")

    # ---- construction ------------------------------------------------------------------
    @staticmethod
    def zeros(shape, dtype=torch.float32, device="cuda"):
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        return KnetArray(torch.zeros(_prod(shape), dtype=dtype, device=device), shape)

    @staticmethod
    def empty(shape, dtype=torch.float32, device="cuda"):
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        return KnetArray(torch.empty(_prod(shape), dtype=dtype, device=device), shape)

    def similar(self, shape=None):
        shape = self.shape if shape is None else tuple(shape)
        return KnetArray(torch.empty(_prod(shape), dtype=self.dtype, device=self.data.device), shape)

    def copy(self):
        return KnetArray(self.data.clone(), self.shape)

    # ---- properties ----------------------------------------------------------------------
    @property
    def dtype(self):
        return self.data.dtype

    @property
    def ndim(self):
        return len(self.shape)

    def __len__(self):
        return self.data.numel()

    length = property(lambda self: self.data.numel())

    def size(self, d=None):
        """1-based like Julia; dims beyond ndims have size 1."""
        if d is None:
            return self.shape
        return self.shape[d - 1] if d <= len(self.shape) else 1

    def stride(self, d):
        return _prod(self.shape[:d - 1])

    def reshape(self, *shape):
        shape = shape[0] if len(shape) == 1 and not isinstance(shape[0], int) else shape
        return KnetArray(self.data, tuple(shape))

    def vec(self):
        return KnetArray(self.data, (self.data.numel(),))

    def view(self, start, length):
        """Contiguous range [start, start+length) (0-based) as a vector aliasing the memory."""
        return KnetArray(self.data[start:start + length], (length,))

    def numpy(self):
        return np.asfortranarray(self.data.detach().cpu().numpy().reshape(self.shape, order="F"))

    def as_rowmajor(self):
        """The same memory as a torch tensor with reversed dims (a (m,n) column-major matrix
        is a (n,m) row-major one); used to hand matrices to cuBLAS through torch."""
        return self.data.view(tuple(reversed(self.shape)))

    def __repr__(self):
        return f"KnetArray{{{self.dtype},{self.ndim}}}{self.shape}"

    # ---- indexing: Julia's index kinds, 1-based (see indexing.py) -----------------------------
    def __getitem__(self, I):
        from . import indexing
        return indexing.getindex(self, *(I if isinstance(I, tuple) else (I,)))

    def __setitem__(self, I, v):
        from . import indexing
        indexing.setindex_(self, v, *(I if isinstance(I, tuple) else (I,)))

    # ---- broadcasting operators (Julia's dotted forms) ------------------------------------
    def __add__(self, o):
        from . import ops
        if hasattr(o, "grad") and hasattr(o, "value"):      # a tracked value: its reflected method records
            return NotImplemented
        return ops.broadcast("add", self, o)

    def __radd__(self, o):
        from . import ops
        return ops.broadcast("add", o, self)

    def __sub__(self, o):
        from . import ops
        if hasattr(o, "grad") and hasattr(o, "value"):      # a tracked value: its reflected method records
            return NotImplemented
        return ops.broadcast("sub", self, o)

    def __rsub__(self, o):
        from . import ops
        return ops.broadcast("sub", o, self)

    def __mul__(self, o):
        from . import ops
        if hasattr(o, "grad") and hasattr(o, "value"):      # a tracked value: its reflected method records
            return NotImplemented
        return ops.broadcast("mul", self, o)

    def __rmul__(self, o):
        from . import ops
        return ops.broadcast("mul", o, self)

    def __truediv__(self, o):
        from . import ops
        if hasattr(o, "grad") and hasattr(o, "value"):      # a tracked value: its reflected method records
            return NotImplemented
        return ops.broadcast("div", self, o)

    def __rtruediv__(self, o):
        from . import ops
        return ops.broadcast("div", o, self)

    def __neg__(self):
        from . import ops
        return ops.unary("neg", self)

    def __matmul__(self, o):
        from . import ops
        if hasattr(o, "grad") and hasattr(o, "value"):
            return NotImplemented
        return ops.matmul(self, o)
