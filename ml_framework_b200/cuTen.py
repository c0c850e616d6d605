"""`cuten`: the raw-pointer device tensor of the Seera Python layer, for the B200 engine.

Same class surface as the reference's cuTen.py (cuTen.py:9-806): plain attributes
`main_ptr` (device address as int), `shape`, `size`, `dtype`, `_owns_memory`; the constructor
uploads a NumPy array or list, or makes an empty shell (`cuten(data=None)`) whose fields the
caller assigns; operators have value semantics; every method maps to one `seera_cuda` call.

What is different underneath:
  * constants are lazy.  `zeros_like`, `ones_like`, `zeros`, `ones` (and a constant times a
    Python scalar) return a tensor that records only its fill value; device memory is allocated
    and filled on the first read of `main_ptr`.  The reference uploads a host array for each
    (cuTen.py:95-111), five per graph node (Seera_init.py:75-80), most of which are never read.
  * `0 + x`, `x + 0`, `1 * x`, `x * 1` with a lazy constant of the same shape return a view
    of `x` (same memory, own metadata): gradient accumulation `cp = cp + dX` (Seera_Engine.py:269-583) then costs nothing.
    Nothing in this class mutates device memory in place, so sharing is not observable.
  * a view (`reshape`, `flatten`) keeps its owner alive through `_base`, so the owner's memory
    cannot return to the pool while the view is reachable.
"""
from __future__ import annotations

import numpy as np

from . import seera_cuda

_UPLOAD = {"float32": seera_cuda.to_device_f32, "int32": seera_cuda.to_device_i32, "int16": seera_cuda.to_device_i16}
_NP = {"float32": np.float32, "int32": np.int32, "int16": np.int16}


def _numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


class cuten:
    supported_types = ["float32", "int32", "int16"]

    def __init__(self, data=None, dtype="float32"):
        if dtype not in self.supported_types:
            raise ValueError("[cuTen]:Not Supported by cuTen, try in CPU")
        self.dtype = dtype
        self._ptr = None
        self._const = None            # pending fill value of a lazy constant
        self._base = None             # owner of the memory this tensor views
        self._owns_memory = False
        if isinstance(data, (list, tuple)):
            data = np.array(data, dtype=dtype)
        if isinstance(data, np.ndarray):
            arr = np.ascontiguousarray(data.astype(dtype))
            self._ptr = _UPLOAD[dtype](arr)
            self.shape = arr.shape
            self.size = arr.size
            self._owns_memory = True
        else:
            self.shape = None
            self.size = None
            self._owns_memory = True     # an empty shell: the caller assigns a fresh address it owns

    # ---- the device address: plain attribute for callers, lazy for constants ----------------
    @property
    def main_ptr(self):
        if self._ptr is None and self._const is not None:
            n = int(self.size)
            if self._const == 0.0:
                self._ptr = seera_cuda.cuda_zeros_f(n)
            else:
                self._ptr = seera_cuda.cuda_ones_f(n)
                if self._const != 1.0:
                    seera_cuda.cuda_scaler_multiply_f(self._ptr, float(self._const), n)
            self._const = None
        return self._ptr

    @main_ptr.setter
    def main_ptr(self, value):
        self._ptr = value
        self._const = None

    def _lazy_value(self):
        """Fill value if this tensor is an unmaterialised constant, else None."""
        return self._const if self._ptr is None else None

    def __del__(self):
        ptr = getattr(self, "_ptr", None)
        if getattr(self, "_owns_memory", False) and ptr is not None and getattr(self, "_base", None) is None:
            try:
                seera_cuda.cuda_free(ptr)
            except Exception:
                pass
            self._ptr = None

    # ---- construction helpers -------------------------------------------------------------------
    @classmethod
    def _wrap(cls, ptr, shape, dtype="float32"):
        t = cls(None, dtype)
        t._ptr = ptr
        t.shape = tuple(shape)
        t.size = _numel(shape)
        return t

    @classmethod
    def _constant(cls, shape, value, dtype="float32"):
        t = cls(None, dtype)
        t.shape = tuple(shape)
        t.size = _numel(shape)
        t._const = float(value)
        return t

    @classmethod
    def ones_like(cls, arr):
        return cls._constant(arr.shape, 1.0)

    @classmethod
    def zeros_like(cls, arr):
        return cls._constant(arr.shape, 0.0)

    @classmethod
    def ones_like_fromnumpy(cls, arr):
        return cls(arr, dtype=str(arr.dtype))

    @classmethod
    def zeros_like_fromnumpy(cls, arr):
        return cls(arr, dtype=str(arr.dtype))

    @classmethod
    def zeros(cls, shape):
        return cls._constant(tuple(shape), 0.0)

    @classmethod
    def ones(cls, shape):
        return cls._constant(tuple(shape), 1.0)

    # ---- transfers --------------------------------------------------------------------------------
    def to_host_f32(self):
        c = self._lazy_value()
        if c is not None:
            return np.full(self.shape, c, np.float32)
        return seera_cuda.to_host_f32(self.main_ptr, tuple(self.shape))

    def to_host_i32(self):
        return seera_cuda.to_host_i32(self.main_ptr, tuple(self.shape))

    # ---- broadcasting helpers -----------------------------------------------------------------------
    @staticmethod
    def _pad_shape_4d(shape):
        return (1,) * (4 - len(shape)) + tuple(shape)

    @staticmethod
    def _broadcast_out_shape(a_shape, b_shape):
        nd = max(len(a_shape), len(b_shape))
        a = (1,) * (nd - len(a_shape)) + tuple(a_shape)
        b = (1,) * (nd - len(b_shape)) + tuple(b_shape)
        out = []
        for x, y in zip(a, b):
            if x != y and x != 1 and y != 1:
                raise ValueError(f"[cuTen]: Shapes {a_shape} and {b_shape} not broadcastable")
            out.append(max(x, y))
        return tuple(out)

    def _scalar_op(self, kernel, k):
        """Out-of-place scalar op: copy, then the in-place kernel on the copy (self is never mutated)."""
        p = seera_cuda.cuda_malloc_f32(self.size)
        seera_cuda.cuda_memcopy_devicetodevice(p, self.main_ptr, self.size)
        kernel(p, float(k), self.size)
        return cuten._wrap(p, self.shape)

    def _binary(self, other, flat_kernel, bcast_kernel, identity):
        if tuple(self.shape) == tuple(other.shape):
            if other._lazy_value() == identity:
                return self.reshape(self.shape)       # a view: shares memory, owns its own metadata
            if self._lazy_value() == identity:
                return other.reshape(other.shape)
            p = seera_cuda.cuda_malloc_f32(self.size)
            flat_kernel(self.main_ptr, other.main_ptr, p, self.size)
            return cuten._wrap(p, self.shape)
        out_shape = cuten._broadcast_out_shape(self.shape, other.shape)
        if len(out_shape) > 4:
            raise ValueError(f"[cuTen]: Shapes {self.shape} and {other.shape} not broadcastable")
        p = seera_cuda.cuda_malloc_f32(_numel(out_shape))
        bcast_kernel(self.main_ptr, other.main_ptr, p, *cuten._pad_shape_4d(self.shape), *cuten._pad_shape_4d(other.shape))
        return cuten._wrap(p, out_shape)

    # ---- arithmetic ---------------------------------------------------------------------------------------
    def __add__(self, other):
        if isinstance(other, cuten):
            return self._binary(other, seera_cuda.cuda_elemadd, seera_cuda.broadcast_add_4d, 0.0)
        if isinstance(other, (int, float)):
            c = self._lazy_value()
            if c is not None:
                return cuten._constant(self.shape, c + other)
            return self._scalar_op(seera_cuda.cuda_scaler_add_f, other)
        return None          # the reference falls through for unsupported operands

    def __mul__(self, other):
        if isinstance(other, cuten):
            return self._binary(other, seera_cuda.cuda_elemmult, seera_cuda.broadcast_mul_4d, 1.0)
        if isinstance(other, (int, float)):
            c = self._lazy_value()
            if c is not None:
                return cuten._constant(self.shape, c * other)
            return self._scalar_op(seera_cuda.cuda_scaler_multiply_f, other)
        raise ValueError("[cuTen]: Not Supported, Can be Device Mismatch")

    def __pow__(self, other):
        if isinstance(other, (int, float)):
            return self._scalar_op(seera_cuda.cuda_power_of, other)
        return None

    def __neg__(self):
        return self * (-1)

    def __sub__(self, other):
        return self + (-other)

    def __radd__(self, other):
        return self + other

    def __rsub__(self, other):
        return other + (self * -1)

    def __rmul__(self, other):
        return self * other

    def __truediv__(self, other):
        return self * other ** -1

    def __rtruediv__(self, other):
        return other * self ** -1

    # ---- views ----------------------------------------------------------------------------------------------
    def reshape(self, shape):
        shape = tuple(shape)
        if self.size != _numel(shape):
            raise ValueError(f"[cuTen]: Cannot reshape cuten of size: {self.size} to shape {shape}")
        c = self._lazy_value()
        if c is not None:
            return cuten._constant(shape, c, self.dtype)
        v = cuten._wrap(self.main_ptr, shape, self.dtype)
        v._owns_memory = False
        v._base = self if self._base is None else self._base
        return v

    def flatten(self):
        return self.reshape((self.shape[0], int(self.size / self.shape[0])))

    def __repr__(self):
        host = self.to_host_i32() if self.dtype == "int32" else self.to_host_f32()
        return f"cuten(shape={tuple(self.shape)}, dtype={self.dtype})\n{host}"

    @property
    def T(self):
        nd = len(self.shape)
        if nd < 2:
            p = seera_cuda.cuda_malloc_f32(self.size)
            seera_cuda.cuda_memcopy_devicetodevice(p, self.main_ptr, self.size)
            return cuten._wrap(p, self.shape)
        if nd == 2:
            r, c = self.shape
            p = seera_cuda.cuda_malloc_f32(self.size)
            seera_cuda.cuda_transpose_2d(self.main_ptr, p, r, c)
            return cuten._wrap(p, (c, r))
        if nd == 3:
            b, m, k = self.shape
            p = seera_cuda.cuda_malloc_f32(self.size)
            seera_cuda.cuda_transpose_3d(self.main_ptr, p, b, m, k)
            return cuten._wrap(p, (b, k, m))
        return cuten(self.to_host_f32().T.copy(), dtype="float32")     # >= 4-D: host round trip, as in the reference

    # ---- unary ops (the engine writes value and local gradient; the gradient is discarded here) -----------
    def _unary(self, kernel, *scalars):
        out = seera_cuda.cuda_malloc_f32(self.size)
        grad = seera_cuda.cuda_malloc_f32(self.size)
        kernel(self.main_ptr, *scalars, out, grad, self.size)
        seera_cuda.cuda_free(grad)
        return cuten._wrap(out, self.shape)

    def relu(self):
        return self._unary(seera_cuda.cuda_relu_fwd)

    def sigmoid(self):
        return self._unary(seera_cuda.cuda_sigmoid_fwd)

    def tanh(self):
        return self._unary(seera_cuda.cuda_tanh_fwd)

    def log(self):
        return self._unary(seera_cuda.cuda_log_fwd)

    def exp(self):
        return self._unary(seera_cuda.cuda_exp_fwd)

    def absolute(self):
        return self._unary(seera_cuda.cuda_abs_fwd)

    abs = absolute

    def sqrt(self):
        return self._unary(seera_cuda.cuda_sqrt_fwd)

    def clip(self, lo, hi):
        return self._unary(seera_cuda.cuda_clip_fwd, float(lo), float(hi))

    def softmax(self):
        if len(self.shape) < 2:
            raise ValueError("[cuTen]: softmax requires at least a 2-D tensor")
        C = self.shape[-1]
        p = seera_cuda.cuda_malloc_f32(self.size)
        seera_cuda.cuda_softmax_fwd(self.main_ptr, p, self.size // C, C)
        return cuten._wrap(p, self.shape)

    # ---- matmul: (M,K) or (B,M,K) times a shared (K,N) ---------------------------------------------------------
    def matmul(self, other):
        if len(self.shape) < 2 or len(other.shape) < 2:
            raise ValueError("[cuTen]: matmul requires at least 2-D tensors")
        M, K = self.shape[-2], self.shape[-1]
        N = other.shape[-1]
        if other.shape[-2] != K:
            raise ValueError(f"[cuTen]: matmul: inner dimensions must agree, got {self.shape} @ {other.shape}")
        if len(self.shape) > 3:
            raise ValueError("[cuTen] A cannot be of more than 3 Dimensional")
        if len(other.shape) > 2:
            raise ValueError("[cuTen] B cannot be of more than 2 Dimensional")
        nb = self.shape[0] if len(self.shape) == 3 else 1
        p = seera_cuda.cuda_malloc_f32(nb * M * N)
        seera_cuda.cuda_matmul(self.main_ptr, other.main_ptr, p, M, N, K, nb)
        return cuten._wrap(p, (M, N) if nb == 1 else (nb, M, N))

    __matmul__ = matmul

    # ---- single-axis reductions ----------------------------------------------------------------------------------
    def _reduction_meta(self, dim):
        nd = len(self.shape)
        if dim < 0:
            dim += nd
        if dim < 0 or dim >= nd:
            raise ValueError(f"[cuTen]: dim {dim} out of range for shape {self.shape}")
        out_shape = tuple(d for i, d in enumerate(self.shape) if i != dim) or (1,)
        return out_shape, _numel(out_shape), nd, dim, np.array(self.shape, dtype=np.int32)

    def _reduce(self, kernel, dim):
        out_shape, out_size, nd, dim, dimarr = self._reduction_meta(dim)
        p = seera_cuda.cuda_malloc_f32(out_size)
        kernel(self.main_ptr, p, nd, dim, dimarr)
        return cuten._wrap(p, out_shape)

    def sum(self, dim):
        return self._reduce(seera_cuda.cuda_sum_fwd, dim)

    def mean(self, dim):
        return self._reduce(seera_cuda.cuda_mean_fwd, dim)

    def max(self, dim):
        return self._reduce(seera_cuda.cuda_max_fwd, dim)

    def min(self, dim):
        return self._reduce(seera_cuda.cuda_min_fwd, dim)

    def _argreduce(self, kernel, dim):
        out_shape, out_size, nd, dim, dimarr = self._reduction_meta(dim)
        p = seera_cuda.cuda_malloc_i32(out_size)
        kernel(self.main_ptr, p, nd, dim, dimarr)
        return cuten._wrap(p, out_shape, "int32")

    def argmax(self, dim):
        return self._argreduce(seera_cuda.cuda_argmax_fwd, dim)

    def argmin(self, dim):
        return self._argreduce(seera_cuda.cuda_argmin_fwd, dim)

    # ---- convolution family (NCHW) ------------------------------------------------------------------------------------
    def conv2d(self, kernel, strideh=1, stridew=1, padh=0, padw=0):
        if len(self.shape) != 4 or len(kernel.shape) != 4:
            raise ValueError("[cuTen]: conv2d expects 4-D tensors (N,C,H,W) and (F,C,KH,KW)")
        N, C, H, W = self.shape
        F, _, KH, KW = kernel.shape
        OH = (H + 2 * padh - KH) // strideh + 1
        OW = (W + 2 * padw - KW) // stridew + 1
        p = seera_cuda.cuda_malloc_f32(N * F * OH * OW)
        seera_cuda.cuda_conv2d_fwd(self.main_ptr, kernel.main_ptr, p, N, C, H, W, F, KH, KW, padh, padw, strideh, stridew)
        return cuten._wrap(p, (N, F, OH, OW))

    def maxpool2d(self, KH, KW, strideh=1, stridew=1, padh=0, padw=0):
        if len(self.shape) != 4:
            raise ValueError("[cuTen]: maxpool2d expects 4-D tensor (N,C,H,W)")
        N, C, H, W = self.shape
        OH = (H + 2 * padh - KH) // strideh + 1
        OW = (W + 2 * padw - KW) // stridew + 1
        out = seera_cuda.cuda_malloc_f32(N * C * OH * OW)
        mask_ptr = seera_cuda.cuda_malloc_i32(self.size)
        seera_cuda.cuda_maxpool_fwd(self.main_ptr, out, mask_ptr, N, C, H, W, KH, KW, padh, padw, strideh, stridew)
        mask = cuten._wrap(mask_ptr, self.shape, "int32")
        return cuten._wrap(out, (N, C, OH, OW)), mask

    def unpool(self, sh, sw):
        if len(self.shape) != 4:
            raise ValueError("[cuTen]:unpool expects 4-D tensor (N,C,H,W)")
        N, C, H, W = self.shape
        p = seera_cuda.cuda_malloc_f32(self.size * sh * sw)
        seera_cuda.cuda_unpooling_fwd(self.main_ptr, p, N, C, H, W, sh, sw)
        return cuten._wrap(p, (N, C, H * sh, W * sw))

    def conv2d_transpose(self, kernel, strideh=1, stridew=1, padh=0, padw=0):
        if len(self.shape) != 4 or len(kernel.shape) != 4:
            raise ValueError("[cuTen]: conv2d_transpose expects 4-D tensors (N,Cin,H,W) and (Cin,Cout,KH,KW)")
        N, Cin, H, W = self.shape
        _, Cout, KH, KW = kernel.shape
        Ho = (H - 1) * strideh - 2 * padh + KH
        Wo = (W - 1) * stridew - 2 * padw + KW
        p = seera_cuda.cuda_malloc_f32(N * Cout * Ho * Wo)
        seera_cuda.cuda_conv2DTranpose_fwd(self.main_ptr, kernel.main_ptr, p, N, Cin, H, W, Cout, KH, KW,
                                           strideh, stridew, padh, padw)
        return cuten._wrap(p, (N, Cout, Ho, Wo))

    # ---- concatenation along axis 1: one strided-copy launch each way (the reference loops over the samples) ---------------
    def _concat(self, other, out_shape):
        N = self.shape[0]
        n1, n2 = self.size // N, other.size // N
        p = seera_cuda.cuda_malloc_f32(self.size + other.size)
        seera_cuda.concat_fwd(self.main_ptr, other.main_ptr, p, N, n1, n2)
        return cuten._wrap(p, out_shape)

    def concatenate2D(self, other):
        if self.shape[0] != other.shape[0]:
            raise ValueError(f"[cuTen]: No of Batches should be same, received {self.shape[0]} and {other.shape[0]}")
        if self.shape[2:] != other.shape[2:]:
            raise ValueError(f"[cuTen]: H x W should be same, received ({self.shape[2]},{self.shape[3]}) and "
                             f"({other.shape[2]},{other.shape[3]})")
        return self._concat(other, (self.shape[0], self.shape[1] + other.shape[1], self.shape[2], self.shape[3]))

    def concatenate1D(self, other):
        if self.shape[0] != other.shape[0]:
            raise ValueError(f"[cuTen]: No of Batches should be same, received {self.shape[0]} and {other.shape[0]}")
        return self._concat(other, (self.shape[0], self.shape[1] + other.shape[1]))

    @classmethod
    def _concat_backward(cls, dout, a, b):
        if dout.shape[0] != a.shape[0]:
            raise ValueError("[cuTen]: Batch mismatch in backward")
        N = a.shape[0]
        n1, n2 = a.size // N, b.size // N
        p1, p2 = seera_cuda.cuda_malloc_f32(a.size), seera_cuda.cuda_malloc_f32(b.size)
        seera_cuda.concat_bwd(dout.main_ptr, p1, p2, N, n1, n2)
        return cls._wrap(p1, a.shape), cls._wrap(p2, b.shape)

    @classmethod
    def concatenate2D_backward(cls, dout, self, other):
        return cls._concat_backward(dout, self, other)

    @classmethod
    def concatenate1D_backward(cls, dout, self, other):
        return cls._concat_backward(dout, self, other)
