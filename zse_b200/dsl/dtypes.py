"""Element types and the tensor descriptor of the kernel language
(zse-compiler/zse_compiler/types/dtypes.py:6-59, tensor.py:14-107)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class DType:
    name: str
    bits: int
    c_name: str              # spelling in CUDA C
    kind: str                # "float" | "int" | "uint"
    torch_name: Optional[str] = None

    @property
    def nbytes(self) -> float:
        return self.bits / 8

    def size_bytes(self) -> int:
        """Whole bytes one element occupies (4-bit types round up to 1), the reference's accessor
        (zse-compiler/zse_compiler/types/dtypes.py:14-15)."""
        return (self.bits + 7) // 8

    @property
    def size_bits(self) -> int:
        return self.bits

    @property
    def is_float(self) -> bool:
        return self.kind == "float"

    @property
    def is_packed(self) -> bool:
        return self.bits < 8

    def __repr__(self) -> str:
        return self.name

    def __getitem__(self, _):      # lets ``Tensor[float16]``-style annotations be written with any nesting
        return self


float32 = DType("float32", 32, "float", "float", "float32")
float16 = DType("float16", 16, "__half", "float", "float16")
bfloat16 = DType("bfloat16", 16, "__nv_bfloat16", "float", "bfloat16")
int32 = DType("int32", 32, "int", "int", "int32")
int16 = DType("int16", 16, "short", "int", "int16")
int8 = DType("int8", 8, "signed char", "int", "int8")
uint32 = DType("uint32", 32, "unsigned int", "uint", None)
uint16 = DType("uint16", 16, "unsigned short", "uint", None)
uint8 = DType("uint8", 8, "unsigned char", "uint", "uint8")
int4 = DType("int4", 4, "unsigned char", "int", None)        # two per byte, low nibble first
uint4 = DType("uint4", 4, "unsigned char", "uint", None)

ALL = {d.name: d for d in (float32, float16, bfloat16, int32, int16, int8, uint32, uint16, uint8, int4, uint4)}


def from_string(name: str) -> DType:
    """``"float16"`` / ``"fp16"`` / ``"half"`` ... -> element type."""
    alias = {"fp32": "float32", "float": "float32", "fp16": "float16", "half": "float16", "bf16": "bfloat16",
             "int": "int32", "uint": "uint32"}
    key = alias.get(name.lower(), name.lower())
    if key not in ALL:
        raise ValueError(f"unknown element type '{name}'")
    return ALL[key]


def from_torch(dtype) -> DType:
    name = str(dtype).replace("torch.", "")
    for d in ALL.values():
        if d.torch_name == name:
            return d
    raise TypeError(f"no kernel element type for {dtype}")


class _TensorMeta(type):
    def __getitem__(cls, dtype: DType) -> "TensorSpec":
        """``Tensor[float16]`` as a parameter annotation fixes the element type of that parameter."""
        if not isinstance(dtype, DType):
            raise TypeError("Tensor[...] takes an element type")
        return TensorSpec(dtype)


@dataclass(frozen=True)
class TensorSpec:
    dtype: DType


class Tensor(metaclass=_TensorMeta):
    """Shape + element type + (optionally) device storage.  As an annotation it marks a pointer parameter; as an
    object it describes a buffer: ``numel``, ``nbytes`` (packed types count bits), ``ndim``, ``data_ptr``."""

    def __init__(self, shape: Tuple[int, ...], dtype: DType = float32, data=None):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        self.data = data            # a torch tensor that owns the storage, or None for a bare description

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return (self.numel * self.dtype.bits + 7) // 8

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def data_ptr(self) -> int:
        return int(self.data.data_ptr()) if self.data is not None else 0

    # descriptor helpers of the reference (zse-compiler/zse_compiler/types/tensor.py:69-107)
    @property
    def device(self) -> str:
        return str(self.data.device) if self.data is not None else "cpu"

    @property
    def strides(self) -> Tuple[int, ...]:
        """Row-major strides in elements (descriptors are always dense)."""
        out, acc = [], 1
        for dim in reversed(self.shape):
            out.append(acc)
            acc *= dim
        return tuple(reversed(out))

    def is_contiguous(self) -> bool:
        return self.data is None or not hasattr(self.data, "is_contiguous") or bool(self.data.is_contiguous())

    def reshape(self, *new_shape: int) -> "Tensor":
        """A descriptor of the same storage under another shape (the element count must match)."""
        if len(new_shape) == 1 and isinstance(new_shape[0], (tuple, list)):
            new_shape = tuple(new_shape[0])
        n = 1
        for dim in new_shape:
            n *= int(dim)
        if n != self.numel:
            raise ValueError(f"Cannot reshape {self.shape} ({self.numel} elements) to {tuple(new_shape)} ({n} elements)")
        data = self.data
        if data is not None and self.dtype.torch_name and hasattr(data, "reshape"):
            data = data.reshape(tuple(int(d) for d in new_shape))
        return Tensor(tuple(new_shape), self.dtype, data)

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, {'allocated' if self.data is not None else 'no storage'})"


def _storage(shape, dtype: DType, device, zero: bool):
    import torch
    t_dtype = getattr(torch, dtype.torch_name) if dtype.torch_name else None
    n = 1
    for s in shape:
        n *= int(s)
    make = torch.zeros if zero else torch.empty
    if t_dtype is None:            # packed or unsigned types without a torch twin: raw bytes
        return make((n * dtype.bits + 7) // 8, dtype=torch.uint8, device=device)
    return make(tuple(shape), dtype=t_dtype, device=device)


def empty(shape, dtype: DType = float32, device=None) -> Tensor:
    import torch
    device = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
    return Tensor(shape, dtype, _storage(shape, dtype, device, False))


def zeros(shape, dtype: DType = float32, device=None) -> Tensor:
    import torch
    device = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
    return Tensor(shape, dtype, _storage(shape, dtype, device, True))
