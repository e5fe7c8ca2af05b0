"""Host mirror of the reference's `SavedFormat` (crates/trainer/src/model/weights.rs:183-335).

A list of entries describes the bytes an engine loads: custom bytes, or a weight id that passes
through transforms and a quantisation.  The builder calls read like the reference's:

    SavedFormat.id("l0w").merge_factoriser().round().quantise("i16", 255)
    SavedFormat.id("l1w").round().quantise("i16", 64).transpose()
    SavedFormat.custom(b"header")

`merge_factoriser` stands for the closure of examples/progression/3_input_buckets.rs:46-53
(value + l0f repeated over the input buckets); the library applies merge, then transpose, then
quantises, whatever order the calls were made in, as the reference quantises last too.
All arithmetic is done by the C library (b200_quantise / b200_saved_format_write).
"""
from __future__ import annotations

import ctypes
import dataclasses

import numpy as np

from . import _lib

QUANT = {"f32": 0, "float": 0, "i8": 1, "i16": 2, "i32": 3}
QUANT_DTYPE = {0: np.dtype("<f4"), 1: np.dtype("i1"), 2: np.dtype("<i2"), 3: np.dtype("<i4")}


@dataclasses.dataclass(frozen=True)
class SavedFormat:
    weight: str | None = None
    custom_bytes: bytes | None = None
    quant: int = 0
    multiplier: int = 1
    rounded: bool = False
    transposed: bool = False
    merged: bool = False

    @staticmethod
    def id(weight: str) -> "SavedFormat":
        return SavedFormat(weight=weight)

    @staticmethod
    def custom(data: bytes) -> "SavedFormat":
        return SavedFormat(custom_bytes=bytes(data))

    def _weight_only(self) -> None:
        if self.custom_bytes is not None:
            raise ValueError("custom bytes take no transform or quantisation")  # the reference asserts the same

    def round(self) -> "SavedFormat":
        self._weight_only()
        return dataclasses.replace(self, rounded=True)

    def quantise(self, target: str, multiplier: int) -> "SavedFormat":
        self._weight_only()
        return dataclasses.replace(self, quant=QUANT[target], multiplier=int(multiplier))

    def transpose(self) -> "SavedFormat":
        self._weight_only()
        if self.weight is None:
            raise ValueError("transpose needs a weight id")
        return dataclasses.replace(self, transposed=True)

    def merge_factoriser(self) -> "SavedFormat":
        self._weight_only()
        return dataclasses.replace(self, merged=True)


def c_formats(formats):
    """(array of b200_saved_format, objects to keep alive while it is used)"""
    arr = (_lib.CSavedFormat * max(1, len(formats)))()
    keep = []
    for i, f in enumerate(formats):
        if f.custom_bytes is not None:
            buf = ctypes.create_string_buffer(f.custom_bytes, len(f.custom_bytes))
            keep.append(buf)
            arr[i].id = None
            arr[i].custom = ctypes.cast(buf, ctypes.c_void_p)
            arr[i].custom_len = len(f.custom_bytes)
        else:
            arr[i].id = f.weight.encode()
            arr[i].quant, arr[i].multiplier = f.quant, f.multiplier
            arr[i].round, arr[i].transpose, arr[i].merge_factoriser = int(f.rounded), int(f.transposed), int(f.merged)
    return arr, keep


def quantise(values: np.ndarray, target: str, multiplier: int, round: bool = False) -> np.ndarray:
    """QuantTarget::quantise (weights.rs:281-331): raises B200Error(-4) if a value does not fit."""
    v = np.ascontiguousarray(values, dtype=np.float32).ravel()
    q = QUANT[target]
    out = np.empty(v.size, dtype=QUANT_DTYPE[q])
    _lib.check(_lib.load().b200_quantise(v.ctypes.data, v.size, q, int(multiplier), int(round), out.ctypes.data))
    return out


def transpose(values: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """SavedFormat::transpose_impl (weights.rs:254-269) on a column-major rows x cols matrix."""
    v = np.ascontiguousarray(values, dtype=np.float32).ravel()
    if v.size != rows * cols:
        raise ValueError("shape does not match the number of values")
    out = np.empty_like(v)
    _lib.check(_lib.load().b200_transpose(v.ctypes.data, rows, cols, out.ctypes.data))
    return out
