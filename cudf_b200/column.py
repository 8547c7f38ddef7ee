"""Device columns: torch tensors holding the reference's Arrow layout
(cudf::column / column_view, cpp/include/cudf/column/column_view.hpp:236-243,469).

torch is used for device memory and streams only; all compute happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .types import HostColumn, STORAGE_DTYPE, TypeId


def _to_device(arr: Optional[np.ndarray], device, pinned: bool):
    if arr is None:
        return None
    a = np.ascontiguousarray(arr)
    t = torch.from_numpy(a.view(np.uint8).reshape(-1))
    if pinned:
        t = t.pin_memory()
    return t.to(device, non_blocking=pinned)


class Column:
    """A column on the device.  ``data``/``mask``/``offsets`` are uint8 torch tensors (raw bytes)."""

    def __init__(self, type_id: int, size: int, data: Optional[torch.Tensor], mask: Optional[torch.Tensor] = None,
                 offset: int = 0, null_count: int = -1, offsets: Optional[torch.Tensor] = None,
                 offsets_type: TypeId = TypeId.INT32, scale: int = 0, children: Optional[list] = None):
        self.type_id = TypeId(type_id)
        self.scale = int(scale)  # DECIMAL32/64 only
        self.size = int(size)
        self.data = data
        self.mask = mask
        self.offset = int(offset)
        self.null_count = int(null_count) if mask is not None else 0
        self.offsets = offsets
        self.offsets_type = TypeId(offsets_type)
        self.children = children  # STRUCT results (SUM_OVERFLOW): the child columns

    # -- construction ---------------------------------------------------------------------
    @staticmethod
    def from_host(hc: HostColumn, device="cuda", pinned: bool = False) -> "Column":
        """Copies a host column to the device (pinned=True stages through pinned memory and
        copies asynchronously on the current stream)."""
        offs_t = TypeId.INT32
        if hc.offsets is not None and hc.offsets.dtype == np.int64:
            offs_t = TypeId.INT64
        if hc.children:  # DICTIONARY32 values: {indices, keys}
            kids = [Column.from_host(c, device, pinned) for c in hc.children]
            return Column(hc.type_id, hc.size, None, _to_device(hc.mask, device, pinned), hc.offset,
                          hc.null_count if hc.mask is not None else 0, children=kids)
        return Column(hc.type_id, hc.size, _to_device(hc.data, device, pinned), _to_device(hc.mask, device, pinned),
                      hc.offset, hc.null_count if hc.mask is not None else 0, _to_device(hc.offsets, device, pinned),
                      offs_t, getattr(hc, "scale", 0))

    @staticmethod
    def from_tensor(values: torch.Tensor, mask_words: Optional[torch.Tensor] = None, type_id: Optional[int] = None,
                    null_count: int = -1) -> "Column":
        """Wraps a 1-D device tensor (no copy).  ``mask_words`` is an int32/uint8 tensor of bitmask words."""
        tmap = {torch.int8: TypeId.INT8, torch.int16: TypeId.INT16, torch.int32: TypeId.INT32,
                torch.int64: TypeId.INT64, torch.uint8: TypeId.UINT8, torch.float32: TypeId.FLOAT32,
                torch.float64: TypeId.FLOAT64, torch.bool: TypeId.BOOL8}
        t = TypeId(type_id) if type_id is not None else tmap[values.dtype]
        v = values.contiguous()
        raw = v.view(torch.uint8) if v.dtype != torch.bool else v.to(torch.uint8)
        m = None if mask_words is None else mask_words.contiguous().view(torch.uint8)
        return Column(t, v.numel(), raw.reshape(-1), m, 0, null_count)

    # -- host copies ----------------------------------------------------------------------
    def to_host(self) -> HostColumn:
        def np_of(t, dtype):
            return None if t is None else t.cpu().numpy().view(dtype).copy()
        mask = np_of(self.mask, np.uint32)
        if self.type_id in (TypeId.STRUCT, TypeId.DICTIONARY32):
            return HostColumn(self.type_id, self.size, None, mask, self.offset, None, 0,
                              [c.to_host() for c in (self.children or [])])
        if self.type_id == TypeId.STRING:
            od = np.int64 if self.offsets_type == TypeId.INT64 else np.int32
            chars = np.zeros(0, np.uint8) if self.data is None else self.data.cpu().numpy().copy()
            return HostColumn(self.type_id, self.size, chars, mask, self.offset, np_of(self.offsets, od))
        dt = np.dtype(STORAGE_DTYPE[self.type_id])
        data = np.zeros(0, dt) if self.data is None else self.data.cpu().numpy()[: (self.offset + self.size) * dt.itemsize].view(dt).copy()
        return HostColumn(self.type_id, self.size, data, mask, self.offset, None, self.scale)

    # -- C view ---------------------------------------------------------------------------
    def c_view(self, keep: list) -> _lib.ColumnView:
        """The b2_column_view of this column; objects that must outlive the call go to ``keep``."""
        v = _lib.ColumnView()
        v.type_id = int(self.type_id)
        v.scale = self.scale
        v.size = self.size
        v.null_count = self.null_count if self.mask is not None else 0
        v.data = self.data.data_ptr() if self.data is not None and self.data.numel() else None
        v.null_mask = self.mask.data_ptr() if self.mask is not None else None
        v.offset = self.offset
        v.num_children = 0
        v.children = None
        if self.type_id == TypeId.STRING:
            child = (_lib.ColumnView * 1)()
            child[0].type_id = int(self.offsets_type)
            child[0].size = self.size + 1
            child[0].data = self.offsets.data_ptr() if self.offsets is not None and self.offsets.numel() else None
            child[0].offset = 0
            keep.append(child)
            v.num_children = 1
            v.children = child
        elif self.children:
            kids = (_lib.ColumnView * len(self.children))(*[c.c_view(keep) for c in self.children])
            keep.append(kids)
            v.num_children = len(self.children)
            v.children = kids
        keep.append(self)
        return v


class Table:
    """An ordered set of equally sized columns (cudf::table_view)."""

    def __init__(self, columns: Sequence[Column]):
        self._columns: List[Column] = list(columns)

    def columns(self) -> List[Column]:
        return self._columns

    def num_columns(self) -> int:
        return len(self._columns)

    def num_rows(self) -> int:
        return self._columns[0].size if self._columns else 0


class TorchAllocator:
    """b2_allocator backed by torch's caching allocator: the stand-in for an rmm memory resource.
    Buffers the library asks for are uint8 tensors; finished results adopt them."""

    def __init__(self, device):
        self.device = device
        self.live = {}
        self._alloc_cb = _lib.ALLOC_FN(self._alloc)
        self._free_cb = _lib.FREE_FN(self._free)
        self.struct = _lib.Allocator(self._alloc_cb, self._free_cb, None)

    def _alloc(self, nbytes, stream, ctx):
        try:
            t = torch.empty(max(int(nbytes), 8), dtype=torch.uint8, device=self.device)
        except Exception:
            return None
        self.live[t.data_ptr()] = t
        return t.data_ptr()

    def _free(self, ptr, nbytes, stream, ctx):
        self.live.pop(ptr, None)

    def adopt(self, ptr) -> Optional[torch.Tensor]:
        return None if not ptr else self.live.pop(ptr)


_ALLOCATORS = {}


def allocator_for(device) -> TorchAllocator:
    """One allocator per device, reused across calls (building the ctypes callbacks is the
    expensive part; the allocator itself only keeps the buffers of calls in flight)."""
    key = str(device)
    a = _ALLOCATORS.get(key)
    if a is None:
        a = _ALLOCATORS[key] = TorchAllocator(device)
    return a
