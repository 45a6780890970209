"""Device buffers for the host side of the MoE layer.

``DeviceStorage`` carries the same fields the upstream ``CUDAStorage`` exposes (``ptr``, ``size``,
``dtype``, ``nbytes``, ``device``; src/qutai/backends/cuda.py:20-58), so every function of
``qutai_b200.cuda_lm`` accepts either kind — all they read is ``ptr``/``size``/``dtype``.  A storage
either owns an allocation made through the library, or wraps memory owned by someone else (an
upstream ``CUDAStorage``, a ``torch`` tensor's ``data_ptr()``), or is a view into another storage
(how the stacked expert weights are handed out as separate parameters).

Every storage carries a ``generation`` counter that the host-visible write paths of this package bump
(``upload_bytes``, ``fill_zero``, ``fill_normal``, ``copy_from``, the optimizer step); a view shares its
parent's counter.  A reader that keeps something derived from the contents (the layer's bf16 operand
copies of the fp32 weights) compares generations instead of rebuilding it on every use.  Code that
writes through the raw ``ptr`` calls ``touch()`` afterwards.
"""
from __future__ import annotations

import ctypes
import os
import struct
from array import array

from . import lib

_FORMATS = {"float32": "f", "float64": "d", "int32": "i", "int64": "q"}
_cache: dict[int, list[int]] = {}
_cached_bytes = 0
# Freed blocks are kept for reuse up to this many bytes (a B200 has 180 GB; activations and gradients of the
# benchmark shapes are hundreds of MB each, and a block that is really freed costs a device-wide synchronisation:
# with 16 GB the 64-expert layer's step filled the cache and every later gradient buffer was freed and allocated
# anew, 10 ms a time); QUTAI_MOE_CACHE_BYTES overrides it.
CACHE_LIMIT_BYTES = int(os.environ.get("QUTAI_MOE_CACHE_BYTES", 64 << 30))


def _bucket(nbytes):
    step = 512 if nbytes < (1 << 16) else 1 << 16
    return max(step, (nbytes + step - 1) // step * step)


def _allocate(nbytes):
    global _cached_bytes
    size = _bucket(nbytes)
    free = _cache.get(size)
    if free:
        _cached_bytes -= size
        address = free.pop()
        if not free:
            del _cache[size]
        return address, size
    address = ctypes.c_uint64()
    try:
        lib.call("qmoe_malloc", ctypes.byref(address), size)
    except RuntimeError:
        empty_cache()  # out of memory: drop cached blocks and try once more
        lib.call("qmoe_malloc", ctypes.byref(address), size)
    return address.value, size


def _release(address, size):
    """Keep the block for reuse.  Over the limit the blocks that have waited longest go first (the one just released
    is the likeliest to be asked for again: a gradient buffer of the next step)."""
    global _cached_bytes
    if size > CACHE_LIMIT_BYTES:
        lib.load().qmoe_free(address)
        return
    while _cached_bytes + size > CACHE_LIMIT_BYTES and _cache:
        oldest = next(iter(_cache))            # dicts keep insertion order: the size that entered the cache first
        blocks = _cache[oldest]
        lib.load().qmoe_free(blocks.pop(0))
        _cached_bytes -= oldest
        if not blocks:
            del _cache[oldest]
    _cache.setdefault(size, []).append(address)
    _cached_bytes += size


def empty_cache():
    global _cached_bytes
    handle = lib.load()
    for blocks in _cache.values():
        for address in blocks:
            handle.qmoe_free(address)
    _cache.clear()
    _cached_bytes = 0


def bf16_bits(value):
    """Round one float to bfloat16 (nearest, ties to even) and return its 16 bits."""
    bits = struct.unpack("<I", struct.pack("<f", value))[0]
    if (bits & 0x7F800000) == 0x7F800000 and bits & 0x007FFFFF:
        return (bits >> 16) | 0x40  # NaN stays NaN
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF


class DeviceStorage:
    device = "cuda"

    def __init__(self, size, dtype="float32", *, ptr=None, owner=None):
        if dtype not in lib.ITEM_BYTES:
            raise ValueError(f"unsupported dtype {dtype!r}")
        if size < 0:
            raise ValueError("size must not be negative")
        self.size, self.dtype = int(size), dtype
        self.nbytes = self.size * lib.ITEM_BYTES[dtype]
        self._owner = owner
        self._block = None
        self._parent = None        # a view shares the generation counter of the storage it was cut from; an owning
                                   # storage refers to nobody (a reference to itself would keep its block from
                                   # being released until the cycle collector runs)
        self._generation = 0
        self._synced = {}          # id(source root) -> generation of the source this storage was last derived from
        if ptr is None:
            self.ptr, self._block = _allocate(max(self.nbytes, 1))
        else:
            self.ptr = int(ptr)

    def __del__(self):
        block, self._block = getattr(self, "_block", None), None
        if block is not None:
            try:
                _release(self.ptr, block)
            except Exception:
                pass

    # -- construction ---------------------------------------------------------------------
    @classmethod
    def wrap(cls, ptr, size, dtype, owner=None):
        """Storage over memory owned elsewhere; ``owner`` is kept alive with it."""
        return cls(size, dtype, ptr=ptr, owner=owner)

    def view(self, start, size):
        """Elements [start, start + size) of this storage as a storage of their own."""
        if start < 0 or size < 0 or start + size > self.size:
            raise ValueError("view exceeds the storage")
        out = DeviceStorage(size, self.dtype, ptr=self.ptr + start * lib.ITEM_BYTES[self.dtype], owner=self)
        out._parent = self._root
        return out

    # -- change tracking ------------------------------------------------------------------
    @property
    def _root(self):
        return self._parent if self._parent is not None else self

    @property
    def generation(self):
        """Grows with every write made through this package (shared by all views of one allocation)."""
        return self._root._generation

    def touch(self):
        """Declare the contents changed (for writers that went through the raw address)."""
        self._root._generation += 1

    def mark_derived_from(self, source):
        """Record that this storage now holds what was computed from ``source`` as it is now."""
        self._root._synced[id(source._root)] = source.generation

    def is_derived_from(self, source):
        """True while ``source`` has not been written since the last ``mark_derived_from(source)``."""
        return self._root._synced.get(id(source._root)) == source.generation

    @classmethod
    def zeros(cls, size, dtype="float32", stream=0):
        out = cls(size, dtype)
        out.fill_zero(stream)
        return out

    @classmethod
    def from_bytes(cls, data, dtype, stream=0):
        item = lib.ITEM_BYTES[dtype]
        if len(data) % item:
            raise ValueError("byte length is not a multiple of the item size")
        out = cls(len(data) // item, dtype)
        out.upload_bytes(data, stream)
        return out

    @classmethod
    def from_values(cls, values, dtype="float32", stream=0):
        values = list(values)
        if dtype == "bfloat16":
            data = array("H", (bf16_bits(float(v)) for v in values)).tobytes()
        else:
            data = array(_FORMATS[dtype], values).tobytes()
        return cls.from_bytes(data, dtype, stream)

    # -- transfers ------------------------------------------------------------------------
    def fill_zero(self, stream=0):
        lib.call("qmoe_memset", self.ptr, 0, self.nbytes, stream)
        self.touch()

    def fill_normal(self, mean, std, seed, stream=0):
        """N(mean, std) draws of the library's counter-based generator keyed by ``seed``."""
        lib.call("qmoe_normal_fill", self.ptr, lib.DTYPE_CODES[self.dtype], self.size, float(mean), float(std),
                 int(seed) & (2 ** 64 - 1), stream)
        self.touch()

    def copy_from(self, other, stream=0):
        if other.dtype != self.dtype or other.size != self.size:
            raise ValueError("copy_from needs a storage of the same dtype and size")
        lib.call("qmoe_memcpy_d2d", self.ptr, other.ptr, self.nbytes, stream)
        self.touch()

    def upload_bytes(self, data, stream=0):
        if len(data) != self.nbytes:
            raise ValueError("byte length does not match the storage")
        buffer = (ctypes.c_char * len(data)).from_buffer_copy(data) if len(data) else None
        if buffer is not None:
            lib.call("qmoe_memcpy_h2d", self.ptr, ctypes.cast(buffer, ctypes.c_void_p), self.nbytes, stream)
            lib.call("qmoe_stream_sync", stream)  # the staging buffer dies with this call
            self.touch()

    def tobytes(self, stream=0):
        buffer = ctypes.create_string_buffer(self.nbytes)
        if self.nbytes:
            lib.call("qmoe_memcpy_d2h", ctypes.cast(buffer, ctypes.c_void_p), self.ptr, self.nbytes, stream)
            lib.call("qmoe_stream_sync", stream)
        return buffer.raw

    def tolist(self, stream=0):
        data = self.tobytes(stream)
        if self.dtype == "bfloat16":
            halves = array("H")
            halves.frombytes(data)
            return [struct.unpack("<f", struct.pack("<I", h << 16))[0] for h in halves]
        out = array(_FORMATS[self.dtype])
        out.frombytes(data)
        return out.tolist()

    def copy(self, stream=0):
        out = DeviceStorage(self.size, self.dtype)
        lib.call("qmoe_memcpy_d2d", out.ptr, self.ptr, self.nbytes, stream)
        return out

    def __len__(self):
        return self.size
