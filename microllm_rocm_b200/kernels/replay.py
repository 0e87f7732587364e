"""Record the launcher calls of one layer and issue them again for the other layers of the same structure
from native code (csrc/replay.cu), with the layer's own tensors swapped in.

`Recorder` is switched on around one layer's forward; every launcher the layer calls through `ops.lib()` is
noted as (function address, arguments as 64-bit slots, floats apart, which slots are pointers).  `Recording`
holds the packed records; `replay(swaps)` issues them with pointers replaced.  What may be swapped is decided
by the caller (parts/build.py): the tensors a layer owns, matched by address.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_uint, c_ulonglong, c_void_p
from typing import Dict, List, Optional, Sequence, Tuple

from . import build
from .build import KernelError


def _register():
    from . import ops
    ops.register_signatures("replay.cu", {
        "mlb_replay_calls": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
        "mlb_replay_probe": [c_void_p, ctypes.c_longlong, c_int, c_float, c_void_p, c_int, c_int, c_int, ctypes.c_longlong,
                             c_float, c_int, c_void_p],
    })

MAX_SLOTS = 28
MAX_FLOATS = 4


class CallRecord(ctypes.Structure):
    _fields_ = [("function", c_void_p), ("slots", c_ulonglong * MAX_SLOTS), ("floats", c_float * MAX_FLOATS),
                ("pointer_mask", c_uint), ("num_slots", c_int), ("num_floats", c_int), ("library", c_int)]


import struct

# the layout of CallRecord (native alignment): function, slots, floats, pointer_mask, num_slots, num_floats, library
_RECORD = struct.Struct(f"@P{MAX_SLOTS}Q{MAX_FLOATS}fIiii")
assert _RECORD.size == ctypes.sizeof(CallRecord), "the packed record must have the layout of the ctypes structure"

_active: Optional["Recorder"] = None


class Recorder:
    """Collects the launcher calls made while it is active (`with Recorder() as rec:`)."""

    def __init__(self):
        self.calls: List[Tuple[object, int, Tuple[int, ...], Tuple[float, ...], int]] = []
        self.unrecordable: Optional[str] = None

    def __enter__(self):
        global _active
        if _active is not None:
            raise RuntimeError("a recorder is already active")
        _active = self
        return self

    def __exit__(self, *exc):
        global _active
        _active = None

    def note(self, library, function, argtypes, args) -> None:
        slots, floats, mask = [], [], 0
        if len(args) != len(argtypes):
            self.unrecordable = f"{function.__name__}: {len(args)} arguments for {len(argtypes)} declared"
            return
        for kind, value in zip(argtypes, args):
            if kind is c_float:
                floats.append(float(value))
            elif kind is c_void_p:
                mask |= 1 << len(slots)
                slots.append(0 if value is None else int(value))
            else:
                slots.append(int(value) & 0xFFFFFFFFFFFFFFFF)
        if len(slots) > MAX_SLOTS or len(floats) > MAX_FLOATS:
            self.unrecordable = f"{function.__name__} takes more arguments than a record holds"
            return
        address = ctypes.cast(function, c_void_p).value
        self.calls.append((library, address, tuple(slots), tuple(floats), mask))


class Launcher:
    """A launcher of a loaded library: calls through, and tells the active recorder what it was called with."""
    __slots__ = ("library", "function", "argtypes", "__name__")

    def __init__(self, library, function, argtypes):
        self.library, self.function, self.argtypes = library, function, tuple(argtypes)
        self.__name__ = function.__name__

    def __call__(self, *args):
        if _active is not None:
            _active.note(self.library, self.function, self.argtypes, args)
        return self.function(*args)


_replay_lib = None


def _lib():
    global _replay_lib
    if _replay_lib is None:
        from . import ops
        L = ops.lib("replay.cu")
        L.mlb_replay_record_bytes.restype = c_int
        if L.mlb_replay_record_bytes() != ctypes.sizeof(CallRecord) or L.mlb_replay_max_slots() != MAX_SLOTS \
                or L.mlb_replay_max_floats() != MAX_FLOATS:
            raise KernelError("replay: the record layout of the library differs from the binding's")
        _replay_lib = L
    return _replay_lib


def sources():
    return [("replay.cu", {})]


_register()


class Recording:
    """The packed calls of one layer, ready to be issued again."""

    def __init__(self, recorder: Recorder):
        if recorder.unrecordable:
            raise KernelError(f"replay: {recorder.unrecordable}")
        self.libraries = []
        n = len(recorder.calls)
        self.count = n
        self.pointers = set()
        # the records are packed in one go (one struct.pack per call): field-by-field assignment through ctypes
        # costs more host time than the calls themselves
        blob = bytearray()
        for library, address, slots, floats, mask in recorder.calls:
            if library not in self.libraries:
                self.libraries.append(library)
            for j, v in enumerate(slots):
                if (mask >> j) & 1 and v:
                    self.pointers.add(v)
            blob += _RECORD.pack(address, *slots, *([0] * (MAX_SLOTS - len(slots))), *floats, *([0.0] * (MAX_FLOATS - len(floats))),
                                 mask, len(slots), len(floats), self.libraries.index(library))
        self.records = (CallRecord * max(1, n)).from_buffer_copy(bytes(blob) if n else bytes(ctypes.sizeof(CallRecord)))
        self._failed = c_int(-1)
        self._launched = c_int(0)
        self._swap_cache: Dict[Tuple[int, ...], Tuple[object, object, int]] = {}

    def swaps(self, pairs: Sequence[Tuple[int, int]]):
        """(from array, to array, count) for pointer pairs that differ; kept per target layer."""
        key = tuple(b for _, b in pairs)
        got = self._swap_cache.get(key)
        if got is None:
            used = [(a, b) for a, b in pairs if a != b and a in self.pointers]
            n = len(used)
            src = (c_ulonglong * max(1, n))(*[a for a, _ in used])
            dst = (c_ulonglong * max(1, n))(*[b for _, b in used])
            got = self._swap_cache[key] = (src, dst, n)
        return got

    def replay(self, pairs: Sequence[Tuple[int, int]]) -> int:
        """Issue the recorded calls with every pointer `a` replaced by `b` for (a, b) in pairs; returns how many
        launchers were called."""
        src, dst, n = self.swaps(pairs)
        L = _lib()
        status = L.mlb_replay_calls(ctypes.addressof(self.records), self.count, ctypes.addressof(src), ctypes.addressof(dst), n,
                                    ctypes.addressof(self._failed), ctypes.addressof(self._launched))
        build.LaunchCounter.own += self._launched.value
        if status != 0:
            where = self._failed.value
            message = None
            if 0 <= where < self.count:
                message = self.libraries[self.records[where].library].mlb_last_error()
            else:
                message = L.mlb_last_error()
            raise KernelError(message.decode("utf-8", "replace") if message else f"a replayed launcher returned {status}")
        return self._launched.value
