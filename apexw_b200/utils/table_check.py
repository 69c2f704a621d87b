"""Debug mode of the persistent kernels: table checks before every chunk.

The fused state kernels index memory only through their segment table (one record per tensor: pointers, sizes,
formats, first chunk).  With ``APEXW_B200_DEBUG_BOUNDS=1`` (or inside ``table_checks()``) every thread block validates
the record of each chunk before it indexes with it - segment number, the chunk's place in its segment and in the
tensor, null pointers, alignment, quantisation block size, formats - skips a chunk that fails, and records the first
failure in a device word.  ``ApexW.step`` and ``ApexWZeRO.step`` read that word after their launches while the mode is
on (one device synchronisation per step) and raise ``TableFaultError``.

This replaces what a memory checker would report for these kernels on machines where none can be run; it costs one
predicate per chunk when off.
"""

from __future__ import annotations

import contextlib
import os
from typing import Dict, Optional

from .. import _native

ENV = "APEXW_B200_DEBUG_BOUNDS"

FAULT_TEXT = {
    0: "ok",
    1: "segment index outside the table",
    2: "chunk before its segment's first chunk",
    3: "chunk past its segment's last chunk",
    4: "chunk past the tensor's elements",
    5: "null pointer in the record",
    6: "pointer not aligned to its element size",
    7: "quantisation block size outside 64..2048",
    8: "null scale pointer in a quantised record",
    9: "format code not known to this kernel class",
    10: "negative offset into the flat buffers",
}


class TableFaultError(RuntimeError):
    """A kernel found a segment-table record it must not index with; the chunks concerned were skipped."""

    def __init__(self, report: Dict[str, Dict[str, int]]):
        self.report = report
        parts = []
        for module, r in report.items():
            if r["code"]:
                parts.append(f"{module}: {FAULT_TEXT.get(r['code'], r['code'])} (segment {r['segment']}, chunk {r['chunk']}, "
                             f"{r['skipped']} chunk(s) skipped)")
        super().__init__("segment-table check failed - " + "; ".join(parts))


def enabled() -> bool:
    return os.environ.get(ENV, "0") not in ("", "0")


@contextlib.contextmanager
def table_checks(on: bool = True):
    """Switch the checks on (or off) for the launches made inside the block."""
    old = os.environ.get(ENV)
    os.environ[ENV] = "1" if on else "0"
    try:
        yield
    finally:
        if old is None:
            os.environ.pop(ENV, None)
        else:
            os.environ[ENV] = old


def report(clear: bool = True) -> Optional[Dict[str, Dict[str, int]]]:
    """The kernels' fault words (synchronises the current device); None without the native library or a GPU."""
    nat = _native.load()
    if nat is None or not hasattr(nat, "table_fault_report"):
        return None
    import torch
    if not torch.cuda.is_available():
        return None
    w = nat.table_fault_report(clear)
    keys = ("code", "segment", "chunk", "skipped")
    return {"state": dict(zip(keys, w[:4])), "zero": dict(zip(keys, w[4:8]))}


def check() -> None:
    """Raise ``TableFaultError`` when a kernel recorded a fault since the last call (clears the record)."""
    r = report(clear=True)
    if r is not None and any(m["code"] for m in r.values()):
        raise TableFaultError(r)


def selftest() -> int:
    """Run the device-side checker on 15 hand-made records (nothing is dereferenced).  Bit i set: case i behaved;
    0x7FFF when all did."""
    import torch
    nat = _native.load()
    if nat is None:
        raise RuntimeError("native library not available: " + str(_native.load_error()))
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    return int(nat.table_check_selftest(scratch))
