"""The timeline of the kernel launches of a step, from records the kernels write themselves.

With ABACUS_TRACE=1 in the environment the kernel libraries are built with the records of
csrc/common.cuh compiled in: the first CTA of every launch notes when it reached its dependency wait
and when it was let go. `read()` collects them from every loaded library; `timeline()` orders them and
gives, for each launch, how long after the previous launch's release its own came: the time the
launch before it took, as the step really ran (no profiler serialising the launches).

    import os; os.environ["ABACUS_TRACE"] = "1"      # before the package is imported
    ... run some steps ...
    trace.read()                                      # drop what came before
    ... run the step to look at ...
    for row in trace.timeline(trace.read()): print(row)
"""
import ctypes

from . import build


class Record(ctypes.Structure):
    _fields_ = [("reached", ctypes.c_ulonglong), ("released", ctypes.c_ulonglong), ("file", ctypes.c_int),
                ("grid", ctypes.c_int), ("block", ctypes.c_int), ("pad", ctypes.c_int)]


def read(max_records=16384, lives=False):
    """All records of launches made since the last call, over every loaded kernel library, ordered by
    release time. lives=True: instead the records some kernels keep of every CTA's life (begin, end,
    what it worked on: `grid`, how much: `block`, and on which SM)."""
    if not build.TRACE:
        raise RuntimeError("the kernel libraries are built without records: set ABACUS_TRACE=1 before importing")
    out = []
    for module, lib in list(build._loaded.items()):
        if not hasattr(lib, "abk_trace_read"):  # a library without device code keeps no records
            continue
        buf = (Record * max_records)()
        n = lib.abk_trace_read(buf, ctypes.c_int(max_records))
        if n < 0:
            raise RuntimeError(f"reading the records of {module} failed")
        out += [dict(module=module, reached=r.reached, released=r.released, grid=r.grid, block=r.block, sm=r.pad - 1)
                for r in buf[:n] if (r.pad != 0) == lives]
    return sorted(out, key=lambda r: r["released"])


def timeline(records):
    """For each launch: its library and sizes, how long its first CTA waited, and how long after the
    launch before it it was released (microseconds)."""
    rows, last = [], None
    for r in records:
        rows.append(dict(module=r["module"], grid=r["grid"], block=r["block"],
                         waited_us=(r["released"] - r["reached"]) / 1e3,
                         after_previous_us=None if last is None else (r["released"] - last) / 1e3))
        last = r["released"]
    return rows
