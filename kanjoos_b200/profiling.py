"""Device-clock spans of the layer launches, in the shape the reference's
profiler consumes (`Profiler::device_span(name, start_ns, end_ns, stream)`,
src/profiler/profiler.h:98-137): recording is switched on around a run, the
epoch is marked on the stream, and the spans are handed over after the run.

    with DeviceSpans(capacity=256) as spans:
        for _ in range(steps):
            layer.prefill(x, out=out)
    for name, start_ns, end_ns in spans.rows: ...
    spans.table()   # name -> (count, total ns), the rows of the --profiling table

Launches captured into a CUDA graph record nothing (events inside a capture
cannot be timed); profile eager launches.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib

_CB = C.CFUNCTYPE(None, C.c_char_p, C.c_uint64, C.c_uint64, C.c_int, C.c_void_p)


class DeviceSpans:
    def __init__(self, capacity: int = 1024, stream: torch.cuda.Stream | None = None):
        self.capacity, self.stream = capacity, stream
        self.rows: list[tuple[str, int, int]] = []
        self.dropped = 0

    def _s(self):
        st = self.stream or torch.cuda.current_stream()
        return C.c_void_p(st.cuda_stream)

    def __enter__(self):
        check(lib().knj_spans_enable(self.capacity))
        check(lib().knj_spans_epoch(self._s()))
        return self

    def span(self, name: str):
        """Bracket caller-side work (e.g. a whole step) with a span of its own."""
        outer = self

        class _Scope:
            def __enter__(self_inner):
                self_inner.h = lib().knj_span_begin(name.encode(), outer._s())
                return self_inner

            def __exit__(self_inner, *exc):
                check(lib().knj_span_end(self_inner.h, outer._s()))
                return False
        return _Scope()

    def __exit__(self, *exc):
        rows = self.rows

        def on_span(name, a, b, stream, user):
            rows.append((name.decode(), int(a), int(b)))
        cb = _CB(on_span)
        try:
            self.dropped = int(lib().knj_spans_dropped())
            check(lib().knj_spans_flush(C.cast(cb, C.c_void_p), None))
        finally:
            lib().knj_spans_disable()
        return False

    def table(self) -> dict:
        """Self time per name: a span contained in another is subtracted from its parent
        (the folding rule of the reference's device rows)."""
        rows = sorted(self.rows, key=lambda r: (r[1], -r[2]))
        self_ns = [b - a for _, a, b in rows]
        stack = []
        for i, (_, a, b) in enumerate(rows):
            while stack and rows[stack[-1]][2] <= a:
                stack.pop()
            if stack and b <= rows[stack[-1]][2]:
                self_ns[stack[-1]] -= b - a
            stack.append(i)
        out = {}
        for (name, _, _), ns in zip(rows, self_ns):
            c, t = out.get(name, (0, 0))
            out[name] = (c + 1, t + ns)
        return out
