"""Context (one GPU) and Tensor (device `Array2<f64>`) over the C ABI."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import RstError, check


class Context:
    """One GPU: streams, caching allocator, result ring (rst_ctx_create)."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        h = C.c_void_p()
        check(self._lib.rst_ctx_create(int(device), C.byref(h)))
        self.handle = h
        self.device = int(device)
        self._next_slot = 0

    # -- lifecycle ---------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "handle", None) is not None and self.handle.value:
            self._lib.rst_ctx_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        check(status, self.handle)

    # -- tensors -----------------------------------------------------------
    def empty(self, rows: int, cols: int) -> "Tensor":
        h = C.c_void_p()
        self._check(self._lib.rst_tensor_alloc(self.handle, int(rows), int(cols), C.byref(h)))
        return Tensor(self, h, int(rows), int(cols))

    def zeros(self, rows: int, cols: int) -> "Tensor":
        t = self.empty(rows, cols)
        t.fill(0.0)
        return t

    def tensor(self, array) -> "Tensor":
        """Uploads a 2-D array (any layout; copied to standard row-major f64 first)."""
        a = np.ascontiguousarray(array, dtype=np.float64)
        if a.ndim != 2:
            raise ValueError(f"expected a 2-D array, got shape {a.shape}")
        t = self.empty(a.shape[0], a.shape[1])
        t.upload(a)
        return t

    # -- misc --------------------------------------------------------------
    def synchronize(self) -> None:
        self._check(self._lib.rst_ctx_synchronize(self.handle))

    def check_device(self) -> None:
        self._check(self._lib.rst_ctx_check_device(self.handle))

    def launch_count(self) -> int:
        n = C.c_uint64()
        self._check(self._lib.rst_ctx_launch_count(self.handle, C.byref(n)))
        return n.value

    def memory_stats(self) -> dict:
        s = (C.c_uint64 * 6)()
        self._check(self._lib.rst_ctx_memory_stats(self.handle, s))
        keys = ("in_use", "reserved", "peak", "requests", "cache_hits", "driver_allocs")
        return dict(zip(keys, (int(v) for v in s)))

    def set_memory_limit(self, max_reserved_bytes: int) -> None:
        self._check(self._lib.rst_ctx_set_memory_limit(self.handle, int(max_reserved_bytes)))

    def empty_cache(self) -> None:
        self._check(self._lib.rst_ctx_empty_cache(self.handle))

    def stream_pointer(self) -> int:
        p = C.c_void_p()
        self._check(self._lib.rst_ctx_stream(self.handle, C.byref(p)))
        return p.value or 0

    def next_result_slot(self) -> int:
        s = self._next_slot
        self._next_slot = (s + 1) % self._lib.rst_xent_slots()
        return s

    def flush_l2(self, nbytes: int = 256 << 20) -> None:
        self._check(self._lib.rst_flush_l2(self.handle, int(nbytes)))

    def probe_fp64_peak(self, kind: int = 0, iters: int = 4096) -> float:
        v = C.c_double()
        self._check(self._lib.rst_probe_fp64_peak(self.handle, kind, iters, C.byref(v)))
        return v.value

    def probe_hbm_copy(self, nbytes: int = 1 << 30, iters: int = 5) -> float:
        v = C.c_double()
        self._check(self._lib.rst_probe_hbm_copy(self.handle, int(nbytes), iters, C.byref(v)))
        return v.value

    def profile_begin(self) -> None:
        self._check(self._lib.rst_profile_begin(self.handle))

    def profile_end(self) -> dict:
        """{kernel class: (launch groups, milliseconds)} since profile_begin."""
        buf = C.create_string_buffer(8192)
        self._check(self._lib.rst_profile_end(self.handle, buf, len(buf)))
        out = {}
        for line in buf.value.decode().splitlines():
            name, count, ms = line.split()
            out[name] = (int(count), float(ms))
        return out

    def timer(self) -> "Timer":
        return Timer(self)

    def capture(self) -> "GraphCapture":
        """`with ctx.capture() as cap: <one step>` then `cap.graph.launch()`."""
        return GraphCapture(self)


class Tensor:
    """Dense row-major f64 matrix in HBM; the stand-in for `Array2<f64>`."""

    __slots__ = ("ctx", "handle", "rows", "cols", "_base", "_owns", "t")

    def __init__(self, ctx: Context, handle, rows: int, cols: int, base: "Tensor | None" = None,
                 owns: bool = True):
        self.ctx, self.handle, self.rows, self.cols, self._base = ctx, handle, rows, cols, base
        self._owns = owns
        # transposed companion (cols, rows) that a backward pass may attach to a gradient it
        # has just produced; valid only as long as nothing writes this tensor again
        self.t: "Tensor | None" = None

    @property
    def shape(self) -> tuple[int, int]:
        return (self.rows, self.cols)

    @property
    def numel(self) -> int:
        return self.rows * self.cols

    def upload(self, array) -> "Tensor":
        a = np.ascontiguousarray(array, dtype=np.float64)
        if a.size != self.numel:
            raise ValueError(f"upload of {a.shape} into tensor {self.shape}")
        self.ctx._check(self.ctx._lib.rst_tensor_upload(self.handle, a.ctypes.data_as(C.c_void_p)))
        self.t = None
        return self

    def numpy(self) -> np.ndarray:
        out = np.empty((self.rows, self.cols), dtype=np.float64)
        self.ctx._check(self.ctx._lib.rst_tensor_download(self.handle, out.ctypes.data_as(C.c_void_p)))
        return out

    def fill(self, value: float) -> "Tensor":
        self.ctx._check(self.ctx._lib.rst_tensor_fill(self.handle, float(value)))
        self.t = None
        return self

    def checksum(self) -> int:
        """64-bit digest of the bit patterns, computed on the device (blocking)."""
        v = C.c_uint64()
        self.ctx._check(self.ctx._lib.rst_tensor_checksum(self.handle, C.byref(v)))
        return int(v.value)

    def clone(self) -> "Tensor":
        t = self.ctx.empty(self.rows, self.cols)
        self.ctx._check(self.ctx._lib.rst_tensor_copy(t.handle, self.handle))
        return t

    def slice(self, elem_offset: int, rows: int, cols: int) -> "Tensor":
        h = C.c_void_p()
        self.ctx._check(self.ctx._lib.rst_tensor_slice(self.handle, int(elem_offset), int(rows), int(cols),
                                                       C.byref(h)))
        return Tensor(self.ctx, h, int(rows), int(cols), base=self)

    def data_ptr(self) -> int:
        p = C.c_void_p()
        self.ctx._check(self.ctx._lib.rst_tensor_data(self.handle, C.byref(p)))
        return p.value or 0

    def free(self) -> None:
        h = self.handle
        if h is not None and h.value:
            self.handle = C.c_void_p()
            ctx = self.ctx
            if not self._owns or ctx.handle is None or not ctx.handle.value:
                return                      # something else, or the (destroyed) context, owns the memory
            ctx._lib.rst_tensor_free(h)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def __repr__(self) -> str:
        return f"Tensor({self.rows}x{self.cols}, f64, cuda:{self.ctx.device})"


def handle_array(tensors) -> "C.Array":
    arr = (C.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.handle.value
    return arr


class Timer:
    """CUDA events on the library's compute stream (torch events do not see it)."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        h = C.c_void_p()
        ctx._check(ctx._lib.rst_timer_create(ctx.handle, C.byref(h)))
        self.handle = h

    def start(self) -> None:
        self.ctx._check(self.ctx._lib.rst_timer_start(self.handle))

    def stop(self) -> None:
        self.ctx._check(self.ctx._lib.rst_timer_stop(self.handle))

    def elapsed_ms(self) -> float:
        v = C.c_double()
        self.ctx._check(self.ctx._lib.rst_timer_elapsed_ms(self.handle, C.byref(v)))
        return v.value

    def __del__(self):
        try:
            if self.handle.value and self.ctx.handle.value:
                self.ctx._lib.rst_timer_destroy(self.handle)
        except Exception:
            pass


class Graph:
    """A recorded step.  The library keeps every block the recorded kernels address out of
    its allocator until the graph is destroyed, so tensors made during the capture may be
    dropped freely; tensors made before it (weights, inputs) must outlive the graph."""

    def __init__(self, ctx: Context, handle):
        self.ctx, self.handle = ctx, handle

    def launch(self) -> None:
        self.ctx._check(self.ctx._lib.rst_graph_launch(self.handle))

    def destroy(self) -> None:
        if self.handle is not None and self.handle.value and self.ctx.handle.value:
            self.ctx._lib.rst_graph_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class GraphCapture:
    """Records one step into a CUDA graph.  Nothing is allocated from the driver while
    recording: run the same step once, unrecorded, directly before each capture, so that
    every allocation of the recorded run is served from the allocator's cache."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        self.graph: Graph | None = None

    def __enter__(self) -> "GraphCapture":
        self.ctx._check(self.ctx._lib.rst_graph_capture_begin(self.ctx.handle))
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        h = C.c_void_p()
        status = self.ctx._lib.rst_graph_capture_end(self.ctx.handle, C.byref(h))
        if exc_type is None:
            self.ctx._check(status)
            self.graph = Graph(self.ctx, h)
        elif status == 0 and h.value:
            self.ctx._lib.rst_graph_destroy(h)
        return False
