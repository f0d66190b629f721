"""Python face of the device-resident graph runtime (``include/one_net.h``).

``Net`` loads a ``.one`` image onto one GPU for a fixed batch and runs it with the Conv / Gemm /
MatMul operators on the sm_100a backend.  It is the counterpart of the reference's
``net`` + ``extractor`` (host/net.h:223-235, :378-397, :613-641).  torch is used for pinned host
buffers only; all device memory belongs to the runtime.
"""
import ctypes as C

import numpy as np

from . import capi

NO_FUSE, NO_GRAPH = 0x1000, 0x2000
NET_SYMBOLS = [
    "one_net_create", "one_net_create_from_memory", "one_net_destroy", "one_net_last_error", "one_net_io_count",
    "one_net_io_info", "one_net_io_ptr", "one_net_stream", "one_net_run", "one_net_sync", "one_net_run_host",
    "one_net_fetch", "one_net_operands", "one_net_trace", "one_net_work", "one_net_describe", "one_net_submit_host", "one_net_operand_ptr", "one_net_autotune", "one_net_set_tile", "one_net_trace_ex", "one_net_write_timeline_csv", "one_net_activation_table",
    "one_net_group_create", "one_net_group_create_from_memory", "one_net_group_destroy", "one_net_group_size", "one_net_group_shard",
    "one_net_group_member", "one_net_group_partition", "one_net_group_submit_host", "one_net_group_sync", "one_net_group_set_fault_hook",
]
_bound = False


def _lib():
    global _bound
    L = capi.lib()
    if not _bound:
        L.one_net_last_error.restype = C.c_char_p
        L.one_net_create.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
        L.one_net_create_from_memory.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_size_t,
                                                 C.POINTER(C.c_void_p)]
        L.one_net_describe.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_char_p, C.c_size_t]
        L.one_net_destroy.argtypes = [C.c_void_p]
        L.one_net_destroy.restype = None
        L.one_net_io_count.argtypes = [C.c_void_p, C.c_int]
        L.one_net_io_info.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.one_net_io_ptr.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.one_net_io_ptr.restype = C.c_void_p
        L.one_net_stream.argtypes = [C.c_void_p]
        L.one_net_stream.restype = C.c_void_p
        L.one_net_run.argtypes = [C.c_void_p]
        L.one_net_sync.argtypes = [C.c_void_p]
        L.one_net_run_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.one_net_submit_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.one_net_fetch.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t]
        L.one_net_operands.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
        L.one_net_operand_ptr.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_longlong),
                                          C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.one_net_trace.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.one_net_trace_ex.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_char_p, C.c_double]
        L.one_net_autotune.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t]
        L.one_net_set_tile.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.one_net_work.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_ulonglong)]
        _bound = True
    return L


def _check(rc):
    if rc != 0:
        raise capi.OneCudaError(rc, _lib().one_net_last_error().decode())


def describe(image, batch=1, precision="tf32", fuse=True):
    """The runtime's execution plan for a ``.one`` image as a list of text lines (no GPU needed)."""
    flags = capi.PRECISIONS[precision] | (0 if fuse else NO_FUSE)
    buf = C.create_string_buffer(1 << 20)
    image = bytes(image)
    _check(_lib().one_net_describe(image, len(image), batch, flags, buf, len(buf)))
    return [ln for ln in buf.value.decode().split("\n") if ln]


class Net:
    def __init__(self, image, device=0, batch=1, precision="tf32", fuse=True, graph=True, workspace_bytes=0):
        """``image``: path of a ``.one`` file or its bytes."""
        L = _lib()
        flags = capi.PRECISIONS[precision]
        flags |= (0 if fuse else NO_FUSE) | (0 if graph else NO_GRAPH)
        self.handle = C.c_void_p()
        if isinstance(image, (bytes, bytearray)):
            self._image = bytes(image)
            _check(L.one_net_create_from_memory(self._image, len(self._image), device, batch, flags, workspace_bytes,
                                                C.byref(self.handle)))
        else:
            _check(L.one_net_create(str(image).encode(), device, batch, flags, workspace_bytes, C.byref(self.handle)))
        self.device, self.batch, self.precision = device, batch, precision
        self.tuned_split = {}   # per operator: the split-K choice the last autotune() kept
        self.inputs = [self._io(0, i) for i in range(L.one_net_io_count(self.handle, 0))]
        self.outputs = [self._io(1, i) for i in range(L.one_net_io_count(self.handle, 1))]

    def _io(self, is_out, i):
        name = C.create_string_buffer(256)
        shape = (C.c_int * 8)()
        nd = C.c_int()
        _check(_lib().one_net_io_info(self.handle, is_out, i, name, shape, C.byref(nd)))
        return name.value.decode(), tuple(shape[k] for k in range(nd.value))

    def io_ptr(self, is_output, index=0):
        return _lib().one_net_io_ptr(self.handle, int(is_output), index)

    @property
    def stream(self):
        return _lib().one_net_stream(self.handle)

    def run(self):
        """Enqueue one inference over the device-resident input."""
        _check(_lib().one_net_run(self.handle))

    def sync(self):
        _check(_lib().one_net_sync(self.handle))

    def run_host(self, host_in, host_out):
        """H2D copy of input 0, run, D2H copy of output 0, wait.  Arguments are contiguous fp32
        numpy arrays or torch CPU tensors (pinned for asynchronous copies)."""
        _check(_lib().one_net_run_host(self.handle, _ptr(host_in), _ptr(host_out)))

    def submit_host(self, host_in, host_out):
        """Pipelined run_host: returns at once; the H2D copy of this batch overlaps the previous batch's
        inference.  Call sync() before reading ``host_out`` or reusing ``host_in``."""
        _check(_lib().one_net_submit_host(self.handle, _ptr(host_in), _ptr(host_out)))

    def __call__(self, x):
        x = np.ascontiguousarray(x, np.float32)
        assert x.shape == self.inputs[0][1], (x.shape, self.inputs[0][1])
        y = np.empty(self.outputs[0][1], np.float32)
        self.run_host(x, y)
        return y

    def operands(self):
        buf = C.create_string_buffer(1 << 20)
        _check(_lib().one_net_operands(self.handle, buf, len(buf)))
        return [n for n in buf.value.decode().split("\n") if n]

    def fetch(self, operand, shape):
        out = np.empty(shape, np.float32)
        _check(_lib().one_net_fetch(self.handle, operand.encode(), out.ctypes.data, out.size))
        return out

    def operand_ptr(self, operand):
        """(device pointer, element count, dtype, layout) of a materialised operand."""
        dev, n, dt, lay = C.c_void_p(), C.c_longlong(), C.c_int(), C.c_int()
        _check(_lib().one_net_operand_ptr(self.handle, operand.encode(), C.byref(dev), C.byref(n), C.byref(dt), C.byref(lay)))
        return dev.value, n.value, dt.value, lay.value

    def trace(self, csv_path, runs=3, model_name="model", hw_gops=0.0):
        """Per-operator CUDA-event timing written as the reference's tracing CSV (read by its
        tools/perf_profiling/gen_timeline_json.py); ``hw_gops`` <= 0 takes the nominal tensor peak."""
        _check(_lib().one_net_trace_ex(self.handle, str(csv_path).encode(), runs, model_name.encode(), float(hw_gops)))

    def autotune(self, runs=5):
        """Time every Conv / Gemm / MatMul at each tile width and keep the fastest (one inference must
        have run).  Returns {op name: (out_width, heuristic_us, best_tile_n, best_us)}; best_tile_n 0
        means the library's own choice stayed."""
        buf = C.create_string_buffer(1 << 20)
        _check(_lib().one_net_autotune(self.handle, runs, buf, len(buf)))
        out = {}
        for line in buf.value.decode().splitlines()[1:]:
            name, _type, width, h_us, bn, b_us, split = line.rsplit(",", 6)
            out[name] = (int(width), float(h_us), int(bn), float(b_us))
            self.tuned_split[name] = int(split)
        return out

    def set_tile(self, op_name, tile_n):
        """Force one operator's tile width (0 = heuristic): replays a saved tuning."""
        _check(_lib().one_net_set_tile(self.handle, op_name.encode(), tile_n))

    def work(self):
        f, b, n = C.c_double(), C.c_double(), C.c_ulonglong()
        _check(_lib().one_net_work(self.handle, C.byref(f), C.byref(b), C.byref(n)))
        return f.value, b.value, n.value

    def close(self):
        if self.handle:
            _lib().one_net_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ptr(a):
    if isinstance(a, np.ndarray):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    return a.data_ptr()   # torch CPU tensor


def write_timeline_csv(csv_path, rows, gpu="", gpu_hw_info="", hw_gops=1.0, model_name="model"):
    """Write rows ``(op_name, op_type, st_us, ed_us, mflop[, bytes[, detail]])`` in the reference's
    tracing CSV schema (host only; no GPU is touched)."""
    L = _lib()
    n = len(rows)
    strs = lambda k: (C.c_char_p * n)(*[str(r[k]).encode() if len(r) > k else b"" for r in rows])
    dbls = lambda k: (C.c_double * n)(*[float(r[k]) if len(r) > k else 0.0 for r in rows])
    L.one_net_write_timeline_csv.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), C.POINTER(C.c_double),
                                             C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_char_p),
                                             C.c_char_p, C.c_char_p, C.c_double, C.c_char_p]
    _check(L.one_net_write_timeline_csv(str(csv_path).encode(), n, strs(0), strs(1), dbls(2), dbls(3), dbls(4), dbls(5), strs(6),
                                        gpu.encode(), gpu_hw_info.encode(), float(hw_gops), model_name.encode()))


FAULT_HOOK = C.CFUNCTYPE(C.c_int, C.c_int)


class NetGroup:
    """One model on several GPUs of the box from one calling thread (``one_net_group``): the batch is cut
    into contiguous shards, one per device, each run by its own replica on its own host thread; nothing
    is exchanged between devices."""

    def __init__(self, image, devices, batch, precision="tf32", fuse=True, graph=True, workspace_bytes=0):
        L = _lib()
        flags = capi.PRECISIONS[precision]
        flags |= (0 if fuse else NO_FUSE) | (0 if graph else NO_GRAPH)
        self.handle = C.c_void_p()
        devs = (C.c_int * len(devices))(*devices)
        L.one_net_group_create_from_memory.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int, C.c_size_t,
                                                       C.POINTER(C.c_void_p)]
        L.one_net_group_create.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
        L.one_net_group_destroy.argtypes = [C.c_void_p]
        L.one_net_group_destroy.restype = None
        L.one_net_group_size.argtypes = [C.c_void_p]
        L.one_net_group_shard.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.one_net_group_member.argtypes = [C.c_void_p, C.c_int]
        L.one_net_group_member.restype = C.c_void_p
        L.one_net_group_submit_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.one_net_group_sync.argtypes = [C.c_void_p]
        L.one_net_group_set_fault_hook.argtypes = [C.c_void_p, C.c_void_p]
        if isinstance(image, (bytes, bytearray)):
            self._image = bytes(image)
            _check(L.one_net_group_create_from_memory(self._image, len(self._image), devs, len(devices), batch, flags, workspace_bytes,
                                                      C.byref(self.handle)))
        else:
            _check(L.one_net_group_create(str(image).encode(), devs, len(devices), batch, flags, workspace_bytes, C.byref(self.handle)))
        self.batch = batch
        self._hook = None

    @property
    def shards(self):
        """[(device, first image, image count)] in shard order."""
        L, out = _lib(), []
        for i in range(L.one_net_group_size(self.handle)):
            d, f, c = C.c_int(), C.c_int(), C.c_int()
            _check(L.one_net_group_shard(self.handle, i, C.byref(d), C.byref(f), C.byref(c)))
            out.append((d.value, f.value, c.value))
        return out

    def submit_host(self, host_in, host_out):
        _check(_lib().one_net_group_submit_host(self.handle, _ptr(host_in), _ptr(host_out)))

    def sync(self):
        _check(_lib().one_net_group_sync(self.handle))

    def set_fault_hook(self, fn):
        """``fn(device) -> int`` runs on the device's host thread before each shard; non-zero = that shard fails."""
        self._hook = FAULT_HOOK(fn) if fn else None
        _check(_lib().one_net_group_set_fault_hook(self.handle, C.cast(self._hook, C.c_void_p) if self._hook else None))

    def close(self):
        if self.handle:
            _lib().one_net_group_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def activation_table(kind):
    """The runtime's SiLU (``"silu"``) or Gelu (``"gelu"``) look-up table, 8192 floats."""
    out = np.empty(8192, np.float32)
    _check(_lib().one_net_activation_table({"silu": 0, "gelu": 1}[kind], out.ctypes.data_as(C.c_void_p)))
    return out
