"""The host surface of the matrix-multiply path, named after the reference's:

    gpu = Gpu(0)                       Gpu::new(0)              crates/gpurs/src/host/context.rs:69
    stream = gpu.stream()              gpu.stream()             context.rs:125
    a = gpu.upload(host_array)         gpu.upload(&host)        context.rs:132
    c = gpu.zeros(np.float32, n)       gpu.zeros::<f32>(n)      context.rs:151
    matmul(stream, a, b, c, [m, n, k]) the launcher             crates/macros/src/launcher.rs:110-223
    c.download()                       output.download()        crates/gpurs/src/host/memory/buffer.rs:251-271

Everything here is a thin object layer over the C ABI (include/gpurs_b200.h) through ctypes: no
computation happens in Python and there is no fallback when the native library is absent.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _ffi

# Element types of the operands.  16-bit and 8-bit float formats have no numpy dtype: buffers of those
# carry their bit patterns in uint16 / uint8 arrays and name the format explicitly.
F16, F32, BF16, I8, I32, E4M3 = _ffi.F16, _ffi.F32, _ffi.BF16, _ffi.I8, _ffi.I32, _ffi.E4M3
ELEMENT_BYTES = {F16: 2, F32: 4, BF16: 2, I8: 1, I32: 4, E4M3: 1}
_STORAGE = {F16: np.uint16, BF16: np.uint16, F32: np.float32, I8: np.int8, I32: np.int32, E4M3: np.uint8}
_FROM_NUMPY = {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.int8): I8, np.dtype(np.int32): I32}


class GpursError(RuntimeError):
    """A failed call: `code` is the CUresult or the GPURS_E_* value (the reference's `gpurs::Error`,
    crates/gpurs/src/error.rs:13-71, and `driver::Error`, crates/driver/src/error.rs:8-16)."""

    def __init__(self, code: int):
        operation, name, description = C.c_char_p(), C.c_char_p(), C.c_char_p()
        _ffi.load().gpurs_last_error(C.byref(operation), C.byref(name), C.byref(description))
        self.code = code
        self.operation = (operation.value or b"").decode()
        self.name = (name.value or b"").decode()
        self.description = (description.value or b"").decode()
        super().__init__(f"`{self.operation}` failed: {self.name} ({self.description}, code {code})")


def _check(code: int) -> None:
    if code != _ffi.OK:
        raise GpursError(code)


@dataclass
class LaunchConfig:
    """`LaunchConfig` (crates/gpurs/src/host/stream.rs:28-52) with the cluster dimension added."""

    grid: tuple = (1, 1, 1)
    block: tuple = (1, 1, 1)
    shared_bytes: int = 0
    cluster: tuple = (1, 1, 1)

    def _struct(self) -> _ffi.LaunchConfigStruct:
        s = _ffi.LaunchConfigStruct()
        for i in range(3):
            s.grid[i] = self.grid[i] if i < len(self.grid) else 1
            s.block[i] = self.block[i] if i < len(self.block) else 1
            s.cluster[i] = self.cluster[i] if i < len(self.cluster) else 1
        s.shared_bytes = self.shared_bytes
        return s


class Event:
    def __init__(self, gpu: "Gpu", handle):
        self._gpu, self._handle = gpu, handle

    def synchronize(self) -> None:
        _check(self._gpu._lib.gpurs_event_synchronize(self._handle))

    def elapsed_ms(self, later: "Event") -> float:
        """Milliseconds from this event to `later` (`Event::elapsed`)."""
        ms = C.c_float()
        _check(self._gpu._lib.gpurs_event_elapsed_ms(self._handle, later._handle, C.byref(ms)))
        return ms.value

    def __del__(self):
        if getattr(self, "_handle", None) and self._gpu._handle:
            self._gpu._lib.gpurs_event_free(self._handle)
            self._handle = None


class Stream:
    """`Stream` (crates/gpurs/src/host/stream.rs): launches are asynchronous, `synchronize` waits."""

    def __init__(self, gpu: "Gpu", handle):
        self.gpu, self._handle = gpu, handle

    def synchronize(self) -> None:
        _check(self.gpu._lib.gpurs_stream_synchronize(self._handle))

    def record_timed(self) -> Event:
        handle = C.c_void_p()
        _check(self.gpu._lib.gpurs_event_record_timed(self._handle, C.byref(handle)))
        return Event(self.gpu, handle)

    def capture(self, record) -> "Graph":
        """Run `record(stream)` with this stream recording instead of executing, and return the recording
        (`Stream::capture`, crates/gpurs/src/host/graph/capture.rs:112-149).  Buffers the recorded operations use must
        stay alive and in place while the graph exists."""
        _check(self.gpu._lib.gpurs_stream_capture_begin(self._handle))
        handle = C.c_void_p()
        try:
            record(self)
        except BaseException:
            # the capture must end whatever happened; what was recorded so far is dropped
            if self.gpu._lib.gpurs_stream_capture_end(self._handle, C.byref(handle)) == _ffi.OK:
                self.gpu._lib.gpurs_graph_free(handle)
            raise
        _check(self.gpu._lib.gpurs_stream_capture_end(self._handle, C.byref(handle)))
        return Graph(self.gpu, handle)

    @property
    def raw(self) -> int:
        return self.gpu._lib.gpurs_stream_raw(self._handle) or 0

    def copy_to_device(self, destination: "DeviceBuffer", host_pointer: int, nbytes: int) -> None:
        _check(self.gpu._lib.gpurs_copy_to_device(self._handle, destination.pointer, host_pointer, nbytes))

    def copy_to_host(self, host_pointer: int, source: "DeviceBuffer", nbytes: int) -> None:
        _check(self.gpu._lib.gpurs_copy_to_host(self._handle, host_pointer, source.pointer, nbytes))

    def __del__(self):
        if getattr(self, "_handle", None) and self.gpu._handle:
            self.gpu._lib.gpurs_stream_free(self._handle)
            self._handle = None


class GraphExec:
    """An instantiated recording (`GraphExec`, crates/gpurs/src/host/graph/exec.rs:15-72)."""

    def __init__(self, graph: "Graph"):
        self._graph = graph

    def launch(self, stream: "Stream") -> None:
        """Enqueue one replay of the whole recording on `stream`; does not wait."""
        _check(self._graph.gpu._lib.gpurs_graph_launch(self._graph._handle, stream._handle))


class Graph:
    """What `Stream.capture` returns (`Graph`, crates/gpurs/src/host/graph/capture.rs:99-110).  The library instantiates
    at the end of the capture, so `instantiate` only hands out the launcher."""

    def __init__(self, gpu: "Gpu", handle):
        self.gpu, self._handle = gpu, handle

    def instantiate(self) -> GraphExec:
        return GraphExec(self)

    def __del__(self):
        if getattr(self, "_handle", None) and self.gpu._handle:
            self.gpu._lib.gpurs_graph_free(self._handle)
            self._handle = None


class DeviceBuffer:
    """A typed device allocation or a view of one: the `DeviceSlice` / `DeviceSliceMut` of the
    reference (crates/gpurs/src/host/memory/buffer.rs:23-83).  `len` counts elements."""

    def __init__(self, gpu: "Gpu", pointer: int, length: int, element: int, owner: "DeviceBuffer | None" = None, owned: bool = True):
        self.gpu, self.pointer, self.len, self.element = gpu, pointer, length, element
        self._owner, self._owned = owner, owned and owner is None

    @property
    def nbytes(self) -> int:
        return self.len * ELEMENT_BYTES[self.element]

    def slice(self, start: int, stop: int) -> "DeviceBuffer":
        """Elements [start, stop) of this buffer, sharing its storage."""
        if not (0 <= start <= stop <= self.len):
            raise ValueError("slice out of range")
        return DeviceBuffer(self.gpu, self.pointer + start * ELEMENT_BYTES[self.element], stop - start, self.element, owner=self._owner or self)

    def download(self) -> np.ndarray:
        """Copy back to the host and wait (`DeviceSlice::download`).  16-bit and 8-bit float formats come
        back as their bit patterns."""
        out = np.empty(self.len, dtype=_STORAGE[self.element])
        _check(self.gpu._lib.gpurs_download(self.gpu._handle, self.pointer, out.ctypes.data, out.nbytes))
        return out

    def __del__(self):
        if getattr(self, "_owned", False) and self.pointer and self.gpu._handle:
            self.gpu._lib.gpurs_free(self.gpu._handle, self.pointer)
            self.pointer = 0


class Kernel:
    """`raw::Kernel` (crates/gpurs/src/raw/module.rs:86-207)."""

    def __init__(self, module: "Module", handle, name: str):
        self.module, self._handle, self.name = module, handle, name

    def reserve_shared(self, nbytes: int) -> None:
        _check(self.module.gpu._lib.gpurs_kernel_reserve_shared(self._handle, nbytes))

    @property
    def registers(self) -> int:
        value = C.c_int()
        _check(self.module.gpu._lib.gpurs_kernel_registers(self._handle, C.byref(value)))
        return value.value

    def launch(self, stream: Stream, config: LaunchConfig, params: list) -> None:
        """`params` are ctypes objects; their addresses form the driver's parameter array."""
        array = (C.c_void_p * len(params))(*[C.cast(C.pointer(p), C.c_void_p) for p in params])
        struct = config._struct()
        _check(self.module.gpu._lib.gpurs_kernel_launch(self._handle, stream._handle, C.byref(struct), array))


class Module:
    """`raw::Module` (crates/gpurs/src/raw/module.rs:36-92)."""

    def __init__(self, gpu: "Gpu", handle, image: bytes):
        self.gpu, self._handle, self._image = gpu, handle, image

    def kernel(self, name: str) -> Kernel:
        handle = C.c_void_p()
        _check(self.gpu._lib.gpurs_module_kernel(self._handle, name.encode(), C.byref(handle)))
        return Kernel(self, handle, name)

    def __del__(self):
        if getattr(self, "_handle", None) and self.gpu._handle:
            self.gpu._lib.gpurs_module_free(self._handle)
            self._handle = None


class Gpu:
    """`Gpu` (crates/gpurs/src/host/context.rs:26-168): one device's primary context."""

    def __init__(self, ordinal: int = 0):
        self._lib = _ffi.load()
        self._handle = C.c_void_p()
        _check(self._lib.gpurs_gpu_new(ordinal, C.byref(self._handle)))
        major, minor, sms, total = C.c_int(), C.c_int(), C.c_int(), C.c_size_t()
        _check(self._lib.gpurs_gpu_properties(self._handle, C.byref(major), C.byref(minor), C.byref(sms), C.byref(total)))
        self.ordinal = ordinal
        self.compute_capability = (major.value, minor.value)
        self.multiprocessors = sms.value
        self.total_bytes = total.value

    def stream(self) -> Stream:
        handle = C.c_void_p()
        _check(self._lib.gpurs_stream_new(self._handle, C.byref(handle)))
        return Stream(self, handle)

    def borrow_stream(self, raw: int) -> Stream:
        """Wrap a CUstream made elsewhere (for example `torch.cuda.current_stream().cuda_stream`)."""
        handle = C.c_void_p()
        _check(self._lib.gpurs_stream_borrow(self._handle, C.c_void_p(raw), C.byref(handle)))
        return Stream(self, handle)

    def upload(self, host: np.ndarray, element: int | None = None) -> DeviceBuffer:
        """Allocate, copy `host` and wait for the copy.  `element` names the format when the array holds
        bit patterns (uint16 for F16 / BF16, uint8 for E4M3)."""
        host = np.ascontiguousarray(host)
        if element is None:
            element = _FROM_NUMPY.get(host.dtype)
            if element is None:
                raise TypeError(f"name the element format of a {host.dtype} array")
        if host.dtype.itemsize != ELEMENT_BYTES[element]:
            raise TypeError("array item size does not match the element format")
        pointer = C.c_uint64()
        _check(self._lib.gpurs_upload(self._handle, host.ctypes.data, host.nbytes, C.byref(pointer)))
        return DeviceBuffer(self, pointer.value, host.size, element)

    def zeros(self, element: int, length: int) -> DeviceBuffer:
        pointer = C.c_uint64()
        _check(self._lib.gpurs_zeros(self._handle, length * ELEMENT_BYTES[element], C.byref(pointer)))
        return DeviceBuffer(self, pointer.value, length, element)

    def allocate(self, element: int, length: int) -> DeviceBuffer:
        """Uninitialised storage (`Gpu::allocate`, crates/gpurs/src/raw/allocation.rs:54-74)."""
        pointer = C.c_uint64()
        _check(self._lib.gpurs_alloc(self._handle, length * ELEMENT_BYTES[element], C.byref(pointer)))
        return DeviceBuffer(self, pointer.value, length, element)

    def import_allocation(self, pointer: int, length: int, element: int) -> DeviceBuffer:
        """Borrow device memory owned by someone else (`Gpu::import_allocation`)."""
        return DeviceBuffer(self, pointer, length, element, owned=False)

    def load_module(self, image: bytes) -> Module:
        handle = C.c_void_p()
        _check(self._lib.gpurs_module_load(self._handle, image, len(image), C.byref(handle)))
        return Module(self, handle, image)

    def kernel_image(self) -> bytes:
        size = C.c_size_t()
        pointer = self._lib.gpurs_kernel_image(C.byref(size))
        return C.string_at(pointer, size.value)

    def status(self) -> list[int]:
        words = (C.c_uint32 * 4)()
        _check(self._lib.gpurs_status_read(self._handle, words))
        return list(words)

    @property
    def launches(self) -> int:
        return self._lib.gpurs_launch_count(self._handle)

    def close(self) -> None:
        if self._handle:
            self._lib.gpurs_gpu_free(self._handle)
            self._handle = None

    def __del__(self):
        # Buffers and streams may be finalised after the gpu: they check `_handle` before freeing.
        pass


@dataclass
class MatmulOptions:
    """Optional arguments of `matmul`: row pitches in elements (0 = contiguous), tile algorithm, CTA
    limit, and the two fp32 scale arrays of a block-scaled E4M3 product."""

    lda: int = 0
    ldb: int = 0
    ldc: int = 0
    algorithm: int = _ffi.ALGO_AUTO
    max_ctas: int = 0
    precision: int = _ffi.PRECISION_DEFAULT
    raster_rows: int = 0
    l2_policy: int = 0
    b_row_major: bool = False              # B given as k x n (n contiguous) instead of n x k
    scale_a: DeviceBuffer | None = None
    scale_b: DeviceBuffer | None = None
    bias: DeviceBuffer | None = None       # fp32 [n], added to every row of C
    row_scale: DeviceBuffer | None = None      # fp32 [m]: C = acc * alpha * row_scale[row] * column_scale[column] + bias[column]
    column_scale: DeviceBuffer | None = None   # fp32 [n]
    alpha: float = 0.0                         # 0 = 1
    batches: int = 0                           # > 1: a batch of products of one shape in one launch
    stride_a: int = 0                          # elements between successive matrices; 0 = packed
    stride_b: int = 0
    stride_c: int = 0
    row_absmax: DeviceBuffer | None = None     # fp32 [m], zeroed by the caller: max |C[row, :]| is folded in
    scale_kind: int = _ffi.SCALES_FP32_BLOCKS  # SCALES_MX: scale_a / scale_b are tiled UE8M0 bytes from quantize_mx_e4m3
    metadata: DeviceBuffer | None = None   # 2:4-sparse A: `a` holds the kept values, see compress_24
    row_bias: DeviceBuffer | None = None       # fp32 [m], added to every element of its row (after the bias)
    residual: DeviceBuffer | None = None       # m x n matrix of C's element type, added as beta * residual (may be C itself)
    ldr: int = 0                               # its row pitch in elements; 0 = n
    beta: float = 0.0                          # 0 = 1
    row_sum: DeviceBuffer | None = None        # fp32 [m], zeroed by the caller: the sum of each row of the result is added in
    accumulate: bool = False                   # fp32 output: add the product to what C holds (atomic adds)
    launch: LaunchConfig | None = None         # explicit geometry (`stream.launch(LaunchConfig)` in the reference)
    extra: dict = field(default_factory=dict)


def matmul(stream: Stream, a: DeviceBuffer, b: DeviceBuffer, c: DeviceBuffer, shape, options: MatmulOptions | None = None) -> None:
    """C[m, n] = sum_k A[m, k] * B[n, k], enqueued on `stream`; shape = [m, n, k].

    `a` is the m x k left operand, `b` the n x k "right_transposed" operand of the reference's examples
    (examples/blackwell/examples/blackwell_matrix.rs:32-36), `c` the m x n row-major output.  Like a
    launcher generated by the reference's `#[gpu]` macro it validates before it submits and does not
    wait for the kernel."""
    options = options or MatmulOptions()
    if a.gpu is not stream.gpu or b.gpu is not stream.gpu or c.gpu is not stream.gpu:
        raise GpursErrorLocal(_ffi.E_CONTEXT_MISMATCH, "buffers and stream belong to different Gpu handles")
    if a.element != b.element:
        raise GpursErrorLocal(_ffi.E_INVALID_ARGUMENT, "A and B must have the same element format")
    m, n, k = (int(x) for x in shape)
    desc = _ffi.MatmulDesc()
    desc.a_type, desc.c_type = a.element, c.element
    desc.m, desc.n, desc.k = m, n, k
    desc.lda, desc.ldb, desc.ldc = options.lda, options.ldb, options.ldc
    desc.a_len, desc.b_len, desc.c_len = a.len, b.len, c.len
    desc.algorithm, desc.max_ctas = options.algorithm, options.max_ctas
    desc.precision, desc.raster_rows = options.precision, options.raster_rows
    desc.scale_a = options.scale_a.pointer if options.scale_a else 0
    desc.scale_b = options.scale_b.pointer if options.scale_b else 0
    desc.metadata = options.metadata.pointer if options.metadata else 0
    desc.l2_policy = options.l2_policy
    desc.b_row_major = 1 if options.b_row_major else 0
    desc.bias = options.bias.pointer if options.bias else 0
    desc.row_scale = options.row_scale.pointer if options.row_scale else 0
    desc.column_scale = options.column_scale.pointer if options.column_scale else 0
    desc.alpha = options.alpha
    desc.batches = options.batches
    desc.stride_a, desc.stride_b, desc.stride_c = options.stride_a, options.stride_b, options.stride_c
    desc.row_absmax = options.row_absmax.pointer if options.row_absmax else 0
    desc.scale_kind = options.scale_kind
    desc.row_bias = options.row_bias.pointer if options.row_bias else 0
    desc.residual = options.residual.pointer if options.residual else 0
    desc.ldr, desc.beta = options.ldr, options.beta
    desc.row_sum = options.row_sum.pointer if options.row_sum else 0
    desc.accumulate = 1 if options.accumulate else 0
    launch = options.launch._struct() if options.launch else None     # kept alive until the call returns
    if launch is not None:
        desc.launch = C.pointer(launch)
    _check(stream.gpu._lib.gpurs_matmul(stream._handle, C.byref(desc), a.pointer, b.pointer, c.pointer))


def matmul_host(stream: Stream, host_a: int, host_b: int, host_c: int, a: DeviceBuffer, b: DeviceBuffer, c: DeviceBuffer, shape,
                options: MatmulOptions | None = None) -> None:
    """The product with operands and result in host memory (addresses `host_a`, `host_b`, `host_c`, page-locked for
    the copies to overlap), staged through the device buffers a, b, c: the upload / upload / launch / download of the
    reference's example (examples/blackwell/examples/blackwell_matrix.rs:58-83) as one call that overlaps the copy in,
    the product and the copy out by blocks of rows.  Does not wait: synchronise `stream` before reading `host_c`."""
    options = options or MatmulOptions()
    m, n, k = (int(x) for x in shape)
    desc = _ffi.MatmulDesc()
    desc.a_type, desc.c_type = a.element, c.element
    desc.m, desc.n, desc.k = m, n, k
    desc.lda, desc.ldb, desc.ldc = options.lda, options.ldb, options.ldc
    desc.algorithm, desc.max_ctas = options.algorithm, options.max_ctas
    desc.precision, desc.raster_rows = options.precision, options.raster_rows
    desc.scale_a = options.scale_a.pointer if options.scale_a else 0
    desc.scale_b = options.scale_b.pointer if options.scale_b else 0
    desc.l2_policy = options.l2_policy
    desc.b_row_major = 1 if options.b_row_major else 0
    desc.bias = options.bias.pointer if options.bias else 0
    desc.row_scale = options.row_scale.pointer if options.row_scale else 0
    desc.column_scale = options.column_scale.pointer if options.column_scale else 0
    desc.alpha = options.alpha
    desc.row_absmax = options.row_absmax.pointer if options.row_absmax else 0
    desc.row_bias = options.row_bias.pointer if options.row_bias else 0
    desc.residual = options.residual.pointer if options.residual else 0
    desc.ldr, desc.beta = options.ldr, options.beta
    desc.row_sum = options.row_sum.pointer if options.row_sum else 0
    _check(stream.gpu._lib.gpurs_matmul_host(stream._handle, C.byref(desc), host_a, host_b, host_c, a.pointer, b.pointer, c.pointer))


class GatheredMatrix:
    """A total_rows x n matrix of which every GPU of one box keeps a copy.  Each process allocates its own copy and maps
    the others' through CUDA IPC; `exchange(handle: bytes) -> list[bytes]` hands this rank's 64-byte handle to the other
    ranks and returns all ranks' handles in rank order (an all-gather of objects of any process group will do).

    No counterpart in the reference, which drives one GPU."""

    def __init__(self, gpu: "Gpu", element: int, total_rows: int, n: int, rank: int, world: int, exchange):
        self.gpu, self.element, self.total_rows, self.n, self.rank, self.world = gpu, element, total_rows, n, rank, world
        self.local = gpu.zeros(element, total_rows * n)
        handle = (C.c_uint8 * 64)()
        _check(gpu._lib.gpurs_ipc_export(gpu._handle, self.local.pointer, handle))
        handles = exchange(bytes(handle))
        if len(handles) != world:
            raise ValueError("exchange must return one handle per rank")
        self.pointers = []
        for peer, raw in enumerate(handles):
            if peer == rank:
                self.pointers.append(self.local.pointer)
                continue
            pointer = C.c_uint64()
            _check(gpu._lib.gpurs_ipc_open(gpu._handle, (C.c_uint8 * 64).from_buffer_copy(raw), C.byref(pointer)))
            self.pointers.append(pointer.value)

    def close(self) -> None:
        """Unmap the peers' copies.  Call on every rank, after the last product into the matrix has completed everywhere."""
        for peer, pointer in enumerate(self.pointers):
            if peer != self.rank and pointer and self.gpu._handle:
                self.gpu._lib.gpurs_ipc_close(self.gpu._handle, pointer)
        self.pointers = []


def comm_unique_id() -> bytes:
    """A fresh 128-byte communicator id (made on one rank, handed to all ranks by any means the host has)."""
    raw = (C.c_uint8 * _ffi.COMM_ID_BYTES)()
    _check(_ffi.load().gpurs_comm_unique_id(raw))
    return bytes(raw)


class Communicator:
    """One rank's end of an NCCL communicator over the GPUs of the box, for the all-gather of C that may follow an
    M-sharded product.  `exchange(id: bytes | None) -> bytes` takes rank 0's id and returns it on every rank (a broadcast
    of any process group will do).  No counterpart in the reference, which drives one GPU."""

    def __init__(self, gpu: "Gpu", rank: int, world: int, exchange):
        self.gpu, self.rank, self.world = gpu, rank, world
        unique = exchange(comm_unique_id() if rank == 0 else None)
        if not isinstance(unique, (bytes, bytearray)) or len(unique) != _ffi.COMM_ID_BYTES:
            raise ValueError("exchange must return the 128-byte id of rank 0 on every rank")
        self._handle = C.c_void_p()
        _check(gpu._lib.gpurs_comm_init(gpu._handle, (C.c_uint8 * _ffi.COMM_ID_BYTES).from_buffer_copy(bytes(unique)), world, rank, C.byref(self._handle)))

    def allgather(self, stream: Stream, full: DeviceBuffer, block_bytes: int) -> None:
        """In place on `full` (world * block_bytes bytes, this rank's block already at position `rank`); does not wait."""
        if full.nbytes < self.world * block_bytes:
            raise GpursErrorLocal(_ffi.E_LENGTH_MISMATCH, "the gathered buffer is smaller than world * block_bytes")
        _check(self.gpu._lib.gpurs_comm_allgather(self._handle, stream._handle, full.pointer, block_bytes))

    def close(self) -> None:
        if self._handle and self.gpu._handle:
            self.gpu._lib.gpurs_comm_free(self._handle)
        self._handle = None


def matmul_allgather(stream: Stream, a: DeviceBuffer, b: DeviceBuffer, gathered: GatheredMatrix, shape, row_offset: int,
                     options: MatmulOptions | None = None) -> None:
    """This rank's block of rows of the gathered matrix, C[row_offset : row_offset + m, :] = A[m, k] * B[n, k]^T, computed
    and stored into EVERY rank's copy by one kernel (the all-gather rides on the GEMM's epilogue as remote stores over
    NVLink).  The matrix is complete everywhere once every rank has synchronised its stream and the ranks have met at
    a barrier.  shape = [m, n, k] of the local product."""
    options = options or MatmulOptions()
    m, n, k = (int(x) for x in shape)
    if n != gathered.n:
        raise GpursErrorLocal(_ffi.E_INVALID_ARGUMENT, "n differs from the gathered matrix")
    desc = _ffi.MatmulDesc()
    desc.a_type, desc.c_type = a.element, gathered.element
    desc.m, desc.n, desc.k = m, n, k
    desc.lda, desc.ldb = options.lda, options.ldb
    desc.a_len, desc.b_len = a.len, b.len
    desc.algorithm, desc.max_ctas, desc.raster_rows = options.algorithm, options.max_ctas, options.raster_rows
    desc.b_row_major = 1 if options.b_row_major else 0
    desc.bias = options.bias.pointer if options.bias else 0
    desc.row_scale = options.row_scale.pointer if options.row_scale else 0
    desc.column_scale = options.column_scale.pointer if options.column_scale else 0
    desc.alpha = options.alpha
    desc.metadata = options.metadata.pointer if options.metadata else 0     # 2:4-sparse A (bf16 -> bf16)
    gather = _ffi.GatherDesc()
    gather.world, gather.rank, gather.row_offset, gather.total_rows, gather.ld_full = gathered.world, gathered.rank, row_offset, gathered.total_rows, 0
    for peer, pointer in enumerate(gathered.pointers):
        gather.full[peer] = pointer
    _check(stream.gpu._lib.gpurs_matmul_allgather(stream._handle, C.byref(desc), C.byref(gather), a.pointer, b.pointer))


def matmul_grouped(stream: Stream, inputs: DeviceBuffer, routes: DeviceBuffer, offsets: DeviceBuffer, weight: DeviceBuffer,
                   output: DeviceBuffer, rows: int, tokens: int, n: int, k: int, experts: int) -> None:
    """output[r] = inputs[routes[r]] @ weight[e]^T for offsets[e] <= r < offsets[e + 1]: the grouped (mixture-of-experts)
    product of the reference's `experts` example (examples/ada/examples/grouped_matrix.rs:30-60).  `routes` and `offsets`
    are I32 buffers holding unsigned values; weight is [experts][n][k]."""
    desc = _ffi.GroupedDesc(inputs.element, output.element, rows, tokens, n, k, experts, 0, 0)
    _check(stream.gpu._lib.gpurs_matmul_grouped(stream._handle, C.byref(desc), inputs.pointer, routes.pointer, offsets.pointer,
                                                weight.pointer, output.pointer))


def quantize_e4m3(stream: Stream, source: DeviceBuffer, rows: int, k: int, block_rows: int, ld: int = 0):
    """Block quantisation of a rows x k fp32 matrix on the device: returns (codes, scales) with one fp32 scale per
    block_rows x 128 block (block_rows = 1 for the left operand of a block-scaled product, 128 for the right one)."""
    gpu = stream.gpu
    codes = gpu.allocate(E4M3, rows * k)
    scales = gpu.allocate(F32, -(-rows // block_rows) * -(-k // 128))
    _check(gpu._lib.gpurs_quantize_e4m3(stream._handle, rows, k, source.pointer, ld, block_rows, codes.pointer, scales.pointer))
    return codes, scales


def quantize_mx_e4m3(stream: Stream, source: DeviceBuffer, rows: int, k: int, right_operand: bool, ld: int = 0):
    """MX quantisation of a rows x k fp32 matrix on the device: returns (codes, scales) with one power-of-two scale
    (UE8M0 byte) per 32 elements of a row, in the tiled order the MX-scaled product reads for its left
    (right_operand = False) or right operand.  Pass them to `matmul` with `scale_kind=SCALES_MX`."""
    gpu = stream.gpu
    codes = gpu.allocate(E4M3, rows * k)
    scales = gpu.allocate(I8, gpu._lib.gpurs_mx_scale_bytes(rows, k, 1 if right_operand else 0))
    _check(gpu._lib.gpurs_quantize_mx_e4m3(stream._handle, rows, k, source.pointer, ld, 1 if right_operand else 0, codes.pointer, scales.pointer))
    return codes, scales


def compress_24(stream: Stream, dense: DeviceBuffer, m: int, k: int, ld: int = 0):
    """2:4 compression of an m x k 16-bit matrix on the device: returns (values, metadata, violations) where
    `values` is the m x k/2 buffer of kept elements, `metadata` the byte buffer of their positions in the layout
    the sparse kernels read, and `violations` a one-element I32 buffer counting groups that were not 2:4."""
    gpu = stream.gpu
    values = gpu.allocate(dense.element, m * k // 2)
    metadata = gpu.zeros(I8, gpu._lib.gpurs_metadata_bytes(m, k))
    violations = gpu.zeros(I32, 1)
    _check(gpu._lib.gpurs_compress_24(stream._handle, dense.element, m, k, dense.pointer, ld, values.pointer, metadata.pointer, violations.pointer))
    return values, metadata, violations


class GpursErrorLocal(GpursError):
    """A rejection raised by this layer before the C ABI is reached."""

    def __init__(self, code: int, message: str):
        RuntimeError.__init__(self, message)
        self.code, self.operation, self.name, self.description = code, "matmul", "GPURS_ERROR", message
