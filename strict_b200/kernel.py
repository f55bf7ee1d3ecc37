"""Host-side mirror of the reference's kernel-launch surface.

`Kernel` plays the role of Strict.Compiler.Cuda.Kernel (Strict.Compiler.Cuda/Kernel.cs:7-58):
it opens device 0 and owns the native context; `DeviceVariable` plays the role of ManagedCuda's
CudaDeviceVariable<T> as the reference's tests use it
(Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:64,75-76,56): construct from a size
or a host array, read back as a host array, index one element.
"""
import ctypes as C

import numpy as np

from . import native as N


class Context:
    """One device + one stream (replaces `new CudaContext(0)`, Kernel.cs:9)."""

    def __init__(self, device=0):
        self.h = C.c_void_p()
        N.check(N.lib().strictb200_create(device, C.byref(self.h)))
        self.device = device

    def synchronize(self):
        N.check(N.lib().strictb200_synchronize(self.h))

    def timer_begin(self):
        N.check(N.lib().strictb200_timer_begin(self.h))

    def timer_end(self):
        ms = C.c_float()
        N.check(N.lib().strictb200_timer_end(self.h, C.byref(ms)))
        return ms.value

    def record(self):
        """Context manager: the calls made inside are recorded, not run; yields nothing and leaves
        the recorded sequence in ``self.last_graph`` (replay with ``replay(graph, times)``)."""
        ctx = self

        class _Rec:
            def __enter__(self):
                N.check(N.lib().strictb200_graph_begin(ctx.h))

            def __exit__(self, et, ev, tb):
                g = C.c_void_p()
                st = N.lib().strictb200_graph_end(ctx.h, C.byref(g))
                if et is None:
                    N.check(st)
                    ctx.last_graph = g
                return False

        return _Rec()

    def replay(self, graph, times=1):
        N.check(N.lib().strictb200_graph_launch(self.h, graph, times))

    def free_graph(self, graph):
        N.check(N.lib().strictb200_graph_destroy(graph))

    def launch_count(self):
        n = C.c_uint64()
        N.check(N.lib().strictb200_launch_count(self.h, C.byref(n)))
        return n.value

    def device_status(self):
        """Synchronise and raise KernelException if a kernel's bounded wait expired."""
        code = C.c_int()
        N.check(N.lib().strictb200_device_status(self.h, C.byref(code)))
        return code.value

    def set_option(self, name, value):
        """A switch of this context (see strictb200_set_option); also settable once, at creation,
        through the environment variable STRICTB200_<NAME>."""
        N.check(N.lib().strictb200_set_option(self.h, name.encode(), int(value)))

    def get_option(self, name):
        v = C.c_int()
        N.check(N.lib().strictb200_get_option(self.h, name.encode(), C.byref(v)))
        return v.value

    def trace(self, capacity=1 << 18):
        """Context manager: per-block time stamps of the instrumented decode kernels launched inside
        (strictb200_trace_begin/_end). The object's ``records`` is an (n, 8) uint64 array afterwards:
        start, after the dependency wait, end (ns of the GPU's global timer),
        kernel id | tag << 8 | SM << 48, three optional marks inside the kernel, 0; ``reported`` counts the blocks, also beyond the capacity."""
        ctx = self

        class _Trace:
            records = None
            reported = 0

            def __enter__(self):
                N.check(N.lib().strictb200_trace_begin(ctx.h, capacity))
                return self

            def __exit__(self, et, ev, tb):
                buf = np.empty((capacity, 8), np.uint64)
                n = C.c_int()
                st = N.lib().strictb200_trace_end(ctx.h, N.ptr(buf), capacity, C.byref(n))
                self.reported = n.value
                self.records = buf[:min(n.value, capacity)].copy()
                if et is None:
                    N.check(st)
                return False

        return _Trace()

    def option(self, name, value):
        """Context manager: the option holds `value` inside the block and its old value after it."""
        ctx = self

        class _Opt:
            def __enter__(self):
                self.old = ctx.get_option(name)
                ctx.set_option(name, value)

            def __exit__(self, *a):
                ctx.set_option(name, self.old)
                return False

        return _Opt()

    def flush_l2(self):
        N.check(N.lib().strictb200_flush_l2(self.h))

    def tp_init(self, world, rank, unique_id):
        N.check(N.lib().strictb200_tp_init(self.h, world, rank, unique_id))

    def tp_open_peer_buffers(self, all_gather):
        """Enable the fused peer-memory all-reduce: all_gather(uint8[64]) -> uint8[world, 64] must
        return every rank's array in rank order (any host transport)."""
        mine = np.zeros(64, np.uint8)
        N.check(N.lib().strictb200_tp_comm_handle(self.h, N.ptr(mine)))
        handles = np.ascontiguousarray(all_gather(mine), dtype=np.uint8)
        N.check(N.lib().strictb200_tp_comm_open(self.h, N.ptr(handles)))

    def dispose(self):
        if self.h:
            N.lib().strictb200_destroy(self.h)
            self.h = C.c_void_p()

    Dispose = dispose

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.dispose()


class DeviceVariable:
    """Typed device array. DeviceVariable(ctx, n, dtype) allocates; DeviceVariable.of(ctx, host)
    uploads; .to_host() downloads; v[i] reads one element (device -> host)."""

    def __init__(self, ctx, count, dtype=np.float32):
        self.ctx, self.dtype, self.count = ctx, np.dtype(dtype), int(count)
        self.p = C.c_void_p()
        N.check(N.lib().strictb200_malloc(ctx.h, self.nbytes, C.byref(self.p)))

    @property
    def nbytes(self):
        return self.count * self.dtype.itemsize

    @property
    def device_pointer(self):
        return self.p

    DevicePointer = device_pointer

    @classmethod
    def of(cls, ctx, host):
        host = np.ascontiguousarray(host)
        v = cls(ctx, host.size, host.dtype)
        v.upload(host)
        return v

    def upload(self, host):
        host = np.ascontiguousarray(host, dtype=self.dtype)
        if host.size != self.count:
            raise ValueError("size mismatch")
        N.check(N.lib().strictb200_upload(self.ctx.h, self.p, N.ptr(host), self.nbytes))

    def to_host(self, shape=None):
        out = np.empty(self.count, self.dtype)
        N.check(N.lib().strictb200_download(self.ctx.h, N.ptr(out), self.p, self.nbytes))
        return out.reshape(shape) if shape is not None else out

    def zero(self):
        N.check(N.lib().strictb200_memset(self.ctx.h, self.p, 0, self.nbytes))

    def __getitem__(self, i):
        if not 0 <= i < self.count:
            raise IndexError(i)
        out = np.empty(1, self.dtype)
        src = C.c_void_p(self.p.value + i * self.dtype.itemsize)
        N.check(N.lib().strictb200_download(self.ctx.h, N.ptr(out), src, self.dtype.itemsize))
        return out[0]

    def free(self):
        if self.p:
            N.lib().strictb200_free(self.ctx.h, self.p)
            self.p = C.c_void_p()


class FlatNumbers:
    """Device-side counterpart of the flat numeric backing of ValueArrayInstance
    (Strict.Expressions/ValueArrayInstance.cs:9-16): one contiguous fp32 array holding `Count`
    elements of `FlatWidth` numbers each (an array of structs, e.g. Color = 4 floats), element i
    member m at ``offset + i*FlatWidth + m`` (ValueArrayInstance.cs:128,339). Slices share the
    backing array and only move `offset` (ValueArrayInstance.cs:63-64); the host array is uploaded
    unchanged."""

    def __init__(self, backing, flat_width, offset=0, count=None):
        if flat_width < 1 or offset < 0:
            raise ValueError("FlatWidth must be positive and offset non-negative")
        self.backing, self.FlatWidth, self.offset = backing, int(flat_width), int(offset)
        self.Count = (backing.count - self.offset) // self.FlatWidth if count is None else int(count)
        if self.Count < 0 or self.offset + self.Count * self.FlatWidth > backing.count:
            raise ValueError("view exceeds the backing array")

    @classmethod
    def of(cls, ctx, flat_numbers, flat_width, offset=0, count=None):
        host = np.ascontiguousarray(flat_numbers, dtype=np.float32).reshape(-1)
        return cls(DeviceVariable.of(ctx, host), flat_width, offset, count)

    def slice(self, first, count):
        """Elements [first, first+count) as a view over the same device memory."""
        if first < 0 or count < 0 or first + count > self.Count:
            raise IndexError((first, count))
        return FlatNumbers(self.backing, self.FlatWidth, self.offset + first * self.FlatWidth, count)

    def GetFlat(self, index):
        """One number by flat index, as ValueArrayInstance.GetFlat (flatNumbers[offset + index])."""
        return self.backing[self.offset + index]

    def __getitem__(self, i):
        """Element i as a tuple of its FlatWidth members."""
        if not 0 <= i < self.Count:
            raise IndexError(i)
        return tuple(float(self.backing[self.offset + i * self.FlatWidth + m]) for m in range(self.FlatWidth))

    def to_host(self):
        """[Count, FlatWidth] host copy of the view."""
        flat = self.backing.to_host()
        return flat[self.offset:self.offset + self.Count * self.FlatWidth].reshape(self.Count, self.FlatWidth).copy()

    def adjust_brightness(self, brightness, channels=3, clamp=False):
        """ImageProcessing/AdjustBrightness.strict over this view, in place on the device."""
        N.check(N.lib().strictb200_adjust_brightness(self.backing.ctx.h, self.backing.p, self.offset, self.Count, self.FlatWidth, channels,
                                                     float(brightness), 1 if clamp else 0))
        return self


def blur5x5_rgb8(ctx, pixels, width, height, iterations=1):
    """The reference harness's in-place 5x5 box blur (BlurPerformanceTests.cs:52-67) on the device:
    uploads `pixels` (uint8, width*height*3), runs `iterations` passes between two device buffers,
    returns the blurred bytes."""
    host = np.ascontiguousarray(pixels, dtype=np.uint8).reshape(-1)
    if host.size != width * height * 3:
        raise ValueError("pixels must hold width*height*3 bytes")
    a, b = DeviceVariable.of(ctx, host), DeviceVariable(ctx, max(host.size, 1), np.uint8)
    for _ in range(iterations):
        N.check(N.lib().strictb200_blur5x5_rgb8(ctx.h, a.p, b.p, width, height))
        a, b = b, a
    out = a.to_host()[:host.size]
    a.free(), b.free()
    return out


class CudaBlasHandle:
    """Stand-in for the lazily created cuBLAS handle of the reference's Kernel (Kernel.cs:10-11).
    The reference never calls a cuBLAS routine through it; the GEMMs of this library are its own
    kernels, so the handle only carries the context it belongs to and a Dispose."""

    def __init__(self, context):
        self.Context = context
        self.disposed = False

    def Dispose(self):
        self.disposed = True


class Kernel:
    """Mirror of Strict.Compiler.Cuda.Kernel (Kernel.cs:7-58): `Context` is opened on device 0 at
    construction and released by Dispose together with the handle (Kernel.cs:13-17); `Handle` is
    created on first use (Kernel.cs:10-11); CompileKernelAndSaveAsPtxFile compiles the same saxpy
    text with NVRTC and writes VectorAdd.ptx (Kernel.cs:19-33,54-58), for compute_100a instead of
    the reference's compute_61. Kernels that run are compiled ahead of time: `Run` launches the
    ahead-of-time equivalent of an emitted kernel."""

    # the text the reference compiles (Kernel.cs:22-28)
    SAXPY = ('extern "C" __global__ void saxpy(float a, float *x, float *y, float *out, size_t n)\n'
             "{\n"
             "  size_t tid = blockIdx.x * blockDim.x + threadIdx.x;\n"
             "  if (tid < n) {\n"
             "    out[tid] = a * x[tid] + y[tid];\n"
             "  }\n"
             "}")
    GPU_ARCHITECTURE = "--gpu-architecture=compute_100a"

    def __init__(self, device=0):
        self.Context = Context(device)
        self._handle = None

    @property
    def Handle(self):
        if self._handle is None:
            self._handle = CudaBlasHandle(self.Context)
        return self._handle

    def CompileKernelAndSaveAsPtxFile(self, path="VectorAdd.ptx"):
        """Returns True and writes the PTX on success; False on a compile error, which the
        reference swallows into an nvrtcResult (Kernel.cs:35-52). NotImplementedError where
        NVRTC is not installed."""
        try:
            ptx = N.compile_to_ptx(self.SAXPY, "saxpy", (self.GPU_ARCHITECTURE,))
        except ValueError:
            return False
        with open(path, "w") as f:
            f.write(ptx)
        return True

    def run(self, method, *args):
        """Launch the ahead-of-time equivalent of a kernel emitted by InstructionsToCuda: `method`
        is a CompiledMethod (instructions_to_cuda.py); args follow the emitted signature —
        array parameters (DeviceVariable), scalars, then `output`, then `count` if the
        signature has one (Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:73-87)."""
        return method.launch(self.Context, *args)

    Run = run

    def dispose(self):
        self.Context.dispose()
        if self._handle is not None:
            self._handle.Dispose()

    Dispose = dispose

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.dispose()
