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


class Kernel:
    """Mirror of Strict.Compiler.Cuda.Kernel: `Context` is opened on device 0 at construction
    and released by Dispose (Kernel.cs:9,13-17). The cuBLAS `Handle` of the reference is never
    used for any routine (Kernel.cs:10-11) and has no counterpart here; kernels are compiled ahead
    of time, so CompileKernelAndSaveAsPtxFile has nothing to compile and `run` launches directly."""

    def __init__(self, device=0):
        self.Context = Context(device)

    def run(self, method, *args):
        """Launch the ahead-of-time equivalent of a kernel emitted by InstructionsToCuda: `method`
        is a CompiledMethod (instructions_to_cuda.py); args follow the emitted signature —
        array parameters (DeviceVariable), scalars, then `output`, then `count` if the
        signature has one (Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:73-87)."""
        return method.launch(self.Context, *args)

    Run = run

    def dispose(self):
        self.Context.dispose()

    Dispose = dispose

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.dispose()
