"""CUDA-backed runtime with the surface of the reference's Vulkan runtime.

Same names and meanings as BrettKnox/vkgrad vk.py -- `Device` (vk.py:892),
`Buffer` (vk.py:507-616), `Graph` (vk.py:807-889), `VkError` (vk.py:128) -- so
code written against that module (autograd, transformer, dataparallel, the
reference's tests and examples) keeps its shape.  Underneath it is one CUDA
stream per device, CUDA graphs for recorded steps, and the C ABI of
libvkgrad_b200.so; numpy is the host array type and torch is not involved.

Memory kinds (vk.py:1161-1200):
  "device"  HBM only; array() raises VkError as in the reference.
  "shared"  pinned host memory mapped into the GPU: host writes are visible to
            the next submit without flush() (callers rely on that,
            examples/mnist.py:170-171).  "bar" is treated the same.
  "cached"  HBM plus a pinned host mirror: flush() uploads, invalidate()
            downloads, exactly where the reference calls them
            (autograd.py:142-149, 277-279).
"""

import ctypes as C

import numpy as np

from . import _lib

_KINDS = {"device": 0, "shared": 1, "bar": 1, "cached": 2}


class VkError(RuntimeError):
    """Every failed runtime or kernel call (reference: vk.py:128-134)."""


def _check(status, what):
    if status != 0:
        raise VkError(f"{what}: {_lib.last_error()}")


class Buffer:
    """A block of GPU-visible memory.  `dptr` is what kernels receive."""

    def __init__(self, dev, size, kind="shared", _parent=None, _offset=0):
        if kind not in _KINDS and kind != "view":
            raise VkError(f"no memory type for kind={kind!r}")
        self.dev = dev
        self.size = int(size)
        self.kind = kind if _parent is None else _parent.kind
        self._parent = _parent
        self._alive = True
        if _parent is not None:
            self.dptr = _parent.dptr + _offset
            self.hptr = None if _parent.hptr is None else _parent.hptr + _offset
            return
        d, h = C.c_void_p(), C.c_void_p()
        _check(dev.lib.vkg_alloc(dev.handle, self.size, _KINDS[kind], C.byref(d), C.byref(h)),
               f"buffer({self.size}, {kind!r})")
        self.dptr = d.value
        self.hptr = h.value
        dev._live += 1

    @property
    def host_visible(self):
        return self.hptr is not None

    def view(self, offset, size):
        """A sub-range of this buffer (no ownership); used for flat arenas."""
        if offset < 0 or offset + size > self.size:
            raise VkError(f"view [{offset}, {offset + size}) outside buffer of {self.size} bytes")
        return Buffer(self.dev, size, "view", _parent=self, _offset=int(offset))

    def array(self, dtype, shape=None):
        """Live numpy view of the host-visible bytes (vk.py:583-595)."""
        if self.hptr is None:
            raise VkError(f"buffer kind={self.kind!r} is not host-visible")
        raw = (C.c_ubyte * self.size).from_address(self.hptr)
        a = np.frombuffer(raw, dtype=dtype)
        return a if shape is None else a.reshape(shape)

    def flush(self):
        """CPU writes -> visible to the GPU (vk.py:598-603)."""
        if self.kind == "cached":
            _check(self.dev.lib.vkg_upload(self.dev.handle, self.dptr, self.hptr, self.size),
                   "flush")

    def invalidate(self):
        """GPU writes -> visible to the CPU (vk.py:605-610)."""
        if self.kind == "cached":
            _check(self.dev.lib.vkg_download(self.dev.handle, self.hptr, self.dptr, self.size),
                   "invalidate")
        else:
            self.dev.sync()

    def destroy(self):
        if not self._alive:
            return
        self._alive = False
        if self._parent is None and self.dev.handle:
            self.dev.sync()
            _check(self.dev.lib.vkg_free(self.dev.handle, self.dptr, self.hptr, _KINDS[self.kind]),
                   "free")
            self.dev._live -= 1
        self.dptr = None
        self.hptr = None


class Graph:
    """A recorded sequence of launches replayed with one submit (vk.py:807-889).

    record() stores a thunk per dispatch; finish() replays the thunks under CUDA
    stream capture and instantiates the graph; submit() launches it, waits, and
    returns GPU seconds.  Several graphs can be recorded interleaved (one per
    stage, transformer.py:339-345) because nothing is captured until finish().
    """

    def __init__(self, dev, name="graph"):
        self.dev = dev
        self.name = name
        self.n_dispatch = 0
        self.traffic = []
        self.mm_split = []
        self._ops = []
        self._finished = False
        self._handle = None
        self.n_kernels = 0

    def add(self, thunk, name="op", nbytes=0, hint=None):
        if self._finished:
            raise VkError(f"{self.name}: already finished")
        self._ops.append(thunk)
        self.traffic.append((name, nbytes, nbytes if hint is None else hint))
        self.n_dispatch += 1

    def record(self, kernel, buffers, groups=None, push=b"", bytes_hint=None):
        """Reference-shaped entry: `kernel` is any object with launch(buffers, push)."""
        self.add(lambda: kernel.launch(buffers, push), getattr(kernel, "name", "kernel"),
                 sum(b.size for b in buffers), bytes_hint)

    def finish(self):
        if self._finished:
            raise VkError(f"{self.name}: already finished")
        lib, h = self.dev.lib, self.dev.handle
        _check(lib.vkg_graph_begin(h), f"{self.name}: begin capture")
        err = None
        try:
            for op in self._ops:
                op()
        except Exception as e:  # end the capture before reporting
            err = e
        g = C.c_void_p()
        status = lib.vkg_graph_end(h, C.byref(g))
        if err is not None:
            if status == 0:
                lib.vkg_graph_destroy(g)
            raise err
        _check(status, f"{self.name}: end capture")
        self._handle = g
        n = C.c_int(0)
        lib.vkg_graph_kernel_count(g, C.byref(n))
        self.n_kernels = n.value
        self._finished = True
        return self

    def submit(self):
        if not self._finished:
            raise VkError(f"{self.name}: call finish() before submit()")
        s = C.c_double(0.0)
        _check(self.dev.lib.vkg_graph_launch(self.dev.handle, self._handle, C.byref(s)),
               f"{self.name}: submit")
        return s.value

    def submit_async(self):
        """Enqueue without waiting; pair with dev.sync()."""
        if not self._finished:
            raise VkError(f"{self.name}: call finish() before submit()")
        _check(self.dev.lib.vkg_graph_launch_async(self.dev.handle, self._handle),
               f"{self.name}: submit")

    def destroy(self):
        if self._handle is not None:
            self.dev.lib.vkg_graph_destroy(self._handle)
            self._handle = None
        self._ops = []


class Device:
    """One B200.  Mirrors the attributes callers of vk.Device read."""

    has_coop_matrix = True        # tcgen05 tensor cores
    has_atomic_float = True
    row_subgroup_size = 32
    can_set_subgroup_size = True
    has_pipeline_stats = False

    def __init__(self, ordinal=0, validate=None, prefer_async_compute=True):
        self.lib = _lib.load()
        self.handle = None
        self._live = 0
        h = C.c_void_p()
        _check(self.lib.vkg_device_create(int(ordinal), C.byref(h)), f"Device({ordinal})")
        self.handle = h
        self.ordinal = int(ordinal)
        name = C.create_string_buffer(128)
        sms, total, maj, mnr = C.c_int(), C.c_size_t(), C.c_int(), C.c_int()
        _check(self.lib.vkg_device_info(h, name, 128, C.byref(sms), C.byref(total),
                                        C.byref(maj), C.byref(mnr)), "device_info")
        self.name = name.value.decode()
        self.sm_count = sms.value
        self.total_bytes = total.value
        self.compute_capability = (maj.value, mnr.value)
        self.features = {"tcgen05": True, "tma": True, "atomic_float": True}
        self.extensions = []
        self._scratch = []     # grow-only list so recorded graphs keep valid pointers
        self._staging = {}

    def __repr__(self):
        return (f"<Device {self.ordinal}: {self.name}, {self.sm_count} SMs, "
                f"{self.total_bytes / 2**30:.0f} GiB, sm_{self.compute_capability[0]}"
                f"{self.compute_capability[1]}>")

    # -- memory -----------------------------------------------------------
    def buffer(self, size, kind="shared", usage=None):
        return Buffer(self, size, kind)

    def scratch(self, nbytes):
        """Device scratch of at least nbytes, shared by ops on this stream."""
        for b in self._scratch:
            if b.size >= nbytes:
                return b
        b = Buffer(self, max(int(nbytes), 1 << 20), "device")
        self._scratch.append(b)
        return b

    def staging(self, key, nbytes):
        """Per-call-site device copy of a host-mapped GEMM operand."""
        b = self._staging.get(key)
        if b is None or b.size < nbytes:
            b = Buffer(self, nbytes, "device")
            self._staging[key] = b   # the old one stays alive with its graphs
        return b

    def import_host_buffer(self, ptr, size, usage=None):
        raise VkError("import_host_buffer: the shared host arena is replaced by NCCL "
                      "all-reduce on this backend (see dataparallel.Replica)")

    # -- execution --------------------------------------------------------
    def graph(self, name="graph"):
        return Graph(self, name)

    def run_op(self, thunk, repeat=1):
        """Eager launch: enqueue `repeat` times, wait, return GPU seconds."""
        _check(self.lib.vkg_timer_begin(self.handle), "timer")
        for _ in range(repeat):
            thunk()
        s = C.c_double(0.0)
        _check(self.lib.vkg_timer_end(self.handle, C.byref(s)), "run")
        return s.value

    def copy(self, src, dst, size=None, repeat=1):
        size = size if size is not None else min(src.size, dst.size)

        def go():
            _check(self.lib.vkg_copy(self.handle, dst.dptr, src.dptr, size), "copy")
        return self.run_op(go, repeat)

    def sync(self):
        _check(self.lib.vkg_sync(self.handle), "sync")

    def destroy(self):
        if self.handle:
            for b in list(self._scratch) + list(self._staging.values()):
                b.destroy()
            self._scratch, self._staging = [], {}
            self.lib.vkg_device_destroy(self.handle)
            self.handle = None
