"""ctypes mirror of the reference's ``Backend`` / ``Session`` traits
(crates/onyxia-ir/src/backend.rs:24-54) over ``libonyxia_cuda.so``.

Same names and argument meaning as the reference: ``prepare`` consumes the
module; ``run`` takes named device tensors and returns all outputs, on the
device, in signature order; ``upload`` / ``download`` cross the host boundary.
There is no CPU path behind this class.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _ffi
from ._ffi import check
from .ir import HostTensor, Module


class DeviceTensor:
    """A device-resident tensor handle; cheap to clone, released on garbage collection."""

    def __init__(self, handle):
        self._h = handle

    @property
    def handle(self):
        return self._h

    def describe(self):
        dt, rank = C.c_int32(), C.c_int32()
        shape = (C.c_uint64 * 8)()
        check(_ffi.cuda_lib().ox_tensor_describe(self._h, C.byref(dt), shape, 8, C.byref(rank)))
        return dt.value, tuple(shape[i] for i in range(rank.value))

    @property
    def dtype(self) -> int:
        return self.describe()[0]

    @property
    def shape(self) -> tuple:
        return self.describe()[1]

    @property
    def nbytes(self) -> int:
        return _ffi.cuda_lib().ox_tensor_nbytes(self._h)

    def clone(self) -> "DeviceTensor":
        return DeviceTensor(_ffi.cuda_lib().ox_tensor_clone(self._h))

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                _ffi.cuda_lib().ox_tensor_release(self._h)
            except Exception:
                pass
            self._h = None


class CudaSession:
    """≙ ``impl Session`` of the reference GPU backend (session.rs:510-649)."""

    def __init__(self, handle):
        self._h = handle
        self._lib = _ffi.cuda_lib()

    def upload(self, t: HostTensor) -> DeviceTensor:
        shape = (C.c_uint64 * max(len(t.shape), 1))(*t.shape)
        out = C.c_void_p()
        check(self._lib.ox_session_upload(self._h, t.dtype, shape, len(t.shape), t.data.ctypes.data_as(C.c_void_p),
                                          t.data.size, C.byref(out)))
        return DeviceTensor(out)

    def run(self, inputs) -> list:
        """inputs: dict or sequence of (name, DeviceTensor) → [(name, DeviceTensor)] in signature order."""
        items = list(inputs.items()) if isinstance(inputs, dict) else list(inputs)
        n = len(items)
        names = (C.c_char_p * max(n, 1))(*[k.encode() for k, _ in items])
        handles = (C.c_void_p * max(n, 1))(*[t.handle for _, t in items])
        cap = 4096
        out_names = (C.c_char_p * cap)()
        out_tensors = (C.c_void_p * cap)()
        n_out = C.c_int32()
        check(self._lib.ox_session_run(self._h, names, handles, n, out_names, out_tensors, cap, C.byref(n_out)))
        return [(out_names[i].decode(), DeviceTensor(C.c_void_p(out_tensors[i]))) for i in range(n_out.value)]

    def download(self, t: DeviceTensor) -> HostTensor:
        dtype, shape = t.describe()
        nbytes = t.nbytes
        buf = np.empty(nbytes, dtype=np.uint8)
        written = C.c_size_t()
        check(self._lib.ox_session_download(self._h, t.handle, buf.ctypes.data_as(C.c_void_p), nbytes, C.byref(written)))
        return HostTensor(dtype, shape, buf)

    def argmax_last(self, t: DeviceTensor) -> DeviceTensor:
        out = C.c_void_p()
        check(self._lib.ox_session_argmax_last(self._h, t.handle, C.byref(out)))
        return DeviceTensor(out)

    def sample_last(self, t: DeviceTensor, temperature: float, top_k: int, top_p: float, uniform) -> DeviceTensor:
        """One token per row by temperature / top-k / top-p sampling on the device (≙ sampling::sample,
        crates/onyxia-cli/src/sampling.rs:36-65); `uniform` holds one number in [0, 1] per row."""
        u = np.ascontiguousarray(np.asarray(uniform, dtype=np.float32).reshape(-1))
        out = C.c_void_p()
        check(self._lib.ox_session_sample_last(self._h, t.handle, float(temperature), int(top_k), float(top_p),
                                               u.ctypes.data_as(C.POINTER(C.c_float)), u.size, C.byref(out)))
        return DeviceTensor(out)

    def argmax_last_into(self, t: DeviceTensor, out: DeviceTensor) -> None:
        """Argmax over the last axis written into `out` (I64, one element per row); allocates nothing."""
        check(self._lib.ox_session_argmax_last_into(self._h, t.handle, out.handle))

    # inherent methods of the reference session (session.rs:280-340)
    def wait_idle(self) -> None:
        check(self._lib.ox_session_wait_idle(self._h))

    def resident_bytes(self) -> int:
        return self._lib.ox_session_resident_bytes(self._h)

    def peak_resident_bytes(self) -> int:
        return self._lib.ox_session_peak_resident_bytes(self._h)

    def pool_stats(self) -> tuple:
        a, b = C.c_uint64(), C.c_uint64()
        self._lib.ox_session_pool_stats(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def enable_profiling(self, on: bool = True) -> bool:
        return bool(self._lib.ox_session_enable_profiling(self._h, int(on)))

    def take_timings(self) -> list:
        cap = 1 << 16
        arr = (_ffi.KernelTiming * cap)()
        n = self._lib.ox_session_take_timings(self._h, arr, cap)
        return [(arr[i].kernel.decode(), arr[i].node.decode(), arr[i].time_ns) for i in range(min(n, cap))]

    def timer_start(self) -> None:
        check(self._lib.ox_session_timer_start(self._h))

    def timer_stop(self) -> float:
        ms = C.c_float()
        check(self._lib.ox_session_timer_stop(self._h, C.byref(ms)))
        return ms.value

    def plan_stats(self) -> dict:
        out = (C.c_uint64 * 9)()
        self._lib.ox_session_plan_stats(self._h, out)
        return dict(zip(("built", "updated", "reused", "graph_launches", "graph_node_updates", "runs", "bind_us",
                         "plan_us", "launch_us"), [int(v) for v in out]))

    def launch_count(self) -> int:
        return self._lib.ox_session_launch_count(self._h)

    def close(self) -> None:
        if self._h:
            self._lib.ox_session_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def nccl_library_path():
    """libnccl.so.2 as shipped beside torch (None if it cannot be found: the loader path is searched then)."""
    try:
        import nvidia.nccl  # type: ignore
        import os
        for d in nvidia.nccl.__path__:
            p = os.path.join(d, "lib", "libnccl.so.2")
            if os.path.exists(p):
                return p
    except Exception:  # noqa: BLE001 - optional
        pass
    return None


class CudaBackend:
    """≙ ``impl Backend`` (session.rs:107-242)."""

    def __init__(self, devices: Sequence[int] = (0,), *, without_fused_kernels: bool = False,
                 disable_graphs: bool = False, disable_pattern_fusion: bool = False,
                 disable_persistent_step: bool = False):
        self._lib = _ffi.cuda_lib()
        self.devices = tuple(int(d) for d in devices)
        opts = _ffi.BackendOptions()
        opts.without_fused_kernels = int(without_fused_kernels)
        opts.disable_graphs = int(disable_graphs)
        opts.disable_pattern_fusion = int(disable_pattern_fusion)
        opts.disable_persistent_step = int(disable_persistent_step)
        devs = (C.c_int32 * max(len(devices), 1))(*devices)
        h = C.c_void_p()
        check(self._lib.ox_backend_create_ex(devs, len(devices), C.byref(opts), C.byref(h)))
        self._h = h

    @classmethod
    def without_fused_kernels(cls, devices: Sequence[int] = (0,)) -> "CudaBackend":
        """≙ ``WgpuBackend::without_fused_kernels`` (session.rs:125-134)."""
        return cls(devices, without_fused_kernels=True)

    def supports(self, composite: str) -> bool:
        return bool(self._lib.ox_backend_supports(self._h, composite.encode()))

    # tensor parallelism: one process per GPU, the id travels by whatever channel the host has
    @staticmethod
    def tp_unique_id(nccl_path: str | None = None) -> bytes:
        out = (C.c_uint8 * 128)()
        check(_ffi.cuda_lib().ox_tp_unique_id(nccl_path.encode() if nccl_path else None, out))
        return bytes(out)

    def join_tp(self, rank: int, world: int, unique_id: bytes, nccl_path: str | None = None) -> None:
        """Collective: returns when all `world` ranks have joined. Afterwards the backend executes
        modules made by ``Module.tp_partition(world, rank)``."""
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(self._lib.ox_backend_join_tp(self._h, rank, world, buf, nccl_path.encode() if nccl_path else None))

    def peer_allreduce(self) -> bool:
        """True when the joined group's f16 all-reduces run as the library's own kernel over peer memory."""
        return bool(self._lib.ox_backend_peer_allreduce(self._h))

    def join_tp_torch(self, group=None) -> tuple:
        """Join the group formed by a torch.distributed process group (used only to pass the id around)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [self.tp_unique_id(nccl_library_path()) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=group)
        self.join_tp(rank, world, box[0], nccl_library_path())
        return rank, world

    def prepare(self, module: Module) -> CudaSession:
        keep = module._keep
        out = C.c_void_p()
        check(self._lib.ox_backend_prepare(self._h, module._take(), C.byref(out)))
        del keep  # weights are on the device now
        return CudaSession(out)

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                self._lib.ox_backend_free(self._h)
            except Exception:
                pass
            self._h = None


def run_once(backend: CudaBackend, module: Module, inputs: dict) -> list:
    """prepare + upload + run + download, for tests (≙ the helper in gpu_test.rs:22-74)."""
    sess = backend.prepare(module)
    dev = {k: sess.upload(v) for k, v in inputs.items()}
    outs = sess.run(dev)
    return [(name, sess.download(t)) for name, t in outs]
