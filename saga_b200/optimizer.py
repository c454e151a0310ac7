"""Host-side mirror of Saga's optimizer ops over the b200opt C ABI.

Names follow the reference (paths relative to the Saga project root):

* ``FlatLayout``       CudaProgram::create_optimizer's flat [weights | gradients]
                       buffer with 16-element padding (src/cuda/cuda_optimizer.cpp:196-260)
* ``AdamGroup``        the AdamF32 + AdamMixed pair of one rank
                       (src/cuda/cuda_optimizer.cpp:64-194); ``exec`` is their ``exec``
* ``LossScaler``       CudaProgram::m_mp_scaling and its update policy
                       (src/cuda/cuda_program.cpp:295-302)
* ``TrainingStepTail`` the end of CudaProgram::step: run the optimizer ops, get the
                       flag sums, update the scale (src/cuda/cuda_program.cpp:264,282-307)

All arithmetic happens in libb200opt.so; nothing here computes on the CPU
except through the library's own host-only entry points.
"""
import ctypes as C

import numpy as np

from . import capi
from .capi import check, lib


def policy_update(scale, flags, policy=capi.POLICY_REFERENCE, state=0, interval=2000):
    """Returns (new_scale as np.float32, new_state) from b200opt_policy_update."""
    s = C.c_float(float(scale))
    st = C.c_int(int(state))
    fl = (C.c_uint32 * 3)(*[int(x) for x in flags])
    check(lib().b200opt_policy_update(C.byref(s), fl, policy, C.byref(st), interval))
    return np.float32(s.value), st.value


def bias_corrections(it):
    b1, b2 = C.c_float(), C.c_float()
    check(lib().b200opt_bias_corrections(int(it), C.byref(b1), C.byref(b2)))
    return np.float32(b1.value), np.float32(b2.value)


class FlatLayout:
    """Offsets of tensors inside the flat buffer (each padded to 16 elements)."""

    def __init__(self, sizes):
        self.sizes = [int(s) for s in sizes]
        k = len(self.sizes)
        arr = (C.c_size_t * max(k, 1))(*self.sizes)
        offs = (C.c_size_t * max(k, 1))()
        total = C.c_size_t()
        check(lib().b200opt_layout(arr, k, offs, C.byref(total)))
        self.offsets = [int(offs[j]) for j in range(k)]
        self.total = int(total.value)

    def slices(self):
        return [slice(o, o + s) for o, s in zip(self.offsets, self.sizes)]


class _DeviceArray:
    """Zero-copy view of library-owned device memory for torch.as_tensor."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {
            "shape": (int(n),), "typestr": typestr, "data": (int(ptr), False),
            "version": 2, "strides": None,
        }


class LossScaler:
    """The program's loss scale (a float32, like CudaProgram::m_mp_scaling)."""

    def __init__(self, initial, policy=capi.POLICY_REFERENCE, interval=2000):
        self.scale = np.float32(initial)
        self.policy = policy
        self.interval = interval
        self.state = 0

    def update(self, flags):
        self.scale, self.state = policy_update(self.scale, flags, self.policy,
                                               self.state, self.interval)
        return self.scale


class AdamGroup:
    """One rank's optimizer: both dtype groups behind one b200opt handle."""

    def __init__(self, handle, rank, nranks, device, n_half, n_float, owns=True):
        self._h = C.c_void_p(handle)
        self.flags_created = 0
        self.rank, self.nranks, self.device = rank, nranks, device
        self.n_half, self.n_float = int(n_half), int(n_float)
        self._owns = owns

    # ------------------------------------------------------------ creation
    @classmethod
    def create(cls, rank, nranks, device, n_half, n_float=0, flags=0):
        """One rank; flags = capi.CREATE_FABRIC / capi.CREATE_MULTICAST for an arena that is
        shared by file descriptor and can be bound to an NVSwitch multicast object."""
        h = C.c_void_p()
        check(lib().b200opt_create_ex(C.byref(h), rank, nranks, device, n_half, n_float, flags))
        g = cls(h.value, rank, nranks, device, n_half, n_float)
        g.flags_created = flags
        return g

    @classmethod
    def create_group(cls, devices, n_half, n_float=0, flags=0):
        """All ranks in this process, wired to one another (Saga's threading model)."""
        n = len(devices)
        hs = (C.c_void_p * n)()
        devs = (C.c_int * n)(*devices)
        check(lib().b200opt_create_group_ex(hs, n, devs, n_half, n_float, flags))
        out = [cls(hs[r], r, n, devices[r], n_half, n_float) for r in range(n)]
        for g in out:
            g.flags_created = flags
        return out

    @staticmethod
    def multicast_supported(device):
        yes = C.c_int()
        check(lib().b200opt_multicast_supported(device, C.byref(yes)))
        return bool(yes.value)

    def destroy(self):
        if self._h and self._owns:
            lib().b200opt_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    # -------------------------------------------------------------- wiring
    def ipc_export(self):
        buf = (C.c_ubyte * capi.IPC_HANDLE_BYTES)()
        check(lib().b200opt_ipc_export(self._h, buf), self._h)
        return bytes(buf)

    def ipc_attach(self, peer_rank, handle_bytes):
        buf = (C.c_ubyte * capi.IPC_HANDLE_BYTES).from_buffer_copy(handle_bytes)
        check(lib().b200opt_ipc_attach(self._h, peer_rank, buf), self._h)

    def fd_export(self):
        """File descriptor of this rank's arena (CREATE_FABRIC); the caller closes it."""
        fd = C.c_int(-1)
        check(lib().b200opt_fd_export(self._h, C.byref(fd)), self._h)
        return fd.value

    def fd_attach(self, peer_rank, fd):
        check(lib().b200opt_fd_attach(self._h, peer_rank, fd), self._h)

    def mc_create(self):
        """Rank 0: creates the multicast object; returns its descriptor for the other ranks."""
        fd = C.c_int(-1)
        check(lib().b200opt_mc_create(self._h, C.byref(fd)), self._h)
        return fd.value

    def mc_join(self, fd):
        check(lib().b200opt_mc_join(self._h, fd), self._h)

    def mc_bind(self):
        check(lib().b200opt_mc_bind(self._h), self._h)

    def nccl_init(self, unique_id):
        buf = (C.c_ubyte * capi.NCCL_ID_BYTES).from_buffer_copy(unique_id)
        check(lib().b200opt_nccl_init(self._h, buf), self._h)

    @staticmethod
    def nccl_unique_id():
        buf = (C.c_ubyte * capi.NCCL_ID_BYTES)()
        check(lib().b200opt_nccl_unique_id(buf))
        return bytes(buf)

    # ------------------------------------------------------------- buffers
    def buffer_pointers(self, dtype):
        w, g, n = C.c_void_p(), C.c_void_p(), C.c_size_t()
        check(lib().b200opt_buffers(self._h, dtype, C.byref(w), C.byref(g), C.byref(n)), self._h)
        return w.value, g.value, n.value

    def buffers(self, dtype):
        """(weights, gradients) as torch tensors aliasing the library's memory."""
        import torch
        w, g, n = self.buffer_pointers(dtype)
        tdt = torch.float16 if dtype == capi.HALF else torch.float32
        dev = torch.device("cuda", self.device)
        if n == 0:
            return torch.empty(0, dtype=tdt, device=dev), torch.empty(0, dtype=tdt, device=dev)
        ts = "<f2" if dtype == capi.HALF else "<f4"
        with torch.cuda.device(dev):
            return (torch.as_tensor(_DeviceArray(w, n, ts), device=dev),
                    torch.as_tensor(_DeviceArray(g, n, ts), device=dev))

    def init_master(self, stream=0):
        check(lib().b200opt_init_master(self._h, C.c_void_p(stream)), self._h)

    # ---------------------------------------------------------------- step
    def exec(self, lr, l2_lambda, scale, stream=0):
        """AdamF32::exec + AdamMixed::exec of this rank; asynchronous."""
        check(lib().b200opt_step(self._h, lr, l2_lambda, float(scale), C.c_void_p(stream)), self._h)

    def step_begin(self):
        """Opens a step that is issued bucket by bucket (exec_bucket)."""
        check(lib().b200opt_step_begin(self._h), self._h)

    def exec_bucket(self, half_range, float_range, lr, l2_lambda, scale, stream=0, last=False):
        """Reduce + update + gather of one bucket: (first, count) per dtype group."""
        hf, hc = half_range
        ff, fc = float_range
        check(lib().b200opt_step_bucket(self._h, hf, hc, ff, fc, lr, l2_lambda, float(scale),
                                        C.c_void_p(stream), 1 if last else 0), self._h)

    def flags(self, stream=0):
        out = (C.c_uint32 * 3)()
        check(lib().b200opt_flags(self._h, C.c_void_p(stream), out), self._h)
        return (out[0], out[1], out[2])

    # ------------------------------------------- loss scale kept on the device
    def device_scale_enable(self, initial_scale, policy=capi.POLICY_REFERENCE, interval=2000,
                            log_capacity=4096):
        check(lib().b200opt_device_scale_enable(self._h, float(initial_scale), policy, interval,
                                                log_capacity), self._h)

    def device_scale_ptr(self):
        p = C.c_void_p()
        check(lib().b200opt_device_scale_ptr(self._h, C.byref(p)), self._h)
        return p.value

    def exec_device_scale(self, lr, l2_lambda, stream=0):
        """Like exec, with 1/scale read from and the policy applied on the device."""
        check(lib().b200opt_step_device_scale(self._h, lr, l2_lambda, C.c_void_p(stream)), self._h)

    def device_scale_read(self, stream=0, capacity=4096):
        """(scale, log) after waiting for the stream; log rows = (range, inf, nan, scale)."""
        scale, cnt = C.c_float(), C.c_size_t()
        buf = np.zeros((capacity, 4), dtype=np.uint32)
        check(lib().b200opt_device_scale_read(self._h, C.c_void_p(stream), C.byref(scale),
                                              buf.ctypes.data_as(C.c_void_p), capacity,
                                              C.byref(cnt)), self._h)
        rows = buf[:cnt.value]
        log = [(int(r[0]), int(r[1]), int(r[2]), np.float32(r[3:4].view(np.float32)[0]))
               for r in rows]
        return np.float32(scale.value), log

    def device_scale_peek(self):
        """(scale, step) as the last finished step kernel left them; does not wait."""
        scale, step = C.c_float(), C.c_uint32()
        check(lib().b200opt_device_scale_peek(self._h, C.byref(scale), C.byref(step)), self._h)
        return np.float32(scale.value), int(step.value)

    def step_host(self, grads_half_ptr, grads_float_ptr, lr, l2_lambda, scale, stream=0):
        out = (C.c_uint32 * 3)()
        check(lib().b200opt_step_host(self._h, C.c_void_p(grads_half_ptr),
                                      C.c_void_p(grads_float_ptr), lr, l2_lambda,
                                      float(scale), C.c_void_p(stream), out), self._h)
        return (out[0], out[1], out[2])

    # --------------------------------------------------------------- state
    @property
    def iter(self):
        v = C.c_int()
        check(lib().b200opt_get_iter(self._h, C.byref(v)))
        return v.value

    @iter.setter
    def iter(self, value):
        check(lib().b200opt_set_iter(self._h, int(value)))

    def export_state(self, dtype, which):
        cnt = C.c_size_t()
        check(lib().b200opt_export_state(self._h, dtype, which, None, 0, C.byref(cnt)), self._h)
        out = np.empty(cnt.value, dtype=np.float32)
        check(lib().b200opt_export_state(self._h, dtype, which, out.ctypes.data_as(C.c_void_p),
                                         out.size, C.byref(cnt)), self._h)
        return out

    def import_state(self, dtype, which, array):
        a = np.ascontiguousarray(array, dtype=np.float32)
        check(lib().b200opt_import_state(self._h, dtype, which, a.ctypes.data_as(C.c_void_p),
                                         a.size), self._h)

    def checkpoint_save(self, directory, scale, policy_state=0):
        """m, v, master, iteration counter and loss scale as Saga tensor files in `directory`."""
        check(lib().b200opt_checkpoint_save(self._h, str(directory).encode(), float(scale),
                                            int(policy_state)), self._h)

    def checkpoint_load(self, directory):
        """Restores what checkpoint_save wrote; returns (scale, policy_state)."""
        s, st = C.c_float(), C.c_int()
        check(lib().b200opt_checkpoint_load(self._h, str(directory).encode(), C.byref(s),
                                            C.byref(st)), self._h)
        return np.float32(s.value), st.value

    def set_option(self, option, value):
        check(lib().b200opt_set_option(self._h, option, int(value)), self._h)

    def get_option(self, option):
        v = C.c_long()
        check(lib().b200opt_get_option(self._h, option, C.byref(v)), self._h)
        return v.value

    def peer_copy(self, peer_rank, nbytes, stream=0):
        """Measurement aid: the peer's fp16 weights copied over this rank's (same values)."""
        check(lib().b200opt_peer_copy(self._h, peer_rank, nbytes, C.c_void_p(stream)), self._h)

    def phase_times(self):
        """(entry wait, entry..last CTA done, completion protocol, total) of the last step
        kernel in ns; needs OPT_PHASE_TIMERS and a preceding flags()."""
        out = (C.c_uint64 * 4)()
        check(lib().b200opt_phase_times(self._h, out), self._h)
        return tuple(int(x) for x in out)

    @property
    def launch_count(self):
        v = C.c_uint64()
        check(lib().b200opt_launch_count(self._h, C.byref(v)))
        return v.value


class TrainingStepTail:
    """The part of CudaProgram::step that follows backward, for one rank."""

    def __init__(self, group, scaler, lr, l2_lambda):
        self.group, self.scaler = group, scaler
        self.lr, self.l2_lambda = lr, l2_lambda

    def step(self, stream=0):
        """Runs the optimizer ops, reads the flag sums, updates the scale."""
        self.group.exec(self.lr, self.l2_lambda, self.scaler.scale, stream)
        flags = self.group.flags(stream)
        self.scaler.update(flags)
        return flags


def tensor_save(path, array):
    """A numpy float16/float32 array as a Saga tensor file (Tensor::save's format)."""
    a = np.ascontiguousarray(array)
    dt = {np.dtype(np.float16): capi.HALF, np.dtype(np.float32): capi.FLOAT}[a.dtype]
    dims = (C.c_uint32 * max(a.ndim, 1))(*a.shape)
    check(lib().b200opt_tensor_save(str(path).encode(), dt, a.ndim, dims,
                                    a.ctypes.data_as(C.c_void_p)))


def tensor_load(path):
    """The array stored in a Saga tensor file."""
    dt, rank, nbytes = C.c_int(), C.c_uint(), C.c_size_t()
    dims = (C.c_uint32 * 8)()
    check(lib().b200opt_tensor_load(str(path).encode(), C.byref(dt), C.byref(rank), dims, None, 0,
                                    C.byref(nbytes)))
    out = np.empty(tuple(dims[i] for i in range(rank.value)),
                   dtype=np.float16 if dt.value == capi.HALF else np.float32)
    check(lib().b200opt_tensor_load(str(path).encode(), None, None, None,
                                    out.ctypes.data_as(C.c_void_p), out.nbytes, None))
    return out


def adam_mixed(n, alpha, weights_ptr, grads_ptr, m_ptr, v_ptr, c_ptr, b1t, b2t, lr, l2,
               aux_ptr, stream=0):
    """saga::adam_mixed on caller-owned device memory (raw pointers)."""
    vp = C.c_void_p
    check(lib().b200opt_adam_mixed(n, alpha, vp(weights_ptr), vp(grads_ptr), vp(m_ptr), vp(v_ptr),
                                   vp(c_ptr), b1t, b2t, lr, l2, vp(aux_ptr), vp(stream)))


def adam_float(n, weights_ptr, grads_ptr, m_ptr, v_ptr, b1t, b2t, lr, l2, aux_ptr, stream=0):
    """saga::adam_float on caller-owned device memory (raw pointers)."""
    vp = C.c_void_p
    check(lib().b200opt_adam_float(n, vp(weights_ptr), vp(grads_ptr), vp(m_ptr), vp(v_ptr),
                                   b1t, b2t, lr, l2, vp(aux_ptr), vp(stream)))
