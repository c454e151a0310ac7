"""Helpers for the GPU parity tests: numpy <-> library-owned device buffers."""
import numpy as np
import torch

from saga_b200 import AdamGroup, capi


def dev_u16(a, device=0):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).to(torch.device("cuda", device))


def dev_f32(a, device=0):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32).copy()).to(torch.device("cuda", device))


def host_u16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16).copy()


def stream_ptr(device=0):
    return torch.cuda.current_stream(torch.device("cuda", device)).cuda_stream


class Program:
    """N ranks of the CUDA path with the weights/gradients API the tests need."""

    def __init__(self, nranks, n_half, n_float=0, devices=None, variant=None, path=None,
                 create_flags=0):
        devices = devices or [0] * nranks
        self.N = nranks
        self.devices = devices
        self.groups = (AdamGroup.create_group(devices, n_half, n_float, create_flags) if nranks > 1
                       else [AdamGroup.create(0, 1, devices[0], n_half, n_float, create_flags)])
        self.Wh, self.Gh, self.Wf, self.Gf = [], [], [], []
        for g in self.groups:
            if variant is not None:
                g.set_option(capi.OPT_KERNEL_VARIANT, variant)
            if path is not None:
                g.set_option(capi.OPT_PATH, path)
            w, gr = g.buffers(capi.HALF)
            self.Wh.append(w)
            self.Gh.append(gr)
            w, gr = g.buffers(capi.FLOAT)
            self.Wf.append(w)
            self.Gf.append(gr)

    def set_weights(self, W_bits=None, Wf=None):
        for r, g in enumerate(self.groups):
            if W_bits is not None and g.n_half:
                self.Wh[r].view(torch.int16).copy_(dev_u16(W_bits[r], self.devices[r]))
            if Wf is not None and g.n_float:
                self.Wf[r].copy_(dev_f32(Wf[r], self.devices[r]))
        for r, g in enumerate(self.groups):
            g.init_master(stream_ptr(self.devices[r]))
        self.sync()

    def set_grads(self, G_bits=None, Gf=None):
        for r, g in enumerate(self.groups):
            if G_bits is not None and g.n_half:
                self.Gh[r].view(torch.int16).copy_(dev_u16(G_bits[r], self.devices[r]))
            if Gf is not None and g.n_float:
                self.Gf[r].copy_(dev_f32(Gf[r], self.devices[r]))
        self.sync()

    def sync(self):
        for d in set(self.devices):
            torch.cuda.synchronize(d)

    def step(self, lr, l2, scale):
        """Steps every rank (serially when they share a device) and returns rank 0's flag sums."""
        for r, g in enumerate(self.groups):
            g.exec(lr, l2, scale, stream_ptr(self.devices[r]))
        flags = [g.flags(stream_ptr(self.devices[r])) for r, g in enumerate(self.groups)]
        for f in flags[1:]:
            assert f == flags[0], f"ranks disagree on the flag sums: {flags}"
        return flags[0]

    def weights_half(self, r):
        return host_u16(self.Wh[r])

    def weights_float(self, r):
        return self.Wf[r].cpu().numpy().copy()

    def state(self, r, dtype, which):
        return self.groups[r].export_state(dtype, which)

    def close(self):
        self.Wh = self.Gh = self.Wf = self.Gf = None
        for g in self.groups:
            g.destroy()
