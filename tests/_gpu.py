"""GPU-side helpers for the parity tests: everything goes through the C ABI."""
import ctypes

import numpy as np
import torch

from mojo_rl_b200 import _lib

DEV = torch.device("cuda", 0)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def host(t):
    return t.detach().cpu().numpy()


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def call(fn_name, *args):
    L = _lib.lib()
    conv = [(_lib.ptr(a) if isinstance(a, torch.Tensor) else a) for a in args]
    _lib.check(getattr(L, fn_name)(*conv))


class GpuAgent:
    """mrl_ctx wrapper mirroring tests/_util.OracleAgent."""

    def __init__(self, cfg):
        self.L = _lib.lib()
        self.h = ctypes.c_void_p()
        _lib.check(self.L.mrl_create(ctypes.byref(self.h), ctypes.byref(cfg)))

    def close(self):
        if self.h:
            self.L.mrl_destroy(self.h)
            self.h = None

    def param_size(self, which):
        return self.L.mrl_param_size(self.h, which)

    def set_params(self, which, params, state=None):
        _lib.check(self.L.mrl_set_params(self.h, which, _lib.ptr(params), _lib.ptr(state)))

    def get_params(self, which):
        n = self.param_size(which)
        p, s = np.empty(n, np.float32), np.empty(2 * n, np.float32)
        _lib.check(self.L.mrl_get_params(self.h, which, _lib.ptr(p), _lib.ptr(s)))
        return p, s

    def sync(self):
        torch.cuda.synchronize()

    def buffer(self, which):
        p, n = ctypes.c_void_p(), ctypes.c_int64()
        _lib.check(self.L.mrl_get_buffer(self.h, which, ctypes.byref(p), ctypes.byref(n)))
        out = np.empty(n.value, np.float32)
        _lib.check(self.L.mrl_read_buffer(self.h, which, _lib.ptr(out), n.value))
        return out

    def write_buffer(self, which, arr):
        arr = np.ascontiguousarray(arr, np.float32)
        _lib.check(self.L.mrl_write_buffer(self.h, which, _lib.ptr(arr), arr.size))

    def stats(self):
        st = _lib.Stats()
        _lib.check(self.L.mrl_get_stats(self.h, ctypes.byref(st)))
        return st

    def reset(self, seed=0):
        _lib.check(self.L.mrl_ppo_reset(self.h, seed))

    def rollout(self):
        _lib.check(self.L.mrl_ppo_rollout(self.h))

    def gae(self):
        _lib.check(self.L.mrl_ppo_gae(self.h))

    def update(self, actor_lr, critic_lr, ent, perms=None):
        _lib.check(self.L.mrl_ppo_update(self.h, actor_lr, critic_lr, ent, _lib.ptr(perms)))

    def drain(self, cap=1 << 16):
        r, l = np.empty(cap, np.float32), np.empty(cap, np.float32)
        n = _lib.check(self.L.mrl_drain_episodes(self.h, _lib.ptr(r), _lib.ptr(l), cap))
        return r[:n].copy(), l[:n].copy()
