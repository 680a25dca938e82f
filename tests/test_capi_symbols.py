"""The C-ABI library loads without a GPU and exports every symbol that
include/mojorl_b200.h declares; host-only helpers answer without a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from mojo_rl_b200 import build, _lib
    build.build()
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "mojorl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mrl_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from mojo_rl_b200 import _lib
    names = _declared()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_host_only_helpers(lib):
    from mojo_rl_b200 import _lib
    vals = [ctypes.c_int() for _ in range(4)]
    assert lib.mrl_env_info(2, *[ctypes.byref(v) for v in vals]) == 0
    assert [v.value for v in vals] == [192, 8, 4, 0]
    assert lib.mrl_env_info(99, *[ctypes.byref(v) for v in vals]) < 0
    assert b"99" in lib.mrl_last_error_string()
    spec = _lib.NetSpec(8, 256, 4, 0, 0)
    assert lib.mrl_net_param_size(spec) == 69124      # LunarLander actor
    spec = _lib.NetSpec(8, 256, 1, 0, 0)
    assert lib.mrl_net_param_size(spec) == 68353      # LunarLander critic
    assert lib.mrl_net_cache_per_sample(spec) == 8 + 4 * 256
    cfg = _lib.Config()
    lib.mrl_config_defaults(ctypes.byref(cfg))
    assert cfg.num_epochs == 4 and abs(cfg.clip_epsilon - 0.2) < 1e-7 and cfg.gamma == 0.99


def test_create_without_gpu_fails_loudly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from mojo_rl_b200 import _lib
    cfg = _lib.Config()
    lib.mrl_config_defaults(ctypes.byref(cfg))
    h = ctypes.c_void_p()
    rc = lib.mrl_create(ctypes.byref(h), ctypes.byref(cfg))
    assert rc == -5 and b"no CPU path" in lib.mrl_last_error_string()
    with pytest.raises(_lib.MojoRLError):
        _lib.check(rc)
