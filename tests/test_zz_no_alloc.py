"""mrl_mlp_forward_noalloc: the forward pass for hosts that cannot allocate device
memory (their own pool owns it all, or they must avoid the device-wide stall of
cudaMalloc/cudaFree).  Its scratch is a fixed array inside the library, so the
test checks that it gives exactly what mrl_mlp_forward gives with a caller
workspace - twice in a row, because the array keeps the previous call's bytes -
and that oversize requests are refused.  Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_forward_matches_workspace_forward_twice():
    import torch
    from _gpu import call, dev, host, stream
    from _util import NetSpec, xavier_params
    from mojo_rl_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(0)
    # two different shapes back to back: the second call finds the first call's activations in the array
    for (i, h, o, act, head), batch in (((8, 256, 4, 0, 0), 4096), ((17, 64, 6, 1, 1), 777)):
        spec = NetSpec(i, h, o, act, head)
        p = xavier_params(spec, rng)
        oc = o * (2 if head else 1)
        x = rng.standard_normal((batch, i)).astype(np.float32)
        xg, pg = dev(x), dev(p)
        cps = L.mrl_net_cache_per_sample(spec)
        ws = torch.zeros(L.mrl_mlp_workspace_floats(spec, batch), device="cuda")
        want, want_cache = torch.zeros(batch, oc, device="cuda"), torch.zeros(batch * cps, device="cuda")
        call("mrl_mlp_forward", spec, batch, xg, pg, want, want_cache, ws, stream())
        for _ in range(2):
            got, got_cache = torch.full((batch, oc), -7.0, device="cuda"), torch.zeros(batch * cps, device="cuda")
            call("mrl_mlp_forward_noalloc", spec, batch, xg, pg, got, got_cache, stream())
            torch.cuda.synchronize()
            assert np.array_equal(host(got), host(want))
            assert np.array_equal(host(got_cache), host(want_cache))
        got_nc = torch.zeros(batch, oc, device="cuda")
        call("mrl_mlp_forward_noalloc", spec, batch, xg, pg, got_nc, None, stream())
        assert np.array_equal(host(got_nc), host(want))


def test_noalloc_forward_rejects_oversize():
    import torch
    from mojo_rl_b200 import _lib
    from _util import NetSpec
    L = _lib.lib()
    spec = NetSpec(8, 256, 4, 0, 0)
    t = torch.zeros(16, device="cuda")
    rc = L.mrl_mlp_forward_noalloc(spec, 4097, _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), None, None)
    assert rc == -7 and b"exceeds the built-in scratch" in L.mrl_last_error_string()
    with pytest.raises(_lib.MojoRLError):
        _lib.check(rc)
