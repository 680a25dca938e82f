"""bf16 tcgen05 kernels of the precision-1 update: the two GEMM building blocks
against an fp32 matmul of the same bf16 operands, and one whole PPO update in
precision 1 against precision 0 (the bit-checked fp32 path)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _err_flag():
    import torch
    return torch.zeros(4, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("M", [128, 300, 4096, 60000])
def test_rowtile_gemm(M):
    import torch
    from _gpu import call, stream
    torch.manual_seed(M)
    A = torch.randn(M, 256, device="cuda").to(torch.bfloat16)
    B = (torch.randn(256, 256, device="cuda") / 16).to(torch.bfloat16)
    D = torch.full((M, 256), float("nan"), device="cuda")
    err = _err_flag()
    call("mrl_bf16_rowtile_gemm", M, A, B, D, err, stream())
    torch.cuda.synchronize()
    assert int(err[0]) == 0
    want = A.float() @ B.float().t()
    assert torch.isfinite(D).all()
    assert torch.allclose(D, want, rtol=1e-4, atol=1e-4), float((D - want).abs().max())


@pytest.mark.parametrize("K", [64, 640, 9472, 262144])
def test_splitk_gemm(K):
    import torch
    from _gpu import call, stream
    from mojo_rl_b200 import _lib
    torch.manual_seed(K)
    A = torch.randn(256, K, device="cuda").to(torch.bfloat16)
    B = (torch.randn(256, K, device="cuda") / 16).to(torch.bfloat16)
    ms = _lib.lib().mrl_bf16_max_splits()
    part = torch.full((ms, 256, 256), float("nan"), device="cuda")
    err = _err_flag()
    splits = ctypes.c_int(0)
    _lib.check(_lib.lib().mrl_bf16_splitk_gemm(K, _lib.ptr(A), _lib.ptr(B), _lib.ptr(part), ctypes.byref(splits),
                                               _lib.ptr(err), stream()))
    torch.cuda.synchronize()
    assert int(err[0]) == 0 and 1 <= splits.value <= ms
    got = part[:splits.value].sum(0)
    want = A.float() @ B.float().t()
    scale = float(want.abs().max())
    assert torch.allclose(got, want, rtol=1e-3, atol=1e-4 * scale), float((got - want).abs().max())


@pytest.mark.parametrize("K", [64, 704, 262144])
def test_splitk_gemm_from_row_major_activations(K):
    import torch
    from _gpu import stream
    from mojo_rl_b200 import _lib
    torch.manual_seed(K + 1)
    X = torch.randn(K, 256, device="cuda").to(torch.bfloat16)
    G = (torch.randn(K, 256, device="cuda") / 16).to(torch.bfloat16)
    ms = _lib.lib().mrl_bf16_max_splits()
    part = torch.full((ms, 256, 256), float("nan"), device="cuda")
    err = _err_flag()
    splits = ctypes.c_int(0)
    _lib.check(_lib.lib().mrl_bf16_splitk_gemm_tn(K, _lib.ptr(X), _lib.ptr(G), _lib.ptr(part), ctypes.byref(splits),
                                                  _lib.ptr(err), stream()))
    torch.cuda.synchronize()
    assert int(err[0]) == 0 and 1 <= splits.value <= ms
    got = part[:splits.value].sum(0)
    want = X.float().t() @ G.float()
    scale = float(want.abs().max())
    assert torch.allclose(got, want, rtol=1e-3, atol=1e-4 * scale), float((got - want).abs().max())


@pytest.mark.parametrize("kind,obs,out,act,head,hidden", [(2, 8, 4, 0, 0, 256), (3, 24, 4, 1, 1, 256),
                                                            (4, 17, 6, 1, 1, 512), (2, 8, 4, 0, 0, 512)])
def test_update_precision1_matches_fp32_gradients(kind, obs, out, act, head, hidden):
    """Same rollout (the fp32 context's slab and GAE results are written into the bf16 context, whose
    own rollout policy runs on tensor cores), same permutation, one minibatch: the bf16 tensor-core update's
    gradients agree with the fp32 path to bf16 accuracy, and training state advances.
    LunarLander: ReLU nets, categorical head; BipedalWalker: tanh nets, Gaussian head; HalfCheetah: hidden
    width 512, computed in 256-wide tensor-core blocks."""
    from _gpu import GpuAgent
    from _util import NetSpec, default_config, xavier_params
    rng = np.random.default_rng(0)
    pa = xavier_params(NetSpec(obs, hidden, out, act, head), rng) * (3 if head == 0 else 1)
    pc = xavier_params(NetSpec(obs, hidden, 1, act, 0), rng)
    if head == 1:
        pa[-out:] = -0.5
    total = 256 * 32
    perms = rng.permutation(total).astype(np.int32)[None]
    grads = {}
    params = {}
    for prec in (0, 1):
        cfg = default_config(env_kind=kind, n_envs=256, rollout_len=32, hidden_dim=hidden, minibatch_size=total,
                             num_epochs=1, target_kl=0.0, precision=prec, max_grad_norm=0.0)
        g = GpuAgent(cfg)
        try:
            g.set_params(0, pa, np.zeros(2 * pa.size, np.float32))
            g.set_params(1, pc, np.zeros(2 * pc.size, np.float32))
            g.reset(0); g.rollout(); g.gae()
            if prec == 0:
                slab = {i: g.buffer(i) for i in (2, 3, 4, 5, 6, 7, 8, 9)}
            else:
                for i, arr in slab.items():
                    g.write_buffer(i, arr)
            g.update(3e-4, 1e-3, 0.01, perms)
            st = g.stats()
            assert st.minibatches_done == 1 and st.actor_adam_t == 1
            grads[prec] = (g.buffer(12), g.buffer(13))
            params[prec] = (g.get_params(0)[0], g.get_params(1)[0])
        finally:
            g.close()
    for which in (0, 1):
        a, b = grads[1][which], grads[0][which]
        assert np.isfinite(a).all()
        denom = np.abs(b).max()
        # bf16 rounding of 256 (512) products per sum: 3 % (5 %) of the largest entry
        assert np.abs(a - b).max() <= (3e-2 if hidden == 256 else 5e-2) * denom, (which, np.abs(a - b).max(), denom)
        # cosine similarity of the whole gradient
        cos = float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))
        assert cos > 0.999, (which, cos)
        assert not np.array_equal(params[1][which], pa if which == 0 else pc)


def test_precision1_rejects_unsupported_shapes():
    from mojo_rl_b200 import _lib
    from _util import default_config
    L = _lib.lib()
    cfg = default_config(env_kind=2, n_envs=256, rollout_len=32, hidden_dim=64, minibatch_size=1024, precision=1)
    h = ctypes.c_void_p()
    assert L.mrl_create(ctypes.byref(h), ctypes.byref(cfg)) == -4
    assert b"precision 1" in L.mrl_last_error_string()


def test_rollout_policy_kernel_matches_fp32_policy():
    """One rollout step: the tensor-core policy kernel (precision 1) against the fp32 forward +
    sampler (precision 0) on the same observations, parameters and seeds."""
    from _gpu import GpuAgent
    from _util import NetSpec, default_config, xavier_params
    rng = np.random.default_rng(1)
    # moderate weights: with the reference's whole-model Xavier range the 256-term sums cancel
    # almost completely and bf16 rounding of the operands dominates the (tiny) result
    pa = xavier_params(NetSpec(8, 256, 4, 0, 0), rng) * 0.25
    pc = xavier_params(NetSpec(8, 256, 1, 0, 0), rng) * 0.25
    out = {}
    for prec in (0, 1):
        for det in (0, 1):
            cfg = default_config(env_kind=2, n_envs=1024, rollout_len=2, hidden_dim=256, minibatch_size=2048,
                                 num_epochs=1, precision=prec, deterministic=det)
            g = GpuAgent(cfg)
            try:
                g.set_params(0, pa, np.zeros(2 * pa.size, np.float32))
                g.set_params(1, pc, np.zeros(2 * pc.size, np.float32))
                g.reset(3); g.rollout()
                out[(prec, det)] = {k: g.buffer(i)[:1024 * (8 if k == "obs" else 1)] for k, i in
                                    (("obs", 2), ("act", 3), ("lp", 4), ("val", 5))}
                assert g.stats().total_steps == 2048
            finally:
                g.close()
    for det in (0, 1):
        a, b = out[(1, det)], out[(0, det)]
        assert np.array_equal(a["obs"], b["obs"])                      # step 0 observations are the reset's
        assert np.allclose(a["val"], b["val"], rtol=2e-2, atol=2e-2), np.abs(a["val"] - b["val"]).max()
        agree = (a["act"] == b["act"])
        assert agree.mean() > 0.97, agree.mean()
        assert np.allclose(a["lp"][agree], b["lp"][agree], rtol=0, atol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("kind,obs_dim,A,hidden", [(3, 24, 4, 256), (4, 17, 6, 512)])
def test_rollout_policy_kernel_gaussian_matches_fp32_policy(kind, obs_dim, A, hidden):
    """Same comparison for a tanh / Gaussian policy (state-independent log_std): actions differ from the fp32
    path only through the bf16 means, the noise draws are identical.  BipedalWalker (24 observations, 4 means,
    hidden 256) runs the single policy kernel; HalfCheetah (17, 6, hidden 512) runs the update path's
    tensor-core forward kernels at batch n_envs followed by the fp32 sampler."""
    from _gpu import GpuAgent
    from _util import NetSpec, default_config, xavier_params
    rng = np.random.default_rng(2)
    pa = xavier_params(NetSpec(obs_dim, hidden, A, 1, 1), rng) * 0.25
    pa[-A:] = np.linspace(-1.0, 0.3, A).astype(np.float32)   # log_std
    pc = xavier_params(NetSpec(obs_dim, hidden, 1, 1, 0), rng) * 0.25
    n = 512
    out = {}
    for prec in (0, 1):
        for det in (0, 1):
            cfg = default_config(env_kind=kind, n_envs=n, rollout_len=2, hidden_dim=hidden, minibatch_size=2 * n,
                                 num_epochs=1, precision=prec, deterministic=det)
            g = GpuAgent(cfg)
            try:
                g.set_params(0, pa, np.zeros(2 * pa.size, np.float32))
                g.set_params(1, pc, np.zeros(2 * pc.size, np.float32))
                g.reset(5); g.rollout()
                out[(prec, det)] = {k: g.buffer(i)[:n * w] for k, i, w in
                                    (("obs", 2, obs_dim), ("act", 3, A), ("lp", 4, 1), ("val", 5, 1))}
                assert g.stats().total_steps == 2 * n
            finally:
                g.close()
    for det in (0, 1):
        a, b = out[(1, det)], out[(0, det)]
        assert np.array_equal(a["obs"], b["obs"])
        assert np.allclose(a["val"], b["val"], rtol=2e-2, atol=2e-2), np.abs(a["val"] - b["val"]).max()
        assert np.allclose(a["act"], b["act"], rtol=0, atol=3e-2), np.abs(a["act"] - b["act"]).max()
        # log-prob depends on the noise only (action - mean = std * noise in both paths)
        assert np.allclose(a["lp"], b["lp"], rtol=0, atol=1e-3), np.abs(a["lp"] - b["lp"]).max()


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_reports_timeout():
    """The waits of the tensor-core kernels are bounded: a wait on a barrier nothing completes gives up after its
    poll limit, the kernel returns, the host sees MRL_ERR_TIMEOUT (-6), and the context keeps working."""
    from mojo_rl_b200 import _lib
    L = _lib.lib()
    assert L.mrl_debug_bounded_wait(4096, None) == -6
    assert b"gave up waiting" in L.mrl_last_error_string()
    # the device is still usable: a real tensor-core GEMM right after
    test_rowtile_gemm(256)
