"""Model / Optimizer / PPO-kernel parity through the C ABI."""
import ctypes

import numpy as np
import pytest

from _util import NetSpec, fp, ip, oracle, xavier_params

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dims", [(4, 64, 2), (8, 256, 4), (8, 256, 1), (17, 96, 6)])
@pytest.mark.parametrize("batch", [1, 50, 512])
def test_mlp_forward_backward(dims, batch):
    import torch
    from _gpu import call, dev, host, stream
    from mojo_rl_b200 import _lib
    o = oracle()
    rng = np.random.default_rng(batch + dims[1])
    for act, head in ((0, 0), (1, 0), (1, 1)):
        spec = NetSpec(dims[0], dims[1], dims[2], act, head)
        p = xavier_params(spec, rng)
        if head == 1:
            p[-dims[2]:] = rng.uniform(-6, 3, dims[2]).astype(np.float32)   # exercises the [-5, 2] clamp
        oc = dims[2] * (2 if head else 1)
        x = rng.standard_normal((batch, dims[0])).astype(np.float32)
        out_c = np.empty((batch, oc), np.float32)
        cps = o.orc_net_cache_per_sample(spec)
        cache_c = np.empty(batch * cps, np.float32)
        o.orc_mlp_forward(spec, batch, fp(x), fp(p), fp(out_c), fp(cache_c))
        L = _lib.lib()
        assert L.mrl_net_param_size(spec) == p.size and L.mrl_net_cache_per_sample(spec) == cps
        ws = torch.zeros(L.mrl_mlp_workspace_floats(spec, batch), device="cuda")
        out_g = torch.zeros(batch, oc, device="cuda")
        cache_g = torch.zeros(batch * cps, device="cuda")
        xg, pg = dev(x), dev(p)
        call("mrl_mlp_forward", spec, batch, xg, pg, out_g, cache_g, ws, stream())
        assert np.array_equal(host(out_g), out_c), "forward must be bit-identical (same fma chain)"
        assert np.array_equal(host(cache_g), cache_c)
        out_nc = torch.zeros(batch, oc, device="cuda")
        call("mrl_mlp_forward", spec, batch, xg, pg, out_nc, None, ws, stream())
        assert np.array_equal(host(out_nc), out_c)
        g = (rng.standard_normal((batch, oc)) / batch).astype(np.float32)
        grads_c, gin_c = np.empty_like(p), np.empty((batch, dims[0]), np.float32)
        o.orc_mlp_backward(spec, batch, fp(g), fp(p), fp(cache_c), fp(gin_c), fp(grads_c), 1)
        grads_g = torch.full((p.size,), 123.0, device="cuda")     # overwritten, not accumulated
        gin_g = torch.zeros(batch, dims[0], device="cuda")
        call("mrl_mlp_backward", spec, batch, dev(g), pg, cache_g, gin_g, grads_g, ws, stream())
        scale = np.abs(grads_c).max()
        assert np.allclose(host(grads_g), grads_c, rtol=1e-5, atol=1e-6 * max(scale, 1e-3))
        assert np.allclose(host(gin_g), gin_c, rtol=1e-5, atol=1e-7)


def test_adam_matches_oracle_bitwise():
    import torch
    from _gpu import call, dev, host, stream
    o = oracle()
    rng = np.random.default_rng(0)
    n = 70000
    p = rng.standard_normal(n).astype(np.float32); g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    s = np.abs(rng.standard_normal(2 * n) * 1e-3).astype(np.float32)
    pg, sg, gg = dev(p), dev(s), dev(g)
    for t in range(1, 4):
        b1, b2 = ctypes.c_float(), ctypes.c_float()
        o.orc_adam_bias_corrections(0.9, 0.999, t, ctypes.byref(b1), ctypes.byref(b2))
        o.orc_adam_step(n, fp(p), fp(g), fp(s), 3e-4, 0.9, 0.999, 1e-8, b1.value, b2.value)
        call("mrl_adam_step", n, pg, gg, sg, 3e-4, 0.9, 0.999, 1e-8, b1.value, b2.value, stream())
    assert np.array_equal(host(pg), p) and np.array_equal(host(sg), s)


def test_sampler_argmax_gae_bitwise():
    import torch
    from _gpu import call, dev, host, stream
    o = oracle()
    rng = np.random.default_rng(1)
    for n, A in ((1, 2), (8192, 4), (1000, 7)):
        logits = (rng.standard_normal((n, A)) * 2).astype(np.float32)
        logits[0] = 0.0                                         # ties
        a_c, lp_c = np.empty(n, np.float32), np.empty(n, np.float32)
        a_g, lp_g = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        for seed in (0, 0xdeadbeef):
            o.orc_sample_actions(n, A, fp(logits), fp(a_c), fp(lp_c), seed)
            call("mrl_sample_actions", n, A, dev(logits), a_g, lp_g, seed, stream())
            assert np.array_equal(host(a_g), a_c) and np.array_equal(host(lp_g), lp_c)
        o.orc_argmax_actions(n, A, fp(logits), fp(a_c))
        call("mrl_argmax_actions", n, A, dev(logits), a_g, stream())
        assert np.array_equal(host(a_g), a_c)
    for T, N in ((1, 1), (128, 1000), (37, 5)):
        r = rng.standard_normal((T, N)).astype(np.float32); v = rng.standard_normal((T, N)).astype(np.float32)
        d = (rng.random((T, N)) < 0.05).astype(np.float32); boot = rng.standard_normal(N).astype(np.float32)
        adv_c, ret_c = np.empty((T, N), np.float32), np.empty((T, N), np.float32)
        o.orc_gae(T, N, fp(r), fp(v), fp(d), fp(boot), 0.99, 0.95, fp(adv_c), fp(ret_c))
        adv_g, ret_g = torch.zeros(T, N, device="cuda"), torch.zeros(T, N, device="cuda")
        call("mrl_gae", T, N, dev(r), dev(v), dev(d), dev(boot), 0.99, 0.95, adv_g, ret_g, stream())
        assert np.array_equal(host(adv_g), adv_c) and np.array_equal(host(ret_g), ret_c)


def test_normalise_gather_grads_clip():
    import torch
    from _gpu import call, dev, host, stream
    o = oracle()
    rng = np.random.default_rng(2)
    for n in (1, 257, 1 << 20):
        x = (rng.standard_normal(n) * 3 + 1).astype(np.float32)
        xc = x.copy()
        o.orc_normalize_advantages(n, fp(xc), 1)
        xg = dev(x); scratch = torch.zeros(8, device="cuda")
        call("mrl_normalize_advantages", n, xg, scratch, stream())
        assert np.allclose(host(xg), xc, rtol=1e-5, atol=1e-6)
    # gather
    total, B, OBS = 5000, 777, 8
    idx = rng.permutation(total)[:B].astype(np.int32)
    src = [rng.standard_normal((total, OBS)).astype(np.float32)] + [rng.standard_normal(total).astype(np.float32) for _ in range(5)]
    outs = [torch.zeros(B, OBS, device="cuda")] + [torch.zeros(B, device="cuda") for _ in range(5)]
    call("mrl_ppo_gather_minibatch", B, OBS, dev(idx), *[dev(s) for s in src], *outs, stream())
    for s, og in zip(src, outs):
        assert np.array_equal(host(og), s[idx])
    # actor / critic loss gradients: bit-identical
    Bn, A = 4096, 4
    logits = rng.standard_normal((Bn, A)).astype(np.float32); act = rng.integers(0, A, Bn).astype(np.float32)
    adv = rng.standard_normal(Bn).astype(np.float32); old_lp = (-1.4 + 0.4 * rng.standard_normal(Bn)).astype(np.float32)
    g_c, kl_c = np.empty((Bn, A), np.float32), np.empty(Bn, np.float32)
    o.orc_ppo_actor_grad(Bn, A, fp(logits), fp(old_lp), fp(adv), fp(act), 0.2, 0.01, fp(g_c), fp(kl_c))
    g_g, kl_g = torch.zeros(Bn, A, device="cuda"), torch.zeros(Bn, device="cuda")
    call("mrl_ppo_actor_grad", Bn, A, dev(logits), dev(old_lp), dev(adv), dev(act), 0.2, 0.01, g_g, kl_g, stream())
    assert np.array_equal(host(g_g), g_c) and np.array_equal(host(kl_g), kl_c)
    v = rng.standard_normal(Bn).astype(np.float32); vo = (v + 0.3 * rng.standard_normal(Bn)).astype(np.float32)
    ret = rng.standard_normal(Bn).astype(np.float32)
    for clip in (0, 1):
        gv_c = np.empty(Bn, np.float32)
        o.orc_ppo_critic_grad(Bn, fp(v), fp(vo), fp(ret), 0.5, 0.2, clip, fp(gv_c))
        gv_g = torch.zeros(Bn, device="cuda")
        call("mrl_ppo_critic_grad", Bn, dev(v), dev(vo), dev(ret), 0.5, 0.2, clip, gv_g, stream())
        assert np.array_equal(host(gv_g), gv_c)
    # gradient clipping
    for scale in (1e-4, 1.0):
        g = (rng.standard_normal(69124) * scale).astype(np.float32)
        gc = g.copy()
        norm = o.orc_grad_clip(g.size, fp(gc), 0.5, 1)
        gg = dev(g); scratch = torch.zeros(8, device="cuda")
        call("mrl_grad_clip", g.size, gg, 0.5, scratch, stream())
        assert np.allclose(host(gg), gc, rtol=1e-6, atol=1e-12)
        assert abs(np.sqrt(host(scratch)[0]) - norm) < 1e-5 * max(norm, 1.0)


def test_gaussian_policy_kernels_bitwise():
    """Sampler, loss gradients and log_std clamp of the continuous agent: the same IEEE operations as the
    oracle, so equality; the reward statistics reduce in a different order, so closeness."""
    import torch
    from _gpu import call, dev, host, stream
    o = oracle()
    rng = np.random.default_rng(4)
    for n, A in ((1, 1), (4096, 1), (1000, 6), (33, 16)):
        out = rng.standard_normal((n, 2 * A)).astype(np.float32)
        out[:, A:] *= 3.0                                   # log_std beyond [-5, 2] on some rows
        a_c, lp_c = np.empty((n, A), np.float32), np.empty(n, np.float32)
        a_g, lp_g = torch.zeros(n, A, device="cuda"), torch.zeros(n, device="cuda")
        for seed, greedy in ((0, 0), (0xdeadbeef, 0), (7, 1)):
            o.orc_sample_continuous_actions(n, A, fp(out), fp(a_c), fp(lp_c), seed, greedy)
            call("mrl_sample_continuous_actions", n, A, dev(out), a_g, lp_g, seed, greedy, stream())
            assert np.array_equal(host(a_g), a_c) and np.array_equal(host(lp_g), lp_c)
        adv = rng.standard_normal(n).astype(np.float32)
        old_lp = (lp_c + 0.2 * rng.standard_normal(n)).astype(np.float32)
        g_c, kl_c = np.empty((n, 2 * A), np.float32), np.empty(n, np.float32)
        o.orc_ppo_continuous_actor_grad(n, A, fp(out), fp(old_lp), fp(adv), fp(a_c), 0.2, 0.01, fp(g_c), fp(kl_c))
        g_g, kl_g = torch.zeros(n, 2 * A, device="cuda"), torch.zeros(n, device="cuda")
        call("mrl_ppo_continuous_actor_grad", n, A, dev(out), dev(old_lp), dev(adv), dev(a_c), 0.2, 0.01, g_g, kl_g,
             stream())
        assert np.array_equal(host(g_g), g_c) and np.array_equal(host(kl_g), kl_c)
        assert (g_c == 0).all(1).sum() > 0 or n < 10          # the clipped branch was taken
    Bn = 4096
    v = rng.standard_normal(Bn).astype(np.float32); vo = (v + 0.3 * rng.standard_normal(Bn)).astype(np.float32)
    ret = rng.standard_normal(Bn).astype(np.float32)
    for clip in (0, 1):
        gv_c = np.empty(Bn, np.float32)
        o.orc_ppo_continuous_critic_grad(Bn, fp(v), fp(vo), fp(ret), 0.2, clip, fp(gv_c))
        gv_g = torch.zeros(Bn, device="cuda")
        call("mrl_ppo_continuous_critic_grad", Bn, dev(v), dev(vo), dev(ret), 0.2, clip, gv_g, stream())
        assert np.array_equal(host(gv_g), gv_c)
    ls = dev(np.array([-7.0, -5.0, 0.3, 2.0, 2.5, -4.9], np.float32))
    call("mrl_clamp_log_std", 6, ls, stream())
    assert np.array_equal(host(ls), np.array([-5.0, -5.0, 0.3, 2.0, 2.0, -4.9], np.float32))
    # wide gather
    total, B, OBS, A = 3000, 500, 3, 6
    idx = rng.permutation(total)[:B].astype(np.int32)
    src = [rng.standard_normal((total, OBS)).astype(np.float32), rng.standard_normal((total, A)).astype(np.float32)] + \
          [rng.standard_normal(total).astype(np.float32) for _ in range(4)]
    outs = [torch.zeros(B, OBS, device="cuda"), torch.zeros(B, A, device="cuda")] + \
           [torch.zeros(B, device="cuda") for _ in range(4)]
    call("mrl_ppo_gather_minibatch_continuous", B, OBS, A, dev(idx), *[dev(x) for x in src], *outs, stream())
    for x, og in zip(src, outs):
        assert np.array_equal(host(og), x[idx])
    # reward statistics over three rollouts, then the f64-sqrt advantage normalisation
    st_c = np.zeros(3, np.float64)
    st_g = torch.zeros(3, dtype=torch.float64, device="cuda"); scr = torch.zeros(2, dtype=torch.float64, device="cuda")
    for k in range(3):
        r = (rng.standard_normal(1 << 16) * (k + 1) - 4.0).astype(np.float32)
        out_c = np.empty_like(r)
        o.orc_rms_update_normalize(st_c.ctypes.data_as(ctypes.POINTER(ctypes.c_double)), fp(r), fp(out_c), r.size)
        out_g = torch.zeros(r.size, device="cuda")
        call("mrl_reward_rms_update_normalize", r.size, dev(r), out_g, st_g, scr, stream())
        assert np.allclose(st_g.cpu().numpy(), st_c, rtol=1e-12)
        assert np.allclose(host(out_g), out_c, rtol=1e-6, atol=1e-6)
    x = (rng.standard_normal(100000) * 3 + 1).astype(np.float32)
    xg = dev(x); scratch = torch.zeros(8, device="cuda")
    call("mrl_normalize_advantages_f64sqrt", x.size, xg, scratch, stream())
    assert abs(host(xg).mean()) < 1e-5 and abs(host(xg).std() - 1.0) < 1e-4


@pytest.mark.parametrize("case", [("actor", 4, 2, 0, 0), ("critic", 4, 1, 0, 0), ("gauss", 3, 1, 1, 1),
                                  ("critic_c", 3, 1, 1, 0), ("actor", 8, 4, 0, 0), ("gauss", 8, 4, 1, 1)])
@pytest.mark.parametrize("batch", [1, 200, 4096 + 37])
def test_fused_train_step_matches_layerwise_oracle(case, batch):
    """Forward + loss gradient + backward in one kernel against the oracle's layer-by-layer functions."""
    import torch
    from _gpu import call, dev, host, stream
    from mojo_rl_b200 import _lib
    kind, I, O, act, head = case
    o = oracle()
    L = _lib.lib()
    rng = np.random.default_rng(batch + I + O)
    spec = NetSpec(I, 64, O, act, head)
    p = xavier_params(spec, rng) * 2
    if head == 1:
        p[-O:] = rng.uniform(-1.0, 0.5, O).astype(np.float32)
    oc = O * (2 if head else 1)
    x = rng.standard_normal((batch, I)).astype(np.float32)
    out = np.empty((batch, oc), np.float32)
    cache = np.empty(batch * o.orc_net_cache_per_sample(spec), np.float32)
    o.orc_mlp_forward(spec, batch, fp(x), fp(p), fp(out), fp(cache))
    adv = rng.standard_normal(batch).astype(np.float32)
    ret = rng.standard_normal(batch).astype(np.float32)
    old_v = (out[:, 0] + 0.3 * rng.standard_normal(batch)).astype(np.float32)
    g_out, kl = np.zeros((batch, oc), np.float32), np.zeros(batch, np.float32)
    if kind == "actor":
        actions = rng.integers(0, O, batch).astype(np.float32)
        lp = out - out.max(1, keepdims=True)
        lp = lp - np.log(np.exp(lp).sum(1, keepdims=True))
        old_lp = (lp[np.arange(batch), actions.astype(int)] + 0.15 * rng.standard_normal(batch)).astype(np.float32)
        o.orc_ppo_actor_grad(batch, O, fp(out), fp(old_lp), fp(adv), fp(actions), 0.2, 0.01, fp(g_out), fp(kl))
        mode = 0
    elif kind == "gauss":
        actions = (out[:, :O] + np.exp(out[:, O:]) * rng.standard_normal((batch, O))).astype(np.float32)
        z = (actions - out[:, :O]) / np.exp(out[:, O:])
        old_lp = ((-0.5 * (1.8378770664093453 + 2 * out[:, O:] + z * z)).sum(1)
                  + 0.15 * rng.standard_normal(batch)).astype(np.float32)
        o.orc_ppo_continuous_actor_grad(batch, O, fp(out), fp(old_lp), fp(adv), fp(actions), 0.2, 0.01, fp(g_out),
                                        fp(kl))
        mode = 1
    elif kind == "critic":
        actions, old_lp = np.zeros(batch, np.float32), np.zeros(batch, np.float32)
        o.orc_ppo_critic_grad(batch, fp(out.reshape(-1).copy()), fp(old_v), fp(ret), 0.5, 0.2, 1, fp(g_out.reshape(-1)))
        mode = 2
    else:
        actions, old_lp = np.zeros(batch, np.float32), np.zeros(batch, np.float32)
        o.orc_ppo_continuous_critic_grad(batch, fp(out.reshape(-1).copy()), fp(old_v), fp(ret), 0.2, 1,
                                         fp(g_out.reshape(-1)))
        mode = 3
    grads_c, gin = np.empty_like(p), np.empty((batch, I), np.float32)
    o.orc_mlp_backward(spec, batch, fp(g_out), fp(p), fp(cache), fp(gin), fp(grads_c), 1)
    n_scr = L.mrl_fused_train_scratch_doubles(spec, batch)
    assert n_scr > 0
    scratch = torch.zeros(n_scr, dtype=torch.float64, device="cuda")
    grads_g = torch.full((p.size,), 7.0, device="cuda")
    kl_g = torch.zeros(1, device="cuda")
    call("mrl_fused_train_step", spec, mode, batch, dev(p), dev(x), dev(actions), dev(adv), dev(ret), dev(old_lp),
         dev(old_v), 0.2, 0.01, 0.5, 1, scratch, grads_g, kl_g, stream())
    scale = max(float(np.abs(grads_c).max()), 1e-6)
    assert np.allclose(host(grads_g), grads_c, rtol=2e-5, atol=2e-6 * scale), np.abs(host(grads_g) - grads_c).max() / scale
    if mode < 2:
        assert abs(float(kl_g.item()) - float(kl.astype(np.float64).sum())) <= 1e-5 * max(1.0, abs(float(kl.sum())))
    assert L.mrl_fused_train_scratch_doubles(NetSpec(24, 64, 4, 0, 0), batch) == -1


def test_add_obs_noise_matches_oracle():
    import torch
    from mojo_rl_b200 import _lib
    L, o = _lib.lib(), oracle()
    n, d = 1000, 24
    rng = np.random.default_rng(5)
    obs = rng.standard_normal((n, d)).astype(np.float32)
    want = obs.copy()
    o.orc_add_obs_noise(n, d, fp(want), 0.05, 99)
    t = torch.from_numpy(obs).cuda()
    _lib.check(L.mrl_add_obs_noise(n, d, t.data_ptr(), 0.05, 99, None))
    torch.cuda.synchronize()
    assert np.array_equal(t.cpu().numpy(), want)
