"""CPU checks of the oracle's Gaussian-policy path and PendulumV2 against
closed forms and float64 numpy restatements of the reference formulas
(deep_agents/ppo/kernels.mojo, core/utils/normalization.mojo,
envs/pendulum/pendulum_v2.mojo)."""
import ctypes

import numpy as np

from _util import NetSpec, OracleAgent, default_config, fp, ip, oracle, xavier_params

PENDULUM = 1
LOG_2PI = 1.8378770664093453


def _env(n, seed=0):
    o = oracle()
    s = np.zeros((n, 8), np.float32)
    o.orc_env_reset(PENDULUM, n, fp(s), seed)
    return s


def _step(s, a):
    o = oracle()
    n = s.shape[0]
    r, d, ob = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros((n, 3), np.float32)
    o.orc_env_step(PENDULUM, n, fp(s), fp(np.ascontiguousarray(a, np.float32)), fp(r), fp(d), fp(ob), 0)
    return r, d, ob


def test_pendulum_dims_and_reset_ranges():
    o = oracle()
    dims = [ctypes.c_int() for _ in range(4)]
    assert o.orc_env_info(PENDULUM, *[ctypes.byref(x) for x in dims]) == 0
    assert [x.value for x in dims] == [8, 3, 0, 1]  # constants.mojo:12-60
    s = _env(4096, seed=7)
    theta, theta_dot = s[:, 3], s[:, 2]
    assert np.all(np.abs(theta) <= np.pi + 1e-6) and np.all(np.abs(theta_dot) <= 1.0)
    assert theta.std() > 1.5 and theta_dot.std() > 0.5          # uniform on [-pi, pi] / [-1, 1]
    assert np.allclose(s[:, 0], np.cos(theta), atol=1e-6) and np.allclose(s[:, 1], np.sin(theta), atol=1e-6)
    assert np.all(s[:, 4:] == 0)
    # a different seed gives different states; the same seed the same ones
    assert not np.array_equal(s, _env(4096, seed=8)) and np.array_equal(s, _env(4096, seed=7))


def test_pendulum_step_matches_closed_form():
    rng = np.random.default_rng(0)
    n = 512
    s = np.zeros((n, 8), np.float32)
    theta = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
    theta_dot = rng.uniform(-8, 8, n).astype(np.float32)
    s[:, 3], s[:, 2] = theta, theta_dot
    a = rng.uniform(-1.5, 1.5, n).astype(np.float32)  # beyond +-1: the torque clamp is exercised
    r, d, ob = _step(s, a)
    u = np.clip(a.astype(np.float64) * 2.0, -2.0, 2.0)
    acc = 15.0 * np.sin(theta.astype(np.float64)) + 3.0 * u      # 3g/(2l) sin + 3/(ml^2) u
    nd = theta_dot + acc * 0.05
    nt = theta + nd * 0.05                                        # angle uses the unclipped velocity
    nd = np.clip(nd, -8.0, 8.0)
    nt = (nt + np.pi) % (2 * np.pi) - np.pi
    assert np.allclose(s[:, 2], nd, atol=1e-5)
    assert np.allclose(np.cos(s[:, 3]), np.cos(nt), atol=1e-5) and np.allclose(np.sin(s[:, 3]), np.sin(nt), atol=1e-5)
    assert np.allclose(r, -(nt ** 2 + 0.1 * nd ** 2 + 0.001 * u ** 2), rtol=1e-4, atol=1e-4)
    assert np.array_equal(ob, s[:, :3]) and np.all(d == 0) and np.all(s[:, 4] == 1)
    assert np.allclose(s[:, 7], u, atol=1e-6) and np.allclose(s[:, 6], r)


def test_pendulum_upright_fixed_point_and_truncation():
    s = np.zeros((1, 8), np.float32)
    s[0, 0] = 1.0
    for t in range(200):
        r, d, _ = _step(s, np.zeros(1, np.float32))
        assert r[0] == 0.0 and s[0, 3] == 0.0
        assert d[0] == (1.0 if t == 199 else 0.0)   # MAX_STEPS = 200 is the only termination
    assert s[0, 4] == 200 and s[0, 5] == 1.0


def test_pendulum_selective_reset_clears_done_flags():
    o = oracle()
    s = _env(8, seed=1)
    before = s.copy()
    dones = np.array([0, 1, 0, 0, 1, 0, 0, 0], np.float32)
    s[:, 4] = 17
    o.orc_env_selective_reset(PENDULUM, 8, fp(s), fp(dones), 99)
    assert np.all(dones == 0)                       # pendulum_v2.mojo:381-392
    for i in range(8):
        if i in (1, 4):
            assert s[i, 4] == 0 and not np.array_equal(s[i, :4], before[i, :4])
        else:
            assert s[i, 4] == 17 and np.array_equal(s[i, :4], before[i, :4])


def _sample(out, A, seed, greedy):
    o = oracle()
    n = out.shape[0]
    act, lp = np.zeros((n, A), np.float32), np.zeros(n, np.float32)
    o.orc_sample_continuous_actions(n, A, fp(out), fp(act), fp(lp), seed, greedy)
    return act, lp


def test_gaussian_sampler_statistics_and_log_prob():
    rng = np.random.default_rng(1)
    n, A = 20000, 3
    out = np.zeros((n, 2 * A), np.float32)
    out[:, :A] = rng.normal(size=(n, A))
    out[:, A:] = np.array([-0.5, 0.3, 5.0], np.float32)   # the last one is clamped to 2
    act, lp = _sample(out, A, 1234, 0)
    ls = np.clip(out[:, A:].astype(np.float64), -5, 2)
    std = np.exp(ls)
    z = (act - out[:, :A]) / std
    assert abs(z.mean()) < 0.02 and abs(z.std() - 1.0) < 0.02      # Box-Muller noise is N(0, 1)
    assert abs(np.corrcoef(z[:, 0], z[:, 1])[0, 1]) < 0.03          # independent streams per (env, dim)
    ref = (-0.5 * (LOG_2PI + 2 * ls + ((act - out[:, :A]) / (std + 1e-6)) ** 2)).sum(1)
    assert np.allclose(lp, ref, rtol=1e-4, atol=1e-4)
    g_act, g_lp = _sample(out, A, 1234, 1)
    assert np.array_equal(g_act, out[:, :A])                         # greedy: the mean
    assert np.allclose(g_lp, (-0.5 * (LOG_2PI + 2 * ls)).sum(1), rtol=1e-5, atol=1e-5)
    act2, _ = _sample(out, A, 1235, 0)
    assert not np.array_equal(act, act2)
    # seed + i * A + j: env i, dim j with seed s draws what env 0, dim 0 draws with seed s + i * A + j
    one, _ = _sample(out[:1] * 0, A, 1234 + 5 * A + 2, 0)
    many, _ = _sample(out * 0, A, 1234, 0)
    assert many[5, 2] == one[0, 0]


def _actor_grad(out, old_lp, adv, act, clip_eps, ent):
    o = oracle()
    B, A = act.shape
    g, kl = np.zeros((B, 2 * A), np.float32), np.zeros(B, np.float32)
    o.orc_ppo_continuous_actor_grad(B, A, fp(out), fp(old_lp), fp(adv), fp(act), clip_eps, ent, fp(g), fp(kl))
    return g, kl


def test_gaussian_actor_grad_matches_float64_restatement():
    rng = np.random.default_rng(2)
    B, A = 256, 2
    out = rng.normal(size=(B, 2 * A)).astype(np.float32) * 0.5
    act = (out[:, :A] + rng.normal(size=(B, A)) * 0.7).astype(np.float32)
    adv = rng.normal(size=B).astype(np.float32)
    ls = out[:, A:].astype(np.float64)
    std = np.exp(ls)
    an = (act - out[:, :A]) / (std + 1e-6)
    new_lp = (-0.5 * (LOG_2PI + 2 * ls + an ** 2)).sum(1)
    old_lp = (new_lp + rng.normal(size=B) * 0.15).astype(np.float32)
    g, kl = _actor_grad(out, old_lp, adv, act, 0.2, 0.01)
    diff = np.clip(new_lp - old_lp, -20, 20)
    ratio = np.exp(diff)
    assert np.allclose(kl, np.clip(ratio - 1 - diff, 0, 100), atol=2e-5)
    clipped = np.clip(ratio, 0.8, 1.2) * adv < ratio * adv
    margin = np.abs(np.clip(ratio, 0.8, 1.2) - ratio) > 1e-4   # away from the float tie
    assert 10 < clipped.sum() < B - 10
    gm = np.clip(-adv[:, None] * ratio[:, None] * an / (std + 1e-6) / B, -10, 10)
    gs = np.clip((-adv[:, None] * ratio[:, None] * (an ** 2 - 1) - 0.01) / B, -10, 10)
    gm[clipped] = 0
    gs[clipped] = 0
    ok = margin | ~clipped
    assert np.allclose(g[ok, :A], gm[ok], rtol=1e-3, atol=1e-6) and np.allclose(g[ok, A:], gs[ok], rtol=1e-3, atol=1e-6)
    # zero gradient exactly where the clipped objective is the smaller one
    assert np.all(g[clipped & margin] == 0)


def test_gaussian_critic_grad_cases():
    o = oracle()
    v = np.array([1.0, 1.0, 1.5, 0.5, 1.05], np.float32)
    old = np.array([1.0, 1.0, 1.0, 1.0, 1.0], np.float32)
    ret = np.array([2.0, 0.0, 3.0, 0.9, 1.2], np.float32)
    g = np.zeros(5, np.float32)
    o.orc_ppo_continuous_critic_grad(5, fp(v), fp(old), fp(ret), 0.2, 0, fp(g))
    assert np.allclose(g, (v - ret) / 5)                                # kernels.mojo:416-438
    o.orc_ppo_continuous_critic_grad(5, fp(v), fp(old), fp(ret), 0.2, 1, fp(g))
    # row 2: clipped value 1.2 is farther from 3.0 -> clipped loss is larger and the value moved out of the band -> 0
    # row 3: clipped value 0.8, target 0.9: clipped loss (0.01) < unclipped (0.16) -> plain gradient
    assert np.allclose(g, [(1 - 2) / 5, (1 - 0) / 5, 0.0, (0.5 - 0.9) / 5, (1.05 - 1.2) / 5], atol=1e-7)


def test_running_mean_std_matches_concatenated_population_moments():
    o = oracle()
    rng = np.random.default_rng(3)
    batches = [rng.normal(-3, 5, 1000).astype(np.float32), rng.normal(2, 1, 300).astype(np.float32),
               rng.normal(0, 9, 4096).astype(np.float32)]
    st = np.zeros(3, np.float64)
    seen = []
    for b in batches:
        out = np.zeros_like(b)
        o.orc_rms_update_normalize(st.ctypes.data_as(ctypes.POINTER(ctypes.c_double)), fp(b), fp(out), b.size)
        seen.append(b.astype(np.float64))
        allv = np.concatenate(seen)
        assert st[0] == allv.size and abs(st[1] - allv.mean()) < 1e-9
        assert abs(st[2] / st[0] - allv.var()) < 1e-8
        s = np.sqrt(allv.var() + 1e-8)
        assert np.allclose(out, (b - allv.mean()) / (s + 1e-8), rtol=1e-6, atol=1e-6)


def test_pendulum_agent_runs_and_clamps_log_std():
    cfg = default_config(env_kind=PENDULUM, n_envs=64, rollout_len=210, hidden_dim=32, minibatch_size=256,
                         num_epochs=2, target_kl=0.0)
    a = OracleAgent(cfg)
    try:
        rng = np.random.default_rng(4)
        a_spec, c_spec = NetSpec(3, 32, 1, 1, 1), NetSpec(3, 32, 1, 1, 0)
        pa, pc = xavier_params(a_spec, rng), xavier_params(c_spec, rng)
        assert pa.size == 3 * 32 + 32 + 32 * 32 + 32 + 32 + 1 + 1 == a.param_size(0)
        pa[-1] = 2.0005   # the first clamp brings it back unless Adam already did
        a.set_params(0, pa, np.zeros(2 * pa.size, np.float32))
        a.set_params(1, pc, np.zeros(2 * pc.size, np.float32))
        a.o.orc_agent_reset(a.h, 0)
        a.o.orc_agent_rollout(a.h)
        st = a.stats()
        assert st.total_steps == 64 * 210 and st.completed_episodes == 64     # every env truncates at 200 once
        acts = a.buffer(3)
        assert acts.size == 64 * 210 and acts.std() > 1.0                      # std = exp(2) before clamping
        a.o.orc_agent_gae(a.h, 1)
        adv = a.buffer(8)
        assert abs(adv.mean()) < 1e-4 and abs(adv.std() - 1.0) < 1e-3
        perms = np.stack([rng.permutation(64 * 210) for _ in range(2)]).astype(np.int32)
        a.o.orc_agent_update(a.h, 3e-4, 1e-3, 0.0, ip(perms), 1)
        p, _ = a.get_params(0)
        assert np.isfinite(p).all() and -5.0 <= p[-1] <= 2.0
        assert a.stats().minibatches_done == 2 * (64 * 210 // 256)
    finally:
        a.close()


# ---------------------------------------------------------------- planar HalfCheetah
CHEETAH = 4
B0, F0, J0, JC, META = 17, 108, 129, 231, 245     # HalfCheetahLayout offsets (physics2d/layout.mojo:290-299)


def _cheetah(n, seed=0):
    o = oracle()
    s = np.zeros((n, 253), np.float32)
    o.orc_env_reset(CHEETAH, n, fp(s), seed)
    return s


def _cstep(s, a):
    o = oracle()
    n = s.shape[0]
    r, d, ob = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros((n, 17), np.float32)
    o.orc_env_step(CHEETAH, n, fp(s), fp(np.ascontiguousarray(a, np.float32)), fp(r), fp(d), fp(ob), 0)
    return r, d, ob


def test_cheetah_reset_fields():
    o = oracle()
    dims = [ctypes.c_int() for _ in range(4)]
    assert o.orc_env_info(CHEETAH, *[ctypes.byref(x) for x in dims]) == 0
    assert [x.value for x in dims] == [253, 17, 0, 6]
    s = _cheetah(64, seed=5)
    body = s[:, B0:B0 + 7 * 13].reshape(64, 7, 13)
    assert np.all(body[:, 0, 0] == 0) and np.allclose(body[:, 0, 1], 0.7)       # torso at INIT_HEIGHT
    assert np.allclose(body[:, 1:4, 0], -0.5) and np.allclose(body[:, 4:7, 0], 0.5)   # hips at the torso ends
    drops = [0.0725, 0.145 + 0.075, 0.145 + 0.15 + 0.047, 0.0665, 0.133 + 0.053, 0.133 + 0.106 + 0.035]
    assert np.allclose(body[:, 1:, 1], 0.7 - np.array(drops, np.float32), atol=1e-6)
    assert np.all(body[:, :, 2] == 0) and np.all(body[:, :, 5] == 0)
    assert np.all(np.abs(body[:, 0, 3]) <= 0.1) and np.all(np.abs(body[:, 0, 4]) <= 0.1)
    assert np.all(body[:, :, 3] == body[:, :1, 3]) and np.all(body[:, :, 4] == body[:, :1, 4])
    assert np.allclose(body[:, 0, 10], 1 / 6.25) and np.allclose(body[:, 0, 11], 12 / 6.25)
    assert np.allclose(body[:, 1, 11], 12 / 0.145 ** 2, rtol=1e-6) and np.all(body[:, 1:, 10] == 1.0)
    assert np.array_equal(body[0, :, 12], np.arange(7, dtype=np.float32))        # shape index = body index
    joints = s[:, J0:J0 + 6 * 17].reshape(64, 6, 17)
    assert np.all(s[:, JC] == 6)
    assert np.array_equal(joints[0, :, 1], [0, 1, 2, 0, 4, 5]) and np.array_equal(joints[0, :, 2], [1, 2, 3, 4, 5, 6])
    assert np.allclose(joints[0, :, 8], [-0.52, -0.785, -0.4, -1.0, -1.2, -0.5])
    assert np.allclose(joints[0, :, 9], [1.05, 0.785, 0.785, 0.7, 0.87, 0.5])
    assert np.all(joints[:, :, 14] == 3) and np.all(joints[:, :, 10] == 1.0) and np.all(joints[:, :, 11] == 0)
    # joint anchors coincide in world space at reset
    for j in range(6):
        a, b = int(joints[0, j, 1]), int(joints[0, j, 2])
        pa = body[0, a, :2] + joints[0, j, 3:5]
        pb = body[0, b, :2] + joints[0, j, 5:7]
        assert np.allclose(pa, pb, atol=1e-6)
    assert np.allclose(s[:, 0], 0.7) and np.all(s[:, 1:8] == 0) and np.array_equal(s[:, 8], body[:, 0, 3])
    assert np.all(s[:, META:META + 8] == 0)
    assert not np.array_equal(_cheetah(4, 1), _cheetah(4, 2))


def test_cheetah_free_fall_then_rest():
    s = _cheetah(8, seed=3)
    vy0, x0 = s[:, B0 + 4].copy(), s[:, B0 + 0].copy()
    vx0 = s[:, B0 + 3].copy()
    r, d, ob = _cstep(s, np.zeros((8, 6), np.float32))
    # the feet start 0.7 - 0.389 = 0.31 above the ground: one step (5 x 0.01 s) is pure free fall of a rigid assembly
    assert np.allclose(s[:, B0 + 4], vy0 - 9.81 * 0.05, atol=2e-4)
    assert np.allclose(s[:, B0 + 0], x0 + vx0 * 0.05, atol=1e-4)
    # reward: forward velocity + height bonus (0.5, saturated) - no control cost, no illegal contact
    assert np.allclose(r, vx0 + 0.5, atol=2e-3)
    assert np.all(s[:, META] == 1) and np.all(d == 0) and np.array_equal(ob, s[:, :17])
    for _ in range(300):
        r, d, ob = _cstep(s, np.zeros((8, 6), np.float32))
    # with limp motors (|a| = 0 -> zero torque) the body ends up lying on the ground, at rest
    assert np.isfinite(s).all()
    assert np.all(s[:, B0 + 1] < 0.4) and np.all(s[:, B0 + 1] > -0.05)
    assert np.all(np.abs(s[:, B0 + 4]) < 0.5)
    joints = s[:, J0:J0 + 6 * 17].reshape(8, 6, 17)
    assert np.all(joints[:, :, 10] == 0) and np.all(joints[:, :, 11] == 1000.0)   # torque 0, speed +1000 for a >= 0


def test_cheetah_motor_limits_truncation_and_penalty():
    s = _cheetah(4, seed=9)
    a = np.tile(np.array([[1.5, -2.0, 0.3, -0.3, 1.0, -1.0]], np.float32), (4, 1))
    r, d, ob = _cstep(s, a)
    joints = s[:, J0:J0 + 6 * 17].reshape(4, 6, 17)
    assert np.allclose(joints[0, :, 10], [1.0, 1.0, 0.3, 0.3, 1.0, 1.0])           # MAX_TORQUE * |clamped action|
    assert np.array_equal(joints[0, :, 11], [1000, -1000, 1000, -1000, 1000, -1000])
    ctrl = 0.1 * (1 + 1 + 0.09 + 0.09 + 1 + 1)
    body_vx = (s[:, B0] - 0.0) / 0.05
    assert np.allclose(r, body_vx - ctrl + 0.5, atol=1e-4)
    rng = np.random.default_rng(0)
    dones = 0
    min_r = 0.0
    for t in range(2, 1001):
        r, d, ob = _cstep(s, rng.uniform(-1, 1, (4, 6)).astype(np.float32))
        assert np.all(np.abs(ob[:, 2:8]) <= 2 * np.pi + 1e-5)   # differences of angles kept in [-pi, pi]
        min_r = min(min_r, float(r.min()))
        assert np.all(d == (1.0 if t == 1000 else 0.0))
    assert np.isfinite(s).all() and min_r < -0.5      # illegal ground contacts were penalised at some point
    o = oracle()
    dd = d.copy()
    o.orc_env_selective_reset(CHEETAH, 4, fp(s), fp(dd), 77)
    assert np.all(dd == 0) and np.all(s[:, META] == 0) and np.allclose(s[:, B0 + 1], 0.7)


# ---------------------------------------------------------------- BipedalWalker
BIPEDAL = 3
BW_B0, BW_J0, BW_E0, BW_EC, BW_META = 24, 104, 173, 941, 942   # BipedalWalkerLayout (physics2d/layout.mojo:268-277)


def _walker(n, seed=0):
    o = oracle()
    s = np.zeros((n, 950), np.float32)
    o.orc_env_reset(BIPEDAL, n, fp(s), seed)
    return s


def _wstep(s, a):
    o = oracle()
    n = s.shape[0]
    r, d, ob = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros((n, 24), np.float32)
    o.orc_env_step(BIPEDAL, n, fp(s), fp(np.ascontiguousarray(a, np.float32)), fp(r), fp(d), fp(ob), 0)
    return r, d, ob


def test_bipedal_reset_terrain_bodies_and_lidar():
    o = oracle()
    dims = [ctypes.c_int() for _ in range(4)]
    assert o.orc_env_info(BIPEDAL, *[ctypes.byref(x) for x in dims]) == 0
    assert [x.value for x in dims] == [950, 24, 0, 4]
    s = _walker(32, seed=2)
    assert np.all(s[:, BW_EC] == 128)                       # min(TERRAIN_LENGTH - 1, MAX_TERRAIN_EDGES)
    edges = s[:, BW_E0:BW_E0 + 768].reshape(32, 128, 6)
    step = np.float32(14.0 / 30.0)
    assert np.array_equal(edges[0, :, 0], np.arange(128, dtype=np.float32) * step)
    assert np.array_equal(edges[:, 1:, 0], edges[:, :-1, 2]) and np.array_equal(edges[:, 1:, 1], edges[:, :-1, 3])
    assert np.allclose(np.hypot(edges[:, :, 4], edges[:, :, 5]), 1.0, atol=1e-6) and np.all(edges[:, :, 5] > 0)
    # the start pad (edges 0..20) is the same deterministic ripple in every environment; the rest is random
    assert np.array_equal(edges[0, :21], edges[7, :21]) and not np.array_equal(edges[0, 21:], edges[7, 21:])
    assert np.all(np.abs(edges[:, :21, 3] - 10.0 / 3.0) < 0.05)
    body = s[:, BW_B0:BW_B0 + 65].reshape(32, 5, 13)
    leg_h = 34.0 / 30.0
    assert np.allclose(body[:, :, 0], 20 * 14.0 / 30.0) and np.allclose(body[:, 0, 1], 10.0 / 3.0 + 2 * leg_h)
    assert np.allclose(body[:, 1, 1], body[:, 0, 1] - 8.0 / 30.0 - leg_h / 2, atol=1e-6)
    assert np.allclose(body[:, 2, 1], body[:, 1, 1] - leg_h, atol=1e-6)
    assert np.array_equal(body[:, 1, :2], body[:, 3, :2]) and np.array_equal(body[:, 2, :2], body[:, 4, :2])
    assert np.allclose(body[:, :, 10], [0.2, 1.25, 2.0, 1.25, 2.0]) and np.allclose(body[:, :, 11], [0.5, 10, 20, 10, 20])
    joints = s[:, BW_J0:BW_J0 + 68].reshape(32, 4, 17)
    assert np.array_equal(joints[0, :, 1], [0, 1, 0, 3]) and np.array_equal(joints[0, :, 2], [1, 2, 3, 4])
    assert np.allclose(joints[0, :, 8], [-0.8, -1.6, -0.8, -1.6]) and np.allclose(joints[0, :, 9], [1.1, -0.1, 1.1, -0.1])
    assert np.all(joints[:, :, 10] == 80.0) and np.all(joints[:, :, 14] == 3)
    # lidar: ray 0 points straight down from the hull centre: height above the pad over the range
    h = body[:, 0, 1] - edges[:, 20, 1]
    assert np.allclose(s[:, 14], h / (160.0 / 30.0), atol=2e-3)
    assert np.all(np.diff(s[:, 14:24], axis=1) >= -1e-6)    # flatter rays travel farther over near-flat ground
    assert np.all(s[:, 22:24] == 1.0)                       # the last rays (>= 1.33 rad from vertical) miss
    assert np.all(s[:, 0:2] == 0) and np.all(s[:, 4:14] == 0)
    assert np.array_equal(s[:, BW_META + 1], body[:, 0, 0]) and np.all(s[:, BW_META + 2:BW_META + 8] == 0)


def test_bipedal_step_rewards_and_terminations():
    s = _walker(16, seed=4)
    x0 = s[:, BW_B0].copy()
    a = np.tile(np.array([[0.5, -2.0, -0.25, 1.0]], np.float32), (16, 1))
    r, d, ob = _wstep(s, a)
    joints = s[:, BW_J0:BW_J0 + 68].reshape(16, 4, 17)
    assert np.array_equal(joints[0, :, 11], [4.0, -6.0, -4.0, 6.0])            # SPEED_HIP / SPEED_KNEE with the sign
    assert np.allclose(joints[0, :, 10], [40.0, 80.0, 20.0, 80.0])             # MOTORS_TORQUE * |clamped action|
    assert np.array_equal(ob, s[:, :24]) and np.all(d == 0) and np.all(s[:, BW_META] == 1)
    hull = s[:, BW_B0:BW_B0 + 13]
    vel_x = hull[:, 3] * np.float32(600.0 / 30.0 / 50.0)
    want = (130.0 / 30.0) * (hull[:, 0] - x0) - 5.0 * np.abs(hull[:, 2]) - 0.00035 * 80.0 * (0.5 + 2.0 + 0.25 + 1.0)
    want = want + np.where(vel_x > 0, 3.0 * vel_x, 5.0 * vel_x)                # energy uses the unclamped actions
    assert np.allclose(r, want, atol=1e-4)
    assert np.array_equal(s[:, BW_META + 1], hull[:, 0])                        # prev_x follows the hull
    # limp motors: the walker sinks until the hull is lower than TERRAIN_HEIGHT + 1.2 LEG_H -> done, reward -50
    s = _walker(16, seed=5)
    seen = np.zeros(16, bool)
    for t in range(200):
        r, d, ob = _wstep(s, np.zeros((16, 4), np.float32))
        newly = (d > 0.5) & ~seen
        if newly.any():
            crit = 10.0 / 3.0 + 1.2 * 34.0 / 30.0
            low = s[newly, BW_B0 + 1] < crit
            assert np.all(np.where(low, r[newly] == -50.0, r[newly] == -100.0))
        seen |= d > 0.5
        if seen.all():
            break
    assert seen.all() and t < 150
    # foot contacts reach the observation and the metadata
    assert np.array_equal(ob[:, 8], s[:, BW_META + 5]) and np.array_equal(ob[:, 13], s[:, BW_META + 6])
    # time limit: a state parked at step 1999 terminates on the next step
    s = _walker(2, seed=6)
    s[:, BW_META] = 1999
    r, d, ob = _wstep(s, np.zeros((2, 4), np.float32))
    assert np.all(d == 1.0) and np.all(s[:, BW_META] == 2000)
    # leaving the terrain to the left is a crash
    s = _walker(2, seed=6)
    s[:, BW_B0:BW_B0 + 65:13] = -0.5      # every body, so that the joints stay satisfied
    r, d, ob = _wstep(s, np.zeros((2, 4), np.float32))
    assert np.all(d == 1.0) and np.all(r == -100.0)


# ---------------------------------------------------------------- LunarLander, continuous controls
LUNAR, LUNAR_C = 2, 5


def _lunar_pair(n, seed):
    o = oracle()
    a, b = np.zeros((n, 192), np.float32), np.zeros((n, 192), np.float32)
    o.orc_env_reset(LUNAR, n, fp(a), seed)
    o.orc_env_reset(LUNAR_C, n, fp(b), seed)
    assert np.array_equal(a, b)                       # one reset serves both traits
    return a, b


def _lstep(kind, s, act):
    o = oracle()
    n = s.shape[0]
    r, d, ob = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros((n, 8), np.float32)
    o.orc_env_step(kind, n, fp(s), fp(np.ascontiguousarray(act, np.float32)), fp(r), fp(d), fp(ob), 0)
    return r, d, ob


def test_lunar_continuous_matches_discrete_at_full_throttle_and_charges_fuel_proportionally():
    o = oracle()
    dims = [ctypes.c_int() for _ in range(4)]
    assert o.orc_env_info(LUNAR_C, *[ctypes.byref(x) for x in dims]) == 0
    assert [x.value for x in dims] == [192, 8, 0, 2]
    n = 64
    # full main throttle (+1) == discrete action 2; side control -1 / +1 == discrete actions 1 / 3 (power 1)
    for disc, cont in ((2, (1.0, 0.0)), (1, (-1.0, -1.0)), (3, (-1.0, 1.0)), (0, (-1.0, 0.2))):
        a, b = _lunar_pair(n, seed=3)
        for t in range(20):
            ra, da, oa = _lstep(LUNAR, a, np.full(n, disc, np.float32))
            rb, db, ob = _lstep(LUNAR_C, b, np.tile(np.array([cont], np.float32), (n, 1)))
            assert np.array_equal(a, b) and np.array_equal(oa, ob) and np.array_equal(da, db)
            assert np.allclose(ra, rb, atol=1e-5)    # same fuel charge: 0.30 main / 0.03 side / none
    # half throttle: half the main impulse and half the fuel charge; side engine off inside +-0.5
    a, b = _lunar_pair(n, seed=4)
    vy0 = a[:, 8 + 4].copy()
    r_full, _, _ = _lstep(LUNAR_C, a, np.tile(np.array([[1.0, 0.4]], np.float32), (n, 1)))
    r_half, _, _ = _lstep(LUNAR_C, b, np.tile(np.array([[0.0, -0.4]], np.float32), (n, 1)))
    dv_full, dv_half = a[:, 12] - vy0, b[:, 12] - vy0
    g = -10.0 * 0.02
    assert np.allclose(dv_half - g, 0.5 * (dv_full - g), rtol=2e-3, atol=2e-4)
    # side power ramps from 0 at |a| = 0.5 to 1 at |a| = 1: at 0.75 the lander gets half the angular impulse
    a, b = _lunar_pair(n, seed=5)
    c, _ = _lunar_pair(n, seed=5)
    _lstep(LUNAR_C, a, np.tile(np.array([[-1.0, 0.5]], np.float32), (n, 1)))     # exactly at the threshold: off
    _lstep(LUNAR_C, b, np.tile(np.array([[-1.0, 0.75]], np.float32), (n, 1)))
    _lstep(LUNAR_C, c, np.tile(np.array([[-1.0, 1.0]], np.float32), (n, 1)))
    w_off, w_half, w_full = a[:, 8 + 5], b[:, 8 + 5], c[:, 8 + 5]
    assert np.all(np.abs(w_full - w_off) > 1e-3)
    assert np.allclose(w_half - w_off, 0.5 * (w_full - w_off), rtol=5e-2, atol=1e-4)
    # actions beyond the range are clamped for the impulse; the side fuel term uses the unclamped control
    a, b = _lunar_pair(n, seed=6)
    _lstep(LUNAR_C, a, np.tile(np.array([[5.0, 0.0]], np.float32), (n, 1)))
    _lstep(LUNAR_C, b, np.tile(np.array([[1.0, 0.0]], np.float32), (n, 1)))
    assert np.array_equal(a[:, 8:47], b[:, 8:47])


def test_observation_noise_kernel_math():
    """add_obs_noise_kernel (kernels.mojo:882-925): obs += std * Box-Muller noise on the Philox stream
    seed + env * obs_dim + dim -- the same stream and transform as the Gaussian sampler's noise, which
    gives an independent check: with mean 0 and log_std 0 the sampler's action IS the noise."""
    from _util import fp, oracle
    o = oracle()
    n, d = 4096, 5
    obs = np.zeros((n, d), np.float32)
    o.orc_add_obs_noise(n, d, fp(obs), 0.25, 1234)
    assert abs(obs.mean()) < 0.01 and abs(obs.std() - 0.25) < 0.01
    actor_out = np.zeros((n, 2 * d), np.float32)          # means 0, log_std 0 -> std 1
    actions, lp = np.zeros((n, d), np.float32), np.zeros(n, np.float32)
    o.orc_sample_continuous_actions(n, d, fp(actor_out), fp(actions), fp(lp), 1234, 0)
    assert np.allclose(obs, actions * np.float32(0.25), rtol=0, atol=1e-7)
    # std <= 0 leaves the observations untouched; the call is deterministic
    ref = np.arange(n * d, dtype=np.float32).reshape(n, d)
    a = ref.copy(); o.orc_add_obs_noise(n, d, fp(a), 0.0, 7)
    assert np.array_equal(a, ref)
    b, c = ref.copy(), ref.copy()
    o.orc_add_obs_noise(n, d, fp(b), 0.1, 7); o.orc_add_obs_noise(n, d, fp(c), 0.1, 7)
    assert np.array_equal(b, c) and not np.array_equal(b, ref)
