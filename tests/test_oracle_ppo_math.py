"""Oracle self-checks for the PPO maths against straightforward numpy."""
import numpy as np

from _util import NetSpec, fp, oracle, xavier_params


def _np_forward(spec, x, p):
    I, H, O = spec.in_dim, spec.hidden_dim, spec.out_dim
    W0 = p[:I * H].reshape(I, H); b0 = p[I * H:I * H + H]; o = I * H + H
    W1 = p[o:o + H * H].reshape(H, H); b1 = p[o + H * H:o + H * H + H]; o += H * H + H
    W2 = p[o:o + H * O].reshape(H, O); b2 = p[o + H * O:o + H * O + O]
    x = x.astype(np.float64)
    h0 = np.maximum(x @ W0 + b0, 0); h1 = np.maximum(h0 @ W1 + b1, 0)
    return h1 @ W2 + b2


def test_mlp_forward_backward_against_numpy():
    o = oracle()
    rng = np.random.default_rng(0)
    spec = NetSpec(8, 32, 4, 0, 0)
    p = xavier_params(spec, rng)
    B = 64
    x = rng.standard_normal((B, 8)).astype(np.float32)
    out = np.empty((B, 4), np.float32)
    cache = np.empty(B * o.orc_net_cache_per_sample(spec), np.float32)
    o.orc_mlp_forward(spec, B, fp(x), fp(p), fp(out), fp(cache))
    assert np.allclose(out, _np_forward(spec, x, p.astype(np.float64)), rtol=1e-5, atol=1e-6)
    # cache layout: [B x (in + H)] [B x (H + H)] [B x H]
    c0 = cache[:B * 40].reshape(B, 40)
    assert np.array_equal(c0[:, :8], x)
    # backward vs central finite differences of sum(out * g)
    g = rng.standard_normal((B, 4)).astype(np.float32)
    grads = np.empty_like(p)
    gin = np.empty((B, 8), np.float32)
    o.orc_mlp_backward(spec, B, fp(g), fp(p), fp(cache), fp(gin), fp(grads), 1)
    f = lambda q: float((_np_forward(spec, x, q) * g).sum())
    idx = rng.choice(p.size, 40, replace=False)
    for i in idx:
        q = p.astype(np.float64); q[i] += 1e-4; fp1 = f(q); q[i] -= 2e-4; fm1 = f(q)
        assert abs((fp1 - fm1) / 2e-4 - grads[i]) < 2e-3 * max(1.0, abs(grads[i]))
    # fp32-accumulated variant agrees with the f64 one
    grads32 = np.empty_like(p)
    o.orc_mlp_backward(spec, B, fp(g), fp(p), fp(cache), fp(gin), fp(grads32), 0)
    assert np.allclose(grads, grads32, rtol=1e-4, atol=1e-5)


def test_gae_matches_reference_recurrence():
    o = oracle()
    rng = np.random.default_rng(1)
    T, N = 16, 5
    r = rng.standard_normal((T, N)).astype(np.float32); v = rng.standard_normal((T, N)).astype(np.float32)
    d = (rng.random((T, N)) < 0.2).astype(np.float32); boot = rng.standard_normal(N).astype(np.float32)
    adv, ret = np.empty((T, N), np.float32), np.empty((T, N), np.float32)
    o.orc_gae(T, N, fp(r), fp(v), fp(d), fp(boot), 0.99, 0.95, fp(adv), fp(ret))
    for e in range(N):
        g = 0.0
        for t in range(T - 1, -1, -1):
            nv = boot[e] if t == T - 1 else v[t + 1, e]
            if d[t, e] > 0.5:
                nv, g = 0.0, 0.0
            g = (r[t, e] + 0.99 * nv - v[t, e]) + 0.99 * 0.95 * g
            assert abs(adv[t, e] - g) < 1e-4 and abs(ret[t, e] - (g + v[t, e])) < 1e-4


def test_sampler_fallthrough_and_logprob():
    o = oracle()
    n, A = 4096, 4
    rng = np.random.default_rng(2)
    logits = rng.standard_normal((n, A)).astype(np.float32)
    a, lp = np.empty(n, np.float32), np.empty(n, np.float32)
    o.orc_sample_actions(n, A, fp(logits), fp(a), fp(lp), 1234)
    p = np.exp(logits - logits.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    assert np.allclose(lp, np.log(p[np.arange(n), a.astype(int)] + 1e-8), atol=1e-5)
    freq = np.bincount(a.astype(int), minlength=A) / n
    assert np.abs(freq - p.mean(0)).max() < 0.03
    g = np.empty(n, np.float32)
    o.orc_argmax_actions(n, A, fp(logits), fp(g))
    assert np.array_equal(g, logits.argmax(1).astype(np.float32))


def test_actor_critic_grads_clip_adam():
    o = oracle()
    rng = np.random.default_rng(3)
    B, A = 256, 4
    logits = rng.standard_normal((B, A)).astype(np.float32)
    act = rng.integers(0, A, B).astype(np.float32)
    adv = rng.standard_normal(B).astype(np.float32)
    p = np.exp(logits - logits.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    old_lp = (np.log(p[np.arange(B), act.astype(int)]) + 0.3 * rng.standard_normal(B)).astype(np.float32)
    g, kl = np.empty((B, A), np.float32), np.empty(B, np.float32)
    o.orc_ppo_actor_grad(B, A, fp(logits), fp(old_lp), fp(adv), fp(act), 0.2, 0.01, fp(g), fp(kl))
    new_lp = np.log(p[np.arange(B), act.astype(int)] + 1e-8)
    ratio = np.exp(new_lp - old_lp)
    clipped = (ratio < 0.8) | (ratio > 1.2)
    assert np.all(g[clipped] == 0) and np.any(clipped) and np.any(~clipped)   # zero outside the band, any sign of A
    assert np.allclose(kl, old_lp - new_lp, atol=1e-5)
    onehot = np.eye(A)[act.astype(int)]
    want = (-adv[:, None] * ratio[:, None] * (onehot - p) + 0.01 * p * (1 + np.log(p + 1e-8))) / B
    assert np.allclose(g[~clipped], want[~clipped], rtol=1e-4, atol=1e-7)
    # critic, clipped: zero gradient when the clipped loss is the larger one and v moved past the band
    v = np.array([1.0, 1.0, 0.0], np.float32); vo = np.array([0.0, 0.9, 0.0], np.float32)
    ret = np.array([-1.0, 2.0, 1.0], np.float32); gv = np.empty(3, np.float32)
    o.orc_ppo_critic_grad(3, fp(v), fp(vo), fp(ret), 0.5, 0.2, 1, fp(gv))
    assert np.allclose(gv, [0.5 * 2 * 2.0 / 3, 0.5 * 2 * -1.0 / 3, 0.5 * 2 * -1.0 / 3])
    o.orc_ppo_critic_grad(3, fp(v), fp(vo), fp(ret), 0.5, 0.2, 0, fp(gv))
    assert np.allclose(gv, 2 * 0.5 * (v - ret) / 3)
    # clip: scale = max / (norm + 1e-8) only above the threshold
    gr = np.full(100, 0.1, np.float32)
    norm = o.orc_grad_clip(100, fp(gr), 0.5, 0)
    assert abs(norm - 1.0) < 1e-6 and np.allclose(gr, 0.05)
    gr = np.full(100, 0.01, np.float32)
    o.orc_grad_clip(100, fp(gr), 0.5, 0)
    assert np.allclose(gr, 0.01)
    # Adam first step: p -= lr * g / (|g| + eps) up to bias-correction rounding
    prm = np.zeros(8, np.float32); grd = np.linspace(-1, 1, 8).astype(np.float32); st = np.zeros(16, np.float32)
    import ctypes
    b1, b2 = ctypes.c_float(), ctypes.c_float()
    o.orc_adam_bias_corrections(0.9, 0.999, 1, ctypes.byref(b1), ctypes.byref(b2))
    o.orc_adam_step(8, fp(prm), fp(grd), fp(st), 0.001, 0.9, 0.999, 1e-8, b1.value, b2.value)
    assert np.allclose(prm, -0.001 * np.sign(grd), atol=1e-6)
    assert np.allclose(st[0::2], 0.1 * grd, atol=1e-7) and np.allclose(st[1::2], 0.001 * grd * grd, atol=1e-8)
