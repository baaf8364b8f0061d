"""Kubolorn on the GPU against the plain restatement in tests/kubolorn_oracle.py: every mechanism alone (op-level entry points that launch
the family's kernels), then whole models with small random configurations — prompts in one pass, token by token, in portions, after a
release, long decoding, greedy generation through the host entry points and the command line."""
import json
import math
import os
import subprocess

import numpy as np
import pytest

import kubolorn_oracle as O
from xalm_b200 import build, capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import InferenceState, Model, Sampler, generate

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4   # IEEE fp32 path against float64, on values of order one
BF16_TOL = 6e-2  # serving mode: bf16 weights (exact here), a bf16 key cache, fp16 operands on the tensor cores


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if got.size == 0:
        return
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err < tol, f"max error {err:.3e} (tolerance {tol})"


# ---- mechanisms alone ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W,groups,taps", [(24, 3, 4), (10, 1, 2), (64, 64, 3), (130, 5, 1), (4096, 4, 4), (12, 2, 9)])
@pytest.mark.parametrize("cuts", [[40], [1], [2, 1, 17, 3, 8, 9], [7, 33]])
def test_reader_norm_and_convolution_over_cuts(W, groups, taps, cuts):
    """Grouped norm, h + conv(h) and the carried rows for two readers at once; one group is made loud (a norm over the whole row would
    show), steps of 1 .. 33 rows take the one-CTA path that rewrites the carried rows itself and the many-CTA path that stages them."""
    rng = np.random.default_rng(W + taps)
    T = 40
    x = rng.standard_normal((T, W))
    x[:, : W // groups] *= 30.0
    w, cw = 1 + 0.3 * rng.standard_normal((2, W)), 0.5 * rng.standard_normal((2, W, taps))
    want = []
    for r in range(2):
        hn = O.group_norm(x, w[r], groups, 1e-4)
        want.append(hn + O.short_conv(hn, cw[r], np.zeros((taps - 1, W)))[0])
    hist, got, p, i = np.zeros((2, taps - 1, W)), [], 0, 0
    while p < T:
        n = min(cuts[min(i, len(cuts) - 1)], T - p)
        out, hist = capi.norm_conv(x[p:p + n], w, cw, hist, groups, eps=1e-4)
        got.append(out)
        p, i = p + n, i + 1
    close(np.concatenate(got, axis=1), np.stack(want), F32_TOL)
    if taps > 1:
        close(hist[1], O.group_norm(x, w[1], groups, 1e-4)[T - (taps - 1):], F32_TOL)


@pytest.mark.parametrize("C,taps", [(5, 4), (130, 2), (64, 8), (300, 1), (7, 3)])
@pytest.mark.parametrize("cuts", [[50], [1], [2, 1, 1, 20, 3], [16, 17]])
def test_short_convolution_over_cuts(C, taps, cuts):
    rng = np.random.default_rng(C + taps)
    T = 50
    x, w, b = rng.standard_normal((T, C)), rng.standard_normal((C, taps)), rng.standard_normal(C)
    want = O.silu(O.short_conv(x, w, np.zeros((taps - 1, C)), b)[0])
    hist, got, p, i = np.zeros((taps - 1, C)), [], 0, 0
    while p < T:
        n = min(cuts[min(i, len(cuts) - 1)], T - p)
        out, hist = capi.short_conv(x[p:p + n], w, hist, bias=b, act=3)
        got.append(out)
        p, i = p + n, i + 1
    close(np.concatenate(got), want, F32_TOL)
    close(hist, x[T - (taps - 1):] if taps > 1 else np.zeros((0, C)), 1e-6)
    close(capi.short_conv(x, w, np.zeros((taps - 1, C)))[0], O.short_conv(x, w, np.zeros((taps - 1, C)))[0], F32_TOL)   # no bias, no activation


def test_pair_embedding_rows():
    rng = np.random.default_rng(3)
    V, W, buckets = 70000, 12, 101
    cfg = O.make_config(V, W, [], groups=3, scale=5.0, bigram=(buckets, 1000003, 999983), eps=1e-5)      # products beyond 32 bits
    w = {"embed": rng.standard_normal((V, W)), "bigram": rng.standard_normal((buckets + 1, W)), "embed.norm": 1 + 0.2 * rng.standard_normal(W)}
    tokens = [69999, 0, 69999, 5, 5, 12345]
    kw = dict(scale=5.0, pair=w["bigram"], mul_prev=1000003, mul_cur=999983, w=w["embed.norm"], groups=3)
    close(capi.embed_pair(tokens, None, w["embed"], **kw), O.embed_rows(cfg, w, tokens, None), F32_TOL)  # the first row takes the table's last row
    close(capi.embed_pair(tokens[2:], tokens[1], w["embed"], **kw), O.embed_rows(cfg, w, tokens[2:], tokens[1]), F32_TOL)
    assert np.abs(capi.embed_pair(tokens[:1], None, w["embed"], **kw) - capi.embed_pair(tokens[:1], 7, w["embed"], **kw)).max() > 1e-2
    plain = capi.embed_pair(tokens, None, w["embed"], scale=2.0)
    close(plain, 2.0 * w["embed"][tokens], 1e-6)


def gla_reference(q, k, v, alpha, S):
    out = np.zeros((q.shape[0],) + v.shape[1:])
    for t in range(q.shape[0]):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hij,hi->hj", S, q[t])
    return out, S


@pytest.mark.parametrize("H,d,dv", [(2, 5, 7), (1, 32, 32), (3, 48, 64), (2, 100, 24), (1, 130, 40), (2, 260, 12), (1, 8, 300)])
def test_channel_decay_recurrence(H, d, dv):
    """S_t = diag(alpha_t) S_{t-1} + k_t v_t^T with a decay per key channel and token, head norm with a weight, silu gate; the state handed
    over cuts of 2, 1, 1 and 17 tokens equals one run."""
    rng = np.random.default_rng(H * d + dv)
    T = 21
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    alpha, gate, nw = rng.uniform(0.3, 1.0, (T, H, d)), rng.standard_normal((T, H * dv)), 1 + 0.2 * rng.standard_normal(dv)
    o, S = gla_reference(q * d ** -0.5, k, v, alpha, np.zeros((H, d, dv)))
    want = (o / np.sqrt((o ** 2).mean(-1, keepdims=True) + 1e-5) * nw).reshape(T, -1) * O.silu(gate)
    f = lambda a: a.reshape(T, -1)
    kw = dict(q_scale=d ** -0.5, norm_w=nw, eps=1e-5)
    got, st = capi.keyed_recurrence(f(q), f(k), f(v), f(alpha), np.zeros((H, d, dv)), H, 1, d, dv, 1, gate=gate, **kw)
    close(got, want, F32_TOL)
    close(st, S, F32_TOL)
    st, rows, p = np.zeros((H, d, dv)), [], 0
    for n in (2, 1, 1, 17):
        out, st = capi.keyed_recurrence(f(q)[p:p + n], f(k)[p:p + n], f(v)[p:p + n], f(alpha)[p:p + n], st, H, 1, d, dv, 1, gate=gate[p:p + n], **kw)
        rows.append(out)
        p += n
    close(np.concatenate(rows), want, F32_TOL)
    close(st, S, F32_TOL)


def test_a_value_written_once_is_read_back_after_hundreds_of_tokens():
    """Channel 0 never decays and channel 1 halves every token: a value written at the first token through both is still read through
    channel 0 after 500 tokens and gone from channel 1."""
    T, d, dv = 500, 2, 3
    q, k, v, alpha = np.zeros((T, d)), np.zeros((T, d)), np.zeros((T, dv)), np.ones((T, d))
    alpha[:, 1] = 0.5
    k[0], v[0] = [1.0, 1.0], [3.0, -2.0, 7.0]
    q[-1] = [1.0, 0.0]
    q[-2] = [0.0, 1.0]
    got, st = capi.keyed_recurrence(q, k, v, alpha, np.zeros((1, d, dv)), 1, 1, d, dv, 1)
    close(got[-1], v[0], 1e-6)
    assert np.abs(got[-2]).max() < 1e-30
    close(st[0, 0], v[0], 1e-6)


@pytest.mark.parametrize("H,rep,N,P", [(4, 2, 6, 5), (1, 1, 32, 16), (8, 4, 48, 48), (2, 2, 128, 64), (3, 1, 70, 9), (6, 3, 16, 130)])
def test_step_size_recurrence(H, rep, N, P):
    """S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t with B and C shared by `rep` neighbouring heads and
    dt = softplus(raw + bias); cuts as above."""
    rng = np.random.default_rng(H * N + P)
    T, G = 23, H // rep
    x, B, C = rng.standard_normal((T, H, P)), rng.standard_normal((T, G, N)), rng.standard_normal((T, G, N))
    raw, bias, A_log, D = 2 * rng.standard_normal((T, H)), rng.standard_normal(H), rng.uniform(-2, 1, H), rng.standard_normal(H)
    dt = O.softplus(raw + bias)
    S, want = np.zeros((H, N, P)), np.zeros((T, H, P))
    for t in range(T):
        for h in range(H):
            S[h] = math.exp(-math.exp(A_log[h]) * dt[t, h]) * S[h] + dt[t, h] * np.outer(B[t, h // rep], x[t, h])
            want[t, h] = S[h].T @ C[t, h // rep] + D[h] * x[t, h]
    f = lambda a: a.reshape(T, -1)
    kw = dict(dt_bias=bias, A_log=A_log, skip=D)
    got, st = capi.keyed_recurrence(f(C), f(B), f(x), raw, np.zeros((H, N, P)), H, rep, N, P, 2, **kw)
    close(got, f(want), F32_TOL)
    close(st, S, F32_TOL)
    st, rows, p = np.zeros((H, N, P)), [], 0
    for n in (2, 1, 1, 19):
        out, st = capi.keyed_recurrence(f(C)[p:p + n], f(B)[p:p + n], f(x)[p:p + n], raw[p:p + n], st, H, rep, N, P, 2, **kw)
        rows.append(out)
        p += n
    close(np.concatenate(rows), f(want), F32_TOL)
    close(st, S, F32_TOL)


def sink_reference(q, k, v, pos0, H, G, scale, sink):
    T, d, dv = q.shape[0], q.shape[2], v.shape[2]
    out = np.zeros((T, H, dv))
    for t in range(T):
        n = pos0 + t + 1
        for h in range(H):
            s = k[:n, h // (H // G)] @ q[t, h] * scale
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            out[t, h] = (e @ v[:n, h // (H // G)]) / (e.sum() + math.exp(sink[h] - m))
    return out.reshape(T, -1)


@pytest.mark.parametrize("H,G,d", [(4, 1, 8), (2, 2, 5), (6, 3, 16), (8, 2, 64), (1, 1, 130)])
@pytest.mark.parametrize("T,pos0,splits", [(1, 0, 1), (1, 300, 1), (1, 300, 5), (3, 97, 1), (40, 0, 1), (37, 60, 2)])
def test_sink_attention(H, G, d, T, pos0, splits):
    """The sink is one more term of the denominator: per head one that dwarfs every score (the output nearly vanishes), one that is
    negligible, ordinary ones.  One, a few and many queries take three kernels; key splits join partial sums before the sink is added."""
    rng = np.random.default_rng(H * d + T + pos0)
    n = pos0 + T
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((n, G, d)), rng.standard_normal((n, G, d))
    sink = rng.standard_normal(H)
    sink[0] = 60.0
    if H > 1:
        sink[1] = -60.0
    want = sink_reference(q, k, v, pos0, H, G, 0.3, sink)
    f = lambda a: a.reshape(a.shape[0], -1)
    got = capi.sink_attention(f(q), f(k), f(v), pos0, H, G, d, d, 0.3, sink=sink, n_splits=splits)
    close(got, want, F32_TOL)
    assert np.abs(got[:, :d]).max() < 1e-12 * max(1.0, np.abs(v).max()) * 1e3           # head 0: exp(-60) of an ordinary output
    close(capi.sink_attention(f(q), f(k), f(v), pos0, H, G, d, d, 0.3, sink=sink, out_scale=1.7, n_splits=splits), 1.7 * want, F32_TOL)
    close(capi.sink_attention(f(q), f(k), f(v), pos0, H, G, d, d, 0.3, sink=sink, n_splits=splits, cache_bf16=True),
          sink_reference(q, O.bf16_round(k), O.bf16_round(v), pos0, H, G, 0.3, sink), F32_TOL)


@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 255, 256, 700])
@pytest.mark.parametrize("T", [1, 3, 40])
def test_one_far_key_among_hundreds(far, T):
    """One query and one key are scaled so that their score stands out: the output is that key's value, wherever the key lies (the first
    row, either side of a key-block border, far back)."""
    rng = np.random.default_rng(far + T)
    H, G, d, n = 2, 1, 16, 760
    pos0 = n - T
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((n, G, d)), rng.standard_normal((n, G, d))
    k[far, 0] = 0.0
    k[far, 0, 3] = 40.0
    q[-1, 1] = 0.0
    q[-1, 1, 3] = 40.0
    sink = np.array([0.5, -0.5])
    f = lambda a: a.reshape(a.shape[0], -1)
    got = capi.sink_attention(f(q), f(k), f(v), pos0, H, G, d, d, 0.25, sink=sink, n_splits=4 if T == 1 else 1)
    close(got[-1, d:], v[far, 0], 1e-4)
    close(got, sink_reference(q, k, v, pos0, H, G, 0.25, sink), F32_TOL)


@pytest.mark.parametrize("H,G,d,dims", [(4, 2, 8, 4), (2, 1, 6, 6), (3, 3, 10, 0), (2, 2, 64, 32)])
def test_rescaled_rotation_and_cache_rows(H, G, d, dims):
    """Queries and keys turn with YaRN-rescaled frequencies and magnitude; the value rows are the keys as they came."""
    rng = np.random.default_rng(d + dims)
    T, pos0 = 5, 300
    rot = {"dims": dims, "base": 50.0, "scaling": {"factor": 5.0, "fast": 6.0, "slow": 0.5, "original": 64}} if dims else None
    proj = rng.standard_normal((T, (H + G) * d))
    q, k = proj[:, :H * d].reshape(T, H, d), proj[:, H * d:].reshape(T, G, d)
    pos = np.arange(pos0, pos0 + T)
    freq, mag = O.yarn_table(rot) if rot else (None, 0.0)
    if rot:
        plain = rot["base"] ** (-2.0 * np.arange(dims // 2) / dims)
        assert mag > 1.0 and ((freq < plain * 0.999).any() or dims <= 4)                      # the rescaling bites somewhere
    gq, kc, vc = capi.qk_post(proj, pos0, H, G, d, freq=freq, rot_mag=mag)
    close(gq, O.rotate(q, pos, rot).reshape(T, -1), 2e-3)                                    # angles of hundreds of radians in fp32
    close(kc[pos0:], O.rotate(k, pos, rot).reshape(T, -1), 2e-3)
    close(vc[pos0:], k.reshape(T, -1), 1e-6)


def test_decay_activation_and_gelu_epilogues():
    rng = np.random.default_rng(8)
    for T, N, K in ((1, 7, 4), (3, 66, 16), (9, 33, 3), (70, 130, 8)):
        x, w, b = rng.standard_normal((T, K)) * 6, rng.standard_normal((N, K)), rng.standard_normal(N) * 4
        z = x @ w.T + b
        close(capi.rows_act_bias(x, w, 5, bias=b, act_pow=1 / 16.0), O.sigmoid(z) ** (1 / 16.0), F32_TOL)
        close(capi.rows_act_bias(x, w, 5, bias=b, act_pow=1.0), O.sigmoid(z), F32_TOL)
        close(capi.rows_act_bias(x, w, 4), O.gelu_tanh(x @ w.T), F32_TOL)
    big = capi.rows_act_bias(np.array([[-200.0], [200.0]]), np.array([[1.0]]), 5, act_pow=0.25)
    close(big[:, 0], [math.exp(-50.0), 1.0], 1e-6)                                           # where the sigmoid itself would be 0 in fp32


@pytest.mark.parametrize("W,groups,ld", [(12, 3, 12), (64, 1, 80), (384, 2, 640), (30, 30, 33)])
def test_gate_before_grouped_norm(W, groups, ld):
    rng = np.random.default_rng(W)
    T = 6
    y, g, w = rng.standard_normal((T, W)), rng.standard_normal((T, W)) * 2, 1 + 0.2 * rng.standard_normal(W)
    y[:, : W // groups] *= 25.0
    got = capi.gated_group_norm(y, w, groups, gate=g, eps=1e-4, out_scale=0.5, ld_out=ld)
    close(got[:, :W], 0.5 * O.group_norm(y * O.silu(g), w, groups, 1e-4), F32_TOL)
    assert (got[:, W:] == 0).all()
    close(capi.gated_group_norm(y, w, groups, eps=1e-4), O.group_norm(y, w, groups, 1e-4), F32_TOL)


# ---- whole models ----------------------------------------------------------------------------------------------------------
YARN = {"dims": 4, "base": 80.0, "scaling": {"factor": 3.0, "fast": 6.0, "slow": 0.5, "original": 24}}
CONFIGS = {
    # attention + state space first, a loop over two layers, three norm groups, a layer without a feed-forward
    "mixed": O.make_config(vocab=41, width=24, groups=3, taps=3, scale=3.0, loop=(1, 3, 2), layers=[
        O.parallel_layer(4, 2, 6, 0.3, YARN, 3, 4, 5, 1, 3, 2, 1.3, 0.7, mlp=O.dense(20)),
        O.gla_layer(2, 5, 7, 4.0, rank=3, mlp=O.moe(6, 5, 2)),
        O.gla_layer(3, 4, 4, 8.0, rank=2, mlp=None),
        O.parallel_layer(2, 2, 8, 0.2, {"dims": 8, "base": 30.0}, 4, 3, 6, 4, 2, 1, 0.5, 2.0, mlp=O.moe(5, 3, 3))]),
    # recurrence first; sizes of one: one head, one group, one expert chosen, one tap (no convolution), no rotation, no loop
    "ones": O.make_config(vocab=17, width=16, groups=1, taps=1, bigram=(1, 3, 2), layers=[
        O.gla_layer(1, 6, 5, 1.0, rank=1, mlp=O.moe(4, 3, 1)),
        O.parallel_layer(1, 1, 10, 0.25, None, 1, 8, 4, 1, 1, 1, mlp=O.dense(9))]),
    # the whole model is one loop run three times; head sizes above a warp; taps at the kernels' limit
    "loop_all": O.make_config(vocab=29, width=32, groups=4, taps=5, scale=0.5, loop=(0, 2, 3), layers=[
        O.parallel_layer(6, 3, 40, 0.15, {"dims": 12, "base": 500.0, "scaling": {"factor": 8.0, "fast": 16.0, "slow": 2.0, "original": 40}},
                         4, 36, 33, 2, 8, 4, 0.8, 1.1, mlp=O.moe(7, 4, 4)),
        O.gla_layer(2, 34, 40, 12.0, rank=5, mlp=O.dense(50))]),
    # shapes the tensor-core GEMM takes (K multiples of 64)
    "k64_tiles": O.make_config(vocab=64, width=64, groups=2, taps=4, layers=[
        O.parallel_layer(4, 2, 16, 0.25, {"dims": 8, "base": 100.0}, 4, 16, 16, 4, 3, 1, 0.9, 1.4, mlp=O.dense(128)),
        O.gla_layer(2, 32, 32, 4.0, rank=8, mlp=O.moe(64, 4, 2))]),
}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def case(request):
    cfg = CONFIGS[request.param]
    W = O.random_weights(cfg, seed=len(request.param))
    tokens = np.random.default_rng(11).integers(0, cfg["vocab"], 75).tolist()
    layers = []
    logits = O.forward(cfg, W, tokens, {}, layers)
    return cfg, W, tokens, logits, layers


def on_gpu(cfg, W, precision, chunk=None, max_tokens=256):
    if chunk:
        capi.tune("seq_chunk", chunk)
    try:
        return Model.from_json(cfg, W, "F32" if precision == capi.PRECISION_F32 else "BF16").cuda(max_tokens=max_tokens, precision=precision)
    finally:
        capi.tune("seq_chunk", 256)


def step_all(m, tokens, cuts):
    """Feed `tokens` in portions of the given sizes (the last size repeats), every position's logits."""
    rows, p, i = [], 0, 0
    while p < len(tokens):
        n = min(cuts[min(i, len(cuts) - 1)], len(tokens) - p)
        rows.append(m.prefill(tokens[p:p + n], p, 2).reshape(n, -1))
        p += n
        i += 1
    return np.concatenate(rows)


@pytest.mark.parametrize("precision,tol", [(capi.PRECISION_F32, F32_TOL), (capi.PRECISION_BF16, BF16_TOL)])
def test_prompt_in_one_pass_and_layer_runs(case, precision, tol, monkeypatch):
    cfg, W, tokens, logits, layers = case
    monkeypatch.setenv("XALM_SEQ_KEEP_LAYERS", "1")
    m = on_gpu(cfg, W, precision)
    got = m.prefill(tokens, 0, 2)
    assert m.info("n_layers") == len(O.layer_runs(cfg)) == len(layers)
    if precision == capi.PRECISION_F32:
        close(got, logits, tol)
        for r in range(len(layers)):         # the first run that differs names the mechanism
            close(m.read_state(100 + r, len(tokens) * cfg["width"]).reshape(len(tokens), -1), layers[r], tol)
    else:
        # 16-bit cache rows and operands move a router logit a little: an expert choice decided by less flips, and the recurrent states carry
        # the other expert's output on for some tokens.  Most rows are within rounding of the oracle, and so is every run before the first mixture.
        def row_errors(a, b):
            return np.abs(np.asarray(a, dtype=np.float64) - b).max(axis=1) / max(1.0, np.abs(b).max())
        err = row_errors(got, logits)
        assert np.median(err) < tol / 4 and (err > tol).mean() <= 0.2
        for r, (_, li) in enumerate(O.layer_runs(cfg)):
            e = row_errors(m.read_state(100 + r, len(tokens) * cfg["width"]).reshape(len(tokens), -1), layers[r])
            assert np.median(e) < tol / 4
            if (cfg["layers"][li].get("mlp") or {}).get("kind") == "moe":
                break
            assert e.max() < tol
    m.close()


@pytest.mark.parametrize("chunk", [8, 16, 256])
@pytest.mark.parametrize("cuts", [[1], [2], [3, 2, 7, 1, 30], [40, 1], [75]])
def test_portions_and_token_by_token(case, chunk, cuts):
    """However the prompt is cut — into steps by the caller, into passes by the engine (chunk) — every position's logits agree with the
    oracle: prefill against token-by-token decoding, portions down to two tokens, states, carried rows and cache rows handed from pass to pass."""
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=chunk)
    close(step_all(m, tokens, cuts), logits, F32_TOL)
    m.close()


def rows_within(got, want, tol, share=0.2):
    """16-bit mode: most rows within rounding of the oracle (a bf16 key cache under a sharp softmax, an expert choice flipped on a close call
    and carried on by the recurrent states move a few rows further)."""
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=1) / max(1.0, np.abs(want).max())
    assert np.median(err) < tol / 4 and (err > tol).mean() <= share, f"median {np.median(err):.3e}, over {(err > tol).mean():.2f}"


def test_tensor_core_passes_match_the_fp32_kernels():
    cfg = CONFIGS["k64_tiles"]
    W = O.random_weights(cfg, seed=9)
    tokens = np.random.default_rng(4).integers(0, cfg["vocab"], 130).tolist()
    logits = O.forward(cfg, W, tokens, {})
    launches, outputs = {}, {}
    for tc in (1, 2, 0):
        capi.tune("seq_tc", tc)
        try:
            m = on_gpu(cfg, W, capi.PRECISION_BF16, chunk=64)
        finally:
            capi.tune("seq_tc", 1)
        got = []
        for cuts in ([130], [40, 33, 5, 18, 34]):        # passes of 32 tokens or more take the tensor cores, shorter ones the fp32 kernels
            outputs[tc] = step_all(m, tokens, cuts)
            rows_within(outputs[tc], logits, BF16_TOL)
            got.append(m.last_launch_count())
            m.release()
        m.close()
        launches[tc] = got
    assert launches[1] != launches[0]                    # the tensor-core path really ran (pack + GEMM + epilogue)
    rows_within(outputs[2], outputs[0], BF16_TOL / 4)    # hi + lo operand planes: the fp32 kernels' numbers but for rounding
    rows_within(outputs[1], outputs[0], BF16_TOL)


def test_forward_steps_use_the_graph_and_match(case):
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=16)
    state = InferenceState(m.config)
    m.prefill(tokens[:30], 0, 0)
    for p in range(30, len(tokens)):
        m.forward(state, tokens[p], p)
        close(state.logits(), logits[p], F32_TOL)
    with pytest.raises(capi.XalmError):        # a step must continue where the sequence stands
        m.forward(state, 1, 3)
    m.close()


def test_release_gives_state_and_rows_back(case):
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=8)
    other = [(t * 7 + 3) % cfg["vocab"] for t in tokens]
    for _ in range(2):
        step_all(m, other[:50], [13])          # leaves cache rows, carried rows and states of another sequence behind
        m.release()
        close(step_all(m, tokens, [20, 1, 1, 9]), logits, F32_TOL)
        m.release()
    m.close()


def test_long_decoding():
    cfg = CONFIGS["mixed"]
    W = O.random_weights(cfg, seed=5)
    tokens = np.random.default_rng(2).integers(0, cfg["vocab"], 200).tolist()
    logits = O.forward(cfg, W, tokens, {})
    for precision, tol in ((capi.PRECISION_F32, 4 * F32_TOL), (capi.PRECISION_BF16, BF16_TOL)):
        m = on_gpu(cfg, W, precision, chunk=8, max_tokens=200)
        got = step_all(m, tokens, [4, 1])      # four prompt tokens, then 196 single steps up to the cache's last row
        if precision == capi.PRECISION_F32:
            close(got, logits, tol)
        else:
            # 16-bit cache rows move a router logit a little: an expert choice decided by less flips, and the recurrent states carry the other
            # expert's output on for a few tokens.  Such rows are few; every other row is within rounding.
            err = np.abs(got - logits).max(axis=1) / max(1.0, np.abs(logits).max())
            assert (err > tol).mean() <= 0.05 and np.median(err) < tol / 4
        with pytest.raises(capi.XalmError):    # the cache is full
            m.prefill(tokens[:1], 200, 1)
        m.close()


def test_first_tokens_and_tiny_sequences(case):
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32)
    for n in (1, 2, 3):
        close(m.prefill(tokens[:n], 0, 2), logits[:n], F32_TOL)
        m.release()
    m.close()


def test_a_far_token_decides_the_answer():
    """The attention's sinks are pushed far down and its query / key matrices up, so that single keys dominate: logits then depend on
    tokens hundreds of positions back, in a prompt and when decoding, across pass borders (chunk 64) and key blocks."""
    cfg = O.make_config(vocab=31, width=32, groups=2, taps=2, layers=[
        O.parallel_layer(2, 1, 16, 1.0, {"dims": 4, "base": 10.0}, 2, 8, 8, 1, 2, 1, 1.5, 0.3, mlp=None)])
    W = O.random_weights(cfg, seed=3)
    W["l0.mix.left.q"] = O.bf16_round(W["l0.mix.left.q"] * 3.0)
    W["l0.mix.left.k"] = O.bf16_round(W["l0.mix.left.k"] * 3.0)
    W["l0.mix.left.sink"][:] = -30.0
    tokens = np.random.default_rng(6).integers(0, 31, 600).tolist()
    logits = O.forward(cfg, W, tokens, {})
    other = list(tokens)
    other[15] = (other[15] + 1) % 31
    assert np.abs(O.forward(cfg, W, other, {})[-1] - logits[-1]).max() > 1.0        # position 15 decides the logits at position 599
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=64, max_tokens=600)
    close(step_all(m, tokens, [600]), logits, 2 * F32_TOL)
    m.release()
    close(step_all(m, tokens, [570, 1]), logits, 2 * F32_TOL)
    m.close()


def test_greedy_generation_through_the_host_entry_points(case, tmp_path):
    cfg, W, tokens, _, _ = case
    prompt, steps = tokens[:12], 10
    seq = list(prompt)                         # the oracle generates greedily, recomputing the whole sequence each step
    for _ in range(steps):
        seq.append(int(np.argmax(O.forward(cfg, W, seq, {})[-1])))
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=8)
    state, sampler = InferenceState(m.config), Sampler(m.config)
    assert generate(m, state, sampler, prompt, steps) == seq
    m.release()
    assert generate(m, state, sampler, prompt, steps, portion=5) == seq
    m.close()
    # the same through the command line on a model folder
    ST.write_model_dir(str(tmp_path / "model"), cfg, W, "BF16")
    build.build_host()
    out = subprocess.run([build.MAIN, str(tmp_path / "model"), "-p", "f32", "-T", "64", "-n", str(steps), "-i", " ".join(map(str, prompt))],
                         capture_output=True, text=True, check=True).stdout
    ids = [int(x) for x in out.split("\n")[1].split()]
    assert ids == seq[len(prompt):]


def test_trace_mode_of_the_command_line(case, tmp_path):
    cfg, W, tokens, logits, _ = case
    ST.write_model_dir(str(tmp_path / "model"), cfg, W, "BF16")
    (tmp_path / "out").mkdir()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[32:33], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": tokens[:5], "want": [4]}], "end": ["b"]}]
    runner = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([runner, "--model", str(tmp_path / "model"), "--dtype", "float32", "--out", str(tmp_path / "out"), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, check=True)
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    V = cfg["vocab"]
    close(np.fromfile(tmp_path / "out" / "0.f32", dtype=np.float32).reshape(2, V), logits[[0, 29]], F32_TOL)
    assert not (tmp_path / "out" / "1.f32").exists()
    close(np.fromfile(tmp_path / "out" / "2.f32", dtype=np.float32).reshape(1, V), logits[[32]], F32_TOL)
    close(np.fromfile(tmp_path / "out" / "3.f32", dtype=np.float32).reshape(1, V), logits[[4]], F32_TOL)


def test_config_errors_are_reported():
    cfg = json.loads(json.dumps(CONFIGS["mixed"]))
    cfg["layers"][0]["type"] = "convolution"
    with pytest.raises(capi.XalmError, match="convolution"):
        Model.from_json(cfg, {}).cuda()
    W = O.random_weights(CONFIGS["mixed"], 1)
    del W["l0.mix.left.sink"]
    with pytest.raises(capi.XalmError, match="l0.mix.left.sink"):
        Model.from_json(CONFIGS["mixed"], W).cuda()
    W = O.random_weights(CONFIGS["mixed"], 1)
    W["l1.mix.a2"] = W["l1.mix.a2"][:, :2]
    with pytest.raises(capi.XalmError, match="decay"):
        Model.from_json(CONFIGS["mixed"], W).cuda()
