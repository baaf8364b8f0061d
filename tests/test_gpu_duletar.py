"""Duletar on the GPU against the plain restatement in tests/duletar_oracle.py: every mechanism alone (op-level entry points that launch
the family's kernels), then whole models with small random configurations — prompts in one pass, token by token, in portions, after a
release, long decoding, greedy generation through the host entry points and the command line."""
import json
import os
import subprocess

import numpy as np
import pytest

import duletar_oracle as O
from xalm_b200 import build, capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import InferenceState, Model, Sampler, generate

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4   # IEEE fp32 path against float64, on values of order one
BF16_TOL = 6e-2  # serving mode: bf16 weights (exact here), a bf16 latent cache, fp16 operands on the tensor cores


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err < tol, f"max error {err:.3e} (tolerance {tol})"


# ---- mechanisms alone ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,N,K", [(1, 7, 24), (3, 66, 40), (9, 33, 17), (70, 130, 64)])
def test_row_product_epilogues(T, N, K):
    rng = np.random.default_rng(T + N)
    x, w = rng.standard_normal((T, K)), rng.standard_normal((N, K)) / np.sqrt(K)
    z = x @ w.T
    close(capi.rows_act(x, w, act=1), np.maximum(z, 0) ** 2, F32_TOL)                         # relu squared: negative columns are exactly 0
    assert (capi.rows_act(x, w, act=1)[z < -1e-3] == 0).all()
    close(capi.rows_act(x, w * 9, cap=4.0), 4.0 * np.tanh(9 * z / 4.0), F32_TOL)              # soft cap: |z| well past the cap
    g = rng.standard_normal((T, N)) * 3
    close(capi.rows_act(x, w, mul=g, mul_act=2), z * O.sigmoid(g), F32_TOL)
    close(capi.rows_act(x, w, mul=g, mul_act=3), z * O.silu(g), F32_TOL)
    wb = O.bf16_round(w)
    close(capi.rows_act(x, wb, act=1, w_bf16=True), np.maximum(x @ wb.T, 0) ** 2, F32_TOL)


@pytest.mark.parametrize("q_rank,kv_rank,rot", [(10, 12, 6), (33, 7, 0), (5, 130, 34), (600, 520, 64)])
def test_latent_post_norms_turn_and_rows(q_rank, kv_rank, rot):
    rng = np.random.default_rng(q_rank + rot)
    T, pos0, ring = 6, 1000, 1004                                  # positions 1000 .. 1005 of a cache of 1004 rows: the last two wrap
    proj = rng.standard_normal((T, q_rank + kv_rank + rot)) * 3
    proj[:, q_rank:q_rank + kv_rank] *= 20.0                       # a loud kv latent: a norm taken over the wrong columns would show
    qn, kn = 1 + 0.3 * rng.standard_normal(q_rank), 1 + 0.3 * rng.standard_normal(kv_rank)
    freqs = O.rotary_frequencies(rot, 300.0) if rot else None
    cq, cache = capi.latent_post(proj, pos0, q_rank, kv_rank, rot, qn, kn, freqs, eps=1e-4, ring=ring)
    close(cq, O.rms_norm(proj[:, :q_rank], qn, 1e-4), F32_TOL)
    want_c = O.rms_norm(proj[:, q_rank:q_rank + kv_rank], kn, 1e-4)
    want_k = O.rotate(proj[:, q_rank + kv_rank:], np.arange(pos0, pos0 + T), freqs) if rot else np.zeros((T, 0))
    for t in range(T):
        row = cache[(pos0 + t) % ring]
        close(row[:kv_rank], want_c[t], F32_TOL)
        if rot:
            close(row[kv_rank:], want_k[t], 2e-3)                      # angles near 1000 rad in fp32
    _, cache16 = capi.latent_post(proj, pos0, q_rank, kv_rank, rot, qn, kn, freqs, eps=1e-4, ring=ring, cache_bf16=True)
    assert (cache16 == O.bf16_round(cache16)).all()
    close(cache16[(pos0 + 1) % ring][:kv_rank], want_c[1], 1e-2)


def latent_case(rng, n, H, d, r, dv, R, extra=0):
    c, k_rot = rng.standard_normal((n, R)), rng.standard_normal((n, r))
    rows = np.concatenate([c, k_rot, 7 * np.ones((n, extra))], axis=1)   # `extra`: another layer's columns that this one must not read
    uk, uv = rng.standard_normal((H * d, R)) / np.sqrt(R), rng.standard_normal((H * dv, R)) / np.sqrt(R)
    return c, k_rot, rows, uk, uv


@pytest.mark.parametrize("H,d,r,dv,R", [(4, 8, 6, 12, 16), (1, 5, 0, 7, 12), (3, 16, 2, 4, 40), (2, 64, 32, 48, 72), (6, 3, 4, 5, 9),
                                       (32, 4, 2, 3, 560)])   # the last: 32 heads over a latent of 560 do not fit one CTA; the heads run in two launches
@pytest.mark.parametrize("T,pos0", [(1, 0), (1, 200), (3, 97), (40, 0), (37, 60)])
def test_latent_attention_over_rows(H, d, r, dv, R, T, pos0):
    """Queries mapped into the latent, one shared key/value head read in place, values expanded afterwards: the same numbers as keys and
    values expanded per head.  One, a few and many queries take three different kernels; pos0 > 0 reads rows of earlier steps."""
    rng = np.random.default_rng(H * d + T + pos0)
    n = pos0 + T
    c, k_rot, rows, uk, uv = latent_case(rng, n, H, d, r, dv, R)
    q, gate = rng.standard_normal((T, H * (d + r))), rng.standard_normal((T, H * dv))
    freqs = O.rotary_frequencies(r, 50.0) if r else None
    scale = 0.7 / np.sqrt(d + r)
    want = O.attend_latents(q, c, k_rot, uk, uv, H=H, d=d, r=r, dv=dv, scale=scale, freqs=freqs, first_pos=pos0)
    close(capi.latent_attend(q, rows, pos0, H, d, r, dv, R, uk, uv, scale, freqs), want, F32_TOL)
    close(capi.latent_attend(q, rows, pos0, H, d, r, dv, R, uk, uv, scale, freqs, gate=gate, n_splits=3), want * O.sigmoid(gate), F32_TOL)


@pytest.mark.parametrize("T,pos0,far", [(1, 700, 3), (1, 700, 699), (2, 350, 31), (2, 350, 32), (48, 400, 0), (48, 400, 430)])
@pytest.mark.parametrize("n_splits", [0, 1, 5])
def test_latent_attention_finds_one_far_key(T, pos0, far, n_splits):
    """One key among hundreds matches the last query far better than the rest (both scaled up): the output is that position's value, wherever
    the key sits — the first row, a key-block border (32), another split's share, a row written by this very step."""
    H, d, r, dv, R, extra = 2, 8, 4, 6, 16, 5
    rng = np.random.default_rng(far + T)
    n = pos0 + T
    c, k_rot, rows, uk, uv = latent_case(rng, n, H, d, r, dv, R, extra)
    q = rng.standard_normal((T, H * (d + r))) * 0.1
    kf = (c[far] @ uk.T).reshape(H, d)
    for h in range(H):
        q[-1, h * (d + r): h * (d + r) + d] = 6.0 * kf[h] / np.linalg.norm(kf[h])     # the last query points at the far key's expansion
    rows[far, :R] *= 5.0
    c = rows[:, :R].copy()
    freqs = O.rotary_frequencies(r, 50.0)
    want = O.attend_latents(q, c, k_rot, uk, uv, H=H, d=d, r=r, dv=dv, scale=1.0, freqs=freqs, first_pos=pos0)
    got = capi.latent_attend(q, rows, pos0, H, d, r, dv, R, uk, uv, 1.0, freqs, n_splits=n_splits)
    close(got, want, F32_TOL)
    close(got[-1], (c[far] @ uv.T), 2e-2)                                                 # the softmax is all but one-hot
    got16 = capi.latent_attend(q, O.bf16_round(rows), pos0, H, d, r, dv, R, O.bf16_round(uk), O.bf16_round(uv), 1.0, freqs, n_splits=n_splits,
                               cache_bf16=True, w_bf16=True)
    c16 = O.bf16_round(c)
    close(got16, O.attend_latents(q, c16, O.bf16_round(k_rot), O.bf16_round(uk), O.bf16_round(uv), H=H, d=d, r=r, dv=dv, scale=1.0, freqs=freqs,
                                  first_pos=pos0), F32_TOL)


@pytest.mark.parametrize("H,d,dv,rot_dims", [(3, 8, 12, 8), (2, 5, 7, 0), (1, 64, 130, 16), (4, 40, 16, 40), (2, 132, 24, 6), (1, 260, 9, 4), (2, 16, 1000, 0)])
def test_retention_states_and_cuts(H, d, dv, rot_dims):
    """The recurrence in the kernels' column layout (registers, one to eight channels per lane), the cluster per head, and the one-CTA
    fallback (d > 256); state handed over cuts of 2, 1, 1 and 17 tokens at positions that matter to the turn."""
    rng = np.random.default_rng(H * d + dv)
    T, pos0 = 21, 90
    q, k = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d))
    v, gate = rng.standard_normal((T, H, dv)), rng.standard_normal((T, H * dv))
    decay = [1.0, 0.5, 0.97, 0.999, 0.25][:H]                      # no two heads alike: a head reading another's decay would show
    freqs = O.rotary_frequencies(rot_dims, 40.0) if rot_dims else None
    s0 = rng.standard_normal((H, d, dv))
    want, s_want = O.retention_heads(q, k, v, decay=decay, freqs=freqs, eps=1e-5, state=s0, first_pos=pos0, gate=gate)
    flat = lambda a: a.reshape(T, -1)
    got, s_got = capi.retention(flat(q), flat(k), flat(v), s0, H, d, dv, decay, pos0=pos0, freq=freqs, gate=gate, eps=1e-5)
    close(got, want, 4 * F32_TOL)
    close(s_got, s_want, F32_TOL)
    st, at, rows = s0, 0, []
    for n in (2, 1, 1, 17):
        o, st = capi.retention(flat(q)[at:at + n], flat(k)[at:at + n], flat(v)[at:at + n], st, H, d, dv, decay, pos0=pos0 + at, freq=freqs,
                               gate=gate[at:at + n], eps=1e-5)
        rows.append(o)
        at += n
    close(np.concatenate(rows), want, 4 * F32_TOL)
    close(st, s_want, F32_TOL)
    no_gate, _ = capi.retention(flat(q), flat(k), flat(v), s0, H, d, dv, decay, pos0=pos0, freq=freqs, eps=1e-5)
    close(no_gate, O.retention_heads(q, k, v, decay=decay, freqs=freqs, eps=1e-5, state=s0, first_pos=pos0)[0], 4 * F32_TOL)


def test_retention_reads_a_value_back_after_500_tokens():
    H, d, dv, T = 2, 16, 8, 500
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((T, H, x)) * 0.01 for x in (d, d, dv))
    key = rng.standard_normal((H, d))
    k[0], v[0] = 30 * key, 5 + rng.standard_normal((H, dv))       # written once, at the first token
    q[-1] = key                                                    # asked for at the last
    decay = [0.999, 0.9]                                           # head 0 still holds it (0.999^499 = 0.61), head 1 has lost it (0.9^499 = 1.5e-23)
    want, _ = O.retention_heads(q, k, v, decay=decay, eps=1e-6)
    got, _ = capi.retention(q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), np.zeros((H, d, dv)), H, d, dv, decay, eps=1e-6)
    close(got, want, 4 * F32_TOL)
    direction = v[0, 0] / np.sqrt(np.mean(v[0, 0] ** 2))
    close(got[-1, :dv], direction, 5e-2)                           # head 0's normed output is the stored value's direction


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (12, 2, 4, 2), (6, 6, 0, 0), (5, 1, 5, 2), (9, 4, 3, 2), (40, 5, 0, 0)])
def test_softmax_router_groups_weights_and_clamped_experts(E, top, groups, keep):
    rng = np.random.default_rng(E * top)
    T, K, ff, limit = 11, 24, 10, 0.8
    h = rng.standard_normal((T, K))
    wr = rng.standard_normal((E, K)) / 2
    wg, wu, wd = rng.standard_normal((E, ff, K)) / 2, rng.standard_normal((E, ff, K)) / 2, rng.standard_normal((E, K, ff)) / 3
    x = rng.standard_normal((T, K))
    idx, wgt, out, xo = capi.moe_ffn_routed(h, wr, wg, wu, wd, top, groups, keep, act=0, limit=limit, x=x)
    want = O.route(h, wr, top=top, n_groups=groups, keep_groups=keep)
    acc = x.copy()
    for t in range(T):
        assert list(idx[t]) == list(want[t][0])
        close(wgt[t], want[t][1], F32_TOL)
        assert abs(wgt[t].sum() - 1) < 1e-5
        for s_, e in enumerate(idx[t]):
            y = O.expert(h[t:t + 1], wg[e], wu[e], wd[e], limit)[0]   # gate and up beyond +-0.8 are clamped for most entries
            close(out[t, s_], y, F32_TOL)
            acc[t] += want[t][1][s_] * y
    close(xo, acc, F32_TOL)


def test_router_group_limit_passes_over_a_large_score():
    """Two groups of three, one kept.  Expert 4 has the second largest score overall but lies in the group whose best is smaller: it is not
    chosen.  A group scoring the sum of its two best would have kept the other group."""
    K = 8
    h = np.zeros((1, K)); h[0, 0] = 1.0
    wr = np.zeros((6, K))
    wr[:, 0] = [3.0, -4.0, -4.0, 2.9, 2.8, -4.0]                   # logits; group 0 best 3.0, group 1 best 2.9 (its two best sum to far more)
    z = np.zeros((6, 4, K))
    idx, wgt, _, _ = capi.moe_ffn_routed(h, wr, z, z, np.zeros((6, K, 4)), 2, 2, 1)
    assert list(idx[0]) == [0, 1]
    s = np.exp(wr[:, 0]) / np.exp(wr[:, 0]).sum()
    close(wgt[0], s[[0, 1]] / s[[0, 1]].sum(), F32_TOL)
    idx, _, _, _ = capi.moe_ffn_routed(h, wr, z, z, np.zeros((6, K, 4)), 2, 2, 1, group="top2")
    assert list(idx[0]) == [3, 4]


# ---- whole models ---------------------------------------------------------------------------------------------------------
CONFIGS = {
    # every mixer and feed-forward kind; a gated layer reading a gated layer's rows and one reading a rotary layer's rows (row stride R + r)
    "mixed": O.make_config(vocab=67, width=48, embed_scale=3.5, softcap=9.0, layers=[
        O.retention_layer(3, 8, 12, [0.9, 0.99, 0.5], rot_dims=4, base=200.0, mlp=O.dense(56)),
        O.gated_latent_layer(4, 8, 6, 20, 14, mlp=O.moe(10, 6, 2, groups=3, keep=2)),
        O.latent_layer(3, 8, 6, 10, 20, 18, base=500.0, mlp=O.moe(6, 4, 4)),
        O.gated_latent_layer(2, 12, 9, 20, 10, kv_from=1, scale=0.3, mlp=None),
        O.gated_latent_layer(5, 4, 4, 20, 7, kv_from=2, mlp=O.dense(24)),
        O.retention_layer(2, 10, 5, [1.0, 0.75], mlp=O.moe(8, 5, 1, groups=5, keep=2, limit=0.6))]),
    # attention first, one head, sizes of 1, no soft cap, embedding as it is, rotation on the whole head of the retention
    "latent_first": O.make_config(vocab=31, width=40, eps=1e-3, layers=[
        O.latent_layer(1, 5, 2, 7, 9, 6, base=50.0, mlp=None),
        O.retention_layer(1, 6, 1, [0.8], rot_dims=6, base=30.0, mlp=O.moe(12, 3, 3, limit=4.0)),
        O.gated_latent_layer(1, 1, 1, 3, 2, mlp=O.dense(20))]),
    # every product a whole number of 64-wide K tiles: the 16-bit mode's long passes run on the tensor cores
    "k64_tiles": O.make_config(vocab=68, width=64, embed_scale=8.0, softcap=20.0, layers=[
        O.latent_layer(4, 16, 16, 16, 64, 64, mlp=O.dense(128)),
        O.gated_latent_layer(2, 32, 32, 64, 64, kv_from=0, mlp=O.moe(64, 4, 2, groups=2, keep=1)),
        O.retention_layer(4, 16, 16, [0.97, 0.99, 0.995, 0.9], rot_dims=16, mlp=O.dense(64))]),
    # a wide retention head (state in shared memory), many heads over a small latent
    "wide": O.make_config(vocab=90, width=72, softcap=5.0, layers=[
        O.retention_layer(1, 260, 9, [0.95], rot_dims=8, mlp=None),
        O.gated_latent_layer(8, 12, 20, 10, 30, mlp=O.moe(5, 7, 3)),
        O.latent_layer(6, 6, 10, 3, 33, 12, base=1e6, mlp=O.dense(30))]),
}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def case(request):
    cfg = CONFIGS[request.param]
    W = O.random_weights(cfg, seed=len(request.param))
    rng = np.random.default_rng(11)
    tokens = rng.integers(0, cfg["vocab"], 75).tolist()
    logits, layers = O.forward(cfg, W, tokens, return_layers=True)
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
def test_prompt_in_one_pass_and_layers(case, precision, tol, monkeypatch):
    cfg, W, tokens, logits, layers = case
    monkeypatch.setenv("XALM_SEQ_KEEP_LAYERS", "1")
    m = on_gpu(cfg, W, precision)
    close(m.prefill(tokens, 0, 2), logits, tol)
    for l in range(len(cfg["layers"])):      # the first layer that differs names the mechanism
        close(m.read_state(100 + l, len(tokens) * cfg["width"]).reshape(len(tokens), -1), layers[l], tol)
    m.close()


@pytest.mark.parametrize("chunk", [8, 16, 256])
@pytest.mark.parametrize("cuts", [[1], [2], [3, 2, 7, 1, 30], [40, 1], [75]])
def test_portions_and_token_by_token(case, chunk, cuts):
    """However the prompt is cut — into steps by the caller, into passes by the engine (chunk) — every position's logits agree with the
    oracle: prefill against token-by-token decoding, portions down to two tokens, the state and the cache rows handed from pass to pass."""
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=chunk)
    close(step_all(m, tokens, cuts), logits, F32_TOL)
    m.close()


def test_tensor_core_passes_match_the_fp32_kernels():
    cfg = CONFIGS["k64_tiles"]
    W = O.random_weights(cfg, seed=9)
    tokens = np.random.default_rng(4).integers(0, cfg["vocab"], 130).tolist()
    logits = O.forward(cfg, W, tokens)
    launches = {}
    for tc in (1, 2, 0):
        capi.tune("seq_tc", tc)
        try:
            m = on_gpu(cfg, W, capi.PRECISION_BF16, chunk=64)
        finally:
            capi.tune("seq_tc", 1)
        got = []
        for cuts in ([130], [40, 33, 5, 18, 34]):        # passes of 32 tokens or more take the tensor cores, shorter ones the fp32 kernels
            close(step_all(m, tokens, cuts), logits, BF16_TOL)
            got.append(m.last_launch_count())
            m.release()
        m.close()
        launches[tc] = got
    assert launches[1] != launches[0]                    # the tensor-core path really ran (pack + GEMM + epilogue)


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
        step_all(m, other[:50], [13])          # leaves the cache rows full of another sequence and the recurrent states non-zero
        m.release()
        close(step_all(m, tokens, [20, 1, 1, 9]), logits, F32_TOL)
        m.release()
    m.close()


def test_long_decoding():
    cfg = O.make_config(vocab=50, width=32, embed_scale=2.0, softcap=7.0, layers=[
        O.latent_layer(2, 4, 4, 6, 8, 8, base=20.0, mlp=O.moe(6, 4, 2, groups=2, keep=1)),
        O.retention_layer(2, 6, 4, [0.99, 0.9], rot_dims=2, base=7.0, mlp=O.dense(20)),
        O.gated_latent_layer(3, 5, 2, 8, 4, kv_from=0, mlp=None)])
    W = O.random_weights(cfg, seed=5)
    tokens = np.random.default_rng(2).integers(0, 50, 200).tolist()
    logits = O.forward(cfg, W, tokens)
    for precision, tol in ((capi.PRECISION_F32, 4 * F32_TOL), (capi.PRECISION_BF16, BF16_TOL)):
        m = on_gpu(cfg, W, precision, chunk=8, max_tokens=200)
        got = step_all(m, tokens, [4, 1])      # four prompt tokens, then 196 single steps up to the cache's last row
        if precision == capi.PRECISION_F32:
            close(got, logits, tol)
        else:
            # 16-bit cache rows move a router logit by about 1e-2: an expert choice decided by less flips, and the retention state carries
            # the other expert's output on for a few tokens.  Such rows are few; every other row is within rounding.
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


def test_greedy_generation_through_the_host_entry_points(case, tmp_path):
    cfg, W, tokens, _, _ = case
    prompt, steps = tokens[:12], 10
    seq = list(prompt)                         # the oracle generates greedily, recomputing the whole sequence each step
    for _ in range(steps):
        seq.append(int(np.argmax(O.forward(cfg, W, seq)[-1])))
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
    del W["l2.mix.dkv.norm"]
    with pytest.raises(capi.XalmError, match="l2.mix.dkv.norm"):
        Model.from_json(CONFIGS["mixed"], W).cuda()
