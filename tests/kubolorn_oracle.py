"""Plain float64 restatement of the Kubolorn design, one function per mechanism, token by token where the design is a recurrence.

Nothing here is shared with the product: the tests hold the CUDA path against these functions.  A model is a dict `cfg` (the parsed
config.json) and a dict `w` of numpy arrays by tensor name.  Notation: `h` is what a sublayer reads (T, width), `p0` the position of
its first row, `state` a dict that carries whatever the sequence keeps between calls (so a prompt can be fed in portions).
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def group_norm(x, w, groups, eps):
    """Each of `groups` equal consecutive parts of a row over its own root mean square; then the weight."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / np.sqrt((parts ** 2).mean(-1, keepdims=True) + eps)
    return parts.reshape(T, W) * w


def short_conv(h, w, hist, bias=None):
    """Causal depthwise convolution over time.  w (channels, taps): the last column multiplies the current row.  hist (taps - 1,
    channels): the rows before h[0], oldest first (zeros at a sequence's start).  Returns (conv(h), new hist)."""
    taps = w.shape[1]
    ext = np.concatenate([hist, h], 0)
    out = np.zeros_like(h)
    for j in range(taps):
        out += ext[j:j + h.shape[0]] * w[:, j]
    if bias is not None:
        out = out + bias
    return out, ext[ext.shape[0] - (taps - 1):]


def embed_rows(cfg, w, tokens, prev):
    """Scaled embedding row + hashed bigram row, then the grouped norm.  prev: the token before tokens[0], None at a sequence's start."""
    e = cfg["embedding"]
    bg = e["bigram"]
    rows = []
    for t in tokens:
        r = bg["buckets"] if prev is None else (prev * bg["mul_prev"] + t * bg["mul_cur"]) % bg["buckets"]
        rows.append(w["embed"][t] * e["scale"] + w["bigram"][r])
        prev = t
    return group_norm(np.stack(rows), w["embed.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"])


def yarn_table(rot):
    """Per rotated pair: the angle's frequency and the magnitude that multiplies cos and sin."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    def dim_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(sc["fast"])), 0)
    hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, pos, rot):
    """x (T, heads, dim); the first rot.dims entries of every head turn, entry i with entry i + dims/2."""
    if not rot or not rot.get("dims"):
        return x
    f, mag = yarn_table(rot)
    half = rot["dims"] // 2
    ang = np.asarray(pos, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def sink_attention(h, mx, w, pre, p0, state):
    """Causal softmax attention whose values are the unrotated keys and whose denominator also holds exp(sink_h)."""
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).reshape(T, H, d)
    k = (h @ w[pre + "k"].T).reshape(T, G, d)
    pos = np.arange(p0, p0 + T)
    qr, kr = rotate(q, pos, mx.get("rot")), rotate(k, pos, mx.get("rot"))
    keys = kr if state.get("k") is None else np.concatenate([state["k"], kr], 0)
    vals = k if state.get("v") is None else np.concatenate([state["v"], k], 0)
    state["k"], state["v"] = keys, vals
    out = np.zeros((T, H, d))
    for t in range(T):
        n = p0 + t + 1
        for hh in range(H):
            g = hh // (H // G)
            s = keys[:n, g] @ qr[t, hh] * mx["scale"]
            m = max(s.max(), w[pre + "sink"][hh])
            e = np.exp(s - m)
            out[t, hh] = (e @ vals[:n, g]) / (e.sum() + math.exp(w[pre + "sink"][hh] - m))
    return out.reshape(T, H * d) @ w[pre + "o"].T


def ssd_mixer(h, mx, w, pre, state, eps):
    """Mamba-2: S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t, per head; gate, grouped norm, projection."""
    H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner, T = H * P, h.shape[0]
    u = h @ w[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    taps = w[pre + "conv"].shape[1]
    hist = state.get("conv")
    if hist is None:
        hist = np.zeros((taps - 1, xbc.shape[1]))
    xbc, state["conv"] = short_conv(xbc, w[pre + "conv"], hist, w[pre + "conv.b"])
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    S = state.get("S")
    if S is None:
        S = np.zeros((H, N, P))
    y = np.zeros((T, H, P))
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = math.exp(-math.exp(w[pre + "A_log"][hh]) * dt[t, hh]) * S[hh] + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + w[pre + "D"][hh] * x[t, hh]
    state["S"] = S
    y = y.reshape(T, inner) * silu(z)
    y = group_norm(y, w[pre + "norm"], mx["norm_groups"], eps)
    return y @ w[pre + "o"].T


def gla_mixer(h, mx, w, pre, state, eps):
    """Gated linear attention: S_t = diag(alpha_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; per-head norm over the value channels, silu gate."""
    H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).reshape(T, H, d)
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    zz = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = (sigmoid(zz) ** (1.0 / mx["tau"])).reshape(T, H, d)
    S = state.get("S")
    if S is None:
        S = np.zeros((H, d, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hij,hi->hj", S, q[t])
    state["S"] = S
    o = o / np.sqrt((o ** 2).mean(-1, keepdims=True) + eps) * w[pre + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    return gelu_tanh(h @ w[pre + "up"].T) @ w[pre + "down"].T


def expert_ff(h, mlp, w, pre):
    """The `top` experts with the largest router logits, weighted by the softmax over those logits; an expert is W_down relu(W_up h)^2."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ w[pre + "router"].T
    out = np.zeros((h.shape[0], w[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-logits[t, e], e))[:top]
        z = logits[t, order]
        p = np.exp(z - z.max())
        p /= p.sum()
        for pe, e in zip(p, order):
            a = np.maximum(h[t] @ w[f"{pre}e{e}.up"].T, 0.0) ** 2
            out[t] += pe * (a @ w[f"{pre}e{e}.down"].T)
    return out


def layer_runs(cfg):
    """(layer index, run index) in the order the layers run: layers start .. stop-1 `times` times in a row, then the rest."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    order = list(range(n))
    if lp and lp.get("times", 1) > 1:
        order = list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))
    return list(enumerate(order))


def forward(cfg, w, tokens, state, keep=None):
    """Runs `tokens` from where `state` (a dict, {} at a sequence's start) stands; returns logits (T, vocab).  keep: a list that receives the
    residual stream after every layer run."""
    eps, groups, taps = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["canon"]["taps"]
    W = cfg["width"]
    p0 = state.get("pos", 0)
    x = embed_rows(cfg, w, tokens, state.get("prev"))
    state["prev"], state["pos"] = tokens[-1], p0 + len(tokens)
    for run, li in layer_runs(cfg):
        lc, pre = cfg["layers"][li], f"l{li}."
        st = state.setdefault(("run", run), {})
        def read(norm, canon, key):
            hn = group_norm(x, w[pre + norm], groups, eps)
            hist = st.get(key)
            if hist is None:
                hist = np.zeros((taps - 1, W))
            c, st[key] = short_conv(hn, w[pre + canon], hist)
            return hn + c
        h1 = read("norm1", "canon1", "c1")
        mx = lc["mixer"]
        if lc["type"] == "gla":
            y = gla_mixer(h1, mx, w, pre + "mix.", st.setdefault("gla", {}), eps)
        elif lc["type"] == "parallel":
            y = mx["left_scale"] * sink_attention(h1, mx["left"], w, pre + "mix.left.", p0, st.setdefault("att", {})) \
                + mx["right_scale"] * ssd_mixer(h1, mx["right"], w, pre + "mix.right.", st.setdefault("ssd", {}), eps)
        else:
            raise ValueError(lc["type"])
        mlp = lc.get("mlp")
        if mlp:
            h2 = read("norm2", "canon2", "c2")
            y = y + (dense_ff(h2, w, pre + "mlp.") if mlp["kind"] == "dense" else expert_ff(h2, mlp, w, pre + "mlp."))
        x = x + y
        if keep is not None:
            keep.append(x.copy())
    return group_norm(x, w["final.norm"], groups, eps) @ w["embed"].T


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this configuration holds, in file order."""
    W, V = cfg["width"], cfg["vocab"]
    taps = cfg["canon"]["taps"]
    out = {"embed": (V, W), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, W), "embed.norm": (W,)}
    for li, lc in enumerate(cfg["layers"]):
        p, mx = f"l{li}.", lc["mixer"]
        out[p + "norm1"] = (W,)
        if lc.get("mlp"):
            out[p + "norm2"] = (W,)
        if lc["type"] == "parallel":
            a, b = mx["left"], mx["right"]
            out[p + "mix.left.q"] = (a["heads"] * a["dim"], W)
            out[p + "mix.left.k"] = (a["kv_heads"] * a["dim"], W)
            out[p + "mix.left.sink"] = (a["heads"],)
            out[p + "mix.left.o"] = (W, a["heads"] * a["vdim"])
            inner, gn = b["heads"] * b["vdim"], b["groups"] * b["state"]
            out[p + "mix.right.in"] = (2 * inner + 2 * gn + b["heads"], W)
            out[p + "mix.right.conv"] = (inner + 2 * gn, b["conv"])
            out[p + "mix.right.conv.b"] = (inner + 2 * gn,)
            for nm in ("dt_bias", "A_log", "D"):
                out[p + "mix.right." + nm] = (b["heads"],)
            out[p + "mix.right.norm"] = (inner,)
            out[p + "mix.right.o"] = (W, inner)
        else:
            H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
            rank = mx.get("rank", 8)
            out[p + "mix.q"] = (H * d, W)
            out[p + "mix.k"] = (H * d, W)
            out[p + "mix.v"] = (H * dv, W)
            out[p + "mix.g"] = (H * dv, W)
            out[p + "mix.o"] = (W, H * dv)
            out[p + "mix.norm"] = (dv,)
            out[p + "mix.a1"] = (rank, W)
            out[p + "mix.a2"] = (H * d, rank)
            out[p + "mix.a2.b"] = (H * d,)
        mlp = lc.get("mlp")
        if mlp and mlp["kind"] == "dense":
            out[p + "mlp.up"] = (mlp["ff"], W)
            out[p + "mlp.down"] = (W, mlp["ff"])
        elif mlp:
            for e in range(mlp["router"]["experts"]):
                out[f"{p}mlp.e{e}.up"] = (mlp["expert"]["ff"], W)
                out[f"{p}mlp.e{e}.down"] = (W, mlp["expert"]["ff"])
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
        out[p + "canon1"] = (W, taps)
        if mlp:
            out[p + "canon2"] = (W, taps)
    out["final.norm"] = (W,)
    return out


# ---- test models -------------------------------------------------------------------------------------------------------------------------
def bf16_round(a):
    """Round to the nearest bfloat16 (ties to even), as float64."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def gla_layer(heads, dim, vdim, tau, rank=4, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}, "mlp": mlp}


def parallel_layer(heads, kv_heads, dim, scale, rot, s_heads, s_vdim, s_state, s_groups, conv, norm_groups, left_scale=1.0, right_scale=1.0, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot:
        left["rot"] = rot
    right = {"heads": s_heads, "vdim": s_vdim, "state": s_state, "groups": s_groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(vocab, width, layers, groups=1, taps=3, eps=1e-5, scale=1.0, bigram=(13, 5, 3), loop=None):
    cfg = {"architecture": "Kubolorn", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps},
           "embedding": {"scale": scale, "bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed):
    """name -> float64 array, every value exactly representable in bfloat16 (so that both storage modes hold the same numbers)."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and not leaf.startswith("canon") and leaf != "conv":
            a = rng.standard_normal(shape) / math.sqrt(shape[1])
            if leaf in ("q", "k", "embed", "bigram"):
                a *= 2.0
            if name in ("embed", "bigram"):
                a *= math.sqrt(shape[1])
        elif leaf.startswith("canon") or leaf == "conv":
            a = 0.4 * rng.standard_normal(shape)
        elif leaf in ("norm", "norm1", "norm2"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "A_log":
            a = rng.uniform(-2.0, 0.5, shape)
        elif leaf == "b" and name.endswith("a2.b"):
            a = 2.0 + rng.standard_normal(shape)         # decays mostly near one, some well below
        else:
            a = 0.5 * rng.standard_normal(shape)         # sink, dt_bias, D, conv.b
        w[name] = bf16_round(a)
    return w
