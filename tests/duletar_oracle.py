"""Plain, slow float64 restatement of the Duletar design, one function per mechanism.

It shares nothing with the CUDA path: no cache, no passes, no absorbed products, no fused steps.  Every mixer works on the whole
sequence at once (T rows), keys and values are expanded per head from the latent, the retention is a token-by-token loop over an
explicit state.  Notation: W = model width, H = heads of a mixer, d = per-head query/key size, r = per-head rotated size of a latent
attention, dv = per-head value size, R = latent size of keys and values, Rq = latent size of queries.
"""
import math

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-f64(z)))


def silu(z):
    z = f64(z)
    return z * sigmoid(z)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight (None: no weight)."""
    x = f64(x)
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * f64(w)


def rotary_frequencies(dims, base):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])


def rotate(x, positions, freqs):
    """x (T, ..., n): the first 2 * len(freqs) entries of the last axis turn, entry i with entry i + len(freqs), by positions[t] * freqs[i]."""
    x = f64(x).copy()
    n = len(freqs)
    for t, p in enumerate(positions):
        for i in range(n):
            a = p * freqs[i]
            u, v = x[t, ..., i].copy(), x[t, ..., i + n].copy()
            x[t, ..., i] = u * math.cos(a) - v * math.sin(a)
            x[t, ..., i + n] = v * math.cos(a) + u * math.sin(a)
    return x


def causal_softmax_attention(q, k, v, scale, first_pos=0):
    """q (T, H, n) for positions first_pos .. first_pos + T - 1; k (first_pos + T, H, n), v (first_pos + T, H, dv) for every position from 0:
    position i sees every j <= i; ordinary softmax; returns (T, H, dv)."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[-1]))
    for h in range(H):
        for t in range(T):
            i = first_pos + t
            s = (k[: i + 1, h] @ q[t, h]) * scale
            p = np.exp(s - s.max())
            out[t, h] = (p / p.sum()) @ v[: i + 1, h]
    return out


def attend_latents(q, c, k_rot, uk, uv, *, H, d, r, dv, scale, freqs, first_pos=0, gate=None):
    """Attention of un-turned queries q (T, H (d + r)) at positions first_pos.. over latents c (n, R) and already turned shared keys k_rot (n, r):
    keys and values are expanded per head; returns (T, H dv), times sigmoid(gate) when given."""
    T, n = q.shape[0], c.shape[0]
    q = f64(q).reshape(T, H, d + r)
    k = (f64(c) @ f64(uk).T).reshape(n, H, d)
    v = (f64(c) @ f64(uv).T).reshape(n, H, dv)
    if r:
        q = np.concatenate([q[:, :, :d], rotate(q[:, :, d:], np.arange(first_pos, first_pos + T), freqs)], axis=-1)
        k = np.concatenate([k, np.repeat(f64(k_rot)[:, None, :], H, axis=1)], axis=-1)
    o = causal_softmax_attention(q, k, v, scale, first_pos).reshape(T, H * dv)
    return o if gate is None else o * sigmoid(gate)


def latent(h, w_down, w_norm, rank, eps):
    """The normed latent (the first `rank` rows of the down projection) and whatever rows follow it, un-normed."""
    z = f64(h) @ f64(w_down).T
    return rms_norm(z[:, :rank], w_norm, eps), z[:, rank:]


def latent_attention(h, p, *, H, d, r, dv, R, Rq, scale, base, eps):
    """Rotary latent attention.  p: dict of the mixer's matrices (dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o)."""
    T = h.shape[0]
    pos = np.arange(T)
    cq, _ = latent(h, p["dq"], p["dq.norm"], Rq, eps)
    q = (cq @ f64(p["uq"]).T).reshape(T, H, d + r)
    c, k_rot = latent(h, p["dkv"], p["dkv.norm"], R, eps)
    freqs = rotary_frequencies(r, base)
    q_rot = rotate(q[:, :, d:], pos, freqs)
    k_rot = rotate(k_rot, pos, freqs)                                # one rotated key part for all heads
    k = (c @ f64(p["uk"]).T).reshape(T, H, d)
    v = (c @ f64(p["uv"]).T).reshape(T, H, dv)
    qq = np.concatenate([q[:, :, :d], q_rot], axis=-1)
    kk = np.concatenate([k, np.repeat(k_rot[:, None, :], H, axis=1)], axis=-1)
    o = causal_softmax_attention(qq, kk, v, scale)
    return o.reshape(T, H * dv) @ f64(p["o"]).T, c


def latent_attention_gated(h, p, *, H, d, dv, R, Rq, scale, eps, c_from=None):
    """Latent attention without positions and with a sigmoid output gate.  c_from: another layer's latents (T, R) used instead of an own
    down projection."""
    T = h.shape[0]
    cq, _ = latent(h, p["dq"], p["dq.norm"], Rq, eps)
    q = (cq @ f64(p["uq"]).T).reshape(T, H, d)
    c = c_from if c_from is not None else latent(h, p["dkv"], p["dkv.norm"], R, eps)[0]
    k = (c @ f64(p["uk"]).T).reshape(T, H, d)
    v = (c @ f64(p["uv"]).T).reshape(T, H, dv)
    o = causal_softmax_attention(q, k, v, scale).reshape(T, H * dv)
    o = o * sigmoid(f64(h) @ f64(p["g"]).T)
    return o @ f64(p["o"]).T, c


def retention_heads(q, k, v, *, decay, freqs=None, eps, state=None, first_pos=0, gate=None):
    """q, k (T, H, d), v (T, H, dv): q and k turned, k times d^-1/2, then per head S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t from the
    given state (zero when None); o over its root mean square, times silu(gate) when given.  Returns (T, H dv) and the state after the last token."""
    T, H, d = q.shape
    dv = v.shape[-1]
    q, k, v = f64(q), f64(k), f64(v)
    if freqs is not None and len(freqs):
        pos = np.arange(first_pos, first_pos + T)
        q, k = rotate(q, pos, freqs), rotate(k, pos, freqs)
    k = k * d ** -0.5
    S = np.zeros((H, d, dv)) if state is None else f64(state).copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = rms_norm(o, None, eps).reshape(T, H * dv)
    return (o if gate is None else o * silu(gate)), S


def retention(h, p, *, H, d, dv, decay, rot_dims, base, eps, state=None, first_pos=0):
    """The retention mixer on its input rows h; returns the output and the state after the last token."""
    T = h.shape[0]
    h = f64(h)
    q = (h @ f64(p["q"]).T).reshape(T, H, d)
    k = (h @ f64(p["k"]).T).reshape(T, H, d)
    v = (h @ f64(p["v"]).T).reshape(T, H, dv)
    o, S = retention_heads(q, k, v, decay=decay, freqs=rotary_frequencies(rot_dims, base) if rot_dims else None, eps=eps, state=state, first_pos=first_pos,
                           gate=h @ f64(p["g"]).T)
    return o @ f64(p["o"]).T, S


def dense_ff(h, up, down):
    """W_down relu(W_up h)^2."""
    z = np.maximum(f64(h) @ f64(up).T, 0.0)
    return (z * z) @ f64(down).T


def expert(h, gate, up, down, limit):
    g = np.minimum(f64(h) @ f64(gate).T, limit)
    u = np.clip(f64(h) @ f64(up).T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ f64(down).T


def route(h, router, *, top, n_groups=0, keep_groups=0):
    """Softmax scores over all experts; with groups, only experts of the keep_groups groups with the largest best score can be chosen;
    the `top` largest scores are chosen and divided by their sum.  Returns per row (chosen experts, weights)."""
    z = f64(h) @ f64(router).T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s = s / s.sum(axis=-1, keepdims=True)
    E = s.shape[-1]
    out = []
    for row in s:
        allowed = np.ones(E, bool)
        if n_groups and n_groups > 1:
            gsz = E // n_groups
            best = row.reshape(n_groups, gsz).max(axis=1)
            kept = np.argsort(-best, kind="stable")[:keep_groups]
            allowed = np.zeros(E, bool)
            for g in kept:
                allowed[g * gsz:(g + 1) * gsz] = True
        masked = np.where(allowed, row, -np.inf)
        idx = np.argsort(-masked, kind="stable")[:top]
        w = row[idx] / (row[idx].sum() + 1e-20)
        out.append((idx, w))
    return out


def moe_ff(h, router, experts, *, top, limit, n_groups=0, keep_groups=0):
    """experts: list of (gate, up, down)."""
    h = f64(h)
    out = np.zeros((h.shape[0], experts[0][2].shape[0]))
    for t, (idx, w) in enumerate(route(h, router, top=top, n_groups=n_groups, keep_groups=keep_groups)):
        for e, we in zip(idx, w):
            out[t] += we * expert(h[t:t + 1], *experts[e], limit)[0]
    return out


def softcap(z, cap):
    return cap * np.tanh(f64(z) / cap) if cap else f64(z)


def forward(cfg, w, tokens, return_layers=False):
    """The whole model on one sequence from position 0.  cfg: the config dict; w: name -> array.  Returns logits (T, vocab) and, asked
    for, the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = f64(w["embed"])[np.asarray(tokens)] * cfg["embedding"]["scale"]
    latents, sums = {}, []
    for li, L in enumerate(cfg["layers"]):
        pre = f"l{li}."
        mx = L["mixer"]
        p = {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mix.")}
        h = rms_norm(x, w[pre + "norm1"], eps)
        if L["type"] == "latent_attention":
            y, latents[li] = latent_attention(h, p, H=mx["heads"], d=mx["dim"], r=mx["rot_dim"], dv=mx["vdim"], R=mx["kv_rank"], Rq=mx["q_rank"],
                                              scale=mx["scale"], base=mx["rot"]["base"], eps=eps)
        elif L["type"] == "latent_attention_2":
            y, latents[li] = latent_attention_gated(h, p, H=mx["heads"], d=mx["dim"], dv=mx["vdim"], R=mx["kv_rank"], Rq=mx["q_rank"], scale=mx["scale"],
                                                    eps=eps, c_from=latents[mx["kv_from"]] if "kv_from" in mx else None)
        elif L["type"] == "retention":
            rot = mx.get("rot") or {}
            y, _ = retention(h, p, H=mx["heads"], d=mx["dim"], dv=mx["vdim"], decay=mx["decay"], rot_dims=rot.get("dims", 0), base=rot.get("base", 1.0),
                             eps=eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        ml = L.get("mlp")
        if ml:
            h = rms_norm(x, w[pre + "norm2"], eps)
            if ml["kind"] == "dense":
                x = x + dense_ff(h, w[pre + "mlp.up"], w[pre + "mlp.down"])
            else:
                r = ml["router"]
                ex = [(w[f"{pre}mlp.e{e}.gate"], w[f"{pre}mlp.e{e}.up"], w[f"{pre}mlp.e{e}.down"]) for e in range(r["experts"])]
                g = r.get("groups") or {}
                x = x + moe_ff(h, w[pre + "mlp.router"], ex, top=r["top"], limit=ml["expert"]["limit"], n_groups=g.get("count", 0),
                               keep_groups=g.get("keep", 0))
        sums.append(x.copy())
    logits = softcap(rms_norm(x, w["final.norm"], eps) @ f64(w["head"]).T, cfg.get("logit_softcap", 0))
    return (logits, np.stack(sums)) if return_layers else logits


# ---- small configurations and random weights for the tests -----------------------------------------------------------------------------
def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=0, keep=0, limit=1.5):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, scale=None, mlp=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale or (dim + rot_dim) ** -0.5,
          "rot": {"base": base, "dims": rot_dim}}
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def gated_latent_layer(heads, dim, vdim, kv_rank, q_rank, scale=None, kv_from=None, mlp=None):
    mx = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale or dim ** -0.5}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention_2", "mixer": mx, "mlp": mlp}


def retention_layer(heads, dim, vdim, decay, rot_dims=0, base=10000.0, mlp=None):
    mx = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        mx["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "retention", "mixer": mx, "mlp": mlp}


def make_config(vocab, width, layers, eps=1e-6, embed_scale=1.0, softcap=0.0):
    c = {"architecture": "Duletar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}
    if softcap:
        c["logit_softcap"] = softcap
    return c


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def random_weights(cfg, seed):
    """name -> fp32 array, every value exactly representable in bfloat16 (so that both storage modes hold the same numbers)."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    w = {}

    def mat(name, rows, cols, gain=1.0):
        w[name] = bf16_round(rng.standard_normal((rows, cols)) * gain / math.sqrt(cols))

    def vec(name, n):
        w[name] = bf16_round(1.0 + 0.2 * rng.standard_normal(n))

    w["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], W)))
    for li, L in enumerate(cfg["layers"]):
        p, mx = f"l{li}.", L["mixer"]
        H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
        vec(p + "norm1", W)
        if L["type"] == "retention":
            mat(p + "mix.q", H * d, W, 2.0); mat(p + "mix.k", H * d, W, 2.0); mat(p + "mix.v", H * dv, W); mat(p + "mix.g", H * dv, W)
        else:
            r, R, Rq = mx.get("rot_dim", 0), mx["kv_rank"], mx["q_rank"]
            mat(p + "mix.dq", Rq, W); vec(p + "mix.dq.norm", Rq); mat(p + "mix.uq", H * (d + r), Rq, 2.0)
            if "kv_from" not in mx:
                mat(p + "mix.dkv", R + r, W); vec(p + "mix.dkv.norm", R)
            mat(p + "mix.uk", H * d, R, 2.0); mat(p + "mix.uv", H * dv, R)
            if L["type"] == "latent_attention_2":
                mat(p + "mix.g", H * dv, W)
        mat(p + "mix.o", W, H * dv)
        ml = L.get("mlp")
        if ml:
            vec(p + "norm2", W)
            if ml["kind"] == "dense":
                mat(p + "mlp.up", ml["ff"], W); mat(p + "mlp.down", W, ml["ff"])
            else:
                ff = ml["expert"]["ff"]
                for e in range(ml["router"]["experts"]):
                    mat(f"{p}mlp.e{e}.gate", ff, W, 2.0); mat(f"{p}mlp.e{e}.up", ff, W, 2.0); mat(f"{p}mlp.e{e}.down", W, ff)
                mat(p + "mlp.router", ml["router"]["experts"], W, 3.0)
    vec("final.norm", W)
    mat("head", cfg["vocab"], W, 3.0)
    return w
