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


def causal_softmax_attention(q, k, v, scale):
    """q, k (T, H, n), v (T, H, dv): position i sees every j <= i; ordinary softmax; returns (T, H, dv)."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[-1]))
    for h in range(H):
        for i in range(T):
            s = (k[: i + 1, h] @ q[i, h]) * scale
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ v[: i + 1, h]
    return out


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


def retention(h, p, *, H, d, dv, decay, rot_dims, base, eps, state=None, first_pos=0):
    """S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head; o over its root mean square, times silu(W_g h), then W_o.
    Returns the output and the state after the last token."""
    T = h.shape[0]
    h = f64(h)
    pos = np.arange(first_pos, first_pos + T)
    q = (h @ f64(p["q"]).T).reshape(T, H, d)
    k = (h @ f64(p["k"]).T).reshape(T, H, d)
    v = (h @ f64(p["v"]).T).reshape(T, H, dv)
    if rot_dims:
        freqs = rotary_frequencies(rot_dims, base)
        q, k = rotate(q, pos, freqs), rotate(k, pos, freqs)
    k = k * d ** -0.5
    S = np.zeros((H, d, dv)) if state is None else f64(state).copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = rms_norm(o, None, eps).reshape(T, H * dv) * silu(h @ f64(p["g"]).T)
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
