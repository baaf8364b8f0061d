"""ctypes binding of the C ABI in include/xalm_cuda.h (libxalm_cuda.so).

Fails loudly: if the shared library is missing it is (re)built with nvcc; if that is impossible, or no CUDA
device is present, the calls raise — there is no CPU or PyTorch fallback behind this module.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

HYDRATE_KV_CACHE, OUTPUT_LOGITS = 0, 1          # InferenceMode, model.h:249-252
GELU, SILU = 0, 1                               # ActivationType, model.h:12-15
S_X, S_XB2, S_HB, S_Q, S_LOGITS = 0, 2, 3, 5, 9


class XalmError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"xalm_cuda status {status}: {msg}")
        self.status = status


class XalmConfig(C.Structure):
    # xalm_config (include/xalm_cuda.h) == Config (model.h:25-42)
    _fields_ = [("dim", C.c_int), ("hidden_dim", C.c_int), ("head_dim", C.c_int), ("n_layers", C.c_int),
                ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("vocab_size", C.c_int), ("max_seq_len", C.c_int),
                ("rope_theta", C.c_float), ("rotary_dim", C.c_int), ("norm_eps", C.c_float), ("act", C.c_int),
                ("norm_type", C.c_int), ("qkv_clip", C.c_float), ("tie_word_embeddings", C.c_int)]

    @classmethod
    def from_dict(cls, c: dict) -> "XalmConfig":
        return cls(c["dim"], c["hidden_dim"], c["head_dim"], c["n_layers"], c["n_heads"], c["n_kv_heads"], c["vocab_size"],
                   c["max_seq_len"], c["rope_theta"], c["rotary_dim"], c["norm_eps"], c["act"], c.get("norm_type", 0),
                   c.get("qkv_clip", float(np.finfo(np.float32).max)), int(c["tie_word_embeddings"]))


# every symbol include/xalm_cuda.h declares: (restype, argtypes)
_vp, _i, _sz, _fp = C.c_void_p, C.c_int, C.c_size_t, C.POINTER(C.c_float)
SYMBOLS = {
    "xalm_cuda_abi_version": (_i, []),
    "xalm_cuda_last_error": (C.c_char_p, []),
    "xalm_cuda_device_count": (_i, [C.POINTER(_i)]),
    "xalm_cuda_type_info": (_i, [_i, C.POINTER(_i), C.POINTER(_i)]),
    "xalm_cuda_create": (_i, [C.POINTER(XalmConfig), _i, _i, _i, C.POINTER(_vp)]),
    "xalm_cuda_upload_tensor": (_i, [_vp, C.c_char_p, _i, C.POINTER(_i), _i, _vp, _sz]),
    "xalm_cuda_host_alloc": (_vp, [_sz]),
    "xalm_cuda_host_free": (None, [_vp]),
    "xalm_cuda_shard_range": (_i, [_vp, C.c_char_p, C.POINTER(_i)]),
    "xalm_cuda_upload_tensor_shard": (_i, [_vp, C.c_char_p, _i, C.POINTER(_i), _i, C.POINTER(_i), _vp, _sz]),
    "xalm_cuda_finalize": (_i, [_vp]),
    "xalm_cuda_destroy": (None, [_vp]),
    "xalm_cuda_comm_unique_id": (_i, [_vp]),
    "xalm_cuda_comm_init": (_i, [_vp, _vp]),
    "xalm_cuda_ipc_export": (_i, [_vp, _vp]),
    "xalm_cuda_ipc_import": (_i, [_vp, _vp]),
    "xalm_cuda_set_stream": (_i, [_vp, _vp]),
    "xalm_cuda_forward": (_i, [_vp, _i, _i, _i, _vp]),
    "xalm_cuda_forward_async": (_i, [_vp, _i, _i, _i]),
    "xalm_cuda_forward_argmax": (_i, [_vp, _i, _i, C.POINTER(_i)]),
    "xalm_cuda_sync": (_i, [_vp]),
    "xalm_cuda_logits_host": (_fp, [_vp]),
    "xalm_cuda_active_bytes": (_i, [_vp, C.c_longlong, C.POINTER(C.c_longlong)]),
    "xalm_cuda_last_launch_count": (_i, [_vp, C.POINTER(_i)]),
    "xalm_cuda_read_state": (_i, [_vp, _i, _vp, _sz]),
    "xalm_cuda_read_kv": (_i, [_vp, _i, _i, _vp, _sz]),
    "xalm_cuda_dequant": (_i, [_i, _vp, _sz, _vp]),
    "xalm_cuda_matmul": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "xalm_cuda_mha": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "xalm_cuda_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, C.c_float]),
    "xalm_cuda_rope": (_i, [_vp, _i, _i, _i, C.c_float, _i]),
    "xalm_cuda_ffn": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "xalm_cuda_tune": (_i, [C.c_char_p, _i]),
    "xalm_cuda_timeline": (_i, [_i, _vp, C.POINTER(_i)]),
    "xalm_cuda_mega_timeline": (_i, [_vp, _vp, C.c_size_t, C.POINTER(_i), C.POINTER(_i)]),
    "xalm_cuda_bench_matvec": (_i, [_i, _i, _i, _i, _i, _i, _i, _fp]),
    "xalm_cuda_prefill": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "xalm_cuda_prefill_async": (_i, [_vp, _vp, _i, _i, _i]),
    "xalm_cuda_gemm": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "xalm_cuda_bench_gemm": (_i, [_i, _i, _i, _i, _i, _fp]),
    "xalm_cuda_create_json": (_i, [C.c_char_p, _i, _i, _i, C.POINTER(_vp)]),
    "xalm_cuda_family_count": (_i, []),
    "xalm_cuda_family_name": (C.c_char_p, [_i]),
    "xalm_cuda_release": (_i, [_vp]),
    "xalm_cuda_expected_tensor": (_i, [_vp, _i, C.c_char_p, _sz, C.POINTER(_i), C.POINTER(_i)]),
    "xalm_cuda_model_info": (_i, [_vp, C.c_char_p, C.POINTER(C.c_longlong)]),
    "xalm_cuda_swa_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, C.c_float, C.c_float, _vp, _vp, _vp, _i, _i, _i]),
    "xalm_cuda_hgrn2": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, C.c_float]),
    "xalm_cuda_hyper_norm": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _i, C.c_float]),
    "xalm_cuda_dual_norm_hyper": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_float, _i, _i, _i, _vp, _vp, _vp]),
    "xalm_cuda_glu_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, C.c_float, C.c_float, _i]),
    "xalm_cuda_swa_attention_kept": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, C.c_float, _i, _i, _i]),
    "xalm_cuda_group_norm_residual": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, C.c_float, _vp, _vp, _i, _vp, _i, _i]),
    "xalm_cuda_qkv_post": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, C.c_float, _i, _i]),
    "xalm_cuda_delta_rule": (_i, [_vp] * 9 + [_i] * 6 + [_vp] * 6 + [C.c_float] * 3),
    "xalm_cuda_moe_ffn": (_i, [_vp] * 8 + [_i] * 9),
    "xalm_cuda_moe_ffn_routed": (_i, [_vp] * 9 + [_i] * 12 + [C.c_float]),
    "xalm_cuda_retention": (_i, [_vp] * 6 + [_i] * 5 + [_vp, _vp, _i, C.c_float, C.c_float]),
    "xalm_cuda_latent_post": (_i, [_vp] * 3 + [_i] * 5 + [_vp] * 3 + [C.c_float, _i, _i]),
    "xalm_cuda_latent_attend": (_i, [_vp] * 4 + [_i] * 8 + [_vp] * 3 + [C.c_float, _i, _i, _i]),
    "xalm_cuda_rows_act": (_i, [_vp] * 3 + [_i] * 4 + [C.c_float, _vp, _i, _i]),
    "xalm_cuda_norm_conv": (_i, [_vp] * 3 + [_i] * 5 + [_vp, _vp, C.c_float]),
    "xalm_cuda_short_conv": (_i, [_vp] * 3 + [_i] * 3 + [_vp, _vp, _i]),
    "xalm_cuda_embed_pair": (_i, [_vp, _vp, _i, _i, _vp, _i, _vp, _i, _i, _i, C.c_float, _vp, _i, _i, C.c_float]),
    "xalm_cuda_keyed_recurrence": (_i, [_vp] * 6 + [_i] * 6 + [C.c_float] + [_vp] * 5 + [C.c_float]),
    "xalm_cuda_sink_attention": (_i, [_vp] * 4 + [_i] * 6 + [C.c_float, _vp, C.c_float, _i, _i]),
    "xalm_cuda_qk_post": (_i, [_vp] * 4 + [_i] * 5 + [_vp, _i, C.c_float, _i]),
    "xalm_cuda_rows_act_bias": (_i, [_vp] * 3 + [_i] * 4 + [_vp, C.c_float, _i]),
    "xalm_cuda_gated_group_norm": (_i, [_vp] * 4 + [_i] * 3 + [C.c_float, C.c_float, _i]),
}
PRECISION_BF16, PRECISION_F32 = 0, 1            # enum xalm_precision

_LIB = None


def lib_path() -> str:
    return _build.LIB


def lib():
    """Load (building first if needed) libxalm_cuda.so and type every entry point."""
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path):
            _build.build_cuda()
        L = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)          # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(status: int):
    if status != 0:
        raise XalmError(status, lib().xalm_cuda_last_error().decode("utf-8", "replace"))


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def device_count() -> int:
    n = C.c_int(0)
    check(lib().xalm_cuda_device_count(C.byref(n)))
    return n.value


def device_count_or_zero() -> int:
    """CUDA devices this process can use; 0 when there is no driver."""
    try:
        return device_count()
    except XalmError:
        return 0


def families() -> list:
    """Model families linked into the library ("Llama", "Nabalix", "Bolovik", ...)."""
    L = lib()
    return [L.xalm_cuda_family_name(i).decode() for i in range(L.xalm_cuda_family_count())]


def tune(key: str, value: int):
    check(lib().xalm_cuda_tune(key.encode(), int(value)))


# ---- op-level entry points -----------------------------------------------------------------------------------
def dequant(type_id: int, raw: np.ndarray, n_elems: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw)
    out = np.empty(n_elems, dtype=np.float32)
    check(lib().xalm_cuda_dequant(type_id, _p(raw), n_elems, _p(out)))
    return out


def matmul(x: np.ndarray, w_raw: np.ndarray, type_id: int, n: int, d: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w_raw = np.ascontiguousarray(w_raw)
    out = np.empty(d, dtype=np.float32)
    check(lib().xalm_cuda_matmul(_p(out), _p(x), _p(w_raw), type_id, n, d))
    return out


def mha(q, kb, vb, head_dim, kv_len, max_seq_len, n_heads, n_kv_heads, want_att=False):
    q = np.ascontiguousarray(q, dtype=np.float32)
    kb, vb = np.ascontiguousarray(kb), np.ascontiguousarray(vb)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    att = np.zeros(n_heads * max_seq_len, dtype=np.float32) if want_att else None
    check(lib().xalm_cuda_mha(_p(out), _p(att) if want_att else None, _p(kb), _p(vb), _p(q), head_dim, kv_len, max_seq_len,
                              n_heads, n_kv_heads))
    return (out, att) if want_att else out


def rmsnorm(x, w_raw, wtype, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w_raw = np.ascontiguousarray(w_raw)
    out = np.empty_like(x)
    check(lib().xalm_cuda_rmsnorm(_p(out), _p(x), _p(w_raw), wtype, x.size, eps))
    return out


def rope(vec, head_dim, pos, theta, rotary_dim):
    v = np.array(vec, dtype=np.float32, copy=True)
    check(lib().xalm_cuda_rope(_p(v), v.size, head_dim, pos, theta, rotary_dim))
    return v


def ffn(x, w1, w2, w3, type_id, hidden_dim, dim, act):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(dim, dtype=np.float32)
    check(lib().xalm_cuda_ffn(_p(out), _p(x), _p(np.ascontiguousarray(w1)), _p(np.ascontiguousarray(w2)),
                              _p(np.ascontiguousarray(w3)), type_id, hidden_dim, dim, act))
    return out


def timeline_start(n_records: int):
    check(lib().xalm_cuda_timeline(n_records, None, None))


def timeline_stop(n_records: int) -> np.ndarray:
    out = np.zeros((n_records, 4), dtype=np.uint64)
    n = C.c_int(0)
    check(lib().xalm_cuda_timeline(n_records, _p(out), C.byref(n)))
    return out[: n.value]


def mega_timeline(handle):
    """(stamps of CTA 0 [n_phases, 8], arrival stamps of every CTA [n_phases, grid]) of the last token kernel, in ns;
    (None, None) when the one-kernel-per-token path is not in use.  Needs tune("mega_timeline", 1) before the first forward."""
    n_ph, grid = C.c_int(0), C.c_int(0)
    check(lib().xalm_cuda_mega_timeline(handle, None, 0, C.byref(n_ph), C.byref(grid)))
    if not n_ph.value:
        return None, None
    words = n_ph.value * (8 + grid.value)
    out = np.zeros(words, dtype=np.uint64)
    check(lib().xalm_cuda_mega_timeline(handle, _p(out), words, C.byref(n_ph), C.byref(grid)))
    return out[: 8 * n_ph.value].reshape(n_ph.value, 8), out[8 * n_ph.value:].reshape(n_ph.value, grid.value)


def bench_matvec(type_id: int, n: int, d: int, n_buffers: int, iters: int, epi: int = 0, with_norm: bool = False) -> float:
    ms = C.c_float(0)
    check(lib().xalm_cuda_bench_matvec(type_id, n, d, epi, int(with_norm), n_buffers, iters, C.byref(ms)))
    return ms.value


def gemm(a: np.ndarray, w_raw: np.ndarray, type_id: int, K: int, N: int, split: int = 1) -> np.ndarray:
    """out(T,N) = a(T,K) . W(N,K)^T on the tensor-core path."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    T = a.shape[0]
    w_raw = np.ascontiguousarray(w_raw)
    out = np.empty((T, N), dtype=np.float32)
    check(lib().xalm_cuda_gemm(_p(out), _p(a), _p(w_raw), type_id, T, K, N, split))
    return out


def bench_gemm(T: int, N: int, K: int, split: int = 1, iters: int = 20) -> float:
    ms = C.c_float(0)
    check(lib().xalm_cuda_bench_gemm(T, N, K, split, iters, C.byref(ms)))
    return ms.value


# ---- mechanism ops of the config.json families (include/xalm_cuda.h, "mechanism ops") --------------------------------------
def _f(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _pn(a):
    return None if a is None else _p(a)


def swa_attention(q, k, v, pos0, H, G, d, dv, window, scale, softcap=0.0, r1=None, r2=None, talk=None, gate=None, ring=None,
                  n_splits=1, cache_bf16=False):
    q, k, v, gate, r1, r2, talk = _f(q), _f(k), _f(v), _f(gate), _f(r1), _f(r2), _f(talk)
    T = q.shape[0]
    if ring is None:
        ring = min(pos0 + T, window - 1 + T)
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_swa_attention(_p(out), _p(q), _pn(gate), _p(k), _p(v), T, pos0, H, G, d, dv, window, scale, softcap, _pn(r1), _pn(r2),
                                        _pn(talk), ring, n_splits, int(cache_bf16)))
    return out


def hgrn2(qz, fz, v, state, H, d, dv, f_bias=None, lower=None, norm_w=None, eps=1e-5):
    """Returns (out, new state); `state` (H, d, dv) is not modified."""
    qz, fz, v, f_bias, lower, norm_w = _f(qz), _f(fz), _f(v), _f(f_bias), _f(lower), _f(norm_w)
    st = np.array(state, dtype=np.float32, copy=True)
    T = qz.shape[0]
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_hgrn2(_p(out), _p(st), _p(qz), _p(fz), _p(v), T, H, d, dv, _pn(f_bias), _pn(lower), _pn(norm_w), eps))
    return out, st


def hyper_norm(xs, a, w, one_plus, eps):
    xs, a, w = _f(xs), _f(a), _f(w)
    S, T, W = xs.shape
    h = np.empty((T, W), dtype=np.float32)
    check(lib().xalm_cuda_hyper_norm(_p(h), _p(xs), S, T, W, _pn(a), _p(w), int(one_plus), eps))
    return h


def dual_norm_hyper(xs, a, b, wa, wb, eps, mix=None, out_coef=None, scale=None):
    xs = np.array(xs, dtype=np.float32, copy=True)
    a, b, wa, wb, mix, out_coef, scale = _f(a), _f(b), _f(wa), _f(wb), _f(mix), _f(out_coef), _f(scale)
    S, T, W = xs.shape
    check(lib().xalm_cuda_dual_norm_hyper(_p(xs), _p(a), _p(b), _p(wa), _p(wb), eps, S, T, W, _pn(mix), _pn(out_coef), _pn(scale)))
    return xs


def glu_rows(x, w_gate, w_up, limit, alpha=1.702, w_bf16=False):
    x, w_gate, w_up = _f(x), _f(w_gate), _f(w_up)
    T, K = x.shape
    ff = w_gate.shape[0]
    out = np.empty((T, ff), dtype=np.float32)
    check(lib().xalm_cuda_glu_rows(_p(out), _p(x), _p(w_gate), _p(w_up), T, ff, K, limit, alpha, int(w_bf16)))
    return out


def swa_attention_kept(q, k, v, pos0, H, G, d, dv, window, keep_first, scale, ring=None, n_splits=1, cache_bf16=False):
    """Window attention in which the first keep_first positions stay visible; `ring` = slots behind the keep_first pinned ones."""
    q, k, v = _f(q), _f(k), _f(v)
    T = q.shape[0]
    if ring is None:
        ring = max(1, min(pos0 + T - keep_first, window - 1 + T))
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_swa_attention_kept(_p(out), _p(q), _p(k), _p(v), T, pos0, H, G, d, dv, window, keep_first, scale, ring, n_splits, int(cache_bf16)))
    return out


def group_norm_residual(y, w, groups, eps, x_in=None, part_w=None, hist=None, dwa=None):
    """y (T, W) or (T, parts, W).  Returns x_out, or (x_out, depth average) when dwa is given."""
    y, w, x_in, part_w, hist, dwa = _f(y), _f(w), _f(x_in), _f(part_w), _f(hist), _f(dwa)
    parts = y.shape[1] if y.ndim == 3 else 1
    T, W = y.shape[0], y.shape[-1]
    n_hist = 0 if dwa is None else dwa.shape[0] - 1
    out, avg = np.empty((T, W), dtype=np.float32), np.empty((T, W), dtype=np.float32)
    check(lib().xalm_cuda_group_norm_residual(_p(out), _p(avg), _p(y), parts, _pn(part_w), _p(w), groups, eps, _pn(x_in), _pn(hist), n_hist, _pn(dwa), T, W))
    return out if dwa is None else (out, avg)


def qkv_post(proj, pos0, H, G, d, dv, bq=None, bk=None, bv=None, freq=None, norm_qk=True, norm_v=True, eps=1e-5, keep_first=0, ring=None):
    """Returns (q rows, K cache, V cache) with the caches slot by slot."""
    proj, bq, bk, bv, freq = _f(proj), _f(bq), _f(bk), _f(bv), _f(freq)
    T = proj.shape[0]
    if ring is None:
        ring = max(1, pos0 + T - keep_first)
    slots = keep_first + ring
    q, kc, vc = np.empty((T, H * d), dtype=np.float32), np.empty((slots, G * d), dtype=np.float32), np.empty((slots, G * dv), dtype=np.float32)
    check(lib().xalm_cuda_qkv_post(_p(q), _p(kc), _p(vc), _p(proj), T, pos0, H, G, d, dv, _pn(bq), _pn(bk), _pn(bv), _pn(freq),
                                   0 if freq is None else freq.shape[0], int(norm_qk), int(norm_v), eps, keep_first, ring))
    return q, kc, vc


def delta_rule(q, k, v, gate, b, a, state, conv_state, H, G, d, dv, wq, wk, wv, A_log, dt_bias, norm_w=None, eps=1e-5, unit_eps=1e-6, q_scale=None):
    """Returns (out, new state, new conv_state); the inputs are not modified."""
    q, k, v, gate, b, a, wq, wk, wv, A_log, dt_bias, norm_w = (_f(x) for x in (q, k, v, gate, b, a, wq, wk, wv, A_log, dt_bias, norm_w))
    taps = wq.shape[1]
    st = np.array(state, dtype=np.float32, copy=True)
    cs = np.array(conv_state, dtype=np.float32, copy=True).reshape(-1)
    if cs.size == 0:
        cs = np.zeros(2 * G * d + H * dv, dtype=np.float32)
    T = q.shape[0]
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_delta_rule(_p(out), _p(st), _p(cs), _p(q), _p(k), _p(v), _p(gate), _p(b), _p(a), T, H, G, d, dv, taps, _p(wq), _p(wk), _p(wv),
                                     _p(A_log), _p(dt_bias), _pn(norm_w), eps, unit_eps, d ** -0.5 if q_scale is None else q_scale))
    return out, st, cs.reshape(max(1, taps - 1), -1)[: taps - 1]


def moe_ffn(h, w_router, w_gate, w_up, w_down, top, n_groups=0, keep_groups=0, act=1, w_bf16=False):
    """Returns (idx (T, top), wgt (T, top), out (T, top, K)): the chosen experts, their scores, and each chosen expert's output."""
    h, w_router, w_gate, w_up, w_down = _f(h), _f(w_router), _f(w_gate), _f(w_up), _f(w_down)
    T, K = h.shape
    E, ff = w_gate.shape[0], w_gate.shape[1]
    idx, wgt, out = np.empty((T, top), dtype=np.int32), np.empty((T, top), dtype=np.float32), np.empty((T, top, K), dtype=np.float32)
    check(lib().xalm_cuda_moe_ffn(_p(out), _p(idx), _p(wgt), _p(h), _p(w_router), _p(w_gate), _p(w_up), _p(w_down), T, K, E, top, ff, n_groups, keep_groups,
                                  act, int(w_bf16)))
    return idx, wgt, out


def moe_ffn_routed(h, w_router, w_gate, w_up, w_down, top, n_groups=0, keep_groups=0, act=0, limit=float("inf"), score="softmax", group="max",
                   renormalise=True, x=None, w_bf16=False):
    """The router's variants.  Returns (idx, wgt, out (T, top, K), x + weighted sum or None)."""
    h, w_router, w_gate, w_up, w_down = _f(h), _f(w_router), _f(w_gate), _f(w_up), _f(w_down)
    T, K = h.shape
    E, ff = w_gate.shape[0], w_gate.shape[1]
    idx, wgt, out = np.empty((T, top), dtype=np.int32), np.empty((T, top), dtype=np.float32), np.empty((T, top, K), dtype=np.float32)
    xo = None if x is None else np.array(x, dtype=np.float32, copy=True)
    check(lib().xalm_cuda_moe_ffn_routed(_p(out), _p(idx), _p(wgt), _pn(xo), _p(h), _p(w_router), _p(w_gate), _p(w_up), _p(w_down), T, K, E, top, ff,
                                         n_groups, keep_groups, act, int(w_bf16), {"sigmoid": 0, "softmax": 1}[score], {"top2": 0, "max": 1}[group],
                                         int(renormalise), limit))
    return idx, wgt, out, xo


def retention(q, k, v, state, H, d, dv, decay, pos0=0, freq=None, gate=None, k_scale=None, eps=1e-6):
    """Returns (out (T, H dv), new state); `state` (H, d, dv) is not modified."""
    q, k, v, gate, decay, freq = _f(q), _f(k), _f(v), _f(gate), _f(decay), _f(freq)
    st = np.array(state, dtype=np.float32, copy=True)
    T = q.shape[0]
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_retention(_p(out), _p(st), _p(q), _p(k), _p(v), _pn(gate), T, pos0, H, d, dv, _p(decay), _pn(freq),
                                    0 if freq is None else freq.shape[0], d ** -0.5 if k_scale is None else k_scale, eps))
    return out, st


def latent_post(proj, pos0, q_rank, kv_rank, rot, q_norm, kv_norm, freq=None, eps=1e-6, ring=None, cache_bf16=False):
    """Returns (normed query latent (T, q_rank), cache rows (ring, kv_rank + rot))."""
    proj, q_norm, kv_norm, freq = _f(proj), _f(q_norm), _f(kv_norm), _f(freq)
    T = proj.shape[0]
    ring = pos0 + T if ring is None else ring
    cq, cache = np.zeros((T, q_rank), dtype=np.float32), np.zeros((ring, kv_rank + rot), dtype=np.float32)
    check(lib().xalm_cuda_latent_post(_p(cq), _p(cache), _p(proj), T, pos0, q_rank, kv_rank, rot, _pn(q_norm), _pn(kv_norm), _pn(freq), eps, ring,
                                      int(cache_bf16)))
    return cq, cache


def latent_attend(q, cache, pos0, H, d, r, dv, R, uk, uv, scale, freq=None, gate=None, n_splits=0, cache_bf16=False, w_bf16=False):
    q, cache, uk, uv, freq, gate = _f(q), _f(cache), _f(uk), _f(uv), _f(freq), _f(gate)
    T = q.shape[0]
    assert cache.shape[0] == pos0 + T
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_latent_attend(_p(out), _p(q), _p(cache), _pn(gate), T, pos0, H, d, r, dv, R, cache.shape[1], _p(uk), _p(uv), _pn(freq), scale,
                                        n_splits, int(cache_bf16), int(w_bf16)))
    return out


def rows_act(x, w, act=0, cap=0.0, mul=None, mul_act=2, w_bf16=False):
    x, w, mul = _f(x), _f(w), _f(mul)
    T, K = x.shape
    out = np.empty((T, w.shape[0]), dtype=np.float32)
    check(lib().xalm_cuda_rows_act(_p(out), _p(x), _p(w), T, w.shape[0], K, act, cap, _pn(mul), mul_act, int(w_bf16)))
    return out


def norm_conv(x, w, cw, hist, groups, eps=1e-5):
    """w (readers, W), cw (readers, W, taps), hist (readers, taps - 1, W).  Returns (out (readers, T, W), new hist); hist is not modified."""
    x, w, cw = _f(x), _f(w), _f(cw)
    readers, W, taps = cw.shape
    T = x.shape[0]
    hs = np.zeros((readers, max(taps - 1, 1), W), dtype=np.float32)
    hs[:, :taps - 1] = hist
    out = np.empty((readers, T, W), dtype=np.float32)
    check(lib().xalm_cuda_norm_conv(_p(out), _p(hs), _p(x), T, W, groups, taps, readers, _p(w), _p(cw), eps))
    return out, hs[:, :taps - 1]


def short_conv(x, w, hist, bias=None, act=0):
    """Returns (out (T, C), new hist (taps - 1, C)); hist is not modified."""
    x, w, bias = _f(x), _f(w), _f(bias)
    T, Cn = x.shape
    taps = w.shape[1]
    hs = np.zeros((max(taps - 1, 1), Cn), dtype=np.float32)
    hs[:taps - 1] = hist
    out = np.empty((T, Cn), dtype=np.float32)
    check(lib().xalm_cuda_short_conv(_p(out), _p(hs), _p(x), T, Cn, taps, _p(w), _pn(bias), act))
    return out, hs[:taps - 1]


def embed_pair(tokens, prev, table, scale=1.0, pair=None, mul_prev=0, mul_cur=0, w=None, groups=1, eps=1e-5):
    table, pair, w = _f(table), _f(pair), _f(w)
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    V, W = table.shape
    out = np.empty((len(tokens), W), dtype=np.float32)
    check(lib().xalm_cuda_embed_pair(_p(out), _p(tokens), len(tokens), -1 if prev is None else prev, _p(table), V, _pn(pair),
                                     0 if pair is None else pair.shape[0] - 1, mul_prev, mul_cur, scale, _pn(w), groups, W, eps))
    return out


def keyed_recurrence(q, k, v, f, state, H, rep, d, dv, mode, q_scale=0.0, dt_bias=None, A_log=None, skip=None, norm_w=None, gate=None, eps=1e-5):
    """Returns (out (T, H dv), new state); `state` (H, d, dv) is not modified."""
    q, k, v, f, dt_bias, A_log, skip, norm_w, gate = (_f(a) for a in (q, k, v, f, dt_bias, A_log, skip, norm_w, gate))
    st = np.array(state, dtype=np.float32, copy=True)
    T = q.shape[0]
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_keyed_recurrence(_p(out), _p(st), _p(q), _p(k), _p(v), _p(f), T, H, rep, d, dv, mode, q_scale, _pn(dt_bias), _pn(A_log),
                                           _pn(skip), _pn(norm_w), _pn(gate), eps))
    return out, st


def sink_attention(q, k, v, pos0, H, G, d, dv, scale, sink=None, out_scale=0.0, n_splits=1, cache_bf16=False):
    q, k, v, sink = _f(q), _f(k), _f(v), _f(sink)
    T = q.shape[0]
    out = np.empty((T, H * dv), dtype=np.float32)
    check(lib().xalm_cuda_sink_attention(_p(out), _p(q), _p(k), _p(v), T, pos0, H, G, d, dv, scale, _pn(sink), out_scale, n_splits, int(cache_bf16)))
    return out


def qk_post(proj, pos0, H, G, d, freq=None, rot_mag=0.0, ring=None):
    """Returns (turned q rows, cache of turned keys, cache of the keys as they came), the caches row by row."""
    proj, freq = _f(proj), _f(freq)
    T = proj.shape[0]
    ring = pos0 + T if ring is None else ring
    q, kc, vc = np.empty((T, H * d), dtype=np.float32), np.empty((ring, G * d), dtype=np.float32), np.empty((ring, G * d), dtype=np.float32)
    check(lib().xalm_cuda_qk_post(_p(q), _p(kc), _p(vc), _p(proj), T, pos0, H, G, d, _pn(freq), 0 if freq is None else freq.shape[0], rot_mag, ring))
    return q, kc, vc


def rows_act_bias(x, w, act, bias=None, act_pow=1.0, w_bf16=False):
    x, w, bias = _f(x), _f(w), _f(bias)
    T, K = x.shape
    out = np.empty((T, w.shape[0]), dtype=np.float32)
    check(lib().xalm_cuda_rows_act_bias(_p(out), _p(x), _p(w), T, w.shape[0], K, act, _pn(bias), act_pow, int(w_bf16)))
    return out


def gated_group_norm(y, w, groups, gate=None, eps=1e-5, out_scale=0.0, ld_out=None):
    y, w, gate = _f(y), _f(w), _f(gate)
    T, W = y.shape
    ld_out = W if ld_out is None else ld_out
    out = np.zeros((T, ld_out), dtype=np.float32)
    check(lib().xalm_cuda_gated_group_norm(_p(out), _p(y), _pn(gate), _p(w), T, W, groups, eps, out_scale, ld_out))
    return out
