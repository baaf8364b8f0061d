"""Host-side pieces of the Duletar family that need no GPU: the registry, config validation (done before a device is touched), the
model-folder round trip, and the oracle's own invariants."""
import json

import numpy as np
import pytest

import duletar_oracle as O
from xalm_b200 import capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import Model

CFG = O.make_config(vocab=19, width=16, embed_scale=2.0, softcap=6.0, layers=[
    O.retention_layer(2, 4, 6, [0.9, 0.5], rot_dims=2, mlp=O.dense(12)),
    O.latent_layer(2, 4, 2, 6, 8, 5, mlp=O.moe(6, 4, 2, groups=2, keep=1)),
    O.gated_latent_layer(3, 2, 2, 8, 4, kv_from=1, mlp=None)])


def test_registry_lists_the_family():
    assert {"Llama", "Nabalix", "Bolovik", "Duletar"} <= set(capi.families())


def test_model_folder_roundtrip(tmp_path):
    W = O.random_weights(CFG, 1)
    ST.write_model_dir(str(tmp_path), CFG, W, "BF16")
    back = ST.read_tensors(str(tmp_path / "model.safetensors"))
    assert set(back) == set(W)
    for n, (t, shape, raw) in back.items():
        assert np.array_equal(ST.bf16_bits_to_f32(raw.view(np.uint16)).reshape(shape), W[n])   # the test weights are bf16-exact
    m = Model.from_pretrained(str(tmp_path))
    assert m.config["architecture"] == "Duletar" and m.config["vocab_size"] == 19
    assert "l2.mix.dkv" not in W and "l2.mix.uk" in W                                          # a layer that reads another's latents has no down projection


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "convolution"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 0), "mixer sizes"),
    (lambda c: c["layers"][0]["mixer"]["decay"].pop(), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 6), "rotary"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("rot_dim", 3), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 4), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 0), "latent sizes"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 0), "no latents"),                # a retention layer has none
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 9), "no latents"),                # sizes must agree
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "routed"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "experts"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 3), "expert groups"),          # one kept group of two cannot give three
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configs_are_named_before_any_device_is_touched(edit, needle):
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(capi.XalmError, match=needle):
        Model.from_json(c, {}).cuda()


def test_oracle_invariants():
    """The restatement itself: a retention run cut in two equals one run; a decay of one keeps everything, of zero only the current token;
    attention over latents equals attention with the key expansion moved to the query side; one expert group is no grouping; renormalised
    weights sum to one; the soft cap is the identity near zero and bounded by the cap."""
    rng = np.random.default_rng(0)
    T, H, d, dv = 9, 2, 4, 3
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    f = O.rotary_frequencies(4, 100.0)
    assert np.allclose(f[1:] / f[:-1], 100.0 ** (-2 / 4))
    whole, s = O.retention_heads(q, k, v, decay=[0.9, 0.6], freqs=f, eps=1e-6)
    o1, s1 = O.retention_heads(q[:4], k[:4], v[:4], decay=[0.9, 0.6], freqs=f, eps=1e-6)
    o2, s2 = O.retention_heads(q[4:], k[4:], v[4:], decay=[0.9, 0.6], freqs=f, eps=1e-6, state=s1, first_pos=4)
    assert np.allclose(np.concatenate([o1, o2]), whole) and np.allclose(s2, s)
    _, s_all = O.retention_heads(q, k, v, decay=[1.0, 0.0], eps=1e-6)
    assert np.allclose(s_all[0], sum(np.outer(k[t, 0], v[t, 0]) for t in range(T)) / 2.0)       # keys carry d^-1/2 = 1/2
    assert np.allclose(s_all[1], np.outer(k[-1, 1], v[-1, 1]) / 2.0)
    n, R, r = 7, 6, 2
    c, kr = rng.standard_normal((n, R)), rng.standard_normal((n, r))
    uk, uv = rng.standard_normal((H * d, R)), rng.standard_normal((H * dv, R))
    qq = rng.standard_normal((n, H * (d + r)))
    a = O.attend_latents(qq, c, kr, uk, uv, H=H, d=d, r=r, dv=dv, scale=0.4, freqs=O.rotary_frequencies(r, 10.0))
    q3 = qq.reshape(n, H, d + r)
    qa = np.einsum("thd,hdr->thr", q3[:, :, :d], uk.reshape(H, d, R))                           # queries in the latent
    qr = O.rotate(q3[:, :, d:], np.arange(n), O.rotary_frequencies(r, 10.0))
    kk = np.repeat(np.concatenate([c, kr], axis=1)[:, None, :], H, axis=1)
    lat = O.causal_softmax_attention(np.concatenate([qa, qr], axis=-1), kk, np.repeat(c[:, None, :], H, axis=1), 0.4)
    assert np.allclose(np.einsum("thr,hvr->thv", lat, uv.reshape(H, dv, R)).reshape(n, -1), a)
    h, wr = rng.standard_normal((5, 7)), rng.standard_normal((6, 7))
    plain, grouped = O.route(h, wr, top=2), O.route(h, wr, top=2, n_groups=1, keep_groups=1)
    assert all(np.array_equal(a_[0], b_[0]) for a_, b_ in zip(plain, grouped))
    assert all(abs(w.sum() - 1) < 1e-12 for _, w in plain)
    assert np.allclose(O.softcap(np.array([1e-3]), 5.0), 1e-3, rtol=1e-6) and abs(O.softcap(np.array([1e3]), 5.0)[0]) <= 5.0
