"""Host-side pieces of the Kubolorn family that need no GPU: the registry, config validation (done before a device is touched), the
model-folder round trip, and the oracle's own invariants."""
import json
import math

import numpy as np
import pytest

import kubolorn_oracle as O
from xalm_b200 import capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import Model

ROT = {"dims": 4, "base": 60.0, "scaling": {"factor": 4.0, "fast": 8.0, "slow": 0.5, "original": 32}}
CFG = O.make_config(vocab=19, width=16, groups=2, taps=3, loop=(0, 2, 2), layers=[
    O.gla_layer(2, 4, 6, 8.0, rank=3, mlp=O.moe(6, 4, 2)),
    O.parallel_layer(4, 2, 6, 0.3, ROT, 2, 4, 5, 1, 3, 2, 1.1, 0.6, mlp=O.dense(12)),
    O.gla_layer(1, 5, 3, 2.0, rank=2, mlp=None)])


def test_registry_lists_the_family():
    assert {"Llama", "Nabalix", "Bolovik", "Duletar", "Kubolorn"} <= set(capi.families())


def test_model_folder_roundtrip(tmp_path):
    W = O.random_weights(CFG, 1)
    ST.write_model_dir(str(tmp_path), CFG, W, "BF16")
    back = ST.read_tensors(str(tmp_path / "model.safetensors"))
    assert set(back) == set(W) == set(O.tensor_shapes(CFG))
    for n, (t, shape, raw) in back.items():
        assert np.array_equal(ST.bf16_bits_to_f32(raw.view(np.uint16)).reshape(shape), W[n])   # the test weights are bf16-exact
    m = Model.from_pretrained(str(tmp_path))
    assert m.config["architecture"] == "Kubolorn"
    assert "head" not in W and "l2.norm2" not in W and "l2.canon2" not in W                   # tied head; a layer without a feed-forward has one reader


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "convolution"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 0), "mixer sizes"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("tau", 0.0), "mixer sizes"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "query heads"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("vdim", 4), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 8), "rotary"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("conv", 40), "taps"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("norm_groups", 3), "norm groups"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"), "routed"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "experts"),
    (lambda c: c["norm"].__setitem__("groups", 3), "norm groups"),
    (lambda c: c["canon"].__setitem__("taps", 0), "canon.taps"),
    (lambda c: c["loop"].__setitem__("stop", 4), "loop"),
    (lambda c: c["embedding"]["bigram"].__setitem__("buckets", 0), "bigram"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configs_are_named_before_any_device_is_touched(edit, needle):
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(capi.XalmError, match=needle):
        Model.from_json(c, {}).cuda()


def test_oracle_invariants():
    """The restatement itself: a run cut into portions equals one run; the loop's order; a decay of one keeps everything; a sink far below
    every score is plain softmax attention, one far above silences the head; the rescaled frequencies lie between f / factor and f; the
    chosen experts' weights sum to one; a convolution of one tap is a per-channel scale."""
    rng = np.random.default_rng(0)
    W = O.random_weights(CFG, 2)
    tokens = rng.integers(0, 19, 20).tolist()
    whole = O.forward(CFG, W, tokens, {})
    st = {}
    parts = np.concatenate([O.forward(CFG, W, tokens[a:b], st) for a, b in ((0, 7), (7, 9), (9, 10), (10, 20))])
    assert np.allclose(parts, whole, atol=1e-10)
    assert [li for _, li in O.layer_runs(CFG)] == [0, 1, 0, 1, 2]
    assert [li for _, li in O.layer_runs(O.make_config(5, 4, [{}] * 4, loop=(1, 2, 3)))] == [0, 1, 1, 1, 2, 3]
    f, mag = O.yarn_table(ROT)
    plain = ROT["base"] ** (-2.0 * np.arange(2) / 4)
    assert (f <= plain + 1e-15).all() and (f >= plain / 4.0 - 1e-15).all() and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-15
    mx = {"heads": 2, "kv_heads": 1, "dim": 4, "scale": 0.5}
    h = rng.standard_normal((6, 8))
    w = {"q": rng.standard_normal((8, 8)), "k": rng.standard_normal((4, 8)), "o": np.eye(8), "sink": np.array([-200.0, 200.0])}
    out = O.sink_attention(h, mx, w, "", 0, {})
    q, k = (h @ w["q"].T).reshape(6, 2, 4), h @ w["k"].T
    s = (q[:, 0] @ k.T) * 0.5
    s[np.triu_indices(6, 1)] = -np.inf
    p = np.exp(s - s.max(-1, keepdims=True))
    assert np.allclose(out[:, :4], (p / p.sum(-1, keepdims=True)) @ k) and np.abs(out[:, 4:]).max() < 1e-60
    mlp = O.moe(3, 4, 2)
    hh = rng.standard_normal((5, 6))
    we = {"router": rng.standard_normal((4, 6))}
    for e in range(4):
        we[f"e{e}.up"], we[f"e{e}.down"] = np.ones((3, 6)), np.ones((6, 3))                    # every expert the same: the mixture is that expert
    assert np.allclose(O.expert_ff(hh, mlp, we, ""), (np.maximum(hh.sum(-1), 0) ** 2 * 3)[:, None] * np.ones(6))
    x = rng.standard_normal((4, 3))
    y, hist = O.short_conv(x, np.array([[2.0], [3.0], [4.0]]), np.zeros((0, 3)))
    assert np.allclose(y, x * [2.0, 3.0, 4.0]) and hist.shape == (0, 3)
