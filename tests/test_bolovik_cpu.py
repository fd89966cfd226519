"""Host-side pieces of the Bolovik family that need no GPU: the registry, config validation (done before a device is touched), the
model-folder round trip, and the oracle's own invariants."""
import json

import numpy as np
import pytest

import bolovik_oracle as O
from xalm_b200 import capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import Model

CFG = O.make_config(vocab=19, width=16, groups=2, layers=[
    O.attention_layer(2, 1, 4, 6, window=5, keep_first=2, rot={"base": 100.0, "dims": 2}, mlp=O.moe(6, 4, 2, groups=2, keep=1)),
    O.delta_layer(2, 2, 4, 4, conv=3, mlp=O.dense(12))])


def test_registry_lists_the_family():
    assert {"Llama", "Nabalix", "Bolovik"} <= set(capi.families())


def test_model_folder_roundtrip(tmp_path):
    W = O.random_weights(CFG, 1)
    ST.write_model_dir(str(tmp_path), CFG, W, "BF16")
    back = ST.read_tensors(str(tmp_path / "model.safetensors"))
    assert set(back) == set(W)
    for n, (t, shape, raw) in back.items():
        assert np.array_equal(ST.bf16_bits_to_f32(raw.view(np.uint16)).reshape(shape), W[n])   # the test weights are bf16-exact
    m = Model.from_pretrained(str(tmp_path))
    assert m.config["architecture"] == "Bolovik" and m.config["vocab_size"] == 19


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "convolution"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "mixer sizes"),
    (lambda c: c["norm"].__setitem__("groups", 3), "norm groups"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"), "routed"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "experts"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 3), "expert groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 3), "expert groups"),          # one kept group of two cannot give three
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 5), "rotary"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("conv", 0), "conv"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configs_are_named_before_any_device_is_touched(edit, needle):
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(capi.XalmError, match=needle):
        Model.from_json(c, {}).cuda()


def test_oracle_invariants():
    """The restatement itself: a window over everything equals keeping everything; a run of the delta rule cut in two equals one run;
    one norm group is the plain RMS norm; one expert group of all experts is no grouping; unscaled frequencies are a geometric series."""
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((6, 8)), rng.standard_normal((6, 4)), rng.standard_normal((6, 6))
    kw = dict(H=2, G=1, d=4, dv=6, scale=0.5)
    full = O.kept_window_attention(q, k, v, window=6, keep_first=0, **kw)
    assert np.allclose(full, O.kept_window_attention(q, k, v, window=1, keep_first=6, **kw))
    assert not np.allclose(full[-1], O.kept_window_attention(q, k, v, window=5, keep_first=0, **kw)[-1])
    assert np.allclose(full[-1], O.kept_window_attention(q, k, v, window=5, keep_first=1, **kw)[-1])
    H, G, d, dv, T, taps = 2, 1, 3, 5, 9, 3
    a = [rng.standard_normal((T, n)) for n in (G * d, G * d, H * dv, H * dv, H, H)]
    par = dict(H=H, G=G, d=d, dv=dv, wq=rng.standard_normal((G * d, taps)), wk=rng.standard_normal((G * d, taps)), wv=rng.standard_normal((H * dv, taps)),
               A_log=rng.standard_normal(H), dt_bias=rng.standard_normal(H), norm_w=np.ones(dv))
    z, c0 = np.zeros((H, d, dv)), np.zeros((taps - 1, 2 * G * d + H * dv))
    whole, s, c = O.delta_rule(*a, z, c0, **par)
    o1, s1, c1 = O.delta_rule(*[x[:4] for x in a], z, c0, **par)
    o2, s2, c2 = O.delta_rule(*[x[4:] for x in a], s1, c1, **par)
    assert np.allclose(np.concatenate([o1, o2]), whole) and np.allclose(s2, s) and np.allclose(c2, c)
    x, w = rng.standard_normal((3, 12)), rng.standard_normal(12)
    assert np.allclose(O.group_norm(x, w, 1, 1e-5), O.unit_rms(x, 1e-5) * w)
    assert not np.allclose(O.group_norm(x, w, 3, 1e-5), O.group_norm(x, w, 1, 1e-5))
    h, wr = rng.standard_normal((5, 7)), rng.standard_normal((6, 7))
    assert np.array_equal(O.route(h, wr, 2, 1, 1)[0], O.route(h, wr, 2)[0])
    f = O.rotary_frequencies(8, 10000.0)
    assert np.allclose(f[1:] / f[:-1], 10000.0 ** (-2 / 8))
