"""Host-side pieces of the config.json families that need no GPU: the model-folder reader / writer, the family registry, config
validation (done before a device is touched), the command line's argument handling, and the oracle's own invariants."""
import json
import subprocess

import numpy as np
import pytest

import nabalix_oracle as O
from xalm_b200 import build, capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import Model

CFG = O.make_config(vocab=19, width=16, streams=2,
                    layers=[dict(H=2, G=1, d=4, dv=6, window=5, Hr=1, dr=3, dvr=5, ff=12), dict(H=2, G=2, d=4, dv=4, window=3, Hr=2, dr=2, dvr=2, ff=None)])


def test_registry_lists_both_families():
    assert {"Llama", "Nabalix"} <= set(capi.families())


def test_model_folder_roundtrip(tmp_path):
    W = O.random_weights(CFG, 1)
    ST.write_model_dir(str(tmp_path), CFG, W, "BF16")
    back = ST.read_tensors(str(tmp_path / "model.safetensors"))
    assert set(back) == set(W)
    for n, (t, shape, raw) in back.items():
        assert t.name == "BF16" and shape == W[n].shape
        assert np.array_equal(ST.bf16_bits_to_f32(raw.view(np.uint16)).reshape(shape), W[n])   # the test weights are bf16-exact
    m = Model.from_pretrained(str(tmp_path))
    assert m.config["architecture"] == "Nabalix" and m.config["vocab_size"] == 19


def test_bf16_rounding_is_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e-39, 65504.0], dtype=np.float32)   # 1 + 2^-8 is a tie -> 1.0; 1 + 3 * 2^-8 -> 1 + 2^-6
    got = ST.bf16_bits_to_f32(ST.f32_to_bf16_bits(x))
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == np.float32(1.015625)
    assert np.array_equal(O.bf16_round(x), got)


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "serial"), "serial"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "attention sizes"),
    (lambda c: c.__setitem__("streams", 99), "streams"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "routed"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.__setitem__("architecture", "Unknown"), "Unknown"),
])
def test_bad_configs_are_named_before_any_device_is_touched(edit, needle):
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(capi.XalmError, match=needle):
        Model.from_json(c, {}).cuda()


def test_command_line_on_a_model_folder_without_a_device(tmp_path):
    """Argument handling and the folder reader run before the device is needed; what then fails is the device, by name."""
    ST.write_model_dir(str(tmp_path / "m"), CFG, O.random_weights(CFG, 2), "BF16")
    build.build_host()
    r = subprocess.run([build.MAIN, str(tmp_path / "m"), "-m", "trace"], capture_output=True, text=True)
    assert r.returncode == 1 and "-o" in r.stderr
    r = subprocess.run([build.MAIN, str(tmp_path / "m"), "-m", "passkey"], capture_output=True, text=True)
    assert r.returncode == 1 and "tokenizer" in r.stderr
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{}")
    r = subprocess.run([build.MAIN, str(tmp_path / "bad"), "-i", "1 2"], capture_output=True, text=True)
    assert r.returncode == 1 and "architecture" in r.stderr
    if capi.device_count_or_zero() == 0:
        r = subprocess.run([build.MAIN, str(tmp_path / "m"), "-i", "1 2 3", "-n", "2"], capture_output=True, text=True)
        assert r.returncode == 1 and "cuda" in r.stderr.lower()      # no CPU fallback


def test_oracle_invariants():
    """The restatement itself: a window that covers everything equals no window; the recurrence split in two equals one run;
    one stream with unit coefficients is the plain residual sum."""
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((6, 8)), rng.standard_normal((6, 4)), rng.standard_normal((6, 6))
    kw = dict(H=2, G=1, d=4, dv=6, scale=0.5)
    assert np.allclose(O.window_attention(q, k, v, window=6, **kw), O.window_attention(q, k, v, window=100, **kw))
    assert not np.allclose(O.window_attention(q, k, v, window=5, **kw)[-1], O.window_attention(q, k, v, window=6, **kw)[-1])
    qz, fz, vv = rng.standard_normal((9, 6)), rng.standard_normal((9, 6)), rng.standard_normal((9, 10))
    whole, s = O.hgrn2(qz, fz, vv, np.zeros((2, 3, 5)), H=2, d=3, dv=5)
    a, sa = O.hgrn2(qz[:4], fz[:4], vv[:4], np.zeros((2, 3, 5)), H=2, d=3, dv=5)
    b, sb = O.hgrn2(qz[4:], fz[4:], vv[4:], sa, H=2, d=3, dv=5)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(sb, s)
    xs = rng.standard_normal((1, 3, 4))
    y = rng.standard_normal((3, 4))
    assert np.allclose(O.hyper_write(xs, y, np.eye(1), np.ones(1))[0], xs[0] + y)
