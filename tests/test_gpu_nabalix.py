"""Nabalix on the GPU against the plain restatement in tests/nabalix_oracle.py: every mechanism alone (op-level entry points that
launch the family's kernels), then whole models with small random configurations — prompts in one pass, token by token, in
portions, across ring wrap and release, long decoding, greedy generation through the host entry points."""
import json
import os
import subprocess

import numpy as np
import pytest

import nabalix_oracle as O
from xalm_b200 import build, capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import InferenceState, Model, Sampler, generate

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4   # IEEE fp32 path against float64, on values of order one
BF16_TOL = 6e-2  # serving mode: bf16 weights (exact here) and a bf16 K/V ring


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err < tol, f"max error {err:.3e} (tolerance {tol})"


# ---- mechanisms alone ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 8, 12), (3, 3, 16, 4), (6, 1, 4, 20), (1, 1, 32, 32)])
@pytest.mark.parametrize("pos0,T,window,splits", [(0, 9, 4, 1), (0, 40, 64, 1), (37, 1, 16, 3), (50, 6, 7, 1), (129, 1, 130, 4), (65, 2, 33, 2)])
def test_window_attention_op(H, G, d, dv, pos0, T, window, splits):
    rng = np.random.default_rng(H * 100 + pos0 + window)
    n = pos0 + T
    q = rng.standard_normal((T, H * d)) * 1.5
    k = rng.standard_normal((n, G * d))
    v = rng.standard_normal((n, G * dv))
    gate = rng.standard_normal((T, H * dv))
    r1, r2 = rng.uniform(0.1, 1, H), rng.uniform(0.1, 2, H)
    talk = np.eye(H) + 0.4 * rng.standard_normal((H, H))
    kw = dict(H=H, G=G, d=d, dv=dv, window=window, scale=0.4, softcap=3.0, r1=r1, r2=r2, talk=talk, gate=gate)
    want = O.window_attention(q, k, v, first_pos=pos0, **kw)
    close(capi.swa_attention(q, k, v, pos0, n_splits=splits, **kw), want, F32_TOL)
    # every optional part off: plain windowed softmax
    kw0 = dict(H=H, G=G, d=d, dv=dv, window=window, scale=0.7)
    close(capi.swa_attention(q, k, v, pos0, n_splits=splits, **kw0), O.window_attention(q, k, v, first_pos=pos0, **kw0), F32_TOL)
    # the bf16 ring
    kb, vb = O.bf16_round(k), O.bf16_round(v)
    close(capi.swa_attention(q, kb, vb, pos0, n_splits=splits, cache_bf16=True, **kw), O.window_attention(q, kb, vb, first_pos=pos0, **kw), F32_TOL)


@pytest.mark.parametrize("T,splits", [(5, 1), (1, 1), (1, 3)])
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("dv", [4, 8])                       # 8: a one-token step copies its key block to shared memory first
def test_window_edge_stands_out(T, splits, offset, dv):
    """One key carries a score far above the rest and a value nobody else has; it sits on the last visible place of the window
    (offset 0) or one further back (offset 1), for the last row of a prompt portion and for a token decoded alone."""
    H, G, d, window, pos0 = 2, 1, 8, 24, 60
    n = pos0 + T
    i = n - 1
    target = i - (window - 1) - offset
    rng = np.random.default_rng(7)
    k = 0.05 * rng.standard_normal((n, G * d))
    v = 0.05 * rng.standard_normal((n, G * dv))
    k[target, 0] = 6.0
    v[target] = 100.0
    q = 0.05 * rng.standard_normal((T, H * d))
    q[:, 0] = 5.0
    q[:, d] = 5.0
    got = capi.swa_attention(q, k, v, pos0, H, G, d, dv, window, 1.0, n_splits=splits)
    want = O.window_attention(q, k, v, H=H, G=G, d=d, dv=dv, window=window, scale=1.0, first_pos=pos0)
    close(got, want, F32_TOL)
    assert (got[-1].min() > 90.0) == (offset == 0)           # seen exactly when it is inside the window
    if T > 1 and offset == 1:
        assert got[-2].min() > 90.0                          # the row before still sees it


@pytest.mark.parametrize("dv", [4, 16])
def test_window_far_key_among_hundreds(dv):
    H, G, d, pos0, T = 2, 2, 8, 700, 1
    n = pos0 + T
    rng = np.random.default_rng(3)
    k = 0.05 * rng.standard_normal((n, G * d))
    v = 0.05 * rng.standard_normal((n, G * dv))
    k[5, 0] = k[5, d] = 8.0
    v[5] = 50.0
    q = np.zeros((T, H * d))
    q[:, 0] = q[:, d] = 4.0
    for splits in (1, 5):
        got = capi.swa_attention(q, k, v, pos0, H, G, d, dv, 1000, 1.0, n_splits=splits)
        close(got, O.window_attention(q, k, v, H=H, G=G, d=d, dv=dv, window=1000, scale=1.0, first_pos=pos0), F32_TOL)
        assert got.min() > 45.0
    # a ring that no longer holds position 5 cannot see it, whatever the window says
    with pytest.raises(capi.XalmError):
        capi.swa_attention(q, k, v, pos0, H, G, d, dv, 1000, 1.0, ring=64)


@pytest.mark.parametrize("H,d,dv", [(2, 8, 8), (3, 16, 5), (1, 4, 40), (2, 33, 7)])
def test_hgrn2_op_and_carried_state(H, d, dv):
    rng = np.random.default_rng(H + d + dv)
    T = 21
    qz, fz, v = rng.standard_normal((T, H * d)), 2 * rng.standard_normal((T, H * d)), rng.standard_normal((T, H * dv))
    fb, lower, nw = rng.standard_normal(H * d), rng.uniform(0, 1, H * d), 1 + 0.2 * rng.standard_normal(dv)
    s0 = rng.standard_normal((H, d, dv))
    kw = dict(H=H, d=d, dv=dv, f_bias=fb, lower=lower, norm_w=nw, eps=1e-5)
    want, s_want = O.hgrn2(qz, fz, v, s0, **kw)
    got, s_got = capi.hgrn2(qz, fz, v, s0, **kw)
    close(got, want, F32_TOL)
    close(s_got, s_want, F32_TOL)
    # the same tokens in three calls that hand the state on (cuts of 2, 1 and the rest)
    st, outs = s0, []
    for a, b in ((0, 2), (2, 3), (3, T)):
        o, st = capi.hgrn2(qz[a:b], fz[a:b], v[a:b], st, **kw)
        outs.append(o)
    close(np.concatenate(outs), want, F32_TOL)
    close(st, s_want, F32_TOL)
    # no bias, no lower bound, no norm
    kw0 = dict(H=H, d=d, dv=dv)
    close(capi.hgrn2(qz, fz, v, s0, **kw0)[0], O.hgrn2(qz, fz, v, s0, **kw0)[0], F32_TOL)


def test_hgrn2_far_memory():
    """A channel whose forget gate is held at 1 - 2^-12 by its lower bound still carries the first token after 600 steps."""
    H, d, dv, T = 1, 4, 4, 600
    qz = np.full((T, d), 3.0)
    fz = np.full((T, d), -30.0)          # sigmoid ~ 0: the gate sits on its lower bound
    lower = np.array([1 - 2.0 ** -12, 0.5, 0.5, 0.5])
    v = np.zeros((T, dv))
    v[0] = 1000.0
    got, _ = capi.hgrn2(qz, fz, v, np.zeros((H, d, dv)), H, d, dv, lower=lower)
    want, _ = O.hgrn2(qz, fz, v, np.zeros((H, d, dv)), H=H, d=d, dv=dv, lower=lower)
    close(got, want, F32_TOL)
    assert got[-1].min() > 0.1


@pytest.mark.parametrize("S,W", [(1, 48), (2, 40), (3, 130), (4, 1024)])
def test_hyper_connection_ops(S, W):
    rng = np.random.default_rng(S * W)
    T = 7
    xs = rng.standard_normal((S, T, W))
    a, w = rng.standard_normal(S), 0.3 * rng.standard_normal(W)
    close(capi.hyper_norm(xs, a, w, True, 1e-5), O.norm_one_plus(O.hyper_read(xs, a), w, 1e-5), F32_TOL)
    close(capi.hyper_norm(xs, None, w, False, 1e-3), O.norm_plain(xs.sum(0), w, 1e-3), F32_TOL)
    ya, yb = rng.standard_normal((T, W)) * 3, rng.standard_normal((T, W)) * 0.01
    wa, wb = 1 + 0.2 * rng.standard_normal(W), 1 + 0.2 * rng.standard_normal(W)
    mix, oc, ls = rng.standard_normal((S, S)), rng.standard_normal(S), rng.standard_normal(W)
    y = O.join_mixers(ya, yb, wa, wb, 1e-5) * ls
    close(capi.dual_norm_hyper(xs, ya, yb, wa, wb, 1e-5, mix, oc, ls), O.hyper_write(xs, y, mix, oc), F32_TOL)


@pytest.mark.parametrize("T", [1, 3, 37])
@pytest.mark.parametrize("bf16", [False, True])
def test_clamped_glu_op(T, bf16):
    rng = np.random.default_rng(T)
    K, ff, limit = 40, 23, 1.25
    x = rng.standard_normal((T, K))
    wg, wu = O.bf16_round(rng.standard_normal((ff, K)) * 0.4), O.bf16_round(rng.standard_normal((ff, K)) * 0.4)
    want = O.glu_clamped(x, wg, wu, limit)
    assert (np.abs(x @ wu.T) > limit).any() and (x @ wg.T > limit).any()     # the clamps are in play
    close(capi.glu_rows(x, wg, wu, limit, w_bf16=bf16), want, F32_TOL)


# ---- whole models ---------------------------------------------------------------------------------------------------------
LAYER_A = dict(H=4, G=2, d=8, dv=12, window=9, softcap=6.0, Hr=2, dr=8, dvr=6, ff=56, limit=1.0)
LAYER_B = dict(H=3, G=3, d=16, dv=8, window=21, softcap=4.0, Hr=1, dr=4, dvr=24, ff=None)
LAYER_C = dict(H=2, G=1, d=4, dv=4, window=5, scale=0.9, softcap=2.0, Hr=3, dr=5, dvr=7, ff=40, limit=3.0)
LAYER_T = dict(H=4, G=2, d=8, dv=16, window=19, softcap=5.0, Hr=2, dr=6, dvr=32, ff=128, limit=1.5)   # every product a whole number of 64-wide K tiles
LAYER_W = dict(H=12, G=2, d=40, dv=24, window=1, softcap=8.0, Hr=5, dr=24, dvr=200, ff=None)             # six query heads per kv head, a window of one
LAYER_X = dict(H=16, G=2, d=16, dv=32, window=200, softcap=5.0, Hr=1, dr=130, dvr=8, ff=72, limit=0.5)   # eight per kv head, a window beyond the prompt
LAYER_1 = dict(H=1, G=1, d=64, dv=8, window=2, softcap=1.0, Hr=1, dr=1, dvr=1, ff=8, limit=1.0)          # sizes of one
CONFIGS = {
    "wide_groups": O.make_config(vocab=130, width=80, streams=4, layers=[LAYER_W, LAYER_X, LAYER_1]),
    "k64_tiles": O.make_config(vocab=68, width=64, streams=2, layers=[LAYER_T, dict(LAYER_T, ff=None), LAYER_T]),
    "mixed3": O.make_config(vocab=67, width=48, streams=2, layers=[LAYER_A, LAYER_B, LAYER_C]),
    "one_stream": O.make_config(vocab=31, width=40, streams=1, layers=[LAYER_C, LAYER_A]),
    "three_streams": O.make_config(vocab=90, width=72, streams=3, layers=[LAYER_B, LAYER_A], eps=1e-3),
}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def case(request):
    cfg = CONFIGS[request.param]
    W = O.random_weights(cfg, seed=len(request.param))
    rng = np.random.default_rng(11)
    tokens = rng.integers(0, cfg["vocab"], 75).tolist()
    logits, layers = O.forward(cfg, W, tokens)
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
    """However the prompt is cut — into steps by the caller, into passes by the engine (chunk), the ring wrapping several times
    (chunk 8 with windows up to 21 gives rings of 12-28 slots for 75 tokens) — every position's logits agree with the oracle."""
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=chunk)
    close(step_all(m, tokens, cuts), logits, F32_TOL)
    m.close()


def test_tensor_core_passes_match_the_fp32_kernels():
    """16-bit mode: passes of 32 tokens or more run their products on the tcgen05 GEMM (where every K is a multiple of 64), shorter
    ones on the fp32 FMA kernels; both agree with the oracle, with one activation plane and with hi + lo planes."""
    cfg = CONFIGS["k64_tiles"]
    W = O.random_weights(cfg, seed=9)
    tokens = np.random.default_rng(4).integers(0, cfg["vocab"], 160).tolist()
    logits, _ = O.forward(cfg, W, tokens)
    for tc, tol in ((1, BF16_TOL), (2, BF16_TOL), (0, BF16_TOL)):
        capi.tune("seq_tc", tc)
        try:
            m = on_gpu(cfg, W, capi.PRECISION_BF16, chunk=64)
        finally:
            capi.tune("seq_tc", 1)
        launches = []
        for cuts in ([160], [40, 33, 5, 18, 64]):        # both end in a pass of 32 tokens or more
            close(step_all(m, tokens, cuts), logits, tol)
            launches.append(m.last_launch_count())
            m.release()
        m.close()
        if tc == 0:
            base = launches
        else:
            tc_launches = launches
    assert tc_launches[1] != base[1] or tc_launches[0] != base[0]      # the tensor-core path really ran (it launches pack + GEMM + epilogue)


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


def test_release_gives_state_and_slots_back(case):
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=8)
    other = [(t * 7 + 3) % cfg["vocab"] for t in tokens]
    for _ in range(2):
        step_all(m, other[:50], [13])          # leaves the ring full of another sequence and a non-zero recurrent state
        m.release()
        close(step_all(m, tokens, [20, 1, 1, 9]), logits, F32_TOL)
        m.release()
    m.close()


def test_long_decoding_past_every_window():
    cfg = O.make_config(vocab=50, width=32, streams=2, layers=[LAYER_C, dict(LAYER_A, window=33)])
    W = O.random_weights(cfg, seed=5)
    tokens = np.random.default_rng(2).integers(0, 50, 260).tolist()
    logits, _ = O.forward(cfg, W, tokens)
    for precision, tol in ((capi.PRECISION_F32, 4 * F32_TOL), (capi.PRECISION_BF16, BF16_TOL)):
        m = on_gpu(cfg, W, precision, chunk=8, max_tokens=300)
        got = step_all(m, tokens, [4, 1])      # four prompt tokens, then 256 single steps: the 12- and 40-slot rings wrap many times
        close(got, logits, tol)
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
        lg, _ = O.forward(cfg, W, seq)
        seq.append(int(np.argmax(lg[-1])))
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
    cfg = json.loads(json.dumps(CONFIGS["one_stream"]))
    cfg["layers"][0]["type"] = "serial"
    with pytest.raises(capi.XalmError, match="serial"):
        Model.from_json(cfg, {}).cuda()
    cfg = json.loads(json.dumps(CONFIGS["one_stream"]))
    cfg["architecture"] = "NoSuchFamily"
    with pytest.raises(capi.XalmError, match="NoSuchFamily"):
        Model.from_json(cfg, {}).cuda()
    W = O.random_weights(CONFIGS["one_stream"], 1)
    del W["l1.mix.right.f"]
    with pytest.raises(capi.XalmError, match="l1.mix.right.f"):
        Model.from_json(CONFIGS["one_stream"], W).cuda()
