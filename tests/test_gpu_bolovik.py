"""Bolovik on the GPU against the plain restatement in tests/bolovik_oracle.py: every mechanism alone (op-level entry points that launch
the family's kernels), then whole models with small random configurations — prompts in one pass, token by token, in portions, across
ring wrap and release, long decoding past every window, greedy generation through the host entry points and the command line."""
import json
import os
import subprocess

import numpy as np
import pytest

import bolovik_oracle as O
from xalm_b200 import build, capi
from xalm_b200 import safetensors_io as ST
from xalm_b200.model import InferenceState, Model, Sampler, generate

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4   # IEEE fp32 path against float64, on values of order one
BF16_TOL = 6e-2  # serving mode: bf16 weights (exact here), a bf16 K/V cache, fp16 operands on the tensor cores


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err < tol, f"max error {err:.3e} (tolerance {tol})"


# ---- mechanisms alone ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W,groups", [(48, 1), (48, 4), (130, 5), (1024, 8), (36, 36)])
def test_group_norm_residual_and_depth_average(W, groups):
    rng = np.random.default_rng(W + groups)
    T, parts, n_hist = 7, 3, 4
    y, w, x = rng.standard_normal((T, W)) * 3, 1 + 0.2 * rng.standard_normal(W), rng.standard_normal((T, W))
    y[:, : W // groups] *= 40.0                                   # one group far louder than the rest: a norm over the whole row would flatten the others
    close(capi.group_norm_residual(y, w, groups, 1e-5, x_in=x), x + O.group_norm(y, w, groups, 1e-5), F32_TOL)
    close(capi.group_norm_residual(y, w, groups, 1e-3), O.group_norm(y, w, groups, 1e-3), F32_TOL)          # no residual: the closing norm
    yp, pw = rng.standard_normal((T, parts, W)), rng.uniform(0.1, 1, (T, parts))
    want = x + O.group_norm((yp * pw[:, :, None]).sum(1), w, groups, 1e-5)
    close(capi.group_norm_residual(yp, w, groups, 1e-5, x_in=x, part_w=pw), want, F32_TOL)
    hist, coef = rng.standard_normal((n_hist, T, W)), rng.standard_normal(n_hist + 1)
    got_x, got_avg = capi.group_norm_residual(yp, w, groups, 1e-5, x_in=x, part_w=pw, hist=hist, dwa=coef)
    close(got_x, want, F32_TOL)
    close(got_avg, O.depth_average(list(hist) + [want], coef), F32_TOL)


@pytest.mark.parametrize("H,G,d,dv,rot_dims", [(4, 2, 8, 12, 4), (3, 3, 16, 4, 16), (6, 1, 20, 20, 0), (1, 1, 64, 8, 32), (2, 2, 6, 3, 2)])
def test_qkv_post_rotation_norms_and_slots(H, G, d, dv, rot_dims):
    rng = np.random.default_rng(H * d + rot_dims)
    T, pos0, keep, ring = 6, 1000, 3, 7
    proj = rng.standard_normal((T, H * d + G * d + G * dv)) * 2
    bq, bk, bv = rng.standard_normal(H * d), rng.standard_normal(G * d), rng.standard_normal(G * dv)
    scaling = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    freqs = O.rotary_frequencies(rot_dims, 100.0, scaling) if rot_dims else None
    if rot_dims >= 16:     # the three bands are all in play: some kept, some slowed by the factor
        plain = O.rotary_frequencies(rot_dims, 100.0)
        assert np.isclose(freqs[0], plain[0]) and np.isclose(freqs[-1], plain[-1] / 8.0)
    q, k, v = O.qkv_heads(proj, H=H, G=G, d=d, dv=dv, first_pos=pos0, bq=bq, bk=bk, bv=bv, freqs=freqs, eps=1e-5)
    gq, kc, vc = capi.qkv_post(proj, pos0, H, G, d, dv, bq, bk, bv, freqs, eps=1e-5, keep_first=keep, ring=ring)
    close(gq, q.reshape(T, -1), F32_TOL)
    for t in range(T):                                             # position p sits in slot keep + (p - keep) % ring: these six run over the ring's end
        slot = keep + (pos0 + t - keep) % ring
        close(kc[slot], k[t].reshape(-1), F32_TOL)
        close(vc[slot], v[t].reshape(-1), F32_TOL)
    assert not kc[:keep].any()                                     # nobody wrote the pinned slots: these positions are past them
    # the first positions of a sequence land in the pinned slots, unrotated at position 0
    gq0, kc0, _ = capi.qkv_post(proj[:4], 0, H, G, d, dv, None, None, None, freqs, norm_qk=False, norm_v=False, keep_first=keep, ring=ring)
    q0, k0, _ = O.qkv_heads(proj[:4], H=H, G=G, d=d, dv=dv, freqs=freqs, norm_qk=False, norm_v=False)
    close(gq0, q0.reshape(4, -1), F32_TOL)
    close(kc0[:4], k0.reshape(4, -1), F32_TOL)
    close(gq0[0], proj[0, :H * d], 1e-6)


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 8, 12), (3, 3, 16, 4), (6, 1, 4, 20), (1, 1, 32, 32), (8, 2, 24, 8)])
@pytest.mark.parametrize("pos0,T,window,keep,splits", [(0, 9, 4, 2, 1), (0, 40, 64, 5, 1), (37, 1, 16, 6, 3), (50, 6, 7, 3, 1), (129, 1, 30, 20, 4),
                                                       (65, 2, 33, 1, 2), (70, 24, 12, 40, 1), (3, 5, 2, 0, 1), (90, 1, 8, 8, 1)])
def test_kept_window_attention_op(H, G, d, dv, pos0, T, window, keep, splits):
    rng = np.random.default_rng(H * 100 + pos0 + window)
    n = pos0 + T
    q, k, v = rng.standard_normal((T, H * d)) * 1.5, rng.standard_normal((n, G * d)), rng.standard_normal((n, G * dv))
    kw = dict(H=H, G=G, d=d, dv=dv, window=window, keep_first=keep, scale=0.4)
    want = O.kept_window_attention(q, k, v, first_pos=pos0, **kw)
    close(capi.swa_attention_kept(q, k, v, pos0, n_splits=splits, **kw), want, F32_TOL)
    kb, vb = O.bf16_round(k), O.bf16_round(v)
    close(capi.swa_attention_kept(q, kb, vb, pos0, n_splits=splits, cache_bf16=True, **kw), O.kept_window_attention(q, kb, vb, first_pos=pos0, **kw), F32_TOL)


@pytest.mark.parametrize("T,splits", [(5, 1), (1, 1), (1, 3), (12, 1)])
@pytest.mark.parametrize("where", ["window_in", "window_out", "kept_in", "kept_out"])
@pytest.mark.parametrize("dv", [4, 8])
def test_edges_of_window_and_kept_positions_stand_out(T, splits, where, dv):
    """One key carries a score far above the rest and a value nobody else has.  It sits on the last place the window still shows, one
    further back, on the last kept position, or on the first one that is not kept — for the last row of a portion and for a token alone."""
    H, G, d, window, keep, pos0 = 2, 1, 8, 24, 6, 90
    n = pos0 + T
    i = n - 1
    target = {"window_in": i - (window - 1), "window_out": i - window, "kept_in": keep - 1, "kept_out": keep}[where]
    rng = np.random.default_rng(7)
    k, v = 0.05 * rng.standard_normal((n, G * d)), 0.05 * rng.standard_normal((n, G * dv))
    k[target, 0] = 6.0
    v[target] = 100.0
    q = 0.05 * rng.standard_normal((T, H * d))
    q[:, 0] = q[:, d] = 5.0
    kw = dict(H=H, G=G, d=d, dv=dv, window=window, keep_first=keep, scale=1.0)
    got = capi.swa_attention_kept(q, k, v, pos0, n_splits=splits, **kw)
    close(got, O.kept_window_attention(q, k, v, first_pos=pos0, **kw), F32_TOL)
    assert (got[-1].min() > 90.0) == where.endswith("_in")         # seen exactly when it should be
    if T > 1 and where == "window_out":
        assert got[-2].min() > 90.0                                # the row before still sees it


def test_far_key_among_hundreds_with_and_without_keeping():
    H, G, d, dv, pos0, T = 2, 2, 8, 16, 700, 1
    n = pos0 + T
    rng = np.random.default_rng(3)
    k, v = 0.05 * rng.standard_normal((n, G * d)), 0.05 * rng.standard_normal((n, G * dv))
    k[5, 0] = k[5, d] = 8.0
    v[5] = 50.0
    q = np.zeros((T, H * d))
    q[:, 0] = q[:, d] = 4.0
    for splits in (1, 5):
        kw = dict(H=H, G=G, d=d, dv=dv, scale=1.0, n_splits=splits)
        assert capi.swa_attention_kept(q, k, v, pos0, window=1000, keep_first=0, **kw).min() > 45.0     # a window over everything
        assert capi.swa_attention_kept(q, k, v, pos0, window=64, keep_first=6, **kw).min() > 45.0       # kept although 695 positions back
        assert capi.swa_attention_kept(q, k, v, pos0, window=64, keep_first=5, **kw).max() < 5.0        # position 5 is the first not kept


@pytest.mark.parametrize("H,G,d,dv,taps", [(2, 1, 8, 8, 3), (3, 3, 16, 5, 2), (4, 2, 33, 7, 4), (2, 2, 64, 40, 1), (2, 1, 128, 32, 3), (1, 1, 136, 12, 3), (6, 3, 4, 70, 5)])
def test_delta_rule_op_and_carried_state(H, G, d, dv, taps):
    rng = np.random.default_rng(H + d + dv + taps)
    T, nq, nv = 37, G * d, H * dv
    q, k, v = rng.standard_normal((T, nq)) * 2, rng.standard_normal((T, nq)) * 2, rng.standard_normal((T, nv)) * 2
    gate, b, a = rng.standard_normal((T, nv)), rng.standard_normal((T, H)) * 2, rng.standard_normal((T, H)) * 2
    par = dict(wq=rng.standard_normal((nq, taps)) * 0.6, wk=rng.standard_normal((nq, taps)) * 0.6, wv=rng.standard_normal((nv, taps)) * 0.6,
               A_log=rng.standard_normal(H) - 1, dt_bias=rng.standard_normal(H), norm_w=1 + 0.2 * rng.standard_normal(dv), eps=1e-5)
    s0, c0 = rng.standard_normal((H, d, dv)) * 0.3, rng.standard_normal((taps - 1, 2 * nq + nv))
    want, s_want, c_want = O.delta_rule(q, k, v, gate, b, a, s0, c0, H=H, G=G, d=d, dv=dv, **par)
    got, s_got, c_got = capi.delta_rule(q, k, v, gate, b, a, s0, c0, H, G, d, dv, **par)
    close(got, want, F32_TOL)
    close(s_got, s_want, F32_TOL)
    if taps > 1:
        close(c_got, c_want, 1e-6)
    # the same tokens in calls that hand state and convolution inputs on: cuts of 2, 1, 1 (shorter than the taps), 17 (past a staging tile), the rest
    st, cs, outs = s0, c0, []
    for lo, hi in ((0, 2), (2, 3), (3, 4), (4, 21), (21, T)):
        o, st, cs = capi.delta_rule(q[lo:hi], k[lo:hi], v[lo:hi], gate[lo:hi], b[lo:hi], a[lo:hi], st, cs, H, G, d, dv, **par)
        outs.append(o)
    close(np.concatenate(outs), want, F32_TOL)
    close(st, s_want, F32_TOL)
    # no output norm
    par0 = dict(par, norm_w=None)
    close(capi.delta_rule(q, k, v, gate, b, a, s0, c0, H, G, d, dv, **par0)[0], O.delta_rule(q, k, v, gate, b, a, s0, c0, H=H, G=G, d=d, dv=dv, **par0)[0], F32_TOL)


def test_delta_rule_remembers_and_overwrites():
    """With decay held at one, a value written under a key is read back 500 tokens later through the same key; writing the same key again with
    full strength replaces it (the rule subtracts what the state already returns for the key)."""
    H, G, d, dv, T = 1, 1, 4, 4, 500
    big = 30.0                                                     # silu(30) = 30: the convolution (one tap of 1) passes it on
    q, k, v = np.zeros((T, d)), np.zeros((T, d)), np.zeros((T, dv))
    k[:, 1] = big                                                  # everybody else writes zeros under key 1
    k[0] = k[T - 1] = [big, 0, 0, 0]
    q[T - 1] = [big, 0, 0, 0]
    v[0] = [big, 0, 0, 0]
    v[T - 1] = [0, 0, big, 0]
    one = np.ones((d, 1))
    par = dict(wq=one, wk=one, wv=np.ones((dv, 1)), A_log=np.array([-40.0]), dt_bias=np.zeros(1))    # exp(-40): no decay to speak of
    gate, a = np.full((T, dv), big), np.zeros((T, H))
    z = np.zeros((H, d, dv))
    weak, strong = np.full((T, H), -40.0), np.full((T, H), -40.0)
    weak[0] = strong[0] = strong[T - 1] = 40.0                      # beta: 1 where a write should land, 0 elsewhere
    got, _, _ = capi.delta_rule(q, k, v, gate, weak, a, z, np.zeros((0, 0)), H, G, d, dv, **par)
    want, _, _ = O.delta_rule(q, k, v, gate, weak, a, z, np.zeros((0, 3 * d)), H=H, G=G, d=d, dv=dv, **par)
    close(got, want, F32_TOL)
    assert got[-1, 0] > 0.4 * big * 0.5 * big and abs(got[-1, 2]) < 1e-3   # token 0's value comes back, the last token's write (beta 0) does not show
    got2, _, _ = capi.delta_rule(q, k, v, gate, strong, a, z, np.zeros((0, 0)), H, G, d, dv, **par)
    close(got2, O.delta_rule(q, k, v, gate, strong, a, z, np.zeros((0, 3 * d)), H=H, G=G, d=d, dv=dv, **par)[0], F32_TOL)
    assert abs(got2[-1, 0]) < 1e-3 * got[-1, 0] and got2[-1, 2] > 0.9 * got[-1, 0]                   # replaced, not added


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 0, 0), (12, 3, 4, 2), (6, 6, 3, 3), (5, 1, 5, 2), (16, 4, 2, 1), (9, 2, 3, 1)])
@pytest.mark.parametrize("bf16", [False, True])
def test_router_and_experts_op(E, top, groups, keep, bf16):
    rng = np.random.default_rng(E * 10 + top)
    T, K, ff = 70, 40, 12                                          # 70 x top pairs: several row tiles for a popular expert
    h = rng.standard_normal((T, K))
    wr = O.bf16_round(rng.standard_normal((E, K)) * 0.5)
    wg, wu, wd = (O.bf16_round(rng.standard_normal(s) * 0.3) for s in ((E, ff, K), (E, ff, K), (E, K, ff)))
    idx, wgt = O.route(h, wr, top, groups, keep)
    gi, gw, out = capi.moe_ffn(h, wr, wg, wu, wd, top, groups, keep, w_bf16=bf16)
    assert np.array_equal(gi, idx)                                 # best first, as the restatement orders them
    close(gw, wgt, F32_TOL)
    for t in range(0, T, 7):
        for s in range(top):
            close(out[t, s], O.expert(h[t], wg[idx[t, s]], wu[idx[t, s]], wd[idx[t, s]]), F32_TOL)
    if groups > 1 and keep < groups and E // groups > 1:           # the groups bite: somewhere an expert with a larger score was passed over
        free, _ = O.route(h, wr, top)
        assert not np.array_equal(np.sort(free, 1), np.sort(idx, 1))


def test_group_limit_passes_over_the_largest_score():
    """Expert 0 has the largest score of all but sits alone in a weak group; groups 1 and 2 hold two good experts each and are the ones kept."""
    K, E = 6, 6
    wr = np.zeros((E, K))
    wr[0, 0] = 3.0
    wr[1, 0] = -6.0
    for e in (2, 3, 4, 5):
        wr[e, 0] = 2.0 + 0.1 * e
    h = np.zeros((1, K))
    h[0, 0] = 1.0
    wg = wu = np.ones((E, 2, K))
    wd = np.ones((E, K, 2))
    idx, wgt, _ = capi.moe_ffn(h, wr, wg, wu, wd, 2, 3, 2)
    assert list(idx[0]) == [5, 4]
    idx, _, _ = capi.moe_ffn(h, wr, wg, wu, wd, 2)
    assert list(idx[0]) == [0, 5]


# ---- whole models ---------------------------------------------------------------------------------------------------------
ROT = {"base": 10000.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 40}}
CONFIGS = {
    # attention first and last, grouped experts, three norm groups, rotation on part of the head
    "mixed": O.make_config(vocab=67, width=48, groups=3, layers=[
        O.attention_layer(4, 2, 8, 12, window=9, keep_first=3, rot=ROT, mlp=O.moe(10, 6, 2, groups=3, keep=2)),
        O.delta_layer(4, 2, 8, 6, conv=3, mlp=O.dense(56)),
        O.attention_layer(3, 3, 16, 8, window=21, keep_first=0, rot={"base": 500.0, "dims": 16}, scale=0.31, mlp=None)]),
    # delta first; kv heads = heads; one norm group; experts without groups; a window of one; no rotation; taps 2 and 4
    "delta_first": O.make_config(vocab=31, width=40, groups=1, eps=1e-3, layers=[
        O.delta_layer(2, 2, 5, 7, conv=4, mlp=O.moe(8, 4, 1)),
        O.attention_layer(2, 1, 4, 4, window=1, keep_first=2, mlp=O.dense(24)),
        O.delta_layer(3, 1, 12, 3, conv=2, mlp=None),
        O.attention_layer(5, 5, 6, 10, window=5, keep_first=1, rot={"base": 50.0, "dims": 6}, mlp=O.moe(6, 3, 3, groups=3, keep=3))]),
    # every product a whole number of 64-wide K tiles: the 16-bit mode's long passes run on the tensor cores; no window in the second layer
    "k64_tiles": O.make_config(vocab=68, width=64, groups=4, layers=[
        O.attention_layer(4, 2, 16, 16, window=19, keep_first=4, rot={"base": 1000.0, "dims": 8}, mlp=O.dense(128)),
        O.attention_layer(2, 1, 32, 32, mlp=O.moe(64, 4, 2, groups=2, keep=1)),
        O.delta_layer(4, 2, 16, 16, conv=3, mlp=O.dense(64))]),
    # a wide delta head (state in shared memory), eight heads per kv head, keep_first beyond the window
    "wide": O.make_config(vocab=90, width=72, groups=2, layers=[
        O.delta_layer(1, 1, 132, 9, conv=3, mlp=None),
        O.attention_layer(8, 1, 12, 20, window=6, keep_first=11, rot={"base": 100.0, "dims": 12, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 16}},
                          mlp=O.moe(5, 7, 3))]),
}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def case(request):
    cfg = CONFIGS[request.param]
    W = O.random_weights(cfg, seed=len(request.param), depth_average=request.param != "wide")
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
    """However the prompt is cut — into steps by the caller, into passes by the engine (chunk), the rings wrapping several times
    (chunk 8 with windows of 1 to 21 gives rings of 8 to 28 slots for 75 tokens) — every position's logits agree with the oracle."""
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=chunk)
    close(step_all(m, tokens, cuts), logits, F32_TOL)
    m.close()


def test_tensor_core_passes_match_the_fp32_kernels():
    cfg = CONFIGS["k64_tiles"]
    W = O.random_weights(cfg, seed=9)
    tokens = np.random.default_rng(4).integers(0, cfg["vocab"], 130).tolist()
    logits, _ = O.forward(cfg, W, tokens)
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


def test_release_gives_state_and_slots_back(case):
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=8)
    other = [(t * 7 + 3) % cfg["vocab"] for t in tokens]
    for _ in range(2):
        step_all(m, other[:50], [13])          # leaves pinned slots and rings full of another sequence, recurrent and convolution state non-zero
        m.release()
        close(step_all(m, tokens, [20, 1, 1, 9]), logits, F32_TOL)
        m.release()
    m.close()


def test_long_decoding_past_every_window():
    cfg = O.make_config(vocab=50, width=32, groups=2, layers=[
        O.attention_layer(2, 1, 4, 6, window=33, keep_first=5, rot={"base": 20.0, "dims": 4}, mlp=O.moe(6, 4, 2, groups=2, keep=1)),
        O.delta_layer(2, 1, 6, 4, conv=3, mlp=O.dense(20))])
    W = O.random_weights(cfg, seed=5)
    tokens = np.random.default_rng(2).integers(0, 50, 200).tolist()
    logits, _ = O.forward(cfg, W, tokens)
    for precision, tol in ((capi.PRECISION_F32, 4 * F32_TOL), (capi.PRECISION_BF16, BF16_TOL)):
        m = on_gpu(cfg, W, precision, chunk=8, max_tokens=220)
        got = step_all(m, tokens, [4, 1])      # four prompt tokens, then 196 single steps: the 40-slot ring wraps many times, five positions stay pinned
        close(got, logits, tol)
        m.close()


def test_first_tokens_and_tiny_sequences(case):
    cfg, W, tokens, logits, _ = case
    m = on_gpu(cfg, W, capi.PRECISION_F32)
    for n in (1, 2, 3):
        close(m.prefill(tokens[:n], 0, 2), logits[:n], F32_TOL)
        m.release()
    m.close()


def test_without_depth_average_and_without_biases():
    cfg = CONFIGS["mixed"]
    W = O.random_weights(cfg, seed=21, depth_average=False)
    for n in [n for n in W if n.endswith(".b") and ".mix." in n and n.count(".") == 3]:
        del W[n]                               # q.b / k.b / v.b of the attention layers
    tokens = np.random.default_rng(8).integers(0, cfg["vocab"], 40).tolist()
    logits, _ = O.forward(cfg, W, tokens)
    m = on_gpu(cfg, W, capi.PRECISION_F32, chunk=16)
    close(step_all(m, tokens, [17, 2, 1]), logits, F32_TOL)
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
    cfg = json.loads(json.dumps(CONFIGS["mixed"]))
    cfg["layers"][0]["type"] = "convolution"
    with pytest.raises(capi.XalmError, match="convolution"):
        Model.from_json(cfg, {}).cuda()
    W = O.random_weights(CONFIGS["mixed"], 1)
    del W["l1.mix.A_log"]
    with pytest.raises(capi.XalmError, match="l1.mix.A_log"):
        Model.from_json(CONFIGS["mixed"], W).cuda()
