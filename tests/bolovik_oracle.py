"""Plain, slow float64 restatement of the Bolovik design, one function per mechanism, position by position.

It shares nothing with the CUDA path: no cache slots, no passes, no fused steps — every position recomputes what it sees from the
full history.  Notation: W = model width, H / G = heads / key-value heads of a mixer, d / dv = per-head key and value sizes.
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


def gelu_tanh(z):
    z = f64(z)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return np.logaddexp(0.0, f64(z))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = f64(x)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def group_norm(x, w, groups, eps):
    """The row cut into `groups` equal consecutive parts, each divided by its own root mean square; then the weight."""
    x = f64(x)
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    return unit_rms(parts, eps).reshape(x.shape) * f64(w)


def depth_average(results, coef):
    """sum_j coef[j] * results[j] over the embedding output and every layer result so far."""
    return sum(c * f64(r) for c, r in zip(f64(coef), results))


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` the long wavelengths are slowed down by `factor`, the short ones kept, and the band
    between original/high and original/low blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            lam = 2.0 * math.pi / f
            lo_edge, hi_edge = scaling["original"] / scaling["high"], scaling["original"] / scaling["low"]
            if lam > hi_edge:
                f = f / scaling["factor"]
            elif lam >= lo_edge:
                s = (scaling["original"] / lam - scaling["low"]) / (scaling["high"] - scaling["low"])
                f = (1.0 - s) * f / scaling["factor"] + s * f
        out.append(f)
    return np.array(out)


def rotate(x, pos, freqs):
    """x (..., n): the first 2*len(freqs) entries are rotated, entry i with entry i + len(freqs), by angle pos * freqs[i]."""
    x = f64(x).copy()
    r = len(freqs)
    for i in range(r):
        a = pos * freqs[i]
        u, v = x[..., i].copy(), x[..., i + r].copy()
        x[..., i] = u * math.cos(a) - v * math.sin(a)
        x[..., i + r] = v * math.cos(a) + u * math.sin(a)
    return x


def qkv_heads(proj, *, H, G, d, dv, first_pos=0, bq=None, bk=None, bv=None, freqs=None, eps=1e-5, norm_qk=True, norm_v=True):
    """proj (T, H*d + G*d + G*dv) -> q (T, H, d), k (T, G, d), v (T, G, dv) after bias, rotation and the weightless norms."""
    proj = f64(proj)
    T = proj.shape[0]
    q = proj[:, :H * d] + (0 if bq is None else f64(bq))
    k = proj[:, H * d:H * d + G * d] + (0 if bk is None else f64(bk))
    v = proj[:, H * d + G * d:] + (0 if bv is None else f64(bv))
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    if freqs is not None and len(freqs):
        for t in range(T):
            q[t] = rotate(q[t], first_pos + t, freqs)
            k[t] = rotate(k[t], first_pos + t, freqs)
    if norm_qk:
        q, k = unit_rms(q, eps), unit_rms(k, eps)
    if norm_v:
        v = unit_rms(v, eps)
    return q, k, v


def visible(i, j, window, keep_first):
    return j <= i and (i - j < window or j < keep_first)


def kept_window_attention(q, k, v, *, H, G, d, dv, window, keep_first, scale, first_pos=0):
    """q (T, H*d) for positions first_pos..; k (n, G*d), v (n, G*dv) for positions 0..n-1.  Returns (T, H*dv)."""
    q, k, v = f64(q).reshape(-1, H, d), f64(k).reshape(-1, G, d), f64(v).reshape(-1, G, dv)
    out = np.zeros((q.shape[0], H, dv))
    for t in range(q.shape[0]):
        i = first_pos + t
        seen = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = np.array([scale * float(q[t, h] @ k[j, g]) for j in seen])
            p = np.exp(s - s.max())
            p /= p.sum()
            out[t, h] = sum(pj * v[j, g] for pj, j in zip(p, seen))
    return out.reshape(-1, H * dv)


def causal_conv(x, w, before):
    """x (T, C), w (C, taps) with the last column on the current row, `before` (taps-1, C) the rows ahead of x.  Returns (y, new before)."""
    x, w, before = f64(x), f64(w), f64(before)
    taps = w.shape[1]
    full = np.concatenate([before.reshape(taps - 1, x.shape[1]), x], axis=0)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for tau in range(taps):
            y[t] += w[:, tau] * full[t + tau]
    return y, full[full.shape[0] - (taps - 1):]


def delta_rule(q, k, v, gate, b, a, state, before, *, H, G, d, dv, wq, wk, wv, A_log, dt_bias, norm_w=None, eps=1e-5, unit_eps=1e-6):
    """One run of T tokens.  q, k (T, G*d), v, gate (T, H*dv), b, a (T, H): the projections; state (H, d, dv); before (taps-1, 2*G*d + H*dv).
    Returns (out (T, H*dv), state, before)."""
    T = f64(q).shape[0]
    nq = G * d
    before = f64(before).reshape(-1, 2 * nq + H * dv)
    cq, bq_ = causal_conv(q, wq, before[:, :nq])
    ck, bk_ = causal_conv(k, wk, before[:, nq:2 * nq])
    cv, bv_ = causal_conv(v, wv, before[:, 2 * nq:])
    cq, ck, cv = silu(cq).reshape(T, G, d), silu(ck).reshape(T, G, d), silu(cv).reshape(T, H, dv)
    cq = cq / np.sqrt((cq * cq).sum(-1, keepdims=True) + unit_eps) * d ** -0.5
    ck = ck / np.sqrt((ck * ck).sum(-1, keepdims=True) + unit_eps)
    beta = sigmoid(b)
    decay = np.exp(-np.exp(f64(A_log)) * softplus(f64(a) + f64(dt_bias)))
    S = f64(state).copy()
    out = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h]
            u = beta[t, h] * (cv[t, h] - S[h].T @ ck[t, g])
            S[h] = S[h] + np.outer(ck[t, g], u)
            out[t, h] = S[h].T @ cq[t, g]
    if norm_w is not None:
        out = unit_rms(out, eps) * f64(norm_w)
    out = out.reshape(T, H * dv) * silu(gate)
    return out, S, np.concatenate([bq_, bk_, bv_], axis=1)


def route(h, w_router, top, n_groups=0, keep_groups=0):
    """Scores sigmoid(h W^T); experts in equal groups of neighbours, a group's score = its two largest scores summed, only the keep_groups
    best groups can be chosen from.  Returns (idx (T, top) best first, scores (T, top))."""
    s = sigmoid(f64(h) @ f64(w_router).T)
    T, E = s.shape
    idx, wgt = np.zeros((T, top), dtype=np.int64), np.zeros((T, top))
    for t in range(T):
        allowed = np.ones(E, dtype=bool)
        if n_groups > 1:
            size = E // n_groups
            gs = [np.sort(s[t, g * size:(g + 1) * size])[-2:].sum() for g in range(n_groups)]
            best = sorted(range(n_groups), key=lambda g: (-gs[g], g))[:keep_groups]
            allowed = np.array([(e // size) in best for e in range(E)])
        order = sorted([e for e in range(E) if allowed[e]], key=lambda e: (-s[t, e], e))[:top]
        idx[t], wgt[t] = order, s[t, order]
    return idx, wgt


def expert(h, w_gate, w_up, w_down, act=silu):
    h = f64(h)
    return (act(h @ f64(w_gate).T) * (h @ f64(w_up).T)) @ f64(w_down).T


def mixture(h, w_router, experts, top, n_groups=0, keep_groups=0):
    """experts: list of (gate, up, down).  Weighted sum of the chosen experts' outputs, weights = their scores."""
    idx, wgt = route(h, w_router, top, n_groups, keep_groups)
    h = f64(h)
    out = np.zeros((h.shape[0], f64(experts[0][2]).shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wgt[t]):
            out[t] += w * expert(h[t], *experts[e])
    return out


def forward(config, W, tokens):
    """Logits (n, vocab) of every position and what each layer hands on (layers, n, W), recomputed from the whole history."""
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    n = len(tokens)
    x = f64(W["embed"])[list(tokens)]
    results, handed = [x], []
    for li, L in enumerate(config["layers"]):
        p, mx = f"l{li}.", L["mixer"]
        H, G, d, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
        if L["type"] == "attention":
            proj = np.concatenate([x @ f64(W[p + "mix.q"]).T, x @ f64(W[p + "mix.k"]).T, x @ f64(W[p + "mix.v"]).T], axis=1)
            rot = mx.get("rot")
            freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot and rot["dims"] else None
            q, k, v = qkv_heads(proj, H=H, G=G, d=d, dv=dv, bq=W.get(p + "mix.q.b"), bk=W.get(p + "mix.k.b"), bv=W.get(p + "mix.v.b"), freqs=freqs, eps=eps)
            mask = mx.get("mask") or {}
            o = kept_window_attention(q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), H=H, G=G, d=d, dv=dv, window=mask.get("size", 10 ** 9),
                                      keep_first=mask.get("keep_first", 0), scale=mx["scale"])
        else:
            taps = mx.get("conv", 1)
            o, _, _ = delta_rule(x @ f64(W[p + "mix.q"]).T, x @ f64(W[p + "mix.k"]).T, x @ f64(W[p + "mix.v"]).T, x @ f64(W[p + "mix.g"]).T,
                                 x @ f64(W[p + "mix.b"]).T, x @ f64(W[p + "mix.a"]).T, np.zeros((H, d, dv)), np.zeros((taps - 1, 2 * G * d + H * dv)),
                                 H=H, G=G, d=d, dv=dv, wq=W[p + "mix.q.conv"], wk=W[p + "mix.k.conv"], wv=W[p + "mix.v.conv"], A_log=W[p + "mix.A_log"],
                                 dt_bias=W[p + "mix.dt_bias"], norm_w=W[p + "mix.norm"], eps=eps)
        x = x + group_norm(o @ f64(W[p + "mix.o"]).T, W[p + "norm1"], groups, eps)
        mlp = L.get("mlp")
        if mlp:
            if mlp.get("kind", "dense") == "dense":
                y = expert(x, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"], act=gelu_tanh)
            else:
                r = mlp["router"]
                ex = [(W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"]) for e in range(r["experts"])]
                gr = r.get("groups") or {}
                y = mixture(x, W[p + "mlp.router"], ex, r["top"], gr.get("count", 0), gr.get("keep", 0))
            x = x + group_norm(y, W[p + "norm2"], groups, eps)
        results.append(x)
        if p + "dwa" in W:
            x = depth_average(results, W[p + "dwa"])
        handed.append(x)
    return group_norm(x, W["final.norm"], groups, eps) @ f64(W["head"]).T, np.stack(handed)


# ---- configurations and weights for the tests -------------------------------------------------------------------------------------
def bf16_round(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def attention_layer(H, G, d, dv, window=None, keep_first=0, rot=None, scale=None, mlp=None):
    mx = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale if scale is not None else d ** -0.5}
    if window is not None:
        mx["mask"] = {"size": window, "keep_first": keep_first}
    if rot:
        mx["rot"] = rot
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def delta_layer(H, G, d, dv, conv=3, mlp=None):
    return {"type": "delta", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": conv}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=None, keep=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def make_config(*, vocab, width, layers, groups=1, eps=1e-5):
    return {"architecture": "Bolovik", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}


def random_weights(config, seed, depth_average=True):
    """bf16-exact random weights for every tensor the configuration names."""
    rng = np.random.default_rng(seed)
    W, Wd = {}, config["width"]

    def mat(rows, cols, gain=1.0):
        return bf16_round(rng.standard_normal((rows, cols)) * gain / math.sqrt(cols))

    def vec(n, mean=0.0, spread=1.0):
        return bf16_round(mean + spread * rng.standard_normal(n))

    W["embed"] = bf16_round(rng.standard_normal((config["vocab"], Wd)))
    for li, L in enumerate(config["layers"]):
        p, mx = f"l{li}.", L["mixer"]
        H, G, d, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
        W[p + "norm1"] = vec(Wd, 0.5, 0.1)
        if L["type"] == "attention":
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * d, Wd, 2.0), mat(G * d, Wd, 2.0), mat(G * dv, Wd)
            W[p + "mix.q.b"], W[p + "mix.k.b"], W[p + "mix.v.b"] = vec(H * d, 0, 0.3), vec(G * d, 0, 0.3), vec(G * dv, 0, 0.3)
        else:
            taps = mx.get("conv", 1)
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(G * d, Wd, 2.0), mat(G * d, Wd, 2.0), mat(H * dv, Wd, 2.0)
            for n_, c in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[p + f"mix.{n_}.conv"] = bf16_round(rng.standard_normal((c, taps)) * 0.6)
            W[p + "mix.b"], W[p + "mix.a"], W[p + "mix.g"] = mat(H, Wd, 2.0), mat(H, Wd, 2.0), mat(H * dv, Wd, 2.0)
            W[p + "mix.A_log"], W[p + "mix.dt_bias"], W[p + "mix.norm"] = vec(H, -1.0, 0.7), vec(H, 0.0, 1.0), vec(dv, 1.0, 0.2)
        W[p + "mix.o"] = mat(Wd, H * dv)
        mlp = L.get("mlp")
        if mlp:
            W[p + "norm2"] = vec(Wd, 0.5, 0.1)
            if mlp.get("kind", "dense") == "dense":
                W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = mat(mlp["ff"], Wd, 2.0), mat(mlp["ff"], Wd), mat(Wd, mlp["ff"])
            else:
                ff = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(ff, Wd, 2.0), mat(ff, Wd), mat(Wd, ff)
                W[p + "mlp.router"] = mat(mlp["router"]["experts"], Wd, 3.0)
        if depth_average:
            W[p + "dwa"] = bf16_round(np.r_[0.3 * rng.standard_normal(li + 1) / (li + 1), 1.0 + 0.1 * rng.standard_normal()])
    W["final.norm"] = vec(Wd, 1.0, 0.1)
    W["head"] = mat(config["vocab"], Wd)
    return W
