"""Plain, slow float64 restatement of the Nabalix design, one function per mechanism, token by token.

It shares nothing with the CUDA path: no ring, no passes, no fused steps — every position recomputes what it sees from
the full history.  Notation: W = model width, S = residual streams, H / G = query / key-value heads of the attention
mixer ("left"), d / dv its per-head key and value sizes; the recurrent mixer ("right") has its own heads and sizes.
"""
import math

import numpy as np


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return unit_rms(x, eps) * (1.0 + np.asarray(w, dtype=np.float64))


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * np.asarray(w, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, dtype=np.float64)))


def hyper_read(streams, coef):
    """u[t] = sum_s coef[s] * streams[s][t]; streams (S, T, W)."""
    return np.tensordot(np.asarray(coef, dtype=np.float64), np.asarray(streams, dtype=np.float64), axes=(0, 0))


def hyper_write(streams, y, mix, out_coef):
    """new[t'] = sum_s mix[s, t'] * old[s] + out_coef[t'] * y, every new stream from the OLD ones."""
    streams = np.asarray(streams, dtype=np.float64)
    new = np.empty_like(streams)
    for to in range(streams.shape[0]):
        acc = np.zeros_like(streams[0])
        for frm in range(streams.shape[0]):
            acc += mix[frm][to] * streams[frm]
        new[to] = acc + out_coef[to] * y
    return new


def window_attention(q, k, v, *, H, G, d, dv, window, scale, softcap=0.0, r1=None, r2=None, talk=None, gate=None, first_pos=0):
    """q (T, H*d) belongs to positions first_pos .. first_pos+T-1; k (n, G*d), v (n, G*dv) to positions 0 .. n-1, n = first_pos+T.
    Position i sees j with 0 <= i - j < window.  Returns (T, H*dv)."""
    q = np.asarray(q, dtype=np.float64).reshape(-1, H, d)
    k = np.asarray(k, dtype=np.float64).reshape(-1, G, d)
    v = np.asarray(v, dtype=np.float64).reshape(-1, G, dv)
    T = q.shape[0]
    out = np.zeros((T, H, dv))
    per = H // G
    for t in range(T):
        i = first_pos + t
        seen = [j for j in range(i + 1) if i - j < window]
        raw = np.zeros((H, len(seen)))
        for h in range(H):
            g = h // per
            for c, j in enumerate(seen):
                s = float(np.dot(q[t, h], k[j, g])) * scale
                if softcap:
                    s = softcap * math.tanh(s / softcap)
                if r1 is not None:
                    s -= float(r1[h]) * math.log(1.0 + float(r2[h]) * (i - j))
                raw[h, c] = s
        mixed = np.asarray(talk, dtype=np.float64) @ raw if talk is not None else raw
        for h in range(H):
            e = np.exp(mixed[h] - mixed[h].max())
            p = e / e.sum()
            for c, j in enumerate(seen):
                out[t, h] += p[c] * v[j, h // per]
    out = out.reshape(T, H * dv)
    if gate is not None:
        out = out * sigmoid(gate)
    return out


def hgrn2(qz, fz, v, state, *, H, d, dv, f_bias=None, lower=None, norm_w=None, eps=1e-5):
    """Gated linear recurrence; returns (out (T, H*dv), state after the last token).  state (H, d, dv)."""
    qz = np.asarray(qz, dtype=np.float64).reshape(-1, H, d)
    fz = np.asarray(fz, dtype=np.float64).reshape(-1, H, d)
    v = np.asarray(v, dtype=np.float64).reshape(-1, H, dv)
    S = np.array(state, dtype=np.float64, copy=True)
    lo = np.zeros((H, d)) if lower is None else np.asarray(lower, dtype=np.float64).reshape(H, d)
    fb = np.zeros((H, d)) if f_bias is None else np.asarray(f_bias, dtype=np.float64).reshape(H, d)
    out = np.zeros((qz.shape[0], H, dv))
    for t in range(qz.shape[0]):
        qa = qz[t] * sigmoid(qz[t])
        f = lo + (1.0 - lo) * sigmoid(fz[t] + fb)
        for h in range(H):
            S[h] = f[h][:, None] * S[h] + (1.0 - f[h])[:, None] * v[t, h][None, :]
            o = S[h].T @ qa[h]
            out[t, h] = norm_plain(o, norm_w, eps) if norm_w is not None else o
    return out.reshape(-1, H * dv), S


def join_mixers(a, b, wa, wb, eps):
    return 0.5 * (norm_plain(a, wa, eps) + norm_plain(b, wb, eps))


def glu_clamped(x, w_gate, w_up, limit, alpha=1.702):
    g = np.minimum(np.asarray(x, dtype=np.float64) @ np.asarray(w_gate, dtype=np.float64).T, limit)
    u = np.clip(np.asarray(x, dtype=np.float64) @ np.asarray(w_up, dtype=np.float64).T, -limit, limit)
    return g * sigmoid(alpha * g) * (u + 1.0)


def forward(config, W, tokens):
    """Logits (T, vocab) and the sum of the streams after every layer (L, T, width) for one sequence from position 0."""
    eps = config["norm"]["eps"]
    S = config.get("streams", 1)
    W = {n: np.asarray(a, dtype=np.float64) for n, a in W.items()}
    x = W["embed"][np.asarray(tokens)]
    T = x.shape[0]
    streams = np.stack([x.copy() for _ in range(S)])
    after = []
    for li, layer in enumerate(config["layers"]):
        p = "l%d." % li
        ones = np.ones(S)

        def sub(q, fn):
            nonlocal streams
            hp = p + "hc%d." % q
            cin = W.get(hp + "in", ones)
            h = norm_one_plus(hyper_read(streams, cin), W[p + "norm%d" % q], eps)
            y = fn(h)
            if p + "ls%d" % q in W:
                y = y * W[p + "ls%d" % q]
            streams = hyper_write(streams, y, W.get(hp + "mix", np.eye(S)), W.get(hp + "out", ones))

        def mixer(h):
            lc, rc = layer["mixer"]["left"], layer["mixer"]["right"]
            m = p + "mix.left."
            H, G, d, dv = lc["heads"], lc.get("kv_heads", lc["heads"]), lc["dim"], lc.get("vdim", lc["dim"])
            window = lc["mask"]["size"] if lc.get("mask") else T + 1
            att = window_attention(h @ W[m + "q"].T, h @ W[m + "k"].T, h @ W[m + "v"].T, H=H, G=G, d=d, dv=dv, window=window,
                                   scale=lc["scale"], softcap=lc.get("softcap", 0.0), r1=W.get(m + "r1"), r2=W.get(m + "r2"),
                                   talk=W.get(m + "talk"), gate=(h @ W[m + "g"].T) if m + "g" in W else None)
            left = att @ W[m + "o"].T
            r = p + "mix.right."
            Hr, dr, dvr = rc["heads"], rc["dim"], rc.get("vdim", rc["dim"])
            rec, _ = hgrn2(h @ W[r + "q"].T, h @ W[r + "f"].T, h @ W[r + "v"].T, np.zeros((Hr, dr, dvr)), H=Hr, d=dr, dv=dvr,
                           f_bias=W.get(r + "f.b"), lower=W.get(r + "lower"), norm_w=W.get(r + "norm"), eps=eps)
            right = rec @ W[r + "o"].T
            return join_mixers(left, right, W[p + "mix.left.out"], W[p + "mix.right.out"], eps)

        sub(1, mixer)
        if layer.get("mlp"):
            mc = layer["mlp"]
            sub(2, lambda h: glu_clamped(h, W[p + "mlp.gate"], W[p + "mlp.up"], mc["limit"]) @ W[p + "mlp.down"].T)
        after.append(streams.sum(axis=0))
    x = streams.sum(axis=0)
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T, np.stack(after)


# ---- small random models ------------------------------------------------------------------------------------------------
def bf16_round(a):
    """fp32 values rounded to the nearest bf16 (ties to even), so that 16-bit and 32-bit uploads hold the same numbers."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def make_config(*, vocab=67, width=48, streams=2, layers=None, eps=1e-5):
    """layers: list of dicts with keys H, G, d, dv, window, scale, softcap, Hr, dr, dvr, ff (None: no feed-forward), limit."""
    out = []
    for L in layers:
        left = {"heads": L["H"], "kv_heads": L["G"], "dim": L["d"], "vdim": L["dv"], "scale": L.get("scale", L["d"] ** -0.5),
                "softcap": L.get("softcap", 12.0), "mask": {"size": L["window"]}}
        right = {"heads": L["Hr"], "dim": L["dr"], "vdim": L["dvr"]}
        mlp = None if L.get("ff") is None else {"kind": "dense", "ff": L["ff"], "limit": L.get("limit", 2.0)}
        out.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp})
    return {"architecture": "Nabalix", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps}, "layers": out}


def random_weights(config, seed, spread=1.0):
    """Weights scaled so that every mechanism matters: scores of a few units (peaky softmax, soft cap in reach), distance bias and
    head mixing of order one, forget gates spread over (0, 1) with some lower bounds near 1, gate / up values reaching the clamp."""
    rng = np.random.default_rng(seed)
    Wd, S, V = config["width"], config.get("streams", 1), config["vocab"]
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)) * gain / math.sqrt(cols))

    def vec(name, n, center, dev):
        W[name] = bf16_round(center + dev * rng.standard_normal(n))

    W["embed"] = bf16_round(rng.standard_normal((V, Wd)))
    for li, layer in enumerate(config["layers"]):
        p = "l%d." % li
        lc, rc = layer["mixer"]["left"], layer["mixer"]["right"]
        H, G, d, dv = lc["heads"], lc["kv_heads"], lc["dim"], lc["vdim"]
        Hr, dr, dvr = rc["heads"], rc["dim"], rc["vdim"]
        vec(p + "norm1", Wd, 0.0, 0.2)
        mat(p + "mix.left.q", H * d, Wd, 2.5 * spread / math.sqrt(lc["scale"] * math.sqrt(d)))
        mat(p + "mix.left.k", G * d, Wd, 2.5 * spread / math.sqrt(lc["scale"] * math.sqrt(d)))
        mat(p + "mix.left.v", G * dv, Wd)
        W[p + "mix.left.r1"] = bf16_round(rng.uniform(0.1, 1.0, H))
        W[p + "mix.left.r2"] = bf16_round(rng.uniform(0.05, 2.0, H))
        W[p + "mix.left.talk"] = bf16_round(np.eye(H) + 0.3 * rng.standard_normal((H, H)))
        mat(p + "mix.left.g", H * dv, Wd, 2.0)
        mat(p + "mix.left.o", Wd, H * dv)
        mat(p + "mix.right.q", Hr * dr, Wd, 1.5)
        mat(p + "mix.right.f", Hr * dr, Wd, 2.0)
        vec(p + "mix.right.f.b", Hr * dr, 1.0, 1.0)
        W[p + "mix.right.lower"] = bf16_round(rng.uniform(0.0, 1.0, Hr * dr) ** 0.3)
        mat(p + "mix.right.v", Hr * dvr, Wd)
        vec(p + "mix.right.norm", dvr, 1.0, 0.2)
        mat(p + "mix.right.o", Wd, Hr * dvr)
        vec(p + "mix.left.out", Wd, 1.0, 0.2)
        vec(p + "mix.right.out", Wd, 1.0, 0.2)
        vec(p + "ls1", Wd, 0.7, 0.2)
        subs = [1]
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            vec(p + "norm2", Wd, 0.0, 0.2)
            mat(p + "mlp.gate", ff, Wd, 1.5 * layer["mlp"]["limit"])
            mat(p + "mlp.up", ff, Wd, 1.5 * layer["mlp"]["limit"])
            mat(p + "mlp.down", Wd, ff)
            vec(p + "ls2", Wd, 0.7, 0.2)
            subs.append(2)
        for q in subs:
            hp = p + "hc%d." % q
            vec(hp + "in", S, 1.0 / S, 0.2)
            vec(hp + "out", S, 1.0, 0.3)
            W[hp + "mix"] = bf16_round(np.eye(S) + 0.2 * rng.standard_normal((S, S)))
    vec("final.norm", Wd, 0.0, 0.2)
    mat("head", V, Wd)
    return W
