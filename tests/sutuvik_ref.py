"""Plain float64 restatement of the Sutuvik design, one function per mechanism, numpy only.

It shares no code with the product path: whole sequences, loops over tokens and heads, no cache,
no state slots.  `forward(cfg_json, weights, tokens)` returns the logits of every position.

Notation: x [T, W] is the residual stream, h what a sublayer reads, names of `weights` are the
checkpoint's ("l<i>.mix.q", ...), linears are [out, in]."""
import math

import numpy as np


# ------------------------------------------------------------------ small pieces
def rms_parts(x, weight, parts, eps):
    """Split every row into `parts` equal consecutive pieces, divide each piece by
    sqrt(mean(piece^2) + eps), multiply the whole row by `weight`."""
    T, n = x.shape
    p = x.reshape(T, parts, n // parts)
    p = p / np.sqrt((p * p).mean(axis=-1, keepdims=True) + eps)
    return p.reshape(T, n) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def causal_conv(u, taps_w, bias=None):
    """y_t = sum_j taps_w[:, j] * u_(t - n + 1 + j), n taps, the last column meets u_t itself;
    u is zero before the sequence's start.  u [T, C], taps_w [C, n]."""
    T, C = u.shape
    n = taps_w.shape[1]
    y = np.zeros((T, C))
    for t in range(T):
        for j in range(n):
            src = t - n + 1 + j
            if src >= 0:
                y[t] += taps_w[:, j] * u[src]
    return y if bias is None else y + bias


def rotation_frequencies(rot):
    """f_i = base^(-2i / dims); with `scaling`, by wavelength l = 2 pi / f: short ones (l < original /
    high) stay, long ones (l > original / low) become f / factor, the rest is blended."""
    dims = rot["dims"]
    f = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f
    out = []
    for fi in f:
        wl = 2.0 * math.pi / fi
        if wl < sc["original"] / sc["high"]:
            out.append(fi)
        elif wl > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * fi / sc["factor"] + s * fi)
    return np.array(out)


def rotate_pairs(x, freqs, positions):
    """Entries (2i, 2i + 1) of every head turn by the angle position * freqs[i]; entries past
    2 len(freqs) stay.  x [T, heads, dim]."""
    y = x.copy()
    for i, f in enumerate(freqs):
        ang = positions * f
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        a, b = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        y[:, :, 2 * i] = a * c - b * s
        y[:, :, 2 * i + 1] = b * c + a * s
    return y


def softmax_with_sink(scores, sink):
    """Rows of `scores` ([T, T], -inf where a key is hidden) to weights whose denominator holds one
    more term exp(sink): weights sum to less than one."""
    m = np.maximum(scores.max(axis=-1, keepdims=True), sink)
    e = np.exp(scores - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def mix_values(v, mx, w, pre, shared):
    """Layers that mix values: the first one's values are kept for the others, which blend
    theirs with them token by token."""
    if not mx.get("v_mix"):
        return v
    if "v_first" not in shared:
        shared["v_first"] = v
        return v
    lam = float(np.asarray(w[pre + "vmix"]).reshape(-1)[0])
    return (1.0 - lam) * v + lam * shared["v_first"]


# ------------------------------------------------------------------ mixers
def attention_biased(h, mx, w, pre, eps, shared):
    """Grouped heads; q and k normed per head with a shared weight; q grows with the position;
    a penalty linear in the distance; a learned sink per head; a gate per head."""
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, dk)
    k = (h @ w[pre + "k"].T).reshape(T, G, dk)
    v = (h @ w[pre + "v"].T).reshape(T, G, dv)
    q = q / np.sqrt((q * q).mean(-1, keepdims=True) + eps) * w[pre + "q.norm"]
    k = k / np.sqrt((k * k).mean(-1, keepdims=True) + eps) * w[pre + "k.norm"]
    pos = np.arange(T)
    qt = mx.get("q_temp")
    if qt:
        q = q * (1.0 + qt["coef"] * np.log(np.floor((pos + 1) / qt["every"]) + 1.0))[:, None, None]
    v = mix_values(v, mx, w, pre, shared)
    dist = pos[:, None] - pos[None, :]
    hidden = dist < 0
    gate = sigmoid(h @ w[pre + "g"].T)
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * mx["scale"] - 2.0 ** (-8.0 * (a + 1) / H) * dist
        s[hidden] = -np.inf
        out[:, a] = softmax_with_sink(s, float(w[pre + "sink"][a])) @ v[:, g] * gate[:, a:a + 1]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def attention_rotary(h, mx, w, pre, eps, shared):
    """Grouped heads; q and k rotated (leading entries, neighbouring pairs) and then divided by
    their root mean square; a multiplier per head; capped scores; a sink of score zero."""
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, dk)
    k = (h @ w[pre + "k"].T).reshape(T, G, dk)
    v = (h @ w[pre + "v"].T).reshape(T, G, dv)
    pos = np.arange(T, dtype=np.float64)
    if mx.get("rot"):
        f = rotation_frequencies(mx["rot"])
        q, k = rotate_pairs(q, f, pos), rotate_pairs(k, f, pos)
    q = q / np.sqrt((q * q).mean(-1, keepdims=True) + eps)
    k = k / np.sqrt((k * k).mean(-1, keepdims=True) + eps)
    v = mix_values(v, mx, w, pre, shared)
    hidden = pos[None, :] > pos[:, None]
    cap = mx.get("softcap")
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * mx["scale"] * w[pre + "temp"][a]
        if cap:
            s = cap * np.tanh(s / cap)
        s[hidden] = -np.inf
        out[:, a] = softmax_with_sink(s, 0.0) @ v[:, g]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def state_space_scan(x, B, C, dt, a_log, d_skip, heads_per_group):
    """Per head: S <- exp(-exp(a_log) dt_t) S + dt_t B_t x_t^T, y_t = S^T C_t + d_skip x_t.
    x [T, heads, p], B / C [T, groups, n], dt [T, heads]."""
    T, nh, p = x.shape
    y = np.zeros((T, nh, p))
    for a in range(nh):
        g = a // heads_per_group
        S = np.zeros((B.shape[2], p))
        for t in range(T):
            S = math.exp(-math.exp(a_log[a]) * dt[t, a]) * S + dt[t, a] * np.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + d_skip[a] * x[t, a]
    return y


def mamba2(h, mx, w, pre, eps):
    T = h.shape[0]
    nh, p, n, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = nh * p
    u = h @ w[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * n], u[:, 2 * inner + 2 * G * n:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, nh, p)
    B = xbc[:, inner:inner + G * n].reshape(T, G, n)
    C = xbc[:, inner + G * n:].reshape(T, G, n)
    dt = softplus(dt + w[pre + "dt_bias"])
    y = state_space_scan(x, B, C, dt, w[pre + "A_log"], w[pre + "D"], nh // G).reshape(T, inner)
    y = rms_parts(y * silu(z), w[pre + "norm"], mx["norm_groups"], eps)  # the gate comes before the norm
    return y @ w[pre + "o"].T


# ------------------------------------------------------------------ feed-forward
def choose_experts(scores, correction, router):
    """Indices of the experts a token uses: ranked by score + correction; with groups only the
    experts of the `keep` groups whose two best ranked scores add up highest take part."""
    E, top = router["experts"], router["top"]
    rank = scores + correction
    g = router.get("groups")
    if g and g["count"] > 1 and g["keep"] < g["count"]:
        per = E // g["count"]
        gs = [np.sort(rank[i * per:(i + 1) * per])[::-1][:2].sum() for i in range(g["count"])]
        kept = sorted(range(g["count"]), key=lambda i: (-gs[i], i))[:g["keep"]]
        rank = np.array([rank[e] if e // per in kept else -np.inf for e in range(E)])
    return sorted(range(E), key=lambda e: (-rank[e], e))[:top]


def experts(h, m, w, pre):
    T = h.shape[0]
    s = sigmoid(h @ w[pre + "router"].T)
    out = np.zeros_like(h)
    for t in range(T):
        idx = choose_experts(s[t], w[pre + "correction"], m["router"])
        total = sum(s[t, e] for e in idx) + 1e-20
        for e in idx:
            p = f"{pre}e{e}."
            out[t] += s[t, e] / total * (w[p + "down"] @ (silu(w[p + "gate"] @ h[t]) * (w[p + "up"] @ h[t])))
    return out


def token_side(x, tokens, i, dim, w, pre, eps):
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[pre + "gate"].T) * e) @ w[pre + "proj"].T
    return y / np.sqrt((y * y).mean(-1, keepdims=True) + eps) * w[pre + "norm"]


# ------------------------------------------------------------------ the model
def forward(j, weights, tokens, stream=None):
    """Logits [T, vocab].  `stream`: a list that receives x after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps, parts = j["norm"]["eps"], j["norm"].get("groups", 1)
    tokens = np.asarray(tokens)
    x = rms_parts(w["embed"][tokens], w["embed.norm"], parts, eps)
    side = (j.get("token_side") or {}).get("dim", 0)
    taps = (j.get("canon") or {}).get("taps", 0)
    shared = {}
    for i, lc in enumerate(j["layers"]):
        p = f"l{i}."
        h = rms_parts(x, w[p + "norm1"], parts, eps)
        if taps > 1:
            h = h + causal_conv(h, w[p + "canon1"])
        if lc["type"] == "attention":
            x = x + attention_biased(h, lc["mixer"], w, p + "mix.", eps, shared)
        elif lc["type"] == "attention_2":
            x = x + attention_rotary(h, lc["mixer"], w, p + "mix.", eps, shared)
        elif lc["type"] == "mamba2":
            x = x + mamba2(h, lc["mixer"], w, p + "mix.", eps)
        else:
            raise ValueError(lc["type"])
        if lc.get("mlp"):
            x = x + experts(rms_parts(x, w[p + "norm2"], parts, eps), lc["mlp"], w, p + "mlp.")
        if side:
            x = x + token_side(x, tokens, i, side, w, p + "side.", eps)
        if stream is not None:
            stream.append(x.copy())
    return rms_parts(x, w["final.norm"], parts, eps) @ w["embed"].T * j.get("logit_scale", 1.0)


def greedy(cfg_json, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(cfg_json, w, toks)[-1])))
    return toks[len(prompt):]
