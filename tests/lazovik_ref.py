"""Plain float64 restatement of the Lazovik design, one function per mechanism, for the tests.
Nothing here is shared with the product path: numpy only, whole sequences at once, no cache.

Notation: x [T, W] the residual stream of one sequence, tokens at positions 0 .. T-1; a linear
map with weight M [out, in] is x @ M.T; w maps tensor names to arrays."""
import numpy as np


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


# ------------------------------------------------------------------ attention side
def short_conv(u, taps_w):
    """Causal convolution over time per channel, no activation: taps_w [C, taps], its last
    column multiplies the current token; inputs before position 0 are zero."""
    T = u.shape[0]
    taps = taps_w.shape[1]
    out = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += taps_w[:, j] * u[src]
    return out


def rotation_tables(rot, T):
    """cos / sin [T, dims / 2].  f_i = base^(-2i / dims); with "scaling" the entries between two
    wavelengths are interpolated towards f_i / factor and both tables get the factor 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        def entry(turns):
            return dims * np.log(sc["original"] / (2.0 * np.pi * turns)) / (2.0 * np.log(base))
        lo = max(np.floor(entry(sc["fast"])), 0.0)
        hi = min(np.ceil(entry(sc["slow"])), dims - 1.0)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mult = 0.1 * np.log(sc["factor"]) + 1.0
    ang = np.arange(T, dtype=np.float64)[:, None] * f[None, :]
    return np.cos(ang) * mult, np.sin(ang) * mult


def rotate(x, cos, sin, dims):
    """x [T, heads, d]: entry i < dims / 2 pairs with entry i + dims / 2; the rest passes."""
    half = dims // 2
    a, b = x[..., :half], x[..., half:dims]
    c, s = cos[:, None, :], sin[:, None, :]
    out = x.copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def chunk_mask(T, size):
    """[T, T] bool: i sees j <= i inside its own block of `size` positions counted from 0."""
    p = np.arange(T)
    return (p[None, :] <= p[:, None]) & (p[None, :] // size == p[:, None] // size)


def capped_softmax_attention(q, k, v, scale, cap, vis):
    """One head.  q, k [T, d], v [T, vd]; scores scaled, squashed by cap * tanh(. / cap), masked."""
    s = q @ k.T * scale
    if cap:
        s = cap * np.tanh(s / cap)
    s = np.where(vis, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)) @ v


def conv_attention(h, w, p, m, eps):
    """The attention side: biased projections, convolution, whole-row norms, rotation, capped and
    chunk-masked softmax, sigmoid output gate, biased output projection."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"])
    k = short_conv(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"])
    v = short_conv(h @ w[p + "v"].T + w[p + "v.b"], w[p + "v.conv"])
    q = (rms_div(q, eps) * w[p + "q.norm"]).reshape(T, H, d)
    k = (rms_div(k, eps) * w[p + "k.norm"]).reshape(T, G, d)
    v = v.reshape(T, G, vd)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        cos, sin = rotation_tables(rot, T)
        q, k = rotate(q, cos, sin, rot["dims"]), rotate(k, cos, sin, rot["dims"])
    vis = chunk_mask(T, m["mask"]["size"])
    o = np.stack([capped_softmax_attention(q[:, i], k[:, i // (H // G)], v[:, i // (H // G)], m["scale"],
                                           m.get("softcap"), vis) for i in range(H)], axis=1)
    o = o.reshape(T, H * vd) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------ recurrences
def decayed_outer_product_scan(q, k, v, decay, bonus=None):
    """One head, state S [d, vd] from zero.  Without bonus: S <- diag(decay_t) S + k_t v_t^T, then
    o_t = S^T q_t.  With bonus u [d]: o_t = (S + diag(u) k_t v_t^T)^T q_t first, then the update."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]))
    o = np.zeros_like(v)
    for t in range(T):
        kv = np.outer(k[t], v[t])
        if bonus is None:
            S = decay[t][:, None] * S + kv
            o[t] = S.T @ q[t]
        else:
            o[t] = (S + bonus[:, None] * kv).T @ q[t]
            S = decay[t][:, None] * S + kv
    return o


def gated_linear_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d) / np.sqrt(d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, vd)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    decay = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, d)
    o = np.stack([decayed_outer_product_scan(q[:, i], k[:, i], v[:, i], decay[:, i]) for i in range(H)], axis=1)
    o = rms_div(o, eps) * w[p + "norm"]  # per head over vd, one weight for all heads
    return (o.reshape(T, H * vd) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu, h_{-1} = 0."""
    prev = np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)
    return h + (prev - h) * mu


def time_mixing(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (token_shift(h, w[p + "mu.r"]) @ w[p + "r"].T).reshape(T, H, d)
    k = (token_shift(h, w[p + "mu.k"]) @ w[p + "k"].T).reshape(T, H, d)
    v = (token_shift(h, w[p + "mu.v"]) @ w[p + "v"].T).reshape(T, H, d)
    gate = silu(token_shift(h, w[p + "mu.g"]) @ w[p + "g"].T)
    z = np.tanh(token_shift(h, w[p + "mu.w"]) @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    decay = np.exp(-np.exp(z)).reshape(T, H, d)
    o = np.stack([decayed_outer_product_scan(r[:, i], k[:, i], v[:, i], decay[:, i], w[p + "u"][i]) for i in range(H)], axis=1)
    o = rms_div(o, eps).reshape(T, H * d) * w[p + "norm"]
    return (o * gate) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward
def squared_relu_expert(x, up, down):
    return (np.maximum(x @ up.T, 0.0) ** 2) @ down.T


def expert_mixture(h, w, p, m):
    """Scores sigmoid(router h); the `top` best experts (ties to the lower index) each run on
    score * h; an always-on expert is added times sigmoid(sg . h)."""
    top = m["router"]["top"]
    s = sigmoid(h @ w[p + "router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-s[t], kind="stable")[:top]:
            out[t] += squared_relu_expert(s[t, e] * h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if m.get("shared"):
        out += squared_relu_expert(h, w[p + "shared.up"], w[p + "shared.down"]) * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------ the model
def execution_order(cfg_json):
    """(layer, pass it opens or None): a repeated run of layers counts once per pass."""
    n = len(cfg_json["layers"])
    lp = cfg_json.get("loop")
    if not lp or lp["times"] < 1 or lp["stop"] <= lp["start"]:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        order += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return order + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg_json, w, tokens):
    """Logits [T, vocab] of one sequence."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = cfg_json["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for i, opens in execution_order(cfg_json):
        lc = cfg_json["layers"][i]
        p = f"l{i}."
        if opens is not None:
            x = x + w["loop.step"][opens]
        h = rms_div(x, eps) * w[p + "norm1"]
        if lc["type"] == "gla":
            x = x + gated_linear_attention(h, w, p + "mix.", lc["mixer"], eps)
        else:
            m = lc["mixer"]
            x = x + m["left_scale"] * conv_attention(h, w, p + "mix.left.", m["left"], eps) \
                  + m["right_scale"] * time_mixing(h, w, p + "mix.right.", m["right"], eps)
        if lc.get("mlp"):
            h = rms_div(x, eps) * w[p + "norm2"]
            x = x + expert_mixture(h, w, p + "mlp.", lc["mlp"])
    return (rms_div(x, eps) * w["final.norm"]) @ w["head"].T


def greedy(cfg_json, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(cfg_json, w, toks)[-1])))
    return toks[len(prompt):]
