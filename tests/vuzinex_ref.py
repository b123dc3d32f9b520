"""A plain, slow restatement of the Vuzinex decoder in numpy float64: one function per mechanism, token by token where a mechanism is a
recurrence, whole score matrices where it is attention.  It shares no code with the package; the tests compare the package against it.

Notation: h [T, D] a sublayer's input, rows are the positions 0 .. T-1 of ONE sequence; W matrices are [out, in] and applied as h W^T."""
import math

import numpy as np


# ---- small pieces -----------------------------------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def log_sigmoid(z):
    return -softplus(-z)


def unit_rms(x, eps):
    """every row of the last axis divided by its root mean square (eps inside the root)"""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    """the layer norms: the stored weight is an offset from one"""
    return unit_rms(x, eps) * (1.0 + w)


# ---- embedding --------------------------------------------------------------------------------------------------------------------------
def embed(conf, w, tokens):
    e = conf["embedding"]
    x = w["embed"][tokens] * e["scale"]
    b = e.get("bigram")
    if b:
        rows = [b["buckets"] if t == 0 else (tokens[t - 1] * b["mul_prev"] + tokens[t] * b["mul_cur"]) % b["buckets"] for t in range(len(tokens))]
        x = x + w["bigram"][rows]
    return x


# ---- rotary positions ---------------------------------------------------------------------------------------------------------------------
def rot_frequencies(rot):
    """-> (frequency of every pair [dims / 2], factor on cos and sin)"""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    if "low" in sc:                                  # wavelength bands: short waves stay, long waves slow down, a blend between
        wave = 2.0 * math.pi / f
        short, long_ = sc["original"] / sc["high"], sc["original"] / sc["low"]
        s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
        mid = (1.0 - s) * f / sc["factor"] + s * f
        return np.where(wave < short, f, np.where(wave > long_, f / sc["factor"], mid)), 1.0

    def pair_at(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_at(sc["fast"])), 0)
    hi = min(math.ceil(pair_at(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, rot, pos0=0):
    """x [T, heads, dim]: neighbouring coordinates (2i, 2i+1) of the first rot.dims turn by position * frequency_i"""
    if not rot or rot["dims"] <= 0:
        return x
    f, mag = rot_frequencies(rot)
    T, n = x.shape[0], rot["dims"]
    a = (pos0 + np.arange(T, dtype=np.float64))[:, None] * f[None, :]
    c, s = (np.cos(a) * mag)[:, None, :], (np.sin(a) * mag)[:, None, :]
    out = x.copy()
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# ---- softmax attention ----------------------------------------------------------------------------------------------------------------------
def visible(T, block, window=0):
    """[T, T] booleans: j <= i; with block > 0 only inside i's block of `block` positions counted from position 0; with window > 0 only
    the last `window` positions, i itself included"""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    ok = j <= i
    if block and block > 0:
        ok &= (i // block) == (j // block)
    if window and window > 0:
        ok &= (i - j) < window
    return ok


def attention(h, m, w, p, eps):
    """the softmax mixer; m: its sizes, p: tensor-name prefix.  Biases, query/key norms, the sink and the output gate are used where the
    model has their tensors."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def proj(name):
        y = h @ w[p + name].T
        return y + w[p + name + ".b"] if p + name + ".b" in w else y
    q, k, v = proj("q").reshape(T, H, dk), proj("k").reshape(T, G, dk), proj("v").reshape(T, G, dv)
    if p + "q.norm" in w:
        q = unit_rms(q, eps) * w[p + "q.norm"]
        k = unit_rms(k, eps) * w[p + "k.norm"]
    q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
    ok = visible(T, (m.get("mask") or {}).get("size", 0), (m.get("mask") or {}).get("window", 0))
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = np.where(ok, s, -np.inf)
        top = s.max(-1, keepdims=True)
        if p + "sink" in w:
            top = np.maximum(top, w[p + "sink"][hd])
        e = np.exp(s - top)
        den = e.sum(-1, keepdims=True)
        if p + "sink" in w:
            den = den + np.exp(w[p + "sink"][hd] - top)
        out[:, hd] = (e / den) @ v[:, g]
    out = out.reshape(T, H * dv)
    if p + "g" in w:
        out = out * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---- matrix memory with exponential gates -------------------------------------------------------------------------------------------------
def matrix_memory(h, m, w, p, eps):
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S, n, top = np.zeros((dk, dv)), np.zeros(dk), 0.0
        for t in range(T):
            new_top = max(gf[t, hd] + top, gi[t, hd])
            keep, take = math.exp(gf[t, hd] + top - new_top), math.exp(gi[t, hd] - new_top)
            S = keep * S + take * np.outer(k[t, hd], v[t, hd])
            n = keep * n + take * k[t, hd]
            top = new_top
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(n @ q[t, hd]), math.exp(-top)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---- linear attention with a decay per key channel ------------------------------------------------------------------------------------------
def decayed_linear_attention(h, m, w, p, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    decay = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, dk)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[t, hd][:, None] * S + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = (unit_rms(out, eps) * w[p + "norm"]).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---- the two-branch mixers --------------------------------------------------------------------------------------------------------------------
def side_by_side(h, m, w, p, eps):
    right = matrix_memory if "gate_cap" in m["right"] else decayed_linear_attention
    return m["left_scale"] * attention(h, m["left"], w, p + "left.", eps) + m["right_scale"] * right(h, m["right"], w, p + "right.", eps)


# ---- state-space mixer ------------------------------------------------------------------------------------------------------------------------
def state_space(h, m, w, p, eps):
    T = h.shape[0]
    H, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    padded = np.concatenate([np.zeros((K - 1, xbc.shape[1])), xbc], 0)
    conv = sum(padded[j:j + T] * w[p + "conv"][:, j] for j in range(K)) + w[p + "conv.b"]
    xbc = silu(conv)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = np.zeros((T, H, P))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((N, P))
        rate = math.exp(w[p + "A_log"][hd])
        for t in range(T):
            S = math.exp(-rate * dt[t, hd]) * S + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ---- feed-forward -----------------------------------------------------------------------------------------------------------------------------
def feed_forward(h, w, p):
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


# ---- the stack ----------------------------------------------------------------------------------------------------------------------------------
MIXERS = {"parallel": side_by_side, "parallel_2": side_by_side, "mamba2": state_space}


def layer_runs(conf):
    """the order in which the layers run: the looped block repeats"""
    n = len(conf["layers"])
    lp = conf.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = lp["start"], lp["stop"], lp["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(conf, weights, tokens, residuals=None):
    """logits [T, vocab] of one sequence fed at once; residuals (a list) receives the stream after every layer run"""
    w = {k: np.asarray(v, np.float64) for k, v in weights.items()}
    eps, mult = conf["norm"]["eps"], conf.get("residual_mult", 1.0)
    x = embed(conf, w, list(tokens))
    for li in layer_runs(conf):
        L, p = conf["layers"][li], f"l{li}."
        y = MIXERS[L["type"]](norm_around_zero(x, w[p + "norm1"], eps), L["mixer"], w, p + "mix.", eps)
        x = x + mult * norm_around_zero(y, w[p + "norm1b"], eps)
        if L.get("mlp"):
            y = feed_forward(norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + mult * norm_around_zero(y, w[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.copy())
    return (norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T) * conf.get("logit_scale", 1.0)
