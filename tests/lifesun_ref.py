"""Plain, slow statement of the Lifesun decoder family in float64 numpy: one function per mechanism, whole sequences only, recurrences
walked token by token.  It shares no code with the package; the tests compare the package's kernels and runner with it.

The stack.  x = embed[token]; x0 keeps that row.  A layer run is x += mixer(h) + ff(h) with ONE norm h = LN(x) (mean and variance, weight
and bias) feeding both sublayers.  `loop` repeats layers start .. stop-1 `times` times with the same weights; right before the first layer
of every repetition x = W_in [x ; x0].  Two mixers, each a softmax attention (left) beside a recurrence (right), joined as
left_scale * left + right_scale * right:
  parallel    left: no positions, queries and keys scaled to unit RMS per head, a mask of blocks of positions counted from 0, one extra
              term 1 in the softmax denominator, a sigmoid gate per head on the result.
              right: a gated diagonal recurrence (RG-LRU) behind a short convolution, times a gelu branch.
  parallel_2  left: RMS norm with weights over the whole query / key projection, rotation of (i, i + dims/2) pairs, tanh cap on the
              scores, sliding window.
              right: retention -- rotated q and k, S = decay_h S + k v^T, read-out S^T q, unit RMS per head, silu gate.
Feed-forward: W_down (gelu_tanh(W_gate h) * (W_up h)).  Output: LN, head, times logit_scale.
"""
import numpy as np


# ---- small functions -----------------------------------------------------------------------------------------------------------
def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / np.sqrt(np.mean(x * x, -1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rotate_half(x, pos, dims, base):
    """x: [T, heads, dim]; in every head column i < dims/2 turns together with column i + dims/2 by pos * base^(-2i/dims)"""
    half = dims // 2
    f = float(base) ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(pos, np.float64)[:, None, None] * f[None, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * np.cos(a) - v * np.sin(a)
    out[..., half:dims] = v * np.cos(a) + u * np.sin(a)
    return out


# ---- masks ---------------------------------------------------------------------------------------------------------------------
def block_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def window_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i - j < size)


# ---- softmax attention ---------------------------------------------------------------------------------------------------------
def attention(q, k, v, scale, mask, softcap=0.0, one_in_denominator=False):
    """q: [T, H, dk], k: [T, G, dk], v: [T, G, dv]; query head h reads key/value head h // (H / G).  -> [T, H, dv]"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        if softcap > 0:
            s = softcap * np.tanh(s / softcap)
        s = np.where(mask, s, -np.inf)
        m = s.max(1, keepdims=True)
        if one_in_denominator:
            m = np.maximum(m, 0.0)
        e = np.exp(s - m)
        den = e.sum(1, keepdims=True) + (np.exp(-m) if one_in_denominator else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out


def left_blocks(h, W, p, c, eps):
    """attention of the `parallel` mixer.  W: name -> array, p: prefix of the left mixer's tensors, c: its config"""
    T = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit_rms((h @ W[p + "q"].T).reshape(T, H, dk), eps)
    k = unit_rms((h @ W[p + "k"].T).reshape(T, G, dk), eps)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    o = attention(q, k, v, c["scale"], block_mask(T, c["mask"]["size"]), one_in_denominator=True)
    o = o * sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def left_window(h, W, p, c, eps):
    """attention of the `parallel_2` mixer"""
    T = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    pos = np.arange(T)
    q = (unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]).reshape(T, H, dk)
    k = (unit_rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]).reshape(T, G, dk)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    rot = c.get("rot")
    if rot and rot.get("dims", 0) > 0:
        q, k = rotate_half(q, pos, rot["dims"], rot["base"]), rotate_half(k, pos, rot["dims"], rot["base"])
    o = attention(q, k, v, c["scale"], window_mask(T, c["mask"]["size"]), softcap=c.get("softcap", 0.0) or 0.0)
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ---- recurrences ---------------------------------------------------------------------------------------------------------------
def causal_conv(x, w, b):
    """x: [T, C], w: [C, K] (last column: the current token), zeros before the start"""
    T, C = x.shape
    K = w.shape[1]
    xp = np.concatenate([np.zeros((K - 1, C)), x], 0)
    y = np.zeros((T, C))
    for j in range(K):
        y += xp[j:j + T] * w[:, j]
    return y + b


def gated_diagonal_recurrence(u, r, i, lam, c=8.0):
    """S_t = a_t S_{t-1} + sqrt(1 - a_t^2) i_t u_t, a_t = exp(-c r_t softplus(lam)), S_{-1} = 0.  all [T, C] but lam [C]"""
    S = np.zeros(u.shape[1])
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        a = np.exp(-c * r[t] * softplus(lam))
        S = a * S + np.sqrt(1.0 - a * a) * (i[t] * u[t])
        out[t] = S
    return out


def right_rglru(h, W, p, c):
    T = h.shape[0]
    C, B = c["width"], c["blocks"]
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = causal_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    ub = u.reshape(T, B, C // B)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, W[p + "ra"]) + W[p + "ra.b"]).reshape(T, C)
    i = sigmoid(np.einsum("tbi,boi->tbo", ub, W[p + "ri"]) + W[p + "ri.b"]).reshape(T, C)
    S = gated_diagonal_recurrence(u, r, i, W[p + "lam"])
    return (S * y) @ W[p + "o"].T


def retention(q, k, v, decay):
    """q, k: [T, H, dk], v: [T, H, dv], decay: [H].  S_t = decay S_{t-1} + k_t v_t^T ; o_t = S_t^T q_t"""
    T, H, dk = q.shape
    S = np.zeros((H, dk, v.shape[2]))
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        S = np.asarray(decay)[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hkv,hk->hv", S, q[t])
    return out


def right_retention(h, W, p, c, eps):
    T = h.shape[0]
    H, dk, dv = c["heads"], c["dim"], c["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dk)
    k = (h @ W[p + "k"].T).reshape(T, H, dk)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    rot = c.get("rot")
    if rot and rot.get("dims", 0) > 0:
        pos = np.arange(T)
        q, k = rotate_half(q, pos, rot["dims"], rot["base"]), rotate_half(k, pos, rot["dims"], rot["base"])
    o = unit_rms(retention(q, k * dk ** -0.5, v, c["decay"]), eps).reshape(T, H * dv)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


# ---- layers and the model ------------------------------------------------------------------------------------------------------
def feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def mixer(kind, h, W, p, m, eps):
    if kind == "parallel":
        left, right = left_blocks(h, W, p + "left.", m["left"], eps), right_rglru(h, W, p + "right.", m["right"])
    elif kind == "parallel_2":
        left, right = left_window(h, W, p + "left.", m["left"], eps), right_retention(h, W, p + "right.", m["right"], eps)
    else:
        raise ValueError(kind)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


def layer_run(x, W, i, L, eps):
    p = f"l{i}."
    h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
    y = mixer(L["type"], h, W, p + "mix.", L["mixer"], eps)
    if L.get("mlp"):
        y = y + feed_forward(h, W, p + "mlp.")
    return x + y


def run_order(conf):
    """-> [(layer index, whether x = W_in [x ; x0] comes right before it)]"""
    n, lp = len(conf["layers"]), conf.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(conf, W, tokens, taps=None):
    """-> logits [T, vocab]; taps (a list) receives the residual stream after every layer run"""
    W = {k: np.asarray(v, np.float64) for k, v in W.items()}
    eps = conf["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    x0 = x
    for i, re_enter in run_order(conf):
        if re_enter:
            x = np.concatenate([x, x0], 1) @ W["loop.in"].T
        x = layer_run(x, W, i, conf["layers"][i], eps)
        if taps is not None:
            taps.append(x.copy())
    return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T * conf.get("logit_scale", 1.0)
