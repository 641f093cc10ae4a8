"""A plain, slow float64 implementation of the Botalorn design: one function per mechanism, one request at a time,
written from the design's equations and sharing nothing with the engine.

Notation: T tokens, W the width, n streams; N(y) = y / sqrt(mean(y^2) + eps) over the last axis.
"""
import numpy as np

SLOPE_EXPONENT = 8.0
SINUSOID_BASE = 10000.0
UNIT_EPS = 1e-6


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(y, eps):
    return y / np.sqrt((y * y).mean(-1, keepdims=True) + eps)


def sinusoid(positions, width, base=SINUSOID_BASE):
    """[T, width]: column 2i = sin(p * base^(-2i/width)), column 2i+1 = cos of the same angle."""
    p = np.asarray(positions, dtype=np.float64)[:, None]
    out = np.zeros((len(positions), width))
    for c in range(width):
        ang = p[:, 0] * base ** (-(c - c % 2) / width)
        out[:, c] = np.sin(ang) if c % 2 == 0 else np.cos(ang)
    return out


def embed(table, tokens, scale, first_position=0):
    T = len(tokens)
    return table[np.asarray(tokens)] * scale + sinusoid(range(first_position, first_position + T), table.shape[1])


def causal_conv(u, w, before=None):
    """u [T, C], w [C, taps] (last column: the current token).  ``before`` [taps-1, C]: the rows ahead of u (zeros)."""
    T, C = u.shape
    taps = w.shape[1]
    head = np.zeros((taps - 1, C)) if before is None else np.asarray(before, dtype=np.float64)
    ext = np.concatenate([head, u], 0)
    y = np.zeros((T, C))
    for t in range(T):
        for j in range(taps):
            y[t] += w[:, j] * ext[t + j]
    return y


def token_shift(h, shift, before=None):
    """h [T, W] -> h + (h_prev - h) * shift; h_prev the row above as it was (``before`` or zeros for the first)."""
    first = np.zeros((1, h.shape[1])) if before is None else np.asarray(before, dtype=np.float64)[None]
    prev = np.concatenate([first, h[:-1]], 0)
    return h + (prev - h) * shift


def stream_read(xs, w_in):
    """xs [n, T, W] -> sum_s in[s] xs[s]."""
    return np.einsum("s,stw->tw", w_in, xs)


def stream_write(xs, y, w_mix, w_out):
    """All copies at once from the old ones: new[t] = sum_s mix[s, t] old[s] + out[t] y."""
    return np.einsum("sr,stw->rtw", w_mix, xs) + w_out[:, None, None] * y[None]


def slopes(heads, exponent=SLOPE_EXPONENT):
    return np.array([2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)])


def biased_window_attention(q, k, v, positions_q, positions_k, scale, temp, window, slope):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, V] -> [Tq, H, V].  Query at position i sees key at position j when
    0 <= i - j < window (window 0: every j <= i); score = q.k * scale * temp[h] - slope[h] * (i - j); softmax."""
    Tq, H, D = q.shape
    G = k.shape[1]
    out = np.zeros((Tq, H, v.shape[2]))
    pk = np.asarray(positions_k)
    for t in range(Tq):
        i = positions_q[t]
        seen = np.where((pk <= i) & ((i - pk < window) if window else True))[0]
        for h in range(H):
            g = h // (H // G)
            s = (k[seen, g] @ q[t, h]) * scale * temp[h] - slope[h] * (i - pk[seen])
            e = np.exp(s - s.max())
            out[t, h] = (e / e.sum()) @ v[seen, g]
    return out


def attention_keys_values(m, Wt, p, h, eps):
    """What an attention layer with projections of its own caches: keys after convolution and the norm over the whole
    row; values after convolution, each head divided by its root mean square."""
    T = h.shape[0]
    G, V = m["kv_heads"], m.get("vdim") or m["dim"]
    k = rms(causal_conv(h @ Wt[p + "k"].T, Wt[p + "k.conv"]), eps) * Wt[p + "k.norm"]
    v = causal_conv(h @ Wt[p + "v"].T, Wt[p + "v.conv"])
    v = rms(v.reshape(T, G, V), eps).reshape(T, G * V)
    return k, v


def attention_mixer(m, Wt, p, h, eps, kv):
    """h [T, W] (whole request from position 0); kv = (k [T, G*D], v [T, G*V]) as cached by this layer or another."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    V = m.get("vdim") or D
    q = rms(causal_conv(h @ Wt[p + "q"].T, Wt[p + "q.conv"]), eps) * Wt[p + "q.norm"]
    k, v = kv
    window = int((m.get("mask") or {}).get("size") or 0)
    pos = list(range(T))
    o = biased_window_attention(q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, V), pos, pos, m["scale"], Wt[p + "temp"], window,
                                slopes(H))
    o = o * sigmoid(h @ Wt[p + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ Wt[p + "o"].T


def delta_inputs(m, Wt, p, h):
    """q, k [T, G, D] unit vectors (q times D^-1/2), v [T, H, V], beta and decay [T, H]."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    V = m.get("vdim") or D
    q = silu(causal_conv(h @ Wt[p + "q"].T, Wt[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ Wt[p + "k"].T, Wt[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ Wt[p + "v"].T, Wt[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + UNIT_EPS) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(h @ Wt[p + "b"].T)
    decay = np.exp(-np.exp(Wt[p + "A_log"])[None] * softplus(h @ Wt[p + "a"].T + Wt[p + "dt_bias"][None]))
    return q, k, v, beta, decay


def delta_recurrence(q, k, v, beta, decay, S=None):
    """Per value head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns (o [T, H, V], S [H, D, V])."""
    T, H, V = v.shape
    G, D = q.shape[1], q.shape[2]
    S = np.zeros((H, D, V)) if S is None else np.array(S, dtype=np.float64)
    o = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, g])
            S[h] = S[h] + np.outer(k[t, g], u)
            o[t, h] = S[h].T @ q[t, g]
    return o, S


def delta_mixer(m, Wt, p, h, eps):
    T = h.shape[0]
    q, k, v, beta, decay = delta_inputs(m, Wt, p, h)
    o, _ = delta_recurrence(q, k, v, beta, decay)
    o = rms(o, eps) * Wt[p + "norm"][None, None]
    return (o.reshape(T, -1) * silu(h @ Wt[p + "g"].T)) @ Wt[p + "o"].T


def feed_forward(Wt, p, h):
    return (np.maximum(h @ Wt[p + "up"].T, 0.0) ** 2) @ Wt[p + "down"].T


def forward(cfg, Wt, tokens, layers_out=None):
    """Logits [T, vocab] of one request from its first token; ``layers_out`` collects the sum of the streams after
    every layer."""
    eps, n = cfg["norm"]["eps"], cfg.get("streams")
    x = embed(Wt["embed"], tokens, (cfg.get("embedding") or {}).get("scale", 1.0))
    xs = np.stack([x] * (n or 1), 0)
    one = np.ones(1)
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        for q, sub in ((1, "mix"), (2, "mlp")):
            if sub == "mlp" and not layer.get("mlp"):
                continue
            w_in, w_out, w_mix = (Wt[L + f"hc{q}.in"], Wt[L + f"hc{q}.out"], Wt[L + f"hc{q}.mix"]) if n else (one, one, one[:, None])
            h = rms(stream_read(xs, w_in), eps) * Wt[L + f"norm{q}"]
            if sub == "mix":
                h = token_shift(h, Wt[L + "shift"])
                m = layer["mixer"]
                if layer["type"] == "attention":
                    src = m.get("kv_from")
                    if src is None:
                        cached[i] = attention_keys_values(m, Wt, L + "mix.", h, eps)
                        src = i
                    y = attention_mixer(m, Wt, L + "mix.", h, eps, cached[src])
                else:
                    y = delta_mixer(m, Wt, L + "mix.", h, eps)
            else:
                y = feed_forward(Wt, L + "mlp.", h)
            xs = stream_write(xs, y, w_mix, w_out)
        if layers_out is not None:
            layers_out.append(xs.sum(0))
    return (rms(xs.sum(0), eps) * Wt["final.norm"]) @ Wt["head"].T
