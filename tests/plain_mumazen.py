"""A plain, slow float64 implementation of the Mumazen design: one function per mechanism, one request at a time,
written from the design's equations and sharing nothing with the engine.

Notation: T tokens, W the width; N(y) = y / sqrt(mean(y^2) + eps) over the last axis; a weight W_foo is stored
[out, in] and applied as h @ W_foo.T.  ``Wt`` maps tensor names to float64 arrays, ``p`` is a layer's prefix.
"""
import numpy as np

QUICK_GELU = 1.702           # the dense feed-forward's gate: g * sigmoid(1.702 g)
WEIGHT_SUM_EPS = 1e-20       # added to the sum of the chosen experts' scores


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(y, eps):
    return y / np.sqrt((y * y).mean(-1, keepdims=True) + eps)


def causal_conv(u, w, bias=None, before=None):
    """u [T, C], w [C, taps] (last column: the current token's), zeros (or ``before`` [taps-1, C]) ahead of u."""
    T, C = u.shape
    taps = w.shape[1]
    head = np.zeros((taps - 1, C)) if before is None else np.asarray(before, dtype=np.float64)
    ext = np.concatenate([head, u], 0)
    y = np.zeros((T, C))
    for t in range(T):
        for j in range(taps):
            y[t] += w[:, j] * ext[t + j]
    return y if bias is None else y + bias


def rotate_halves(x, positions, dims, base, factor):
    """x [T, H, D]: dimension i < dims/2 of every head turns with dimension i + dims/2 by the angle
    p * base^(-2i/dims) / factor; dimensions from ``dims`` on pass unchanged."""
    out = x.copy()
    half = dims // 2
    p = np.asarray(positions, dtype=np.float64)
    for i in range(half):
        a = p * (base ** (-2.0 * i / dims) / factor)
        c, s = np.cos(a)[:, None], np.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def capped_causal_attention(q, k, v, pos_q, pos_k, scale, cap):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, V] -> [Tq, H, V]; score = q.k * scale, then cap * tanh(score / cap)
    (cap 0: none); the query at position i sees every key at position j <= i; ordinary softmax."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((Tq, H, v.shape[2]))
    for t in range(Tq):
        see = [j for j in range(k.shape[0]) if pos_k[j] <= pos_q[t]]
        for h in range(H):
            g = h // (H // G)
            s = np.array([q[t, h] @ k[j, g] for j in see]) * scale
            if cap:
                s = cap * np.tanh(s / cap)
            w = np.exp(s - s.max())
            w /= w.sum()
            out[t, h] = sum(w[n] * v[j, g] for n, j in enumerate(see))
    return out


def gated_attention(m, Wt, p, h, positions=None):
    """The left half of the mixer 'parallel': grouped-query attention with a partial rotation, a capped score and an
    element-wise output gate sigmoid(W_g h) on the concatenated heads before W_o."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ Wt[p + "q"].T).reshape(T, H, D)
    k = (h @ Wt[p + "k"].T).reshape(T, G, D)
    v = (h @ Wt[p + "v"].T).reshape(T, G, V)
    rot = m.get("rot")
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor") or 1.0)
        q = rotate_halves(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_halves(k, pos, rot["dims"], rot["base"], factor)
    o = capped_causal_attention(q, k, v, pos, pos, m["scale"], float(m.get("softcap") or 0.0)).reshape(T, H * V)
    o = o * sigmoid(h @ Wt[p + "g"].T)
    return o @ Wt[p + "o"].T


def ssd_recurrence(x, B, C, dt, A, D, S=None):
    """x [T, heads, V], B and C [T, groups, N], dt [T, heads] (after its softplus), A = exp(A_log) [heads], D [heads].
    Per head: S <- exp(-A dt) S + dt B x^T (S is N x V); y = S^T C + D x."""
    T, heads, V = x.shape
    groups, N = B.shape[1], B.shape[2]
    S = np.zeros((heads, N, V)) if S is None else S.copy()
    y = np.zeros((T, heads, V))
    for t in range(T):
        for h in range(heads):
            g = h // (heads // groups)
            S[h] = np.exp(-A[h] * dt[t, h]) * S[h] + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y, S


def ssd_mixer(m, Wt, p, h, eps):
    """The right half of the mixer 'parallel': W_in h = [z | x | B | C | dt]; x, B, C pass the convolution and silu;
    the recurrence; y * silu(z); an RMS norm per part of ``norm_groups`` equal parts; W_o."""
    T = h.shape[0]
    heads, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * V
    u = h @ Wt[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, Wt[p + "conv"], Wt[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + Wt[p + "dt_bias"])
    y, _ = ssd_recurrence(x, B, C, dt, np.exp(Wt[p + "A_log"]), Wt[p + "D"])
    y = y.reshape(T, inner) * silu(z)
    parts = int(m.get("norm_groups") or 1)
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * Wt[p + "norm"]
    return y @ Wt[p + "o"].T


def parallel_mixer(m, Wt, p, h, eps):
    return m["left_scale"] * gated_attention(m["left"], Wt, p + "left.", h) + m["right_scale"] * ssd_mixer(m["right"], Wt, p + "right.", h, eps)


def selective_scan(x, dt, A, B, C, D, S=None):
    """x and dt [T, inner], A [inner, N] (negative), B and C [T, N], D [inner].  Per channel c and state n:
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c."""
    T, inner = x.shape
    S = np.zeros(A.shape) if S is None else S.copy()
    y = np.zeros((T, inner))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y, S


def mamba_mixer(m, Wt, p, h):
    """The mixer 'mamba1': W_in h = [x | z]; x through the convolution and silu; W_x x = [dt | B | C];
    dt = softplus(W_dt dt + b); the scan; y * silu(z); W_o."""
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    u = h @ Wt[p + "in"].T
    x, z = u[:, :inner], u[:, inner:]
    x = silu(causal_conv(x, Wt[p + "conv"], Wt[p + "conv.b"]))
    xp = x @ Wt[p + "x"].T
    dt = softplus(xp[:, :R] @ Wt[p + "dt"].T + Wt[p + "dt.b"])
    y, _ = selective_scan(x, dt, -np.exp(Wt[p + "A_log"]), xp[:, R:R + N], xp[:, R + N:R + 2 * N], Wt[p + "D"])
    return (y * silu(z)) @ Wt[p + "o"].T


def dense_ff(f, Wt, p, h):
    """g = min(W_gate h + b, limit), u = clamp(W_up h + b, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1)) + b."""
    lim = float(f["limit"])
    g = np.minimum(h @ Wt[p + "gate"].T + Wt[p + "gate.b"], lim)
    u = np.clip(h @ Wt[p + "up"].T + Wt[p + "up.b"], -lim, lim)
    return (g * sigmoid(QUICK_GELU * g) * (u + 1.0)) @ Wt[p + "down"].T + Wt[p + "down.b"]


def route(z, correction, top):
    """z [T, E] router logits -> (ids [T, top], weights [T, top]): s = softmax(z); the ``top`` largest s + correction
    are chosen; the weights are the chosen s divided by their sum."""
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(-1, keepdims=True)
    ids = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, ids, -1)
    return ids, w / (w.sum(-1, keepdims=True) + WEIGHT_SUM_EPS)


def relu2_expert(Wt, p, h):
    return np.maximum(h @ Wt[p + "up"].T, 0.0) ** 2 @ Wt[p + "down"].T


def moe_ff(f, Wt, p, h):
    """Routed experts (the last ``identity`` ones return their input), plus the shared expert times sigmoid(W_sg h)."""
    r = f["router"]
    E, ident, top = r["experts"], int(r.get("identity") or 0), r["top"]
    ids, w = route(h @ Wt[p + "router"].T, Wt[p + "correction"], top)
    out = np.zeros((h.shape[0], Wt[p + "router"].shape[1]))
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t], w[t]):
            out[t] += wt * (h[t] if e >= E else relu2_expert(Wt, f"{p}e{e}.", h[t:t + 1])[0])
    if f.get("shared"):
        out += sigmoid(h @ Wt[p + "shared.sg"].T) * relu2_expert(Wt, p + "shared.", h)
    return out


def run_order(cfg):
    """[(layer, pass number or None, first of its pass)]: layers start..stop-1 run ``times`` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


def forward(cfg, Wt, tokens, layers_out=None):
    """Logits [T, vocab] of one request's whole token list."""
    eps, mult = cfg["norm"]["eps"], float(cfg.get("residual_mult", 1.0))
    x0 = Wt["embed"][np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    x = x0.copy()
    for i, t, first in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if first:
            if t > 0:
                x = x + x0
            x = x + Wt["loop.step"][t]
        h = rms(x, eps) * Wt[p + "norm1"]
        if layer["type"] == "parallel":
            y = parallel_mixer(layer["mixer"], Wt, p + "mix.", h, eps)
        elif layer["type"] == "mamba1":
            y = mamba_mixer(layer["mixer"], Wt, p + "mix.", h)
        else:
            raise ValueError(layer["type"])
        x = x + mult * Wt[p + "ls1"] * y
        f = layer.get("mlp")
        if f:
            h = rms(x, eps) * Wt[p + "norm2"]
            y = dense_ff(f, Wt, p + "mlp.", h) if f["kind"] == "dense" else moe_ff(f, Wt, p + "mlp.", h)
            x = x + mult * Wt[p + "ls2"] * y
        if layers_out is not None:
            layers_out.append(x.copy())
    return (rms(x, eps) * Wt["final.norm"]) @ Wt["head"].T
