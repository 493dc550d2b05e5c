"""A plain, slow Kisepel: every mechanism as one numpy function over a whole sequence, float64 throughout.

Nothing here is shared with the package: no cache, no state carried between calls, no kernels.  A sequence goes in
whole and every position's result comes out, so that the engine's cuttings (portions, decoding, batches) can be
held against it.  Weights are a dict of numpy arrays by tensor name; the configuration is the plain dict of
config.json.

Notation: T tokens, E the model's width, H heads, G key (or group) heads, D key width, V value width, N state width.
"""
import numpy as np

F = np.float64


def rms_norm(x, w, eps, one_plus=False):
    """x / sqrt(mean(x^2) + eps) times w, or times (1 + w) for a weight stored around zero; w None: no weight."""
    x = np.asarray(x, dtype=F)
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    if w is None:
        return y
    return y * ((1.0 + w.astype(F)) if one_plus else w.astype(F))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


def lin(h, w):
    return h @ w.astype(F).T


def causal_conv(x, taps_w, bias=None):
    """y[t, c] = b[c] + sum_j w[c, j] x[t - (taps - 1) + j, c]: the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), x.astype(F)], axis=0)
    y = np.zeros((T, C), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j].astype(F)[None, :]
    if bias is not None:
        y += bias.astype(F)[None, :]
    return y


# ---- lightning ---------------------------------------------------------------------------------------------------
def decayed_linear_attention(q, k, v, decay):
    """Per head: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, D]; v [T, H, V]; decay [H]."""
    T, H, D = q.shape
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        S = np.zeros((D, v.shape[2]), dtype=F)
        for t in range(T):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def lightning_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(lin(h, w[pre + "q"])).reshape(T, H, D)
    k = silu(lin(h, w[pre + "k"])).reshape(T, H, D)
    v = silu(lin(h, w[pre + "v"])).reshape(T, H, V)
    o = decayed_linear_attention(q, k, v, np.asarray(m["decay"], dtype=F)).reshape(T, H * V)
    o = rms_norm(o, w[pre + "norm"], eps) * sigmoid(lin(h, w[pre + "g"]))
    return lin(o, w[pre + "o"])


# ---- state-space duality -----------------------------------------------------------------------------------------
def selective_scan(x, B, C, dt, a_log, skip):
    """Per head h of group g: S_t = exp(-exp(a_log_h) dt) S_{t-1} + dt B_t x_t^T (S is N x V); y_t = S_t^T C_t + skip_h x_t.
    x [T, H, V]; B, C [T, G, N]; dt [T, H] (already positive)."""
    T, H, V = x.shape
    G, N = B.shape[1], B.shape[2]
    y = np.zeros((T, H, V), dtype=F)
    for h in range(H):
        g = h // (H // G)
        S = np.zeros((N, V), dtype=F)
        for t in range(T):
            S = np.exp(-np.exp(a_log[h]) * dt[t, h]) * S + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + skip[h] * x[t, h]
    return y


def mamba2_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    p = lin(h, w[pre + "in"])
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"].astype(F)[None, :])
    y = selective_scan(x, B, C, dt, w[pre + "A_log"].astype(F), w[pre + "D"].astype(F)).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * w[pre + "norm"].astype(F)[None, :]
    return lin(y, w[pre + "o"])


# ---- softmax attention inside chunks ------------------------------------------------------------------------------
def rotate_half(x, positions, base, dims, factor=1.0):
    """The first `dims` entries of the last axis: entry i pairs with entry i + dims/2; the pair (u, v) at position p
    becomes (u cos a - v sin a, v cos a + u sin a), a = p base^(-2i/dims) / factor.  x [T, heads, D]."""
    out = np.asarray(x, dtype=F).copy()
    half = dims // 2
    if half == 0:
        return out
    i = np.arange(half, dtype=F)
    angle = np.asarray(positions, dtype=F)[:, None] * (np.power(F(base), -2.0 * i / dims) / factor)[None, :]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    u, v = out[..., :half].copy(), out[..., half:dims].copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def chunked_softmax_attention(q, k, v, scale, chunk):
    """q [T, H, D]; k [T, G, D]; v [T, G, V]; position i sees j <= i with floor(i / chunk) = floor(j / chunk)
    (chunk None: every j <= i); query head h reads key/value head floor(h / (H / G))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for i in range(T):
        lo = 0 if chunk is None else (i // chunk) * chunk
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ v[lo:i + 1, g]
    return out


def attention_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(lin(h, w[pre + "q"]).reshape(T, H, D), w[pre + "q.norm"], eps)
    k = rms_norm(lin(h, w[pre + "k"]).reshape(T, G, D), w[pre + "k.norm"], eps)
    v = lin(h, w[pre + "v"]).reshape(T, G, V)
    rot = m.get("rot") or {}
    dims = rot.get("dims", 0)
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    pos = np.arange(T)
    if dims:
        q = rotate_half(q, pos, rot["base"], dims, factor)
        k = rotate_half(k, pos, rot["base"], dims, factor)
    chunk = (m.get("mask") or {}).get("size")
    o = chunked_softmax_attention(q, k, v, m["scale"], chunk).reshape(T, H * V)
    return lin(o, w[pre + "o"])


# ---- the gated delta rule with a decay per key channel --------------------------------------------------------------
def channel_gated_delta_rule(q, k, v, beta, g):
    """Per head: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k [T, H, D]; v [T, H, V];
    beta [T, H]; g [T, H, D] (one decay per key channel, on the rows of S)."""
    T, H, D = q.shape
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        S = np.zeros((D, v.shape[2]), dtype=F)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            out[t, h] = S.T @ q[t, h]
    return out


def delta_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(lin(h, w[pre + "q"]), w[pre + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(lin(h, w[pre + "k"]), w[pre + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(lin(h, w[pre + "v"]), w[pre + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    group = np.arange(H) // (H // G)
    q, k = q[:, group], k[:, group]
    beta = sigmoid(lin(h, w[pre + "b"]))
    a = lin(lin(h, w[pre + "a1"]), w[pre + "a2"]) + w[pre + "dt_bias"].astype(F)[None, :]
    g = np.exp(-np.exp(w[pre + "A_log"].astype(F))[None, :, None] * softplus(a).reshape(T, H, D))
    o = channel_gated_delta_rule(q, k, v, beta, g)
    o = rms_norm(o, w[pre + "norm"], eps).reshape(T, H * V)
    o = o * sigmoid(lin(lin(h, w[pre + "g1"]), w[pre + "g2"]))
    return lin(o, w[pre + "o"])


def parallel_mixer(h, w, pre, m, eps):
    """Half the sum of the two sides, each normed over the model's width with a plain weight of its own."""
    left = attention_mixer(h, w, pre + "left.", m["left"], eps)
    right = delta_mixer(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[pre + "left.out"], eps) + rms_norm(right, w[pre + "right.out"], eps))


MIXERS = {"lightning": lightning_mixer, "mamba2": mamba2_mixer, "parallel": parallel_mixer}


# ---- feed-forward -------------------------------------------------------------------------------------------------
def gated_unit(h, w, pre):
    return lin(silu(lin(h, w[pre + "gate"])) * lin(h, w[pre + "up"]), w[pre + "down"])


def table_routed_experts(h, ids, w, pre, mlp):
    """Each token's experts are the row of the table its id names, each weighing 1 / top; a shared expert (when the
    configuration has one) is added for every token."""
    top = mlp["router"]["top"]
    table = w[pre + "table"]
    out = np.zeros((h.shape[0], w[pre + "e0.down"].shape[0]), dtype=F)
    for t, tok in enumerate(ids):
        for e in table[tok][:top]:
            out[t] += gated_unit(h[t:t + 1], w, f"{pre}e{int(e)}.")[0] / top
    if mlp.get("shared") is not None:
        out += gated_unit(h, w, pre + "shared.")
    return out


# ---- the model ----------------------------------------------------------------------------------------------------
def layer_runs(config):
    """The layers in the order they run: layers start .. stop-1 `times` times in a row, the rest once.  Each item is
    (layer index, whether the embedding output is added before it)."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(start)]
    for p in range(times if stop > start else 0):
        runs += [(i, p > 0 and i == start) for i in range(start, stop)]
    runs += [(i, False) for i in range(max(stop, start), n)]
    return runs


def forward(config, w, ids, layers_out=None):
    """Logits [T, vocab] of a whole sequence.  `layers_out`: a list that receives the residual stream after every layer run."""
    eps = config["norm"]["eps"]
    ids = np.asarray(ids)
    x0 = w["embed"].astype(F)[ids] * (config.get("embedding") or {}).get("scale", 1.0)
    x = x0.copy()
    for i, inject in layer_runs(config):
        layer = config["layers"][i]
        pre = f"l{i}."
        if inject:
            x = x + x0
        h = rms_norm(x, w[pre + "norm1"], eps, one_plus=True)
        y = MIXERS[layer["type"]](h, w, pre + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + table_routed_experts(h, ids, w, pre + "mlp.", mlp)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    h = rms_norm(x, w["final.norm"], eps, one_plus=True)
    return lin(h, w["embed"]) * config.get("logit_scale", 1.0)
