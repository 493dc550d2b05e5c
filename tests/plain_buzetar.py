"""A plain, slow Buzetar: every mechanism as one numpy function over a whole sequence, float64 throughout.

Nothing here is shared with the package: no cache, no state carried between calls, no kernels.  A sequence goes in
whole and every position's result comes out, so that the engine's cuttings (portions, decoding, batches) can be
held against it.  Weights are a dict of numpy arrays by tensor name; the configuration is the plain dict of
config.json.

Notation: T tokens, E the model's width, H heads, D key width per head, V value width per head.
"""
import math

import numpy as np

F = np.float64


def layer_norm(x, w, eps):
    """Centred norm with a weight and no bias: (x - mean) / sqrt(var + eps) * w, var = mean of squared deviations."""
    x = x.astype(F)
    xc = x - x.mean(axis=-1, keepdims=True)
    return xc / np.sqrt((xc * xc).mean(axis=-1, keepdims=True) + eps) * w.astype(F)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w (eps inside the root; the weight is plain, not 1 + w)."""
    x = x.astype(F)
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if w is None else y * w.astype(F)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


def clamped_glu(h, w_gate, w_up, w_down, limit, alpha=1.702):
    """g = min(h Wg^T, limit), u = clamp(h Wu^T, -limit, limit), y = g sigmoid(alpha g) (u + 1); out = y Wd^T."""
    g = np.minimum(h @ w_gate.astype(F).T, limit)
    u = np.clip(h @ w_up.astype(F).T, -limit, limit)
    return (g * sigmoid(alpha * g) * (u + 1.0)) @ w_down.astype(F).T


def decayed_linear_attention(q, k, v, decay):
    """Per head: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, D]; v [T, H, V]; decay [H]."""
    T, H, D = q.shape
    V = v.shape[2]
    out = np.zeros((T, H, V), dtype=F)
    for h in range(H):
        S = np.zeros((D, V), dtype=F)
        for t in range(T):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def lightning_mixer(h, w, pre, m, eps):
    """silu on q, k and v; the decayed recurrence; one RMS norm over all heads' outputs; a sigmoid gate; W_o."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].astype(F).T).reshape(T, H, D)
    k = silu(h @ w[pre + "k"].astype(F).T).reshape(T, H, D)
    v = silu(h @ w[pre + "v"].astype(F).T).reshape(T, H, V)
    o = decayed_linear_attention(q, k, v, np.asarray(m["decay"], dtype=F)).reshape(T, H * V)
    o = rms_norm(o, w[pre + "norm"], eps) * sigmoid(h @ w[pre + "g"].astype(F).T)
    return o @ w[pre + "o"].astype(F).T


def rotate_interleaved(x, positions, base, dims):
    """Pairs (2i, 2i+1) of the first `dims` entries of the last axis turned by position * base^(-2i / dims)."""
    out = x.astype(F).copy()
    i = np.arange(dims // 2, dtype=F)
    angle = np.asarray(positions, dtype=F)[:, None] * np.power(F(base), -2.0 * i / dims)[None, :]
    c, s = np.cos(angle), np.sin(angle)
    while c.ndim < x.ndim:
        c, s = c[:, None], s[:, None]
    a, b = x[..., 0:dims:2].astype(F), x[..., 1:dims:2].astype(F)
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def windowed_softmax_attention(q, k, v, scale, window):
    """q, k [T, H, D]; v [T, H, V]; position i sees j with 0 <= i - j < window (window None: all j <= i)."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ v[lo:i + 1, h]
    return out


def latent_attention_mixer(h, w, pre, m, eps):
    """Queries and keys/values through low-rank latents; one rotated key part shared by the heads."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = rms_norm(h @ w[pre + "dq"].astype(F).T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].astype(F).T).reshape(T, H, D + R)
    kv = h @ w[pre + "dkv"].astype(F).T
    c = rms_norm(kv[:, :C], w[pre + "dkv.norm"], eps)
    k_rot = rotate_interleaved(kv[:, C:], pos, m["rot"]["base"], m["rot"]["dims"])               # [T, R]
    q_rot = rotate_interleaved(q[:, :, D:], pos, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[pre + "uk"].astype(F).T).reshape(T, H, D)
    v = (c @ w[pre + "uv"].astype(F).T).reshape(T, H, V)
    qq = np.concatenate([q[:, :, :D].astype(F), q_rot], axis=2)
    kk = np.concatenate([k_plain, np.broadcast_to(k_rot[:, None, :], (T, H, R))], axis=2)
    window = (m.get("mask") or {}).get("size")
    o = windowed_softmax_attention(qq, kk, v, m["scale"], window).reshape(T, H * V)
    return o @ w[pre + "o"].astype(F).T


def causal_conv(x, taps_w):
    """y[t, c] = sum_j w[c, j] x[t - (taps - 1) + j, c]: the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), x.astype(F)], axis=0)
    y = np.zeros((T, C), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j].astype(F)[None, :]
    return y


def gated_delta_rule(q, k, v, beta, g):
    """Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k [T, H, D]; v [T, H, V]; beta, g [T, H]."""
    T, H, D = q.shape
    V = v.shape[2]
    out = np.zeros((T, H, V), dtype=F)
    for h in range(H):
        S = np.zeros((D, V), dtype=F)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            out[t, h] = S.T @ q[t, h]
    return out


def delta_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[pre + "q"].astype(F).T, w[pre + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ w[pre + "k"].astype(F).T, w[pre + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ w[pre + "v"].astype(F).T, w[pre + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    group = np.arange(H) // (H // G)
    q, k = q[:, group], k[:, group]
    beta = sigmoid(h @ w[pre + "b"].astype(F).T)
    g = np.exp(-np.exp(w[pre + "A_log"].astype(F))[None, :] * softplus(h @ w[pre + "a"].astype(F).T + w[pre + "dt_bias"].astype(F)[None, :]))
    o = gated_delta_rule(q, k, v, beta, g)                                                        # [T, H, V]
    o = rms_norm(o, w[pre + "norm"], eps)
    o = o.reshape(T, H * V) * silu(h @ w[pre + "g"].astype(F).T)
    return o @ w[pre + "o"].astype(F).T


MIXERS = {"lightning": lightning_mixer, "latent_attention": latent_attention_mixer, "delta": delta_mixer}


def forward(config, w, ids, layers_out=None):
    """Logits [T, vocab] of a whole sequence.  `layers_out`: a list that receives the residual stream after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"].astype(F)[np.asarray(ids)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        h = layer_norm(x, w[pre + "norm1"], eps)
        y = MIXERS[layer["type"]](h, w, pre + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] != "dense":
                raise ValueError(mlp["kind"])
            y = y + clamped_glu(h, w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"], mlp["limit"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    h = layer_norm(x, w["final.norm"], eps)
    return (h @ w["head"].astype(F).T) * config["logit_scale"]
