"""Plain, slow implementation of the Gozatar decoder: whole sequences, no cache, no state carried between calls.

One function per mechanism, plain tensor arithmetic on the CPU (float64 unless told otherwise). It shares no code
with ``spissa_b200``: it reads config.json keys and a dict of tensors by their checkpoint names. Notation: X is the
set of residual streams [S, T, W]; a is what a sublayer reads.

    embedding       every stream starts as E[id_t]
    layer norm      n(x) = (x − mean) / sqrt(var + eps) ⊙ w
    hyper-conn.     a = n(Σ_s in_s X_s);  y = sublayer(a);  X_t ← Σ_s mix[s, t] X_s + out_t y
    mixer           y = c_l · window_attention(a) + c_r · gated_linear_attention(a)
    feed-forward    dense (tanh gelu) or routed experts with a shared expert
    head            logits = n_f(Σ_s X_s) · Hᵀ
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, w, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def unit_rms(v, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y_t = Σ_j w[:, j] ⊙ u_{t − taps + 1 + j}, zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * taps_w[:, j]
    return y


def rotate_half(v, dims: int, base: float, start: int = 0):
    """v [T, heads, dim]: dim i pairs with dim i + dims/2 (i < dims/2), turned by (start + t) · base^(−2i/dims)."""
    if dims <= 0:
        return v
    T, half = v.shape[0], dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    ang = (start + torch.arange(T, dtype=v.dtype))[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = v.clone()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def window_attention(a, w, p, m, eps):
    """The left branch: grouped-query softmax attention over the last ``mask.size`` positions, with a short
    convolution behind each projection, a partial rotation and a weightless rms norm of q and k per head."""
    T = a.shape[0]
    H, G, d, vd = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q, k, v = a @ w[p + "q"].T, a @ w[p + "k"].T, a @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = (short_conv(t, w[p + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, vd)
    rot = m.get("rot")
    if rot:
        q, k = rotate_half(q, rot["dims"], rot["base"]), rotate_half(k, rot["dims"], rot["base"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    size = (m.get("mask") or {}).get("size")
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = (j <= i) if not size else ((j <= i) & (i - j < size))
    out = torch.zeros(T, H, vd, dtype=a.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~see, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def gated_linear_attention(a, w, p, m, eps):
    """The right branch, token by token: S_t = diag(α_t) S_{t−1} + k_t v_tᵀ, o_t = S_tᵀ q_t per head."""
    T = a.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T * d ** -0.5).view(T, H, d)
    k = (a @ w[p + "k"].T).view(T, H, d)
    v = (a @ w[p + "v"].T).view(T, H, vd)
    z = (a @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(T, H, d)
    S = torch.zeros(H, d, vd, dtype=a.dtype)
    o = torch.zeros(T, H, vd, dtype=a.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * vd) * silu(a @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(a, w, p, m, eps):
    return m["left_scale"] * window_attention(a, w, p + "left.", m["left"], eps) + \
        m["right_scale"] * gated_linear_attention(a, w, p + "right.", m["right"], eps)


def dense_ff(a, w, p):
    return gelu_tanh(a @ w[p + "up"].T) @ w[p + "down"].T


def clamped_expert(a, w, p, limit):
    g = torch.clamp(a @ w[p + "gate"].T, max=limit)
    u = torch.clamp(a @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(a, w, p, r):
    """(chosen experts [T, top], their weights [T, top]) of the sigmoid router with a correction that only the
    choice sees and groups of neighbouring experts of which only the best may be chosen from."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(a @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        n, keep = groups["count"], groups["keep"]
        per = choice.view(-1, n, E // n)
        score = per.topk(min(2, E // n), dim=-1).values.sum(dim=-1)
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, E // n).reshape(-1, E), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def moe_ff(a, w, p, mlp):
    idx, wt = route(a, w, p, mlp["router"])
    y = torch.zeros_like(a)
    for t in range(a.shape[0]):
        for e, c in zip(idx[t].tolist(), wt[t]):
            y[t] += c * clamped_expert(a[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        y = y + clamped_expert(a, w, p + "shared.", mlp["shared"]["limit"])
    return y


def feed_forward(a, w, p, mlp):
    return dense_ff(a, w, p) if mlp["kind"] == "dense" else moe_ff(a, w, p, mlp)


def forward(cfg: dict, weights: dict, ids, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence. ``layers_out``: gets the sum of the streams after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    S = cfg.get("streams")
    X = x[None].repeat(S or 1, 1, 1)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [("1", lambda a: parallel_mixer(a, w, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append(("2", lambda a: feed_forward(a, w, p + "mlp.", layer["mlp"])))
        for q, f in subs:
            if S:
                u = torch.einsum("s,stw->tw", w[f"{p}hc{q}.in"], X)
                y = f(layer_norm(u, w[p + "norm" + q], eps))
                X = torch.einsum("sr,stw->rtw", w[f"{p}hc{q}.mix"], X) + w[f"{p}hc{q}.out"][:, None, None] * y[None]
            else:
                X = X + f(layer_norm(X[0], w[p + "norm" + q], eps))[None]
        if layers_out is not None:
            layers_out.append(X.sum(dim=0))
    return layer_norm(X.sum(dim=0), w["final.norm"], eps) @ w["head"].T
