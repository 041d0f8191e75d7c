"""Plain, slow implementation of the Duzinex decoder: whole sequences, no cache, no state carried between calls.

One function per mechanism, plain tensor arithmetic on the CPU (float64 unless told otherwise). It shares no code
with ``spissa_b200``: it reads config.json keys and the safetensors file itself (through the reader of
``llama_plain``, which is test code too). Notation: x is the residual stream [T, W]; a is what a mixer reads.

    embedding      x_t = E[id_t] · s
    dynamic tanh   n(x) = tanh(α x) ⊙ w + b
    token shift    a_t ← a_t + (a_{t-1} − a_t) ⊙ μ,  a_{-1} = 0
    layer          x ← x + mixer(shift(n₁(x)));  x ← x + ff(n₂(x))  (ff may be missing)
    loop           layers lo … hi−1 run r times; passes 2 … r first add the embedding's output to x
    head           logits = n_f(x) · Eᵀ
"""
from __future__ import annotations

import math

import torch

from .llama_plain import read_model_folder  # noqa: F401  (re-exported for the tests)


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v²) + eps) over the last axis."""
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def dynamic_tanh(x, w, name):
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def token_shift(a, mu):
    before = torch.cat([torch.zeros_like(a[:1]), a[:-1]], dim=0)
    return a + (before - a) * mu


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_neighbours(v, rot_dims: int, base: float):
    """v [T, heads, maps, dim]: dims 2i and 2i+1 (2i < rot_dims) turn by t · base^(−2i/rot_dims)."""
    if rot_dims <= 0:
        return v
    T = v.shape[0]
    freq = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)], dtype=v.dtype)
    ang = torch.arange(T, dtype=v.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, None, :], torch.sin(ang)[:, None, None, :]
    out = v.clone()
    even, odd = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
    out[..., 0:rot_dims:2] = even * c - odd * s
    out[..., 1:rot_dims:2] = odd * c + even * s
    return out


def visible(T: int, window, keep_first: int):
    """[T, T] bool: query i sees key j when j ≤ i and (i − j < window or j < keep_first); no window: causal."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    causal = j <= i
    if not window:
        return causal
    return causal & ((i - j < window) | (j < keep_first))


def diff_lambda(w, p, diff):
    return math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff


def differential_attention(a, w, p, m, eps):
    T = a.shape[0]
    H, G, d, vd = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T + w[p + "q.b"]).view(T, H, 2, d)
    k = (a @ w[p + "k"].T + w[p + "k.b"]).view(T, G, 2, d)
    v = (a @ w[p + "v"].T + w[p + "v.b"]).view(T, G, vd)
    rot = m.get("rot")
    if rot:
        q, k = rotate_neighbours(q, rot["dims"], rot["base"]), rotate_neighbours(k, rot["dims"], rot["base"])
    mask = m.get("mask")
    see = visible(T, mask["size"] if mask else None, (mask.get("keep_first") or 0) if mask else 0)
    lam = diff_lambda(w, p, m["diff"])
    cap = m.get("softcap")
    heads = []
    for h in range(H):
        g = h // (H // G)
        maps = []
        for i in range(2):
            s = (q[:, h, i] @ k[:, g, i].T) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~see, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        heads.append(unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"]))
    return torch.cat(heads, dim=-1) @ w[p + "o"].T + w[p + "o.b"]


def retention(a, w, p, m, eps):
    T = a.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T).view(T, H, d)
    k = (a @ w[p + "k"].T).view(T, H, d) / math.sqrt(d)
    v = (a @ w[p + "v"].T).view(T, H, vd)
    gamma = torch.tensor(m["decay"], dtype=a.dtype)[:, None, None]
    S = torch.zeros(H, d, vd, dtype=a.dtype)
    rows = []
    for t in range(T):
        S = gamma * S + k[t][:, :, None] * v[t][:, None, :]
        rows.append(torch.einsum("hij,hi->hj", S, q[t]))
    o = unit_rms(torch.stack(rows), eps).reshape(T, H * vd)
    return (o * silu(a @ w[p + "g"].T)) @ w[p + "o"].T


def mingru(a, w, p, m):
    z = torch.sigmoid(a @ w[p + "z"].T + w[p + "z.b"])
    u = a @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(m["width"], dtype=a.dtype)
    rows = []
    for t in range(a.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S)
    return (torch.stack(rows) * silu(a @ w[p + "g"].T)) @ w[p + "o"].T


def polynorm_ff(a, w, p, eps):
    z = a @ w[p + "up"].T
    c = [float(x) for x in w[p + "act"]]
    return (c[0] * unit_rms(z, eps) + c[1] * unit_rms(z * z, eps) + c[2] * unit_rms(z * z * z, eps) + c[3]) @ w[p + "down"].T


def layer_runs(cfg) -> list:
    n = len(cfg["layers"])
    loop = cfg.get("loop") or dict(start=0, stop=0, times=1)
    runs = [(i, False) for i in range(loop["start"])]
    for r in range(loop["times"]):
        runs += [(i, r > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def model_logits(cfg, weights, ids, dtype=torch.float64, stream_out=None):
    """Logits [T, vocab] of the whole sequence ``ids``; ``stream_out`` (a list) receives x after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(ids), dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    first = x.clone()
    for i, again in layer_runs(cfg):
        if again:
            x = x + first
        layer, p = cfg["layers"][i], f"l{i}."
        a = token_shift(dynamic_tanh(x, w, p + "norm1"), w[p + "shift"])
        if layer["type"] == "attention":
            y = differential_attention(a, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "retention":
            y = retention(a, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "mingru":
            y = mingru(a, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + polynorm_ff(dynamic_tanh(x, w, p + "norm2"), w, p + "mlp.", eps)
        if stream_out is not None:
            stream_out.append(x.clone())
    return dynamic_tanh(x, w, "final.norm") @ w["embed"].T


def generate_greedy(cfg, weights, prompt, n_new: int) -> list:
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(model_logits(cfg, weights, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out
