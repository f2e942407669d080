"""A plain, slow implementation of the Pipilix decoder, for tests only.

Whole sequences, no cache, one function per mechanism, torch on the CPU in float32 or
float64; it shares no code with ``rocml_b200`` (the model folder is read with the
``safetensors`` package).  Notation: W is stored [out, in] and applied as W x; rms(x) =
x / sqrt(mean(x^2) + eps).

    embedding        x_t = E[id_t] * s_e + pe(t),  pe(t)[2i] = sin(t * 10000^(-2i/D)), pe(t)[2i+1] = cos(same)
    layer            x += n1b(mix(n1(x)));  x += n2b(ff(n2(x)))          (n*: rms(.) * w)
    latent attention q = Wq h;  c = rms(Wdkv h) * w_c;  k = Wuk c;  v = Wuv c  (head by head)
                     a_ij = softmax_j((q_i . k_j) * s_a) over 0 <= i - j < window
                     o_i = sigmoid(Wg h_i)_head * sum_j a_ij v_j;  out = Wo concat(o)
    dense ff         Wdown (silu(Wgate h) * (Wup h))
    routed ff        z = Wr h;  s = sigmoid(z);  chosen = top_k(s + b);  weights = s[chosen]
                     expert: g = min(Wgate h, L);  u = clamp(Wup h, -L, L);  Wdown (g * sigmoid(1.702 g) * (u + 1))
    loop             layers [start, stop) run `times` times with the same weights; before every pass but
                     the first the embedding output is added, then (every pass) row `pass` of loop.step
    output           logits = Whead (rms(x) * w_f) * s_l
"""
from __future__ import annotations

import json
import math
import os

import torch


def sinusoid(positions, width, dtype):
    """pe[p, 2i] = sin(p * 10000^(-2i / width)), pe[p, 2i + 1] = cos of the same angle."""
    half = (width + 1) // 2
    i = torch.arange(half, dtype=torch.float64)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * inv[None, :]
    pe = torch.zeros((len(positions), 2 * half), dtype=torch.float64)
    pe[:, 0::2] = torch.sin(ang)
    pe[:, 1::2] = torch.cos(ang)
    return pe[:, :width].to(dtype)


def embed(table, ids, scale, dtype):
    ids = torch.as_tensor(ids, dtype=torch.long)
    return table[ids] * scale + sinusoid(list(range(len(ids))), table.shape[1], dtype)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w


def latent_attention(h, w, pre, heads, dim, vdim, window, scale, eps):
    """h [T, D] -> [T, D].  ``w`` maps tensor names to tensors, ``pre`` is '<layer>.mix.'."""
    T = h.shape[0]
    q = (h @ w[pre + "q"].t()).reshape(T, heads, dim)
    c = norm(h @ w[pre + "dkv"].t(), w[pre + "dkv.norm"], eps)           # [T, rank]
    k = (c @ w[pre + "uk"].t()).reshape(T, heads, dim)
    v = (c @ w[pre + "uv"].t()).reshape(T, heads, vdim)
    gate = torch.sigmoid(h @ w[pre + "g"].t())                           # [T, heads]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < window)
    out = torch.empty((T, heads, vdim), dtype=h.dtype)
    for n in range(heads):
        s = (q[:, n] @ k[:, n].t()) * scale
        s = s.masked_fill(~seen, float("-inf"))
        a = torch.softmax(s, dim=-1)
        out[:, n] = (a @ v[:, n]) * gate[:, n:n + 1]
    return out.reshape(T, heads * vdim) @ w[pre + "o"].t()


def dense_ff(h, w, pre):
    g = h @ w[pre + "gate"].t()
    u = h @ w[pre + "up"].t()
    return (g * torch.sigmoid(g) * u) @ w[pre + "down"].t()


def expert_ff(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].t(), max=limit)
    u = torch.clamp(h @ w[pre + "up"].t(), min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].t()


MARGINS = None      # a list, while a test wants to know how close the routers' choices were


def route(h, w, pre, top):
    """(chosen [T, top] expert numbers, weights [T, top]): sigmoid scores; the correction only chooses."""
    s = torch.sigmoid(h @ w[pre + "router"].t())
    choice = s + w[pre + "correction"]
    chosen = torch.topk(choice, top, dim=-1).indices
    if MARGINS is not None and top < choice.shape[-1]:
        best = torch.topk(choice, top + 1, dim=-1).values
        MARGINS.append(best[:, top - 1] - best[:, top])        # per token: the last chosen over the first left out
    return chosen, torch.gather(s, 1, chosen)


def closest_calls(w, cfg, ids):
    """Per token, the smallest margin by which any router of any layer run chose its last expert over the next
    (infinite where no router has a choice to make).  A token whose margin is within rounding may be routed otherwise
    by an implementation that rounds otherwise, and so may every later token that sees it."""
    global MARGINS
    MARGINS = []
    try:
        forward(w, cfg, ids, torch.float64)
        got = MARGINS
    finally:
        MARGINS = None
    out = torch.full((len(ids),), float("inf"), dtype=torch.float64)
    for m in got:
        out = torch.minimum(out, m)
    return out


def routed_ff(h, w, pre, experts, top, limit):
    chosen, weights = route(h, w, pre, top)
    out = torch.zeros_like(h)
    for e in range(experts):
        for slot in range(top):
            rows = torch.nonzero(chosen[:, slot] == e)[:, 0]
            if rows.numel():
                out[rows] += weights[rows, slot:slot + 1] * expert_ff(h[rows], w, f"{pre}e{e}.", limit)
    return out


def layer(x, w, cfg, i):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    if L["type"] != "latent_attention":
        raise ValueError(f"unknown mixer {L['type']!r}")
    m = L["mixer"]
    y = latent_attention(norm(x, w[p + "norm1"], eps), w, p + "mix.", m["heads"], m["dim"], m["vdim"],
                         m["mask"]["size"], m["scale"], eps)
    x = x + norm(y, w[p + "norm1b"], eps)
    f = L.get("mlp")
    if f is None:
        return x
    hn = norm(x, w[p + "norm2"], eps)
    if f["kind"] == "dense":
        y = dense_ff(hn, w, p + "mlp.")
    elif f["kind"] == "moe":
        y = routed_ff(hn, w, p + "mlp.", f["router"]["experts"], f["router"]["top"], f["expert"]["limit"])
    else:
        raise ValueError(f"unknown feed-forward {f['kind']!r}")
    return x + norm(y, w[p + "norm2b"], eps)


def layer_runs(cfg):
    """The order the layers run in: [(layer, pass or None)], the looped span repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, None, False) for i in range(b, n)]


def forward(w, cfg, ids, dtype=torch.float32, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run if asked)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    x0 = embed(w["embed"], ids, cfg["embedding"]["scale"], dtype)
    x = x0
    after = []
    for i, t, first in layer_runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = layer(x, w, cfg, i)
        after.append(x)
    logits = (norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].t()) * cfg["logit_scale"]
    return (logits, torch.stack(after)) if keep_layers else logits


def load_folder(folder):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return load_file(os.path.join(folder, "model.safetensors")), cfg
