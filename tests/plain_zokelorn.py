"""A plain, slow implementation of the Zokelorn decoder, for tests only.

Whole sequences, no cache, one function per mechanism, torch on the CPU in float32 or
float64; it shares no code with ``rocml_b200`` (the model folder is read with the
``safetensors`` package).  Notation: W is stored [out, in] and applied as W x; rms(x) =
x / sqrt(mean(x^2) + eps); n(x) = rms(x) * w.

    layer               h = n1(x);  x += mix(h) + ff(h)                      (one norm, both sublayers read it)
    attention           q = Wq h, k = Wk h, v = Wv h;  the first `dims` entries of every q and k head are rotated in
                        neighbouring pairs (2i, 2i+1) by p * f_i;  query i sees key j when j <= i and both lie in the
                        same block of `size` positions;  softmax((q . k) * scale);  head n's result times
                        sigmoid(Wg h)_n;  Wo
    frequencies         f_i = base^(-2i / dims), then by wavelength L = 2 pi / f:  L < original / high: f;
                        L > original / low: f / factor;  between: s = (original / L - low) / (high - low),
                        (1 - s) f / factor + s f
    lightning           q, k, v = silu(W. h);  S_t = d_n S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                        Wo (n_all_heads(o) * sigmoid(Wg h))
    retention           q, k, v = W. h;  k *= dim^(-1/2);  same recurrence;  Wo (rms_per_head(o) * silu(Wg h))
    dense ff            Wdown (gelu_tanh(Wgate h) * (Wup h))
    routed ff           s = sigmoid(Wr h);  groups of neighbouring experts, a group's score = its two largest s added;
                        only the `keep` best groups stay;  of those the `top` largest s are chosen;
                        weights = s / (sum of the chosen s + 1e-20);  experts: Wdown (silu(Wgate h) * (Wup h));
                        plus sigmoid(Wsg h) * shared expert (same form)
    loop                layers [start, stop) run `times` times in a row with the same weights
    output              logits = Whead n_f(x)
"""
from __future__ import annotations

import json
import math
import os

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot, dtype=torch.float64):
    """f_i for i < dims / 2, with the piecewise stretch of long wavelengths when `scaling` is given."""
    dims, base = rot["dims"], rot["base"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if sc:
            wave = 2.0 * math.pi / f
            if wave < sc["original"] / sc["high"]:
                pass
            elif wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=dtype)


def rotate_pairs(x, positions, rot):
    """x [T, heads, dim]: entries (2i, 2i + 1), i < dims / 2, turned by positions * f_i; the rest unchanged."""
    dims = rot["dims"]
    f = frequencies(rot, x.dtype)
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * f[None, :]            # [T, dims / 2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attention(h, w, pre, m, positions=None):
    """h [T, D] -> [T, D]; ``m`` is the layer's mixer dictionary."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = list(range(T)) if positions is None else positions
    q = (h @ w[pre + "q"].t()).reshape(T, H, dim)
    k = (h @ w[pre + "k"].t()).reshape(T, G, dim)
    v = (h @ w[pre + "v"].t()).reshape(T, G, vdim)
    q, k = rotate_pairs(q, pos, m["rot"]), rotate_pairs(k, pos, m["rot"])
    gate = torch.sigmoid(h @ w[pre + "g"].t())                                       # [T, H]
    p = torch.as_tensor(pos)
    size = m["mask"]["size"]
    seen = (p[None, :] <= p[:, None]) & ((p[:, None] // size) == (p[None, :] // size))
    out = torch.empty((T, H, vdim), dtype=h.dtype)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].t()) * m["scale"]
        a = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1)
        out[:, n] = (a @ v[:, g]) * gate[:, n:n + 1]
    return out.reshape(T, H * vdim) @ w[pre + "o"].t()


def decayed_sum(q, k, v, decay, state=None):
    """Per head: S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, dim], v [T, H, vdim].
    Returns (o [T, H, vdim], the last state [H, dim, vdim])."""
    T, H, dim = q.shape
    vdim = v.shape[-1]
    S = torch.zeros((H, dim, vdim), dtype=q.dtype) if state is None else state.clone()
    d = torch.as_tensor(decay, dtype=q.dtype)[:, None, None]
    o = torch.empty((T, H, vdim), dtype=q.dtype)
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = (S * q[t][:, :, None]).sum(dim=1)
    return o, S


def lightning(h, w, pre, m, eps):
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].t()).reshape(T, H, dim)
    k = silu(h @ w[pre + "k"].t()).reshape(T, H, dim)
    v = silu(h @ w[pre + "v"].t()).reshape(T, H, vdim)
    o, _ = decayed_sum(q, k, v, m["decay"])
    o = norm(o.reshape(T, H * vdim), w[pre + "norm"], eps) * torch.sigmoid(h @ w[pre + "g"].t())
    return o @ w[pre + "o"].t()


def retention(h, w, pre, m, eps):
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].t()).reshape(T, H, dim)
    k = (h @ w[pre + "k"].t()).reshape(T, H, dim) * dim ** -0.5
    v = (h @ w[pre + "v"].t()).reshape(T, H, vdim)
    o, _ = decayed_sum(q, k, v, m["decay"])
    o = rms(o, eps).reshape(T, H * vdim) * silu(h @ w[pre + "g"].t())
    return o @ w[pre + "o"].t()


def gated_ff(h, w, pre, act):
    return (act(h @ w[pre + "gate"].t()) * (h @ w[pre + "up"].t())) @ w[pre + "down"].t()


MARGINS = None      # a list, while a test wants to know how close the routers' choices were


def route(h, w, pre, r):
    """(chosen [T, top], weights [T, top]) from sigmoid scores, after the groups' cut."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[pre + "router"].t())                                     # [T, E]
    allowed = torch.ones_like(s, dtype=torch.bool)
    gr = r.get("groups")
    margin = torch.full((h.shape[0],), float("inf"), dtype=s.dtype)
    if gr and gr["count"] > 1 and gr["keep"] < gr["count"]:
        n, keep = gr["count"], gr["keep"]
        per = E // n
        by_group = s.reshape(-1, n, per)
        score = torch.topk(by_group, min(2, per), dim=-1).values.sum(dim=-1)         # [T, n]
        order = torch.topk(score, keep + 1, dim=-1)
        kept = order.indices[:, :keep]
        margin = order.values[:, keep - 1] - order.values[:, keep]
        mask = torch.zeros_like(score, dtype=torch.bool)
        mask.scatter_(1, kept, True)
        allowed = mask[:, :, None].expand(-1, -1, per).reshape(-1, E)
    choice = s.masked_fill(~allowed, -1.0)
    best = torch.topk(choice, min(top + 1, E), dim=-1)
    chosen = best.indices[:, :top]
    if top < E:
        margin = torch.minimum(margin, best.values[:, top - 1] - best.values[:, top])
    if MARGINS is not None:
        MARGINS.append(margin)
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def routed_ff(h, w, pre, f):
    r = f["router"]
    chosen, weights = route(h, w, pre, r)
    out = torch.zeros((h.shape[0], w[pre + "e0.down"].shape[0]), dtype=h.dtype)
    for e in range(r["experts"]):
        for slot in range(r["top"]):
            rows = torch.nonzero(chosen[:, slot] == e)[:, 0]
            if rows.numel():
                out[rows] += weights[rows, slot:slot + 1] * gated_ff(h[rows], w, f"{pre}e{e}.", silu)
    if f.get("shared"):
        out = out + torch.sigmoid(h @ w[pre + "shared.sg"].t()) * gated_ff(h, w, pre + "shared.", silu)
    return out


def closest_calls(w, cfg, ids):
    """Per token, the smallest margin by which any router of any layer run made a choice (infinite where none had
    one to make).  A token whose margin is within rounding may be routed otherwise by an implementation that rounds
    otherwise; in a model with recurrent or attention layers every later token may then differ too."""
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


def layer(x, w, cfg, i):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = norm(x, w[p + "norm1"], eps)
    m = L["mixer"]
    if L["type"] == "attention":
        y = attention(h, w, p + "mix.", m)
    elif L["type"] == "lightning":
        y = lightning(h, w, p + "mix.", m, eps)
    elif L["type"] == "retention":
        y = retention(h, w, p + "mix.", m, eps)
    else:
        raise ValueError(f"unknown mixer {L['type']!r}")
    f = L.get("mlp")
    if f is None:
        return x + y
    if f["kind"] == "dense":
        return x + (y + gated_ff(h, w, p + "mlp.", gelu_tanh))
    if f["kind"] == "moe":
        return x + (y + routed_ff(h, w, p + "mlp.", f))
    raise ValueError(f"unknown feed-forward {f['kind']!r}")


def layer_runs(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(w, cfg, ids, dtype=torch.float32, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run if asked)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    after = []
    for i in layer_runs(cfg):
        x = layer(x, w, cfg, i)
        after.append(x)
    logits = norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].t()
    return (logits, torch.stack(after)) if keep_layers else logits


def load_folder(folder):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return load_file(os.path.join(folder, "model.safetensors")), cfg
