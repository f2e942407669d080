"""Zokelorn on the GPU against the plain implementation (tests/plain_zokelorn.py): each mechanism alone, then
the engine in every way of cutting and batching, in 32-bit and in bfloat16.

Tolerances are a fraction of the largest |logit| of the row compared.  float32: sums of a few hundred terms
in another order than the plain implementation's float64, through up to seven layer runs with a softmax made to
pick few keys.  bfloat16: activations are rounded to 8 bits of mantissa between kernels, a dozen roundings a
layer run.
"""
import json
import math

import pytest
import torch

import plain_zokelorn as P
from tiny_models import ZOKELORN, prompt, write_zokelorn

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 3e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"

# A router's choice between two scores that differ by less than rounding can fall either way; the token's logits
# then differ by much more than rounding, and so do those of every later token, which sees it through the
# attention and the running sums.  The plain implementation reports, per token, the smallest margin of any of its
# routers' choices; rows from the first such token on are excused (and must be few).
CLOSE = {"float32": 2e-5, "bfloat16": 4e-3}


def rel_err(got, want):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


def assert_rows(got, want, calls, dtype, what, first_row=0):
    """``calls`` are the margins of ALL the sequence's tokens; the rows compared start at token ``first_row``."""
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    scale = want.abs().amax(dim=-1).clamp_min(1e-30)
    err = (got - want).abs().amax(dim=-1) / scale
    near = torch.nonzero(calls < CLOSE[dtype])[:, 0]
    n_ok = len(err) if not len(near) else max(0, int(near[0]) - first_row)
    bad = err[:n_ok] >= TOL[dtype]
    if dtype == "bfloat16":
        # a row whose running sums nearly cancel before they are normalised multiplies the rounding of its input
        # many times (measured: single rows at 20 times the median): a few rows may lie above the tolerance, none
        # at the size of a fault (32-bit is the sharp comparison; the kernels that only bfloat16 uses have their own)
        few = int(bad.sum()) <= max(2, 0.1 * n_ok)
        bad = (err[:n_ok] >= 10 * TOL[dtype]) if few else bad
    assert not bool(bad.any()), f"{what}: rows {torch.nonzero(bad)[:, 0].tolist()[:8]} off by up to {float(err[:n_ok][bad].max()):.3g}"
    assert n_ok >= 0.7 * len(err), f"{what}: only {n_ok} of {len(err)} rows lie before the first near tie"
    assert bool(torch.isfinite(got).all()), what


def close(got, want, tol):
    want = want.double()
    got = got.double().cpu()
    return float((got - want).abs().max()) <= tol * max(1e-30, float(want.abs().max()))


# ---- each mechanism alone -------------------------------------------------------------------------------------

@pytest.mark.parametrize("rot", [
    {"base": 10000.0, "dims": 16},
    {"base": 1e6, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
    {"base": 500.0, "dims": 32, "scaling": {"factor": 3.0, "low": 0.5, "high": 3.0, "original": 40}},
    {"base": 100.0, "dims": 12, "scaling": {"factor": 2.0, "low": 0.25, "high": 1.0, "original": 16}},
])
def test_frequencies_with_stretched_long_waves(rot):
    """The position part's table against the plain implementation: all three pieces of the stretch occur."""
    from rocml_b200.config.specs import PositionSpec, _frozen_params
    from rocml_b200.parts import BuildEnv, build_position
    params = {"scaling": rot["scaling"]} if "scaling" in rot else {}
    enc = build_position(PositionSpec("rope_pairs", theta=rot["base"], rot_dim=rot["dims"], params_items=_frozen_params(params)),
                         64, BuildEnv(torch.device(DEV), torch.bfloat16))
    want = P.frequencies(rot)
    assert enc.interleaved and enc.rot_dim == rot["dims"]
    assert float((enc.inv_freq.cpu().double() - want).abs().max() / want.max()) < 1e-7
    if "scaling" in rot and rot["scaling"]["original"] == 40:
        plain = P.frequencies({"base": rot["base"], "dims": rot["dims"]})
        ratio = (want / plain).tolist()
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 3.0) < 1e-12 and any(1 / 3.0 + 1e-6 < r < 1 - 1e-6 for r in ratio)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, hd, vd, rot_dims, parts", [(4, 2, 32, 16, 16, 1), (3, 3, 20, 28, 12, 3), (8, 1, 64, 64, 64, 2),
                                                                (2, 2, 128, 64, 128, 1), (5, 1, 16, 16, 0, 1)])
def test_rotation_of_neighbouring_pairs_padding_and_gates(dtype, nq, nkv, hd, vd, rot_dims, parts):
    """Queries and keys turned in pairs (2i, 2i + 1) over the first rot_dims entries, value heads of another width,
    every head padded with zeros to one width in q and in the pages, sigmoid gates from the row's last columns;
    from one result and from partial sums."""
    from rocml_b200 import kernels
    torch.manual_seed(nq * hd + vd)
    dt = DT[dtype]
    T = 70
    hdp = -(-max(hd, vd) // 16) * 16
    width = nq * hd + nkv * (hd + vd) + nq
    width_p = -(-width // 8) * 8
    rows = torch.randn(parts, T, width_p) if parts > 1 else torch.randn(T, width_p).to(dt)
    pos = torch.arange(5, 5 + T, dtype=torch.int32)
    pos[-1] = 4000
    rot = {"base": 10000.0, "dims": rot_dims}
    inv = P.frequencies(rot).float().to(DEV) if rot_dims else None
    n_pages = 70
    kc = torch.full((n_pages, nkv, 64, hdp), 7.0, dtype=dt, device=DEV)
    vc = torch.full((n_pages, nkv, 64, hdp), 7.0, dtype=dt, device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, n_pages).contiguous().to(DEV)
    q = torch.full((T, nq * hdp), 7.0, dtype=dt, device=DEV)
    gates = torch.empty((T, nq), dtype=torch.float32, device=DEV)
    kernels.qk_norm_rope_cache(rows.to(DEV), q, T, nq, nkv, hd, None, None, 1e-6, inv, rot_dims, pos.to(DEV),
                               torch.zeros(T, dtype=torch.int32, device=DEV), table, kc, vc, v_head_dim=vd,
                               padded_head_dim=hdp, interleaved=True, gates=gates)
    x = (rows.double().sum(0) if parts > 1 else rows.double())
    wq = x[:, :nq * hd].reshape(T, nq, hd)
    wk = x[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    wv = x[:, (nq + nkv) * hd:(nq + nkv) * hd + nkv * vd].reshape(T, nkv, vd)
    wg = torch.sigmoid(x[:, width - nq:width])
    if rot_dims:
        wq, wk = P.rotate_pairs(wq, pos.tolist(), rot), P.rotate_pairs(wk, pos.tolist(), rot)
    tol = 1e-2 if dtype == "bfloat16" else (2e-3 if rot_dims else 1e-6)     # a 32-bit angle of 4000 radians
    got_q = q.reshape(T, nq, hdp)
    assert close(got_q[:, :, :hd], wq, tol) and float(got_q[:, :, hd:].abs().sum()) == 0
    assert close(got_q[:-1, :, :hd], wq[:-1], 1e-2 if dtype == "bfloat16" else 2e-5)
    assert close(gates, wg, 1e-6)
    for t in range(T):
        p = int(pos[t])
        page = n_pages - 1 - p // 64
        assert close(kc[page, :, p % 64, :hd], wk[t], tol), t
        assert close(vc[page, :, p % 64, :vd], wv[t], 1e-2 if dtype == "bfloat16" else 1e-6), t
        assert float(kc[page, :, p % 64, hd:].abs().sum()) == 0 and float(vc[page, :, p % 64, vd:].abs().sum()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, vdim, acts, k_scale", [(3, 16, 24, "silu", 1.0), (2, 24, 8, "none", 24 ** -0.5),
                                                             (1, 40, 12, "none", 0.3), (7, 4, 4, "silu", 1.0),
                                                             (2, 72, 136, "silu", 1.0), (4, 128, 128, "none", 0.1)])
def test_decayed_running_sum(dtype, heads, dim, vdim, acts, k_scale):
    """Three sequences in one step, whole; then the same tokens in pieces of unequal sizes and one by one, the state
    carried in the slots; a slot that is zeroed and used again; from one result and from partial sums.  Decays of 0
    and 1 are among them.  32-bit: pieces give the same bits as the whole."""
    from rocml_b200 import kernels
    torch.manual_seed(heads * dim + vdim)
    dt = DT[dtype]
    lens = [37, 1, 90]
    decay = [0.0, 1.0, 0.9, 0.5, 0.99, 0.97, 0.3][:heads]
    qk, vw = heads * dim, heads * vdim
    N = 2 * qk + 2 * vw + 8
    rows = [torch.randn(n, N).to(dt) for n in lens]
    state = torch.full((5, heads, dim, vdim), 3.0, dtype=torch.float32, device=DEV)
    slots = [4, 0, 2]
    d_dev = torch.tensor(decay, dtype=torch.float32, device=DEV)

    def run(pieces):
        """pieces: per step a list of (sequence, start, stop)."""
        outs = {i: [] for i in range(len(lens))}
        for step in pieces:
            x = torch.cat([rows[i][a:b] for i, a, b in step]).to(DEV)
            cu = [0]
            for i, a, b in step:
                cu.append(cu[-1] + b - a)
            T = cu[-1]
            o = torch.full((T, vw), float("nan"), dtype=torch.float32, device=DEV)
            ss = torch.tensor([slots[i] for i, _, _ in step] + [-1], dtype=torch.int32, device=DEV)
            cu_t = torch.tensor(cu + [cu[-1]], dtype=torch.int32, device=DEV)
            kernels.decay_scan(x, T, 8, 8 + qk, 8 + 2 * qk, heads, dim, vdim, acts, acts, k_scale, d_dev, state, ss, cu_t,
                               len(step) + 1, o)
            for j, (i, a, b) in enumerate(step):
                outs[i].append(o[cu[j]:cu[j + 1]].cpu())
        return [torch.cat(outs[i]) for i in range(len(lens))]

    def fresh():
        for s in slots:
            state[s].zero_()

    act = P.silu if acts == "silu" else (lambda z: z)
    want, want_state = [], []
    for r in rows:
        x = r.double()
        q = act(x[:, 8:8 + qk]).reshape(-1, heads, dim)
        k = act(x[:, 8 + qk:8 + 2 * qk]).reshape(-1, heads, dim) * k_scale
        v = act(x[:, 8 + 2 * qk:8 + 2 * qk + vw]).reshape(-1, heads, vdim)
        o, S = P.decayed_sum(q, k, v, decay)
        want.append(o.reshape(-1, vw))
        want_state.append(S)
    fresh()
    whole = run([[(0, 0, 37), (1, 0, 1), (2, 0, 90)]])
    tol = 2e-5                                      # bfloat16 inputs are exact in 32-bit sums
    for i in range(3):
        assert close(whole[i], want[i], tol), i
        assert close(state[slots[i]], want_state[i], tol), i
    assert float((state[1] - 3.0).abs().max()) == 0 and float((state[3] - 3.0).abs().max()) == 0     # other slots untouched
    fresh()
    cut = run([[(0, 0, 2), (2, 0, 9)], [(2, 9, 73), (0, 2, 36), (1, 0, 1)], [(0, 36, 37), (2, 73, 74)]] +
              [[(2, t, t + 1)] for t in range(74, 90)])
    for i in range(3):
        assert torch.equal(cut[i], whole[i]), i
    # partial sums: the same rows as three 32-bit parts
    fresh()
    parts = [torch.randn(3, n, N) for n in lens]
    x3 = torch.cat(parts, dim=1).to(DEV)
    o = torch.empty((sum(lens), vw), dtype=torch.float32, device=DEV)
    kernels.decay_scan(x3, sum(lens), 8, 8 + qk, 8 + 2 * qk, heads, dim, vdim, acts, acts, k_scale, d_dev, state,
                       torch.tensor(slots, dtype=torch.int32, device=DEV),
                       torch.tensor([0, 37, 38, 128], dtype=torch.int32, device=DEV), 3, o)
    x = parts[2].double().sum(0)
    ow, _ = P.decayed_sum(act(x[:, 8:8 + qk]).reshape(-1, heads, dim), act(x[:, 8 + qk:8 + 2 * qk]).reshape(-1, heads, dim) * k_scale,
                          act(x[:, 8 + 2 * qk:8 + 2 * qk + vw]).reshape(-1, heads, vdim), decay)
    assert close(o[38:], ow.reshape(-1, vw), 2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, vdim, acts, k_scale", [(3, 16, 24, "silu", 1.0), (2, 24, 8, "none", 24 ** -0.5),
                                                             (7, 4, 4, "silu", 1.0), (2, 72, 120, "silu", 1.0),
                                                             (4, 128, 128, "none", 0.1), (2, 64, 64, "silu", 1.0)])
def test_decayed_running_sum_by_blocks_of_tokens(dtype, heads, dim, vdim, acts, k_scale):
    """The prompts' way: blocks of 64 tokens side by side, against the plain implementation and against the kernel that
    goes token after token; sequences of 1, 64, 65, 200 and 131 tokens, one of them going on from a state; a padding
    entry; decays of 0 and 1."""
    from rocml_b200 import kernels
    torch.manual_seed(heads * dim + vdim + 1)
    dt = DT[dtype]
    lens = [1, 64, 65, 200, 131]
    decay = [0.0, 1.0, 0.9, 0.5, 0.99, 0.97, 0.3][:heads]
    qk, vw = heads * dim, heads * vdim
    N = 2 * qk + 2 * vw
    rows = [torch.randn(n, N).to(dt) for n in lens]
    slots = [3, 0, 5, 1, 4]
    start = torch.randn(heads, dim, vdim)
    d_dev = torch.tensor(decay, dtype=torch.float32, device=DEV)
    x = torch.cat(rows).to(DEV)
    T = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    ss = torch.tensor(slots[:2] + [-1] + slots[2:], dtype=torch.int32, device=DEV)
    cu_t = torch.tensor(cu[:3] + [cu[2]] + cu[3:], dtype=torch.int32, device=DEV)
    got = {}
    for way in ("blocks", "tokens"):
        state = torch.zeros((6, heads, dim, vdim), dtype=torch.float32, device=DEV)
        state[1] = start.to(DEV)
        o = torch.full((T, vw), float("nan"), dtype=torch.float32, device=DEV)
        if way == "blocks":
            work = torch.empty((T // 64 + 6, heads, dim, vdim), dtype=torch.float32, device=DEV)
            assert kernels.decay_scan_blocks(x, T, 0, qk, 2 * qk, heads, dim, vdim, acts, acts, k_scale, d_dev, state, ss, cu_t, 6, o, work)
        else:
            kernels.decay_scan(x, T, 0, qk, 2 * qk, heads, dim, vdim, acts, acts, k_scale, d_dev, state, ss, cu_t, 6, o)
        got[way] = (o.cpu(), state.cpu())
    act = P.silu if acts == "silu" else (lambda z: z)
    for i, r in enumerate(rows):
        xx = r.double()
        q = act(xx[:, :qk]).reshape(-1, heads, dim)
        k = act(xx[:, qk:2 * qk]).reshape(-1, heads, dim) * k_scale
        v = act(xx[:, 2 * qk:2 * qk + vw]).reshape(-1, heads, vdim)
        ow, S = P.decayed_sum(q, k, v, decay, state=start.double() if slots[i] == 1 else None)
        for way in ("blocks", "tokens"):
            assert close(got[way][0][cu[i]:cu[i + 1]], ow.reshape(-1, vw), 3e-5), (way, i)
            assert close(got[way][1][slots[i]], S, 3e-5), (way, i)
    assert float(got["blocks"][1][2].abs().max()) == 0          # a slot that no sequence of the step holds


@pytest.mark.parametrize("heads, dim, vdim, acts", [(3, 16, 24, "silu"), (2, 24, 8, "none"), (7, 4, 4, "silu"), (2, 72, 136, "silu"),
                                                   (4, 128, 128, "none"), (1, 300, 40, "none")])
def test_decayed_running_sum_one_token_a_sequence(heads, dim, vdim, acts):
    """A decode step's kernel: twenty steps of four sequences (one entry of the batch is padding) from given states,
    from partial sums, against the plain implementation; decays of 0 and 1."""
    from rocml_b200 import kernels
    torch.manual_seed(heads * dim + vdim + 2)
    steps, B = 20, 4
    decay = [0.0, 1.0, 0.9, 0.5, 0.99, 0.97, 0.3][:heads]
    qk, vw = heads * dim, heads * vdim
    N = 2 * qk + vw
    rows = torch.randn(steps, 2, B, N)                       # two partial sums a step
    start = torch.randn(B, heads, dim, vdim)
    state = torch.zeros((6, heads, dim, vdim), dtype=torch.float32, device=DEV)
    slots = [5, 0, 3, 2]
    for i, s in enumerate(slots):
        state[s] = start[i].to(DEV)
    d_dev = torch.tensor(decay, dtype=torch.float32, device=DEV)
    ss = torch.tensor(slots[:2] + [-1] + slots[2:], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1, 2, 2, 3, 4], dtype=torch.int32, device=DEV)
    got = []
    for t in range(steps):
        o = torch.full((B, vw), float("nan"), dtype=torch.float32, device=DEV)
        kernels.decay_scan(rows[t].to(DEV), B, 0, qk, 2 * qk, heads, dim, vdim, acts, acts, 0.5, d_dev, state, ss, cu, 5, o,
                           one_token_each=True)
        got.append(o.cpu())
    got = torch.stack(got)                                   # [steps, B, vw]
    act = P.silu if acts == "silu" else (lambda z: z)
    for i in range(B):
        x = rows[:, :, i].double().sum(1)
        ow, S = P.decayed_sum(act(x[:, :qk]).reshape(-1, heads, dim), act(x[:, qk:2 * qk]).reshape(-1, heads, dim) * 0.5,
                              act(x[:, 2 * qk:]).reshape(-1, heads, vdim), decay, state=start[i].double())
        assert close(got[:, i], ow.reshape(steps, vw), 3e-5), i
        assert close(state[slots[i]], S, 3e-5), i
    assert float(state[1].abs().max()) == 0 and float(state[4].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("groups, gw, weight, gate", [(1, 72, True, "sigmoid"), (6, 8, False, "silu"), (3, 136, True, "silu"),
                                                      (1, 1000, False, "sigmoid"), (40, 4, False, "sigmoid"),
                                                      (5, 6, True, "silu"), (1, 30, True, "sigmoid")])
def test_norm_over_groups_of_columns_and_gate(dtype, groups, gw, weight, gate):
    from rocml_b200 import kernels
    torch.manual_seed(groups + gw)
    dt = DT[dtype]
    T, W = 11, groups * gw
    o = torch.randn(T, W) * 4
    proj = torch.randn(2, T, W + 16)
    w = (torch.rand(W) + 0.5).to(dt) if weight else None
    out = torch.empty((T, W), dtype=dt, device=DEV)
    slot = torch.zeros(T, dtype=torch.int32, device=DEV)
    kernels.group_norm_gate(o.to(DEV), proj.to(DEV), 16, None if w is None else w.to(DEV), 1e-5, groups, gate, out, slot, T)
    z = proj.double().sum(0)[:, 16:]
    g = torch.sigmoid(z) if gate == "sigmoid" else P.silu(z)
    want = P.rms(o.double().reshape(T, groups, gw), 1e-5).reshape(T, W) * (w.double() if weight else 1.0) * g
    assert close(out, want, 1e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("E, top, groups, keep", [(6, 2, 3, 2), (16, 4, 4, 3), (9, 2, 3, 1), (4, 4, 2, 2), (64, 6, 8, 4),
                                                  (8, 3, 1, 1), (12, 2, 12, 5), (256, 8, 8, 4)])
def test_choice_among_the_best_groups(E, top, groups, keep):
    """Scores, the groups' cut, the choice and the weights that sum to one, against the plain implementation; every
    choice also gets a place of its own among its expert's rows."""
    from rocml_b200 import kernels
    torch.manual_seed(E + top)
    T, K = 200, 24
    h = torch.randn(T, K)
    wr = torch.randn(E, K) * 0.5
    r = {"experts": E, "top": top}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    P.MARGINS = []
    chosen, weights = P.route(h.double(), {"x.router": wr.double()}, "x.", r)
    margins, P.MARGINS = P.MARGINS[0], None
    z = (h.double() @ wr.double().t()).float()
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    place = torch.empty((T, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((T, top), dtype=torch.float32, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    slot = torch.zeros(T, dtype=torch.int32, device=DEV)
    slot[7] = -1
    kernels.moe_route(z.to(DEV), None, slot, T, top, ids, wts, place, counts, n_groups=groups, keep_groups=keep,
                      renormalize=True, norm_eps=1e-20)
    decided = margins > 1e-6
    decided[7] = False
    assert int(decided.sum()) > 0.95 * T
    got = torch.sort(ids.cpu()[decided].long(), dim=-1)
    want = torch.sort(chosen[decided], dim=-1)
    assert torch.equal(got.values, want.values)
    gw = torch.gather(wts.cpu()[decided].double(), 1, got.indices)
    ww = torch.gather(weights[decided], 1, want.indices)
    assert float((gw - ww).abs().max()) < 1e-6
    assert float((wts.cpu()[decided].double().sum(-1) - 1).abs().max()) < 1e-6
    assert int(ids[7].max()) == -1
    assert int(counts.sum()) == (T - 1) * top
    for e in range(E):
        pl = place.cpu()[ids.cpu() == e]
        assert sorted(pl.tolist()) == list(range(len(pl)))


def test_the_sum_over_choices_takes_a_gated_shared_result_along():
    from rocml_b200 import kernels
    torch.manual_seed(3)
    T, H, top, R = 9, 40, 3, 50
    y = torch.randn(R, H)
    row_of = torch.randint(0, R, (T, top), dtype=torch.int32)
    row_of[2, 1] = -1
    wts = torch.rand(T, top)
    extra = torch.randn(2, T, H)
    z = torch.randn(T, 5)
    out = torch.empty((T, H), dtype=torch.float32, device=DEV)
    kernels.moe_combine(y.to(DEV), row_of.to(DEV), wts.to(DEV), T, top, out, extra=extra.to(DEV), extra_gate=z.to(DEV)[:, 4])
    want = torch.zeros(T, H, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            if row_of[t, j] >= 0:
                want[t] += wts[t, j].double() * y[row_of[t, j]].double()
    want += torch.sigmoid(z[:, 4:5].double()) * extra.double().sum(0)
    assert close(out, want, 1e-6)
    kernels.moe_combine(y.to(DEV), row_of.to(DEV), wts.to(DEV), T, top, out, extra=extra.to(DEV))
    assert close(out, want - torch.sigmoid(z[:, 4:5].double()) * extra.double().sum(0) + extra.double().sum(0), 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gelu_gate_and_head_gate(dtype):
    from rocml_b200 import kernels
    torch.manual_seed(1)
    dt = DT[dtype]
    T, I = 7, 52
    gu = torch.randn(3, T, 2 * I) * 2
    out = torch.empty((T, I), dtype=dt, device=DEV)
    kernels.gated_act(gu.to(DEV), out, "gelu_tanh")
    x = gu.double().sum(0)
    assert close(out, P.gelu_tanh(x[:, :I]) * x[:, I:], 1e-6 if dtype == "float32" else 1e-2)
    for heads, in_w, out_w in ((5, 32, 20), (3, 30, 18), (2, 128, 128)):
        a = torch.randn(T, heads * in_w).to(dt)
        g = torch.rand(T, heads)
        o = torch.empty((T, heads * out_w), dtype=dt, device=DEV)
        kernels.head_gate(a.to(DEV), o, g.to(DEV), heads, in_w, out_w, T)
        want = a.double().reshape(T, heads, in_w)[:, :, :out_w] * g.double()[:, :, None]
        assert close(o, want.reshape(T, -1), 1e-6 if dtype == "float32" else 1e-2)
        kernels.head_gate(a.to(DEV), o, None, heads, in_w, out_w, T)
        assert close(o, a.double().reshape(T, heads, in_w)[:, :, :out_w].reshape(T, -1), 1e-6 if dtype == "float32" else 1e-2)


# ---- the engine -----------------------------------------------------------------------------------------------

class Folder:
    """A model folder with its plain implementation (logits and the routers' margins, kept per prompt)."""

    def __init__(self, folder):
        self.folder = folder
        self.w, self.cfg = P.load_folder(folder)
        self.kept = {}

    def __call__(self, ids):
        key = tuple(ids)
        if key not in self.kept:
            self.kept[key] = (P.forward(self.w, self.cfg, list(ids), torch.float64), P.closest_calls(self.w, self.cfg, list(ids)))
        return self.kept[key][0]

    def calls(self, ids):
        self(ids)
        return self.kept[tuple(ids)][1]


@pytest.fixture(scope="module", params=sorted(ZOKELORN))
def models(request, tmp_path_factory):
    """Two folders a configuration.  In the first the routers' choices follow the tokens; the 32-bit runs use it.
    Over hundreds of tokens some choice is always closer than bfloat16's rounding, and a choice that falls the other
    way moves every later token; the bfloat16 runs therefore use a second folder in which every token makes the same
    choices by a wide margin (the routing kernel's own test keeps choices that follow the tokens)."""
    name = request.param
    a = str(tmp_path_factory.mktemp(f"zokelorn_{name}"))
    b = str(tmp_path_factory.mktemp(f"zokelorn_{name}_fixed"))
    write_zokelorn(a, ZOKELORN[name], seed=60 + ord(name[-1]), std=0.06, sharp=3.0)
    write_zokelorn(b, ZOKELORN[name], seed=60 + ord(name[-1]), std=0.06, sharp=3.0, fixed_routes=True)
    return name, ZOKELORN[name], {"float32": Folder(a), "bfloat16": Folder(b)}


@pytest.fixture
def model(models, request):
    name, cfg, by_dtype = models
    dtype = request.node.callspec.params.get("dtype", "float32")
    f = by_dtype[dtype]
    return name, f.folder, cfg, f


def engine(folder, dtype, **kw):
    from rocml_b200 import Engine
    kw.setdefault("max_tokens", 1024)
    return Engine.from_folder(folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype):
    """Lengths around the pages' borders (64) and around every block of positions of the four configurations (1, 37,
    64, 90, 130, 300), every place compared: the first tokens, keys just inside and just outside a block."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    eng = engine(folder, dtype)
    for n in (1, 2, 3, 37, 38, 63, 64, 65, 75, 91, 128, 129, 131, 261, 302):
        ids = prompt(n, n, cfg["vocab"])
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(n)))])
        eng.release(slot)
        assert_rows(got, plain(ids), plain.calls(ids), dtype, f"{name} {dtype} n={n}")
    eng.cache.check_invariants()


def test_a_block_one_position_off_would_show(model):
    """The weights make the softmax pick few keys: the plain implementation with every block of positions one longer,
    or one shorter, is far from itself, so the comparisons of this file would see such a fault."""
    name, folder, cfg, plain = model
    w, _ = P.load_folder(folder)
    ids = prompt(5, 200, cfg["vocab"])
    want = plain(ids)
    for off in (1, -1):
        other = json.loads(json.dumps(cfg))
        changed = False
        for L in other["layers"]:
            if L["type"] == "attention" and L["mixer"]["mask"]["size"] + off >= 1 and L["mixer"]["mask"]["size"] < 150:
                L["mixer"]["mask"]["size"] += off
                changed = True
        if not changed:
            assert name == "ZC" and off == -1          # its only attention layer has blocks of one position
            continue
        err = rel_err(P.forward(w, other, ids, torch.float64), want)
        assert err > 3 * TOL["bfloat16"], f"{name} block {off:+d}: {err}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_prompt_then_token_by_token(model, dtype, graphs):
    """The last tokens one by one (blocks of up to 130 positions begin and end under decoded tokens; pages begin and
    end; layers with blocks give pages back; the running sums go on from the prompt's state), against the same
    positions of the whole prompt."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    eng = engine(folder, dtype, use_graphs=graphs)
    for n, tail in ((150, 80), (81, 80), (290, 170)):
        ids = prompt(300 + n, n, cfg["vocab"])
        want = plain(ids)
        slot = eng.new_sequence()
        head = n - tail
        got = [eng.step([StepEntry(slot, ids[:head], [head - 1])]).clone()]
        for t in range(head, n):
            got.append(eng.step([StepEntry(slot, [ids[t]], [0])]).clone())
        eng.release(slot)
        assert_rows(torch.cat(got, dim=0), want[head - 1:], plain.calls(ids), dtype, f"{name} {dtype} n={n} graphs={graphs}",
                    first_row=head - 1)
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_very_first_token(model, dtype):
    """A sequence grown one token at a time from nothing, across page borders, blocks and the graphs' context
    buckets, every row compared."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    n = 270
    ids = prompt(9, n, cfg["vocab"])
    eng = engine(folder, dtype)
    slot = eng.new_sequence()
    got = [eng.step([StepEntry(slot, [ids[t]], [0])]).clone() for t in range(n)]
    eng.release(slot)
    assert_rows(torch.cat(got, dim=0), plain(ids), plain.calls(ids), dtype, f"{name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("piece", [2, 5, 64, 100])
def test_prompts_in_pieces(model, dtype, piece):
    """Steps cut into pieces of 2 to 100 tokens (the engine's work space is that small): two sequences side by
    side, every place wanted, then a few tokens one by one."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    eng = engine(folder, dtype, max_step_tokens=piece)
    lens = (140, 70) if piece > 2 else (67, 9)
    seqs = [prompt(700 + i, n + 4, cfg["vocab"]) for i, n in enumerate(lens)]
    slots = [eng.new_sequence() for _ in seqs]
    got = eng.step([StepEntry(s, ids[:-4], list(range(len(ids) - 4))) for s, ids in zip(slots, seqs)])
    rows, at = [], 0
    for ids in seqs:
        rows.append([got[at:at + len(ids) - 4].clone()])
        at += len(ids) - 4
    for k in range(4, 0, -1):
        out = eng.step([StepEntry(s, [ids[-k]], [0]) for s, ids in zip(slots, seqs)])
        for i in range(len(seqs)):
            rows[i].append(out[i:i + 1].clone())
    for i, ids in enumerate(seqs):
        assert_rows(torch.cat(rows[i], dim=0), plain(ids), plain.calls(ids), dtype, f"{name} {dtype} piece={piece} seq {i}")
        eng.release(slots[i])
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_against_each_alone_and_reuse(model, dtype):
    """Batches of unequal prompts, then one token each until the shorter ones end; later batches get the slots, pages
    and states that earlier ones gave back.  Every request is compared with the plain implementation of it alone, and
    in 32-bit the batched rows equal the rows of the request stepped alone in the same engine."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    eng = engine(folder, dtype, max_tokens=640)
    batches = [[(5, 8), (70, 3), (130, 12), (1, 5)], [(64, 4), (2, 9), (33, 1)], [(190, 6), (90, 2)]]
    for r, batch in enumerate(batches):
        seqs = []
        for j, (plen, ndec) in enumerate(batch):
            ids = prompt(1000 * r + j, plen + ndec, cfg["vocab"])
            seqs.append({"ids": ids, "plen": plen, "slot": eng.new_sequence(), "got": []})
        out = eng.step([StepEntry(s["slot"], s["ids"][:s["plen"]], [s["plen"] - 1]) for s in seqs])
        for i, s in enumerate(seqs):
            s["got"].append(out[i].clone())
            s["pos"] = s["plen"]
        live = list(seqs)
        while live:
            for s in [s for s in live if s["pos"] >= len(s["ids"])]:
                eng.release(s["slot"])
            live = [s for s in live if s["pos"] < len(s["ids"])]
            if not live:
                break
            out = eng.step([StepEntry(s["slot"], [s["ids"][s["pos"]]], [0]) for s in live])
            for i, s in enumerate(live):
                s["got"].append(out[i].clone())
                s["pos"] += 1
        for j, s in enumerate(seqs):
            got = torch.stack(s["got"])
            assert_rows(got, plain(s["ids"])[s["plen"] - 1:], plain.calls(s["ids"]), dtype,
                        f"{name} {dtype} batch {r} seq {j}", first_row=s["plen"] - 1)
            if dtype == "float32" and j == 2:
                slot = eng.new_sequence()
                alone = [eng.step([StepEntry(slot, s["ids"][:s["plen"]], [s["plen"] - 1])]).clone()]
                for t in range(s["plen"], len(s["ids"])):
                    alone.append(eng.step([StepEntry(slot, [s["ids"][t]], [0])]).clone())
                eng.release(slot)
                assert rel_err(got, torch.cat(alone).cpu()) < 2e-6
        eng.cache.check_invariants()
    assert eng.cache.slots.n_held == 0
    for g in eng.cache.kv_groups:
        assert g.pool.n_held == 0


def _one_layer(layer, width=64, vocab=40):
    return {"architecture": "Zokelorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [layer]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_that_must_and_must_not_be_seen(tmp_path, dtype):
    """One attention layer, no feed-forward, no rotation, blocks of 150 positions in a prompt of 460.  The weights
    are made so that one key among the block's stands out: the first 16 entries of a token's row are its 'key part',
    the next 16 its 'value part'; queries and keys compare key parts, values come from value parts.  Tokens 7 and 9
    share a key part and nothing else.  Token 7 sits at place 155 (the block from 150 to 299), token 9 at places 298
    to 301: places 298 and 299 still see place 155 (144 back, across two page borders) and mix the two tokens' values;
    places 300 and 301 start the next block and do not.  Whole, in pieces, and decoding over the edge."""
    from safetensors.torch import load_file, save_file
    from rocml_b200 import StepEntry
    from tiny_models import write_model
    cfg = _one_layer({"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 1.0,
                                                    "mask": {"size": 150}, "rot": {"base": 10000.0, "dims": 0}}, "mlp": None})
    folder = str(tmp_path / "far")
    write_model(folder, cfg, 3)
    path = folder + "/model.safetensors"
    w = load_file(path)
    g = torch.Generator().manual_seed(1)
    E = torch.zeros(40, 64)
    E[:, :16] = torch.randn(40, 16, generator=g)
    E[:, 16:32] = torch.randn(40, 16, generator=g)
    E[:, 32:] = 0.3 * torch.randn(40, 32, generator=g)
    E[9, :16] = E[7, :16]
    E[9, 16:] *= E[7, 16:].norm() / E[9, 16:].norm()       # rows of equal length: equal keys after the norm
    pick_key = torch.zeros(16, 64)
    pick_key[:, :16] = torch.eye(16)
    pick_val = torch.zeros(16, 64)
    pick_val[:, 16:32] = torch.eye(16)
    w["embed"] = E.to(torch.bfloat16)
    w["l0.norm1"] = torch.ones(64, dtype=torch.bfloat16)
    w["l0.mix.q"] = torch.cat([pick_key, pick_key]).to(torch.bfloat16)
    w["l0.mix.k"] = pick_key.to(torch.bfloat16)
    w["l0.mix.v"] = pick_val.to(torch.bfloat16)
    w["l0.mix.g"] = torch.zeros(2, 64, dtype=torch.bfloat16)
    o = torch.zeros(64, 32)
    o[32:64, :] = torch.eye(32) * 4
    w["l0.mix.o"] = o.to(torch.bfloat16)
    w["final.norm"] = torch.ones(64, dtype=torch.bfloat16)
    w["head"] = (torch.randn(40, 64, generator=g) * 0.3).to(torch.bfloat16)
    save_file(w, path)
    others = [t for t in range(40) if t not in (7, 9)]
    ids = [others[i % len(others)] for i in range(460)]
    ids[155] = 7
    for p in (298, 299, 300, 301):
        ids[p] = 9
    wf, c = P.load_folder(folder)
    want = P.forward(wf, c, ids, torch.float64)
    # the test is worth something: seeing place 155 or not moves these rows by far more than the tolerance
    other = json.loads(json.dumps(c))
    other["layers"][0]["mixer"]["mask"]["size"] = 500
    assert rel_err(P.forward(wf, other, ids, torch.float64)[300:302], want[300:302]) > 0.2
    other["layers"][0]["mixer"]["mask"]["size"] = 140
    assert rel_err(P.forward(wf, other, ids, torch.float64)[298:300], want[298:300]) > 0.2
    tol = TOL[dtype]
    eng = engine(folder, dtype)
    slot = eng.new_sequence()
    got = eng.step([StepEntry(slot, ids, list(range(460)))])
    eng.release(slot)
    assert rel_err(got, want) < tol
    eng = engine(folder, dtype, max_step_tokens=100)        # pieces: 298 to 301 lie in two pieces, 155 in another
    slot = eng.new_sequence()
    got = eng.step([StepEntry(slot, ids, list(range(460)))])
    eng.release(slot)
    assert rel_err(got, want) < tol
    for graphs in (False, True):
        eng = engine(folder, dtype, use_graphs=graphs)
        slot = eng.new_sequence()
        eng.step([StepEntry(slot, ids[:290], [])])
        rows = [eng.step([StepEntry(slot, [ids[t]], [0])]).clone() for t in range(290, 310)]
        eng.release(slot)
        assert rel_err(torch.cat(rows), want[290:310]) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["lightning", "retention"])
def test_a_running_sum_remembers_one_token_hundreds_back(tmp_path, dtype, kind):
    """One linear-attention layer with a decay of 1 on its first head and 0.9 on its second.  Only the first head can
    still see what the tokens 120 and more places back wrote into the state; other tokens there move the last rows by
    far more than the tolerance, so a state that is lost, zeroed or mixed up between steps or slots shows.  Whole,
    in pieces, decoding, and in a slot that another sequence used before."""
    from rocml_b200 import StepEntry
    from tiny_models import write_model
    cfg = _one_layer({"type": kind, "mixer": {"heads": 2, "dim": 16, "vdim": 16, "decay": [1.0, 0.9]}, "mlp": None})
    folder = str(tmp_path / kind)
    write_model(folder, cfg, 8, std=0.3)
    wf, c = P.load_folder(folder)
    ids = prompt(2, 430, 40)
    want = P.forward(wf, c, ids, torch.float64)
    swapped = [(t + 1) % 40 for t in ids[:300]] + ids[300:]
    assert rel_err(P.forward(wf, c, swapped, torch.float64)[420:], want[420:]) > 3 * TOL["bfloat16"]
    tol = TOL[dtype]
    eng = engine(folder, dtype, max_step_tokens=128)
    slot = eng.new_sequence()
    got = eng.step([StepEntry(slot, ids, list(range(430)))])
    assert rel_err(got, want) < tol
    eng.release(slot)
    again = eng.new_sequence()
    assert again == slot                                   # the same slot, whose state must start from zero again
    eng.step([StepEntry(again, ids[:300], [])])
    rows = [eng.step([StepEntry(again, [ids[t]], [0])]).clone() for t in range(300, 430)]
    eng.release(again)
    assert rel_err(torch.cat(rows), want[300:]) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(model, dtype):
    """Engine.generate (its scheduler, sampler and run-ahead loop) against greedy decoding with the plain
    implementation, for prompts of unequal length in one batch; compared until the first step whose two best logits
    are closer than the tolerance."""
    from rocml_b200 import SamplingParams
    name, folder, cfg, plain = model
    eng = engine(folder, dtype)
    prompts = [prompt(50 + i, n, cfg["vocab"]) for i, n in enumerate((3, 70, 35))]
    outs = eng.generate(prompts, max_new_tokens=12, sampling=SamplingParams(temperature=0.0), ignore_eos=True)
    for ids, out in zip(prompts, outs):
        seq = list(ids)
        for tok in out.tokens:
            logits = P.forward(plain.w, plain.cfg, seq, torch.float64)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 5 * TOL[dtype] * float(logits.abs().max()):
                break
            assert tok == int(logits.argmax()), f"{name} {dtype}: after {len(seq)} tokens"
            seq.append(tok)
    assert eng.cache.slots.n_held == 0


def test_trace_replay_and_command_line(models, tmp_path):
    """bin/trace_run on a folder of this architecture: a prompt in two steps and two decoded tokens, a second request
    beside it; the logits are the plain implementation's."""
    import io
    import os
    import subprocess
    import sys
    import numpy as np
    name, cfg, by_dtype = models
    f = by_dtype["float32"]
    a, b = prompt(1, 40, cfg["vocab"]), prompt(2, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:38], "want": [0, 37]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[38:39], "want": [0]}, {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[39:], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["a", "b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", f.folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = f(a), f(b)
    V = cfg["vocab"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got0, torch.stack([wa[0], wa[37], wb[6]])) < TOL["float32"]
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got1, wa[38:39]) < TOL["float32"]
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(got2, torch.stack([wa[39], wb[8]])) < TOL["float32"]
    r = subprocess.run([sys.executable, "-m", "rocml_b200", "generate", "--model", f.folder, "--prompt-ids", "1,2,3", "-n", "5"],
                       capture_output=True, text=True, timeout=600, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]


# ---- configurations drawn at random -----------------------------------------------------------------------------

def random_configuration(seed):
    """A Zokelorn configuration whose every size, option and constant is drawn from a seed (sizes stay small)."""
    import random
    r = random.Random(seed)
    width = r.choice([48, 64, 72, 96, 128, 160, 256])
    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice(["attention", "lightning", "retention"])
        if kind == "attention":
            heads = r.choice([1, 2, 3, 4, 6, 8, 12])
            kv = r.choice([g for g in (1, 2, 3, 4, 6, 8, 12) if heads % g == 0])
            dim = r.choice([8, 16, 24, 32, 40, 64, 96, 128])
            rot = {"base": r.choice([100.0, 10000.0, 1e6]), "dims": r.choice([0, 2, dim // 2 // 2 * 2, dim])}
            if r.random() < 0.6:
                low = r.choice([0.5, 1.0, 2.0])
                rot["scaling"] = {"factor": r.choice([2.0, 8.0, 32.0]), "low": low, "high": low * r.choice([2.0, 4.0]),
                                  "original": r.choice([16, 64, 1024, 8192])}
            mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": r.choice([8, 16, 24, 32, 40, 64, 96, 128]),
                     "scale": r.uniform(0.05, 0.4), "mask": {"size": r.choice([1, 2, 7, 31, 64, 65, 100, 128, 200, 1000])}, "rot": rot}
        else:
            heads = r.randint(1, 6)
            mixer = {"heads": heads, "dim": r.choice([4, 8, 16, 20, 32, 64, 72, 128, 136]), "vdim": r.choice([4, 8, 12, 32, 64, 96, 128, 160]),
                     "decay": [r.choice([0.0, 1.0, r.uniform(0.3, 0.9), 1.0 - 2.0 ** -r.randint(3, 10)]) for _ in range(heads)]}
        u = r.random()
        if u < 0.1:
            mlp = None
        elif u < 0.5:
            mlp = {"kind": "dense", "ff": 4 * r.randint(2, 50)}
        else:
            experts = r.choice([1, 2, 4, 6, 8, 12, 16, 24])
            groups = r.choice([g for g in (1, 2, 3, 4, 6, 8) if experts % g == 0])
            keep = r.randint(1, groups)
            top = r.randint(1, min(6, keep * (experts // groups)))
            router = {"experts": experts, "top": top}
            if groups > 1 or r.random() < 0.3:
                router["groups"] = {"count": groups, "keep": keep}
            mlp = {"kind": "moe", "expert": {"ff": 4 * r.randint(1, 16)}, "router": router}
            if r.random() < 0.6:
                mlp["shared"] = {"ff": 4 * r.randint(1, 24)}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Zokelorn", "vocab": r.randint(40, 700), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])},
           "layers": layers}
    if r.random() < 0.6:
        a = r.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": a, "stop": r.randint(a + 1, len(layers)), "times": r.randint(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Ten configurations whose sizes, options and constants come from a seed: in 32-bit a whole prompt, the same prompt
    as a first piece and single tokens, and two unequal requests side by side, against the plain implementation; in
    bfloat16 the whole prompt, loosely (it must run and stay near)."""
    from rocml_b200 import StepEntry
    cfg = random_configuration(seed)
    folder = str(tmp_path / "m")
    write_zokelorn(folder, cfg, seed=seed, std=0.06, sharp=2.0)
    plain = Folder(folder)
    n = 150
    ids = prompt(seed, n, cfg["vocab"])
    other = prompt(seed + 100, 70, cfg["vocab"])
    want, calls = plain(ids), plain.calls(ids)
    eng = engine(folder, "float32")
    slot = eng.new_sequence()
    got = eng.step([StepEntry(slot, ids, list(range(n)))])
    eng.release(slot)
    assert_rows(got, want, calls, "float32", f"seed {seed} whole")
    a, b = eng.new_sequence(), eng.new_sequence()
    out = eng.step([StepEntry(a, ids[:97], [96]), StepEntry(b, other[:66], list(range(66)))])
    rows_a, rows_b = [out[:1].clone()], [out[1:].clone()]
    for t in range(97, n):
        entries = [StepEntry(a, [ids[t]], [0])] + ([StepEntry(b, [other[t - 97 + 66]], [0])] if t - 97 + 66 < 70 else [])
        out = eng.step(entries)
        rows_a.append(out[:1].clone())
        if len(entries) > 1:
            rows_b.append(out[1:2].clone())
        elif t - 97 + 66 == 70:
            eng.release(b)
    eng.release(a)
    assert_rows(torch.cat(rows_a), want[96:], calls, "float32", f"seed {seed} decoded", first_row=96)
    assert_rows(torch.cat(rows_b), plain(other), plain.calls(other), "float32", f"seed {seed} second request")
    eng.cache.check_invariants()
    eng = engine(folder, "bfloat16")
    slot = eng.new_sequence()
    got = eng.step([StepEntry(slot, ids, list(range(n)))]).double().cpu()
    eng.release(slot)
    assert bool(torch.isfinite(got).all())
    near = torch.nonzero(calls < CLOSE["bfloat16"])[:, 0]
    upto = n if not len(near) else int(near[0])
    if upto >= 20:
        err = (got[:upto] - want[:upto]).abs().amax(-1) / want[:upto].abs().amax(-1)
        assert float(err.median()) < TOL["bfloat16"], f"seed {seed} bfloat16: median {float(err.median()):.3g}"
