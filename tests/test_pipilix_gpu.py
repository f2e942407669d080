"""Pipilix on the GPU against the plain implementation (tests/plain_pipilix.py): each mechanism alone, then
the engine in every way of cutting and batching, in 32-bit and in bfloat16.

Tolerances are a fraction of the largest |logit| of the row compared.  float32: sums of a few hundred terms
in another order than the plain implementation's float64.  bfloat16: activations are rounded to 8 bits of
mantissa between kernels, a dozen roundings a layer run.
"""
import json

import pytest
import torch

import plain_pipilix as P
from tiny_models import PIPILIX, prompt, write_pipilix

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-5, "bfloat16": 3e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel_err(got, want):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


# A router's choice between two experts whose scores differ by less than rounding can fall either way, and the
# token's logits then differ by much more than rounding.  The plain implementation reports, per token, the smallest
# margin of any of its routers' choices; rows below these margins are excused (and must be few).
CLOSE = {"float32": 2e-5, "bfloat16": 1e-2}


def assert_rows(got, want, calls, dtype, what):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    scale = want.abs().amax(dim=-1).clamp_min(1e-30)
    err = (got - want).abs().amax(dim=-1) / scale
    excused = calls < CLOSE[dtype]
    bad = (err >= TOL[dtype]) & ~excused
    assert not bool(bad.any()), f"{what}: rows {torch.nonzero(bad)[:, 0].tolist()[:8]} off by up to {float(err[bad].max()):.3g}"
    assert int(excused.sum()) <= max(2, 0.3 * len(err)), f"{what}: {int(excused.sum())} of {len(err)} rows are near ties"
    assert bool(torch.isfinite(got).all()), what


def close(got, want, tol):
    want = want.double()
    got = got.double().cpu()
    return float((got - want).abs().max()) <= tol * max(1e-30, float(want.abs().max()))


# ---- each mechanism alone -------------------------------------------------------------------------------------

def test_embedding_with_multiplier_and_sinusoid():
    from rocml_b200 import kernels
    from rocml_b200.config.specs import PositionSpec
    from rocml_b200.parts import BuildEnv, build_position
    dev = torch.device("cuda:0")
    for width in (10, 64, 257):
        table = torch.randn(50, width).to(torch.bfloat16)
        ids = torch.tensor([3, 49, 0, 3, 7], dtype=torch.int32)
        pos = torch.tensor([0, 1, 900, 12345, 65], dtype=torch.int32)
        enc = build_position(PositionSpec("sinusoid", theta=10000.0), width, BuildEnv(dev, torch.bfloat16))
        out = torch.empty((5, width), dtype=torch.float32, device=dev)
        copy = torch.empty_like(out)
        kernels.embedding_pos(ids.to(dev), table.to(dev), out, 2.5, pos.to(dev), enc.inv_freq, copy=copy)
        want = table.double()[ids.long()] * 2.5 + P.sinusoid(pos.tolist(), width, torch.float64)
        # a 32-bit angle of 12345 radians is off by up to 12345 * 2^-24
        assert float((out.double().cpu() - want).abs().max()) < 2e-3
        assert float((out[:3].double().cpu() - want[:3]).abs().max()) < 1e-4
        assert torch.equal(out, copy)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width, parts", [(72, 1), (256, 3), (1000, 8)])
def test_norm_after_a_sublayer_then_add_then_norm(dtype, width, parts):
    from rocml_b200 import kernels
    dev = torch.device("cuda:0")
    torch.manual_seed(width + parts)
    T = 9
    wdt = DT[dtype]
    resid = torch.randn(T, width) * 3
    delta = torch.randn(parts, T, width) * 5
    w1 = (torch.rand(width) + 0.5).to(wdt)
    w2 = (torch.rand(width) + 0.5).to(wdt)
    r = resid.to(dev)
    out = torch.empty((T, width), dtype=wdt, device=dev)
    kernels.postnorm_add_norm(r, delta.to(dev), w1.to(dev), 1e-5, w2.to(dev), 2e-6, out)
    d = delta.double().sum(0)
    want_r = resid.double() + P.norm(d, w1.double(), 1e-5)
    want_o = P.norm(want_r, w2.double(), 2e-6)
    assert close(r, want_r, 1e-6)
    assert close(out, want_o, 1e-6 if dtype == "float32" else 1e-2)
    r2 = resid.to(dev)
    kernels.postnorm_add_norm(r2, delta.to(dev), w1.to(dev), 1e-5)      # the last sublayer of a layer: no norm follows
    assert torch.equal(r2, r)


def test_additions_between_layers():
    from rocml_b200 import kernels
    dev = torch.device("cuda:0")
    T, H = 5, 24
    resid, other, delta = torch.randn(T, H), torch.randn(T, H), torch.randn(2, T, H)
    vec = torch.randn(H).to(torch.bfloat16)
    r = resid.to(dev)
    kernels.residual_inject(r, delta.to(dev), other.to(dev), vec.to(dev))
    assert close(r, resid.double() + delta.double().sum(0) + other.double() + vec.double(), 1e-6)
    r = resid.to(dev)
    kernels.residual_inject(r, None, None, vec.float().to(dev))
    assert close(r, resid.double() + vec.double(), 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("G, N, K, T", [(3, 20, 12, 7), (4, 32, 16, 16), (7, 88, 48, 70), (2, 40, 24, 200), (5, 8, 36, 33)])
def test_products_head_by_head(dtype, G, N, K, T):
    """Both row tiles, the tensor-core and the FMA kernel (sizes off 8 take the latter), strided rows, a gate a row."""
    from rocml_b200 import kernels
    dev = torch.device("cuda:0")
    torch.manual_seed(G * N + K)
    dt = DT[dtype]
    wide = torch.randn(T, G * K + 8).to(dt)
    x = wide[:, :G * K]
    w = torch.randn(G, N, K).to(dt)
    gate = torch.rand(T, G)
    out = torch.full((T, G * N), 7.0, dtype=dt, device=dev)
    kernels.head_matmul(wide.to(dev)[:, :G * K], w.to(dev), out, T, row_scale=gate.to(dev))
    want = torch.einsum("tgk,gnk->tgn", x.double().reshape(T, G, K), w.double()) * gate.double()[:, :, None]
    assert close(out, want.reshape(T, G * N), 1e-6 if dtype == "float32" else 1e-2)
    out32 = torch.empty((T, G * N), dtype=torch.float32, device=dev)
    kernels.head_matmul(wide.to(dev)[:, :G * K], w.to(dev), out32, T)
    want = torch.einsum("tgk,gnk->tgn", x.double().reshape(T, G, K), w.double())
    assert close(out32, want.reshape(T, G * N), 1e-6)      # bfloat16 operands are exact in 32-bit sums


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, E, K", [(1, 3, 20), (8, 32, 256), (13, 7, 72), (70, 64, 1024), (5, 9, 5000)])
def test_router_logits_are_32_bit(dtype, T, E, K):
    from rocml_b200 import kernels
    dev = torch.device("cuda:0")
    torch.manual_seed(T + E + K)
    x = torch.randn(T + 2, K + 3).to(DT[dtype])[:, :K]            # rows with a stride of their own
    w = torch.randn(E, K)
    z = torch.full((T, E), 9.0, dtype=torch.float32, device=dev)
    kernels.router_logits(x.to(dev), w.to(dev), z, T)
    assert close(z, x[:T].double() @ w.double().t(), 2e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_norm_into_the_cache_and_gates(dtype):
    from rocml_b200 import kernels
    dev = torch.device("cuda:0")
    torch.manual_seed(5)
    dt = DT[dtype]
    T, qw, rank, H = 6, 24, 20, 3
    proj = torch.randn(2, T, qw + rank + H + 1)          # two partial sums, one column of padding
    w = (torch.rand(rank) + 0.5).to(dt)
    cache = torch.zeros((4, 1, 64, rank), dtype=dt, device=dev)
    table = torch.tensor([[2, 0, -1], [3, 1, -1]], dtype=torch.int32, device=dev)
    positions = torch.tensor([0, 63, 64, 5, 70, 9], dtype=torch.int32, device=dev)
    slots = torch.tensor([0, 0, 0, 1, 1, -1], dtype=torch.int32, device=dev)
    q = torch.empty((T, qw), dtype=dt, device=dev)
    gates = torch.zeros((T, H), dtype=torch.float32, device=dev)
    kernels.latent_prep(proj.to(dev), T, qw, rank, H, w.to(dev), 1e-5, q, gates, cache, positions, slots, table)
    full = proj.double().sum(0)
    c = P.norm(full[:, qw:qw + rank], w.double(), 1e-5)
    tol = 1e-6 if dtype == "float32" else 1e-2
    where = [(2, 0), (2, 63), (0, 0), (3, 5), (1, 6)]
    for t, (page, off) in enumerate(where):
        assert close(cache[page, 0, off], c[t], tol), t
    assert int((cache.float().abs().sum(-1) > 0).sum()) == 5          # the padding token wrote nothing
    assert close(q[:5], full[:5, :qw], tol)
    assert close(gates[:5], torch.sigmoid(full[:5, qw + rank:qw + rank + H]), 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, E, top, D, F", [(5, 3, 3, 24, 20), (40, 7, 2, 64, 48), (300, 16, 1, 32, 16), (130, 5, 4, 40, 12),
                                             (300, 16, 4, 128, 64), (600, 4, 2, 256, 160), (1100, 9, 1, 72, 48)])
def test_routed_feed_forward_alone(dtype, T, E, top, D, F):
    """The routed part by itself: choices, weights and the weighted sum of the chosen experts; padding tokens
    (slot -1) get zeros.  Row tiles of 16, 64 and (the last three cases in bfloat16) 128 on the tcgen05 product,
    with feature tiles of 128 and 256, an expert without rows, and sizes that are no multiple of a tile."""
    from rocml_b200.config.specs import FeedForwardSpec
    from rocml_b200.parts import BuildEnv, build_feed_forward
    dev = torch.device("cuda:0")
    torch.manual_seed(T + E)
    dt = DT[dtype]
    spec = FeedForwardSpec.make("routed_mlp", experts=E, top=top, intermediate=F, activation="clamped_swish", limit=0.6,
                                alpha=1.702, choice_bias=True,
                                names={"router": "router", "choice_bias": "correction", "expert": "e{e}.", "gate": "gate",
                                       "up": "up", "down": "down"})
    part = build_feed_forward(spec, D, BuildEnv(dev, dt))
    w = {"router": torch.randn(E, D), "correction": torch.randn(E)}
    for e in range(E):
        w.update({f"e{e}.gate": torch.randn(F, D) * 0.3, f"e{e}.up": torch.randn(F, D) * 0.3, f"e{e}.down": torch.randn(D, F) * 0.3})
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    assert sorted(d.name for d in part.declare("")) == sorted(k + ".weight" for k in w)
    part.load({k + ".weight": v.to(dev).to(dt) for k, v in w.items()}, "")
    x = torch.randn(T, D).to(dt)

    class Batch:
        n_tokens = T
        slot_of_token = torch.zeros(T, dtype=torch.int32, device=dev)
    Batch.slot_of_token[T - 1] = -1
    got = part.forward(x.to(dev), Batch)[0]
    wd = {k: v.double() for k, v in w.items()}
    want = P.routed_ff(x.double(), wd, "", E, top, 0.6)
    assert float(got[T - 1].abs().max()) == 0.0
    # rows whose choice is a near tie (in the plain implementation's own scores) may be routed otherwise
    decided = torch.ones(T, dtype=torch.bool)
    if top < E:
        best = torch.topk(torch.sigmoid(x.double() @ wd["router"].t()) + wd["correction"], top + 1, dim=-1).values
        decided = (best[:, top - 1] - best[:, top]) > (1e-5 if dtype == "float32" else 1e-2)
    decided[T - 1] = False
    assert int(decided.sum()) >= 0.8 * (T - 1)
    assert close(got[decided], want[decided], 2e-6 if dtype == "float32" else 2e-2)


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


@pytest.fixture(scope="module", params=sorted(PIPILIX))
def models(request, tmp_path_factory):
    """Two folders a configuration.  In the first the routers' choices follow the tokens; the 32-bit runs use it.
    A choice between two scores that differ by less than bfloat16's rounding falls either way, moves that token's
    logits by far more than rounding, and through the attention every later token's: over hundreds of tokens some
    choice is always that close.  The bfloat16 runs therefore use a second folder whose choice biases lie far apart,
    so that every choice rests on them (the routed part's own bfloat16 test keeps choices that follow the tokens)."""
    name = request.param
    a = str(tmp_path_factory.mktemp(f"pipilix_{name}"))
    b = str(tmp_path_factory.mktemp(f"pipilix_{name}_fixed"))
    write_pipilix(a, PIPILIX[name], seed=40 + ord(name[-1]), std=0.06, sharp=3.0)
    write_pipilix(b, PIPILIX[name], seed=40 + ord(name[-1]), std=0.06, sharp=3.0, bias_std=40.0)
    return name, PIPILIX[name], {"float32": Folder(a), "bfloat16": Folder(b)}


@pytest.fixture
def model(models, request):
    """(name, folder, configuration, plain implementation) for the test's ``dtype`` (32-bit where it has none)."""
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
    """Lengths around the pages' borders (64) and around every window of the three configurations (1, 9, 17, 33, 64,
    70, 100, 200, 300), every place compared: the first tokens, keys just inside and just outside a window."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    eng = engine(folder, dtype)
    for n in (1, 2, 9, 10, 18, 34, 63, 64, 65, 71, 101, 128, 129, 201, 310):
        ids = prompt(n, n, cfg["vocab"])
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(n)))])
        eng.release(slot)
        assert_rows(got, plain(ids), plain.calls(ids), dtype, f"{name} {dtype} n={n}")
    eng.cache.check_invariants()


def test_a_window_one_token_off_would_show(model):
    """The weights make the softmax pick few keys: the plain implementation with every window one token longer, or
    one shorter, is far from itself, so the comparisons of this file would see such a fault."""
    name, folder, cfg, plain = model
    w, _ = P.load_folder(folder)
    ids = prompt(5, 200, cfg["vocab"])
    want = plain(ids)
    for off in (1, -1):
        other = json.loads(json.dumps(cfg))
        changed = False
        for L in other["layers"]:
            if L["mixer"]["mask"]["size"] + off >= 1 and L["mixer"]["mask"]["size"] < 150:
                L["mixer"]["mask"]["size"] += off
                changed = True
        assert changed
        err = rel_err(P.forward(w, other, ids, torch.float64), want)
        assert err > 3 * TOL["bfloat16"], f"{name} window {off:+d}: {err}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_prompt_then_token_by_token(model, dtype, graphs):
    """The last 80 tokens one by one (windows of up to 70 tokens pass wholly over decoded tokens; pages begin and
    end; windowed layers give pages back), against the same positions of the whole prompt."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    eng = engine(folder, dtype, use_graphs=graphs)
    for n, tail in ((150, 80), (81, 80), (260, 40)):
        ids = prompt(300 + n, n, cfg["vocab"])
        want = plain(ids)
        slot = eng.new_sequence()
        head = n - tail
        got = [eng.step([StepEntry(slot, ids[:head], [head - 1])]).clone()]
        for t in range(head, n):
            got.append(eng.step([StepEntry(slot, [ids[t]], [0])]).clone())
        eng.release(slot)
        assert_rows(torch.cat(got, dim=0), want[head - 1:], plain.calls(ids)[head - 1:], dtype, f"{name} {dtype} n={n} graphs={graphs}")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_very_first_token(model, dtype):
    """A sequence grown one token at a time from nothing, across two page borders and the graphs' context
    buckets, every row compared."""
    from rocml_b200 import StepEntry
    name, folder, cfg, plain = model
    n = 140
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
    lens = (131, 70) if piece > 2 else (67, 9)
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
    """Batches of unequal prompts, then one token each until the shorter ones end; later batches get the slots and
    pages that earlier ones gave back.  Every request is compared with the plain implementation of it alone, and
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
            assert_rows(got, plain(s["ids"])[s["plen"] - 1:], plain.calls(s["ids"])[s["plen"] - 1:], dtype,
                        f"{name} {dtype} batch {r} seq {j}")
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_that_must_and_must_not_be_seen(tmp_path, dtype):
    """One layer, no feed-forward, a window of 150 tokens in a prompt of 400.  The weights are made so that one key
    among the 150 stands out: the first 16 dimensions of a token's row are its 'key part', the next 16 its 'value
    part'; the latent keeps both, queries and keys compare key parts, values come from value parts.  Tokens 7 and 9
    share a key part and nothing else.  Token 7 sits at place 200, token 9 at places 349 to 351: place 349 still sees
    place 200 (149 back, across two page borders) and mixes the two tokens' values; place 350 does not.  The engine
    agrees with the plain implementation at both, in a prompt's piece and decoding, and the plain implementation
    shows that the far key moves place 349 a lot and place 350 not at all."""
    from rocml_b200 import StepEntry
    from safetensors.torch import load_file, save_file
    D, R, dim = 48, 32, 16
    cfg = {"architecture": "Pipilix", "vocab": 64, "width": D, "embedding": {"scale": 300.0}, "norm": {"eps": 1e-6},
           "logit_scale": 1.0,
           "layers": [{"type": "latent_attention",
                       "mixer": {"heads": 2, "dim": dim, "vdim": 16, "kv_rank": R, "scale": 1.0, "mask": {"size": 150}},
                       "mlp": None}]}
    folder = write_pipilix(str(tmp_path / "far"), cfg, seed=8, std=0.1)
    path = folder + "/model.safetensors"
    w = load_file(path)
    eye = torch.eye(dim)
    down = torch.zeros(R, D)
    down[:, :R] = torch.eye(R)                                   # the latent: key part, then value part
    w["l0.mix.dkv"] = down.to(torch.bfloat16)
    w["l0.mix.dkv.norm"] = torch.ones(R).to(torch.bfloat16)
    w["l0.norm1"] = torch.ones(D).to(torch.bfloat16)
    w["l0.mix.q"] = torch.cat([torch.cat([eye, torch.zeros(dim, D - dim)], dim=1)] * 2).to(torch.bfloat16)
    w["l0.mix.uk"] = torch.cat([torch.cat([eye, torch.zeros(dim, R - dim)], dim=1)] * 2).to(torch.bfloat16)
    w["l0.mix.uv"] = torch.cat([torch.cat([torch.zeros(16, R - 16), torch.eye(16)], dim=1)] * 2).to(torch.bfloat16)
    w["l0.norm1b"] = torch.full((D,), 100.0).to(torch.bfloat16)        # the mixer's result outweighs the stream it joins
    w["embed"][9, :dim] = w["embed"][7, :dim]
    save_file(w, path)
    w, cfg = P.load_folder(folder)
    ids = [t if t not in (7, 9) else 8 for t in prompt(3, 400, 64)]
    ids[200] = 7
    ids[349] = ids[350] = ids[351] = 9
    want = P.forward(w, cfg, ids, torch.float64)
    without = list(ids)
    without[200] = 8
    blind = P.forward(w, cfg, without, torch.float64)
    assert rel_err(blind[349:350], want[349:350]) > 0.1                   # seen: the far token matters
    assert rel_err(blind[350:], want[350:]) < 1e-9                        # out of the window: it cannot
    places = [200, 201, 263, 264, 320, 349, 350, 351, 399]
    eng = engine(folder, dtype)
    for cut in (340, 352):                                               # the three places decoded alone, or in the prompt
        slot = eng.new_sequence()
        got = [eng.step([StepEntry(slot, ids[:cut], [p for p in places if p < cut])]).clone()]
        for t in range(cut, 400):
            out = eng.step([StepEntry(slot, [ids[t]], [0] if t in places else [])])
            if out is not None:
                got.append(out.clone())
        eng.release(slot)
        assert rel_err(torch.cat(got), want[places]) < TOL[dtype], cut


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_latent_wider_than_the_tensor_core_kernels_take(tmp_path, dtype):
    """A latent of 320 numbers (the plain attention kernel's wide variant), a prompt across a page border and a
    window's edge, then six tokens one by one."""
    from rocml_b200 import StepEntry
    cfg = {"architecture": "Pipilix", "vocab": 80, "width": 96, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
           "logit_scale": 1.0,
           "layers": [{"type": "latent_attention",
                       "mixer": {"heads": 2, "dim": 24, "vdim": 16, "kv_rank": 320, "scale": 0.2, "mask": {"size": 40}},
                       "mlp": {"kind": "dense", "ff": 64}}]}
    folder = write_pipilix(str(tmp_path / "wide"), cfg, seed=12, std=0.06, sharp=2.0)
    f = Folder(folder)
    ids = prompt(21, 106, 80)
    eng = engine(folder, dtype)
    slot = eng.new_sequence()
    got = [eng.step([StepEntry(slot, ids[:100], list(range(100)))]).clone()]
    got += [eng.step([StepEntry(slot, [ids[t]], [0])]).clone() for t in range(100, 106)]
    eng.release(slot)
    assert_rows(torch.cat(got), f(ids), f.calls(ids), dtype, f"latent 320 {dtype}")


def test_greedy_generation_through_the_entry_point(model):
    """Engine.generate (the loop, the scheduler of batches, the GPU sampler) in 32-bit gives the plain
    implementation's greedy tokens; more requests than a batch holds, so slots are used again."""
    name, folder, cfg, plain = model
    eng = engine(folder, "float32", max_tokens=64 * 12, max_slots=3)
    prompts = [prompt(50 + i, n, cfg["vocab"]) for i, n in enumerate([5, 11, 70, 1, 40])]
    outs = eng.generate(prompts, max_new_tokens=6, stop_tokens=[], max_batch=3)
    for p, o in zip(prompts, outs):
        ids = list(p)
        for t in o.tokens:
            logits = plain(ids)[-1]
            best = int(torch.argmax(logits))
            if t != best:                     # only where the two best logits nearly tie
                top2 = torch.topk(logits, 2).values
                assert float(top2[0] - logits[t]) < 1e-4 * float(top2[0].abs()), f"{name}: {t} instead of {best}"
            ids.append(t)
        assert len(o.tokens) == 6 and o.finish_reason == "length"
    eng.cache.check_invariants()
    assert eng.cache.slots.n_held == 0


def test_trace_replay_writes_what_the_step_returns(model, tmp_path):
    """bin/trace_run on a Pipilix folder: a batch of two unequal requests, then one token each, one ending early."""
    import os
    import subprocess
    import sys
    import numpy as np
    name, folder, cfg, plain = model
    a, b = prompt(1, 40, cfg["vocab"]), prompt(2, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[37:38], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[38:39], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[39:40], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out, "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not os.path.exists(os.path.join(out, "2.f32"))
    V = cfg["vocab"]
    got0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(-1, V))
    want0 = torch.stack([plain(a)[0], plain(a)[36], plain(b)[7]])
    assert rel_err(got0, want0) < TOL["float32"]
    got3 = torch.from_numpy(np.fromfile(os.path.join(out, "3.f32"), dtype="<f4").reshape(-1, V))
    assert rel_err(got3, plain(a)[39:40]) < TOL["float32"]


def test_the_command_line_generates_and_profiles(models):
    """`python -m rocml_b200 generate` on a Pipilix folder: greedy tokens equal the plain implementation's (32-bit),
    and --profile lists the design's own kernels."""
    import os
    import subprocess
    import sys
    name, cfg, by_dtype = models
    f = by_dtype["float32"]
    ids = prompt(12, 9, cfg["vocab"])
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "rocml_b200", "generate", "--model", f.folder, "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, ids)), "-n", "5", "-t", "0", "--profile"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    toks = [int(x) for x in p.stdout.split("limits (")[0].split()]
    seq = list(ids)
    for t in toks:
        logits = f(seq)[-1]
        best = int(torch.argmax(logits))
        if t != best:
            top2 = torch.topk(logits, 2).values
            assert float(top2[0] - logits[t]) < 1e-4 * float(top2[0].abs())
        seq.append(t)
    assert len(toks) == 5
    for label in ("latent_norm_cache", "fold_queries", "unfold_values", "mixer_post_norm", "q+dkv"):
        assert label in p.stdout, label
    if any(L["mlp"] and L["mlp"]["kind"] == "moe" for L in cfg["layers"]):
        assert "router" in p.stdout and "experts_gate_up" in p.stdout
