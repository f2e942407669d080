"""Zokelorn without a GPU: the configuration, the parts it is spelled as, the tensors it declares, the cache it
asks for, and the plain implementation's own mechanisms."""
import json

import pytest
import torch

import plain_zokelorn as P
from tiny_models import ZOKELORN


def spec_of(cfg):
    from rocml_b200.config import config_from_dict
    return config_from_dict(cfg).to_model_spec()


@pytest.mark.parametrize("name", sorted(ZOKELORN))
def test_config_round_trip(name):
    from rocml_b200.config import ZokelornConfig, config_from_dict
    cfg = config_from_dict(ZOKELORN[name])
    assert isinstance(cfg, ZokelornConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert len(cfg.layers) == len(ZOKELORN[name]["layers"])


@pytest.mark.parametrize("broken, needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "type"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 5), "groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5, 0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("decay", [0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["loop"].__setitem__("stop", 7), "loop"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_named(broken, needle):
    from rocml_b200.config import config_from_dict
    from rocml_b200.errors import ConfigError
    cfg = json.loads(json.dumps(ZOKELORN["ZA"]))
    broken(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert needle in str(e.value)


def test_schedule_follows_the_loop_and_every_run_has_a_cache_of_its_own():
    from rocml_b200.cache.requirements import KVRequirement, StateRequirement
    from rocml_b200.engine.model import Model
    from rocml_b200.parts import BuildEnv
    spec = spec_of(ZOKELORN["ZA"])
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 1, 0, 1, 2]
    assert all(e.reads_cache_of is None and not e.add_input and e.add_row is None for e in spec.schedule)
    assert [e.layer for e in spec_of(ZOKELORN["ZB"]).schedule] == [0, 1, 2, 3]
    assert [e.layer for e in spec_of(ZOKELORN["ZD"]).schedule] == [0, 1, 2, 1, 2]
    model = Model(spec, BuildEnv(torch.device("cpu"), torch.bfloat16))
    reqs = model.cache_requirements()
    assert [type(r) for r in reqs] == [StateRequirement, KVRequirement] * 3 + [StateRequirement]
    assert reqs[0].shape == (3, 16, 24) and reqs[0].dtype == torch.float32
    assert reqs[1] == KVRequirement(2, 32, None, chunk=37)         # heads of 32 and 16 share pages 32 wide
    assert reqs[6].shape == (2, 24, 8)


def test_layers_are_spelled_as_parts_with_the_designs_constants():
    spec = spec_of(ZOKELORN["ZA"])
    light, attn, ret = (spec.layers[i] for i in range(3))
    assert {l.arrangement for l in spec.layers} == {"parallel"}
    p = light.mixer.params
    assert light.mixer.kind == "linear_attention" and p["qk_activation"] == "silu" and p["v_activation"] == "silu"
    assert p["out_norm"] == "all_heads" and p["out_norm_weight"] and p["gate_activation"] == "sigmoid" and p["k_scale"] == 1.0
    p = ret.mixer.params
    assert p["qk_activation"] == "none" and p["out_norm"] == "per_head" and not p["out_norm_weight"]
    assert p["gate_activation"] == "silu" and abs(p["k_scale"] - 24 ** -0.5) < 1e-15 and ret.feed_forward is None
    p = attn.mixer.params
    assert attn.mixer.kind == "attention" and p["chunk"] == 37 and p["gated"] and p["v_head_dim"] == 16 and p["scale"] == 0.3
    assert attn.mixer.position.kind == "rope_pairs" and attn.mixer.position.rot_dim == 16
    assert dict(attn.mixer.position.params["scaling"]) == {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 64.0}
    f = attn.feed_forward.params
    assert attn.feed_forward.kind == "routed_mlp" and f["groups"] == 3 and f["keep_groups"] == 2 and f["renormalize"]
    assert f["renormalize_eps"] == 1e-20 and f["shared"] == 40 and f["shared_gate"] and f["activation"] == "silu"
    assert light.feed_forward.params["activation"] == "gelu_tanh"
    # no rotation at all, no groups, no shared expert
    d = spec_of(ZOKELORN["ZD"])
    assert d.layers[0].mixer.position.kind == "none"
    b = spec_of(ZOKELORN["ZB"]).layers[0].feed_forward.params
    assert b["groups"] == 1 and not b["shared"] and not b["shared_gate"]


def test_declared_tensors():
    from rocml_b200.engine.model import declared_tensors
    decl = {d.name: tuple(d.shape) for d in declared_tensors(spec_of(ZOKELORN["ZA"]))}
    assert decl["embed"] == (211, 64) and decl["head"] == (211, 64) and decl["final.norm"] == (64,)
    assert decl["l0.mix.q"] == (48, 64) and decl["l0.mix.v"] == (72, 64) and decl["l0.mix.g"] == (72, 64)
    assert decl["l0.mix.norm"] == (72,) and decl["l0.mix.o"] == (64, 72)
    assert decl["l1.mix.q"] == (128, 64) and decl["l1.mix.k"] == (64, 64) and decl["l1.mix.v"] == (32, 64)
    assert decl["l1.mix.g"] == (4, 64) and decl["l1.mix.o"] == (64, 64)
    assert decl["l1.mlp.router"] == (6, 64) and decl["l1.mlp.e5.down"] == (64, 24) and decl["l1.mlp.shared.gate"] == (40, 64)
    assert decl["l1.mlp.shared.sg"] == (1, 64)
    assert decl["l2.mix.g"] == (16, 64) and "l2.mix.norm" not in decl and not any(k.startswith("l2.mlp") for k in decl)
    assert "l0.norm2" not in decl and decl["l0.mlp.gate"] == (96, 64)


def test_pages_of_earlier_blocks_come_back():
    """A layer whose queries read only their own block of positions keeps no page that lies wholly before the
    block of the next position; the plan on numbers agrees with what growth then does."""
    from rocml_b200.cache import SequenceCache
    from rocml_b200.cache.requirements import KVRequirement
    req = KVRequirement(1, 16, None, chunk=150)
    assert [req.first_needed(n) for n in (0, 1, 149, 150, 151, 299, 300, 460)] == [0, 0, 0, 150, 150, 150, 300, 450]
    c = SequenceCache([req, KVRequirement(1, 16)], [None, None], 1024, 2, 1024, torch.bfloat16, "cpu", 128)
    blk = next(g for g in c.kv_groups if g.req.chunk)
    full = next(g for g in c.kv_groups if not g.req.chunk)
    s = c.alloc_slot()
    c.plan([[(s, 128)], [(s, 128)], [(s, 128)], [(s, 77)]])
    for n in (128, 128, 128, 77):
        c.grow(s, n); c.commit(s, n)
    # 461 tokens: the next query sits at 461, in the block from 450, on page 7; pages 0 to 6 lie wholly before it
    assert list(blk.table_host[s][:9] >= 0) == [False] * 7 + [True, False]
    assert full.pool.n_held == 8
    for _ in range(200):
        c.grow(s, 1); c.commit(s, 1)
        assert blk.pool.n_held <= 4
    c.check_invariants()
    c.free_slot(s)
    assert blk.pool.n_held == 0 and full.pool.n_held == 0


# ---- the plain implementation's own mechanisms ---------------------------------------------------------------------

def test_plain_running_sum_in_pieces_and_as_a_sum_over_keys():
    torch.manual_seed(0)
    T, H, dim, vdim = 23, 3, 5, 7
    q, k, v = torch.randn(T, H, dim).double(), torch.randn(T, H, dim).double(), torch.randn(T, H, vdim).double()
    decay = [0.5, 1.0, 0.0]
    o, S = P.decayed_sum(q, k, v, decay)
    o1, S1 = P.decayed_sum(q[:9], k[:9], v[:9], decay)
    o2, S2 = P.decayed_sum(q[9:], k[9:], v[9:], decay, state=S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # the same thing as attention without softmax: o_t = sum_{s <= t} d^(t - s) (q_t . k_s) v_s
    for h, d in enumerate(decay):
        for t in (0, 7, 22):
            want = sum((d ** (t - s) if t > s else 1.0) * float(q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-10)


def test_plain_rotation_keeps_lengths_and_depends_on_distance_only():
    torch.manual_seed(1)
    rot = {"base": 100.0, "dims": 6, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    x = torch.randn(1, 2, 10).double()
    a = P.rotate_pairs(x.expand(3, 2, 10).clone(), [0, 5, 11], rot)
    assert torch.equal(a[0], x[0])                                  # position 0: unchanged
    assert torch.equal(a[:, :, 6:], x.expand(3, 2, 10)[:, :, 6:])   # beyond dims: unchanged
    assert torch.allclose(a.norm(dim=-1), x.norm(dim=-1).expand(3, 2))
    y = torch.randn(1, 2, 10).double()
    b = P.rotate_pairs(y.expand(3, 2, 10).clone(), [20, 25, 31], rot)
    c = P.rotate_pairs(y.expand(3, 2, 10).clone(), [0, 5, 11], rot)
    assert torch.allclose((a[2] * c[1]).sum(-1), (P.rotate_pairs(x.expand(3, 2, 10).clone(), [31, 0, 0], rot)[0] * b[1]).sum(-1))
    f, plain = P.frequencies(rot), P.frequencies({"base": 100.0, "dims": 6})
    assert f[0] == plain[0] and abs(float(f[2] / plain[2]) - 0.25) < 1e-12 and 0.25 < float(f[1] / plain[1]) < 1.0


def test_plain_route_groups_and_weights():
    h = torch.eye(8).double()[:1]                                # one token that reads row 0 of the router
    scores = torch.tensor([0.9, 0.1, 0.5, 0.55, 0.8, 0.3, 0.2, 0.84], dtype=torch.float64)
    wr = torch.zeros(8, 8).double()
    wr[:, 0] = torch.log(scores / (1 - scores))
    r = {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}}
    # groups' scores: 1.0, 1.05, 1.1, 1.04 -> groups 2 and 1 stay; the best three of 0.5 0.55 0.8 0.3
    chosen, weights = P.route(h, {"x.router": wr}, "x.", r)
    assert sorted(chosen[0].tolist()) == [2, 3, 4]
    assert abs(float(weights.sum()) - 1.0) < 1e-12
    by = dict(zip(chosen[0].tolist(), weights[0].tolist()))
    assert abs(by[4] - 0.8 / 1.85) < 1e-12
    chosen, _ = P.route(h, {"x.router": wr}, "x.", {"experts": 8, "top": 3})
    assert sorted(chosen[0].tolist()) == [0, 4, 7]


def test_plain_block_mask_and_gelu():
    torch.manual_seed(2)
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "mask": {"size": 3}, "rot": {"base": 10.0, "dims": 2}}
    w = {"x.q": torch.randn(8, 10).double(), "x.k": torch.randn(4, 10).double(), "x.v": torch.randn(6, 10).double(),
         "x.g": torch.randn(2, 10).double(), "x.o": torch.randn(10, 12).double()}
    h = torch.randn(7, 10).double()
    whole = P.attention(h, w, "x.", m)
    # positions 3..5 form a block of their own: the same rows come out when only they are given, at their positions
    alone = P.attention(h[3:6], w, "x.", m, positions=[3, 4, 5])
    assert torch.allclose(whole[3:6], alone, atol=1e-12)
    assert not torch.allclose(whole[3:6], P.attention(h[3:6], w, "x.", m, positions=[2, 3, 4]), atol=1e-3)
    z = torch.tensor([-3.0, 0.0, 0.5, 4.0]).double()
    assert torch.allclose(P.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-12)
