"""Pipilix without a GPU: the configuration, the parts it is spelled as, the tensors it declares, the cache it
asks for, and the plain implementation's own mechanisms."""
import json

import pytest
import torch

import plain_pipilix as P
from tiny_models import PIPILIX


def spec_of(cfg):
    from rocml_b200.config import config_from_dict
    return config_from_dict(cfg).to_model_spec()


@pytest.mark.parametrize("name", sorted(PIPILIX))
def test_config_round_trip(name):
    from rocml_b200.config import PipilixConfig, config_from_dict
    cfg = config_from_dict(PIPILIX[name])
    assert isinstance(cfg, PipilixConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert len(cfg.layers) == len(PIPILIX[name]["layers"])


def test_architecture_is_chosen_by_either_key():
    from rocml_b200.config import PipilixConfig, Qwen3Config, config_from_dict
    from rocml_b200.errors import ConfigError, UnsupportedArchitecture
    from tiny_models import TINY_A
    assert isinstance(config_from_dict(PIPILIX["PA"]), PipilixConfig)
    assert isinstance(config_from_dict({**PIPILIX["PA"], "architecture": None, "architectures": ["Pipilix"]}), PipilixConfig)
    assert isinstance(config_from_dict(TINY_A), Qwen3Config)
    with pytest.raises(UnsupportedArchitecture):
        config_from_dict({**PIPILIX["PA"], "architecture": "Nobody"})
    with pytest.raises(ConfigError):
        config_from_dict({k: v for k, v in PIPILIX["PA"].items() if k != "architecture"})


@pytest.mark.parametrize("broken, needle", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "type"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["loop"].__setitem__("stop", 7), "loop"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_named(broken, needle):
    from rocml_b200.config import config_from_dict
    from rocml_b200.errors import ConfigError
    cfg = json.loads(json.dumps(PIPILIX["PA"]))
    broken(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert needle in str(e.value)


def test_schedule_follows_the_loop():
    spec = spec_of(PIPILIX["PA"])          # layers 0, 1 three times, then 2
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 1, 0, 1, 2]
    assert [e.add_input for e in spec.schedule] == [False, False, True, False, True, False, False]
    rows = [e.add_row[1] if e.add_row else None for e in spec.schedule]
    assert rows == [0, None, 1, None, 2, None, None]
    assert all(e.reads_cache_of is None for e in spec.schedule)
    assert [(i, t) for i, t, _ in P.layer_runs(PIPILIX["PA"])] == [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (2, None)]
    spec = spec_of(PIPILIX["PC"])          # a loop that runs once still adds its row
    assert [e.layer for e in spec.schedule] == [0, 1, 2]
    assert [e.add_row is not None for e in spec.schedule] == [False, True, False]
    assert not any(e.add_input for e in spec.schedule)
    assert all(e.add_row is None for e in spec_of(PIPILIX["PB"]).schedule)


def test_declared_tensors_carry_the_files_names():
    from rocml_b200.engine.model import declared_tensors
    cfg = PIPILIX["PA"]
    got = {d.name: tuple(d.shape) for d in declared_tensors(spec_of(cfg))}
    D = cfg["width"]
    assert got["embed"] == (cfg["vocab"], D) and got["head"] == (cfg["vocab"], D) and got["final.norm"] == (D,)
    assert got["loop.step"] == (3, D)
    m = cfg["layers"][1]["mixer"]
    assert got["l1.mix.q"] == (m["heads"] * m["dim"], D)
    assert got["l1.mix.dkv"] == (m["kv_rank"], D) and got["l1.mix.dkv.norm"] == (m["kv_rank"],)
    assert got["l1.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"])
    assert got["l1.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
    assert got["l1.mix.g"] == (m["heads"], D) and got["l1.mix.o"] == (D, m["heads"] * m["vdim"])
    assert got["l1.mlp.router"] == (5, D) and got["l1.mlp.correction"] == (5,)
    assert got["l1.mlp.e4.gate"] == (40, D) and got["l1.mlp.e4.down"] == (D, 40)
    assert got["l0.mlp.up"] == (96, D)
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert got[f"l0.{n}"] == (D,)
    assert "l2.norm2" not in got and "l2.norm2b" not in got and not any(k.startswith("l2.mlp") for k in got)
    assert not any(k.endswith(".weight") for k in got)
    assert "loop.step" not in {d.name for d in declared_tensors(spec_of(PIPILIX["PB"]))}


def test_every_run_of_a_layer_has_a_cache_of_its_own():
    from rocml_b200.cache import SequenceCache
    from rocml_b200.engine.model import Model
    from rocml_b200.parts import BuildEnv
    model = Model(spec_of(PIPILIX["PA"]), BuildEnv(torch.device("cpu"), torch.float32))
    reqs = model.cache_requirements()
    assert len(reqs) == 7 and all(r.shared_values and r.n_kv_heads == 1 for r in reqs)
    assert [r.head_dim for r in reqs] == [32, 24, 32, 24, 32, 24, 48]
    assert [r.window for r in reqs] == [9, 70, 9, 70, 9, 70, 200]
    cache = SequenceCache(reqs, model.reads_cache_of(), 512, 4, 512, torch.float32, "cpu", 64)
    places = {(id(v.group), v.index) for v in cache.views}
    assert len(places) == 7                      # no two runs share storage
    for g in cache.kv_groups:
        assert g.v is g.k                        # keys and values are one tensor
        assert g.bytes() == g.k.numel() * 4


def test_a_random_folder_reads_back(tmp_path):
    from tiny_models import write_pipilix
    from rocml_b200.config import load_model_spec
    folder = write_pipilix(str(tmp_path / "pc"), PIPILIX["PC"], seed=3)
    w, cfg = P.load_folder(folder)
    assert cfg == json.loads(json.dumps(PIPILIX["PC"]))
    assert load_model_spec(folder).hidden == 72
    assert float(w["l0.mlp.correction"].float().abs().max()) > 0.1


# ---- the plain implementation's mechanisms, each against a direct restatement ------------------------------------

def test_plain_sinusoid_and_embedding():
    pe = P.sinusoid([0, 1, 5], 6, torch.float64)
    assert torch.allclose(pe[0], torch.tensor([0.0, 1.0] * 3, dtype=torch.float64))
    a = 5 * 10000.0 ** (-2.0 / 6)
    assert abs(float(pe[2, 2]) - torch.sin(torch.tensor(a, dtype=torch.float64))) < 1e-12
    assert abs(float(pe[2, 3]) - torch.cos(torch.tensor(a, dtype=torch.float64))) < 1e-12
    table = torch.arange(12, dtype=torch.float64).reshape(2, 6)
    x = P.embed(table, [1, 1], 2.0, torch.float64)
    assert torch.allclose(x[1] - x[0], pe[1] - pe[0])
    assert torch.allclose(x[0], table[1] * 2.0 + pe[0])


def test_plain_window_sees_itself_and_the_tokens_before():
    torch.manual_seed(0)
    D, H, dim, vdim, rank, T = 16, 2, 4, 3, 5, 12
    w = {"q": torch.randn(H * dim, D), "dkv": torch.randn(rank, D), "dkv.norm": torch.rand(rank) + 0.5,
         "uk": torch.randn(H * dim, rank), "uv": torch.randn(H * vdim, rank), "g": torch.randn(H, D),
         "o": torch.randn(D, H * vdim)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, D, dtype=torch.float64)
    full = P.latent_attention(h, w, "", H, dim, vdim, T, 0.5, 1e-6)
    for window in (1, 3, 7):
        got = P.latent_attention(h, w, "", H, dim, vdim, window, 0.5, 1e-6)
        for i in range(T):
            lo = max(0, i - window + 1)
            alone = P.latent_attention(h[lo:i + 1], w, "", H, dim, vdim, T, 0.5, 1e-6)[-1]
            assert torch.allclose(got[i], alone, atol=1e-10)
        assert torch.allclose(got[:window], full[:window], atol=1e-10)
        assert not torch.allclose(got[window:], full[window:], atol=1e-6)


def test_plain_routing_and_experts():
    torch.manual_seed(1)
    D, E, F, T = 8, 4, 6, 9
    w = {"router": torch.randn(E, D), "correction": torch.tensor([0.0, 5.0, -5.0, 0.0])}
    for e in range(E):
        w.update({f"e{e}.gate": torch.randn(F, D), f"e{e}.up": torch.randn(F, D), f"e{e}.down": torch.randn(D, F)})
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, D, dtype=torch.float64)
    chosen, weights = P.route(h, w, "", 2)
    assert (chosen[:, 0] == 1).all() and not (chosen == 2).any()       # the bias decides the choice
    s = torch.sigmoid(h @ w["router"].t())
    assert torch.allclose(weights, torch.gather(s, 1, chosen))          # and stays out of the weights
    assert float(weights.sum(-1).max()) <= 2.0 and not torch.allclose(weights.sum(-1), torch.ones(T, dtype=torch.float64))
    out = P.routed_ff(h, w, "", E, 2, 0.5)
    t = 3
    want = sum(weights[t, j] * P.expert_ff(h[t:t + 1], w, f"e{int(chosen[t, j])}.", 0.5)[0] for j in range(2))
    assert torch.allclose(out[t], want, atol=1e-12)
    g = torch.tensor([[-3.0, 0.2, 9.0]], dtype=torch.float64)
    y = P.expert_ff(torch.ones((1, 1), dtype=torch.float64), {"gate": g.t(), "up": g.t(), "down": torch.eye(3, dtype=torch.float64)}, "", 0.5)
    gg, uu = torch.clamp(g, max=0.5), torch.clamp(g, -0.5, 0.5)
    assert torch.allclose(y, gg * torch.sigmoid(1.702 * gg) * (uu + 1))
