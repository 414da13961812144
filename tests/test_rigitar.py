"""Rigitar without a GPU: the configuration reader, the plan and its tensor list, random models on disk, the
cache's bookkeeping for rows shared between layers and per-sequence state, and hand-computed checks of the plain
implementation's mechanisms."""
import json
import math
import os

import pytest
import torch

from exl3_server_b200.cache.kv import SequenceCache
from exl3_server_b200.config import ConfigError, resolve_architecture
from exl3_server_b200.config.rigitar import RigitarConfig
from exl3_server_b200.engine.model import plan_manifest
from exl3_server_b200.parts.base import KVRequest, StateRequest
import plain_rigitar as P
from rigitar_configs import CONFIGS, make_rigitar


def test_config_round_trip_and_plan():
    cfg = CONFIGS["mixed"]
    obj = json.loads(json.dumps(cfg.to_dict()))
    arch = resolve_architecture(obj)
    again = arch.config_class.from_dict(obj)
    assert again.to_dict() == cfg.to_dict()
    plan = arch.build_plan(again)
    assert [l.mixer.kind for l in plan.layers] == ["latent_attention", "mingru", "latent_attention",
                                                   "latent_attention", "mingru"]
    assert [e.cache_from for e in plan.schedule] == [None, None, 0, None, None]
    assert plan.layers[1].feed_forward is None and plan.layers[0].feed_forward.inner == 160
    names = {s.name: s.shape for s in plan_manifest(plan)}
    assert names["l0.mix.dkv"] == (48, 96) and "l2.mix.dkv" not in names and names["l2.mix.uk"] == (32, 40)
    assert names["l3.mix.uq"] == (48, 48) and names["l4.mix.z.b"] == (130,) and names["l4.mlp.act"] == (2,)
    assert "l1.norm2" not in names and names["l0.norm2"] == (96,) and names["final.norm"] == (96,)
    assert "l1.norm2" in plan.ignorable


@pytest.mark.parametrize("change, message", [
    (lambda o: o["layers"][2]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda o: o["layers"][2]["mixer"].__setitem__("kv_rank", 48), "kv_rank"),
    (lambda o: o["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda o: o["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda o: o["layers"][0]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda o: o["layers"][3]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda o: o["norm"].pop("eps"), "eps"),
    (lambda o: o.__setitem__("layers", []), "layers"),
])
def test_config_errors_name_the_key(change, message):
    obj = CONFIGS["mixed"].to_dict()
    change(obj)
    with pytest.raises(ConfigError, match=message):
        RigitarConfig.from_dict(obj)


def test_random_model_on_disk(tmp_path):
    folder = make_rigitar("mixed", str(tmp_path / "m"))
    w = P.read_weights(folder)
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architecture"] == "Rigitar" and len(cfg["layers"]) == 5
    assert w["l0.mix.g"].shape == (3, 96) and w["head"].shape == (211, 96)
    logits = P.PlainRigitar(folder).logits([1, 2, 3, 4])
    assert logits.shape == (4, 211) and torch.isfinite(logits).all()


def test_cache_rows_shared_between_layers_and_state():
    row = KVRequest(kv_heads=1, head_dim=48, values_in_keys=True)
    state = StateRequest((72,))
    cache = SequenceCache([(row, None, None), (None, state, None), (row, None, 0), (KVRequest(1, 80, values_in_keys=True), None, None)],
                          max_tokens=256, device="cpu", dtype=torch.float32)
    assert len(cache.groups) == 2 and cache.entry_owns == [True, False, False, True]
    assert cache.groups[0].v is cache.groups[0].k and cache.groups[0].k.shape == (1, 5, 1, 64, 48)
    s = cache.open()
    cache.state[1][s].fill_(3.0)
    cache.reserve({s: 70})
    cache.commit(s, 70)
    assert cache.tokens_held() == 128
    cache.close(s)
    s2 = cache.open()
    assert s2 == s and float(cache.state[1][s2].abs().max()) == 0.0      # a reused slot starts from zero state
    cache.check()
    with pytest.raises(Exception, match="head shapes differ"):
        SequenceCache([(row, None, None), (KVRequest(1, 48), None, 0)], max_tokens=64, device="cpu")


def test_plain_mechanisms_by_hand():
    # rms norm
    x = torch.tensor([[3.0, 4.0]], dtype=P.F)
    assert torch.allclose(P.rms_norm(x, torch.tensor([2.0, 1.0], dtype=P.F), 0.0), torch.tensor([[6.0, 4.0]], dtype=P.F) / math.sqrt(12.5))
    # rotation: pairs (0, 2) and (1, 3) of the first four features, the fifth passes
    v = torch.tensor([[1.0, 0.0, 0.0, 1.0, 9.0]], dtype=P.F)
    r = P.rotate(v, torch.tensor([2]), 100.0, 4)
    a0, a1 = 2.0, 2.0 * 100.0 ** -0.5
    assert torch.allclose(r, torch.tensor([[math.cos(a0), -math.sin(a1), math.sin(a0), math.cos(a1), 9.0]], dtype=P.F))
    # xielu at both sides of zero
    pq = torch.tensor([0.3, -0.2], dtype=P.F)
    sp = lambda t: math.log1p(math.exp(t))
    assert math.isclose(float(P.xielu(torch.tensor(2.0, dtype=P.F), pq)), sp(0.3) * 4 + 1.0)
    assert math.isclose(float(P.xielu(torch.tensor(-1.0, dtype=P.F), pq)), (0.5 + sp(-0.2)) * (math.exp(-1) - 1 + 1) - 0.5)
    assert float(P.xielu(torch.tensor(0.0, dtype=P.F), pq)) == 0.0
    # minGRU: two steps of one channel
    w = {"z": torch.tensor([[1.0]], dtype=P.F), "z.b": torch.tensor([0.0], dtype=P.F), "x": torch.tensor([[2.0]], dtype=P.F),
         "x.b": torch.tensor([-1.0], dtype=P.F), "g": torch.tensor([[1.0]], dtype=P.F), "o": torch.tensor([[1.0]], dtype=P.F)}
    h = torch.tensor([[1.0], [0.0]], dtype=P.F)
    sig = lambda t: 1 / (1 + math.exp(-t))
    s1 = sig(1.0) * (1.0 + 0.5)                                   # u = 1 >= 0: candidate u + 1/2
    s2 = (1 - sig(0.0)) * s1 + sig(0.0) * sig(-1.0)               # u = -1 < 0: candidate sigmoid(u)
    y = P.mingru(h, {"p." + k: v for k, v in w.items()}, "p.")
    assert math.isclose(float(y[0]), s1 * 1.0 * sig(1.0)) and math.isclose(float(y[1]), s2 * 0.0 * sig(0.0), abs_tol=1e-15)
