"""Nikodra without a GPU: the configuration reader, the plan and its tensor list, random models on disk, the cache's
bookkeeping for blocks of positions and for per-sequence state of several owners, and hand-computed checks of the
plain implementation's mechanisms."""
import json
import math

import pytest
import torch

from exl3_server_b200.cache.kv import SequenceCache
from exl3_server_b200.config import ConfigError, resolve_architecture
from exl3_server_b200.engine.model import plan_manifest
from exl3_server_b200.parts.base import KVRequest, StateRequest
from exl3_server_b200.parts.position import RotaryPosition
from exl3_server_b200.parts.spec import PositionSpec
import plain_nikodra as P
from nikodra_configs import CONFIGS, make_nikodra


def test_config_round_trip_and_plan():
    cfg = CONFIGS["mixed"]
    obj = json.loads(json.dumps(cfg.to_dict()))
    arch = resolve_architecture(obj)
    again = arch.config_class.from_dict(obj)
    assert again.to_dict() == cfg.to_dict()
    plan = arch.build_plan(again)
    assert [l.mixer.kind for l in plan.layers] == ["normed_attention", "wkv", "normed_attention", "normed_attention",
                                                   "parallel", "normed_attention"]
    # the first layer with v_mix gives its values, the later ones mix them in, a layer without the key does neither
    assert [l.mixer.params.get("v_mix") for l in plan.layers] == ["source", None, None, "mix", None, "mix"]
    assert all(l.arrangement == "sandwich" and l.residual_scale == 0.7 for l in plan.layers)
    assert plan.layers[1].feed_forward is None and plan.layers[0].feed_forward.inner == 160
    left, right = plan.layers[4].mixer.params["branches"]
    assert left.params["chunk"] == 50 and left.params["qk_norm"] == "unit" and left.position is None
    assert right.kind == "retention" and right.params["decay"] == [0.9, 0.97, 0.995]
    assert plan.layers[0].mixer.position.params["layout"] == "interleaved" and "yarn" in plan.layers[0].mixer.position.params
    assert "yarn" not in plan.layers[2].mixer.position.params and right.position.params["layout"] == "half"
    names = {s.name: s.shape for s in plan_manifest(plan)}
    assert names["l0.mix.q"] == (96, 96) and names["l0.mix.v"] == (32, 96) and names["l0.mix.o"] == (96, 64)
    assert names["l2.mix.v.b"] == (120,) and names["l2.mix.q.norm"] == (16,) and names["l0.mix.vmix"] == ()
    assert "l2.mix.vmix" not in names and names["l4.mix.left.out"] == (96,) and names["l4.mix.right.g"] == (72, 96)
    assert names["l1.mix.w1"] == (8, 96) and names["l1.mix.u"] == (3, 16) and names["l1.mix.mu.w"] == (96,)
    assert "l1.norm2" not in names and names["l1.norm1b"] == (96,) and names["l0.norm2b"] == (96,)
    assert names["bigram"] == (98, 96) and names["head"] == (211, 96)
    assert "l1.norm2b" in plan.ignorable


def test_a_rank_the_configuration_does_not_give_is_the_checkpoints():
    from exl3_server_b200.weights.loader import check_manifest
    obj = CONFIGS["only_wkv"].to_dict()                  # no decay_rank key
    arch = resolve_architecture(obj)
    man = plan_manifest(arch.build_plan(arch.config_class.from_dict(obj)))
    found = {s.name: tuple(11 if d == -1 else d for d in s.shape) for s in man}
    assert found["l0.mix.w1"] == (11, 80) and found["l0.mix.w2"] == (96, 11)
    check_manifest(man, found)
    found["l0.mix.w1"] = (11, 81)
    with pytest.raises(Exception, match="l0.mix.w1"):
        check_manifest(man, found)


@pytest.mark.parametrize("change, message", [
    (lambda o: o["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda o: o["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda o: o["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda o: o["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda o: o["layers"][4]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda o: o["layers"][4]["mixer"].pop("left"), "left"),
    (lambda o: o["layers"][5]["mixer"].__setitem__("vdim", 24), "v_mix"),
    (lambda o: o["layers"][1].__setitem__("type", "conv"), "type"),
    (lambda o: o["layers"][0]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda o: o["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda o: o["norm"].pop("eps"), "eps"),
    (lambda o: o.__setitem__("layers", []), "layers"),
])
def test_config_errors_name_the_key(change, message):
    obj = CONFIGS["mixed"].to_dict()
    change(obj)
    with pytest.raises(ConfigError, match=message):
        resolve_architecture(obj).config_class.from_dict(obj)


def test_random_model_on_disk(tmp_path):
    folder = make_nikodra("odd", str(tmp_path / "m"))
    pm = P.PlainNikodra(folder)
    assert pm.w["l1.mix.w1"].shape == (5, 100) and pm.w["l0.mix.right.q"].shape == (24, 100)
    assert 0.2 <= float(pm.w["l2.mix.vmix"]) <= 0.6
    out = pm.logits([3, 1, 4, 1, 5])
    assert out.shape == (5, 77) and torch.isfinite(out).all()


def test_cache_blocks_of_positions_and_state_of_several_owners():
    """A group whose queries see only their own block of 50 positions gives back the pages wholly before the block
    of the next position; state of a mixer with two tensors and of the embedding is zeroed when a slot is reused."""
    reqs = [(KVRequest(2, 16, chunk=50), None, None), (None, (StateRequest((8,)), StateRequest((2, 4, 4))), None),
            (KVRequest(2, 16), StateRequest((3,)), None)]
    c = SequenceCache(reqs, max_tokens=64 * 8, dtype=torch.float32, device="cpu", page_size=64,
                      extra_states={"embedding": StateRequest((), torch.int32)})
    assert len(c.groups) == 2 and c.groups[0].request.chunk == 50
    assert isinstance(c.state_of(1), tuple) and c.state_of(1)[1].shape[1:] == (2, 4, 4)
    assert c.state_of("embedding").dtype == torch.int32 and c.state_of(0) is None
    s = c.open()
    c.state_of(1)[0][s] += 3.0
    c.state_of(1)[1][s] += 2.0
    c.state_of("embedding")[s] = 9
    c.reserve({s: 130})
    c.commit(s, 130)                                     # next position 130 lies in block 100..149: page 0 (0..63) is free
    assert c.groups[0].pages[s][0] == -1 and c.groups[0].pages[s][1] >= 0 and c.groups[1].pages[s][0] >= 0
    assert c.gives_back_at(150) and not c.gives_back_at(149) and c.gives_back_at(200) and c.gives_back_at(100) and not c.gives_back_at(101) and not c.gives_back_at(50)
    c.reserve({s: 200})
    c.commit(s, 200)                                     # block 200..249 starts in page 3
    assert [p >= 0 for p in c.groups[0].pages[s]] == [False, False, False, True]
    c.check()
    c.close(s)
    s2 = c.open()
    assert s2 == s
    assert float(c.state_of(1)[0][s2].abs().sum()) == 0 and float(c.state_of(1)[1][s2].abs().sum()) == 0
    assert int(c.state_of("embedding")[s2]) == 0
    c.check()


def test_plain_mechanisms_by_hand():
    # the second table's rows: the last row first, then the hash of (token before, token)
    assert P.pair_rows([5, 2, 9], 97, 31, 7) == [97, (5 * 31 + 2 * 7) % 97, (2 * 31 + 9 * 7) % 97]
    # a softmax with one more in the denominator: a single key of score 0 gets 1/2, the rest is lost
    s = torch.tensor([[0.0, -math.inf], [math.log(3.0), 0.0]], dtype=P.F)
    p = P.sink_softmax(s)
    assert torch.allclose(p, torch.tensor([[0.5, 0.0], [0.6, 0.2]], dtype=P.F))
    # blocks of 2 positions: token 2 sees only itself, token 3 sees 2 and 3
    q = torch.zeros(4, 1, 2, dtype=P.F)
    k = torch.zeros(4, 1, 2, dtype=P.F)
    v = torch.tensor([[[1.0]], [[10.0]], [[100.0]], [[1000.0]]], dtype=P.F)
    o = P.grouped_attention(q, k, v, 1.0, 2)
    assert torch.allclose(o[:, 0], torch.tensor([0.5, 11.0 / 3.0, 50.0, 1100.0 / 3.0], dtype=P.F))
    o = P.grouped_attention(q, k, v, 1.0, 0)
    assert torch.allclose(o[3, 0], torch.tensor(1111.0 / 5.0, dtype=P.F))
    # rotation: a quarter turn of the pair, in both layouts; features beyond dims stay
    rot = {"base": 1.0, "dims": 2}
    x = torch.tensor([[[1.0, 0.0, 7.0]], [[1.0, 0.0, 7.0]]], dtype=P.F)
    y = P.rotate(x, rot, True)
    assert torch.allclose(y[1, 0], torch.tensor([math.cos(1.0), math.sin(1.0), 7.0], dtype=P.F))
    x4 = torch.tensor([[[1.0, 2.0, 0.0, 0.0]], [[1.0, 2.0, 0.0, 0.0]]], dtype=P.F)
    y = P.rotate(x4, {"base": 1.0, "dims": 4}, False)
    assert torch.allclose(y[1, 0], torch.tensor([math.cos(1.0), 2 * math.cos(1.0), math.sin(1.0), 2 * math.sin(1.0)], dtype=P.F))
    # the stretched table: slow pairs are divided by the factor, fast ones stay, and the factor on sines and cosines
    f, factor = P.rotary_frequencies({"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}})
    plain, one = P.rotary_frequencies({"base": 10000.0, "dims": 32})
    assert one == 1.0 and abs(factor - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert float(f[0]) == float(plain[0]) and abs(float(f[-1]) - float(plain[-1]) / 4.0) < 1e-15
    assert all(float(plain[i]) / 4.0 - 1e-15 <= float(f[i]) <= float(plain[i]) + 1e-15 for i in range(16))
    # the package's table is the same
    spec = PositionSpec(kind="rope", dims=32, theta=10000.0, params={"layout": "interleaved", "yarn": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}})
    assert torch.allclose(RotaryPosition.frequencies(spec), f, rtol=1e-13, atol=0)
    # retention, two tokens by hand: o_1 = (decay k_0 v_0^T + k_1 v_1^T)^T q_1
    q = torch.tensor([[[1.0, 2.0]], [[3.0, 4.0]]], dtype=P.F)
    k = torch.tensor([[[0.5, 1.0]], [[2.0, -1.0]]], dtype=P.F)
    v = torch.tensor([[[1.0, 10.0, 100.0]], [[2.0, 20.0, 200.0]]], dtype=P.F)
    o = P.retention(q, k, v, [0.5])
    assert torch.allclose(o[0, 0], 2.5 * v[0, 0])
    assert torch.allclose(o[1, 0], 0.5 * (3 * 0.5 + 4 * 1.0) * v[0, 0] + (3 * 2.0 - 4 * 1.0) * v[1, 0])
    # wkv, three tokens: the bonus counts for the current token only; a token's decay acts on what the tokens after
    # it read, not on its own output
    r = torch.tensor([[[1.0, 1.0]], [[1.0, 2.0]], [[1.0, 1.0]]], dtype=P.F)
    k3 = torch.tensor([[[0.5, 1.0]], [[2.0, -1.0]], [[1.0, 1.0]]], dtype=P.F)
    w = torch.tensor([[[9.0, 9.0]], [[0.5, 0.25]], [[9.0, 9.0]]], dtype=P.F)
    u = torch.tensor([[3.0, 0.0]], dtype=P.F)
    vv = torch.tensor([[[1.0, 10.0]], [[2.0, 20.0]], [[4.0, 40.0]]], dtype=P.F)
    o = P.wkv(r, k3, vv, w, u)
    assert torch.allclose(o[0, 0], (1 * 3.0 * 0.5) * vv[0, 0])
    assert torch.allclose(o[1, 0], (1 * 0.5 + 2 * 1.0) * vv[0, 0] + (1 * 3.0 * 2.0) * vv[1, 0])
    assert torch.allclose(o[2, 0], (0.5 * 0.5 + 0.25 * 1.0) * vv[0, 0] + (2.0 - 1.0) * vv[1, 0] + 3.0 * vv[2, 0])
