"""The Kizezen decoder without a device: configuration, plan, tensor names against the naming rule, what the cache keeps
(the pages of kept first keys are held on to, a latent's values live in its key rows), refusals, the frequency laws, and
the plain implementation against closed forms."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_kizezen as pk
from kizezen_models import CONFIGS, MIXED, ODD, tensor_shapes

from camelid_b200.cache.book import PAGE, CacheBook, KVSpec, StateSpec, flatten_specs
from camelid_b200.config.kizezen import KizezenConfig, kizezen_plan
from camelid_b200.engine.model import DecoderModel
from camelid_b200.errors import ConfigError
from camelid_b200.parts.position import rotary_frequencies


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_follow_the_naming_rule(name):
    model = DecoderModel.from_config(CONFIGS[name], dtype=torch.bfloat16, device="cpu")
    got = {k: tuple(v.shape) for k, v in model.tensor_specs().items()}
    assert got == {k: v[0] for k, v in tensor_shapes(CONFIGS[name]).items()}


def test_plan_names_the_parts_and_their_constants():
    plan = kizezen_plan(KizezenConfig.from_dict(MIXED))
    kinds = [L.mixer.kind for L in plan.layers]
    assert kinds == ["retention", "window_attention", "latent_attention", "window_attention", "retention"]
    assert all(L.arrangement == "prenorm" for L in plan.layers)
    assert plan.layers[2].ffn is None and plan.layers[2].norm2 is None
    a = plan.layers[1].mixer.params
    assert (a["window"], a["keep_first"], a["num_kv_heads"], a["qk_norm"], a["bias"], a["sink"]) == (9, 3, 2, "full", True, True)
    assert a["position"].params["scaling"]["rope_type"] == "llama3" and a["position"].params["pairing"] == "split"
    assert plan.layers[3].mixer.params["window"] is None and plan.layers[3].mixer.params["position"] is None
    la = plan.layers[2].mixer.params
    assert la["position"].params["scaling"]["rope_type"] == "ramp" and la["position"].params["pairing"] == "interleaved"
    assert plan.layers[0].mixer.params["decay"] == (0.9, 0.99, 0.999)
    assert plan.layers[0].ffn.params["activation"] == "gelu_erf"
    assert plan.embedding.params["scale"] == 3.0 and plan.head.params["scale"] == 0.7


def test_what_the_cache_keeps():
    model = DecoderModel.from_config(ODD, dtype=torch.bfloat16, device="cpu")
    specs = [flatten_specs(b.cache_spec()) for b in model.blocks]
    assert specs[0] == [KVSpec(1, 12, 70, 20, None, 65)]
    assert specs[1] == [KVSpec(1, 24, None, 18, None, 0, True)] and specs[1][0].stored_value_dim == 0
    assert specs[2] == [StateSpec((1, 4, 20), "float32", "retention")]
    assert specs[3][0].kept_blocks == 1 and specs[0][0].kept_blocks == 2


def test_pages_of_kept_first_keys_are_held_on_to():
    book = CacheBook([KVSpec(1, 8, 70, None, None, 65), KVSpec(1, 8, 70)], n_pages=16, n_slots=2, max_position=10000)
    slot = book.alloc_slot()
    for n in (300, 1, 1, 200):
        book.check_extend([(slot, n)])
        book.extend(slot, n)
        book.commit(slot, n)
        book.audit()
    kept, plain = book.pages[0][slot], book.pages[1][slot]
    first = (502 - 70 + 1) // PAGE
    assert all(p >= 0 for p in kept[:2]) and all(p < 0 for p in kept[2:first]) and all(p >= 0 for p in kept[first:])
    assert all(p < 0 for p in plain[:first]) and all(p >= 0 for p in plain[first:])
    book.free_slot(slot)
    assert all(p.n_free == p.n for p in book.pools)


@pytest.mark.parametrize("path,value,key", [
    (("layers", 1, "mixer", "kv_heads"), 4, "kv_heads"), (("layers", 0, "mixer", "decay"), [0.5], "decay"),
    (("layers", 2, "mixer", "rot", "dims"), 6, "rot.dims"), (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "type"), "convolution", "type"), (("layers", 0, "mlp", "kind"), "moe", "mlp.kind"),
    (("layers", 1, "mixer", "mask", "keep_first"), -1, "keep_first"), (("vocab",), 0, "vocab"),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), 0.0, "scaling")])
def test_refusals_name_the_key(path, value, key):
    cfg = copy.deepcopy(MIXED)
    d = cfg
    for p in path[:-1]:
        d = d[p]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        KizezenConfig.from_dict(cfg)
    assert key in str(e.value)


def test_missing_keys_take_their_defaults():
    cfg = copy.deepcopy(MIXED)
    del cfg["embedding"], cfg["logit_scale"], cfg["layers"][1]["mixer"]["kv_heads"], cfg["layers"][1]["mixer"]["vdim"]
    c = KizezenConfig.from_dict(cfg)
    assert (c.embedding_scale, c.logit_scale) == (1.0, 1.0)
    assert c.layers[1]["mixer"]["kv_heads"] == 6 and c.layers[1]["mixer"]["vdim"] == 24


def test_frequency_laws_match_the_plain_ones():
    for rot, law in ((MIXED["layers"][1]["mixer"]["rot"], "llama3"), (MIXED["layers"][2]["mixer"]["rot"], "ramp"),
                     (ODD["layers"][1]["mixer"]["rot"], "ramp"), (CONFIGS["wide"]["layers"][0]["mixer"]["rot"], "llama3")):
        want, amp = pk.frequencies(rot)
        m = KizezenConfig.from_dict({**MIXED, "layers": [{"type": "retention", "mlp": None,
                                                          "mixer": {"dim": rot["dims"], "heads": 1, "decay": [0.5], "rot": rot}}]})
        p = m.layers[0]["mixer"]["rot"]
        assert p["scaling"]["rope_type"] == law
        got = rotary_frequencies(p["rotary_dim"], p["theta"], p["scaling"])
        assert np.allclose(got, want, rtol=2e-6, atol=0)
        assert (amp == 1.0) == (law == "llama3")
    # the ramp law by hand: two pairs, the first untouched, the second wholly divided
    f, amp = pk.ramped_frequencies(4, 100.0, {"factor": 4.0, "fast": 16.0 / (2 * math.pi), "slow": 16.0 / (2 * math.pi * 10.0),
                                             "original": 16.0})
    assert np.allclose(f, [1.0, 0.1 / 4.0]) and amp == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_plain_mechanisms_against_closed_forms():
    # the window with kept first keys
    see = pk.visible(8, 3, 2)
    assert see[7].tolist() == [True, True, False, False, False, True, True, True] and see[2].tolist() == [True] * 3 + [False] * 5
    # a sink of ln 3 beside one key of score 0 leaves a quarter
    w = pk.sink_softmax(np.zeros((1, 1)), np.ones((1, 1), bool), math.log(3.0))
    assert w[0, 0] == pytest.approx(0.25)
    # retention by hand: two tokens, one head, keys and queries of one channel
    m = {"heads": 1, "dim": 1, "vdim": 2, "decay": (0.5,)}
    out = pk.retention_core(np.array([[1.0], [2.0]]), np.array([[3.0], [1.0]]), np.array([[1.0, -1.0], [4.0, 0.0]]), m)
    assert np.allclose(out[0, 0], [3.0, -3.0]) and np.allclose(out[1, 0], [2 * (1.5 + 4.0), 2 * -1.5])
    # a turn by a quarter circle, pairs of halves and pairs of neighbours
    x = np.array([[[1.0, 2.0, 3.0, 4.0]]])
    assert np.allclose(pk.turn(x, [1], np.array([math.pi / 2, 0.0]), 1.0, 4, "half")[0, 0], [-3.0, 2.0, 1.0, 4.0])
    assert np.allclose(pk.turn(x, [1], np.array([math.pi / 2, 0.0]), 2.0, 4, "pairs")[0, 0], [-4.0, 2.0, 6.0, 8.0])
    # the latent form equals attention with per-head keys and values written out
    rng = np.random.default_rng(0)
    mm = {"heads": 2, "dim": 3, "rot_dim": 2, "vdim": 4, "kv_rank": 5, "scale": 0.4, "rot": {"dims": 2, "base": 10.0}}
    t = {"uk": rng.normal(size=(6, 5)), "uv": rng.normal(size=(8, 5)), "dkv.norm": np.ones(5), "sink": np.array([-np.inf, -np.inf])}
    q, down, gate = rng.normal(size=(4, 10)), rng.normal(size=(4, 7)), np.full((4, 2), 50.0)
    got = pk.latent_core(q, down, gate, t, mm, 1e-6)
    c = pk.rms_norm(down[:, :5], None, 1e-6)
    kt = pk.turn(down[:, None, 5:], np.arange(4), np.array([1.0]), 1.0, 2, "pairs")[:, 0]
    qt = pk.turn(q.reshape(4, 2, 5)[:, :, 3:], np.arange(4), np.array([1.0]), 1.0, 2, "pairs")
    for h in range(2):
        keys = np.concatenate([c @ t["uk"][3 * h:3 * h + 3].T, kt], 1)
        qs = np.concatenate([q.reshape(4, 2, 5)[:, h, :3], qt[:, h]], 1)
        s = np.where(np.tril(np.ones((4, 4), bool)), qs @ keys.T * 0.4, -np.inf)
        w = np.exp(s - s.max(-1, keepdims=True))
        w /= w.sum(-1, keepdims=True)
        assert np.allclose(got.reshape(4, 2, 4)[:, h], w @ (c @ t["uv"][4 * h:4 * h + 4].T))
