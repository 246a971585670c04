"""The Nudusun decoder without a device: its configuration and plan against the tensor naming rule, refusals, what the
cache keeps for its mixers, and the plain implementation (tests/plain_nudusun.py) against closed forms."""
import copy

import numpy as np
import pytest

import plain_nudusun as pn
from nudusun_models import CONFIGS, tensor_shapes


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes_follow_the_naming_rule(name):
    from camelid_b200.engine.model import DecoderModel
    model = DecoderModel.from_config(CONFIGS[name], device="cpu")
    specs = {n: tuple(s.shape) for n, s in model.tensor_specs().items()}
    assert specs == {n: tuple(shape) for n, (shape, _) in tensor_shapes(CONFIGS[name]).items()}
    assert model.use_graphs and model.capture_steps           # every part runs inside captured graphs
    assert model.memory_plan(256).total > 0


def test_the_plan_reads_every_size_from_the_configuration():
    from camelid_b200.config.registry import load_config
    arch, cfg, plan = load_config(CONFIGS["mixed"])
    assert arch.name == "Nudusun" and cfg.alpha == 1.5 and cfg.embed_scale == 4.0 and len(plan.layers) == 4
    assert plan.max_position == 512 and plan.embedding.params["positions"] == 512 and plan.embedding.params["scale"] == 4.0
    l0, l1, l2, l3 = plan.layers
    assert all(L.arrangement == "postnorm" and L.residual_scale == 1.5 for L in plan.layers)
    assert l0.mixer.kind == "gated_delta" and l0.mixer.params["conv_taps"] == 3 and l0.mixer.params["num_qk_heads"] == 2
    assert l0.ffn.params["identity"] == 1 and l0.ffn.params["groups"] == (3, 2) and l0.ffn.params["route_scale"] == 1.7
    assert l0.ffn.params["gate_act"] == (1.702, 1.5, 1.0) and l0.ffn.params["shared_gate_act"] == (1.702, 3.0, 1.0)
    assert l1.mixer.kind == "window_attention" and l1.mixer.params["window"] == 9 and l1.mixer.params["softcap"] == 5.0
    assert l1.mixer.params["difference"] == 0.25 and l1.mixer.params["qk_norm"] == "head"
    assert l2.ffn is None and l2.norm2 is None and l2.mixer.params["softcap"] is None
    assert l3.ffn.params["shared_size"] is None and l3.ffn.params["groups"] is None and l3.ffn.params["identity"] == 0
    assert l2.after.kind == "token_side" and l2.after.params["layer"] == 2 and l2.after.params["dim"] == 8
    _, open_cfg, open_plan = load_config(CONFIGS["open"])
    assert open_cfg.alpha == 1.0 and open_plan.layers[0].mixer.params["window"] is None and open_plan.layers[0].after is None


def test_what_the_cache_keeps():
    from camelid_b200.cache.book import KVSpec, StateSpec
    from camelid_b200.engine.model import DecoderModel
    specs = DecoderModel.from_config(CONFIGS["mixed"], device="cpu").entry_cache_specs()
    # a delta layer: the matrix per head (values x keys) and the convolution's last inputs; an attention layer: both maps
    # of a key head as one row, values of their own size, pages given back behind the window
    assert specs[0] == [StateSpec((4, 24, 16), "float32", "memory"), StateSpec((2, 2 * 2 * 16 + 4 * 24), "float32", "conv")]
    assert specs[1] == KVSpec(2, 16, 9, 12, None) and specs[2] == KVSpec(3, 32, 70, 40, None)
    assert specs[3][1] == StateSpec((1, 2 * 24 + 2 * 8), "float32", "conv")       # one tap: nothing is read from it
    assert specs[4] is None                                                      # the embedding keeps nothing


@pytest.mark.parametrize("path,value,key", [
    (("layers", 0, "type"), "recurrent", "layers[0].type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "layers[0].mixer.kv_heads"),
    (("layers", 1, "mixer", "mask", "size"), 0, "layers[1].mixer.mask.size"),
    (("layers", 1, "mixer", "softcap"), -1.0, "layers[1].mixer.softcap"),
    (("layers", 1, "mixer", "diff"), None, "layers[1].mixer.diff"),
    (("layers", 0, "mlp", "router", "top"), 7, "layers[0].mlp.router.top"),
    (("layers", 0, "mlp", "router", "top"), 5, "layers[0].mlp.router.top"),       # more than the open groups hold
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "layers[0].mlp.router.groups"),
    (("layers", 0, "mlp", "kind"), "dense", "layers[0].mlp.kind"),
    (("layers", 0, "mlp", "expert", "limit"), 0.0, "layers[0].mlp.expert.limit"),
    (("max_positions",), None, "max_positions"),
    (("width",), -3, "width"),
])
def test_refusals_name_the_key(path, value, key):
    from camelid_b200.config.registry import load_config
    from camelid_b200.errors import ConfigError
    cfg = copy.deepcopy(CONFIGS["mixed"])
    d = cfg
    for p in path[:-1]:
        d = d[p]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(cfg)
    assert key in str(e.value)


def test_a_sequence_may_not_outgrow_the_position_table():
    from camelid_b200.cache.book import CacheBook
    from camelid_b200.engine.model import DecoderModel
    from camelid_b200.errors import CacheError
    from camelid_b200.cache.book import KVSpec
    model = DecoderModel.from_config({**CONFIGS["odd"], "max_positions": 70}, device="cpu")
    kv = [s for s in model.entry_cache_specs() if isinstance(s, KVSpec)]
    book = CacheBook(kv, 8, 2, model.plan.max_position)
    slot = book.alloc_slot()
    book.check_extend([(slot, 70)])
    with pytest.raises(CacheError):
        book.check_extend([(slot, 71)])


# ---- the plain implementation against closed forms ----------------------------------------------

def test_plain_delta_rule_by_hand():
    # one head, two key channels: write v1 under k = e0, then v2 under k = e1 with a decay of one half in between
    q = np.array([[[1.0, 0.0]], [[1.0, 1.0]]])
    k = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    v = np.array([[[2.0, 4.0]], [[6.0, 8.0]]])
    o = pn.delta_rule(q, k, v, beta=np.array([[1.0], [0.5]]), decay=np.array([[1.0], [0.5]]))
    assert np.allclose(o[0, 0], [2.0, 4.0])                     # the read-out sees the token's own write
    assert np.allclose(o[1, 0], [0.5 * 2.0 + 0.5 * 6.0, 0.5 * 4.0 + 0.5 * 8.0])
    # a second write under the same key replaces a share beta of what stands there
    o = pn.delta_rule(np.ones((2, 1, 1)), np.ones((2, 1, 1)), np.array([[[3.0]], [[5.0]]]), np.array([[1.0], [0.25]]), np.ones((2, 1)))
    assert np.allclose(o[:, 0, 0], [3.0, 3.0 + 0.25 * (5.0 - 3.0)])


def test_plain_convolution_starts_from_zeros():
    x = np.arange(1.0, 5.0)[:, None]
    y = pn.causal_conv(x, np.array([[100.0, 10.0, 1.0]]))      # the last tap is the current token's
    assert np.allclose(y[:, 0], [1.0, 12.0, 123.0, 234.0])


def test_plain_window_and_cap():
    m = pn.window_mask(5, 2)
    assert m[3].tolist() == [False, False, True, True, False] and m[0].tolist() == [True, False, False, False, False]
    assert pn.window_mask(3, None)[2].all()
    w = pn.capped_softmax(np.array([[1000.0, 0.0]]), np.ones((1, 2), dtype=bool), 2.0)
    assert np.allclose(w[0, 0] / w[0, 1], np.exp(2.0 * np.tanh(500.0)))


def test_plain_routing_keeps_closed_groups_closed_below_zero():
    # six experts in three groups of two, one group stays open; the correction makes every choice score negative:
    # the chosen two are the open group's, although closed groups hold "larger" numbers than zero would be
    cfg = {"router": {"experts": 5, "identity": 1, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}}
    h = np.eye(6)[:1]
    t = {"router": np.diag([0.0, 0.0, 2.0, 0.5, 1.0, 1.5]), "correction": np.full(6, -1.0)}
    z = np.array([0.0, 0.0, 0.0, 0.0, 0.0, 0.0])
    z[0] = 0.0                                                  # only expert 0's logit is touched by the row e0: all equal
    chosen, weights = pn.route(h, t, cfg)
    assert chosen[0].tolist() == [0, 1]                         # all scores equal 1/6: ties go to the lower index and group
    assert np.allclose(weights, 3.0 / 6.0)
    t["router"] = np.array([[0.0], [0.0], [0.0], [0.0], [0.0], [3.0]]) * np.ones((1, 6))
    chosen, weights = pn.route(h, t, cfg)                       # the identity expert's group wins: experts 5 and 4
    assert chosen[0].tolist() == [5, 4]
    s = np.exp([0, 0, 0, 0, 0, 3.0]) / np.exp([0, 0, 0, 0, 0, 3.0]).sum()
    assert np.allclose(weights[0], 3.0 * s[[5, 4]])


def test_plain_expert_clamps_before_the_gate():
    t = {"e0.gate": np.array([[10.0], [-10.0]]), "e0.up": np.array([[10.0], [-10.0]]), "e0.down": np.eye(2)}
    y = pn.clamped_expert(np.array([[1.0]]), t, "e0", 2.0)[0]
    assert np.allclose(y[0], 2.0 / (1.0 + np.exp(-1.702 * 2.0)) * 3.0)          # both at the upper limit
    assert np.allclose(y[1], -10.0 / (1.0 + np.exp(17.02)) * (-2.0 + 1.0))       # the gate has no lower limit, the other has


def test_plain_identity_experts_hand_the_row_back():
    cfg = {"router": {"experts": 1, "identity": 1, "top": 1, "scale": 2.0}, "expert": {"limit": 1.0}}
    t = {"router": np.array([[0.0, 0.0], [5.0, 0.0]]), "correction": np.zeros(2), "e0.gate": np.ones((1, 2)), "e0.up": np.ones((1, 2)),
         "e0.down": np.ones((2, 1))}
    h = np.array([[1.0, 3.0]])
    s = 1.0 / (1.0 + np.exp(-5.0))
    assert np.allclose(pn.routed_ff(h, t, cfg), 2.0 * s * h)


def test_plain_difference_of_two_maps():
    # one head, one key: both maps see the same single value, so the difference is (1 - lambda) v, normed and scaled
    t = {"q": np.ones((4, 2)), "k": np.ones((4, 2)), "v": np.eye(2), "q.norm": np.ones(2), "k.norm": np.ones(2), "o": np.eye(2),
         "lq1": np.array([0.5, 0.0]), "lk1": np.array([1.0, 0.0]), "lq2": np.zeros(2), "lk2": np.zeros(2)}
    cfg = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "diff": 0.25}
    lam = np.exp(0.5) - 1.0 + 0.25
    assert np.isclose(pn.difference_factor(t, 0.25), lam)
    out = pn.differential_attention(np.array([[3.0, 4.0]]), t, cfg, 0.0)
    want = np.array([3.0, 4.0]) * (1 - lam)
    assert np.allclose(out[0], want / np.sqrt(np.mean(want ** 2)) * 0.75)
