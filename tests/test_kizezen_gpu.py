"""The Kizezen decoder on the device against the plain implementation (tests/plain_kizezen.py): whole prompts, decoding
through the cache and the state, portions down to two tokens, unequal batches against each sequence alone, slots and
pages used again, long decoding past every window, greedy generation through the library's entry point, the trace
runner, and the kernels of each mechanism alone with inputs made so that a window's edge, a kept first key, a far key,
the sink or a lost state shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_kizezen as pk
from kizezen_models import CONFIGS, as_float64, write_model
import helpers
from helpers import assert_same_engine, tokens

pytestmark = pytest.mark.gpu

SEEDS = {"mixed": 31, "odd": 32, "wide": 33}
LENGTHS = {"mixed": 150, "odd": 171, "wide": 330}
# bfloat16: a retention state carried over hundreds of tokens and per-head norms without weight pass rounding on, which
# a dense decoder does not; single rows get a wider bound than the library's, the mean error a tight one
BF16_ROW, BF16_MEAN = 8e-2, 6e-3


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp("kizezen_" + name))
        out[name] = (d, as_float64(write_model(d, cfg, SEEDS[name])))
    return out


_models: dict = {}
_plain: dict = {}


def model(folders, name, dtype):
    import camelid_b200
    if (name, dtype) not in _models:
        _models[(name, dtype)] = camelid_b200.load(folders[name][0], dtype=dtype)
    return _models[(name, dtype)]


def plain(folders, name, ids):
    key = (name, tuple(ids))
    if key not in _plain:
        _plain[key] = torch.from_numpy(pk.forward(CONFIGS[name], folders[name][1], list(ids)))
    return _plain[key]


def well_conditioned(cfg, weights, ids, floor=0.005):
    """Rows whose retention read-outs are not just what cancellation left (see `plain_kizezen.retention_core`): the norm
    behind a read-out keeps only its direction, so a first token whose q and k are nearly orthogonal, say, comes out
    with whatever sign rounding gives it in bfloat16."""
    cond = []
    pk.forward(cfg, weights, list(ids), conditioning=cond)
    if not cond:
        return np.ones(len(ids), bool)
    return np.min(np.stack(cond), axis=0) > floor


def assert_close(got, ref, dtype, what="", rows_ok=None):
    if dtype == "float32":
        return helpers.assert_close(got, ref, dtype, what)
    if rows_ok is not None and not rows_ok.all():              # bfloat16: the few ill-conditioned rows are left out
        assert rows_ok.mean() > 0.95, f"{what}: too many ill-conditioned rows for a test"
        keep = torch.from_numpy(np.nonzero(rows_ok)[0])
        got, ref = torch.as_tensor(got)[keep], ref[keep]
    rows = helpers.row_errors(torch.as_tensor(got), ref)
    assert float(rows.max()) <= BF16_ROW, f"{what}: row {int(rows.argmax())} is off by {float(rows.max()):.3e} of its largest logit"
    assert float(rows.median()) <= helpers.TOL[dtype], f"{what}: the median row is off by {float(rows.median()):.3e}"
    m = helpers.mean_err(got, ref)
    assert m <= BF16_MEAN, f"{what}: mean error {m:.3e}"


def run_cut(lm, cache, ids, cut):
    """Feed ``ids`` in portions of the sizes ``cut`` (the rest one by one); logits of every position."""
    from camelid_b200.engine.model import StepEntry
    slot = cache.alloc_slot()
    out, at = [], 0
    for n in list(cut) + [1] * (len(ids) - sum(cut)):
        out.append(lm.step(cache, [StepEntry(slot, ids[at:at + n], list(range(n)))]).cpu())
        at += n
    cache.free_slot(slot)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_decoding_match_plain(cuda, folders, name, dtype):
    lm = model(folders, name, dtype)
    ids = tokens(SEEDS[name], LENGTHS[name], CONFIGS[name]["vocab"])
    ref = plain(folders, name, ids)
    cache = lm.new_cache(1024)
    whole = run_cut(lm, cache, ids, [len(ids)])
    assert_close(whole, ref, dtype, f"{name} whole prompt")
    decoded = run_cut(lm, cache, ids, [len(ids) - 40])         # the last tokens one by one (captured steps)
    assert_close(decoded, ref, dtype, f"{name} decoded")
    if dtype == "float32":
        assert_same_engine(whole, decoded, f"{name} whole against decoded", tol=2e-5)
    lm.model.check_device_errors()
    cache.book.audit()


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(cuda, tmp_path, seed):
    """Sizes, head counts, the order of the layers, windows, kept keys, turned channels and scaling laws drawn from a
    seed: a whole prompt, the same tokens with the last 30 decoded one by one, and two sequences in one batch."""
    import camelid_b200
    from camelid_b200.engine.model import StepEntry
    from kizezen_models import random_config
    cfg = random_config(seed)
    weights = as_float64(write_model(str(tmp_path), cfg, 50 + seed))
    lm = camelid_b200.load(str(tmp_path), dtype="float32")
    ids, short = tokens(seed, 160, cfg["vocab"]), tokens(90 + seed, 21, cfg["vocab"])
    ref, ref_short = torch.from_numpy(pk.forward(cfg, weights, ids)), torch.from_numpy(pk.forward(cfg, weights, short))
    cache = lm.new_cache(512)
    assert_close(run_cut(lm, cache, ids, [len(ids)]), ref, "float32", f"seed {seed} whole prompt")
    assert_close(run_cut(lm, cache, ids, [len(ids) - 30]), ref, "float32", f"seed {seed} decoded")
    a, b = cache.alloc_slot(), cache.alloc_slot()
    both = lm.step(cache, [StepEntry(a, short[:20], list(range(20))), StepEntry(b, ids[:150], list(range(150)))]).cpu()
    one = lm.step(cache, [StepEntry(a, short[20:], [0]), StepEntry(b, ids[150:151], [0])]).cpu()
    assert_close(torch.cat([both[:20], one[:1]]), ref_short, "float32", f"seed {seed} the short sequence of a batch")
    assert_close(torch.cat([both[20:], one[1:]]), ref[:151], "float32", f"seed {seed} the long sequence of a batch")
    cache.free_slot(a)
    cache.free_slot(b)
    cache.book.audit()
    lm.model.check_device_errors()


@pytest.mark.parametrize("seed", range(5))
def test_configurations_for_the_tensor_core_kernels_in_bfloat16(cuda, tmp_path, seed):
    """Drawn configurations whose attention heads and latents have sizes the bfloat16 prompt kernels take: whole prompts,
    portions, decoding and a batch, against the plain implementation at the bounds of bfloat16."""
    import camelid_b200
    from camelid_b200.engine.model import StepEntry
    from kizezen_models import random_config
    cfg = random_config(seed, tensor_cores=True)
    weights = as_float64(write_model(str(tmp_path), cfg, 70 + seed))
    lm = camelid_b200.load(str(tmp_path), dtype="bfloat16")
    ids, short = tokens(seed, 300, cfg["vocab"]), tokens(90 + seed, 21, cfg["vocab"])
    ref, ref_short = torch.from_numpy(pk.forward(cfg, weights, ids)), torch.from_numpy(pk.forward(cfg, weights, short))
    ok, ok_short = well_conditioned(cfg, weights, ids), well_conditioned(cfg, weights, short)
    cache = lm.new_cache(1024)
    assert_close(run_cut(lm, cache, ids, [len(ids)]), ref, "bfloat16", f"seed {seed} whole prompt", ok)
    assert_close(run_cut(lm, cache, ids, [130, 2, 138]), ref, "bfloat16", f"seed {seed} portions and decoding", ok)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    both = lm.step(cache, [StepEntry(a, short[:20], list(range(20))), StepEntry(b, ids[:290], list(range(290)))]).cpu()
    one = lm.step(cache, [StepEntry(a, short[20:], [0]), StepEntry(b, ids[290:291], [0])]).cpu()
    assert_close(torch.cat([both[:20], one[:1]]), ref_short, "bfloat16", f"seed {seed} the short sequence of a batch", ok_short)
    assert_close(torch.cat([both[20:], one[1:]]), ref[:291], "bfloat16", f"seed {seed} the long sequence of a batch", ok[:291])
    cache.free_slot(a)
    cache.free_slot(b)
    lm.model.check_device_errors()


def test_every_token_decoded_alone(cuda, folders):
    """From the first token on: the first tokens of a sequence, the kept keys and the windows as they fill."""
    for name in ("mixed", "odd"):
        lm = model(folders, name, "float32")
        ids = tokens(7, 100, CONFIGS[name]["vocab"])
        got = run_cut(lm, lm.new_cache(256), ids, [])
        assert_close(got, plain(folders, name, ids), "float32", f"{name} token by token")


@pytest.mark.parametrize("name,cut", [("mixed", [7, 2, 3, 2, 50, 1, 1, 2, 64, 2]), ("odd", [64, 2, 63, 1, 2, 5]),
                                      ("wide", [2, 126, 2, 3, 128, 2, 60]), ("odd", [1, 2, 2, 3, 70, 71])])
def test_portions_of_a_prompt(cuda, folders, name, cut):
    lm = model(folders, name, "float32")
    ids = tokens(SEEDS[name], LENGTHS[name], CONFIGS[name]["vocab"])
    got = run_cut(lm, lm.new_cache(1024), ids, cut)
    assert_close(got, plain(folders, name, ids), "float32", f"{name} in portions {cut}")


def test_portions_in_bfloat16_on_the_tensor_core_attention(cuda, folders):
    lm = model(folders, "wide", "bfloat16")
    ids = tokens(SEEDS["wide"], LENGTHS["wide"], CONFIGS["wide"]["vocab"])
    got = run_cut(lm, lm.new_cache(1024), ids, [150, 2, 70, 100])
    assert_close(got, plain(folders, "wide", ids), "bfloat16", "wide in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
def test_unequal_batch_against_each_alone(cuda, folders, name, dtype):
    """Prompts of 1, 17 and 135 tokens start together, are decoded together and end one after the other."""
    from camelid_b200.engine.model import StepEntry
    lm = model(folders, name, dtype)
    vocab = CONFIGS[name]["vocab"]
    seqs = [tokens(100 + i, n, vocab) for i, n in enumerate((9, 30, 150))]
    prompt = [1, 17, 135]
    cache = lm.new_cache(1024)
    slots = [cache.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    logits = lm.step(cache, [StepEntry(s, q[:p], list(range(p))) for s, q, p in zip(slots, seqs, prompt)]).cpu()
    at = 0
    for i, p in enumerate(prompt):
        got[i].append(logits[at:at + p])
        at += p
    done, live = list(prompt), [0, 1, 2]
    while live:
        logits = lm.step(cache, [StepEntry(slots[i], [seqs[i][done[i]]], [0]) for i in live]).cpu()
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
            done[i] += 1
        for i in [i for i in live if done[i] == len(seqs[i])]:
            cache.free_slot(slots[i])
        live = [i for i in live if done[i] < len(seqs[i])]
    for i, q in enumerate(seqs):
        assert_close(torch.cat(got[i]), plain(folders, name, q), dtype, f"{name} sequence {i} of a batch")
    cache.book.audit()


def test_slots_and_pages_used_again(cuda, folders):
    """A cache of four pages and one slot: every sequence gets the slot, the state and the pages the one before gave
    back. The windowed layers give old pages back on the way but hold on to those of their kept first keys."""
    lm = model(folders, "odd", "float32")
    cache = lm.new_cache(256, max_slots=1)
    for i, n in enumerate((200, 75, 250)):
        ids = tokens(200 + i, n, CONFIGS["odd"]["vocab"])
        got = run_cut(lm, cache, ids, [n - 10])
        assert_close(got, plain(folders, "odd", ids), "float32", f"sequence {i} in a slot used before")
        cache.book.audit()
    assert cache.book.slots.n_free == 1 and all(p.n_free == p.n for p in cache.book.pools)


def test_long_decoding_past_every_window(cuda, folders):
    lm = model(folders, "mixed", "float32")
    ids = tokens(5, 300, CONFIGS["mixed"]["vocab"])
    got = run_cut(lm, lm.new_cache(512), ids, [3])
    assert_close(got, plain(folders, "mixed", ids), "float32", "297 tokens decoded one by one")
    lm = model(folders, "wide", "float32")
    ids = tokens(6, 300, CONFIGS["wide"]["vocab"])
    got = run_cut(lm, lm.new_cache(512), ids, [190])
    assert_close(got, plain(folders, "wide", ids), "float32", "110 tokens decoded past windows of 130 and 64")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(cuda, folders, dtype):
    """``generate`` (scheduler, batches, the decode loop on the device) picks the plain implementation's tokens."""
    lm = model(folders, "mixed", dtype)
    cfg = CONFIGS["mixed"]
    prompts = [tokens(300, 5, cfg["vocab"]), tokens(301, 19, cfg["vocab"]), tokens(302, 1, cfg["vocab"])]
    for _ in range(2):                                         # the second call uses the slots again
        out = lm.generate(prompts, max_tokens=12)
        for p, new in zip(prompts, out):
            assert len(new) == 12
            seq = list(p)
            for tok in new:
                ref = plain(folders, "mixed", seq)
                top2 = torch.topk(ref[-1], 2).values
                if dtype == "float32" or float(top2[0] - top2[1]) > 0.25:
                    assert tok == int(ref[-1].argmax()), (seq, new)
                seq.append(tok)


def test_weights_drawn_on_the_device_match_the_folder(cuda, tmp_path):
    import camelid_b200
    from camelid_b200.weights.random_init import write_random_model
    cfg = CONFIGS["mixed"]
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=5)
    a = camelid_b200.load(folder, dtype="bfloat16")
    b = camelid_b200.from_random(cfg, seed=5, dtype="bfloat16")
    prompts = [tokens(1, 12, cfg["vocab"]), tokens(2, 3, cfg["vocab"])]
    assert a.generate(prompts, max_tokens=6) == b.generate(prompts, max_tokens=6)


def test_trace_runner_replays_a_kizezen_model(cuda, folders, tmp_path):
    folder, _ = folders["odd"]
    cfg = CONFIGS["odd"]
    a, b = tokens(1, 40, cfg["vocab"]), tokens(2, 4, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:38], "want": [0, 32, 33, 37]}, {"id": "b", "tokens": b[:1], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[38:39], "want": []}, {"id": "b", "tokens": b[1:2], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[39:40], "want": [0]}, {"id": "b", "tokens": b[2:3], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[3:4], "want": [0]}], "end": ["b"]}]
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", folder, "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain(folders, "odd", a), plain(folders, "odd", b)
    want = {0: torch.stack([ra[0], ra[32], ra[33], ra[37], rb[0]]), 1: rb[1:2], 2: torch.stack([ra[39], rb[2]]), 3: rb[3:4]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        helpers.assert_close(got, ref, "float32", f"step {i}")


# ---- each mechanism's kernels alone -------------------------------------------------------------

def arrays(cuda, starts, news, slots=None):
    """The packed-row arrays of a step."""
    dev = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.int32, device=cuda)      # noqa: E731
    row0 = np.concatenate([[0], np.cumsum(news)[:-1]])
    return {"row_seq": dev(np.repeat(np.arange(len(news)), news)),
            "row_pos": dev(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, news)])),
            "seq_row0": dev(row0), "seq_new": dev(news), "seq_start": dev(starts),
            "seq_slot": dev(slots if slots is not None else np.arange(len(news)))}


def portions(n, cut):
    at = 0
    for s in list(cut) + [1] * (n - sum(cut)):
        yield at, s
        at += s


def _paged(cuda, T, G, D, Dv, dtype):
    pages = (T + 63) // 64
    order = list(range(pages))[::-1]                                   # pages in another order than positions
    table = torch.tensor([order + [-1]], dtype=torch.int32, device=cuda)
    k = torch.full((pages + 1, G, 64, D), float("nan"), dtype=dtype, device=cuda)
    v = torch.full((pages + 1, G, 64, Dv), float("nan"), dtype=dtype, device=cuda) if Dv else k
    return table, k, v


def _windowed_case(T, H, G, D, Dv, window, kept, rot, seed=1):
    """Inputs in which some keys are loved by every query: inside and just outside the kept first keys, at the window's
    edge as seen from later rows, at page borders and far back. Returns the plain result as well."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H * D, generator=gen) * 0.3
    k = torch.randn(T, G * D, generator=gen) * 0.3
    v = torch.randn(T, G * Dv, generator=gen)
    loved = sorted({0, kept - 1, kept, 63, 64, 65, 127, 128, T - window - 1, T - window, T - window + 1} & set(range(T)))
    for j in loved:                                                    # a channel outside the turned ones stands out
        k.view(T, G, D)[j] = 0.0
        k.view(T, G, D)[j, :, D - 1] = 6.0
    q.view(T, H, D)[:, :, D - 1] = 2.0
    sink = torch.linspace(-3.0, 3.0, H)
    gate = torch.randn(T, H, generator=gen)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.5, "mask": {"size": window, "keep_first": kept}}
    if rot:
        m["rot"] = {"dims": rot, "base": 50.0}
    ref = pk.attention_core(q.double().numpy(), k.double().numpy(), v.double().numpy(), gate.double().numpy(),
                            sink.double().numpy(), m)
    return q, k, v, gate, sink, m, torch.from_numpy(ref)


@pytest.mark.parametrize("cut", [[400], [100, 2, 60, 130, 2], [5]])
@pytest.mark.parametrize("window,kept", [(70, 20), (33, 65), (5, 12), (200, 0), (64, 64), (1, 1)])
def test_window_with_kept_first_keys(cuda, cut, window, kept):
    """A key that every query loves is seen while it is inside the window or among the kept first keys and not a row
    longer; the rows' outputs jump where it leaves. Prompts, portions and single tokens; three query heads per kv head."""
    from camelid_b200.csrc import ops
    T, H, G, D, Dv, rot = 400, 6, 2, 24, 40, 8
    q, k, v, gate, sink, m, ref = _windowed_case(T, H, G, D, Dv, window, kept, rot)
    if kept and kept + window < T:                                     # the first key outside the kept ones is lost one row later
        assert float((ref[kept + window - 1] - ref[kept + window]).abs().max()) > 0.05
    proj = torch.cat([q, k, v, gate], 1).to(cuda)
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=cuda)
    table, kp, vp = _paged(cuda, T, G, D, Dv, torch.float32)
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        qo = torch.empty(n, H * D, device=cuda)
        ops.qkv_prepare(proj[at:at + n], None, None, 0, 0.0, inv_freq, rot, False, a["row_seq"], a["row_pos"], table, qo, kp, vp,
                        H, G, D, Dv)
        out = torch.empty(n, H * Dv, device=cuda)
        ops.window_attention(qo, kp, vp, table, a["row_seq"], a["row_pos"], None, None, proj[at:at + n], H * D + G * D + G * Dv,
                             out, H, G, D, Dv, window, 0.5, sink=sink.to(cuda), gate_per_head=True, keep_first=kept)
        got.append(out.cpu())
    got = torch.cat(got).double()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) < 2e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,Dv,group,window,kept", [(64, 64, 3, 70, 20), (128, 128, 2, 200, 65), (128, 64, 1, 33, 130),
                                                    (64, 128, 4, 130, 64)])
def test_prompt_attention_on_tensor_cores_with_kept_first_keys(cuda, D, Dv, group, window, kept):
    """The tcgen05 prompt kernel with a window, kept first keys, sink and gate against the plain attention and the
    general kernel: a whole prompt and a portion that starts mid-sequence."""
    from camelid_b200.csrc import ops
    from camelid_b200.parts import linear
    T, G = 450, 2
    H = G * group
    q, k, v, gate, sink, m, ref = _windowed_case(T, H, G, D, Dv, window, kept, 0, seed=3)
    m["scale"] = 0.125
    q, k, v = (x.to(torch.bfloat16).float() for x in (q, k, v))         # what the kernels are given
    ref = torch.from_numpy(pk.attention_core(q.double().numpy(), k.double().numpy(), v.double().numpy(), gate.double().numpy(),
                                             sink.double().numpy(), m))
    bf = torch.bfloat16
    table, kp, vp = _paged(cuda, T, G, D, Dv, bf)
    qd, gd = q.to(cuda, bf), gate.to(cuda)
    a = arrays(cuda, [0], [T])
    kp.zero_(); vp.zero_()
    pages = table[0].tolist()
    for j in range(T):
        kp[pages[j // 64], :, j % 64] = k.view(T, G, D)[j].to(cuda, bf)
        vp[pages[j // 64], :, j % 64] = v.view(T, G, Dv)[j].to(cuda, bf)
    general = torch.empty(T, H * Dv, device=cuda, dtype=bf)
    ops.window_attention(qd, kp, vp, table, a["row_seq"], a["row_pos"], None, None, gd, 0, general, H, G, D, Dv, window, 0.125,
                         sink=sink.to(cuda), gate_per_head=True, keep_first=kept)
    rows, hpc, chunks = ops.attn_tc_tiling(H, G)
    for start in (0, 190):
        n = T - start
        tiles = [(0, q0) for q0 in range(0, n, rows)]
        tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device=cuda)
        tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device=cuda)
        b = arrays(cuda, [start], [n])
        out = torch.empty(n, H * Dv, device=cuda, dtype=bf)
        ops.attn_prefill_tc(qd[start:], out, kp, vp, table, tile_seq, tile_q0, len(tiles), b["seq_row0"], b["seq_start"],
                            b["seq_new"], H, G, D, rows, hpc, chunks, window, 0.125, linear._err_word(cuda), None, None, 0,
                            sink.to(cuda), gd[start:], 0, 1, 0.0, Dv, kept)
        torch.cuda.synchronize()
        linear.check_errors()
        got = out.double().cpu()
        scale = max(1.0, float(ref.abs().max()))
        assert float((got - ref[start:]).abs().max()) < 3e-2 * scale, (start, float((got - ref[start:]).abs().max()))
        assert float((got - general[start:].double().cpu()).abs().max()) < 3e-2 * scale


def test_sink_alone_takes_its_share(cuda):
    """One key with score 0 beside a sink of ln 3: the output is a quarter of the value."""
    from camelid_b200.csrc import ops
    H, D, Dv = 2, 16, 8
    table, kp, vp = _paged(cuda, 1, 1, D, Dv, torch.float32)
    kp.zero_()
    vp.fill_(4.0)
    a = arrays(cuda, [0], [1])
    out = torch.empty(1, H * Dv, device=cuda)
    sink = torch.tensor([np.log(3.0), -np.inf], dtype=torch.float32, device=cuda)
    ops.window_attention(torch.ones(1, H * D, device=cuda), kp, vp, table, a["row_seq"], a["row_pos"], None, None, None, 0, out,
                         H, 1, D, Dv, 5, 1.0, sink=sink, keep_first=3)
    assert torch.allclose(out.cpu(), torch.tensor([[1.0] * Dv + [4.0] * Dv]), atol=1e-6)


def test_projection_biases_and_scaled_rotation_in_the_preparation_kernel(cuda):
    """Biases are added to the summed splits before the norm over the whole projection; sines and cosines carry an
    amplitude; pairs of halves."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(2)
    T, H, G, D, Dv, rot, eps, amp = 70, 3, 1, 12, 20, 6, 1e-5, 1.3
    width = H * D + G * D + G * Dv
    parts = torch.randn(3, T, width + H, generator=gen)
    bias = torch.randn(width + H, generator=gen)
    bias[width:] = 0.0
    qw, kw = 1 + 0.3 * torch.randn(H * D, generator=gen), 1 + 0.3 * torch.randn(G * D, generator=gen)
    rows = (parts.sum(0) + bias).double().numpy()
    freq = np.array([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)])
    qn = pk.turn(pk.rms_norm(rows[:, :H * D], qw.double().numpy(), eps).reshape(T, H, D), np.arange(T), freq, amp, rot, "half")
    kn = pk.turn(pk.rms_norm(rows[:, H * D:H * D + G * D], kw.double().numpy(), eps).reshape(T, G, D), np.arange(T), freq, amp, rot, "half")
    table, kp, vp = _paged(cuda, T, G, D, Dv, torch.float32)
    a = arrays(cuda, [0], [T])
    qo = torch.empty(T, H * D, device=cuda)
    extra = torch.empty(T, H, device=cuda)
    ops.qkv_prepare(parts.to(cuda), qw.to(cuda), kw.to(cuda), 2, eps, torch.tensor(freq, dtype=torch.float32, device=cuda), rot,
                    False, a["row_seq"], a["row_pos"], table, qo, kp, vp, H, G, D, Dv, extra, bias.to(cuda), amp)
    pages = table[0].tolist()
    k_got = torch.stack([kp[pages[j // 64], :, j % 64] for j in range(T)]).cpu().double()
    v_got = torch.stack([vp[pages[j // 64], :, j % 64] for j in range(T)]).cpu().double()
    assert float((qo.cpu().double() - torch.from_numpy(qn.reshape(T, -1))).abs().max()) < 1e-5
    assert float((k_got - torch.from_numpy(kn)).abs().max()) < 1e-5
    assert float((v_got.reshape(T, -1) - torch.from_numpy(rows[:, H * D + G * D:width])).abs().max()) < 1e-5
    assert float((extra.cpu().double() - torch.from_numpy(rows[:, width:])).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("cut", [[330], [100, 2, 60, 130, 2], [3]])
def test_latent_attention_finds_a_far_key(cuda, cut, dtype, tol):
    """The kernels of the attention over a latent, from the projections' rows on: the latent of position 2 is what the
    queries of the last rows ask for, among hundreds of others; the turned part alone decides at position 5. Prompts,
    portions and single tokens give the same rows."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(4)
    T, H, D, R, Dv, C, eps = 330, 3, 16, 8, 12, 40, 1e-5
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": C, "scale": 0.3,
         "rot": {"dims": R, "base": 50.0, "scaling": {"factor": 4.0, "fast": 8.0, "slow": 1.0, "original": 16}}}
    t = {"uk": torch.randn(H * D, C, generator=gen) / C ** 0.5, "uv": torch.randn(H * Dv, C, generator=gen) / C ** 0.5,
         "dkv.norm": 1 + 0.3 * torch.randn(C, generator=gen), "sink": torch.tensor([-2.0, 0.0, 2.0])}
    t = {n: x.to(torch.bfloat16).double() for n, x in t.items()}
    q = torch.randn(T, H * (D + R), generator=gen) * 0.3
    down = torch.randn(T, C + R, generator=gen)
    gate = torch.randn(T, H, generator=gen)
    # the last rows' unturned queries point at head h's key of position 2
    c2 = pk.rms_norm(down[2:3, :C].double().numpy(), t["dkv.norm"].numpy(), eps)[0]
    k2 = (t["uk"].numpy() @ c2).reshape(H, D)
    q.view(T, H, D + R)[300:, :, :D] = torch.from_numpy(k2).float() * 3.0
    tn = {n: x.numpy() for n, x in t.items()}
    ref = torch.from_numpy(pk.latent_core(q.double().numpy(), down.double().numpy(), gate.double().numpy(), tn, m, eps))
    lost = dict(m)
    without = pk.latent_core(q.double().numpy()[3:], down.double().numpy()[3:], gate.double().numpy()[3:], tn, lost, eps,
                             positions=np.arange(3, T))
    assert float(np.abs(without[-1] - ref[-1].numpy()).max()) > 0.05          # the far key matters to the last row
    freq, amp = pk.frequencies(m["rot"])
    inv_freq = torch.tensor(freq, dtype=torch.float32, device=cuda)
    proj = torch.cat([q, down, gate], 1).to(cuda)
    table, kp, _ = _paged(cuda, T, 1, C + R, 0, dtype)
    uk_t = t["uk"].view(H, D, C).transpose(1, 2).contiguous().to(cuda, dtype)
    uv = t["uv"].view(H, Dv, C).contiguous().to(cuda, dtype)
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        q_plain = torch.empty(n, H * D, device=cuda, dtype=dtype)
        q_full = torch.empty(n, H * (C + R), device=cuda, dtype=dtype)
        g = torch.empty(n, H, device=cuda)
        ops.latent_prepare(proj[at:at + n], t["dkv.norm"].float().to(cuda), eps, inv_freq, True, amp, a["row_seq"], a["row_pos"],
                           table, q_plain, q_full, kp, H, D, R, C, g)
        ops.head_product(q_plain, D, uk_t, q_full, C + R)
        mixed = torch.empty(n, H * C, device=cuda, dtype=dtype)
        ops.window_attention(q_full, kp, kp, table, a["row_seq"], a["row_pos"], None, None, g, 0, mixed, H, 1, C + R, C, 0, 0.3,
                             sink=t["sink"].float().to(cuda), gate_per_head=True, values_in_keys=True)
        out = torch.empty(n, H * Dv, device=cuda, dtype=dtype)
        ops.head_product(mixed, C, uv, out, Dv)
        got.append(out.cpu())
    got = torch.cat(got).double()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("rows,heads,n,k", [(1, 3, 40, 16), (70, 2, 7, 18), (33, 5, 130, 70), (16, 4, 24, 512), (8, 2, 130, 36),
                                            (200, 3, 96, 48), (65, 2, 512, 128), (130, 2, 70, 512)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_product_per_head(cuda, rows, heads, n, k, dtype):
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(rows, heads * k + 8, generator=gen).to(dtype)
    w = torch.randn(heads, n, k, generator=gen).to(dtype)
    out = torch.zeros(rows, heads * (n + 5), dtype=dtype, device=cuda)
    ops.head_product(x.to(cuda), k, w.to(cuda), out, n + 5)
    ref = torch.einsum("rhk,hnk->rhn", x[:, :heads * k].double().view(rows, heads, k), w.double())
    got = out.cpu().double().view(rows, heads, n + 5)
    assert float((got[:, :, :n] - ref).abs().max()) < (1e-4 if dtype == torch.float32 else 5e-2) * float(ref.abs().max())
    assert float(got[:, :, n:].abs().max()) == 0.0


@pytest.mark.parametrize("D,Dv,rot", [(24, 40, 16), (128, 64, 128), (20, 4, 0), (64, 130, 32)])
def test_retention_keeps_a_far_key_through_portions_and_slots(cuda, D, Dv, rot):
    """A head that barely decays is asked at row 290 for the key written at row 2; a head that halves its state every
    token has forgotten it. Portions and single tokens, two sequences side by side, in slots that held other states."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(6)
    T, decay = 300, (0.9995, 0.5, 1.0)
    H = len(decay)
    m = {"heads": H, "dim": D, "vdim": Dv, "decay": decay}
    if rot:
        m["rot"] = {"dims": rot, "base": 100.0}
    seqs = []
    for s in range(2):
        q, k = torch.randn(T, H, D, generator=gen) * 0.3, torch.randn(T, H, D, generator=gen) * 0.3
        v = torch.randn(T, H * Dv, generator=gen)
        if not rot:                                # (with rotation a fixed direction does not survive 288 positions)
            q[290] = k[2] * 8.0
        seqs.append((q.reshape(T, -1), k.reshape(T, -1), v))
    refs = [torch.from_numpy(pk.retention_core(q.double().numpy(), k.double().numpy(), v.double().numpy(), m).reshape(T, -1))
            for q, k, v in seqs]
    if not rot:
        assert float(refs[0][290, :Dv].abs().max()) > 3 * float(refs[0][289, :Dv].abs().max())
    state = torch.full((4, H, Dv, D), 7.0, device=cuda)                 # slots that held something else
    dec = torch.tensor(decay, dtype=torch.float64).float().to(cuda)
    inv_freq = torch.tensor([100.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32, device=cuda)
    got = [[], []]
    cuts = ([150, 2, 100], [7, 64, 3])
    plans = [list(portions(T, c)) for c in cuts]
    # the two sequences' portions differ, so steps mix a portion of one with single tokens of the other
    at = [0, 0]
    while at[0] < T or at[1] < T:
        live = [s for s in range(2) if at[s] < T]
        news = [next(n for a0, n in plans[s] if a0 == at[s]) for s in live]
        a = arrays(cuda, [at[s] for s in live], news, slots=[3 - s for s in live])
        proj = torch.cat([torch.cat([seqs[s][i][at[s]:at[s] + n] for i in range(3)], 1) for s, n in zip(live, news)]).to(cuda)
        ops.rotate_rows_(proj, 0, 2 * H, D, rot, False, inv_freq, 1.0, a["row_pos"], H, D ** -0.5)
        out = torch.empty(proj.shape[0], H * Dv, device=cuda)
        ops.retention_scan(proj, (0, H * D, 2 * H * D), dec, state, a["seq_row0"], a["seq_new"], a["seq_start"], a["seq_slot"],
                           out, len(live), H, D, Dv)
        r0 = 0
        for s, n in zip(live, news):
            got[s].append(out[r0:r0 + n].cpu())
            r0 += n
            at[s] += n
    for s in range(2):
        g = torch.cat(got[s]).double()
        assert torch.isfinite(g).all()
        assert float((g - refs[s]).abs().max()) < 3e-5 * max(1.0, float(refs[s].abs().max())), s


def test_head_norm_without_weight_and_exact_gelu(cuda):
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(8)
    rows, H, Dv, eps = 9, 3, 20, 1e-5
    raw, gate = torch.randn(rows, H * Dv, generator=gen) * 5, torch.randn(rows, H * Dv + 4, generator=gen)
    out = torch.empty(rows, H * Dv, device=cuda)
    ops.head_norm_gate(raw.to(cuda), False, None, False, gate.to(cuda), 4, out, H, Dv, eps, gate_silu=True)
    ref = pk.rms_norm(raw.double().numpy().reshape(rows, H, Dv), None, eps).reshape(rows, -1) * pk.silu(gate.double().numpy()[:, 4:])
    assert float((out.cpu().double() - torch.from_numpy(ref)).abs().max()) < 1e-5
    x = torch.linspace(-6, 6, 96).reshape(4, 24)
    y = x.to(cuda).clone()
    ops.bias_act_(y, None, ops.ACT_GELU_ERF)
    assert float((y.cpu().double() - torch.from_numpy(pk.gelu_erf(x.double().numpy()))).abs().max()) < 1e-6
    part = torch.randn(3, 4, 24, generator=gen)
    y2 = torch.empty(4, 24, device=cuda)
    ops.act_from_partials(part.to(cuda), y2, act=ops.ACT_GELU_ERF)
    assert float((y2.cpu().double() - torch.from_numpy(pk.gelu_erf(part.sum(0).double().numpy()))).abs().max()) < 1e-5


@pytest.mark.parametrize("H,C,R", [(3, 32, 16), (4, 128, 32), (8, 96, 0), (70, 64, 16), (16, 512, 64)])
def test_latent_prompts_on_tensor_cores(cuda, H, C, R):
    """The prompt kernel of the attention over a latent against the plain softmax and the general kernel: two sequences
    in one step, the first a portion that starts at position 150 of its sequence; sink and gate; a loved key far back."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(9)
    bf = torch.bfloat16
    D, scale = C + R, 0.2
    lens, starts = [230, 67], [150, 0]
    total = [s + n for s, n in zip(starts, lens)]
    qs = [(torch.randn(t, H, D, generator=gen) * 0.4).to(bf) for t in total]
    ks = [(torch.randn(t, D, generator=gen) * 0.4).to(bf) for t in total]
    ks[0][3] = 0
    ks[0][3, 0] = 6.0
    qs[0][:, :, 0] = 2.0
    sink = torch.linspace(-2.0, 2.0, H)
    gates = [torch.randn(t, H, generator=gen) for t in total]
    refs = []
    for q, k, g, t, st in zip(qs, ks, gates, total, starts):
        out = np.zeros((t, H, C))
        see = pk.visible(t)
        for h in range(H):
            w = pk.sink_softmax(q[:, h].double().numpy() @ k.double().numpy().T * scale, see, float(sink[h]))
            out[:, h] = (w @ k[:, :C].double().numpy()) * pk.sigmoid(g[:, h:h + 1].double().numpy())
        refs.append(torch.from_numpy(out.reshape(t, H * C))[st:])
    ref = torch.cat(refs)
    pages = [(t + 63) // 64 for t in total]
    table = torch.full((2, max(pages)), -1, dtype=torch.int32)
    table[0, :pages[0]] = torch.arange(pages[0]) + pages[1]
    table[1, :pages[1]] = torch.arange(pages[1])
    kp = torch.zeros(sum(pages), 1, 64, D, dtype=bf)
    for s in range(2):
        for j in range(total[s]):
            kp[int(table[s, j // 64]), 0, j % 64] = ks[s][j]
    kp, table = kp.to(cuda), table.to(cuda)
    a = arrays(cuda, starts, lens)
    q = torch.cat([x[st:].reshape(t - st, -1) for x, t, st in zip(qs, total, starts)]).to(cuda)
    gate = torch.cat([x[st:] for x, st in zip(gates, starts)]).to(cuda)
    tpt = ops.latent_prompt_tokens(H)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=cuda)      # noqa: E731
    tile_seq = [s for s, n in enumerate(lens) for _ in range(0, n, tpt)]
    tile_q0 = [q0 for n in lens for q0 in range(0, n, tpt)]
    assert ops.latent_prompt_usable(q, C, R)
    assert not ops.latent_prompt_usable(q, 512, 128) and not ops.latent_prompt_usable(q, 40, 16) and not ops.latent_prompt_usable(q.float(), C, R)
    out = torch.empty(sum(lens), H * C, dtype=bf, device=cuda)
    ops.latent_prompt(q, kp, out, table, dev(tile_seq), dev(tile_q0), len(tile_seq), a["seq_row0"], a["seq_start"], a["seq_new"],
                      H, C, R, scale, sink.to(cuda), gate, 0)
    general = torch.empty_like(out)
    ops.window_attention(q, kp, kp, table, a["row_seq"], a["row_pos"], None, None, gate, 0, general, H, 1, D, C, 0, scale,
                         sink=sink.to(cuda), gate_per_head=True, values_in_keys=True)
    top = max(1.0, float(ref.abs().max()))
    for got, what in ((out, "tensor cores"), (general, "general kernel")):
        err = float((got.cpu().double() - ref).abs().max())
        assert err < 2e-2 * top, f"{what}: {err}"
    # the sequences' last tokens alone, their pages dealt to three blocks each (the shorter sequence leaves two of them empty)
    last = [lens[0] - 1, sum(lens) - 1]
    b = arrays(cuda, [t - 1 for t in total], [1, 1])
    partial = torch.full((3, 2, H, C + 2), float("nan"), device=cuda)
    one = torch.empty(2, H * C, dtype=bf, device=cuda)
    ops.latent_prompt(q[last].contiguous(), kp, one, table, dev([0, 1]), dev([0, 0]), 2, b["seq_row0"], b["seq_start"], b["seq_new"],
                      H, C, R, scale, sink.to(cuda), gate[last].contiguous(), 0, partial, 2)
    err = float((one.cpu().double() - ref[last]).abs().max())
    assert err < 2e-2 * top, f"single tokens in three shares: {err}"
