"""The Nudusun decoder on the device against the plain implementation (tests/plain_nudusun.py): whole prompts, decoding
through cache and state, portions down to two tokens, unequal batches against each sequence alone, slots and pages used
again, long decoding past every window, greedy generation through the library's entry point, the trace runner, and the
kernels of each mechanism alone with inputs made so that a window's edge, a far key, a closed group, an identity expert
or a lost state shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_nudusun as pn
from nudusun_models import CONFIGS, as_float64, write_model
import helpers
from helpers import assert_same_engine, tokens

pytestmark = pytest.mark.gpu

SEEDS = {"mixed": 31, "odd": 32, "wide": 33, "open": 34, "all_experts": 35, "paired": 36}
LENGTHS = {"mixed": 150, "odd": 141, "wide": 270, "open": 90, "all_experts": 230, "paired": 200}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp("nudusun_" + name))
        out[name] = (d, as_float64(write_model(d, cfg, SEEDS[name])))
    return out


_models: dict = {}


def model(folders, name, dtype):
    import camelid_b200
    if (name, dtype) not in _models:
        _models[(name, dtype)] = camelid_b200.load(folders[name][0], dtype=dtype)
    return _models[(name, dtype)]


_plain: dict = {}


def bf16(x):
    return torch.from_numpy(np.asarray(x)).to(torch.bfloat16).to(torch.float64).numpy()


def plain(folders, name, ids):
    """(logits float64 [tokens, vocab]; per row the smallest margin of a router's choice over all routed layers; a
    function that gives the plain logits with 16-bit storage between the steps, computed when first asked for)."""
    key = (name, tuple(ids))
    if key not in _plain:
        margins = []
        logits = pn.forward(CONFIGS[name], folders[name][1], list(ids), margins=margins)
        margin = np.min(np.stack(margins), axis=0) if margins else np.full(len(ids), np.inf)
        kept = []

        def rounded():
            if not kept:
                kept.append(torch.from_numpy(pn.forward(CONFIGS[name], folders[name][1], list(ids), r=bf16)))
            return kept[0]
        _plain[key] = (torch.from_numpy(logits), margin, rounded)
    return _plain[key]


def assert_close(got, reference, dtype, what=""):
    """float32: the library's tolerances on every row. bfloat16: this design norms a row again after most steps (the
    head's difference of two maps, the read-out of a state that holds a few writes, the token input's product of a few
    channels, every residual sum), and where such a row is small by cancellation the norm blows up whatever rounding it
    carries: single rows move ten times as far as the median row, in the plain implementation too once it stores 16 bits
    between the steps. So a row is given the library's bound plus one and a half times the distance that 16-bit storage
    moves that row of the plain implementation, the median row half the bound plus one and a half times the median
    distance. A router scores rows that carry rounding, so a near tie may fall the other way, and every later row moves,
    through a window or a state: rows are held up to the sequence's first near tie, and the rows behind it only to a
    median within a tenth of the largest logit (a lost state or a wrong key moves them by more)."""
    ref, margin, rounded = reference
    got = torch.as_tensor(got)
    if dtype != "bfloat16":
        return helpers.assert_close(got, ref, dtype, what)
    rows, moved = helpers.row_errors(got, ref), helpers.row_errors(rounded(), ref)
    assert float(rows.median()) <= 0.1, f"{what}: the median row is off by {float(rows.median()):.3e}"
    n = len(margin) if np.isinf(margin).all() else int((np.minimum.accumulate(margin) > 0.01).sum())
    if n == 0:
        return
    middle, bound = float(rows[:n].median()), helpers.TOL[dtype] / 2 + 1.5 * float(moved[:n].median())
    assert middle <= bound, f"{what}: the median row before the first near tie is off by {middle:.3e}, more than {bound:.3e}"
    over = rows[:n] - (helpers.TOL[dtype] + 1.5 * moved[:n])
    worst = int(over.argmax())
    assert float(over[worst]) <= 0, (f"{what}: row {worst} is off by {float(rows[worst]):.3e} of its largest logit; 16-bit storage "
                                     f"moves it by {float(moved[worst]):.3e} in the plain implementation")
    mean = helpers.mean_err(got[:n], ref[:n])
    bound = helpers.MEAN_TOL[dtype] + 1.5 * helpers.mean_err(rounded()[:n], ref[:n])
    assert mean <= bound, f"{what}: mean error {mean:.3e} exceeds {bound:.3e}"


# Two cuts of the same work in float32 differ by the order of a few sums; the rows that the norms blow up (above) carry
# thirty times the median row's rounding, so the cuts are held to half the bound against the plain implementation.
CUTS = 5e-5


def run_cut(lm, cache, ids, cut):
    """Feed ``ids`` in portions of the sizes ``cut`` (the rest one by one); logits of every position."""
    from camelid_b200.engine.model import StepEntry
    slot = cache.alloc_slot()
    out, at = [], 0
    sizes = list(cut) + [1] * (len(ids) - sum(cut))
    for n in sizes:
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
    n = len(ids)
    decoded = run_cut(lm, cache, ids, [n - 40])                # the last tokens one by one (captured steps)
    assert_close(decoded, ref, dtype, f"{name} decoded")
    if dtype == "float32":
        assert_same_engine(whole, decoded, f"{name} whole against decoded", tol=CUTS)
    lm.model.check_device_errors()
    cache.book.audit()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_token_decoded_alone_matches_the_prompt(cuda, folders, name):
    """The first tokens of a sequence go through the state and the windows one by one: nothing before them, a
    convolution that still reads its zeros, a window that is not yet full."""
    lm = model(folders, name, "float32")
    ids = tokens(SEEDS[name] + 50, 48, CONFIGS[name]["vocab"])
    cache = lm.new_cache(256)
    one_by_one = run_cut(lm, cache, ids, [])
    assert_close(one_by_one, plain(folders, name, ids), "float32", f"{name} token by token from the first")
    assert_same_engine(run_cut(lm, cache, ids, [len(ids)]), one_by_one, f"{name} prompt against token by token", tol=CUTS)


@pytest.mark.parametrize("name,cut", [("mixed", [7, 2, 3, 2, 50, 1, 1, 2, 64, 2]), ("odd", [64, 2, 63, 1, 2, 5]),
                                      ("open", [1, 2, 2, 3, 70]), ("wide", [2, 126, 2, 3, 128, 2]),
                                      ("all_experts", [2, 2, 97, 100, 3]), ("paired", [99, 2, 64, 3])])
def test_portions_of_a_prompt(cuda, folders, name, cut):
    lm = model(folders, name, "float32")
    ids = tokens(SEEDS[name], LENGTHS[name], CONFIGS[name]["vocab"])
    cache = lm.new_cache(1024)
    got = run_cut(lm, cache, ids, cut)
    assert_close(got, plain(folders, name, ids), "float32", f"{name} in portions {cut}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "paired"])
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
    done = list(prompt)
    live = [0, 1, 2]
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
    """One slot and few pages: every sequence gets the slot, the recurrent state and the convolution's inputs of the one
    before (zeroed when the slot is handed out) and the pages it gave back; the windowed layer gives pages back on the
    way, the layer that sees every key keeps them."""
    lm = model(folders, "open", "float32")
    cache = lm.new_cache(192, max_slots=1)
    for i, n in enumerate((130, 75, 190)):
        ids = tokens(200 + i, n, CONFIGS["open"]["vocab"])
        got = run_cut(lm, cache, ids, [n - 10])
        assert_close(got, plain(folders, "open", ids), "float32", f"sequence {i} in a slot used before")
        cache.book.audit()
    assert cache.book.slots.n_free == 1 and all(p.n_free == p.n for p in cache.book.pools)


def test_long_decoding_past_every_window(cuda, folders):
    lm = model(folders, "wide", "float32")
    ids = tokens(5, 420, CONFIGS["wide"]["vocab"])
    cache = lm.new_cache(512)
    got = run_cut(lm, cache, ids, [3])
    assert_close(got, plain(folders, "wide", ids), "float32", "417 tokens decoded one by one")


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
                ref, margin, _ = plain(folders, "mixed", seq)
                top2 = torch.topk(ref[-1], 2).values
                if dtype == "float32" or (float(top2[0] - top2[1]) > 0.25 and margin.min() > 0.05):
                    assert tok == int(ref[-1].argmax()), (seq, new)
                seq.append(tok)


def test_weights_drawn_on_the_device_match_the_folder(cuda, tmp_path):
    """``from_random`` (what the benchmark uses) and a folder written on the host hold the same model."""
    import camelid_b200
    from camelid_b200.weights.random_init import write_random_model
    cfg = CONFIGS["mixed"]
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=5)
    a = camelid_b200.load(folder, dtype="bfloat16")
    b = camelid_b200.from_random(cfg, seed=5, dtype="bfloat16")
    prompts = [tokens(1, 12, cfg["vocab"]), tokens(2, 3, cfg["vocab"])]
    assert a.generate(prompts, max_tokens=6) == b.generate(prompts, max_tokens=6)


def test_trace_runner_replays_a_nudusun_model(cuda, folders, tmp_path):
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
    ra, rb = plain(folders, "odd", a)[0], plain(folders, "odd", b)[0]
    want = {0: torch.stack([ra[0], ra[32], ra[33], ra[37], rb[0]]), 1: rb[1:2], 2: torch.stack([ra[39], rb[2]]), 3: rb[3:4]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        helpers.assert_close(got, ref, "float32", f"step {i}")


# ---- each mechanism's kernels alone -------------------------------------------------------------

def arrays(cuda, starts, news, slots=None):
    """The packed-row arrays of a step; sequence s sits in slot ``slots[s]`` (its own index unless given)."""
    row_seq = np.repeat(np.arange(len(news)), news)
    row_pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, news)])
    row0 = np.concatenate([[0], np.cumsum(news)[:-1]])
    dev = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.int32, device=cuda)      # noqa: E731
    return {"row_seq": dev(row_seq), "row_pos": dev(row_pos), "seq_row0": dev(row0), "seq_new": dev(news), "seq_start": dev(starts),
            "seq_slot": dev(slots if slots is not None else list(range(len(news))))}


def portions(n, cut):
    sizes = list(cut) + [1] * (n - sum(cut))
    at = 0
    for s in sizes:
        yield at, s
        at += s


def _paged(cuda, T, G, D, Dv, dtype):
    pages = (T + 63) // 64
    order = list(range(pages))[::-1]                                   # pages in another order than positions
    table = torch.tensor([order + [-1]], dtype=torch.int32, device=cuda)
    k = torch.full((pages + 1, G, 64, D), float("nan"), dtype=dtype, device=cuda)
    v = torch.full((pages + 1, G, 64, Dv), float("nan"), dtype=dtype, device=cuda)
    return table, k, v


@pytest.mark.parametrize("cut", [[640], [100, 2, 60, 300, 2], [5]])
@pytest.mark.parametrize("window,cap", [(70, 4.0), (600, 0.0), (0, 9.0), (1, 0.0), (64, 0.0)])
def test_differential_attention_at_a_windows_edge_and_far_back(cuda, cut, window, cap):
    """Keys that every query loves stand at the first positions, at the edges of cache pages and far back, some loved by the
    first score map only, some by the second: a query's output jumps when the key leaves its window, `window` positions
    later and not one earlier. With a window of 600 a loved key at position 2 is found by position 601, among hundreds of
    others, and gone at 602; without a window it is still found at 639. A window of 1 sees the token itself alone. Keys
    and values of different sizes, 3 query heads per kv head, the cap on or off."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(1)
    T, H, G, D, Dv, scale, eps, diff = 640, 6, 2, 24, 40, 0.6, 1e-5, 0.3
    q = torch.randn(T, H, 2, D, generator=gen) * 0.3
    k = torch.randn(T, G, 2, D, generator=gen) * 0.3
    v = torch.randn(T, G * Dv, generator=gen)
    loved = {0: 0, 2: 1, 63: 0, 64: 1, 69: 0, 70: 1, 139: 0, 140: 1, 300: 0, 575: 1}      # position -> the map that loves it
    for j, m in loved.items():
        k[j, :, m] = 0.0
        k[j, :, m, D - 1] = 4.0
    q[:, :, :, D - 1] = 1.5
    qw, kw = 1.0 + 0.3 * torch.randn(D, generator=gen), 1.0 + 0.3 * torch.randn(D, generator=gen)
    lam = {n: 0.4 * torch.randn(D, generator=gen) for n in ("lq1", "lk1", "lq2", "lk2")}
    Wq, Wk, Wv = H * 2 * D, G * 2 * D, G * Dv
    h = torch.cat([q.reshape(T, Wq), k.reshape(T, Wk), v], 1)
    sel = lambda a, n: np.eye(Wq + Wk + Wv)[a:a + n]                     # noqa: E731   the plain projections pick q, k, v out of h
    t = {"q": sel(0, Wq), "k": sel(Wq, Wk), "v": sel(Wq + Wk, Wv), "q.norm": qw.double().numpy(), "k.norm": kw.double().numpy(),
         "o": np.eye(H * Dv), **{n: x.double().numpy() for n, x in lam.items()}}
    cfg = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": scale, "diff": diff}
    if window:
        cfg["mask"] = {"size": window}
    if cap:
        cfg["softcap"] = cap
    ref = torch.from_numpy(pn.differential_attention(h.double().numpy(), t, cfg, eps))
    if window in (70, 600):                                            # the plain result itself shows the edge
        for j in (2, 0):
            if j + window < T:
                assert float((ref[j + window - 1] - ref[j + window]).abs().max()) > 0.05
    factor = pn.difference_factor(t, diff)
    proj = h.to(cuda)
    table, kp, vp = _paged(cuda, T, G, 2 * D, Dv, torch.float32)
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        qo = torch.empty(n, Wq, device=cuda)
        ops.qk_norm_kv_write(proj[at:at + n], qw.to(cuda), kw.to(cuda), eps, a["row_seq"], a["row_pos"], table, qo, kp, vp, H, G, D, Dv, 2)
        out = torch.empty(n, H * Dv, device=cuda)
        ops.window_attention(qo, kp, vp, table, a["row_seq"], a["row_pos"], None, None, None, 0, out, H, G, D, Dv, window, scale,
                             softcap=cap, difference=(factor, eps, 1.0 - diff))
        got.append(out.cpu())
    got = torch.cat(got).double()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) < 3e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("cut", [[640], [100, 2, 60, 300, 2, 113, 63]])
@pytest.mark.parametrize("D,Dv,group,window,cap", [(64, 64, 3, 70, 4.0), (128, 128, 2, 600, 0.0), (64, 128, 1, 0, 9.0),
                                                   (128, 64, 4, 64, 30.0), (64, 128, 2, 600, 50.0)])
def test_differential_attention_of_prompts_on_tensor_cores(cuda, cut, D, Dv, group, window, cap):
    """bfloat16 prompts whose keys (of one map) and values have 64 or 128 channels, alike or not: each score map runs as an attention of its own on the
    tcgen05 kernel (its slice of the key rows, the shared values, the cap inside), and a second kernel takes the difference
    and the norm. Loved keys at the first positions, at page edges and far back, for one map or the other, so that a window
    that is one token off shows; against the plain formula and against the general kernel on the same rows."""
    from camelid_b200.csrc import ops
    from camelid_b200.parts import linear
    gen = torch.Generator().manual_seed(11)
    T, G, scale, eps, diff = 640, 2, 0.5 * D ** -0.5, 1e-5, 0.3
    H = G * group
    q = torch.randn(T, H, 2, D, generator=gen) * 0.3
    k = torch.randn(T, G, 2, D, generator=gen) * 0.3
    v = torch.randn(T, G * Dv, generator=gen)
    loved = {0: 0, 2: 1, 63: 0, 64: 1, 69: 0, 70: 1, 139: 0, 140: 1, 300: 0, 575: 1}
    for j, m in loved.items():
        k[j, :, m] = 0.0
        k[j, :, m, D - 1] = 3.0
    q[:, :, :, D - 1] = 2.0
    qw, kw = 1.0 + 0.3 * torch.randn(D, generator=gen), 1.0 + 0.3 * torch.randn(D, generator=gen)
    lam = {n: 0.1 * torch.randn(D, generator=gen) for n in ("lq1", "lk1", "lq2", "lk2")}
    Wq, Wk, Wv = H * 2 * D, G * 2 * D, G * Dv
    h = torch.cat([q.reshape(T, Wq), k.reshape(T, Wk), v], 1).to(torch.bfloat16).float()
    sel = lambda a, n: np.eye(Wq + Wk + Wv)[a:a + n]                     # noqa: E731
    t = {"q": sel(0, Wq), "k": sel(Wq, Wk), "v": sel(Wq + Wk, Wv), "q.norm": qw.double().numpy(), "k.norm": kw.double().numpy(),
         "o": np.eye(H * Dv), **{n: x.double().numpy() for n, x in lam.items()}}
    cfg = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": scale, "diff": diff}
    if window:
        cfg["mask"] = {"size": window}
    if cap:
        cfg["softcap"] = cap
    ref = torch.from_numpy(pn.differential_attention(h.double().numpy(), t, cfg, eps))
    if window in (70, 600):
        for j in (2, 0):
            assert float((ref[j + window - 1] - ref[j + window]).abs().max()) > 0.3
    factor = pn.difference_factor(t, diff)
    proj = h.to(cuda)
    table, kp, vp = _paged(cuda, T, G, 2 * D, Dv, torch.bfloat16)
    tile_rows, hpc, chunks = ops.attn_tc_tiling(H, G)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=cuda)      # noqa: E731
    got, general = [], []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        qo = torch.empty(n, Wq, dtype=torch.bfloat16, device=cuda)
        ops.qk_norm_kv_write(proj[at:at + n], qw.to(cuda), kw.to(cuda), eps, a["row_seq"], a["row_pos"], table, qo, kp, vp, H, G, D, Dv, 2)
        maps_out = torch.full((n, 2 * H * Dv), float("nan"), device=cuda)
        out = torch.empty(n, H * Dv, dtype=torch.bfloat16, device=cuda)
        assert ops.attn_tc_usable(qo, maps_out, D, Dv)
        tile_q0 = list(range(0, n, tile_rows))
        ops.attn_prefill_tc(qo, maps_out, kp, vp, table, dev([0] * len(tile_q0)), dev(tile_q0), len(tile_q0), a["seq_row0"],
                            a["seq_start"], a["seq_new"], H, G, D, tile_rows, hpc, chunks, window, scale, linear._err_word(cuda),
                            maps=2, softcap=cap, value_dim=Dv)
        ops.maps_difference(maps_out, factor, eps, 1.0 - diff, out, H, Dv)
        got.append(out.cpu())
        out2 = torch.empty_like(out)
        ops.window_attention(qo, kp, vp, table, a["row_seq"], a["row_pos"], None, None, None, 0, out2, H, G, D, Dv, window, scale,
                             softcap=cap, difference=(factor, eps, 1.0 - diff))
        general.append(out2.cpu())
    linear.check_errors()
    got, general = torch.cat(got).double(), torch.cat(general).double()
    assert torch.isfinite(got).all()
    for x, what in ((got, "tensor cores"), (general, "general kernel")):
        err = float((x - ref).abs().max())
        assert err < 6e-2, f"{what}: {err}"
    assert float((got - general).abs().max()) < 6e-2


def test_two_maps_of_one_key_give_nothing_but_the_norms_floor(cuda):
    """When both maps score alike, a1 = a2 and the head's output is (1 - L) a1 normed: its direction is a1's, its size
    the norm's. With L = 1 exactly the difference is zero and eps alone keeps the division finite."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(2)
    T, H, G, D, Dv, eps = 20, 2, 1, 8, 16, 1e-5
    q1, k1 = torch.randn(T, H, 1, D, generator=gen), torch.randn(T, G, 1, D, generator=gen)
    q, k = q1.expand(T, H, 2, D).reshape(T, -1), k1.expand(T, G, 2, D).reshape(T, -1)
    v = torch.randn(T, G * Dv, generator=gen)
    proj = torch.cat([q, k, v], 1).contiguous().to(cuda)
    table, kp, vp = _paged(cuda, T, G, 2 * D, Dv, torch.float32)
    a = arrays(cuda, [0], [T])
    qo = torch.empty(T, H * 2 * D, device=cuda)
    ops.qk_norm_kv_write(proj, None, None, eps, a["row_seq"], a["row_pos"], table, qo, kp, vp, H, G, D, Dv, 2)
    for factor, diff in ((0.25, 0.4), (1.0, 0.2)):
        out = torch.empty(T, H * Dv, device=cuda)
        ops.window_attention(qo, kp, vp, table, a["row_seq"], a["row_pos"], None, None, None, 0, out, H, G, D, Dv, 7, 0.5,
                             difference=(factor, eps, 1.0 - diff))
        s = torch.einsum("thd,jd->thj", q1[:, :, 0].double(), k1[:, 0, 0].double()) * 0.5
        mask = torch.from_numpy(pn.window_mask(T, 7))[:, None, :]
        p = torch.softmax(s.masked_fill(~mask, -np.inf), -1)
        a1 = torch.einsum("thj,jc->thc", p, v.double())
        ref = torch.from_numpy(pn.rms(((1.0 - factor) * a1).numpy(), eps)) * (1.0 - diff)
        # at L = 1 what float32 leaves of a1 - a2 (1e-7 of a1) is divided by sqrt(eps)
        assert torch.allclose(out.cpu().double().view(T, H, Dv), ref, atol=2e-5 if factor != 1.0 else 3e-4)


@pytest.mark.parametrize("cut", [[131], [2, 2, 61, 3, 40], []])
@pytest.mark.parametrize("G,share,D,Dv,taps", [(2, 2, 16, 24, 4), (1, 3, 20, 8, 2), (3, 1, 64, 64, 1), (1, 1, 128, 32, 5)])
def test_gated_delta_rule_kernels_carry_their_state(cuda, cut, G, share, D, Dv, taps):
    """Convolution with SiLU, unit q and k, the decays, the rule itself and the gated norm of the read-out against the
    plain functions: two sequences in one step whose slots are not their order, cut into portions down to two tokens and
    single tokens, so the matrix and the convolution's last inputs pass from step to step. One head's decay is almost 1 (a
    write of the first tokens is still read at the end), one head forgets within a few tokens."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(3)
    H, eps = G * share, 1e-5
    lens = [131, 57]
    qk, vw = G * D, H * Dv
    channels = 2 * qk + vw
    width = channels + H + H + vw                                      # q, k, v, the write strength's, the decay's and the gate's inputs
    projs = [torch.randn(n, width, generator=gen) for n in lens]
    conv_w = 0.25 + 0.3 * torch.randn(channels, taps, generator=gen)
    a_log = torch.linspace(-7.0, 1.0, H)
    dt_bias, norm_w = 0.3 * torch.randn(H, generator=gen), 1.0 + 0.3 * torch.randn(Dv, generator=gen)
    refs = []
    for p in projs:
        x = p.double().numpy()
        n = x.shape[0]
        cw = conv_w.double().numpy()
        c = pn.silu(pn.causal_conv(x[:, :channels], cw))
        q = pn.unit(c[:, :qk].reshape(n, G, D)) * D ** -0.5
        k = pn.unit(c[:, qk:2 * qk].reshape(n, G, D))
        v = c[:, 2 * qk:].reshape(n, H, Dv)
        beta = 1.0 / (1.0 + np.exp(-x[:, channels:channels + H]))
        decay = np.exp(-np.exp(a_log.double().numpy()) * pn.softplus(x[:, channels + H:channels + 2 * H] + dt_bias.double().numpy()))
        o = pn.delta_rule(np.repeat(q, share, 1), np.repeat(k, share, 1), v, beta, decay)
        o = pn.rms(o, eps) * norm_w.double().numpy() * pn.silu(x[:, channels + 2 * H:]).reshape(n, H, Dv)
        refs.append(torch.from_numpy(o.reshape(n, vw)))
    slots = [2, 0]
    memory = torch.zeros(3, H, Dv, D, device=cuda)
    conv_state = torch.zeros(3, max(taps - 1, 1), channels, device=cuda)
    memory[1], conv_state[1] = float("nan"), float("nan")              # a slot that belongs to nobody is never read
    steps = [list(portions(n, [c for c in cut if c <= n])) for n in lens]
    got = [[] for _ in lens]
    for i in range(max(len(s) for s in steps)):
        live = [s for s in range(len(lens)) if i < len(steps[s])]
        starts, news = [steps[s][i][0] for s in live], [steps[s][i][1] for s in live]
        a = arrays(cuda, starts, news, [slots[s] for s in live])
        proj = torch.cat([projs[s][st:st + n] for s, st, n in zip(live, starts, news)]).to(cuda)
        rows = proj.shape[0]
        qkv, decays = torch.empty(rows, channels, device=cuda), torch.empty(rows, H, device=cuda)
        single = all(n == 1 for n in news)
        high = proj[:, channels + H:]
        ops.conv_unit(proj, conv_w.to(cuda), conv_state, a["row_seq"], a["row_pos"], a["seq_row0"], a["seq_slot"], qkv, G, H, D, Dv,
                      D ** -0.5, update_state=single, decay=(high[:, :H], a_log.to(cuda), dt_bias.to(cuda), decays))
        if taps > 1 and not single:
            ops.keep_last_rows(proj, 0, channels, conv_state, a["seq_row0"], a["seq_new"], a["seq_start"], a["seq_slot"], len(live))
        raw = torch.empty(rows, vw, device=cuda)
        ops.delta_scan(qkv, proj, channels, decays, a_log.to(cuda), dt_bias.to(cuda), memory, a["seq_row0"], a["seq_new"],
                       a["seq_start"], a["seq_slot"], raw, len(live), H, G, D, Dv, decay_ready=True)
        out = torch.empty(rows, vw, device=cuda)
        ops.head_norm_gate(raw, False, norm_w.to(cuda), False, high, H, out, H, Dv, eps, gate_silu=True)
        at = 0
        for s, n in zip(live, news):
            got[s].append(out[at:at + n].cpu())
            at += n
    for s, ref in enumerate(refs):
        g = torch.cat(got[s]).double()
        assert torch.isfinite(g).all()
        assert float((g - ref).abs().max()) < 5e-5 * max(1.0, float(ref.abs().max())), f"sequence {s}"


@pytest.mark.parametrize("E,identity,top,groups,shift", [(12, 4, 4, (4, 3), -0.5), (5, 1, 2, (3, 2), 0.0), (7, 2, 2, (3, 1), -1.0),
                                                          (6, 0, 3, None, 0.0), (3, 1, 4, (2, 2), 0.3), (30, 2, 6, (8, 3), -0.2)])
def test_routing_in_groups_with_a_correction(cuda, E, identity, top, groups, shift):
    """The choice is made on softmax scores plus a correction, inside the best groups only, and the weights are the
    uncorrected scores times a factor. With a correction that makes every choice score negative, an expert of a closed
    group must count as minus infinity: counted as zero it would win. Logits as split sums too."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(4)
    rows, W, total = 200, 24, E + identity
    h = torch.randn(rows, W, generator=gen)
    t = {"router": (torch.randn(total, W, generator=gen) * 0.6).double().numpy(),
         "correction": (shift + 0.08 * torch.randn(total, generator=gen)).float().double().numpy()}
    cfg = {"router": {"experts": E, "identity": identity, "top": top, "scale": 1.7}}
    if groups:
        cfg["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    margins = []
    chosen, weights = pn.route(h.double().numpy(), t, cfg, margins)
    logits = (h.double() @ torch.from_numpy(t["router"]).T).float()
    clear = margins[0] > 1e-5
    assert clear.sum() > rows * 0.9
    for parts in (logits[None], torch.stack([logits * 0.25, logits * 0.5, logits * 0.25])):
        ids = torch.empty(rows * top, dtype=torch.int32, device=cuda)
        wts = torch.empty(rows * top, device=cuda)
        ops.route_topk(parts.to(cuda).contiguous(), top, True, False, ids, wts, torch.from_numpy(t["correction"]).float().to(cuda),
                       groups[0] if groups else 1, groups[1] if groups else 1, 1.7)
        ids, wts = ids.cpu().view(rows, top).numpy(), wts.cpu().view(rows, top).double().numpy()
        assert (ids[clear] == chosen[clear]).all()
        assert np.abs(wts[clear] - weights[clear]).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,E,identity,top,ff,limit", [(1, 5, 1, 2, 24, 0.7), (9, 3, 2, 3, 16, 2.0), (300, 4, 3, 2, 48, 1.0),
                                                            (150, 2, 2, 4, 32, 30.0)])
def test_clamped_experts_and_identity_experts(cuda, dtype, rows, E, identity, top, ff, limit):
    """The routed feed-forward from its kernels against the plain one: experts whose gate and up reach the clamps (a small
    limit) and that never do (a large one), identity experts that hand back the row times its weight and own no rows of
    the grouped products, rows that choose identity experts only, experts without rows."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(6)
    W, total = 48, E + identity
    x = torch.randn(rows, W, generator=gen).to(dtype)
    t = {"router": torch.randn(total, W, generator=gen) * 0.5}
    t["router"][E:] += 0.5 * x[0].float()                              # the first row chooses an identity expert
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = torch.randn(ff, W, generator=gen) * 0.3, torch.randn(ff, W, generator=gen) * 0.3
        t[f"e{e}.down"] = torch.randn(W, ff, generator=gen) * 0.2
    t = {n: w.to(dtype) for n, w in t.items()}
    t["router"] = t["router"].float()
    tn = {n: w.double().numpy() for n, w in t.items()}
    cfg = {"router": {"experts": E, "identity": identity, "top": top, "scale": 1.3}, "expert": {"ff": ff, "limit": limit}}
    ref = torch.from_numpy(pn.routed_ff(x.double().numpy(), tn, cfg))
    chosen, _ = pn.route(x.double().numpy(), tn, cfg)
    assert (chosen >= E).any()
    logits = (x.float() @ t["router"].T).to(cuda).contiguous()
    pairs = rows * top
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=cuda)      # noqa: E731
    ids, wts = i32(pairs), torch.empty(pairs, device=cuda)
    ops.route_topk(logits, top, True, False, ids, wts, None, 1, 1, 1.3)
    rank, counts, offsets, tiles, place = i32(pairs), i32(total), i32(total + 1), i32(total + 1), i32(pairs)
    ops.expert_plan(ids, total, rank, counts, offsets, tiles)
    xd = x.to(cuda)
    xs = torch.zeros(pairs, W, dtype=dtype, device=cuda)
    ops.expert_gather(xd, ids, wts, rank, offsets, top, False, xs, place, E)
    stack = lambda n: torch.stack([t[f"e{e}.{n}"] for e in range(E)]).to(cuda).contiguous()      # noqa: E731
    act = torch.zeros(pairs, ff, dtype=dtype, device=cuda)
    gate_act = ops.GateAct(1.702, limit, 1.0)
    ops.expert_gemm(xs, stack("gate"), stack("up"), act, offsets, tiles, gate_act)
    ys = torch.zeros(pairs, W, device=cuda)
    ops.expert_gemm(act, stack("down"), None, ys, offsets, tiles)
    out = torch.empty(rows, W, device=cuda)
    ops.expert_combine(ys, place, wts, top, True, None, out, (ids, E, xd))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((out.double().cpu() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
    if dtype == torch.bfloat16 and ff % 16 == 0:
        # the same through the grouped products on the tensor cores (stretches cut into tiles of 128 rows)
        from camelid_b200.parts import linear
        ops.expert_plan(ids, total, rank, counts, offsets, tiles, ops.EXPERT_TILE_ROWS_TC)
        ops.expert_gather(xd, ids, wts, rank, offsets, top, False, xs, place, E)
        packed = torch.stack([linear.pack_gate_up(t[f"e{e}.gate"], t[f"e{e}.up"], 16) for e in range(E)]).to(cuda).contiguous()
        err = torch.zeros(1, dtype=torch.int32, device=cuda)
        act2, ys2 = torch.zeros_like(act), torch.zeros_like(ys)
        ops.gemm_tc_grouped(xs, packed, act2, ops.TC_SWIGLU, offsets, tiles, err, gate_act)
        ops.gemm_tc_grouped(act2, stack("down"), ys2, ops.TC_STORE_F32, offsets, tiles, err)
        ops.expert_combine(ys2, place, wts, top, True, None, out, (ids, E, xd))
        assert int(err.item()) == 0
        assert float((out.double().cpu() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("width", [40, 37, 256])
def test_norm_after_the_sum_and_the_token_input(cuda, width):
    """x <- rmsnorm(a x + y) * w in place from rows and from split sums, with the rows in bfloat16 beside them; then the
    per-layer token input: the layer's own columns of the second table, GELU of the gate, the product, its norm, the add.
    A width that allows no 16-byte pieces too."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(8)
    rows, eps, alpha, dim, vocab, layer = 7, 1e-5, 1.7, 6, 19, 2
    y = torch.randn(3, rows, width, generator=gen)
    stream, w = torch.randn(rows, width, generator=gen) * 3, 1 + 0.3 * torch.randn(width, generator=gen)
    want = torch.from_numpy(pn.rms((alpha * stream.double() + y.double().sum(0)).numpy(), eps)) * w.double()
    for parts in (y.sum(0), y):
        s, x = stream.to(cuda), torch.empty(rows, width, dtype=torch.bfloat16, device=cuda)
        ops.sum_norm(parts.to(cuda).contiguous(), None, w.to(cuda), eps, alpha, s, x)
        assert torch.allclose(s.cpu().double(), want, atol=2e-5)
        assert torch.equal(x.cpu(), s.cpu().to(torch.bfloat16))
    table = torch.randn(vocab, 4 * dim, generator=gen)
    toks = torch.tensor([3, 18, 0, 7, 7, 11, 5], dtype=torch.int32)
    t = {"gate": torch.randn(dim, width, generator=gen) * 0.3, "proj": torch.randn(width, dim, generator=gen), "norm": w}
    x0 = want.float()
    add = pn.token_input(x0.double().numpy(), toks.numpy(), table.double().numpy(), layer, {n: v.double().numpy() for n, v in t.items()}, dim, eps)
    z = (x0 @ t["gate"].T).to(cuda)
    g = torch.empty(rows, dim, device=cuda)
    ops.gelu_mul_lookup(z, table[:, layer * dim:(layer + 1) * dim].contiguous().to(cuda), 0, toks.to(cuda), g)
    yy = (g.cpu() @ t["proj"].T).to(cuda)
    s = x0.to(cuda)
    ops.post_norm_add(yy, None, w.to(cuda), eps, 1.0, s, None, 0.0, None)
    assert torch.allclose(s.cpu().double(), x0.double() + torch.from_numpy(add), atol=3e-5)


def test_embedding_with_a_multiplier_and_position_rows(cuda):
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(9)
    vocab, width, positions = 23, 44, 50
    table, pos = torch.randn(vocab, width, generator=gen), torch.randn(positions, width, generator=gen)
    toks = torch.tensor([0, 22, 5, 5, 9], dtype=torch.int32, device=cuda)
    row_pos = torch.tensor([0, 49, 7, 8, 1], dtype=torch.int32, device=cuda)
    out, err = torch.empty(5, width, device=cuda), torch.zeros(1, dtype=torch.int32, device=cuda)
    ops.embed_positions(table.to(cuda), toks, 6.5, pos.to(cuda), row_pos, out, err)
    want = 6.5 * table[toks.cpu().long()] + pos[row_pos.cpu().long()]
    assert torch.allclose(out.cpu(), want, atol=1e-6) and int(err.item()) == 0
    ops.embed_positions(table.to(cuda), toks, 6.5, pos.to(cuda), torch.tensor([0, 50, 7, 8, 1], dtype=torch.int32, device=cuda), out, err)
    assert int(err.item()) != 0                                       # a position beyond the table is reported, not read
