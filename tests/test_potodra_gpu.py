"""The Potodra decoder in the engine against the plain implementation (tests/plain_potodra.py): each mechanism alone,
whole prompts against token-by-token decoding, portions, unequal batches with slots, pages and state rows used again,
keys far back, at page borders, on both sides of a window's edge and of the kept first keys' edge, first tokens, long
decoding, generation through the entry point, the replay program; float32 and bfloat16, on configurations that differ
in every size and option.

Routers: a token whose choice between two experts (or two groups) is nearly a tie may choose the other way when its
input carries bfloat16 rounding, and then that position's logits differ by far more than rounding.  float32 runs are
compared at every position (requests whose closest decision in the plain implementation is nearer than 1e-4 are drawn
again); bfloat16 runs of configurations with routers may have a share of positions beyond the bound (a flipped pick
also changes the recurrent states behind it), and the median must be well within it.
"""
import json
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import batched_trace, random_requests, rel_err, run_trace, tail_trace, whole_trace
from plain_potodra import PlainPotodra
from potodra_configs import CONFIGS, ROUTED, make_potodra

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"mixed": [1, 2, 9, 64, 65, 150], "odd": [1, 3, 20, 64, 66, 131], "wide": [3, 17, 63, 128, 129, 300]}
ONLY_LENGTHS = [1, 2, 31, 64, 129, 140]
# bfloat16 with routers: the share of positions that may be beyond the bound.  A token makes two decisions (the groups,
# then the picks), and a pick that falls the other way changes the states of the recurrences after it, and with them
# every later position of the sequence, not only its own.
FLIP_SHARE = 0.35
# Bounds on rounding, as shares of the largest logit.  float32: the gates of the matrix memory are exponentials of sums
# of up to the gates' cap (relative error |x| * 6e-8, thirty times a plain operation's), the dense feed-forward squares
# and the read-out divides by a normaliser that may sit at its floor, so rounding reaches 2e-5 where the other designs
# stay under 1e-5; any indexing, masking or state fault shows as 1e-2 and more.  bfloat16 as for the other designs.
TOL = {"float32": 4e-5, "bfloat16": 5e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("potodra")
    return {name: make_potodra(name, str(root / name)) for name in CONFIGS}


_plain = {}


def plain(folder):
    if folder not in _plain:
        _plain[folder] = PlainPotodra(folder)
    return _plain[folder]


def engine_for(folder, dtype, max_tokens=2048):
    from exl3_server_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)


def requests_for(name, folder, lengths, seed):
    """Random requests none of whose routers' decisions is a close call in the plain implementation."""
    pm = plain(folder)
    out = {}
    for i, n in enumerate(lengths):
        for attempt in range(20):
            toks = random_requests(CONFIGS[name].vocab, [n], seed=seed + 1000 * i + 17 * attempt)["r0"]
            if pm.closest_call(toks) >= 1e-4:
                break
        out[f"r{i}"] = toks
    return out


def position_errors(got, want):
    return np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)), axis=1) / max(1e-30, np.max(np.abs(want)))


def close_enough(got, want, dtype, name, what):
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    err = position_errors(got, want)
    bad = err > TOL[dtype]
    if dtype == "bfloat16" and name in ROUTED:
        assert bad.sum() <= max(1, int(FLIP_SHARE * len(err))) and np.median(err) <= TOL[dtype] / 2, \
            f"{what}: {bad.sum()} of {len(err)} positions beyond the bound, median error {np.median(err):.3e}"
        return
    assert not bad.any(), (f"{what}: differs from the plain implementation by {err.max():.3e} (bound {TOL[dtype]:.0e}); "
                           f"first wrong position {int(np.argmax(bad))} of {len(err)}")


def check(got, want, dtype, name, what):
    assert set(got) == set(want)
    for rid in want:
        close_enough(got[rid], want[rid], dtype, name, f"{what}, request {rid}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", [n for n in CONFIGS if not n.startswith("random")])
def test_whole_decoded_and_batched(folders, name, dtype):
    folder = folders[name]
    requests = requests_for(name, folder, LENGTHS.get(name, ONLY_LENGTHS), seed=3)
    pm = plain(folder)
    want = {rid: pm.logits(t).numpy() for rid, t in requests.items()}
    eng = engine_for(folder, dtype)
    check(run_trace(eng, whole_trace(requests)), want, dtype, name, "whole")
    check(run_trace(eng, tail_trace(requests, 45)), want, dtype, name, "last 45 one by one")
    # everything but the first token decoded: the prompt path and the one-token path must walk the same sums
    short = {rid: t for rid, t in requests.items() if len(t) <= 70}
    check(run_trace(eng, tail_trace(short, 1000)), {rid: want[rid] for rid in short}, dtype, name, "token by token")
    ids = list(requests)
    # two batches one after the other, so that slots, pages and state rows are used again
    batches = [[ids[5], ids[0], ids[2], ids[3]], [ids[1], ids[4], ids[0]]]
    prompt_len = {rid: max(1, len(requests[rid]) - k) for rid, k in zip(ids, (0, 1, 4, 40, 33, 70))}
    check(run_trace(eng, batched_trace(requests, batches, prompt_len)),
          {rid: want[rid] for b in batches for rid in b}, dtype, name, "batched")
    assert eng.cache.tokens_held() == 0
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", [n for n in CONFIGS if n.startswith("random")])
def test_configurations_drawn_from_a_seed(folders, name, dtype):
    """Layer orders, sizes, counts and constants that nobody chose: whole prompts, the last tokens one by one, and
    a batch of unequal requests decoded together."""
    folder = folders[name]
    requests = requests_for(name, folder, [1, 2, 40, 66, 150], seed=41)
    pm = plain(folder)
    want = {rid: pm.logits(t).numpy() for rid, t in requests.items()}
    eng = engine_for(folder, dtype)
    check(run_trace(eng, whole_trace(requests)), want, dtype, name, "whole")
    check(run_trace(eng, tail_trace(requests, 70)), want, dtype, name, "last 70 one by one")
    ids = list(requests)
    prompt_len = {rid: max(1, len(requests[rid]) - k) for rid, k in zip(ids, (0, 1, 35, 3, 80))}
    check(run_trace(eng, batched_trace(requests, [ids[::-1]], prompt_len)), want, dtype, name, "batched")
    assert eng.cache.tokens_held() == 0
    eng.check_kernels()


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_float32_cuttings_agree_closely(folders, name):
    requests = requests_for(name, folders[name], LENGTHS[name], seed=5)
    eng = engine_for(folders[name], "float32")
    a = run_trace(eng, whole_trace(requests))
    b = run_trace(eng, tail_trace(requests, 32))
    for rid in requests:
        assert rel_err(b[rid], a[rid]) <= 2e-6, rid


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
def test_portions_of_a_prompt(folders, name, dtype):
    """A prompt fed in portions of many sizes, down to two tokens, some ending on a page border, on a window's edge
    and inside one, shorter than the convolution's taps reach back, and one long enough for the experts to take the
    many-rows product."""
    from exl3_server_b200 import StepEntry
    folder = folders[name]
    toks = requests_for(name, folder, [430], seed=9)["r0"]
    want = plain(folder).logits(toks).numpy()
    eng = engine_for(folder, dtype)
    for cuts in ([2, 2, 60, 3, 61, 2, 100, 200], [64, 64, 2, 37, 63, 200], [7, 121, 2, 2, 2, 96, 199, 1], [429, 1],
                 [50, 50, 50, 130, 150], [1, 300, 129], [1, 1, 1, 2, 1, 3, 421]):
        assert sum(cuts) == len(toks)
        s = eng.open()
        got, at = [], 0
        for n in cuts:
            got.append(eng.step([StepEntry(s, toks[at:at + n], "all")]).float().cpu().numpy())
            at += n
        eng.close(s)
        close_enough(np.concatenate(got), want, dtype, name, f"portions {cuts}")
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_portions_in_one_batch(folders, dtype):
    """Rows that go on by portions of different sizes in the same steps, beside a row that starts."""
    from exl3_server_b200 import StepEntry
    folder = folders["mixed"]
    reqs = requests_for("mixed", folder, [150, 90, 40], seed=13)
    pm = plain(folder)
    want = {r: pm.logits(t).numpy() for r, t in reqs.items()}
    eng = engine_for(folder, dtype)
    sa, sb = eng.open(), eng.open()
    got = {r: [] for r in reqs}
    out = eng.step([StepEntry(sa, reqs["r0"][:70], "all"), StepEntry(sb, reqs["r1"][:3], "all")]).float().cpu().numpy()
    got["r0"].append(out[:70]); got["r1"].append(out[70:])
    sc = eng.open()
    out = eng.step([StepEntry(sb, reqs["r1"][3:66], "all"), StepEntry(sc, reqs["r2"], "all"),
                    StepEntry(sa, reqs["r0"][70:72], "all")]).float().cpu().numpy()
    got["r1"].append(out[:63]); got["r2"].append(out[63:103]); got["r0"].append(out[103:])
    eng.close(sc)
    out = eng.step([StepEntry(sa, reqs["r0"][72:], "all"), StepEntry(sb, reqs["r1"][66:], "all")]).float().cpu().numpy()
    got["r0"].append(out[:78]); got["r1"].append(out[78:])
    for r in reqs:
        close_enough(np.concatenate(got[r]), want[r], dtype, "mixed", r)


def _rewrite(src, folder, change):
    os.makedirs(folder)
    shutil.copy(os.path.join(src, "config.json"), folder)
    from safetensors import safe_open
    from exl3_server_b200.weights.safetensors_io import write_safetensors
    with safe_open(os.path.join(src, "model.safetensors"), framework="pt") as f:
        tensors = {k: f.get_tensor(k).float() for k in f.keys()}
    change(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), ((k, v.to(torch.bfloat16)) for k, v in tensors.items()),
                      metadata={"format": "pt"})


MARKED = 77


def _mark_features(t):
    """Feature 0 of the model is on for the marked token only and feature 1 for every token; the first norm passes
    both (after it feature 1 is about 5 for an ordinary token and 2 for the marked one, whose feature 0 is about 7)."""
    t["embed"][:, 0] = 0.0
    t["embed"][:, 1] = 0.5
    t["embed"][MARKED, 0] = 2.0
    t["l0.norm1"][:2] = 1.0


def _marked_attention(src, folder, prefix, heads_dim, rot_dims):
    """A copy of a one-layer model in which one token's key stands out for every query of the attention under
    ``prefix``.  Feature 0 of the model is on for the marked token only and feature 1 for every token (the other
    embedding features stay random); the streams' read weights and the norm pass both; the key matrix sends feature 0,
    and the query matrix feature 1, to the same features of every head (those the rotation leaves alone, or all of
    them where nothing is left alone and the rotation is slow), so the marked key's score is far above the spread of
    the others' wherever the query stands."""
    def change(t):
        _mark_features(t)
        d = heads_dim
        for name, col in ((prefix + "q", 1), (prefix + "k", 0)):
            w = t[name]
            w[:, col] = 0.0
            w.view(-1, d, w.shape[1])[:, rot_dims:, col] = 3.0
            t[name + ".b"][:] = 0.0
        t[prefix + "v"][:, 0] = 1.0             # and its value is several times the others'
    _rewrite(src, folder, change)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, prefix, places", [
    ("only_full_attention", "l0.mix.left.", [0, 1, 63, 64, 127, 128, 300]),
    ("only_attention", "l0.mix.", [0, 8, 9, 64, 610, 629, 630, 631, 640, 699])])
def test_a_key_that_stands_out(folders, tmp_path, name, prefix, places, dtype):
    """The marked key sits first, second, on both sides of page borders and hundreds of tokens back (no window); and,
    with a window of 70 positions that keeps the first 9 keys, at the last kept place (8), the first one not kept (9),
    and around the window's edge: the last query (699) sees 630 .. 699, the twenty before it see from 610 .. 629 on.
    Losing the key, reading a neighbour instead, seeing it across an edge or not seeing a kept one changes the logits
    by far more than the bound.  Whole prompts, and the last 95 tokens decoded one by one, so that the window passes
    over the key while decoding."""
    folder = str(tmp_path / "m")
    mixer = CONFIGS[name].layers[0].mixer
    m = mixer["left"] if "left" in mixer else mixer
    rot = m["rot"]["dims"] if m.get("rot") else 0
    _marked_attention(folders[name], folder, prefix, m["dim"], rot if rot < m["dim"] else m["dim"] // 2)
    pm = PlainPotodra(folder)
    vocab = CONFIGS[name].vocab
    base = [t if t != MARKED else 5 for t in random_requests(vocab, [700], seed=21)["r0"]]
    mask = m.get("mask") or {}
    window, keep = mask.get("size", 10 ** 9), mask.get("keep_first", 0)
    eng = engine_for(folder, dtype)
    for place in places:
        toks = list(base)
        toks[place] = MARKED
        want = pm.logits(toks).numpy()
        seen = [q for q in range(680, 700) if 0 <= q - place < window or place < keep]
        unseen = [q for q in range(680, 700) if q - place >= window and place >= keep]
        plainly = pm.logits(base).numpy()
        if seen:
            assert rel_err(plainly[seen], want[seen]) > 0.2, place      # the test can see the key
        if unseen:
            assert rel_err(plainly[unseen], want[unseen]) < 1e-9, place  # and the window hides it
        got = run_trace(eng, whole_trace({"a": toks}))["a"]
        assert rel_err(got, want) <= TOL[dtype], ("whole", place)
        got = run_trace(eng, tail_trace({"a": toks}, 95))["a"]
        assert rel_err(got, want) <= TOL[dtype], ("decoded", place)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_counts(folders, tmp_path, dtype):
    """Sinks of 6 (far above the scores): leaving the sink out, scaling or capping it would change every row."""
    folder = str(tmp_path / "m")

    def change(t):
        t["l0.mix.sink"][:] = torch.tensor([6.0, 5.0, 7.0, 4.0])
    _rewrite(folders["only_attention"], folder, change)
    pm = PlainPotodra(folder)
    toks = random_requests(128, [200], seed=33)["r0"]
    want = pm.logits(toks).numpy()
    assert rel_err(plain(folders["only_attention"]).logits(toks).numpy(), want) > 0.05
    eng = engine_for(folder, dtype)
    assert rel_err(run_trace(eng, whole_trace({"a": toks}))["a"], want) <= TOL[dtype]
    assert rel_err(run_trace(eng, tail_trace({"a": toks}, 90))["a"], want) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["only_mlstm", "only_delta"])
def test_a_token_far_back_in_the_state(folders, tmp_path, name, dtype):
    """One token 600 positions back that writes far more strongly than the others (the norm before the mixer makes
    every token's input the same size, so the mark goes through the gates: an input gate at its cap for the marked
    token and low for the others, or a beta near one against betas near zero with a large value), with forget gates
    and decays near one: a state that is lost, reset or decayed once too often shows."""
    folder = str(tmp_path / "m")

    def change(t):
        _mark_features(t)
        if name == "only_mlstm":
            t["l0.mix.f.b"][:] = 7.0                 # forget gates of 0.998
            t["l0.mix.f"] *= 0.1
            t["l0.mix.i"][:, 0] = 5.0
            t["l0.mix.i"][:, 1] = -0.6
            t["l0.mix.o"] *= 12.0                    # the mixer's share of the logits
        else:
            t["l0.mix.right.A_log"][:] = -6.0        # decays of 0.998 and slower
            t["l0.mix.right.b"][:] = 0.0
            t["l0.mix.right.b"][:, 0] = 2.0
            t["l0.mix.right.b"][:, 1] = -1.5
            t["l0.mix.right.v"][:, 0] = 3.0
            t["l0.mix.right.o"] *= 14.0              # the mixer's share of the logits
    _rewrite(folders[name], folder, change)
    pm = PlainPotodra(folder)
    base = [t if t != MARKED else 5 for t in random_requests(128, [700], seed=27)["r0"]]
    toks = list(base)
    toks[90] = MARKED
    want = pm.logits(toks).numpy()
    assert rel_err(pm.logits(base).numpy()[-20:], want[-20:]) > 0.15
    eng = engine_for(folder, dtype)
    assert rel_err(run_trace(eng, whole_trace({"a": toks}))["a"], want) <= TOL[dtype]
    assert rel_err(run_trace(eng, tail_trace({"a": toks}, 64))["a"], want) <= TOL[dtype]
    from exl3_server_b200 import StepEntry
    s = eng.open()
    got = [eng.step([StepEntry(s, toks[a:b], "all")]).float().cpu().numpy()
           for a, b in ((0, 89), (89, 91), (91, 300), (300, 302), (302, 700))]
    eng.close(s)
    assert rel_err(np.concatenate(got), want) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
def test_long_decoding(folders, name, dtype):
    """Three tokens of prompt, then 200 decoded one by one over three page borders and past every window, two
    sequences side by side."""
    from exl3_server_b200 import StepEntry
    folder = folders[name]
    reqs = requests_for(name, folder, [203, 180], seed=17)
    pm = plain(folder)
    want = [pm.logits(reqs["r0"]).numpy(), pm.logits(reqs["r1"]).numpy()]
    eng = engine_for(folder, dtype)
    s = [eng.open(), eng.open()]
    got = [[], []]
    out = eng.step([StepEntry(s[0], reqs["r0"][:3], "all"), StepEntry(s[1], reqs["r1"][:3], "all")]).float().cpu().numpy()
    got[0].append(out[:3]); got[1].append(out[3:])
    for i in range(3, 203):
        live = [k for k in (0, 1) if i < len(reqs[f"r{k}"])]
        out = eng.step([StepEntry(s[k], [reqs[f"r{k}"][i]], "all") for k in live]).float().cpu().numpy()
        for j, k in enumerate(live):
            got[k].append(out[j:j + 1])
    for k in (0, 1):
        close_enough(np.concatenate(got[k]), want[k], dtype, name, k)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_reused_slot_shows_nothing_of_its_former_owner(folders, dtype):
    """A sequence's state rows and pages go to the next sequence; the next one must start from zero state (also the
    convolutions' last inputs and the running maximum) and see none of the old rows, also when it is shorter than the
    old one."""
    from exl3_server_b200 import StepEntry
    folder = folders["mixed"]
    reqs = requests_for("mixed", folder, [190, 30], seed=23)
    want = plain(folder).logits(reqs["r1"]).numpy()
    eng = engine_for(folder, dtype, max_tokens=256)
    for _ in range(3):
        s = eng.open()
        eng.step([StepEntry(s, reqs["r0"], None)])
        eng.close(s)
        s2 = eng.open()
        assert s2 == s
        got = [eng.step([StepEntry(s2, reqs["r1"][:9], "all")]).float().cpu().numpy()]
        for t in reqs["r1"][9:]:
            got.append(eng.step([StepEntry(s2, [t], "all")]).float().cpu().numpy())
        eng.close(s2)
        close_enough(np.concatenate(got), want, dtype, "mixed", "after reuse")
    eng.cache.check()


@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
def test_greedy_generation_through_the_entry_point(folders, name):
    from exl3_server_b200 import GenerateOptions
    folder = folders[name]
    prompts = list(requests_for(name, folder, [5, 70, 1, 33], seed=29).values())
    eng = engine_for(folder, "float32")
    res = eng.generate(prompts, GenerateOptions(max_tokens=24, ignore_eos=True, max_batch=3))
    pm = plain(folder)
    for p, r in zip(prompts, res):
        assert r.tokens == pm.greedy(p, 24)
        assert r.finish_reason == "length"
    assert eng.cache.tokens_held() == 0
    # bfloat16: the same call runs and every token is in range (near-ties may fall the other way)
    eng = engine_for(folder, "bfloat16")
    res = eng.generate(prompts, GenerateOptions(max_tokens=24, ignore_eos=True))
    assert all(len(r.tokens) == 24 and all(0 <= t < CONFIGS[name].vocab for t in r.tokens) for r in res)
    eng.check_kernels()


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_residual_stream_layer_by_layer(folders, name):
    """The float32 sum of the streams after every layer against the plain implementation's."""
    from exl3_server_b200 import StepEntry
    folder = folders[name]
    toks = requests_for(name, folder, [75], seed=31)["r0"]
    want = plain(folder).layers(toks)
    eng = engine_for(folder, "float32")
    S = CONFIGS[name].streams
    seen = []
    for b in eng.model.blocks:
        def wrapped(stream, *args, f=b.forward, **kwargs):
            f(stream, *args, **kwargs)
            seen.append(stream.h.view(stream.h.shape[0], S, -1).sum(dim=1))
        b.forward = wrapped
    s = eng.open()
    eng.step([StepEntry(s, toks, None)])
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        assert rel_err(a.cpu().numpy(), b.numpy()) <= TOL["float32"], i


def test_replay_program_and_command_line(folders, tmp_path):
    folder = folders["mixed"]
    vocab = CONFIGS["mixed"].vocab
    reqs = requests_for("mixed", folder, [40, 7], seed=4)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": reqs["r0"][:38], "want": [0, 37]},
                                {"id": "b", "tokens": reqs["r1"][:6], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [reqs["r0"][38]], "want": [0]},
                                {"id": "b", "tokens": [reqs["r1"][6]], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [reqs["r0"][39]], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "b", "tokens": reqs["r1"], "want": [6]}], "end": ["b"]},
    ]
    pm = plain(folder)
    la, lb = pm.logits(reqs["r0"]).numpy(), pm.logits(reqs["r1"]).numpy()
    out = tmp_path / "float32"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, vocab)
    s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, vocab)
    s3 = np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, vocab)
    assert rel_err(s0, la[[0, 37]]) <= TOL["float32"]
    assert rel_err(s1, np.stack([la[38], lb[6]])) <= TOL["float32"]
    assert rel_err(s3, lb[6:7]) <= TOL["float32"]
    p = subprocess.run([sys.executable, "-m", "exl3_server_b200", "--model", folder, "-p", "5,6,7", "--max-tokens", "5",
                        "--ignore-eos", "--dtype", "float32"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.strip() == ",".join(map(str, pm.greedy([5, 6, 7], 5)))
