"""The Tabedra decoder inside the engine against the plain float64 implementation (tests/plain_tabedra.py).

Every mechanism alone (one-layer models), whole prompts against token-by-token decoding, portions down to two tokens,
mixed batches against each request alone, pages and state slots that are freed and used again, keys just inside and
just outside a window (in prompts and in decoding, with peaked attention and large distance biases), a reader of
another layer's cache whose window is wider than the owner's, the first tokens of a sequence, long decoding, several
sizes, the residual stream layer by layer, greedy generation through the scheduler, and the command line.

The bfloat16 engine rounds what the router reads, so its models space the router's corrections far apart
(``steady_router``): which experts are chosen then does not hang on the last bits of a score, while their weights still
come from the live scores.  The 32-bit engine runs the live router.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_tabedra as P
import tabedra_models as M
from helpers import ROOT

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 4e-2}         # max |difference| / max |reference logit|
# With peaked attention (scores scaled up sixfold) a rounding of a score moves the weights of the keys by as much more.
TOL_SHARP = {"float32": 1.5e-3, "bfloat16": 8e-2}
DTYPES = ["float32", "bfloat16"]


def rel_err(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - ref)) / np.max(np.abs(ref)))


def runner_for(path, dtype, page_size=16, pool_tokens=1024, max_seqs=4, max_batch_tokens=1024):
    from rustingstrata_b200.config import EngineConfig
    from rustingstrata_b200.engine import ModelRunner
    eng = EngineConfig(dtype=dtype, page_size=page_size, num_pages=(pool_tokens + page_size - 1) // page_size,
                       max_seqs=max_seqs, max_batch_tokens=max_batch_tokens, max_logit_rows=max_batch_tokens)
    return ModelRunner.from_dir(path, eng)


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def plain_logits(cfg, w, toks):
    return P.forward(toks, w, cfg).numpy()


_MODELS = {}


def model(tmp_path_factory, key, cfg, dtype, seed=0, sharp=False):
    """(folder, config, weights) of a model made for ``dtype`` (see the module's text on the router)."""
    steady = dtype == "bfloat16"
    key = f"{key}{'_sharp' if sharp else ''}{'_steady' if steady else ''}"
    if key not in _MODELS:
        path = str(tmp_path_factory.mktemp("tabedra") / key)
        _MODELS[key] = (path,) + M.make(path, cfg, seed, sharp, steady)
    return _MODELS[key]


def step_all(r, rid, toks, want=None):
    from rustingstrata_b200.engine import StepEntry
    out = r.step([StepEntry(rid, toks, list(range(len(toks))) if want is None else want)])
    r.check_status()
    return None if out is None else out.cpu().numpy()


# ----------------------------------------------------------------------------- each mechanism alone
ONE_LAYER = {
    "attention_plain": M.config(97, 64, [(M.attn(4, 2, 16, 16, conv=None, rows=8, bias_max=30.0), None)], streams=None, bigram=None),
    "attention_window_not_a_page": M.config(97, 64, [(M.attn(3, 1, 16, 32, conv=None, rows=12, bias_max=17.0, window=11), None)],
                                            streams=None, bigram=None),
    "attention_convolved": M.config(97, 64, [(M.attn(2, 2, 32, 16, conv=4, rows=6, bias_max=60.0, window=29), None)],
                                    streams=None, bigram=None),
    "attention_padded_heads": M.config(97, 72, [(M.attn(5, 1, 20, 36, conv=2, rows=10, bias_max=44.0), None)], streams=None, bigram=None),
    "bigram_embedding": M.config(97, 64, [(M.attn(2, 1, 16, 16, conv=None, rows=4, bias_max=9.0), None)], streams=None, bigram=(23, 5, 3)),
    "streams_nine_taps_twenty": M.config(97, 64, [(M.attn(2, 1, 16, 16, conv=20, rows=4, bias_max=9.0), None)], streams=9, bigram=None),
    "streams_four": M.config(97, 64, [(M.attn(2, 1, 16, 16, conv=None, rows=4, bias_max=9.0), None)], streams=4, bigram=None),
    "experts_top2_shared": M.config(97, 64, [(M.attn(2, 1, 16, 16, conv=None), M.moe(6, 2, 24, shared=40))], streams=None, bigram=None),
    "experts_top1_unshared": M.config(97, 64, [(M.attn(2, 1, 16, 16, conv=None), M.moe(4, 1, 40))], streams=2, bigram=None),
    "experts_all_chosen": M.config(33, 56, [(M.attn(2, 1, 16, 16, conv=2), M.moe(3, 3, 16, shared=8))], streams=None, bigram=None),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_mechanism_alone(tmp_path_factory, name, dtype):
    """A one-layer model per mechanism: the stream after the layer and the logits of a whole prompt, the same prompt
    in portions, and token by token."""
    path, cfg, w = model(tmp_path_factory, "one_" + name, ONE_LAYER[name], dtype, seed=len(name))
    toks = tokens_for(cfg, 45, 3)
    streams = []
    ref = P.forward(toks, w, cfg, streams).numpy()
    r = runner_for(path, dtype, page_size=8, pool_tokens=256)
    from rustingstrata_b200.engine import StepEntry
    got_streams = []
    logits = r.step([StepEntry("a", toks, list(range(len(toks))))],
                    on_layer=lambda k, x: got_streams.append(x.float().cpu().numpy().copy()))
    r.check_status()
    assert len(got_streams) == len(streams)
    for i, (g, s) in enumerate(zip(got_streams, streams)):
        assert rel_err(g, s.numpy()) <= TOL[dtype], f"{name} {dtype}: stream after layer {i}"
    assert rel_err(logits.cpu().numpy(), ref) <= TOL[dtype]
    r.release("a")
    got, pos = [], 0
    for n in [2, 5, 1, 2, 17, 3, 2, 13]:
        got.append(step_all(r, "b", toks[pos:pos + n]))
        pos += n
    assert pos == len(toks)
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], f"{name} {dtype}: portions"
    r.release("b")
    got = [step_all(r, "c", [t]) for t in toks]
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], f"{name} {dtype}: token by token"


def test_router_choice_weights_and_correction():
    """The router kernel alone against the plain router: choice by corrected score, weights from the uncorrected
    scores, for several expert counts (more experts than a warp has lanes among them)."""
    from rustingstrata_b200.kernels import ops
    rng = np.random.default_rng(5)
    for E, top, T in [(5, 2, 9), (12, 5, 40), (70, 8, 33), (3, 3, 4), (130, 1, 17)]:
        logits = torch.from_numpy(rng.standard_normal((T, E)) * 2).float()
        corr = torch.from_numpy(rng.standard_normal(E) * 0.2).float()
        s = torch.softmax(logits.double(), dim=-1)
        idx = torch.topk(s + corr.double(), top, dim=-1).indices
        w = torch.gather(s, 1, idx)
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
        choice = torch.empty(T * top, dtype=torch.int32, device="cuda")
        weights = torch.empty(T * top, dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.router_topk(logits.cuda(), corr.cuda(), top, T, choice, weights, status)
        assert int(status.item()) == 0
        assert torch.equal(choice.cpu().view(T, top).long(), idx), (E, top)
        assert torch.allclose(weights.cpu().view(T, top).double(), w, rtol=1e-5, atol=1e-7)


# ----------------------------------------------------------------------------- whole models, every cutting
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_cuttings_of_a_prompt(tmp_path_factory, name, dtype):
    """Whole, last tokens one by one (captured steps), portions of several sizes down to two tokens."""
    path, cfg, w = model(tmp_path_factory, name, name, dtype, seed=11)
    toks = tokens_for(cfg, 150, 5)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=512)
    assert rel_err(step_all(r, "w", toks), ref) <= TOL[dtype], "whole"
    r.release("w")
    n = len(toks) - 40
    got = [step_all(r, "d", toks[:n])] + [step_all(r, "d", [t]) for t in toks[n:]]
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], "decoding"
    if r.model.capturable:
        assert r.graph_replays > 0
    r.release("d")
    got, pos, k = [], 0, 0
    sizes = [7, 2, 13, 2, 5, 3, 29, 2, 16, 4, 11, 2, 1, 1, 31]
    while pos < len(toks):
        m = min(sizes[k % len(sizes)], len(toks) - pos)
        got.append(step_all(r, "p", toks[pos:pos + m]))
        pos, k = pos + m, k + 1
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], "portions"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R"])
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path_factory, name, dtype):
    """Up to three live requests of unequal length in a pool that cannot hold all seven at once: portions of some
    beside single tokens of others, requests left out of steps, and every row equal to the request run alone.  A slot
    that a request has left (with its convolution tails and its previous token) is taken by the next one, which must
    start from zero."""
    from rustingstrata_b200.engine import StepEntry
    path, cfg, w = model(tmp_path_factory, name, name, dtype, seed=21, sharp=True)
    tol = TOL_SHARP[dtype]
    lengths = [70, 33, 121, 9, 64, 1, 47]
    toks = {f"r{i}": tokens_for(cfg, n, 40 + i) for i, n in enumerate(lengths)}
    ref = {k: plain_logits(cfg, w, t) for k, t in toks.items()}
    r = runner_for(path, dtype, page_size=16, pool_tokens=256, max_seqs=3)
    rng = np.random.default_rng(9)
    waiting, live, pos = list(toks), [], {}
    worst, rows, slots_seen = 0.0, 0, {}
    while waiting or live:
        while waiting and len(live) < 3 and sum((len(toks[x]) + 15) // 16 for x in live + [waiting[0]]) <= 16:
            live.append(waiting.pop(0))
            pos[live[-1]] = 0
        chosen = [x for x in live if rng.random() < 0.7] or [live[0]]
        entries, where = [], []
        for rid in chosen:
            left = len(toks[rid]) - pos[rid]
            n = 1 if left <= 12 else int(min(rng.choice([2, 3, 5, 9, 17, 31]), left - 12))
            want = list(range(n))
            entries.append(StepEntry(rid, toks[rid][pos[rid]:pos[rid] + n], want))
            where += [(rid, pos[rid] + j) for j in want]
            pos[rid] += n
        out = r.step(entries).cpu().numpy()
        r.check_status()
        for rid in chosen:
            slots_seen.setdefault(r.cache.slot(rid), set()).add(rid)
        for row, (rid, p) in zip(out, where):
            e = float(np.max(np.abs(row - ref[rid][p])) / np.max(np.abs(ref[rid])))
            worst, rows = max(worst, e), rows + 1
            assert e <= tol, f"{name} {dtype}: request {rid} position {p}: {e:.3e}"
        for rid in [x for x in live if pos[x] == len(toks[x])]:
            live.remove(rid)
            r.release(rid)
    r.cache.check()
    assert rows == sum(lengths)
    print(f"mixed {name} {dtype}: worst {worst:.3e}")
    assert max(len(v) for v in slots_seen.values()) >= 2, "no state slot was used again"
    assert all(p.reuses > 0 for p in r.cache.pools), "no page was used again"


# ----------------------------------------------------------------------------- windows, far keys, page borders
@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_in_prompts_and_decoding(tmp_path_factory, dtype):
    """Peaked attention with large biases on the far rows of the distance tables: every position of a prompt that
    crosses each layer's window several times, then decoding across page borders and window edges, then the rest as a
    portion.  A window that is one key too wide or too narrow, or a bias row that is one off, moves these logits."""
    path, cfg, w = model(tmp_path_factory, "P", "P", dtype, seed=21, sharp=True)
    toks = tokens_for(cfg, 330, 77)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=512, max_batch_tokens=512)
    n = 200
    got = [step_all(r, "a", toks[:n])] + [step_all(r, "a", [t]) for t in toks[n:n + 70]] + [step_all(r, "a", toks[n + 70:])]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / np.max(np.abs(ref))
    print(f"window edges {dtype}: worst {err.max():.3e}")
    assert err.max() <= TOL_SHARP[dtype], f"first wrong position {int(np.argmax(err > TOL_SHARP[dtype]))}"


def test_sharp_weights_see_the_window_edge(tmp_path_factory):
    """The premise of the test above, checked on the plain implementation: a window one key narrower or wider in any
    windowed layer, or a bias table read one row off, changes the logits by more than the tolerance of either engine
    (by a hundred times that of the 32-bit engine)."""
    path, cfg, w = model(tmp_path_factory, "P", "P", "float32", seed=21, sharp=True)
    toks = tokens_for(cfg, 120, 77)
    full = plain_logits(cfg, w, toks)[-40:]
    for layer in (0, 2, 3):
        for by in (-1, 1):
            other = json.loads(json.dumps(cfg))
            other["layers"][layer]["mixer"]["mask"]["size"] += by
            moved = np.max(np.abs(full - plain_logits(other, w, toks)[-40:])) / np.max(np.abs(full))
            assert moved > 1.5 * TOL_SHARP["bfloat16"], (layer, by, moved)
    shifted = dict(w)
    shifted["l0.mix.rel"] = torch.roll(w["l0.mix.rel"], 1, dims=0)
    assert np.max(np.abs(full - plain_logits(cfg, shifted, toks)[-40:])) / np.max(np.abs(full)) > 3 * TOL_SHARP["bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_without_a_window(tmp_path_factory, dtype):
    """A layer that sees every earlier key (no mask), peaked: 600 positions, decoding across the border of an
    attention split and page borders, keys hundreds of tokens back; beside it a reader with a window of 200 on a cache
    whose owner's window is 128."""
    path, cfg, w = model(tmp_path_factory, "R", "R", dtype, seed=21, sharp=True)
    toks = tokens_for(cfg, 600, 78)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=640, max_batch_tokens=640)
    n = 500
    got = [step_all(r, "a", toks[:n])] + [step_all(r, "a", [t]) for t in toks[n:n + 60]] + [step_all(r, "a", toks[n + 60:])]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / np.max(np.abs(ref))
    print(f"far keys {dtype}: worst {err.max():.3e}")
    assert err.max() <= TOL_SHARP[dtype], f"first wrong position {int(np.argmax(err > TOL_SHARP[dtype]))}"


def test_sharp_weights_look_far_back(tmp_path_factory):
    """The premise of the test above: keys more than 250 back carry weight (more than either engine's tolerance)."""
    path, cfg, w = model(tmp_path_factory, "R", "R", "float32", seed=21, sharp=True)
    toks = tokens_for(cfg, 400, 78)
    full = plain_logits(cfg, w, toks)[-20:]
    # the same tokens at the same positions, but the unwindowed layer sees the last 250 keys only
    cut = json.loads(json.dumps(cfg))
    cut["layers"][1]["mixer"]["mask"] = {"size": 250}
    assert np.max(np.abs(full - plain_logits(cut, w, toks)[-20:])) / np.max(np.abs(full)) > 1.5 * TOL_SHARP["bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_short_sequences(tmp_path_factory, dtype):
    """Sequences shorter than the convolutions' taps, single-token prompts (the bigram table's own row), and a first
    step of one token beside longer ones in the same batch."""
    from rustingstrata_b200.engine import StepEntry
    path, cfg, w = model(tmp_path_factory, "P", "P", dtype, seed=11)
    r = runner_for(path, dtype, page_size=16, pool_tokens=256)
    seqs = {"one": tokens_for(cfg, 1, 1), "two": tokens_for(cfg, 2, 2), "three": tokens_for(cfg, 3, 3), "ten": tokens_for(cfg, 10, 4)}
    out = r.step([StepEntry(k, t, list(range(len(t)))) for k, t in seqs.items()]).cpu().numpy()
    r.check_status()
    at = 0
    for k, t in seqs.items():
        assert rel_err(out[at:at + len(t)], plain_logits(cfg, w, t)) <= TOL[dtype], k
        at += len(t)
    # each grows by one token (the step is all single tokens: the captured form), three times
    for _ in range(3):
        for k in seqs:
            seqs[k] = seqs[k] + tokens_for(cfg, 1, len(seqs[k]) + 50)
        out = r.step([StepEntry(k, t[-1:], [0]) for k, t in seqs.items()]).cpu().numpy()
        for row, (k, t) in zip(out, seqs.items()):
            assert rel_err(row, plain_logits(cfg, w, t)[-1]) <= TOL[dtype], k


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path_factory, dtype):
    """300 tokens one by one after a short prompt (replayed graphs, several attention splits, pages taken and, behind
    the windows, given back as it goes)."""
    path, cfg, w = model(tmp_path_factory, "P", "P", dtype, seed=21, sharp=True)
    toks = tokens_for(cfg, 320, 8)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=8, pool_tokens=384)
    got = [step_all(r, "a", toks[:20])] + [step_all(r, "a", [t]) for t in toks[20:]]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / np.max(np.abs(ref))
    print(f"long decoding {dtype}: worst {err.max():.3e}")
    assert err.max() <= TOL_SHARP[dtype], f"first wrong position {int(np.argmax(err > TOL_SHARP[dtype]))}"


WIDE = {
    # many experts (more than a warp's lanes), eight streams, a long portion (the grouped products' large tiles),
    # head size 128, a kv group of 8
    "many_experts": M.config(300, 512, [(M.attn(8, 1, 128, 128, conv=4, rows=64, bias_max=500.0, window=256), M.moe(40, 4, 128, shared=256)),
                                         (M.attn(8, 1, 128, 128, conv=4, rows=64, bias_max=500.0, window=300, kv_from=0), M.moe(3, 1, 512))],
                            streams=8, bigram=(1021, 300, 7)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(WIDE))
def test_wider_shapes_and_long_portions(tmp_path_factory, name, dtype):
    """A portion of 700 tokens, 40 single tokens, a portion of 160: the forms of the kernels that only large steps and
    wide rows reach."""
    path, cfg, w = model(tmp_path_factory, "wide_" + name, WIDE[name], dtype, seed=7)
    toks = tokens_for(cfg, 900, 3)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=1024, max_batch_tokens=1024)
    got = [step_all(r, "a", toks[:700])] + [step_all(r, "a", [t]) for t in toks[700:740]] + [step_all(r, "a", toks[740:])]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / np.max(np.abs(ref))
    assert err.max() <= TOL[dtype], f"first wrong position {int(np.argmax(err > TOL[dtype]))}"


# ----------------------------------------------------------------------------- the engine's own entry points
@pytest.mark.parametrize("chunk", [None, 7])
def test_greedy_generation_through_the_scheduler(tmp_path_factory, chunk):
    """Engine.generate (scheduler, admission, prompt portions of 7 tokens, decode steps launched ahead) gives the plain
    implementation's greedy tokens in 32-bit, for several prompts of unequal length at once."""
    from rustingstrata_b200 import Engine
    path, cfg, w = model(tmp_path_factory, "P", "P", "float32", seed=11)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (5, 23, 1, 40)]
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(plain_logits(cfg, w, seq)[-1])))
        want.append(seq[len(p):])
    eng = Engine(path, dtype="float32", page_size=8, max_tokens=512, max_batch_tokens=64, max_seqs=4, prefill_chunk=chunk)
    assert eng.generate(prompts, max_new_tokens=12) == want
    # and once more through the same engine: slots and pages of the finished requests are taken again
    assert eng.generate(prompts[::-1], max_new_tokens=12) == want[::-1]


def test_bfloat16_generation_picks_top_tokens(tmp_path_factory):
    from rustingstrata_b200 import Engine
    path, cfg, w = model(tmp_path_factory, "R", "R", "bfloat16", seed=11)
    prompt = tokens_for(cfg, 30, 2)
    eng = Engine(path, dtype="bfloat16", page_size=16, max_tokens=256, max_batch_tokens=64, max_seqs=2)
    got = eng.generate(prompt, max_new_tokens=10)
    logits = plain_logits(cfg, w, prompt + got)
    for i, t in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        assert row[t] >= row.max() - 0.08 * np.abs(logits).max()


def test_trace_replay_and_command_line(tmp_path_factory, tmp_path):
    """bin/trace_run on a model folder (logits of a request cut in two steps), and ``init-random`` + ``generate`` of
    the package's command line for this architecture."""
    path, cfg, w = model(tmp_path_factory, "Q", "Q", "float32", seed=11)
    toks = tokens_for(cfg, 40, 1)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[25:], "want": [14]}, {"id": "y", "tokens": toks[:3], "want": [2]}],
              "end": ["x", "y"]}]
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1"]
    ref = plain_logits(cfg, w, toks)
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, cfg["vocab"])
    b = np.fromfile(out / "1.f32", dtype="<f4").reshape(2, cfg["vocab"])
    assert rel_err(a, ref[[0, 24]]) <= TOL["float32"]
    assert rel_err(b, np.stack([ref[39], ref[2]])) <= TOL["float32"]
    # random weights for a configuration of this architecture, then generation from the command line
    cfg_path = tmp_path / "cfg.json"
    small = dict(M.CONFIGS["Q"][0])
    small["layers"] = [dict(L, mixer=dict(L["mixer"], bias_rows=12)) for L in small["layers"]]
    cfg_path.write_text(json.dumps(small))
    made = tmp_path / "made"
    env = dict(os.environ, PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-m", "rustingstrata_b200", "init-random", "--config", str(cfg_path), "--out", str(made),
                          "--seed", "3"], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    res = subprocess.run([sys.executable, "-m", "rustingstrata_b200", "generate", "--model", str(made), "--dtype", "float32",
                          "--prompt", "1,2,3", "-n", "5"], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-2000:]


# ----------------------------------------------------------------------------- kernels against torch, one by one
def test_kernels_of_the_new_parts_against_torch():
    from rustingstrata_b200.kernels import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)                          # noqa: E731
    # layer norm of a weighted sum of streams, with gathered rows
    S, D, T = 3, 70, 9
    x, coef, w, b = rn(T, S * D), rn(S), rn(D), rn(D)
    rows = torch.tensor([4, 0, 8], dtype=torch.int32)
    out = torch.empty(3, D, device=dev)
    ops.stream_layernorm(x.to(dev), S, coef.to(dev), w.to(dev), b.to(dev), 1e-5, out, 3, rows=rows.to(dev))
    u = torch.einsum("s,tsd->td", coef.double(), x.double().view(T, S, D))[rows.long()]
    assert torch.allclose(out.cpu().double(), P.layer_norm(u, w.double(), b.double(), 1e-5), atol=1e-5)
    # all streams rewritten at once, and the next reader's norm in the same pass
    y, mix, oc, coef2 = rn(T, D), rn(S, S), rn(S), rn(S)
    xs, h = x.clone().to(dev), torch.empty(T, D, device=dev)
    ops.stream_update(xs, S, y.to(dev), mix.to(dev), oc.to(dev), T, next_coef=coef2.to(dev), next_weight=w.to(dev),
                      next_bias=b.to(dev), next_eps=1e-6, next_out=h)
    X = x.double().view(T, S, D)
    new = torch.einsum("st,tsd->ttd" if False else "sq,tsd->tqd", mix.double(), X) + oc.double()[None, :, None] * y.double()[:, None, :]
    assert torch.allclose(xs.cpu().double().view(T, S, D), new, atol=1e-5)
    assert torch.allclose(h.cpu().double(), P.layer_norm(torch.einsum("s,tsd->td", coef2.double(), new), w.double(), b.double(), 1e-6),
                          atol=1e-5)
    # the distance table the attention kernels read, against the plain bucket function
    from rustingstrata_b200.parts.conv_attention import distance_rows
    for rows_, far in [(16, 120.0), (10, 33.5), (4, 9.0), (32, 100.0), (64, 500.0)]:
        got = distance_rows(rows_, far, 700)
        assert got.tolist() == [P.distance_bucket(n, rows_, far) for n in range(700)]
