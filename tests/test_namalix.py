"""Namalix through the library's own step function, cache and generation loop, against the plain float64 implementation of
`plain_namalix.py`, on small configurations made here (`namalix_cases.py`).

32-bit runs: every schedule of a sequence (whole, cut into portions, token by token, inside a batch, in pages and slots
that were used before) must give the same bits, and those must lie within 32-bit rounding of the plain result.
bfloat16 runs are judged position by position (`check`).  The mechanisms alone are in `test_namalix_kernels.py`."""

import numpy as np
import pytest
import torch

import plain_namalix as pn
from helpers import check_logits
from namalix_cases import CONFIGS, as_float64, random_weights, write_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, folder, float64 weights)."""
    out = {}
    for i, (name, make) in enumerate(CONFIGS.items()):
        cfg = make()
        w = random_weights(cfg, seed=71 + i)
        out[name] = (cfg, write_model(tmp_path_factory.mktemp(f"nam_{name}"), cfg, w), as_float64(w))
    return out


def ref_logits(cfg, w, toks):
    return pn.plain_logits(cfg, w, toks).numpy()


def check(got, ref, dtype, what=""):
    if dtype == "float32":
        return check_logits(got, ref, dtype, what)
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
    assert np.median(err) <= 2.5e-2, f"{what}: median error {np.median(err):.3f} of the range"
    if len(err) >= 10:
        assert np.quantile(err, 0.9) <= 6e-2, f"{what}: 90 % of the positions within {np.quantile(err, 0.9):.3f} of the range"
        assert (err > 0.15).mean() <= 0.05, f"{what}: {(err > 0.15).sum()} of {len(err)} positions differ by more than 0.15 of the range"
    else:
        assert (err > 0.15).sum() <= 1, f"{what}: errors {np.round(err, 3)} of the range"


def tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def load(folder, dtype, max_tokens=64 * 12, max_seqs=4, **kw):
    import rusty_llama_b200 as rl

    return rl.load(folder, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs, **kw)


def run_cut(llm, toks, cuts):
    """One sequence fed in portions of the given sizes (the rest one by one); logits of every position."""
    from rusty_llama_b200 import StepEntry

    s = llm.open_sequence()
    out, at = [], 0
    sizes = list(cuts) + [1] * (len(toks) - sum(cuts))
    for n in sizes:
        out.append(llm.step([StepEntry(s, toks[at : at + n], list(range(n)))]).cpu().numpy())
        at += n
    llm.close_sequence(s)
    llm.engine.check_device_status()
    return np.concatenate(out, axis=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_against_the_plain_model(models, name, dtype):
    cfg, folder, w = models[name]
    llm = load(folder, dtype)
    for n, seed in ((1, 0), (5, 1), (150, 2)):
        toks = tokens(cfg, n, seed)
        check(run_cut(llm, toks, [n]), ref_logits(cfg, w, toks), dtype, f"{name}: prompt of {n}")


def test_the_stream_after_every_layer(models, monkeypatch):
    """The residual stream after each layer in a 32-bit run, against the plain model's."""
    from rusty_llama_b200 import StepEntry
    from rusty_llama_b200.parts import block

    got = []
    plain_forward = block.SharedNormBlock.forward

    def forward_and_keep(self, stream, step, cache, shared_cache=False):
        plain_forward(self, stream, step, cache, shared_cache)
        stream.flush()
        got.append(stream.x.detach().to(torch.float64).cpu())

    monkeypatch.setattr(block.SharedNormBlock, "forward", forward_and_keep)
    for name in CONFIGS:
        cfg, folder, w = models[name]
        toks = tokens(cfg, 70, 3)
        want = pn.plain_streams(cfg, w, toks)[1]
        llm = load(folder, "float32", use_graphs=False)
        s = llm.open_sequence()
        got.clear()
        llm.step([StepEntry(s, toks, [len(toks) - 1])])
        llm.close_sequence(s)
        assert len(got) == len(want) == len(cfg["layers"])
        for i, (g, r) in enumerate(zip(got, want)):
            assert float((g.view_as(r) - r).abs().max()) <= 2e-5 * max(1.0, float(r.abs().max())), f"{name}: layer {i}"


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_of_a_sequence_gives_the_same_bits_in_32_bit(models, name):
    """Whole, token by token from the first token on, and portions down to two tokens across page borders; the convolution's
    record is shorter than, as long as, and longer than a portion."""
    cfg, folder, w = models[name]
    toks = tokens(cfg, 140, 5)
    llm = load(folder, "float32")
    whole = run_cut(llm, toks, [140])
    check_logits(whole, ref_logits(cfg, w, toks), "float32", name)
    for cuts in ([], [2, 3, 61, 64, 7], [63, 2, 64], [1, 1, 126, 2], [16, 17, 15, 32], [2, 2, 2, 2, 1, 2]):
        got = run_cut(llm, toks, cuts)
        assert np.array_equal(got, whole), f"{name}: cut {cuts} changes bits, first at row {np.nonzero((got != whole).any(1))[0][:3]}"
    llm.engine.cache.check_consistent()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_decoding_in_bfloat16(models, name):
    """Portions long enough for the chunked retention (32 tokens and more) and short ones that go token by token."""
    cfg, folder, w = models[name]
    toks = tokens(cfg, 200, 6)
    ref = ref_logits(cfg, w, toks)
    llm = load(folder, "bfloat16")
    for cuts in ([], [2, 62, 2, 30], [190], [33, 64, 65, 31]):
        check(run_cut(llm, toks, cuts), ref, "bfloat16", f"{name}: cut {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_with_leavers_and_reused_slots(models, name, dtype):
    """Three requests of unequal lengths start together and decode together; the shortest leaves first, a fourth starts in
    its slot (whose states and input records must read zero again) and pages; each against itself alone (same bits in
    32-bit) and against the plain model."""
    from rusty_llama_b200 import StepEntry

    cfg, folder, w = models[name]
    reqs = {"a": tokens(cfg, 131, 7), "b": tokens(cfg, 70, 8), "c": tokens(cfg, 3, 9), "d": tokens(cfg, 66, 10)}
    refs = {k: ref_logits(cfg, w, v) for k, v in reqs.items()}
    llm = load(folder, dtype, max_tokens=64 * 6, max_seqs=3)
    got = {k: [] for k in reqs}
    prompt = {"a": 120, "b": 64, "c": 1}
    slots = {k: llm.open_sequence() for k in prompt}
    out = llm.step([StepEntry(slots[k], reqs[k][: prompt[k]], list(range(prompt[k]))) for k in prompt]).cpu().numpy()
    at = 0
    for k in prompt:
        got[k].append(out[at : at + prompt[k]])
        at += prompt[k]
    pos = dict(prompt)
    live = list(prompt)
    while live:
        out = llm.step([StepEntry(slots[k], [reqs[k][pos[k]]], [0]) for k in live]).cpu().numpy()
        for i, k in enumerate(live):
            got[k].append(out[i : i + 1])
            pos[k] += 1
        for k in [k for k in live if pos[k] == len(reqs[k])]:
            llm.close_sequence(slots[k])
            live.remove(k)
            if k == "c":  # the freed slot and pages are taken at once by a new request, alone in its prompt step
                slots["d"] = llm.open_sequence()
                assert slots["d"] == slots["c"]
                got["d"].append(llm.step([StepEntry(slots["d"], reqs["d"][:60], list(range(60)))]).cpu().numpy())
                pos["d"] = 60
                live.append("d")
    llm.engine.cache.check_consistent()
    llm.engine.check_device_status()
    alone = load(folder, dtype, max_tokens=64 * 3, max_seqs=1)
    for k in reqs:
        mine = np.concatenate(got[k], axis=0)
        check(mine, refs[k], dtype, f"{name}: request {k} in the batch")
        if dtype == "float32":
            assert np.array_equal(mine, run_cut(alone, reqs[k], [len(reqs[k])])), f"{name}: request {k} depends on its batch"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_pages_and_graph_buckets(models, dtype):
    """300 tokens one by one after a prompt of 10: page borders at 64, 128, 192, 256, the step from a page table of 4 to one
    of 8; with and without CUDA graphs the 32-bit bits are equal."""
    cfg, folder, w = models["a"]
    toks = tokens(cfg, 310, 12)
    ref = ref_logits(cfg, w, toks)
    got = run_cut(load(folder, dtype), toks, [10])
    check(got, ref, dtype, "long decoding")
    if dtype == "float32":
        assert np.array_equal(got, run_cut(load(folder, dtype, use_graphs=False), toks, [10]))


def test_greedy_generation_through_the_generation_loop(models):
    """`LLM.generate` with temperature 0 (scheduler, batching, sampler) against greedy decoding of the plain model."""
    cfg, folder, w = models["a"]
    llm = load(folder, "float32", max_tokens=64 * 8, max_seqs=4)
    prompts = [tokens(cfg, 9, 20), tokens(cfg, 70, 21), tokens(cfg, 2, 22)]
    outs = llm.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:
            logits = ref_logits(cfg, w, seq)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] > 1e-3 * np.abs(logits).max():  # a clear winner must be the engine's token
                assert int(np.argmax(logits)) == t
            seq.append(t)
        assert len(o) == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_and_command_line(models, dtype, tmp_path):
    """The two programs a user starts: `bin/trace_run` (a prompt whole, then cut, then two requests decoded together in a
    cache that the first run has used) and `bin/rusty_llama` (greedy ids)."""
    import os
    import subprocess
    import sys

    from helpers import REPO, TraceRun

    cfg, folder, w = models["b"]
    a, b = tokens(cfg, 90, 30), tokens(cfg, 7, 31)
    ref = {"a": ref_logits(cfg, w, a), "b": ref_logits(cfg, w, b)}
    run = TraceRun(folder, dtype, str(tmp_path / "out"), 64 * 3, cfg["vocab"])
    try:
        check(run.step([("w", a, range(90))], end=["w"]), ref["a"], dtype, "whole")
        rows = [run.step([("x", a[:80], range(80)), ("y", b[:3], range(3))])]
        got = {"x": [rows[0][:80]], "y": [rows[0][80:]]}
        for t in range(10):
            live = [("x", [a[80 + t]], [0])] + ([("y", [b[3 + t]], [0])] if t < 4 else [])
            end = (["x"] if t == 9 else []) + (["y"] if t == 3 else [])
            out = run.step(live, end=end)
            got["x"].append(out[:1])
            if t < 4:
                got["y"].append(out[1:2])
        check(np.concatenate(got["x"]), ref["a"], dtype, "cut and batched")
        check(np.concatenate(got["y"]), ref["b"], dtype, "the short one")
    finally:
        run.close()
    if dtype == "float32":
        out = subprocess.run(
            [sys.executable, os.path.join(REPO, "bin", "rusty_llama"), folder, "-t", "0", "-n", "12", "-i", " ".join(map(str, b)), "--dtype", "float32"],
            capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        ids = [int(t) for t in out.stdout.split()]
        new = ids[-(12 - len(b)):]
        seq = list(b)
        for t in new:
            logits = ref_logits(cfg, w, seq)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] > 1e-3 * np.abs(logits).max():
                assert int(np.argmax(logits)) == t
            seq.append(t)
