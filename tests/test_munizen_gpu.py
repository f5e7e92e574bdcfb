"""The Munizen design in the engine against the plain implementation of tests/plain_munizen.py.

Every test makes its own small configuration and random weights (tests/munizen_cases.py), writes a model
folder with the engine's random-weights mode, reads it back with the plain reader, and compares logits:
float32 to 2e-4 of the largest logit, bfloat16 to 6e-2 (tiny widths average little out).  In float32 the rows
of every cut must also EQUAL the rows of the whole request bit for bit: the 32-bit kernels take a token's
sums in an order that depends on its position only.
"""
import numpy as np
import pytest
import torch

import plain_munizen as plain
from munizen_cases import CASES, SINGLE, Harness, attention_layer, config, delta_layer, rel_err, write_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def plain_logits(folder, tokens):
    cfg, w = plain.read_model(folder)
    return plain.forward(cfg, w, list(tokens)).numpy()


def tokens_of(rng, n, vocab):
    return rng.integers(0, vocab, n).tolist()


# ---- each mechanism alone ------------------------------------------------------------------------
def test_group_norm_of_weighted_streams_kernel():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(1)
    for T, S, W, groups in ((5, 3, 48, 3), (2, 1, 40, 1), (7, 4, 60, 4), (3, 16, 32, 2)):
        x = torch.randn(T, S, W, generator=g) * 3
        coef, w = torch.randn(S, generator=g), 1 + 0.1 * torch.randn(W, generator=g)
        want = plain.grouped_rms_norm(plain.hyper_read(x.double().permute(1, 0, 2), coef.double()), w.double(), 1e-5, groups)
        out = torch.empty(T, W, device="cuda")
        ops.streams_norm(x.cuda(), w.cuda(), out, 1e-5, groups, coef.cuda())
        assert rel_err(out.cpu().numpy(), want.numpy()) < 1e-5
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")         # chosen rows, the plain sum of the streams
        out2 = torch.empty(2, W, device="cuda", dtype=torch.bfloat16)
        ops.streams_norm(x.cuda(), w.cuda(), out2, 1e-5, groups, None, rows)
        want2 = plain.grouped_rms_norm(x.double().sum(1), w.double(), 1e-5, groups)[[T - 1, 0]]
        assert rel_err(out2.float().cpu().numpy(), want2.numpy()) < 1e-2


def test_streams_write_and_broadcast_kernels():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(2)
    for T, S, W in ((6, 3, 48), (1, 1, 40), (9, 5, 24), (4, 16, 16)):
        x0 = torch.randn(T, W, generator=g)
        x = torch.empty(T, S, W, device="cuda")
        ops.streams_broadcast(x0.cuda(), x)
        assert torch.equal(x.cpu(), x0[:, None, :].expand(T, S, W))
        x = torch.randn(T, S, W, generator=g)
        y, mix, out = torch.randn(T, W, generator=g), torch.randn(S, S, generator=g), torch.randn(S, generator=g)
        want = plain.hyper_write(x.double().permute(1, 0, 2), y.double(), mix.double(), out.double()).permute(1, 0, 2)
        xd = x.cuda()
        ops.streams_write(xd, y.cuda(), mix.cuda(), out.cuda())
        assert rel_err(xd.cpu().numpy(), want.numpy()) < 1e-5


def test_token_shift_kernel_over_two_steps():
    """Two sequences in two steps (one of them a single token in the second): the first token of every portion
    takes the row the step before left in the slot's state, zeros at position 0."""
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(3)
    W = 40
    mu = torch.rand(W, generator=g)
    seqs = [torch.randn(7, W, generator=g), torch.randn(4, W, generator=g)]
    want = [plain.token_shift(s.double(), mu.double()).numpy() for s in seqs]
    state = torch.full((3, W), float("nan"), device="cuda")
    slots = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    got = [[], []]
    for cut0, cut1 in (((0, 5), (0, 3)), ((5, 7), (3, 4))):
        h = torch.cat([seqs[0][cut0[0]:cut0[1]], seqs[1][cut1[0]:cut1[1]]]).cuda()
        n0, n1 = cut0[1] - cut0[0], cut1[1] - cut1[0]
        out = torch.empty_like(h)
        ops.token_shift(h, mu.cuda(), state, out, i32(list(range(cut0[0], cut0[1])) + list(range(cut1[0], cut1[1]))),
                        i32([0] * n0 + [1] * n1), slots, i32([0, n0, n0 + n1]))
        got[0].append(out[:n0].cpu()); got[1].append(out[n0:].cpu())
    for b in range(2):
        assert rel_err(torch.cat(got[b]).numpy(), want[b]) < 1e-6
    assert torch.equal(state[2].cpu(), seqs[0][-1]) and torch.equal(state[0].cpu(), seqs[1][-1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_layer_of_each_kind(tmp_path, name, dtype):
    folder = write_model(SINGLE[name], str(tmp_path / name), seed=7)
    rng = np.random.default_rng(5)
    toks = tokens_of(rng, 45, SINGLE[name]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, dtype)
    whole = h.run(toks)
    assert rel_err(whole, want) < TOL[dtype]
    one_by_one = h.run(toks, [1])
    assert rel_err(one_by_one, want) < TOL[dtype]
    if dtype == "float32":
        assert np.array_equal(whole, one_by_one)


def test_layers_outputs_one_after_another(tmp_path):
    """The residual after every call of the schedule (a looped layer counts each time)."""
    from carbon_engine_b200.engine.batch import StepEntry
    folder = write_model(CASES["P"], str(tmp_path / "P"))
    cfg, w = plain.read_model(folder)
    toks = tokens_of(np.random.default_rng(1), 30, cfg["vocab"])
    trace = []
    plain.forward(cfg, w, toks, trace)
    h = Harness(folder, "float32")
    rid = h.open()
    ctx, rows, commits = h.runner.prepare([StepEntry(rid, toks, [0])])
    got = []
    h.model.forward(ctx, h.storage, tap=lambda i, x: got.append(x.sum(1).cpu().numpy()))
    assert len(got) == len(trace) == 6
    for i, (a, b) in enumerate(zip(got, trace)):
        assert rel_err(a, b.numpy()) < 1e-4, i


# ---- whole models: cuts, batches, reuse ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompt_portions_and_decoding(tmp_path, name, dtype):
    from carbon_engine_b200 import ops
    folder = write_model(CASES[name], str(tmp_path / name), seed=11)
    rng = np.random.default_rng(3)
    toks = tokens_of(rng, 83, CASES[name]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, dtype, page_size=8, pages=16)          # 128 tokens of pages: every run reuses the last one's
    ops.reset_kernel_counts()
    whole = h.run(toks)
    if name in ("T", "U", "V"):           # head sizes of the tensor-core kernel: bfloat16 must have taken it, float32 never
        assert ("diff_attention_mma_kernel" in ops.kernel_counts()) == (dtype == "bfloat16")
    assert rel_err(whole, want) < TOL[dtype], "whole"
    for cuts in ([1], [2], [3, 2, 7, 2, 16, 5], [40, 1, 1, 1], [64, 19]):
        got = h.run(toks, cuts)
        assert rel_err(got, want) < TOL[dtype], cuts
        if dtype == "float32":
            assert np.array_equal(got, whole), cuts
    assert h.storage.manager.free_pages(0) == 16 and h.storage.manager.free_slots() == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_reused_pages_and_slots(tmp_path, dtype):
    """Up to three live requests in two slots more than needed, portions beside single tokens, a request left out
    of some steps, finished requests' pages and slots taken by the next: every row equals the request alone."""
    name = "P"
    folder = write_model(CASES[name], str(tmp_path / name), seed=13)
    rng = np.random.default_rng(9)
    lengths = [61, 17, 40, 1, 2, 33, 25]
    reqs = [tokens_of(rng, n, CASES[name]["vocab"]) for n in lengths]
    want = [plain_logits(folder, t) for t in reqs]
    h = Harness(folder, dtype, page_size=8, pages=20, slots=3)          # 160 tokens: three live requests at most
    alone = [h.run(t) for t in reqs] if dtype == "float32" else None
    waiting, live, done_rows = list(range(len(reqs))), {}, {i: [] for i in range(len(reqs))}
    portions, k, step_no = [2, 5, 1, 9, 3, 14], 0, 0
    while waiting or live:
        while waiting and len(live) < 3 and sum(-(-len(reqs[i]) // 8) for i in live) + -(-len(reqs[waiting[0]]) // 8) <= 20:
            i = waiting.pop(0)
            live[i] = [h.open(), 0]
        entries, who = [], []
        for i, (rid, pos) in list(live.items()):
            if step_no % 4 == 3 and i % 2 == 0 and len(live) > 1:
                continue                                     # left out of this step
            left = len(reqs[i]) - pos
            n = 1 if left <= 6 else min(portions[k % len(portions)], left - 6)      # the last tokens one by one
            k += 1
            entries.append((rid, reqs[i][pos:pos + n], range(n)))
            who.append((i, n))
        step_no += 1
        if not entries:
            continue
        rows = h.step(entries)
        at = 0
        for i, n in who:
            done_rows[i].append(rows[at:at + n])
            at += n
            live[i][1] += n
            if live[i][1] == len(reqs[i]):
                h.close(live.pop(i)[0])
    for i in range(len(reqs)):
        got = np.concatenate(done_rows[i])
        assert rel_err(got, want[i]) < TOL[dtype], i
        if alone is not None:
            assert np.array_equal(got, alone[i]), i
    assert h.storage.manager.free_pages(0) == 20 and h.storage.manager.free_slots() == 3


# ---- keys that stand out: far away, at page borders, around every block of the mask -----------------------
def standout_model(tmp_path, mask, page=8, aligned=False):
    """One attention layer (and a delta layer behind it) whose marker token's key stands out: the marker's
    embedding is made several times larger, so wherever a query may see it, its score dominates the map (with
    either sign).  ``aligned``: in map 1, one unrotated element of every query is given a large bias and the same
    element of the keys is made to read the marker's embedding, so that EVERY query scores the marker's key
    far above hundreds of others."""
    from helpers import read_raw_safetensors, write_safetensors_plain
    import os
    raw = config([attention_layer(heads=2, kv_heads=1, dim=16, vdim=16, rot=(4, 10000.0), mask=mask, ff=None, scale=0.6),
                  delta_layer(heads=2, dim=8, rank=2)], width=32, vocab=50, groups=1, streams=2)
    folder = write_model(raw, str(tmp_path / f"standout{mask}"), seed=21)
    path = os.path.join(folder, "model.safetensors")
    t = read_raw_safetensors(path)
    t["embed"][7] = t["embed"][7] * 6.0
    for n in ("l0.mix.q", "l0.mix.k"):
        t[n] = t[n] * 3.0
    if aligned:
        j, d = 10, 16                                # an element past the rotated ones
        e = t["embed"][7].float()
        t["l0.mix.k"][j] = (2.0 * e / e.norm()).to(t["l0.mix.k"].dtype)
        for head in range(2):
            t["l0.mix.q.b"][head * 2 * d + j] = 4.0
    write_safetensors_plain(path, t)
    return folder, raw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_that_stands_out_is_seen_exactly_inside_its_block(tmp_path, dtype):
    mask = 21                                   # no multiple of the page size (8), so block and page borders differ
    folder, raw = standout_model(tmp_path, mask)
    rng = np.random.default_rng(4)
    n = 150
    base = [int(t) for t in rng.integers(8, 50, n)]
    h = Harness(folder, dtype, page_size=8, pages=64)
    for marker_at in (0, 20, 21, 41, 42, 63, 64, 100):          # first token, last and first of a block, page borders
        toks = list(base)
        toks[marker_at] = 7
        want = plain_logits(folder, toks)
        # the plain model itself must tell "inside" from "outside": the marker moves the rows of its own block only
        plain_base = plain_logits(folder, base)
        block_end = (marker_at // mask + 1) * mask
        moved = np.abs(want - plain_base).max(axis=1) / np.abs(plain_base).max()
        assert moved[marker_at:block_end].min() > 0.02
        whole = h.run(toks)
        assert rel_err(whole, want) < TOL[dtype], marker_at
        # the block's edge met in a portion's middle, at its start, and by tokens decoded one by one
        for cuts in ([block_end - 1, 1, 1, 1, 1, 40], [block_end, 2, 2, 50], [max(marker_at, 1), 1, 1, 1, 30], [13]):
            got = h.run(toks, cuts)
            assert rel_err(got, want) < TOL[dtype], (marker_at, cuts)
            if dtype == "float32":
                assert np.array_equal(got, whole)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(tmp_path, dtype):
    """No mask block in reach: the marker at the start must still carry its weight 700 tokens later, in a
    prompt and in decoding, across many pages."""
    folder, raw = standout_model(tmp_path, 100000, page=16, aligned=True)
    rng = np.random.default_rng(6)
    toks = [int(t) for t in rng.integers(8, 50, 720)]
    toks[3] = 7
    want = plain_logits(folder, toks)
    without = list(toks)
    without[3] = 9
    moved = np.abs(want - plain_logits(folder, without)).max(axis=1) / np.abs(want).max()
    assert moved[700:].min() > 0.02                       # the plain model says the far key matters
    h = Harness(folder, dtype, page_size=16, pages=48, max_step_tokens=1024)
    assert rel_err(h.run(toks), want) < TOL[dtype]
    rid = h.open()
    rows = [h.step([(rid, toks[:690], [689])])]
    for p in range(690, 720):
        rows.append(h.step([(rid, toks[p:p + 1], [0])]))
    h.close(rid)
    assert rel_err(np.concatenate(rows), want[689:]) < TOL[dtype]


def test_long_decoding_keeps_the_state(tmp_path):
    """300 tokens one by one after a short prompt, in float32: the recurrent state, the shift's row and the
    cache must carry every token (bit for bit the rows of the whole prompt)."""
    folder = write_model(CASES["S"], str(tmp_path / "S"), seed=2)
    toks = tokens_of(np.random.default_rng(8), 310, CASES["S"]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, "float32", page_size=8, pages=48)
    whole = h.run(toks)
    got = h.run(toks, [10] + [1] * 300)
    assert rel_err(got, want) < TOL["float32"] and np.array_equal(got, whole)


def test_first_tokens_of_a_sequence_in_a_reused_slot(tmp_path):
    """A slot and pages that held a longer request: the next request's first tokens must start from nothing
    (zero state, no previous row, no keys)."""
    folder = write_model(CASES["P"], str(tmp_path / "P"), seed=5)
    rng = np.random.default_rng(12)
    h = Harness(folder, "float32", page_size=8, pages=12, slots=1, poison=False)
    h.run(tokens_of(rng, 90, CASES["P"]["vocab"]))
    for n in (1, 2, 3, 9):
        toks = tokens_of(rng, n, CASES["P"]["vocab"])
        want = plain_logits(folder, toks)
        assert rel_err(h.run(toks), want) < TOL["float32"]
        assert rel_err(h.run(toks, [1]), want) < TOL["float32"]


# ---- through the entry point -------------------------------------------------------------------------
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(tmp_path, graphs):
    from carbon_engine_b200 import Engine, SamplingParams
    folder = write_model(CASES["P"], str(tmp_path / "P"), seed=17)
    cfg, w = plain.read_model(folder)
    rng = np.random.default_rng(2)
    prompts = [tokens_of(rng, n, cfg["vocab"]) for n in (23, 5, 41)]
    eng = Engine(folder, dtype="float32", page_size=8, max_running_requests=3, max_prefill_tokens=16, kv_tokens=256,
                 cuda_graphs=graphs)
    assert eng.cuda_graphs == graphs
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == 12 and out.finish_reason == "length"
        toks = list(prompt)
        for t in out.token_ids:
            row = plain.forward(cfg, w, toks)[-1]
            assert t == int(row.argmax()) or float(row.max() - row[t]) < 4e-4 * float(row.abs().max())
            toks.append(t)
    eng.storage.manager.check()


def test_trace_replay_program_on_a_munizen_folder(tmp_path):
    import json, os, subprocess, sys
    from helpers import ROOT
    folder = write_model(CASES["Q"], str(tmp_path / "Q"), seed=1)
    toks = tokens_of(np.random.default_rng(3), 40, CASES["Q"]["vocab"])
    want = plain_logits(folder, toks)
    out = str(tmp_path / "out")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[25:27], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[27:], "want": [12]}, {"id": "b", "tokens": toks[:3], "want": [2]}],
              "end": ["a", "b"]}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                           "--out", out, "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    got0 = np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(2, -1)
    assert not os.path.exists(os.path.join(out, "1.f32"))
    assert rel_err(got0, want[[0, 24]]) < 2e-4 and rel_err(got2, want[[39, 2]]) < 2e-4


def test_command_line_writes_and_generates_a_munizen_model(tmp_path):
    """``tiny-model --arch munizen`` then ``generate``: the printed ids are the plain implementation's greedy ones."""
    import ast, os, re, subprocess, sys
    from helpers import ROOT
    carbon = [sys.executable, os.path.join(ROOT, "bin", "carbon")]
    out = str(tmp_path / "tiny_m")
    p = subprocess.run(carbon + ["tiny-model", "--arch", "munizen", "--out", out, "--layers", "4", "--hidden", "48", "--heads", "3",
                                 "--kv-heads", "1", "--head-dim", "16", "--vocab", "120", "--seed", "9", "--streams", "3",
                                 "--mask-size", "6", "--max-positions", "256"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "wrote" in p.stdout, p.stderr[-2000:]
    cfg, w = plain.read_model(out)
    assert cfg["architecture"] == "Munizen" and cfg["streams"] == 3 and len(cfg["layers"]) == 4
    prompt = tokens_of(np.random.default_rng(5), 17, 120)
    p = subprocess.run(carbon + ["generate", "--model", out, "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "8",
                                 "--ignore-eos", "--print-ids", "--dtype", "f32", "--kv-tokens", "256", "--page-size", "16"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = [ast.literal_eval(m) for m in re.findall(r"output_ids: (\[[^\]]*\])", p.stderr)][0]
    toks = list(prompt)
    for t in ids:
        row = plain.forward(cfg, w, toks)[-1]
        assert t == int(row.argmax()) or float(row.max() - row[t]) < 4e-4 * float(row.abs().max())
        toks.append(t)
    assert len(ids) == 8
