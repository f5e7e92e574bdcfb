"""The Lunerax design in the engine against the plain implementation of tests/plain_lunerax.py.

Every test makes its own small configuration and random weights (tests/lunerax_cases.py), writes a model folder with
the engine's random-weights mode, reads it back with the plain reader, and compares logits: float32 to 2e-4 of the
largest logit, bfloat16 to 6e-2 (tiny widths average little out).  In float32 the rows of every cut must also EQUAL
the rows of the whole request bit for bit: the 32-bit kernels take a token's sums in an order that depends on its
position only.
"""
import os

import numpy as np
import pytest
import torch

import plain_lunerax as plain
from lunerax_cases import CASES, SINGLE, Harness, attention, config, delta, latent, rel_err, write_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def plain_logits(folder, tokens, layers_out=None):
    cfg, w = plain.read_model(folder)
    return plain.forward(cfg, w, list(tokens), layers_out).numpy()


def tokens_of(rng, n, vocab):
    return rng.integers(0, vocab, n).tolist()


# ---- each mechanism alone: the kernels --------------------------------------------------------------------
def test_layer_norm_kernel_with_row_gather():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(1)
    for T, W in ((5, 40), (3, 192), (2, 2500), (7, 33)):
        x = torch.randn(T, W, generator=g) * 3 + 1.5
        w, b = 1 + 0.1 * torch.randn(W, generator=g), 0.2 * torch.randn(W, generator=g)
        want = plain.layer_norm(x.double(), w.double(), b.double(), 1e-5)
        out = torch.empty(T, W, device="cuda")
        ops.layernorm(x.cuda(), w.cuda(), b.cuda(), out, 1e-5)
        assert rel_err(out.cpu().numpy(), want.numpy()) < 1e-5
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
        out2 = torch.empty(2, W, device="cuda", dtype=torch.bfloat16)
        ops.layernorm(x.cuda(), w.cuda(), b.cuda(), out2, 1e-5, rows)
        assert rel_err(out2.float().cpu().numpy(), want[[T - 1, 0]].numpy()) < 1e-2


def test_rms_norm_add_tanh_cap_copy_and_side_gate_kernels():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(2)
    T, W, D, V = 6, 52, 7, 19
    y, w, x = torch.randn(T, W, generator=g), 1 + 0.1 * torch.randn(W, generator=g), torch.randn(T, W, generator=g)
    xd = x.cuda()
    ops.rmsnorm_add(y.cuda(), w.cuda(), xd, 1e-6)
    assert rel_err(xd.cpu().numpy(), (x.double() + plain.rms_norm(y.double(), w.double(), 1e-6)).numpy()) < 1e-6
    z = (torch.randn(T, W, generator=g) * 20).cuda()
    want = 7.5 * torch.tanh(z.double().cpu() / 7.5)
    ops.tanh_cap(z, 7.5)
    assert rel_err(z.cpu().numpy(), want.numpy()) < 1e-6
    src = torch.randn(T, W, generator=g).cuda()
    out = torch.empty(T, 9, device="cuda", dtype=torch.bfloat16)
    ops.copy_cols(src, 13, 9, out)
    assert torch.equal(out.cpu(), src[:, 13:22].cpu().to(torch.bfloat16))
    table = torch.randn(V, 3 * D, generator=g)
    toks = torch.tensor([3, 0, 18, 18, 7, 1], dtype=torch.int32)
    zz = torch.randn(T, D, generator=g) * 2
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gate = torch.empty(T, D, device="cuda")
    ops.side_gate(zz.cuda(), table.cuda(), toks.cuda(), gate, D, status)
    want = plain.gelu_tanh(zz.double()) * table.double()[toks.long()][:, D:2 * D]
    assert rel_err(gate.cpu().numpy(), want.numpy()) < 1e-6 and int(status.item()) == 0


def test_relu_gated_product_on_both_kernels_and_scaled_embedding():
    from carbon_engine_b200 import ops, ops_tensor
    g = torch.Generator().manual_seed(3)
    for M, N, K in ((5, 24, 40), (70, 136, 64), (300, 256, 128)):
        a, w = torch.randn(M, K, generator=g), torch.randn(2 * N, K, generator=g) * 0.2
        want = (torch.relu(a.double() @ w[:N].double().T) * (a.double() @ w[N:].double().T)).numpy()
        out = torch.empty(M, N, device="cuda")
        ops.gemm_plain(a.cuda(), w.cuda(), out, ops.GEMM_RELUGLU)
        assert rel_err(out.cpu().numpy(), want) < 1e-5
        ab, wb = a.cuda().bfloat16(), w.cuda().bfloat16()
        outb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        assert ops_tensor.gemm_bf16(ab, wb, outb, ops.GEMM_RELUGLU)
        wantb = (torch.relu(ab.double() @ wb[:N].double().T) * (ab.double() @ wb[N:].double().T)).cpu().numpy()
        assert rel_err(outb.float().cpu().numpy(), wantb) < 1e-2
    table = torch.randn(11, 20, generator=g).cuda()
    toks = torch.tensor([4, 10, 0], dtype=torch.int32, device="cuda")
    x = torch.empty(3, 20, device="cuda")
    ops.embed(table, toks, x, torch.zeros(1, dtype=torch.int32, device="cuda"), 2.5)
    assert torch.allclose(x, table[toks.long()] * 2.5)


def test_product_per_head_with_gate_and_value_blend_kernels():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(4)
    for T, H, N, K in ((5, 3, 20, 14), (33, 2, 70, 45), (1, 5, 8, 96)):
        x = torch.randn(T, H * K + 6, generator=g)
        w = torch.randn(H, N, K, generator=g) * 0.3
        gate = torch.randn(T, H * N + 4, generator=g)
        want = torch.einsum("thk,hnk->thn", x[:, 3:3 + H * K].reshape(T, H, K).double(), w.double())
        out = torch.zeros(T, H * N, device="cuda")
        ops.head_matmul(x.cuda()[:, 3:], K, w.cuda(), out, N, H, N, K)
        assert rel_err(out.cpu().numpy(), want.reshape(T, -1).numpy()) < 1e-5
        ops.head_matmul(x.cuda()[:, 3:], K, w.cuda(), out, N, H, N, K, gate=gate.cuda()[:, 4:])
        want_g = want * torch.sigmoid(gate[:, 4:].double()).reshape(T, H, N)
        assert rel_err(out.cpu().numpy(), want_g.reshape(T, -1).numpy()) < 1e-5
    # bfloat16 with sizes in multiples of 16: the tensor-core form, with a ragged last tile of tokens and of outputs
    ops.reset_kernel_counts()
    for T, H, N, K in ((70, 3, 48, 32), (5, 2, 128, 80), (130, 1, 16, 16)):
        x = torch.randn(T, H * K, generator=g).cuda().bfloat16()
        w = (torch.randn(H, N, K, generator=g) * 0.3).cuda().bfloat16()
        gate = torch.randn(T, H * N, generator=g).cuda()
        want = torch.einsum("thk,hnk->thn", x.double().reshape(T, H, K), w.double()) * torch.sigmoid(gate.double()).reshape(T, H, N)
        out = torch.zeros(T, H * N, device="cuda", dtype=torch.bfloat16)
        ops.head_matmul(x, K, w, out, N, H, N, K, gate=gate)
        assert rel_err(out.float().cpu().numpy(), want.reshape(T, -1).cpu().numpy()) < 1e-2
    assert ops.kernel_counts().get("head_matmul_wmma_kernel") == 3
    rows, first = torch.randn(6, 30, generator=g), torch.randn(6, 25, generator=g)
    rd = rows.cuda()
    ops.value_mix(rd, 8, 12, first.cuda(), 5, 0.3)
    want = rows.clone()
    want[:, 8:20] = 0.7 * rows[:, 8:20] + 0.3 * first[:, 5:17]
    assert torch.allclose(rd.cpu(), want, atol=1e-6)


# ---- each mechanism alone: one layer of each kind ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_layer_of_each_kind(tmp_path, name, dtype):
    folder = write_model(SINGLE[name], str(tmp_path / name), seed=7)
    toks = tokens_of(np.random.default_rng(5), 45, SINGLE[name]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, dtype)
    whole = h.run(toks)
    assert rel_err(whole, want) < TOL[dtype]
    one_by_one = h.run(toks, [1])
    assert rel_err(one_by_one, want) < TOL[dtype]
    if dtype == "float32":
        assert np.array_equal(whole, one_by_one)


def test_layers_outputs_one_after_another(tmp_path):
    """The residual after every layer, so that a fault shows in the layer it is in."""
    from carbon_engine_b200.engine.batch import StepEntry
    folder = write_model(CASES["A"], str(tmp_path / "A"))
    cfg, w = plain.read_model(folder)
    toks = tokens_of(np.random.default_rng(1), 30, cfg["vocab"])
    trace = []
    plain.forward(cfg, w, toks, trace)
    h = Harness(folder, "float32")
    rid = h.open()
    ctx, rows, commits = h.runner.prepare([StepEntry(rid, toks, [0])])
    got = []
    h.model.forward(ctx, h.storage, tap=lambda i, x: got.append(x.cpu().numpy().copy()))
    assert len(got) == len(trace) == 5
    for i, (a, b) in enumerate(zip(got, trace)):
        assert rel_err(a, b.numpy()) < 1e-4, i


# ---- whole models: cuts, batches, reuse ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompt_portions_and_decoding(tmp_path, name, dtype):
    from carbon_engine_b200 import ops
    folder = write_model(CASES[name], str(tmp_path / name), seed=11)
    toks = tokens_of(np.random.default_rng(3), 140 if name in ("T", "V") else 83, CASES[name]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, dtype, page_size=8, pages=24)          # 192 tokens of pages: every run reuses the last one's
    ops.reset_kernel_counts()
    whole = h.run(toks)
    if name in ("T", "V"):        # head sizes of the tensor-core kernel: bfloat16 must have taken it, float32 never
        assert ("masked_attention_mma_kernel" in ops.kernel_counts()) == (dtype == "bfloat16")
    assert rel_err(whole, want) < TOL[dtype], "whole"
    for cuts in ([1], [2], [3, 2, 7, 2, 16, 5], [40, 1, 1, 1], [64, 19]):
        got = h.run(toks, cuts)
        assert rel_err(got, want) < TOL[dtype], cuts
        if dtype == "float32":
            assert np.array_equal(got, whole), cuts
    m = h.storage.manager
    assert all(m.free_pages(g) == h.storage.groups[g].num_pages for g in range(len(h.storage.groups))) and m.free_slots() == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_reused_pages_and_slots(tmp_path, dtype):
    """Up to three live requests, portions beside single tokens, a request left out of some steps, finished requests'
    pages and slots taken by the next: every row equals the request alone."""
    name = "A"
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
    assert h.storage.manager.free_slots() == 3


# ---- keys that stand out: far away, at page borders, around the window's edge and the kept first tokens ----------
def standout_model(tmp_path, layer, tag):
    """One attention layer in which EVERY query scores the marker token's key far above hundreds of others, wherever it
    may see it.  The norm's bias is a constant vector (its output's other part has zero mean, so a query row of equal
    entries reads the constant and little else): one element of every query head becomes a constant.  The same element
    of the keys reads the direction of the marker's normed embedding: large for the marker, noise for all others.  In
    the latent layer the two travel through the first element of the query latent and of the key latent."""
    from helpers import read_raw_safetensors, write_safetensors_plain
    W = 32
    raw = config([layer], width=W, vocab=50, side=0, logit_cap=0, scale=2.0)
    folder = write_model(raw, str(tmp_path / f"standout_{tag}"), seed=21)
    path = os.path.join(folder, "model.safetensors")
    t = read_raw_safetensors(path)
    m, j = layer["mixer"], 10
    e = t["embed"][7].float()
    mark = (e - e.mean()) / e.std(unbiased=False)                 # the marker's normed embedding: orthogonal to equal entries
    t["l0.norm1"] = torch.ones(W)
    t["l0.norm1.b"] = torch.full((W,), W ** -0.5)                # its product with a row of equal entries 1/sqrt(W) is 1
    ones = torch.full((W,), W ** -0.5)
    if layer["type"] == "attention":
        d = m["dim"]
        for head in range(m["heads"]):
            t["l0.mix.q"][head * d + j] = ones.to(t["l0.mix.q"].dtype)
        for head in range(m["kv_heads"]):
            t["l0.mix.k"][head * d + j] = (0.6 * mark).to(t["l0.mix.k"].dtype)
    else:
        d, dr = m["dim"], m["rot_dim"]
        t["l0.mix.dq"][0] = ones.to(t["l0.mix.dq"].dtype)
        t["l0.mix.dkv"][0] = (0.02 * mark).to(t["l0.mix.dkv"].dtype)
        t["l0.mix.dq.norm"] = torch.ones(m["q_rank"])
        t["l0.mix.dkv.norm"] = torch.ones(m["kv_rank"])
        for head in range(m["heads"]):
            t["l0.mix.uq"][head * (d + dr) + j] = 0.0
            t["l0.mix.uq"][head * (d + dr) + j, 0] = 1.2
            t["l0.mix.uk"][head * d + j] = 0.0
            t["l0.mix.uk"][head * d + j, 0] = 1.2
    write_safetensors_plain(path, t)
    return folder, raw


def marker_effect(folder, toks, at):
    """How far the plain model's rows move when the marker at ``at`` is replaced by an ordinary token."""
    want = plain_logits(folder, toks)
    other = list(toks)
    other[at] = 9
    return want, np.abs(want - plain_logits(folder, other)).max(axis=1) / np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_a_key_that_stands_out_is_seen_exactly_inside_the_window(tmp_path, kind, dtype):
    window, keep = 21, 3                        # no multiple of the page size (8), so window and page borders differ
    layer = attention(heads=2, kv_heads=1, dim=16, vdim=16, window=window, keep_first=keep, scale=0.6, softcap=9.0, ff=None) \
        if kind == "attention" else latent(heads=2, dim=16, rot_dim=4, rot_dims=4, vdim=16, q_rank=12, kv_rank=24, window=window, scale=0.6)
    folder, raw = standout_model(tmp_path, layer, kind)
    rng = np.random.default_rng(4)
    n = 120
    base = [int(t) for t in rng.integers(10, 50, n)]
    h = Harness(folder, dtype, page_size=8, pages=64)
    for marker_at in (0, 2, 3, 15, 16, 40, 63, 64):          # kept tokens and the first one that is not, page borders
        toks = list(base)
        toks[marker_at] = 7
        want, moved = marker_effect(folder, toks, marker_at)
        last_seen = marker_at + window - 1
        # the plain model itself must tell "inside" from "outside": the marker moves the rows that see it only
        assert moved[marker_at:last_seen + 1].min() > 1e-3
        kept = kind == "attention" and marker_at < keep
        assert (moved[last_seen + 1:].min() > 1e-3) if kept else (moved[last_seen + 1:].max() < 1e-9)
        whole = h.run(toks)
        assert rel_err(whole, want) < TOL[dtype], marker_at
        # the window's edge met in a portion's middle, at its start, and by tokens decoded one by one
        for cuts in ([last_seen, 1, 1, 1, 1, 40], [last_seen + 1, 2, 2, 50], [max(marker_at, 1), 1, 1, 1, 30], [13]):
            got = h.run(toks, cuts)
            assert rel_err(got, want) < TOL[dtype], (marker_at, cuts)
            if dtype == "float32":
                assert np.array_equal(got, whole)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["kept_first", "no_window", "latent_no_window"])
def test_a_far_key_among_hundreds(tmp_path, kind, dtype):
    """The marker near the start must still carry its weight 700 tokens later, in a prompt and in decoding, across many
    pages: as a kept first token of a short window, and without any window."""
    layer = {"kept_first": attention(heads=2, kv_heads=1, dim=16, vdim=16, window=12, keep_first=4, scale=0.6, softcap=0, ff=None),
             "no_window": attention(heads=2, kv_heads=2, dim=16, vdim=8, window=0, scale=0.6, softcap=9.0, ff=None),
             "latent_no_window": latent(heads=2, dim=16, rot_dim=4, rot_dims=2, vdim=16, q_rank=12, kv_rank=24, window=0, scale=0.6)}[kind]
    folder, raw = standout_model(tmp_path, layer, kind)
    rng = np.random.default_rng(6)
    toks = [int(t) for t in rng.integers(10, 50, 720)]
    toks[3] = 7
    want, moved = marker_effect(folder, toks, 3)
    assert moved[700:].min() > 1e-3                       # the plain model says the far key matters
    h = Harness(folder, dtype, page_size=16, pages=48, max_step_tokens=1024)
    assert rel_err(h.run(toks), want) < TOL[dtype]
    rid = h.open()
    rows = [h.step([(rid, toks[:690], [689])])]
    for p in range(690, 720):
        rows.append(h.step([(rid, toks[p:p + 1], [0])]))
    h.close(rid)
    assert rel_err(np.concatenate(rows), want[689:]) < TOL[dtype]


def test_long_decoding_keeps_the_state(tmp_path):
    """300 tokens one by one after a short prompt, in float32: the recurrent state, the convolution's kept rows and the
    caches must carry every token (bit for bit the rows of the whole prompt)."""
    folder = write_model(CASES["C"], str(tmp_path / "C"), seed=2)
    toks = tokens_of(np.random.default_rng(8), 310, CASES["C"]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, "float32", page_size=8, pages=48)
    whole = h.run(toks)
    got = h.run(toks, [10] + [1] * 300)
    assert rel_err(got, want) < TOL["float32"] and np.array_equal(got, whole)


def test_first_tokens_of_a_sequence_in_a_reused_slot(tmp_path):
    """A slot and pages that held a longer request: the next request's first tokens must start from nothing (zero
    state, no kept convolution inputs, no keys), also when it is shorter than the convolution."""
    folder = write_model(CASES["A"], str(tmp_path / "A"), seed=5)
    rng = np.random.default_rng(12)
    h = Harness(folder, "float32", page_size=8, pages=12, slots=1, poison=False)
    h.run(tokens_of(rng, 90, CASES["A"]["vocab"]))
    for n in (1, 2, 3, 9):
        toks = tokens_of(rng, n, CASES["A"]["vocab"])
        want = plain_logits(folder, toks)
        assert rel_err(h.run(toks), want) < TOL["float32"]
        assert rel_err(h.run(toks, [1]), want) < TOL["float32"]


# ---- through the entry point -------------------------------------------------------------------------
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(tmp_path, graphs):
    from carbon_engine_b200 import Engine, SamplingParams
    folder = write_model(CASES["A"], str(tmp_path / "A"), seed=17)
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


def test_trace_replay_program_on_a_lunerax_folder(tmp_path):
    import json, subprocess, sys
    from helpers import ROOT
    folder = write_model(CASES["C"], str(tmp_path / "C"), seed=1)
    toks = tokens_of(np.random.default_rng(3), 40, CASES["C"]["vocab"])
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


def test_command_line_writes_and_generates_a_lunerax_model(tmp_path):
    """``tiny-model --arch lunerax`` then ``generate``: the printed ids are the plain implementation's greedy ones."""
    import ast, re, subprocess, sys
    from helpers import ROOT
    carbon = [sys.executable, os.path.join(ROOT, "bin", "carbon")]
    out = str(tmp_path / "tiny_l")
    p = subprocess.run(carbon + ["tiny-model", "--arch", "lunerax", "--out", out, "--layers", "5", "--hidden", "48", "--heads", "3",
                                 "--kv-heads", "1", "--head-dim", "16", "--vocab", "120", "--seed", "9", "--side-dim", "6",
                                 "--mask-size", "6", "--max-positions", "256"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "wrote" in p.stdout, p.stderr[-2000:]
    cfg, w = plain.read_model(out)
    assert cfg["architecture"] == "Lunerax" and cfg["token_side"]["dim"] == 6 and len(cfg["layers"]) == 5
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
