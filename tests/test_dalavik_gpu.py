"""The Dalavik decoder through the engine, and each of its mechanisms alone (GPU), against the plain
64-bit statement in plain_dalavik.py.  The configurations are in dalavik_cases.py: P (odd sizes, exact
kernels, a cache read across another latent layer), Q (the tensor-core kernels' sizes), R (one norm group, no
side input, one head, one kv head, a temperature that steps at every position).
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dalavik_cases as cases
import plain_dalavik as plain
from helpers import ROOT, Trace, assert_close, random_tokens, run_trace_inprocess

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ENGINE_CASES = [(n, d) for n in ("P", "Q", "R", "S") for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("dalavik"))


def stored(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


def runner_for(root, name, dtype, pages=64, requests=4, page=None):
    from inferloop_b200.engine import ModelRunner
    _, _, page_size = cases.CASES[name]
    return ModelRunner.from_folder(cases.folder(root, name, stored(dtype)), dtype=dtype, device=DEV,
                                   page_size=page or page_size, num_pages=pages, max_requests=requests)


def tokens_for(name, n, seed):
    return random_tokens(n, cases.CASES[name][0]["vocab"], seed)


def reference(root, name, dtype, tokens):
    return cases.plain_model(root, name, stored(dtype)).forward(tokens)


# Every sublayer's output is normed to unit size before it joins the stream, so each adds its own rounding at full
# weight, and the test weights are spread out to make the softmaxes sharp: measured against the 64-bit statement, the
# 32-bit engine's worst logit is off by 2e-6 of the largest logit and the bfloat16 engine's by 1.2e-2 (3.8e-3 root mean
# square).  A lost key, a position one off or a sink left out moves logits by tenths.
F32_REL_OF_MAX = 5e-6
BF16_REL_OF_MAX = 2.5e-2


def close(got, ref, dtype, what):
    if dtype == "float32":
        got, ref = got.double().cpu(), ref.double().cpu()
        assert got.shape == ref.shape and torch.isfinite(got).all(), what
        err = float((got - ref).abs().max())
        assert err <= F32_REL_OF_MAX * float(ref.abs().max()), f"{what}: max error {err:.3e}, max |ref| {float(ref.abs().max()):.3e}"
    else:
        assert_close(got, ref, dtype, what, bf16_rel_of_max=BF16_REL_OF_MAX)


def check_trace(outputs, trace, ref_logits, dtype, what):
    """32-bit: every step's rows against the plain logits.  bfloat16: a single row's rounding error varies with the
    position (measured: up to 1e-2 of the largest logit in root mean square, single elements a few times that; the same
    in a whole prompt, token by token, and in the exact kernels), so every element is held to twice the bound, a row's
    root mean square to the bound, and the root mean square over all rows of the trace to a quarter of it."""
    got_all, ref_all = [], []
    for step, rows in trace.rows.items():
        ref = torch.stack([ref_logits[rid][pos] for rid, pos in rows])
        got = torch.from_numpy(outputs[step])
        if dtype == "float32":
            close(got, ref, dtype, f"{what} step {step} rows {rows[:4]}...")
            continue
        assert got.shape == ref.shape and torch.isfinite(got).all(), f"{what} step {step}"
        bound = BF16_REL_OF_MAX * float(ref.abs().max())
        err = (got.double() - ref.double().cpu()).abs()
        assert float(err.max()) <= 2 * bound, f"{what} step {step} rows {rows[:4]}...: max error {float(err.max()):.3e} exceeds {2 * bound:.3e}"
        row_rms = err.pow(2).mean(1).sqrt()
        assert float(row_rms.max()) <= bound, \
            f"{what} step {step} row {rows[int(row_rms.argmax())]}: root-mean-square error {float(row_rms.max()):.3e} exceeds {bound:.3e}"
        got_all.append(got)
        ref_all.append(ref)
    if got_all:
        close(torch.cat(got_all), torch.cat(ref_all), dtype, f"{what}, all rows")


# ------------------------------------------------------------------------------ the engine
@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_whole_prompt_and_every_layer(root, name, dtype):
    """One prompt in one step: the residual stream after every layer, and all logits."""
    from inferloop_b200.engine import StepEntry
    r = runner_for(root, name, dtype)
    toks = tokens_for(name, 45, 1)
    ref, after = cases.plain_model(root, name, stored(dtype)).forward(toks, keep_layers=True)
    got = []
    for b in r.model.blocks:
        def hooked(hidden, step, cache, orig=b.forward):
            orig(hidden, step, cache)
            got.append(hidden.cpu().clone())
        b.forward = hooked
    logits = r.step([StepEntry("a", toks, list(range(len(toks))))])
    assert len(got) == len(after)
    for i, (g, w) in enumerate(zip(got, after)):
        close(g, w, dtype, f"{name} layer {i}")
    close(logits, ref, dtype, f"{name} logits")


@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_prefill_against_token_by_token_and_portions(root, name, dtype):
    """The same sequence whole, token by token from the first token on, and in portions of changing size
    down to two tokens with the last tokens one by one."""
    toks = tokens_for(name, 70, 2)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=80)
    t = Trace()
    for i, tok in enumerate(toks[:40]):
        t.step([("a", [tok], [0])], end=["a"] if i == 39 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} token by token")
    t = Trace()
    at = 0
    for n in (2, 5, 3, 17, 2, 9, 16, 1, 2, 7):
        t.step([("a", toks[at:at + n], [0, n - 1])])
        at += n
    while at < len(toks):
        t.step([("a", toks[at:at + 1], [0])], end=["a"] if at == len(toks) - 1 else [])
        at += 1
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} portions")
    r.cache.check()
    assert all(n == g.pool.num_pages for g, n in zip(r.cache.groups, r.cache.free_pages().values()))


@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_mixed_batches_with_pages_and_slots_used_again(root, name, dtype):
    """Up to four live requests of unequal length, portions beside single tokens, four slots for seven requests
    and a pool that cannot hold all of them: what ends gives its pages to the next.  Every row equals the
    request alone."""
    lens = {"a": 37, "b": 5, "c": 64, "d": 21, "e": 50, "f": 2, "g": 33}
    toks = {k: tokens_for(name, n, 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: reference(root, name, dtype, v) for k, v in toks.items()}
    page = cases.CASES[name][2]
    pages = -(-64 // page) + -(-50 // page) + -(-37 // page) + -(-33 // page) + 1
    r = runner_for(root, name, dtype, pages=pages, requests=4)
    t = Trace()
    cursor = {k: 0 for k in lens}
    waiting, live = list(lens), []
    portion = {"a": [2, 16, 3], "b": [5], "c": [31, 2, 20], "d": [8, 8], "e": [3, 40], "f": [2], "g": [30]}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4:
            need = sum(-(-lens[k] // page) for k in live + [waiting[0]])
            if need > pages:
                break
            live.append(waiting.pop(0))
        entries, ended = [], []
        for k in live:
            plan = portion[k]
            n = plan.pop(0) if plan else 1
            n = min(n, lens[k] - cursor[k])
            entries.append((k, toks[k][cursor[k]:cursor[k] + n], sorted({0, n - 1})))
            cursor[k] += n
            if cursor[k] == lens[k]:
                ended.append(k)
        t.step(entries, end=ended)
        live = [k for k in live if k not in ended]
        step += 1
        assert step < 400
    out = run_trace_inprocess(r, t)
    check_trace(out, t, ref, dtype, f"{name} mixed")
    info = r.cache.inspect()
    assert info["begun"] == len(lens) and info["live_requests"] == 0
    assert any(g["reuses"] > 0 for g in info["groups"]), "no page was used again"
    r.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "bfloat16"), ("R", "float32"), ("Q", "float32")])
def test_long_decoding_through_recorded_graphs(root, name, dtype):
    """A short prompt, then 200 single tokens (recorded decode graphs after the first): the temperature's steps and
    many pages' borders are passed by decoded tokens."""
    toks = tokens_for(name, 220, 3)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=-(-230 // cases.CASES[name][2]))
    t = Trace()
    t.step([("a", toks[:20], [19])])
    for i in range(20, len(toks)):
        t.step([("a", [toks[i]], [0])], end=["a"] if i == len(toks) - 1 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} long decoding")
    assert r.graphs is not None and r.graphs.whole and r.graphs.replays > 150


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "float32"), ("Q", "bfloat16"), ("R", "bfloat16")])
def test_a_long_prompt_whole_and_in_portions(root, name, dtype):
    """600 tokens in one step against the plain model, and against the same prompt in portions of 128, 100 and 37:
    the logits at a position do not depend on the cut."""
    from inferloop_b200.engine import StepEntry
    toks = tokens_for(name, 600, 77)
    want = list(range(5, 600, 10)) + [599]
    r = runner_for(root, name, dtype, pages=-(-600 // cases.CASES[name][2]) + 2)
    whole = r.step([StepEntry("w", toks, want)]).float().cpu().clone()
    r.end("w")
    close(whole, reference(root, name, dtype, toks)[want], dtype, f"{name} 600 tokens whole")
    for portion in (128, 100, 37):
        rows = []
        for at in range(0, 600, portion):
            part = toks[at:at + portion]
            out = r.step([StepEntry("p", part, [w - at for w in want if at <= w < at + len(part)])])
            rows.append(out.float().cpu().clone())
        r.end("p")
        close(torch.cat(rows), whole, dtype, f"{name} portions of {portion} against the whole prompt")


@pytest.mark.parametrize("name,dtype", [("Q", "bfloat16"), ("Q", "float32")])
def test_single_tokens_on_both_sides_of_a_chunk_of_keys(root, name, dtype):
    """Two unequal requests decode together while one of them passes key 256, where the kernel for single tokens
    starts a second chunk of keys (its first token there reads one key of the new chunk); the other stays
    inside its first chunk.  Each against the plain model of its own tokens."""
    toks = {"a": tokens_for(name, 270, 11), "b": tokens_for(name, 60, 12)}
    ref = {k: reference(root, name, dtype, v) for k, v in toks.items()}
    page = cases.CASES[name][2]
    r = runner_for(root, name, dtype, pages=-(-270 // page) + -(-60 // page) + 2)
    t = Trace()
    t.step([("a", toks["a"][:250], [0, 249]), ("b", toks["b"][:40], [39])])
    for i in range(20):
        t.step([("a", [toks["a"][250 + i]], [0]), ("b", [toks["b"][40 + i]], [0])], end=["a", "b"] if i == 19 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} two requests around key 256")
    r.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "bfloat16"), ("R", "float32")])
def test_greedy_generation_through_the_entry_point(root, name, dtype):
    from inferloop_b200 import Engine, SamplingParams
    config, _, page = cases.CASES[name]
    model = cases.plain_model(root, name, stored(dtype))
    prompts = [tokens_for(name, n, 30 + n) for n in (3, 12, 31, 64)]
    engine = Engine(cases.folder(root, name, stored(dtype)), dtype=dtype, block_size=page, num_gpu_blocks_override=96,
                    max_num_seqs=4, prefill_chunk_tokens=32, max_num_batched_tokens=40)
    new = 12
    got = engine.generate(prompts, SamplingParams(), max_new_tokens=new)
    for p, g in zip(prompts, got):
        assert len(g) == new
        ref = model.forward(list(p) + list(g))[len(p) - 1:-1]
        bound = (1e-2 if dtype == "bfloat16" else 1e-5) * float(ref.abs().max())
        for i, tok in enumerate(g):        # teacher-forced: every chosen token is the best one within the bound
            assert ref[i, tok] >= ref[i].max() - 2 * bound
    info = engine.inspect()
    assert info["running"] == 0 and all(g["free"] == g["total"] for g in info["cache"]["groups"])


def test_the_command_line_generates_from_a_dalavik_folder(root):
    name, dtype = "R", "float32"
    prompt = tokens_for(name, 9, 41)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "generate", cases.folder(root, name, stored(dtype)),
                          "--tokens", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", dtype, "--block-size", "16",
                          "--num-gpu-blocks-override", "8"], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["tokens"]
    ref = cases.plain_model(root, name, stored(dtype)).forward(list(prompt) + got)[len(prompt) - 1:-1]
    for i, tok in enumerate(got):
        assert ref[i, tok] >= ref[i].max() - 2e-5 * float(ref.abs().max())


def test_the_trace_program_replays_a_dalavik_folder(root, tmp_path):
    name, dtype = "P", "float32"
    toks = {"x": tokens_for(name, 40, 5), "y": tokens_for(name, 9, 6)}
    ref = {k: reference(root, name, dtype, v) for k, v in toks.items()}
    t = Trace()
    t.step([("x", toks["x"][:33], [0, 32]), ("y", toks["y"][:2], [1])])
    t.step([("x", toks["x"][33:34], [0]), ("y", toks["y"][2:], [0, 6])], end=["y"])
    for i in range(34, 40):
        t.step([("x", toks["x"][i:i + 1], [0])], end=["x"] if i == 39 else [])
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", cases.folder(root, name, stored(dtype)), "--dtype", dtype,
           "--out", str(tmp_path), "--max-tokens", "128", "--block-size", "4"]
    proc = subprocess.run(cmd, input=t.lines(), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr
    vocab = cases.CASES[name][0]["vocab"]
    out = {s: np.fromfile(os.path.join(str(tmp_path), f"{s}.f32"), dtype="<f4").reshape(len(rows), vocab) for s, rows in t.rows.items()}
    check_trace(out, t, ref, dtype, "trace program")


# ------------------------------------------------------------------------------ each mechanism alone
class FakeStep:
    """The device arrays of a batch, for kernels called without an engine: sequences of `lens` tokens that
    start at `starts`."""

    def __init__(self, lens, starts, tokens=None):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.h_q_len = list(lens)
        self.n_seqs, self.n_tokens = len(lens), sum(lens)
        self.max_q_len = max(lens)
        self.decode_only = all(n == 1 for n in lens)
        self.cu_q = i32([sum(lens[:i]) for i in range(len(lens) + 1)])
        self.positions = i32([s + j for n, s in zip(lens, starts) for j in range(n)])
        self.seq_of_token = i32([i for i, n in enumerate(lens) for _ in range(n)])
        self.h_kv_len = [s + n for n, s in zip(lens, starts)]
        self.max_kv_len = max(self.h_kv_len)
        self.tokens = i32(tokens if tokens is not None else [0] * self.n_tokens)
        self.position_tables = {}


def f32(t):
    return t.float().to(DEV).contiguous()


def name_of(dtype):
    return "bfloat16" if dtype == torch.bfloat16 else "float32"


@pytest.mark.parametrize("width,groups", [(72, 3), (256, 2), (64, 1), (4096, 8), (100, 50), (129, 1), (2048, 64)])
def test_grouped_norm_alone_and_added_to_the_stream(width, groups):
    """The grouped norm as a plain norm (also of a slice of wider rows), and as the step between two sublayers: the
    stream gets the normed rows, the next sublayer its input, the buffer is zero again."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(width + groups)
    rows, eps = 7, 1e-5
    y = torch.randn(rows, width + 8, generator=g) * torch.linspace(0.1, 30.0, width + 8)      # parts of very unequal size
    w = 1 + 0.1 * torch.randn(width, generator=g)
    x = torch.randn(rows, width, generator=g)
    ref = plain.group_norm(y[:, 4:4 + width].double(), w.double(), eps, groups)
    for out_dtype in (torch.float32, torch.bfloat16):
        yd = y.to(DEV)
        out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
        ops.group_norm_add(yd[:, 4:4 + width], f32(w), eps, groups, out=out)
        assert_close(out, ref, "float32" if out_dtype == torch.float32 else "bfloat16", "grouped norm of a slice")
        assert torch.equal(yd.cpu(), y)
        yc = y[:, 4:4 + width].contiguous().to(DEV)
        xd = x.to(DEV)
        ops.group_norm_add(yc, f32(w), eps, groups, x=xd, out=out, zero=True)
        assert_close(xd, x.double() + ref, "float32", "stream after the sublayer")
        assert torch.equal(out.float(), xd.to(out_dtype).float())
        assert not yc.any()
        yc = y[:, 4:4 + width].contiguous().to(DEV)
        xd = x.to(DEV)
        ops.group_norm_add(yc, f32(w), eps, groups, x=xd)
        assert_close(xd, x.double() + ref, "float32", "stream after the last sublayer")
        assert torch.equal(yc.cpu(), y[:, 4:4 + width])


@pytest.mark.parametrize("n", [1, 5, 72 * 3, 4096 * 3 + 4])
def test_cast_and_zero(n):
    from inferloop_b200.csrc import ops
    x = torch.randn(n, generator=torch.Generator().manual_seed(n)).view(1, n).to(DEV)
    for dt in (torch.float32, torch.bfloat16):
        xc = torch.empty(1, n, dtype=dt, device=DEV)
        y = torch.full((1, n), 3.0, device=DEV)
        ops.cast_zero(x, xc, y)
        assert torch.equal(xc, x.to(dt)) and not y.any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_slice_of_a_token_table(dtype):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    V, layers, dim, T = 37, 3, 5, 11
    table = torch.randn(V, layers * dim, generator=g).to(dtype)
    a = (3 * torch.randn(T, dim, generator=g)).to(dtype)
    toks = random_tokens(T, V, 9)
    for i in range(layers):
        out = torch.empty(T, dim, dtype=dtype, device=DEV)
        ops.gated_rows(a.to(DEV), table.to(DEV), i * dim, torch.tensor(toks, dtype=torch.int32, device=DEV), out)
        ref = plain.gelu_tanh(a.double()) * table.double()[torch.tensor(toks)][:, i * dim:(i + 1) * dim]
        assert_close(out, ref, name_of(dtype), f"gated slice {i}", bf16_rel_of_max=2.0 ** -8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_relu_gate_of_the_feed_forward(dtype):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    for rows, width in ((3, 40), (9, 64)):
        gu = torch.randn(rows, 2 * width, generator=g).to(dtype)
        out = torch.empty(rows, width, dtype=dtype, device=DEV)
        ops.silu_mul(gu.to(DEV), out, "relu")
        ref = torch.relu(gu.double()[:, :width]) * gu.double()[:, width:]
        assert_close(out, ref, name_of(dtype), "relu gate", bf16_rel_of_max=2.0 ** -8)


@pytest.mark.parametrize("tokens", [1, 8, 70, 300])
@pytest.mark.parametrize("gate", ["relu", "silu"])
def test_the_gate_inside_the_tensor_core_product(tokens, gate):
    """relu(gate) * up (or silu) formed in the epilogue of the product over the weight whose rows interleave
    blocks of 64 gate rows and 64 up rows, for a single token, a few, and many tokens."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(7 + tokens)
    width, inter = 192, 320 if tokens < 100 else 1024
    x = torch.randn(tokens, width, generator=g).bfloat16()
    wg = (torch.randn(inter, width, generator=g) / width ** 0.5).bfloat16()
    wu = (torch.randn(inter, width, generator=g) / width ** 0.5).bfloat16()
    blocks = inter // 64
    w = torch.stack([wg.view(blocks, 64, width), wu.view(blocks, 64, width)], dim=1).reshape(2 * inter, width).contiguous()
    out = torch.empty(tokens, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x.to(DEV), w.to(DEV), out, swiglu=True, gate=gate)
    a, b = x.double() @ wg.double().T, x.double() @ wu.double().T
    ref = (torch.relu(a) if gate == "relu" else a * torch.sigmoid(a)) * b
    assert_close(out, ref, "bfloat16", f"{gate} gate in the product, {tokens} tokens", bf16_rel_of_max=2.0 ** -7)


def paged(rows, page, order):
    """rows [n, width] laid into pages in the order given: (cache [pages, 1, page, width], block table row)."""
    n, width = rows.shape
    n_pages = -(-n // page)
    cache = torch.zeros(len(order), 1, page, width, dtype=rows.dtype)
    for p in range(n_pages):
        part = rows[p * page:(p + 1) * page]
        cache[order[p], 0, :part.shape[0]] = part
    return cache, list(order[:n_pages])


@pytest.mark.parametrize("rank,tail,rot,heads,d", [(18, 6, 4, 3, 8), (96, 32, 32, 8, 32), (24, 2, 2, 1, 24), (10, 5, 4, 2, 7), (16, 0, 0, 2, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_row_with_a_rotated_part_and_the_queries_tails(rank, tail, rot, heads, d, dtype):
    """The cache row [normed latent | rotated shared key part] at the token's place of its page, pages out of order,
    two sequences that start in the middle of a page; only the first `rot` elements of the part turn; the queries'
    tails turn the same way into their place behind the mapped query; a layer without a cache of its own turns
    its queries only."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.config.spec import PartSpec
    from inferloop_b200.parts import registry
    from inferloop_b200.parts.base import BuildContext, Workspace
    g = torch.Generator().manual_seed(rank * 10 + tail)
    page, eps, base = 4, 1e-5, 77.0
    lens, starts = [9, 3], [6, 1]
    T = sum(lens)
    step = FakeStep(lens, starts)
    col0 = 5
    proj = torch.randn(T, col0 + rank + tail + 3, generator=g).to(dtype if dtype == torch.bfloat16 else torch.float32)
    w = 1 + 0.1 * torch.randn(rank, generator=g)
    qh = d + tail
    q_src = torch.randn(T, heads * qh, generator=g).to(dtype)
    pos = step.positions.cpu()
    angles = None
    if rot:
        ctx = BuildContext(dtype=dtype, device=torch.device(DEV), workspace=Workspace(torch.device(DEV)))
        angles = registry.build("position", PartSpec.make("rope_interleaved", theta=base, rotary_dim=rot), ctx).table(step)
    table = torch.tensor([[5, 2, 7, 0, -1], [3, 1, -1, -1, -1]], dtype=torch.int32, device=DEV)
    cache = torch.zeros(8, 1, page, rank + tail, dtype=dtype, device=DEV)
    row = rank + tail
    q_dst = torch.zeros(T, heads * row, dtype=dtype, device=DEV)
    ops.latent_write_rot(proj.to(DEV), col0, rank, tail, rot, angles, f32(w), eps, step, table, cache,
                         q_src.to(DEV) if tail else None, q_dst if tail else None, q_col0=d, q_head_stride=qh, heads=heads)
    c = plain.rms(proj.double()[:, col0:col0 + rank], eps) * w.double()
    part = proj.double()[:, col0 + rank:col0 + rank + tail]
    if rot:
        part = plain.rotate_pairs(part, pos, base, rot)
    want_rows = torch.cat([c, part], dim=1)
    seq = step.seq_of_token.cpu()
    for t in range(T):
        p = int(pos[t])
        got = cache[int(table[int(seq[t]), p // page]), 0, p % page].float().cpu()
        assert_close(got, want_rows[t], name_of(dtype), f"cache row of token {t}", bf16_rel_of_max=2.0 ** -7)
    if tail:
        qt = q_src.double().view(T, heads, qh)[..., d:]
        if rot:
            qt = plain.rotate_pairs(qt, pos, base, rot)
        got = q_dst.float().cpu().view(T, heads, row)
        assert_close(got[..., rank:], qt, name_of(dtype), "queries' tails", bf16_rel_of_max=2.0 ** -7)
        assert not got[..., :rank].any()
        # a layer that reads another layer's cache: its queries' tails only, the cache untouched
        before = cache.clone()
        q_dst.zero_()
        ops.latent_write_rot(proj.to(DEV), col0, rank, tail, rot, angles, None, eps, step, None, None,
                             q_src.to(DEV), q_dst, q_col0=d, q_head_stride=qh, heads=heads)
        assert torch.equal(before, cache)
        assert_close(q_dst.float().cpu().view(T, heads, row)[..., rank:], qt, name_of(dtype), "queries' tails alone", bf16_rel_of_max=2.0 ** -7)


@pytest.mark.parametrize("T,heads,K,N,xhs,ohs", [(5, 3, 8, 18, 14, 24), (70, 8, 32, 96, 64, 128), (33, 4, 96, 48, 128, 48), (1, 2, 7, 5, 7, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_head_products_with_strides(T, heads, K, N, xhs, ohs, dtype):
    """A head's input may be a part of a wider head row, and its output may land in one; what lies beside stays."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(T + K)
    x = torch.randn(T, heads * xhs + 3, generator=g).to(dtype)
    w = torch.randn(heads, K, N, generator=g).to(dtype)
    out = torch.full((T, heads * ohs), 7.0, dtype=dtype, device=DEV)
    ops.head_matmul(x.to(DEV), w.to(DEV), out, x_head_stride=xhs, out_head_stride=ohs)
    xs = torch.stack([x.double()[:, i * xhs:i * xhs + K] for i in range(heads)], 1)
    ref = torch.einsum("thk,hkn->thn", xs, w.double())
    got = out.float().cpu().view(T, heads, ohs)
    assert_close(got[..., :N], ref, name_of(dtype), "per-head product", bf16_rel_of_max=2.0 ** -7)
    assert (got[..., N:] == 7.0).all()


def shaped_attention_reference(q, k, v, positions, scale, per, cap, temp, r1, r2, mix, sink):
    """q [T, H, d] of ONE sequence whose keys k [n, G, d], v [n, G, dv] are all cached; returns [T, H, dv]."""
    T, H, _ = q.shape
    n = k.shape[0]
    kh, vh = k.repeat_interleave(per, 1), v.repeat_interleave(per, 1)
    pos = positions.double()
    f = torch.ones(T, dtype=torch.float64)
    if temp is not None:
        f = 1.0 + temp[0] * torch.log(torch.floor((pos + 1) / temp[1]) + 1.0)
    s = torch.einsum("ihd,jhd->hij", q * f[:, None, None], kh) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    dist = (pos[:, None] - torch.arange(n, dtype=torch.float64)[None, :]).clamp(min=0)
    if r1 is not None:
        s = s - r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None])
    if mix is not None:
        s = torch.einsum("hg,gij->hij", mix, s)
    seen = torch.arange(n)[None, :] <= positions[:, None]
    s = s.masked_fill(~seen[None], -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(s - top)
    total = e.sum(-1, keepdim=True) + (torch.exp(sink[:, None, None] - top) if sink is not None else 0.0)
    return torch.einsum("hij,jhd->ihd", e / total, vh)


MIX_GEOMETRIES = [  # H, G, d, dv, page, cap, temp, with distance, with mixing, with sink
    (4, 2, 12, 20, 4, 5.0, (0.7, 3), True, True, True),
    (8, 2, 64, 64, 16, 30.0, (0.5, 16), True, True, True),
    (4, 4, 128, 128, 16, 0.0, None, True, True, False),
    (3, 1, 16, 8, 8, 2.0, (1.0, 1), False, True, True),
    (1, 1, 32, 8, 8, 0.0, None, True, False, True),
    (6, 3, 80, 96, 32, 25.0, (0.4, 48), True, True, True),
    (12, 12, 32, 48, 8, 10.0, (0.2, 100), True, True, True),
    (16, 16, 64, 128, 16, 0.0, None, False, True, True),
    (16, 4, 128, 128, 16, 15.0, (0.3, 128), True, True, True),
]


@pytest.mark.parametrize("geometry", MIX_GEOMETRIES)
@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "exact"), (torch.bfloat16, "exact"), (torch.bfloat16, "tensor cores")])
def test_attention_with_shaped_and_mixed_scores(geometry, dtype, kernel):
    """A sequence of 300 cached keys with its pages out of order, read by a portion of the prompt (positions in
    the middle and at the end) and by single tokens of other sequences in the same launch.  One far key (position 3)
    and one at a page's last place stand out: their keys are aligned with one head's queries and scaled, so a
    kernel that lost them, or a distance that is one off, shows; the mixing matrix is far from the identity."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts.base import Workspace
    H, G, d, dv, page, cap, temp, with_dist, with_mix, with_sink = geometry
    if kernel == "tensor cores" and not ops.attention_mix_tc_supported(H, G, d, dv):
        pytest.skip("the tensor-core kernel does not take this geometry")
    g = torch.Generator().manual_seed(H * 100 + d)
    n, per, scale = 300, H // G, 1.0 / math.sqrt(d)
    k = torch.randn(n, G, d, generator=g).to(dtype)
    v = torch.randn(n, G, dv, generator=g).to(dtype)
    lens, starts = [37, 1, 1, 20], [n - 37, 150, 4, 100]       # all four read (a prefix of) the same cached sequence
    q = torch.randn(sum(lens), H, d, generator=g)
    hot = torch.randn(d, generator=g)
    hot = hot / hot.norm() * 3.0
    q[:, 0] += hot * 2.0                                       # head 0 of every query looks for the hot keys
    kk = k.float()
    kk[3, 0] = hot * 4.0
    kk[page * 4 - 1, 0] = hot * 3.0
    k = kk.to(dtype)
    q = q.to(dtype)
    r1 = torch.linspace(0.2, 1.5, H) if with_dist else None
    r2 = torch.linspace(2.0, 0.05, H) if with_dist else None
    mix = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)) if with_mix else None
    sink = torch.linspace(-1.0, 3.0, H) if with_sink else None
    n_pages = -(-n // page)
    order = torch.randperm(n_pages + 3, generator=g).tolist()
    k_cache = torch.zeros(n_pages + 3, G, page, d, dtype=dtype)
    v_cache = torch.zeros(n_pages + 3, G, page, dv, dtype=dtype)
    for p in range(n_pages):
        part = slice(p * page, min(n, (p + 1) * page))
        k_cache[order[p], :, :part.stop - part.start] = k[part].transpose(0, 1)
        v_cache[order[p], :, :part.stop - part.start] = v[part].transpose(0, 1)
    table = torch.tensor([order[:n_pages]] * len(lens), dtype=torch.int32, device=DEV)
    step = FakeStep(lens, starts)
    out = torch.zeros(sum(lens), H * dv, dtype=dtype, device=DEV)
    args = dict(sink=None if sink is None else f32(sink), head_mix=None if mix is None else f32(mix),
                dist_r1=None if r1 is None else f32(r1), dist_r2=None if r2 is None else f32(r2),
                softcap=cap, temp_coef=temp[0] if temp else 0.0, temp_every=temp[1] if temp else 1,
                workspace=Workspace(torch.device(DEV)) if kernel == "tensor cores" else None, decode_chunk=64)
    ops.attention_mixed_heads(q.view(-1, H * d).to(DEV), out, k_cache.to(DEV), v_cache.to(DEV), step, table, 0, scale, H, G, d, dv, **args)
    if kernel == "tensor cores":
        # single tokens alone: their keys cut into chunks of 64 whose records are added by a second launch
        singles = FakeStep([1, 1, 1], [150, 4, n - 1])
        rows = [37, 38, 36]
        out1 = torch.zeros(3, H * dv, dtype=dtype, device=DEV)
        ops.attention_mixed_heads(q.view(-1, H * d)[rows].to(DEV).contiguous(), out1, k_cache.to(DEV), v_cache.to(DEV), singles,
                                  table[:3].contiguous(), 0, scale, H, G, d, dv, **args)
        got1 = out1.float().cpu()
        # the same launch as the first, with the blocks' keys cut into chunks of 64 (as few blocks with many keys are):
        # portions that end inside a chunk, at positions before and after several borders, beside single tokens
        chunk, ops.MIX_PROMPT_CHUNK = ops.MIX_PROMPT_CHUNK, 64
        try:
            out2 = torch.zeros(sum(lens), H * dv, dtype=dtype, device=DEV)
            ops.attention_mixed_heads(q.view(-1, H * d).to(DEV), out2, k_cache.to(DEV), v_cache.to(DEV), step, table, 0, scale, H, G, d, dv, **args)
        finally:
            ops.MIX_PROMPT_CHUNK = chunk
    dd = lambda t: None if t is None else t.double()
    ref = shaped_attention_reference(q.double(), k.double(), v.double(), step.positions.cpu(), scale, per, cap, temp,
                                     dd(r1), dd(r2), dd(mix), dd(sink))
    bound = 2.0 ** -8 * (1.0 + float(v.float().abs().max()) / max(1e-9, float(ref.abs().max())))
    assert_close(out.float().cpu().view(-1, H, dv), ref, name_of(dtype), "attention with mixed heads", bf16_rel_of_max=bound)
    if kernel == "tensor cores":
        assert_close(got1.view(3, H, dv), ref[rows], "bfloat16", "single tokens in chunks", bf16_rel_of_max=bound)
        assert_close(out2.float().cpu().view(-1, H, dv), ref, "bfloat16", "portions with their keys in chunks", bf16_rel_of_max=bound)
    # the hot keys carry weight: without them the result differs by far more than the bound
    k2 = k.double().clone()
    k2[3, 0] = 0
    ref2 = shaped_attention_reference(q.double(), k2, v.double(), step.positions.cpu(), scale, per, cap, temp,
                                      dd(r1), dd(r2), dd(mix), dd(sink))
    assert float((ref2 - ref).abs().max()) > 5 * bound * float(ref.abs().max())
