"""The Zebivik decoder through the engine, and each of its mechanisms alone (GPU), against the plain 64-bit
statement in plain_zebivik.py.  The configurations are in zebivik_cases.py: K (odd sizes, exact kernels, groups of
experts of which two of three stay, a layer without feed-forward), L (the tensor-core kernels' sizes, values as wide
as keys and narrower, one group of four kept), M (everything plural is one, sizes that are multiples of nothing),
N (recurrences only: no pages, only state slots), P (heads and values of 128, dense units only).
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zebivik as plain
import zebivik_cases as cases
from helpers import ROOT, Trace, assert_close, check_trace, random_tokens, run_trace_inprocess

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ENGINE_CASES = [(n, d) for n in ("K", "L", "M", "N", "P") for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("zebivik"))


def stored(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


def runner_for(root, name, dtype, pages=64, requests=4, page=None):
    from inferloop_b200.engine import ModelRunner
    _, _, page_size = cases.CASES[name]
    return ModelRunner.from_folder(cases.folder(root, name, stored(dtype)), dtype=dtype, device=DEV,
                                   page_size=page or page_size, num_pages=pages, max_requests=requests)


_TOKENS = {}


def tokens_for(root, name, dtype, n, seed):
    key = (name, dtype, n, seed)
    if key not in _TOKENS:
        model = cases.plain_model(root, name, stored(dtype))
        _TOKENS[key] = cases.decided_tokens(model, n, cases.CASES[name][0]["vocab"], seed, 2e-2 if dtype == "bfloat16" else 1e-4)
    return _TOKENS[key]


def reference(root, name, dtype, tokens):
    return cases.plain_model(root, name, stored(dtype)).forward(tokens)


# ------------------------------------------------------------------------------ the engine
@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_whole_prompt_and_every_layer(root, name, dtype):
    """One prompt in one step: the residual stream after every layer, and all logits."""
    from inferloop_b200.engine import StepEntry
    r = runner_for(root, name, dtype)
    toks = tokens_for(root, name, dtype, 45, 1)
    per_layer = []
    ref = cases.plain_model(root, name, stored(dtype)).forward(toks, per_layer)
    got = []
    for b in r.model.blocks:
        def hooked(hidden, step, cache, orig=b.forward):
            orig(hidden, step, cache)
            got.append(hidden.cpu().clone())
        b.forward = hooked
    logits = r.step([StepEntry("a", toks, list(range(len(toks))))])
    assert len(got) == len(per_layer) == len(cases.CASES[name][0]["layers"])
    for i, (g, w) in enumerate(zip(got, per_layer)):
        assert_close(g, w, dtype, f"{name} layer {i}", bf16_rel_of_max=2e-2)
    assert_close(logits, ref, dtype, f"{name} logits")


@pytest.mark.parametrize("name,dtype", ENGINE_CASES)
def test_prefill_against_token_by_token_and_portions(root, name, dtype):
    """The same sequence whole, token by token from the first token on, and in portions of changing size
    down to two tokens with the last tokens one by one."""
    toks = tokens_for(root, name, dtype, 70, 2)
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
    """Up to four live requests of unequal length, portions beside single tokens, four state slots for seven
    requests and a pool that cannot hold all of them: what ends gives its pages and its slot (both recurrences'
    states, the convolution's inputs) to the next.  Every row equals the request alone."""
    lens = {"a": 37, "b": 5, "c": 64, "d": 21, "e": 50, "f": 2, "g": 33}
    toks = {k: tokens_for(root, name, dtype, n, 10 + i) for i, (k, n) in enumerate(lens.items())}
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
    if r.cache.groups:
        assert any(g["reuses"] > 0 for g in info["groups"]), "no page was used again"
    r.cache.check()


@pytest.mark.parametrize("name,dtype", [("K", "float32"), ("L", "bfloat16"), ("M", "float32"), ("N", "bfloat16")])
def test_long_decoding_through_recorded_graphs(root, name, dtype):
    """A short prompt, then 200 single tokens (recorded decode graphs after the first): the slow heads of the linear
    attention and the slow channels of the recurrence still carry the prompt at the end."""
    toks = tokens_for(root, name, dtype, 220, 3)
    ref = {"a": reference(root, name, dtype, toks)}
    r = runner_for(root, name, dtype, pages=-(-230 // cases.CASES[name][2]))
    t = Trace()
    t.step([("a", toks[:20], [19])])
    for i in range(20, len(toks)):
        t.step([("a", [toks[i]], [0])], end=["a"] if i == len(toks) - 1 else [])
    check_trace(run_trace_inprocess(r, t), t, ref, dtype, f"{name} long decoding")
    assert r.graphs is not None and r.graphs.whole and r.graphs.replays > 150


@pytest.mark.parametrize("name,dtype", [("K", "float32"), ("L", "float32"), ("L", "bfloat16"), ("M", "float32"), ("N", "float32")])
def test_a_long_prompt_whole_and_in_portions(root, name, dtype):
    """700 tokens in one step (both recurrences run in chunks side by side; keys hundreds of tokens back at every page
    border) against the same prompt in portions of 128 (chunks again, other borders), 100 and 37 (one pass each): the
    logits at a position do not depend on the cut; in 32-bit, where no routing decision is close, also against the
    plain model."""
    from inferloop_b200.engine import StepEntry
    toks = random_tokens(700, cases.CASES[name][0]["vocab"], 77)
    want = list(range(5, 700, 10)) + [699]
    r = runner_for(root, name, dtype, pages=-(-700 // cases.CASES[name][2]) + 2)
    whole = r.step([StepEntry("w", toks, want)]).float().cpu().clone()
    r.end("w")
    if dtype == "float32":
        model = cases.plain_model(root, name, stored(dtype))
        if model.least_margin(toks) > 1e-4:
            assert_close(whole, model.forward(toks)[want], dtype, f"{name} 700 tokens whole")
    for portion in (128, 100, 37):
        rows = []
        for at in range(0, 700, portion):
            part = toks[at:at + portion]
            out = r.step([StepEntry("p", part, [w - at for w in want if at <= w < at + len(part)])])
            rows.append(out.float().cpu().clone())
        r.end("p")
        if dtype == "float32":
            err = (torch.cat(rows).double() - whole.double()).abs().max()
            assert err <= 2e-5 * whole.abs().max(), f"{name} portions of {portion}: {float(err):.3e}"
        else:
            assert_close(torch.cat(rows), whole, dtype, f"{name} portions of {portion} against the whole prompt")


@pytest.mark.parametrize("name,dtype", [("K", "float32"), ("L", "bfloat16"), ("M", "float32")])
def test_greedy_generation_through_the_entry_point(root, name, dtype):
    from inferloop_b200 import Engine, SamplingParams
    config, _, page = cases.CASES[name]
    model = cases.plain_model(root, name, stored(dtype))
    prompts = [tokens_for(root, name, dtype, n, 30 + n) for n in (3, 12, 31, 64)]
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


def test_the_command_line_generates_from_a_zebivik_folder(root):
    name, dtype = "M", "float32"
    prompt = tokens_for(root, name, dtype, 9, 41)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "generate", cases.folder(root, name, stored(dtype)),
                          "--tokens", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", dtype, "--block-size", "16",
                          "--num-gpu-blocks-override", "8"], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["tokens"]
    ref = cases.plain_model(root, name, stored(dtype)).forward(list(prompt) + got)[len(prompt) - 1:-1]
    for i, tok in enumerate(got):
        assert ref[i, tok] >= ref[i].max() - 2e-5 * float(ref.abs().max())


def test_the_trace_program_replays_a_zebivik_folder(root, tmp_path):
    name, dtype = "K", "float32"
    toks = {"x": tokens_for(root, name, dtype, 40, 5), "y": tokens_for(root, name, dtype, 9, 6)}
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
    start at `starts`, in slots `slots`."""

    def __init__(self, lens, starts, slots):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.h_q_len = list(lens)
        self.n_seqs, self.n_tokens = len(lens), sum(lens)
        self.max_q_len = max(lens)
        self.decode_only = all(n == 1 for n in lens)
        self.cu_q = i32([sum(lens[:i]) for i in range(len(lens) + 1)])
        self.positions = i32([s + j for n, s in zip(lens, starts) for j in range(n)])
        self.seq_of_token = i32([i for i, n in enumerate(lens) for _ in range(n)])
        self.slots = i32(slots)
        self.h_kv_len = [s + n for n, s in zip(lens, starts)]
        self.max_kv_len = max(self.h_kv_len)
        self.position_tables = {}


def f32(t):
    return t.float().to(DEV).contiguous()


@pytest.mark.parametrize("width", [1, 50, 256, 4100])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_without_statistics_alone_and_with_the_residual_sum(width, dtype):
    """tanh(alpha x) g + b on rows of every width, into another buffer and over its own input; then the norm on a
    sublayer's output, the sum into the stream times a constant, the next sublayer's input and the zeroed buffer
    as one launch."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    T = 9
    x, y = 2 * torch.randn(T, width, generator=g), 3 * torch.randn(T, width, generator=g)
    w = {"n": 1 + 0.2 * torch.randn(width, generator=g), "n.b": 0.3 * torch.randn(width, generator=g), "n.alpha": torch.tensor(0.7),
         "m": 1 + 0.2 * torch.randn(width, generator=g), "m.b": 0.3 * torch.randn(width, generator=g), "m.alpha": torch.tensor(1.3)}
    wd = {k: v.double() for k, v in w.items()}
    n = (f32(w["n.alpha"].reshape(1)), f32(w["n"]), f32(w["n.b"]))
    m = (f32(w["m.alpha"].reshape(1)), f32(w["m"]), f32(w["m.b"]))
    tol = "float32" if dtype == torch.float32 else "bfloat16"
    out = torch.empty(T, width, dtype=dtype, device=DEV)
    ops.dyt(f32(x), *n, out)
    assert_close(out, plain.dyt(x.double(), wd, "n"), tol, "norm")
    own = f32(x)
    ops.dyt(own, *n, own)
    assert_close(own, plain.dyt(x.double(), wd, "n"), "float32", "norm over its input")
    xs, ys = f32(x), f32(y)
    ops.dyt_add(ys, n, 0.4, xs, next_norm=m, out=out, zero=True)
    new = x.double() + 0.4 * plain.dyt(y.double(), wd, "n")
    assert_close(xs, new, "float32", "stream")
    assert_close(out, plain.dyt(new, wd, "m"), tol, "next input")
    assert float(ys.abs().max()) == 0.0
    xs, ys = f32(x), f32(y)
    ops.dyt_add(ys, n, -1.5, xs)
    assert_close(xs, x.double() - 1.5 * plain.dyt(y.double(), wd, "n"), "float32", "stream alone")
    assert torch.equal(ys.cpu(), y)


def test_rotation_frequencies_rescaled_by_wavelength():
    """The three bands (kept, blended, divided) against the plain statement; no rescaling without the key."""
    from inferloop_b200.config.spec import PartSpec
    from inferloop_b200.parts import registry
    from inferloop_b200.parts.base import BuildContext, Workspace
    ctx = BuildContext(dtype=torch.float32, device=torch.device(DEV), workspace=Workspace(torch.device(DEV)))
    for base, dims, scaling in ((50.0, 8, (4.0, 1.0, 3.0, 40.0)), (10000.0, 64, (8.0, 1.0, 4.0, 512.0)), (7.0, 2, (2.0, 0.5, 8.0, 16.0)), (300.0, 12, None)):
        part = registry.build("position", PartSpec.make("rope_neox", theta=base, rotary_dim=dims, scaling=scaling), ctx)
        rot = {"base": base, "dims": dims}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
        want = plain.frequencies(rot)
        got = part.inv_freq().cpu()
        assert torch.allclose(got, want, rtol=1e-14, atol=0)
        if scaling:
            plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
            assert dims < 8 or ((got == plainf).any() and (got < plainf).any())
        step = FakeStep([5], [1000], [0])
        table = part.table(step).cpu().double()
        ang = torch.arange(1000, 1005).double()[:, None] * want[None, :]
        assert (table[..., 0] - torch.cos(ang)).abs().max() < 1e-6 and (table[..., 1] - torch.sin(ang)).abs().max() < 1e-6


@pytest.mark.parametrize("heads,dv,pad", [(1, 9, 3), (5, 10, 0), (8, 64, 8), (6, 128, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_gate_a_head(heads, dv, pad, dtype):
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(heads * dv)
    T = 21
    o = torch.randn(T, heads * dv, generator=g).to(dtype)
    z = (3 * torch.randn(T, 7 + heads + pad, generator=g)).to(dtype)
    od = o.to(DEV)
    ops.head_gate(od, z.to(DEV)[:, 7:], heads, 1.2)
    ref = (o.double().view(T, heads, dv) * torch.sigmoid(z.double()[:, 7:7 + heads])[:, :, None] * 1.2).reshape(T, heads * dv)
    if dtype == torch.float32:
        assert_close(od, ref, "float32", "head gate")
    else:
        assert (od.double().cpu() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()


@pytest.mark.parametrize("heads,K,N", [(1, 16, 8), (3, 48, 96), (4, 64, 128), (8, 256, 512), (2, 80, 24)])
def test_per_block_product_on_the_tensor_cores_keeps_32_bit_accuracy(heads, K, N):
    """32-bit rows times bfloat16 matrices, the rows cut into three exact bfloat16 pieces: as accurate as 32-bit
    multiply-adds, for many tokens, few, and one; inputs of very different sizes in one row."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(heads * K + N)
    x = torch.randn(150, heads * K, generator=g) * torch.logspace(-3, 3, heads * K)
    w = (torch.randn(heads, K, N, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    for T in (150, 64, 17, 1):
        out = torch.empty(T, heads * N, dtype=torch.float32, device=DEV)
        ops.head_matmul_split(x[:T].to(DEV), w.to(DEV), out)
        xs = x.double()[:T].reshape(T, heads, K)
        ref = torch.einsum("thk,hkn->thn", xs, w.double()).reshape(T, heads * N)
        size = torch.einsum("thk,hkn->thn", xs.abs(), w.double().abs()).reshape(T, heads * N)      # what a 32-bit sum's error scales with
        assert ((out.double().cpu() - ref).abs() <= 4e-7 * size + 1e-30).all(), f"{T} tokens: {float(((out.double().cpu() - ref).abs() / size).max()):.3e}"


@pytest.mark.parametrize("width,blocks", [(24, 1), (60, 3), (256, 4), (35, 1), (1280, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_linear_recurrence_in_one_pass_in_chunks_and_in_portions(width, blocks, dtype):
    """The gates' block-diagonal products and the scan against the token-by-token recurrence in 64-bit: a whole sequence
    in one pass, in chunks side by side, and in portions through the state slot; two sequences; channels whose decay is
    so slow that the first token, made to stand out, still decides the last output."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts.base import Workspace
    g = torch.Generator().manual_seed(width + blocks)
    bw = width // blocks
    lens = [300, 45]
    u = [torch.randn(n, width, generator=g) for n in lens]
    u[0][0] *= 30.0                                                      # the first token's input stands out
    yraw = [torch.randn(n, width + 6, generator=g).to(dtype) for n in lens]
    bf = lambda t: t.to(torch.bfloat16).float()            # (the matrices are stored in bfloat16 on one of the two paths)
    w = {"ra": bf(2 * torch.randn(blocks, bw, bw, generator=g) / math.sqrt(bw)), "ri": bf(2 * torch.randn(blocks, bw, bw, generator=g) / math.sqrt(bw)),
         "ra.b": torch.randn(blocks, bw, generator=g), "ri.b": torch.randn(blocks, bw, generator=g), "lam": torch.linspace(-9.0, 1.0, width)}
    wd = {k: v.double() for k, v in w.items()}
    ref = []
    for uu, yy in zip(u, yraw):
        uu = uu.double()
        r = torch.sigmoid(plain.block_diagonal(uu, wd["ra"], wd["ra.b"]))
        i = torch.sigmoid(plain.block_diagonal(uu, wd["ri"], wd["ri.b"]))
        a = torch.exp(-plain.DECAY_RATE * r * plain.softplus(wd["lam"]))
        b = torch.sqrt(1.0 - a * a) * i * uu
        S, out = torch.zeros(width, dtype=torch.float64), []
        for t in range(uu.shape[0]):
            S = a[t] * S + b[t]
            out.append(S * plain.gelu_tanh(yy.double()[t, 3:3 + width]))
        ref.append(torch.stack(out))
    assert float(ref[0][-1, :4].abs().max()) > 1e-3 * float(ref[0].abs().max())        # the slowest channels still carry the first token
    gates_w = f32(torch.cat([w["ra"].transpose(1, 2), w["ri"].transpose(1, 2)], dim=2))
    ws = Workspace(torch.device(DEV))
    for mode, cuts in (("one pass", [[300], [45]]), ("chunks", [[300], [45]]), ("portions", [[1, 2, 130, 17, 150], [40, 5]])):
        state = torch.full((3, width), 5.0, dtype=torch.float32, device=DEV)
        state[0].zero_(); state[2].zero_()
        at = [0, 0]
        for k in range(max(len(c) for c in cuts)):
            parts = [(s, at[s], at[s] + cuts[s][k]) for s in (0, 1) if k < len(cuts[s])]
            step = FakeStep([b - a for _, a, b in parts], [a for _, a, _ in parts], [2 if s == 0 else 0 for s, _, _ in parts])
            x = torch.cat([u[s][a:b] for s, a, b in parts]).to(DEV)
            yy = torch.cat([yraw[s][a:b] for s, a, b in parts]).to(DEV)
            gates = torch.empty(x.shape[0], 2 * width, dtype=torch.float32, device=DEV)
            if dtype == torch.bfloat16 and ops.head_matmul_split_supported(bw, 2 * bw, width, 2 * width):
                ops.head_matmul_split(x, gates_w.to(torch.bfloat16), gates)
            else:
                ops.head_matmul(x, gates_w, gates)
            out = torch.empty(x.shape[0], width, dtype=dtype, device=DEV)
            chunk = {"one pass": 0, "chunks": 64, "portions": None}[mode]
            ops.lru_scan(gates, x, yy, 3, f32(w["ra.b"].reshape(-1)), f32(w["ri.b"].reshape(-1)), f32(w["lam"]), plain.DECAY_RATE, state, out,
                         step, bw, workspace=ws, chunk=chunk)
            want = torch.cat([ref[s][a:b] for s, a, b in parts])
            err = (out.double().cpu() - want).abs().max() / want.abs().max()
            assert err < (2e-5 if dtype == torch.float32 else 2.0 ** -7), f"{mode} step {k}: {float(err):.3e}"
            for s, a, b in parts:
                at[s] = b
        assert float(state[1].min()) == 5.0


@pytest.mark.parametrize("heads,d,dv,decay", [(3, 10, 6, (0.0, 0.8, 0.995)), (1, 4, 20, (1.0,)), (4, 64, 64, (0.5, 0.9, 0.99, 0.999)),
                                              (2, 128, 32, (0.97, 0.6)), (2, 200, 80, (0.999, 0.3))])
def test_linear_attention_with_a_constant_decay(heads, d, dv, decay):
    """silu of the projection's leading columns, the scan with stored decays and unit steps (one pass, chunks, portions
    through the slot), then the norm over all heads with its sigmoid gate and constant: against the plain statement.
    Decays of nothing, of one, and so slow that the first token, made to stand out, decides the last output."""
    from inferloop_b200.csrc import ops
    from inferloop_b200.parts.base import Workspace
    g = torch.Generator().manual_seed(heads * d + dv)
    inner, channels = heads * dv, heads * dv + 2 * heads * d
    lens = [300, 45]
    proj = [torch.randn(n, channels + inner + 4, generator=g) for n in lens]        # v | k | q | gate | unused
    proj[0][0, :inner] += 20.0
    norm_w = 1 + 0.2 * torch.randn(inner, generator=g)
    ref_y, ref_out = [], []
    for p in proj:
        n = p.shape[0]
        a = plain.silu(p.double()[:, :channels])
        v, k, q = a[:, :inner].view(n, heads, dv), a[:, inner:inner + heads * d].view(n, heads, d), a[:, inner + heads * d:].view(n, heads, d)
        out = torch.zeros(n, heads, dv, dtype=torch.float64)
        for h in range(heads):
            S = torch.zeros(d, dv, dtype=torch.float64)
            for t in range(n):
                S = decay[h] * S + torch.outer(k[t, h], v[t, h])
                out[t, h] = S.T @ q[t, h]
        ref_y.append(out.reshape(n, inner))
        ref_out.append(plain.rms(out.reshape(n, inner), 1e-5) * norm_w.double() * torch.sigmoid(p.double()[:, channels:channels + inner]) * 0.5)
    ws = Workspace(torch.device(DEV))
    decays = f32(torch.tensor(decay))
    for mode, cuts in (("one pass", [[300], [45]]), ("chunks", [[300], [45]]), ("portions", [[1, 2, 130, 17, 150], [40, 5]])):
        state = torch.full((3, heads, d, dv), 5.0, dtype=torch.float32, device=DEV)
        state[0].zero_(); state[2].zero_()
        at = [0, 0]
        for i in range(max(len(c) for c in cuts)):
            parts = [(s, at[s], at[s] + cuts[s][i]) for s in (0, 1) if i < len(cuts[s])]
            step = FakeStep([b - a for _, a, b in parts], [a for _, a, _ in parts], [2 if s == 0 else 0 for s, _, _ in parts])
            x = torch.cat([proj[s][a:b] for s, a, b in parts]).to(DEV)
            act = torch.empty(x.shape[0], channels, dtype=torch.float32, device=DEV)
            ops.silu_rows(x, channels, act)
            y = torch.empty(x.shape[0], inner, dtype=torch.float32, device=DEV)
            chunk = {"one pass": 0, "chunks": 64, "portions": None}[mode]
            ops.ssm_scan(act, None, 0, None, decays, None, state, y, step, heads, dv, d, heads, workspace=ws, chunk=chunk, fixed_decay=True)
            want = torch.cat([ref_y[s][a:b] for s, a, b in parts])
            err = (y.double().cpu() - want).abs().max() / want.abs().max()
            assert err < 2e-5, f"{mode} step {i}: {float(err):.3e}"
            out = torch.empty(x.shape[0], inner, dtype=torch.float32, device=DEV)
            ops.rms_gate(y, x[:, channels:], f32(norm_w), 1e-5, out, 0.5)
            want = torch.cat([ref_out[s][a:b] for s, a, b in parts])
            assert (out.double().cpu() - want).abs().max() < 3e-5 * want.abs().max(), f"{mode} step {i}: norm and gate"
            for s, a, b in parts:
                at[s] = b
        assert float(state[1].min()) == 5.0


@pytest.mark.parametrize("width,pad", [(18, 3), (64, 4), (1024, 8), (5000, 0), (4100, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_whole_rows_with_a_sigmoid_gate(width, pad, dtype):
    """Rows on 16-byte boundaries (four elements an access, a row read once up to 4,096 elements, longer rows read twice) and
    others; the gate's columns lie behind other columns of a wider matrix."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(width + pad)
    T = 11
    y = 3 * torch.randn(T, width, generator=g)
    z = (2 * torch.randn(T, 8 + width + pad, generator=g)).to(dtype)
    w = 1 + 0.2 * torch.randn(width, generator=g)
    out = torch.empty(T, width, dtype=dtype, device=DEV)
    ops.rms_gate(f32(y), z.to(DEV)[:, 8:], f32(w), 1e-5, out, 0.75)
    ref = plain.rms(y.double(), 1e-5) * w.double() * torch.sigmoid(z.double()[:, 8:8 + width]) * 0.75
    if dtype == torch.float32:
        assert_close(out, ref, "float32", "norm and gate")
    else:
        assert (out.double().cpu() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()


@pytest.mark.parametrize("width,extra", [(24, 8), (30, 3), (256, 64), (1000, 24)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_of_a_projections_leading_columns(width, extra, dtype):
    """Rows on 16-byte boundaries (eight elements an access) and others; the columns behind the leading ones are left alone."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    x = (3 * torch.randn(37, width + extra, generator=g)).to(dtype)
    out = torch.full((37, width), 7.0, dtype=torch.float32, device=DEV)
    ops.silu_rows(x.to(DEV), width, out)
    assert_close(out, plain.silu(x.double()[:, :width]), "float32", "silu of rows")


@pytest.mark.parametrize("taps,channels", [(1, 40), (2, 130), (4, 256), (5, 33)])
def test_short_convolution_without_activation(taps, channels):
    """The state-space layer's convolution with its activation switched off: whole and in portions through the slot."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(taps * 100 + channels)
    raw = torch.randn(61, channels + 7, generator=g)
    w, b = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    ref = plain.causal_conv(raw.double()[:, 3:3 + channels], w.double(), b.double())
    state = torch.zeros(2, max(taps - 1, 0), channels, dtype=torch.float32, device=DEV)
    at = 0
    for n in (1, 2, 17, 40, 1):
        step = FakeStep([n], [at], [1])
        out = torch.empty(n, channels, dtype=torch.float32, device=DEV)
        ops.ssm_conv(raw[at:at + n].to(DEV), 3, channels, f32(w), f32(b), state, step, out, activation="none")
        assert_close(out, ref[at:at + n], "float32", f"conv at {at}")
        at += n


@pytest.mark.parametrize("experts,top,groups,keep", [(6, 2, 3, 2), (10, 3, 2, 1), (8, 2, 4, 1), (1, 1, 1, 1), (12, 4, 1, 1), (64, 6, 8, 3), (40, 8, 4, 4)])
def test_routing_with_a_ranking_correction_and_groups(experts, top, groups, keep):
    """Softmax scores; the ranking adds a correction, the weights do not; a group ranks by its best member and only the
    best groups' experts can win, also when every ranking score is negative; weights divided by their sum and scaled."""
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(experts * 10 + top)
    T = 200
    logits = 3 * torch.randn(T, experts, generator=g)
    for shift in (0.0, -5.0):              # -5: every ranking score is negative (the scores are at most 1)
        corr = 0.2 * torch.randn(experts, generator=g) + shift
        choice = torch.empty(T * top, dtype=torch.int32, device=DEV)
        weight = torch.empty(T * top, dtype=torch.float32, device=DEV)
        ops.moe_route(f32(logits), experts, top, True, True, choice, weight, correction=f32(corr), groups=groups, keep=keep, scale=1.5,
                      renorm_eps=1e-20)
        scores = torch.softmax(logits.double(), dim=-1)
        want_e, want_w = plain.route(scores, corr.double(), top, {"count": groups, "keep": keep} if groups > 1 else None, 1.5)
        router = {"experts": experts, "top": top}
        if groups > 1:
            router["groups"] = {"count": groups, "keep": keep}
        decided = plain.routing_margin({"router": torch.eye(experts, dtype=torch.float64), "correction": corr.double()}, "",
                                       {"router": router}, logits.double()) > 1e-5
        assert decided.float().mean() > 0.9
        got_e = choice.view(T, top).cpu().long()
        assert torch.equal(got_e[decided], want_e[decided]), "the chosen experts differ where no call is close"
        assert (weight.view(T, top).cpu().double()[decided] - want_w[decided]).abs().max() < 1e-6
        if groups > 1:                     # the winners really come from `keep` groups
            per = experts // groups
            assert all(len({int(e) // per for e in row}) <= keep for row in got_e)


def test_routing_without_the_new_options_is_what_it_was():
    from inferloop_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(50, 10, generator=g)
    choice = torch.empty(50 * 3, dtype=torch.int32, device=DEV)
    weight = torch.empty(50 * 3, dtype=torch.float32, device=DEV)
    ops.moe_route(f32(logits), 10, 3, True, True, choice, weight)
    s = torch.softmax(logits.double(), -1)
    top = torch.sort(s, dim=-1, descending=True, stable=True)
    assert torch.equal(choice.view(50, 3).cpu().long(), top.indices[:, :3])
    want = top.values[:, :3] / top.values[:, :3].sum(-1, keepdim=True)
    assert (weight.view(50, 3).cpu().double() - want).abs().max() < 1e-6
