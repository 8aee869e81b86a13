"""Python face of the CUDA kernels: thin, checked ctypes calls on torch tensors.

Every function launches on torch's current stream of the tensors' device and returns
without synchronising.  There is no CPU path: a tensor that is not on a CUDA device, or
a library that cannot be built or loaded, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_module

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    """torch's current stream on the tensor's device, as the raw handle the launchers take."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(t.device.index))


def _need(t: Optional[torch.Tensor], what: str, dtype: Optional[torch.dtype] = None,
          contiguous: bool = True) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; inferloop_b200 kernels run on CUDA only")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, found {t.dtype}")


LAUNCHES = 0          # kernels launched through this module since import


_FUNCTIONS: dict = {}  # launcher name -> (function, its library)


SCOPE = "other"       # the op class the next launches belong to (see `scope`)
TIMER = None          # an engine.timing.DeviceTimer in "node" mode, or None


def scope(name: str) -> None:
    """Name the op class of the launches that follow (a part calls this before its kernels);
    it costs one assignment and only the per-kernel device timer reads it."""
    global SCOPE
    SCOPE = name


def _call(module: str, fn: str, *args) -> None:
    global LAUNCHES
    LAUNCHES += 1
    entry = _FUNCTIONS.get(fn)
    if entry is None:
        lib = load_module(module)
        f = getattr(lib, fn)
        f.restype = ctypes.c_int
        entry = _FUNCTIONS[fn] = (f, lib)
    timer = TIMER
    begin = timer.node_begin() if timer is not None else None
    rc = entry[0](*args)
    if rc != 0:
        raise KernelError(entry[1].ilb_last_error().decode())
    if begin is not None:
        timer.node_end(SCOPE, fn, begin)


def _i(v) -> ctypes.c_int:
    return ctypes.c_int(int(v))


def _f(v) -> ctypes.c_float:
    return ctypes.c_float(float(v))


# --------------------------------------------------------------------------- rows
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0, streams: int = 1) -> None:
    """out[t, s, :] = table[tokens[t], :] * scale, widened to 32-bit, for each of `streams`
    copies of the residual stream (out is [T, streams * H])."""
    _need(tokens, "embed tokens", torch.int32); _need(table, "embed table"); _need(out, "embed out", torch.float32)
    T, H = out.shape[0], table.shape[1]
    if tokens.numel() != T or out.shape[1] != H * streams:
        raise KernelError("embed: shapes do not agree")
    _call("elementwise", "ilb_embed", _ptr(tokens), _ptr(table), _i(_code(table)), _ptr(out),
          _i(T), _i(H), _i(table.shape[0]), _f(scale), _i(streams), _stream(out))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = x / sqrt(mean(x^2) + eps) * weight over the last dimension; x is 32-bit."""
    _need(x, "rmsnorm x", torch.float32); _need(weight, "rmsnorm weight", torch.float32); _need(out, "rmsnorm out")
    width = x.shape[-1]
    if weight.numel() != width or out.shape != x.shape:
        raise KernelError("rmsnorm: shapes do not agree")
    rows = x.numel() // width
    _call("elementwise", "ilb_rmsnorm", _ptr(x), _ptr(weight), _ptr(out), _i(_code(out)),
          _i(rows), _i(width), _f(eps), _stream(x))


GATE_ACTIVATIONS = {"silu": 0, "relu": 1}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out = act(gate_up[:, :I]) * gate_up[:, I:2I], act = silu (default) or relu."""
    _need(gate_up, "silu_mul in"); _need(out, "silu_mul out", gate_up.dtype)
    rows, width = out.shape
    if gate_up.shape[0] != rows or gate_up.shape[1] != 2 * width:
        raise KernelError("silu_mul: shapes do not agree")
    _call("elementwise", "ilb_silu_mul", _ptr(gate_up), _ptr(out), _i(_code(out)), _i(rows),
          _i(width), _i(gate_up.shape[1]), _i(GATE_ACTIVATIONS[activation]), _stream(out))


def glu_mul(gate_up: torch.Tensor, out: torch.Tensor, limit: float = 0.0, sharpness: float = 1.0, up_offset: float = 0.0) -> None:
    """out = g * sigmoid(sharpness * g) * (u + up_offset) with g = min(gate, limit), u = clamp(up, -limit, limit)
    (limit 0: no clamping); gate = gate_up[:, :I], up = gate_up[:, I:2I]."""
    _need(gate_up, "glu_mul in"); _need(out, "glu_mul out", gate_up.dtype)
    rows, width = out.shape
    if gate_up.shape[0] != rows or gate_up.shape[1] != 2 * width:
        raise KernelError("glu_mul: shapes do not agree")
    _call("elementwise", "ilb_glu_mul", _ptr(gate_up), _ptr(out), _i(_code(out)), _i(rows), _i(width), _i(gate_up.shape[1]),
          _f(limit), _f(sharpness), _f(up_offset), _stream(out))


def embed_pairs(step, table: torch.Tensor, pairs: Optional[torch.Tensor], buckets: int, mul_prev: int, mul_cur: int,
                prev_state: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                keep: Optional[torch.Tensor] = None) -> None:
    """out[t] = norm(table[token] + pairs[(previous token * mul_prev + token * mul_cur) mod buckets]) (the last row
    of `pairs` for a sequence's first token); the token before a step's first one comes from `prev_state`
    [slots] int32.  `keep`, if given, receives the same rows.  See elementwise.cu."""
    _need(table, "embed table"); _need(pairs, "pair table", table.dtype); _need(prev_state, "previous tokens", torch.int32)
    _need(norm_weight, "embed norm weight", torch.float32); _need(out, "embed out", torch.float32); _need(keep, "embed keep", torch.float32)
    T, H = out.shape
    if table.shape[1] != H or (pairs is not None and tuple(pairs.shape) != (buckets + 1, H)) or (keep is not None and keep.shape != out.shape):
        raise KernelError("embed_pairs: shapes do not agree")
    _call("elementwise", "ilb_embed_pairs", _ptr(step.tokens), _ptr(step.positions), _ptr(step.seq_of_token), _ptr(step.cu_q),
          _ptr(step.slots), _ptr(table), _ptr(pairs), _i(_code(table)), _i(buckets if pairs is not None else 0), _i(mul_prev), _i(mul_cur),
          _ptr(prev_state), _ptr(norm_weight), _f(eps), _ptr(out), _ptr(keep), _i(T), _i(H), _i(table.shape[0]), _stream(out))


def store_last_tokens(step, prev_state: torch.Tensor) -> None:
    """prev_state[slot] = the last token each sequence brings in this step."""
    _need(prev_state, "previous tokens", torch.int32)
    _call("elementwise", "ilb_store_last_tokens", _ptr(step.tokens), _ptr(step.cu_q), _ptr(step.slots), _ptr(prev_state),
          _i(step.n_seqs), _stream(prev_state))


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = [a[r], b[r]] of two 32-bit matrices, in out's dtype."""
    _need(a, "concat a", torch.float32); _need(b, "concat b", torch.float32); _need(out, "concat out")
    rows, width = a.shape
    if b.shape != a.shape or tuple(out.shape) != (rows, 2 * width):
        raise KernelError("concat_cast: shapes do not agree")
    _call("elementwise", "ilb_concat_cast", _ptr(a), _ptr(b), _ptr(out), _i(_code(out)), _i(rows), _i(width), _stream(out))


# --------------------------------------------------------------------------- state-space recurrence
SSM_CONV_TILE = 16         # tokens of a sequence per block of the convolution
SSM_CHUNK = 64             # tokens per chunk when a long portion's recurrence runs chunks side by side
SSM_CHUNK_FROM = 128       # portions from this many tokens on are cut into chunks


def ssm_conv(proj: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: torch.Tensor, state: torch.Tensor,
             step, out: torch.Tensor, activation: str = "silu") -> None:
    """out[t, c] = silu(bias[c] + sum_k weight[c, k] * raw[t - (taps - 1) + k, c]) over columns col0 .. of `proj`; the raw
    inputs ahead of the step come from state [slots, taps - 1, channels], which is brought up to date.  `activation`
    "none" leaves the sum as it is."""
    if activation not in ("silu", "none"):
        raise KernelError(f"ssm_conv: unknown activation {activation!r}")
    _need(proj, "ssm projection"); _need(weight, "conv weight", torch.float32); _need(bias, "conv bias", torch.float32)
    _need(state, "conv state", torch.float32); _need(out, "conv out", torch.float32)
    T, taps = proj.shape[0], weight.shape[1]
    if tuple(weight.shape) != (channels, taps) or bias.numel() != channels or tuple(out.shape) != (T, channels) \
            or tuple(state.shape[1:]) != (max(taps - 1, 0), channels):
        raise KernelError("ssm_conv: shapes do not agree")
    n_tiles = sum(-(-n // SSM_CONV_TILE) for n in step.h_q_len) + (step.n_seqs - len(step.h_q_len))
    _call("ssm", "ilb_ssm_conv", _ptr(proj), _i(_code(proj)), _i(proj.stride(0)), _i(col0), _i(channels), _i(taps), _ptr(weight),
          _ptr(bias), _ptr(state), _ptr(step.cu_q), _ptr(step.slots), _i(step.n_seqs), _i(n_tiles), _ptr(out),
          _i(1 if activation == "silu" else 0), _stream(out))


def ssm_scan(act: torch.Tensor, proj: Optional[torch.Tensor], dt_col0: int, dt_bias: Optional[torch.Tensor], a_log: torch.Tensor,
             skip: Optional[torch.Tensor], state: torch.Tensor, y: torch.Tensor, step, heads: int, head_dim: int, n_state: int,
             groups: int, workspace=None, chunk: Optional[int] = None, fixed_decay: bool = False) -> None:
    """The recurrence S_t = exp(-exp(a_log) d_t) S_{t-1} + d_t B_t u_t^T, y_t = S_t^T C_t + skip * u_t per head over the
    step's tokens, from and to state [slots, heads, n_state, head_dim] (see ssm.cu).  `chunk`: None picks by the
    longest portion; 0 runs every sequence in one go; n cuts portions into chunks of n tokens.  `fixed_decay`: every
    step size is one and `a_log` holds each head's decay itself (S_t = decay S_{t-1} + B_t u_t^T, y_t = S_t^T C_t);
    `proj`, `dt_bias` and `skip` are None then."""
    _need(act, "ssm activations", torch.float32); _need(proj, "ssm projection"); _need(state, "ssm state", torch.float32)
    _need(y, "ssm y", torch.float32)
    if fixed_decay != (proj is None) or fixed_decay != (dt_bias is None) or fixed_decay != (skip is None):
        raise KernelError("ssm_scan: a fixed decay takes no step sizes, and step sizes no fixed decay")
    for t, w in ((dt_bias, "dt bias"), (a_log, "decay logarithms"), (skip, "skip weights")):
        _need(t, "ssm " + w, torch.float32)
        if t is not None and t.numel() != heads:
            raise KernelError("ssm_scan: one " + w + " per head")
    T, channels = act.shape
    if channels != heads * head_dim + 2 * groups * n_state or tuple(y.shape) != (T, heads * head_dim) \
            or tuple(state.shape[1:]) != (heads, n_state, head_dim):
        raise KernelError("ssm_scan: shapes do not agree")
    if chunk is None:
        chunk = 0
        if step.max_q_len >= SSM_CHUNK_FROM:
            # chunks of 64, 128 or 256 tokens: the launch runs in rounds of about four blocks an SM, a round takes as
            # long as a chunk, and of equal products the longer chunk wins (fewer states to carry)
            room = 4 * _sm_count(act.device)
            tiles = heads * -(-head_dim // 64)
            cost = lambda c: -(-(sum(-(-n // c) for n in step.h_q_len) * tiles) // room) * c
            chunk = min((SSM_CHUNK, 2 * SSM_CHUNK, 4 * SSM_CHUNK), key=lambda c: (cost(c), -c))
    chunk_state = chunk_decay = None
    n_blocks = step.n_seqs
    if chunk:
        if workspace is None:
            raise KernelError("ssm_scan: chunks need a workspace")
        n_blocks = sum(-(-n // chunk) for n in step.h_q_len) + (step.n_seqs - len(step.h_q_len))
        chunk_state = workspace.buffer("ssm.chunk_state", (n_blocks, heads, n_state, head_dim), torch.float32)
        chunk_decay = workspace.buffer("ssm.chunk_decay", (n_blocks, heads), torch.float32)
    _call("ssm", "ilb_ssm_scan", _ptr(act), _ptr(proj), _i(F32 if proj is None else _code(proj)), _i(0 if proj is None else proj.stride(0)),
          _i(dt_col0), _i(channels), _ptr(dt_bias),
          _ptr(a_log), _ptr(skip), _ptr(state), _ptr(chunk_state), _ptr(chunk_decay), _ptr(y), _ptr(step.cu_q), _ptr(step.slots),
          _i(step.n_seqs), _i(heads), _i(head_dim), _i(n_state), _i(groups), _i(chunk), _i(n_blocks), _i(1 if fixed_decay else 0), _stream(y))


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out: torch.Tensor) -> None:
    """out = rms over each of `groups` equal parts of (y * silu(gate[:, :width])) * weight; y is 32-bit."""
    _need(y, "gated norm y", torch.float32); _need(gate, "gated norm gate", contiguous=False); _need(weight, "gated norm weight", torch.float32)
    _need(out, "gated norm out", gate.dtype)
    T, width = y.shape
    if gate.shape[0] != T or gate.shape[1] < width or gate.stride(1) != 1 or weight.numel() != width or out.shape != y.shape or width % groups:
        raise KernelError("gated_group_norm: shapes do not agree")
    _call("ssm", "ilb_gated_group_norm", _ptr(y), _ptr(gate), _i(_code(gate)), _i(gate.stride(0)), _ptr(weight), _ptr(out), _i(T), _i(width),
          _i(groups), _f(eps), _stream(out))


# --------------------------------------------------------------------------- attention over a cached latent
def latent_write(proj: torch.Tensor, col0: int, rank: int, weight: torch.Tensor, eps: float, step, block_table: torch.Tensor,
                 cache: torch.Tensor) -> None:
    """cache[page of t, place of t] = rms(proj[t, col0 : col0 + rank]) * weight; cache is [pages, 1, page_size, rank]."""
    _need(proj, "latent projection"); _need(weight, "latent norm weight", torch.float32); _need(cache, "latent cache")
    _need(block_table, "block table", torch.int32)
    if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != rank or weight.numel() != rank:
        raise KernelError("latent_write: cache must be [pages, 1, page_size, rank]")
    if proj.shape[0] != step.n_tokens:
        raise KernelError(f"latent_write: {proj.shape[0]} rows for a step of {step.n_tokens} tokens")
    _call("latent", "ilb_latent_write", _ptr(proj), _i(_code(proj)), _i(proj.stride(0)), _i(col0), _i(rank), _ptr(weight), _f(eps),
          _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table), _i(block_table.shape[1]), _i(cache.shape[2]),
          _i(cache.shape[0]), _ptr(cache), _i(_code(cache)), _i(proj.shape[0]), _stream(cache))


LATENT_INPUT_TOKENS = 16      # steps of up to this many tokens run the latent write and the queries' map as one launch


def latent_input(proj: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, col0: int, rank: int, weight: torch.Tensor, eps: float,
                 step, block_table: torch.Tensor, cache: torch.Tensor) -> None:
    """`latent_write` and `head_matmul(proj, w, q_out)` of a step of few tokens in one launch (see latent.cu)."""
    _need(proj, "latent projection"); _need(w, "head_matmul w", proj.dtype); _need(q_out, "mapped queries", proj.dtype)
    _need(weight, "latent norm weight", torch.float32); _need(cache, "latent cache", proj.dtype); _need(block_table, "block table", torch.int32)
    heads, K, N = w.shape
    if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != rank or weight.numel() != rank:
        raise KernelError("latent_input: cache must be [pages, 1, page_size, rank]")
    if proj.shape[0] != step.n_tokens or proj.shape[1] < max(heads * K, col0 + rank) or tuple(q_out.shape) != (proj.shape[0], heads * N):
        raise KernelError("latent_input: shapes do not agree")
    _call("latent", "ilb_latent_input", _ptr(proj), _i(_code(proj)), _i(proj.stride(0)), _ptr(w), _ptr(q_out), _i(_code(q_out)),
          _i(q_out.stride(0)), _i(proj.shape[0]), _i(heads), _i(K), _i(N), _i(col0), _i(rank), _ptr(weight), _f(eps), _ptr(step.positions),
          _ptr(step.seq_of_token), _ptr(block_table), _i(block_table.shape[1]), _i(cache.shape[2]), _i(cache.shape[0]), _ptr(cache),
          _i(_code(cache)), _stream(cache))


def head_matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_head_stride: Optional[int] = None,
                out_head_stride: Optional[int] = None) -> None:
    """out[t, i, :N] = x[t, i, :K] @ w[i] for every head i; w [heads, K, N]; head i of x starts at column
    i * x_head_stride (default K), head i of out at i * out_head_stride (default N); row strides are free."""
    _need(x, "head_matmul x", contiguous=False); _need(w, "head_matmul w", x.dtype); _need(out, "head_matmul out", contiguous=False)
    heads, K, N = w.shape
    xhs = K if x_head_stride is None else int(x_head_stride)
    ohs = N if out_head_stride is None else int(out_head_stride)
    if (x.stride(1) != 1 or out.stride(1) != 1 or xhs < K or ohs < N or x.shape[1] < (heads - 1) * xhs + K
            or out.shape[0] != x.shape[0] or out.shape[1] < (heads - 1) * ohs + N):
        raise KernelError("head_matmul: shapes do not agree")
    _call("latent", "ilb_head_matmul", _ptr(x), _i(_code(x)), _i(x.stride(0)), _ptr(w), _ptr(out), _i(_code(out)), _i(out.stride(0)),
          _i(x.shape[0]), _i(heads), _i(K), _i(N), _i(xhs), _i(ohs), _stream(out))


def head_matmul_split_supported(K: int, N: int, ldx: int, ldo: int) -> bool:
    """Sizes that :func:`head_matmul_split` takes."""
    return K % 16 == 0 and N % 8 == 0 and ldx % 2 == 0 and ldo % 2 == 0


def head_matmul_split(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i, :N] = x[t, i, :K] @ w[i] for 32-bit x and out and a bfloat16 w [heads, K, N], on the tensor cores with
    32-bit accuracy: x is cut into three bfloat16 pieces whose products with w are exact and are added in 32-bit."""
    _need(x, "head_matmul_split x", torch.float32); _need(w, "head_matmul_split w", torch.bfloat16); _need(out, "head_matmul_split out", torch.float32)
    heads, K, N = w.shape
    if x.shape[1] != heads * K or tuple(out.shape) != (x.shape[0], heads * N) or not head_matmul_split_supported(K, N, x.stride(0), out.stride(0)):
        raise KernelError("head_matmul_split: shapes do not agree or are not served")
    _call("latent", "ilb_head_matmul_split", _ptr(x), _i(x.stride(0)), _ptr(w), _ptr(out), _i(out.stride(0)), _i(x.shape[0]), _i(heads), _i(K),
          _i(N), _i(K), _i(N), _stream(out))


def latent_write_rot(proj: torch.Tensor, col0: int, rank: int, tail: int, rot: int, angles: Optional[torch.Tensor],
                     weight: Optional[torch.Tensor], eps: float, step, block_table: Optional[torch.Tensor],
                     cache: Optional[torch.Tensor], q_src: Optional[torch.Tensor] = None, q_dst: Optional[torch.Tensor] = None,
                     q_col0: int = 0, q_head_stride: int = 0, heads: int = 0) -> None:
    """A latent with a rotated part behind it: cache row of token t = [rms(proj[t, col0 : col0 + rank]) * weight |
    turn(proj[t, col0 + rank : + tail])], the first `rot` elements of the part turned in neighbouring pairs by
    `angles` [T, rot / 2, 2] (cos, sin); cache is [pages, 1, page_size, rank + tail] (None: nothing stored).  With
    `q_src` [T, >= q_col0 + heads * q_head_stride]: head i's `tail` columns from q_col0 + i * q_head_stride are
    turned the same way into q_dst[t, i, rank:], q_dst [T, heads * (rank + tail)]."""
    _need(proj, "latent projection", contiguous=False); _need(weight, "latent norm weight", torch.float32); _need(cache, "latent cache")
    _need(block_table, "block table", torch.int32); _need(angles, "rotation table", torch.float32)
    _need(q_src, "queries", contiguous=False); _need(q_dst, "mapped queries", None if q_src is None else q_src.dtype)
    T = step.n_tokens
    if cache is not None and (cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != rank + tail or weight is None
                              or weight.numel() != rank or block_table is None):
        raise KernelError("latent_write_rot: cache must be [pages, 1, page_size, rank + tail]")
    if proj.shape[0] != T or (angles is not None and tuple(angles.shape) != (T, rot // 2, 2)):
        raise KernelError("latent_write_rot: rows do not match the step")
    if q_src is not None and (q_dst is None or q_src.shape[0] != T or tuple(q_dst.shape) != (T, heads * (rank + tail))):
        raise KernelError("latent_write_rot: the queries do not match the step")
    ref = cache if cache is not None else q_dst
    _call("latent", "ilb_latent_write_rot", _ptr(proj), _i(_code(proj)), _i(proj.stride(0)), _i(col0), _i(rank), _i(tail), _i(rot),
          _ptr(angles), _ptr(weight), _f(eps), _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table),
          _i(0 if block_table is None else block_table.shape[1]), _i(0 if cache is None else cache.shape[2]),
          _i(0 if cache is None else cache.shape[0]), _ptr(cache), _i(_code(ref)), _ptr(q_src), _ptr(q_dst),
          _i(_code(ref if q_src is None else q_src)), _i(0 if q_src is None else q_src.stride(0)), _i(q_col0), _i(q_head_stride),
          _i(heads), _i(T), _stream(ref))


# --------------------------------------------------------------------------- norm on a sublayer's output
def cast_zero(x: torch.Tensor, xc: torch.Tensor, y: torch.Tensor) -> None:
    """xc = x in xc's dtype; y = 0 (x and y 32-bit, all of one shape)."""
    _need(x, "cast_zero x", torch.float32); _need(xc, "cast_zero out"); _need(y, "cast_zero y", torch.float32)
    if xc.shape != x.shape or y.shape != x.shape:
        raise KernelError("cast_zero: shapes do not agree")
    _call("sublayer_norm", "ilb_cast_zero", _ptr(x), _ptr(xc), _i(_code(xc)), _ptr(y), ctypes.c_longlong(x.numel()), _stream(x))


def group_norm_add(y: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, x: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, zero: bool = False) -> None:
    """n = y cut into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times weight.
    With `x`: x += n and out (if given) = the new x; without: out = n.  `zero` leaves y at zero.  y [rows, width]
    32-bit with a free row stride."""
    _need(y, "group_norm y", torch.float32, contiguous=False); _need(weight, "group_norm weight", torch.float32)
    _need(x, "group_norm x", torch.float32); _need(out, "group_norm out")
    rows, width = y.shape
    if y.stride(1) != 1 or weight.numel() != width or (x is not None and x.shape != y.shape) or (out is not None and out.shape != y.shape):
        raise KernelError("group_norm_add: shapes do not agree")
    _call("sublayer_norm", "ilb_group_norm_add", _ptr(y), _i(y.stride(0)), _ptr(weight), _f(eps), _i(groups), _i(rows), _i(width),
          _ptr(x), _ptr(out), _i(F32 if out is None else _code(out)), _i(1 if zero else 0), _stream(y))


def dyt(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(alpha * x) * weight + bias, element by element (alpha one stored number); x 32-bit, out of any dtype
    and possibly x itself."""
    _need(x, "dyt x", torch.float32); _need(alpha, "dyt alpha", torch.float32); _need(weight, "dyt weight", torch.float32)
    _need(bias, "dyt bias", torch.float32); _need(out, "dyt out")
    width = x.shape[-1]
    if alpha.numel() != 1 or weight.numel() != width or bias.numel() != width or out.shape != x.shape:
        raise KernelError("dyt: shapes do not agree")
    _call("sublayer_norm", "ilb_dyt", _ptr(x), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out), _i(_code(out)), _i(x.numel() // width),
          _i(width), _stream(x))


def dyt_add(y: torch.Tensor, norm, mult: float, x: torch.Tensor, next_norm=None, out: Optional[torch.Tensor] = None,
            zero: bool = False) -> None:
    """x += mult * (tanh(a y) g + b) with (a, g, b) = `norm`; then, with `next_norm` and `out`, out = tanh(a2 x) g2 + b2 in
    out's dtype; `zero` leaves y at zero.  y and x are 32-bit and of one shape."""
    _need(y, "dyt_add y", torch.float32); _need(x, "dyt_add x", torch.float32); _need(out, "dyt_add out")
    width = x.shape[-1]
    if y.shape != x.shape or (out is not None and out.shape != x.shape) or (out is None) != (next_norm is None):
        raise KernelError("dyt_add: shapes do not agree")
    for n in (norm, next_norm):
        if n is not None:
            a, g, b = n
            _need(a, "dyt alpha", torch.float32); _need(g, "dyt weight", torch.float32); _need(b, "dyt bias", torch.float32)
            if a.numel() != 1 or g.numel() != width or b.numel() != width:
                raise KernelError("dyt_add: a norm's tensors do not fit the row")
    a2, g2, b2 = next_norm if next_norm is not None else (None, None, None)
    _call("sublayer_norm", "ilb_dyt_add", _ptr(y), _ptr(norm[0]), _ptr(norm[1]), _ptr(norm[2]), _f(mult), _ptr(x), _ptr(a2), _ptr(g2),
          _ptr(b2), _ptr(out), _i(F32 if out is None else _code(out)), _i(1 if zero else 0), _i(x.numel() // width), _i(width), _stream(x))


# --------------------------------------------------------------------------- linear recurrences over channels, gates
LRU_CHUNK = 16             # tokens per chunk when a long portion's recurrence runs chunks side by side
LRU_CHUNK_FROM = 128       # portions from this many tokens on are cut into chunks


def lru_scan(gates: torch.Tensor, u: torch.Tensor, proj: torch.Tensor, y_col0: int, r_bias: torch.Tensor, i_bias: torch.Tensor,
             lam: torch.Tensor, rate: float, state: torch.Tensor, out: torch.Tensor, step, block_width: int, workspace=None,
             chunk: Optional[int] = None) -> None:
    """The gated linear recurrence over channels (see recurrent.cu): gates [T, 2 W] 32-bit (per block of `block_width`
    channels its r logits, then its i logits), u [T, W] 32-bit, the raw output branch at columns y_col0 .. of `proj`;
    from and to state [slots, W]; out [T, W] = S * gelu_tanh(y) in proj's dtype.  `chunk`: None picks by the longest
    portion; 0 runs every sequence in one go; n cuts portions into chunks of n tokens."""
    _need(gates, "lru gates", torch.float32, contiguous=False); _need(u, "lru input", torch.float32); _need(proj, "lru projection", contiguous=False)
    _need(state, "lru state", torch.float32); _need(out, "lru out", proj.dtype)
    T, W = u.shape
    for t, w in ((r_bias, "r bias"), (i_bias, "i bias"), (lam, "decay parameter")):
        _need(t, "lru " + w, torch.float32)
        if t.numel() != W:
            raise KernelError("lru_scan: one " + w + " per channel")
    if gates.shape[0] != T or gates.shape[1] < 2 * W or gates.stride(1) != 1 or proj.shape[0] != T or proj.stride(1) != 1 \
            or tuple(out.shape) != (T, W) or tuple(state.shape[1:]) != (W,) or W % block_width:
        raise KernelError("lru_scan: shapes do not agree")
    if chunk is None:
        chunk = LRU_CHUNK if step.max_q_len >= LRU_CHUNK_FROM else 0
    chunk_state = chunk_decay = None
    n_blocks = step.n_seqs
    if chunk:
        if workspace is None:
            raise KernelError("lru_scan: chunks need a workspace")
        n_blocks = sum(-(-n // chunk) for n in step.h_q_len) + (step.n_seqs - len(step.h_q_len))
        chunk_state = workspace.buffer("lru.chunk_state", (n_blocks, W), torch.float32)
        chunk_decay = workspace.buffer("lru.chunk_decay", (n_blocks, W), torch.float32)
    _call("recurrent", "ilb_lru_scan", _ptr(gates), _i(gates.stride(0)), _ptr(u), _ptr(proj), _i(_code(proj)), _i(proj.stride(0)), _i(y_col0),
          _ptr(r_bias), _ptr(i_bias), _ptr(lam), _f(rate), _ptr(state), _ptr(chunk_state), _ptr(chunk_decay), _ptr(out), _ptr(step.cu_q),
          _ptr(step.slots), _i(step.n_seqs), _i(W), _i(block_width), _i(chunk), _i(n_blocks), _stream(out))


def silu_rows(x: torch.Tensor, width: int, out: torch.Tensor) -> None:
    """out[t, :width] = silu(x[t, :width]) in 32-bit; x may have more columns."""
    _need(x, "silu_rows x", contiguous=False); _need(out, "silu_rows out", torch.float32)
    if x.stride(1) != 1 or x.shape[1] < width or tuple(out.shape) != (x.shape[0], width):
        raise KernelError("silu_rows: shapes do not agree")
    _call("recurrent", "ilb_silu_rows", _ptr(x), _i(_code(x)), _i(x.stride(0)), _ptr(out), _i(x.shape[0]), _i(width), _stream(out))


def rms_gate(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, scale: float = 1.0) -> None:
    """out = y / sqrt(mean(y^2) + eps) * weight * sigmoid(gate) * scale over whole rows; y 32-bit, gate [T, >= width]
    (its first `width` columns) and out [T, width] (rows of any stride) in the compute dtype."""
    _need(y, "rms_gate y", torch.float32); _need(gate, "rms_gate gate", contiguous=False); _need(weight, "rms_gate weight", torch.float32)
    _need(out, "rms_gate out", gate.dtype, contiguous=False)
    T, width = y.shape
    if gate.shape[0] != T or gate.shape[1] < width or gate.stride(1) != 1 or weight.numel() != width or out.shape != y.shape \
            or out.stride(1) != 1:
        raise KernelError("rms_gate: shapes do not agree")
    _call("recurrent", "ilb_rms_gate", _ptr(y), _ptr(gate), _i(_code(gate)), _i(gate.stride(0)), _ptr(weight), _ptr(out), _i(out.stride(0)),
          _i(T), _i(width), _f(eps), _f(scale), _stream(out))


def head_gate(o: torch.Tensor, gate: torch.Tensor, heads: int, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :] = o[t, h, :] * sigmoid(gate[t, h]) * scale; o [T, heads * dv], gate [T, >= heads] (its first `heads`
    columns), out [T, heads * dv] with rows of any stride (default: o itself, in place), all in the compute dtype."""
    _need(o, "head_gate o"); _need(gate, "head_gate gate", o.dtype, contiguous=False); _need(out, "head_gate out", o.dtype, contiguous=False)
    T, width = o.shape
    dst = o if out is None else out
    if width % heads or gate.shape[0] != T or gate.shape[1] < heads or gate.stride(1) != 1 or dst.shape != o.shape or dst.stride(1) != 1:
        raise KernelError("head_gate: shapes do not agree")
    _call("recurrent", "ilb_head_gate", _ptr(o), _ptr(dst), _i(dst.stride(0)), _ptr(gate), _i(_code(o)), _i(gate.stride(0)), _i(T), _i(heads),
          _i(width // heads), _f(scale), _stream(o))


def gated_rows(a: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, k] = gelu_tanh(a[t, k]) * table[tokens[t], col0 + k]."""
    _need(a, "gated_rows a"); _need(table, "gated_rows table", a.dtype); _need(out, "gated_rows out", a.dtype)
    _need(tokens, "gated_rows tokens", torch.int32)
    rows, width = a.shape
    if out.shape != a.shape or tokens.numel() != rows or table.shape[1] < col0 + width:
        raise KernelError("gated_rows: shapes do not agree")
    _call("sublayer_norm", "ilb_gated_rows", _ptr(a), _ptr(table), _i(_code(a)), _i(table.stride(0)), _i(col0), _ptr(tokens),
          _i(table.shape[0]), _ptr(out), _i(rows), _i(width), _stream(out))


def gather_rows(x: torch.Tensor, index: torch.Tensor, out: torch.Tensor, streams: int = 1) -> None:
    """out[r, :] = the sum of the `streams` copies of row index[r] of x [rows, streams * width]."""
    _need(x, "gather x", torch.float32); _need(index, "gather index", torch.int32); _need(out, "gather out", torch.float32)
    if out.shape[0] != index.numel() or out.shape[1] * streams != x.shape[1]:
        raise KernelError("gather_rows: shapes do not agree")
    _call("elementwise", "ilb_gather_rows", _ptr(x), _ptr(index), _ptr(out), _i(out.shape[0]),
          _i(out.shape[1]), _i(x.shape[0]), _i(streams), _stream(x))


# --------------------------------------------------------------------------- several residual streams
def streams_read(x: torch.Tensor, coef: torch.Tensor, streams: int, norm_weight: Optional[torch.Tensor] = None,
                 eps: float = 0.0, normed: Optional[torch.Tensor] = None, u_out: Optional[torch.Tensor] = None,
                 y_zero: Optional[torch.Tensor] = None) -> None:
    """u = sum_s coef[s] x[:, s, :] of x [T, streams * H] (32-bit); `normed` = RMS norm of u with
    `norm_weight` (any compute dtype), `u_out` = u, `y_zero` is set to zero (see hyper.cu)."""
    _need(x, "streams x", torch.float32); _need(coef, "streams coefficients", torch.float32)
    _need(norm_weight, "streams norm weight", torch.float32); _need(normed, "streams normed")
    _need(u_out, "streams u", torch.float32); _need(y_zero, "streams y", torch.float32)
    T, H = x.shape[0], x.shape[1] // streams
    if x.shape[1] != H * streams or coef.numel() != streams or (norm_weight is not None and norm_weight.numel() != H):
        raise KernelError("streams_read: shapes do not agree")
    for t in (normed, u_out, y_zero):
        if t is not None and tuple(t.shape) != (T, H):
            raise KernelError("streams_read: outputs must be [tokens, width]")
    _call("hyper", "ilb_streams_read", _ptr(x), _ptr(coef), _ptr(norm_weight), _ptr(normed),
          _i(_code(normed) if normed is not None else F32), _ptr(u_out), _ptr(y_zero), _i(T), _i(H), _i(streams), _f(eps),
          _stream(x))


def streams_write(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, out_coef: torch.Tensor, streams: int) -> None:
    """In place on x [T, streams * H]: x[:, t, :] = sum_s mix[s, t] x[:, s, :] + out_coef[t] * y."""
    _need(x, "streams x", torch.float32); _need(y, "streams y", torch.float32)
    _need(mix, "streams mix", torch.float32); _need(out_coef, "streams out", torch.float32)
    T, H = y.shape
    if tuple(x.shape) != (T, H * streams) or mix.numel() != streams * streams or out_coef.numel() != streams:
        raise KernelError("streams_write: shapes do not agree")
    _call("hyper", "ilb_streams_write", _ptr(x), _ptr(y), _ptr(mix), _ptr(out_coef), _i(T), _i(H), _i(streams), _stream(x))


# --------------------------------------------------------------------------- routed feed-forward
def moe_limits() -> tuple:
    """(most experts, most experts per token) the routing kernels take."""
    lib = load_module("moe")
    return int(lib.ilb_moe_max_experts()), int(lib.ilb_moe_max_top())


def moe_plan_rows(n_pairs: int, experts: int, block_rows: int) -> int:
    """Rows that `n_pairs` (token, expert) pairs need once every expert's rows start at a
    multiple of `block_rows` (the worst case over all routings)."""
    most = min(n_pairs, experts)
    rows = n_pairs + most * (block_rows - 1)
    return -(-rows // block_rows) * block_rows


def moe_logits(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, e] = x[t] . w[e] in 32-bit for the few rows of a router's matrix (same dtype as x)."""
    _need(x, "router x"); _need(w, "router matrix", x.dtype); _need(out, "router logits", torch.float32)
    if w.shape[1] != x.shape[1] or tuple(out.shape) != (x.shape[0], w.shape[0]):
        raise KernelError("moe_logits: shapes do not agree")
    _call("moe", "ilb_moe_logits", _ptr(x), _ptr(w), _i(_code(x)), _ptr(out), _i(x.shape[0]), _i(w.shape[0]), _i(x.shape[1]), _stream(x))


def moe_route(logits: torch.Tensor, experts: int, top: int, softmax: bool, renormalize: bool,
              choice: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
              correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1, scale: float = 1.0,
              renorm_eps: float = 0.0) -> None:
    """The `top` experts with the largest scores of every token and their weights; `bias` [experts]
    is added to the logits first.  `correction` [experts] is added to the scores for the ranking alone (the
    weights stay the scores); with `groups` > 1 the experts form that many equal groups of neighbours, a group
    ranks by its best member, and only the best `keep` groups' experts can be chosen.  The weights are divided by
    their sum + `renorm_eps` when `renormalize`, then multiplied by `scale`."""
    _need(logits, "router logits", torch.float32); _need(choice, "moe choice", torch.int32); _need(weight, "moe weight", torch.float32)
    _need(bias, "router bias", torch.float32); _need(correction, "router correction", torch.float32)
    T = logits.shape[0]
    if choice.numel() != T * top or weight.numel() != T * top or logits.shape[1] < experts or (bias is not None and bias.numel() != experts) \
            or (correction is not None and correction.numel() != experts):
        raise KernelError("moe_route: shapes do not agree")
    _call("moe", "ilb_moe_route", _ptr(logits), _ptr(bias), _i(logits.stride(0)), _i(T), _i(experts), _i(top), _i(1 if softmax else 0),
          _i(1 if renormalize else 0), _ptr(choice), _ptr(weight), _ptr(correction), _i(groups), _i(keep), _f(scale), _f(renorm_eps),
          _stream(logits))


def moe_plan(choice: torch.Tensor, experts: int, block_rows: int, pos: torch.Tensor, block_expert: torch.Tensor) -> None:
    """pos[pair] = the pair's row once the pairs are sorted by expert with every expert's rows
    starting at a multiple of `block_rows`; block_expert[b] = the expert of rows b * block_rows
    ..., or -1."""
    for t, w in ((choice, "choice"), (pos, "pos"), (block_expert, "block_expert")):
        _need(t, "moe " + w, torch.int32)
    rows = block_expert.numel() * block_rows
    if pos.numel() != choice.numel():
        raise KernelError("moe_plan: shapes do not agree")
    _call("moe", "ilb_moe_plan", _ptr(choice), _i(choice.numel()), _i(experts), _i(block_rows), _i(rows), _ptr(pos),
          _ptr(block_expert), _stream(choice))


def moe_gather(x: torch.Tensor, weight: Optional[torch.Tensor], pos: torch.Tensor, top: int, out: torch.Tensor) -> None:
    """out[pos[p]] = (weight[p] *) x[p // top] for every pair p; other rows of `out` are left alone."""
    _need(x, "moe x"); _need(out, "moe rows", x.dtype); _need(weight, "moe weight", torch.float32); _need(pos, "moe pos", torch.int32)
    if pos.numel() != x.shape[0] * top or out.shape[1] != x.shape[1]:
        raise KernelError("moe_gather: shapes do not agree")
    _call("moe", "ilb_moe_gather", _ptr(x), _i(_code(x)), _ptr(weight), _ptr(pos), _i(pos.numel()), _i(top), _i(x.shape[1]),
          _ptr(out), _stream(x))


def moe_combine(routed: torch.Tensor, pos: torch.Tensor, weight: Optional[torch.Tensor], top: int,
                shared: Optional[torch.Tensor], gate_logit: Optional[torch.Tensor], y: torch.Tensor) -> None:
    """y[t] += sum_j (weight[t, j] *) routed[pos[t, j]] (+ sigmoid(gate_logit[t]) * shared[t]); `gate_logit`
    is a [T] column (any row stride) of a 32-bit matrix."""
    _need(routed, "moe routed", torch.float32); _need(pos, "moe pos", torch.int32); _need(weight, "moe weight", torch.float32)
    _need(shared, "moe shared", torch.float32); _need(y, "moe y", torch.float32)
    T, H = y.shape
    if routed.shape[1] != H or pos.numel() != T * top or (shared is not None and tuple(shared.shape) != (T, H)):
        raise KernelError("moe_combine: shapes do not agree")
    gate_ld = 0
    if gate_logit is not None:
        _need(gate_logit, "moe gate", torch.float32, contiguous=False)
        if gate_logit.dim() != 1 or gate_logit.numel() != T:
            raise KernelError("moe_combine: the gate must be one logit per token")
        gate_ld = gate_logit.stride(0)
    _call("moe", "ilb_moe_combine", _ptr(routed), _ptr(pos), _ptr(weight), _i(top), _ptr(shared), _ptr(gate_logit), _i(gate_ld),
          _i(T), _i(H), _ptr(y), _stream(y))


GROUP_ROWS_SIMT = 16       # rows of a block of the grouped exact product (ilb_gemm_simt_group_rows)
GROUP_ROWS_TC = 128        # rows of a block of the grouped tensor-core product: 128 x 128 tiles, two CTAs to an SM
GROUP_ROWS_TC_WIDE = 256   # or 256 x 256 tiles, when experts have hundreds of rows


def moe_gemm_tc_eligible(a: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """bfloat16 operands whose rows are multiples of 16 bytes (TMA's rule); gate and up rows in
    blocks of 64 for the SwiGLU epilogue."""
    return (TC_ENABLED and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (not swiglu or w.shape[1] % 128 == 0))


MOE_WIDE_BLOCKS = False    # blocks of 256 rows (256 x 256 tiles) once an expert gets a thousand rows on average: measured slower than the persistent 128 x 256 form
MOE_TILE_N = 0             # tests and measurements force 128, 256 or 257 (256 with persistent CTAs) weight rows per tile of 128 rows; 0: the default choice


def moe_gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, block_group: torch.Tensor, swiglu: bool = False,
                block_rows: int = GROUP_ROWS_TC, tile_n: int = 0, act: tuple = (0.0, 1.0, 0.0)) -> None:
    """out[rows of block b] = a[rows of block b] @ w[block_group[b]].T on tcgen05 tensor cores for
    blocks of 128 or 256 rows (moe_gemm_tcgen05.cu); with `swiglu`, w holds blocks of 64 gate rows
    followed by their 64 up rows and out is [rows, N / 2] = silu(gate) * up; or, with `act` = (limit, sharpness, up_offset), the gated
    unit of `glu_mul`."""
    _need(a, "moe gemm a", torch.bfloat16); _need(w, "moe gemm w", torch.bfloat16); _need(out, "moe gemm out")
    _need(block_group, "moe gemm groups", torch.int32)
    M, K = a.shape
    if w.dim() != 3 or w.shape[2] != K or block_group.numel() * block_rows != M:
        raise KernelError(f"moe_gemm_tc: shapes do not agree: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    N = w.shape[1]
    if tuple(out.shape) != (M, N // 2 if swiglu else N) or out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"moe_gemm_tc: output {tuple(out.shape)} {out.dtype} does not fit")
    if block_rows == GROUP_ROWS_TC_WIDE:
        tile_n = 256
    elif not tile_n:
        # many rows: persistent CTAs over 128 x 256 tiles with two accumulators (a tile is written out under the
        # next one's products); few rows: 128 x 128 tiles, two CTAs an SM, a stream of the chosen experts' weights
        tile_n = MOE_TILE_N or (257 if M >= 2048 and N >= 512 else 128)
    st = _tc_state(a.device)
    _call("moe_gemm_tcgen05", "ilb_moe_gemm_tc", _ptr(a), _ptr(w), _ptr(out), _i(1 if out.dtype == torch.float32 else 0), _i(M),
          _i(w.shape[0]), _i(N), _i(K), _i(a.stride(0)), _i(out.stride(0)), _i(1 if swiglu else 0), _ptr(block_group),
          _i(block_rows), _i(tile_n), _ptr(st.error), _f(act[0]), _f(act[1]), _f(act[2]), _stream(out))


def gemm_simt_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, block_group: torch.Tensor) -> None:
    """out[rows of block b] = a[rows of block b] @ w[block_group[b]].T for blocks of 16 rows; w is
    [groups, N, K]; blocks whose group is negative are left alone."""
    _need(a, "gemm a"); _need(w, "gemm w", a.dtype); _need(out, "gemm out"); _need(block_group, "gemm groups", torch.int32)
    M, K = a.shape
    if w.dim() != 3 or w.shape[2] != K or tuple(out.shape) != (M, w.shape[1]) or block_group.numel() * GROUP_ROWS_SIMT != M:
        raise KernelError(f"gemm_simt_grouped: shapes do not agree: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    N = w.shape[1]
    _call("gemm_simt", "ilb_gemm_simt_grouped", _ptr(a), _ptr(w), _ptr(out), _i(_code(a)), _i(_code(out)), _i(M), _i(N), _i(K),
          _i(K), _i(K), _i(N), _ptr(block_group), ctypes.c_longlong(N * K), _stream(out))


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = (cos, sin)(positions[t] * inv_freq[i]); inv_freq is 64-bit."""
    _need(positions, "rope positions", torch.int32); _need(inv_freq, "rope inv_freq", torch.float64)
    _need(out, "rope table", torch.float32)
    T, half = positions.numel(), inv_freq.numel()
    if tuple(out.shape) != (T, half, 2):
        raise KernelError("rope_table: out must be [T, rotary_dim/2, 2]")
    _call("elementwise", "ilb_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(out), _i(T),
          _i(half), _stream(out))


def add_inplace(x: torch.Tensor, y: torch.Tensor) -> None:
    _need(x, "add x", torch.float32); _need(y, "add y", torch.float32)
    if x.numel() != y.numel():
        raise KernelError("add_inplace: sizes differ")
    _call("elementwise", "ilb_add_inplace", _ptr(x), _ptr(y), ctypes.c_longlong(x.numel()), _stream(x))


def scale_cap_inplace(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> None:
    """x = x * scale, then (cap > 0) x = cap * tanh(x / cap); x is 32-bit."""
    _need(x, "scale_cap x", torch.float32)
    _call("elementwise", "ilb_scale_cap_inplace", _ptr(x), _f(scale), _f(cap), ctypes.c_longlong(x.numel()), _stream(x))


def decode_advance(tokens: torch.Tensor, positions: torch.Tensor, kv_len: torch.Tensor,
                   drawn: torch.Tensor, n_live: int) -> None:
    """tokens[:n_live] = drawn[:n_live]; positions and kv_len of those advance by one."""
    for t, what in ((tokens, "tokens"), (positions, "positions"), (kv_len, "kv_len"), (drawn, "drawn")):
        _need(t, what, torch.int32)
    _call("elementwise", "ilb_decode_advance", _ptr(tokens), _ptr(positions), _ptr(kv_len), _ptr(drawn),
          _i(n_live), _i(tokens.numel()), _stream(tokens))


# --------------------------------------------------------------------------- GEMM
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              bias: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """out (+)= a @ w.T (+ bias) with 32-bit fused multiply-adds in a fixed order."""
    _need(a, "gemm a"); _need(w, "gemm w", a.dtype); _need(out, "gemm out")
    _need(bias, "gemm bias", torch.float32)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or (bias is not None and bias.numel() != N):
        raise KernelError(f"gemm: shapes do not agree: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulation needs a 32-bit output")
    _call("gemm_simt", "ilb_gemm_simt", _ptr(a), _ptr(w), _ptr(bias), _ptr(out), _i(_code(a)),
          _i(_code(out)), _i(M), _i(N), _i(K), _i(K), _i(K), _i(N), _i(1 if accumulate else 0),
          _stream(out))


# --------------------------------------------------------------------------- attention
ROPE_INTERLEAVED, NORM_AFTER_ROTATION, NORM_UNWEIGHTED = 1, 2, 4      # bits of `mode` (qk_norm_rope.cu)


def qk_norm_rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], eps: float,
                       rope: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                       seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                       page_size: int, k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], nq: int, nkv: int, d: int, dv: Optional[int] = None,
                       mode: int = 0, v_first: Optional[torch.Tensor] = None, v_lambda: Optional[torch.Tensor] = None,
                       v_keep: bool = False) -> None:
    """Per-head q/k RMSNorm, rotation, q -> q_out, k/v -> cache pages (see qk_norm_rope.cu).
    `dv`: head size of the values (default d).  `mode`: ROPE_INTERLEAVED | NORM_AFTER_ROTATION |
    NORM_UNWEIGHTED.  `v_first` [T, nkv * dv]: with `v_keep` it receives this layer's values;
    with `v_lambda` (a device scalar) the values become (1 - lambda) v + lambda v_first first."""
    dv = d if dv is None else int(dv)
    _need(qkv, "qkv", contiguous=False); _need(q_out, "q_out", qkv.dtype)
    if qkv.stride(1) != 1 or qkv.shape[1] < (nq + nkv) * d + nkv * dv:
        raise KernelError("qk_norm_rope_cache: the projection's rows must hold q | k | v side by side")
    _need(q_weight, "q_norm weight", torch.float32); _need(k_weight, "k_norm weight", torch.float32)
    _need(rope, "rope table", torch.float32); _need(positions, "positions", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32); _need(block_table, "block table", torch.int32)
    _need(k_cache, "k cache"); _need(v_cache, "v cache")
    _need(v_first, "first values", qkv.dtype); _need(v_lambda, "value mixing coefficient", torch.float32)
    T = qkv.shape[0]
    if k_cache is not None:
        if tuple(k_cache.shape[1:]) != (nkv, page_size, d) or tuple(v_cache.shape) != (k_cache.shape[0], nkv, page_size, dv):
            raise KernelError(f"cache shapes {tuple(k_cache.shape)} / {tuple(v_cache.shape)} are not [pages, {nkv}, {page_size}, {d} / {dv}]")
        if block_table is None:
            raise KernelError("a cache write needs a block table")
    v_mode = 0
    if v_keep or v_lambda is not None:
        if v_first is None or tuple(v_first.shape) != (T, nkv * dv) or (v_keep and v_lambda is not None):
            raise KernelError("value mixing needs first values [tokens, nkv * dv], and either keeps or mixes them")
        v_mode = 1 if v_keep else 2
    max_blocks = 0 if block_table is None else block_table.shape[1]
    num_pages = 0 if k_cache is None else k_cache.shape[0]
    cache_code = _code(k_cache) if k_cache is not None else _code(qkv)
    _call("qk_norm_rope", "ilb_qk_norm_rope_cache", _ptr(qkv), _ptr(q_out), _i(_code(qkv)),
          _ptr(q_weight), _ptr(k_weight), _f(eps), _ptr(rope), _i(rotary_dim), _ptr(positions),
          _ptr(seq_of_token), _ptr(block_table), _i(max_blocks), _i(page_size), _i(num_pages),
          _ptr(k_cache), _ptr(v_cache), _i(cache_code), _i(T), _i(nq), _i(nkv), _i(d), _i(dv),
          _i(qkv.stride(0)), _i(q_out.shape[1]), _i(mode), _i(v_mode), _ptr(v_lambda), _ptr(v_first if v_mode else None),
          _stream(qkv))


def paged_attention_simple(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, positions: torch.Tensor,
                           seq_of_token: torch.Tensor, block_table: torch.Tensor, window: int,
                           scale: float, nq: int, nkv: int, d: int, dv: Optional[int] = None,
                           sink: Optional[torch.Tensor] = None) -> None:
    dv = d if dv is None else int(dv)
    _need(q, "attention q"); _need(out, "attention out", q.dtype); _need(sink, "attention sink", torch.float32)
    if sink is not None and sink.numel() != nq:
        raise KernelError("attention: one sink logit per query head")
    _need(k_cache, "k cache"); _need(v_cache, "v cache", k_cache.dtype)
    _need(positions, "positions", torch.int32); _need(seq_of_token, "seq_of_token", torch.int32)
    _need(block_table, "block table", torch.int32)
    num_pages, nkv_c, page_size, d_c = k_cache.shape
    if (nkv_c, d_c) != (nkv, d) or tuple(v_cache.shape) != (num_pages, nkv, page_size, dv):
        raise KernelError("attention: cache shape does not match the heads")
    _call("attention_simple", "ilb_paged_attention_simple", _ptr(q), _ptr(out), _i(_code(q)),
          _ptr(k_cache), _ptr(v_cache), _i(_code(k_cache)), _ptr(positions), _ptr(seq_of_token),
          _ptr(block_table), _i(block_table.shape[1]), _i(page_size), _i(num_pages),
          _i(window or 0), _f(scale), _i(q.shape[0]), _i(nq), _i(nkv), _i(d), _i(dv), _i(q.shape[1]),
          _i(out.shape[1]), _ptr(sink), _stream(q))


def attention_mixed_heads(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step,
                          block_table: torch.Tensor, window: int, scale: float, nq: int, nkv: int, d: int, dv: int,
                          sink: Optional[torch.Tensor] = None, head_mix: Optional[torch.Tensor] = None,
                          dist_r1: Optional[torch.Tensor] = None, dist_r2: Optional[torch.Tensor] = None,
                          softcap: float = 0.0, temp_coef: float = 0.0, temp_every: int = 1, workspace=None,
                          decode_chunk: int = 256) -> None:
    """Causal attention whose scores are capped, shifted by a distance term and mixed across heads before the
    softmax (see attention_mix.cu): s = scale * (1 + temp_coef ln(floor((i + 1) / temp_every) + 1)) q.k;
    s <- softcap tanh(s / softcap); s <- s - r1 ln(1 + r2 (i - j)); z_h = sum_g head_mix[h, g] s_g; softmax with `sink`."""
    _need(q, "attention q"); _need(out, "attention out", q.dtype); _need(k_cache, "k cache"); _need(v_cache, "v cache", k_cache.dtype)
    for t, what, n in ((sink, "sink", nq), (head_mix, "head mixing matrix", nq * nq), (dist_r1, "distance r1", nq), (dist_r2, "distance r2", nq)):
        _need(t, "attention " + what, torch.float32)
        if t is not None and t.numel() != n:
            raise KernelError(f"attention: the {what} has {t.numel()} elements, {n} are needed")
    num_pages, nkv_c, page_size, d_c = k_cache.shape
    if (nkv_c, d_c) != (nkv, d) or tuple(v_cache.shape) != (num_pages, nkv, page_size, dv):
        raise KernelError("attention: cache shape does not match the heads")
    if (MIX_TC_ENABLED and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and workspace is not None
            and attention_mix_tc_supported(nq, nkv, d, dv) and q.shape[1] % 8 == 0):
        # the tensor-core kernel: a block owns 16 tokens of a sequence with all heads; a step of single tokens cuts
        # every sequence's keys into chunks (by key index alone) whose records a second launch adds in order
        split = decode_chunk if step.decode_only else 0
        max_chunks, scratch = 0, None
        if split:
            # the chunk depends on the width of the block table alone (a constant of the engine, not of the batch):
            # at most MIX_MAX_CHUNKS records a sequence
            while block_table.shape[1] * page_size > split * MIX_MAX_CHUNKS:
                split *= 2
            max_chunks = max(1, -(-(block_table.shape[1] * page_size) // split))
            scratch = workspace.buffer("attn.mix_scratch", (step.n_seqs * max_chunks * nq * (dv + 2),), torch.float32)
        n_blocks = 0 if split else sum(-(-n // 16) for n in step.h_q_len)
        per_token = 0
        if not split and n_blocks <= MIX_FEW_BLOCKS and step.max_kv_len > MIX_PROMPT_CHUNK:
            # few blocks of 16 tokens with many keys each (a long prompt alone): the blocks also cut their keys into
            # chunks, so that the longest walk is a chunk and not the whole prompt; a second launch adds a token's records
            chunks = -(-step.max_kv_len // MIX_PROMPT_CHUNK)
            floats = q.shape[0] * chunks * nq * (dv + 2)
            if floats * 4 <= MIX_PROMPT_SCRATCH_BYTES:
                per_token, split, max_chunks = 1, MIX_PROMPT_CHUNK, chunks
                scratch = workspace.buffer("attn.mix_scratch", (floats,), torch.float32)
        _call("attention_mix", "ilb_attention_mix_tc", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(step.positions),
              _ptr(step.cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size), _i(num_pages), _i(window or 0), _f(scale),
              _i(step.n_seqs), _i(n_blocks), _i(nq), _i(nkv), _i(d), _i(dv), _i(q.shape[1]), _i(out.shape[1]), _ptr(sink),
              _ptr(head_mix), _ptr(dist_r1), _ptr(dist_r2), _f(softcap), _f(temp_coef), _i(temp_every), _i(split), _i(max_chunks),
              _ptr(scratch), ctypes.c_longlong(0 if scratch is None else scratch.numel()), _i(per_token), _i(q.shape[0]), _stream(q))
        return
    _call("attention_mix", "ilb_attention_mix", _ptr(q), _ptr(out), _i(_code(q)), _ptr(k_cache), _ptr(v_cache), _i(_code(k_cache)),
          _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table), _i(block_table.shape[1]), _i(page_size), _i(num_pages),
          _i(window or 0), _f(scale), _i(q.shape[0]), _i(nq), _i(nkv), _i(d), _i(dv), _i(q.shape[1]), _i(out.shape[1]),
          _ptr(sink), _ptr(head_mix), _ptr(dist_r1), _ptr(dist_r2), _f(softcap), _f(temp_coef), _i(temp_every), _stream(q))


MIX_TC_ENABLED = True      # tests switch it off to run the exact kernel on bfloat16
MIX_PROMPT_CHUNK = 1024    # keys a block of 16 tokens walks when the blocks of a step are few and their keys many
MIX_FEW_BLOCKS = 296       # "few": up to two blocks a multiprocessor
MIX_PROMPT_SCRATCH_BYTES = 256 << 20
MIX_MAX_CHUNKS = 512       # the most chunk records of a single token's keys (131,072 keys in chunks of 256; 4 MB of scratch a sequence at 16 heads of 128)


def attention_mix_tc_supported(nq: int, nkv: int, d: int, dv: int) -> bool:
    """Geometries the tensor-core kernel for mixed heads takes: at most 16 heads, head sizes in multiples of 16."""
    lib = load_module("attention_mix")
    lib.ilb_attention_mix_tc_supported.restype = ctypes.c_int
    return bool(lib.ilb_attention_mix_tc_supported(_i(nq), _i(nkv), _i(d), _i(dv)))


# --------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor, bad: Optional[torch.Tensor] = None) -> None:
    _need(logits, "argmax logits", torch.float32); _need(out, "argmax out", torch.int32)
    _need(bad, "argmax flags", torch.int32)
    rows, vocab = logits.shape
    _call("sampling", "ilb_argmax", _ptr(logits), _ptr(out), _ptr(bad), _i(rows), _i(vocab),
          _i(logits.stride(0)), _stream(logits))


def sample_filter_max_vocab() -> int:
    """Largest vocabulary whose draws can be filtered (top-k, top-p, min-p) on the device."""
    lib = load_module("sampling")
    lib.ilb_sample_filter_max_vocab.restype = ctypes.c_int
    return int(lib.ilb_sample_filter_max_vocab())


def mark_tokens(rows: torch.Tensor, tokens: torch.Tensor, is_generated: torch.Tensor, seen: torch.Tensor,
                generated: torch.Tensor, vocab: int) -> None:
    """Set bit t of row r of `seen` ([rows, ceil(vocab / 32)] int32, zeroed by the caller) for
    every entry (r, t), and of `generated` for entries flagged as generated."""
    for t, w in ((rows, "rows"), (tokens, "tokens"), (is_generated, "flags"), (seen, "seen bits"), (generated, "generated bits")):
        _need(t, "mark_tokens " + w, torch.int32)
    _call("sampling", "ilb_mark_tokens", _ptr(rows), _ptr(tokens), _ptr(is_generated), _i(tokens.numel()), _ptr(seen),
          _ptr(generated), _i(seen.shape[0]), _i(vocab), _stream(seen))


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                       out: torch.Tensor, bad: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
                       top_p: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
                       penalties: Optional[tuple] = None) -> None:
    """One draw per row from softmax(logits / T) by the reference's sorted-walk rule, after
    its filters if given: top_k [rows] int32 (0 = none), top_p and min_p [rows] float32;
    `penalties` = (seen bits, generated bits, repetition [rows], presence [rows]) applies
    the reference's penalties to the logits first (see mark_tokens)."""
    _need(logits, "sample logits", torch.float32); _need(temperature, "temperature", torch.float32)
    _need(uniform, "uniform", torch.float64); _need(out, "sample out", torch.int32)
    _need(bad, "sample flags", torch.int32); _need(top_k, "top-k", torch.int32)
    _need(top_p, "top-p", torch.float32); _need(min_p, "min-p", torch.float32)
    rows, vocab = logits.shape
    seen = gen = rep = pres = None
    if penalties is not None:
        seen, gen, rep, pres = penalties
        _need(seen, "seen bits", torch.int32); _need(gen, "generated bits", torch.int32)
        _need(rep, "repetition penalty", torch.float32); _need(pres, "presence penalty", torch.float32)
        if tuple(seen.shape) != (rows, (vocab + 31) // 32) or tuple(gen.shape) != tuple(seen.shape):
            raise KernelError("sample: token bitmaps must be [rows, ceil(vocab / 32)]")
    _call("sampling", "ilb_sample_temperature", _ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(top_k), _ptr(top_p),
          _ptr(min_p), _ptr(seen), _ptr(gen), _ptr(rep), _ptr(pres), _ptr(out), _ptr(bad), _i(rows), _i(vocab),
          _i(logits.stride(0)), _stream(logits))


# --------------------------------------------------------------------------- tensor-core GEMM
class _TcState:
    """Per-device scratch of the tensor-core kernels: the GEMM's split-K workspace and tile
    tickets (zero between launches), and the flag a kernel raises when a bounded wait runs out."""

    def __init__(self, device: torch.device) -> None:
        lib = load_module("gemm_tcgen05")
        lib.ilb_gemm_tc_workspace_floats.restype = ctypes.c_longlong
        self.floats = int(lib.ilb_gemm_tc_workspace_floats())
        self.n_tickets = int(lib.ilb_gemm_tc_max_tickets())
        self.workspace = torch.empty(self.floats, dtype=torch.float32, device=device)
        self.tickets = torch.zeros(self.n_tickets, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        # decode attention of few, long sequences: records of the clusters that share a sequence, and their tickets
        self.attn_scratch = torch.empty(1 << 20, dtype=torch.float32, device=device)
        self.attn_counters = torch.zeros(1 << 14, dtype=torch.int32, device=device)


_TC: dict = {}
TC_ENABLED = True          # tests switch it off to exercise the fallback


def _tc_state(device: torch.device) -> _TcState:
    st = _TC.get(device)
    if st is None:
        st = _TC[device] = _TcState(device)
    return st


def gemm_tc_eligible(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """bfloat16 operands whose rows are multiples of 16 bytes (TMA's rule)."""
    if not TC_ENABLED or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.shape[0] > 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, max_ctas: int = 0, swiglu: bool = False, gate: str = "silu", glu=None) -> None:
    """out (+)= a @ w.T (+ bias) on tcgen05 tensor cores (see gemm_tcgen05.cu).  With
    `swiglu`, `w` holds blocks of 64 gate rows followed by their 64 up rows and `out` is
    [M, N/2] = act(gate) * up, act = `gate` ("silu" or "relu"); or, with `glu` = (limit, sharpness, up_offset), the
    clamped unit a(min(gate, limit)) * (clamp(up, -limit, limit) + up_offset), a(g) = g * sigmoid(sharpness * g)."""
    if gate not in ("silu", "relu"):
        raise KernelError(f"gemm: the gated epilogue has no activation {gate!r}")
    if glu is not None and (not swiglu or float(glu[0]) <= 0):
        raise KernelError("gemm: the clamped gated unit belongs to the gated epilogue and needs a positive limit")
    _need(a, "gemm a", torch.bfloat16); _need(w, "gemm w", torch.bfloat16); _need(out, "gemm out")
    _need(bias, "gemm bias", torch.float32)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or (bias is not None and bias.numel() != N):
        raise KernelError(f"gemm: shapes do not agree: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and (out.dtype != torch.float32 or swiglu):
        raise KernelError("gemm: accumulation needs a 32-bit output and no SwiGLU epilogue")
    st = _tc_state(a.device)
    mode = (4 if glu is not None else 3 if gate == "relu" else 2) if swiglu else (1 if accumulate else 0)
    limit, sharp, offset = glu if glu is not None else (0.0, 1.0, 0.0)
    _call("gemm_tcgen05", "ilb_gemm_tc", _ptr(a), _ptr(w), _ptr(bias), _ptr(out),
          _i(1 if out.dtype == torch.float32 else 0), _i(M), _i(N), _i(K), _i(a.stride(0)), _i(w.stride(0)),
          _i(out.stride(0)), _i(mode), _ptr(st.workspace), ctypes.c_longlong(st.floats),
          _ptr(st.tickets), _i(st.n_tickets), _ptr(st.error), _i(max_ctas), _f(limit), _f(sharp), _f(offset), _stream(out))


def gemm_sums_in_memory(on: bool) -> None:
    """Whether products that accumulate into a 32-bit output may let the K ranges of a tile meet
    in memory: the tiles of the last round of many tokens (on single CTAs or on pairs), and every
    tile of up to eight tokens when the weight is large (faster; the order of that 32-bit sum
    is not fixed, so two runs agree beyond rounding but not bit for bit).  On by default;
    off gives sums whose bits do not change from run to run."""
    load_module("gemm_tcgen05").ilb_gemm_tc_sums_in_memory(_i(1 if on else 0))


def gemm_pairs(mode: int) -> None:
    """Products of many tokens on pairs of CTAs that the tensor cores treat as one unit
    (256 x 256 tiles, `tcgen05.mma.cta_group::2`): 0 never, 1 where the sizes favour it (the
    default), 2 wherever the kernel can run (tests use it at small sizes)."""
    load_module("gemm_tcgen05").ilb_gemm_tc_pairs(_i(int(mode)))


def gemm_tuning(few_tokens_in_memory: Optional[int] = None, few_tokens_ranges: int = 8,
                pair_ranges: Optional[int] = None, pair_fill_plain: float = 0.75, pair_fill_adding: float = 0.85) -> None:
    """Knobs behind the measured defaults, for A/B runs (the defaults are what the profiles
    report).  `few_tokens_in_memory`: accumulating products of up to this many tokens (and a
    weight of at least 2,048 x 2,048) add the K ranges of a tile in memory instead of inside a
    cluster, cut into up to `few_tokens_ranges` ranges (default 8 tokens; 0: never).
    `pair_ranges`: the most K ranges a tile of a pair of CTAs is cut into (default 8), with
    the shares of busy pairs that plain and adding products ask for before they take pairs."""
    lib = load_module("gemm_tcgen05")
    if few_tokens_in_memory is not None:
        lib.ilb_gemm_tc_red_few(_i(int(few_tokens_in_memory)), _i(int(few_tokens_ranges)))
    if pair_ranges is not None:
        lib.ilb_gemm_tc_pair_tuning(_i(int(pair_ranges)), _i(int(round(pair_fill_plain * 1000))),
                                    _i(int(round(pair_fill_adding * 1000))))


def gemm_tc_plan(M: int, N: int, K: int, accumulate: bool = False, swiglu: bool = False) -> dict:
    """How `gemm_tc` deals out a product of these sizes (needs a device: the answer depends
    on how many CTAs fit it).  `pairs` > 0: the product runs on that many pairs of CTAs, each
    tile left over after the whole rounds (or every tile) cut into `pair_split` K ranges, and
    `sums_meet_in_memory` speaks of those; the other fields then describe the single-CTA deal
    that `gemm_pairs(0)` would use."""
    lib = load_module("gemm_tcgen05")
    out = (ctypes.c_int * 11)()
    lib.ilb_gemm_tc_plan.restype = ctypes.c_int
    if lib.ilb_gemm_tc_plan(_i(M), _i(N), _i(K), _i(2 if swiglu else (1 if accumulate else 0)), out) != 0:
        raise KernelError(lib.ilb_last_error().decode())
    keys = ("swap", "tile_n", "row_blocks", "grid", "cluster", "rounds", "tiles", "tiles_stream_k", "sums_meet_in_memory",
            "pairs", "pair_split")
    return dict(zip(keys, list(out)))


def device_error_tensor(device) -> Optional[torch.Tensor]:
    """The one-int flag that kernels on `device` raise when a bounded wait runs out (None
    while no tensor-core kernel has run there yet)."""
    st = _TC.get(torch.device(device))
    return None if st is None else st.error


def check_device_errors() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (synchronises)."""
    for dev, st in _TC.items():
        if int(st.error.item()) != 0:
            st.error.zero_()
            st.tickets.zero_()
            raise KernelError(f"a tensor-core kernel on {dev} gave up waiting on a barrier; its output is invalid")


# --------------------------------------------------------------------------- attention dispatch
DECODE_CHUNK_MIN = 256      # keys per decode CTA; boundaries depend on the key index alone


def decode_chunk_for(max_positions: int) -> int:
    """Chunk length of split-KV decode for a model that reaches `max_positions`: 256 keys,
    or more for very long contexts so that a sequence never has more than 32 chunks."""
    chunk = DECODE_CHUNK_MIN
    while chunk * 32 < max_positions:
        chunk *= 2
    return chunk


def attention_flash_supported(d: int) -> bool:
    return d in (32, 64, 96, 128)


def attention_tc_supported(nq: int, nkv: int, d: int, page_size: int) -> bool:
    """Geometries the tcgen05 prefill attention is built for."""
    if nkv <= 0 or nq % nkv:
        return False
    g = nq // nkv
    return d in (64, 128) and g <= 128 and page_size in (16, 32, 64, 128)


def attention_prefill_tc(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                         n_tiles, nq, nkv, d, row_blocks: int = 1, skip_single: bool = False, sink=None) -> None:
    """Prefill attention on tcgen05 tensor cores (attention_tc.cu); a CTA takes `row_blocks`
    (1 or 2) blocks of 128 // (nq / nkv) tokens of one sequence, and n_tiles counts the CTAs
    over the sequences (with `skip_single`, over those that bring more than one token: the
    others' rows of `out` are left alone)."""
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    num_pages, _, page_size, _ = k_cache.shape
    st = _tc_state(q.device)
    _call("attention_tc", "ilb_attention_prefill_tc", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(q.shape[0]), _i(n_seqs), _i(n_tiles), _i(row_blocks), _i(1 if skip_single else 0), _i(nq), _i(nkv),
          _i(d), _i(q.shape[1]), _i(out.shape[1]), _ptr(st.error), _ptr(sink), _stream(q))


def attention_prefill(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                      n_tiles, nq, nkv, d, sink=None) -> None:
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    num_pages, _, page_size, _ = k_cache.shape
    _call("attention_flash", "ilb_attention_prefill", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(n_seqs), _i(n_tiles), _i(nq), _i(nkv), _i(d),
          _i(q.shape[1]), _i(out.shape[1]), _ptr(sink), _stream(q))


def attention_decode(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                     nq, nkv, d, chunk, max_chunks, scratch, tickets, sink=None) -> None:
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    _need(scratch, "attention scratch", torch.float32); _need(tickets, "attention tickets", torch.int32)
    num_pages, _, page_size, _ = k_cache.shape
    _call("attention_flash", "ilb_attention_decode", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(n_seqs), _i(nq), _i(nkv), _i(d), _i(q.shape[1]),
          _i(out.shape[1]), _i(chunk), _i(max_chunks), _ptr(scratch), ctypes.c_longlong(scratch.numel()),
          _ptr(tickets), _i(tickets.numel()), _ptr(sink), _stream(q))


def attention_decode_tma_supported(nq: int, nkv: int, d: int, page_size: int) -> bool:
    """Geometries the cluster-merged TMA decode attention is built for."""
    return nkv > 0 and nq > 0 and nq % nkv == 0 and d in (64, 128) and page_size in (16, 32, 64, 128)


# A decode step whose longest sequence holds at least this many keys is launched for the most
# CTAs at work: narrower clusters, several of them sharing a (sequence, kv head) when the
# sequences are few.  Recorded decode graphs are kept apart by this flag.
DECODE_LONG_CONTEXT = 8192


def attention_decode_plan(n_seqs: int, nq: int, nkv: int, d: int, page_size: int, long_context: bool = False) -> tuple:
    """(CTAs of a cluster, stages of the tile ring, clusters that may share a long sequence)
    that a decode step of this geometry gets."""
    lib = load_module("attention_decode")
    split, stages, chunks = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    lib.ilb_attention_decode_plan.restype = ctypes.c_int
    if lib.ilb_attention_decode_plan(_i(n_seqs), _i(nq), _i(nkv), _i(d), _i(page_size), _i(1 if long_context else 0), ctypes.byref(split),
                                     ctypes.byref(stages), ctypes.byref(chunks)) != 0:
        raise KernelError(lib.ilb_last_error().decode())
    return split.value, stages.value, chunks.value


def attention_decode_tma(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                         nq, nkv, d, long_context: bool = False) -> None:
    """Split-KV decode whose tiles come by TMA and whose partial results meet inside a
    thread-block cluster (no scratch)."""
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    num_pages, _, page_size, _ = k_cache.shape
    st = _tc_state(q.device)
    _call("attention_decode", "ilb_attention_decode_tma", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(n_seqs), _i(nq), _i(nkv), _i(d), _i(q.shape[1]),
          _i(out.shape[1]), _i(1 if long_context else 0), _ptr(st.attn_scratch), ctypes.c_longlong(st.attn_scratch.numel()), _ptr(st.attn_counters),
          ctypes.c_longlong(st.attn_counters.numel()), _ptr(st.error), _stream(q))


def attention_decode_fused_supported(dtype: torch.dtype, cache_dtype: torch.dtype, nq: int, nkv: int, d: int,
                                     page_size: int, rotary_dim: int, has_rope: bool, interleaved: bool = False) -> bool:
    """Whether a decode-only step can take q/k/v straight from the fused projection output:
    the TMA decode kernel's geometry, bfloat16 throughout, rotation over the whole head (pairs
    of neighbours: over any even part of it)."""
    return (DECODE_CLUSTER_ENABLED and DECODE_FUSED_ENABLED and FLASH_ENABLED and dtype == torch.bfloat16
            and cache_dtype == torch.bfloat16 and attention_decode_tma_supported(nq, nkv, d, page_size)
            and (not has_rope or rotary_dim == d or (interleaved and 0 < rotary_dim <= d and rotary_dim % 2 == 0)))


def attention_decode_fused(qkv, out, q_weight, k_weight, eps, rope_table, k_cache, v_cache, write_kv, positions, cu_q,
                           block_table, window, scale, n_seqs, nq, nkv, d, long_context: bool = False, mode: int = 0,
                           rotary_dim: Optional[int] = None, v_first: Optional[torch.Tensor] = None,
                           v_lambda: Optional[torch.Tensor] = None, v_keep: bool = False) -> None:
    """Decode attention with the per-head q/k norm, the rotation and the cache write of the
    step's own key and value inside the attention kernel (one launch instead of two).  `mode`,
    `rotary_dim`, `v_first`, `v_lambda` and `v_keep` as in `qk_norm_rope_cache`."""
    v_mode = 0
    if v_keep or v_lambda is not None:
        _need(v_first, "first values", torch.bfloat16); _need(v_lambda, "value mixing coefficient", torch.float32)
        if v_first is None or tuple(v_first.shape) != (qkv.shape[0], nkv * d) or (v_keep and v_lambda is not None):
            raise KernelError("value mixing needs first values [tokens, nkv * d], and either keeps or mixes them")
        v_mode = 1 if v_keep else 2
    _need(qkv, "attention qkv", torch.bfloat16, contiguous=False)
    if qkv.stride(1) != 1 or qkv.shape[1] < (nq + 2 * nkv) * d:
        raise KernelError("attention_decode_fused: the projection's rows must hold q | k | v side by side")
    for t, w in ((out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    for t, w in ((q_weight, "q norm weight"), (k_weight, "k norm weight"), (rope_table, "rope table")):
        if t is not None:
            _need(t, "attention " + w, torch.float32)
    num_pages, _, page_size, _ = k_cache.shape
    st = _tc_state(qkv.device)
    _call("attention_decode", "ilb_attention_decode_fused", _ptr(qkv), _i(qkv.stride(0)), _ptr(q_weight), _ptr(k_weight),
          _f(eps if eps and eps > 0 else 1e-6), _ptr(rope_table), _i(mode), _i(d if rotary_dim is None else rotary_dim), _i(v_mode),
          _ptr(v_first if v_mode else None), _ptr(v_lambda if v_mode == 2 else None), _i(1 if write_kv else 0), _ptr(out),
          _ptr(k_cache), _ptr(v_cache), _ptr(positions),
          _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size), _i(num_pages), _i(window or 0),
          _f(scale), _i(n_seqs), _i(nq), _i(nkv), _i(d), _i(out.shape[1]), _i(1 if long_context else 0), _ptr(st.attn_scratch),
          ctypes.c_longlong(st.attn_scratch.numel()), _ptr(st.attn_counters), ctypes.c_longlong(st.attn_counters.numel()),
          _ptr(st.error), _stream(qkv))


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              step, block_table: torch.Tensor, window: int, scale: float, nq: int, nkv: int,
              d: int, workspace=None, decode_chunk: int = DECODE_CHUNK_MIN, dv: Optional[int] = None,
              sink: Optional[torch.Tensor] = None) -> None:
    """Causal attention of the step's tokens over the cache; picks the kernel: the
    tensor-core kernels for a bfloat16 cache and a head size they are built for (split-KV
    when every sequence brings one token), else the exact kernel.  `sink` [nq] 32-bit: a logit
    per query head that joins the softmax's denominator (no key, no value, no scale)."""
    dv = d if dv is None else int(dv)
    _need(sink, "attention sink", torch.float32)
    fast = (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and attention_flash_supported(d) and dv == d
            and workspace is not None and FLASH_ENABLED)
    if not fast:          # the 32-bit path, and values of another head size than the keys'
        paged_attention_simple(q, out, k_cache, v_cache, step.positions, step.seq_of_token,
                               block_table, window, scale, nq, nkv, d, dv, sink)
        return
    G = nq // nkv
    # (the cluster-merged decode kernel takes no sink: single tokens of such layers go to the ticketed split-KV kernel)
    if step.decode_only and DECODE_CLUSTER_ENABLED and sink is None and attention_decode_tma_supported(nq, nkv, d, k_cache.shape[2]):
        attention_decode_tma(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                             step.n_seqs, nq, nkv, d, getattr(step, "max_kv_len", 0) >= DECODE_LONG_CONTEXT)
    elif step.decode_only:
        page_size = k_cache.shape[2]
        capacity = block_table.shape[1] * page_size
        max_chunks = max(1, -(-capacity // decode_chunk))
        if window:                       # a token reads the chunks its window touches, counted from the first of them
            max_chunks = min(max_chunks, (window - 1) // decode_chunk + 2)
        scratch = workspace.buffer("attn.decode_scratch", (step.n_seqs * nkv * max_chunks * G * (d + 2),), torch.float32)
        tickets = workspace.zeroed("attn.decode_tickets", (max(step.n_seqs * nkv, 4096),), torch.int32)
        attention_decode(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                         step.n_seqs, nq, nkv, d, decode_chunk, max_chunks, scratch, tickets, sink)
    elif TC_ATTENTION_ENABLED and attention_tc_supported(nq, nkv, d, k_cache.shape[2]):
        # A mixed step: the sequences that bring one token go to the split-KV decode kernel
        # (it leaves the others alone), the portions to the prefill kernel (which leaves those).
        lens = step.h_q_len
        kv_lens = getattr(step, "h_kv_len", None) or lens
        split = (MIXED_SPLIT_ENABLED and DECODE_CLUSTER_ENABLED and sink is None and 1 in lens and max(lens) > 1
                 and attention_decode_tma_supported(nq, nkv, d, k_cache.shape[2]))
        if split:
            attention_decode_tma(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                                 step.n_seqs, nq, nkv, d, False)
            kv_lens = [k for n, k in zip(lens, kv_lens) if n > 1]
            lens = [n for n in lens if n > 1]
        per_block = 128 // G
        n_one = sum(-(-n // per_block) for n in lens)
        n_two = sum(-(-n // (2 * per_block)) for n in lens)
        blocks = TC_ATTENTION_ROW_BLOCKS or tc_row_blocks(n_one * nkv, n_two * nkv, _sm_count(q.device),
                                                          all(k >= 2 * n for n, k in zip(lens, kv_lens)))
        n_tiles = n_two if blocks == 2 else n_one
        attention_prefill_tc(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                             step.n_seqs, n_tiles, nq, nkv, d, blocks, skip_single=split, sink=sink)
    else:
        n_tiles = sum(-(-n * G // 64) for n in step.h_q_len)
        attention_prefill(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                          step.n_seqs, n_tiles, nq, nkv, d, sink)


def tc_row_blocks(ctas_one: int, ctas_two: int, sms: int, behind_cache: bool) -> int:
    """Row blocks per CTA of the tcgen05 prefill kernel.  Two blocks share the K and V tiles
    and keep the tensor core busier, but a tile then takes 4,150 clocks for the pair against
    2,400 for one block (measured), and there are half as many CTAs.
    Portions behind a long cached prefix: every CTA walks about as many keys, the launch runs
    in rounds of one CTA per SM, and the cheaper of rounds x tile time wins (512 tokens of 40 / 8
    heads behind 3,584: 168 CTAs in two rounds, or 88 in one).  Prompts from their start: the
    CTAs' runs differ and pack well, and two blocks pay once there is a CTA for every SM."""
    if behind_cache:
        return 2 if -(-ctas_two // sms) * 1.7 < -(-ctas_one // sms) else 1
    return 2 if ctas_two >= sms else 1


DECODE_FUSED_ENABLED = True     # tests switch it off to run q/k norm + rotation + cache write as a launch of its own
DECODE_CLUSTER_ENABLED = True   # tests switch it off to reach the ticketed split-KV decode kernel
FLASH_ENABLED = True       # tests switch it off to exercise the exact kernel in bfloat16
TC_ATTENTION_ENABLED = True   # tests switch it off to reach the mma.sync prefill kernel at its geometries
TC_ATTENTION_ROW_BLOCKS = 0   # tests set 1 or 2 to force the row blocks per CTA of the tcgen05 prefill kernel
MIXED_SPLIT_ENABLED = True    # tests switch it off to send a mixed step's single tokens through the prefill kernel

_SM_COUNT: dict = {}


def _sm_count(device) -> int:
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n
