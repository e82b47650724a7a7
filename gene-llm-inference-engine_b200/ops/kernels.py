"""Python faces of the kernel entry points: tensors in, launches on the current stream.

Each function checks device, dtype, contiguity and sizes of what it is given (a kernel never sees
a pointer it could misread) and raises ``KernelError`` with the library's message when the library
refuses a size. Nothing here computes on the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError, check, lib

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype} (float32 and bfloat16 only)") from None


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (each wrapper call launches one)."""
    return _launches


def count_launches(n: int) -> None:
    """Adjusts the count for kernels that run from a replayed CUDA graph (or were only captured)."""
    global _launches
    _launches += n


_scoped_stream: Optional[int] = None


class on_current_stream:
    """Within this block every kernel goes to the stream that is current at its entry: the handle is
    looked up once instead of at every launch (a few microseconds each, a third of a millisecond of a
    step that launches 150 kernels). Blocks nest (a graph capture inside a step has its own stream)."""

    def __enter__(self):
        global _scoped_stream
        self._outer = _scoped_stream
        _scoped_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._outer
        return False


def _stream() -> int:
    global _launches
    _launches += 1
    return _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream


class Program:
    """A recorded sequence of this library's launches (csrc/program.cu): ``run()`` repeats it on the
    current stream with one call into the library. It holds raw addresses and sizes, so it is valid
    only while every buffer it was recorded with is."""

    def __init__(self, handle: int, launches: int):
        self._handle = handle
        self.launches = launches

    def run(self) -> None:
        global _launches
        stream = _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream
        check(lib().gi_program_run(self._handle, stream), "program")
        _launches += self.launches

    def __len__(self) -> int:
        return int(lib().gi_program_size(self._handle))

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                lib().gi_program_free(handle)
            except Exception:       # interpreter shutdown
                pass


class record:
    """``with record() as r: ...`` runs the block's kernel calls as usual and records them;
    ``r.program`` repeats them afterwards. Recordings do not nest."""

    program: Optional[Program] = None

    def __enter__(self):
        check(lib().gi_program_begin(), "program")
        self._before = _launches
        return self

    def __exit__(self, exc_type, exc, tb):
        handle = lib().gi_program_end()
        if exc_type is None:
            self.program = Program(handle, _launches - self._before)
        elif handle:
            lib().gi_program_free(handle)
        return False


def _dev(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t: Optional[torch.Tensor], name: str, dtype: torch.dtype) -> int:
    return 0 if t is None else _dev(t, name, dtype)


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
          feedback: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = table[tokens[t], :] * scale, widened to 32-bit. A negative tokens[t] = -(k + 1)
    stands for feedback[k], a token id that a sampling kernel left on the device."""
    T, D = out.shape
    if table.shape[1] != D or tokens.numel() != T:
        raise KernelError("embed: shapes of table, tokens and out do not agree")
    check(lib().gi_embed(_dev(table, "table"), dtype_code(table.dtype), _dev(tokens, "tokens", torch.int32),
                         _opt(feedback, "feedback", torch.int32), _dev(out, "out", torch.float32), T, D, float(scale),
                         _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = weight * (x[row_r, :] / sqrt(mean(x^2) + eps)); ``rows`` gathers rows of x."""
    n, D = out.shape
    if x.shape[1] != D or weight.numel() != D:
        raise KernelError("rmsnorm: shapes of x, weight and out do not agree")
    if rows is None and x.shape[0] < n:
        raise KernelError("rmsnorm: x has fewer rows than out")
    if rows is not None and rows.numel() != n:
        raise KernelError("rmsnorm: rows and out do not agree")
    check(lib().gi_rmsnorm(_dev(x, "x", torch.float32), _opt(rows, "rows", torch.int32),
                           _dev(weight, "weight", torch.float32), _dev(out, "out"), dtype_code(out.dtype),
                           n, D, float(eps), _stream()), "rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError("swiglu: gate_up must be [T, 2I] for out [T, I]")
    check(lib().gi_swiglu(_dev(gate_up, "gate_up", torch.float32), _dev(out, "out"), dtype_code(out.dtype), T, I,
                          _stream()), "swiglu")


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_tables: torch.Tensor,
               cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], interleaved: bool,
               q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
               num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool = True) -> None:
    """Rotates query and key heads of ``qkv`` [T, (H+2Hkv)*hd] by the rows of the cos/sin table at
    each token's position, writes queries to ``q_out`` [T, H*hd] and keys/values into the token's
    row of the paged cache [pages, Hkv, page_size, hd]."""
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("rope_store: qkv width does not match the head counts")
    if q_out.shape != (T, num_heads * head_dim):
        raise KernelError("rope_store: q_out must be [T, H*hd]")
    if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
        raise KernelError("rope_store: q_out and the cache must have one dtype")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("rope_store: the cache must be [pages, Hkv, page_size, hd]")
    rot_half = 0 if cos is None else cos.shape[1]
    if cos is not None and (sin is None or sin.shape != cos.shape):
        raise KernelError("rope_store: cos and sin tables must have one shape")
    check(lib().gi_rope_store(
        _dev(qkv, "qkv", torch.float32), _dev(positions, "positions", torch.int32),
        _dev(row_req, "row_req", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), rot_half,
        int(interleaved), _dev(q_out, "q_out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
        dtype_code(q_out.dtype), T, num_heads, num_kv_heads, head_dim, page_size, int(write_kv), _stream()),
        "rope_store")


# what a gated feed-forward applies to (gate, up): act(gate) * up, except "capped_swish" (with ``limit`` L):
# g = min(gate, L), u = clamp(up, -L, L), g * sigmoid(1.702 g) * (u + 1)
ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "capped_swish": 3}


def scale_cast(x: torch.Tensor, acc: torch.Tensor, xn: Optional[torch.Tensor], alpha: float) -> None:
    """acc = alpha * x (32-bit) and, when given, xn = x in xn's dtype."""
    if acc.shape != x.shape or (xn is not None and xn.shape != x.shape):
        raise KernelError("scale_cast: shapes do not agree")
    check(lib().gi_scale_cast(_dev(x, "x", torch.float32), _dev(acc, "acc", torch.float32), 0 if xn is None else _dev(xn, "xn"),
                              F32 if xn is None else dtype_code(xn.dtype), float(alpha), x.numel(), _stream()), "scale_cast")


def residual_norm(acc: torch.Tensor, weight: torch.Tensor, x_out: torch.Tensor, eps: float, alpha: float = 1.0,
                  acc_out: Optional[torch.Tensor] = None, xn_out: Optional[torch.Tensor] = None) -> None:
    """x_out = weight * (acc / sqrt(mean(acc^2) + eps)) per row, in 32-bit; optionally also acc_out = alpha * x_out
    (it may be ``acc`` itself) and xn_out = x_out in xn_out's dtype: what the next sublayer of a layer that
    normalises after the residual sum adds to and reads."""
    n, D = acc.shape
    if x_out.shape != acc.shape or weight.numel() != D:
        raise KernelError("residual_norm: shapes of acc, weight and x_out do not agree")
    for t, name in ((acc_out, "acc_out"), (xn_out, "xn_out")):
        if t is not None and t.shape != acc.shape:
            raise KernelError(f"residual_norm: {name} has the wrong shape")
    check(lib().gi_residual_norm(_dev(acc, "acc", torch.float32), _dev(weight, "weight", torch.float32),
                                 _dev(x_out, "x_out", torch.float32), _opt(acc_out, "acc_out", torch.float32),
                                 0 if xn_out is None else _dev(xn_out, "xn_out"),
                                 F32 if xn_out is None else dtype_code(xn_out.dtype), n, D, float(eps), float(alpha),
                                 _stream()), "residual_norm")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str, limit: float = 0.0,
              bias: Optional[torch.Tensor] = None) -> None:
    """out = act(gate_up[:, :I]) * gate_up[:, I:] for act in ACTIVATIONS (``limit``: the bound of "capped_swish");
    ``bias`` [2I] 32-bit is added to gate_up first."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or (bias is not None and bias.numel() != 2 * I):
        raise KernelError("gated_act: gate_up must be [T, 2I] for out [T, I] (and the bias [2I])")
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {', '.join(sorted(ACTIVATIONS))})")
    check(lib().gi_gated_act(_dev(gate_up, "gate_up", torch.float32), _opt(bias, "bias", torch.float32), _dev(out, "out"),
                             dtype_code(out.dtype), T, I, ACTIVATIONS[activation], float(limit), _stream()), "gated_act")


def norm_rope_store(proj: torch.Tensor, q_offset: int, k_offset: int, v_offset: int, q_norm: Optional[torch.Tensor],
                    k_norm: Optional[torch.Tensor], eps: float, freq: Optional[torch.Tensor], interleaved: bool,
                    positions: torch.Tensor, row_req: torch.Tensor, block_tables: torch.Tensor, q_out: torch.Tensor,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                    page_size: int, write_kv: bool = True, value_dim: Optional[int] = None, wide_norm: bool = False) -> None:
    """From the 32-bit projections ``proj`` [T, ld] (query heads from column q_offset, key heads from k_offset,
    value heads from v_offset, which may be the keys' columns): per head an optional unit-RMS norm with the
    shared weight ``q_norm`` / ``k_norm`` [hd] (``wide_norm``: one norm over all query heads' values together and one
    over all key heads', with weights [H*hd] and [Hkv*hd]), then the rotation of the first 2 * len(freq) dimensions by
    position * freq[i] (angles computed on the device in 32-bit), queries to ``q_out`` [T, H*hd], keys and
    values into the token's page row. ``value_dim``: the width of a value head when it is not the head size."""
    T, ld = proj.shape
    vd = head_dim if value_dim is None else int(value_dim)
    if q_out.shape != (T, num_heads * head_dim):
        raise KernelError("norm_rope_store: q_out must be [T, H*hd]")
    if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
        raise KernelError("norm_rope_store: q_out and the cache must have one dtype")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != (k_cache.shape[0], num_kv_heads, page_size, vd):
        raise KernelError("norm_rope_store: the cache must be [pages, Hkv, page_size, hd] (values: their own width)")
    for w, name, heads in ((q_norm, "q_norm", num_heads), (k_norm, "k_norm", num_kv_heads)):
        if w is not None and w.numel() != (heads * head_dim if wide_norm else head_dim):
            raise KernelError(f"norm_rope_store: {name} must have head_dim values (all heads' with wide_norm)")
    check(lib().gi_norm_rope_store(
        _dev(proj, "proj", torch.float32), ld, int(q_offset), int(k_offset), int(v_offset),
        _opt(q_norm, "q_norm", torch.float32), _opt(k_norm, "k_norm", torch.float32), float(eps),
        _opt(freq, "freq", torch.float32), 0 if freq is None else freq.numel(), int(interleaved),
        _dev(positions, "positions", torch.int32), _dev(row_req, "row_req", torch.int32),
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], _dev(q_out, "q_out"),
        _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), dtype_code(q_out.dtype), T, num_heads, num_kv_heads,
        head_dim, vd, page_size, int(write_kv), int(bool(wide_norm)), _stream()), "norm_rope_store")


def add_normed(y: torch.Tensor, weight: torch.Tensor, x: torch.Tensor, eps: float, xn_out: Optional[torch.Tensor] = None,
               clear_y: bool = False) -> None:
    """x += weight * (y / sqrt(mean(y^2) + eps)) per row, in 32-bit; optionally also xn_out = x in xn_out's dtype and
    y = 0: what the next sublayer of a layer whose norms stand on the sublayers' outputs reads and adds to."""
    n, D = y.shape
    if x.shape != y.shape or weight.numel() != D or (xn_out is not None and xn_out.shape != y.shape):
        raise KernelError("add_normed: shapes of y, weight, x and xn_out do not agree")
    check(lib().gi_add_normed(_dev(y, "y", torch.float32), _dev(weight, "weight", torch.float32), _dev(x, "x", torch.float32),
                              0 if xn_out is None else _dev(xn_out, "xn_out"), F32 if xn_out is None else dtype_code(xn_out.dtype),
                              n, D, float(eps), int(bool(clear_y)), _stream()), "add_normed")


def add_rows_at(x: torch.Tensor, table: torch.Tensor, index: torch.Tensor) -> None:
    """x[t, :] += table[index[t], :] in 32-bit (a learned vector per position added to the embedding's output)."""
    T, D = x.shape
    if table.dim() != 2 or table.shape[1] != D or index.numel() != T:
        raise KernelError("add_rows_at: shapes of x, table and index do not agree")
    check(lib().gi_add_rows_at(_dev(x, "x", torch.float32), _dev(table, "table"), dtype_code(table.dtype), _dev(index, "index", torch.int32),
                               T, D, table.shape[0], _stream()), "add_rows_at")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[t, :] += bias, 32-bit."""
    T, D = y.shape
    if bias.numel() != D:
        raise KernelError("add_bias: the bias must have one value per column")
    check(lib().gi_add_bias(_dev(y, "y", torch.float32), _dev(bias, "bias", torch.float32), T, D, _stream()), "add_bias")


def sigmoid_gate(a: torch.Tensor, gate: torch.Tensor, gate_offset: int, out: torch.Tensor) -> None:
    """out[t, c] = a[t, c] * sigmoid(gate[t, gate_offset + c]); a and gate 32-bit, out 32-bit or bfloat16."""
    T, N = a.shape
    if out.shape != a.shape or gate.dim() != 2 or gate.shape[0] != T or gate_offset + N > gate.shape[1]:
        raise KernelError("sigmoid_gate: shapes do not agree")
    check(lib().gi_sigmoid_gate(_dev(a, "a", torch.float32), _dev(gate, "gate", torch.float32), gate.shape[1], int(gate_offset),
                                _dev(out, "out"), dtype_code(out.dtype), T, N, _stream()), "sigmoid_gate")


def softcap(z: torch.Tensor, cap: float) -> None:
    """z <- cap * tanh(z / cap) in place, 32-bit."""
    check(lib().gi_softcap(_dev(z, "z", torch.float32), z.numel(), float(cap), _stream()), "softcap")


def scale(z: torch.Tensor, factor: float) -> None:
    """z <- factor * z in place, 32-bit."""
    check(lib().gi_scale(_dev(z, "z", torch.float32), z.numel(), float(factor), _stream()), "scale")


def depth_mix(x: torch.Tensor, y: torch.Tensor, mult: float, history: Optional[torch.Tensor] = None, slot: int = 0,
              weights: Optional[torch.Tensor] = None, first: bool = False, next_weight: Optional[torch.Tensor] = None,
              eps: float = 0.0, xn_out: Optional[torch.Tensor] = None, y_bias: Optional[torch.Tensor] = None) -> None:
    """The end of a layer whose sublayers were summed into ``y``: fresh = x + mult * y and y = 0 (``y_bias`` [D]: a bias
    that a sublayer's last product left to this kernel, added to every row of y first). With ``history``
    [T, slots, D] (every layer's fresh result, slot 0 what the first layer read: written too when ``first``) and
    ``weights`` [slot + 1]: history[:, slot] = fresh and x = sum_j weights[j] * history[:, j] over j <= slot; without,
    x = fresh. ``xn_out``: also next_weight[0] * x / sqrt(mean(x^2) + eps) in xn_out's dtype (the next layer's normed
    input when its norm has a single weight)."""
    T, D = x.shape
    if y.shape != x.shape or (xn_out is not None and xn_out.shape != x.shape) or (y_bias is not None and y_bias.numel() != D):
        raise KernelError("depth_mix: shapes do not agree")
    slots = 0
    if history is not None:
        if history.dim() != 3 or history.shape[0] != T or history.shape[2] != D or weights is None or weights.numel() != slot + 1:
            raise KernelError("depth_mix: the history must be [T, slots, D] and the layer needs slot + 1 weights")
        slots = history.shape[1]
    check(lib().gi_depth_mix(_dev(x, "x", torch.float32), _dev(y, "y", torch.float32), _opt(y_bias, "y_bias", torch.float32), float(mult), _opt(history, "history", torch.float32),
                             slots, int(slot), _opt(weights, "weights", torch.float32), int(bool(first)),
                             _opt(next_weight, "next_weight", torch.float32), float(eps), 0 if xn_out is None else _dev(xn_out, "xn_out"),
                             F32 if xn_out is None else dtype_code(xn_out.dtype), T, D, _stream()), "depth_mix")


def streams(X: torch.Tensor, single: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None, clear_y: bool = False,
            mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None, in_w: Optional[torch.Tensor] = None,
            norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, xn_out: Optional[torch.Tensor] = None,
            sum_out: Optional[torch.Tensor] = None) -> None:
    """Several copies of the residual stream, X [T, S, D] 32-bit. In one pass per row, any of: ``single`` [T, D]: the
    copies are all this row (X is written from it); ``y`` [T, D] with ``mix`` [S, S] (indexed [from, to]) and ``out_w`` [S]:
    every copy is rewritten at once, X'[t] = sum_s mix[s, t] X[s] + out_w[t] y (``clear_y``: y = 0 afterwards); ``in_w``
    [S] with ``norm_weight`` [D] and ``eps``: xn_out = norm_weight * u / sqrt(mean(u^2) + eps) for u = sum_s in_w[s] X'[s];
    ``sum_out`` [T, D] = sum_s X'[s]."""
    T, S, D = X.shape
    for t, name in ((single, "single"), (y, "y"), (xn_out, "xn_out"), (sum_out, "sum_out")):
        if t is not None and t.shape != (T, D):
            raise KernelError(f"streams: {name} must be [T, D]")
    if (y is not None and (mix is None or out_w is None or mix.numel() != S * S or out_w.numel() != S)) or \
            (in_w is not None and (in_w.numel() != S or norm_weight is None or norm_weight.numel() != D or xn_out is None)):
        raise KernelError("streams: a rewrite needs mix [S, S] and out_w [S]; a read needs in_w [S], the norm's weight [D] and xn_out")
    check(lib().gi_streams(_dev(X, "X", torch.float32), _opt(single, "single", torch.float32), _opt(y, "y", torch.float32),
                           int(bool(clear_y)), _opt(mix, "mix", torch.float32), _opt(out_w, "out_w", torch.float32),
                           _opt(in_w, "in_w", torch.float32), _opt(norm_weight, "norm_weight", torch.float32), float(eps),
                           0 if xn_out is None else _dev(xn_out, "xn_out"), F32 if xn_out is None else dtype_code(xn_out.dtype),
                           _opt(sum_out, "sum_out", torch.float32), T, S, D, _stream()), "streams")


def latent_store(proj: torch.Tensor, q_offset: int, q_weight: Optional[torch.Tensor], q_latent: Optional[torch.Tensor],
                 c_offset: int, c_weight: torch.Tensor, rot_offset: int, freq: Optional[torch.Tensor], amplitude: float,
                 eps: float, positions: torch.Tensor, row_req: torch.Tensor, block_tables: torch.Tensor, cache: torch.Tensor,
                 page_size: int, write_cache: bool = True) -> None:
    """From the 32-bit projections ``proj`` [T, ld]: the query latent (columns from q_offset, len(q_weight) wide) is
    brought to unit RMS, weighted and written to ``q_latent`` [T, q_rank]; the key/value latent (from c_offset,
    len(c_weight) wide) likewise into the first columns of the token's page row of ``cache`` [pages, 1, page_size,
    rank + rot]; the 2 * len(freq) columns from rot_offset are rotated pair by pair (2i, 2i+1) by position * freq[i],
    cos and sin times ``amplitude``, and written behind it."""
    T, ld = proj.shape
    rank = c_weight.numel()
    rot = 0 if freq is None else 2 * freq.numel()
    if cache.dim() != 4 or cache.shape[1:] != (1, page_size, rank + rot):
        raise KernelError("latent_store: the cache must be [pages, 1, page_size, rank + rot]")
    if q_latent is not None and (q_weight is None or q_latent.shape != (T, q_weight.numel()) or q_latent.dtype != cache.dtype):
        raise KernelError("latent_store: q_latent must be [T, q_rank] of the cache's dtype")
    check(lib().gi_latent_store(
        _dev(proj, "proj", torch.float32), ld, int(q_offset), 0 if q_weight is None else q_weight.numel(),
        _opt(q_weight, "q_weight", torch.float32), 0 if q_latent is None else _dev(q_latent, "q_latent"), int(c_offset), rank,
        _dev(c_weight, "c_weight", torch.float32), int(rot_offset), rot, _opt(freq, "freq", torch.float32), float(amplitude),
        float(eps), _dev(positions, "positions", torch.int32), _dev(row_req, "row_req", torch.int32),
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], _dev(cache, "cache"), dtype_code(cache.dtype), T,
        page_size, int(write_cache), _stream()), "latent_store")


def attention_rows_supported(head_dim: int, value_dim: int) -> bool:
    """Whether the row-form attention kernel serves these sizes."""
    return bool(lib().gi_attention_rows_supported(int(head_dim), int(value_dim)))


def attention_rows_tensor_cores(on: Optional[bool] = None) -> bool:
    """With a bfloat16 cache, at least eight query heads to a key/value head, a head size in whole 16s and a value size in
    whole 64s the row-form attention runs on the tensor cores; ``on`` False makes the CUDA-core form run there too (for
    comparisons). Returns the old setting."""
    old = bool(lib().gi_attention_rows_set_mma(1))
    lib().gi_attention_rows_set_mma(int(old if on is None else on))
    return old


def attention_rows_tile_tokens(num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, values_in_keys: bool) -> int:
    """How many consecutive tokens of one request share a tile of the tensor-core form of ``attention_rows`` over a
    bfloat16 cache (64 // heads per key/value head for head and value sizes up to 128, where every warp owns sixteen
    rows; 2 for larger heads with sixteen or more heads per key/value head; else 16 // heads per key/value head, at
    least 1); 0 when that form does not serve these sizes."""
    return int(lib().gi_attention_rows_tile_tokens(num_heads, num_kv_heads, head_dim, value_dim, int(values_in_keys)))


_ROWS_BLOCKS = 296          # about two blocks an SM: what the ranges of keys of a small launch are to fill


def attention_rows_splits(n_tiles: int, num_heads: int, num_kv_heads: int, span: int) -> int:
    """Into how many ranges the keys of every tile of a launch of ``n_tiles`` tiles are cut (1: none): few tiles
    (decoding) with many keys to see would leave most SMs idle. ``span``: the most keys a row sees."""
    blocks = n_tiles * num_kv_heads * ((num_heads // num_kv_heads + 15) // 16)
    if blocks <= 0 or blocks >= sm_count():
        return 1
    return max(1, min(16, _ROWS_BLOCKS // blocks, (span + 63) // 64))


def attention_rows_workspace_rows(n_tiles: int, num_heads: int, num_kv_heads: int, splits: int) -> int:
    """Rows [value_dim + 2] of 32-bit workspace that a launch cut into ``splits`` ranges of keys needs."""
    return n_tiles * num_kv_heads * ((num_heads // num_kv_heads + 15) // 16) * splits * 64 if splits > 1 else 0      # up to 64 rows a tile


def attention_rows(q: torch.Tensor, k_cache: torch.Tensor, v_cache: Optional[torch.Tensor], out: torch.Tensor,
                   row_req: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor, num_heads: int,
                   num_kv_heads: int, head_dim: int, value_dim: int, page_size: int, scale: float,
                   window: Optional[int] = None, chunk: Optional[int] = None, slopes: Optional[torch.Tensor] = None,
                   sinks: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                   tiles: Optional[torch.Tensor] = None, splits: int = 1, workspace: Optional[torch.Tensor] = None,
                   softcap: Optional[float] = None) -> None:
    """Attention of every row of ``q`` [T, H*hd] (32-bit or bfloat16) over its request's pages, 32-bit arithmetic.
    ``v_cache`` None: the values are the first ``value_dim`` columns of the key rows. ``window``: the last w positions;
    ``chunk``: only keys of the query's own block of c positions; ``slopes`` [H]: slope_h * distance is taken off a
    score; ``sinks`` [H]: exp(sinks_h) more in the softmax's denominator; ``softcap`` c: the scaled score s becomes
    c tanh(s / c). ``out`` [T, H*vd], 32-bit or bfloat16.
    (See attention_rows_tensor_cores for the form that rounds queries and softmax weights to bfloat16.)
    Tensor-core form only (attention_rows_tile_tokens() > 0): ``rows`` [n] lists the step rows to work on, a tile each;
    ``tiles`` [m, 3] = (first row, tokens (at most attention_rows_tile_tokens()), request) lists tiles of consecutive
    tokens of one request; ``splits`` > 1 cuts every tile's keys into ranges that run side by side and meet in
    ``workspace`` (attention_rows_workspace_rows() rows of value_dim + 2 floats)."""
    if rows is not None and tiles is not None:
        raise KernelError("attention_rows: give rows or tiles, not both")
    lst, kind, n_list = (rows, 1, rows.numel()) if rows is not None else (tiles, 2, tiles.shape[0]) if tiles is not None else (None, 0, 0)
    if tiles is not None and (tiles.dim() != 2 or tiles.shape[1] != 3):
        raise KernelError("attention_rows: tiles must be [m, 3]")
    T = q.shape[0]
    if q.dim() != 2 or q.shape[1] != num_heads * head_dim or out.shape != (T, num_heads * value_dim):
        raise KernelError("attention_rows: q must be [T, H*hd] and out [T, H*vd]")
    if k_cache.dim() != 4 or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim):
        raise KernelError("attention_rows: the keys must be [pages, Hkv, page_size, hd]")
    if v_cache is not None and (v_cache.shape != (k_cache.shape[0], num_kv_heads, page_size, value_dim) or v_cache.dtype != k_cache.dtype):
        raise KernelError("attention_rows: the values must be [pages, Hkv, page_size, vd] of the keys' dtype")
    for t, name in ((slopes, "slopes"), (sinks, "sinks")):
        if t is not None and t.numel() != num_heads:
            raise KernelError(f"attention_rows: {name} must have one value per head")
    check(lib().gi_attention_rows(
        _dev(q, "q"), dtype_code(q.dtype), q.shape[1], _dev(k_cache, "k_cache"), 0 if v_cache is None else _dev(v_cache, "v_cache"),
        dtype_code(k_cache.dtype), _dev(out, "out"), dtype_code(out.dtype), out.shape[1], _dev(row_req, "row_req", torch.int32),
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], T,
        num_heads, num_kv_heads, head_dim, value_dim, head_dim if v_cache is None else value_dim, int(v_cache is None), page_size,
        float(scale), float(softcap or 0.0), int(window or 0), int(chunk or 0), _opt(slopes, "slopes", torch.float32), _opt(sinks, "sinks", torch.float32),
        _opt(lst, "rows or tiles", torch.int32), kind, n_list, int(splits), _opt(workspace, "workspace", torch.float32),
        0 if workspace is None else workspace.numel(), _stream()), "attention_rows")
    if splits > 1:
        count_launches(1)


def attention_rows_of_step(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: Optional[torch.Tensor], out: torch.Tensor,
                           tables: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                           window: Optional[int], chunk: Optional[int], slopes: Optional[torch.Tensor],
                           sinks: Optional[torch.Tensor], softcap: Optional[float] = None, tiles_on=None, singles_on=None) -> None:
    """``attention_rows`` for all rows of a step. Over a bfloat16 cache with sizes that the tensor-core form serves, the
    step's single tokens and the tiles of its prompt portions (``ctx.attention_work``) run as two launches, each with its
    keys cut into ranges when it has few tiles; otherwise one launch works row by row. ``tiles_on`` = (tokens per tile,
    fn(work)): the tiles of prompt portions go to ``fn`` instead, another kernel that serves this form of attention;
    ``singles_on`` = fn(rows, longest context): likewise the rows of requests that bring a single token."""
    common = dict(window=window, chunk=chunk, slopes=slopes, sinks=sinks, softcap=softcap)
    per_tile = attention_rows_tile_tokens(num_heads, num_kv_heads, head_dim, value_dim, v_cache is None) \
        if k_cache.dtype is torch.bfloat16 else 0
    if per_tile == 0 or not hasattr(ctx, "attention_work"):
        attention_rows(q, k_cache, v_cache, out, ctx.row_req, ctx.positions, tables, num_heads, num_kv_heads, head_dim, value_dim,
                       ctx.page_size, scale, **common)
        return
    rows, work, _ = ctx.attention_work(per_tile)
    if tiles_on is not None:
        other = ctx.attention_work(tiles_on[0])[1]
        if other.shape[0]:
            tiles_on[1](other)
        work = work[:0]
    if singles_on is not None:
        if rows.numel():
            singles_on(rows, ctx.attention_work(per_tile)[2])
        rows = rows[:0]
    span = min(v for v in (window, chunk, getattr(ctx, "max_position", None), 1 << 30) if v)
    for name, lst, n in (("rows", rows, rows.numel()), ("tiles", work, work.shape[0])):
        if n == 0:
            continue
        splits = attention_rows_splits(n, num_heads, num_kv_heads, span)
        ws = None
        if splits > 1:
            ws = ctx.scratch("attention_rows_ranges_" + name, (attention_rows_workspace_rows(n, num_heads, num_kv_heads, splits), value_dim + 2),
                             torch.float32, capacity=(_ROWS_BLOCKS + 16) * 64)
        attention_rows(q, k_cache, v_cache, out, ctx.row_req, ctx.positions, tables, num_heads, num_kv_heads, head_dim, value_dim,
                       ctx.page_size, scale, splits=splits, workspace=ws, **{name: lst}, **common)


def attention_rows_launch_key(ctx, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, values_in_keys: bool,
                              dtype: torch.dtype):
    """What the launches of ``attention_rows_of_step`` depend on besides the token count."""
    per_tile = attention_rows_tile_tokens(num_heads, num_kv_heads, head_dim, value_dim, values_in_keys) if dtype is torch.bfloat16 else 0
    if per_tile == 0 or not hasattr(ctx, "attention_work"):
        return ()
    rows, work, _ = ctx.attention_work(per_tile)
    return (rows.numel(), work.shape[0])


def head_product(a: torch.Tensor, a_offset: int, a_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_offset: int,
                 out_head_stride: int, tail: int = 0, freq: Optional[torch.Tensor] = None, amplitude: float = 1.0,
                 positions: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """out[t, out_offset + h * out_head_stride + n] = sum_k w[h, n, k] * a[t, a_offset + h * a_head_stride + k] for
    every head h of ``w`` [H, N, K]: a matrix per head, applied to that head's slice of a row. ``tail`` > 0: the tail
    columns behind a head's K inputs are rotated pair by pair by positions[t] * freq[i] (cos and sin times
    ``amplitude``) and written behind the head's N outputs. ``gate`` [T, ld] 32-bit: output n of head h is multiplied by
    sigmoid(gate[t, gate_offset + h * N + n]) (an element-wise output gate laid out head by head)."""
    T = a.shape[0]
    H, N, K = w.shape
    if gate is not None and (gate.dim() != 2 or gate.shape[0] != T or gate_offset < 0 or gate_offset + H * N > gate.shape[1]):
        raise KernelError("head_product: the gate's columns lie outside its rows")
    if a.dim() != 2 or out.dim() != 2 or out.shape[0] != T:
        raise KernelError("head_product: a and out must be matrices with one row per token")
    if a_offset + (H - 1) * a_head_stride + K + tail > a.shape[1] or out_offset + (H - 1) * out_head_stride + N + tail > out.shape[1]:
        raise KernelError("head_product: a head's slice lies outside a row")
    if tail and (freq is None or positions is None or 2 * freq.numel() != tail):
        raise KernelError("head_product: a rotated tail needs tail / 2 frequencies and the positions")
    check(lib().gi_head_product(
        _dev(a, "a"), dtype_code(a.dtype), a.shape[1], int(a_offset), int(a_head_stride), _dev(w, "w"), dtype_code(w.dtype), N * K,
        _dev(out, "out"), dtype_code(out.dtype), out.shape[1], int(out_offset), int(out_head_stride), T, H, N, K, int(tail),
        _opt(freq, "freq", torch.float32), float(amplitude), 0 if positions is None else _dev(positions, "positions", torch.int32),
        _opt(gate, "gate", torch.float32), 0 if gate is None else gate.shape[1], int(gate_offset), _stream()), "head_product")


def grouped_tile_rows() -> int:
    """Rows per tile of the products that run one matrix per expert."""
    return int(lib().gi_grouped_tile_rows())


TC_TILE_ROWS = 128       # token rows per tile of the tensor-core product that takes a matrix per tile


def route_tiles(n_tokens: int, top: int, experts: int, tile_rows: Optional[int] = None) -> int:
    """An upper bound of the tiles that the (token, choice) pairs of a step make once bucketed by expert."""
    pairs = n_tokens * top
    tm = tile_rows or grouped_tile_rows()
    return (pairs + tm - 1) // tm + min(experts, pairs)


def route(x: torch.Tensor, w: torch.Tensor, correction: Optional[torch.Tensor], top: int, ids: torch.Tensor,
          weights: torch.Tensor, sorted_rows: torch.Tensor, tile_group: torch.Tensor, n_tiles: torch.Tensor,
          tile_rows: Optional[int] = None, pair_row: Optional[torch.Tensor] = None) -> None:
    """Per row of ``x`` [T, D]: s = sigmoid(w x) with ``w`` [E, D] 32-bit; the ``top`` experts with the largest
    s + correction go to ``ids`` [T, top] and their s to ``weights`` [T, top]. The pairs (token, choice) are then
    bucketed by expert into tiles of ``tile_rows`` rows (grouped_tile_rows() by default): ``sorted_rows`` (pair index
    or -1), ``tile_group`` (a tile's expert), ``n_tiles`` [1], and optionally ``pair_row`` [T * top], the row each pair
    landed in. Two launches."""
    T, D = x.shape
    E = w.shape[0]
    max_tiles = tile_group.numel()
    tm = tile_rows or grouped_tile_rows()
    if w.shape != (E, D) or ids.shape != (T, top) or weights.shape != (T, top) or (correction is not None and correction.numel() != E):
        raise KernelError("route: shapes do not agree")
    if sorted_rows.numel() < max_tiles * tm or max_tiles < route_tiles(T, top, E, tm) or (pair_row is not None and pair_row.numel() < T * top):
        raise KernelError("route: the buffers of the tiles are too small")
    check(lib().gi_route(_dev(x, "x"), dtype_code(x.dtype), T, D, _dev(w, "w", torch.float32), _opt(correction, "correction", torch.float32),
                         E, int(top), _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                         _dev(sorted_rows, "sorted_rows", torch.int32), _dev(tile_group, "tile_group", torch.int32),
                         _dev(n_tiles, "n_tiles", torch.int32), max_tiles, tm, _opt(pair_row, "pair_row", torch.int32), _stream()), "route")
    count_launches(1)


def route_table(tokens: torch.Tensor, feedback: Optional[torch.Tensor], table: torch.Tensor, experts: int, ids: torch.Tensor,
                weights: torch.Tensor, sorted_rows: torch.Tensor, tile_group: torch.Tensor, n_tiles: torch.Tensor,
                tile_rows: Optional[int] = None, pair_row: Optional[torch.Tensor] = None) -> None:
    """Experts fixed per token id: ids[t, :] = table[tokens[t], :] (``table`` [vocab, top] int32; a token given as
    -(k + 1) stands for feedback[k]), every weight 1 / top; then the bucketing of ``route``. Two launches."""
    T = tokens.numel()
    vocab, top = table.shape
    max_tiles = tile_group.numel()
    tm = tile_rows or grouped_tile_rows()
    if ids.shape != (T, top) or weights.shape != (T, top):
        raise KernelError("route_table: shapes do not agree")
    if sorted_rows.numel() < max_tiles * tm or max_tiles < route_tiles(T, top, experts, tm) or (pair_row is not None and pair_row.numel() < T * top):
        raise KernelError("route_table: the buffers of the tiles are too small")
    check(lib().gi_route_table(_dev(tokens, "tokens", torch.int32), _opt(feedback, "feedback", torch.int32), _dev(table, "table", torch.int32),
                               vocab, T, int(experts), top, _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                               _dev(sorted_rows, "sorted_rows", torch.int32), _dev(tile_group, "tile_group", torch.int32),
                               _dev(n_tiles, "n_tiles", torch.int32), max_tiles, tm, _opt(pair_row, "pair_row", torch.int32), _stream()),
          "route_table")
    count_launches(1)


def gather_rows(x: torch.Tensor, a_div: int, sorted_rows: torch.Tensor, n_tiles: torch.Tensor, tile_rows: int, out: torch.Tensor) -> None:
    """out[r] = x[sorted_rows[r] // a_div] for the rows of the first n_tiles tiles (zeros where sorted_rows is -1)."""
    if out.shape[1] != x.shape[1] or out.dtype != x.dtype or sorted_rows.numel() < out.shape[0]:
        raise KernelError("gather_rows: shapes do not agree")
    check(lib().gi_gather_rows(_dev(x, "x"), dtype_code(x.dtype), x.shape[1], int(a_div), _dev(sorted_rows, "sorted_rows", torch.int32),
                               _dev(n_tiles, "n_tiles", torch.int32), int(tile_rows), out.shape[0], _dev(out, "out"), _stream()), "gather_rows")


def expert_product_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, n_tiles: torch.Tensor,
                      gated: Optional[str] = None, limit: float = 0.0) -> None:
    """The same on the tensor cores (bfloat16) for rows already in the tiles' order: ``a`` [tiles * 128, K], tile i
    multiplies ``w[tile_group[i]]``; ``out`` [tiles * 128, N] 32-bit, or gated: bfloat16 act(gate) * up."""
    E, rows, K = w.shape
    N = rows // 2 if gated else rows
    M = a.shape[0]
    if a.shape != (M, K) or out.shape != (M, N) or M % TC_TILE_ROWS or tile_group.numel() < M // TC_TILE_ROWS:
        raise KernelError("expert_product_tc: shapes do not agree")
    if gated is not None and gated not in ACTIVATIONS:
        raise KernelError(f"expert_product_tc: unknown activation '{gated}'")
    st = _tc_state(a.device)
    check(lib().gi_gemm_tc_grouped(_dev(a, "a", torch.bfloat16), _dev(w, "w", torch.bfloat16),
                                   _dev(out, "out", torch.bfloat16 if gated else torch.float32),
                                   (2 | (ACTIVATIONS[gated] << 8)) if gated else 0, M, N, K, E,
                                   _dev(tile_group, "tile_group", torch.int32), _dev(n_tiles, "n_tiles", torch.int32),
                                   st.status.data_ptr(), float(limit), _stream()), "expert_product_tc")


def expert_product_tc_supported(N: int, K: int, gated: bool) -> bool:
    """Rows that TMA can address: K a multiple of 8, output rows of a multiple of 16 bytes."""
    return K % 8 == 0 and (N % 8 == 0 if gated else N % 4 == 0)


def expert_product(a: torch.Tensor, a_div: int, w: torch.Tensor, out: torch.Tensor, sorted_rows: torch.Tensor,
                   tile_group: torch.Tensor, n_tiles: torch.Tensor, gated: Optional[str] = None, limit: float = 0.0) -> None:
    """out[pair] = W[expert of pair] a[pair // a_div] for the pairs that ``route`` bucketed, ``w`` [E, N, K] (gated:
    [E, 2N, K], gate rows first, and out = act(gate) * up with ``gated`` one of ACTIVATIONS)."""
    E, rows, K = w.shape
    N = rows // 2 if gated else rows
    if a.dim() != 2 or a.shape[1] != K or out.dim() != 2 or out.shape[1] != N:
        raise KernelError("expert_product: shapes do not agree")
    if gated is not None and gated not in ACTIVATIONS:
        raise KernelError(f"expert_product: unknown activation '{gated}'")
    check(lib().gi_expert_product(_dev(a, "a"), dtype_code(a.dtype), K, int(a_div), _dev(w, "w"), dtype_code(w.dtype), rows * K, K,
                                  N * K if gated else 0, int(gated is not None), ACTIVATIONS.get(gated, 0), float(limit), _dev(out, "out"),
                                  dtype_code(out.dtype), N, N, K, _dev(tile_group, "tile_group", torch.int32),
                                  _dev(sorted_rows, "sorted_rows", torch.int32), _dev(n_tiles, "n_tiles", torch.int32),
                                  tile_group.numel(), _stream()), "expert_product")


def route_combine(part: torch.Tensor, weights: torch.Tensor, y: torch.Tensor, pair_row: Optional[torch.Tensor] = None) -> None:
    """y[t] += sum_k weights[t, k] * part[row of pair t * top + k], in the order of k; all 32-bit. The row of a pair is
    the pair itself, or ``pair_row[pair]`` when given."""
    T, D = y.shape
    top = weights.shape[1]
    if part.dim() != 2 or part.shape[1] != D or weights.shape[0] != T or (pair_row is None and part.shape[0] != T * top) or \
            (pair_row is not None and pair_row.numel() < T * top):
        raise KernelError("route_combine: shapes do not agree")
    check(lib().gi_route_combine(_dev(part, "part", torch.float32), _dev(weights, "weights", torch.float32),
                                 _opt(pair_row, "pair_row", torch.int32), _dev(y, "y", torch.float32), T, D, top, _stream()), "route_combine")


def causal_conv(proj: torch.Tensor, offset: int, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                state_offset: int, row_req: torch.Tensor, seg_start: torch.Tensor, seg_len: torch.Tensor,
                state_slots: torch.Tensor, out: torch.Tensor, activate: bool = True) -> None:
    """out[t, c] = act(bias[c] + sum_j weight[c, j] * u(t - taps + 1 + j, c)) (act: SiLU, or nothing when ``activate``
    is off; ``bias`` may be None) over the channels
    proj[:, offset:offset + C] of each request's rows; inputs before a segment's first row come from the request's
    state (``state`` [slots, floats per slot], the [taps-1, C] block at ``state_offset``), which afterwards
    holds the last taps-1 inputs. Two launches."""
    T, ld = proj.shape
    C, taps = weight.shape
    if out.shape != (T, C) or (bias is not None and bias.numel() != C):
        raise KernelError("causal_conv: shapes of weight, bias and out do not agree")
    if state.dim() != 2 or state_offset < 0 or state_offset + (taps - 1) * C > state.shape[1]:
        raise KernelError("causal_conv: the conv state does not fit the slot")
    R = seg_start.numel()
    check(lib().gi_causal_conv(_dev(proj, "proj", torch.float32), ld, int(offset), _dev(weight, "weight", torch.float32),
                               _opt(bias, "bias", torch.float32), _dev(state, "state", torch.float32), state.shape[1],
                               int(state_offset), _dev(row_req, "row_req", torch.int32), _dev(seg_start, "seg_start", torch.int32),
                               _dev(seg_len, "seg_len", torch.int32), _dev(state_slots, "state_slots", torch.int32),
                               _dev(out, "out", torch.float32), C, taps, T, R, int(bool(activate)), _stream()), "causal_conv")
    if taps > 1:
        count_launches(1)


def linear_scan(q: torch.Tensor, q_offset: int, k: torch.Tensor, k_offset: int, v: torch.Tensor, v_offset: int,
                num_heads: int, group: int, dk: int, dv: int, activate: bool, state: torch.Tensor, state_offset: int,
                seg_start: torch.Tensor, seg_len: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor,
                decay: Optional[torch.Tensor] = None, dt: Optional[torch.Tensor] = None, dt_offset: int = 0,
                dt_bias: Optional[torch.Tensor] = None, a_log: Optional[torch.Tensor] = None,
                skip: Optional[torch.Tensor] = None, part_len: int = 0, ws_state: Optional[torch.Tensor] = None,
                ws_decay: Optional[torch.Tensor] = None, row_gate: Optional[torch.Tensor] = None, row_gate_offset: int = 0,
                row_gate_bias: Optional[torch.Tensor] = None, tau: float = 1.0, q_scale: float = 1.0) -> None:
    """The recurrence S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t + skip * v_t per head over each
    request's rows in order, the state [H, dk, dv] carried in the request's slot of ``state`` [slots, floats]
    at ``state_offset``. q, k [T, ld] hold H / group heads of dk from their offsets (head h reads head
    h // group), v holds H heads of dv. Either ``decay`` [H] (a constant, b = 1) or ``dt`` [T, ld] with
    ``dt_bias`` and ``a_log`` [H] (dt' = softplus(dt + bias), a = exp(-exp(a_log) dt'), b = dt'), or ``row_gate``
    [T, ld] holding z for every head and key channel from ``row_gate_offset`` (plus ``row_gate_bias`` [H*dk]): row i of
    head h's state then fades by its own factor sigmoid(z)^(1/``tau``) per token, b = 1 (group must be 1).
    ``q_scale``: a constant on the queries. ``activate``: SiLU on q, k, v as they are read. All 32-bit.
    ``part_len`` > 0 cuts segments into parts of that many tokens which run side by side (three launches: the
    parts from zero states, the parts' start states, what the start states add); it needs ``ws_state``
    [scan_parts(T, R, part_len), H * dk * dv] and ``ws_decay`` [T, H] ([T, H * dk] with ``row_gate``). Results differ from the one-launch form by
    rounding only."""
    T = out.shape[0]
    if out.shape != (T, num_heads * dv):
        raise KernelError("linear_scan: out must be [T, H*dv]")
    kv_heads = num_heads // group
    for t, off, width, name in ((q, q_offset, kv_heads * dk, "q"), (k, k_offset, kv_heads * dk, "k"), (v, v_offset, num_heads * dv, "v")):
        if t.dim() != 2 or t.shape[0] != T or off < 0 or off + width > t.shape[1]:
            raise KernelError(f"linear_scan: {name} does not hold its heads inside a row")
    if row_gate is not None:
        if decay is not None or dt is not None or group != 1 or row_gate.dim() != 2 or row_gate.shape[0] != T or \
                row_gate_offset < 0 or row_gate_offset + num_heads * dk > row_gate.shape[1] or not tau > 0 or \
                (row_gate_bias is not None and row_gate_bias.numel() != num_heads * dk):
            raise KernelError("linear_scan: per-row decays come alone, one key head per head, their columns inside a row")
    elif decay is None and (dt is None or dt_bias is None or a_log is None or dt_offset + num_heads > dt.shape[1]):
        raise KernelError("linear_scan: give constant decays or step sizes with their bias and rates")
    for t, name in ((decay, "decay"), (dt_bias, "dt_bias"), (a_log, "a_log"), (skip, "skip")):
        if t is not None and t.numel() != num_heads:
            raise KernelError(f"linear_scan: {name} must have one value per head")
    if state.dim() != 2 or state_offset < 0 or state_offset + num_heads * dk * dv > state.shape[1]:
        raise KernelError("linear_scan: the state does not fit the slot")
    R = seg_start.numel()
    max_parts = 0
    if part_len:
        max_parts = (T + part_len - 1) // part_len          # no segment is longer than the step
        if ws_state is None or ws_decay is None or ws_state.numel() < scan_parts(T, R, part_len) * num_heads * dk * dv or \
                ws_decay.numel() < T * num_heads * (dk if row_gate is not None else 1):
            raise KernelError("linear_scan: the workspaces of the parts are missing or too small")
    check(lib().gi_linear_scan(
        _dev(q, "q", torch.float32), q.shape[1], int(q_offset), _dev(k, "k", torch.float32), k.shape[1], int(k_offset),
        _dev(v, "v", torch.float32), v.shape[1], int(v_offset), num_heads, group, dk, dv, int(bool(activate)),
        _opt(decay, "decay", torch.float32), _opt(dt, "dt", torch.float32), 0 if dt is None else dt.shape[1], int(dt_offset),
        _opt(dt_bias, "dt_bias", torch.float32), _opt(a_log, "a_log", torch.float32), _opt(skip, "skip", torch.float32),
        _opt(row_gate, "row_gate", torch.float32), 0 if row_gate is None else row_gate.shape[1], int(row_gate_offset),
        _opt(row_gate_bias, "row_gate_bias", torch.float32), 1.0 / float(tau), float(q_scale),
        _dev(state, "state", torch.float32), state.shape[1], int(state_offset), _dev(seg_start, "seg_start", torch.int32),
        _dev(seg_len, "seg_len", torch.int32), _dev(state_slots, "state_slots", torch.int32), _dev(out, "out", torch.float32),
        R, int(part_len), max_parts, _opt(ws_state, "ws_state", torch.float32), _opt(ws_decay, "ws_decay", torch.float32),
        _stream()), "linear_scan")
    if part_len:
        count_launches(2)


SCAN_PART = 128          # tokens per part of a long segment (see linear_scan)


def scan_parts(T: int, R: int, part_len: int = SCAN_PART) -> int:
    """An upper bound of the parts that R segments of T tokens together make."""
    return T // part_len + R


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, gate_offset: int, weight: torch.Tensor, out: torch.Tensor,
                     groups: int, eps: float, gate_first: bool, out_scale: float = 1.0, gate_act: str = "sigmoid") -> None:
    """Unit-RMS norm of y [T, W] in ``groups`` equal parts, times ``weight`` [W], with a gate from
    gate[:, gate_offset:gate_offset + W]: ``gate_first`` norms y * silu(gate); else the normed values are multiplied
    by sigmoid(gate) or, with ``gate_act`` "silu", by silu(gate). ``out_scale``: a constant factor."""
    T, W = y.shape
    if out.shape != (T, W) or weight.numel() != W or gate.dim() != 2 or gate.shape[0] != T:
        raise KernelError("gated_group_norm: shapes do not agree")
    check(lib().gi_gated_group_norm(_dev(y, "y", torch.float32), _dev(gate, "gate", torch.float32), gate.shape[1],
                                    int(gate_offset), _dev(weight, "weight", torch.float32), _dev(out, "out"),
                                    dtype_code(out.dtype), T, W, int(groups), float(eps),
                                    1 if gate_first else 2 if gate_act == "silu" else 0,
                                    float(out_scale), _stream()), "gated_group_norm")


def copy_pages(cache: torch.Tensor, src: torch.Tensor, dst: torch.Tensor) -> None:
    """cache is [arrays, pages, ...]; copies page src[i] to page dst[i] in every array."""
    n_arrays = cache.shape[0]
    page_bytes = cache[0, 0].numel() * cache.element_size()
    array_stride = cache[0].numel() * cache.element_size()
    check(lib().gi_copy_pages(_dev(cache, "cache"), array_stride, n_arrays, page_bytes,
                              _dev(src, "src", torch.int32), _dev(dst, "dst", torch.int32), src.numel(),
                              _stream()), "copy_pages")


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      row_req: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                      num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: Optional[int] = None, sink: bool = False, gate: Optional[torch.Tensor] = None,
                      gate_offset: int = 0, out_scale: float = 1.0) -> None:
    """Causal attention of every row of ``q`` [T, H*hd] over its request's pages. ``sink``: one more in the
    softmax's denominator; ``gate`` [T, ld] 32-bit: head h's output times sigmoid(gate[t, gate_offset + h]);
    ``out_scale``: a constant factor on the output."""
    T = q.shape[0]
    if gate is not None and (gate.dim() != 2 or gate.shape[0] != T or gate_offset < 0 or gate_offset + num_heads > gate.shape[1]):
        raise KernelError("attention: the gate must be [T, ld] with the heads' columns inside a row")
    if q.shape != (T, num_heads * head_dim) or out.shape != q.shape or out.dtype != q.dtype:
        raise KernelError("attention: q and out must be [T, H*hd] of one dtype")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelError("attention: q and the cache must have one dtype")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    check(lib().gi_attention_generic(
        _dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), _dev(out, "out"), dtype_code(q.dtype),
        _dev(row_req, "row_req", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], T, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), int(bool(sink)), _opt(gate, "gate", torch.float32),
        0 if gate is None else gate.shape[1], int(gate_offset), float(out_scale), _stream()), "attention")


def _epilogue(sink: bool, gate: Optional[torch.Tensor], gate_offset: int, out_scale: float, num_heads: int):
    """The arguments every attention entry point takes for what follows the softmax: a sink in the denominator,
    a sigmoid gate per head read from a 32-bit [T, ld] tensor, a constant factor."""
    if gate is not None and (gate.dim() != 2 or gate_offset < 0 or gate_offset + num_heads > gate.shape[1]):
        raise KernelError("attention: the gate must be [T, ld] with the heads' columns inside a row")
    return (int(bool(sink)), _opt(gate, "gate", torch.float32), 0 if gate is None else gate.shape[1], int(gate_offset),
            float(out_scale))


def attention_tma_pages(page_size: int) -> bool:
    """Whether the TMA-fed attention kernels can tile pages of this size."""
    return page_size % 8 == 0 and (32 % page_size == 0 or page_size % 32 == 0)


def attention_supported(head_dim: int) -> bool:
    """Whether any attention kernel of the library serves this head size (up to 256)."""
    return bool(lib().gi_attention_generic_supported(head_dim))


def attention_fast_supported(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    """Whether the tensor-core attention kernels are built for this head size and grouping."""
    return bool(lib().gi_attention_fast_supported(head_dim, num_heads, num_kv_heads))


def attention_prefill_rows(page_size: int, head_dim: int) -> int:
    """Query rows (tokens x heads of one key/value group) per work item of the prefill kernel."""
    return int(lib().gi_attention_prefill_rows(page_size, head_dim))


def attention_chunk_keys() -> int:
    """Positions per chunk of the decode kernel's split over the context (a fixed length)."""
    return int(lib().gi_attention_chunk_keys())


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     rows: torch.Tensor, row_req: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                     num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: Optional[int], part_o: torch.Tensor, part_ml: torch.Tensor, max_chunks: int,
                     n_chunks: int, sink: bool = False, gate: Optional[torch.Tensor] = None, gate_offset: int = 0,
                     out_scale: float = 1.0, softcap: Optional[float] = None) -> None:
    """Attention of single decoded tokens (bfloat16): ``rows`` lists their step rows; the context is
    split into fixed chunks whose partial results go through ``part_o`` / ``part_ml``. ``sink``, ``gate``,
    ``gate_offset``, ``out_scale``: as in ``attention_generic``. ``softcap`` c (pages that ``attention_tma_pages`` accepts
    only): the scaled score s becomes c tanh(s / c)."""
    n = rows.numel()
    if part_o.numel() < n * num_heads * max_chunks * head_dim or part_ml.numel() < n * num_heads * max_chunks * 2:
        raise KernelError("attention_decode: the workspace is too small")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, H*hd]")
    check(lib().gi_attention_decode(
        _dev(q, "q", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16), _dev(v_cache, "v_cache", torch.bfloat16),
        _dev(out, "out", torch.bfloat16), _dev(rows, "rows", torch.int32), n, _dev(row_req, "row_req", torch.int32),
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), max_chunks, n_chunks,
        k_cache.shape[0], _tc_state(q.device).status.data_ptr(), *_epilogue(sink, gate, gate_offset, out_scale, num_heads),
        float(softcap or 0.0), _stream()), "attention_decode")
    tma = page_size % 8 == 0 and (32 % page_size == 0 or page_size % 32 == 0)
    if n_chunks > 1 or not tma:
        count_launches(1)     # the kernel that merges the chunks (not needed when every context is one chunk)


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      work: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, scale: float, window: Optional[int],
                      sink: bool = False, gate: Optional[torch.Tensor] = None, gate_offset: int = 0,
                      out_scale: float = 1.0) -> None:
    """Attention of prompt portions (bfloat16): ``work`` [n, 3] = (first step row of a tile, tokens
    in it (at most attention_prefill_rows() // group size), request index)."""
    if work.dim() != 2 or work.shape[1] != 3:
        raise KernelError("attention_prefill: work must be [n, 3]")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, H*hd]")
    check(lib().gi_attention_prefill(
        _dev(q, "q", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16), _dev(v_cache, "v_cache", torch.bfloat16),
        _dev(out, "out", torch.bfloat16), _dev(work, "work", torch.int32), work.shape[0],
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        k_cache.shape[0], _tc_state(q.device).status.data_ptr(), *_epilogue(sink, gate, gate_offset, out_scale, num_heads),
        _stream()), "attention_prefill")


def attention_prefill_tc_supported(head_dim: int, num_heads: int, num_kv_heads: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention serves this shape (head size 64 or 128, pages TMA can tile)."""
    return bool(lib().gi_attention_prefill_tc_supported(head_dim, num_heads, num_kv_heads, page_size))


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         work: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor, num_heads: int,
                         num_kv_heads: int, head_dim: int, page_size: int, scale: float, window: Optional[int],
                         sink: bool = False, gate: Optional[torch.Tensor] = None, gate_offset: int = 0,
                         out_scale: float = 1.0, softcap: Optional[float] = None) -> None:
    """Attention of prompt portions on the tcgen05 tensor cores: ``work`` [n, 3] = (first step row of
    a tile, tokens in it (at most 128 // group size), request index). ``softcap`` c: the scaled score s becomes c tanh(s / c)."""
    if work.dim() != 2 or work.shape[1] != 3:
        raise KernelError("attention_prefill_tc: work must be [n, 3]")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, H*hd]")
    check(lib().gi_attention_prefill_tc(
        _dev(q, "q", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16), _dev(v_cache, "v_cache", torch.bfloat16),
        _dev(out, "out", torch.bfloat16), _dev(work, "work", torch.int32), work.shape[0],
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        k_cache.shape[0], _tc_state(q.device).status.data_ptr(), *_epilogue(sink, gate, gate_offset, out_scale, num_heads),
        float(softcap or 0.0), _stream()), "attention_prefill_tc")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T with 32-bit fused multiply-adds on the CUDA cores."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes do not agree (a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)})")
    check(lib().gi_gemm_simt(_dev(a, "a"), dtype_code(a.dtype), _dev(w, "w"), dtype_code(w.dtype), _dev(out, "out"),
                             dtype_code(out.dtype), int(accumulate), M, N, K, K, K, N, _stream()), "gemm")


class _TensorCoreState:
    """Per-device buffers of the tensor-core matrix product: the workspace and tile counters of the
    split over K, and the status word in which a kernel records a wait that gave up."""

    WORKSPACE_FLOATS = 8 * 1024 * 1024
    COUNTERS = 4096

    def __init__(self, device: torch.device):
        self.device = device
        self._workspace = None
        self.counters = torch.zeros(self.COUNTERS, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    @property
    def workspace(self) -> torch.Tensor:
        if self._workspace is None:        # only products split over K need it (the 32-bit path never does)
            self._workspace = torch.empty(self.WORKSPACE_FLOATS, dtype=torch.float32, device=self.device)
        return self._workspace


_tc_states = {}


def _tc_state(device: torch.device) -> _TensorCoreState:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _tc_states:
        _tc_states[key] = _TensorCoreState(device)
    return _tc_states[key]


_B200_SMS = 148          # only for looking at plans on a machine without a device
_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the device the kernels run on (asked once); the plans below
    size their grids by it. Without a device (plans examined on a CPU) the B200's count."""
    global _sm_count
    if _sm_count is None:
        if torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        else:
            return _B200_SMS
    return _sm_count


# Many-token products on pairs of CTAs (tcgen05 cta_group::2): the two CTAs of a pair share a 256-row tile of
# tokens and each fetches half of the weights' tile, so an SM takes in 32 KB instead of 48 KB per 64 columns of K.
PAIRED_PRODUCTS = True


def _paired(M: int, block_q: int) -> int:
    return int(PAIRED_PRODUCTS and M > 128 and block_q == 256)


def _persistent_plan(M: int, N: int, K: int):
    block_q = 256 if N >= 256 else 128 if N > 64 else 64
    splits = 1
    if block_q >= 128 and N % 4 == 0:
        # few output tiles (a prompt portion of a few hundred tokens, a narrow matrix): K is cut as well
        # so that about as many work items as SMs exist, each with at least 8 steps of 64
        tiles = ((M + 127) // 128) * ((N + block_q - 1) // block_q)
        k_blocks = (K + 63) // 64
        splits = max(1, min(8, sm_count() // tiles, k_blocks // 8))
        if splits < 3 and k_blocks < 64:
            splits = 1           # measured: two ranges of a short K cost more (a second kernel adds them) than they save
    return False, block_q, splits


def gemm_tc_plan(M: int, N: int, K: int, accumulate: bool = False):
    """(swap, block_q, splits) for a product of these sizes; the choice depends on the sizes (and on whether the
    product is added into its output) only.
    Few tokens put the weights on the 128-row side (the tokens are the N of the MMA) and split K until
    the grid fills the GPU. Many tokens put the tokens on the 128-row side, one persistent CTA per SM,
    K cut into ranges when the output has few tiles. Between 65 and 128 tokens a narrow matrix with a long K (one
    that the first form would split) is faster in the second form, whose ranges are added up by a
    kernel of their own instead of by one CTA per tile (measured at the Llama-3.2-1B widths: the down product of
    128 tokens 30 -> 17 us); with a short K, token tiles of 32 (or, for a product that is stored, of 64) in the first
    form are faster still (the O product of 128 tokens 11.5 -> 8.6 us, [q; k; v] 12.3 -> 9.6 us; at the Llama-3.1-8B
    widths [q; k; v] 30.5 -> 17.6 us)."""
    if M <= 128:
        tiles, k_blocks = (N + 127) // 128, (K + 63) // 64
        if M > 64 and k_blocks <= 64:
            if tiles * ((M + 31) // 32) * 2 <= sm_count():
                return True, 32, 2 if k_blocks >= 8 else 1
            if not accumulate and tiles * ((M + 63) // 64) <= sm_count():
                return True, 64, 1
        swap, block_q, splits = _swap_plan(M, N, K)
        if M > 32 and N >= 256 and N % 4 == 0 and (splits >= 6 or (M > 64 and splits > 1)):
            return _persistent_plan(M, N, K)
        return swap, block_q, splits
    return _persistent_plan(M, N, K)


_STREAMING_SHARE = 0.75


def _swap_plan(M: int, N: int, K: int):
    block_q = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = (N + 127) // 128
    k_blocks = (K + 63) // 64
    if 32 < M <= 64 and 2 * tiles * 2 <= sm_count():
        # 33 to 64 tokens over a matrix of few row tiles: two tiles of 32 tokens, each with its own CTAs (the second reads the
        # weights from L2), so that what the 32-token form has applies: ranges of K added up in a cluster, residual values
        # and rotation tables requested early, rotation in the epilogue. Measured at the Llama-3.2-1B widths, 64 tokens:
        # the O product 11.1 -> 7.3 us, down 16.1 -> 12.3, [q; k; v] 10.1 -> 8.6 (and no rotation kernel after it).
        splits = 1
        while 2 * tiles * (splits + 1) <= sm_count() and k_blocks // (splits + 1) >= 4 and splits < 5:
            splits += 1
        return True, 32, splits
    # split K until about three quarters of the SMs stream weights (112 CTAs on a B200), keeping at least
    # 4 steps of 64 per CTA (measured on B200 at the Llama-3.2-1B widths: 4 splits for 24 tiles, 6..8 for 16, 1 for 128)
    streaming = int(sm_count() * _STREAMING_SHARE) + 1
    # (17 to 32 tokens: at most 5 ranges, whose partial tiles have a place of their own beside four stages; measured at the
    # Llama-3.2-1B widths, 32 tokens: the O product 9.9 -> 8.6 us, down 13.4 -> 12.8)
    most = 5 if block_q == 32 else 8
    splits = 1
    while tiles * (splits + 1) <= streaming and k_blocks // (splits + 1) >= 4 and splits < most:
        splits += 1
    return True, block_q, splits


_cluster_splits_cache = {}


def gemm_tc_cluster_splits(block_q: int, tiles: int, splits: int, tiled: bool = False) -> int:
    """The split count to run: the planned one, or up to two fewer if only then all the launch's
    clusters (one per tile, a CTA per split) are resident at once, which lets the splits be added up
    in shared memory instead of through global memory. A property of the device, asked once."""
    key = (block_q, tiles, splits, tiled)
    if key not in _cluster_splits_cache:
        chosen = None
        # first with the partial tiles in shared memory of their own (no split waits for another), then
        # in the first split's pipeline stages (it tells the others when they are free)
        # (the first only while it keeps three quarters of the planned splits: fewer CTAs streaming the
        # weights cost more than the wait)
        for sign in (-1, 1):
            for s in range(splits, max(1, splits - 3), -1):
                if sign < 0 and 4 * s < 3 * splits:
                    continue
                if chosen is None and s >= 2 and lib().gi_gemm_tc_cluster_capacity(block_q, sign * s, int(tiled)) >= tiles:
                    chosen = s
        _cluster_splits_cache[key] = chosen or splits
    return _cluster_splits_cache[key]


def tile_weight(w: torch.Tensor) -> torch.Tensor:
    """A copy of the bfloat16 matrix w [N, K] laid out as the few-token product reads it: tiles of
    128 rows x 64 columns in the order [row tile][column block], each tile 16 KB in the swizzled
    K-major layout of the tensor cores (row r at r * 128 bytes, its 16-byte pieces permuted by
    piece ^ (r % 8)), rows padded with zeros to a multiple of 128 and columns to a multiple of 128.
    One untiled bulk copy then brings two neighbouring tiles (32 KB) into shared memory, which a B200
    SM does at 1.5 times the rate of tiled TMA boxes, with half as many waits and commits."""
    N, K = w.shape
    Np, Kp = (N + 127) // 128 * 128, (K + 127) // 128 * 128
    wp = torch.zeros((Np, Kp), dtype=w.dtype, device=w.device)
    wp[:N, :K] = w
    t = wp.view(Np // 128, 128, Kp // 64, 8, 8).permute(0, 2, 1, 3, 4)          # [row tile, k block, row, piece, 8]
    r = torch.arange(128, device=w.device).view(128, 1)
    piece = torch.arange(8, device=w.device).view(1, 8)
    src = (piece ^ (r % 8)).view(1, 1, 128, 8, 1).expand(t.shape[0], t.shape[1], 128, 8, 8)
    return torch.gather(t, 3, src).contiguous().view(-1)        # place q of row r holds piece q ^ (r % 8)


_gemm_choice = {}      # (M, N, K, output dtype, tiled weights) -> (swap, block_q, splits, persistent): the sizes decide, once


# How much of the weights that a later product will stream a few-token product asks into L2 (measured on B200 at the
# Llama-3.2-1B widths: 16 to 24 MiB ahead of the [gate; up] product make a decode step 1 to 3 % faster, 48 MiB slower)
AHEAD_BYTES = 24 << 20


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False, plan=None,
            w_tiles: Optional[torch.Tensor] = None, ahead: Optional[torch.Tensor] = None) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T on the tensor cores: bfloat16 operands, 32-bit accumulation,
    output 32-bit (optionally accumulated into) or bfloat16. K must be a multiple of 8. ``w_tiles``
    (tile_weight(w)) lets products of few tokens fetch the weights with bulk copies. ``ahead``: a tensor
    that a later kernel of the step streams (the tile-by-tile weights of the next large product); a product of few
    tokens asks its first AHEAD_BYTES into L2 while it runs, so that memory keeps streaming between the kernels."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes do not agree (a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)})")
    key = (M, N, K, out.dtype, w_tiles is not None, bool(accumulate)) if plan is None else None
    chosen = _gemm_choice.get(key) if key is not None else None
    if chosen is None:
        swap, block_q, splits = plan or gemm_tc_plan(M, N, K, bool(accumulate))
        persistent = not swap and out.dtype is torch.float32 and N % 4 == 0 and block_q >= 128
        if not swap and not persistent:
            if plan is None and M <= 128:
                swap, block_q, splits = _swap_plan(M, N, K)      # the persistent kernel cannot write this output
            else:
                splits = 1
        if plan is None and swap and splits > 1:
            splits = gemm_tc_cluster_splits(block_q, (N + 127) // 128 * ((M + block_q - 1) // block_q), splits,
                                            w_tiles is not None and block_q <= 128)
        chosen = (swap, block_q, splits, persistent)
        if key is not None:
            _gemm_choice[key] = chosen
    swap, block_q, splits, persistent = chosen
    st = _tc_state(a.device)
    if persistent:
        # many tokens, 32-bit output: the persistent kernel (epilogue overlapped, TMA stores)
        need = splits * ((M + 255) // 256 * 256) * N
        if splits > 1 and need > st.workspace.numel():
            splits = 1
        check(lib().gi_gemm_tc_persistent(_dev(a, "a", torch.bfloat16), _dev(w, "w", torch.bfloat16),
                                          _dev(out, "out", torch.float32), 1 if accumulate else 0, M, N, K, K, K, N,
                                          block_q, st.status.data_ptr(), splits, st.workspace.data_ptr() if splits > 1 else 0,
                                          st.workspace.numel() if splits > 1 else 0, _paired(M, block_q), 0.0, 0, _stream()), "gemm_tc")
        if splits > 1:
            count_launches(1)     # the kernel that adds the ranges up
        return
    check(lib().gi_gemm_tc(_dev(a, "a", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"),
                           dtype_code(out.dtype), int(accumulate), M, N, K, K, K, N, int(swap), block_q, splits,
                           st.workspace.data_ptr(), st.workspace.numel(), st.counters.data_ptr(), st.counters.numel(),
                           st.status.data_ptr(), _opt(w_tiles, "w_tiles", torch.bfloat16),
                           ahead.data_ptr() if ahead is not None and swap and M <= 32 else 0,
                           min(AHEAD_BYTES, ahead.numel() * ahead.element_size()) if ahead is not None else 0,
                           _stream()), "gemm_tc")


def gemm_swiglu_supported(M: int, I: int, K: int) -> bool:
    """The fused gate/up product needs many tokens (tokens on the 128-row side) and TMA-addressable rows."""
    return M > 128 and K % 8 == 0 and I % 8 == 0


def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", limit: float = 0.0,
                bias: Optional[torch.Tensor] = None) -> None:
    """out[M, I] = act(a @ w_gate^T) * (a @ w_up^T) as bfloat16, w_gate_up = [gate rows; up rows]
    [2I, K]: one tensor-core kernel whose epilogue applies the activation (the [M, 2I] intermediate
    never exists in memory). ``activation``: one of ACTIVATIONS (``limit``: see gated_act); ``bias`` [2I] 32-bit is added
    to the gate and up values before the activation."""
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_swiglu: unknown activation '{activation}'")
    M, K = a.shape
    I = out.shape[1]
    if w_gate_up.shape != (2 * I, K) or out.shape[0] != M or (bias is not None and bias.numel() != 2 * I):
        raise KernelError("gemm_swiglu: shapes do not agree")
    st = _tc_state(a.device)
    check(lib().gi_gemm_tc_persistent(_dev(a, "a", torch.bfloat16), _dev(w_gate_up, "w_gate_up", torch.bfloat16),
                                      _dev(out, "out", torch.bfloat16), 2 | (ACTIVATIONS[activation] << 8), M, I, K, K, K, I, 256,
                                      st.status.data_ptr(), 1, 0, 0, _paired(M, 256), float(limit), _opt(bias, "bias", torch.float32),
                                      _stream()), "gemm_swiglu")


_ROPE_FEW_TOKENS = 64      # up to here the few-token product (weights on the 128-row side, token tiles of at most 32) does
                           # the rotation: measured in whole decode steps, 2.4 % faster at 16 tokens (with 64-token tiles
                           # it was 1.7 % slower at 64 tokens)


def gemm_rope_store_supported(M: int, K: int, num_heads: int, num_kv_heads: int, head_dim: int,
                              cos: Optional[torch.Tensor], interleaved: bool) -> bool:
    """Whether the [q; k; v] product of M tokens can rotate and store in its own epilogue. Few tokens: the
    head size must divide 128 (both members of a pair in one tile of weight rows), any rotation. Many
    tokens: head sizes 32, 64, 128, whole heads rotated in the half-split pairing (or no rotation), and
    enough output tiles that K is not cut into ranges. Between the two, and otherwise, the product and
    the rope+store kernel run one after the other."""
    if K % 8:
        return False
    N = (num_heads + 2 * num_kv_heads) * head_dim
    if M <= 32 or (M <= _ROPE_FEW_TOKENS and _swap_plan(M, N, K)[1] == 32):      # token tiles of at most 32
        return 128 % head_dim == 0
    if head_dim not in (32, 64, 128) or not (cos is None or (not interleaved and 2 * cos.shape[1] == head_dim)):
        return False
    return M > 128 and _persistent_plan(M, N, K)[2] == 1


def gemm_rope_store(a: torch.Tensor, w_qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                    block_tables: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                    interleaved: bool, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool = True,
                    w_tiles: Optional[torch.Tensor] = None) -> None:
    """``rope_store`` of ``a @ w_qkv^T`` in one tensor-core kernel: the product's epilogue rotates the
    query and key heads and writes queries to ``q_out`` and keys/values into the pages; the
    [T, (H+2Hkv)*hd] intermediate never exists in memory. All operands bfloat16."""
    M, K = a.shape
    N = (num_heads + 2 * num_kv_heads) * head_dim
    if w_qkv.shape != (N, K):
        raise KernelError("gemm_rope_store: the weight must be [(H+2Hkv)*hd, K]")
    if q_out.shape != (M, num_heads * head_dim):
        raise KernelError("gemm_rope_store: q_out must be [T, H*hd]")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("gemm_rope_store: the cache must be [pages, Hkv, page_size, hd]")
    if cos is not None and (sin is None or sin.shape != cos.shape):
        raise KernelError("gemm_rope_store: cos and sin tables must have one shape")
    if not gemm_rope_store_supported(M, K, num_heads, num_kv_heads, head_dim, cos, interleaved):
        raise KernelError(f"gemm_rope_store: not built for {M} tokens, head size {head_dim} and this rotation")
    st = _tc_state(a.device)
    rope_args = (_dev(positions, "positions", torch.int32), _dev(row_req, "row_req", torch.int32),
                 _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], _opt(cos, "cos", torch.float32),
                 _opt(sin, "sin", torch.float32), 0 if cos is None else cos.shape[1], int(interleaved),
                 _dev(q_out, "q_out", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16),
                 _dev(v_cache, "v_cache", torch.bfloat16), num_heads, num_kv_heads, head_dim, page_size, int(write_kv))
    if M <= _ROPE_FEW_TOKENS:
        _, block_q, splits = _swap_plan(M, N, K)
        if splits > 1:
            splits = gemm_tc_cluster_splits(block_q, (N + 127) // 128 * ((M + block_q - 1) // block_q), splits, w_tiles is not None)
        check(lib().gi_gemm_tc_rope(_dev(a, "a", torch.bfloat16), _dev(w_qkv, "w_qkv", torch.bfloat16), M, K, K, K, block_q,
                                    splits, st.workspace.data_ptr(), st.workspace.numel(), st.counters.data_ptr(),
                                    st.counters.numel(), st.status.data_ptr(), _opt(w_tiles, "w_tiles", torch.bfloat16),
                                    *rope_args, _stream()), "gemm_rope_store")
    else:
        check(lib().gi_gemm_tc_persistent_rope(_dev(a, "a", torch.bfloat16), _dev(w_qkv, "w_qkv", torch.bfloat16), M, K, K, K,
                                               *rope_args, st.status.data_ptr(), _paired(M, 256), _stream()), "gemm_rope_store")


def l2_streaming(weights: Optional[bool] = None, keys_values: Optional[bool] = None):
    """In steps of few tokens the weights of the matrix products and the keys and values of decode attention, which
    a step reads once, are loaded with the "evict first" L2 policy, so that they do not push out what the step's
    kernels read again soon. Sets either switch (None leaves it) and returns the old (weights, keys_values)."""
    old_w = bool(lib().gi_gemm_tc_set_stream_weights(1))
    lib().gi_gemm_tc_set_stream_weights(int(old_w if weights is None else weights))
    old_kv = bool(lib().gi_attention_set_stream_kv(1))
    lib().gi_attention_set_stream_kv(int(old_kv if keys_values is None else keys_values))
    return old_w, old_kv


def specialised_products(on: Optional[bool] = None) -> bool:
    """The forms of the few-token product that a decode step runs (rotating [q; k; v], added into the residual stream,
    stored unsplit; up to 16 tokens over tiled weights) have kernels of their own with nothing else compiled in;
    ``on`` False makes the kernel of every form run them too (same results). Returns the old setting."""
    old = bool(lib().gi_gemm_tc_set_specialised(1))
    lib().gi_gemm_tc_set_specialised(int(old if on is None else on))
    return old


def status_word(device: torch.device) -> torch.Tensor:
    """The device word [1] (int32) in which a kernel records a bounded wait that gave up (0 = none)."""
    return _tc_state(device).status


def gemm_tc_status(device: torch.device) -> int:
    """0 when no bounded wait of a tensor-core kernel ever gave up on this device (synchronises)."""
    import ctypes
    st = _tc_state(device)
    out = ctypes.c_int(0)
    check(lib().gi_gemm_tc_status(st.status.data_ptr(), torch.cuda.current_stream().cuda_stream, ctypes.byref(out)),
          "gemm_tc_status")
    return out.value


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r (the lowest index among equals)."""
    rows, V = logits.shape
    key = logits.device.index
    buf = _argmax_scratch.get(key)
    if buf is None or buf[0].numel() < rows * 32:
        n = max(rows, 64) * 32
        buf = (torch.empty(n, dtype=torch.float32, device=logits.device), torch.empty(n, dtype=torch.int32, device=logits.device))
        _argmax_scratch[key] = buf
    check(lib().gi_argmax(_dev(logits, "logits", torch.float32), rows, V, _dev(out, "out", torch.int32),
                          buf[0].data_ptr(), buf[1].data_ptr(), _stream()), "argmax")
    global _launches
    _launches += 1            # two kernels


def sample(logits: torch.Tensor, scratch: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    rows, V = logits.shape
    if scratch.numel() < rows * V:
        raise KernelError("sample: scratch must hold rows x vocab floats")
    check(lib().gi_sample(_dev(logits, "logits", torch.float32), _dev(scratch, "scratch", torch.float32), rows, V,
                          _dev(temperature, "temperature", torch.float32), _dev(top_k, "top_k", torch.int32),
                          _dev(top_p, "top_p", torch.float32), _dev(uniform, "uniform", torch.float32),
                          _dev(out, "out", torch.int32), _stream()), "sample")
