"""The hot ops of the forward pass: thin, checked wrappers over the sm_100a kernels.

Every function takes CUDA tensors, checks element types, shapes and contiguity, and launches on
the current stream.  A size that a kernel does not take is refused with an error; nothing here
falls back to a tensor library's model code or to the CPU.  Matrix products in bfloat16 go to the
library GEMM (cuBLAS through `torch.mm`), as the reference's go to its tensor library
(crates/model/src/layers.rs:82); in float32 they go to this package's own FFMA kernel so that
no reduced-precision matrix mode can enter.
"""

from __future__ import annotations

import functools

import torch

from . import library
from .library import KernelError, check, debug_set, lib

_DT = {torch.float32: 0, torch.bfloat16: 1}

# Number of launches of this package's kernels since the last reset (a claim the benchmark
# reports; launches replayed from a captured graph are counted by the graph's owner).
launch_count = 0


def set_programmatic_launch(on: bool) -> None:
    """Whether kernels are launched with the programmatic-serialization attribute (on unless
    switched off, here or by RLIS_DEBUG=pdl=0): the next kernel's CTAs start their prologue while
    the current kernel drains; see csrc/kernels/common.cuh."""
    debug_set("pdl", 1 if on else 0)


def _code(dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)") from None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  (The raw lookup takes a microsecond; building a
    `torch.cuda.Stream` object for it took eighteen, three times a decode step.)"""
    if _raw_stream is not None:
        return _raw_stream(-1)
    return torch.cuda.current_stream().cuda_stream


def _req(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor, got strides {t.stride()}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None:
        if t.dim() != len(shape) or any(s is not None and s != g for s, g in zip(shape, t.shape)):
            raise KernelError(f"{name}: expected shape {shape}, got {tuple(t.shape)}")


# The same by kernel, for tests that have to know which kernel a step went through:
# {"stream_gemm.sink": 12, "attention_decode_qkv.mma.tma": 4, ...}.
launches_by_kernel: dict = {}


def _count(name: str) -> None:
    global launch_count
    launch_count += 1
    launches_by_kernel[name] = launches_by_kernel.get(name, 0) + 1


def _decode_variant() -> str:
    """Which decode-attention kernel the launcher just chose."""
    v = lib().rlis_attention_decode_last_variant()
    if not v & 1:
        return ".cuda_core"
    return ".mma" + (".tma" if v & 2 else "") + (".cluster" if v & 4 else "")


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to float32 (times `scale` if given).  ids int32 [T];
    out float32 [T, H]."""
    V, H = table.shape
    T = ids.shape[0]
    _req(ids, "ids", torch.int32, (T,))
    _req(table, "table")
    _req(out, "out", torch.float32, (T, H))
    check(lib().rlis_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, V,
                               1.0 if scale is None else float(scale), _code(table.dtype), _stream()), "embedding")
    _count("embedding")
    return out


def embedding_sink(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float | None, sink):
    """`embedding` for a step whose first norm is left to the product after it (`sink`, a
    ResidualSink over `out`): also returns that norm's ScaledRows, bf16(row * weight) and the sums of
    squares of every 128 features.  bfloat16 tables whose width is a multiple of 8."""
    V, H = table.shape
    T = ids.shape[0]
    _req(ids, "ids", torch.int32, (T,))
    _req(table, "table", torch.bfloat16)
    _req(out, "out", torch.float32, (T, H))
    _req(sink.weight, "sink.weight", torch.float32, (H,))
    if sink.resid.data_ptr() != out.data_ptr() or H % 8:
        raise KernelError("embedding_sink: the sink is over another residual stream, or the width is no multiple of 8")
    xn = torch.empty((T, H), dtype=torch.bfloat16, device=out.device)
    partials = torch.empty(((H + 127) // 128, T), dtype=torch.float32, device=out.device)
    check(lib().rlis_embedding_sink(ids.data_ptr(), table.data_ptr(), out.data_ptr(), sink.weight.data_ptr(),
                                    xn.data_ptr(), partials.data_ptr(), T, H, V,
                                    1.0 if scale is None else float(scale), _stream()), "embedding_sink")
    _count("embedding.sink")
    return ScaledRows(xn, partials, H, sink.eps)


def logit_transform(logits: torch.Tensor, scale: float | None, soft_cap: float | None) -> torch.Tensor:
    """In place on float32 logits [R, V]: x <- x * scale, then x <- cap * tanh(x / cap) (each only
    where given)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("logit_transform: logits must be float32 CUDA rows with unit stride")
    if soft_cap is not None and not soft_cap > 0:
        raise KernelError(f"logit_transform: the cap must be positive, got {soft_cap}")
    check(lib().rlis_logit_transform(logits.data_ptr(), R, V, logits.stride(0), 1.0 if scale is None else float(scale),
                                     0.0 if soft_cap is None else float(soft_cap), _stream()), "logit_transform")
    _count("logit_transform")
    return logits


def rmsnorm(resid: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
    """If `delta` is given: resid += delta (float32).  out = rmsnorm(resid) * weight, rounded once.

    resid float32 [T, H] (updated in place), weight float32 [H], out and delta in the activation
    type.  With `rows` (int32 [R]): out [R, H] is computed from rows resid[rows] (+ delta[rows])
    and resid is left unchanged."""
    T, H = resid.shape
    _req(resid, "resid", torch.float32)
    _req(weight, "weight", torch.float32, (H,))
    n_out = T
    if rows is not None:
        _req(rows, "rows", torch.int32, (None,))
        n_out = rows.shape[0]
    _req(out, "out", None, (n_out, H))
    if delta is not None:
        _req(delta, "delta", out.dtype, (T, H))
    check(lib().rlis_rmsnorm(resid.data_ptr(), delta.data_ptr() if delta is not None else None,
                             weight.data_ptr(), out.data_ptr(),
                             rows.data_ptr() if rows is not None else None, n_out, H, float(eps),
                             _code(out.dtype), _stream()), "rmsnorm")
    _count("rmsnorm" if rows is None else "rmsnorm.rows")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i; gate_up [T, 2I], out [T, I].  interleave 0: gate columns
    first, then up columns; B > 0: blocks of B gate columns each followed by their B up columns."""
    T, I2 = gate_up.shape
    if I2 % 2:
        raise KernelError(f"swiglu: the fused gate|up width must be even, got {I2}")
    _req(gate_up, "gate_up")
    _req(out, "out", gate_up.dtype, (T, I2 // 2))
    check(lib().rlis_swiglu(gate_up.data_ptr(), out.data_ptr(), T, I2 // 2, int(interleave),
                            _code(out.dtype), _stream()), "swiglu")
    _count("swiglu")
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FFMA, fixed order over K)."""
    M, K = a.shape
    N = w.shape[0]
    _req(a, "a", torch.float32)
    _req(w, "w", torch.float32, (N, K))
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _req(out, "out", torch.float32, (M, N))
    check(lib().rlis_gemm_f32_nt(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _stream()),
          "gemm_f32")
    _count("gemm_f32")
    return out


FUSE_NORMS = True          # debug switch "fuse_norms": 0 runs every norm as a kernel
STREAM_MAX_ROWS = 128     # what the weight-streaming kernel takes
DECODE_GEMM_ROWS = 16     # up to this many rows its sink epilogue works: the norms go into the products
STREAM_GEMM_ROWS = 16     # up to this many rows `linear` uses it; longer batches go to the library GEMM
                          # (debug switch "stream_rows"; measured in the decode step with 32 rows: at the 1B
                          # sizes, context 4096, 1.540 ms with it and 1.541 ms with the library; at the 8B
                          # sizes, two layers, context 8192, 0.863 against 0.770 ms; with 48 and 64 rows at
                          # the 1B sizes 1.976 and 2.369 ms against 1.894 and 2.226 ms)


class ScaledRows:
    """Rows of a norm's output whose scale is still to be applied: `x` = bf16(resid * weight) [T, dim]
    and `partials` float32 [P, T], the sums of resid^2 over P slices of the width.  The product that
    takes them multiplies its result by 1 / sqrt(sum of a row's partials / dim + eps): the norm
    between two decode products without a kernel of its own.  Made by `stream_gemm(..., sink=)`."""

    def __init__(self, x, partials, dim, eps):
        self.x, self.partials, self.dim, self.eps = x, partials, int(dim), float(eps)

    shape = property(lambda self: self.x.shape)
    dtype = property(lambda self: self.x.dtype)
    device = property(lambda self: self.x.device)


class ResidualSink:
    """Where the last product of a part may put its result itself: added to the float32 residual
    stream `resid` [T, dim] in place, and handed on as the ScaledRows of the RMSNorm that follows
    (`weight` float32 [dim], `eps`)."""

    def __init__(self, resid, weight, eps):
        self.resid, self.weight, self.eps = resid, weight, float(eps)


def stream_gemm(x, w: torch.Tensor, out_dtype=torch.bfloat16, swiglu4: bool = False, sink: ResidualSink | None = None):
    """y = x @ w^T for at most 128 rows of bfloat16 x: the decode step's weight-streaming product on
    the tcgen05 tensor cores (TMA-fed, weights as the M side, k split over CTAs).  `swiglu4`: w is a
    gate|up matrix interleaved in blocks of 4 rows and the result is silu(gate) * up, [M, N / 2].
    `x` may be ScaledRows: the rows' scale is applied to the result.  `sink` (up to 16 rows): the
    result, rounded to bfloat16, is added to sink.resid in place and the ScaledRows of the norm that
    follows are returned instead of y."""
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is not None:
        x = scaled.x
    M, K = x.shape
    N = w.shape[0]
    _req(x, "x", torch.bfloat16)
    _req(w, "w", torch.bfloat16, (N, K))
    if M > STREAM_MAX_ROWS or K % 8 or (swiglu4 and N % 8):
        raise KernelError(f"stream_gemm: takes up to {STREAM_MAX_ROWS} rows and K a multiple of 8, got M={M}, K={K}")
    if scaled is None and sink is None:
        out = torch.empty((M, N // 2 if swiglu4 else N), dtype=out_dtype, device=x.device)
        check(lib().rlis_stream_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _code(out_dtype),
                                          1 if swiglu4 else 0, _stream()), "stream_gemm")
        _count("stream_gemm.swiglu" if swiglu4 else "stream_gemm")
        return out
    in_p, n_p, dim, eps = 0, 0, 0, 0.0
    if scaled is not None:
        if sink is not None:
            raise KernelError("stream_gemm: scaled rows into a sink are not supported")
        n_p = scaled.partials.shape[0]
        _req(scaled.partials, "partials", torch.float32, (n_p, M))
        if scaled.dim != K:
            raise KernelError(f"stream_gemm: scaled rows of width {scaled.dim} for a product over {K}")
        in_p, dim, eps = scaled.partials.data_ptr(), scaled.dim, scaled.eps
    if sink is None:
        out = torch.empty((M, N // 2 if swiglu4 else N), dtype=out_dtype, device=x.device)
        check(lib().rlis_stream_gemm_fused(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _code(out_dtype),
                                           1 if swiglu4 else 0, in_p, n_p, dim, eps, 0, 0, 0, 0, _stream()),
              "stream_gemm")
        _count("stream_gemm.scaled.swiglu" if swiglu4 else "stream_gemm.scaled")
        return out
    if swiglu4 or M > DECODE_GEMM_ROWS:
        raise KernelError(f"stream_gemm: a sink takes a plain product of up to {DECODE_GEMM_ROWS} rows")
    _req(sink.resid, "sink.resid", torch.float32, (M, N))
    _req(sink.weight, "sink.weight", torch.float32, (N,))
    xn = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    partials = torch.empty(((N + 127) // 128, M), dtype=torch.float32, device=x.device)
    check(lib().rlis_stream_gemm_fused(x.data_ptr(), w.data_ptr(), 0, M, N, K, _code(torch.bfloat16), 2, 0, 0, 0, 0.0,
                                       sink.resid.data_ptr(), sink.weight.data_ptr(), xn.data_ptr(),
                                       partials.data_ptr(), _stream()), "stream_gemm")
    _count("stream_gemm.sink")
    return ScaledRows(xn, partials, N, sink.eps)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, epilogue: str = "plain") -> torch.Tensor:
    """y = x @ w^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory), bfloat16
    operands.  epilogue "plain": bf16 [M, N]; "float32": float32 [M, N]; "swiglu4": w is a gate|up
    matrix interleaved in blocks of 4 rows and the result is silu(gate) * up, bf16 [M, N / 2]."""
    M, K = x.shape
    N = w.shape[0]
    _req(x, "x", torch.bfloat16)
    _req(w, "w", torch.bfloat16, (N, K))
    code = {"plain": 0, "swiglu4": 1, "float32": 2}[epilogue]
    if M < 128 or N < 256 or K % 8 or N % (16 if code == 1 else 8):
        raise KernelError(f"gemm_tcgen05: takes M >= 128, N >= 256, K a multiple of 8 and N a multiple of 8 "
                          f"(16 with the SwiGLU epilogue); got M={M}, N={N}, K={K}")
    out = torch.empty((M, N // 2 if code == 1 else N), dtype=torch.float32 if code == 2 else torch.bfloat16,
                      device=x.device)
    check(lib().rlis_gemm_tcgen05(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, code, _stream()),
          "gemm_tcgen05")
    _count("gemm_tcgen05." + epilogue)
    return out


def take_device_errors(out: torch.Tensor) -> torch.Tensor:
    """Reads and clears, in stream order, the error words of the kernels' bounded waits and leaves
    their union in `out` (int32 [1] on the device): non-zero when a wait ran out in a kernel launched
    before this call and after the last one.  No synchronisation; copy `out` to the host with
    whatever else the step brings back."""
    _req(out, "out", torch.int32, (1,))
    check(lib().rlis_take_errors(out.data_ptr(), _stream()), "take_errors")
    _count("take_errors")
    return out


def stream_timeline(on: bool) -> None:
    """Switches the streaming products' timeline on or off (and empties it): the first CTA of every
    launch stamps the device's global timer at its phases.  A measurement tool; synchronises.  Only in
    a library built with it: set RLIS_TIMELINE=1 in the environment before the first use."""
    torch.cuda.synchronize()
    check(lib().rlis_stream_gemm_timeline(1 if on else 0), "stream_timeline")


def read_stream_timeline(last: int) -> list:
    """The last `last` launches of the streaming product (oldest first), each a dict with N, K and,
    in nanoseconds of the global timer: start, wait_passed (the kernel before has finished),
    products_done, cluster_barrier, sent, sums_arrived (the last three None for a launch that does
    not split k), end, and grid_before_done: the latest end of any CTA of the streaming product launched
    before this one (meaningful when that product is the kernel right before)."""
    import ctypes
    torch.cuda.synchronize()
    buf = (ctypes.c_ulonglong * (512 * 10))()
    n = ctypes.c_uint(0)
    check(lib().rlis_stream_gemm_timeline_read(buf, ctypes.byref(n)), "stream_timeline_read")
    count = min(int(last), n.value, 512)
    out = []
    for i in range(n.value - count, n.value):
        r = buf[(i % 512) * 10:(i % 512) * 10 + 10]
        split = r[3] >= r[2] and r[3] <= r[7]          # records of launches without a split keep stale stamps there
        out.append({"N": int(r[6] // 100000), "K": int(r[6] % 100000), "start": int(r[0]), "wait_passed": int(r[1]),
                    "products_done": int(r[2]), "cluster_barrier": int(r[3]) if split else None,
                    "sent": int(r[4]) if split else None, "sums_arrived": int(r[5]) if split else None,
                    "end": int(r[7]), "grid_before_done": int(r[8])})
    return out


def check_device_errors() -> None:
    """Raises if a bounded wait inside a kernel ever ran out on this device (the kernel then
    finished without its data; results since are not to be trusted).  Synchronises the device."""
    code = (lib().rlis_gemm_tcgen05_error() or lib().rlis_stream_gemm_error() or lib().rlis_attention_prefill_tc_error()
            or lib().rlis_attention_decode_error())
    if code != 0:
        raise KernelError(f"a bounded mbarrier wait of a tcgen05 kernel ran out on the device (code {code})")


def fuses_norms(n_rows: int, dtype, *widths: int) -> bool:
    """Whether products over `widths` of a step of `n_rows` rows go to the kernel that takes
    ScaledRows and a ResidualSink."""
    return (FUSE_NORMS and dtype == torch.bfloat16 and 0 < n_rows <= DECODE_GEMM_ROWS
            and all(w % 8 == 0 for w in widths))


def linear(x, w: torch.Tensor, out_dtype=None, sink: ResidualSink | None = None):
    """y = x @ w^T for w stored (out, in).  float32: this package's FFMA kernel.  bfloat16: up to
    16 rows go to this package's weight-streaming tcgen05 kernel, more to the library GEMM; both
    accumulate in float32, and `out_dtype=torch.float32` keeps that precision (used for logits).
    ScaledRows as x and a `sink` are for the streaming kernel only (see `fuses_norms`)."""
    if isinstance(x, ScaledRows) or sink is not None:
        if not fuses_norms(x.shape[0], x.dtype, x.shape[1]):
            raise KernelError("linear: scaled rows or a sink with a product that does not take them")
        return stream_gemm(x, w, out_dtype or torch.bfloat16, sink=sink)
    if x.dtype == torch.float32:
        return gemm_f32(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: expected matching float32 or bfloat16 operands, got {x.dtype}, {w.dtype}")
    if not x.is_cuda:
        raise KernelError("linear: expected CUDA tensors; there is no CPU path")
    if x.shape[1] % 8 == 0 and x.is_contiguous() and (
            x.shape[0] <= STREAM_GEMM_ROWS or (x.shape[0] <= STREAM_MAX_ROWS and w.shape[0] >= 256 * num_sms())):
        # few rows, or up to 128 rows over a matrix so tall that the streaming kernel does not split k
        # (two tiles of 128 features an SM and more: an LM head).  Measured at 128256 x 2048: 48 rows
        # 88 against 97 us for the library, 64 rows 91 against 99, 128 rows 104 against 111; at 17 to
        # 32 rows the two are within 1 us.
        return stream_gemm(x, w, out_dtype or torch.bfloat16)
    if out_dtype is None or out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
               v_cache: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor | None,
               inv_freq: torch.Tensor | None, n_heads: int, n_kv_heads: int, head_dim: int,
               page_size: int) -> torch.Tensor:
    """Rotates q and k by their positions and stores k, v at `slots` of one layer's paged cache.

    qkv [T, (nh + 2 nkv) d]; q_out [T, nh d]; caches [pages, nkv, page_size, d]; positions and
    slots int32 [T] (slots None: nothing is stored); inv_freq float32 [d/2] (None: no rotation)."""
    T = qkv.shape[0]
    _req(qkv, "qkv", None, (T, (n_heads + 2 * n_kv_heads) * head_dim))
    _req(q_out, "q_out", qkv.dtype, (T, n_heads * head_dim))
    _req(positions, "positions", torch.int32, (T,))
    if slots is not None:
        _req(slots, "slots", torch.int32, (T,))
        for c, nm in ((k_cache, "k_cache"), (v_cache, "v_cache")):
            _req(c, nm, qkv.dtype, (None, n_kv_heads, page_size, head_dim))
    if inv_freq is not None:
        _req(inv_freq, "inv_freq", torch.float32, (head_dim // 2,))
    check(lib().rlis_rope_cache(
        qkv.data_ptr(), q_out.data_ptr(),
        k_cache.data_ptr() if slots is not None else None,
        v_cache.data_ptr() if slots is not None else None,
        positions.data_ptr(), slots.data_ptr() if slots is not None else None,
        inv_freq.data_ptr() if inv_freq is not None else None,
        T, n_heads, n_kv_heads, head_dim, page_size, _code(qkv.dtype), _stream()), "rope_cache")
    _count("rope_cache")
    return q_out


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      out: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                      block_tables: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      page_size: int, scale: float, window: int = 0,
                      token_rows: torch.Tensor | None = None) -> torch.Tensor:
    """Causal grouped-query attention over paged keys and values for any mix of query lengths.

    q, out [T, nh d]; caches [pages, nkv, page_size, d]; seq_of_token, positions int32 [T];
    block_tables int32 [B, max_blocks].  window 0 = all earlier keys.  `token_rows` (int32):
    compute these rows of the step only."""
    T = q.shape[0]
    _req(q, "q", None, (T, n_heads * head_dim))
    _req(out, "out", q.dtype, (T, n_heads * head_dim))
    _req(k_cache, "k_cache", q.dtype, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", q.dtype, (None, n_kv_heads, page_size, head_dim))
    _req(seq_of_token, "seq_of_token", torch.int32, (T,))
    _req(positions, "positions", torch.int32, (T,))
    _req(block_tables, "block_tables", torch.int32, (None, None))
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head sizes are multiples of 16 up to 256, got {head_dim}")
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
    check(lib().rlis_attention_generic(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        seq_of_token.data_ptr(), positions.data_ptr(), block_tables.data_ptr(),
        token_rows.data_ptr() if token_rows is not None else None,
        block_tables.shape[1], T if token_rows is None else token_rows.shape[0], n_heads,
        n_kv_heads, head_dim, page_size, float(scale), int(window), _code(q.dtype), _stream()),
        "attention_generic")
    _count("attention_generic")
    return out


DECODE_MIN_KEYS_PER_SPLIT = 128


@functools.lru_cache(maxsize=None)
def num_sms() -> int:
    """Streaming multiprocessors of the current device (what the launchers ask the runtime for)."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device; there is no CPU path")
    return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)


def decode_splits(n_decode: int, n_kv_heads: int, max_ctx: int, sms: int | None = None) -> int:
    """How many pieces the context is cut into for decode attention on a device of `sms`
    multiprocessors (None: the current device); see `_decode_splits`."""
    return _decode_splits(n_decode, n_kv_heads, max_ctx, num_sms() if sms is None else int(sms))


@functools.lru_cache(maxsize=4096)
def _decode_splits(n_decode: int, n_kv_heads: int, max_ctx: int, sms: int) -> int:
    """Role of `split_plan`, crates/model/src/paged_attention.rs:21-36, re-tuned by measurement
    (on 148 multiprocessors, which the numbers below are for).  Few requests:
    enough CTAs (kv heads x requests x pieces) to fill the SMs about twice, each piece at least
    128 keys long.  From 64 (request, kv head) pairs on, pieces of at least 512 keys and no more
    than about 384 CTAs; from 256 pairs on, one piece at every context: the pairs fill the SMs by
    themselves, and cutting only adds the merge (batch 32, context 2048: 22.6 us whole, 33.8 us
    in 4 pieces; batch 64, context 4096: 82.5 against 95.9 us).  Up to 8 pieces of a small grid are
    merged inside a thread-block cluster, and clusters of 2, 4 and 8 are the sizes that schedule
    well (batch 8, context 4096: 17.4 us with 4 pieces, 29.2 with 5)."""
    groups = max(1, n_decode * n_kv_heads)
    cluster_max_ctas = 4 * sms     # larger grids merge their pieces through global memory instead
    want = -(-2 * sms // groups)
    min_keys = DECODE_MIN_KEYS_PER_SPLIT
    if groups >= 64:
        want = min(want, max(1, 384 // groups))
        min_keys = 512
    want = max(1, min(want, max_ctx // min_keys, 32))
    if want > 1 and groups * min(want, 8) <= cluster_max_ctas:
        # merged inside a cluster: 2, 4 or 8 pieces; with few requests 8, until a piece gets long
        # (batch 1, context 4096: 6.7 us with 8 pieces in a cluster, 12.6 us with 32 and tickets)
        pieces = 1 << (min(want, 8).bit_length() - 1)
        while 8 <= pieces < 32 and want >= 2 * pieces and max_ctx // pieces > 1536:
            pieces *= 2
        want = pieces
    return want


def attention_decode(q, k_cache, v_cache, out, dec_rows, dec_seqs, ctx_lens, block_tables,
                     n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: int, splits: int, scratch: torch.Tensor | None) -> torch.Tensor:
    """Attention of single decoded tokens (bfloat16): request i's token sits in row dec_rows[i] of
    q/out and belongs to batch entry dec_seqs[i]; it sees keys 0 .. ctx_lens[seq]-1.  `scratch`:
    float32, at least n_decode * n_heads * splits * (d + 2) elements when splits > 1."""
    n = dec_rows.shape[0]
    _req(q, "q", torch.bfloat16, (None, n_heads * head_dim))
    _req(out, "out", torch.bfloat16, tuple(q.shape))
    _req(k_cache, "k_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    for t, nm in ((dec_rows, "dec_rows"), (dec_seqs, "dec_seqs"), (ctx_lens, "ctx_lens")):
        _req(t, nm, torch.int32, (None,))
    _req(block_tables, "block_tables", torch.int32, (None, None))
    if head_dim % 8 or head_dim > 256 or n_heads % n_kv_heads or n_heads // n_kv_heads > 8:
        raise KernelError(f"decode attention: head size {head_dim} / group of {n_heads // max(1, n_kv_heads)} "
                          "heads is not taken (multiples of 8 up to 256, groups up to 8)")
    if splits > 1:
        need = n * n_heads * splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"decode attention: scratch of {need} float32 elements is needed")
    check(lib().rlis_attention_decode_pages(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        scratch.data_ptr() if splits > 1 else None, dec_rows.data_ptr(), dec_seqs.data_ptr(),
        ctx_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n, n_heads,
        n_kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), int(splits),
        _code(q.dtype), _stream()), "attention_decode")
    _count("attention_decode" + _decode_variant())
    return out


def decode_attention_takes_qkv(dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether `attention_decode_from_qkv` exists for these sizes (the tensor-core decode kernel)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv_heads == 0
            and n_heads // n_kv_heads <= 8)


def attention_decode_from_qkv(qkv, k_cache, v_cache, out, step, group: int, inv_freq, store: bool,
                              n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                              scale: float, window: int = 0) -> torch.Tensor:
    """Decode attention of a step of single tokens straight from the q|k|v projection
    [T, (nh + 2 nkv) d]: rotates q and each request's newest key (`inv_freq` float32 [d / 2], None:
    no rotation) inside the attention kernel, which also stores the newest key and value at the
    step's slots (`store` False: the layer reads another layer's cache)."""
    T = qkv.shape[0]
    n = step.n_decode
    _req(qkv, "qkv", torch.bfloat16, (T, (n_heads + 2 * n_kv_heads) * head_dim))
    _req(out, "out", torch.bfloat16, (T, n_heads * head_dim))
    _req(k_cache, "k_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    if not decode_attention_takes_qkv(qkv.dtype, n_heads, n_kv_heads, head_dim):
        raise KernelError(f"decode attention from q|k|v: head size {head_dim} / {n_heads}:{n_kv_heads} heads is not taken")
    if inv_freq is not None:
        _req(inv_freq, "inv_freq", torch.float32, (head_dim // 2,))
    slots = step.slots[group] if store else None
    tables = step.block_tables[group]
    splits = decode_splits(n, n_kv_heads, step.max_decode_ctx)
    scratch = None
    if splits > 1:
        scratch = step.buffer("attn_partial", (n * n_heads * splits * (head_dim + 2),), torch.float32)
    check(lib().rlis_attention_decode_qkv(
        qkv.data_ptr(), step.positions.data_ptr(), slots.data_ptr() if slots is not None else None,
        inv_freq.data_ptr() if inv_freq is not None else None, k_cache.data_ptr(), v_cache.data_ptr(),
        out.data_ptr(), scratch.data_ptr() if splits > 1 else None, step.dec_rows.data_ptr(),
        step.dec_seqs.data_ptr(), step.ctx_lens.data_ptr(), tables.data_ptr(), tables.shape[1], n, n_heads,
        n_kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), int(splits),
        _code(qkv.dtype), _stream()),
        "attention_decode_qkv")
    _count("attention_decode_qkv" + _decode_variant())
    return out


@functools.lru_cache(maxsize=None)
def prefill_tile() -> int:
    """Tokens of a portion that one CTA of the flash kernels for prompt portions takes; the step's
    tile list (`attention_prefill`'s `tiles`) is cut to this size."""
    return int(lib().rlis_attention_prefill_tile())


PREFILL_TCGEN05 = True     # debug switch "prefill_tcgen05": 0 takes the mma.sync kernel for every size


def _set_flag(name):
    def setter(value):
        globals()[name] = bool(value)
    return setter


def _set_stream_rows(value):
    global STREAM_GEMM_ROWS
    STREAM_GEMM_ROWS = max(DECODE_GEMM_ROWS, min(int(value), STREAM_MAX_ROWS))


library.PYTHON_SWITCHES.update(fuse_norms=_set_flag("FUSE_NORMS"), prefill_tcgen05=_set_flag("PREFILL_TCGEN05"),
                               stream_rows=_set_stream_rows)


def attention_prefill(q, k_cache, v_cache, out, tiles, cu_seqlens, ctx_lens, block_tables,
                      n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: int = 0, max_ctx: int = 0) -> torch.Tensor:
    """Causal flash attention of portions of prompts over the paged cache (bfloat16, head sizes 64
    and 128).  tiles int32 [n, 2] = (batch entry, first token of the tile within the entry's
    portion; a tile is `prefill_tile()` tokens); cu_seqlens int32 [B + 1] = rows of the entries' first tokens.  max_ctx: the
    longest context of the step if known (with few tiles and long contexts several CTAs then
    share a tile's keys)."""
    _req(q, "q", torch.bfloat16, (None, n_heads * head_dim))
    _req(out, "out", torch.bfloat16, tuple(q.shape))
    _req(k_cache, "k_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(v_cache, "v_cache", torch.bfloat16, (None, n_kv_heads, page_size, head_dim))
    _req(tiles, "tiles", torch.int32, (None, 2))
    _req(cu_seqlens, "cu_seqlens", torch.int32, (None,))
    _req(ctx_lens, "ctx_lens", torch.int32, (None,))
    _req(block_tables, "block_tables", torch.int32, (None, None))
    if head_dim not in (64, 128) or n_heads % n_kv_heads:
        raise KernelError(f"prefill attention: head size {head_dim} is not taken (64 and 128 are)")
    if PREFILL_TCGEN05 and lib().rlis_attention_prefill_tc_takes(n_heads, n_kv_heads, head_dim, page_size):
        # the tcgen05 kernel: head sizes 64 and 128, two or more query heads a kv head, pages that divide a block of keys
        check(lib().rlis_attention_prefill_tc(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), tiles.data_ptr(),
            tiles.shape[0], cu_seqlens.data_ptr(), ctx_lens.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], q.shape[0], k_cache.shape[0], n_heads, n_kv_heads, head_dim, page_size,
            float(scale), int(window), _code(q.dtype), int(max_ctx), _stream()), "attention_prefill_tc")
        _count("attention_prefill.tcgen05")
        return out
    check(lib().rlis_attention_prefill(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), tiles.data_ptr(),
        tiles.shape[0], cu_seqlens.data_ptr(), ctx_lens.data_ptr(), block_tables.data_ptr(),
        block_tables.shape[1], n_heads, n_kv_heads, head_dim, page_size, float(scale), int(window),
        _code(q.dtype), _stream()), "attention_prefill")
    _count("attention_prefill.mma")
    return out


def attention(q, k_cache, v_cache, out, step, group: int, n_heads: int, n_kv_heads: int,
              head_dim: int, page_size: int, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of every token of the step over its request's cached keys, by the kernels that
    fit the step.  bfloat16: single decoded tokens go to the split decode kernel, portions of
    prompts to the flash kernel (head sizes 64 and 128); everything else, and all of float32, to
    the kernel for any query length.  The choice never changes the result beyond rounding."""
    tables = step.block_tables[group]
    bf = q.dtype == torch.bfloat16
    dec_fast = bf and step.n_decode > 0 and n_heads // n_kv_heads <= 8 and head_dim % 8 == 0
    pf_fast = bf and step.n_prefill_tiles > 0 and head_dim in (64, 128)
    if dec_fast:
        splits = decode_splits(step.n_decode, n_kv_heads, step.max_decode_ctx)
        scratch = None
        if splits > 1:
            scratch = step.buffer("attn_partial", (step.n_decode * n_heads * splits * (head_dim + 2),), torch.float32)
        attention_decode(q, k_cache, v_cache, out, step.dec_rows, step.dec_seqs, step.ctx_lens, tables,
                         n_heads, n_kv_heads, head_dim, page_size, scale, window, splits, scratch)
    if pf_fast:
        attention_prefill(q, k_cache, v_cache, out, step.prefill_tiles, step.cu_seqlens, step.ctx_lens,
                          tables, n_heads, n_kv_heads, head_dim, page_size, scale, window,
                          getattr(step, "max_ctx_len", 0))
    if dec_fast and pf_fast:
        return out
    if not dec_fast and not pf_fast:
        rows = None                                   # every token of the step
    elif dec_fast:
        if step.n_prefill_tokens == 0:
            return out
        rows = step.prefill_rows                      # the portions only
    else:
        if step.n_decode == 0:
            return out
        rows = step.dec_rows                          # the single tokens only
    return attention_generic(q, k_cache, v_cache, out, step.seq_of_token, step.positions, tables,
                             n_heads, n_kv_heads, head_dim, page_size, scale, window, token_rows=rows)


def sample_rows(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of float32 logits [R, V].  params int32 [R, 2] = (key, bits of 1/T);
    (0, 0) is greedy.  Returns int32 [R]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("sample_rows: logits must be float32 CUDA rows with unit stride")
    _req(params, "params", torch.int32, (R, 2))
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _req(out, "out", torch.int32, (R,))
    check(lib().rlis_sample_rows(logits.data_ptr(), params.data_ptr(), out.data_ptr(), R, V,
                                 logits.stride(0), _stream()), "sample_rows")
    _count("sample_rows")
    return out


def repetition_penalty(logits: torch.Tensor, rows: torch.Tensor, history: torch.Tensor, offsets: torch.Tensor,
                       penalties: torch.Tensor) -> torch.Tensor:
    """In place on float32 logits [R, V]: for row rows[i], every distinct token of
    history[offsets[i]:offsets[i + 1]] has its logit divided by penalties[i] if positive, multiplied
    otherwise (once, however often the token occurs)."""
    R, V = logits.shape
    n = rows.shape[0]
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("repetition_penalty: logits must be float32 CUDA rows with unit stride")
    _req(rows, "rows", torch.int32, (n,))
    _req(history, "history", torch.int32, (None,))
    _req(offsets, "offsets", torch.int32, (n + 1,))
    _req(penalties, "penalties", torch.float32, (n,))
    check(lib().rlis_repetition_penalty(logits.data_ptr(), rows.data_ptr(), history.data_ptr(), offsets.data_ptr(),
                                        penalties.data_ptr(), n, V, logits.stride(0), _stream()), "repetition_penalty")
    _count("repetition_penalty")
    return logits


def sample_filtered(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of float32 logits [R, V] by temperature sampling with top-k and/or
    top-p filtering on the device.  params int32 [R, 5] = (bits of 1/T, top_k (0: off), bits of
    top_p, low word, high word of a 53-bit uniform).  Returns int32 [R]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("sample_filtered: logits must be float32 CUDA rows with unit stride")
    _req(params, "params", torch.int32, (R, 5))
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _req(out, "out", torch.int32, (R,))
    check(lib().rlis_sample_filtered(logits.data_ptr(), params.data_ptr(), out.data_ptr(), R, V,
                                     logits.stride(0), _stream()), "sample_filtered")
    _count("sample_filtered")
    return out


def nll_rows(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Negative log-likelihood of targets[r] under softmax(logits[r]); float32 [R]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise KernelError("nll_rows: logits must be float32 CUDA rows with unit stride")
    _req(targets, "targets", torch.int32, (R,))
    out = torch.empty((R,), dtype=torch.float32, device=logits.device)
    check(lib().rlis_nll_rows(logits.data_ptr(), targets.data_ptr(), out.data_ptr(), R, V,
                              logits.stride(0), _stream()), "nll_rows")
    _count("nll_rows")
    return out
