"""Python face of the CUDA kernels: torch tensors in, a launch on the current stream out.

There is no CPU or library fallback here: every function launches a kernel of ``csrc/``
and raises :class:`KernelError` if the library is missing, the tensors are not on a CUDA
device, or a size is outside what the kernel takes.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build


class KernelError(RuntimeError):
    pass


F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, not {dtype}") from None


def _ptr(t: torch.Tensor | None):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(
            "a tensor on the CPU reached a CUDA kernel: this engine has no CPU path"
        )
    return c_void_p(t.data_ptr())


_scoped_stream = None


def _stream():
    if _scoped_stream is not None:
        return _scoped_stream
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks the current CUDA stream up once for every launch made inside the ``with`` block (the
    look-up costs a third of a launch's host time).  The stream must not be switched inside."""

    def __enter__(self):
        global _scoped_stream
        self.prev = _scoped_stream
        _scoped_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self.prev


launches = 0   # kernels launched through this module (a captured graph counts its launches once)


def _check(lib, code: int, what: str):
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: {lib.mhb_last_error().decode()}")


def _contig(t: torch.Tensor, name: str):
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------------------
def embed(table, tokens, out, status=None, scale: float = 1.0, copy=None):
    """out[t] = table[tokens[t]] * scale as float32; ids outside the table give zeros and set status
    bit 0.  ``copy`` (bfloat16 [T, H]): the same rows once more, rounded, for a block whose products
    read the stream itself."""
    lib = build.load("elementwise")
    T, H = out.shape
    if scale == 1.0 and copy is None:
        _check(lib, lib.mhb_embed(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(tokens), _ptr(out),
                                  c_int(T), c_int(H), c_int(table.shape[0]), _ptr(status), _stream()),
               "embed")
        return
    if copy is not None and (copy.dtype != torch.bfloat16 or tuple(copy.shape) != (T, H) or not copy.is_contiguous()):
        raise KernelError("embed: the copy must be a contiguous bfloat16 matrix of the output's shape")
    _check(lib, lib.mhb_embed_scaled(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(tokens), _ptr(out),
                                     c_int(T), c_int(H), c_int(table.shape[0]), _ptr(status), c_float(scale),
                                     _ptr(copy), _stream()), "embed")


def norm_mix(x, weight, eps, *, delta=None, nsplit=1, split_stride=0, alpha=1.0, keep=0.0, copy=None):
    """x <- keep * x + rms(alpha * x + delta) * weight, row by row in float32, in place; ``copy`` (compute
    dtype, same shape) receives the new rows too.  alpha = 0 leaves x out of the norm (a normalised branch
    that is ADDED to the stream: keep = 1); keep = 0 replaces the stream by the norm (a post-norm block).
    ``delta`` may be ``nsplit`` float32 partial matrices ``split_stride`` elements apart."""
    lib = build.load("postnorm")
    R, H = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("norm_mix: the stream must be a contiguous float32 matrix")
    if delta is None and alpha == 0.0:
        raise KernelError("norm_mix: nothing to normalise")
    ddt = dtype_code(delta.dtype) if delta is not None else F32
    cdt = dtype_code(copy.dtype) if copy is not None else F32
    _check(lib, lib.mhb_norm_mix(_ptr(x), _ptr(delta), c_int(ddt), c_int(nsplit), c_longlong(split_stride),
                                 _ptr(weight), c_float(eps), c_float(alpha), c_float(keep), _ptr(copy), c_int(cdt),
                                 c_int(R), c_int(H), _stream()), "norm_mix")


ACTIVATIONS = {"relu2": 0, "silu": 1, "gelu_tanh": 2, "copy": 3}
GLU_ACTS = {"silu": 0, "gelu_tanh": 1}          # activations of a gated feed-forward's gate


def act_rows(z, out, act: str, nsplit=1, split_stride=0):
    """out = act(z) element by element in float32; z may be split-K parts.  act: relu2 (the square of
    relu), silu, gelu_tanh, copy (a conversion only)."""
    lib = build.load("postnorm")
    if act not in ACTIVATIONS:
        raise KernelError(f"act_rows: unknown activation {act!r}; known: {sorted(ACTIVATIONS)}")
    _check(lib, lib.mhb_act_rows(_ptr(z), c_int(dtype_code(z.dtype)), c_int(nsplit), c_longlong(split_stride),
                                 _ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
                                 c_int(ACTIVATIONS[act]), _stream()), "act_rows")


def table_gate(z, table, column0, tokens, out, nsplit=1, split_stride=0, status=None):
    """out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], column0 + j]."""
    lib = build.load("postnorm")
    T, D = out.shape
    if not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("table_gate: table and output must be contiguous")
    _check(lib, lib.mhb_table_gate(_ptr(z), c_int(dtype_code(z.dtype)), c_int(nsplit), c_longlong(split_stride),
                                   _ptr(table), c_int(dtype_code(table.dtype)), c_int(table.shape[1]),
                                   c_int(column0), c_int(table.shape[0]), _ptr(tokens), _ptr(out),
                                   c_int(dtype_code(out.dtype)), c_int(T), c_int(D), _ptr(status), _stream()),
           "table_gate")


def _gate_args(gate, gate_nsplit, gate_split_stride):
    """(pointer, parts, stride between parts, row stride) of a gate that is a run of columns of a float32 product."""
    if gate is None:
        return c_void_p(0), c_int(1), c_longlong(0), c_int(0)
    if gate.dtype != torch.float32 or gate.stride(-1) != 1:
        raise KernelError("a gate must be float32 columns of a product")
    return _ptr(gate), c_int(gate_nsplit), c_longlong(gate_split_stride), c_int(gate.stride(-2))


def gated_rmsnorm(o, weight, eps, out, gate=None, gate_nsplit=1, gate_split_stride=0):
    """out = rms(o) * weight * sigmoid(gate): o float32 [R, N]; ``gate`` [R, N] is a view of columns of
    a float32 product (its parts ``gate_split_stride`` elements apart)."""
    lib = build.load("postnorm")
    R, N = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or not out.is_contiguous():
        raise KernelError("gated_rmsnorm: o must be contiguous float32, out contiguous")
    g = _gate_args(gate, gate_nsplit, gate_split_stride)
    _check(lib, lib.mhb_gated_rmsnorm(_ptr(o), g[0], g[1], g[2], g[3], _ptr(weight), c_float(eps), _ptr(out),
                                      c_int(dtype_code(out.dtype)), c_int(R), c_int(N), _stream()), "gated_rmsnorm")


def qknorm_rope_append(qkv, q_weight, k_weight, eps, positions, tok_seg, block_table, inv_freq, rotary_dim, q_out,
                       cache, *, nq, nkv, dk, dv, page_size, has_kv=True, nsplit=1, split_stride=0, status=None,
                       per_head=False, v_eps=0.0, page_extra=0):
    """RMS norm over the whole q projection and over the whole k projection, rotation of the first
    ``rotary_dim`` elements of every head (pairs (i, i + rotary_dim/2)), q to ``q_out`` [T, nq dk], k and v
    into the pages of ``cache`` (one layer's pool; a page holds [nkv][P][dk] keys then [nkv][P][dv] values).
    ``qkv`` float32 [.., T, ld] holds [q | k | v | ...] per row; with ``has_kv`` False it holds [q | ...]
    and nothing is appended.  ``per_head``: the norms run over each head alone with weights [dk] shared by the
    heads.  ``v_eps`` > 0: every head's value is divided by its root mean square before it is stored.
    ``page_extra``: elements of a page behind its keys and values, which this kernel leaves alone."""
    lib = build.load("postnorm")
    T = q_out.shape[0]
    if qkv.dtype != torch.float32 or qkv.stride(-1) != 1:
        raise KernelError("qknorm_rope_append: the product must be float32 with contiguous rows")
    if has_kv and (cache is None or cache.dtype != q_out.dtype or not cache.is_contiguous()):
        raise KernelError("qknorm_rope_append: the pool must be contiguous and of the activations' dtype")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError(f"qknorm_rope_append: {rotary_dim} rotated elements need {rotary_dim // 2} frequencies")
    _check(lib, lib.mhb_qknorm_rope_append_opts(
        _ptr(qkv), c_int(nsplit), c_longlong(split_stride), c_int(qkv.stride(-2)), _ptr(q_weight), _ptr(k_weight),
        c_float(eps), _ptr(positions), _ptr(tok_seg), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(inv_freq), c_int(rotary_dim), _ptr(q_out), _ptr(cache if has_kv else None), c_int(dtype_code(q_out.dtype)),
        c_int(T), c_int(nq), c_int(nkv), c_int(dk), c_int(dv), c_int(page_size),
        c_int(cache.shape[0] if has_kv else 0), c_int(1 if has_kv else 0), _ptr(status), c_int(1 if per_head else 0),
        c_float(v_eps or 0.0), c_longlong(page_extra), _stream()),
        "qknorm_rope_append")


def _lightning_head(proj, q0, k0, v0, decay, state, out, ctx_arrays, H, dk, dv, nsplit, split_stride, writable):
    tok_seg, seg_slot, positions = ctx_arrays
    if proj.dtype != torch.float32 or proj.stride(-1) != 1 or state.dtype != torch.float32 or out.dtype != torch.float32:
        raise KernelError("lightning: the product, the state and the output are float32")
    if not state.is_contiguous() or not out.is_contiguous() or tuple(state.shape[1:]) != (H, dk, dv):
        raise KernelError(f"lightning: the state must be contiguous [slots, {H}, {dk}, {dv}]")
    return (_ptr(proj), c_int(nsplit), c_longlong(split_stride), c_int(proj.stride(-2)), c_int(q0), c_int(k0),
            c_int(v0), _ptr(decay), _ptr(state), _ptr(out), _ptr(tok_seg), _ptr(seg_slot), _ptr(positions))


def lightning_scan(proj, q0, k0, v0, decay, state, out, tok_seg, seg_slot, positions, *, heads, dk, dv, nsplit=1,
                   split_stride=0, writable=True, max_tokens=0):
    """Linear attention with decay, token by token, for every segment of at most ``max_tokens`` tokens
    (0: all).  ``proj`` float32 [.., T, ld] holds silu's inputs: q at column q0, k at k0, v at v0, heads
    side by side; ``state`` [slots, heads, dk, dv]; ``out`` float32 [T, heads * dv]."""
    lib = build.load("lightning")
    T, S = out.shape[0], seg_slot.shape[0]
    head = _lightning_head(proj, q0, k0, v0, decay, state, out, (tok_seg, seg_slot, positions), heads, dk, dv,
                           nsplit, split_stride, writable)
    _check(lib, lib.mhb_lightning_scan(*head, c_int(T), c_int(S), c_int(heads), c_int(dk), c_int(dv),
                                       c_int(1 if writable else 0), c_int(max_tokens), _stream()), "lightning_scan")


def lightning_chunk_smem(dk: int, dv: int, chunk: int) -> int:
    """Shared memory the chunked route needs for chunks of ``chunk`` tokens."""
    lib = build.load("lightning")
    lib.mhb_lightning_chunk_smem.restype = c_longlong
    return int(lib.mhb_lightning_chunk_smem(c_int(dk), c_int(dv), c_int(chunk)))


def lightning_chunked(proj, q0, k0, v0, decay, state, out, tok_seg, seg_slot, positions, chunks, num_chunks,
                      seg_chunks, num_segs, scratch, chunk, *, heads, dk, dv, nsplit=1, split_stride=0, writable=True):
    """The same for the listed segments, cut into the listed chunks of at most ``chunk`` tokens (4 ints
    each: see csrc/lightning.cu); ``scratch`` float32 holds num_chunks * heads * dk * dv."""
    lib = build.load("lightning")
    T = out.shape[0]
    if scratch.dtype != torch.float32 or scratch.numel() < num_chunks * heads * dk * dv:
        raise KernelError("lightning_chunked: the scratch is too small")
    head = _lightning_head(proj, q0, k0, v0, decay, state, out, (tok_seg, seg_slot, positions), heads, dk, dv,
                           nsplit, split_stride, writable)
    _check(lib, lib.mhb_lightning_chunked(*head, c_int(T), c_int(heads), c_int(dk), c_int(dv),
                                          c_int(1 if writable else 0), _ptr(chunks), c_int(num_chunks),
                                          _ptr(seg_chunks), c_int(num_segs), _ptr(scratch), c_int(chunk), _stream()),
           "lightning_chunked")


def add_rmsnorm(x, weight, eps, out, delta=None, nsplit=1, split_stride=0, rows=None):
    """out[r] = rmsnorm(x[s] + delta[s]) * weight with s = rows[r] if rows is given else r.

    Without ``rows`` and with ``delta`` the sum is written back to ``x`` (the residual).
    ``delta`` may be ``nsplit`` float32 partial matrices ``split_stride`` elements apart.
    """
    lib = build.load("elementwise")
    R, H = out.shape
    ddt = dtype_code(delta.dtype) if delta is not None else F32
    _check(lib, lib.mhb_add_rmsnorm(_ptr(x), _ptr(delta), c_int(ddt), c_int(nsplit),
                                    c_longlong(split_stride), _ptr(weight), c_float(eps),
                                    _ptr(rows), _ptr(out), c_int(dtype_code(out.dtype)),
                                    c_int(R), c_int(H), _stream()), "add_rmsnorm")


def residual_add(x, delta, nsplit=1, split_stride=0):
    lib = build.load("elementwise")
    _check(lib, lib.mhb_residual_add(_ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype)),
                                     c_int(nsplit), c_longlong(split_stride),
                                     c_longlong(x.numel()), _stream()), "residual_add")


def rope_append(qkv, bias, positions, tok_seg, block_table, inv_freq, q_out, cache, *, nq, nkv, d,
                page_size, write_kv=True, rotary_dim=None, interleaved=False, nsplit=1, split_stride=0,
                status=None):
    """Bias + rotary encoding of q and k, q to ``q_out``, k and v into the cache pages.

    ``cache`` is one layer's pool [pages, 2, nkv, page_size, d]; ``block_table`` [S, width]
    holds the page ids of each segment of the batch, ``tok_seg`` [T] the segment of a token.
    ``rotary_dim``: how many leading elements of a head are rotated (None: all of them when
    ``inv_freq`` is given, else none); ``interleaved``: pairs (2i, 2i+1) instead of (i, i + rotary_dim/2).
    """
    lib = build.load("elementwise")
    T = q_out.shape[0]
    if cache.dtype != q_out.dtype:
        raise KernelError("rope_append: cache and activations must have one dtype")
    if rotary_dim is None:
        rotary_dim = d if inv_freq is not None else 0
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError(f"rope_append: {rotary_dim} rotated elements need {rotary_dim // 2} frequencies")
    _check(lib, lib.mhb_rope_append(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(nsplit), c_longlong(split_stride),
        _ptr(bias), _ptr(positions), _ptr(tok_seg), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(inv_freq), _ptr(q_out), _ptr(cache),
        c_int(dtype_code(q_out.dtype)), c_int(T), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(1 if write_kv else 0),
        c_int(rotary_dim), c_int(1 if interleaved else 0), _ptr(status), _stream()), "rope_append")


def swiglu(gate_up, out, nsplit=1, split_stride=0, block=None):
    """out[t, i] = silu(gate_i) * up_i; gate_up[t] holds blocks of ``block`` gate values followed by
    the up values of the same indices (default: one block, [gate | up])."""
    lib = build.load("elementwise")
    T, I = out.shape
    _check(lib, lib.mhb_swiglu(_ptr(gate_up), c_int(dtype_code(gate_up.dtype)), c_int(nsplit),
                               c_longlong(split_stride), _ptr(out), c_int(dtype_code(out.dtype)),
                               c_int(T), c_int(I), c_int(block or I), _stream()), "swiglu")


def gemm_simt(a, w, out, bias=None, nsplit=1, split_stride=0):
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias) with float32 accumulation on the CUDA cores."""
    lib = build.load("gemm_simt")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: a is [{M},{K}] but w is {list(w.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(-1) != 1:
        raise KernelError("gemm: the last dimension must be contiguous")
    _check(lib, lib.mhb_gemm_simt(
        _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out),
        c_int(dtype_code(out.dtype)), _ptr(bias), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(-2)),
        c_int(nsplit), c_longlong(split_stride), _stream()), "gemm_simt")


STREAM_K_PARTIAL_FLOATS = 2 * 160 * 128 * 256     # workspace of the persistent product: two tiles per CTA
STREAM_K_FLAGS = 4 << 16                            # a counter for each quarter of each tile


def stream_k_scratch(device):
    """(partials, flags) for the persistent product: CTAs that share a tile's K range exchange
    float32 partial tiles through ``partials`` and count in ``flags`` (zero before and after)."""
    return (torch.empty(STREAM_K_PARTIAL_FLOATS, dtype=torch.float32, device=device),
            torch.zeros(STREAM_K_FLAGS, dtype=torch.int32, device=device))


def _scratch_ptrs(scratch):
    if scratch is None:
        return c_void_p(None), c_void_p(None)
    partials, flags = scratch
    if partials.numel() < STREAM_K_PARTIAL_FLOATS or flags.numel() < STREAM_K_FLAGS:
        raise KernelError("gemm_tc: the stream-K scratch is too small")
    return _ptr(partials), _ptr(flags)


class gemm_tc_wait_limit:
    """Inside the block the bounded waits of the persistent product give up after ``limit`` iterations
    instead of about a million: for tests that make a wait run out on purpose (a flag that nothing
    sets) and check that the kernel reports it (status bit 4) and leaves in order."""

    def __init__(self, limit: int):
        self.limit = limit

    def __enter__(self):
        lib = build.load("gemm_tc")
        lib.mhb_gemm_tc_wait_limit.restype = ctypes.c_uint
        self.before = lib.mhb_gemm_tc_wait_limit(ctypes.c_uint(self.limit))
        return self

    def __exit__(self, *exc):
        build.load("gemm_tc").mhb_gemm_tc_wait_limit(ctypes.c_uint(self.before))


def gemm_tc(a, w, out, *, swap: bool, bn: int, nsplit=1, split_stride=0, status=None, scratch=None):
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulate).

    ``swap`` streams the weights through the 128-row operand (for few tokens, M <= bn <= 64);
    ``bn`` is the tile width along the other operand, or 0 for the persistent kernel (more than
    64 tokens), which balances its CTAs over tiles and K with ``scratch`` from stream_k_scratch()."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: a is [{M},{K}] but w is {list(w.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(-1) != 1:
        raise KernelError("gemm_tc: the last dimension must be contiguous")
    if swap and M > bn:
        raise KernelError(f"gemm_tc: {M} tokens do not fit the swapped tile of {bn}")
    _check(lib, lib.mhb_gemm_tc(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(-2)),
        c_int(1 if swap else 0), c_int(bn), c_int(nsplit), c_longlong(split_stride),
        *_scratch_ptrs(scratch), _ptr(status), _stream()), "gemm_tc")


def gemm_tc_swiglu(a, w, out, *, swap: bool, bn: int, status=None, scratch=None):
    """out[M, I] = silu(a Wg^T) * (a Wu^T); ``w`` [2 I, K] holds gate and up rows interleaved in
    blocks of 16 (rows 32j..32j+15 gate, 32j+16..32j+31 up)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    I = out.shape[1]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_swiglu: operands and output must be bfloat16")
    if w.shape != (2 * I, K):
        raise KernelError(f"gemm_tc_swiglu: w is {list(w.shape)}, expected [{2 * I}, {K}]")
    if swap and M > bn:
        raise KernelError(f"gemm_tc: {M} tokens do not fit the swapped tile of {bn}")
    _check(lib, lib.mhb_gemm_tc_swiglu(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
        c_int(1 if swap else 0), c_int(bn), *_scratch_ptrs(scratch), _ptr(status), _stream()), "gemm_tc_swiglu")


def gemm_tc_glu(a, w, out, act: str, *, swap: bool, bn: int, status=None, scratch=None):
    """gemm_tc_swiglu with the gate's activation as a parameter: "silu" or "gelu_tanh" (taken in float32 on the
    accumulators, in the product's epilogue)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    I = out.shape[1]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_glu: operands and output must be bfloat16")
    if w.shape != (2 * I, K):
        raise KernelError(f"gemm_tc_glu: w is {list(w.shape)}, expected [{2 * I}, {K}]")
    if swap and M > bn:
        raise KernelError(f"gemm_tc: {M} tokens do not fit the swapped tile of {bn}")
    _check(lib, lib.mhb_gemm_tc_glu(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
        c_int(1 if swap else 0), c_int(bn), *_scratch_ptrs(scratch), _ptr(status), c_int(GLU_ACTS[act]), _stream()),
        "gemm_tc_glu")


def rope_table(positions, inv_freq, table):
    """table[t] = cos of token t's rotation angles, then their sin (float32, [T, 2 * angles]), for the
    q/k/v product's rotating epilogue."""
    lib = build.load("elementwise")
    T, rdim = table.shape
    if inv_freq.numel() * 2 != rdim or table.dtype != torch.float32 or not table.is_contiguous():
        raise KernelError("rope_table: the table must be float32 [tokens, 2 * frequencies]")
    _check(lib, lib.mhb_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), c_int(T), c_int(rdim), _stream()),
           "rope_table")


def gemm_tc_qkv_rope_supports(d: int, rotary_dim: int, interleaved: bool) -> bool:
    """Head sizes and rotations the q/k/v product's rotating epilogue is built for."""
    return d in (64, 128) and 0 <= rotary_dim <= d and rotary_dim % (16 if interleaved else 32) == 0


def gemm_tc_qkv_rope(x, w, bias, cos_sin, positions, tok_seg, block_table, q_out, cache, *, nq, nkv, d,
                     page_size, rotary_dim=None, interleaved=False, write_kv=True, status=None):
    """The stacked q/k/v product of more than 64 tokens whose epilogue adds the bias, rotates q and k
    (``cos_sin`` from rope_table, None for no rotation) and writes q to ``q_out`` and k, v into the
    pages of ``cache`` (one layer's pool)."""
    lib = build.load("gemm_tc")
    M, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_qkv_rope: operands, q and the cache must be bfloat16")
    if tuple(w.shape) != ((nq + 2 * nkv) * d, K) or not cache.is_contiguous() or not q_out.is_contiguous():
        raise KernelError(f"gemm_tc_qkv_rope: w is {list(w.shape)}, expected [{(nq + 2 * nkv) * d}, {K}]; q and the pool must be contiguous")
    if rotary_dim is None:
        rotary_dim = cos_sin.shape[1] if cos_sin is not None else 0
    if rotary_dim and (cos_sin is None or cos_sin.shape != (M, rotary_dim) or cos_sin.dtype != torch.float32):
        raise KernelError("gemm_tc_qkv_rope: the cos/sin table must be float32 [tokens, rotated elements]")
    _check(lib, lib.mhb_gemm_tc_qkv_rope(
        _ptr(x), _ptr(w), c_int(M), c_int(K), c_longlong(x.stride(0)), c_longlong(w.stride(0)), _ptr(bias),
        _ptr(cos_sin), c_int(rotary_dim), c_int(1 if interleaved else 0), _ptr(positions), _ptr(tok_seg),
        _ptr(block_table), c_int(block_table.shape[-1]), _ptr(q_out),
        _ptr(cache), c_int(nq), c_int(nkv), c_int(d), c_int(page_size), c_int(cache.shape[0]),
        c_int(1 if write_kv else 0), _ptr(status), _stream()), "gemm_tc_qkv_rope")


def attention_simt(q, cache, out, part_acc, part_ml, items, num_items, max_items, positions,
                   block_table, tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None, dv=None,
                   sink=None, gate=None, gate_nsplit=1, gate_split_stride=0, kparts=1, softcap=0.0,
                   shared_kv=False, gate_per_head=False, keep_first=0, pool=0, all_values=False, value_head=None):
    """CUDA-core attention over the items of a plan.  Options: ``dv`` values of another width than the
    keys (a page then holds the keys of all KV heads followed by their values), ``sink`` float32 [nq]
    (one extra term exp(sink_h) in the softmax's denominator), ``gate`` (the output is multiplied by its
    sigmoid; columns of a float32 product; ``gate_per_head``: one column per head), ``kparts`` score maps
    per KV head (its key row holds kparts keys side by side; ``nq`` counts every map of every head),
    ``softcap`` (s <- softcap tanh(s / softcap)), ``shared_kv`` (the values are the first dv elements of
    the key rows, and a page holds nothing but those rows).  With a window: ``keep_first`` positions at the
    start of a sequence stay visible, or (``pool``) every block of ``pool`` positions that the window has passed
    wholly is seen as one key and value, its means, from the tail of its page (csrc/maskparts.cu).
    ``all_values``: every query head's weights are applied to the values of all KV heads, and ``out`` is
    [T, nq, nkv * dv]; ``value_head``: to the values of that one KV head."""
    lib = build.load("attention_simt")
    if scale is None:
        scale = float(d) ** -0.5
    if keep_first or pool or all_values or value_head is not None:
        if keep_first and pool:
            raise KernelError("attention: kept first positions or pooled blocks, not both")
        if kparts != 1 or softcap or shared_kv or gate_per_head:
            raise KernelError("attention: keys beyond the window go with plain keys and values only")
        g = _gate_args(gate, gate_nsplit, gate_split_stride)
        _check(lib, lib.mhb_attention_simt_masked(
            _ptr(q), _ptr(cache), _ptr(out), c_int(dtype_code(q.dtype)), _ptr(part_acc), _ptr(part_ml),
            _ptr(items), c_int(num_items), c_int(max_items), _ptr(positions), _ptr(block_table),
            c_int(block_table.shape[-1]), _ptr(tok_part_row), c_int(nq), c_int(nkv), c_int(d), c_int(dv or d),
            c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(sink),
            g[0], g[1], g[2], g[3], c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if keep_first else 2 if pool else 0), c_int(keep_first or pool or 0),
            c_int(1 if all_values else 0 if value_head is None else 2 + value_head), _stream()), "attention")
        return
    general = kparts != 1 or softcap or shared_kv or gate_per_head or out.dtype != q.dtype
    if dv is not None or sink is not None or gate is not None or general:
        g = _gate_args(gate, gate_nsplit, gate_split_stride)
        _check(lib, lib.mhb_attention_simt_ext(
            _ptr(q), _ptr(cache), _ptr(out), c_int(dtype_code(q.dtype)), _ptr(part_acc), _ptr(part_ml),
            _ptr(items), c_int(num_items), c_int(max_items), _ptr(positions), _ptr(block_table),
            c_int(block_table.shape[-1]), _ptr(tok_part_row), c_int(nq), c_int(nkv), c_int(d), c_int(dv or d),
            c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(sink),
            g[0], g[1], g[2], g[3], c_int(kparts), c_float(softcap or 0.0), c_int(1 if shared_kv else 0),
            c_int(1 if gate_per_head else 0), c_int(1 if out.dtype == torch.float32 else 0), _stream()),
            "attention")
        return
    _check(lib, lib.mhb_attention_simt(
        _ptr(q), _ptr(cache), _ptr(out), c_int(dtype_code(q.dtype)), _ptr(part_acc), _ptr(part_ml),
        _ptr(items), c_int(num_items), c_int(max_items), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(tok_part_row), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _stream()),
        "attention")


MMA_HEAD_DIMS = (32, 64, 96, 128)   # head sizes the tensor-core attention kernel is built for


def attention_mma(q, cache, out, part_acc, part_ml, items, num_items, rows, positions, block_table,
                  tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None, tok_nsplit=None,
                  counters=None):
    """Tensor-core attention (bfloat16) over ``num_items`` items planned for tiles of ``rows`` rows.

    With ``counters`` (int32, zero, one per (token, KV head, chunk of 16 group heads)) the kernel
    merges the key splits itself and leaves the counters zero; else call attention_combine."""
    lib = build.load("attention_mma")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_mma: q and the cache must be bfloat16")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_mma(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
        c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _stream()),
        "attention_mma")


def lightning_chunked_tc_supports(dk: int, dv: int) -> bool:
    """Widths the tensor-core chunked route takes (tiles padded to 32, 64 or 128)."""
    return 1 <= dk <= 128 and 1 <= dv <= 128


LIGHTNING_TC_CHUNK = 64


def lightning_chunked_tc(proj, q0, k0, v0, decay, state, out, tok_seg, seg_slot, positions, chunks, num_chunks,
                         seg_chunks, num_segs, scratch, *, heads, dk, dv, nsplit=1, split_stride=0, writable=True):
    """lightning_chunked on the tensor cores: chunks of LIGHTNING_TC_CHUNK tokens, q, k and v rounded to
    bfloat16 after silu, every float32 operand of a product as the sum of two bfloat16 numbers."""
    lib = build.load("lightning")
    T = out.shape[0]
    if scratch.dtype != torch.float32 or scratch.numel() < num_chunks * heads * dk * dv:
        raise KernelError("lightning_chunked_tc: the scratch is too small")
    head = _lightning_head(proj, q0, k0, v0, decay, state, out, (tok_seg, seg_slot, positions), heads, dk, dv,
                           nsplit, split_stride, writable)
    _check(lib, lib.mhb_lightning_chunked_tc(*head, c_int(T), c_int(heads), c_int(dk), c_int(dv),
                                             c_int(1 if writable else 0), _ptr(chunks), c_int(num_chunks),
                                             _ptr(seg_chunks), c_int(num_segs), _ptr(scratch), _stream()),
           "lightning_chunked_tc")


def attention_mma_ext_supports(d: int, dv: int) -> bool:
    """Widths of keys and values the tensor-core attention with options takes (tiles padded to multiples of 32)."""
    return 8 <= d <= 128 and d % 8 == 0 and 8 <= dv <= 128 and dv % 8 == 0


def attention_mma_ext(q, cache, out, part_acc, part_ml, items, num_items, rows, positions, block_table,
                      tok_part_row, *, nq, nkv, d, dv, page_size, window=0, scale=None, tok_nsplit=None,
                      counters=None, sink=None, gate=None, gate_nsplit=1, gate_split_stride=0, kparts=1, softcap=0.0,
                      shared_kv=False, gate_per_head=False, keep_first=0, pool=0, value_head=None):
    """attention_mma with the options of attention_simt: values ``dv`` wide in pages that hold the keys of
    all KV heads followed by their values, a ``sink`` per query head, a ``gate`` on the output; the softmax's
    weights enter the value product as two bfloat16 numbers each (16 bits instead of 8).  ``kparts``,
    ``softcap``, ``shared_kv``, ``gate_per_head``, ``keep_first`` and ``pool`` as in attention_simt; ``out`` may be
    float32.  ``value_head``: every query head's weights are applied to the values of that one KV head; "all": to
    the values of every KV head in turn in one launch, ``out`` being [nkv, T, nq, dv] (a plane per KV head), the partial
    buffers [nkv, rows, nq, ...] and the counters [nkv, ...] likewise (for a mixer that mixes the heads' weights)."""
    lib = build.load("attention_mma_ext")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_mma_ext: q and the (contiguous) pool must be bfloat16")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("attention_mma_ext: the output must be bfloat16 or float32")
    if scale is None:
        scale = float(d) ** -0.5
    g = _gate_args(gate, gate_nsplit, gate_split_stride)
    if keep_first or pool or value_head is not None:
        if keep_first and pool:
            raise KernelError("attention: kept first positions or pooled blocks, not both")
        if kparts != 1 or softcap or shared_kv or gate_per_head or sink is not None:
            raise KernelError("attention: keys beyond the window go with plain keys and values only")
        planes = (0, 0, 0)
        if value_head == "all":
            if tuple(out.shape[:1]) != (nkv,) or part_acc.shape[0] != nkv or part_ml.shape[0] != nkv or not out.is_contiguous():
                raise KernelError("attention: with the values of every KV head the output and the partial buffers have a plane per KV head")
            if counters is not None and counters.numel() % nkv:
                raise KernelError("attention: the counters have a plane per KV head")
            planes = (out[0].numel(), part_acc.shape[1], 0 if counters is None else counters.numel() // nkv)
            value_head = -2
        _check(lib, lib.mhb_attention_mma_masked(
            _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
            c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
            _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d), c_int(dv),
            c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), g[0], g[1], g[2], g[3],
            c_int(1 if out.dtype == torch.float32 else 0), c_int(1 if keep_first else 2 if pool else 0),
            c_int(keep_first or pool or 0), c_int(-1 if value_head is None else value_head),
            *(c_longlong(x) for x in planes), _stream()),
            "attention_mma_ext")
        return
    _check(lib, lib.mhb_attention_mma_ext(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
        c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d), c_int(dv),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(sink),
        g[0], g[1], g[2], g[3], c_int(kparts), c_float(softcap or 0.0), c_int(1 if shared_kv else 0),
        c_int(1 if gate_per_head else 0), c_int(1 if out.dtype == torch.float32 else 0), _stream()),
        "attention_mma_ext")


def attention_tma_supports(d: int, page_size: int) -> bool:
    """Head sizes and page sizes the TMA-fed attention kernel is built for."""
    return d in (64, 128) and 2 <= page_size <= 64 and 64 % page_size == 0


def attention_tma(q, cache, out, part_acc, part_ml, items, num_items, rows, positions, block_table,
                  tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None, tok_nsplit=None,
                  counters=None, status=None, fresh=0):
    """attention_mma with keys and values staged by TMA through a ring of mbarrier-guarded stages.

    ``fresh``: how many positions before an item's first token the kernel launched just before this
    one may have written (the append of the step's own keys); older keys are requested while that
    kernel still runs.  0: it may have written any key."""
    lib = build.load("attention_tma")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tma: q and the cache must be bfloat16")
    if not cache.is_contiguous():
        raise KernelError("attention_tma: the layer's pool must be contiguous")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_tma(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
        c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_int(fresh), c_float(scale), _ptr(status),
        _stream()), "attention_tma")


DECODE_MAX_SPLITS = 16      # key splits of a token that the fused decode kernel merges in one cluster


def attention_decode_supports(d: int, page_size: int, groups: int, nsplit: int, rotary_dim: int) -> bool:
    """Sizes the fused decode-attention kernel is built for."""
    return (d in (64, 128) and 2 <= page_size <= 64 and 64 % page_size == 0 and 1 <= groups <= 16
            and 1 <= nsplit <= DECODE_MAX_SPLITS and nsplit * -(-groups // nsplit) <= 16
            and 0 <= rotary_dim <= d and rotary_dim % 8 == 0)


_decode_clusters: dict[tuple[int, int], int] = {}


def attention_decode_max_clusters(d: int, nsplit: int) -> int:
    """How many clusters of ``nsplit`` CTAs of the fused decode kernel the device holds at once."""
    key = (d, nsplit)
    if key not in _decode_clusters:
        lib = build.load("attention_decode")
        n = lib.mhb_attention_decode_max_clusters(c_int(d), c_int(nsplit))
        if n < 0:
            raise KernelError(f"attention_decode: {lib.mhb_last_error().decode()}")
        _decode_clusters[key] = n
    return _decode_clusters[key]


def attention_decode(qkv, bias, inv_freq, cache, out, positions, block_table, *, nq, nkv, d, page_size, nsplit,
                     qkv_nsplit=1, qkv_split_stride=0, rotary_dim=None, interleaved=False, window=0, scale=None,
                     status=None, ngroups=1, part_acc=None, part_ml=None):
    """A batch of single new tokens in one kernel: the q/k/v product's float32 partials ``qkv``
    ([qkv_nsplit, T, (nq + 2 nkv) d], ``qkv_split_stride`` elements apart) are summed, biased and
    rotated, k and v are appended to ``cache`` (one layer's pool), every token attends over its
    ``nsplit`` equal shares of keys and the shares are merged inside a thread-block cluster.
    Token i is segment i: ``block_table`` [T, width], ``positions`` [T]; ``out`` [T, nq d] bfloat16.

    ``ngroups`` > 1 cuts every token's keys into ngroups * nsplit shares, ngroups clusters per token and
    KV head: each cluster leaves its part in ``part_acc`` [T * ngroups, nq, d] and ``part_ml``
    [T * ngroups, nq, 2], and ``out`` is written by attention_combine(..., every=ngroups)."""
    lib = build.load("attention_decode")
    T = out.shape[0]
    if qkv.dtype != torch.float32 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode: the product's parts must be float32, cache and output bfloat16")
    if not cache.is_contiguous() or not out.is_contiguous() or qkv.stride(-1) != 1 or qkv.stride(-2) != (nq + 2 * nkv) * d:
        raise KernelError("attention_decode: the pool, the output and the rows of the product must be contiguous")
    if rotary_dim is None:
        rotary_dim = d if inv_freq is not None else 0
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError(f"attention_decode: {rotary_dim} rotated elements need {rotary_dim // 2} frequencies")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_decode(
        _ptr(qkv), c_int(qkv_nsplit), c_longlong(qkv_split_stride), _ptr(bias), _ptr(inv_freq), c_int(rotary_dim),
        c_int(1 if interleaved else 0), _ptr(cache), _ptr(out), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(page_size),
        c_int(cache.shape[0]), c_int(window or 0), c_int(nsplit), c_int(ngroups), _ptr(part_acc), _ptr(part_ml),
        c_float(scale), _ptr(status), _stream()),
        "attention_decode")
    if ngroups > 1:
        attention_combine(part_acc, part_ml, None, None, out, nq=nq, d=d, every=ngroups)


def attention_tc(q, cache, out, items, num_items, positions, block_table, *, nq, nkv, d, page_size,
                 window=0, scale=None, status=None, part_acc=None, part_ml=None, tok_part_row=None):
    """tcgen05 attention for long portions: ``items`` planned for tiles of 128 rows; items split
    along the keys write to the partial buffers (then call attention_combine)."""
    lib = build.load("attention_tc")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tc: q and the cache must be bfloat16")
    if not cache.is_contiguous():
        raise KernelError("attention_tc: the layer's pool must be contiguous")
    if scale is None:
        scale = float(d) ** -0.5
    _check(lib, lib.mhb_attention_tc(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(items), c_int(num_items), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(tok_part_row), _ptr(part_acc), _ptr(part_ml),
        c_int(nq), c_int(nkv), c_int(d), c_int(page_size),
        c_int(cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(status), _stream()), "attention_tc")


def attention_tma_ext(q, cache, out, part_acc, part_ml, items, num_items, rows, positions, block_table,
                      tok_part_row, *, nq, nkv, d, page_size, window=0, scale=None, tok_nsplit=None,
                      counters=None, status=None, fresh=0, sink=None, gate=None, gate_nsplit=1, gate_split_stride=0,
                      gate_per_head=False, shared_kv=False, softcap=0.0):
    """attention_tma with a ``sink`` per query head, a ``gate`` on the output (``gate_per_head``: one column per
    head) and softmax weights that keep 16 bits in the value product; keys and values are both ``d`` wide.
    ``shared_kv``: the pool is [pages, P, d] and a row is its position's key and value at once; ``softcap`` caps
    the scaled scores; ``out`` may be float32."""
    lib = build.load("attention_tma")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_tma_ext: q and the (contiguous) pool must be bfloat16")
    if scale is None:
        scale = float(d) ** -0.5
    g = _gate_args(gate, gate_nsplit, gate_split_stride)
    _check(lib, lib.mhb_attention_tma_ext(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(items), c_int(num_items),
        c_int(num_items), c_int(rows), _ptr(positions), _ptr(block_table), c_int(block_table.shape[-1]),
        _ptr(tok_part_row), _ptr(tok_nsplit), _ptr(counters), c_int(nq), c_int(nkv), c_int(d),
        c_int(page_size), c_int(cache.shape[0]), c_int(window or 0), c_int(fresh), c_float(scale), _ptr(sink),
        g[0], g[1], g[2], g[3], c_int(1 if gate_per_head else 0), c_int(1 if shared_kv else 0),
        c_float(softcap or 0.0), c_int(1 if out.dtype == torch.float32 else 0), _ptr(status), _stream()),
        "attention_tma_ext")


def attention_tc_ext(q, cache, out, items, num_items, positions, block_table, *, nq, nkv, d, page_size,
                     window=0, scale=None, status=None, part_acc=None, part_ml=None, tok_part_row=None,
                     sink=None, gate=None, gate_nsplit=1, gate_split_stride=0, gate_per_head=False, shared_kv=False,
                     softcap=0.0):
    """attention_tc with a ``sink`` per query head, a ``gate`` on the output (``gate_per_head``: one column
    per head) and softmax weights that keep 16 bits in the value product; keys and values are both ``d``
    wide.  ``shared_kv``: the pool is [pages, P, d] and a row is its position's key and value at once;
    ``softcap`` caps the scaled scores; ``out`` may be float32."""
    lib = build.load("attention_tc")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_tc_ext: q and the (contiguous) pool must be bfloat16")
    if scale is None:
        scale = float(d) ** -0.5
    g = _gate_args(gate, gate_nsplit, gate_split_stride)
    _check(lib, lib.mhb_attention_tc_ext(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(items), c_int(num_items), _ptr(positions), _ptr(block_table),
        c_int(block_table.shape[-1]), _ptr(tok_part_row), _ptr(part_acc), _ptr(part_ml),
        c_int(nq), c_int(nkv), c_int(d), c_int(page_size), c_int(cache.shape[0]), c_int(window or 0),
        c_float(scale), _ptr(sink), g[0], g[1], g[2], g[3], c_int(1 if gate_per_head else 0),
        c_int(1 if shared_kv else 0), c_float(softcap or 0.0), c_int(1 if out.dtype == torch.float32 else 0),
        _ptr(status), _stream()), "attention_tc_ext")


def attention_combine(part_acc, part_ml, tok_part_row, tok_nsplit, out, *, nq, d, every=0, gate=None,
                      gate_nsplit=1, gate_split_stride=0, gate_per_head=False):
    """Merge the parts of every token's attention.  ``every`` > 0: each token has exactly that many parts,
    in the rows t * every ... of the partial buffers (the two index arrays may be None).  ``d`` is the
    width of a head's output; ``gate``: see attention_simt."""
    lib = build.load("attention_simt")
    T = out.shape[0]
    if gate is not None:
        g = _gate_args(gate, gate_nsplit, gate_split_stride)
        _check(lib, lib.mhb_attention_combine_gated(_ptr(part_acc), _ptr(part_ml), _ptr(tok_part_row),
                                                    _ptr(tok_nsplit), _ptr(out), c_int(dtype_code(out.dtype)),
                                                    c_int(T), c_int(nq), c_int(d), c_int(every), g[0], g[1], g[2],
                                                    g[3], c_int(1 if gate_per_head else 0), _stream()),
               "attention_combine")
        return
    _check(lib, lib.mhb_attention_combine(_ptr(part_acc), _ptr(part_ml), _ptr(tok_part_row),
                                          _ptr(tok_nsplit), _ptr(out), c_int(dtype_code(out.dtype)),
                                          c_int(T), c_int(nq), c_int(d), c_int(every), _stream()),
           "attention_combine")


def sample(logits, temperature, seed, counter, out):
    """out[r] = argmax(logits[r]) where temperature[r] <= 0, else a draw from softmax(logits/T)."""
    lib = build.load("sampling")
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with a contiguous last dimension")
    _check(lib, lib.mhb_sample(_ptr(logits), c_longlong(logits.stride(0)), c_int(R), c_int(V),
                               _ptr(temperature), _ptr(seed), _ptr(counter), _ptr(out), _stream()),
           "sample")


# ---- parts of parallel blocks, multi-map attention and latent attention (csrc/mixparts.cu) --------------
def _delta_args(delta):
    """(pointer, parts, stride between parts) of a pending product (None: nothing to add)."""
    if delta is None:
        return c_void_p(0), c_int(1), c_longlong(0)
    return _ptr(delta.tensor), c_int(delta.nsplit), c_longlong(delta.split_stride)


def _delta_dtype(*deltas) -> int:
    kinds = {d.tensor.dtype for d in deltas if d is not None}
    if len(kinds) > 1:
        raise KernelError("products that are added together must have one dtype")
    return dtype_code(kinds.pop()) if kinds else F32


def add_layernorm(x, weight, eps, out, delta=None, delta2=None, rows=None):
    """out[r] = layernorm(x[s] + delta[s] + delta2[s]) * weight (no bias) with s = rows[r] if rows is given
    else r; without ``rows`` and with a delta the sum is written back to ``x``.  The deltas are products
    (objects with tensor, nsplit, split_stride), each possibly float32 split-K parts."""
    lib = build.load("mixparts")
    R, H = out.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("add_layernorm: the stream must be a contiguous float32 matrix")
    if delta is None and delta2 is not None:
        delta, delta2 = delta2, None
    a, b = _delta_args(delta), _delta_args(delta2)
    _check(lib, lib.mhb_add_layernorm(_ptr(x), a[0], a[1], a[2], b[0], b[1], b[2], c_int(_delta_dtype(delta, delta2)),
                                      _ptr(weight), c_float(eps), _ptr(rows), _ptr(out), c_int(dtype_code(out.dtype)),
                                      c_int(R), c_int(H), _stream()), "add_layernorm")


def stream_pack(x, dst, col0: int, delta=None, delta2=None, zero: bool = False):
    """dst[:, col0 : col0 + W] = x + delta + delta2 in dst's dtype (x float32 [T, W]); with ``zero`` the
    stream is left at zero (whoever replaces the stream by a product adds that product into it)."""
    lib = build.load("mixparts")
    T, W = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or dst.stride(1) != 1:
        raise KernelError("stream_pack: the stream must be contiguous float32, the target's rows contiguous")
    if delta is None and delta2 is not None:
        delta, delta2 = delta2, None
    a, b = _delta_args(delta), _delta_args(delta2)
    _check(lib, lib.mhb_stream_pack(_ptr(x), a[0], a[1], a[2], b[0], b[1], b[2], c_int(_delta_dtype(delta, delta2)),
                                    _ptr(dst), c_int(dtype_code(dst.dtype)), c_int(dst.stride(0)), c_int(col0),
                                    c_int(T), c_int(W), c_int(1 if zero else 0), _stream()), "stream_pack")


def glu_act(gate_up, out, act: str, nsplit=1, split_stride=0, block=None):
    """out[t, i] = act(gate_i) * up_i; gate_up[t] holds blocks of ``block`` gate values followed by the up
    values of the same indices (default: one block, [gate | up])."""
    lib = build.load("mixparts")
    T, I = out.shape
    _check(lib, lib.mhb_glu_act(_ptr(gate_up), c_int(dtype_code(gate_up.dtype)), c_int(nsplit), c_longlong(split_stride),
                                _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(I), c_int(block or I),
                                c_int(GLU_ACTS[act]), _stream()), "glu_act")


def rope_append_maps(proj, positions, tok_seg, block_table, inv_freq, rotary_dim, interleaved, q_out, cache, *,
                     nq, nkv, kparts, d, dv, page_size, nsplit=1, split_stride=0, status=None, q_pad=False):
    """Rows of the float32 product [q: nq * d | k: nkv * kparts * d | v: nkv * dv | ...]: the first
    ``rotary_dim`` elements of every q and k map are rotated, q goes to ``q_out`` [T, nq * d], keys and values
    into the page of the position ([keys: nkv][P][kparts * d] then [values: nkv][P][dv]).  ``q_pad``: every q map
    is written as a row as wide as a KV head's key row, [T, nq, kparts * d], at the columns of its own map, zeros
    elsewhere: its product with the whole key row is the map's score."""
    lib = build.load("mixparts")
    T = q_out.shape[0]
    if proj.dtype != torch.float32 or cache.dtype != q_out.dtype:
        raise KernelError("rope_append_maps: a float32 product; cache and q of one dtype")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError(f"rope_append_maps: {rotary_dim} rotated elements need {rotary_dim // 2} frequencies")
    _check(lib, lib.mhb_rope_append_maps(
        _ptr(proj), c_int(nsplit), c_longlong(split_stride), c_int(proj.stride(-2)), _ptr(positions), _ptr(tok_seg),
        _ptr(block_table), c_int(block_table.shape[-1]), _ptr(inv_freq), c_int(rotary_dim or 0),
        c_int(1 if interleaved else 0), _ptr(q_out), _ptr(cache), c_int(dtype_code(q_out.dtype)), c_int(T), c_int(nq),
        c_int(nkv), c_int(kparts), c_int(d), c_int(dv), c_int(page_size), c_int(cache.shape[0]),
        c_int(1 if q_pad else 0), _ptr(status), _stream()), "rope_append_maps")


def latent_prep(proj, weight, eps, positions, tok_seg, block_table, inv_freq, interleaved, q_plain, q_full, cache, *,
                heads, d, dr, rank, page_size, write_kv=True, nsplit=1, split_stride=0, status=None):
    """Rows of the float32 product [q: heads * (d + dr) | latent: rank | key part: dr | ...]: the latent is
    divided by its root mean square and multiplied by ``weight``, the key part and the last dr elements of each
    q head are rotated; the cache row [latent | key part] goes into the position's page ([P][rank + dr]),
    q's unrotated parts to ``q_plain`` [T, heads, d], its rotated parts to the last dr columns of ``q_full``
    [T, heads, rank + dr]."""
    lib = build.load("mixparts")
    T = q_plain.shape[0]
    if proj.dtype != torch.float32 or cache.dtype != q_full.dtype or q_plain.dtype != q_full.dtype:
        raise KernelError("latent_prep: a float32 product; cache and q of one dtype")
    if dr and (inv_freq is None or inv_freq.numel() != dr // 2):
        raise KernelError(f"latent_prep: {dr} rotated elements need {dr // 2} frequencies")
    _check(lib, lib.mhb_latent_prep(
        _ptr(proj), c_int(nsplit), c_longlong(split_stride), c_int(proj.stride(-2)), _ptr(weight), c_float(eps),
        _ptr(positions), _ptr(tok_seg), _ptr(block_table), c_int(block_table.shape[-1]), _ptr(inv_freq),
        c_int(1 if interleaved else 0), _ptr(q_plain), _ptr(q_full), _ptr(cache), c_int(dtype_code(q_full.dtype)),
        c_int(T), c_int(heads), c_int(d), c_int(dr), c_int(rank), c_int(page_size), c_int(cache.shape[0]),
        c_int(1 if write_kv else 0), _ptr(status), _stream()), "latent_prep")


def head_linear(x, w, out):
    """out[t, h, :] = w[h] @ x[t, h, :] with float32 accumulation: x [T, heads, K] and out [T, heads, N] may be
    views with any token and head strides (last dimension contiguous), w [heads, N, K] contiguous."""
    lib = build.load("mixparts")
    T, H, Kd = x.shape
    N = w.shape[1]
    if tuple(w.shape) != (H, N, Kd) or tuple(out.shape) != (T, H, N):
        raise KernelError(f"head_linear: x {list(x.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if x.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous():
        raise KernelError("head_linear: the last dimensions must be contiguous")
    _check(lib, lib.mhb_head_linear(_ptr(x), c_int(dtype_code(x.dtype)), c_longlong(x.stride(0)), c_longlong(x.stride(1)),
                                    _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out), c_int(dtype_code(out.dtype)),
                                    c_longlong(out.stride(0)), c_longlong(out.stride(1)), c_int(T), c_int(H), c_int(N),
                                    c_int(Kd), _stream()), "head_linear")


def maps_combine(a, lam: float, eps: float, post: float, out, gate=None, gate_nsplit=1, gate_split_stride=0):
    """a float32 [T, heads, 2, dv]: o = a[..., 0, :] - lam * a[..., 1, :], divided by its root mean square over
    dv (eps inside the root), times ``post``, times sigmoid(gate[t, h]) (one column per head of a float32
    product); out [T, heads * dv]."""
    lib = build.load("mixparts")
    T, H, two, dv = a.shape
    if two != 2 or a.dtype != torch.float32 or not a.is_contiguous() or not out.is_contiguous():
        raise KernelError("maps_combine: a must be contiguous float32 [T, heads, 2, dv]")
    g = _gate_args(gate, gate_nsplit, gate_split_stride)
    _check(lib, lib.mhb_maps_combine(_ptr(a), c_float(lam), c_float(eps), c_float(post), g[0], g[1], g[2], g[3],
                                     _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(H), c_int(dv),
                                     _stream()), "maps_combine")


# ---- blocks that normalise a sublayer's result; two activations (csrc/gateparts.cu) ---------------------------
def _parts_args(t, nsplit, split_stride):
    if t.dtype != torch.float32 or t.stride(-1) != 1:
        raise KernelError("a product that joins a float32 sum must be float32 with contiguous rows")
    return _ptr(t), c_int(nsplit), c_longlong(split_stride)


def gated_norm_add(x, delta, weight, eps, *, gate=None, bias=None, copy=None, next_weight=None, next_eps=None,
                   next_out=None):
    """x <- x + rms(d * sigmoid(g + bias)) * weight, row by row in float32, in place.  ``delta`` and ``gate`` are
    Products (float32, possibly split-K parts; the gate may be a run of columns of a wider product); without a
    gate y = d.  ``copy``: the new rows once more in the compute dtype; ``next_out`` with ``next_weight``: the
    next norm of the new rows, rms(x) * next_weight, in the compute dtype."""
    lib = build.load("gateparts")
    R, H = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("gated_norm_add: the stream must be a contiguous float32 matrix")
    d = delta.tensor
    if tuple(d.shape[-2:]) != (R, H) or not d[0 if delta.nsplit > 1 else slice(None)].is_contiguous():
        raise KernelError("gated_norm_add: the product must be contiguous and of the stream's shape")
    g = (c_void_p(0), c_int(1), c_longlong(0))
    g_ld = 0
    if gate is not None:
        g = _parts_args(gate.tensor, gate.nsplit, gate.split_stride)
        g_ld = gate.tensor.stride(-2)
    outs = [t for t in (copy, next_out) if t is not None]
    for t in outs:
        if t.dtype != outs[0].dtype or tuple(t.shape) != (R, H) or not t.is_contiguous():
            raise KernelError("gated_norm_add: copy and next_out are contiguous, of one dtype and of the stream's shape")
    odt = dtype_code(outs[0].dtype) if outs else F32
    _check(lib, lib.mhb_gated_norm_add(_ptr(x), *_parts_args(d, delta.nsplit, delta.split_stride), *g, c_int(g_ld),
                                       _ptr(bias), _ptr(weight), c_float(eps), _ptr(copy),
                                       _ptr(next_weight if next_out is not None else None),
                                       c_float(next_eps if next_eps is not None else eps), _ptr(next_out), c_int(odt),
                                       c_int(R), c_int(H), _stream()), "gated_norm_add")


def polynorm_rows(z, coef, eps, out, nsplit=1, split_stride=0):
    """out = a rms(z) + b rms(z^2) + c rms(z^3) + e over every row of the float32 product z (powers element by
    element, each power divided by its own root mean square); coef = (a, b, c, e) float32 on the device."""
    lib = build.load("gateparts")
    R, Fd = out.shape
    if coef.dtype != torch.float32 or coef.numel() != 4 or not out.is_contiguous():
        raise KernelError("polynorm_rows: four float32 coefficients and a contiguous output")
    _check(lib, lib.mhb_polynorm_rows(*_parts_args(z, nsplit, split_stride), _ptr(coef), c_float(eps), _ptr(out),
                                      c_int(dtype_code(out.dtype)), c_int(R), c_int(Fd), _stream()), "polynorm_rows")


def softcap_rows(z, cap: float):
    """z <- cap * tanh(z / cap) in place (float32)."""
    lib = build.load("gateparts")
    if z.dtype != torch.float32 or not z.is_contiguous():
        raise KernelError("softcap_rows: a contiguous float32 tensor")
    _check(lib, lib.mhb_softcap_rows(_ptr(z), c_float(cap), c_longlong(z.numel()), _stream()), "softcap_rows")


# ---- linear attention with a decay per key channel and token (csrc/gatedlinear.cu) ------------------------------
GATED_LINEAR_MODES = {"gla": 0, "hgrn2": 1}


def gated_linear_prep(mode: str, proj, q0, k0, v0, a0, bias, q, k, v, g, *, a2=None, low=None, qscale=1.0, tau=1.0):
    """From the float32 Product ``proj`` (columns q0 / k0 / v0 / a0, heads side by side) the recurrence's float32
    inputs q, k, v and g = log(decay).  "gla": q = zq * qscale, k = zk, g = logsigmoid(z + bias) / tau with
    z = a2 @ (the columns a0 .. a0 + rank of ``proj``), ``a2`` [heads * dim, rank], taken in float32.  "hgrn2":
    q = silu(zq), f = low + (1 - low) sigmoid(za + bias) with za the columns from a0, k = 1 - f, g = log f."""
    lib = build.load("gatedlinear")
    T, QW = q.shape
    VW = v.shape[1]
    for t in (q, k, v, g):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError("gated_linear_prep: q, k, v and g are contiguous float32")
    rank = 0
    if mode == "gla":
        if a2 is None or a2.shape[0] != QW or not a2.is_contiguous():
            raise KernelError("gated_linear_prep: the decay's second matrix is contiguous [heads * dim, rank]")
        rank = a2.shape[1]
    _check(lib, lib.mhb_gated_linear_prep(
        *_parts_args(proj.tensor, proj.nsplit, proj.split_stride), c_int(proj.tensor.stride(-2)), c_int(q0), c_int(k0),
        c_int(v0), c_int(a0), _ptr(a2), c_int(dtype_code(a2.dtype) if a2 is not None else F32), c_int(rank), _ptr(bias),
        _ptr(low), c_float(qscale), c_float(1.0 / tau), c_int(GATED_LINEAR_MODES[mode]),
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), c_int(T), c_int(QW), c_int(VW), _stream()), "gated_linear_prep")


def gated_linear_head_norm(o, weight, eps, out, *, heads, dv, gate=None, gate0=0):
    """out[t, h] = rms(o[t, h]) * weight, one norm per head over its ``dv`` values (``weight`` [dv] is shared by the
    heads), times silu of the columns gate0 .. of the float32 Product ``gate`` if there is one."""
    lib = build.load("gatedlinear")
    T = o.shape[0]
    if o.dtype != torch.float32 or not o.is_contiguous() or not out.is_contiguous() or o.shape[1] != heads * dv:
        raise KernelError("gated_linear_head_norm: o is contiguous float32 [T, heads * dv], out contiguous")
    gp = (c_void_p(0), c_int(1), c_longlong(0))
    g_ld = 0
    if gate is not None:
        gp = _parts_args(gate.tensor, gate.nsplit, gate.split_stride)
        g_ld = gate.tensor.stride(-2)
    _check(lib, lib.mhb_gated_linear_head_norm(_ptr(o), _ptr(weight), c_float(eps), *gp, c_int(g_ld), c_int(gate0),
                                               _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(heads), c_int(dv),
                                               _stream()), "gated_linear_head_norm")


def _gated_linear_head(q, k, g, v, state, out, tok_seg, seg_slot, positions, H, dk, dv):
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (H, dk, dv):
        raise KernelError(f"gated linear attention: the state must be contiguous float32 [slots, {H}, {dk}, {dv}]")
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("gated linear attention: the output is contiguous float32")
    return (_ptr(q), _ptr(k), _ptr(g), _ptr(v), _ptr(state), _ptr(out), _ptr(tok_seg), _ptr(seg_slot), _ptr(positions))


def gated_linear_scan(q, k, g, v, state, out, tok_seg, seg_slot, positions, *, heads, dk, dv, writable=True,
                      max_tokens=0):
    """S <- diag(exp(g_t)) S + k_t v_t^T, o_t = S^T q_t, token by token, for every segment of at most ``max_tokens``
    tokens (0: all); ``state`` [slots, heads, dk, dv], ``out`` float32 [T, heads * dv]."""
    lib = build.load("gatedlinear")
    T, S = out.shape[0], seg_slot.shape[0]
    head = _gated_linear_head(q, k, g, v, state, out, tok_seg, seg_slot, positions, heads, dk, dv)
    _check(lib, lib.mhb_gated_linear_scan(*head, c_int(T), c_int(S), c_int(heads), c_int(dk), c_int(dv),
                                          c_int(1 if writable else 0), c_int(max_tokens), _stream()), "gated_linear_scan")


def gated_linear_chunk_smem(dk: int, dv: int, chunk: int) -> int:
    lib = build.load("gatedlinear")
    lib.mhb_gated_linear_chunk_smem.restype = c_longlong
    return int(lib.mhb_gated_linear_chunk_smem(c_int(dk), c_int(dv), c_int(chunk)))


def gated_linear_chunked(q, k, g, v, state, out, tok_seg, seg_slot, positions, chunks, num_chunks, seg_chunks,
                         num_segs, scratch, chunk, *, heads, dk, dv, writable=True):
    """The same for the listed segments, cut into the listed chunks of at most ``chunk`` tokens; ``scratch`` float32
    holds num_chunks * heads * (dk * dv + dk)."""
    lib = build.load("gatedlinear")
    T = out.shape[0]
    if scratch.dtype != torch.float32 or scratch.numel() < num_chunks * heads * (dk * dv + dk):
        raise KernelError("gated_linear_chunked: the scratch is too small")
    head = _gated_linear_head(q, k, g, v, state, out, tok_seg, seg_slot, positions, heads, dk, dv)
    _check(lib, lib.mhb_gated_linear_chunked(*head, c_int(T), c_int(heads), c_int(dk), c_int(dv),
                                             c_int(1 if writable else 0), _ptr(chunks), c_int(num_chunks),
                                             _ptr(seg_chunks), c_int(num_segs), _ptr(scratch), c_int(chunk), _stream()),
           "gated_linear_chunked")


# ---- routed feed-forward (csrc/moe.cu) --------------------------------------------------------------------------
MOE_TILE_ROWS = 64


def moe_max_tiles(pairs: int, experts: int) -> int:
    """Upper bound of the tiles that ``pairs`` (token, expert) pairs over ``experts`` experts are cut into."""
    return -(-pairs // MOE_TILE_ROWS) + min(experts, pairs)


def moe_plan_words(pairs: int, experts: int) -> int:
    return 1 + 3 * moe_max_tiles(pairs, experts) + 2 * pairs


def moe_route(logits, correction, chosen, weights, *, outputs, top, groups=1, keep=1, bias=None):
    """Per token: softmax over the first ``outputs`` columns of the float32 Product ``logits`` (plus ``bias``, if
    there is one), choice by softmax + correction (None: none) inside the best ``keep`` of ``groups`` groups,
    ``chosen`` int32 [T, top] and the chosen outputs' softmax values divided by their sum as ``weights`` float32
    [T, top]: without a correction that is the choice of the largest logits, weighted by the softmax over the
    chosen logits alone."""
    lib = build.load("moe")
    T = chosen.shape[0]
    _check(lib, lib.mhb_moe_route_biased(*_parts_args(logits.tensor, logits.nsplit, logits.split_stride),
                                         c_int(logits.tensor.stride(-2)), _ptr(bias), _ptr(correction), _ptr(chosen),
                                         _ptr(weights), c_int(T), c_int(outputs), c_int(top), c_int(groups),
                                         c_int(keep), _stream()), "moe_route")


def moe_plan(chosen, plan, *, experts):
    """Group the chosen pairs by expert (outputs at or beyond ``experts`` get no row); ``plan`` int32 of
    moe_plan_words(pairs, experts)."""
    lib = build.load("moe")
    T, top = chosen.shape
    pairs = T * top
    if plan.dtype != torch.int32 or plan.numel() < moe_plan_words(pairs, experts):
        raise KernelError("moe_plan: the plan buffer is too small")
    _check(lib, lib.mhb_moe_plan(_ptr(chosen), c_int(pairs), c_int(top), c_int(experts),
                                 c_int(moe_max_tiles(pairs, experts)), _ptr(plan), _stream()), "moe_plan")


def moe_linear(x, plan, w, out, *, pairs, experts, gather: bool, glu: bool):
    """out[r] = w[expert of row r] applied to x[token of row r] (``gather``) or to x[r]; ``w`` [experts, N, K], or
    [experts, 2 N, K] holding gate above up with ``glu`` (then out = silu(gate x) * (up x)); float32 accumulation."""
    lib = build.load("moe")
    N, Kd = out.shape[1], x.shape[1]
    if w.dtype != x.dtype or tuple(w.shape) != (experts, (2 if glu else 1) * N, Kd) or not w.is_contiguous():
        raise KernelError(f"moe_linear: weights {list(w.shape)} for rows {Kd} wide and outputs {N} wide")
    if x.stride(1) != 1 or not out.is_contiguous():
        raise KernelError("moe_linear: contiguous rows")
    _check(lib, lib.mhb_moe_linear(_ptr(x), c_int(dtype_code(x.dtype)), c_longlong(x.stride(0)), _ptr(plan),
                                   c_int(moe_max_tiles(pairs, experts)), c_int(pairs), c_int(1 if gather else 0), _ptr(w),
                                   _ptr(out), c_int(dtype_code(out.dtype)), c_int(N), c_int(Kd), c_int(1 if glu else 0),
                                   _stream()), "moe_linear")


def moe_combine(y, plan, chosen, weights, h, out, *, experts, shared=None, shared_gate=None):
    """out[t] = sum_k weights[t, k] * (y[row of pair (t, k)], or h[t] for an identity expert) + sigmoid(shared_gate[t])
    * shared[t]; ``shared`` and ``shared_gate`` are float32 Products (the gate one column)."""
    lib = build.load("moe")
    T, top = chosen.shape
    pairs = T * top
    W = out.shape[1]
    if out.dtype != torch.float32 or not out.is_contiguous() or h.stride(1) != 1:
        raise KernelError("moe_combine: a contiguous float32 output and input rows that are contiguous")
    sh = (c_void_p(0), c_int(1), c_longlong(0))
    sg = (c_void_p(0), c_int(1), c_longlong(0))
    g_ld = 0
    if shared is not None:
        sh = _parts_args(shared.tensor, shared.nsplit, shared.split_stride)
        sg = _parts_args(shared_gate.tensor, shared_gate.nsplit, shared_gate.split_stride)
        g_ld = shared_gate.tensor.stride(-2)
    _check(lib, lib.mhb_moe_combine(_ptr(y), _ptr(plan), c_int(moe_max_tiles(pairs, experts)), c_int(pairs), _ptr(chosen),
                                    _ptr(weights), c_int(top), c_int(experts), _ptr(h), c_int(dtype_code(h.dtype)),
                                    c_longlong(h.stride(0)), *sh, *sg, c_int(g_ld), _ptr(out), c_int(T), c_int(W),
                                    _stream()), "moe_combine")


# ---- keys beyond the window, mixed heads (csrc/maskparts.cu) --------------------------------------------------
def pool_slots(page_size: int, pool: int) -> int:
    """Pooled rows a page holds per KV head behind its keys and values: blocks of ``pool`` positions whose last
    position lies in the page."""
    return -(-page_size // pool)


def pool_means(cache, positions, tok_seg, block_table, *, nkv, d, dv, page_size, pool, status=None):
    """For every token of the step that completes a block of ``pool`` positions: the means of the block's cached
    keys and values into the tail of the page of its last position (one layer's pool, pages of
    nkv * page_size * (d + dv) + nkv * pool_slots * (d + dv) elements)."""
    lib = build.load("maskparts")
    T = positions.shape[0]
    want = nkv * (page_size + pool_slots(page_size, pool)) * (d + dv)
    if not cache.is_contiguous() or cache[0].numel() != want:
        raise KernelError(f"pool_means: a page of {cache[0].numel()} elements where {want} are needed")
    _check(lib, lib.mhb_pool_means(_ptr(cache), c_int(dtype_code(cache.dtype)), _ptr(positions), _ptr(tok_seg),
                                   _ptr(block_table), c_int(block_table.shape[-1]), c_int(T), c_int(nkv), c_int(d),
                                   c_int(dv), c_int(page_size), c_int(pool), c_int(cache.shape[0]), _ptr(status),
                                   _stream()), "pool_means")


def talk_mix(a, talk, out, *, nq, nkv, dv, planes=False):
    """out[t, h] = sum_g talk[h, g] * a[t, g, kv(h)]: ``a`` float32 holds every head's weights over the values of
    every KV head, as rows [T, nq, nkv * dv] or (``planes``) as one matrix per KV head, [nkv, T, nq, dv]; ``talk``
    float32 [nq, nq]; ``out`` [T, nq * dv]."""
    lib = build.load("maskparts")
    T = out.shape[0]
    if a.dtype != torch.float32 or not a.is_contiguous() or a.numel() != T * nq * nkv * dv or not out.is_contiguous():
        raise KernelError("talk_mix: a is contiguous float32 with T * nq * nkv * dv numbers, out contiguous")
    if talk.dtype != torch.float32 or tuple(talk.shape) != (nq, nq) or not talk.is_contiguous():
        raise KernelError(f"talk_mix: the mixing matrix is contiguous float32 [{nq}, {nq}]")
    strides = (nq * dv, dv, T * nq * dv) if planes else (nq * nkv * dv, nkv * dv, dv)
    _check(lib, lib.mhb_talk_mix(_ptr(a), _ptr(talk), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(nq),
                                 c_int(nkv), c_int(dv), *(c_longlong(x) for x in strides), _stream()), "talk_mix")


# ---- the gated delta rule (csrc/deltarule.cu) -------------------------------------------------------------------
def delta_prep(proj, c0, b0, a0, taps, A_log, dt_bias, keep, tok_seg, seg_slot, positions, q, k, v, beta, decay, *,
               heads, kv_heads, dk, dv, qscale, unit_eps):
    """From the float32 Product ``proj`` (columns c0 .. hold [q | k | v], b0 .. the write strength's logits, a0 .. the
    decay's): the short causal convolutions (``taps`` float32 [channels, taps]; inputs before the step from
    ``keep`` [slots, >= (taps - 1) * channels]), silu, unit q (times ``qscale``) and k per head, beta = sigmoid,
    decay = exp(-exp(A_log) softplus(a + dt_bias)); all outputs float32."""
    lib = build.load("deltarule")
    T = q.shape[0]
    C, ntaps = taps.shape
    if C != 2 * kv_heads * dk + heads * dv or taps.dtype != torch.float32 or not taps.is_contiguous():
        raise KernelError("delta_prep: the filters are contiguous float32 [2 kv_heads dk + heads dv, taps]")
    if keep.dtype != torch.float32 or keep.stride(-1) != 1 or keep.shape[-1] < (ntaps - 1) * C:
        raise KernelError("delta_prep: a slot keeps (taps - 1) x channels float32 inputs")
    for t in (q, k, v, beta, decay):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError("delta_prep: outputs are contiguous float32")
    _check(lib, lib.mhb_delta_prep(*_parts_args(proj.tensor, proj.nsplit, proj.split_stride), c_int(proj.tensor.stride(-2)),
                                   c_int(c0), c_int(b0), c_int(a0), _ptr(taps), _ptr(A_log), _ptr(dt_bias), _ptr(keep),
                                   c_longlong(keep.stride(0)), _ptr(tok_seg), _ptr(seg_slot), _ptr(positions), _ptr(q),
                                   _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), c_int(T), c_int(heads), c_int(kv_heads),
                                   c_int(dk), c_int(dv), c_int(ntaps), c_float(qscale), c_float(unit_eps), _stream()),
           "delta_prep")


def delta_conv_keep(proj, c0, keep, tok_seg, seg_slot, positions, *, channels, taps):
    """After delta_prep: every segment's last ``taps`` - 1 inputs (columns c0 .. of ``proj``) into its slot of ``keep``."""
    lib = build.load("deltarule")
    T, S = positions.shape[0], seg_slot.shape[0]
    _check(lib, lib.mhb_delta_conv_keep(*_parts_args(proj.tensor, proj.nsplit, proj.split_stride),
                                        c_int(proj.tensor.stride(-2)), c_int(c0), _ptr(keep), c_longlong(keep.stride(0)),
                                        _ptr(tok_seg), _ptr(seg_slot), _ptr(positions), c_int(T), c_int(S), c_int(channels),
                                        c_int(taps), _stream()), "delta_conv_keep")


def delta_scan(q, k, v, beta, decay, state, out, tok_seg, seg_slot, positions, *, heads, kv_heads, dk, dv, writable=True):
    """S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, token by token for every segment; ``state`` float32
    [slots, >= heads * dk * dv] (a slot's rows are [heads, dk, dv]); ``out`` float32 [T, heads * dv]."""
    lib = build.load("deltarule")
    T, S = out.shape[0], seg_slot.shape[0]
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[-1] < heads * dk * dv:
        raise KernelError(f"delta_scan: a slot holds float32 [{heads}, {dk}, {dv}]")
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("delta_scan: the output is contiguous float32")
    _check(lib, lib.mhb_delta_scan(_ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), _ptr(state),
                                   c_longlong(state.stride(0)), _ptr(out), _ptr(tok_seg), _ptr(seg_slot), _ptr(positions),
                                   c_int(T), c_int(S), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
                                   c_int(1 if writable else 0), _stream()), "delta_scan")
