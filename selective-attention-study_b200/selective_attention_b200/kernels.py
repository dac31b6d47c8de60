"""Selective Attention for B200: the reference's operator API over a C-ABI library of sm_100a kernels.

The names, signatures, return types and error behaviour follow the reference module
``src/selective_attention/kernels.py`` so that its callers (``mixers.py:86-98``, its kernel tests, its
bench script) can import this module instead:

    selective_attention(q, k, v, ...)            differentiable, fp32 output      (reference :669-703)
    selective_attention_forward(q, k, v, ...)    forward only, optional aux dict  (reference :526-605)
    selective_logits / selective_attention_reference   the dense paper listing    (reference :61-83)
    check_inputs, supported, _check_exempt, HEAD_DIMS, DTYPES, CARRY_M, HAS_TRITON

What differs underneath: the device work is done by ``libselective_attention_b200.so`` (CUDA-core fp32
engine for "ieee"/"tf32", tcgen05 tensor-core engine for bf16), the launch-tuning keywords are
validated but have no effect, the softmax statistics are kept as one log-sum-exp per row
(``aux["rmax"]`` holds it, ``aux["rden"]`` is all ones, so ``exp2(z - rmax) / rden`` still rebuilds the
attention), and ``aux["carry"]`` has a checkpoint every ``aux["carry_m"]`` query rows (32 or 128).
There is no fallback: without the library every kernel entry raises.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch
from torch.autograd.function import once_differentiable

from . import _lib

HAS_KERNELS = _lib.available()
HAS_TRITON = HAS_KERNELS          # the reference's tests and layer gate on this name
HEAD_DIMS = (16, 32, 64, 128)
DTYPES = (torch.float16, torch.bfloat16, torch.float32)
CARRY_M = 32                      # checkpoint spacing of the CUDA-core engine; the tensor-core engine uses 128
_BLOCK_QUANTUM = 32
_DTYPE_CODE = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}


# ---- the paper listing (dense; the oracle the kernels are tested against, never a fallback) ---------

def selective_logits(q: torch.Tensor, k: torch.Tensor, exempt: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """(L - F) as (B, H, T, T) fp32 with -inf above the diagonal, and the (B, T) selection totals."""
    exempt = _check_exempt(exempt)
    seq, dim = q.shape[-2], q.shape[-1]
    raw = torch.matmul(q.float(), k.float().transpose(-2, -1)) * (1.0 / math.sqrt(dim))
    idx = torch.arange(seq, device=q.device)
    future = idx[None, :] > idx[:, None]
    selectable = (idx[None, :] < idx[:, None]) & (idx[None, :] >= exempt)
    sel = torch.relu(raw[:, 0]) * selectable
    history = sel.cumsum(dim=-2) - sel
    return raw.masked_fill(future, float("-inf")) - history[:, None], sel.sum(dim=-2)


def selective_attention_reference(q, k, v, exempt: int = 1) -> torch.Tensor:
    """softmax(L - F) @ v in fp32, (B, H, T, D)."""
    return torch.matmul(torch.softmax(selective_logits(q, k, exempt)[0], dim=-1), v.float())


# ---- argument contract --------------------------------------------------------------------------------

def check_inputs(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    """ValueError / RuntimeError unless the kernels can take these tensors."""
    if not HAS_KERNELS:
        raise RuntimeError("the CUDA library is not built (python -m selective_attention_b200.build)")
    shapes = tuple(tuple(t.shape) for t in (q, k, v))
    if q.dim() != 4 or shapes[0] != shapes[1] or shapes[0] != shapes[2]:
        raise ValueError(f"q, k, v must all be (B, H, T, D); got {shapes[0]}, {shapes[1]}, {shapes[2]}")
    if not q.is_cuda or k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must be CUDA tensors on one device")
    for t in (q, k, v):
        if t.dtype not in DTYPES:
            raise ValueError(f"dtype must be float16, bfloat16 or float32; got {q.dtype}, {k.dtype}, {v.dtype}")
    if q.shape[3] not in HEAD_DIMS:
        raise ValueError(f"head_dim must be one of {HEAD_DIMS}; got {q.shape[3]}")
    if q.shape[2] < 1:
        raise ValueError("the sequence is empty")


def supported(q: torch.Tensor, k: torch.Tensor | None = None, v: torch.Tensor | None = None) -> bool:
    try:
        check_inputs(q, q if k is None else k, q if v is None else v)
        return True
    except (ValueError, RuntimeError):
        return False


def _check_exempt(exempt: int) -> int:
    if int(exempt) != exempt or exempt < 1:
        raise ValueError(f"exempt must be an integer >= 1 (position 0, <BOS>, is always exempt); got {exempt}")
    return int(exempt)


def _check_blocks(*blocks) -> None:
    for b in blocks:
        if b is not None and (int(b) != b or b < _BLOCK_QUANTUM or b % _BLOCK_QUANTUM):
            raise ValueError(f"block_m and block_n must be multiples of {_BLOCK_QUANTUM}")


def _check_bwd_group(group) -> None:
    if group not in (None, 1, 2):
        raise ValueError(f"bwd_group must be None, 1 or 2; got {group}")


def _lowp(dot_precision: str | None, dtype: torch.dtype) -> bool:
    """True: bf16 tensor-core operands.  None follows the dtype (bf16 -> "bf16", else "tf32")."""
    if dot_precision is None:
        dot_precision = "bf16" if dtype == torch.bfloat16 else "tf32"
    if dot_precision == "bf16":
        return True
    if dot_precision in ("tf32", "ieee"):
        return False       # both run as exact fp32 products here, which is inside the tf32 envelope
    raise ValueError(f"dot_precision must be None, 'bf16', 'tf32' or 'ieee', not {dot_precision!r}")


# ---- library plumbing ---------------------------------------------------------------------------------

def _strided(t: torch.Tensor, tc: bool) -> torch.Tensor:
    """The kernels take any batch/head/token strides with a contiguous last axis; the TMA path also
    needs 16-byte aligned rows."""
    ok = t.stride(3) == 1 or t.shape[3] == 1
    if ok and tc:
        es = t.element_size()
        ok = t.data_ptr() % 16 == 0 and all((s * es) % 16 == 0 for s in t.stride()[:3])
    return t if ok else t.contiguous()


def _engine(lowp: bool, head_dim: int, with_backward: bool) -> int:
    """Tensor-core engine for bf16 operands where it covers the call, else the CUDA-core engine."""
    if os.environ.get("SA_B200_ENGINE", "") == "simt":
        return _lib.ENGINE_SIMT
    if lowp and _lib.load().sa_engine_supports(_lib.ENGINE_TCGEN05, _lib.DTYPE_BF16, head_dim, int(with_backward)):
        return _lib.ENGINE_TCGEN05
    return _lib.ENGINE_SIMT


def _problem(q, k, v, engine: int, exempt: int, damp: int = 0, train_len: int = 0) -> _lib.Problem:
    b, h, t, d = q.shape
    p = _lib.Problem()
    p.struct_bytes = ctypes.sizeof(_lib.Problem)
    p.dtype = _DTYPE_CODE[q.dtype]
    p.engine = engine
    p.batch, p.heads, p.seq, p.head_dim = b, h, t, d
    p.exempt, p.damp, p.train_len = exempt, damp, max(int(train_len), 0)
    for field, ten in (("q_stride", q), ("k_stride", k), ("v_stride", v)):
        getattr(p, field)[:] = list(ten.stride()[:3])
    return p


def _selector_struct(q0: torch.Tensor, k0: torch.Tensor) -> _lib.Selector:
    s = _lib.Selector()
    s.struct_bytes = ctypes.sizeof(_lib.Selector)
    s.q0, s.k0 = q0.data_ptr(), k0.data_ptr()
    s.q0_stride[:] = [q0.stride(0), q0.stride(1)]
    s.k0_stride[:] = [k0.stride(0), k0.stride(1)]
    return s


def _check_selector(selector, q: torch.Tensor):
    """(q0, k0): the selection head's rows, (B, T, D) or (B, 1, T, D), on q's device."""
    if selector is None:
        return None
    try:
        q0, k0 = selector
    except (TypeError, ValueError):
        raise ValueError("selector must be a pair (q0, k0) of tensors") from None
    b, _, t, d = q.shape
    out = []
    for x in (q0, k0):
        if x.dim() == 4 and x.shape[1] == 1:
            x = x[:, 0]
        if tuple(x.shape) != (b, t, d):
            raise ValueError(f"selector tensors must all be (B, T, D) = {(b, t, d)}; got {tuple(x.shape)}")
        if x.device != q.device:
            raise ValueError("selector tensors must be CUDA tensors on q's device")
        if x.dtype not in DTYPES:
            raise ValueError(f"selector dtype must be float16, bfloat16 or float32; got {x.dtype}")
        out.append(x)
    return tuple(out)


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _prepare(q, k, v, lowp: bool):
    """Operand dtype of the engines: bf16 when the products run on bf16 operands, otherwise a common
    input dtype (the CUDA-core engine converts every element to fp32 as it loads it)."""
    if lowp:
        want = torch.bfloat16
    elif q.dtype == k.dtype == v.dtype:
        want = q.dtype
    else:
        want = torch.float32
    return tuple(t if t.dtype == want else t.to(want) for t in (q, k, v))


def _prepare_selector(selector, want: torch.dtype, tc: bool):
    if selector is None:
        return None
    out = []
    for x in selector:
        x = x if x.dtype == want else x.to(want)
        ok = x.stride(2) == 1
        if ok and tc:
            es = x.element_size()
            ok = x.data_ptr() % 16 == 0 and all((st * es) % 16 == 0 for st in x.stride()[:2])
        out.append(x if ok else x.contiguous())
    return tuple(out)


def _carry_rows_request(carry_rows):
    if carry_rows is None:
        env = os.environ.get("SA_B200_CARRY_ROWS", "")
        carry_rows = int(env) if env else None
    if carry_rows not in (None, 32, 128):
        raise ValueError(f"carry_rows must be None, 32 or 128; got {carry_rows}")
    return carry_rows


def _selection_carry32(q, k, sel, exempt: int, zero: bool):
    """Checkpoints every 32 queries (the reference's CARRY layout) from the CUDA-core selection pass."""
    lib = _lib.load()
    b, _, t, _ = q.shape
    alloc = torch.zeros if zero else torch.empty
    carry = alloc(b, lib.sa_carry_checkpoints(_lib.ENGINE_SIMT, t), t, device=q.device, dtype=torch.float32)
    total = torch.empty(b, t, device=q.device, dtype=torch.float32)
    prob = _problem(q, k, q, _lib.ENGINE_SIMT, exempt)
    sel_ref = ctypes.byref(_selector_struct(*sel)) if sel is not None else None
    with torch.cuda.device(q.device):
        st = lib.sa_selection_carry(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), sel_ref, carry.data_ptr(),
                                    total.data_ptr(), _stream(q.device))
    _lib.check("sa_selection_carry", st)
    return carry


def _forward(q, k, v, lowp: bool, exempt: int, damp: int, train_len: int, selector=None, zero_carry: bool = False,
             live_tiles: bool = False):
    lib = _lib.load()
    b, h, t, d = q.shape
    engine = _engine(lowp, d, False)
    if damp and engine == _lib.ENGINE_TCGEN05:
        engine = _lib.ENGINE_SIMT          # row-scaled F is an evaluation-only option of the CUDA-core engine
    tc = engine == _lib.ENGINE_TCGEN05
    q, k, v = (_strided(x, tc) for x in _prepare(q, k, v, lowp))
    sel = _prepare_selector(selector, q.dtype, tc)
    dev = q.device
    carry_m = lib.sa_carry_rows(engine)
    out = torch.empty(b, h, t, d, device=dev, dtype=torch.float32)
    lse2 = torch.empty(b, h, t, device=dev, dtype=torch.float32)
    alloc = torch.zeros if zero_carry else torch.empty
    carry = alloc(b, lib.sa_carry_checkpoints(engine, t), t, device=dev, dtype=torch.float32)
    total = torch.empty(b, t, device=dev, dtype=torch.float32)
    prob = _problem(q, k, v, engine, exempt, damp, train_len)
    sel_ref = ctypes.byref(_selector_struct(*sel)) if sel is not None else None
    table = None
    if live_tiles and tc:
        need = lib.sa_tile_table_bytes(ctypes.byref(prob))
        if need:
            table = torch.empty(need, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        st = lib.sa_forward_live_tiles(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), sel_ref,
                                       out.data_ptr(), None, lse2.data_ptr(), carry.data_ptr(), total.data_ptr(),
                                       table.data_ptr() if table is not None else None,
                                       table.numel() if table is not None else 0, _stream(dev))
    _lib.check("sa_forward", st)
    return out, lse2, carry, total, (q, k, v), sel, engine, carry_m, table


def selective_attention_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dot_precision: str | None = None,
    block_m: int | None = None,
    block_n: int = 32,
    return_aux: bool = False,
    num_warps: int = 4,
    num_stages: int | None = None,
    group: int | None = None,
    exempt: int = 1,
    *,
    damp: str = "none",
    train_len: int = 0,
    selector=None,
    carry_rows: int | None = None,
    skip_dead_tiles: bool = False,
):
    """Forward without autograd: fp32 (B, H, T, D).  With ``return_aux`` also a dict with ``rmax``
    (the row log-sum-exp in log2 units), ``rden`` (ones), ``carry``, ``carry_m`` and
    ``selected_total`` (B, T): the selection each key received from all T queries, i.e. the cached
    decode accumulator after this prefix.  ``damp`` ("none" | "linear" | "sqrt") with ``train_len``
    scales the history term of query i by min(1, train_len / (i + 1)) or its square root
    (evaluation only; the backward does not implement it).  block_m / block_n / num_warps /
    num_stages / group are accepted for signature compatibility and only validated.

    Beyond the reference's signature (keyword-only): ``selector=(q0, k0)`` takes the selection head's
    rows, (B, T, D), from outside q / k (for a call that holds only some heads of each sequence);
    ``carry_rows=32`` (or the environment variable SA_B200_CARRY_ROWS=32) returns ``aux["carry"]`` with the
    reference's checkpoint every 32 queries whichever engine ran (an extra selection pass on the CUDA
    cores); by default the spacing is the engine's own, reported in ``aux["carry_m"]``; ``skip_dead_tiles=True``
    leaves out the (query tile, key tile) pairs whose probabilities are all exactly zero (see
    ``selective_attention``)."""
    check_inputs(q, k, v)
    exempt = _check_exempt(exempt)
    lowp = _lowp(dot_precision, q.dtype)
    _check_blocks(block_m, block_n)
    if damp not in _lib.DAMP_CODES:
        raise ValueError(f"damp must be 'none', 'linear' or 'sqrt'; got {damp!r}")
    if _lib.DAMP_CODES[damp] and train_len < 1:
        raise ValueError("damp needs train_len (the trained context length)")
    selector = _check_selector(selector, q)
    carry_rows = _carry_rows_request(carry_rows) if return_aux else None
    out, lse2, carry, total, operands, sel, _, carry_m, table = _forward(
        q, k, v, lowp, exempt, _lib.DAMP_CODES[damp], train_len, selector=selector, zero_carry=return_aux,
        live_tiles=skip_dead_tiles)
    if not return_aux:
        return out
    b, h, t, _ = q.shape
    if carry_rows is not None and carry_rows != carry_m:
        if carry_rows != 32:
            raise ValueError("carry_rows=128 is only available where the tensor-core engine runs")
        carry, carry_m = _selection_carry32(operands[0], operands[1], sel, exempt, zero=True), 32
    aux = dict(rmax=lse2.view(b * h, t), rden=torch.ones(b * h, t, device=q.device, dtype=torch.float32),
               carry=carry[:, :(t + carry_m - 1) // carry_m], carry_m=carry_m, selected_total=total)
    if table is not None:       # [row, query tile, key tile] != 0 where the tile was computed (entries above the diagonal unused)
        nt = (t + 127) // 128
        aux["live_tiles"] = table[: b * h * nt * nt].view(b * h, nt, nt)
    return out, aux


def _backward_call(ctx, dout, dq0=None, dk0=None):
    q, k, v, out, lse2, carry = ctx.saved_tensors[:6]
    sel = tuple(ctx.saved_tensors[6:8]) if len(ctx.saved_tensors) > 6 else None
    lib = _lib.load()
    dev = q.device
    if dout.dtype not in _DTYPE_CODE:
        dout = dout.float()
    dout = dout.contiguous()
    engine = ctx.engine
    prob = _problem(q, k, v, engine, ctx.exempt)
    need = lib.sa_backward_workspace_bytes(ctypes.byref(prob))
    workspace = torch.empty(max(need, 1), device=dev, dtype=torch.uint8)
    dq, dk, dv = (torch.empty(q.shape, device=dev, dtype=q.dtype) for _ in range(3))
    sel_ref = ctypes.byref(_selector_struct(*sel)) if sel is not None else None
    table = getattr(ctx, "tile_table", None)
    with torch.cuda.device(dev):
        if table is not None:           # the forward left out dead tiles: the backward walks the same live ones
            descs = [_tensor_struct(x) for x in (dout, dq, dk, dv)]
            st = lib.sa_backward_live_tiles(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), sel_ref,
                                            out.data_ptr(), lse2.data_ptr(), carry.data_ptr(),
                                            *(ctypes.byref(x) for x in descs),
                                            dq0.data_ptr() if dq0 is not None else None,
                                            dk0.data_ptr() if dk0 is not None else None, workspace.data_ptr(), need,
                                            table.data_ptr(), _stream(dev))
        else:
            st = lib.sa_backward_selector(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), sel_ref,
                                          out.data_ptr(), lse2.data_ptr(), carry.data_ptr(), dout.data_ptr(),
                                          _DTYPE_CODE[dout.dtype], dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                          dq0.data_ptr() if dq0 is not None else None,
                                          dk0.data_ptr() if dk0 is not None else None, workspace.data_ptr(), need,
                                          _stream(dev))
    _lib.check("sa_backward", st)
    return dq, dk, dv


class _SelectiveAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, dot_precision, block_m, block_n, num_warps, bwd_block_n, bwd_num_warps,
                bwd_num_stages, group, bwd_group, num_stages, exempt, skip_dead_tiles=False):
        check_inputs(q, k, v)
        exempt = _check_exempt(exempt)
        lowp = _lowp(dot_precision, q.dtype)
        _check_blocks(block_m, block_n)
        out, lse2, carry, _, operands, _, engine, _, table = _forward(q, k, v, lowp, exempt, 0, 0,
                                                                      live_tiles=skip_dead_tiles)
        ctx.save_for_backward(*operands, out, lse2, carry)
        ctx.engine, ctx.exempt, ctx.bwd_group, ctx.tile_table = engine, exempt, bwd_group, table
        ctx.grad_dtypes = (q.dtype, k.dtype, v.dtype)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dout):
        _check_bwd_group(ctx.bwd_group)
        grads = _backward_call(ctx, dout)
        grads = tuple(g if g.dtype == want else g.to(want) for g, want in zip(grads, ctx.grad_dtypes))
        return grads + (None,) * 12


class _SelectiveAttentionSelectorFn(torch.autograd.Function):
    """The operator for a call that holds only some heads of each sequence: the selection head's rows come
    in as their own tensors (q0, k0), and the gradient that reaches them through the history term comes
    back as THEIR gradient, in fp32 precision before the cast, not folded into any head of q / k.  Ranks that
    share a sequence sum these partial gradients (all-reduce) like any replicated parameter's."""

    @staticmethod
    def forward(ctx, q, k, v, q0, k0, dot_precision, exempt, skip_dead_tiles=False):
        check_inputs(q, k, v)
        exempt = _check_exempt(exempt)
        lowp = _lowp(dot_precision, q.dtype)
        selector = _check_selector((q0, k0), q)
        out, lse2, carry, _, operands, sel, engine, _, table = _forward(q, k, v, lowp, exempt, 0, 0, selector=selector,
                                                                        live_tiles=skip_dead_tiles)
        ctx.save_for_backward(*operands, out, lse2, carry, *sel)
        ctx.engine, ctx.exempt, ctx.tile_table = engine, exempt, table
        ctx.grad_dtypes = (q.dtype, k.dtype, v.dtype)
        ctx.sel_shapes = (q0.shape, k0.shape, q0.dtype, k0.dtype)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dout):
        q = ctx.saved_tensors[0]
        b, _, t, d = q.shape
        dq0 = torch.empty(b, t, d, device=q.device, dtype=torch.float32)
        dk0 = torch.empty(b, t, d, device=q.device, dtype=torch.float32)
        grads = _backward_call(ctx, dout, dq0, dk0)
        grads = tuple(g if g.dtype == want else g.to(want) for g, want in zip(grads, ctx.grad_dtypes))
        q0_shape, k0_shape, q0_dtype, k0_dtype = ctx.sel_shapes
        return grads + (dq0.reshape(q0_shape).to(q0_dtype), dk0.reshape(k0_shape).to(k0_dtype), None, None, None)


def selective_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dot_precision: str | None = None,
    block_m: int | None = None,
    block_n: int = 32,
    num_warps: int = 4,
    bwd_block_n: int = 32,
    bwd_num_warps: int = 4,
    bwd_num_stages: int = 1,
    group: int | None = None,
    bwd_group: int | None = None,
    num_stages: int | None = None,
    exempt: int = 1,
    *,
    selector=None,
    skip_dead_tiles: bool = False,
) -> torch.Tensor:
    """Differentiable Selective Attention.  q / k / v: (B, H, T, D) CUDA tensors (fp16, bf16 or fp32;
    D in 16, 32, 64, 128; any strides).  Returns fp32 (B, H, T, D); gradients come back in the input
    dtypes.  dot_precision: None -> "bf16" for bf16 inputs, otherwise "tf32"; "ieee" and "tf32" both
    run exact fp32 products.  exempt: keys [0, exempt) are never selected (1 = <BOS>, the paper's rule).
    The remaining positional keywords are the reference's launch-tuning knobs: validated, otherwise unused.

    ``selector=(q0, k0)`` (keyword-only, beyond the reference's signature) shards the heads of a sequence:
    q / k / v hold any subset of its heads and q0 / k0, (B, T, D), are a replica of the selection head's rows.
    Gradients flow to q0 / k0 as this call's partial sums; sum them over the calls that share the selector.

    ``skip_dead_tiles=True`` (keyword-only, beyond the reference, tensor-core engine, T <= 131072): after the selection
    pass, 128 x 128 (query tile, key tile) pairs in which every probability is exactly zero -- far queries of keys that
    many later queries have selected against; decided by a rigorous bound, never by a threshold on the result -- are
    left out of the forward and the backward.  The results are those of the full computation (the forward bit for
    bit); the time saved depends on how strongly the data selects."""
    if selector is not None:
        _check_blocks(block_m, block_n)
        _check_bwd_group(bwd_group)
        q0, k0 = selector
        return _SelectiveAttentionSelectorFn.apply(q, k, v, q0, k0, dot_precision, exempt, bool(skip_dead_tiles))
    return _SelectiveAttentionFn.apply(q, k, v, dot_precision, block_m, block_n, num_warps, bwd_block_n,
                                       bwd_num_warps, bwd_num_stages, group, bwd_group, num_stages, exempt,
                                       bool(skip_dead_tiles))


# ---- layout-fused form for a model's attention layer -------------------------------------------------

def _tensor_struct(t: torch.Tensor) -> _lib.Tensor:
    """sa_tensor for a (B, H, T, D) view with a contiguous last axis."""
    d = _lib.Tensor()
    d.ptr, d.dtype = t.data_ptr(), _DTYPE_CODE[t.dtype]
    d.stride[:] = list(t.stride()[:3])
    return d


def packed_supported(qkv: torch.Tensor) -> bool:
    """True when ``selective_attention_packed`` can take this fused projection output: bf16 on a CUDA device,
    (B, T, 3, H, D) with D = 64 or 128, contiguous, and the library built."""
    return (HAS_KERNELS and qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 5 and qkv.shape[2] == 3
            and qkv.shape[4] in (64, 128) and qkv.is_contiguous() and os.environ.get("SA_B200_ENGINE", "") != "simt")


class _SelectiveAttentionPackedFn(torch.autograd.Function):
    """The operator between a model's fused QKV projection and its output projection, without the copies around it:
    q, k, v are read in place from the (B, T, 3, H, D) projection output (strided TMA descriptors), the result is
    written by the forward kernel as (B, T, H * D) in the activation dtype, the cotangent is read in that layout,
    and dq, dk, dv are written by the backward's kernels into one (B, T, 3, H, D) gradient."""

    @staticmethod
    def forward(ctx, qkv, exempt, skip_dead_tiles=False):
        exempt = _check_exempt(exempt)
        lib = _lib.load()
        b, t, _, h, d = qkv.shape
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))          # (B, H, T, D) views
        dev = qkv.device
        engine = _lib.ENGINE_TCGEN05
        out = torch.empty(b, h, t, d, device=dev, dtype=torch.float32)       # kept for the backward's row sums
        merged = torch.empty(b, t, h * d, device=dev, dtype=qkv.dtype)
        lse2 = torch.empty(b, h, t, device=dev, dtype=torch.float32)
        carry = torch.empty(b, lib.sa_carry_checkpoints(engine, t), t, device=dev, dtype=torch.float32)
        total = torch.empty(b, t, device=dev, dtype=torch.float32)
        prob = _problem(q, k, v, engine, exempt)
        low = _tensor_struct(merged.view(b, t, h, d).transpose(1, 2))
        table = None
        need = lib.sa_tile_table_bytes(ctypes.byref(prob)) if skip_dead_tiles else 0
        if need:
            table = torch.empty(need, device=dev, dtype=torch.uint8)
        with torch.cuda.device(dev):
            st = lib.sa_forward_live_tiles(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
                                           out.data_ptr(), ctypes.byref(low), lse2.data_ptr(), carry.data_ptr(),
                                           total.data_ptr(), table.data_ptr() if need else None, need, _stream(dev))
        _lib.check("sa_forward_fused", st)
        ctx.save_for_backward(qkv, out, lse2, carry)
        ctx.exempt, ctx.tile_table = exempt, table
        return merged

    @staticmethod
    @once_differentiable
    def backward(ctx, d_merged):
        qkv, out, lse2, carry = ctx.saved_tensors
        lib = _lib.load()
        b, t, _, h, d = qkv.shape
        dev = qkv.device
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        d_merged = d_merged.to(qkv.dtype)
        if not d_merged.is_contiguous():
            d_merged = d_merged.contiguous()
        d_qkv = torch.empty_like(qkv)
        dq, dk, dv = (d_qkv[:, :, i].transpose(1, 2) for i in range(3))
        prob = _problem(q, k, v, _lib.ENGINE_TCGEN05, ctx.exempt)
        need = lib.sa_backward_workspace_bytes(ctypes.byref(prob))
        workspace = torch.empty(max(need, 1), device=dev, dtype=torch.uint8)
        descs = [_tensor_struct(x) for x in (d_merged.view(b, t, h, d).transpose(1, 2), dq, dk, dv)]
        table = ctx.tile_table
        with torch.cuda.device(dev):
            st = lib.sa_backward_live_tiles(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
                                            out.data_ptr(), lse2.data_ptr(), carry.data_ptr(),
                                            *(ctypes.byref(x) for x in descs), None, None, workspace.data_ptr(), need,
                                            table.data_ptr() if table is not None else None, _stream(dev))
        _lib.check("sa_backward_fused", st)
        return d_qkv, None, None


def selective_attention_packed(qkv: torch.Tensor, exempt: int = 1, *, skip_dead_tiles: bool = False) -> torch.Tensor:
    """Differentiable Selective Attention on a fused projection output.  qkv: (B, T, 3, H, D) bf16, contiguous
    (``packed_supported``); returns (B, T, H * D) bf16, ready for the output projection.  Head 0 selects for all
    heads.  Same arithmetic as ``selective_attention`` on the three (B, H, T, D) views; what is saved is every
    copy between the projections and the kernels.  ``skip_dead_tiles``: as in ``selective_attention``."""
    if not packed_supported(qkv):
        raise ValueError("qkv must be a contiguous bf16 CUDA tensor (B, T, 3, H, 64 or 128); use selective_attention otherwise")
    return _SelectiveAttentionPackedFn.apply(qkv, exempt, bool(skip_dead_tiles))


# ---- cached decode ------------------------------------------------------------------------------------

def prefill_extend(cache: dict, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, exempt: int = 1, *,
                   skip_dead_tiles: bool = False) -> torch.Tensor:
    """Continues a prefill: appends a chunk of new tokens to the cache and returns their outputs, (B, H, Tn, D)
    fp32, as the full forward over cached + new tokens would give them; ``cache["selected"]`` and ``cache["len"]``
    move on to the new length.  (The reference prefills from position 0 only and then decodes token by token,
    ``mixers.py:105-130``; chunked prefill is what a serving loop does with a long prompt.)

    cache: {"k", "v": (B, H, capacity, D) contiguous bf16, "len": int, "selected": (B, G, capacity) fp32} with G = 1
    (head 0 selects) or G = H (every head its own selector).  q, k, v: (B, H, Tn, D).  bf16 operands on the
    tensor-core engine only (head_dim 64 or 128).  ``skip_dead_tiles``: as in ``selective_attention``; the part of
    the cache whose probabilities are all exactly zero for the new queries is not read."""
    lib = _lib.load()
    exempt = _check_exempt(exempt)
    kc, vc, selected = cache["k"], cache["v"], cache["selected"]
    b, h, cap, d = kc.shape
    cached, tn = int(cache["len"]), q.shape[2]
    total_len = cached + tn
    if total_len > cap:
        raise ValueError("prefill past the cache capacity (context_length)")
    if tuple(q.shape) != (b, h, tn, d) or k.shape != q.shape or v.shape != q.shape:
        raise ValueError(f"q, k, v must all be (B, H, Tn, D) matching the cache; got {tuple(q.shape)}")
    groups = selected.shape[1]
    if not (kc.is_cuda and kc.dtype == torch.bfloat16 and vc.dtype == torch.bfloat16 and kc.is_contiguous()
            and vc.is_contiguous() and selected.is_contiguous() and selected.dtype == torch.float32
            and d in (64, 128) and groups in (1, h)):
        raise ValueError("prefill_extend needs a contiguous bf16 CUDA cache with head_dim 64 or 128 and one selector "
                         "per sequence or per head")
    if cached == 0:
        raise ValueError("the cache is empty: use selective_attention_forward(return_aux=True) for the first chunk")
    kc[:, :, cached:total_len] = k
    vc[:, :, cached:total_len] = v
    if cache.get("key_norms") is not None:
        cache["key_norms"][:, :, cached:total_len] = key_norms(k.to(kc.dtype))
    qn = q.to(torch.bfloat16)
    if groups == h and h > 1:             # every head is its own one-head sequence
        qn = qn.reshape(b * h, 1, tn, d)
        kv, vv = kc.view(b * h, 1, cap, d), vc.view(b * h, 1, cap, d)
    else:
        kv, vv = kc, vc
    qn = _strided(qn, True)
    bb, hh = qn.shape[0], qn.shape[1]
    dev = kc.device
    engine = _lib.ENGINE_TCGEN05
    out = torch.empty(bb, hh, tn, d, device=dev, dtype=torch.float32)
    lse2 = torch.empty(bb, hh, tn, device=dev, dtype=torch.float32)
    carry = torch.empty(bb, lib.sa_carry_checkpoints(engine, total_len), total_len, device=dev, dtype=torch.float32)
    total = torch.empty(bb, total_len, device=dev, dtype=torch.float32)
    prob = _problem(qn, kv, vv, engine, exempt)
    prob.seq = total_len
    need = lib.sa_tile_table_bytes(ctypes.byref(prob)) if skip_dead_tiles else 0
    table = torch.empty(need, device=dev, dtype=torch.uint8) if need else None
    with torch.cuda.device(dev):
        st = lib.sa_prefill_extend_live_tiles(ctypes.byref(prob), cached, qn.data_ptr(), kv.data_ptr(), vv.data_ptr(),
                                              selected.data_ptr(), cap, out.data_ptr(), lse2.data_ptr(),
                                              carry.data_ptr(), total.data_ptr(),
                                              table.data_ptr() if need else None, need, _stream(dev))
    _lib.check("sa_prefill_extend", st)
    selected.view(bb, cap)[:, :total_len] = total
    cache["len"] = total_len
    return out.view(b, h, tn, d)


def key_norms(k: torch.Tensor) -> torch.Tensor:
    """|k_j| of every key, fp32, for a decode cache that leaves out dead keys (``cache["key_norms"]``)."""
    return k.float().norm(dim=-1)


def decode_step(cache: dict, q1: torch.Tensor, k1: torch.Tensor, v1: torch.Tensor, exempt: int = 1) -> torch.Tensor:
    """One cached decode step on the device (the reference does this with PyTorch ops,
    ``mixers.py:115-130`` and ``model.py:86-93``).

    cache: {"k", "v": (B, H, capacity, D) contiguous, "len": int, "selected": (B, G, capacity) fp32}.
    q1, k1, v1: (B, H, 1, D).  Appends k1 / v1 at ``len``, returns y (B, H, 1, D) fp32 and then adds the
    new query's own selection to ``selected`` in place.  G selectors: heads in G contiguous runs, the
    first head of a run selects.

    When the cache also holds ``"key_norms"`` (B, H, capacity) fp32 (``key_norms(k)`` of the cached keys; the slot's
    ``begin_cache(..., live_keys=True)`` creates it), the step leaves out the part of the cache whose weights are
    below 2^-150 for this query and keeps the norms up to date."""
    lib = _lib.load()
    exempt = _check_exempt(exempt)
    kc, vc, selected = cache["k"], cache["v"], cache["selected"]
    b, h, cap, d = kc.shape
    length = int(cache["len"])
    if length >= cap:
        raise ValueError("decode step past the cache capacity (context_length)")
    if not (kc.is_cuda and kc.is_contiguous() and vc.is_contiguous() and selected.is_contiguous()):
        raise ValueError("the cache must be contiguous CUDA tensors")
    if kc.dtype not in _DTYPE_CODE or vc.dtype != kc.dtype or selected.dtype != torch.float32:
        raise ValueError("cache dtype must be float16, bfloat16 or float32 with fp32 `selected`")
    if d not in HEAD_DIMS:
        raise ValueError(f"head_dim must be one of {HEAD_DIMS}; got {d}")
    groups = selected.shape[1]
    q1, k1, v1 = (t.reshape(b, h, d) for t in (q1, k1, v1))
    q1, k1, v1 = (t if (t.dtype == kc.dtype and t.is_contiguous()) else t.to(kc.dtype).contiguous() for t in (q1, k1, v1))
    dev = kc.device
    y = torch.empty(b, h, 1, d, device=dev, dtype=torch.float32)
    need = lib.sa_decode_workspace_bytes(b, h, groups, length, d)
    ws = cache.get("_workspace")                  # scratch of the step, kept with the cache and grown when needed
    if ws is None or ws.numel() < need or ws.device != dev:
        ws = torch.empty(max(2 * need, 1 << 16), device=dev, dtype=torch.uint8)
        cache["_workspace"] = ws
    norms = cache.get("key_norms")
    if norms is not None and not (norms.is_cuda and norms.dtype == torch.float32 and norms.is_contiguous()
                                  and tuple(norms.shape) == (b, h, cap)):
        raise ValueError("cache['key_norms'] must be a contiguous fp32 CUDA tensor (B, H, capacity)")
    with torch.cuda.device(dev):
        st = lib.sa_decode_step_live_keys(_DTYPE_CODE[kc.dtype], b, h, groups, length, cap, d, exempt, q1.data_ptr(),
                                          k1.data_ptr(), v1.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                          selected.data_ptr(), norms.data_ptr() if norms is not None else None,
                                          y.data_ptr(), ws.data_ptr(), need, _stream(dev))
    _lib.check("sa_decode_step", st)
    cache["len"] = length + 1
    return y
