"""The kernel namespace that parts call: tensors in, tensors out, CUDA underneath.

Every function launches hand-written sm_100a kernels from `csrc/` on the current stream.
Matrix products of the bfloat16 path go to cuBLAS through `torch.mm`, where tamnd/fastmlx
calls its library's matmul (compute/models/qwen3_forward.go:111-115 -> mlxgo/binding_cgo.go:
324-328); the 32-bit path uses its own fixed-order kernel and never a reduced-precision
matrix mode.  Nothing here runs on the CPU.
"""
from __future__ import annotations

import torch

from . import lib as _lib
from .lib import KernelError, call, load, loaded_libraries


def launch_count() -> int:
    """Calls into the package's CUDA libraries so far (a graph replay is counted by its owner)."""
    return _lib.launches

F32, BF16 = 0, 1
BAD_TOKEN, BAD_SLOT, BAD_PAGE, BAD_ROW = 1, 2, 3, 4


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {t.dtype}")


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle.  A step makes a hundred and more launches, and building a
    torch.cuda.Stream object for each cost about 5 us of host time per launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


# ----------------------------------------------------------------------------- rows
def gather_rows(table: torch.Tensor, ids: torch.Tensor, status, code: int = BAD_ROW) -> torch.Tensor:
    _need_cuda(table, ids)
    assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    n, d = ids.numel(), table.shape[1]
    out = torch.empty((n, d), dtype=table.dtype, device=table.device)
    call("common", "fmx_gather_rows", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, d, table.shape[0],
         _dt(table), _ptr(status), code, _stream())
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, status, out_dtype=None) -> torch.Tensor:
    """Rows of the table; a table stored in 32-bit can feed bfloat16 activations (rounded here)."""
    if out_dtype == torch.bfloat16 and table.dtype == torch.float32:
        _need_cuda(table, ids)
        assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
        n, d = ids.numel(), table.shape[1]
        out = torch.empty((n, d), dtype=torch.bfloat16, device=table.device)
        call("common", "fmx_gather_rows_f32_to_bf16", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, d,
             table.shape[0], _ptr(status), BAD_TOKEN, _stream())
        return out
    return gather_rows(table, ids, status, BAD_TOKEN)


def add_rmsnorm(x, residual, weight: torch.Tensor, eps: float, stream_dtype=None, out_dtype=None):
    """-> (norm(residual + x) * weight, residual + x); the sum replaces `residual` in place.
    Without a residual, x is the stream's first value: it is returned as the stream, as it is or,
    when `stream_dtype` is float32 beside bfloat16 activations, as a 32-bit copy that the later
    sums then never round.  x may be None when there is a residual (the stream itself is
    normalised; `out_dtype` then names the activations' type)."""
    _need_cuda(x, residual, weight)
    assert weight.dtype == torch.float32
    ref = x if x is not None else residual
    assert ref is not None and ref.dim() == 2 and ref.is_contiguous()
    act = x.dtype if x is not None else (out_dtype or residual.dtype)
    init = 0
    if residual is None and stream_dtype is not None and stream_dtype != act:
        residual = torch.empty(ref.shape, dtype=stream_dtype, device=ref.device)
        init = 1
    assert residual is None or (residual.shape == ref.shape and residual.is_contiguous())
    out = torch.empty(ref.shape, dtype=act, device=ref.device)
    call("common", "fmx_add_rmsnorm", _ptr(x), _ptr(residual), weight.data_ptr(), out.data_ptr(), ref.shape[0], ref.shape[1],
         float(eps), _dt(out), _dt(residual) if residual is not None else _dt(out), init, _stream())
    return out, (residual if residual is not None else x)


def silu_mul(gate_up: torch.Tensor, block: int | None = None) -> torch.Tensor:
    """silu(gate) * up over rows of 2 I values laid out in blocks of `block` gates followed by
    their `block` ups (block = I, the default: all gates, then all ups)."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    call("common", "fmx_silu_mul", gate_up.data_ptr(), out.data_ptr(), rows, inter, int(block or inter), _dt(gate_up),
         _stream())
    return out


def act_mul(gate_up: torch.Tensor, kind: str, block: int | None = None) -> torch.Tensor:
    """act(gate) * up like `silu_mul`, with act = "silu" or "gelu_tanh" (the tanh form of gelu), in 32-bit."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0 and kind in ("silu", "gelu_tanh")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    call("common", "fmx_act_mul", gate_up.data_ptr(), out.data_ptr(), rows, inter, int(block or inter), ACTIVATIONS[kind],
         _dt(gate_up), _stream())
    return out


# ----------------------------------------------------------------------------- matrix products
def gemm_simple(x, w, bias, out_dtype) -> torch.Tensor:
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    call("common", "fmx_gemm_simple", x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
         x.stride(0), w.stride(0), out.stride(0), _dt(x), _dt(w), _dt(out), _stream())
    return out


_tc_status: dict = {}
_props: dict = {}


def _dev_index(device) -> int:
    device = torch.device(device)
    return device.index if device.index is not None else torch.cuda.current_device()


def num_sms(device=None) -> int:
    """Multiprocessors of the device (148 on a B200; fewer under a partition), read once per
    device.  Where no device is visible (host-side arithmetic in tests) a B200's count."""
    if not torch.cuda.is_available():
        return 148
    i = _dev_index(device if device is not None else "cuda")
    n = _props.get(i)
    if n is None:
        n = _props[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return n


def set_status_word(device, status: torch.Tensor) -> None:
    """The word in which kernels called through `linear` report trouble (a bounded wait that
    ran out): the engine registers its own, so that one read after a step covers them."""
    _tc_status[_dev_index(device)] = status


def _status_word(device):
    st = _tc_status.get(_dev_index(device))
    if st is None:
        st = _tc_status[_dev_index(device)] = torch.zeros(4, dtype=torch.int32, device=device)
    return st


# Which kernel multiplies, by the rows M of x (one path per class, no switch):
#   M <= 16                    whole-K weight-streaming kernel (`gemv`), except the vocabulary-sized head
#   M >= 128, full rounds      tcgen05 kernel (`gemm_tcgen05`)
#   everything else in bf16    the library (cuBLAS through torch.mm), as tamnd/fastmlx calls its library's matmul
#   32-bit or mixed types      fixed-order FMA kernel (`gemm_simple`)
GEMV_MAX_ROWS = 16
LIBRARY_MIN_FEATURES = 65536     # from this many output features on (the vocabulary) the library's product streams best
TC_MIN_ROWS = 128
GATE_UP_BLOCK = 128              # gate/up rows of a fused weight alternate in blocks of this many
EPI_PLAIN, EPI_SILU_MUL, EPI_RESIDUAL, EPI_RELU2 = 0, 1, 2, 3
EPI_GELU_MUL = 6                 # the gated epilogue with the tanh form of gelu on the gate
GEMV_GATE_GELU = 1 << 20         # added to a gated whole-K product's block size: gelu on the gate instead of silu


def _bf16_operands(x, w) -> bool:
    """bfloat16 operands laid out as the tensor-core kernels read them (16-byte rows)."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > 0
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def can_gemv(x, w) -> bool:
    """May this product run on the whole-K kernel of decode steps?"""
    return _bf16_operands(x, w) and x.shape[0] <= GEMV_MAX_ROWS


def gemv(x, w, bias=None, out_dtype=torch.bfloat16, residual=None, block: int = 0, out=None, wide=None, warps=None,
         act: str | None = None):
    """x[M <= 16, K] @ w[N, K]^T, one block per `wide` (8, 16, 32) output features and the whole of K:
    nothing is summed across blocks.  residual [M, n_out] is added to the product (out may be
    the residual itself).  block > 0: w's rows alternate in blocks of `block` gate rows and
    their up rows, and the result is silu(gate) * up, [M, N/2] (with act="gelu_tanh": gelu(gate) * up).  act (relu2,
    gelu_tanh, silu) without blocks: the activation of the product (and bias), in the same pass; `out` may be a slice
    of a wider buffer."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if block else N
    if act is not None and block:
        assert block > 0 and act in ("silu", "gelu_tanh") and out_dtype == torch.bfloat16
        block = int(block) + (GEMV_GATE_GELU if act == "gelu_tanh" else 0)
    elif act is not None:
        assert out_dtype == torch.bfloat16
        block = -1 - ACTIVATIONS[act]
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    # wide / warps left open: the library plans them (`fmx_gemv_plan_width`, `fmx_gemv_plan_warps`)
    call("bf16", "fmx_gemv", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _ptr(bias), _ptr(residual),
         residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0), M, N, K, _dt(out), int(block),
         int(wide or 0), int(warps or 0), _stream())
    return out


_greedy_ws: dict = {}


def greedy_workspace(device):
    """The greedy head's 16 best-so-far words and its ticket, one pair per device, made once
    (captured graphs hold their addresses); zero between launches."""
    ws = _greedy_ws.get(_dev_index(device))
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the greedy head's workspace must exist before a CUDA graph is captured")
        ws = _greedy_ws[_dev_index(device)] = (torch.zeros(16, dtype=torch.int64, device=device),
                                               torch.zeros(1, dtype=torch.int32, device=device))
    return ws


GREEDY_HEAD_MAX_ROWS = 8      # beyond, the library's product followed by the split argmax is the faster head


def can_greedy_head(x, w) -> bool:
    """Should the output head choose greedily in the same pass (no logits written)?  Up to 8
    rows (128,256 x 2,048: 84 us against 86 for the library's product and the argmax kernel; at
    16 rows 101 against 88)."""
    return _bf16_operands(x, w) and x.shape[0] <= GREEDY_HEAD_MAX_ROWS


def greedy_head(x, w) -> torch.Tensor:
    """argmax over n of x[m] . w[n]^T for at most 16 rows, the lowest index on ties: the head of
    a decode step whose rows all choose greedily.  The weight streams once; every block keeps the
    best of its 32 logits per row, and the rows' bests meet in one 64-bit atomicMax each.
    -> int32 [M]."""
    M, K = x.shape
    ids = torch.empty(M, dtype=torch.int32, device=x.device)
    best, ticket = greedy_workspace(x.device)
    call("bf16", "fmx_gemv_argmax", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), ids.data_ptr(), best.data_ptr(),
         ticket.data_ptr(), M, w.shape[0], K, _stream())
    return ids


def tile_width(M: int, N: int, sms: int = 148) -> int:
    """The tile width (of 128, 192, 256) whose tiles fill the SMs' rounds best, as the
    tensor-core library plans it (`fmx_gemm_tcgen05_plan_width`)."""
    return int(load("tc").fmx_gemm_tcgen05_plan_width(int(M), int(N), int(sms)))


def tc_fills_the_gpu(M: int, N: int, sms: int = 148) -> bool:
    """Does a product of these sizes fill the GPU on the tensor-memory kernel (else the
    library's product, which splits K, is the faster one)?  The library's own plan
    (`fmx_gemm_tcgen05_plan_fills`)."""
    return bool(load("tc").fmx_gemm_tcgen05_plan_fills(int(M), int(N), int(sms)))


def can_tc(x, w, bias=None, out_dtype=torch.bfloat16, epilogue: int = EPI_PLAIN) -> bool:
    """Does this product go to the tcgen05 kernel?  Only with an epilogue of its own (SiLU-mul over
    blocks of gate and up rows, or a residual), bfloat16 operands, at least 128 rows and tiles
    that fill the GPU.  A plain product runs in the library: with the weights coming from HBM it
    is ahead of the one-CTA kernel at every size measured (2048 x 2048 x 8192: 47 us against 52)."""
    return (epilogue != EPI_PLAIN and _bf16_operands(x, w) and bias is None and out_dtype == torch.bfloat16
            and x.shape[0] >= TC_MIN_ROWS and (epilogue not in (EPI_SILU_MUL, EPI_GELU_MUL) or w.shape[0] % (2 * GATE_UP_BLOCK) == 0)
            and tc_fills_the_gpu(x.shape[0], w.shape[0], num_sms(x.device)))


def gemm_tcgen05(x, w, status=None, epilogue: int = EPI_PLAIN, residual=None, bn: int | None = None, out=None) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory).
    epilogue EPI_SILU_MUL: w's rows come in blocks of bn/2 gate rows then bn/2 up rows, and the
    result is silu(gate) * up, [M, N/2] (EPI_GELU_MUL: the tanh form of gelu on the gate); EPI_RESIDUAL: residual + product; EPI_RELU2: the square of the
    product's positive part.  `out` may be a slice of a wider buffer."""
    M, K = x.shape
    N = w.shape[0]
    sms = num_sms(x.device)
    n_out = N // 2 if epilogue in (EPI_SILU_MUL, EPI_GELU_MUL) else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (M, n_out)
    call("tc", "fmx_gemm_tcgen05", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
         _ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K, int(bn or 0), epilogue, sms,
         _ptr(status if status is not None else _status_word(x.device)), _stream())
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias, out_dtype) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T (+ bias) -> [M, N] in `out_dtype`, accumulated in 32-bit."""
    _need_cuda(x, w, bias)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], (x.shape, w.shape)
    assert x.stride(1) == 1 and w.stride(1) == 1
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[0] == 0:
        return gemm_simple(x, w, bias, out_dtype)
    if can_gemv(x, w) and (w.shape[0] < LIBRARY_MIN_FEATURES or bias is not None):
        return gemv(x, w, bias, out_dtype)
    wt = w.t()
    if bias is not None:
        if out_dtype == torch.bfloat16:
            return torch.addmm(bias.to(torch.bfloat16), x, wt)
        return gemm_simple(x, w, bias, out_dtype)
    return torch.mm(x, wt) if out_dtype == torch.bfloat16 else torch.mm(x, wt, out_dtype=out_dtype)


# ----------------------------------------------------------------------------- positions and cache
def rope_kv_write(qkv, positions, inv_freq, rotary_dim, traditional, slot_mapping, kv, nh, nkv, hd, status) -> None:
    """Rotate q and k of qkv[T, (nh + 2 nkv) hd] in place and store k, v at slot_mapping."""
    _need_cuda(qkv, positions, inv_freq, slot_mapping, kv)
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and positions.dtype == torch.int32
    if kv is not None:
        assert kv.is_contiguous() and kv.dtype == qkv.dtype and kv.shape[1] == 2 and kv.shape[2] == nkv \
            and kv.shape[4] == hd and slot_mapping is not None and slot_mapping.dtype == torch.int64
        num_pages, page_size = kv.shape[0], kv.shape[3]
    else:
        num_pages, page_size = 0, 1
    call("common", "fmx_rope_kv_write", qkv.data_ptr(), positions.data_ptr(), _ptr(inv_freq), _ptr(slot_mapping),
         _ptr(kv), qkv.shape[0], nh, nkv, hd, int(rotary_dim), int(bool(traditional)), page_size, num_pages,
         qkv.stride(0), _dt(qkv), _ptr(status), _stream())


def paged_attention_simple(qkv, kv, ctx, group, nh, nkv, hd, scale, window) -> torch.Tensor:
    T = qkv.shape[0]
    out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    bt = group.block_tables
    call("common", "fmx_paged_attention_simple", qkv.data_ptr(), qkv.stride(0), kv.data_ptr(), bt.data_ptr(),
         bt.stride(0), ctx.token_row.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), T, nh, nkv, hd,
         kv.shape[3], kv.shape[0], float(scale), int(window), bt.shape[0], _dt(qkv), _ptr(ctx.status), _stream())
    return out


def qk_prepare(qkv, positions, inv_freq, rotary_dim, traditional, norm_eps, slot_mapping, kv, nh, nkv, hd, vd,
               status, bias=None, q_weight=None, k_weight=None, norm_first: bool = False, whole: bool = False,
               values_from_keys: bool = False) -> torch.Tensor:
    """Queries and keys of qkv[T, nh*hd + nkv*hd + nkv*vd] made ready for attention: rotated over their
    first `rotary_dim` dimensions, then (norm_eps not None) each head divided by its root mean square;
    keys and values are stored at slot_mapping in pages that hold [nkv, page, hd] keys and then
    [nkv, page, vd] values.  -> the queries in 32-bit, [T, nh*hd].  qkv may be of another type than the
    cache (a product that leaves in 32-bit beside bfloat16 pages).  `bias` (32-bit, a whole row's) is added
    first; `q_weight` / `k_weight` ([hd], 32-bit) multiply the normalised heads; `norm_first` normalises
    before the rotation instead of after it.  `whole` (with `norm_first`): q and k are each divided by the root mean
    square of their whole projection, all heads at once, and the weights are that wide ([nh*hd], [nkv*hd]);
    `values_from_keys`: qkv holds q | k only, and a token's values are its keys as projected (vd = hd)."""
    _need_cuda(qkv, positions, inv_freq, slot_mapping, kv, bias, q_weight, k_weight)
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and positions.dtype == torch.int32
    T = qkv.shape[0]
    q = torch.empty((T, nh * hd), dtype=torch.float32, device=qkv.device)
    if kv is not None:
        assert kv.is_contiguous() and slot_mapping is not None and slot_mapping.dtype == torch.int64
        num_pages = kv.shape[0]
        page_size = kv[0].numel() // (nkv * (hd + vd))
    else:
        num_pages, page_size = 0, 1
    for v in (bias, q_weight, k_weight):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous())
    if whole or values_from_keys:
        assert norm_first or norm_eps is None, "the norm over the whole projection comes before the rotation"
        call("common", "fmx_qk_prepare_whole", qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), _ptr(inv_freq),
             _ptr(slot_mapping), q.data_ptr(), _ptr(kv), T, nh, nkv if kv is not None else 0, hd, vd, int(rotary_dim),
             int(bool(traditional)), -1.0 if norm_eps is None else float(norm_eps), page_size, num_pages, _dt(qkv),
             _dt(kv) if kv is not None else _dt(qkv), _ptr(bias), _ptr(q_weight), _ptr(k_weight), int(bool(values_from_keys)),
             _ptr(status), _stream())
        return q
    call("common", "fmx_qk_prepare_ex", qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), _ptr(inv_freq),
         _ptr(slot_mapping), q.data_ptr(), _ptr(kv), T, nh, nkv if kv is not None else 0, hd, vd, int(rotary_dim),
         int(bool(traditional)), -1.0 if norm_eps is None else float(norm_eps), page_size, num_pages, _dt(qkv),
         _dt(kv) if kv is not None else _dt(qkv), _ptr(bias), _ptr(q_weight), _ptr(k_weight), int(bool(norm_first)),
         _ptr(status), _stream())
    return q


def paged_attention_general(q, kv, ctx, group, nh, nkv, hd, vd, scale, softcap, window, page_size, out=None,
                            keep_first: int = 0, values_are_keys: bool = False, gate=None, chunk: int = 0, sinks=None,
                            gate_group: int = 1) -> torch.Tensor:
    """Attention with 32-bit scores and weights, one warp per (token, head): queries q[T, nh*hd] of their own
    type over pages of [nkv, page, hd] keys and [nkv, page, vd] values; scores are capped by
    softcap * tanh(s / softcap) where softcap > 0.  `out` may be a slice of a wider buffer.  -> [T, nh*vd].
    `keep_first`: beside a window, a request's first tokens that stay visible; `values_are_keys`: pages of keys
    only, which are the values too; `gate` (32-bit [T, nh*vd], rows may be a slice): the output is multiplied
    element by element with sigmoid(gate) (`gate_group` g > 1: one gate value per g output elements).  `chunk` c > 0
    instead of a window: a query sees the keys of its own run of c positions, runs counted from position 0.  `sinks`
    (32-bit [nh]): one more term exp(sink) per head in the softmax's denominator, with no value."""
    _need_cuda(q, kv, gate, sinks)
    assert kv.is_contiguous() and q.stride(1) == 1
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, nh * vd), dtype=kv.dtype, device=q.device)
    assert out.dtype == kv.dtype and out.stride(1) == 1 and out.shape == (T, nh * vd)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (T, nh * vd // gate_group))
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == nh)
    bt = group.block_tables
    if chunk or sinks is not None or gate_group != 1:
        call("common", "fmx_paged_attention_masked_ex", q.data_ptr(), q.stride(0), _dt(q), kv.data_ptr(), bt.data_ptr(),
             bt.stride(0), ctx.token_row.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), out.stride(0), T, nh, nkv, hd,
             vd, int(page_size), kv.shape[0], float(scale), float(softcap or 0.0), int(window), bt.shape[0], _dt(kv),
             _ptr(ctx.status), int(keep_first), int(bool(values_are_keys)), _ptr(gate),
             gate.stride(0) if gate is not None else 0, int(chunk), _ptr(sinks), int(gate_group), _stream())
        return out
    call("common", "fmx_paged_attention_masked", q.data_ptr(), q.stride(0), _dt(q), kv.data_ptr(), bt.data_ptr(),
         bt.stride(0), ctx.token_row.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), out.stride(0), T, nh, nkv, hd, vd,
         int(page_size), kv.shape[0], float(scale), float(softcap or 0.0), int(window), bt.shape[0], _dt(kv),
         _ptr(ctx.status), int(keep_first), int(bool(values_are_keys)), _ptr(gate), gate.stride(0) if gate is not None else 0,
         _stream())
    return out


def wide_attention_ok(q, kv, hd, vd) -> bool:
    """Does the tiled tensor-core kernel with two-term products take this attention?  bfloat16 pages in the common
    layout (values as wide as keys), a head size in steps of 16 up to 256, 32-bit queries in 8-byte pairs."""
    return (kv is not None and kv.dtype == torch.bfloat16 and kv.dim() == 5 and q.dtype == torch.float32 and hd == vd
            and hd % 16 == 0 and hd <= 256 and q.stride(0) % 2 == 0 and q.data_ptr() % 8 == 0)


WIDE_MAX_SPLITS = 16
WIDE_HAS_SINKS = True            # the tiled kernel takes runs of positions and terms without a value too


def wide_attention_splits(rows: int, nkv: int, keys: int, device=None, hd: int = 64) -> int:
    """Blocks that share the keys of a one-token row out among them.  `keys`: the most keys a row sees (its window, its
    run of positions, or the longest context).  A grid that fills the GPU twice over as it is stays whole.  Else the
    count s <= 16 (each share at least two 64-key tiles) with the shortest estimate waves(s) x (tiles / s + 2): the
    grid's blocks run in waves of as many as are resident at once (one per SM with heads wider than 128, whose tiles
    fill the shared memory; two otherwise), and a block costs its share of the tiles plus a fixed part.  Measured at
    64 rows over one kv head of 256 values behind 4,096 keys: 5 shares (320 blocks, a second wave of 24) 288 us,
    2 shares (128 blocks) 241 us; 32 rows: 10 shares 140 us, 4 shares 134 us; 16 rows: 16 shares 104 us, 9 shares 79 us."""
    tiles = -(-max(1, int(keys)) // 64) + 1
    grid = max(1, rows * nkv)
    sms = num_sms(device)
    if grid >= 2 * sms:
        return 1
    slots = sms * (1 if hd > 128 else 2)
    best, best_cost = 1, None
    for s in range(1, max(1, min(tiles // 2, WIDE_MAX_SPLITS)) + 1):
        cost = -(-grid * s // slots) * (-(-tiles // s) + 2)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def wide_attention_takes(q, kv, hd, vd, out=None) -> bool:
    """`wide_attention_ok` for pages in either layout (keys and values, or keys that are the values too) and an
    output that may be a slice of a wider buffer."""
    return (kv is not None and kv.dtype == torch.bfloat16 and kv.dim() == 5 and q.dtype == torch.float32 and hd == vd
            and hd % 16 == 0 and hd <= 256 and q.stride(0) % 2 == 0 and q.data_ptr() % 8 == 0
            and (out is None or (out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0)))


def _wide_launch(q, kv, ctx, group, nh, nkv, hd, scale, softcap, window, out, first_token: int = 0, splits: int = 1,
                 keep_first: int = 0, chunk: int = 0, sinks=None) -> None:
    bt = group.block_tables
    scratch = None
    n_tokens = ctx.R
    if splits > 1:
        scratch = attention_scratch(q.device, (first_token + n_tokens) * nh * splits * (hd + 2))
    call(f"attn_hd{hd}", "fmx_attn_prefill_wide_masked", q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
         ctx.row_start.data_ptr(), ctx.row_ctx.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), out.stride(0), ctx.R,
         int(ctx.max_q_len), nh, nkv, kv.shape[3], kv.shape[0], float(scale), float(softcap or 0.0), int(window),
         _ptr(ctx.status), _ptr(scratch), scratch.numel() if scratch is not None else 0, int(splits),
         first_token + n_tokens, int(keep_first), int(kv.shape[1] == 1), int(chunk), _ptr(sinks), _stream())
    if splits > 1:
        call(f"attn_hd{hd}", "fmx_attn_wide_combine_sinks", scratch.data_ptr(), out.data_ptr(), out.stride(0), int(first_token),
             n_tokens, nh, int(splits), _ptr(sinks), _stream())


def paged_attention_wide(q, kv, ctx, group, nh, nkv, hd, scale, softcap, window, out=None, keep_first: int = 0,
                         gate=None, chunk: int = 0, sinks=None, gate_group: int = 1) -> torch.Tensor:
    """Attention of any mix of rows on the tensor cores with 32-bit scores and weights: the 32-bit queries
    q[T, nh*hd] and the probabilities enter the products as two bfloat16 terms each, sums are 32-bit, scores may be
    capped (softcap > 0).  `out` may be a slice of a wider buffer.  -> [T, nh*hd] in bfloat16.  The one-token rows
    (a whole decode step, or the rows at the head of a mixed step) have their keys shared out over several blocks
    whose parts a second kernel puts together; the portions behind them take a launch of their own.
    `keep_first`: beside a window, a request's first tokens that stay visible; pages of shape [pages, 1, nkv, page, hd]
    hold keys that are the values too; `gate` ([T, nh*hd / gate_group]): the output is multiplied by sigmoid(gate)
    afterwards, one gate value per `gate_group` elements.  `chunk` c > 0 instead of a window: keys are seen within runs
    of c positions counted from position 0; `sinks` (32-bit [nh]): one more term exp(sink) per head in the
    denominator, with no value."""
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == nh)
    out = _paged_attention_wide(q, kv, ctx, group, nh, nkv, hd, scale, softcap, window, out, int(keep_first), int(chunk), sinks)
    if gate is not None:
        sigmoid_gate(out, gate, int(gate_group))
    return out


def _paged_attention_wide(q, kv, ctx, group, nh, nkv, hd, scale, softcap, window, out, keep_first, chunk=0, sinks=None) -> torch.Tensor:
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=q.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0
    d = ctx.R if ctx.all_decode else getattr(ctx, "decode_rows", 0)
    more = dict(chunk=chunk, sinks=sinks)
    if d <= 0:
        _wide_launch(q, kv, ctx, group, nh, nkv, hd, scale, softcap, window, out, keep_first=keep_first, **more)
        return out
    longest = ctx.max_ctx_after if ctx.all_decode else ctx.decode_max_ctx
    keys = min(window + keep_first, longest) if window > 0 else (min(chunk, longest) if chunk > 0 else longest)
    splits = wide_attention_splits(d, nkv, keys, q.device, hd)
    if splits > 1 and d * nh * splits * (hd + 2) > ATTN_SCRATCH_FLOATS:
        splits = 1
    if ctx.all_decode:
        _wide_launch(q, kv, ctx, group, nh, nkv, hd, scale, softcap, window, out, 0, splits, keep_first, **more)
        return out
    key = ("wide attention rows", id(group))
    views = ctx.scratch.get(key)
    if views is None:
        views = ctx.scratch[key] = (_rows_of(ctx, group, 0, d, 1, ctx.decode_max_ctx),
                                    _rows_of(ctx, group, d, ctx.R, ctx.rest_max_q_len, ctx.rest_max_ctx))
    (dctx, dgroup), (rctx, rgroup) = views
    _wide_launch(q, kv, dctx, dgroup, nh, nkv, hd, scale, softcap, window, out, 0, splits, keep_first, **more)     # the one-token rows come first
    _wide_launch(q, kv, rctx, rgroup, nh, nkv, hd, scale, softcap, window, out, keep_first=keep_first, **more)
    return out


# ----------------------------------------------------------------------------- gated delta rule
def delta_prepare(proj, ab, conv_w, a_log, dt_bias, ctx, state, conv_off, H, G, D, Dv, taps):
    """What the recurrence of a gated delta rule layer takes in, from the projections of a step:
    proj[T, >= C] holds q (G*D) | k (G*D) | v (H*Dv) channels, ab[T, 2H] in 32-bit the write strengths'
    and decays' pre-activations.  Channels pass a causal convolution of `taps` taps (weights conv_w[C, taps];
    inputs before a portion's start come from the request's state slot, which then takes the
    portion's last inputs) and SiLU; q and k become unit vectors per head, q times D^-1/2.
    -> (q | k | v in 32-bit [T, C], decay | beta in 32-bit [T, 2H])."""
    _need_cuda(proj, ab, conv_w, a_log, dt_bias, state)
    T = proj.shape[0]
    C = 2 * G * D + H * Dv
    assert proj.stride(1) == 1 and ab.dtype == torch.float32 and ab.stride(1) == 1 and state.dtype == torch.float32
    assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape == (C, taps) and state.is_contiguous()
    qkv = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    gb = torch.empty((T, 2 * H), dtype=torch.float32, device=proj.device)
    call("common", "fmx_delta_prepare", proj.data_ptr(), proj.stride(0), ab.data_ptr(), ab.stride(0), conv_w.data_ptr(),
         a_log.data_ptr(), dt_bias.data_ptr(), ctx.token_row.data_ptr(), ctx.row_start.data_ptr(), ctx.row_slot.data_ptr(),
         state.data_ptr(), state.stride(0), int(conv_off), qkv.data_ptr(), gb.data_ptr(), T, ctx.R, H, G, D, Dv, int(taps),
         state.shape[0], _dt(proj), _ptr(ctx.status), _stream())
    return qkv, gb


def delta_rule(qkv, gb, ctx, state, H, G, D, Dv, lanes: int = 0) -> torch.Tensor:
    """The gated delta rule over every request's tokens of the step, in order, from and into the requests'
    state slots (S^T per head, [H, Dv, D], at the head of a slot): S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q.  `lanes` (2 to 32, a power of two; 0: the library's choice): lanes that share a column of S.
    -> o in 32-bit, [T, H*Dv]."""
    T = qkv.shape[0]
    out = torch.empty((T, H * Dv), dtype=torch.float32, device=qkv.device)
    call("common", "fmx_delta_rule", qkv.data_ptr(), gb.data_ptr(), ctx.row_start.data_ptr(), ctx.row_slot.data_ptr(),
         state.data_ptr(), state.stride(0), out.data_ptr(), ctx.R, H, G, D, Dv, state.shape[0], int(lanes), _stream())
    return out


def gated_rmsnorm(o, gate, weight, eps, H, Dv, out_dtype, out=None) -> torch.Tensor:
    """o[T, H*Dv] (32-bit) per head divided by its root mean square, times weight[Dv], times silu(gate);
    gate and out may be slices of wider buffers."""
    T = o.shape[0]
    if out is None:
        out = torch.empty((T, H * Dv), dtype=out_dtype, device=o.device)
    assert gate.stride(1) == 1 and out.stride(1) == 1 and gate.dtype == out.dtype and o.is_contiguous()
    call("common", "fmx_gated_rmsnorm", o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), out.data_ptr(),
         out.stride(0), T, H, Dv, float(eps), _dt(out), _stream())
    return out


# ----------------------------------------------------------------------------- bigram embedding, rotated latents, state space
def embed_bigram(ids, table, bigram, ctx, state, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """table[id_t] + bigram[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] in 32-bit, [T, d]; a request's first
    token takes row `buckets`.  `state` (int32 [slots, 1]) holds the token before a row's first token of this step and
    is left holding the row's last one.  Rows of slot -1 or tokens at position -1 get zeros."""
    _need_cuda(ids, table, bigram, state)
    assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous() and bigram.is_contiguous()
    assert bigram.shape == (buckets + 1, table.shape[1]) and bigram.dtype == table.dtype
    assert state.dtype == torch.int32 and state.is_contiguous()
    T, d = ids.numel(), table.shape[1]
    out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    call("common", "fmx_embed_bigram", ids.data_ptr(), table.data_ptr(), bigram.data_ptr(), ctx.positions.data_ptr(),
         ctx.token_row.data_ptr(), ctx.row_start.data_ptr(), ctx.row_slot.data_ptr(), state.data_ptr(), state.stride(0),
         out.data_ptr(), T, d, table.shape[0], int(buckets), int(mul_prev), int(mul_cur), ctx.R, state.shape[0], _dt(table),
         _ptr(ctx.status), _stream())
    return out


def latent_rope_prepare(q, dkv, positions, inv_freq, norm_w, eps, slot_mapping, kv, q_lat, H, D, R, r, status,
                        q_offset: int | None = None) -> None:
    """Latent attention with a rotated key part: a token's down-projection dkv[t, :r+R] (32-bit; rows may be a slice)
    becomes its cache row [rmsnorm(dkv[:r]) * norm_w | dkv[r:] rotated] at slot_mapping[t] of `kv` (rows of r + R
    values), and the rotated parts of its query heads (q[t, h, D:D+R], pairs (i, i + R/2)) go, rotated, to
    q_lat[t, h, r:r+R] in 32-bit (with `q_offset` o: q_lat is [T, H * (o + R)] and takes them at [t, h, o:o+R]).
    dkv / kv None: a layer that reads another's cache stores nothing."""
    _need_cuda(q, dkv, positions, inv_freq, norm_w, slot_mapping, kv, q_lat)
    assert q.dim() == 2 and q.stride(1) == 1 and q_lat.dtype == torch.float32 and q_lat.is_contiguous()
    q_off = int(r if q_offset is None else q_offset)
    assert q_lat.shape == (q.shape[0], H * (q_off + R))
    store = kv is not None and dkv is not None
    if store:
        assert dkv.dtype == torch.float32 and dkv.stride(1) == 1 and kv.is_contiguous() and kv.numel() % (r + R) == 0
        assert slot_mapping.dtype == torch.int64
    if not store and R == 0:
        return
    call("common", "fmx_latent_rope_prepare", q.data_ptr(), q.stride(0), _dt(q), _ptr(dkv) if store else None,
         dkv.stride(0) if store else 0, positions.data_ptr(), _ptr(inv_freq), _ptr(norm_w) if store else None, float(eps),
         _ptr(slot_mapping) if store else None, _ptr(kv) if store else None, kv.numel() // (r + R) if store else 0,
         _dt(kv) if store else _dt(q), q_lat.data_ptr(), q.shape[0], H, D, R, r, q_off, _ptr(status), _stream())


def ssm_prepare(proj, conv_w, conv_b, a_log, dt_bias, ctx, state, conv_off, H, G, N, P, taps):
    """What a state-space recurrence takes in, from a step's projection proj[T, z (H*P) | x (H*P) | B (G*N) | C (G*N) |
    dt (H)]: x | B | C pass a causal convolution of `taps` taps with a bias (weights conv_w[C, taps]; inputs before
    a portion's start come from the request's state slot, which then takes the portion's last inputs) and SiLU;
    dt = softplus(dt + dt_bias), decay = exp(-exp(A_log) dt).
    -> (x | B | C in 32-bit [T, C], dt | decay in 32-bit [T, 2H])."""
    _need_cuda(proj, conv_w, conv_b, a_log, dt_bias, state)
    T = proj.shape[0]
    C = H * P + 2 * G * N
    assert proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
    assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape == (C, taps) and conv_b.shape == (C,)
    xbc = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    dd = torch.empty((T, 2 * H), dtype=torch.float32, device=proj.device)
    call("common", "fmx_ssm_prepare", proj.data_ptr(), proj.stride(0), conv_w.data_ptr(), conv_b.data_ptr(), a_log.data_ptr(),
         dt_bias.data_ptr(), ctx.token_row.data_ptr(), ctx.row_start.data_ptr(), ctx.row_slot.data_ptr(), state.data_ptr(),
         state.stride(0), int(conv_off), xbc.data_ptr(), dd.data_ptr(), T, ctx.R, H, G, N, P, int(taps), state.shape[0],
         _dt(proj), _ptr(ctx.status), _stream())
    return xbc, dd


def ssm_scan(xbc, dd, d_skip, ctx, state, H, G, N, P, lanes: int = 0) -> torch.Tensor:
    """The state-space recurrence over every request's tokens of the step, in order, from and into the requests' state
    slots (S^T per head, [H, P, N], at the head of a slot): S <- decay S + dt B x^T; y = S^T C + D x.  `lanes` (2 to 32,
    a power of two; 0: the library's choice): lanes that share a column of S.  -> y in 32-bit, [T, H*P]."""
    T = xbc.shape[0]
    out = torch.empty((T, H * P), dtype=torch.float32, device=xbc.device)
    call("common", "fmx_ssm_scan", xbc.data_ptr(), dd.data_ptr(), d_skip.data_ptr(), ctx.row_start.data_ptr(),
         ctx.row_slot.data_ptr(), state.data_ptr(), state.stride(0), out.data_ptr(), ctx.R, H, G, N, P, state.shape[0],
         int(lanes), _stream())
    return out


def gated_group_rmsnorm(y, z, weight, eps, groups, out_dtype, out=None) -> torch.Tensor:
    """y[T, n] (32-bit) * silu(z), then each of `groups` equal parts of a row divided by its own root mean square,
    times weight[n]; z and out may be slices of wider buffers."""
    T, n = y.shape
    if out is None:
        out = torch.empty((T, n), dtype=out_dtype, device=y.device)
    assert z.stride(1) == 1 and out.stride(1) == 1 and z.dtype == out.dtype and y.is_contiguous() and n % groups == 0
    assert z.shape == (T, n) and weight.dtype == torch.float32 and weight.numel() == n
    call("common", "fmx_gated_group_rmsnorm", y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), out.data_ptr(),
         out.stride(0), T, int(groups), n // groups, float(eps), _dt(out), _stream())
    return out


# ----------------------------------------------------------------------------- scaled embedding, retention, sigmoid attention
def embed_scaled(ids, table, scale: float, status) -> torch.Tensor:
    """table[id_t] * scale in 32-bit, [T, d]: an embedding that starts the 32-bit stream."""
    _need_cuda(table, ids)
    assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    n, d = ids.numel(), table.shape[1]
    out = torch.empty((n, d), dtype=torch.float32, device=table.device)
    call("common", "fmx_embed_scaled", table.data_ptr(), _dt(table), ids.data_ptr(), out.data_ptr(), n, d, table.shape[0],
         float(scale), _ptr(status), BAD_TOKEN, _stream())
    return out


def rmsnorm_pair_mean(a, b, wa, wb, eps: float, out_dtype) -> torch.Tensor:
    """(a / rms(a) * wa + b / rms(b) * wb) / 2, row by row, in 32-bit; rows of a and b may be slices."""
    _need_cuda(a, b, wa, wb)
    assert a.dim() == 2 and a.shape == b.shape and a.dtype == b.dtype and a.stride(1) == 1 and b.stride(1) == 1
    assert wa.dtype == torch.float32 and wb.dtype == torch.float32 and wa.numel() == a.shape[1] == wb.numel()
    T, n = a.shape
    out = torch.empty((T, n), dtype=out_dtype, device=a.device)
    call("common", "fmx_rmsnorm_pair_mean", a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), _dt(a), wa.data_ptr(),
         wb.data_ptr(), float(eps), out.data_ptr(), out.stride(0), _dt(out), T, n, _stream())
    return out


def retention_prepare(proj, positions, inv_freq, decay, H: int, D: int, P: int, rot: int, k_scale: float):
    """What a retention's recurrence takes in, from a step's projection proj[T, q (H*D) | k (H*D) | v (H*P) ...] (rows may be
    a slice): q and k rotated over their first `rot` dimensions (half-split pairing), k times `k_scale` after the
    rotation.  -> (v | k | q in 32-bit [T, H*P + 2*H*D], the layout `ssm_scan` reads as x | B | C with as many groups as
    heads; step size 1 | decay per head in 32-bit [T, 2H])."""
    _need_cuda(proj, positions, inv_freq, decay)
    assert proj.dim() == 2 and proj.stride(1) == 1 and positions.dtype == torch.int32
    assert decay.dtype == torch.float32 and decay.numel() == H
    T = proj.shape[0]
    xbc = torch.empty((T, H * P + 2 * H * D), dtype=torch.float32, device=proj.device)
    dd = torch.empty((T, 2 * H), dtype=torch.float32, device=proj.device)
    call("common", "fmx_retention_prepare", proj.data_ptr(), proj.stride(0), _dt(proj), positions.data_ptr(), _ptr(inv_freq),
         decay.data_ptr(), xbc.data_ptr(), dd.data_ptr(), T, int(H), int(D), int(P), int(rot), float(k_scale), _stream())
    return xbc, dd


def retention_gate_norm(o, gate, eps: float, H: int, P: int, out_dtype, out=None) -> torch.Tensor:
    """o[T, H*P] (32-bit) per head divided by its root mean square (no weight), times silu(gate); gate (of its own type)
    and out may be slices of wider buffers."""
    _need_cuda(o, gate, out)
    T = o.shape[0]
    if out is None:
        out = torch.empty((T, H * P), dtype=out_dtype, device=o.device)
    assert o.is_contiguous() and o.dtype == torch.float32 and gate.stride(1) == 1 and out.stride(1) == 1
    assert gate.shape == (T, H * P) and out.shape == (T, H * P)
    call("common", "fmx_retention_gate_norm", o.data_ptr(), gate.data_ptr(), gate.stride(0), _dt(gate), out.data_ptr(),
         out.stride(0), _dt(out), T, int(H), int(P), float(eps), _stream())
    return out


def _pow2_at_least(n: int, choices=(1, 2, 4, 8)) -> int:
    for c in choices:
        if n <= c:
            return c
    return 0


def mixed_heads_library(nh: int, nkv: int, hd: int, vd: int, q=None, kv=None) -> str | None:
    """The library of the tiled attention with mixed heads that takes these sizes (one per values-per-lane and query
    heads per key head), or None: 32-bit queries over bfloat16 pages, values up to 256 wide, at most 8 query heads per
    key head."""
    if kv is not None and (kv.dtype != torch.bfloat16 or q is None or q.dtype != torch.float32):
        return None
    if q is not None and (q.data_ptr() % 16 or q.stride(0) % 4 or (nh * hd) % 4):
        return None
    vpl, per = _pow2_at_least(-(-vd // 32)), _pow2_at_least(nh // nkv)
    return f"mixattn_v{vpl}_p{per}" if vpl and per else None


def sigmoid_attention(q, kv, ctx, group, nh, nkv, hd, vd, scale, softcap, window, page_size, head_bias, mix, out=None,
                      out_dtype=None, tiled: bool | None = None) -> torch.Tensor:
    """Attention without a softmax: a visible key weighs sigmoid(cap(scale q.k) + head_bias[head]); the heads' weights are
    mixed by `mix` ([nh, nh], 32-bit: row h lists what head h takes of every head's weights) and head h applies its mixed
    weights to the values of its own key/value head.  Queries q[T, nh*hd] of their own type over pages of [nkv, page, hd]
    keys and [nkv, page, vd] values; scores, weights and the sums over keys are 32-bit.  -> [T, nh*vd].

    Two kernels: over bfloat16 pages a block owns all heads of a tile of tokens and mixes the weights before they meet
    the values (prompt portions and single tokens; a single token's keys may be shared out over several blocks); else,
    and on the 32-bit path, one warp per (token, head, value head) sums the unmixed heads' outputs, which a second
    kernel mixes.  `tiled`: force the choice (None: the tiled kernel where it takes the sizes)."""
    _need_cuda(q, kv, head_bias, mix, out)
    assert kv.is_contiguous() and q.stride(1) == 1
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, nh * vd), dtype=out_dtype or kv.dtype, device=q.device)
    assert out.stride(1) == 1 and out.shape == (T, nh * vd)
    assert mix.dtype == torch.float32 and mix.is_contiguous() and mix.shape == (nh, nh)
    assert head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == nh)
    bt = group.block_tables
    name = mixed_heads_library(nh, nkv, hd, vd, q, kv) if tiled is not False and out.dtype == torch.bfloat16 else None
    if name is not None:
        lib = load(name)
        splits = int(lib.fmx_mixattn_plan(T, nh, nkv, hd, vd, int(ctx.max_q_len), int(ctx.max_ctx_after)))
        if splits > 0:
            part = torch.empty((splits, T, nh * vd), dtype=torch.float32, device=q.device) if splits > 1 else None
            call(name, "fmx_mixattn", q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
                 ctx.token_row.data_ptr(), ctx.positions.data_ptr(), ctx.row_start.data_ptr(), _ptr(part), out.data_ptr(),
                 out.stride(0), T, nh, nkv, hd, vd, int(page_size), kv.shape[0], float(scale), float(softcap or 0.0),
                 int(window), bt.shape[0], _ptr(head_bias), mix.data_ptr(), int(ctx.max_q_len), splits, _ptr(ctx.status),
                 _stream())
            return out
    assert tiled is not True, "the tiled kernel does not take these sizes"
    part = torch.empty((T, nh, nkv, vd), dtype=torch.float32, device=q.device)
    call("common", "fmx_sigmoid_attention", q.data_ptr(), q.stride(0), _dt(q), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
         ctx.token_row.data_ptr(), ctx.positions.data_ptr(), part.data_ptr(), T, nh, nkv, hd, vd, int(page_size), kv.shape[0],
         float(scale), float(softcap or 0.0), int(window), bt.shape[0], _dt(kv), _ptr(head_bias), _ptr(ctx.status), _stream())
    call("common", "fmx_head_mix", part.data_ptr(), mix.data_ptr(), out.data_ptr(), out.stride(0), _dt(out), T, nh, nkv, vd,
         _stream())
    return out


# ----------------------------------------------------------------------------- dynamic tanh, latents, gates, routed experts
def dyt_step(y, post, mult, add, residual, pre, out_dtype, out=None, keep_stream: bool = True):
    """One pass over the stream: residual <- residual + mult * post(y) + add, out = pre(residual), all 32-bit.
    post and pre are (alpha, weight, bias) of a dynamic tanh, tanh(alpha x) weight + bias, or None for the identity;
    y (bfloat16 or 32-bit, rows may be a slice) may be None, `add` (a 32-bit vector) too; residual None: the stream
    starts at zero and gets an array of its own; pre False: nothing but the stream is written.  `out` may be a
    slice of a wider buffer.  -> (out or None, residual)."""
    ref = y if y is not None else residual
    _need_cuda(y, residual, add, out)
    assert ref is not None and ref.dim() == 2 and (y is None or y.stride(1) == 1)
    rows, cols = ref.shape
    assert residual is None or (residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape == ref.shape)
    res_in = residual
    if residual is None:
        residual = torch.empty((rows, cols), dtype=torch.float32, device=ref.device)
    want_out = pre is not False
    if want_out and out is None:
        out = torch.empty((rows, cols), dtype=out_dtype, device=ref.device)
    pa, pw, pb = post if post else (0.0, None, None)
    qa, qw, qb = pre if pre else (0.0, None, None)
    call("common", "fmx_dyt_step", _ptr(y), y.stride(0) if y is not None else 0, _dt(y) if y is not None else F32, float(pa),
         _ptr(pw), _ptr(pb), float(mult), _ptr(add), _ptr(res_in), residual.data_ptr() if keep_stream else None, float(qa),
         _ptr(qw), _ptr(qb), _ptr(out) if want_out else None, out.stride(0) if want_out else 0,
         _dt(out) if want_out else F32, rows, cols, _stream())
    return (out if want_out else None), residual


def rmsnorm_rows(x, weight, eps, out=None, out_dtype=None, row_map=None, status=None):
    """x[T, n] (rows may be a slice) / sqrt(mean(x^2) + eps) * weight, in 32-bit, into `out` (a dense array, or any
    array of rows of n where `row_map`, int64 [T], names each token's row: a cache of latents addressed by slot)."""
    _need_cuda(x, weight, out, row_map)
    assert x.dim() == 2 and x.stride(1) == 1 and weight.dtype == torch.float32
    T, n = x.shape
    if out is None:
        out = torch.empty((T, n), dtype=out_dtype or x.dtype, device=x.device)
    if row_map is not None:
        assert row_map.dtype == torch.int64 and out.is_contiguous() and out.numel() % n == 0
        max_rows, stride = out.numel() // n, n
    else:
        assert out.shape == (T, n) and out.stride(1) == 1
        max_rows, stride = T, out.stride(0)
    call("common", "fmx_rmsnorm_rows", x.data_ptr(), x.stride(0), _dt(x), weight.data_ptr(), float(eps), out.data_ptr(), stride,
         _dt(out), _ptr(row_map), max_rows, T, n, _ptr(status), _stream())
    return out


def sigmoid_gate(o, gate, group: int = 1):
    """o[t, j] *= sigmoid(gate[t, j // group]) in place, in 32-bit; rows of either may be slices."""
    _need_cuda(o, gate)
    assert o.dim() == 2 and o.stride(1) == 1 and gate.stride(1) == 1 and gate.shape[1] * group == o.shape[1]
    call("common", "fmx_sigmoid_gate", o.data_ptr(), o.stride(0), _dt(o), gate.data_ptr(), gate.stride(0), _dt(gate), o.shape[0],
         o.shape[1], int(group), _stream())
    return o


def moe_route(logits, top: int, groups: int = 1, keep: int = 1, want_chosen: bool = False, experts: int | None = None,
              correction=None, scale: float = 1.0):
    """Router logits [T, E] (32-bit) -> weights [T, E] (32-bit): the softmax score where an expert is among the token's
    `top` best of the `keep` best groups (of `groups` groups of neighbours, each scored by its best member), else zero;
    not renormalised.  With `want_chosen` also the chosen indices, int32 [T, top].  `experts`: the row's first that many
    columns are the experts' logits (a row may hold other columns behind them).  `correction` (32-bit [E]): added to the
    scores for the choice only; `scale` multiplies the chosen experts' scores."""
    _need_cuda(logits, correction)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    T, E = logits.shape[0], int(experts if experts is not None else logits.shape[1])
    assert E <= logits.shape[1] and (correction is None or (correction.dtype == torch.float32 and correction.numel() == E
                                                             and correction.is_contiguous()))
    w = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device) if want_chosen else None
    call("common", "fmx_moe_route_biased", logits.data_ptr(), logits.stride(0), T, E, int(top), int(groups), int(keep),
         w.data_ptr(), _ptr(chosen), _ptr(correction), float(scale), _stream())
    return (w, chosen) if want_chosen else w


def moe_plain_act(u, weights, E: int, ff: int, act: str, shared_gate=None, out=None):
    """The hidden layers of experts without a gate, side by side: u[T, F], F = E*ff + the shared expert's width;
    -> [T, F]: w * act(u) with w the token's weight for the column's expert, zero where it did not choose it; the shared
    columns at the end weigh sigmoid(shared_gate[t]) (32-bit, one value per token; rows may be a slice) or 1."""
    _need_cuda(u, weights, shared_gate)
    assert u.dim() == 2 and u.stride(1) == 1 and weights.dtype == torch.float32 and weights.is_contiguous()
    T, F = u.shape
    assert weights.shape == (T, E) and (shared_gate is None or (shared_gate.dtype == torch.float32 and shared_gate.shape[0] == T))
    if out is None:
        out = torch.empty((T, F), dtype=u.dtype, device=u.device)
    call("common", "fmx_moe_plain_act", u.data_ptr(), u.stride(0), weights.data_ptr(), _ptr(shared_gate),
         shared_gate.stride(0) if shared_gate is not None else 0, out.data_ptr(), out.stride(0), T, int(E), int(ff), F,
         ACTIVATIONS[act], _dt(u), _stream())
    return out


def moe_expert_act(gu, weights, E: int, ff: int, limit: float, limit_shared: float = 0.0, out=None, block: int = 0):
    """The experts' hidden layers side by side: gu[T, 2F] holds F gates then F ups, F = E*ff + the shared expert's
    width; -> [T, F]: w * g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit), w the
    token's weight for the column's expert (1 for the shared columns at the end), zero where it chose it not.
    `block` > 0: gu holds gates and ups in alternating blocks of that many instead."""
    _need_cuda(gu, weights)
    assert gu.dim() == 2 and gu.stride(1) == 1 and gu.shape[1] % 2 == 0 and weights.dtype == torch.float32
    T, F = gu.shape[0], gu.shape[1] // 2
    assert weights.shape == (T, E) and weights.is_contiguous()
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    call("common", "fmx_moe_expert_act", gu.data_ptr(), gu.stride(0), weights.data_ptr(), out.data_ptr(), out.stride(0), T,
         int(E), int(ff), F, float(limit), float(limit_shared), _dt(gu), int(block), _stream())
    return out


def can_expert_tc(x, w) -> bool:
    """Does a shared expert's gate/up product of these sizes go to the tcgen05 kernel with the expert's activation in its
    epilogue?  As `can_tc` with the SiLU-mul epilogue: bfloat16, at least 128 rows, gate/up rows in blocks of 128, full rounds."""
    return (_bf16_operands(x, w) and x.shape[0] >= TC_MIN_ROWS and w.shape[0] % (2 * GATE_UP_BLOCK) == 0
            and tc_fills_the_gpu(x.shape[0], w.shape[0], num_sms(x.device)))


def expert_gate_up_tc(x, w, limit: float, status=None) -> torch.Tensor:
    """g' sigmoid(1.702 g') (u' + 1) of x w^T, g' = min(g, limit), u' = clamp(u, -limit, limit), for w [2 ff, K] in blocks of 128
    gate rows followed by their up rows: product and activation in one tcgen05 kernel.  -> bfloat16 [M, ff]."""
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    call("tc", "fmx_expert_tcgen05", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
         float(limit), num_sms(x.device), _ptr(status if status is not None else _status_word(x.device)), _stream())
    return out


MOE_TILE_ROWS = 128         # rows of a tile of sorted pairs (`fmx_moe_tile_rows` of the library)


def moe_sort(chosen, weights):
    """The (token, chosen expert) pairs laid out expert by expert, each expert's pairs starting on a multiple of
    MOE_TILE_ROWS rows.  chosen int32 [T, top] (-1: none), weights 32-bit [T, E].  -> a plan for the grouped products: (token of each
    sorted row or -1, weight of each sorted row, sorted row of each pair, expert of each tile of rows or -1, tiles, the
    number of sorted rows in use as a device scalar)."""
    _need_cuda(chosen, weights)
    T, top = chosen.shape
    E = weights.shape[1]
    assert chosen.dtype == torch.int32 and chosen.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
    assert int(load("bf16").fmx_moe_tile_rows()) == MOE_TILE_ROWS
    tiles = -(-(T * top + E * (MOE_TILE_ROWS - 1)) // MOE_TILE_ROWS)
    dev = chosen.device
    sorted_token = torch.empty(tiles * MOE_TILE_ROWS, dtype=torch.int32, device=dev)
    sorted_w = torch.empty(tiles * MOE_TILE_ROWS, dtype=torch.float32, device=dev)
    pair_pos = torch.empty(T * top, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
    used = torch.empty(1, dtype=torch.int32, device=dev)
    call("bf16", "fmx_moe_sort", chosen.data_ptr(), weights.data_ptr(), T, E, top, sorted_token.data_ptr(), sorted_w.data_ptr(),
         pair_pos.data_ptr(), tile_expert.data_ptr(), tiles, used.data_ptr(), _stream())
    return sorted_token, sorted_w, pair_pos, tile_expert, tiles, used


MOE_BLOCK = 128           # gate and up rows of an expert alternate in blocks of this many where its width allows
MOE_TC_MIN_TOKENS = 128   # steps of at least this many tokens run their grouped products on the tcgen05 kernel


def moe_grouped_gate_up(x, plan, gate_up, E: int, ff: int, limit: float, block: int = 0, status=None) -> torch.Tensor:
    """The experts' hidden layers for the sorted pairs of `plan`.  gate_up [2 E ff, K] bfloat16: with block = 0 every
    expert's gate rows and then every expert's up rows; with block = MOE_BLOCK expert after expert, each in blocks of
    `block` gate rows followed by their up rows.  Row r of the result is w g' sigmoid(1.702 g') (u' + 1) of the row's token
    under the row's expert (clamped by `limit`, scaled by the pair's weight); padding rows are not written.
    -> bfloat16 [tiles * MOE_TILE_ROWS, ff].  Steps of MOE_TC_MIN_TOKENS tokens and more, with blocked weights, gather the
    pairs' inputs and multiply on the tcgen05 tensor cores; the others on the tiled mma.sync kernel, which gathers itself."""
    sorted_token, sorted_w, _, tile_expert, tiles, used = plan
    _need_cuda(x, gate_up)
    T, K = x.shape
    assert x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and gate_up.is_contiguous() and x.stride(1) == 1
    assert gate_up.shape == (2 * E * ff, K) and block in (0, MOE_BLOCK) and (block == 0 or ff % block == 0)
    rows = tiles * MOE_TILE_ROWS
    y = torch.empty((rows, ff), dtype=torch.bfloat16, device=x.device)
    if block and T >= MOE_TC_MIN_TOKENS and ff % 8 == 0:
        xs = torch.empty((rows, K), dtype=torch.bfloat16, device=x.device)
        call("bf16", "fmx_moe_gather", x.data_ptr(), x.stride(0), sorted_token.data_ptr(), used.data_ptr(), xs.data_ptr(), rows, K,
             _stream())
        call("tc", "fmx_grouped_tcgen05", xs.data_ptr(), K, gate_up.data_ptr(), K, y.data_ptr(), ff, rows, 2 * ff, K, E,
             used.data_ptr(), tile_expert.data_ptr(), sorted_token.data_ptr(), sorted_w.data_ptr(), float(limit), 1,
             num_sms(x.device), _ptr(status if status is not None else _status_word(x.device)), _stream())
        return y
    if block:
        w_up, stride = gate_up.data_ptr() + 2 * block * K, 2 * ff * K
    else:
        w_up, stride = gate_up.data_ptr() + 2 * E * ff * K, ff * K
    call("bf16", "fmx_moe_grouped_gate_up", x.data_ptr(), x.stride(0), sorted_token.data_ptr(), sorted_w.data_ptr(),
         tile_expert.data_ptr(), gate_up.data_ptr(), w_up, K, stride, y.data_ptr(), tiles, ff, K, float(limit), int(block), _stream())
    return y


def moe_grouped_down(y, plan, down, E: int, ff: int, stacked: bool = False, tokens: int = 0, status=None) -> torch.Tensor:
    """The pairs' outputs.  down bfloat16: [d, E ff], the experts' down matrices side by side, or with `stacked`
    [E d, ff], one under the other.  -> 32-bit [tiles * MOE_TILE_ROWS, d] (padding rows are not written).  `tokens`:
    the step's tokens (stacked matrices and MOE_TC_MIN_TOKENS of them: the tcgen05 kernel)."""
    sorted_token, _, _, tile_expert, tiles, used = plan
    assert down.dtype == torch.bfloat16 and down.is_contiguous() and y.is_contiguous()
    d = down.shape[0] // E if stacked else down.shape[0]
    assert down.shape == ((E * d, ff) if stacked else (d, E * ff))
    rows = tiles * MOE_TILE_ROWS
    out = torch.empty((rows, d), dtype=torch.float32, device=y.device)
    if stacked and tokens >= MOE_TC_MIN_TOKENS:
        call("tc", "fmx_grouped_tcgen05", y.data_ptr(), ff, down.data_ptr(), ff, out.data_ptr(), d, rows, d, ff, E,
             used.data_ptr(), tile_expert.data_ptr(), sorted_token.data_ptr(), None, 0.0, 0, num_sms(y.device),
             _ptr(status if status is not None else _status_word(y.device)), _stream())
        return out
    ldw, stride = (ff, d * ff) if stacked else (E * ff, ff)
    call("bf16", "fmx_moe_grouped_down", y.data_ptr(), sorted_token.data_ptr(), tile_expert.data_ptr(), down.data_ptr(), ldw, stride,
         out.data_ptr(), tiles, d, ff, _stream())
    return out


def moe_combine(pair_out, plan, shared, T: int, top: int, out_dtype) -> torch.Tensor:
    """Each token's pair outputs added in the order of its choices, plus `shared` [T, d] where given; rounded once."""
    pair_pos = plan[2]
    d = pair_out.shape[1]
    out = torch.empty((T, d), dtype=out_dtype, device=pair_out.device)
    assert shared is None or (shared.dtype == out_dtype and shared.stride(1) == 1 and shared.shape == (T, d))
    call("bf16", "fmx_moe_combine", pair_out.data_ptr(), pair_pos.data_ptr(), _ptr(shared), shared.stride(0) if shared is not None else 0,
         _dt(out), out.data_ptr(), out.stride(0), _dt(out), T, d, int(top), _stream())
    return out


def head_linear(x, w, out_dtype, x_head_stride: int | None = None, out=None, out_head_stride: int | None = None) -> torch.Tensor:
    """A product per head: x[T, H*K] (head by head, rows may be a slice) and w[H, N, K] -> [T, H*N], out[t, h] =
    w[h] x[t, h], accumulated in 32-bit.  bfloat16 operands go to the library's batched product; 32-bit ones to
    the fixed-order kernel, head by head.  `x_head_stride` s > K: head h's K inputs are the first K of the s values
    at x[t, h*s]; `out` with `out_head_stride` s' > N: head h's N results go to the first N of the s' places at
    out[t, h*s'], the rest stay as they are."""
    _need_cuda(x, w, out)
    H, N, K = w.shape
    T = x.shape[0]
    xs = int(x_head_stride or K)
    assert x.dim() == 2 and x.shape[1] >= (H - 1) * xs + K and x.stride(1) == 1 and w.is_contiguous()
    if out is None:
        os_ = N
        out = torch.empty((T, H * N), dtype=out_dtype, device=x.device)
    else:
        os_ = int(out_head_stride or N)
        assert out.dim() == 2 and out.shape[0] == T and out.stride(1) == 1 and out.shape[1] >= (H - 1) * os_ + N
        out_dtype = out.dtype
    if T == 0:
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        a = x.as_strided((H, T, K), (xs, x.stride(0), 1), x.storage_offset())
        o = out.as_strided((H, T, N), (os_, out.stride(0), 1), out.storage_offset())
        if out_dtype == torch.bfloat16:
            if os_ == N:
                torch.bmm(a, w.transpose(1, 2), out=o)
            else:
                o.copy_(torch.bmm(a, w.transpose(1, 2)))
        else:
            o.copy_(torch.bmm(a, w.transpose(1, 2), out_dtype=out_dtype))
        return out
    for h in range(H):
        call("common", "fmx_gemm_simple", x.data_ptr() + h * xs * x.element_size(), w[h].data_ptr(), None,
             out.data_ptr() + h * os_ * out.element_size(), T, N, K, x.stride(0), K, out.stride(0), _dt(x), _dt(w), _dt(out),
             _stream())
    return out


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(x, kind: str, out=None) -> torch.Tensor:
    """relu(x)^2, gelu (tanh form) or silu, in 32-bit, over rows that may be slices of wider buffers."""
    _need_cuda(x)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    assert x.dim() == 2 and x.stride(1) == 1 and out.stride(1) == 1 and out.shape == x.shape and out.dtype == x.dtype
    call("common", "fmx_activation", x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), x.shape[0], x.shape[1],
         ACTIVATIONS[kind], _dt(x), _stream())
    return out


MAX_SPLITS = 64
ATTN_SCRATCH_FLOATS = 8 << 20        # 32 MiB of split partials per device
_scratch: dict = {}


def attention_scratch(device, floats: int = 0) -> torch.Tensor:
    """The workspace of the split decode attention (partial outputs, maxima and sums): one per
    device, made once at a fixed size and never replaced, since captured graphs hold its
    address.  The engine's own split counts keep rows * kv heads * splits within a round of
    resident blocks, which needs at most 12 MB; a call that asks for more than the buffer
    holds is refused."""
    i = _dev_index(device)
    buf = _scratch.get(i)
    if buf is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace must exist before a CUDA graph is captured")
        buf = _scratch[i] = torch.empty(ATTN_SCRATCH_FLOATS, dtype=torch.float32, device=device)
    if floats > buf.numel():
        raise KernelError(f"the split decode attention's workspace holds {buf.numel()} floats, {floats} asked for: "
                          "use fewer splits")
    return buf


ATTN_TICKETS = 1 << 16
_tickets: dict = {}


def attention_tickets(device) -> torch.Tensor:
    """Tickets of the split decode attention (one per row and kv head), zero between launches."""
    t = _tickets.get(_dev_index(device))
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention tickets must exist before a CUDA graph is captured")
        t = _tickets[_dev_index(device)] = torch.zeros(ATTN_TICKETS, dtype=torch.int32, device=device)
    return t


def decode_splits(rows: int, nkv: int, max_ctx: int, hd: int = 64, device=None) -> int:
    """Splits over the keys of a decode step, as the attention library of this head size plans
    them from its own tile and shared-memory sizes (`fmx_attn_decode_plan`)."""
    lib = load(f"attn_hd{hd}")
    return int(lib.fmx_attn_decode_plan(int(rows), int(nkv), int(max_ctx), num_sms(device)))


def attn_decode_scratch_floats(rows: int, nkv: int, splits: int, hd: int) -> int:
    return 0 if splits <= 1 else rows * nkv * splits * 16 * (hd + 2)


def paged_attention_decode(qkv, kv, ctx, group, nh, nkv, hd, scale, window, splits=None, rope=None, out=None) -> torch.Tensor:
    """Every row brings one token: split over the keys, all query heads of a kv head together.
    rope = (inv_freq or None, rotary_dim, traditional, store): qkv is as the projection left it;
    the kernel rotates the queries itself and, if `store`, rotates each row's new key and puts
    it and its value into the cache (what rope_kv_write does in a kernel of its own)."""
    T = qkv.shape[0]
    R = ctx.R
    if out is None:
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    if splits is None:
        splits = getattr(ctx, "n_splits", 0) or decode_splits(R, nkv, max(1, ctx.max_ctx_after), hd, qkv.device)
    need = attn_decode_scratch_floats(R, nkv, splits, hd)
    scratch = attention_scratch(qkv.device, need) if need else None
    tickets = attention_tickets(qkv.device) if need and R * nkv <= ATTN_TICKETS else None
    bt = group.block_tables
    inv_freq, rot, trad, mode = None, 0, False, 0
    if rope is not None:
        inv_freq, rot, trad, store = rope
        mode = 1 if store else 2
    call(f"attn_hd{hd}", "fmx_attn_decode", qkv.data_ptr(), qkv.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
         ctx.row_start.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), _ptr(scratch),
         scratch.numel() if scratch is not None else 0, _ptr(tickets), R, splits, nh, nkv, kv.shape[3], kv.shape[0],
         float(scale), int(window), _ptr(ctx.status), _ptr(inv_freq), int(rot), 1 if trad else 0, mode, _stream())
    return out


def paged_attention_prefill(qkv, kv, ctx, group, nh, nkv, hd, scale, window, out=None) -> torch.Tensor:
    """Any mix of rows, tiled over 64 packed query rows and 64 keys."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    bt = group.block_tables
    call(f"attn_hd{hd}", "fmx_attn_prefill", qkv.data_ptr(), qkv.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
         ctx.row_start.data_ptr(), ctx.row_ctx.data_ptr(), out.data_ptr(), ctx.R, int(ctx.max_q_len), nh, nkv,
         kv.shape[3], kv.shape[0], float(scale), int(window), _ptr(ctx.status), _stream())
    return out


TC_ATTN_MIN_TOKENS = 64       # portions at least this long attend on the tensor-memory kernel


def tc_attention_ok(nh: int, nkv: int, hd: int, page_size: int, window: int) -> bool:
    """Sizes the tensor-memory attention kernel takes: head size 64 or 128, at most 16 query
    heads per kv head, a page size that divides 128 (at least 8), no window."""
    rep = nh // nkv
    return (hd in (64, 128) and window <= 0 and rep <= 16
            and page_size >= 8 and 128 % page_size == 0)


def paged_attention_prefill_tc(qkv, kv, ctx, group, nh, nkv, hd, scale, variant: int = 0, out=None, ksplits=None) -> torch.Tensor:
    """Causal attention of prompt portions on the tcgen05 tensor cores (TMA-fed, scores and
    outputs in tensor memory).  variant 0: the library's choice of kernel, 1: one query tile per
    CTA, 2: two.  ksplits: how many CTAs share the keys of a pair of query tiles (the two-tile
    kernel; None: as many as the library plans for a grid that would leave most SMs idle)."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    bt = group.block_tables
    lib = load(f"attn_hd{hd}")
    if ksplits is None:
        ksplits = 1
        if variant != 1 and (128 if hd == 64 else 64) % kv.shape[3] == 0:
            ksplits = int(lib.fmx_attn_prefill_tc_plan_splits(int(ctx.R), int(ctx.max_q_len), int(ctx.max_ctx_after), nh, nkv,
                                                               num_sms(qkv.device)))
            if ksplits > 1 and int(lib.fmx_attn_prefill_tc_scratch_floats(T, nh, ksplits)) > ATTN_SCRATCH_FLOATS:
                ksplits = 1
    scratch = attention_scratch(qkv.device, int(lib.fmx_attn_prefill_tc_scratch_floats(T, nh, ksplits))) if ksplits > 1 else None
    call(f"attn_hd{hd}", "fmx_attn_prefill_tc", qkv.data_ptr(), qkv.stride(0), T, kv.data_ptr(), bt.data_ptr(),
         bt.stride(0), ctx.row_start.data_ptr(), ctx.row_ctx.data_ptr(), out.data_ptr(), ctx.R, int(ctx.max_q_len), nh,
         nkv, kv.shape[3], kv.shape[0], float(scale), int(2 if ksplits > 1 else variant), _ptr(ctx.status), int(ksplits),
         _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream())
    return out


def decode_attention_clusters(hd: int, allow: bool) -> bool:
    """Let the split decode attention of head size `hd` combine a row's splits inside a thread-block
    cluster (the default) or make it take the path through L2 and tickets; -> the old setting."""
    return bool(load(f"attn_hd{hd}").fmx_attn_decode_allow_clusters(int(bool(allow))))


def decode_attention_fuses_rope(qkv, kv, ctx, nh, nkv, hd) -> bool:
    """Will `paged_attention` take this step on the split decode kernel, which can rotate q and
    k and store k and v itself?"""
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and kv is not None and kv.dtype == qkv.dtype
            and hd % 16 == 0 and hd <= 256 and qkv.stride(0) % 2 == 0 and ctx.all_decode and nh // nkv <= 16)


def _rows_of(ctx, group, a: int, b: int, max_q_len: int, max_ctx_after: int):
    """The rows [a, b) of a step as a step of their own for the attention kernels: the arrays per
    row start at row a, token indices and positions stay those of the whole step."""
    from types import SimpleNamespace
    sub = SimpleNamespace(positions=ctx.positions, status=ctx.status, row_start=ctx.row_start[a:], row_ctx=ctx.row_ctx[a:],
                          R=b - a, max_q_len=max_q_len, max_ctx_after=max_ctx_after, all_decode=max_q_len == 1, n_splits=0)
    return sub, SimpleNamespace(block_tables=group.block_tables[a:b])


def paged_attention(qkv, kv, ctx, group, nh, nkv, hd, scale, window, rope=None) -> torch.Tensor:
    """Attention of every token of the step over the pages of its own request.
    qkv[T, >= nh*hd] holds the (rotated) queries first; -> [T, nh*hd].  bfloat16 with a head
    size in steps of 16 (at most 256) runs on the tensor cores; everything else, and all
    of the 32-bit path, on the one-warp-per-query kernel.  In a mixed step the decoding rows at
    its head go to the split decode kernel and the portions behind them to the tiled one: alone
    on a tile, a decoding row would walk its whole context in one block."""
    _need_cuda(qkv, kv)
    assert kv.is_contiguous() and kv.dtype == qkv.dtype and qkv.stride(1) == 1
    tiled = qkv.dtype == torch.bfloat16 and hd % 16 == 0 and hd <= 256 and qkv.stride(0) % 2 == 0
    if tiled and ctx.all_decode and nh // nkv <= 16:
        return paged_attention_decode(qkv, kv, ctx, group, nh, nkv, hd, scale, window, rope=rope)
    if rope is not None:
        raise KernelError("only the split decode kernel rotates by itself: ask decode_attention_fuses_rope first")
    if not tiled:
        return paged_attention_simple(qkv, kv, ctx, group, nh, nkv, hd, scale, window)
    out = None
    d = getattr(ctx, "decode_rows", 0)
    if d > 0 and nh // nkv <= 16:
        key = ("attention rows", id(group))
        views = ctx.scratch.get(key)
        if views is None:
            views = ctx.scratch[key] = (_rows_of(ctx, group, 0, d, 1, ctx.decode_max_ctx),
                                        _rows_of(ctx, group, d, ctx.R, ctx.rest_max_q_len, ctx.rest_max_ctx))
        (dctx, dgroup), (ctx, group) = views
        out = torch.empty((qkv.shape[0], nh * hd), dtype=qkv.dtype, device=qkv.device)
        paged_attention_decode(qkv, kv, dctx, dgroup, nh, nkv, hd, scale, window, out=out)
    if ctx.max_q_len >= TC_ATTN_MIN_TOKENS and tc_attention_ok(nh, nkv, hd, kv.shape[3], window) \
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
        return paged_attention_prefill_tc(qkv, kv, ctx, group, nh, nkv, hd, scale, out=out)
    return paged_attention_prefill(qkv, kv, ctx, group, nh, nkv, hd, scale, window, out=out)


# ----------------------------------------------------------------------------- sampling
ARGMAX_ROWS, ARGMAX_CHUNKS = 1024, 32      # the split greedy choice's workspace: rows x chunks pairs
ARGMAX_MIN_CHUNK = 4096                    # logits per block at least
_argmax_ws: dict = {}


def argmax_workspace(device):
    """Chunk results and tickets of the split greedy choice, one pair per device, made once;
    the tickets are zero between launches."""
    ws = _argmax_ws.get(_dev_index(device))
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the greedy choice's workspace must exist before a CUDA graph is captured")
        ws = (torch.empty(ARGMAX_ROWS * ARGMAX_CHUNKS * 2, dtype=torch.int32, device=device),
              torch.zeros(ARGMAX_ROWS, dtype=torch.int32, device=device))
        _argmax_ws[_dev_index(device)] = ws
    return ws


def argmax_chunks(rows: int, V: int) -> int:
    """Blocks per row of the greedy choice: enough to fill the SMs about once, each with at
    least ARGMAX_MIN_CHUNK logits; 1 = the one-block kernel."""
    if rows > ARGMAX_ROWS:
        return 1
    return max(1, min(ARGMAX_CHUNKS, V // ARGMAX_MIN_CHUNK, -(-num_sms() // max(rows, 1))))


def sample(logits: torch.Tensor, temperature=None, uniform=None, keep=None) -> torch.Tensor:
    """Row-wise token choice: argmax where temperature <= 0 (or None), else a draw from
    softmax(logits / temperature) among keep != 0 by the given uniform numbers."""
    _need_cuda(logits, temperature, uniform, keep)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if keep is not None:
        assert keep.dtype == torch.uint8 and keep.shape == logits.shape and keep.stride(1) == 1
    chunks = argmax_chunks(rows, V) if temperature is None and keep is None else 1
    partial, tickets = argmax_workspace(logits.device) if chunks > 1 else (None, None)
    call("common", "fmx_sample", logits.data_ptr(), logits.stride(0), rows, V, _ptr(temperature), _ptr(uniform),
         _ptr(keep), keep.stride(0) if keep is not None else 0, out.data_ptr(), chunks, _ptr(partial), ARGMAX_CHUNKS,
         _ptr(tickets), ARGMAX_ROWS, _stream())
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return sample(logits)


def filter_mask(logits, top_p=None, min_p=None, top_k=None, min_keep=None) -> torch.Tensor:
    """uint8 [rows, V]: 1 where the row's filters (top-p, then min-p, then top-k) keep the token.
    Each argument is a per-row tensor (float32 / int32) or None for "off"."""
    _need_cuda(logits, top_p, min_p, top_k, min_keep)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    keep = torch.empty((rows, V), dtype=torch.uint8, device=logits.device)
    call("common", "fmx_filter_mask", logits.data_ptr(), logits.stride(0), rows, V, _ptr(top_p), _ptr(min_p),
         _ptr(top_k), _ptr(min_keep), keep.data_ptr(), keep.stride(0), _stream())
    return keep


def filter_sample_takes(V: int) -> bool:
    """Rows of this width can be filtered and sampled by one kernel (`filter_sample`)."""
    return bool(load("common").fmx_filter_sample_takes(int(V)))


def filter_sample(logits, temperature, uniform, top_p=None, min_p=None, top_k=None, min_keep=None) -> torch.Tensor:
    """The token of each row after its filters, in one kernel and without a keep mask in memory:
    what `sample(logits, temperature, uniform, filter_mask(logits, ...))` gives.  A row is spread
    over a thread-block cluster with its logits in registers."""
    _need_cuda(logits, temperature, uniform, top_p, min_p, top_k, min_keep)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    call("common", "fmx_filter_sample", logits.data_ptr(), logits.stride(0), rows, V, _ptr(temperature), _ptr(uniform),
         _ptr(top_p), _ptr(min_p), _ptr(top_k), _ptr(min_keep), out.data_ptr(), _stream())
    return out


def penalties(logits, history, repetition, presence, frequency, windows) -> None:
    """In place on float32 logits [rows, V].  history int32 [rows, H] (oldest first, -1 padded
    in front); repetition/presence/frequency float32 [rows] or None; windows int32 [rows, 3]."""
    _need_cuda(logits, history, repetition, presence, frequency, windows)
    assert logits.dtype == torch.float32 and history.dtype == torch.int32 and windows.dtype == torch.int32
    call("common", "fmx_penalties", logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1],
         history.data_ptr(), history.shape[1], _ptr(repetition), _ptr(presence), _ptr(frequency),
         windows.data_ptr(), _stream())


def logit_bias(logits, rows, ids, values) -> None:
    """logits[rows[i], ids[i]] += values[i], in place."""
    _need_cuda(logits, rows, ids, values)
    call("common", "fmx_logit_bias", logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(),
         ids.data_ptr(), values.data_ptr(), rows.numel(), _stream())
