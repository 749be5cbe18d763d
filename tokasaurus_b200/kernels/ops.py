"""Tensor-level entry points of the hand-written kernels.

Each function checks its arguments, then launches one kernel on the current CUDA stream through
the ctypes library built by ``tokasaurus_b200.kernels.build``.  There is no other
implementation behind these functions: a tensor that is not on a CUDA device, or a library
that cannot be built or loaded, raises.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import torch

from tokasaurus_b200.kernels import build


class KernelError(RuntimeError):
    pass


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}


def _suffix(dtype: torch.dtype) -> str:
    try:
        return _SUFFIX[dtype]
    except KeyError:
        raise KernelError(f"kernels exist for float32 and bfloat16 activations, not {dtype}") from None


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device as a raw handle (the direct binding where torch has
    it: ``torch.cuda.current_stream()`` costs more on the host than a kernel launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "this engine runs on CUDA devices only; got a tensor on " + str(t.device)
            )


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


LAUNCHES = 0  # kernels of this engine launched so far (the benchmark reads and resets it)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        if code > 0:
            raise KernelError(f"{what}: CUDA launch failed with error {code}")
        reason = {-2: "sizes not supported", -3: "grid too large", -4: "size beyond the built-in scratch"}.get(
            code, "refused"
        )
        raise KernelError(f"{what}: {reason} (code {code})")


def _fn(lib: ctypes.CDLL, name: str):
    f = lib.__dict__.get(name)  # ctypes keeps a function it has looked up once as an attribute of the library
    if f is not None:
        return f
    try:
        f = getattr(lib, name)
    except AttributeError:
        raise KernelError(f"compiled kernel library lacks the symbol {name}") from None
    f.restype = c_int
    return f


class _Libs:
    def __init__(self) -> None:
        self._cache: dict[tuple, ctypes.CDLL] = {}

    def get(self, source: str, **defines) -> ctypes.CDLL:
        key = (source, tuple(defines.items())) if len(defines) < 2 else (source, tuple(sorted(defines.items())))
        lib = self._cache.get(key)
        if lib is None:
            lib = build.load_module(source, defines or None)
            self._cache[key] = lib
        return lib


_libs = _Libs()


def check_head_dim(hd: int) -> None:
    if hd % 16 or not 16 <= hd <= 256:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to 256, not {hd}")


def prepare(head_dims=(), dtype: torch.dtype = torch.bfloat16) -> None:
    """Build and load everything a model with these head sizes needs (first call compiles)."""
    from tokasaurus_b200.kernels.modules import all_modules

    for hd in head_dims:
        check_head_dim(hd)
    name = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype)
    for source, defines in all_modules(head_dims, name):
        _libs.get(source, **(defines or {}))


# ---------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                 last_token: torch.Tensor, x_out: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """x_out[t] = table[ids[t]] * scale as float32; ids[t] < 0 takes last_token[seq_slot[token_seq[t]]]."""
    _need_cuda(table, ids, token_seq, seq_slot, last_token, x_out, status)
    n, H = x_out.shape
    V = table.shape[0]
    _need(table.shape[1] == H and table.is_contiguous() and x_out.is_contiguous(), "embed_gather: bad table/x shapes")
    _need(x_out.dtype == torch.float32, "embed_gather: the residual stream is float32")
    _need(ids.dtype == torch.int32 and ids.numel() >= n and token_seq.numel() >= n, "embed_gather: ids int32 [T]")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_embed_gather_{_suffix(table.dtype)}")
    _check(f(_ptr(table), _ptr(ids), _ptr(token_seq), _ptr(seq_slot), _ptr(last_token), _ptr(x_out), c_int(n),
             c_int(H), c_int(V), c_float(scale), _ptr(status), _stream()), "embed_gather")


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """x += delta (float32, in place) if delta is given; out = rmsnorm(x) * weight in out's dtype.

    ``delta`` is [rows, H] in out's dtype, or float32 [slices, rows, H]: the slices of a split matrix
    product (``linear_smallm``), added in slice order."""
    _need_cuda(x, delta, weight, out)
    rows, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_rmsnorm: x must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == H, "add_rmsnorm: weight must be float32 [H]")
    _need(out.shape == x.shape and out.is_contiguous(), "add_rmsnorm: out shape")
    partials, n_part, stride = None, 0, 0
    if delta is not None and delta.dim() == 3:
        _need(delta.dtype == torch.float32 and tuple(delta.shape[1:]) == (rows, H) and delta.is_contiguous(),
              "add_rmsnorm: partial sums must be contiguous float32 [slices, rows, H]")
        partials, n_part, stride, delta = delta, delta.shape[0], rows * H, None
    elif delta is not None:
        _need(delta.shape == x.shape and delta.dtype == out.dtype and delta.is_contiguous(), "add_rmsnorm: delta")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_add_rmsnorm_{_suffix(out.dtype)}")
    _check(f(_ptr(x), _ptr(delta), _ptr(partials), c_int(n_part), ctypes.c_longlong(stride), _ptr(weight), _ptr(out),
             c_float(eps), c_int(rows), c_int(H), _stream()), "add_rmsnorm")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor, page_indptr: torch.Tensor,
                  page_ids: torch.Tensor, inv_freq: torch.Tensor | None, kcache: torch.Tensor, vcache: torch.Tensor,
                  n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  write_cache: bool, status: torch.Tensor, bias: torch.Tensor | None = None,
                  qk_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """Rotate q (in place) and k by position, write rotated k and v into the request's pages.

    kcache/vcache: [pages, n_kv_heads, page_size, head_dim].  The element-wise stage before the rotation:
    ``bias`` float32 [C] is added to the row; ``qk_norm`` float32 [2, head_dim] RMS-normalises every q head (first
    row of weights) and every k head (second row) over the head size, with ``norm_eps``."""
    _need_cuda(qkv, positions, token_seq, page_indptr, page_ids, inv_freq, kcache, vcache, status, bias, qk_norm)
    _check_qkv_stage(bias, qk_norm, (n_heads + 2 * n_kv_heads) * head_dim, head_dim)
    n = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "rope_kv_write: qkv shape")
    _need(kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == qkv.dtype, "rope_kv_write: cache")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "rope_kv_write: cache layout")
    _need(0 <= rotary_dim <= head_dim and rotary_dim % 2 == 0, "rope_kv_write: rotary_dim")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "rope_kv_write: inv_freq must be float32 [rotary_dim/2]")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_rope_kv_write_{_suffix(qkv.dtype)}")
    _check(f(_ptr(qkv), _ptr(positions), _ptr(token_seq), _ptr(page_indptr), _ptr(page_ids), _ptr(inv_freq),
             _ptr(kcache), _ptr(vcache), c_int(n), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
             c_int(rotary_dim), c_int(page_size), c_int(kcache.shape[0]), c_int(1 if write_cache else 0),
             _ptr(status), _ptr(bias), _ptr(qk_norm), c_float(norm_eps), _stream()), "rope_kv_write")


def _check_qkv_stage(bias: torch.Tensor | None, qk_norm: torch.Tensor | None, C: int, head_dim: int) -> None:
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C, "q|k|v bias: float32 [C]")
    if qk_norm is not None:
        _need(qk_norm.dtype == torch.float32 and qk_norm.is_contiguous() and tuple(qk_norm.shape) == (2, head_dim),
              "q/k norm weights: float32 [2, head_dim]")


SMALL_M_MAX = 16   # above this many rows the library product is as fast or faster (measured on B200)
GATED_M_MAX = 8    # the gated small-batch product wins only up to this many rows
DECODE_M_MAX = 16
_EPILOGUES = {"bf16": 0, "add": 1, "gated": 2, "f32": 3}


def can_use_linear_decode(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (w.dtype == torch.bfloat16 and a.dtype in (torch.bfloat16, torch.float32) and 0 < a.shape[0] <= DECODE_M_MAX
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1)


def linear_decode(a: torch.Tensor, w: torch.Tensor, epilogue: str = "bf16", norm_weight: torch.Tensor | None = None,
                  eps: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused product for at most 16 rows: ``prologue(a) @ w^T`` with the epilogue applied in the same kernel.

    ``a``: bfloat16 [M, K], or the float32 residual stream [M, K] with ``norm_weight`` (an RMS norm is
    folded in).  ``epilogue``: "bf16" store; "f32" store; "add" adds into the float32 ``out`` [M, N] in place;
    "gated": ``w`` interleaves gate/up rows (``interleave_gate_up``), result silu(gate)*up [M, N/2]."""
    _need_cuda(a, w, norm_weight, out)
    _need(can_use_linear_decode(a, w), "linear_decode: at most 16 rows, bfloat16 weights, K a multiple of 8")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K, "linear_decode: shapes")
    pro = 1 if a.dtype == torch.float32 else 0
    _need((pro == 1) == (norm_weight is not None), "linear_decode: a float32 input goes with a norm weight")
    if pro:
        _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == K, "linear_decode: norm weight float32 [K]")
    epi = _EPILOGUES[epilogue]
    if epilogue == "add":
        _need(out is not None and out.dtype == torch.float32 and tuple(out.shape) == (M, N) and out.stride(1) == 1,
              "linear_decode: 'add' needs the float32 stream [M, N]")
    elif epilogue == "gated":
        _need(N % 16 == 0, "linear_decode: gated weights come in groups of 16 rows")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    else:
        out = torch.empty((M, N), dtype=torch.bfloat16 if epilogue == "bf16" else torch.float32, device=a.device)
    _check(_fn(_libs.get("linear_decode.cu"), "tkb_linear_decode_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(norm_weight), c_float(eps), _ptr(w), c_int(w.stride(0)), _ptr(out),
        c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(pro), c_int(epi), _stream()), "linear_decode")
    return out


def can_use_smallm(a: torch.Tensor, w: torch.Tensor, max_rows: int | None = None) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < a.shape[0] <= (max_rows or SMALL_M_MAX)
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def linear_smallm(a: torch.Tensor, w: torch.Tensor, max_slices: int = 8) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T for M <= 64 in bfloat16, as float32 slices [slices, M, N] of a K-split
    product (the consumer adds the slices).  ``max_slices=1`` gives the whole product as [1, M, N]."""
    _need_cuda(a, w)
    _need(can_use_smallm(a, w, 64), "linear_smallm: bfloat16, M <= 64, K a multiple of 8")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1, "linear_smallm: shapes")
    lib = _libs.get("linear_smallm.cu")
    slices = lib.tkb_linear_smallm_slices(c_int(N), c_int(K), c_int(max_slices))
    out = torch.empty((slices, M, N), dtype=torch.float32, device=a.device)
    _check(_fn(lib, "tkb_linear_smallm_bf16")(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                                              c_int(M), c_int(N), c_int(K), c_int(slices), _stream()), "linear_smallm")
    return out


def linear_smallm_gated(a: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """silu(a @ gate^T) * (a @ up^T) as bfloat16 [M, I] for M <= 64; ``w_interleaved`` [2I, K] holds gate
    and up rows in groups of 8 (``interleave_gate_up``)."""
    _need_cuda(a, w_interleaved)
    _need(can_use_smallm(a, w_interleaved, 64) and w_interleaved.shape[0] % 16 == 0, "linear_smallm_gated: operands")
    M, K = a.shape
    N = w_interleaved.shape[0]
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    _check(_fn(_libs.get("linear_smallm.cu"), "tkb_linear_smallm_gated_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w_interleaved), c_int(w_interleaved.stride(0)), _ptr(out), c_int(M), c_int(N),
        c_int(K), _stream()), "linear_smallm_gated")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K]: for every 8 features, their 8 gate rows then their 8 up rows.  I must be a multiple of 8."""
    I, K = gate.shape
    _need(I % 8 == 0 and up.shape == gate.shape, "interleave_gate_up: I must be a multiple of 8")
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def rope_kv_write_partials(partials: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                           token_seq: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor,
                           inv_freq: torch.Tensor | None, kcache: torch.Tensor, vcache: torch.Tensor, n_heads: int,
                           n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int, write_cache: bool,
                           status: torch.Tensor, bias: torch.Tensor | None = None,
                           qk_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """``rope_kv_write`` for q|k|v that arrive as float32 slices [slices, T, C] of a split product: the
    slices are added, q is rotated into ``q_out`` [T, n_heads*head_dim] (bfloat16), k and v go to the cache."""
    _need_cuda(partials, q_out, positions, token_seq, page_indptr, page_ids, inv_freq, kcache, vcache, status, bias,
               qk_norm)
    S, T, C = partials.shape
    _check_qkv_stage(bias, qk_norm, C, head_dim)
    _need(partials.dtype == torch.float32 and partials.is_contiguous() and C == (n_heads + 2 * n_kv_heads) * head_dim,
          "rope_kv_write_partials: partials")
    _need(q_out.dtype == torch.bfloat16 and q_out.is_contiguous() and tuple(q_out.shape) == (T, n_heads * head_dim),
          "rope_kv_write_partials: q_out")
    _need(kcache.dtype == torch.bfloat16 and tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim),
          "rope_kv_write_partials: cache layout")
    _need((C + max(rotary_dim, 2)) * 4 <= 160 * 1024, "rope_kv_write_partials: row too wide for shared memory")
    f = _fn(_libs.get("elementwise.cu"), "tkb_rope_kv_write_partials_bf16")
    _check(f(_ptr(partials), c_int(S), ctypes.c_longlong(T * C), _ptr(q_out), _ptr(positions), _ptr(token_seq),
             _ptr(page_indptr), _ptr(page_ids), _ptr(inv_freq), _ptr(kcache), _ptr(vcache), c_int(T), c_int(n_heads),
             c_int(n_kv_heads), c_int(head_dim), c_int(rotary_dim), c_int(page_size), c_int(kcache.shape[0]),
             c_int(1 if write_cache else 0), _ptr(status), _ptr(bias), _ptr(qk_norm), c_float(norm_eps), _stream()),
           "rope_kv_write_partials")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0, act: str = "silu") -> None:
    """out[t, i] = silu(gate[t, i]) * up[t, i].  interleave 0: gate_up = [gate | up]; interleave 8: columns in
    groups of 16, 8 gate columns then the 8 up columns of the same features.  ``act`` "gelu_tanh": the tanh form of
    GELU takes the SiLU's place."""
    _need(act in ("silu", "gelu_tanh"), f"silu_mul: the gate's activation is 'silu' or 'gelu_tanh', not {act!r}")
    _need_cuda(gate_up, out)
    rows, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (rows, two_i // 2), "silu_mul: shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype, "silu_mul: layout")
    f = _fn(_libs.get("elementwise.cu"), f"tkb_{act}_mul_{_suffix(out.dtype)}")
    _check(f(_ptr(gate_up), _ptr(out), c_int(rows), c_int(two_i // 2), c_int(interleave), _stream()), "silu_mul")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = src[rows[r]]."""
    _need_cuda(src, rows, out)
    _need(src.is_contiguous() and out.is_contiguous() and src.dtype == out.dtype, "gather_rows: layout")
    _need(rows.dtype == torch.int32 and out.shape[0] == rows.numel() and out.shape[1:] == src.shape[1:],
          "gather_rows: shapes")
    row_bytes = src[0].numel() * src.element_size() if src.shape[0] else 0
    f = _fn(_libs.get("elementwise.cu"), "tkb_gather_rows")
    _check(f(_ptr(src), _ptr(out), _ptr(rows), c_int(rows.numel()), c_int(row_bytes), _stream()), "gather_rows")


def sgemm_tn(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FP32 FMA, fixed summation order)."""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "sgemm_tn: shapes")
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "sgemm_tn: float32 only")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "sgemm_tn: rows must be contiguous")
    f = _fn(_libs.get("sgemm.cu"), "tkb_sgemm_tn_f32")
    _check(f(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0) if M > 1 else K),
             c_int(w.stride(0) if N > 1 else K), c_int(out.stride(0) if M > 1 else N), _stream()), "sgemm_tn")


def attn_paged(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
               token_seq: torch.Tensor, positions: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor,
               rows: torch.Tensor | None, n_rows: int, n_heads: int, n_kv_heads: int, head_dim: int,
               page_size: int, scale: float, window: int | None, status: torch.Tensor | None = None) -> None:
    """Causal GQA attention over the paged cache on the FP32 pipes (any mix of portions and single tokens).

    q: first n_heads*head_dim columns of each row of a [T, q_stride] buffer; out: [n_rows, n_heads*head_dim].
    ``status``: the device status word; a page id beyond the pool sets its bit 2 and its keys count for nothing."""
    _need_cuda(q, out, kcache, vcache, token_seq, positions, page_indptr, page_ids, rows, status)
    check_head_dim(head_dim)
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim and out.shape[0] >= n_rows, "attn_paged: out")
    _need(kcache.dtype == q.dtype == out.dtype, "attn_paged: dtypes")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_paged: cache layout")
    f = _fn(_libs.get("attention_simt.cu", TKB_HD=head_dim), f"tkb_attn_paged_simt_{_suffix(q.dtype)}")
    _check(f(_ptr(q), c_int(q_stride), _ptr(out), c_int(out.shape[1]), _ptr(kcache), _ptr(vcache), _ptr(token_seq),
             _ptr(positions), _ptr(page_indptr), _ptr(page_ids), _ptr(rows), c_int(n_rows), c_int(n_heads),
             c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0), c_int(kcache.shape[0]), _ptr(status),
             _stream()), "attn_paged")


_COUNTERS: dict = {}
_COUNTER_INTS = 1 << 20


def _decode_counters(device: torch.device, dec_cap: int, n_heads: int, n_kv_heads: int) -> torch.Tensor | None:
    """Arrival counters of the split-key kernel's in-kernel merge: one fixed zero-initialised array per device
    (every launch leaves it zero again).  None if a launch would need more than it holds."""
    group = n_heads // n_kv_heads
    need = dec_cap * n_kv_heads * ((group + 15) // 16)
    if need > _COUNTER_INTS:
        return None
    key = (device.type, device.index)
    t = _COUNTERS.get(key)
    if t is None:
        t = torch.zeros((_COUNTER_INTS,), dtype=torch.int32, device=device)
        _COUNTERS[key] = t
    return t


def attn_decode_mma(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, seq_q_start: torch.Tensor,
                    seq_kv_len: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor, items: torch.Tensor,
                    n_items: torch.Tensor, items_cap: int, dec_seqs: torch.Tensor, dec_item_start: torch.Tensor,
                    n_dec: torch.Tensor, dec_cap: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    page_size: int, scale: float, window: int | None,
                    out_row_of: torch.Tensor | None = None, item_entry: torch.Tensor | None = None,
                    tma: bool = True, status: torch.Tensor | None = None) -> None:
    """bfloat16 split-key attention for requests that bring one token: ``items`` are (request row,
    first key, number of keys) triples, computed into float32 partial results and merged into
    ``out`` [T, n_heads*head_dim] at each request's token row (or at row ``out_row_of[request]``).
    ``n_items``/``n_dec`` are device counters; the launch grids are sized by ``items_cap``/``dec_cap``.
    ``tma``: some work item is longer than three tiles (the kernel variant that fetches tiles by TMA pays)."""
    _need_cuda(qkv, kcache, vcache, seq_q_start, seq_kv_len, page_indptr, page_ids, items, n_items, dec_seqs,
               dec_item_start, n_dec, out, status)
    check_head_dim(head_dim)
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attn_decode_mma: bfloat16 only")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_decode_mma: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_decode_mma: out")
    _need(items.numel() >= 3 * items_cap and dec_item_start.numel() >= dec_cap + 1, "attn_decode_mma: plan arrays")
    lib = _libs.get("attention_mma.cu", TKB_HD=head_dim)
    part_o = torch.empty((items_cap, n_heads, head_dim), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((items_cap, n_heads, 2), dtype=torch.float32, device=qkv.device)
    counters = _decode_counters(qkv.device, dec_cap, n_heads, n_kv_heads) if item_entry is not None else None
    if counters is not None:
        # the merge of the splits happens inside the attention kernel
        _check(_fn(lib, "tkb_attn_decode_merged_bf16")(
            _ptr(qkv), c_int(qkv.shape[1]), _ptr(None), c_int(0), ctypes.c_longlong(0), _ptr(kcache), _ptr(vcache),
            _ptr(seq_q_start), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids), _ptr(items), _ptr(n_items),
            c_int(items_cap), _ptr(part_o), _ptr(part_ml), c_int(n_heads), c_int(n_kv_heads), c_int(page_size),
            c_float(scale), c_int(window or 0), c_int(0), _ptr(None), c_int(0), c_int(0), c_int(kcache.shape[0]),
            c_int(1 if tma else 0), _ptr(status), _ptr(counters), _ptr(item_entry), _ptr(dec_item_start),
            _ptr(out_row_of if out_row_of is not None else seq_q_start), _ptr(out), c_int(out.shape[1]), _ptr(None),
            _ptr(None), c_float(0.0), _stream()), "attn_decode_merged")
        return
    _check(_fn(lib, "tkb_attn_decode_mma_bf16")(
        _ptr(qkv), c_int(qkv.shape[1]), _ptr(kcache), _ptr(vcache), _ptr(seq_q_start), _ptr(seq_kv_len),
        _ptr(page_indptr), _ptr(page_ids), _ptr(items), _ptr(n_items), c_int(items_cap), _ptr(part_o), _ptr(part_ml),
        c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0),
        c_int(kcache.shape[0]), _ptr(status), _stream()), "attn_decode_mma")
    _check(_fn(lib, "tkb_attn_decode_merge_bf16")(
        _ptr(part_o), _ptr(part_ml), _ptr(dec_seqs), _ptr(dec_item_start), _ptr(n_dec), c_int(dec_cap),
        _ptr(out_row_of if out_row_of is not None else seq_q_start), _ptr(out), c_int(out.shape[1]), c_int(n_heads),
        _stream()), "attn_decode_merge")


def attn_decode_rope_mma(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, seq_q_start: torch.Tensor,
                         seq_kv_len: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor,
                         items: torch.Tensor, n_items: torch.Tensor, items_cap: int, dec_seqs: torch.Tensor,
                         dec_item_start: torch.Tensor, n_dec: torch.Tensor, dec_cap: int, out: torch.Tensor,
                         n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                         window: int | None, inv_freq: torch.Tensor | None, rotary_dim: int,
                         write_cache: bool, status: torch.Tensor, item_entry: torch.Tensor | None = None,
                         tma: bool = True, bias: torch.Tensor | None = None, qk_norm: torch.Tensor | None = None,
                         norm_eps: float = 0.0) -> None:
    """``attn_decode_mma`` with rotary encoding and the cache write folded in: ``qkv`` holds the step's
    un-rotated q|k|v rows of requests that bring one token each, as bfloat16 [T, C] or as the float32 slices
    [slices, T, C] of a K-split product (``linear_smallm``); C = (n_heads + 2 n_kv_heads) * head_dim."""
    _need_cuda(qkv, kcache, vcache, seq_q_start, seq_kv_len, page_indptr, page_ids, items, n_items, dec_seqs,
               dec_item_start, n_dec, out, inv_freq, status, bias, qk_norm)
    check_head_dim(head_dim)
    C = (n_heads + 2 * n_kv_heads) * head_dim
    _check_qkv_stage(bias, qk_norm, C, head_dim)
    _need(kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "attn_decode_rope_mma: bfloat16 only")
    _need(qkv.is_contiguous() and qkv.shape[-1] == C, "attn_decode_rope_mma: qkv")
    if qkv.dim() == 3:
        _need(qkv.dtype == torch.float32, "attn_decode_rope_mma: slices are float32")
        parts, n_parts, part_stride, qkv_ptr = qkv, qkv.shape[0], qkv.shape[1] * C, None
    else:
        _need(qkv.dtype == torch.bfloat16, "attn_decode_rope_mma: rows are bfloat16")
        parts, n_parts, part_stride, qkv_ptr = None, 0, 0, qkv
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_decode_rope_mma: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_decode_rope_mma: out")
    _need(rotary_dim % 4 == 0 and 0 <= rotary_dim <= head_dim, "attn_decode_rope_mma: rotary_dim")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "attn_decode_rope_mma: inv_freq")
    lib = _libs.get("attention_mma.cu", TKB_HD=head_dim)
    part_o = torch.empty((items_cap, n_heads, head_dim), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((items_cap, n_heads, 2), dtype=torch.float32, device=qkv.device)
    counters = _decode_counters(qkv.device, dec_cap, n_heads, n_kv_heads) if item_entry is not None else None
    if counters is not None:
        _check(_fn(lib, "tkb_attn_decode_merged_bf16")(
            _ptr(qkv_ptr), c_int(C), _ptr(parts), c_int(n_parts), ctypes.c_longlong(part_stride), _ptr(kcache),
            _ptr(vcache), _ptr(seq_q_start), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids), _ptr(items),
            _ptr(n_items), c_int(items_cap), _ptr(part_o), _ptr(part_ml), c_int(n_heads), c_int(n_kv_heads),
            c_int(page_size), c_float(scale), c_int(window or 0), c_int(1), _ptr(inv_freq),
            c_int(rotary_dim), c_int(1 if write_cache else 0), c_int(kcache.shape[0]), c_int(1 if tma else 0),
            _ptr(status), _ptr(counters),
            _ptr(item_entry), _ptr(dec_item_start), _ptr(seq_q_start), _ptr(out), c_int(out.shape[1]), _ptr(bias),
            _ptr(qk_norm), c_float(norm_eps), _stream()), "attn_decode_merged")
        return
    _check(_fn(lib, "tkb_attn_decode_rope_mma_bf16")(
        _ptr(qkv_ptr), c_int(C), _ptr(parts), c_int(n_parts), ctypes.c_longlong(part_stride), _ptr(kcache),
        _ptr(vcache), _ptr(seq_q_start), _ptr(seq_kv_len),
        _ptr(page_indptr), _ptr(page_ids), _ptr(items), _ptr(n_items), c_int(items_cap), _ptr(part_o), _ptr(part_ml),
        c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0),
        _ptr(inv_freq), c_int(rotary_dim), c_int(1 if write_cache else 0), c_int(kcache.shape[0]),
        c_int(1 if tma else 0), _ptr(status), _ptr(bias), _ptr(qk_norm), c_float(norm_eps), _stream()),
        "attn_decode_rope_mma")
    _check(_fn(lib, "tkb_attn_decode_merge_bf16")(
        _ptr(part_o), _ptr(part_ml), _ptr(dec_seqs), _ptr(dec_item_start), _ptr(n_dec), c_int(dec_cap),
        _ptr(seq_q_start), _ptr(out), c_int(out.shape[1]), c_int(n_heads), _stream()), "attn_decode_merge")


def attn_prefill_mma(qkv: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor,
                     page_indptr: torch.Tensor, page_ids: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor,
                     tiles_cap: int, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: int | None, status: torch.Tensor | None = None) -> None:
    """bfloat16 causal attention for prompt portions: ``tiles`` are (request row, first query of a
    64-query tile within the portion) pairs; results go to ``out`` [T, n_heads*head_dim] at the token rows."""
    _need_cuda(qkv, out, kcache, vcache, seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, tiles, n_tiles)
    check_head_dim(head_dim)
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attn_prefill_mma: bfloat16 only")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "attn_prefill_mma: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_prefill_mma: out")
    _need(tiles.numel() >= 2 * tiles_cap, "attn_prefill_mma: plan arrays")
    lib = _libs.get("attention_mma.cu", TKB_HD=head_dim)
    _check(_fn(lib, "tkb_attn_prefill_mma_bf16")(
        _ptr(qkv), c_int(qkv.shape[1]), _ptr(out), c_int(out.shape[1]), _ptr(kcache), _ptr(vcache), _ptr(seq_q_start),
        _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids), _ptr(tiles), _ptr(n_tiles),
        c_int(tiles_cap), c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_int(window or 0),
        c_int(kcache.shape[0]), _ptr(status), _stream()), "attn_prefill_mma")


ATTN_PREFILL_TC = True  # portions of prompts on the tcgen05 kernels where one takes the head size
# head size -> (source, compile-time constants, entry point).  Both accumulate the output in tensor memory; head
# size 64 has 128-key tiles and one S tile a head (the faster of the two there), head size 128 64-key tiles and two.
ATTN_PREFILL_TC_KERNELS = {
    64: ("attention_tc.cu", {}, "tkb_attn_prefill_tc_bf16"),
    128: ("attention_tc_acc.cu", {"TKB_HD": 128}, "tkb_attn_prefill_acc_bf16"),
}


def can_use_attn_prefill_tc(head_dim: int) -> bool:
    return ATTN_PREFILL_TC and head_dim in ATTN_PREFILL_TC_KERNELS


def attn_prefill_tc(qkv: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor,
                    page_indptr: torch.Tensor, page_ids: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor,
                    tiles_cap: int, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float,
                    window: int | None, status: torch.Tensor, single_heads: bool = False) -> None:
    """bfloat16 causal attention for prompt portions on tcgen05 tensor cores (head sizes 64 and 128): ``tiles`` are
    (request row, first query of a 128-query tile within the portion) pairs; results go to ``out``
    [T, n_heads*head_dim] at the token rows.  ``status`` collects a wait that ran out.  A block takes two query
    heads of a kv head; ``single_heads``: one (twice the blocks, for steps whose tiles are too few to give every
    SM a pair)."""
    _need_cuda(qkv, out, kcache, vcache, seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, tiles, n_tiles,
               status)
    _need(head_dim in ATTN_PREFILL_TC_KERNELS,
          f"attn_prefill_tc: head sizes {sorted(ATTN_PREFILL_TC_KERNELS)} only, got {head_dim}")
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attn_prefill_tc: bfloat16 only")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim) and kcache.is_contiguous()
          and vcache.shape == kcache.shape and vcache.is_contiguous(), "attn_prefill_tc: cache layout")
    _need(out.is_contiguous() and out.shape[1] == n_heads * head_dim, "attn_prefill_tc: out")
    _need(qkv.stride(1) == 1 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0,
          "attn_prefill_tc: rows of q must start on 16-byte boundaries")
    _need(tiles.numel() >= 2 * tiles_cap, "attn_prefill_tc: plan arrays")
    source, defines, entry = ATTN_PREFILL_TC_KERNELS[head_dim]
    _check(_fn(_libs.get(source, **defines), entry)(
        _ptr(qkv), c_int(qkv.stride(0)), _ptr(out), c_int(out.shape[1]), _ptr(kcache), _ptr(vcache),
        c_int(kcache.shape[0]), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(page_indptr), _ptr(page_ids),
        _ptr(tiles), _ptr(n_tiles), c_int(tiles_cap), c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale),
        c_int(window or 0), c_int(1 if single_heads else 0), _ptr(status), _stream()), "attn_prefill_tc")


def sample(logits: torch.Tensor, temperature: torch.Tensor | None, stream_key: torch.Tensor | None,
           sample_pos: torch.Tensor | None, row_slot: torch.Tensor | None, out_ids: torch.Tensor,
           out_logprob: torch.Tensor | None, last_token: torch.Tensor | None) -> None:
    """Greedy (temperature <= 0) or Gumbel-max temperature sampling of one id per row of logits [R, V]."""
    _need_cuda(logits, temperature, stream_key, sample_pos, row_slot, out_ids, out_logprob, last_token)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(out_ids.dtype == torch.int32 and out_ids.numel() >= R, "sample: out_ids int32 [R]")
    if stream_key is not None:
        _need(stream_key.dtype == torch.int64, "sample: stream_key int64 [R]")
    lib = _libs.get("sampling.cu")
    nch = lib.tkb_sample_chunks(c_int(R), c_int(V))
    if nch > 1:
        # few rows, large vocabulary: chunks of the vocabulary in parallel, then a fold in chunk order
        part = torch.empty((R, nch, 4), dtype=torch.float32, device=logits.device)
        _check(_fn(lib, "tkb_sample_two_stage")(
            _ptr(logits), _ptr(temperature), _ptr(stream_key), _ptr(sample_pos), _ptr(row_slot), _ptr(out_ids),
            _ptr(out_logprob), _ptr(last_token), _ptr(part), c_int(nch), c_int(R), c_int(V), _stream()), "sample")
        return
    f = _fn(lib, "tkb_sample")
    _check(f(_ptr(logits), _ptr(temperature), _ptr(stream_key), _ptr(sample_pos), _ptr(row_slot), _ptr(out_ids),
             _ptr(out_logprob), _ptr(last_token), c_int(R), c_int(V), _stream()), "sample")


def noise_of_bits(bits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The uniform number in (0, 1) and the Gumbel value the sampling kernels make of 32 random bits each
    (``bits``: int32 holding the bit patterns).  For tests of the extremes."""
    _need_cuda(bits)
    _need(bits.dtype == torch.int32 and bits.is_contiguous(), "noise_of_bits: bits must be contiguous int32")
    u = torch.empty(bits.numel(), dtype=torch.float32, device=bits.device)
    g = torch.empty_like(u)
    _check(_fn(_libs.get("sampling.cu"), "tkb_noise_of_bits")(_ptr(bits), _ptr(u), _ptr(g), c_int(bits.numel()), _stream()),
           "noise_of_bits")
    return u, g


def topk_logprobs(logits: torch.Tensor, temperature: torch.Tensor | None, k: int, out_idx: torch.Tensor,
                  out_lp: torch.Tensor) -> None:
    _need_cuda(logits, temperature, out_idx, out_lp)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "topk_logprobs: logits")
    _need(out_idx.shape == (R, k) and out_lp.shape == (R, k) and out_idx.dtype == torch.int32, "topk_logprobs: outs")
    f = _fn(_libs.get("sampling.cu"), "tkb_topk_logprobs")
    _check(f(_ptr(logits), _ptr(temperature), _ptr(out_idx), _ptr(out_lp), c_int(R), c_int(V), c_int(k), _stream()),
           "topk_logprobs")


TCGEN05_M_MIN = 128  # from this many rows on the gated tcgen05 product beats library product + activation kernel


def can_use_tcgen05(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and a.shape[1] % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, gated: bool = False) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T in bfloat16 on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).
    ``gated``: ``w`` interleaves gate/up rows (``interleave_gate_up``); the result is silu(gate)*up [M, N/2].
    ``status``: the device status word; a bounded wait that runs out sets its bit 4."""
    _need_cuda(a, w, status)
    _need(can_use_tcgen05(a, w), "gemm_tcgen05: bfloat16 operands, K and strides multiples of 8, 16-byte aligned")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and (not gated or N % 16 == 0), "gemm_tcgen05: shapes")
    out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=a.device)
    _check(_fn(_libs.get("gemm_tcgen05.cu"), "tkb_gemm_tcgen05_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N),
        c_int(K), c_int(1 if gated else 0), _ptr(status), _stream()), "gemm_tcgen05")
    return out


def gemm_tcgen05_clamped(a: torch.Tensor, w_interleaved: torch.Tensor, status: torch.Tensor, limit: float,
                         alpha: float) -> torch.Tensor:
    """The gated tcgen05 product with the clamped unit in its epilogue: ``w_interleaved`` interleaves gate and up rows
    (``interleave_gate_up``); the result is g * sigmoid(alpha g) * (u + 1) [M, N / 2] with g = min(gate, limit),
    u = clamp(up, -limit, limit), taken from the float32 accumulators."""
    _need_cuda(a, w_interleaved, status)
    _need(can_use_tcgen05(a, w_interleaved), "gemm_tcgen05_clamped: bfloat16 operands, K and strides multiples of 8, 16-byte aligned")
    M, K = a.shape
    N = w_interleaved.shape[0]
    _need(w_interleaved.shape[1] == K and N % 16 == 0 and limit > 0, "gemm_tcgen05_clamped: shapes, a positive limit")
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    _check(_fn(_libs.get("gemm_tcgen05.cu"), "tkb_gemm_tcgen05_clamped_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w_interleaved), c_int(w_interleaved.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(M), c_int(N), c_int(K), c_float(limit), c_float(alpha), _ptr(status), _stream()), "gemm_tcgen05_clamped")
    return out


TC_DECODE_M_MAX = 64


def linear_tc_decode(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, max_slices: int = 16,
                     gated: bool = False) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T for M <= 64 on the tcgen05 tensor cores with the weights on the 128-row side
    (TMA-fed ten-stage ring).  Returns float32 slices [slices, M, N] of a K-split product, or with ``gated``
    (``w`` from ``interleave_gate_up``) silu(gate)*up as bfloat16 [M, N/2]."""
    _need_cuda(a, w, status)
    _need(can_use_tcgen05(a, w) and 0 < a.shape[0] <= TC_DECODE_M_MAX, "linear_tc_decode: bfloat16, M <= 64, K % 8 == 0")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and (not gated or N % 16 == 0), "linear_tc_decode: shapes")
    lib = _libs.get("gemm_tcgen05_decode.cu")
    slices = 1 if gated else lib.tkb_linear_tcgen05_decode_slices(c_int(N), c_int(K), c_int(max_slices))
    if gated:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    else:
        out = torch.empty((slices, M, N), dtype=torch.float32, device=a.device)
    _check(_fn(lib, "tkb_linear_tcgen05_decode_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(M), c_int(N), c_int(K),
        c_int(slices), c_int(1 if gated else 0), _ptr(status), _stream()), "linear_tc_decode")
    return out


FEW_ROWS_MAX = 16  # measured on B200: from 17 rows on, library products + separate kernels are faster than the K-split path
# ... except for the attention block's two products, whose weights are small (the library's kernels take 10 us each
# for 2 us worth of bytes at 64 rows) and whose slices the attention kernel and the norm add on their way anyway:
# measured at Llama-3.2-1B sizes, batch 32: 24.2 k -> 25.5 k tok/s, batch 64: 38.1 k -> 38.6 k
ATTN_FEW_ROWS_MAX = 64


def can_use_few_rows(a: torch.Tensor, w: torch.Tensor, max_rows: int | None = None) -> bool:
    """Steps with few rows (decode) use K-split products whose float32 slices the consumer adds."""
    if a.shape[0] <= SMALL_M_MAX:
        return can_use_smallm(a, w)
    return a.shape[0] <= (max_rows or FEW_ROWS_MAX) and can_use_tcgen05(a, w)


def linear_few_rows(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor | None) -> torch.Tensor:
    """Float32 slices [slices, M, N] of a[M, K] @ w[N, K]^T: the mma.sync kernel up to 16 rows (measured
    faster there), the tcgen05 kernel above (if ``FEW_ROWS_MAX`` is raised)."""
    if a.shape[0] <= SMALL_M_MAX:
        return linear_smallm(a, w)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=a.device)
    return linear_tc_decode(a, w, status)


def linear_few_rows_gated(a: torch.Tensor, w_interleaved: torch.Tensor, status: torch.Tensor | None) -> torch.Tensor:
    """silu(gate) * up [M, I] for at most 64 rows: mma.sync kernel up to 8 rows, tcgen05 kernel above."""
    if a.shape[0] <= GATED_M_MAX:
        return linear_smallm_gated(a, w_interleaved)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=a.device)
    return linear_tc_decode(a, w_interleaved, status, gated=True)


def linear(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T.  float32: this engine's FP32 kernel (no tf32).  bfloat16: the library
    matrix product (cuBLAS through torch), float32 accumulation, output bfloat16 or float32."""
    _need_cuda(a, w)
    M = a.shape[0]
    N = w.shape[0]
    if a.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        sgemm_tn(a, w, out)
        return out
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must share the engine dtype")
    if out_dtype is None or out_dtype == torch.bfloat16:
        return torch.mm(a, w.t())
    return torch.mm(a, w.t(), out_dtype=out_dtype)


def softmax_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


# ---------------------------------------------------------------------------------------------
# Layer norm, short convolution, PolyNorm (csrc/norm_conv.cu)
def _split_update(delta: torch.Tensor | None, rows: int, H: int, act_dtype: torch.dtype, what: str):
    """A residual update as (rows in the activation type | None, float32 slices | None, slices, slice stride)."""
    if delta is None:
        return None, None, 0, 0
    if delta.dim() == 3:
        _need(delta.dtype == torch.float32 and tuple(delta.shape[1:]) == (rows, H) and delta.is_contiguous(),
              f"{what}: slices must be contiguous float32 [slices, rows, H]")
        return None, delta, delta.shape[0], rows * H
    _need(tuple(delta.shape) == (rows, H) and delta.is_contiguous(), f"{what}: update shape")
    if delta.dtype == torch.float32 and act_dtype != torch.float32:
        return None, delta, 1, rows * H
    _need(delta.dtype == act_dtype, f"{what}: the update is in the activation type or float32")
    return delta, None, 0, 0


def add_layernorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                  out: torch.Tensor) -> None:
    """x += delta (float32, in place) if given; out = (x - mean) / sqrt(var + eps) * weight + bias in out's dtype."""
    _need_cuda(x, delta, weight, bias, out)
    rows, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_layernorm: x must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == H and bias.dtype == torch.float32 and bias.numel() == H,
          "add_layernorm: weight and bias must be float32 [H]")
    _need(out.shape == x.shape and out.is_contiguous(), "add_layernorm: out shape")
    d, sl, n_sl, stride = _split_update(delta, rows, H, out.dtype, "add_layernorm")
    f = _fn(_libs.get("norm_conv.cu"), f"tkb_add_layernorm_{_suffix(out.dtype)}")
    _check(f(_ptr(x), _ptr(d), _ptr(sl), c_int(n_sl), ctypes.c_longlong(stride), _ptr(weight), _ptr(bias), _ptr(out),
             c_float(eps), c_int(rows), c_int(H), _stream()), "add_layernorm")


def add_layernorm_conv1(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor,
                        eps: float, conv_w: torch.Tensor, carry: torch.Tensor, token_seq: torch.Tensor,
                        seq_slot: torch.Tensor, out: torch.Tensor) -> None:
    """``add_layernorm`` followed by ``short_conv`` for a step in which every request brings one token, in one kernel."""
    _need_cuda(x, delta, weight, bias, conv_w, carry, token_seq, seq_slot, out)
    rows, H = x.shape
    taps = conv_w.shape[1]
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.shape == x.shape and out.is_contiguous(),
          "add_layernorm_conv1: x float32, out of the same shape")
    _need(weight.dtype == torch.float32 and weight.numel() == H and bias.dtype == torch.float32 and bias.numel() == H,
          "add_layernorm_conv1: weight and bias must be float32 [H]")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == H, "add_layernorm_conv1: taps")
    _need(carry.dtype == torch.float32 and carry.is_contiguous() and tuple(carry.shape[1:]) == (max(taps - 1, 0), H),
          "add_layernorm_conv1: carried inputs float32 [slots, taps - 1, H]")
    d, sl, n_sl, stride = _split_update(delta, rows, H, out.dtype, "add_layernorm_conv1")
    f = _fn(_libs.get("norm_conv.cu"), f"tkb_add_layernorm_conv1_{_suffix(out.dtype)}")
    _check(f(_ptr(x), _ptr(d), _ptr(sl), c_int(n_sl), ctypes.c_longlong(stride), _ptr(weight), _ptr(bias),
             _ptr(conv_w), _ptr(carry), _ptr(token_seq), _ptr(seq_slot), _ptr(out), c_float(eps), c_int(rows), c_int(H),
             c_int(taps), _stream()), "add_layernorm_conv1")


def short_conv(h: torch.Tensor, out: torch.Tensor, conv_w: torch.Tensor, carry: torch.Tensor, token_seq: torch.Tensor,
               seq_slot: torch.Tensor, seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, n_seqs: int) -> None:
    """out_t = h_t + sum_j conv_w[:, j] * h_(t - taps + 1 + j) over each request's tokens in order; inputs from before
    the step come from ``carry`` [slots, taps - 1, H] (float32, oldest first), which is then brought forward."""
    _need_cuda(h, out, conv_w, carry, token_seq, seq_slot, seq_q_start, seq_q_len)
    n, H = h.shape
    taps = conv_w.shape[1]
    _need(h.is_contiguous() and out.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype
          and out.data_ptr() != h.data_ptr(), "short_conv: out is another tensor of h's shape and type")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == H, "short_conv: taps float32 [H, taps]")
    _need(carry.dtype == torch.float32 and carry.is_contiguous() and tuple(carry.shape[1:]) == (max(taps - 1, 0), H),
          "short_conv: carried inputs float32 [slots, taps - 1, H]")
    f = _fn(_libs.get("norm_conv.cu"), f"tkb_short_conv_{_suffix(h.dtype)}")
    _check(f(_ptr(h), _ptr(out), _ptr(conv_w), _ptr(carry), _ptr(token_seq), _ptr(seq_slot), _ptr(seq_q_start),
             _ptr(seq_q_len), c_int(n), c_int(n_seqs), c_int(H), c_int(taps), _stream()), "short_conv")


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(u) = u / sqrt(mean(u^2) + eps); z float32, coef float32 [4]."""
    _need_cuda(z, coef, out)
    rows, F = z.shape
    _need(z.dtype == torch.float32 and z.is_contiguous() and out.shape == z.shape and out.is_contiguous(),
          "polynorm: z contiguous float32, out of the same shape")
    _need(coef.dtype == torch.float32 and coef.numel() == 4, "polynorm: four float32 coefficients")
    f = _fn(_libs.get("norm_conv.cu"), f"tkb_polynorm_{_suffix(out.dtype)}")
    _check(f(_ptr(z), _ptr(coef), _ptr(out), c_float(eps), c_int(rows), c_int(F), _stream()), "polynorm")


# ---------------------------------------------------------------------------------------------
# Gated linear recurrence (csrc/recurrence.cu)
def recurrence_defines(dim: int, vdim: int) -> dict:
    """The compile-time constants of the recurrence kernel for heads of ``dim`` x ``vdim``."""
    _need(0 < dim <= 512 and 0 < vdim <= 1024, f"gated recurrence: head sizes up to 512 x 1024, not {dim} x {vdim}")
    return dict(TKB_REC_DPT=(dim + 7) // 8, TKB_REC_CPT=(vdim + 127) // 128)


def gated_recurrence(qfv: torch.Tensor, state: torch.Tensor, f_bias: torch.Tensor, low: torch.Tensor,
                     norm_w: torch.Tensor, out: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor,
                     seq_q_len: torch.Tensor, n_seqs: int, heads: int, dim: int, vdim: int, eps: float,
                     write_state: bool = True, split_heads: bool = True) -> None:
    """The recurrence S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t over each request's tokens, then an
    RMS norm of every head's o.  qfv: float32 [T, heads*dim (q) + heads*dim (f) + heads*vdim (v)] raw projections;
    state: float32 [slots, heads, vdim, dim] (S transposed); out: [T, heads*vdim].  ``split_heads``: a step with more
    tokens than requests may spread a head's columns over several blocks (raw outputs through a float32 buffer)."""
    _need_cuda(qfv, state, f_bias, low, norm_w, out, seq_slot, seq_q_start, seq_q_len)
    T = qfv.shape[0]
    _need(qfv.dtype == torch.float32 and qfv.stride(1) == 1 and qfv.shape[1] == heads * (2 * dim + vdim),
          "gated_recurrence: qfv float32 [T, heads * (2 dim + vdim)]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, dim),
          "gated_recurrence: state float32 [slots, heads, vdim, dim]")
    for v, n, what in ((f_bias, heads * dim, "gate bias"), (low, heads * dim, "lower bound"), (norm_w, vdim, "norm weight")):
        _need(v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n, f"gated_recurrence: {what} float32 [{n}]")
    _need(out.is_contiguous() and tuple(out.shape) == (T, heads * vdim), "gated_recurrence: out [T, heads * vdim]")
    f = _fn(_libs.get("recurrence.cu", **recurrence_defines(dim, vdim)), f"tkb_gated_recurrence_{_suffix(out.dtype)}")
    raw = torch.empty((T, heads * vdim), dtype=torch.float32, device=qfv.device) if (split_heads and T > n_seqs) else None
    _check(f(_ptr(qfv), c_int(qfv.stride(0)), _ptr(state), _ptr(f_bias), _ptr(low), _ptr(norm_w), _ptr(out),
             _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), c_int(n_seqs), c_int(T), c_int(heads), c_int(dim),
             c_int(vdim), c_float(eps), c_int(1 if write_state else 0), _ptr(raw), _stream()), "gated_recurrence")


# ---------------------------------------------------------------------------------------------
# Attention over cached latents (csrc/latent_attention.cu)
def latent_prep(proj: torch.Tensor, q_off: int, q_rank: int, q_norm_w: torch.Tensor | None, cq_out: torch.Tensor | None,
                kv_off: int, rank: int, rot: int, rot_dims: int, kv_norm_w: torch.Tensor | None,
                inv_freq: torch.Tensor | None, cache: torch.Tensor | None, positions: torch.Tensor,
                token_seq: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor, page_size: int, eps: float,
                status: torch.Tensor, act_dtype: torch.dtype, freq64: torch.Tensor | None = None, halves: bool = False,
                mag: float = 1.0) -> None:
    """From float32 projections [T, .]: the RMS-normed query latent (columns q_off..+q_rank) into ``cq_out``; if
    ``kv_off`` >= 0 the RMS-normed latent (rank columns) and the rotated shared key part (rot columns, the first
    ``rot_dims`` rotated in interleaved pairs) into the request's cache rows [pages, page_size, rank + rot].
    ``freq64`` float64 [rot_dims / 2] in place of ``inv_freq``: angles, sines and cosines in float64, times ``mag``;
    ``halves``: channel i turns with channel i + rot_dims / 2."""
    _need_cuda(proj, q_norm_w, cq_out, kv_norm_w, inv_freq, cache, positions, token_seq, page_indptr, page_ids, status, freq64)
    _need(freq64 is None or (freq64.dtype == torch.float64 and freq64.is_contiguous() and freq64.numel() == rot_dims // 2),
          "latent_prep: freq64 float64 [rot_dims / 2]")
    n = proj.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1, "latent_prep: float32 projections")
    if q_rank:
        _need(cq_out is not None and cq_out.is_contiguous() and tuple(cq_out.shape) == (n, q_rank) and cq_out.dtype == act_dtype
              and q_norm_w is not None and q_norm_w.dtype == torch.float32 and q_norm_w.numel() == q_rank,
              "latent_prep: query latent output [T, q_rank] and its float32 norm weight")
    num_pages = 0
    if kv_off >= 0:
        _need(cache is not None and cache.is_contiguous() and cache.dtype == act_dtype
              and tuple(cache.shape[1:]) == (1, page_size, rank + rot), "latent_prep: cache [pages, 1, page_size, rank + rot]")
        _need(kv_norm_w is not None and kv_norm_w.dtype == torch.float32 and kv_norm_w.numel() == rank, "latent_prep: norm weight")
        _need(rot_dims == 0 or freq64 is not None
              or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2),
              "latent_prep: inv_freq float32 [rot_dims / 2]")
        num_pages = cache.shape[0]
    f = _fn(_libs.get("latent_attention.cu", TKB_LAT_RANK=rank), f"tkb_latent_prep_{_suffix(act_dtype)}")
    _check(f(_ptr(proj), c_int(proj.stride(0)), c_int(q_off), c_int(q_rank), _ptr(q_norm_w), _ptr(cq_out), c_int(kv_off),
             c_int(rot), c_int(rot_dims), _ptr(kv_norm_w), _ptr(inv_freq), _ptr(cache), _ptr(positions), _ptr(token_seq),
             _ptr(page_indptr), _ptr(page_ids), c_int(page_size), c_int(num_pages), c_float(eps), c_int(n), _ptr(status),
             _ptr(freq64), c_int(1 if halves else 0), c_float(mag), _stream()), "latent_prep")


def rotate_pairs(x: torch.Tensor, n_heads: int, head_stride: int, off: int, rot: int, rot_dims: int,
                 inv_freq: torch.Tensor | None, positions: torch.Tensor, token_seq: torch.Tensor, rank: int,
                 out: torch.Tensor | None = None, out_head_stride: int = 0, out_off: int = 0,
                 freq64: torch.Tensor | None = None, halves: bool = False, mag: float = 1.0) -> None:
    """Interleaved rotary encoding of the ``rot`` values at column ``off`` of every head of x [T, .]: the pairs
    (2i, 2i + 1), i < rot_dims / 2, are turned by position * inv_freq[i], the rest passes.  In place, or into the
    columns ``out_off`` of every head of ``out`` [T, .].  ``freq64``, ``halves``, ``mag``: as in ``latent_prep``."""
    _need_cuda(x, inv_freq, positions, token_seq, out, freq64)
    _need(freq64 is None or (freq64.dtype == torch.float64 and freq64.is_contiguous() and freq64.numel() == rot_dims // 2),
          "rotate_pairs: freq64 float64 [rot_dims / 2]")
    _need(x.stride(1) == 1 and off + rot <= head_stride and n_heads * head_stride <= x.shape[1], "rotate_pairs: layout")
    _need(rot_dims == 0 or freq64 is not None
          or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2),
          "rotate_pairs: inv_freq float32 [rot_dims / 2]")
    if out is None:
        if rot_dims == 0:
            return
        out, out_head_stride, out_off = x, head_stride, off
    _need(out.dtype == x.dtype and out.stride(1) == 1 and out.shape[0] == x.shape[0] and out_off + rot <= out_head_stride
          and n_heads * out_head_stride <= out.shape[1], "rotate_pairs: out layout")
    f = _fn(_libs.get("latent_attention.cu", TKB_LAT_RANK=rank), f"tkb_rotate_pairs_{_suffix(x.dtype)}")
    _check(f(_ptr(x), c_int(x.stride(0)), c_int(head_stride), c_int(off), _ptr(out), c_int(out.stride(0)),
             c_int(out_head_stride), c_int(out_off), c_int(n_heads), c_int(rot), c_int(rot_dims), _ptr(inv_freq),
             _ptr(positions), _ptr(token_seq), c_int(x.shape[0]), _ptr(freq64), c_int(1 if halves else 0), c_float(mag),
             _stream()), "rotate_pairs")


def head_sigmoid_gate(val: torch.Tensor, gate: torch.Tensor, gate_off: int, rows: torch.Tensor | None, n_heads: int,
                      vdim: int, rank: int) -> None:
    """val [n_rows, heads * vdim] *= sigmoid(gate[token, gate_off + head]) in place: an output gate, one number a
    (token, head).  ``gate`` float32 [T, .]; ``rows`` int32 names the tokens of val's rows (None: row r is token r).
    ``rank``: the latent rank whose kernel module holds the kernel."""
    _need_cuda(val, gate, rows)
    _need(val.is_contiguous() and val.shape[1] == n_heads * vdim, "head_sigmoid_gate: val [rows, heads * vdim]")
    _need(gate.dtype == torch.float32 and gate.stride(1) == 1 and gate_off + n_heads <= gate.shape[1],
          "head_sigmoid_gate: float32 gate logits")
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() == val.shape[0]), "head_sigmoid_gate: rows")
    f = _fn(_libs.get("latent_attention.cu", TKB_LAT_RANK=rank), f"tkb_head_sigmoid_gate_{_suffix(val.dtype)}")
    _check(f(_ptr(val), _ptr(gate), c_int(gate.stride(0)), c_int(gate_off), _ptr(rows), c_int(val.shape[0]), c_int(n_heads),
             c_int(vdim), _stream()), "head_sigmoid_gate")


def latent_attn(q_abs: torch.Tensor, q_rot: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, token_seq: torch.Tensor,
                positions: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor, rows: torch.Tensor | None,
                n_rows: int, page_size: int, scale: float, window: int | None, status: torch.Tensor) -> None:
    """q_abs [T, heads, rank] and q_rot [T, heads, rot] (any strides with a unit last one); cache
    [pages, 1, page_size, rank + rot]; out [n_rows, heads, rank]: softmax((q_abs . c + q_rot . k_rot) * scale) over
    the rows of the last ``window`` positions, times c."""
    _need_cuda(q_abs, q_rot, out, cache, token_seq, positions, page_indptr, page_ids, rows, status)
    T, nh, rank = q_abs.shape
    rot = q_rot.shape[2]
    _need(q_abs.stride(2) == 1 and q_rot.stride(2) == 1 and q_rot.shape[:2] == q_abs.shape[:2], "latent_attn: q layout")
    _need(q_abs.dtype == cache.dtype and q_rot.dtype == cache.dtype and out.dtype == cache.dtype, "latent_attn: one type")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (1, page_size, rank + rot), "latent_attn: cache layout")
    _need(out.is_contiguous() and tuple(out.shape) == (n_rows, nh, rank), "latent_attn: out [rows, heads, rank]")
    # few rows (the wanted rows of a prompt's last layer, decode steps of a float32 engine): a (row, head)'s visible
    # rows are shared out among warps until the SMs hold eight each (a function of the step's shape only, so that the
    # same step replays from a graph); a small kernel puts the shares together
    from tokasaurus_b200.kernels.device import device_limits

    splits, part = 1, None
    warps = n_rows * nh
    sms = device_limits(q_abs.device).sm_count
    if 0 < warps < 4 * sms:
        splits = min(32, (8 * sms) // warps)
        if window:
            splits = min(splits, max(1, -(-window // 32)))
        if splits > 1:
            part = torch.empty((warps * splits * (rank + 2),), dtype=torch.float32, device=q_abs.device)
    f = _fn(_libs.get("latent_attention.cu", TKB_LAT_RANK=rank), f"tkb_latent_attn_simt_{_suffix(cache.dtype)}")
    _check(f(_ptr(q_abs), ctypes.c_longlong(q_abs.stride(0)), ctypes.c_longlong(q_abs.stride(1)), _ptr(q_rot),
             ctypes.c_longlong(q_rot.stride(0)), ctypes.c_longlong(q_rot.stride(1)), c_int(rot), _ptr(out), _ptr(cache),
             _ptr(token_seq), _ptr(positions), _ptr(page_indptr), _ptr(page_ids), _ptr(rows), c_int(n_rows), c_int(nh),
             c_int(page_size), c_float(scale), c_int(window or 0), c_int(cache.shape[0]), _ptr(status), c_int(splits),
             _ptr(part), _stream()), "latent_attn")


# ---------------------------------------------------------------------------------------------
# Routed experts (csrc/moe.cu)
def moe_route(h: torch.Tensor, router_w: torch.Tensor, router_b: torch.Tensor | None, token_seq: torch.Tensor,
              top: int, top_idx: torch.Tensor, top_w: torch.Tensor, scored: dict | None = None,
              over_all: bool = False, scale: float = 1.0) -> None:
    """Router logits h @ router_w^T + router_b in float32, the ``top`` largest per token (int32 [T, top]) and the
    softmax over them (float32 [T, top]).  ``scored`` = dict(correction float32 [E] or None, groups, keep, scale): the
    other way of choosing: scores sigmoid(logits); the choice by score + correction among the experts of the best
    ``keep`` of ``groups`` equal groups of neighbours (a group scores the sum of its two largest choice scores); the
    weights are the chosen scores over their sum, times ``scale``.
    ``over_all`` (the plain way of choosing): the weights are the chosen experts' shares of the softmax over ALL experts,
    not renormalised; ``scale`` multiplies the plain way's weights."""
    _need_cuda(h, router_w, router_b, token_seq, top_idx, top_w)
    T, H = h.shape
    E = router_w.shape[0]
    _need(h.is_contiguous() and router_w.dtype == torch.float32 and router_w.is_contiguous() and router_w.shape[1] == H,
          "moe_route: router weight float32 [E, H]")
    _need(router_b is None or (router_b.dtype == torch.float32 and router_b.numel() == E), "moe_route: bias float32 [E]")
    _need(top_idx.dtype == torch.int32 and top_w.dtype == torch.float32 and tuple(top_idx.shape) == (T, top)
          and tuple(top_w.shape) == (T, top) and top_idx.is_contiguous() and top_w.is_contiguous(), "moe_route: outputs [T, top]")
    logits = torch.empty((T, E), dtype=torch.float32, device=h.device)
    if scored is not None:
        corr, groups, keep = scored.get("correction"), int(scored.get("groups", 1)), int(scored.get("keep", 1))
        _need_cuda(corr)
        _need(corr is None or (corr.dtype == torch.float32 and corr.is_contiguous() and corr.numel() == E),
              "moe_route: correction float32 [E]")
        _need(groups > 0 and E % groups == 0 and 0 < keep <= groups and top <= keep * (E // groups),
              f"moe_route: {E} experts in {groups} groups of which {keep} are kept, {top} chosen")
        f = _fn(_libs.get("moe.cu"), f"tkb_moe_route_scored_{_suffix(h.dtype)}")
        _check(f(_ptr(h), _ptr(router_w), _ptr(router_b), _ptr(corr), _ptr(token_seq), _ptr(top_idx), _ptr(top_w),
                 _ptr(logits), c_int(T), c_int(H), c_int(E), c_int(top), c_int(groups), c_int(keep),
                 c_float(float(scored.get("scale", 1.0))), _stream()), "moe_route")
        return
    f = _fn(_libs.get("moe.cu"), f"tkb_moe_route_{_suffix(h.dtype)}")
    _check(f(_ptr(h), _ptr(router_w), _ptr(router_b), _ptr(token_seq), _ptr(top_idx), _ptr(top_w), _ptr(logits), c_int(T),
             c_int(H), c_int(E), c_int(top), c_int(1 if over_all else 0), c_float(scale), _stream()), "moe_route")


def moe_logits(h: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> None:
    """out [T, E] = h @ w^T (+ bias) with float32 weights w [E, H], float32 sums: the router's first kernel alone, for
    other small products that want float32 (a gate of one number a token)."""
    _need_cuda(h, w, out, bias)
    T, H = h.shape
    E = w.shape[0]
    _need(h.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous() and w.shape[1] == H
          and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (T, E), "moe_logits: shapes")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == E), "moe_logits: bias float32 [E]")
    _check(_fn(_libs.get("moe.cu"), f"tkb_moe_logits_{_suffix(h.dtype)}")(
        _ptr(h), _ptr(w), _ptr(bias), _ptr(out), c_int(T), c_int(H), c_int(E), _stream()), "moe_logits")


def moe_order(top_idx: torch.Tensor, n_experts: int, offsets: torch.Tensor, order: torch.Tensor,
              place_of: torch.Tensor, pad: int = 1, tile_group: torch.Tensor | None = None,
              src_token: torch.Tensor | None = None) -> None:
    """Order the (token, choice) pairs by expert: offsets int32 [E + 1], order int32 (pair at each place),
    place_of int32 [pairs] (place of each pair, -1 for pairs of padding tokens).  ``pad`` > 1: every expert's span
    starts at a multiple of ``pad``; ``tile_group`` int32 [tiles] then receives the expert that owns each tile of
    ``pad`` places (-1: none) and ``src_token`` int32 [places] the token whose row stands at each place (-1: padding);
    ``order`` must then hold as many entries as ``src_token``."""
    _need_cuda(top_idx, offsets, order, place_of, tile_group, src_token)
    n = top_idx.numel()
    top = top_idx.shape[1]
    for t in (top_idx, offsets, order, place_of, tile_group, src_token):
        _need(t is None or (t.dtype == torch.int32 and t.is_contiguous()), "moe_order: int32 arrays")
    _need(offsets.numel() == n_experts + 1 and place_of.numel() == n, "moe_order: sizes")
    cap = n if pad == 1 else (n // pad + n_experts) * pad  # the spans, each rounded up to whole tiles, never take more
    _need(order.numel() >= cap, "moe_order: room for the padded ordering")
    if pad > 1:
        _need(tile_group is not None and src_token is not None and src_token.numel() >= cap
              and tile_group.numel() * pad >= cap, "moe_order: tile groups and source tokens for the padded ordering")
    _check(_fn(_libs.get("moe.cu"), "tkb_moe_order")(
        _ptr(top_idx), c_int(n), c_int(n_experts), c_int(top), c_int(pad), _ptr(offsets), _ptr(order), _ptr(place_of),
        _ptr(tile_group), c_int(tile_group.numel() if tile_group is not None else 0), _ptr(src_token),
        c_int(src_token.numel() if src_token is not None else 0), _stream()), "moe_order")


def moe_gather(src: torch.Tensor, src_token: torch.Tensor, out: torch.Tensor) -> None:
    """out[p] = src[src_token[p]], zeros where src_token[p] < 0."""
    _need_cuda(src, src_token, out)
    _need(src.is_contiguous() and out.is_contiguous() and out.dtype == src.dtype and out.shape[1] == src.shape[1]
          and src_token.dtype == torch.int32 and src_token.numel() == out.shape[0], "moe_gather: shapes")
    f = _fn(_libs.get("moe.cu"), f"tkb_moe_gather_{_suffix(src.dtype)}")
    _check(f(_ptr(src), _ptr(src_token), _ptr(out), c_int(out.shape[0]), c_int(src.shape[1]), _stream()), "moe_gather")


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, status: torch.Tensor,
                         gated: bool = False, gelu: bool = False, clamp: tuple[float, float] | None = None) -> torch.Tensor:
    """Row tile i (128 rows) of a[M, K] times the weights w[tile_group[i]] of w [groups, N, K], bfloat16 on the tcgen05
    tensor cores; tiles with tile_group[i] < 0 are left out (their rows of the result are not written).
    ``gated``: every group's rows interleave gate and up (``interleave_gate_up``); the result is [M, N / 2].
    ``gelu`` (ungated): the exact GELU of every result in the epilogue.  ``clamp`` = (limit, alpha), with ``gated``:
    the clamped unit g * sigmoid(alpha g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit), in the SiLU's
    place."""
    _need_cuda(a, w, tile_group, status)
    G, N, K = w.shape
    _need(can_use_tcgen05(a, w.view(G * N, K)) and a.shape[1] == K, "gemm_tcgen05_grouped: bfloat16, K a multiple of 8")
    M = a.shape[0]
    _need(tile_group.dtype == torch.int32 and tile_group.numel() * 128 >= M, "gemm_tcgen05_grouped: a group for every row tile")
    _need(not gated or N % 16 == 0, "gemm_tcgen05_grouped: gated rows come in groups of 16")
    _need(not (gated and gelu), "gemm_tcgen05_grouped: the GELU epilogue is the ungated form's")
    out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=a.device)
    if clamp is not None:
        _need(gated and clamp[0] > 0, "gemm_tcgen05_grouped: the clamped unit is a gated form with a positive limit")
        _check(_fn(_libs.get("gemm_tcgen05.cu"), "tkb_gemm_tcgen05_grouped_clamped_bf16")(
            _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(K), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N), c_int(K),
            c_float(clamp[0]), c_float(clamp[1]), _ptr(tile_group), c_int(G), _ptr(status), _stream()), "gemm_tcgen05_grouped")
        return out
    _check(_fn(_libs.get("gemm_tcgen05.cu"), "tkb_gemm_tcgen05_grouped_bf16")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(K), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N), c_int(K),
        c_int(1 if gated else (2 if gelu else 0)), _ptr(tile_group), c_int(G), _ptr(status), _stream()), "gemm_tcgen05_grouped")
    return out


def moe_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, order: torch.Tensor | None,
             top: int, gated: bool, gelu: bool = False, clamp: tuple[float, float] | None = None) -> None:
    """The experts' products over the ordering.  w [E, N (2N if gated), K]; a [., K]; row p of ``out`` is made from
    row order[p] // top of ``a`` (row p if ``order`` is None) with the weights of the expert whose span holds p.
    gated: out = silu(a w_gate^T) * (a w_up^T) in a's type [places, N]; gelu: out = gelu(a w^T) (exact) in a's type;
    else float32 [places, N].  ``clamp`` = (limit, alpha), with ``gated``: the clamped unit
    g * sigmoid(alpha g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit), in the SiLU's place."""
    _need_cuda(a, w, out, offsets, order)
    _need(clamp is None or (gated and clamp[0] > 0), "moe_gemm: the clamped unit is a gated form with a positive limit")
    E, NN, K = w.shape
    N = NN // 2 if gated else NN
    _need(a.dtype == w.dtype and a.stride(1) == 1 and a.shape[1] == K and w.is_contiguous(), "moe_gemm: operands")
    _need(not (gated and gelu), "moe_gemm: gated or gelu")
    _need(out.shape[1] == N and out.stride(1) == 1 and out.dtype == (a.dtype if (gated or gelu) else torch.float32), "moe_gemm: out")
    if clamp is not None:
        _check(_fn(_libs.get("moe.cu"), f"tkb_moe_gemm_clamped_{_suffix(a.dtype)}")(
            _ptr(a), c_int(a.stride(0)), _ptr(w), _ptr(out), c_int(out.stride(0)), _ptr(offsets), _ptr(order), c_int(top),
            c_int(out.shape[0]), c_int(E), c_int(N), c_int(K), c_float(clamp[0]), c_float(clamp[1]), _stream()), "moe_gemm")
        return
    name = f"tkb_moe_gemm_{'gated_' if gated else ('gelu_' if gelu else '')}{_suffix(a.dtype)}"
    _check(_fn(_libs.get("moe.cu"), name)(_ptr(a), c_int(a.stride(0)), _ptr(w), _ptr(out), c_int(out.stride(0)),
                                          _ptr(offsets), _ptr(order), c_int(top), c_int(out.shape[0]), c_int(E), c_int(N),
                                          c_int(K), _stream()), "moe_gemm")


def moe_combine(y: torch.Tensor, place_of: torch.Tensor, top_w: torch.Tensor, shared: torch.Tensor | None,
                out: torch.Tensor, shared_gate: torch.Tensor | None = None) -> None:
    """out[t] = sum_k top_w[t, k] * y[place_of[t, k]] (+ shared[t]); y float32 [places, H]; shared [T, H] in out's type
    or float32 slices [slices, T, H].  ``shared_gate`` float32 [T]: the shared part counts sigmoid(shared_gate[t])
    times."""
    _need_cuda(y, place_of, top_w, shared, out, shared_gate)
    _need(shared_gate is None or (shared is not None and shared_gate.dtype == torch.float32 and shared_gate.is_contiguous()
                                  and shared_gate.numel() == out.shape[0]), "moe_combine: shared gate float32 [T]")
    T, H = out.shape
    top = top_w.shape[1]
    _need(y.is_contiguous() and y.shape[1] == H and out.is_contiguous(), "moe_combine: y, out")
    _need(y.dtype in (torch.float32, torch.bfloat16), "moe_combine: expert outputs float32 or bfloat16")
    d, sl, n_sl, stride = _split_update(shared, T, H, out.dtype, "moe_combine")
    f = _fn(_libs.get("moe.cu"), f"tkb_moe_combine_y16_{_suffix(out.dtype)}" if y.dtype == torch.bfloat16
            else f"tkb_moe_combine_{_suffix(out.dtype)}")
    _check(f(_ptr(y), _ptr(place_of), _ptr(top_w), _ptr(d), _ptr(sl), c_int(n_sl), ctypes.c_longlong(stride), _ptr(out),
             c_int(T), c_int(H), c_int(top), _ptr(shared_gate), _stream()), "moe_combine")


# ---------------------------------------------------------------------------------------------
# Blocks that norm a sublayer's output; sinusoidal positions; clamped gated unit; gated norm in parts (csrc/post_norm.cu)
def scaled_norm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor | None, mult: float,
                    eps: float, h_out: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
    """x += mult * scale * weight * N(y + bias) in place (x, y float32; N divides a row by its root mean square);
    ``h_out`` (activation type, x's shape) receives the new x.  ``y``: [rows, H], or [slices, rows, H], the slices of
    a split matrix product (``linear_few_rows``), added in slice order."""
    _need_cuda(x, y, weight, scale, h_out, bias)
    rows, H = x.shape
    n_slices = y.shape[0] if y.dim() == 3 else 1
    _need(x.dtype == torch.float32 and x.is_contiguous() and y.dtype == torch.float32 and y.is_contiguous()
          and tuple(y.shape[-2:]) == (rows, H), "scaled_norm_add: x and y contiguous float32 of one shape")
    for v, what in ((weight, "norm weight"), (scale, "scale"), (bias, "bias")):
        _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == H),
              f"scaled_norm_add: {what} float32 [H]")
    _need(weight is not None, "scaled_norm_add: a norm weight")
    _need(h_out is None or (h_out.shape == x.shape and h_out.is_contiguous()), "scaled_norm_add: h_out of x's shape")
    suf = _suffix(h_out.dtype) if h_out is not None else "f32"
    _check(_fn(_libs.get("post_norm.cu"), f"tkb_scaled_norm_add_{suf}")(
        _ptr(x), _ptr(y), c_int(n_slices), ctypes.c_longlong(rows * H), _ptr(bias), _ptr(weight), _ptr(scale), c_float(mult),
        c_float(eps), _ptr(h_out), c_int(rows), c_int(H), _stream()), "scaled_norm_add")


def linear_out_f32(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor | None) -> torch.Tensor:
    """a[M, K] @ w[N, K]^T for a consumer that reads float32 and can add slices (``scaled_norm_add``): with few rows
    and a matrix of up to 32 M values the K-split product's float32 slices [slices, M, N], else whole float32 rows
    [M, N].  (Measured on B200 at 8 rows: 2,048 x 8,192 14.5 us against the library's 23.5 us; 4,096 x 4,096 11 against
    12.5; 4,096 x 14,336 35 against 29, and its eight slices cost the consumer another 9 us.)"""
    if w.numel() <= (32 << 20) and can_use_few_rows(a, w):
        return linear_few_rows(a, w, status)
    return linear(a, w, out_dtype=torch.float32)


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) in out's type."""
    _need_cuda(x, out)
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape, "cast_rows: shapes")
    _check(_fn(_libs.get("post_norm.cu"), f"tkb_cast_rows_{_suffix(out.dtype)}")(
        _ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _stream()), "cast_rows")


def add_sinusoid(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> None:
    """x[t, 2i] += sin(positions[t] * freq[i]), x[t, 2i + 1] += cos(same); x float32, frequencies and angles float64."""
    _need_cuda(x, positions, freq)
    rows, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_sinusoid: x contiguous float32")
    _need(positions.dtype == torch.int32 and positions.numel() >= rows, "add_sinusoid: positions int32 [T]")
    _need(freq.dtype == torch.float64 and freq.is_contiguous() and freq.numel() == (H + 1) // 2, "add_sinusoid: float64 [ceil(H / 2)] frequencies")
    _check(_fn(_libs.get("post_norm.cu"), "tkb_add_sinusoid")(_ptr(x), _ptr(positions), _ptr(freq), c_int(rows), c_int(H),
                                                              _stream()), "add_sinusoid")


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, interleave: int = 0) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit);
    gate_up [rows, 2 * inner] in out's type or float32: [gate | up], or with ``interleave`` 8 columns in groups of 16,
    8 gate columns then the 8 up columns of the same features (``interleave_gate_up``)."""
    _need_cuda(gate_up, out)
    rows, two_i = gate_up.shape
    _need(two_i % 2 == 0 and tuple(out.shape) == (rows, two_i // 2) and gate_up.is_contiguous() and out.is_contiguous(),
          "clamped_glu: shapes")
    _need(gate_up.dtype in (torch.float32, out.dtype), "clamped_glu: gate_up float32 or in out's type")
    name = f"tkb_clamped_glu_{_suffix(gate_up.dtype)}_{_suffix(out.dtype)}"
    _check(_fn(_libs.get("post_norm.cu"), name)(_ptr(gate_up), _ptr(out), c_int(rows), c_int(two_i // 2), c_float(limit),
                                                c_float(alpha), c_int(interleave), _stream()), "clamped_glu")


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor | None, out: torch.Tensor, groups: int,
                     eps: float, gate_first: bool, silu_gate: bool = False) -> None:
    """Rows of float32 values, RMS-normed in ``groups`` equal parts and gated: ``gate_first`` False:
    N(y) * weight * sigmoid(gate) (``silu_gate``: * silu(gate)); True: N(y * silu(gate)) * weight.  ``y`` and ``gate``
    may be column slices of wider float32 tensors.  ``weight``: a value for every column, or a shorter vector that is
    used round and round (one part's weights, shared by all parts), or None."""
    _need_cuda(y, gate, weight, out)
    rows, width = y.shape
    _need(y.dtype == torch.float32 and gate.dtype == torch.float32 and y.stride(1) == 1 and gate.stride(1) == 1
          and gate.shape == y.shape, "gated_group_norm: float32 values and gates of one shape")
    _need(weight is None or (weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() > 0
                             and width % weight.numel() == 0), "gated_group_norm: weight float32, a divisor of the width long")
    _need(out.stride(1) == 1 and out.shape == y.shape and groups > 0 and width % groups == 0, "gated_group_norm: out, groups")
    _need(not (gate_first and silu_gate), "gated_group_norm: the gate first is a SiLU already")
    _check(_fn(_libs.get("post_norm.cu"), f"tkb_gated_group_norm_{_suffix(out.dtype)}")(
        _ptr(y), c_int(y.stride(0)), _ptr(gate), c_int(gate.stride(0)), _ptr(weight),
        c_int(weight.numel() if weight is not None else 0), _ptr(out), c_int(out.stride(0)),
        c_int(rows), c_int(width), c_int(groups), c_float(eps), c_int(1 if gate_first else (2 if silu_gate else 0)),
        _stream()), "gated_group_norm")


def sum_group_norm(x: torch.Tensor, y: torch.Tensor | None, alpha: float, weight: torch.Tensor, eps: float, groups: int,
                   h_out: torch.Tensor | None = None) -> None:
    """x = weight * N_g(alpha * x + y) in place (x float32): the norm after the residual sum, each of the row's
    ``groups`` equal parts divided by its own root mean square.  ``y``: float32 [rows, H], float32 slices
    [slices, rows, H] of a split product (added in slice order), rows in ``h_out``'s type, or None.  ``h_out``
    (activation type, x's shape) receives the new x."""
    _need_cuda(x, y, weight, h_out)
    rows, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "sum_group_norm: x contiguous float32")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == H, "sum_group_norm: weight float32 [H]")
    _need(groups > 0 and H % groups == 0, f"sum_group_norm: {H} values in {groups} parts")
    _need(h_out is None or (h_out.shape == x.shape and h_out.is_contiguous()), "sum_group_norm: h_out of x's shape")
    y32 = y16 = None
    n_slices = 0
    if y is not None:
        _need(y.is_contiguous() and tuple(y.shape[-2:]) == (rows, H), "sum_group_norm: y of x's shape")
        if y.dtype == torch.float32:
            y32, n_slices = y, (y.shape[0] if y.dim() == 3 else 1)
        else:
            _need(h_out is not None and y.dtype == h_out.dtype and y.dim() == 2, "sum_group_norm: y float32 or in the activation type")
            y16 = y
    suf = _suffix(h_out.dtype) if h_out is not None else "f32"
    _check(_fn(_libs.get("post_norm.cu"), f"tkb_sum_group_norm_{suf}")(
        _ptr(x), _ptr(y32), c_int(n_slices), ctypes.c_longlong(rows * H), _ptr(y16), c_float(alpha), _ptr(weight),
        c_float(eps), _ptr(h_out), c_int(rows), c_int(H), c_int(groups), _stream()), "sum_group_norm")


def gelu_gate_rows(z: torch.Tensor, table: torch.Tensor, off: int, ids: torch.Tensor, token_seq: torch.Tensor,
                   seq_slot: torch.Tensor, last_token: torch.Tensor, rows: torch.Tensor | None, out: torch.Tensor,
                   status: torch.Tensor) -> None:
    """out[r, j] = gelu_tanh(z[r, j]) * table[token(r), off + j]: z float32 [R, dim]; row r belongs to token rows[r] (r
    if ``rows`` is None), whose id is found as the embedding finds it (an id < 0: the request's last sampled token)."""
    _need_cuda(z, table, ids, token_seq, seq_slot, last_token, rows, out, status)
    R, dim = z.shape
    _need(z.dtype == torch.float32 and z.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (R, dim)
          and out.dtype == table.dtype and table.is_contiguous() and off >= 0 and off + dim <= table.shape[1], "gelu_gate_rows: shapes")
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() == R), "gelu_gate_rows: rows int32 [R]")
    _check(_fn(_libs.get("post_norm.cu"), f"tkb_gelu_gate_rows_{_suffix(out.dtype)}")(
        _ptr(z), _ptr(table), c_int(table.shape[1]), c_int(off), c_int(dim), c_int(table.shape[0]), _ptr(ids),
        _ptr(token_seq), _ptr(seq_slot), _ptr(last_token), _ptr(rows), _ptr(out), c_int(R), _ptr(status), _stream()),
        "gelu_gate_rows")


# ---------------------------------------------------------------------------------------------
# The recurrence with one decay a head and token (csrc/decay_recurrence.cu)
def decay_recurrence_defines(dim: int, vdim: int, lanes: int | None = None) -> dict:
    """The compile-time constants of the walk for heads of ``dim`` x ``vdim``: how many threads share a column of the
    state (``lanes``: 8, 16 or 32, at most as many as the head has 16-byte pieces; None: 8) and how many values each
    holds."""
    _need(0 < dim <= 1024 and 0 < vdim, f"decay recurrence: key sizes up to 1024, not {dim}")
    pieces = (dim + 3) // 4
    lanes = min(lanes or 8, 8 if pieces <= 8 else (16 if pieces <= 16 else 32))
    _need(lanes in (8, 16, 32), "decay recurrence: 8, 16 or 32 threads a column")
    return dict(TKB_DR_LANES=lanes, TKB_DR_DPT=4 * ((pieces + lanes - 1) // lanes))


def decay_walk_modules(dim: int, vdim: int) -> list[dict]:
    """Every build of the walk that ``decay_walk`` may choose for heads of this size."""
    out = []
    for lanes in (8, 16, 32):
        d = decay_recurrence_defines(dim, vdim, lanes)
        if d not in out:
            out.append(d)
    return out


def _walk_defines(dim: int, vdim: int, columns: int, single: bool, device) -> dict:
    """Which build walks ``columns`` state columns (requests x heads x vdim).  Single tokens: 8 threads a column, each
    with several 16-byte loads of the state in flight (the time is the state's trip through memory).  Portions: the
    walk over the tokens is a chain, a warp alone issues an instruction every four cycles, so the columns are spread
    over warps until there are about seven an SM (measured on B200 at heads of 128 x 128 and 64 x 128, 2,048 tokens:
    1,024 warps beat 512 and 2,048 at 16, 32 and 64 heads alike), by giving a column more threads with fewer values."""
    if single:
        return decay_recurrence_defines(dim, vdim, 8)
    from tokasaurus_b200.kernels.device import device_limits

    want = 6 * device_limits(device).sm_count
    chosen = None
    for d in decay_walk_modules(dim, vdim):
        chosen = d
        if columns * d["TKB_DR_LANES"] // 32 >= want:
            break
    return chosen


def ssm_prep(proj: torch.Tensor, xbc_off: int, channels: int, conv_w: torch.Tensor, conv_b: torch.Tensor | None,
             state: torch.Tensor, carry_off: int, token_seq: torch.Tensor, seq_slot: torch.Tensor,
             seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, n_seqs: int, xbc: torch.Tensor, dt_off: int,
             heads: int, dt_bias: torch.Tensor, a_log: torch.Tensor, dt_dec: torch.Tensor, defines: dict,
             write_state: bool = True) -> None:
    """From float32 projections [T, .]: xbc = silu(bias + causal convolution over time) of the ``channels`` columns at
    ``xbc_off`` (inputs from before the step out of state[slot, carry_off:] = [taps - 1, channels], brought forward
    afterwards), dt = softplus(proj[:, dt_off + h] + dt_bias[h]) and the decay exp(-exp(a_log[h]) * dt) into
    dt_dec [T, 2 * heads]."""
    _need_cuda(proj, conv_w, conv_b, state, token_seq, seq_slot, seq_q_start, seq_q_len, xbc, dt_bias, a_log, dt_dec)
    T = proj.shape[0]
    taps = conv_w.shape[1]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= max(xbc_off + channels, dt_off + heads),
          "ssm_prep: float32 projections")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == channels, "ssm_prep: taps float32 [channels, taps]")
    _need(conv_b is None or (conv_b.dtype == torch.float32 and conv_b.numel() == channels), "ssm_prep: bias float32 [channels]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
          and state.shape[1] >= carry_off + (taps - 1) * channels, "ssm_prep: state float32 [slots, n]")
    _need(xbc.dtype == torch.float32 and xbc.is_contiguous() and tuple(xbc.shape) == (T, channels), "ssm_prep: xbc float32 [T, channels]")
    _need(dt_dec.dtype == torch.float32 and dt_dec.is_contiguous() and tuple(dt_dec.shape) == (T, 2 * heads), "ssm_prep: dt_dec [T, 2 heads]")
    for v in (dt_bias, a_log):
        _need(v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads, "ssm_prep: float32 [heads] vectors")
    _check(_fn(_libs.get("decay_recurrence.cu", **defines), "tkb_ssm_prep")(
        _ptr(proj), c_int(proj.stride(0)), c_int(xbc_off), c_int(channels), c_int(taps), _ptr(conv_w), _ptr(conv_b),
        _ptr(state), ctypes.c_longlong(state.stride(0)), ctypes.c_longlong(carry_off), _ptr(token_seq), _ptr(seq_slot),
        _ptr(seq_q_start), _ptr(seq_q_len), c_int(T), c_int(n_seqs), _ptr(xbc), c_int(dt_off), c_int(heads),
        _ptr(dt_bias), _ptr(a_log), _ptr(dt_dec), c_int(1 if write_state else 0), _stream()), "ssm_prep")


def decay_walk(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads_per_qk: int, dt_dec: torch.Tensor | None,
               decay_head: torch.Tensor | None, skip: torch.Tensor | None, state: torch.Tensor, out: torch.Tensor,
               seq_slot: torch.Tensor, seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, n_seqs: int, heads: int,
               dim: int, vdim: int, write_state: bool = True, decay_vec: torch.Tensor | None = None) -> None:
    """S_t = a_t S_(t-1) + (c_t k_t) v_t^T, o_t = S_t^T q_t + skip * v_t over each request's tokens.  q, k [T, . * dim]
    and v [T, heads * vdim] are float32 (column slices allowed); head h reads q and k number h // heads_per_qk.
    ``dt_dec`` [T, 2 heads] = (c, a) per token, or ``decay_head`` [heads] with
    c = 1, or ``decay_vec`` float32 [T, heads * dim] (a column slice allowed): a decay for every key channel,
    S_t = diag(f_t) S_(t-1) + k_t v_t^T.  state float32 [slots, n], S^T of the heads first: [heads, vdim, dim]; out
    float32 [T, heads * vdim]."""
    _need_cuda(q, k, v, dt_dec, decay_head, skip, state, out, seq_slot, seq_q_start, seq_q_len, decay_vec)
    T = q.shape[0]
    for t in (q, k, v):
        _need(t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == T, "decay_walk: float32 rows")
    _need(heads_per_qk > 0 and heads % heads_per_qk == 0 and q.shape[1] == (heads // heads_per_qk) * dim
          and k.shape[1] == q.shape[1] and v.shape[1] == heads * vdim, "decay_walk: shapes of q, k, v")
    _need((dt_dec is not None) + (decay_head is not None) + (decay_vec is not None) == 1,
          "decay_walk: decays per token, per head or per key channel")
    _need(decay_vec is None or (decay_vec.dtype == torch.float32 and decay_vec.stride(1) == 1 and heads_per_qk == 1
                                and tuple(decay_vec.shape) == (T, heads * dim)), "decay_walk: decay_vec float32 [T, heads * dim]")
    _need(dt_dec is None or (dt_dec.dtype == torch.float32 and dt_dec.is_contiguous() and tuple(dt_dec.shape) == (T, 2 * heads)),
          "decay_walk: dt_dec float32 [T, 2 heads]")
    for t in (decay_head, skip):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads), "decay_walk: float32 [heads]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] >= heads * vdim * dim,
          "decay_walk: state float32 [slots, n]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (T, heads * vdim), "decay_walk: out float32 [T, heads * vdim]")
    defines = _walk_defines(dim, vdim, n_seqs * heads * vdim, T == n_seqs, q.device)
    _check(_fn(_libs.get("decay_recurrence.cu", **defines), "tkb_decay_walk")(
        _ptr(q), c_int(q.stride(0)), _ptr(k), c_int(k.stride(0)), c_int(heads_per_qk), _ptr(decay_vec),
        c_int(decay_vec.stride(0) if decay_vec is not None else 0), _ptr(v), c_int(v.stride(0)),
        _ptr(dt_dec), _ptr(decay_head), _ptr(skip), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(out),
        _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), c_int(n_seqs), c_int(T), c_int(heads), c_int(dim), c_int(vdim),
        c_int(1 if write_state else 0), _stream()), "decay_walk")


def gla_gates(proj: torch.Tensor, low_off: int, rank: int, a2t: torch.Tensor, bias: torch.Tensor | None, tau: float,
              f_out: torch.Tensor, q_off: int, q_cols: int, q_scale: float, defines: dict) -> None:
    """Decays of gated linear attention from float32 projections [T, .]: f = sigmoid(low @ a2t + bias)^(1 / tau) with
    low = proj[:, low_off : low_off + rank] and a2t float32 [rank, C]; f_out float32 [T, C].  Also scales the ``q_cols``
    columns at ``q_off`` by ``q_scale``, in place."""
    _need_cuda(proj, a2t, bias, f_out)
    T = proj.shape[0]
    C = a2t.shape[1]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= max(low_off + rank, q_off + q_cols),
          "gla_gates: float32 projections")
    _need(a2t.dtype == torch.float32 and a2t.is_contiguous() and a2t.shape[0] == rank, "gla_gates: a2t float32 [rank, C]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C), "gla_gates: bias float32 [C]")
    _need(f_out.dtype == torch.float32 and f_out.is_contiguous() and tuple(f_out.shape) == (T, C) and tau > 0, "gla_gates: f_out, tau")
    _check(_fn(_libs.get("decay_recurrence.cu", **defines), "tkb_gla_gates")(
        _ptr(proj), c_int(proj.stride(0)), c_int(low_off), c_int(rank), _ptr(a2t), _ptr(bias), c_float(1.0 / tau), c_int(C),
        _ptr(f_out), c_int(q_off), c_int(q_cols), c_float(q_scale), c_int(T), _stream()), "gla_gates")


def rotate_scale(proj: torch.Tensor, q_off: int, k_off: int, heads: int, dim: int, rot_dims: int, pairs: bool,
                 freq: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor, q_scale: float, k_scale: float,
                 defines: dict) -> None:
    """Rotation by position of the ``heads`` q heads (at column ``q_off``) and k heads (at ``k_off``) of float32 rows,
    in place, on the first ``rot_dims`` channels of a head (``pairs``: channel 2i with 2i + 1, else i with
    i + rot_dims / 2; freq float64 [rot_dims / 2]), then q * q_scale and k * k_scale."""
    _need_cuda(proj, freq, positions, token_seq)
    T = proj.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= max(q_off, k_off) + heads * dim,
          "rotate_scale: float32 projections")
    _need(0 <= rot_dims <= dim and rot_dims % 2 == 0 and freq.dtype == torch.float64 and freq.is_contiguous()
          and freq.numel() == rot_dims // 2, "rotate_scale: float64 [rot_dims / 2] frequencies")
    _need(positions.dtype == torch.int32 and positions.numel() >= T and token_seq.numel() >= T, "rotate_scale: positions")
    _check(_fn(_libs.get("decay_recurrence.cu", **defines), "tkb_rotate_scale")(
        _ptr(proj), c_int(proj.stride(0)), c_int(q_off), c_int(k_off), c_int(heads), c_int(dim), c_int(rot_dims),
        c_int(1 if pairs else 0), _ptr(freq), _ptr(positions), _ptr(token_seq), c_float(q_scale), c_float(k_scale),
        c_int(T), _stream()), "rotate_scale")


def silu_cols(x: torch.Tensor, ncols: int, defines: dict) -> None:
    """SiLU in place on the first ``ncols`` columns of float32 rows."""
    _need_cuda(x)
    _need(x.dtype == torch.float32 and x.stride(1) == 1 and 0 <= ncols <= x.shape[1], "silu_cols: float32 rows")
    _check(_fn(_libs.get("decay_recurrence.cu", **defines), "tkb_silu_cols")(
        _ptr(x), c_int(x.stride(0)), c_int(ncols), c_int(x.shape[0]), _stream()), "silu_cols")


# ---------------------------------------------------------------------------------------------
# Attention with a score cap and a sink, keys and values of different sizes (csrc/attention_sink.cu)
def sink_attention_defines(dim: int, vdim: int, sigmoid: bool = False, maps: int = 1) -> dict:
    """``sigmoid``: the build whose weights are sigmoid(score), not a softmax.  ``maps``: attention maps a head (each
    with query and key vectors of its own, over the same values)."""
    _need(0 < dim <= 512 and 0 < vdim <= 512, f"sink attention: head sizes up to 512, not {dim} / {vdim}")
    _need(1 <= maps <= 4, f"sink attention: one to four maps a head, not {maps}")
    d = dict(TKB_QK=dim, TKB_VD=vdim)
    if sigmoid:
        d["TKB_SIGMOID"] = 1
    if maps > 1:
        d["TKB_MAPS"] = maps
    return d


def sink_attn_prep(qkv: torch.Tensor, bias: torch.Tensor | None, unit_norm: bool, eps: float, q_out: torch.Tensor,
                   cache: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor, page_indptr: torch.Tensor,
                   page_ids: torch.Tensor, n_heads: int, n_kv_heads: int, dim: int, vdim: int, page_size: int,
                   write_cache: bool, status: torch.Tensor, norm_w: torch.Tensor | None = None,
                   rot_freq: torch.Tensor | None = None, rot_dims: int = 0, rot_pairs: bool = False,
                   values_are_keys: bool = False, sigmoid: bool = False, maps: int = 1) -> None:
    """qkv float32 [T, heads*maps*dim | kv heads*maps*dim | kv heads*vdim | anything else] -> (+ bias, q and k vectors
    divided by their root mean square) q_out [T, heads*maps*dim] and the tokens' [k of every map | v] rows in cache
    [pages, kv heads, page_size, maps*dim + vdim].
    ``norm_w`` float32 [2, dim]: weights of the q heads' and the k heads' norm.  ``rot_freq`` float64 [rot_dims / 2]:
    q and k are rotated by position on their first ``rot_dims`` channels (``rot_pairs``: channel 2i with 2i + 1, else
    i with i + rot_dims / 2).  ``values_are_keys``: the projections hold no v; a token's value is its key as projected
    (before norm and rotation).  ``sigmoid``: the kernel build of the sigmoid form."""
    _need_cuda(qkv, bias, q_out, cache, positions, token_seq, page_indptr, page_ids, status, norm_w, rot_freq)
    T = qkv.shape[0]
    C = (n_heads + n_kv_heads) * maps * dim + (0 if values_are_keys else n_kv_heads * vdim)
    _need(not values_are_keys or (dim == vdim and maps == 1), "sink_attn_prep: values that are the keys have the keys' size")
    _need(norm_w is None or (norm_w.dtype == torch.float32 and norm_w.is_contiguous() and tuple(norm_w.shape) == (2, dim)),
          "sink_attn_prep: norm weights float32 [2, dim]")
    _need(rot_freq is None or (rot_freq.dtype == torch.float64 and rot_freq.is_contiguous() and rot_dims % 2 == 0
                               and 0 < rot_dims <= dim and rot_freq.numel() == rot_dims // 2),
          "sink_attn_prep: float64 [rot_dims / 2] frequencies")
    _need(qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] >= C, "sink_attn_prep: float32 projections")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C), "sink_attn_prep: bias float32")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, n_heads * maps * dim) and q_out.dtype == cache.dtype, "sink_attn_prep: q_out")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (n_kv_heads, page_size, maps * dim + vdim), "sink_attn_prep: cache rows")
    _check(_fn(_libs.get("attention_sink.cu", **sink_attention_defines(dim, vdim, sigmoid, maps)), f"tkb_sink_attn_prep_{_suffix(cache.dtype)}")(
        _ptr(qkv), c_int(qkv.stride(0)), _ptr(bias), c_int(1 if unit_norm else 0), c_float(eps), _ptr(q_out), _ptr(cache),
        _ptr(positions), _ptr(token_seq), _ptr(page_indptr), _ptr(page_ids), c_int(T), c_int(n_heads), c_int(n_kv_heads),
        c_int(page_size), c_int(cache.shape[0]), c_int(1 if write_cache else 0), _ptr(status), _ptr(norm_w), _ptr(rot_freq),
        c_int(rot_dims if rot_freq is not None else 0), c_int(1 if rot_pairs else 0), c_int(1 if values_are_keys else 0),
        _stream()), "sink_attn_prep")


def _head_vectors(n_heads: int, what: str, *vectors):
    for v in vectors:
        _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n_heads), f"{what}: float32 [heads] vectors")


def _sink_out_ok(out: torch.Tensor, rows: int, n_heads: int, vdim: int, maps: int, act: torch.dtype) -> bool:
    """One map: [rows, heads * vdim] in the activation type.  Several: float32 [rows, heads * maps * vdim], the maps'
    outputs side by side, unrounded."""
    return (out.is_contiguous() and tuple(out.shape) == (rows, n_heads * maps * vdim)
            and out.dtype == (act if maps == 1 else torch.float32))


def attn_sink(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
              page_indptr: torch.Tensor, page_ids: torch.Tensor, rows: torch.Tensor | None, n_rows: int,
              sinks: torch.Tensor | None, n_heads: int, n_kv_heads: int, dim: int, vdim: int, page_size: int,
              scale: float, softcap: float | None, window: int | None, status: torch.Tensor,
              head_scale: torch.Tensor | None = None, head_bias: torch.Tensor | None = None, sigmoid: bool = False,
              maps: int = 1, keep_first: int = 0) -> None:
    """Attention of ``n_rows`` tokens (``rows`` names them; None: all) over their requests' cached [k | v] rows.
    ``head_scale`` / ``head_bias`` float32 [heads]: a factor on a head's scale, a number added to its scores.
    ``sigmoid``: weights sigmoid(score) instead of a softmax (no sink).  ``maps`` > 1: so many attention maps a head,
    each a softmax of its own; ``out`` then is float32 [rows, heads * maps * vdim].  ``keep_first``: with a window, the
    request's first so many positions stay visible."""
    _need_cuda(q, out, cache, token_seq, positions, page_indptr, page_ids, rows, sinks, status, head_scale, head_bias)
    _head_vectors(n_heads * maps, "attn_sink", head_scale, head_bias)
    _need(not (sigmoid and sinks is not None), "attn_sink: the sigmoid form has no sink")
    _need(q.is_contiguous() and q.shape[1] == n_heads * maps * dim and q.dtype == cache.dtype
          and _sink_out_ok(out, n_rows, n_heads, vdim, maps, cache.dtype), "attn_sink: q and out")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (n_kv_heads, page_size, maps * dim + vdim), "attn_sink: cache rows")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads * maps), "attn_sink: sinks float32 [heads]")
    _check(_fn(_libs.get("attention_sink.cu", **sink_attention_defines(dim, vdim, sigmoid, maps)), f"tkb_attn_sink_simt_{_suffix(cache.dtype)}")(
        _ptr(q), _ptr(out), _ptr(cache), _ptr(token_seq), _ptr(positions), _ptr(page_indptr), _ptr(page_ids), _ptr(rows),
        c_int(n_rows), _ptr(sinks), c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale),
        c_float(softcap or 0.0), c_int(window or 0), c_int(keep_first if window else 0), c_int(cache.shape[0]),
        _ptr(status), _ptr(head_scale), _ptr(head_bias), _stream()), "attn_sink")


def can_use_attn_sink_tc(dtype: torch.dtype, dim: int, vdim: int, maps: int = 1) -> bool:
    """The tensor-core kernels of csrc/attention_sink.cu take bfloat16 rows whose key and value sizes are multiples of 16
    up to 256, with one, two or four maps a head (a block's four warps are shared out among the maps)."""
    return dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and dim <= 256 and vdim <= 256 and maps in (1, 2, 4)


def attn_sink_tc(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, seq_q_start: torch.Tensor, seq_q_len: torch.Tensor,
                 seq_kv_len: torch.Tensor, page_indptr: torch.Tensor, page_ids: torch.Tensor, n_seqs: int,
                 sinks: torch.Tensor | None, n_heads: int, n_kv_heads: int, dim: int, vdim: int, page_size: int, scale: float,
                 softcap: float | None, window: int | None, status: torch.Tensor, portions: bool = True,
                 singles: bool = True, head_scale: torch.Tensor | None = None, head_bias: torch.Tensor | None = None,
                 sigmoid: bool = False, maps: int = 1, keep_first: int = 0) -> None:
    """Attention of every token of the step on the tensor cores (bfloat16): out [T, heads * vdim] (``maps`` > 1: float32
    [T, heads * maps * vdim]).  ``portions`` / ``singles``: whether the step can hold requests with several tokens /
    with one (a kernel each).  ``keep_first``: as in ``attn_sink``."""
    _need_cuda(q, out, cache, seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, sinks, status, head_scale, head_bias)
    _head_vectors(n_heads * maps, "attn_sink_tc", head_scale, head_bias)
    _need(not (sigmoid and sinks is not None), "attn_sink_tc: the sigmoid form has no sink")
    T = q.shape[0]
    _need(can_use_attn_sink_tc(cache.dtype, dim, vdim, maps), "attn_sink_tc: bfloat16 rows, key and value sizes multiples of 16")
    _need(q.is_contiguous() and q.shape[1] == n_heads * maps * dim and q.dtype == cache.dtype
          and _sink_out_ok(out, T, n_heads, vdim, maps, cache.dtype), "attn_sink_tc: q and out")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (n_kv_heads, page_size, maps * dim + vdim), "attn_sink_tc: cache rows")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads * maps), "attn_sink_tc: sinks float32 [heads]")
    # single tokens: with few requests a request's 64-key tiles are shared out among blocks until the SMs are covered
    # twice (a function of the step's shape only: the same step replays from a graph)
    splits, part = 1, None
    if singles:
        from tokasaurus_b200.kernels.device import device_limits

        blocks = n_seqs * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16)  # (a block serves every map of its heads)
        splits = max(1, min(8, (2 * device_limits(q.device).sm_count) // max(1, blocks)))
        if window:
            splits = min(splits, max(1, (window + 63) // 64))
        if splits > 1:
            part = torch.empty((n_seqs * n_heads * maps * splits * (vdim + 2),), dtype=torch.float32, device=q.device)
    _check(_fn(_libs.get("attention_sink.cu", **sink_attention_defines(dim, vdim, sigmoid, maps)), "tkb_attn_sink_tc_bf16")(
        _ptr(q), _ptr(out), _ptr(cache), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(page_indptr),
        _ptr(page_ids), c_int(T), c_int(n_seqs), c_int(1 if portions else 0), c_int(1 if singles else 0), _ptr(sinks),
        c_int(n_heads), c_int(n_kv_heads), c_int(page_size), c_float(scale), c_float(softcap or 0.0), c_int(window or 0),
        c_int(keep_first if window else 0), c_int(cache.shape[0]), _ptr(status), _ptr(part), c_int(splits), _ptr(head_scale),
        _ptr(head_bias), _stream()), "attn_sink_tc")


def diff_combine(a: torch.Tensor, lam: torch.Tensor, eps: float, mult: float, gate: torch.Tensor | None, gate_off: int,
                 rows: torch.Tensor | None, out: torch.Tensor, n_heads: int, dim: int, vdim: int) -> None:
    """The differential form's combination of two attention maps: a float32 [n_rows, heads * 2 * vdim] ->
    out [n_rows, heads * vdim] = N(a_0 - lam * a_1) * mult * sigmoid(gate[token, gate_off + head]), N the division of a
    head's vdim values by their root mean square (float32, ``eps``).  ``lam`` float32 [1] on the device; ``gate``
    float32 [T, .] or None; ``rows`` int32 names the tokens of a's rows (None: row r is token r)."""
    _need_cuda(a, lam, gate, rows, out)
    n_rows = a.shape[0]
    _need(a.dtype == torch.float32 and a.is_contiguous() and a.shape[1] == n_heads * 2 * vdim
          and out.is_contiguous() and tuple(out.shape) == (n_rows, n_heads * vdim), "diff_combine: a and out")
    _need(lam.dtype == torch.float32 and lam.numel() == 1, "diff_combine: lambda float32 [1]")
    _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate_off + n_heads <= gate.shape[1]),
          "diff_combine: float32 gate logits")
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() == n_rows), "diff_combine: rows")
    f = _fn(_libs.get("attention_sink.cu", **sink_attention_defines(dim, vdim, False, 2)), f"tkb_diff_combine_{_suffix(out.dtype)}")
    _check(f(_ptr(a), _ptr(lam), c_float(eps), c_float(mult), _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
             c_int(gate_off), _ptr(rows), _ptr(out), c_int(n_rows), c_int(n_heads), _stream()), "diff_combine")


def prepare_modules(modules) -> None:
    """Build and load the listed (source file, constants) modules."""
    for source, defines in modules:
        _libs.get(source, **(defines or {}))
