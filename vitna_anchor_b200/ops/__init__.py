"""Python faces of the engine's CUDA kernels.

The kernels live in one shared library (csrc/, built by ops.build) with a C
interface; this module checks tensors (device, dtype, contiguity, shapes) and
passes raw pointers and the current CUDA stream.  There is no CPU fallback and
no library stand-in: if the library cannot be built or loaded, or a tensor is
not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib = None

class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded kernel library; built at the first call if need be."""
    global _lib
    if _lib is None:
        # VITNA_KERNEL_LIB names a library that was built elsewhere from these sources (a read-only installation, a build
        # with other compiler flags); otherwise the in-tree library, compiled now if it is missing or out of date
        path = os.environ.get("VITNA_KERNEL_LIB") or _build.library_path(build=True)
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the kernel library {path} could not be loaded: {e}") from None
    return _lib


_launches = 0

# The 32-bit path has two routings.  Exact (the default): every operation has ONE kernel, whatever the batch (the
# tile product, the row-wise norm, attention_rows), and each of them sums an output's terms in an order that
# depends on that output alone, so the logits of a position are the same BITS however the tokens are cut into
# steps, whatever else is in the batch and wherever the pages lie.  Fast (VITNA_FLOAT32_FAST=1 in the environment,
# or set_float32_exact(False)): the float32 twins of the serving kernels (few-rows products with fused norm,
# rotation and SwiGLU, split-key decode attention) are chosen by batch size as in bfloat16; the result then
# differs between ways of cutting by float32 rounding.
_float32_exact = os.environ.get("VITNA_FLOAT32_FAST", "") in ("", "0")


def set_float32_exact(exact: bool) -> bool:
    """Choose the routing of the 32-bit path (see above); returns the setting that was in force."""
    global _float32_exact
    before, _float32_exact = _float32_exact, bool(exact)
    return before


def float32_exact() -> bool:
    return _float32_exact


def launch_count() -> int:
    """Kernels of this library launched so far by this process (a graph replay counts the kernels it holds)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    fn = lib().vk_error_string
    fn.restype = ctypes.c_char_p
    text = fn(status).decode()
    if status < 0:
        raise KernelError(f"{what}: refused, {text}")
    raise KernelError(f"{what}: CUDA error {status}: {text}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not one of float32, bfloat16")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _req(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device; the engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, expected {dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# ---------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :]); table [V, H] (float32 or bfloat16), ids int32 [T], out float32 [T, H]."""
    _req(table, "table", dims=2); _req(ids, "ids", torch.int32, 1); _req(out, "out", torch.float32, 2)
    if out.shape != (ids.shape[0], table.shape[1]):
        raise KernelError("embed_rows: out is not [tokens, hidden]")
    _check(lib().vk_embed_rows(_p(table), _p(ids), _p(out), ids.shape[0], table.shape[1], table.shape[0], _dt(table),
                               _stream()), "embed_rows")
    return out


def rmsnorm_rows(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r, :] = rmsnorm(x[rows[r], :]) * w; x float32 [T, n], w float32 [n], out [R, n] float32 or bfloat16."""
    _req(x, "x", torch.float32, 2); _req(w, "w", torch.float32, 1); _req(out, "out", dims=2)
    n = x.shape[1]
    if w.shape[0] != n or out.shape[1] != n:
        raise KernelError("rmsnorm_rows: widths differ")
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        if rows.shape[0] != out.shape[0]:
            raise KernelError("rmsnorm_rows: rows and out differ in length")
    elif out.shape[0] != x.shape[0]:
        raise KernelError("rmsnorm_rows: out and x differ in rows")
    _check(lib().vk_rmsnorm_rows(_p(x), _p(w), _p(rows), _p(out), out.shape[0], n, ctypes.c_float(eps), _dt(out),
                                 _stream()), "rmsnorm_rows")
    return out


LINEAR_SAME, LINEAR_F32, LINEAR_ACC_F32 = 0, 1, 2


def linear_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, few_rows: int = 8) -> torch.Tensor:
    """out = x @ w.T on CUDA cores in float32 arithmetic.  x [M, K] (rows may be strided), w [N, K],
    out [M, N]: mode 0 stores in x's dtype, 1 stores float32, 2 adds into a float32 out."""
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("linear: x must be a CUDA matrix with unit column stride")
    _req(w, "w", x.dtype, 2); _req(out, "out", x.dtype if mode == LINEAR_SAME else torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    ldx = x.stride(0) if M > 1 else max(K, x.stride(0))
    _check(lib().vk_linear_simt(_p(x), _p(w), _p(out), M, N, K, ldx, _dt(x), mode, few_rows, _stream()), "linear_simt")
    return out


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               slot_mapping: Optional[torch.Tensor], q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
               nh: int, nkv: int, hd: int, rot: int, page_size: int) -> torch.Tensor:
    """Rotate q and k (half-split pairs within the first `rot` dimensions), write q to q_out and k, v into
    the layer's pages at slot_mapping (page * page_size + offset, or -1 for no write)."""
    _req(qkv, "qkv", dims=2); _req(positions, "positions", torch.int32, 1); _req(q_out, "q_out", qkv.dtype, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd or q_out.shape != (T, nh * hd) or positions.shape[0] != T:
        raise KernelError("rope_store: shapes do not fit the head counts")
    if rot > 0:
        _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError("rope_store: tables are not [positions, rot/2]")
    if cache_layer is not None:
        _req(cache_layer, "cache_layer", qkv.dtype)
        _req(slot_mapping, "slot_mapping", torch.int32, 1)
        if tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd) or slot_mapping.shape[0] != T:
            raise KernelError("rope_store: the cache layer is not [pages, 2, nkv, page_size, hd]")
    _check(lib().vk_rope_store(_p(qkv), _p(positions), _p(cos if rot > 0 else None), _p(sin if rot > 0 else None),
                               _p(slot_mapping if cache_layer is not None else None), _p(q_out), _p(cache_layer), T, nh,
                               nkv, hd, rot, page_size, _dt(qkv), _stream()), "rope_store")
    return q_out


def attention_rows(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor,
                   positions: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float,
                   window: int = 0, tok_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token (or of those in tok_list) over its request's pages (any sizes,
    float32 arithmetic)."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype, 5); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    if q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd):
        raise KernelError("attention_rows: shapes do not fit the head counts")
    if token_seg.shape[0] != T or positions.shape[0] != T:
        raise KernelError("attention_rows: per-token arrays differ in length")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    _check(lib().vk_attention_rows(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list), _p(out),
                                   n, nh, nkv, hd, page_size, block_tables.shape[1], ctypes.c_float(scale), window, _dt(q),
                                   _stream()), "attention_rows")
    return out


def attention_decode_scratch_bytes(tokens: int, nh: int, nkv: int, hd: int, max_context: int) -> int:
    fn = lib().vk_attention_decode_scratch_bytes
    fn.restype = ctypes.c_size_t
    return int(fn(tokens, nh, nkv, hd, max_context))


def attention_decode_takes(dtype: torch.dtype, hd: int, max_context: int = 0) -> bool:
    """Whether the split-key decode kernel takes this head size and context (else attention_rows does the work)."""
    vec = 4 if dtype == torch.float32 else 8
    return hd % vec == 0 and hd <= 256 and hd // vec <= 32 and max_context <= 128 * 256


def attention_decode(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, scratch_tokens: int, nh: int, nkv: int,
                     hd: int, scale: float, max_context: int, grid_context: int, window: int = 0,
                     tok_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of single decoded tokens, split over the keys in runs of 256 absolute positions.
    scratch: a byte buffer of attention_decode_scratch_bytes(scratch_tokens, ...) that was zero at first use
    and is used by no other shape; max_context fixes its layout, grid_context (<= max_context) bounds the
    positions of this launch."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype, 5); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    _req(scratch, "scratch", torch.uint8, 1)
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    if q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd):
        raise KernelError("attention_decode: shapes do not fit the head counts")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    if scratch.numel() < attention_decode_scratch_bytes(scratch_tokens, nh, nkv, hd, max_context):
        raise KernelError("attention_decode: the scratch is too small")
    _check(lib().vk_attention_decode(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list),
                                     _p(out), _p(scratch), scratch_tokens, n, nh, nkv, hd, page_size, cache_layer.shape[0],
                                     block_tables.shape[1], max_context, grid_context, ctypes.c_float(scale), window, _dt(q),
                                     _p(error_word()), _stream()),
           "attention_decode")
    return out


def set_decode_tma(mode: int) -> int:
    """Which decode-attention launches the persistent TMA kernel takes: 0 none, 1 all whose sizes it takes, 2 those its
    size rule gives it (the default).  Returns the mode that was in force."""
    return int(lib().vk_set_decode_tma(int(mode)))


def set_decode_tma_few(mode: int) -> int:
    """Whether the persistent TMA decode attention takes head groups of at most eight with the keys as the rows of its
    products (1, the default; VITNA_DECODE_TMA_FEW=0 sets the other at start) or with the heads as rows (0), as it takes
    larger groups.  Returns what was in force."""
    return int(lib().vk_set_decode_tma_few(int(mode)))


def set_skinny_stream(mode: int) -> int:
    """Which few-rows products the streaming tensor-core kernel takes: 0 none, 1 all whose sizes it takes, 2 those its
    size rule gives it (the default; VITNA_SKINNY_STREAM sets the initial mode).  Returns the mode that was in force."""
    return int(lib().vk_set_skinny_stream(int(mode)))


def silu_mul(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gu[:, :I]) * gu[:, I:]."""
    _req(gu, "gu", dims=2); _req(out, "out", gu.dtype, 2)
    T, two_i = gu.shape
    if two_i % 2 or out.shape != (T, two_i // 2):
        raise KernelError("silu_mul: out is not [tokens, width/2]")
    _check(lib().vk_silu_mul(_p(gu), _p(out), T, two_i // 2, _dt(gu), _stream()), "silu_mul")
    return out


def add_inplace(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """y (float32) += x (float32 or bfloat16)."""
    _req(y, "y", torch.float32); _req(x, "x")
    if y.numel() != x.numel():
        raise KernelError("add_inplace: sizes differ")
    _check(lib().vk_add_inplace(_p(y), _p(x), ctypes.c_size_t(y.numel()), _dt(x), _stream()), "add_inplace")
    return y


def take_tokens(tokens: torch.Tensor, ids: torch.Tensor, src: torch.Tensor) -> None:
    """tokens[i] = ids[src[i]] where src[i] >= 0 (all int32, on the device)."""
    _req(tokens, "tokens", torch.int32, 1); _req(ids, "ids", torch.int32, 1); _req(src, "src", torch.int32, 1)
    if src.shape[0] != tokens.shape[0]:
        raise KernelError("take_tokens: tokens and src differ in length")
    _check(lib().vk_take_tokens(_p(tokens), _p(ids), _p(src), tokens.shape[0], _stream()), "take_tokens")


_argmax_scratch = None


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = the lowest id among the maxima of logits[r, :]."""
    _req(logits, "logits", torch.float32, 2); _req(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax_rows: out and logits differ in rows")
    global _argmax_scratch
    rows = logits.shape[0]
    if _argmax_scratch is None or _argmax_scratch.numel() < rows * 12 or _argmax_scratch.device != logits.device:
        _argmax_scratch = torch.zeros(max(rows, 256) * 12, dtype=torch.uint8, device=logits.device)
    _check(lib().vk_argmax_rows(_p(logits), _p(out), _p(_argmax_scratch), rows, logits.shape[1], _stream()), "argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                uniform: torch.Tensor, probs_scratch: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row: greedy where temperature <= 0, else temperature / top-k / top-p with the row's uniform."""
    _req(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _req(temperature, "temperature", torch.float32, 1); _req(top_k, "top_k", torch.int32, 1)
    _req(top_p, "top_p", torch.float32, 1); _req(uniform, "uniform", torch.float64, 1)
    _req(probs_scratch, "probs_scratch", torch.float32); _req(out, "out", torch.int32, 1)
    if min(temperature.shape[0], top_k.shape[0], top_p.shape[0], uniform.shape[0], out.shape[0]) < R:
        raise KernelError("sample_rows: a per-row array is shorter than the rows")
    if probs_scratch.numel() < R * V:
        raise KernelError("sample_rows: the scratch is smaller than [rows, vocab]")
    _check(lib().vk_sample_rows(_p(logits), _p(temperature), _p(top_k), _p(top_p), _p(uniform), _p(probs_scratch), _p(out),
                                R, V, _stream()), "sample_rows")
    return out


_error_word = None


def error_word() -> torch.Tensor:
    """A pinned host word that kernels with bounded waits set when a wait runs out (the device writes it
    through the mapped address; the host reads it for free after any synchronisation)."""
    global _error_word
    if _error_word is None:
        _error_word = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_word


class KernelGaveUp(KernelError):
    """A kernel's bounded wait ran out; what it and the kernels after it wrote is not valid."""


def device_error_code() -> int:
    """The code the last kernel that gave up a wait left (0: none), without clearing it.  The word is host memory,
    so reading it costs nothing; it is up to date after any synchronisation with the kernels in question."""
    return 0 if _error_word is None else int(_error_word[0])


def check_device_errors() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (call after a synchronisation)."""
    code = device_error_code()
    if code != 0:
        _error_word[0] = 0
        raise KernelGaveUp(f"a kernel gave up waiting on an mbarrier (code {code}); its results are not valid")


def set_wait_limit_ms(ms: float) -> None:
    """The limit of one wait inside the kernels that wait on mbarriers, for every launch from now on, in
    milliseconds at the device's highest clock (0 or less: the default, about a second).  Launches that a CUDA
    graph already holds keep the limit they were captured with."""
    status = lib().vk_set_wait_limit_ms(ctypes.c_double(float(ms)))
    if status != 0:
        raise KernelError(f"set_wait_limit_ms: CUDA error {status}")


WAIT_FAMILIES = {"linear_tcgen05": 1, "linear_tcgen05_wide": 2, "attention_prefill_tcgen05": 3, "attention_decode_tma": 4}


def skip_stage_once(family: str, stage: int) -> None:
    """For tests of the give-up path: the next launch of the named kernel family leaves one pipeline stage of
    every block unarmed and unfilled, so its waits run out, the error word is set and the kernel returns by
    itself.  Nothing faults: no address is out of range and nothing traps."""
    lib().vk_test_skip_stage(WAIT_FAMILIES[family], int(stage))


def tcgen05_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands (bfloat16, K and the row stride multiples of 8, aligned)."""
    return (x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> torch.Tensor:
    """out (=, or += in mode 2) x @ w.T in bfloat16 on the tcgen05 tensor cores, float32 accumulation in tensor memory."""
    if not tcgen05_takes(x, w):
        raise KernelError("linear_tcgen05: operands must be bfloat16, 16-byte aligned, with K and the row stride multiples of 8")
    _req(w, "w", torch.bfloat16, 2); _req(out, "out", torch.bfloat16 if mode == LINEAR_SAME else torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    _check(lib().vk_linear_tcgen05(_p(x), _p(w), _p(out), M, N, K, x.stride(0), mode, _p(error_word()), _stream()), "linear_tcgen05")
    return out


def linear_tcgen05_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [M, I] = silu(x @ gate.T) * (x @ up.T) in one tcgen05 kernel; w_gate_up [2I, K], gate rows then up rows."""
    if not tcgen05_takes(x, w_gate_up):
        raise KernelError("linear_tcgen05_swiglu: operands must be bfloat16, 16-byte aligned, with K and the row stride multiples of 8")
    _req(w_gate_up, "w_gate_up", torch.bfloat16, 2); _req(out, "out", torch.bfloat16, 2)
    M, K = x.shape
    inter = w_gate_up.shape[0] // 2
    if w_gate_up.shape != (2 * inter, K) or out.shape != (M, inter) or inter % 8:
        raise KernelError("linear_tcgen05_swiglu: shapes do not fit")
    _check(lib().vk_linear_tcgen05_swiglu(_p(x), _p(w_gate_up), _p(out), M, inter, K, x.stride(0), _p(error_word()), _stream()),
           "linear_tcgen05_swiglu")
    return out


def linear_tcgen05_rope(x: torch.Tensor, wqkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor,
                        sin: torch.Tensor, slot_mapping: torch.Tensor, cache_layer: torch.Tensor, nh: int, nkv: int,
                        hd: int) -> torch.Tensor:
    """q, k, v projections with the rotation of q and k and the write of k and v into the pages in the product's
    epilogue (head sizes 64 and 128; the whole head is rotated)."""
    if not tcgen05_takes(x, wqkv):
        raise KernelError("linear_tcgen05_rope: operands must be bfloat16, 16-byte aligned, with K and the row stride multiples of 8")
    _req(wqkv, "wqkv", torch.bfloat16, 2); _req(q_out, "q_out", torch.bfloat16, 2); _req(positions, "positions", torch.int32, 1)
    _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2); _req(slot_mapping, "slot_mapping", torch.int32, 1)
    _req(cache_layer, "cache_layer", torch.bfloat16, 5)
    M, K = x.shape
    ps = cache_layer.shape[3]
    if (wqkv.shape != ((nh + 2 * nkv) * hd, K) or q_out.shape != (M, nh * hd) or cos.shape[1] != hd // 2 or sin.shape != cos.shape
            or tuple(cache_layer.shape[1:]) != (2, nkv, ps, hd) or positions.shape[0] < M or slot_mapping.shape[0] < M):
        raise KernelError("linear_tcgen05_rope: shapes do not fit the head counts")
    _check(lib().vk_linear_tcgen05_rope(_p(x), _p(wqkv), _p(q_out), M, K, x.stride(0), _p(positions), _p(cos), _p(sin),
                                        _p(slot_mapping), _p(cache_layer), nh, nkv, hd, ps, _p(error_word()), _stream()),
           "linear_tcgen05_rope")
    return q_out


EPI_SAME, EPI_F32, EPI_ACC, EPI_SWIGLU, EPI_ROPE = 0, 1, 2, 3, 4
SKINNY_MAX_ROWS = 64
FUSED_NORM_MAX_ROWS = 16     # a block of the few-rows kernel norms every row it stages: beyond this many a norm kernel runs once
NORM_IN_REGISTERS_MAX_K = 640    # the tensor-core few-rows kernel norms rows of up to this many columns without staging them


def _mma_rows_per_block(M: int, N: int, K: int) -> int:
    """Batch rows a block of the tensor-core few-rows kernel stages (its launcher's rule): all of them in groups
    of eight; at most 16 for weights of up to 16 MB; fewer when the weights make too few tiles to fill the machine."""
    tiles = ((N + 1) // 2 + 7) // 8
    mg = 1 if M <= 8 else 2 if M <= 16 else 4 if M <= 32 else 8
    if mg > 2 and N * K * 2 <= (16 << 20):
        mg = 2
    while mg > 1 and tiles * -(-M // (8 * mg)) < 120:
        mg //= 2
    return 8 * mg


def _mma_norm_smem(M: int, K: int, N: int) -> int:
    """Shared memory of the tensor-core few-rows kernel with the fused norm: a block's rows staged whole in float32."""
    rows = _mma_rows_per_block(M, N, K)
    return rows * (4 * K + 64) + 4 * K + 8 * (rows // 8) * 512


def fused_norm_takes(dtype: torch.dtype, M: int, K: int, N: int) -> bool:
    """Whether norm and product should be one launch.  Every block norms the rows it stages, so the rows of a
    block must be few (at most 16) and, in float32, small enough that two blocks share a multiprocessor."""
    if not skinny_takes(dtype, M, K, N):
        return False
    if dtype == torch.float32 or K % 32 != 0:
        return M <= FUSED_NORM_MAX_ROWS
    rows = _mma_rows_per_block(M, N, K)
    # Rows of up to 640 columns are normed in registers, and a block may norm 16 of them; longer rows are staged in
    # float32 first, and beyond eight of them a norm kernel that runs once is faster (measured at K = 960 and 16 / 64
    # decode rows: 1.48 against 1.53 and 2.73 against 2.91 ms a step; at K = 576 the fused form wins: 1.42 against 1.53).
    if rows > (FUSED_NORM_MAX_ROWS if K <= NORM_IN_REGISTERS_MAX_K else min(8, FUSED_NORM_MAX_ROWS)):
        return False
    return _mma_norm_smem(M, K, N) <= 112 * 1024


def skinny_takes(dtype: torch.dtype, M: int, K: int, N: int = 0) -> bool:
    """Whether the few-rows kernel should take this product (else the tile kernels do the work).  Every block
    stages all M rows for itself, so many rows times many blocks (a large N) is left to the tile kernels."""
    if dtype == torch.float32 and _float32_exact:
        return False
    if not (0 < M <= SKINNY_MAX_ROWS and K % (4 if dtype == torch.float32 else 8) == 0):
        return False
    return M <= 8 or N <= 8192 or dtype == torch.float32


def linear_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, *, norm_weight: Optional[torch.Tensor] = None,
                  eps: float = 0.0, rows: Optional[torch.Tensor] = None, rope: Optional[tuple] = None,
                  force_simt: bool = False) -> torch.Tensor:
    """out = epilogue(x' @ w.T) for at most 64 rows, where x' is x, or rmsnorm(x[rows]) * norm_weight when
    norm_weight is given (x float32 then).  epi: EPI_SAME / EPI_F32 / EPI_ACC as LINEAR_*; EPI_SWIGLU: out [M, N/2] =
    silu(first half) * second half; EPI_ROPE: out = rotated q [M, nh*hd], rotated k and v go into the cache;
    rope = (positions, cos, sin, slot_mapping, cache_layer, nh, nkv, hd)."""
    _req(w, "w", dims=2)
    N, K = w.shape
    if norm_weight is not None:
        _req(x, "x", torch.float32, 2); _req(norm_weight, "norm_weight", torch.float32, 1)
        if x.shape[1] != K or norm_weight.shape[0] != K:
            raise KernelError("linear_skinny: widths differ")
        M = x.shape[0]
        if rows is not None:
            _req(rows, "rows", torch.int32, 1)
            M = rows.shape[0]
        ldx = x.stride(0)
    else:
        if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1 or x.dtype != w.dtype:
            raise KernelError("linear_skinny: x must be a CUDA matrix of the weights' dtype with unit column stride")
        if x.shape[1] != K or rows is not None:
            raise KernelError("linear_skinny: widths differ, or rows given without a norm")
        M = x.shape[0]
        ldx = x.stride(0) if M > 1 else max(K, x.stride(0))
    want = {EPI_SAME: ((M, N), w.dtype), EPI_F32: ((M, N), torch.float32), EPI_ACC: ((M, N), torch.float32),
            EPI_SWIGLU: ((M, N // 2), w.dtype)}
    pos = cos = sin = slot = cache = None
    nh = nkv = hd = ps = 0
    if epi == EPI_ROPE:
        pos, cos, sin, slot, cache, nh, nkv, hd = rope
        _req(pos, "positions", torch.int32, 1); _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2)
        _req(slot, "slot_mapping", torch.int32, 1); _req(cache, "cache_layer", w.dtype, 5)
        ps = cache.shape[3]
        if (cos.shape[1] != hd // 2 or tuple(cache.shape[1:]) != (2, nkv, ps, hd) or pos.shape[0] < M or slot.shape[0] < M
                or N != (nh + 2 * nkv) * hd):
            raise KernelError("linear_skinny: the rotary epilogue's arrays do not fit the head counts")
        want[EPI_ROPE] = ((M, nh * hd), w.dtype)
    _req(out, "out", want[epi][1], 2)
    if tuple(out.shape) != want[epi][0]:
        raise KernelError(f"linear_skinny: out is {tuple(out.shape)}, expected {want[epi][0]}")
    if (w.dtype == torch.bfloat16 and K % 32 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and not force_simt
            and (ldx % 4 == 0 and norm_weight.data_ptr() % 16 == 0 and _mma_norm_smem(M, K, N) <= 220 * 1024
                 if norm_weight is not None else ldx % 8 == 0)):
        # bfloat16: the tensor-core kernel
        _check(lib().vk_linear_skinny_mma(_p(x), _p(rows), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(out), M, N, K, ldx,
                                          epi, _p(pos), _p(cos), _p(sin), _p(slot), _p(cache), nh, nkv, hd, ps, _stream()),
               "linear_skinny_mma")
        return out
    _check(lib().vk_linear_skinny(_p(x), _p(rows), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(out), M, N, K, ldx, epi,
                                  _p(pos), _p(cos), _p(sin), _p(slot), _p(cache), nh, nkv, hd, ps, _dt(w), _stream()),
           "linear_skinny")
    return out


# ---------------------------------------------------------------------------
# Dispatch: which kernel a part's call runs, by dtype and size.
# ---------------------------------------------------------------------------

def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> torch.Tensor:
    """out (=, or += in mode LINEAR_ACC_F32) x @ w.T.  float32 runs on CUDA cores in float32 arithmetic
    (no reduced-precision matrix mode); bfloat16 runs the tensor-core kernel where it takes the sizes."""
    if skinny_takes(x.dtype, x.shape[0], x.shape[1], w.shape[0]) and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return linear_skinny(x, w, out, mode)
    if tcgen05_takes(x, w) and out.data_ptr() % 16 == 0:
        return linear_tcgen05(x, w, out, mode)
    if x.dtype == torch.float32 and _float32_exact:
        return linear_simt(x, w, out, mode, few_rows=0)        # the tile kernel for every batch: one order of sums
    return linear_simt(x, w, out, mode)


PREFILL_HEAD_SIZES = (16, 32, 64, 96, 128)


def attention_prefill(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor,
                      out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions in bfloat16 on the tensor cores.  tiles int32 [n, 4]: first token,
    rows (1..64), position of the first token, segment."""
    _req(q, "q", torch.bfloat16, 2); _req(cache_layer, "cache_layer", torch.bfloat16, 5)
    _req(block_tables, "block_tables", torch.int32, 2); _req(tiles, "tiles", torch.int32, 2); _req(out, "out", torch.bfloat16, 2)
    page_size = cache_layer.shape[3]
    if q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd) or tiles.shape[1] != 4:
        raise KernelError("attention_prefill: shapes do not fit the head counts")
    if hd not in PREFILL_HEAD_SIZES:
        raise KernelError(f"attention_prefill: head size {hd} is not one of {PREFILL_HEAD_SIZES}")
    _check(lib().vk_attention_prefill(_p(q), _p(cache_layer), _p(block_tables), _p(tiles), _p(out), tiles.shape[0], nh, nkv, hd,
                                      page_size, block_tables.shape[1], ctypes.c_float(scale), window, _stream()),
           "attention_prefill")
    return out


def set_prefill_streams(mode: int) -> int:
    """Which tcgen05 prompt-attention kernel a launch takes: 0 the kernel with two threads a query row, 1 the kernel with
    two streams of key steps, 2 by the size of the launch (the default).  Returns the mode that was in force."""
    return int(lib().vk_set_prefill_streams(int(mode)))


def attention_prefill_tcgen05_takes(q: torch.Tensor, cache_layer: torch.Tensor, hd: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these operands: bfloat16, head size 64, pages of 8, 16, 32
    or a multiple of 64 slots, q rows dense and 16-byte aligned."""
    ps = cache_layer.shape[3]
    return (q.dtype == torch.bfloat16 and hd == 64 and ps % 8 == 0 and (64 % ps == 0 or ps % 64 == 0) and q.dim() == 2
            and q.stride(1) == 1 and q.stride(0) == q.shape[1] and q.data_ptr() % 16 == 0 and cache_layer.data_ptr() % 16 == 0
            and cache_layer.is_contiguous())


def attention_prefill_tcgen05_scratch_bytes(cap_tiles: int, nh: int, max_context: int) -> int:
    fn = lib().vk_attention_prefill_tcgen05_scratch_bytes
    fn.restype = ctypes.c_size_t
    return int(fn(cap_tiles, nh, max_context))


def attention_prefill_tcgen05(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor,
                              out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: int = 0, *,
                              scratch: Optional[torch.Tensor] = None, cap_tiles: int = 0, max_context: int = 0,
                              grid_context: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions on the tcgen05 tensor cores (scores and P V in tensor memory, keys and
    values by TMA straight from the pages).  tiles int32 [n, 4]: first token, rows (1..128), position of the first
    token, segment.  A tile whose walk over the keys is long is cut into parts that different blocks take; their
    partial results meet in `scratch`: a byte buffer of attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh,
    max_context) that was zero at first use and is used with no other (cap_tiles, nh, max_context); grid_context
    (<= max_context) bounds the positions of this launch.  Without a scratch one is made for this call."""
    _req(q, "q", torch.bfloat16, 2); _req(cache_layer, "cache_layer", torch.bfloat16, 5)
    _req(block_tables, "block_tables", torch.int32, 2); _req(tiles, "tiles", torch.int32, 2); _req(out, "out", torch.bfloat16, 2)
    page_size = cache_layer.shape[3]
    if (q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd) or tiles.shape[1] != 4
            or out.stride(0) != out.shape[1]):
        raise KernelError("attention_prefill_tcgen05: shapes do not fit the head counts")
    if not attention_prefill_tcgen05_takes(q, cache_layer, hd):
        raise KernelError("attention_prefill_tcgen05: bfloat16, head size 64 and pages of 8, 16, 32 or a multiple of 64 slots only")
    if scratch is None:
        cap_tiles = tiles.shape[0]
        max_context = grid_context = max_context or block_tables.shape[1] * page_size
        scratch = torch.zeros(attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, max_context), dtype=torch.uint8, device=q.device)
    _req(scratch, "scratch", torch.uint8, 1)
    if scratch.numel() < attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, max_context):
        raise KernelError("attention_prefill_tcgen05: the scratch is too small")
    _check(lib().vk_attention_prefill_tcgen05(_p(q), _p(cache_layer), _p(block_tables), _p(tiles), _p(out), q.shape[0], tiles.shape[0],
                                              cache_layer.shape[0], nh, nkv, hd, page_size, block_tables.shape[1],
                                              ctypes.c_float(scale), window, _p(scratch), cap_tiles, max_context,
                                              grid_context or max_context, _p(error_word()), _stream()),
           "attention_prefill_tcgen05")
    return out


def attention(q: torch.Tensor, pages: torch.Tensor, meta, ctx, out: torch.Tensor, nh: int, nkv: int, hd: int,
              scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of a mixed batch over the paged cache; `meta` is the page group's GroupMeta.
    Single decoded tokens take the split-key kernel; tokens of prompt portions take the tensor-core kernel
    (bfloat16, head sizes it is built for); whatever is left takes attention_rows, which takes every size."""
    dec_ok = (bool(ctx.num_dec) and attention_decode_takes(q.dtype, hd, ctx.workspace.max_context)
              and not (q.dtype == torch.float32 and _float32_exact))
    pre_ok = (bool(ctx.num_pre) and q.dtype == torch.bfloat16 and hd in PREFILL_HEAD_SIZES and ctx.pre_tiles is not None
              and q.data_ptr() % 16 == 0)
    if dec_ok:
        ws = ctx.workspace
        cap, layout = ws.max_segments, ws.max_context
        nbytes = attention_decode_scratch_bytes(cap, nh, nkv, hd, layout)
        scratch = ws.flat(f"att.dec/{nh}/{nkv}/{hd}/{layout}", nbytes, torch.uint8, zero=True)
        attention_decode(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, scratch, cap, nh, nkv, hd, scale,
                         layout, min(layout, max(1, ctx.max_context)), window, ctx.dec_tokens)
    if pre_ok:
        if ctx.pre_tiles_big is not None and attention_prefill_tcgen05_takes(q, pages, hd) and out.stride(0) == out.shape[1]:
            ws = ctx.workspace
            cap_tiles, layout = ws.max_tokens // 128 + ws.max_segments, ws.max_context
            nbytes = attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, layout)
            scratch = ws.flat(f"att.pre/{nh}/{cap_tiles}/{layout}", nbytes, torch.uint8, zero=True)
            attention_prefill_tcgen05(q, pages, meta.block_tables, ctx.pre_tiles_big, out, nh, nkv, hd, scale, window,
                                      scratch=scratch, cap_tiles=cap_tiles, max_context=layout,
                                      grid_context=min(layout, max(1, ctx.max_context)))
        else:
            attention_prefill(q, pages, meta.block_tables, ctx.pre_tiles, out, nh, nkv, hd, scale, window)
    if not dec_ok and not pre_ok:
        return attention_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, scale, window)
    if ctx.num_pre and not pre_ok:
        attention_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, scale, window, ctx.pre_tokens)
    if ctx.num_dec and not dec_ok:
        attention_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, scale, window, ctx.dec_tokens)
    return out
