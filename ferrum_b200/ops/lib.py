"""The kernel library, loaded once, and thin checked wrappers around its C entry points.

There is no fallback: if the library cannot be built or loaded, or there is no CUDA
device, every op raises `KernelError`.  Wrappers take torch tensors only as typed
memory (pointer, shape, stride); no torch operator runs on the product path.
"""
from __future__ import annotations

import ctypes
import functools
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from . import build

F32, BF16, F16 = 0, 1, 2
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
SIXTEEN_BIT = (torch.bfloat16, torch.float16)       # the tensor-core kernels take either

EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL = 0, 1, 2                       # generic product
TC_STORE_BF16, TC_STORE_F32, TC_RESIDUAL, TC_SWIGLU, TC_GEGLU, TC_SWISH_CLAMP = 0, 1, 2, 3, 4, 5   # tcgen05 product (GEGLU: SWIGLU with gelu_tanh on the gate; SWISH_CLAMP: the clamped unit)

_lib = None
_lock = threading.Lock()
ABI = 17


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.build_kernels()
                try:
                    handle = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"cannot load the kernel library {path}: {e}") from None
                handle.ferrum_last_error.restype = ctypes.c_char_p
                handle.ferrum_gemm_tc_workspace.restype = c_longlong
                handle.ferrum_matrix_memory_state_floats.restype = c_longlong
                if handle.ferrum_kernels_abi() != ABI:
                    raise KernelError(f"{path} is a stale build; delete it and call again")
                if os.environ.get("FERRUM_DEPENDENT_LAUNCH", "1") == "0":
                    handle.ferrum_set_dependent_launch(c_int(0))
                _lib = handle
    return _lib


def require_cuda(device=None):
    if not torch.cuda.is_available():
        raise KernelError("ferrum_b200 runs on a CUDA device only (sm_100a); none is visible")
    lib()


def sm_count():
    """Multiprocessors of the current CUDA device, as the kernels' own grids count them."""
    return int(lib().ferrum_gemm_tc_default_ctas())


def gemm_tc_test_hooks(wait_cycles=0, drop_loads=False):
    """For tests of the failure path only: shorten every bounded wait of the tensor-core product
    kernels to `wait_cycles` clock cycles (0: the default of about a second), and make the
    producer of the single-CTA kernel request nothing, so that the waits run out and the kernel
    leaves with an error code.  Call again without arguments to restore."""
    lib().ferrum_gemm_tc_test_hooks(c_longlong(int(wait_cycles)), c_int(1 if drop_loads else 0))


def set_dependent_launch(on: bool):
    """Programmatic dependent launch between the kernels of a step (on by default): a kernel's
    prologue may overlap the tail of the kernel before it.  Off: plain stream order."""
    lib().ferrum_set_dependent_launch(c_int(1 if on else 0))


launches = 0          # kernel launches made through this module (every entry point launches one kernel)


class _Profile:
    """Per-kernel timing for `profile_begin` / `profile_report`: one CUDA event after every launch;
    a launch's time is the span from the event before it to its own (its wait for the kernel ahead
    of it included).  `work` is (bytes it must move, flops) where the wrapper knows them."""

    def __init__(self):
        self.rows = []        # (name, event after, work)
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def mark(self, name, work):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.rows.append((name, ev, work))


_profile = None
_work = None          # set by a wrapper just before its launch: (bytes, flops)


def profile_begin():
    """Start timing every kernel launched through this module (steps must run without CUDA graphs:
    `Engine(profile=True)` sees to it)."""
    global _profile
    require_cuda()
    _profile = _Profile()


def profile_report(peaks=None):
    """Stops the timing and returns one row per kernel name, largest total first: launches, total
    milliseconds, share of the total, microseconds per launch and, where the wrapper knows the
    kernel's work, GB/s and TFLOP/s (with `peaks` = {"hbm_gbs", "bf16_tflops"} also the fraction of
    whichever bound is nearer)."""
    global _profile
    prof, _profile = _profile, None
    if prof is None:
        return []
    torch.cuda.synchronize()
    acc, prev = {}, prof.start
    for name, ev, work in prof.rows:
        r = acc.setdefault(name, {"kernel": name, "launches": 0, "ms": 0.0, "bytes": 0, "flops": 0.0, "known": 0})
        r["launches"] += 1
        r["ms"] += prev.elapsed_time(ev)
        if work is not None:
            r["bytes"] += work[0]
            r["flops"] += work[1]
            r["known"] += 1
        prev = ev
    total = sum(r["ms"] for r in acc.values()) or 1.0
    out = []
    for r in sorted(acc.values(), key=lambda r: -r["ms"]):
        row = {"kernel": r["kernel"], "launches": r["launches"], "ms": round(r["ms"], 3), "share": round(r["ms"] / total, 4),
               "us_per_launch": round(r["ms"] * 1e3 / r["launches"], 2)}
        if r["known"] == r["launches"] and r["ms"] > 0:
            row["GBps"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9, 1)
            row["TFLOPs"] = round(r["flops"] / (r["ms"] * 1e-3) / 1e12, 2)
            if peaks:
                row["frac_of_roofline"] = round(max(row["GBps"] / peaks["hbm_gbs"], row["TFLOPs"] / peaks["bf16_tflops"]), 4)
        out.append(row)
    return out


def _check(rc, name):
    global launches, _work
    if rc != 0:
        _work = None
        raise KernelError(f"{name}: {lib().ferrum_last_error().decode()}")
    launches += 1
    if _profile is not None:
        _profile.mark(name, _work)
    _work = None


def _gemm_work(x, w, out, M, N, K, products=1):
    """(bytes, flops) of a product for the profile: every weight once, the tokens and the result."""
    global _work
    if _profile is not None:
        _work = (products * N * K * w.element_size() + M * K * x.element_size() + M * N * out.element_size(),
                 2.0 * products * M * N * K)


def _bytes_work(*tensors_rows):
    """(bytes, 0 flops) for the profile: (tensor, rows) pairs give rows x row bytes each."""
    global _work
    if _profile is not None:
        _work = (sum(int(r) * t.shape[-1] * t.element_size() for t, r in tensors_rows if t is not None), 0.0)


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle (the capture stream inside a graph capture)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype, name, ndim=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, found {t.dim()}")
    if t.dim() and t.stride(-1) != 1 and t.shape[-1] > 1:
        raise KernelError(f"{name} must be contiguous in its last dimension")


def _need16(t, name, ndim=None, like=None):
    """A CUDA tensor of a 16-bit float type (the same as `like`'s when given)."""
    _need(t, like.dtype if like is not None else None, name, ndim)
    if t.dtype not in SIXTEEN_BIT:
        raise KernelError(f"{name} must be bfloat16 or float16, found {t.dtype}")


def dtype_code(dtype):
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"unsupported compute dtype {dtype}") from None


# ----------------------------------------------------------------------------- ops
def embedding(table, ids, out, err, scale=1.0, pos_table=None, positions=None, copies=1):
    """out[t] = table[ids[t]] as float32; with `scale` the row is multiplied by it, with `pos_table`
    ([positions, E], the table's dtype) row positions[t] of it is added.  copies > 1: out is
    [>=T, copies * E] and receives the row that many times."""
    _need(table, None, "table", 2); _need(ids, torch.int32, "ids", 1); _need(out, torch.float32, "out", 2)
    V, E = table.shape
    T = ids.shape[0]
    if out.shape[0] < T or out.shape[1] != E * copies or not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("embedding: out must be contiguous [>=T, copies * E] and table contiguous")
    if scale != 1.0 or pos_table is not None:
        if copies != 1:
            raise KernelError("embedding: a scaled or positioned embedding writes one copy")
        if pos_table is not None:
            _need(pos_table, table.dtype, "pos_table", 2); _need(positions, torch.int32, "positions", 1)
            if pos_table.shape[1] != E or not pos_table.is_contiguous() or positions.shape[0] < T:
                raise KernelError("embedding: pos_table must be contiguous [positions, E]")
        _check(lib().ferrum_embedding_scaled(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), c_int(T), c_int(E),
                                             c_int(V), c_float(scale), _ptr(pos_table), _ptr(positions),
                                             c_int(pos_table.shape[0] if pos_table is not None else 0), _ptr(err),
                                             _stream()), "embedding_scaled")
        return
    _check(lib().ferrum_embedding(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), c_int(T), c_int(E),
                                  c_int(V), _ptr(err), c_int(copies), _stream()), "embedding")


class Partials:
    """A product that the tensor-core kernel left as float32 partials (see gemm_tc_deferred):
    the workspace that holds them and the four numbers a consumer needs to sum them."""

    def __init__(self, workspace, layout):
        self.workspace, self.layout = workspace, layout
        self._c = (c_int * 4)(*layout)


def rmsnorm(x, weight, out, eps, rows=None, n_rows=None, partials=None, groups=1):
    """out[r] = rmsnorm(x[rows[r] if rows else r]) * weight; x float32, out float32 or bfloat16.
    With `partials` (a deferred residual product) the rows of x first get the partials added,
    in place.  groups > 1: the row is cut into that many equal consecutive parts and each is
    divided by its own root mean square."""
    _need(x, torch.float32, "x", 2); _need(weight, torch.float32, "weight", 1); _need(out, None, "out", 2)
    E = x.shape[1]
    if n_rows is None:
        n_rows = rows.shape[0] if rows is not None else x.shape[0]
    if weight.shape[0] != E or out.shape[1] != E or out.shape[0] < n_rows or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("rmsnorm: shapes do not agree")
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    if partials is None:
        _bytes_work((x, n_rows), (out, n_rows))
    if groups != 1:
        if partials is not None:
            raise KernelError("rmsnorm: a grouped norm takes no pending product")
        _check(lib().ferrum_group_norm(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows), c_int(n_rows),
                                       c_int(E), c_int(groups), c_float(eps), _stream()), "group_norm")
        return
    if partials is not None:
        _check(lib().ferrum_rmsnorm_reduce(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows),
                                           c_int(n_rows), c_int(E), c_float(eps), _ptr(partials.workspace), partials._c,
                                           _stream()), "rmsnorm_reduce")
        return
    _check(lib().ferrum_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows), c_int(n_rows),
                                c_int(E), c_float(eps), _stream()), "rmsnorm")


def residual_reduce(h, n_rows, partials):
    """h[:n_rows] += the deferred product."""
    _need(h, torch.float32, "h", 2)
    _check(lib().ferrum_residual_reduce(_ptr(h), c_int(n_rows), c_int(h.shape[1]), _ptr(partials.workspace), partials._c,
                                        _stream()), "residual_reduce")


def swiglu_reduce(act, n_tokens, F, partials):
    """act[t, f] = silu(gate) * up from a deferred two-product launch."""
    _need16(act, "act", 2)
    _check(lib().ferrum_swiglu_reduce(_ptr(act), dtype_code(act.dtype), c_int(n_tokens), c_int(F), c_int(act.stride(0)), _ptr(partials.workspace),
                                      partials._c, _stream()), "swiglu_reduce")


@functools.lru_cache(maxsize=4096)
def gemm_tc_can_defer(M, N, K, dual):
    """(A pure function of the shape, asked for every product of every step: remembered.)"""
    return bool(lib().ferrum_gemm_tc_can_defer(c_int(M), c_int(N), c_int(K), c_int(1 if dual else 0), c_int(0)))


def gemm_tc_deferred(x, w, err, workspace, M=None, N=None, dual_offset=0, n_ctas=0):
    """The tensor-core product without its final reduction: returns `Partials` for the kernel
    that consumes the product.  Only for shapes that `gemm_tc_can_defer` accepts."""
    _need16(x, "x", 2); _need16(w, "w", 2, like=x); _need(workspace, torch.float32, "workspace")
    M = x.shape[0] if M is None else M
    K = w.shape[1]
    N = (w.shape[0] - dual_offset) if N is None else N
    if x.shape[1] != K or x.shape[0] < M:
        raise KernelError(f"gemm_tc_deferred: shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)}")
    layout = (c_int * 4)()
    _gemm_work(x, w, workspace, M, N, K, 2 if dual_offset else 1)
    _check(lib().ferrum_gemm_tc_deferred(_ptr(x), _ptr(w), dtype_code(x.dtype), c_int(M), c_int(N), c_int(K), c_int(x.stride(0)),
                                         c_int(w.stride(0)), c_int(w.shape[0]), c_int(dual_offset), c_int(n_ctas),
                                         _ptr(workspace), c_longlong(workspace.numel()), layout, _ptr(err), _stream()),
           "gemm_tc_deferred")
    return Partials(workspace, tuple(layout))


def gemm_generic(x, w, out, epilogue, M=None):
    """out[t, n] (=, or += for EPI_RESIDUAL) sum_k x[t, k] w[n, k]; CUDA cores, float32 accumulate."""
    _need(x, None, "x", 2); _need(w, x.dtype, "w", 2); _need(out, None, "out", 2)
    M = x.shape[0] if M is None else M
    N, K = w.shape
    if x.shape[1] != K or out.shape[1] < N or out.shape[0] < M or x.shape[0] < M:
        raise KernelError(f"gemm: shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    want = x.dtype if epilogue == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: out must be {want} for epilogue {epilogue}")
    _gemm_work(x, w, out, M, N, K)
    _check(lib().ferrum_gemm_generic(_ptr(x), _ptr(w), _ptr(out), dtype_code(x.dtype), c_int(M), c_int(N), c_int(K),
                                     c_int(x.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(epilogue),
                                     _stream()), "gemm_generic")


def gemm_tc_supported(x, w):
    """True when the tcgen05 kernel takes these operands (one 16-bit type, 16-byte rows)."""
    return (x.dtype in SIXTEEN_BIT and w.dtype == x.dtype and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_token_tile(M, dual):
    return lib().ferrum_gemm_tc_token_tile(c_int(M), c_int(1 if dual else 0))


@functools.lru_cache(maxsize=4096)
def gemm_tc_workspace(M, N, K, dual, n_ctas=0):
    """(workspace floats, tile counters) that a launch needs."""
    tiles = c_int(0)
    need = lib().ferrum_gemm_tc_workspace(c_int(M), c_int(N), c_int(K), c_int(1 if dual else 0), c_int(n_ctas),
                                          ctypes.byref(tiles))
    return int(need), tiles.value


def gemm_tc(x, w, out, epilogue, err, workspace, counters, M=None, N=None, dual_offset=0, n_ctas=0, glu_limit=0.0):
    """16-bit (bfloat16 or float16) tensor-core product; see csrc/kernels/gemm_tc.cu.  `N` is the number of
    output features (rows of w used per product); with dual_offset > 0 rows dual_offset + n
    feed the second product of the SwiGLU epilogue.  `workspace` (float32) and `counters`
    (int32, all zero) are scratch for tiles that several CTAs share; n_ctas = 0 means one CTA
    per SM."""
    _need16(x, "x", 2); _need16(w, "w", 2, like=x); _need(out, None, "out", 2)
    M = x.shape[0] if M is None else M
    K = w.shape[1]
    N = (w.shape[0] - dual_offset) if N is None else N
    if x.shape[1] != K or out.shape[1] < N or out.shape[0] < M or x.shape[0] < M:
        raise KernelError(f"gemm_tc: shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    want = x.dtype if epilogue in (TC_STORE_BF16, TC_SWIGLU, TC_GEGLU, TC_SWISH_CLAMP) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc: out must be {want} for epilogue {epilogue}")
    _need(workspace, torch.float32, "workspace")
    _need(counters, torch.int32, "counters")
    _gemm_work(x, w, out, M, N, K, 2 if dual_offset else 1)
    _check(lib().ferrum_gemm_tc(_ptr(x), _ptr(w), _ptr(out), dtype_code(x.dtype), c_int(M), c_int(N), c_int(K), c_int(x.stride(0)),
                                c_int(w.stride(0)), c_int(out.stride(0)), c_int(w.shape[0]), c_int(epilogue),
                                c_int(dual_offset), c_int(n_ctas), _ptr(workspace), c_longlong(workspace.numel()),
                                _ptr(counters), c_int(counters.numel()), _ptr(err), c_float(glu_limit), _stream()), "gemm_tc")


def rope_cache_write(qkv, n_tokens, positions, req_of_token, block_table, cos_sin, kv_plane, page_stride, page_size,
                     Hq, Hkv, D, R, pairing, write_kv, err, partials=None):
    """Rotate q (in place) and k, store k and v into the paged cache plane.  With `partials`
    the q, k, v rows are first summed from a deferred product into `qkv`."""
    _need(qkv, None, "qkv", 2); _need(positions, torch.int32, "positions", 1)
    _need(req_of_token, torch.int32, "req_of_token", 1); _need(block_table, torch.int32, "block_table", 2)
    if R:
        _need(cos_sin, torch.float32, "cos_sin", 3)
        if cos_sin.shape[1] != R // 2 or cos_sin.shape[2] != 2 or not cos_sin.is_contiguous():
            raise KernelError("rope: cos_sin must be contiguous [positions, rope_dim/2, 2]")
    if write_kv:
        _need(kv_plane, qkv.dtype, "kv_plane")
    if not block_table.is_contiguous():
        raise KernelError("rope: block_table must be contiguous")
    global _work
    if _profile is not None and partials is None:
        _work = (n_tokens * (2 * Hq + (3 * Hkv if write_kv else 0)) * D * qkv.element_size(), 0.0)
    _check(lib().ferrum_rope_cache_write(_ptr(qkv), dtype_code(qkv.dtype), c_int(n_tokens), c_int(qkv.stride(0)),
                                         _ptr(positions), _ptr(req_of_token), _ptr(block_table),
                                         c_int(block_table.shape[1]), _ptr(cos_sin if R else None),
                                         c_int(cos_sin.shape[0] if R else 0), _ptr(kv_plane if write_kv else None),
                                         c_longlong(page_stride), c_int(page_size), c_int(Hq), c_int(Hkv), c_int(D),
                                         c_int(R), c_int(pairing), c_int(1 if write_kv else 0), _ptr(err),
                                         _ptr(partials.workspace if partials is not None else None),
                                         partials._c if partials is not None else None, _stream()),
           "rope_cache_write")


def attention_generic_split():
    """Keys per split of the generic attention kernel's split mode."""
    return int(lib().ferrum_attention_generic_split())


def attention_generic(q, out, n_tokens, positions, req_of_token, block_table, kv_plane, page_stride, page_size, Hq,
                      Hkv, D, scale, window, err, part=None, split_slots=0, q_start=None, n_reqs=0, distance_penalty=None,
                      chunked=False, softcap=0.0, sink=False):
    """Causal GQA attention of every token over its request's pages on the CUDA cores, float32
    arithmetic.  part=None: one CTA per (token, group of heads) walks the whole key range (many
    tokens).  With `part` (float32, n_tokens * Hq * split_slots * (D + 2) elements) every row's keys
    are cut at multiples of `attention_generic_split()` among split_slots CTAs and folded by a
    second launch (few tokens); split_slots must cover the longest row.  With q_start (the device's
    n_reqs + 1 token offsets of the requests, tokens of a request in ascending positions) and no
    `part`, up to eight tokens of a request that follow each other share every tile of keys.
    distance_penalty=(r1, r2), float32 per query head: r1[h] * ln(1 + r2[h] * (position - key position))
    is taken off the scaled score; with r2 None it is the straight line r1[h] * (position - key position).
    chunked: `window` is the length of a chunk (positions are cut into chunks from 0; a query sees its own
    chunk's keys up to itself) instead of a sliding window.  softcap c > 0: the scaled score becomes c * tanh(score / c).
    sink: a key of score 0 without a value joins every softmax (one more term in its denominator).  `out` may be float32 whatever the cache's type
    (a kernel after this one still works on the heads' results)."""
    _need(q, None, "q", 2); _need(out, None, "out", 2); _need(kv_plane, q.dtype, "kv_plane")
    if out.dtype not in (q.dtype, torch.float32):
        raise KernelError(f"attention: out must be {q.dtype} or float32, found {out.dtype}")
    r1 = r2 = None
    if distance_penalty is not None:
        r1, r2 = distance_penalty
        _need(r1, torch.float32, "r1", 1)
        if r2 is not None:
            _need(r2, torch.float32, "r2", 1)
        if r1.shape[0] != Hq or (r2 is not None and r2.shape[0] != Hq):
            raise KernelError("attention: the distance penalty has one pair of numbers per query head")
    _need(positions, torch.int32, "positions", 1); _need(req_of_token, torch.int32, "req_of_token", 1)
    _need(block_table, torch.int32, "block_table", 2)
    if not block_table.is_contiguous():
        raise KernelError("attention: block_table must be contiguous")
    if part is not None:
        _need(part, torch.float32, "part")
        if part.numel() < n_tokens * Hq * split_slots * (D + 2):
            raise KernelError("attention: the partials buffer is too small")
    _check(lib().ferrum_attention_generic(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)),
                                          dtype_code(q.dtype), c_int(n_tokens), _ptr(positions), _ptr(req_of_token),
                                          _ptr(block_table), c_int(block_table.shape[1]), _ptr(kv_plane),
                                          c_longlong(page_stride), c_int(page_size), c_int(Hq), c_int(Hkv), c_int(D),
                                          c_float(scale), c_int(window), _ptr(err), _ptr(part), c_int(split_slots),
                                          _ptr(q_start) if part is None else None, c_int(n_reqs), _ptr(r1), _ptr(r2),
                                          c_int(1 if out.dtype == torch.float32 and q.dtype != torch.float32 else 0),
                                          c_int(1 if chunked else 0), c_float(softcap or 0.0), c_int(1 if sink else 0), _stream()),
           "attention_generic")


def attention_flash_supported(dtype, D, page_stride=0):
    """True when the tensor-core attention kernel is built for this dtype and head size."""
    return dtype in SIXTEEN_BIT and bool(lib().ferrum_attention_flash_supported(c_int(D), c_int(16)))


def attention_work(ctx, Hq, Hkv, D, window, esize):
    """(bytes, flops) of causal attention for the step in `ctx`, for the profile: every visible key
    and value row once, the queries and outputs; two products per (query, visible key) pair."""
    keys, pairs = visible_keys(ctx, window)
    return (keys * 2 * Hkv * D * esize + 2 * ctx.n_tokens * Hq * D * esize, 4.0 * pairs * Hq * D)


def visible_keys(ctx, window):
    """(cached rows the step's requests read, (query, visible key) pairs) of the step in `ctx`."""
    keys = pairs = 0
    for p, n in zip(ctx.h_pos0, ctx.h_q_len):
        keys += min(p + n, window + n - 1) if window > 0 else p + n
        for i in range(n):
            pairs += min(p + i + 1, window) if window > 0 else p + i + 1
    return keys, pairs


def set_work(work):
    """A part that knows its kernel's work tells the profile before the launch."""
    global _work
    if _profile is not None:
        _work = work


def profiling():
    return _profile is not None


def attention_flash(q, out, kv_plane, page_stride, page_size, block_table, q_start, pos0, work, n_work, part_o,
                    part_ml, Hq, Hkv, D, scale, window, bm, err, cta_items=None, n_ctas=0, trigger_early=False):
    """Tensor-core attention over the work items of one row-tile class (bm 16 or 64).
    trigger_early: the kernels that follow in the stream may start while this one runs."""
    _need16(q, "q", 2); _need16(out, "out", 2, like=q); _need16(kv_plane, "kv_plane", like=q)
    _need(block_table, torch.int32, "block_table", 2); _need(work, torch.int32, "work", 1)
    _check(lib().ferrum_attention_flash(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), dtype_code(q.dtype),
                                        _ptr(kv_plane),
                                        c_longlong(page_stride), c_int(page_size), _ptr(block_table),
                                        c_int(block_table.shape[1]), _ptr(q_start), _ptr(pos0), _ptr(work),
                                        c_int(n_work), _ptr(cta_items), c_int(n_ctas), _ptr(part_o), _ptr(part_ml),
                                        c_int(Hq), c_int(Hkv), c_int(D),
                                        c_float(scale), c_int(window), c_int(bm), c_int(1 if trigger_early else 0),
                                        _ptr(err), _stream()), "attention_flash")


def attention_tc_tokens(D, G, page_size, kv_plane=None, page_stride=0):
    """Tokens per work item of the tcgen05 attention kernel for this head size, group size and
    page size (an item has that many tokens x G rows); 0 where the kernel does not apply (other
    sizes, float32, pages that are not dense in the plane)."""
    if kv_plane is not None and (kv_plane.dtype not in SIXTEEN_BIT or kv_plane.dim() != 5 or
                                 page_stride != kv_plane[0].numel()):
        return 0
    return int(lib().ferrum_attention_tc_tokens(c_int(D), c_int(G), c_int(page_size)))


def set_attention_pair_kernel(on: bool):
    """Head size 128 runs the tcgen05 attention on CTA pairs (on by default); off: the single-CTA
    kernel takes the same work items (for comparisons)."""
    lib().ferrum_set_attention_pair_kernel(c_int(1 if on else 0))


def attention_tc(q, out, kv_plane, page_stride, page_size, block_table, q_start, pos0, work, n_work, part_o, part_ml,
                 Hq, Hkv, D, scale, window, err):
    """tcgen05 attention over work items of attention_tc_tokens * G rows (prompt portions)."""
    _need16(q, "q", 2); _need16(out, "out", 2, like=q); _need16(kv_plane, "kv_plane", like=q)
    _need(block_table, torch.int32, "block_table", 2); _need(work, torch.int32, "work", 1)
    _check(lib().ferrum_attention_tc(_ptr(q), c_int(q.stride(0)), c_longlong(q.shape[0]), _ptr(out), c_int(out.stride(0)),
                                     dtype_code(q.dtype), _ptr(kv_plane), c_longlong(page_stride), c_longlong(kv_plane.shape[0]),
                                     c_int(page_size), _ptr(block_table), c_int(block_table.shape[1]), _ptr(q_start),
                                     _ptr(pos0), _ptr(work), c_int(n_work), _ptr(part_o), _ptr(part_ml), c_int(Hq),
                                     c_int(Hkv), c_int(D), c_float(scale), c_int(window), _ptr(err), _stream()),
           "attention_tc")


def attention_combine(out, part_o, part_ml, q_start, req_of_token, req_tile0, tile_info, token_list, n_tokens, Hq, Hkv,
                      D, bm, n_warps=1):
    """Merges the key-range splits written by attention_flash into `out`.  n_warps (1..8): warps
    per (token, head) that share its splits; more than one pays from about 16 splits on."""
    _need16(out, "out", 2)
    _check(lib().ferrum_attention_combine(_ptr(out), c_int(out.stride(0)), dtype_code(out.dtype), _ptr(part_o), _ptr(part_ml), _ptr(q_start),
                                          _ptr(req_of_token), _ptr(req_tile0), _ptr(tile_info), _ptr(token_list),
                                          c_int(n_tokens), c_int(Hq), c_int(Hkv), c_int(D), c_int(bm), c_int(n_warps), _stream()),
           "attention_combine")


def swiglu(gu, act, n_tokens, F):
    """act[t, f] = silu(gu[t, f]) * gu[t, F + f]."""
    _need(gu, None, "gu", 2); _need(act, gu.dtype, "act", 2)
    _check(lib().ferrum_swiglu(_ptr(gu), _ptr(act), dtype_code(gu.dtype), c_int(n_tokens), c_int(F),
                               c_int(gu.stride(0)), c_int(act.stride(0)), _stream()), "swiglu")


def sample(logits, n_rows, out_ids, err, inv_temperature=None, seeds=None, counters=None, also_to=None):
    """out_ids[r] = argmax, or the Gumbel-max draw where inv_temperature[r] != 0.  `also_to`
    (int32) receives the ids as well."""
    _need(logits, torch.float32, "logits", 2); _need(out_ids, torch.int32, "out_ids", 1)
    if inv_temperature is not None:
        _need(inv_temperature, torch.float32, "inv_temperature", 1)
        _need(seeds, torch.int64, "seeds", 1); _need(counters, torch.int32, "counters", 1)
    _check(lib().ferrum_sample(_ptr(logits), c_int(logits.stride(0)), c_int(n_rows), c_int(logits.shape[1]),
                               _ptr(inv_temperature), _ptr(seeds), _ptr(counters), _ptr(out_ids), _ptr(also_to),
                               _ptr(err), _stream()), "sample")


# ----------------------------------------------------------------------------- parallel gated block
def norm_pair_shift(x, w1, w2, shift, a, m, b, n_tokens, ctx, state, stage, groups, eps):
    """Both norms of a parallel block and the token shift of the mixer's input (gated_block.cu):
    a = n * w1, b = n * w2 (b, w2 may be None), m = a + (previous a - a) * shift (shift None: m = a).
    `ctx` gives positions, req_of_token, q_start and slots; state [slots, E] and stage [requests, E]
    are float32."""
    _need(x, torch.float32, "x", 2); _need(w1, torch.float32, "w1", 1); _need(a, None, "a", 2); _need(m, a.dtype, "m", 2)
    E = x.shape[1]
    if not (x.is_contiguous() and a.is_contiguous() and m.is_contiguous()) or a.shape[1] != E or m.shape[1] != E:
        raise KernelError("norm_pair_shift: rows must be contiguous [T, E]")
    if b is not None:
        _need(b, a.dtype, "b", 2); _need(w2, torch.float32, "w2", 1)
    if shift is not None:
        _need(shift, torch.float32, "shift", 1); _need(state, torch.float32, "state", 2); _need(stage, torch.float32, "stage", 2)
        if state.shape[1] != E or stage.shape[1] != E or stage.shape[0] < ctx.n_reqs or not state.is_contiguous():
            raise KernelError("norm_pair_shift: state and stage rows must have E elements")
    _bytes_work((x, n_tokens), (a, n_tokens), (m, n_tokens), (b, n_tokens))
    _check(lib().ferrum_norm_pair_shift(_ptr(x), _ptr(w1), _ptr(w2), _ptr(shift), _ptr(a), _ptr(m), _ptr(b), dtype_code(a.dtype),
                                        c_int(n_tokens), _ptr(ctx.positions), _ptr(ctx.req_of_token), _ptr(ctx.q_start),
                                        _ptr(ctx.slots), _ptr(state), _ptr(stage), c_int(E), c_int(groups), c_float(eps),
                                        _stream()), "norm_pair_shift")


GLU_ACTS = {"silu": 0, "gelu_tanh": 1, "swish_clamp": 2}      # swish_clamp: min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)


def bias_glu(gu, bias_gate, bias_up, act, n_tokens, F, kind="silu", limit=0.0):
    """act[t, f] = f(gu[t, f] + bias_gate[f]) * (gu[t, F + f] + bias_up[f]); gu float32."""
    _need(gu, torch.float32, "gu", 2); _need(act, None, "act", 2)
    for bias in (bias_gate, bias_up):
        if bias is not None:
            _need(bias, torch.float32, "bias", 1)
    global _work
    if _profile is not None:
        _work = (n_tokens * F * (8 + act.element_size()), 0.0)
    _check(lib().ferrum_bias_glu(_ptr(gu), c_int(gu.stride(0)), _ptr(bias_gate), _ptr(bias_up), _ptr(act), dtype_code(act.dtype),
                                 c_int(act.stride(0)), c_int(n_tokens), c_int(F), c_int(GLU_ACTS[kind]), c_float(limit), _stream()), "bias_glu")


def bias_glu_reduce(partials, bias_gate, bias_up, act, n_tokens, F, kind="silu", extra=None, limit=0.0):
    """`bias_glu` on a product of 2F + n rows (gate | up | extra) that was left in deferred mode; the n
    extra columns are summed into `extra` (float32 [T, n], contiguous)."""
    _need(act, None, "act", 2)
    n_extra = 0
    if extra is not None:
        _need(extra, torch.float32, "extra", 2)
        if not extra.is_contiguous():
            raise KernelError("bias_glu_reduce: extra must be contiguous")
        n_extra = extra.shape[1]
    _check(lib().ferrum_bias_glu_reduce(_ptr(bias_gate), _ptr(bias_up), _ptr(act), dtype_code(act.dtype), c_int(act.stride(0)),
                                        c_int(n_tokens), c_int(F), c_int(GLU_ACTS[kind]), c_float(limit), _ptr(extra), c_int(n_extra),
                                        _ptr(partials.workspace), partials._c, _stream()), "bias_glu_reduce")


def gated_residual(x, n_tokens, y1, g1, c1, y2=None, c2=None, g2=None, c3=None, ctx=None, stage=None, state=None, p1=None,
                   p2=None):
    """x += y1 * sigmoid(g1 + c1) + (y2 + c2) * sigmoid(g2 + c3), all float32 (the second term only with
    y2 or p2).  p1 / p2: y1 / y2 as a product left in deferred mode (`Partials`), summed while read.
    With `state` the staged row of every request whose portion ends in this batch is copied into its
    state row."""
    _need(x, torch.float32, "x", 2)
    for t in (y1, g1, y2, g2):
        if t is not None:
            _need(t, torch.float32, "operand", 2)
    ld = lambda t: c_int(t.stride(0) if t is not None else 0)
    global _work
    if _profile is not None:
        _work = (n_tokens * x.shape[1] * 4 * (2 + sum(t is not None for t in (y1, g1, y2, g2))), 0.0)
    _check(lib().ferrum_gated_residual(_ptr(x), c_int(n_tokens), c_int(x.shape[1]), _ptr(y1), ld(y1), _ptr(g1), ld(g1), _ptr(c1),
                                       _ptr(y2), ld(y2), _ptr(c2), _ptr(g2), ld(g2), _ptr(c3),
                                       _ptr(ctx.req_of_token if state is not None else None),
                                       _ptr(ctx.q_start if state is not None else None),
                                       _ptr(ctx.slots if state is not None else None), _ptr(stage), _ptr(state),
                                       _ptr(p1.workspace if p1 is not None else None), p1._c if p1 is not None else None,
                                       _ptr(p2.workspace if p2 is not None else None), p2._c if p2 is not None else None,
                                       _stream()), "gated_residual")


# ----------------------------------------------------------------------------- attention over a cached latent
def latent_prep(proj, n_tokens, off_q, q_rank, wq, off_kv, kv_rank, rot_dim, wkv, off_gate, n_gate, ctx, block_table, rot,
                plane, page_stride, page_size, cq, gate, eps, partials=None):
    """From a token's float32 down-projections: the normalised query latent `cq`, the cache row
    (normalised latent, rotated key part) at the token's page (off_kv < 0: no cache write) and the
    sigmoid of the gate logits (latent.cu).  With `partials` (the product left in deferred mode) the
    projections are summed from them and `proj` may be None."""
    if partials is None:
        _need(proj, torch.float32, "proj", 2)
    _need(cq, None, "cq", 2); _need(gate, torch.float32, "gate", 2)
    if off_kv >= 0:
        _need(plane, cq.dtype, "plane")
    cos_sin = rot.cos_sin if rot is not None else None
    global _work
    if _profile is not None:
        _work = (n_tokens * ((off_gate + n_gate) * 4 + (q_rank + (kv_rank + rot_dim if off_kv >= 0 else 0)) * cq.element_size()), 0.0)
    _check(lib().ferrum_latent_prep(_ptr(proj), c_int(proj.stride(0) if proj is not None else 0), c_int(n_tokens), c_int(off_q), c_int(q_rank), _ptr(wq),
                                    c_int(off_kv), c_int(kv_rank), c_int(rot_dim), _ptr(wkv), c_int(off_gate), c_int(n_gate),
                                    _ptr(ctx.positions), _ptr(ctx.req_of_token), _ptr(block_table), c_int(block_table.shape[1]),
                                    _ptr(cos_sin), c_int(cos_sin.shape[0] if rot is not None else 0),
                                    c_int(rot.rope_dim if rot is not None else 0), _ptr(plane if off_kv >= 0 else None),
                                    c_longlong(page_stride), c_int(page_size), _ptr(cq), c_int(cq.stride(0)),
                                    dtype_code(cq.dtype), _ptr(gate), c_float(eps), _ptr(ctx.err),
                                    _ptr(partials.workspace if partials is not None else None),
                                    partials._c if partials is not None else None, _stream()), "latent_prep")


def latent_q_rope(q, qf, n_tokens, positions, rot, H, Dn, Rr, R, err):
    """The rotated part of every query head (q: heads of Dn + Rr) into qf (heads of R + Rr) at R."""
    _need(q, None, "q", 2); _need(qf, q.dtype, "qf", 2)
    cos_sin = rot.cos_sin if rot is not None else None
    _check(lib().ferrum_latent_q_rope(_ptr(q), c_int(q.stride(0)), _ptr(qf), c_int(qf.stride(0)), dtype_code(q.dtype),
                                      c_int(n_tokens), _ptr(positions), _ptr(cos_sin),
                                      c_int(cos_sin.shape[0] if rot is not None else 0),
                                      c_int(rot.rope_dim if rot is not None else 0), c_int(H), c_int(Dn), c_int(Rr), c_int(R),
                                      _ptr(err), _stream()), "latent_q_rope")


@functools.lru_cache(maxsize=1)
def attention_latent_split():
    """Keys per split of the latent attention kernel's split mode."""
    return int(lib().ferrum_attention_latent_split())


def attention_latent(qf, out, gate, n_tokens, ctx, block_table, plane, page_stride, page_size, H, Dk, Dv, scale, window,
                     single_tokens, part=None, split_slots=0, tensor_cores=None):
    """Attention of every token over its request's cached rows of Dk elements, whose first Dv
    elements are the values; qf: heads of Dk, out: heads of Dv, times gate[t, h] (latent.cu).
    tensor_cores: None picks the mma.sync kernel where it takes the shape (16-bit storage, Dk a
    multiple of 16, Dv of 32), else the CUDA-core kernel; False forces the latter.
    With `part` (float32, n_tokens * H * split_slots * (Dv + 2) elements; single tokens only) every
    token's keys are cut at multiples of `attention_latent_split()` among split_slots CTAs and folded
    by a second launch."""
    if part is not None:
        _need(part, torch.float32, "part")
        if part.numel() < n_tokens * H * split_slots * (Dv + 2):
            raise KernelError("attention_latent: the partials buffer is too small")
    _need(qf, None, "qf", 2); _need(out, qf.dtype, "out", 2); _need(plane, qf.dtype, "plane")
    if gate is not None:
        _need(gate, torch.float32, "gate", 2)
    global _work
    if _profile is not None:
        keys, pairs = visible_keys(ctx, window)
        _work = (keys * Dk * plane.element_size() + n_tokens * H * (Dk + Dv) * qf.element_size(), 2.0 * pairs * H * (Dk + Dv))
    args = (_ptr(qf), c_int(qf.stride(0)), _ptr(out), c_int(out.stride(0)), dtype_code(qf.dtype),
            _ptr(gate), c_int(n_tokens), _ptr(ctx.positions), _ptr(ctx.q_start), c_int(ctx.n_reqs),
            _ptr(block_table), c_int(block_table.shape[1]), _ptr(plane), c_longlong(page_stride),
            c_int(page_size), c_int(H), c_int(Dk), c_int(Dv), c_float(scale), c_int(window),
            c_int(1 if single_tokens else 0), _ptr(part), c_int(split_slots), _ptr(ctx.err), _stream())
    if tensor_cores is None:
        tensor_cores = attention_latent_mma_supported(qf, out, plane, page_stride, Dk, Dv)
    if tensor_cores:
        _check(lib().ferrum_attention_latent_mma(*args), "attention_latent_mma")
        if part is not None:
            _check(lib().ferrum_attention_latent_combine(_ptr(out), c_int(out.stride(0)), dtype_code(out.dtype), _ptr(part), _ptr(gate),
                                                         c_int(n_tokens), _ptr(ctx.positions), c_int(H), c_int(Dv), c_int(window),
                                                         c_int(split_slots), _stream()), "attention_latent_combine")
        return
    _check(lib().ferrum_attention_latent(*args), "attention_latent")
    if part is not None:
        globals()["launches"] += 1        # (the merge of the splits is a second kernel)


def attention_latent_mma_stage(keys=0):
    """For tests and measurements: force the tensor-core kernel's stage size (32 or 64 keys) wherever it
    fits; 0 restores its own rule (attention_latent_mma.cu)."""
    lib().ferrum_attention_latent_mma_stage(c_int(int(keys)))


def attention_latent_mma_supported(qf, out, plane, page_stride, Dk, Dv):
    """True where the tensor-core kernel (attention_latent_mma.cu) takes the shape and the pointers."""
    return qf.dtype in SIXTEEN_BIT and bool(lib().ferrum_attention_latent_mma_supported(
        dtype_code(qf.dtype), c_int(Dk), c_int(Dv), c_int(qf.stride(0)), c_int(out.stride(0)), c_longlong(page_stride),
        _ptr(qf), _ptr(out), _ptr(plane)))


@functools.lru_cache(maxsize=1)
def head_linear_max_tokens():
    return int(lib().ferrum_head_linear_max_tokens())


def head_linear_mma_supported(x, x_head_stride, w, y, y_head_stride):
    """True where the tensor-core kernel for many tokens takes the operands (16-bit, 16-byte rows)."""
    return x.dtype in SIXTEEN_BIT and bool(lib().ferrum_head_linear_mma_supported(
        dtype_code(x.dtype), c_int(w.shape[2]), c_int(x.stride(0)), c_int(x_head_stride), c_int(y.stride(0)), c_int(y_head_stride),
        _ptr(x), _ptr(w), _ptr(y)))


def head_linear(x, x_head_stride, w, y, y_head_stride, n_tokens):
    """y[t, h * y_head_stride + n] = sum_k x[t, h * x_head_stride + k] * w[h, n, k]: one small product
    per head in one launch; w: [H, N, K] contiguous.  Up to `head_linear_max_tokens()` tokens on the
    CUDA cores (latent.cu: the time is the weights' read); more tokens on mma.sync where
    `head_linear_mma_supported` (attention_latent_mma.cu)."""
    _need(x, None, "x", 2); _need(y, x.dtype, "y", 2); _need(w, x.dtype, "w", 3)
    if not w.is_contiguous():
        raise KernelError("head_linear: w must be contiguous [H, N, K]")
    H, N, K = w.shape
    if n_tokens > head_linear_max_tokens():
        global _work
        if _profile is not None:
            _work = (w.numel() * w.element_size() + n_tokens * H * (N + K) * x.element_size(), 2.0 * n_tokens * H * N * K)
        _check(lib().ferrum_head_linear_mma(_ptr(x), c_int(x.stride(0)), c_int(x_head_stride), _ptr(w), _ptr(y), c_int(y.stride(0)),
                                            c_int(y_head_stride), dtype_code(x.dtype), c_int(n_tokens), c_int(H), c_int(N), c_int(K),
                                            _stream()), "head_linear_mma")
        return
    if _profile is not None:
        _work = (w.numel() * w.element_size() + n_tokens * H * (N + K) * x.element_size(), 2.0 * n_tokens * H * N * K)
    _check(lib().ferrum_head_linear(_ptr(x), c_int(x.stride(0)), c_int(x_head_stride), _ptr(w), _ptr(y), c_int(y.stride(0)),
                                    c_int(y_head_stride), dtype_code(x.dtype), c_int(n_tokens), c_int(H), c_int(N), c_int(K),
                                    _stream()), "head_linear")


# ----------------------------------------------------------------------------- shaped attention heads
def qkv_shape(proj, n_tokens, ctx, block_table, rot, qk_pairing, value_rot, value_pairing, unit_norm, eps, q_out, plane,
              page_stride, page_size, Hq, Hkv, Dk, Dv, Dp, writes, bias=None, q_norm=None, k_norm=None, q_temp=None,
              value_mix=None, whole_norm=False, value_from_key=False):
    """Per head of a float32 product row [q | k | v | ...]: rotary turn of q and k (table `rot`:
    `.cos_sin` [positions, R/2, 2], `.rope_dim`; None: none), optional division by the head's root
    mean square, a turn of the value over all its elements (`value_rot`: a table [positions, Dv/2, 2]
    or None); q -> q_out [T, Hq * Dp], k and v -> the token's place in the cache (rows of Dp elements).
    bias: float32 [Hq*Dk + Hkv*(Dk+Dv)] added first.  q_norm / k_norm: float32 [Dk] weights of an RMS norm
    of every query / key head before the turn.  q_temp = (coef, every): a query at position p is multiplied
    by 1 + coef * ln(floor((p + 1) / every) + 1).  value_mix = ("store", v_first) leaves the float32 values
    in v_first [T, Hkv*Dv]; ("blend", v_first, lam) caches (1 - lam) v + lam v_first (lam: one float on the device).
    whole_norm: q_norm [Hq*Dk] and k_norm [Hkv*Dk] are the weights of an RMS norm over the token's whole query / key
    projection (all heads at once).  value_from_key: the row is [q | k] and a KV head's value is its key as projected."""
    for t, n in ((bias, Hq * Dk + Hkv * (Dk + Dv)), (q_norm, Hq * Dk if whole_norm else Dk), (k_norm, Hkv * Dk if whole_norm else Dk)):
        if t is not None:
            _need(t, torch.float32, "qkv_shape vector", 1)
            if t.shape[0] != n or not t.is_contiguous():
                raise KernelError("qkv_shape: a bias or norm weight has the wrong length")
    coef, every = q_temp if q_temp is not None else (0.0, 0)
    mode, v_first, lam = 0, None, None
    if value_mix is not None:
        mode = {"store": 1, "blend": 2}[value_mix[0]]
        v_first = value_mix[1]
        _need(v_first, torch.float32, "v_first", 2)
        if v_first.shape[0] < n_tokens or v_first.shape[1] < Hkv * Dv:
            raise KernelError("qkv_shape: v_first is too small")
        if mode == 2:
            lam = value_mix[2]
            _need(lam, torch.float32, "lambda")
    _need(proj, torch.float32, "proj", 2); _need(q_out, plane.dtype, "q_out", 2); _need(block_table, torch.int32, "block_table", 2)
    if proj.shape[1] < Hq * Dk + ((Hkv * Dk if value_from_key else Hkv * (Dk + Dv)) if writes else 0) or q_out.shape[1] < Hq * Dp:
        raise KernelError("qkv_shape: a row is too short for the heads")
    cs = rot.cos_sin if rot is not None else None
    _check(lib().ferrum_qkv_shape(_ptr(proj), c_int(proj.stride(0)), c_int(n_tokens), _ptr(ctx.positions), _ptr(ctx.req_of_token),
                                  _ptr(block_table), c_int(block_table.shape[1]), _ptr(cs), c_int(rot.rope_dim if rot is not None else 0),
                                  c_int(qk_pairing), c_int(cs.shape[0] if cs is not None else 0), _ptr(value_rot),
                                  c_int(value_pairing), c_int(value_rot.shape[0] if value_rot is not None else 0),
                                  c_int(1 if unit_norm else 0), c_float(eps), _ptr(q_out), c_int(q_out.stride(0)), _ptr(plane),
                                  c_longlong(page_stride), c_int(page_size), dtype_code(plane.dtype), c_int(Hq), c_int(Hkv),
                                  c_int(Dk), c_int(Dv), c_int(Dp), c_int(1 if writes else 0), _ptr(ctx.err), _ptr(bias),
                                  _ptr(q_norm), _ptr(k_norm), c_float(coef), c_int(every), c_int(mode), _ptr(v_first),
                                  c_int(v_first.stride(0) if v_first is not None else 0), _ptr(lam), c_int(1 if whole_norm else 0),
                                  c_int(1 if value_from_key else 0), _stream()),
           "qkv_shape")


def attention_finish(o, n_tokens, ctx, value_rot, value_pairing, gate, out, Hq, Dv, Dp):
    """out[t, h] = turn_back(o[t, h], position) * sigmoid(gate[t, h]) in the compute type; `value_rot`
    (None: no turn) and `gate` (float32 logits [T, Hq * Dv], may be a view into wider rows; None: no gate)."""
    _need(o, torch.float32, "o", 2); _need(out, None, "out", 2)
    if gate is not None:
        _need(gate, torch.float32, "gate", 2)
    _bytes_work((o, n_tokens), (out, n_tokens))
    _check(lib().ferrum_attention_finish(_ptr(o), c_int(o.stride(0)), c_int(n_tokens), _ptr(ctx.positions), _ptr(value_rot),
                                         c_int(value_pairing), c_int(value_rot.shape[0] if value_rot is not None else 0),
                                         _ptr(gate), c_int(gate.stride(0) if gate is not None else 0), _ptr(out),
                                         c_int(out.stride(0)), dtype_code(out.dtype), c_int(Hq), c_int(Dv), c_int(Dp),
                                         _ptr(ctx.err), _stream()), "attention_finish")


# ----------------------------------------------------------------------------- state-space mixer
def mamba2_mix(proj, n_tokens, ctx, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, heads, P, N, groups, norm_groups, eps,
               state, xbc, y, out):
    """Everything of the state-space mixer between its two products: short convolution + silu over
    x, B, C (its last inputs kept in the request's state row), the recurrence per head, the gate by
    silu(z) and the grouped RMS norm.  proj: float32 rows [z | x | B | C | dt]; state: float32
    [max_requests, heads * P * N + (taps - 1) * channels]; xbc, y: float32 scratch; out: compute type."""
    global launches
    _need(proj, torch.float32, "proj", 2); _need(state, torch.float32, "state", 2); _need(out, None, "out", 2)
    inner, C = heads * P, heads * P + 2 * groups * N
    taps = conv_w.shape[1]
    for t, n in ((conv_w, "conv_w"), (conv_b, "conv_b"), (dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip"), (norm_w, "norm_w")):
        _need(t, torch.float32, n)
    if (proj.shape[1] < inner + C + heads or conv_w.shape[0] != C or state.shape[1] != inner * N + (taps - 1) * C
            or xbc.numel() < n_tokens * C or y.numel() < n_tokens * inner or out.shape[1] != inner or not conv_w.is_contiguous()):
        raise KernelError("mamba2_mix: shapes do not agree")
    _check(lib().ferrum_mamba2_mix(_ptr(proj), c_int(proj.stride(0)), c_int(n_tokens), c_int(ctx.n_reqs), _ptr(ctx.req_of_token),
                                   _ptr(ctx.q_start), _ptr(ctx.slots), _ptr(conv_w), _ptr(conv_b), c_int(taps), _ptr(dt_bias),
                                   _ptr(a_log), _ptr(d_skip), _ptr(norm_w), c_int(heads), c_int(P), c_int(N), c_int(groups),
                                   c_int(norm_groups), c_float(eps), _ptr(state), c_longlong(state.stride(0)), _ptr(xbc), _ptr(y),
                                   _ptr(out), c_int(out.stride(0)), dtype_code(out.dtype), c_int(ctx.max_q_len), _stream()),
           "mamba2_mix")
    launches += 3 if taps > 1 else 2       # (the entry point launches the convolution, its state, the walk and the norm)


# ----------------------------------------------------------------------------- parallel block
def _partials_args(p):
    return (_ptr(p.workspace), p._c) if p is not None else (c_void_p(0), None)


def scaled_sum(x, y1, y2, mult, n_tokens, xc=None, p1=None, p2=None):
    """x[:n] += mult * (y1 + y2) in float32 (y2 may be None); xc, when given, also receives the new rows
    in its own type.  p1 / p2 (`Partials`) stand in for y1 / y2 when the sublayers left their last
    products in deferred mode."""
    _need(x, torch.float32, "x", 2)
    E = x.shape[1]
    for y, p in ((y1, p1), (y2, p2)):
        if p is None and y is not None:
            _need(y, torch.float32, "y", 2)
            if not y.is_contiguous() or y.shape[1] != E:
                raise KernelError("scaled_sum: rows must be contiguous and of one width")
    if (y1 is None and p1 is None) or not x.is_contiguous() or (xc is not None and (not xc.is_contiguous() or xc.shape[1] != E)):
        raise KernelError("scaled_sum: rows must be contiguous and of one width")
    _bytes_work((x, 2 * n_tokens), (y1, n_tokens), (y2, n_tokens), (xc, n_tokens))
    _check(lib().ferrum_scaled_sum(_ptr(x), _ptr(y1 if p1 is None else None), _ptr(y2 if p2 is None else None), c_float(mult),
                                   _ptr(xc), dtype_code(xc.dtype if xc is not None else torch.float32), c_int(n_tokens), c_int(E),
                                   *_partials_args(p1), *_partials_args(p2), _stream()), "scaled_sum")


def gated_table_rows(s, table, token_ids, offset, dim, out, n_tokens, err, partials=None):
    """out[t, j] = gelu_tanh(s[t, j]) * table[token_ids[t], offset + j]; s float32 (or a deferred product,
    `partials`), table and out in the compute type."""
    _need(table, out.dtype, "table", 2); _need(token_ids, torch.int32, "token_ids", 1)
    if partials is None:
        _need(s, torch.float32, "s", 2)
    _check(lib().ferrum_gated_table_rows(_ptr(s if partials is None else None), c_int(s.stride(0) if partials is None else 0),
                                         _ptr(table), c_int(table.stride(0)), c_int(table.shape[0]),
                                         _ptr(token_ids), c_int(offset), c_int(dim), _ptr(out), c_int(out.stride(0)),
                                         dtype_code(out.dtype), c_int(n_tokens), _ptr(err), *_partials_args(partials), _stream()),
           "gated_table_rows")


def norm_scaled_add_max_width():
    """The widest row whose product `norm_scaled_add` can take as partials."""
    return int(lib().ferrum_norm_scaled_add_max_width())


def norm_scaled_add(x, y, w, mult, eps, n_tokens, partials=None):
    """x[:n] += mult * y / sqrt(mean(y^2) + eps) * w, all float32; y a buffer or a deferred product (`partials`)."""
    _need(x, torch.float32, "x", 2); _need(w, torch.float32, "w", 1)
    E = x.shape[1]
    if partials is None:
        _need(y, torch.float32, "y", 2)
        if y.shape[1] != E or not y.is_contiguous():
            raise KernelError("norm_scaled_add: shapes do not agree")
    if w.shape[0] != E or not x.is_contiguous():
        raise KernelError("norm_scaled_add: shapes do not agree")
    _bytes_work((x, 2 * n_tokens), (x, n_tokens))
    _check(lib().ferrum_norm_scaled_add(_ptr(x), _ptr(y if partials is None else None), _ptr(w), c_float(mult), c_float(eps),
                                        c_int(n_tokens), c_int(E), *_partials_args(partials), _stream()), "norm_scaled_add")


# ----------------------------------------------------------------------------- several residual streams
HYPER_MAX_STREAMS = 8        # (the kernel's own limit, which it checks again)


class StreamWrite:
    """What a sublayer leaves for the kernel that reads the streams next: its result (`y` float32 [T, E], or
    `partials`, or `y` with `y_rows` int32 [T, top] naming the rows to add per token) and its carry matrix
    `mix` [S, S] and write vector `out` [S] (float32 on the device)."""

    def __init__(self, mix, out, y=None, partials=None, y_rows=None, top=0):
        self.mix, self.out, self.y, self.partials, self.y_rows, self.top = mix, out, y, partials, y_rows, int(top)


def hyper_step(X, S, E, n_rows, write=None, rows=None, store=True, in_w=None, norm_w=None, eps=0.0, out=None):
    """One pass over the residual streams X [tokens, S * E] (float32): first the pending `write` of the sublayer
    before (X'[t] = sum_s mix[s, t] X[s] + out[t] y), stored when `store`; then, when `out` is given, the read
    u = sum_s in_w[s] X[s] (in_w None: the plain sum) and out = rms(u) * norm_w in out's type.  `rows` (int32):
    work on these tokens only, storing nothing."""
    _need(X, torch.float32, "X", 2)
    if X.shape[1] != S * E or not X.is_contiguous():
        raise KernelError("hyper_step: X must be contiguous [tokens, S * E]")
    y = ldy = y_rows = part = layout = mix = out_w = None
    top = 0
    if write is not None:
        mix, out_w = write.mix, write.out
        _need(mix, torch.float32, "mix", 2); _need(out_w, torch.float32, "out", 1)
        if tuple(mix.shape) != (S, S) or out_w.shape[0] != S or not mix.is_contiguous():
            raise KernelError("hyper_step: the carry matrix is [S, S], the write vector [S]")
        if write.partials is not None:
            part, layout = write.partials.workspace, write.partials._c
        else:
            y = write.y
            _need(y, torch.float32, "y", 2)
            ldy = y.stride(0)
            if write.y_rows is not None:
                y_rows, top = write.y_rows, write.top
                _need(y_rows, torch.int32, "y_rows")
    if out is not None:
        _need(out, None, "out", 2); _need(norm_w, torch.float32, "norm_w", 1)
        if out.shape[1] != E or out.shape[0] < n_rows or norm_w.shape[0] != E or not out.is_contiguous():
            raise KernelError("hyper_step: out must be contiguous [>= rows, E]")
    if in_w is not None:
        _need(in_w, torch.float32, "in_w", 1)
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    global _work
    if _profile is not None:
        _work = (n_rows * E * (4 * S * (2 if write is not None and store else 1) + (4 if y is not None else 0)
                               + (out.element_size() if out is not None else 0)), 0.0)
    _check(lib().ferrum_hyper_step(_ptr(X), c_int(S), c_int(E), _ptr(rows), c_int(n_rows), _ptr(y), c_int(ldy or 0), _ptr(y_rows),
                                   c_int(top), _ptr(part), layout, _ptr(mix), _ptr(out_w), c_int(1 if store and rows is None else 0),
                                   _ptr(in_w), _ptr(norm_w), c_float(eps), _ptr(out),
                                   dtype_code(out.dtype) if out is not None else c_int(0), _stream()), "hyper_step")


# ----------------------------------------------------------------------------- routed feed-forward
MOE_SCORES = {"sigmoid": 0, "softmax": 1}


MOE_MAX_EXPERTS, MOE_MAX_TOP = 256, 8      # (the routing kernel's own limits, which it checks again)


def moe_route(logits, n_tokens, n_exp, top, x, scale_input, expert_of, rank_of, weight_of, counts, xg, row_of, scores="sigmoid",
              renormalize=False, correction=None, weight_scale=1.0, n_identity=0):
    """From the router's float32 logits [T, >= n_exp]: every token's `top` experts and their weights, and the
    tokens' input rows x [T, E] gathered into xg [T * top, E] sorted by expert (times the weight when
    `scale_input`); row_of [T * top] says where each (token, choice) went; counts [n_exp] the rows per expert.
    correction (float32 [n_exp]) is added to the scores for the choice only; the weights are the plain scores times
    weight_scale.  The last n_identity of the n_exp router outputs are identity experts: they get no rows (row_of -1)."""
    global launches
    _need(logits, torch.float32, "logits", 2); _need(x, None, "x", 2); _need(xg, x.dtype, "xg", 2)
    for t in (expert_of, rank_of, counts, row_of):
        _need(t, torch.int32, "routing table")
    _need(weight_of, torch.float32, "weight_of")
    E = x.shape[1]
    if xg.shape[1] != E or xg.shape[0] < n_tokens * top or not xg.is_contiguous() or counts.numel() < n_exp - n_identity:
        raise KernelError("moe_route: buffers are too small")
    if correction is not None:
        _need(correction, torch.float32, "correction", 1)
        if correction.shape[0] != n_exp or not correction.is_contiguous():
            raise KernelError("moe_route: the correction has one number per router output")
    _check(lib().ferrum_moe_route(_ptr(logits), c_int(logits.stride(0)), c_int(n_tokens), c_int(n_exp), c_int(top),
                                  c_int(MOE_SCORES[scores]), c_int(1 if renormalize else 0), _ptr(x), c_int(x.stride(0)), c_int(E),
                                  dtype_code(x.dtype), c_int(1 if scale_input else 0), _ptr(expert_of), _ptr(rank_of),
                                  _ptr(weight_of), _ptr(counts), _ptr(xg), _ptr(row_of), _ptr(correction), c_float(weight_scale),
                                  c_int(n_identity), _stream()), "moe_route")
    launches += 1          # (the entry point launches the routing and the gather)


_moe_tcgen05 = True
MOE_TCGEN05_ROWS_PER_EXPERT = 32      # more rows an expert than this on average: the tcgen05 grouped product


def set_moe_tcgen05(on: bool):
    """Tests and measurements: False keeps the grouped products of many rows on the mma.sync kernel."""
    global _moe_tcgen05
    _moe_tcgen05 = bool(on)


def moe_gemm(a, w, counts, n_rows, out, N, glu=None, err=None, limit=0.0):
    """out[row] = a[row] @ w[expert of row].T over rows sorted by expert (`counts` rows each, on the device).
    w: [n_exp, rows, K]; glu ("silu" / "gelu_tanh"): w holds N gate rows then N up rows per expert and out
    (compute type) gets act(gate) * up; else out is float32 [n_rows, N].  With `err` (the step's error flag) 16-bit
    products of many rows (more than about 32 an expert) run on the tcgen05 kernel, the others on mma.sync tiles
    or, float32 and unaligned rows, on the CUDA cores."""
    _need(a, None, "a", 2); _need(w, a.dtype, "w", 3); _need(out, a.dtype if glu else torch.float32, "out", 2)
    n_exp, w_rows, K = w.shape
    if not w.is_contiguous() or a.shape[1] != K or a.shape[0] < n_rows or out.shape[0] < n_rows or out.shape[1] < N:
        raise KernelError("moe_gemm: shapes do not agree")
    global _work
    if _profile is not None:
        _work = (w.numel() * w.element_size() + n_rows * (K * a.element_size() + N * out.element_size()),
                 2.0 * n_rows * K * N * (2 if glu else 1))
    if (err is not None and _moe_tcgen05 and a.dtype in SIXTEEN_BIT and n_rows > MOE_TCGEN05_ROWS_PER_EXPERT * n_exp and w_rows == (2 * N if glu else N)
            and lib().ferrum_gemm_tc_grouped_supported(_ptr(a), _ptr(w), c_int(n_rows), c_int(n_exp), c_int(K), c_int(a.stride(0)))):
        _check(lib().ferrum_gemm_tc_grouped(_ptr(a), _ptr(w), _ptr(out), dtype_code(a.dtype), c_int(n_rows), c_int(a.shape[0]), c_int(N),
                                            c_int(K), c_int(a.stride(0)), c_int(out.stride(0)), c_int(n_exp), c_int(w_rows), _ptr(counts),
                                            c_int(1 + GLU_ACTS[glu] if glu else 0), _ptr(err), c_float(limit), _stream()), "moe_gemm")
        return
    _check(lib().ferrum_moe_gemm(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w_rows), c_int(K), c_int(N), c_int(n_exp), _ptr(counts),
                                 c_int(n_rows), dtype_code(a.dtype), c_int(1 if glu else 0), c_int(GLU_ACTS[glu] if glu else 0), c_float(limit),
                                 _ptr(out), c_int(out.stride(0)), _stream()), "moe_gemm")


def set_moe_cuda_cores(on: bool):
    """Tests and measurements: send 16-bit grouped products to the CUDA-core kernel too."""
    lib().ferrum_moe_cuda_cores(c_int(1 if on else 0))


def moe_combine(rows, row_of, top, n_tokens, y, weight_of=None, x=None, add=None):
    """y[t] = sum_j rows[row_of[t, j]] (times weight_of[t, j] when given), float32.  x [T, E] (any type): the tokens'
    own input rows, which stand in for choices without a row (row_of < 0: identity experts); add (float32 [T, E]): rows
    that join the sum last."""
    _need(rows, torch.float32, "rows", 2); _need(y, torch.float32, "y", 2); _need(row_of, torch.int32, "row_of")
    E = y.shape[1]
    if not y.is_contiguous() or rows.shape[1] < E:
        raise KernelError("moe_combine: shapes do not agree")
    if x is not None:
        _need(x, None, "x", 2)
    if add is not None:
        _need(add, torch.float32, "add", 2)
    if (x is not None and x.shape[1] < E) or (add is not None and add.shape[1] < E):
        raise KernelError("moe_combine: shapes do not agree")
    _check(lib().ferrum_moe_combine(_ptr(rows), c_int(rows.stride(0)), _ptr(row_of), _ptr(weight_of), c_int(top), c_int(n_tokens),
                                    c_int(E), _ptr(y), _ptr(x), c_int(x.stride(0) if x is not None else 0),
                                    dtype_code(x.dtype) if x is not None else c_int(F32), _ptr(add),
                                    c_int(add.stride(0) if add is not None else 0), _stream()), "moe_combine")


def softcap(x, n_rows, cap):
    """x[:n_rows] <- cap * tanh(x / cap) in place (float32)."""
    _need(x, torch.float32, "x", 2)
    _check(lib().ferrum_softcap(_ptr(x), c_int(x.stride(0)), c_int(n_rows), c_int(x.shape[1]), c_float(cap), _stream()), "softcap")


# ----------------------------------------------------------------------------- norms on the sublayers' results
def post_norm_add(h, n_tokens, y=None, w=None, ls=None, eps=0.0, xc=None):
    """h[:n] += ls * (y / sqrt(mean(y^2) + eps) * w), all float32 (ls: a per-element layer scale or None); xc (a
    compute-type buffer or None) receives the new rows.  Without y only that copy is made."""
    _need(h, torch.float32, "h", 2)
    E = h.shape[1]
    if not h.is_contiguous():
        raise KernelError("post_norm_add: the residual rows must be contiguous")
    if y is not None:
        _need(y, torch.float32, "y", 2); _need(w, torch.float32, "w", 1)
        if y.shape[1] < E or w.shape[0] != E or (ls is not None and (ls.dtype != torch.float32 or ls.shape[0] != E)):
            raise KernelError("post_norm_add: shapes do not agree")
    if xc is not None:
        _need(xc, None, "xc", 2)
        if xc.shape[1] < E:
            raise KernelError("post_norm_add: shapes do not agree")
    _bytes_work((h, 2 * n_tokens), (y, n_tokens), (xc, n_tokens))
    _check(lib().ferrum_post_norm_add(_ptr(h), c_int(E), _ptr(y), c_int(y.stride(0) if y is not None else 0), _ptr(w), _ptr(ls),
                                      c_float(eps), _ptr(xc), c_int(xc.stride(0) if xc is not None else 0),
                                      dtype_code(xc.dtype) if xc is not None else c_int(F32), c_int(n_tokens), _stream()),
           "post_norm_add")


def dual_norm_mean(a, b, wa, wb, eps, out, n_tokens):
    """out[:n] = (rms(a) * wa + rms(b) * wb) / 2 with rms(v) = v / sqrt(mean(v^2) + eps), all float32 [T, E]."""
    for t, n in ((a, "a"), (b, "b"), (out, "out")):
        _need(t, torch.float32, n, 2)
    E = out.shape[1]
    _need(wa, torch.float32, "wa", 1); _need(wb, torch.float32, "wb", 1)
    if a.shape[1] < E or b.shape[1] < E or wa.shape[0] != E or wb.shape[0] != E:
        raise KernelError("dual_norm_mean: shapes do not agree")
    _bytes_work((a, n_tokens), (b, n_tokens), (out, n_tokens))
    _check(lib().ferrum_dual_norm_mean(_ptr(a), c_int(a.stride(0)), _ptr(b), c_int(b.stride(0)), _ptr(wa), _ptr(wb), c_float(eps),
                                       c_int(E), _ptr(out), c_int(out.stride(0)), c_int(n_tokens), _stream()), "dual_norm_mean")


def head_gate_norm(o, gate, w, eps, n_tokens, H, Dv, out):
    """out[t, h] = rms(o[t, h]) * w * sigmoid(gate[t, h]) per head of Dv elements, rounded once to out's type.  o, gate:
    float32 rows (gate may be a view into wider rows, or None); w: float32 [Dv] (one for all heads) or [H * Dv]."""
    _need(o, torch.float32, "o", 2); _need(out, None, "out", 2); _need(w, torch.float32, "w", 1)
    if gate is not None:
        _need(gate, torch.float32, "gate", 2)
    if w.shape[0] not in (Dv, H * Dv) or o.shape[1] < H * Dv or out.shape[1] < H * Dv:
        raise KernelError("head_gate_norm: shapes do not agree")
    _bytes_work((o, n_tokens), (gate, n_tokens), (out, n_tokens))
    _check(lib().ferrum_head_gate_norm(_ptr(o), c_int(o.stride(0)), _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
                                       _ptr(w), c_int(1 if w.shape[0] == H * Dv and H > 1 else 0), c_float(eps), c_int(n_tokens),
                                       c_int(H), c_int(Dv), _ptr(out), c_int(out.stride(0)), dtype_code(out.dtype), _stream()),
           "head_gate_norm")


# ----------------------------------------------------------------------------- recurrent mixers with a matrix per head
DELTA_MAX_TAPS, RECURRENT_MAX_DIM = 16, 256      # (the kernels' own limits, which they check again)


def delta_rule(proj, logit, n_tokens, ctx, conv_w, dt_bias, a_log, H, G, D, Dv, state, qkv, dec, o):
    """Everything of the gated delta rule between its products: short convolution + silu over q, k, v (its last
    inputs kept in the request's state row), unit norm of q and k, the decays, the walk over the tokens.
    proj: float32 rows [q: G D | k: G D | v: H Dv | beta logits: H]; logit: float32 rows [H D] (decay logits before
    dt_bias); state: float32 [max_requests, H D Dv + (taps - 1) C]; qkv [T, C], dec [T, H D + H]: float32 scratch;
    o: float32 [T, H Dv]."""
    global launches
    _need(proj, torch.float32, "proj", 2); _need(logit, torch.float32, "logit", 2); _need(state, torch.float32, "state", 2)
    _need(o, torch.float32, "o", 2)
    C = 2 * G * D + H * Dv
    taps = conv_w.shape[1]
    for t, n in ((conv_w, "conv_w"), (dt_bias, "dt_bias"), (a_log, "a_log")):
        _need(t, torch.float32, n)
    if (conv_w.shape[0] != C or not conv_w.is_contiguous() or dt_bias.numel() != H * D or a_log.numel() != H
            or state.shape[1] != H * D * Dv + (taps - 1) * C or qkv.numel() < n_tokens * C or dec.numel() < n_tokens * (H * D + H)):
        raise KernelError("delta_rule: shapes do not agree")
    if _profile is not None:
        global _work
        _work = (4 * (n_tokens * (2 * C + 2 * H * D + H * Dv) + 2 * ctx.n_reqs * H * D * Dv), 6.0 * n_tokens * H * D * Dv)
    _check(lib().ferrum_delta_rule(_ptr(proj), c_int(proj.stride(0)), _ptr(logit), c_int(logit.stride(0)), c_int(n_tokens),
                                   c_int(ctx.n_reqs), _ptr(ctx.req_of_token), _ptr(ctx.q_start), _ptr(ctx.slots), _ptr(conv_w),
                                   c_int(taps), _ptr(dt_bias), _ptr(a_log), c_int(H), c_int(G), c_int(D), c_int(Dv), _ptr(state),
                                   c_longlong(state.stride(0)), _ptr(qkv), _ptr(dec), _ptr(o), c_int(o.stride(0)), c_int(ctx.max_q_len), _stream()),
           "delta_rule")
    launches += 2 if taps > 1 else 1       # (the entry point launches the preparation, the convolution's state and the walk)


def matrix_memory_state_size(H, D, Dv):
    """Floats of a request's state row: S [H, D, Dv] and, per eight value columns, a copy of n [H, D] and m [H] (the
    kernel's own layout: it is asked when the library is there, so that a cache layout can also be made without it)."""
    if _lib is not None:
        return int(_lib.ferrum_matrix_memory_state_floats(c_int(H), c_int(D), c_int(Dv)))
    return H * D * Dv + ((Dv + 7) // 8) * (H * D + H)


def matrix_memory(proj, offsets, bias_i, bias_f, cap, n_tokens, ctx, H, D, Dv, state, gates, o):
    """The walk of the matrix-memory recurrence (see csrc/kernels/matrix_memory.cu).  proj: float32 rows holding q, k,
    v and the two gates' logits at `offsets` = (q, k, v, i, f); state: float32 [max_requests, matrix_memory_state_size];
    gates: float32 scratch of T * 2 H elements; o: float32 [T, H Dv]."""
    global launches
    _need(proj, torch.float32, "proj", 2); _need(state, torch.float32, "state", 2); _need(o, torch.float32, "o", 2)
    _need(gates, torch.float32, "gates")
    if gates.numel() < n_tokens * 2 * H:
        raise KernelError("matrix_memory: the gates' scratch is too small")
    _need(bias_i, torch.float32, "bias_i", 1); _need(bias_f, torch.float32, "bias_f", 1)
    oq, ok, ov, oi, of = (int(v) for v in offsets)
    if (bias_i.shape[0] != H or bias_f.shape[0] != H or state.shape[1] != matrix_memory_state_size(H, D, Dv)
            or proj.shape[1] < max(oq + H * D, ok + H * D, ov + H * Dv, oi + H, of + H)):
        raise KernelError("matrix_memory: shapes do not agree")
    if _profile is not None:
        global _work
        _work = (4 * (n_tokens * (2 * H * D + 2 * H * Dv) + 2 * ctx.n_reqs * H * D * Dv), 4.0 * n_tokens * H * D * Dv)
    _check(lib().ferrum_matrix_memory(_ptr(proj), c_int(proj.stride(0)), c_int(oq), c_int(ok), c_int(ov), c_int(oi), c_int(of),
                                      _ptr(bias_i), _ptr(bias_f), c_float(cap), c_int(n_tokens), c_int(ctx.n_reqs), _ptr(ctx.q_start),
                                      _ptr(ctx.slots), c_int(H), c_int(D), c_int(Dv), _ptr(state), c_longlong(state.stride(0)),
                                      _ptr(gates), _ptr(o), c_int(o.stride(0)), _stream()), "matrix_memory")
    launches += 1          # (the entry point launches the gates and the walk)
