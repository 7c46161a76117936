"""Python launchers of the hand-written CUDA kernels (ctypes over the libraries csrc/build.py makes).

Tensors are torch tensors used as plain device memory: every launcher checks device, dtype and
layout, passes raw pointers and the current CUDA stream, and turns a non-zero status into a
`KernelError`.  Nothing here computes: if a library cannot be built or loaded the call raises;
there is no CPU or library-op fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_uint64, c_void_p
from typing import Optional, Tuple

import torch

from .csrc import build

DT_F32, DT_BF16 = 0, 1
_STATUS = {-1: "unsupported dtype", -2: "unsupported shape", -3: "misaligned pointer or stride",
           -4: "size beyond the kernel's limit", -5: "device-side wait ran out"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """Kernel launches made through this module since import (launch counting for measurements)."""
    return _launches


def count_launches(n: int) -> None:
    """Account for launches made on this module's behalf elsewhere (a replayed CUDA graph)."""
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")
    raise KernelError(f"{what}: CUDA error {status} (cudaError_t)")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return DT_F32
    if dt == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)     # the short way to the stream's handle
_device_index: Optional[int] = None


def _stream() -> c_void_p:
    """The current stream of the current device (under a graph capture: the capturing stream).  Asked for at
    every launch, so by the shortest route torch offers."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (no CPU path exists)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_sigs_done = set()
_profile: Optional[list] = None          # (function name, start event, end event) per launch while profiling


def profile_start() -> None:
    """From now on every launch made through this module is bracketed by two CUDA events (for launch-by-launch
    runs; launches replayed inside a CUDA graph are not seen)."""
    global _profile
    _profile = []


def profile_report():
    """Stop profiling; [(function, calls, seconds on the device)] sorted by time, the reference's per-kind
    totals (stratum/native/stratum_arch_llama.inc.c:2081-2091) with kernels in place of weight types."""
    global _profile
    rows, _profile = _profile or [], None
    torch.cuda.synchronize()
    totals = {}
    for name, e0, e1 in rows:
        calls, secs = totals.get(name, (0, 0.0))
        totals[name] = (calls + 1, secs + e0.elapsed_time(e1) * 1e-3)
    return sorted(((n, c, t) for n, (c, t) in totals.items()), key=lambda r: -r[2])


class _Timed:
    """A launcher whose calls are bracketed by events while profiling is on."""
    __slots__ = ("f", "name")

    def __init__(self, f, name):
        self.f, self.name = f, name

    def __call__(self, *args):
        if _profile is None:
            return self.f(*args)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        status = self.f(*args)
        e1.record()
        _profile.append((self.name, e0, e1))
        return status


_timed = {}


def _fn(libname: str, fname: str, argtypes):
    key = (libname, fname)
    t = _timed.get(key)
    if t is None:
        lib = build.load(libname)
        f = getattr(lib, fname)
        f.argtypes = argtypes
        f.restype = c_int
        t = _timed[key] = _Timed(f, fname.replace("stratum_", "", 1))
    return t if _profile is not None else t.f


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] as float32.  table [V,H] float32|bfloat16, ids int32 [T], out float32 [T,H]."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    f = _fn("elementwise", "stratum_embed_gather",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), ids.numel(), table.shape[1],
             table.shape[0], _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * gain.  x float32 [*,H], gain float32 [H]."""
    _need(x, "x", torch.float32); _need(gain, "gain", torch.float32); _need(out, "out")
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("rmsnorm: rows and out disagree")
    elif x.shape[0] != n_rows:
        raise KernelError("rmsnorm: x and out disagree")
    f = _fn("elementwise", "stratum_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(x), _ptr(gain), _ptr(rows), _ptr(out), dtype_code(out.dtype), n_rows, x.shape[-1],
             c_float(eps), _stream()), "rmsnorm")


def rmsnorm_heads(x: torch.Tensor, first_col: int, n_heads: int, head_dim: int, gain: torch.Tensor,
                  eps: float) -> None:
    """In place, in every row of x [T, width]: each of the n_heads stretches of head_dim values from column
    first_col on becomes rmsnorm(stretch) * gain.  gain float32 [head_dim]."""
    _need(x, "x", contiguous=False); _need(gain, "gain", torch.float32)
    if x.dim() != 2 or x.stride(1) != 1 or first_col < 0 or first_col + n_heads * head_dim > x.shape[1]:
        raise KernelError("rmsnorm_heads: the heads do not lie inside the rows of x")
    if gain.numel() != head_dim:
        raise KernelError("rmsnorm_heads: gain and head_dim disagree")
    f = _fn("elementwise", "stratum_rmsnorm_heads",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p])
    _check(f(_ptr(x), dtype_code(x.dtype), x.shape[0], x.stride(0), first_col, n_heads, head_dim, _ptr(gain),
             c_float(eps), _stream()), "rmsnorm_heads")


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> None:
    """out[r][j] = silu(gu[r][2j]) * gu[r][2j+1]."""
    _need(gu, "gu"); _need(out, "out", gu.dtype)
    f = _fn("elementwise", "stratum_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gu), _ptr(out), dtype_code(gu.dtype), out.shape[0], out.shape[1], _stream()), "swiglu")


def rope_store(qkv: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
               block_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], interleaved: bool,
               mscale: float, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
               n_q: int, n_kv: int, head_dim: int, page_tokens: int, write_cache: bool) -> None:
    """Rotate q (in place) and k, and store k and v into the paged cache."""
    _need(qkv, "qkv"); _need(token_pos, "token_pos", torch.int32); _need(token_seq, "token_seq", torch.int32)
    n_pairs = 0 if inv_freq is None else inv_freq.numel()
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
    if write_cache:
        _need(k_cache, "k_cache", qkv.dtype); _need(v_cache, "v_cache", qkv.dtype)
        _need(block_table, "block_table", torch.int32)
    if qkv.shape[-1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError("rope_store: qkv width is not (n_q + 2 n_kv) * head_dim")
    f = _fn("elementwise", "stratum_rope_store",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), dtype_code(qkv.dtype), _ptr(token_pos), _ptr(token_seq), _ptr(block_table),
             0 if block_table is None else block_table.stride(0), _ptr(inv_freq), n_pairs, int(interleaved),
             c_float(mscale), _ptr(k_cache), _ptr(v_cache), qkv.shape[0], n_q, n_kv, head_dim, page_tokens,
             int(write_cache), _stream()), "rope_store")


def rope_table(token_pos: torch.Tensor, inv_freq: torch.Tensor, mscale: float, out: torch.Tensor) -> None:
    """out[t][k] = mscale * (cos, sin)((float)pos[t] * inv_freq[k]): float32 [tokens, pairs, 2], once per step, for
    the matrix-product epilogues that rotate queries and keys."""
    _need(token_pos, "token_pos", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _need(out, "out", torch.float32)
    if tuple(out.shape) != (token_pos.numel(), inv_freq.numel(), 2):
        raise KernelError("rope_table: out must be [tokens, pairs, 2]")
    f = _fn("elementwise", "stratum_rope_table", [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(token_pos), _ptr(inv_freq), c_float(mscale), _ptr(out), token_pos.numel(), inv_freq.numel(),
             _stream()), "rope_table")


def fill_normal(out: torch.Tensor, seed: int, std: float) -> None:
    """Fill with std * N(0,1) from a counter-based generator keyed by (seed, element index)."""
    _need(out, "out")
    f = _fn("elementwise", "stratum_fill_normal", [c_void_p, c_int, c_size_t, c_uint64, c_float, c_void_p])
    _check(f(_ptr(out), dtype_code(out.dtype), out.numel(), c_uint64(seed & (2**64 - 1)), c_float(std),
             _stream()), "fill_normal")


# ------------------------------------------------------------------ linear (any shape, CUDA cores)
EPI_STORE, EPI_ADD_F32, EPI_STORE_F32, EPI_SWIGLU = 0, 1, 2, 3
EPI_ADD_F32_EMIT, EPI_QKV_ROPE = 4, 5          # gemm_tc only: see GemmExtra


def linear_simple(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  epilogue: int) -> None:
    """out (=|+=) x @ w.T + bias.  x [M,K] and w [N,K] of one dtype; bias float32; see EPI_*."""
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(out, "out", contiguous=False)
    if x.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError("linear: rows must be contiguous")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    want = x.dtype if epilogue == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"linear: epilogue {epilogue} writes {want}, out is {out.dtype}")
    f = _fn("linear_simple", "stratum_linear_simple",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), dtype_code(x.dtype), epilogue, M, N, K, x.stride(0),
             out.stride(0), _stream()), "linear_simple")


def _linear_shapes(x, w, bias, out, epilogue, what):
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(out, "out", contiguous=False)
    if x.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError(f"{what}: rows must be contiguous")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    M, Kd = x.shape
    N = w.shape[0]
    width = N // 2 if epilogue == EPI_SWIGLU else N
    if w.shape[1] != Kd or out.shape[0] != M or out.shape[1] != width:
        raise KernelError(f"{what}: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    want = x.dtype if epilogue in (EPI_STORE, EPI_SWIGLU) else torch.float32
    if out.dtype != want:
        raise KernelError(f"{what}: epilogue {epilogue} writes {want}, out is {out.dtype}")
    return M, N, Kd


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                epilogue: int) -> None:
    """bfloat16, at most 32 rows of x: the weight-streaming tensor-core kernel (see EPI_*)."""
    M, N, Kd = _linear_shapes(x, w, bias, out, epilogue, "gemm_skinny")
    _need(x, "x", torch.bfloat16, contiguous=False)
    f = _fn("gemm_skinny", "stratum_gemm_skinny",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), epilogue, M, N, Kd, x.stride(0), out.stride(0), _stream()),
           "gemm_skinny")


_scratch_epoch = 0


def scratch_epoch() -> int:
    """Grows whenever a scratch buffer that kernels are given is replaced by a larger one (the old one is freed).
    A captured CUDA graph recorded the old address: whoever replays graphs compares this number with the one
    at capture and captures again when it has moved."""
    return _scratch_epoch


def scratch_regrown() -> None:
    global _scratch_epoch
    _scratch_epoch += 1


_status_word: Optional[torch.Tensor] = None


def status_word() -> torch.Tensor:
    """One int32 on the device that kernels with bounded waits write to when a wait runs out."""
    global _status_word
    if _status_word is None:
        _status_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status_word


def check_status() -> None:
    """Synchronise and raise if a kernel gave up a wait (the word is cleared for the next run)."""
    if _status_word is None:
        return
    code = int(_status_word.item())
    if code != 0:
        _status_word.zero_()
        where = {101: "the TMA producer waiting for a free stage", 102: "the MMA warp waiting for a free accumulator",
                 103: "the MMA warp waiting for a loaded stage", 104: "the epilogue waiting for an accumulator"}
        raise KernelError(f"a device-side wait ran out in {where.get(code, f'code {code}')}; results are invalid")


_gemm_scratch = None


def _gemm_tc_scratch(device):
    """float32 scratch for the partial tiles of tiles that several CTAs share."""
    global _gemm_scratch
    if _gemm_scratch is None or _gemm_scratch.device != device:
        lib = build.load("gemm_tc")
        lib.stratum_gemm_tc_scratch_floats.restype = ctypes.c_longlong
        _gemm_scratch = torch.empty(int(lib.stratum_gemm_tc_scratch_floats()), dtype=torch.float32, device=device)
        scratch_regrown()
    return _gemm_scratch


class _EpiExtra(ctypes.Structure):
    """Mirror of struct EpiExtra in csrc/gemm_tc.cu (pointers first, then 4-byte fields)."""
    _fields_ = [("norm_ss", c_void_p), ("emit_x", c_void_p), ("emit_gain", c_void_p), ("emit_ss", c_void_p),
                ("rope_cs", c_void_p), ("token_pos", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("norm_parts", c_int), ("norm_ld", c_int), ("norm_size", c_float), ("norm_eps", c_float),
                ("emit_ldx", c_int), ("emit_ld", c_int),
                ("rope_pairs", c_int), ("bt_stride", c_int), ("n_q", c_int), ("n_kv", c_int), ("head_dim", c_int),
                ("page_tokens", c_int), ("write_cache", c_int), ("reserved", c_int)]


class GemmExtra:
    """What a gemm_tc call does beyond its basic epilogue (all optional):

    scaled rows   norm_ss float32 [parts, rows] partial sums of squares of the rows a norm handed over as
                  r * gain: the product's rows are multiplied by 1 / sqrt(sum / norm_size + norm_eps);
    EPI_ADD_F32_EMIT   emit_x bfloat16 [rows, N] receives bf16(new residual * emit_gain), emit_ss float32
                  [parts, rows] the sums of squares of the new residual values per tile of columns (how many
                  parts were written: `last_parts()` after the call);
    EPI_QKV_ROPE  the columns are query, key and value heads (pairs of rotated dimensions neighbours): queries
                  are rotated and stored to `out`, keys rotated and written, values written, into the paged cache.
    """

    def __init__(self):
        self.c = _EpiExtra()
        self.keep = []                      # tensors whose memory the struct points into

    def scaled_rows(self, norm_ss: torch.Tensor, parts: int, size: int, eps: float) -> "GemmExtra":
        _need(norm_ss, "norm_ss", torch.float32)
        if norm_ss.dim() != 2 or norm_ss.shape[0] < parts:
            raise KernelError("gemm_tc: norm_ss must be [parts or more, rows]")
        self.c.norm_ss, self.c.norm_parts, self.c.norm_ld = norm_ss.data_ptr(), parts, norm_ss.stride(0)
        self.c.norm_size, self.c.norm_eps = float(size), float(eps)
        self.keep.append(norm_ss)
        return self

    def emit(self, emit_x: torch.Tensor, gain: torch.Tensor, emit_ss: torch.Tensor) -> "GemmExtra":
        _need(emit_x, "emit_x", torch.bfloat16); _need(gain, "gain", torch.float32)
        _need(emit_ss, "emit_ss", torch.float32)
        self.c.emit_x, self.c.emit_gain, self.c.emit_ss = emit_x.data_ptr(), gain.data_ptr(), emit_ss.data_ptr()
        self.c.emit_ldx, self.c.emit_ld = emit_x.stride(0), emit_ss.stride(0)
        self.keep += [emit_x, gain, emit_ss]
        return self

    def qkv_rope(self, rope_cs: Optional[torch.Tensor], token_pos: torch.Tensor, token_seq: torch.Tensor,
                 block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                 v_cache: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int, page_tokens: int,
                 write_cache: bool) -> "GemmExtra":
        _need(token_pos, "token_pos", torch.int32); _need(token_seq, "token_seq", torch.int32)
        if rope_cs is not None:
            _need(rope_cs, "rope_cs", torch.float32)
            if rope_cs.dim() != 3 or rope_cs.shape[0] != token_pos.numel() or rope_cs.shape[2] != 2:
                raise KernelError("gemm_tc: rope_cs must be [rows, pairs, 2]")
            self.c.rope_cs, self.c.rope_pairs = rope_cs.data_ptr(), rope_cs.shape[1]
        if write_cache:
            _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
            _need(block_table, "block_table", torch.int32, contiguous=False)
            self.c.k_cache, self.c.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
            self.c.block_table, self.c.bt_stride = block_table.data_ptr(), block_table.stride(0)
        self.c.token_pos, self.c.token_seq = token_pos.data_ptr(), token_seq.data_ptr()
        self.c.n_q, self.c.n_kv, self.c.head_dim, self.c.page_tokens = n_q, n_kv, head_dim, page_tokens
        self.c.write_cache = int(bool(write_cache))
        self.keep += [rope_cs, token_pos, token_seq, block_table, k_cache, v_cache]
        return self


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            epilogue: int, extra: Optional[GemmExtra] = None) -> int:
    """bfloat16 matrix product on the 5th-generation tensor cores (TMA + tcgen05/TMEM); see EPI_* and GemmExtra.
    The form (k shared inside clusters, stream-K, tiles, tiles on pairs of CTAs) is chosen from the shapes in
    gemm_tc.cu.  Returns the number of parts written per row with EPI_ADD_F32_EMIT (else 0)."""
    basic = {EPI_ADD_F32_EMIT: EPI_ADD_F32, EPI_QKV_ROPE: EPI_STORE}.get(epilogue, epilogue)
    M, N, Kd = _linear_shapes(x, w, bias, out, basic, "gemm_tc")
    _need(x, "x", torch.bfloat16, contiguous=False)
    if epilogue in (EPI_ADD_F32_EMIT, EPI_QKV_ROPE) and extra is None:
        raise KernelError("gemm_tc: this epilogue needs a GemmExtra")
    part = _gemm_tc_scratch(x.device)
    lib = build.load("gemm_tc")
    f = _fn("gemm_tc", "stratum_gemm_tc_ex",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), epilogue, M, N, Kd, x.stride(0), out.stride(0),
             _ptr(status_word()), _ptr(part), None if extra is None else ctypes.addressof(extra.c), _stream()),
           "gemm_tc")
    count_launches(lib.stratum_gemm_tc_last_launches() - 1)      # a second pass, if there was one
    return int(lib.stratum_gemm_tc_last_parts()) if epilogue == EPI_ADD_F32_EMIT else 0


def gemm_tc_last_form() -> Tuple[str, int]:
    """The form the last gemm_tc call took, for tests:
    ("tiles" | "pairs" | "pairs-shared" | "stream-k" | "cluster-k", cluster size)."""
    code = int(build.load("gemm_tc").stratum_gemm_tc_last_form())
    return {1: "tiles", 2: "pairs", 3: "stream-k", 4: "cluster-k", 5: "pairs-shared"}.get(code % 16, "none"), code // 16


# ------------------------------------------------------------------ attention (any sizes, CUDA cores)
def attention_simple(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                     token_seq: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, page_tokens: int, window: int, scale: float) -> None:
    """Causal GQA attention of every token of the step over its sequence's cached keys."""
    _need(qkv, "qkv"); _need(k_cache, "k_cache", qkv.dtype); _need(v_cache, "v_cache", qkv.dtype)
    _need(out, "out", qkv.dtype); _need(block_table, "block_table", torch.int32)
    f = _fn("attention_simple", "stratum_attention_simple",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), dtype_code(qkv.dtype), _ptr(token_pos),
             _ptr(token_seq), _ptr(block_table), block_table.stride(0), _ptr(out), out.stride(0), qkv.shape[0],
             n_q, n_kv, head_dim, page_tokens, window, c_float(scale), _stream()), "attention_simple")


def attention_mma(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                  token_seq: torch.Tensor, block_table: torch.Tensor, qblocks, tokens_per_block: int,
                  out: torch.Tensor, part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], n_q: int,
                  n_kv: int, head_dim: int, page_tokens: int, window: int, scale: float, n_splits: int,
                  chunk: int) -> None:
    """bfloat16 tensor-core attention over the paged cache.  qblocks: None (one token per sequence, block i is
    sequence i) or (seq, first row, tokens) int32 tensors of equal length.  n_splits > 1 needs scratch:
    part_o float32 [tokens*n_q*n_splits*head_dim], part_ml float32 [tokens*n_q*n_splits*2]."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    n_tokens = qkv.shape[0]
    if qblocks is None:
        qs = qt = qn = None
        n_qb = n_tokens
    else:
        qs, qt, qn = qblocks
        n_qb = qs.numel()
    if n_splits > 1:
        need = n_tokens * n_q * n_splits
        _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
            raise KernelError("attention_mma: scratch too small for the splits")
    f = _fn("attention_mma", "stratum_attention_mma",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
             _ptr(block_table), block_table.stride(0), _ptr(qs), _ptr(qt), _ptr(qn), n_qb, tokens_per_block,
             _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), n_tokens, n_q, n_kv, head_dim, page_tokens,
             window, c_float(scale), n_splits, chunk, _stream()), "attention_mma")
    if n_splits > 1:
        count_launches(1)          # the merge kernel


def attention_tile(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                   token_seq: torch.Tensor, block_table: torch.Tensor, qblocks, tokens_per_warp: int,
                   out: torch.Tensor, n_q: int, n_kv: int, head_dim: int, page_tokens: int, window: int,
                   scale: float) -> None:
    """bfloat16 tensor-core attention for prompts: query tiles of 4 * tokens_per_warp tokens share their key
    tiles through shared memory.  qblocks: (seq, first row, tokens) int32 tensors, tokens <= 4 * tokens_per_warp."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    qs, qt, qn = qblocks
    f = _fn("attention_mma", "stratum_attention_tile",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
             _ptr(block_table), block_table.stride(0), _ptr(qs), _ptr(qt), _ptr(qn), qs.numel(), tokens_per_warp,
             _ptr(out), out.stride(0), qkv.shape[0], n_q, n_kv, head_dim, page_tokens, window, c_float(scale),
             _stream()), "attention_tile")


def attention_tc(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                 block_table: torch.Tensor, qblocks, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                 page_tokens: int, window: int, scale: float, halves: int = 1) -> None:
    """bfloat16 attention for prompts on tcgen05/TMEM: query tiles of halves * 128 / (n_q / n_kv) tokens (qblocks
    as for attention_tile).  halves 2: a CTA owns 256 query rows whose two halves share every key and value tile.
    head_dim 64 or 128, group size dividing 128, pages of 64 tokens."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    qs, qt, qn = qblocks
    f = _fn("attention_tc", "stratum_attention_tc",
            [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
             c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(token_pos),
             _ptr(block_table), block_table.stride(0), _ptr(qs), _ptr(qt), _ptr(qn), qs.numel(), _ptr(out),
             out.stride(0), qkv.shape[0], n_q, n_kv, head_dim, page_tokens, window, c_float(scale), halves,
             _ptr(status_word()), _stream()), "attention_tc")


_stream_scratch = None


def attention_stream(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                     token_seq: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, page_tokens: int, window: int, scale: float, late_trigger: bool = True,
                     whole_pages: bool = False) -> None:
    """bfloat16 attention for decode steps (one new token per sequence, row i of qkv): the pages of all
    sequences are spread evenly over the SMs and streamed by TMA.  head_dim 64 or 128, at most 8 query heads per
    kv head, pages of 64 tokens, at most 1024 sequences.  late_trigger: a CTA that has asked for its last page lets
    the kernels after this one start (they then wait on the SMs for this one to end).  whole_pages (head_dim 64):
    eight warps take whole pages in turn, instead of four warps a quarter of every page."""
    global _stream_scratch
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32, contiguous=False)
    gs = n_q // max(n_kv, 1)
    if _stream_scratch is None or _stream_scratch[0] < gs * (head_dim + 2) or _stream_scratch[1].device != qkv.device:
        lib = build.load("attention_stream")
        lib.stratum_attention_stream_scratch_floats.restype = ctypes.c_longlong
        floats = int(lib.stratum_attention_stream_scratch_floats(max(gs, 8), max(head_dim, 128)))
        _stream_scratch = (max(gs, 8) * (max(head_dim, 128) + 2),
                           torch.empty(floats, dtype=torch.float32, device=qkv.device))
        scratch_regrown()
    f = _fn("attention_stream", "stratum_attention_stream",
            [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(token_pos),
             _ptr(token_seq), _ptr(block_table), block_table.stride(0), _ptr(out), out.stride(0), qkv.shape[0],
             n_q, n_kv, head_dim, page_tokens, window, c_float(scale), int(bool(late_trigger)),
             int(bool(whole_pages)), _ptr(_stream_scratch[1]),
             _ptr(status_word()),
             _stream()), "attention_stream")
    count_launches(1)


# ------------------------------------------------------------------ sampling
ARGMAX_SPLITS = 32
_argmax_scratch = None


def _argmax_scratch_for(rows: int, device):
    """(best values, best ids, counters) for the many-blocks-per-row argmax; the counters start at zero and
    every launch leaves them at zero."""
    global _argmax_scratch
    if _argmax_scratch is None or _argmax_scratch[2].numel() < rows:
        n = max(rows, 64)
        _argmax_scratch = (torch.empty(n * ARGMAX_SPLITS, dtype=torch.float32, device=device),
                           torch.empty(n * ARGMAX_SPLITS, dtype=torch.int32, device=device),
                           torch.zeros(n, dtype=torch.int32, device=device))
        scratch_regrown()
    return _argmax_scratch


def argmax(logits: torch.Tensor, ids: torch.Tensor, values: Optional[torch.Tensor] = None) -> None:
    """ids[r] = index of the largest logit of row r, the lowest index among equals."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(ids, "ids", torch.int32)
    if values is not None:
        _need(values, "values", torch.float32)
    pv, pi, cnt = _argmax_scratch_for(logits.shape[0], logits.device)
    f = _fn("sampling", "stratum_argmax",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(ids), _ptr(values),
             _ptr(pv), _ptr(pi), _ptr(cnt), _stream()), "argmax")


def feed_ids(ids: torch.Tensor, feed: torch.Tensor, prev: torch.Tensor) -> None:
    """ids[i] = prev[feed[i]] where feed[i] >= 0 (int32 tensors on the device): picked ids fed back without the host."""
    _need(ids, "ids", torch.int32); _need(feed, "feed", torch.int32); _need(prev, "prev", torch.int32)
    if feed.numel() != ids.numel():
        raise KernelError("feed_ids: ids and feed disagree")
    f = _fn("sampling", "stratum_feed_ids", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(feed), _ptr(prev), ids.numel(), _stream()), "feed_ids")


SAMPLE_SPLITS, SAMPLE_KEEP = 32, 64
_sample_scratch = None


def _sample_scratch_for(rows: int, device):
    """What the many-blocks-per-row sampling kernel leaves between its two stages (per row: the stretches' best
    logits, ids, sums and last kept keys, their lists of candidates, a counter that starts at zero and is left
    at zero, a mark for the one-block kernel)."""
    global _sample_scratch
    if _sample_scratch is None or _sample_scratch[6].numel() < rows:
        n = max(rows, 64)
        f32, i32 = torch.float32, torch.int32
        _sample_scratch = (torch.empty(n * SAMPLE_SPLITS, dtype=f32, device=device),
                           torch.empty(n * SAMPLE_SPLITS, dtype=i32, device=device),
                           torch.empty(n * SAMPLE_SPLITS * 8, dtype=f32, device=device),
                           torch.empty(n * SAMPLE_SPLITS, dtype=i32, device=device),
                           torch.empty(n * SAMPLE_SPLITS * SAMPLE_KEEP, dtype=f32, device=device),
                           torch.empty(n * SAMPLE_SPLITS * SAMPLE_KEEP, dtype=i32, device=device),
                           torch.zeros(n, dtype=i32, device=device),
                           torch.zeros(n, dtype=i32, device=device))
        scratch_regrown()
    return _sample_scratch


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, ids: torch.Tensor, values: Optional[torch.Tensor] = None,
           one_block_per_row: bool = False) -> None:
    """Per row: temperature <= 0 greedy, else a draw by `uniform` from exp((l - max) / T), optionally among the
    top_k largest (0: off, at most 512) cut after the prefix that reaches top_p (1: off).  Rows of 8,192 logits
    or more are cut over 32 blocks each (one_block_per_row: the single-block kernel, for comparison)."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(ids, "ids", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32); _need(uniform, "uniform", torch.float32)
    scratch = (None,) * 8 if one_block_per_row else _sample_scratch_for(logits.shape[0], logits.device)
    f = _fn("sampling", "stratum_sample",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(uniform), _ptr(ids), _ptr(values), *[_ptr(t) for t in scratch], _stream()), "sample")
    if not one_block_per_row and 8192 <= logits.shape[1] <= 262144:
        count_launches(1)                      # the one-block kernel behind, for marked rows
