"""Python faces of the CUDA kernels: argument checks on the host, then one C call.

Every function here launches hand-written sm_100a code from `csrc/kernels/` on the current
CUDA stream. There is no CPU fallback and no library model or attention code: if the extension
cannot be built or loaded, the call raises. Checks that a sanitizer would make on the device
are made here on the host: dtypes, contiguity, shapes, and that index tensors are int32.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

from ..csrc.build import kernel_library

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACTIVATIONS = {None: ACT_NONE, "none": ACT_NONE, "gelu_new": ACT_GELU_TANH, "gelu": ACT_GELU_ERF}

_STATUS = {-1: "unsupported dtype", -2: "bad shape", -3: "bad alignment", -4: "unsupported size or option"}


class KernelError(RuntimeError):
    pass


class KernelTimeout(KernelError):
    """A bounded wait inside a kernel ran out: the kernel recorded a code and returned instead of
    spinning on. What it computed is not to be trusted. `code` is the recorded number."""

    CODES = {
        1: "a product's operand tile did not arrive (tensor copy)",
        2: "a product's operand stage was not released (tensor-core commit)",
        3: "a product's accumulator was not completed",
        4: "a product's normalised token tile was not built",
        5: "a key/value tile of prefill attention did not arrive (tensor copy)",
        6: "a stage of the tensor-core prefill attention did not complete",
        7: "a step of the resident decode kernel did not reach its grid barrier",
        99: "a wait that a test let run out",
    }

    def __init__(self, code: int):
        super().__init__(f"a kernel gave up a bounded wait (code {code}: {self.CODES.get(code, 'unknown')}); "
                         f"the step's results are not valid")
        self.code = code


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


_launches = 0


_uses: dict[str, int] = {}


def kernel_uses() -> dict[str, int]:
    """How often each attention kernel has been chosen (tests check the choice by it)."""
    return dict(_uses)


def _used(name: str) -> None:
    _uses[name] = _uses.get(name, 0) + 1


def launch_count() -> int:
    """How many kernels of this package have been launched (graph replays count their kernels)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_STATUS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows, got shape {tuple(t.shape)} stride {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


_libs: dict[str, C.CDLL] = {}


_pdl = os.environ.get("R2_PDL", "1") != "0"


def use_programmatic_dependent_launch(on: bool) -> bool:
    """Kernels are launched so that each may start its prologue (set-up, weight prefetch) while
    its predecessor still runs; every kernel waits for the predecessor before it reads or writes
    anything the predecessor touches. Returns the previous setting."""
    global _pdl
    before, _pdl = _pdl, bool(on)
    for lib in _libs.values():
        lib.r2_set_pdl(int(_pdl))
    return before


def _lib(source: str) -> C.CDLL:
    lib = _libs.get(source)
    if lib is None:
        lib = kernel_library(source)
        lib.r2_set_pdl(int(_pdl))
        _libs[source] = lib
    return lib


def build_all(head_dims=()) -> None:
    """Compile every kernel library that does not depend on a model, and the attention kernels
    for the given head sizes (a model compiles its own head size at first use otherwise)."""
    for source in ("rowwise", "recurrent", "routing", "gemm_simt", "gemm_tc", "attention_simt", "attention_prefill_tc", "latent_attention",
                   "sampling", "wait_selftest"):
        _lib(source)
    kernel_library("sfu_probe")  # (profiling/sfu_probe.py: a measurement, no part of a step)
    for head_dim in head_dims:
        _lib_for_head_dim("attention_decode", head_dim)
        if head_dim <= 128:
            _lib_for_head_dim("attention_prefill", head_dim)
            _lib_for_head_dim("decode_resident", head_dim)


_tensor_core_gemm = os.environ.get("R2_GEMM", "tc") != "simt"
_fast_attention = os.environ.get("R2_ATTENTION", "fast") != "simt"
_fused_norm = os.environ.get("R2_FUSED_NORM", "1") != "0"
_fused_decode = os.environ.get("R2_FUSED_DECODE", "1") != "0"


def use_fused_decode_attention(on: bool) -> bool:
    """Switch the one-launch decode attention (cache write and slice merge inside) on or off."""
    global _fused_decode
    before, _fused_decode = _fused_decode, bool(on)
    return before


def use_fused_norm(on: bool) -> bool:
    """Switch the LayerNorm inside the matrix product's kernel (few rows, bfloat16) on or off."""
    global _fused_norm
    before, _fused_norm = _fused_norm, bool(on)
    return before


_sm_counts: dict = {}


def sm_count(device) -> int:
    """The device's number of multiprocessors (asked once per device)."""
    device = torch.device(device)
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = int(torch.cuda.get_device_properties(device).multi_processor_count)
    return n


_prefill_tc = {"0": False, "always": "always"}.get(os.environ.get("R2_PREFILL_TC", "1"), True)


def use_prefill_tc(on):
    """The tcgen05 prefill attention kernel (head size 64): False, the mma.sync kernel takes
    every shape; True (or "always", which older callers pass), the tcgen05 kernel takes every
    batch that it can take. Returns the previous setting."""
    global _prefill_tc
    before, _prefill_tc = _prefill_tc, ("always" if on == "always" else bool(on))
    return before


_prefill_tc_extras = os.environ.get("R2_PREFILL_TC_EXTRAS", "1") != "0"


def use_prefill_tc_extras(on: bool) -> bool:
    """Whether attention with kept first keys, a sink or a gate may run on the tcgen05 prefill kernel (head
    size 64); off, it runs on the mma.sync kernel (tests compare the two). Returns the previous setting."""
    global _prefill_tc_extras
    before, _prefill_tc_extras = _prefill_tc_extras, bool(on)
    return before


def use_prefill_tma(on: bool, head_dim: int = 64) -> bool:
    """Switch how the prefill attention kernel brings key and value tiles in: 4-D tensor copies
    (TMA, one per page; head size 64 and page sizes 8, 16, 32 or multiples of 64) or 16-byte
    cp.async pieces (every shape). Returns the previous setting."""
    return bool(_lib_for_head_dim("attention_prefill", head_dim).r2_attention_prefill_set_tma(int(bool(on))))


def use_decode_mma(on: bool, head_dim: int = 64) -> bool:
    """Switch the arithmetic of a decode-attention tile between the warp-level tensor cores
    (mma.sync; head sizes up to 128) and scalar float instructions. Returns the previous setting."""
    return bool(_lib_for_head_dim("attention_decode", head_dim).r2_attention_decode_set_mma(int(bool(on))))


_latent_slices = os.environ.get("R2_LATENT_SLICES", "1") != "0"


def use_latent_slices(on: bool) -> bool:
    """Whether a decode step's attention over a cache of latents cuts a token's keys over several CTAs (and merges them in a
    second launch); returns the old setting."""
    global _latent_slices
    old, _latent_slices = _latent_slices, bool(on)
    return old


def use_fast_attention(on: bool) -> bool:
    """Switch bfloat16 attention between the fast kernels and the general CUDA-core one."""
    global _fast_attention
    before, _fast_attention = _fast_attention, bool(on)
    return before


def decode_slices(n_rows: int, n_kv_heads: int, max_context: int, device="cuda:0") -> int:
    """Slices of the keys per (row, kv head) in decode attention: as many as keep every CTA
    resident at once (four to an SM is what every head size's kernel reaches; a second wave of
    CTAs costs more than the slices gain: 8 rows x 12 heads took 8.4 us with 6 slices, 10.3 us with
    8), never less than 128 keys a slice."""
    ctas = max(1, n_rows * n_kv_heads)
    want = max(1, 4 * sm_count(device) // ctas)
    most = max(1, max_context // 128)
    return max(1, min(want, most, 32))


def _lib_for_head_dim(source: str, head_dim: int) -> C.CDLL:
    key = f"{source}:{head_dim}"
    lib = _libs.get(key)
    if lib is None:
        lib = kernel_library(source, {"HEAD_DIM": head_dim})
        lib.r2_set_pdl(int(_pdl))
        if source == "attention_decode":
            lib.r2_attention_decode_scratch_floats.restype = C.c_longlong
        _libs[key] = lib
    return lib


def use_tensor_core_gemm(on: bool) -> bool:
    """Switch the bfloat16 matrix products between the tcgen05 kernel and the CUDA-core one
    (tests compare the two). Returns the previous setting."""
    global _tensor_core_gemm
    before, _tensor_core_gemm = _tensor_core_gemm, bool(on)
    return before


_exact_weights = os.environ.get("R2_EXACT_WEIGHTS", "1") != "0"


def use_exact_weights(on: bool) -> bool:
    """Attention that has a sink, kept first keys or a gate computes its softmax weights in float32 and, in
    the tensor-core kernels, hands them to the second product as the sum of two bfloat16 terms (16 bits of
    mantissa) instead of one rounded term. Off: one term, as the plain attention does. Returns the previous setting."""
    global _exact_weights
    before, _exact_weights = _exact_weights, bool(on)
    return before


def exact_weights() -> bool:
    return _exact_weights


_kv_in_epilogue = os.environ.get("R2_KV_IN_EPILOGUE", "1") != "0"


def use_kv_in_epilogue(on: bool) -> bool:
    """Switch the writing of keys and values into the cache by the q/k/v product's epilogue (more
    than 64 bfloat16 rows) on or off; off, a kernel of its own writes them. Returns the previous setting."""
    global _kv_in_epilogue
    before, _kv_in_epilogue = _kv_in_epilogue, bool(on)
    return before


def use_pair_gemm(mode):
    """The two-CTA persistent form (tcgen05.mma.cta_group::2, 256-row tiles) of the tensor-core
    product: False never, True where it is the faster form (many tiles per SM), "always" wherever
    it can run (192 rows and 128 columns or more; tests compare it with the single-CTA form).
    Returns the previous setting in the same terms."""
    names = {0: False, 1: True, 2: "always"}
    code = {False: 0, True: 1, "always": 2}[mode]
    return names[_lib("gemm_tc").r2_gemm_tc_set_pair(code)]


def gemm_cta_stamps(buffer: torch.Tensor | None) -> int:
    """Profiling: the tensor-core products launched (or captured into a graph) from now on leave six times of
    the nanosecond clock per CTA in `buffer` (int64 [n, 6] on the device: start, before and after the wait on the
    kernel before, tokens normalised, products complete, end; single-CTA forms only); None switches it off.
    Returns the number of CTAs of the last such launch."""
    if buffer is None:
        return int(_lib("gemm_tc").r2_gemm_tc_set_cta_stamps(None, 0))
    _need(buffer, "buffer", torch.int64, 2)
    if buffer.shape[1] != 6 or not buffer.is_contiguous():
        raise KernelError("gemm_cta_stamps: the buffer must be a contiguous int64 [n, 6]")
    return int(_lib("gemm_tc").r2_gemm_tc_set_cta_stamps(C.c_void_p(buffer.data_ptr()), buffer.shape[0]))


if os.environ.get("R2_PAIR_GEMM", "1") == "0":
    use_pair_gemm(False)


class _Workspace:
    """Scratch of sliced decode attention (the slices' partial results, arrival counters that are
    zero between launches) and the word in which kernels record a bounded wait that ran out.
    One per device, sized once."""

    FLOATS = 4 * 1024 * 1024
    COUNTERS = 4096

    def __init__(self, device):
        self.floats = torch.empty(self.FLOATS, dtype=torch.float32, device=device)
        self.counters = torch.zeros(self.COUNTERS, dtype=torch.int32, device=device)
        self.error = torch.zeros(4, dtype=torch.int32, device=device)


_workspaces: dict = {}


def _workspace(device) -> _Workspace:
    ws = _workspaces.get(device)
    if ws is None:
        ws = _workspaces[device] = _Workspace(device)
    return ws


def device_errors(device="cuda:0") -> int:
    """0, or the code that a kernel left when one of its bounded waits ran out (synchronises)."""
    ws = _workspaces.get(torch.device(device))
    return 0 if ws is None else int(ws.error[0].item())


def error_word(device) -> torch.Tensor:
    """The device's error word (int32 [4]; element 0 holds the code): a step's graph copies it to the
    host beside its tokens, so that a time-out is seen without a transfer of its own."""
    return _workspace(torch.device(device)).error


def raise_on_device_error(device="cuda:0", code: int | None = None) -> None:
    """Raises KernelTimeout if a kernel on `device` has recorded that a bounded wait ran out, and
    clears the word so that later steps are checked on their own. `code` is the word's value when the
    caller has read it already (a graph's pinned copy); else it is read here (synchronises)."""
    if code is None:
        code = device_errors(device)
    if code:
        ws = _workspaces.get(torch.device(device))
        if ws is not None:
            ws.error.zero_()
        raise KernelTimeout(int(code))


def wait_selftest(device="cuda:0", polls: int = 64, code: int = 99) -> None:
    """Launches the kernel that waits `polls` polls on a barrier nothing arrives on and then records
    `code` in the device's error word (csrc/kernels/wait_selftest.cu). For tests of the error path."""
    ws = _workspace(torch.device(device))
    with torch.cuda.device(device):
        _check(_lib("wait_selftest").r2_wait_selftest(_p(ws.error), int(polls), int(code), _stream()), "wait_selftest")


# ---------------------------------------------------------------------------------------------


def embed(ids: torch.Tensor, table: torch.Tensor, positions: torch.Tensor | None = None,
          pos_table: torch.Tensor | None = None, out: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale (+ pos_table[positions[t]]) as float32 [T, width]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", dim=2)
    n, width = ids.shape[0], table.shape[1]
    if not table.is_contiguous():
        raise KernelError("table must be contiguous")
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype, 2)
        _need(positions, "positions", torch.int32, 1)
        if pos_table.shape[1] != width or not pos_table.is_contiguous() or positions.shape[0] != n:
            raise KernelError("pos_table / positions do not fit the token table")
    if out is None:
        out = torch.empty(n, width, dtype=torch.float32, device=ids.device)
    _need(out, "out", torch.float32, 2)
    fn = _lib("rowwise").r2_embed
    status = fn(_p(ids), _p(positions), _p(table), _p(pos_table), _p(out), n, width, table.shape[0],
                0 if pos_table is None else pos_table.shape[0], dtype_code(table.dtype), C.c_float(scale), _stream())
    _check(status, "embed")
    return out


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, out_dtype: torch.dtype,
               rows: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm of float32 rows; `rows` (int32) picks input rows, else all rows in order."""
    _need(x, "x", torch.float32, 2)
    _need(gamma, "gamma", torch.float32, 1)
    _need(beta, "beta", torch.float32, 1)
    if not x.is_contiguous() or gamma.shape[0] != x.shape[1] or beta.shape[0] != x.shape[1]:
        raise KernelError(f"layer_norm: x {tuple(x.shape)} gamma {tuple(gamma.shape)} beta {tuple(beta.shape)}")
    n = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n = rows.shape[0]
    if out is None:
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
    status = _lib("rowwise").r2_layer_norm(_p(x), _p(rows), _p(gamma), _p(beta), _p(out), n, x.shape[1],
                                          C.c_float(eps), dtype_code(out.dtype), _stream())
    _check(status, "layer_norm")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype, rows: torch.Tensor | None = None,
             unit_offset: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w of float32 rows, statistics in float32; with `unit_offset` the gain is
    1 + w (the tensor holds the gain's offset from one). `rows` (int32) picks input rows, else all rows in order."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    if not x.is_contiguous() or weight.shape[0] != x.shape[1]:
        raise KernelError(f"rms_norm: x {tuple(x.shape)} weight {tuple(weight.shape)}")
    n = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n = rows.shape[0]
    if out is None:
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
    status = _lib("rowwise").r2_rms_norm(_p(x), _p(rows), _p(weight), _p(out), n, x.shape[1], C.c_float(eps),
                                        C.c_float(1.0 if unit_offset else 0.0), dtype_code(out.dtype), _stream())
    _check(status, "rms_norm")
    return out


def head_norm(buf: torch.Tensor, n_q_heads: int, n_k_heads: int, head_dim: int, w_q: torch.Tensor, w_k: torch.Tensor,
              eps: float, unit_offset: bool = False, kv: KvScatter | None = None) -> None:
    """RMS norm, in place, of each of the first n_q_heads + n_k_heads heads of every row of `buf` (a fused
    projection whose first columns are the query heads and then the key heads); the query heads take the
    gain `w_q`, the key heads `w_k` (float32 [head_dim], shared by the heads of a kind). With `kv` (see
    `kv_scatter`; `col` the first value column, `width` the values' width, `head_dim` the values' head size)
    the same launch puts the normed keys and the values into the rows' cache slots."""
    _need(buf, "buf", dim=2)
    _need(w_q, "w_q", torch.float32, 1)
    _need(w_k, "w_k", torch.float32, 1)
    if w_q.shape[0] != head_dim or w_k.shape[0] != head_dim or buf.shape[1] < (n_q_heads + n_k_heads) * head_dim:
        raise KernelError(f"head_norm: buf {tuple(buf.shape)} does not hold {n_q_heads} + {n_k_heads} heads of {head_dim}")
    if kv is not None and (kv.width != n_k_heads * kv.head_dim or kv.col + kv.width > buf.shape[1]):
        raise KernelError("head_norm: the value columns do not fit the projection")
    cache = (C.c_void_p(kv.k_cache), C.c_void_p(kv.v_cache), C.c_void_p(kv.slots), kv.col, kv.head_dim, kv.page_size,
             C.c_longlong(kv.page_stride), kv.n_pages) if kv is not None else (None, None, None, 0, 0, 0, C.c_longlong(0), 0)
    status = _lib("rowwise").r2_head_norm(_p(buf), _rows(buf, "buf"), buf.shape[0], n_q_heads, n_k_heads, head_dim, _p(w_q),
                                         _p(w_k), C.c_float(eps), C.c_float(1.0 if unit_offset else 0.0), *cache,
                                         dtype_code(buf.dtype), _stream())
    _check(status, "head_norm")


def gated_act(gate_up: torch.Tensor, limit: float, alpha: float, up_offset: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """y = g * sigmoid(alpha * g) * (u + up_offset) with g = min(gate, limit) and u = clamp(up, -limit, limit);
    a row of `gate_up` [T, 2 F] holds its gate values and then its up values. -> [T, F] in the same dtype."""
    _need(gate_up, "gate_up", dim=2)
    if gate_up.shape[1] % 2:
        raise KernelError(f"gated_act: {tuple(gate_up.shape)} does not hold a gate and an up half")
    inner = gate_up.shape[1] // 2
    if out is None:
        out = torch.empty(gate_up.shape[0], inner, dtype=gate_up.dtype, device=gate_up.device)
    status = _lib("rowwise").r2_gated_act(_p(gate_up), _rows(gate_up, "gate_up"), _p(out), _rows(out, "out"), gate_up.shape[0],
                                         inner, C.c_float(limit), C.c_float(alpha), C.c_float(up_offset),
                                         dtype_code(gate_up.dtype), _stream())
    _check(status, "gated_act")
    return out


def expert_act(gate_up: torch.Tensor, kind: str, limit: float = 0.0, alpha: float = 1.0, up_offset: float = 0.0,
               route: torch.Tensor | None = None, n_experts: int = 0, expert_width: int = 0, tail_limit: float | None = None,
               out: torch.Tensor | None = None, tail_gate: torch.Tensor | None = None) -> torch.Tensor:
    """The inner activation of gated feed-forwards whose projections lie side by side: a row of `gate_up` [T, 2 F] holds
    the gates of all F columns and then their ups. kind "relu": relu(g) * u. kind "clamped_swish": g' sigmoid(alpha g')
    (u' + up_offset) with g' = min(g, limit), u' = clamp(u, -limit, limit). kind "silu": g sigmoid(g) * u. With `route` (float32 [T, n_experts], zero
    for experts that a row does not use) the first n_experts * expert_width columns are the routed experts', each
    multiplied by the row's weight for its expert; the columns after them belong to an expert that every row uses
    (limit `tail_limit`), multiplied by sigmoid(tail_gate[row]) where `tail_gate` (float32 [T] or [T, 1], the gate's logit)
    is given. -> [T, F] in the same dtype."""
    _need(gate_up, "gate_up", dim=2)
    if gate_up.shape[1] % 2:
        raise KernelError(f"expert_act: {tuple(gate_up.shape)} does not hold a gate and an up half")
    kinds = {"clamped_swish": 0, "relu": 1, "silu": 2}
    if kind not in kinds:
        raise KernelError(f"expert_act: unknown kind {kind!r}; known: {sorted(kinds)}")
    inner = gate_up.shape[1] // 2
    if route is not None:
        _need(route, "route", torch.float32, 2)
        if route.shape != (gate_up.shape[0], n_experts) or not route.is_contiguous() or n_experts * expert_width > inner:
            raise KernelError(f"expert_act: route {tuple(route.shape)} does not fit {n_experts} experts of {expert_width} in {inner} columns")
    else:
        n_experts = 0
    tail_gate_stride = 0
    if tail_gate is not None:
        _need(tail_gate, "tail_gate", torch.float32)
        if tail_gate.shape[0] != gate_up.shape[0] or tail_gate.numel() != gate_up.shape[0]:
            raise KernelError(f"expert_act: tail_gate {tuple(tail_gate.shape)} is not one number per row")
        tail_gate_stride = tail_gate.stride(0) if gate_up.shape[0] > 1 else 1
    if out is None:
        out = torch.empty(gate_up.shape[0], inner, dtype=gate_up.dtype, device=gate_up.device)
    status = _lib("routing").r2_expert_act(
        _p(gate_up), _rows(gate_up, "gate_up"), _p(out), _rows(out, "out"), gate_up.shape[0], inner, kinds[kind],
        C.c_float(limit), C.c_float(alpha), C.c_float(up_offset), _p(route), n_experts, expert_width,
        C.c_float(limit if tail_limit is None else tail_limit), _p(tail_gate), tail_gate_stride, dtype_code(gate_up.dtype), _stream())
    _check(status, "expert_act")
    return out


def small_linear(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """h [T, K] (any compute dtype) times w [N, K] float32 (+ bias float32) -> float32 [T, N]: the few outputs per row
    that must stay in 32-bit (gates of a recurrence, one gate per head, step sizes), each one warp's sum."""
    _need(h, "h", dim=2)
    _need(w, "w", torch.float32, 2)
    if w.shape[1] != h.shape[1] or not w.is_contiguous():
        raise KernelError(f"small_linear: h {tuple(h.shape)} does not fit w {tuple(w.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != w.shape[0]:
            raise KernelError(f"small_linear: bias {tuple(bias.shape)} does not fit {w.shape[0]} outputs")
    if out is None:
        out = torch.empty(h.shape[0], w.shape[0], dtype=torch.float32, device=h.device)
    status = _lib("routing").r2_small_linear(_p(h), _rows(h, "h"), _p(w), _p(bias), _p(out), _rows(out, "out"), h.shape[0],
                                            w.shape[0], h.shape[1], dtype_code(h.dtype), _stream())
    _check(status, "small_linear")
    return out


def route_top_k(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, top: int):
    """Router: logits h @ w^T + bias in float32, the `top` largest per row (the lower index wins a tie), softmax over
    the chosen logits only. -> (dense float32 [T, experts]: a row's weights, zero for experts not chosen;
    chosen int32 [T, top]; their weights float32 [T, top])."""
    _need(h, "h", dim=2)
    _need(w, "w", torch.float32, 2)
    if w.shape[1] != h.shape[1] or not w.is_contiguous() or not 1 <= top <= w.shape[0]:
        raise KernelError(f"route_top_k: h {tuple(h.shape)}, w {tuple(w.shape)}, top {top} do not fit")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
    n, e = h.shape[0], w.shape[0]
    dense = torch.empty(n, e, dtype=torch.float32, device=h.device)
    chosen = torch.empty(n, top, dtype=torch.int32, device=h.device)
    weight = torch.empty(n, top, dtype=torch.float32, device=h.device)
    status = _lib("routing").r2_route_top_k(_p(h), _rows(h, "h"), _p(w), _p(bias), _p(dense), _p(chosen), _p(weight), n, e, top,
                                           h.shape[1], dtype_code(h.dtype), _stream())
    _check(status, "route_top_k")
    return dense, chosen, weight


def rotate_half(buf: torch.Tensor, n_heads: int, head_dim: int, rot_dims: int, inv_freq: torch.Tensor, positions: torch.Tensor,
                kv: KvScatter | None = None, n_kv_heads: int = 0, k_col: int = 0, *, q_norm: torch.Tensor | None = None,
                k_norm: torch.Tensor | None = None, n_q_heads: int = 0, norm_eps: float = 0.0, magnitude: float = 1.0) -> None:
    """Rotation by position, in place, of the first `n_heads` heads of every row of `buf` (a stacked projection whose
    first columns are the query heads and then the key heads): of each head the first rot_dims dimensions, dimension i
    paired with i + rot_dims / 2, by the angle position * inv_freq[i] (float32 [rot_dims / 2]). With `kv` (see
    `kv_scatter`: `col` the first value column, `head_dim` the values' head size) the same launch puts the rotated keys
    (n_kv_heads heads from column `k_col`) and the values into the rows' cache slots. With `q_norm` / `k_norm` (float32
    [head_dim]) every head is RMS-normed before its rotation, in float32 and in the same launch: the first `n_q_heads` heads with
    the gain q_norm, the others with k_norm, eps `norm_eps`. `magnitude` multiplies cos and sin."""
    _need(buf, "buf", dim=2)
    _need(inv_freq, "inv_freq", torch.float32, 1)
    for name, t in (("q_norm", q_norm), ("k_norm", k_norm)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.shape[0] != head_dim:
                raise KernelError(f"rotate_half: {name} {tuple(t.shape)} is not [{head_dim}]")
    if (q_norm is not None or k_norm is not None) and ((n_q_heads > 0 and q_norm is None) or (n_q_heads < n_heads and k_norm is None)):
        raise KernelError("rotate_half: a norm needs the gains of every kind of head that the rows hold")
    _need(positions, "positions", torch.int32, 1)
    if rot_dims % 2 or not 0 <= rot_dims <= head_dim or inv_freq.shape[0] != rot_dims // 2 or buf.shape[1] < n_heads * head_dim:
        raise KernelError(f"rotate_half: {rot_dims} of {head_dim} dimensions, {n_heads} heads in rows of {buf.shape[1]}")
    if kv is not None and (kv.width != n_kv_heads * kv.head_dim or kv.col + kv.width > buf.shape[1] or k_col + n_kv_heads * head_dim > buf.shape[1]):
        raise KernelError("rotate_half: the key and value columns do not fit the projection")
    cache = (C.c_void_p(kv.k_cache), C.c_void_p(kv.v_cache), C.c_void_p(kv.slots), k_col, kv.col, n_kv_heads, kv.head_dim, kv.page_size,
             C.c_longlong(kv.page_stride), kv.n_pages) if kv is not None else (None, None, None, 0, 0, 0, 0, 0, C.c_longlong(0), 0)
    status = _lib("rowwise").r2_rotate_half(_p(buf), _rows(buf, "buf"), buf.shape[0], n_heads, head_dim, rot_dims, _p(inv_freq),
                                           _p(positions), *cache, _p(q_norm), _p(k_norm), n_q_heads, C.c_float(norm_eps),
                                           C.c_float(magnitude), dtype_code(buf.dtype), _stream())
    _check(status, "rotate_half")


def pair_norm_add(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, w_a: torch.Tensor, w_b: torch.Tensor, eps: float,
                  share: float = 0.5) -> torch.Tensor:
    """x + share * (rms_norm(a) * w_a + rms_norm(b) * w_b), all float32 [T, D]: two branches join the stream."""
    for name, t in (("x", x), ("a", a), ("b", b)):
        _need(t, name, torch.float32, 2)
        if t.shape != x.shape or not t.is_contiguous():
            raise KernelError(f"pair_norm_add: {name} {tuple(t.shape)} must be contiguous and shaped like x {tuple(x.shape)}")
    for name, t in (("w_a", w_a), ("w_b", w_b)):
        _need(t, name, torch.float32, 1)
        if t.shape[0] != x.shape[1]:
            raise KernelError(f"pair_norm_add: {name} {tuple(t.shape)} does not fit the width {x.shape[1]}")
    out = torch.empty_like(x)
    status = _lib("rowwise").r2_pair_norm_add(_p(x), _p(a), _p(b), _p(w_a), _p(w_b), _p(out), x.shape[0], x.shape[1],
                                             C.c_float(eps), C.c_float(share), _stream())
    _check(status, "pair_norm_add")
    return out


def norm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, next_weight: torch.Tensor | None = None,
             next_eps: float = 0.0, next_dtype: torch.dtype | None = None):
    """x + y / rms(y) * weight, all float32 [T, D]: a sublayer's output is normalised and joins the stream. With
    `next_weight` the same launch also gives the norm of the new stream rows, rms_norm(x_new) * next_weight in `next_dtype`
    (the next sublayer's input): -> (x_new, h_next); else -> x_new."""
    for name, t in (("x", x), ("y", y)):
        _need(t, name, torch.float32, 2)
        if t.shape != x.shape or not t.is_contiguous():
            raise KernelError(f"norm_add: {name} {tuple(t.shape)} must be contiguous and shaped like x {tuple(x.shape)}")
    _need(weight, "weight", torch.float32, 1)
    if weight.shape[0] != x.shape[1]:
        raise KernelError(f"norm_add: weight {tuple(weight.shape)} does not fit the width {x.shape[1]}")
    out = torch.empty_like(x)
    nxt = None
    if next_weight is not None:
        _need(next_weight, "next_weight", torch.float32, 1)
        if next_weight.shape[0] != x.shape[1]:
            raise KernelError(f"norm_add: next_weight {tuple(next_weight.shape)} does not fit the width {x.shape[1]}")
        nxt = torch.empty(x.shape, dtype=next_dtype or torch.float32, device=x.device)
    status = _lib("rowwise").r2_norm_add(_p(x), _p(y), _p(weight), _p(out), _p(next_weight), _p(nxt), x.shape[0], x.shape[1],
                                        C.c_float(eps), C.c_float(next_eps), dtype_code(nxt.dtype) if nxt is not None else F32, _stream())
    _check(status, "norm_add")
    return out if nxt is None else (out, nxt)


def add_norm(x: torch.Tensor, y: torch.Tensor, alpha: float, weight: torch.Tensor, eps: float, rounded_dtype: torch.dtype | None = None):
    """(alpha x + y) / rms(alpha x + y) * weight, all float32 [T, D]: a sublayer's output joins the scaled stream and the sum is
    normalised (the norm AFTER the sum). With `rounded_dtype` the same launch also gives the new rows in that dtype, which the
    next sublayer's products read: -> (x_new, rounded); else -> x_new."""
    for name, t in (("x", x), ("y", y)):
        _need(t, name, torch.float32, 2)
        if t.shape != x.shape or not t.is_contiguous():
            raise KernelError(f"add_norm: {name} {tuple(t.shape)} must be contiguous and shaped like x {tuple(x.shape)}")
    _need(weight, "weight", torch.float32, 1)
    if weight.shape[0] != x.shape[1]:
        raise KernelError(f"add_norm: weight {tuple(weight.shape)} does not fit the width {x.shape[1]}")
    out = torch.empty_like(x)
    rounded = torch.empty(x.shape, dtype=rounded_dtype, device=x.device) if rounded_dtype is not None else None
    status = _lib("rowwise").r2_add_norm(_p(x), _p(y), _p(weight), _p(out), _p(rounded), x.shape[0], x.shape[1], C.c_float(alpha),
                                        C.c_float(eps), dtype_code(rounded_dtype) if rounded is not None else F32, _stream())
    _check(status, "add_norm")
    return out if rounded is None else (out, rounded)


def round_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 rows of the stream in the compute dtype."""
    _need(x, "x", torch.float32, 2)
    if not x.is_contiguous():
        raise KernelError("round_rows: x must be contiguous")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    status = _lib("rowwise").r2_round_rows(_p(x), _p(out), C.c_longlong(x.numel()), dtype_code(dtype), _stream())
    _check(status, "round_rows")
    return out


def xielu(z: torch.Tensor, a_pos: float, a_neg: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """For z > 0: a_pos z^2 + z / 2; for z <= 0: a_neg (e^z - 1 - z) + z / 2, elementwise on [T, F], computed in float32."""
    _need(z, "z", dim=2)
    if out is None:
        out = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    status = _lib("rowwise").r2_xielu(_p(z), _rows(z, "z"), _p(out), _rows(out, "out"), z.shape[0], z.shape[1], C.c_float(a_pos),
                                     C.c_float(a_neg), dtype_code(z.dtype), _stream())
    _check(status, "xielu")
    return out


def route_scored(h: torch.Tensor, w: torch.Tensor, correction: torch.Tensor | None, top: int, n_groups: int = 1, keep_groups: int = 1,
                 n_extra: int = 0, scoring: str = "sigmoid", group_mark: str = "two_best", normalise: bool = True, weight_scale: float = 1.0):
    """Router with sigmoid scores: logits h @ w^T in float32 (w float32 [experts + n_extra, K]); an expert is chosen by
    sigmoid(logit) + correction, only inside the `keep_groups` best of `n_groups` equal groups of neighbouring experts (a
    group counts by the sum of its two largest choice scores; the lower index wins ties), the `top` largest; the chosen
    experts' weights are their sigmoids over the sum of the chosen sigmoids (+ 1e-20). The last n_extra rows of w are further
    gates: their logits come back as they are. `scoring` "softmax": the scores are the softmax of the logits over all experts
    instead of their sigmoids. `group_mark` "best": a group counts by its largest choice score alone. `normalise` False: a chosen
    expert's weight is its score times `weight_scale` (the weights are not made to sum to one).
    -> (dense float32 [T, experts]: a row's weights, zero where not chosen; chosen
    int32 [T, top]; their weights float32 [T, top]; extra float32 [T, n_extra] or None)."""
    if scoring not in ("sigmoid", "softmax") or group_mark not in ("two_best", "best"):
        raise KernelError(f"route_scored: unknown scoring {scoring!r} or group mark {group_mark!r}")
    _need(h, "h", dim=2)
    _need(w, "w", torch.float32, 2)
    e = w.shape[0] - n_extra
    if (w.shape[1] != h.shape[1] or not w.is_contiguous() or e < 1 or n_groups < 1 or e % n_groups or not 1 <= keep_groups <= n_groups
            or not 1 <= top <= e // n_groups * keep_groups):
        raise KernelError(f"route_scored: h {tuple(h.shape)}, w {tuple(w.shape)}, top {top}, {keep_groups} of {n_groups} groups do not fit")
    if correction is not None:
        _need(correction, "correction", torch.float32, 1)
        if correction.shape[0] != e:
            raise KernelError(f"route_scored: correction {tuple(correction.shape)} is not [{e}]")
    n = h.shape[0]
    dense = torch.empty(n, e, dtype=torch.float32, device=h.device)
    chosen = torch.empty(n, top, dtype=torch.int32, device=h.device)
    weight = torch.empty(n, top, dtype=torch.float32, device=h.device)
    extra = torch.empty(n, n_extra, dtype=torch.float32, device=h.device) if n_extra else None
    status = _lib("routing").r2_route_scored(_p(h), _rows(h, "h"), _p(w), _p(correction), _p(dense), _p(chosen), _p(weight), _p(extra),
                                            n, e, n_extra, top, n_groups, keep_groups, h.shape[1], int(scoring == "softmax"),
                                            int(group_mark == "best"), int(bool(normalise)), C.c_float(weight_scale), dtype_code(h.dtype), _stream())
    _check(status, "route_scored")
    return dense, chosen, weight, extra


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, k_scale: float,
                   inv_freq: torch.Tensor | None, rot_dims: int, positions: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
                   state_slot: torch.Tensor, fresh: torch.Tensor, n_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """Retention's recurrence S <- decay[h] S + k v^T, o = S^T q for every entry of a batch, from and to the entries' state
    slots. q, k [T, heads * dim], v [T, heads * vdim] (slices of a projection); the kernel rotates q and k by position on their
    way in (of each head the first rot_dims dimensions, i with i + rot_dims / 2, angle positions[t] * inv_freq[i], in float32)
    and multiplies k by k_scale after that. decay float32 [heads]; state float32 [slots, heads * dim * vdim].
    -> float32 [T, heads * vdim], the heads' outputs before their norm."""
    n = _entries(q_start, state_slot, fresh)
    for name, t, width in (("q", q, n_heads * dim), ("k", k, n_heads * dim), ("v", v, n_heads * vdim)):
        _need(t, name, q.dtype, 2)
        if t.shape[1] != width or t.shape[0] != q.shape[0]:
            raise KernelError(f"retention_scan: {name} {tuple(t.shape)} is not [T, {width}]")
    _need(decay, "decay", torch.float32, 1)
    _need(state, "state", torch.float32, 2)
    _need(positions, "positions", torch.int32, 1)
    if decay.shape[0] != n_heads or state.shape[1] != n_heads * dim * vdim or not state.is_contiguous() or positions.shape[0] < q.shape[0]:
        raise KernelError(f"retention_scan: decay {tuple(decay.shape)} / state {tuple(state.shape)} do not fit {n_heads} heads of {dim} x {vdim}")
    if rot_dims:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if rot_dims % 2 or rot_dims > dim or inv_freq.shape[0] != rot_dims // 2:
            raise KernelError(f"retention_scan: {rot_dims} rotated dimensions of {dim}, {tuple(inv_freq.shape)} frequencies")
    out = torch.empty(q.shape[0], n_heads * vdim, dtype=torch.float32, device=q.device)
    status = _lib("recurrent").r2_retention_scan(
        _p(q), _rows(q, "q"), _p(k), _rows(k, "k"), _p(v), _rows(v, "v"), _p(decay), C.c_float(k_scale), _p(inv_freq if rot_dims else None),
        rot_dims, _p(positions), _p(state), C.c_longlong(state.shape[1]), _p(q_start), _p(state_slot), _p(fresh), n, _p(out),
        _rows(out, "out"), n_heads, dim, vdim, int(q.shape[0] <= n), dtype_code(q.dtype), _stream())
    _check(status, "retention_scan")
    return out


def latent_prepare(buf: torch.Tensor, n_heads: int, q_head_dim: int, q_rot_off: int, rot_dim: int, rot_dims: int, kv_col: int,
                   kv_rank: int, norm_weight: torch.Tensor, eps: float, freq: torch.Tensor, magnitude: float, positions: torch.Tensor,
                   k_cache: torch.Tensor | None = None, slot_mapping: torch.Tensor | None = None, page_size: int = 0,
                   page_stride: int = 0, n_pages: int = 0, q_out: torch.Tensor | None = None, q_out_head_dim: int = 0,
                   q_out_off: int = 0, also_norm: tuple[int, int, torch.Tensor] | None = None) -> None:
    """In place on the rows of a stacked projection [n_heads query heads of q_head_dim | latent: kv_rank | shared key part:
    rot_dim]: RMS norm of the latent (weight float32 [kv_rank], statistics in float32); rotation of the shared key part and of
    every head's last-but-`q_rot_off` part (rot_dim numbers from q_rot_off on): the first rot_dims dimensions, pairs (2i, 2i + 1),
    angle positions[t] * freq[i], cos and sin times `magnitude`. With `k_cache` the row's [latent | key part] goes to its
    cache slot (rows of kv_rank + rot_dim numbers) in the same launch. With `q_out` ([T, n_heads * q_out_head_dim]) head h's
    rotated part is also copied to q_out[t, h, q_out_off:]. The rows may hold no query heads (`n_heads` 0) or no latent
    (`kv_col` < 0: query heads only, from column 0). `also_norm` (column, length, weight float32 [length]): that segment of the
    row is RMS-normed in place too (a latent that the queries are made from), with the same eps."""
    _need(buf, "buf", dim=2)
    _need(freq, "freq", torch.float32, 1)
    _need(positions, "positions", torch.int32, 1)
    if kv_col >= 0:
        _need(norm_weight, "norm_weight", torch.float32, 1)
        if buf.shape[1] < kv_col + kv_rank + rot_dim or norm_weight.shape[0] != kv_rank:
            raise KernelError(f"latent_prepare: rows of {buf.shape[1]} do not hold a latent of {kv_rank} and {rot_dim} more from column {kv_col} on")
    if (buf.shape[1] < n_heads * q_head_dim or (kv_col >= 0 and kv_col < n_heads * q_head_dim) or (kv_col < 0 and n_heads < 1)
            or freq.shape[0] < rot_dims // 2 or positions.shape[0] < buf.shape[0]):
        raise KernelError(f"latent_prepare: rows of {buf.shape[1]} do not hold {n_heads} heads of {q_head_dim}, a latent of {kv_rank} and {rot_dim} more")
    xn_col, xn_rank, xn_w = also_norm if also_norm is not None else (0, 0, None)
    if xn_rank:
        _need(xn_w, "also_norm weight", torch.float32, 1)
        if xn_w.shape[0] != xn_rank or xn_col < 0 or xn_col + xn_rank > buf.shape[1]:
            raise KernelError(f"latent_prepare: a normed segment of {xn_rank} from column {xn_col} on does not fit rows of {buf.shape[1]}")
    if k_cache is not None:
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        if k_cache.dtype != buf.dtype or slot_mapping.shape[0] < buf.shape[0]:
            raise KernelError("latent_prepare: the cache and the projection must share a dtype, and every row needs a slot")
    q_out_stride = 0
    if q_out is not None:
        _need(q_out, "q_out", buf.dtype, 2)
        if q_out.shape != (buf.shape[0], n_heads * q_out_head_dim) or q_out_off + rot_dim > q_out_head_dim:
            raise KernelError(f"latent_prepare: q_out {tuple(q_out.shape)} does not hold {n_heads} heads of {q_out_head_dim}")
        q_out_stride = _rows(q_out, "q_out")
    status = _lib("latent_attention").r2_latent_prepare(
        _p(buf), _rows(buf, "buf"), buf.shape[0], n_heads, q_head_dim, q_rot_off, rot_dim, rot_dims, kv_col, kv_rank, _p(norm_weight),
        C.c_float(eps), _p(freq), C.c_float(magnitude), _p(positions), _p(k_cache), _p(slot_mapping), page_size,
        C.c_longlong(page_stride), n_pages, _p(q_out), q_out_stride, q_out_head_dim, q_out_off, xn_col, xn_rank, _p(xn_w),
        dtype_code(buf.dtype), _stream())
    _check(status, "latent_prepare")


def head_linear(a: torch.Tensor, a_head: int, w: torch.Tensor, w_is_nk: bool, out: torch.Tensor, out_head: int, n_heads: int,
                k: int, n: int, gate: torch.Tensor | None = None) -> torch.Tensor:
    """One small product per head: out[t, h * out_head: h * out_head + n] = a[t, h * a_head: h * a_head + k] @ W[h], float32
    sums. `w` holds the heads' matrices one after the other: [n_heads * k, n] (each [k, n]; w_is_nk False) or [n_heads * n, k]
    (each [n, k], stored [out, in]; w_is_nk True). a and out are 2-D with contiguous rows and may be wider than the heads.
    `gate` (laid out like out: head h's n numbers at gate[t, h * out_head:]) multiplies the outputs by its sigmoid."""
    _need(a, "a", dim=2)
    _need(w, "w", a.dtype, 2)
    _need(out, "out", a.dtype, 2)
    want = (n_heads * n, k) if w_is_nk else (n_heads * k, n)
    if (tuple(w.shape) != want or not w.is_contiguous() or a.shape[0] != out.shape[0] or (n_heads - 1) * a_head + k > a.shape[1]
            or (n_heads - 1) * out_head + n > out.shape[1]):
        raise KernelError(f"head_linear: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit {n_heads} heads of {k} -> {n}")
    gate_stride = 0
    if gate is not None:
        _need(gate, "gate", a.dtype, 2)
        if gate.shape[0] != a.shape[0] or (n_heads - 1) * out_head + n > gate.shape[1]:
            raise KernelError(f"head_linear: gate {tuple(gate.shape)} does not fit {n_heads} heads of {n} at a distance of {out_head}")
        gate_stride = _rows(gate, "gate")
    status = _lib("latent_attention").r2_head_linear(_p(a), _rows(a, "a"), a_head, _p(w), int(w_is_nk), _p(out), _rows(out, "out"),
                                                    out_head, a.shape[0], n_heads, k, n, _p(gate), gate_stride, dtype_code(a.dtype), _stream())
    _check(status, "head_linear")
    return out


def mlstm_state_floats(dim: int, vdim: int) -> int:
    """Floats of one head's matrix-memory state in a request slot (matrix, normaliser, running maximum)."""
    fn = _lib("recurrent").r2_mlstm_state_floats
    fn.restype = C.c_longlong
    return int(fn(dim, vdim))


def _entries(q_start, state_slot, fresh) -> int:
    for name, t in (("q_start", q_start), ("state_slot", state_slot), ("fresh", fresh)):
        _need(t, name, torch.int32, 1)
    n = q_start.shape[0] - 1
    if state_slot.shape[0] < n or fresh.shape[0] < n:
        raise KernelError("entries: state_slot / fresh are shorter than q_start says")
    return n


def mlstm_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, cap: float, q_scale: float,
               state: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, fresh: torch.Tensor, n_heads: int,
               dim: int, vdim: int) -> torch.Tensor:
    """The matrix memory's recurrence for every entry of a batch, from and to the entries' state slots.
    q, k [T, heads * dim], v [T, heads * vdim] (slices of a projection); gates float32 [T, 2 heads]: input gates then
    forget gates before the cap; state float32 [slots, heads * mlstm_state_floats]. -> float32 [T, heads * vdim], the
    heads' outputs before their norm."""
    n = _entries(q_start, state_slot, fresh)
    for name, t, width in (("q", q, n_heads * dim), ("k", k, n_heads * dim), ("v", v, n_heads * vdim)):
        _need(t, name, q.dtype, 2)
        if t.shape[1] != width or t.shape[0] != q.shape[0]:
            raise KernelError(f"mlstm_scan: {name} {tuple(t.shape)} is not [T, {width}]")
    _need(gates, "gates", torch.float32, 2)
    _need(state, "state", torch.float32, 2)
    per_head = mlstm_state_floats(dim, vdim)
    if gates.shape != (q.shape[0], 2 * n_heads) or state.shape[1] != n_heads * per_head or not state.is_contiguous():
        raise KernelError(f"mlstm_scan: gates {tuple(gates.shape)} / state {tuple(state.shape)} do not fit {n_heads} heads of {dim} x {vdim}")
    out = torch.empty(q.shape[0], n_heads * vdim, dtype=torch.float32, device=q.device)
    status = _lib("recurrent").r2_mlstm_scan(
        _p(q), _rows(q, "q"), _p(k), _rows(k, "k"), _p(v), _rows(v, "v"), _p(gates), _rows(gates, "gates"), C.c_float(cap),
        C.c_float(q_scale), _p(state), C.c_longlong(state.shape[1]), _p(q_start), _p(state_slot), _p(fresh), n, _p(out),
        _rows(out, "out"), n_heads, dim, vdim, int(q.shape[0] <= n), dtype_code(q.dtype), _stream())
    _check(status, "mlstm_scan")
    return out


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor, conv_state_off: int,
                row_entry: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, fresh: torch.Tensor) -> torch.Tensor:
    """silu of a causal convolution per channel: x [T, C] (a slice of a projection), taps float32 [C, n_taps] whose last
    column is the current token's. Inputs before an entry's first row come from the request's state slot (float32
    [slots, floats]; at `conv_state_off` the inputs of the last n_taps - 1 positions, [n_taps - 1, C]), zeros before a
    sequence's start. The slot is read only: `ssd_scan` renews it. -> [T, C] in x's dtype."""
    _need(x, "x", dim=2)
    _need(taps, "taps", torch.float32, 2)
    _need(state, "state", torch.float32, 2)
    _entries(q_start, state_slot, fresh)
    _need(row_entry, "row_entry", torch.int32, 1)
    channels, n_taps = taps.shape
    if x.shape[1] != channels or not taps.is_contiguous() or conv_state_off + (n_taps - 1) * channels > state.shape[1]:
        raise KernelError(f"causal_conv: x {tuple(x.shape)}, taps {tuple(taps.shape)}, state {tuple(state.shape)} do not fit")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
    out = torch.empty(x.shape[0], channels, dtype=x.dtype, device=x.device)
    status = _lib("recurrent").r2_causal_conv(
        _p(x), _rows(x, "x"), _p(out), _rows(out, "out"), _p(taps), _p(bias), n_taps, channels, _p(state), C.c_longlong(state.shape[1]),
        C.c_longlong(conv_state_off), _p(row_entry), _p(q_start), _p(state_slot), _p(fresh), x.shape[0], dtype_code(x.dtype), _stream())
    _check(status, "causal_conv")
    return out


def ssd_scan(x: torch.Tensor, b: torch.Tensor, c: torch.Tensor, steps: torch.Tensor, step_bias: torch.Tensor, log_rate: torch.Tensor,
             skip: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, fresh: torch.Tensor,
             n_heads: int, n_groups: int, n_state: int, vdim: int, conv_in: torch.Tensor | None = None, conv_taps: int = 1,
             conv_state_off: int = 0) -> torch.Tensor:
    """The state-space recurrence S <- exp(-exp(log_rate) dt) S + dt B x^T, y = S^T C + skip x, dt = softplus(steps +
    step_bias), for every entry of a batch, from and to the entries' state slots. x [T, heads * vdim], b and c
    [T, groups * n_state]; steps float32 [T, heads]; state float32 [slots, floats]: S [heads, n_state, vdim] first. With
    `conv_in` (the convolution's input rows of this step, [T, channels]) the convolution's last conv_taps - 1 inputs at
    `conv_state_off` are renewed too. -> float32 [T, heads * vdim]."""
    n = _entries(q_start, state_slot, fresh)
    _need(x, "x", dim=2)
    _need(b, "b", x.dtype, 2)
    _need(c, "c", x.dtype, 2)
    _need(steps, "steps", torch.float32, 2)
    _need(state, "state", torch.float32, 2)
    for name, t in (("step_bias", step_bias), ("log_rate", log_rate), ("skip", skip)):
        _need(t, name, torch.float32, 1)
        if t.shape[0] != n_heads:
            raise KernelError(f"ssd_scan: {name} {tuple(t.shape)} is not [{n_heads}]")
    if (x.shape[1] != n_heads * vdim or b.shape[1] != n_groups * n_state or c.shape[1] != n_groups * n_state
            or steps.shape != (x.shape[0], n_heads) or n_heads % n_groups or state.shape[1] < n_heads * n_state * vdim):
        raise KernelError("ssd_scan: shapes do not fit")
    channels = 0
    if conv_in is not None:
        _need(conv_in, "conv_in", x.dtype, 2)
        channels = conv_in.shape[1]
        if conv_state_off < n_heads * n_state * vdim or conv_state_off + (conv_taps - 1) * channels > state.shape[1]:
            raise KernelError("ssd_scan: the convolution's state does not fit the slot")
    out = torch.empty(x.shape[0], n_heads * vdim, dtype=torch.float32, device=x.device)
    status = _lib("recurrent").r2_ssd_scan(
        _p(x), _rows(x, "x"), _p(b), _rows(b, "b"), _p(c), _rows(c, "c"), _p(steps), _rows(steps, "steps"), _p(step_bias),
        _p(log_rate), _p(skip), _p(state), C.c_longlong(state.shape[1]), _p(q_start), _p(state_slot), _p(fresh), n, _p(out),
        _rows(out, "out"), n_heads, n_groups, n_state, vdim, _p(conv_in), 0 if conv_in is None else _rows(conv_in, "conv_in"),
        channels, conv_taps, C.c_longlong(conv_state_off), int(x.shape[0] <= n), dtype_code(x.dtype), _stream())
    _check(status, "ssd_scan")
    return out


def group_norm_gated(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor | None, n_groups: int, eps: float, gate_first,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """RMS norm of float32 rows y [T, C] in n_groups equal parts, each by its own root mean square, times weight [C], with
    a gate [T, C] (a slice of a projection, in out_dtype): `gate_first`: y * silu(gate) is what is normalised; else the
    normalised, weighted result is multiplied by sigmoid(gate), or, with gate_first "silu_after", by silu(gate). `weight` None:
    a gain of one. -> [T, C] in out_dtype."""
    _need(y, "y", torch.float32, 2)
    _need(gate, "gate", out_dtype, 2)
    if weight is not None:
        _need(weight, "weight", torch.float32, 1)
    if gate.shape != y.shape or (weight is not None and weight.shape[0] != y.shape[1]) or y.shape[1] % n_groups:
        raise KernelError(f"group_norm_gated: y {tuple(y.shape)}, gate {tuple(gate.shape)}, weight "
                          f"{None if weight is None else tuple(weight.shape)}, {n_groups} groups")
    out = torch.empty(y.shape[0], y.shape[1], dtype=out_dtype, device=y.device)
    status = _lib("recurrent").r2_group_norm_gated(
        _p(y), _rows(y, "y"), _p(gate), _rows(gate, "gate"), _p(weight), _p(out), _rows(out, "out"), y.shape[0], n_groups,
        y.shape[1] // n_groups, C.c_float(eps), 2 if gate_first == "silu_after" else int(bool(gate_first)), dtype_code(out_dtype), _stream())
    _check(status, "group_norm_gated")
    return out


class NormedRows:
    """LayerNorm of float32 rows that has not been computed yet: `linear` may compute it inside
    its own kernel (few rows, bfloat16), or `materialize()` runs the LayerNorm kernel. With `beta`
    None it is an RMS norm with the gain `gamma`."""

    def __init__(self, x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float, dtype: torch.dtype,
                 rows: torch.Tensor | None = None):
        self.x, self.gamma, self.beta, self.eps, self.dtype, self.rows = x, gamma, beta, eps, dtype, rows
        self.shape = (x.shape[0] if rows is None else rows.shape[0], x.shape[1])
        self.device = x.device

    def materialize(self) -> torch.Tensor:
        if self.beta is None:
            return rms_norm(self.x, self.gamma, self.eps, self.dtype, rows=self.rows)
        return layer_norm(self.x, self.gamma, self.beta, self.eps, self.dtype, rows=self.rows)


def _linear_of_normed(a: NormedRows, w, bias, w_is_nk, act, residual, out_dtype, out):
    """The fused form, or None when the kernel does not take the shape."""
    m, k = a.shape
    n = w.shape[0] if w_is_nk else w.shape[1]
    if not (_tensor_core_gemm and _fused_norm and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and m <= 16 and k <= 1024):
        return None
    if (w.shape[1] if w_is_nk else w.shape[0]) != k:
        raise KernelError(f"linear: normed rows {a.shape} do not fit w {tuple(w.shape)} (w_is_nk={w_is_nk})")
    _need(a.x, "x", torch.float32, 2)
    if not a.x.is_contiguous():
        return None
    if out_dtype is None:
        out_dtype = torch.float32 if residual is not None else a.dtype
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    ldr = _rows(residual, "residual") if residual is not None else 0
    ws = _workspace(a.device)
    status = _lib("gemm_tc").r2_gemm_tc(
        None, 0, _p(w), _rows(w, "w"), int(w_is_nk), _p(bias), _p(residual), ldr, _p(out), _rows(out, "out"), m, n, k,
        ACTIVATIONS[act], dtype_code(out.dtype), _p(ws.error), _p(a.x), a.x.stride(0), _p(a.rows), _p(a.gamma),
        _p(a.beta), C.c_float(a.eps), None, C.c_longlong(0), None, _stream())
    if status == -4:
        return None
    _check(status, "linear (tensor cores, fused norm)")
    return out


def mlp(h, w_in: torch.Tensor, b_in: torch.Tensor, act: str, w_out: torch.Tensor, b_out: torch.Tensor | None,
        residual: torch.Tensor | None = None) -> torch.Tensor:
    """act(h @ w_in + b_in) @ w_out + b_out (+ residual), both matrices stored [in, out]. `h` may be
    NormedRows (the LayerNorm then runs inside the first product's kernel where it can)."""
    inner = linear(h, w_in, b_in, act=act)
    return linear(inner, w_out, b_out, residual=residual)


class KvScatter(C.Structure):
    """Where the key and value columns of a fused q/k/v product go: the rows' cache slots.
    `col` is the first key column, `width` the keys' (and the values') width."""

    _fields_ = [("slots", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("page_stride", C.c_longlong),
                ("page_size", C.c_int), ("n_pages", C.c_int), ("col", C.c_int), ("width", C.c_int), ("head_dim", C.c_int)]


def kv_scatter(slot_mapping: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_stride: int, page_size: int,
               n_pages: int, col: int, width: int, head_dim: int) -> KvScatter:
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    return KvScatter(_p(slot_mapping), _p(k_cache), _p(v_cache), page_stride, page_size, n_pages, col, width, head_dim)


def linear(a, w: torch.Tensor, bias: torch.Tensor | None = None, *, w_is_nk: bool = False,
           act: str | None = None, residual: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None, kv: KvScatter | None = None):
    """act(a @ w + bias) (+ residual). `w` is [K, N], or [N, K] with w_is_nk. `a` and `w`
    share a dtype; bias and residual are float32; a float32 residual makes a float32 result.
    `a` may be NormedRows: the LayerNorm then runs inside the product's kernel where it can.

    With `kv` (a fused q/k/v product) the result is (out, written): where the tensor-core kernel
    takes the case (more than 64 bfloat16 rows), the key and value columns go straight into the
    rows' cache slots, `written` is True and those columns of `out` are left undefined; else
    `written` is False and `out` is whole."""
    if kv is not None:
        rows = a.shape[0]
        if _tensor_core_gemm and _kv_in_epilogue and rows > 64 and act is None and residual is None and out_dtype in (None, torch.bfloat16):
            tokens = a.materialize() if isinstance(a, NormedRows) else a
            if tokens.dtype == torch.bfloat16:
                written = _linear_kv(tokens, w, bias, w_is_nk, out, kv)
                if written is not None:
                    return written, True
            a = tokens
        return linear(a, w, bias, w_is_nk=w_is_nk, act=act, residual=residual, out_dtype=out_dtype, out=out), False
    if isinstance(a, NormedRows):
        if act not in ACTIVATIONS:
            raise KernelError(f"linear: unknown activation {act!r}; known: {sorted(k for k in ACTIVATIONS if k)}")
        fused = _linear_of_normed(a, w, bias, w_is_nk, act, residual, out_dtype, out)
        if fused is not None:
            return fused
        a = a.materialize()
    _need(a, "a", dim=2)
    _need(w, "w", a.dtype, 2)
    m, k = a.shape
    n = w.shape[0] if w_is_nk else w.shape[1]
    if (w.shape[1] if w_is_nk else w.shape[0]) != k:
        raise KernelError(f"linear: a {tuple(a.shape)} does not fit w {tuple(w.shape)} (w_is_nk={w_is_nk})")
    lda, ldw = _rows(a, "a"), _rows(w, "w")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError(f"linear: bias {tuple(bias.shape)} does not fit n={n}")
    if out_dtype is None:
        out_dtype = torch.float32 if residual is not None else a.dtype
    ldr = 0
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
        if tuple(residual.shape) != (m, n):
            raise KernelError(f"linear: residual {tuple(residual.shape)} is not [{m}, {n}]")
        ldr = _rows(residual, "residual")
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    if tuple(out.shape) != (m, n):
        raise KernelError(f"linear: out {tuple(out.shape)} is not [{m}, {n}]")
    if act not in ACTIVATIONS:
        raise KernelError(f"linear: unknown activation {act!r}; known: {sorted(k for k in ACTIVATIONS if k)}")
    if a.dtype == torch.bfloat16 and _tensor_core_gemm:
        ws = _workspace(a.device)
        status = _lib("gemm_tc").r2_gemm_tc(
            _p(a), lda, _p(w), ldw, int(w_is_nk), _p(bias), _p(residual), ldr, _p(out), _rows(out, "out"), m, n, k,
            ACTIVATIONS[act], dtype_code(out.dtype), _p(ws.error), None, 0, None, None, None, C.c_float(0.0),
            None, C.c_longlong(0), None, _stream())
        if status != -4:  # -4: a shape the tensor-core kernel does not take; the CUDA-core kernel does
            _check(status, "linear (tensor cores)")
            return out
    status = _lib("gemm_simt").r2_gemm_simt(
        _p(a), lda, _p(w), ldw, int(w_is_nk), _p(bias), _p(residual), ldr, _p(out), _rows(out, "out"), m, n, k,
        ACTIVATIONS[act], dtype_code(a.dtype), dtype_code(out.dtype), _stream())
    _check(status, "linear")
    return out


def _linear_kv(a: torch.Tensor, w: torch.Tensor, bias, w_is_nk: bool, out, kv: KvScatter):
    """The fused q/k/v product with keys and values written to the cache by the epilogue; None
    where the tensor-core kernel does not take the case."""
    _need(a, "a", torch.bfloat16, 2)
    _need(w, "w", a.dtype, 2)
    m, k = a.shape
    n = w.shape[0] if w_is_nk else w.shape[1]
    if (w.shape[1] if w_is_nk else w.shape[0]) != k:
        raise KernelError(f"linear: a {tuple(a.shape)} does not fit w {tuple(w.shape)} (w_is_nk={w_is_nk})")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    ws = _workspace(a.device)
    status = _lib("gemm_tc").r2_gemm_tc(
        _p(a), _rows(a, "a"), _p(w), _rows(w, "w"), int(w_is_nk), _p(bias), None, 0, _p(out), _rows(out, "out"), m, n, k,
        ACTIVATIONS[None], dtype_code(out.dtype), _p(ws.error), None, 0, None, None, None, C.c_float(0.0),
        None, C.c_longlong(0), C.byref(kv), _stream())
    if status == -4:
        return None
    _check(status, "linear (tensor cores, keys and values into the cache)")
    return out


def kv_write(k_src: torch.Tensor, v_src: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             slot_mapping: torch.Tensor, n_kv_heads: int, head_dim: int, page_size: int, page_stride: int,
             n_pages: int, v_head_dim: int = 0) -> None:
    """Scatter this step's keys [T, n_kv_heads * head_dim] and values [T, n_kv_heads * v_head_dim] (0: the keys'
    head size) into their cache slots."""
    v_head_dim = v_head_dim or head_dim
    _need(k_src, "k_src", dim=2)
    _need(v_src, "v_src", k_src.dtype, 2)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    if k_cache.dtype != k_src.dtype or v_cache.dtype != k_src.dtype:
        raise KernelError("kv_write: the cache and the new keys/values must share a dtype")
    n = k_src.shape[0]
    if (k_src.shape[1] != n_kv_heads * head_dim or v_src.shape[1] != n_kv_heads * v_head_dim or v_src.shape[0] != n
            or slot_mapping.shape[0] < n):
        raise KernelError("kv_write: shapes do not fit")
    status = _lib("rowwise").r2_kv_write(_p(k_src), _p(v_src), _rows(k_src, "k_src"), _rows(v_src, "v_src"), _p(k_cache), _p(v_cache), _p(slot_mapping), n,
                                        n_kv_heads, head_dim, v_head_dim, page_size, C.c_longlong(page_stride), n_pages,
                                        dtype_code(k_src.dtype), _stream())
    _check(status, "kv_write")


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_stride: int, page_size: int,
                    n_pages: int, block_tables: torch.Tensor, row_entry: torch.Tensor, positions: torch.Tensor,
                    seq_lens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                    window: int = 0, out: torch.Tensor | None = None, *, decode_only: bool = False,
                    max_context: int = 0, q_start: torch.Tensor | None = None, n_tiles: int = 0, v_head_dim: int = 0,
                    keep_first: int = 0, sink: bool = False, gate: torch.Tensor | None = None, softcap: float = 0.0,
                    sinks: torch.Tensor | None = None, head_gate: torch.Tensor | None = None,
                    values_in_keys: bool = False) -> torch.Tensor:
    """Causal attention of q [T, n_heads * head_dim] over the paged cache -> [T, n_heads * v_head_dim]
    (`v_head_dim` 0: the keys' head size). With a window, `keep_first` keeps a sequence's first keys visible;
    `sink` adds one to the softmax's denominator (an extra exp(0) term: the weights sum to less than one); `gate`
    [T, n_heads * v_head_dim] multiplies the output by its sigmoid. `softcap` > 0 caps the scaled scores at
    softcap * tanh(s / softcap); `sinks` (float32 [n_heads]) puts exp(sinks[h]) into head h's denominator; `head_gate`
    (float32 [T, n_heads]) multiplies head h's output by the sigmoid of its entry: these three are taken by the general
    kernel, the mma.sync prefill kernel and the fused decode kernel.
    `values_in_keys`: the cache holds key rows only and a key's first v_head_dim numbers are its value (a cache of
    latents; `v_cache` is not read); the general kernel takes it, and for bfloat16 with one key head and `q_start` the
    latent kernel, whose tiles hold all heads of a few tokens (it takes `sinks` as well).
    `decode_only` says that every row is an entry of its own (one new token each) and
    `max_context` bounds the rows' context lengths; `q_start` (int32 [R + 1]) with `n_tiles`, the
    sum over entries of ceil(rows / 64), lets the tensor-core prefill kernel take the batch. They
    only choose the kernel and its slicing."""
    _need(q, "q", dim=2)
    for name, t in (("row_entry", row_entry), ("positions", positions), ("seq_lens", seq_lens)):
        _need(t, name, torch.int32, 1)
    _need(block_tables, "block_tables", torch.int32, 2)
    if not block_tables.is_contiguous():
        raise KernelError("block_tables must be contiguous")
    n = q.shape[0]
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"attention: q {tuple(q.shape)} is not [T, {n_heads} * {head_dim}]")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelError("attention: q and the cache must share a dtype")
    v_head_dim = v_head_dim or head_dim
    if out is None:
        out = torch.empty(n, n_heads * v_head_dim, dtype=q.dtype, device=q.device)
    gate_stride = 0
    if gate is not None:
        _need(gate, "gate", q.dtype, 2)
        if gate.shape != (n, n_heads * v_head_dim):
            raise KernelError(f"attention: gate {tuple(gate.shape)} is not [T, {n_heads} * {v_head_dim}]")
        gate_stride = _rows(gate, "gate")
    group = n_heads // max(n_kv_heads, 1)
    # only the general kernel takes a value head size of its own or a head size that is no multiple of 16; kept
    # first keys, a sink and an output gate are taken by both prefill kernels and the fused decode kernel
    fits = v_head_dim == head_dim and head_dim % 16 == 0 and not values_in_keys
    capped = softcap != 0.0 or sinks is not None or head_gate is not None   # what the tcgen05 kernel does not take
    head_gate_stride = 0
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != n_heads:
            raise KernelError(f"attention: sinks {tuple(sinks.shape)} is not [{n_heads}]")
    if head_gate is not None:
        _need(head_gate, "head_gate", torch.float32, 2)
        if head_gate.shape != (n, n_heads):
            raise KernelError(f"attention: head_gate {tuple(head_gate.shape)} is not [T, {n_heads}]")
        head_gate_stride = _rows(head_gate, "head_gate")
    plain = fits and keep_first == 0 and not sink and gate is None and not capped
    if plain and q.dtype == torch.bfloat16 and decode_only and _fast_attention and group in (1, 2, 4, 8):
        lib = _lib_for_head_dim("attention_decode", head_dim)
        n_slices = decode_slices(n, n_kv_heads, max_context, q.device)
        ws = _workspace(q.device)
        need = lib.r2_attention_decode_scratch_floats(n, n_heads, n_slices)
        if need > ws.floats.numel():
            n_slices, need = 1, 0
        status = lib.r2_attention_decode(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
            page_size, n_pages, _p(block_tables), block_tables.shape[1], _p(row_entry), _p(positions), _p(seq_lens),
            n, n_heads, n_kv_heads, C.c_float(scale), window, n_slices, _p(ws.floats), C.c_longlong(ws.floats.numel()),
            _stream())
        _check(status, "paged_attention (decode)")
        if n_slices > 1:
            count_launches(1)  # the merge kernel
        return out
    if (fits and not capped and q.dtype == torch.bfloat16 and _fast_attention and _prefill_tc and q_start is not None and n_tiles > 0 and head_dim == 64
            and (plain or _prefill_tc_extras)):
        # tcgen05 form (head size 64, pages of 8, 16, 32 or a multiple of 64 keys): 128-row tiles, one entry to a
        # tile. Also where most tiles are mostly empty (single decoded tokens beside a portion: 64 such rows
        # and 448 of a prompt take 40 us against the mma.sync kernel's 49).
        _need(q_start, "q_start", torch.int32, 1)
        n_entries = q_start.shape[0] - 1
        status = _lib("attention_prefill_tc").r2_attention_prefill_tc(
            _p(q), _rows(q, "q"), n, _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
            page_size, n_pages, _p(block_tables), block_tables.shape[1], _p(q_start), _p(seq_lens), n_entries,
            (n_tiles + n_entries + 1) // 2, n_heads, n_kv_heads, C.c_float(scale), window, _p(_workspace(q.device).error),
            keep_first, int(bool(sink)), _p(gate), gate_stride, int(_exact_weights and not plain), _stream())
        if status != -4:
            _check(status, "paged_attention (prefill, tcgen05)")
            _used("attention_prefill_tc")
            return out
    if (fits and q.dtype == torch.bfloat16 and _fast_attention and q_start is not None and n_tiles > 0 and head_dim <= 128
            and _rows(q, "q") % 8 == 0 and q.data_ptr() % 16 == 0 and (gate is None or (gate_stride % 2 == 0 and gate.data_ptr() % 4 == 0))):
        _need(q_start, "q_start", torch.int32, 1)
        lib = _lib_for_head_dim("attention_prefill", head_dim)
        status = lib.r2_attention_prefill_capped(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
            page_size, n_pages, _p(block_tables), block_tables.shape[1], _p(q_start), _p(seq_lens),
            q_start.shape[0] - 1, n_tiles, n_heads, n_kv_heads, C.c_float(scale), window, _p(_workspace(q.device).error),
            keep_first, int(bool(sink)), _p(gate), gate_stride, int(_exact_weights and not plain), C.c_float(softcap), _p(sinks),
            _p(head_gate), head_gate_stride, _stream())
        _check(status, "paged_attention (prefill)")
        _used("attention_prefill")
        return out
    if (values_in_keys and n_kv_heads == 1 and q.dtype == torch.bfloat16 and _fast_attention and q_start is not None and keep_first == 0
            and not sink and gate is None and softcap == 0.0 and head_gate is None and head_dim <= 256 and v_head_dim <= head_dim):
        # a cache of latents: every head reads the same rows, so a tile's rows are (token, head) pairs (mma.sync)
        _need(q_start, "q_start", torch.int32, 1)
        single_rows = decode_only and n == q_start.shape[0] - 1
        n_slices, ws = 1, _workspace(q.device)
        if single_rows and _latent_slices:
            # a decode step's token walks all its keys: cut them over enough CTAs to fill the SMs twice (a tile is 64 keys)
            tiles = -(-(min(max_context, window) if window > 0 else max_context) // 64)
            ctas = n * -(-n_heads // 16)
            n_slices = max(1, min(tiles, 16, -(-2 * sm_count(q.device) // ctas)))
        status = _lib("latent_attention").r2_latent_attention(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), C.c_longlong(page_stride), page_size, n_pages,
            _p(block_tables), block_tables.shape[1], _p(q_start), _p(positions), _p(seq_lens), q_start.shape[0] - 1, n, n_heads,
            head_dim, v_head_dim, C.c_float(scale), window, int(_exact_weights), int(single_rows), _p(sinks), n_slices, _p(ws.floats),
            C.c_longlong(ws.floats.numel()), _stream())
        if n_slices > 1:
            count_launches(1)  # the merge kernel
        _check(status, "paged_attention (latents)")
        _used("latent_attention")
        return out
    status = _lib("attention_simt").r2_attention_simt(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(k_cache if values_in_keys else v_cache), C.c_longlong(page_stride),
        page_size, _p(block_tables), block_tables.shape[1], _p(row_entry), _p(positions), _p(seq_lens), n, n_heads,
        n_kv_heads, head_dim, v_head_dim, C.c_float(scale), window, keep_first, int(bool(sink)), _p(gate), gate_stride,
        n_pages, dtype_code(q.dtype), C.c_float(softcap), _p(sinks), _p(head_gate), head_gate_stride,
        head_dim if values_in_keys else 0, _stream())
    _check(status, "paged_attention")
    _used("attention_simt")
    return out


def decode_attention_fused(q: torch.Tensor, k_new: torch.Tensor | None, v_new: torch.Tensor | None, slot_mapping: torch.Tensor | None,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, page_stride: int, page_size: int, n_pages: int,
                           block_tables: torch.Tensor, row_entry: torch.Tensor, positions: torch.Tensor,
                           seq_lens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                           window: int, max_context: int, keep_first: int = 0, sink: bool = False,
                           gate: torch.Tensor | None = None, exact_weights: bool = False, softcap: float = 0.0,
                           sinks: torch.Tensor | None = None, head_gate: torch.Tensor | None = None) -> torch.Tensor | None:
    """Decode attention in ONE launch for a batch in which every row is an entry of its own: the
    kernel writes the new keys and values to their cache slots, and the slice that finishes last
    merges all slices of its row. Returns None when it does not take the case (the caller then writes
    the cache and calls `paged_attention`). With `k_new` None nothing is written: the rows read a cache that already holds
    their own position (a layer that reads the keys and values another layer wrote in this step).
    `keep_first`, `sink`, `gate`, `softcap`, `sinks` and `head_gate` as in `paged_attention`;
    `exact_weights` carries the softmax's weights into the second product as two bfloat16 terms."""
    group = n_heads // max(n_kv_heads, 1)
    if not (_fast_attention and _fused_decode and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and 1 <= group <= 8 and head_dim % 16 == 0):
        return None
    _need(q, "q", dim=2)
    _need(block_tables, "block_tables", torch.int32, 2)
    n = q.shape[0]
    stride = 0
    if k_new is not None:
        _need(k_new, "k_new", torch.bfloat16, 2)
        _need(v_new, "v_new", torch.bfloat16, 2)
        _need(slot_mapping, "slot_mapping", torch.int32, 1)
        stride = _rows(k_new, "k_new")
        if _rows(v_new, "v_new") != stride or k_new.shape != (n, n_kv_heads * head_dim) or slot_mapping.shape[0] < n:
            raise KernelError("decode attention: the new keys and values do not fit the rows")
    else:
        v_new = slot_mapping = None
    if window > 0:
        max_context = min(max_context, window + keep_first)   # what a row reads at most
    slices = decode_slices(n, n_kv_heads, max_context, q.device)
    lib = _lib_for_head_dim("attention_decode", head_dim)
    ws = _workspace(q.device)
    if (lib.r2_attention_decode_scratch_floats(n, n_heads, slices) > ws.floats.numel()
            or n * n_kv_heads > ws.counters.numel()):
        slices = 1
    gate_stride = 0
    if gate is not None:
        _need(gate, "gate", torch.bfloat16, 2)
        if gate.shape != (n, n_heads * head_dim):
            raise KernelError(f"decode attention: gate {tuple(gate.shape)} is not [T, {n_heads} * {head_dim}]")
        gate_stride = _rows(gate, "gate")
    head_gate_stride = 0
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != n_heads:
            raise KernelError(f"decode attention: sinks {tuple(sinks.shape)} is not [{n_heads}]")
    if head_gate is not None:
        _need(head_gate, "head_gate", torch.float32, 2)
        if head_gate.shape != (n, n_heads):
            raise KernelError(f"decode attention: head_gate {tuple(head_gate.shape)} is not [T, {n_heads}]")
        head_gate_stride = _rows(head_gate, "head_gate")
    out = torch.empty(n, n_heads * head_dim, dtype=q.dtype, device=q.device)
    status = lib.r2_attention_decode_fused_capped(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride), page_size,
        n_pages, _p(block_tables), block_tables.shape[1], _p(row_entry), _p(positions), _p(seq_lens), n, n_heads,
        n_kv_heads, C.c_float(scale), window, slices, _p(k_new), _p(v_new), stride, _p(slot_mapping), _p(ws.floats),
        C.c_longlong(ws.floats.numel()), _p(ws.counters), ws.counters.numel(), keep_first, int(bool(sink)), _p(gate),
        gate_stride, int(bool(exact_weights)), C.c_float(softcap), _p(sinks), _p(head_gate), head_gate_stride, _stream())
    if status == -4:
        return None
    _check(status, "decode attention (fused)")
    _used("attention_decode_fused")
    return out


_resident_decode = os.environ.get("R2_RESIDENT_DECODE", "1") != "0"


def use_resident_decode(on: bool) -> bool:
    """Switch the one-kernel form of a decode step's layers (csrc/kernels/decode_resident.cu) on or
    off; off, every part of a layer launches its own kernels. Returns the previous setting."""
    global _resident_decode
    before, _resident_decode = _resident_decode, bool(on)
    return before


_resident_rows = int(os.environ.get("R2_RESIDENT_ROWS", "16"))


def set_resident_decode_rows(n: int) -> int:
    """The most rows of a decode-only batch that run as the resident kernel (it takes up to 64). The
    default is 16: up to there it measured faster than the chain of kernels at GPT-2 124M sizes (0.39 against
    0.46 ms a step of 8 rows, 0.46 against 0.54 at 12, 0.53 against 0.57 at 16), at 24 rows the same (0.62) and
    beyond it slower (0.73 against 0.69 at 32, 1.07 against 0.88 at 64: every CTA reads all rows of a
    product's input). Returns the previous value."""
    global _resident_rows
    before, _resident_rows = _resident_rows, int(n)
    return before


def resident_decode_rows() -> int:
    return _resident_rows if (_resident_decode and _tensor_core_gemm and _fast_attention) else 0


RESIDENT_MAX_GROUPS = 4


class ResidentLayerC(C.Structure):
    """One layer of the resident decode kernel (R2ResidentLayer in csrc/kernels/decode_resident.cu)."""

    _fields_ = [("w_qkv", C.c_void_p), ("w_out", C.c_void_p), ("w_fc", C.c_void_p), ("w_pr", C.c_void_p),
                ("b_qkv", C.c_void_p), ("b_out", C.c_void_p), ("b_fc", C.c_void_p), ("b_pr", C.c_void_p),
                ("ln1_g", C.c_void_p), ("ln1_b", C.c_void_p), ("ln2_g", C.c_void_p), ("ln2_b", C.c_void_p),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("page_stride", C.c_longlong),
                ("group", C.c_int), ("page_size", C.c_int), ("n_pages", C.c_int), ("window", C.c_int),
                ("scale", C.c_float), ("eps1", C.c_float), ("eps2", C.c_float), ("act", C.c_int)]


class ResidentShapeC(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("width", C.c_int), ("inner", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("n_rows", C.c_int)]


class ResidentBuffersC(C.Structure):
    _fields_ = [("x", C.c_void_p), ("qkv", C.c_void_p), ("mixed", C.c_void_p), ("hidden", C.c_void_p),
                ("barrier", C.c_void_p), ("error_flag", C.c_void_p), ("positions", C.c_void_p), ("seq_lens", C.c_void_p),
                ("block_tables", C.c_void_p * RESIDENT_MAX_GROUPS), ("slot_mapping", C.c_void_p * RESIDENT_MAX_GROUPS),
                ("table_width", C.c_int * RESIDENT_MAX_GROUPS), ("stamps", C.c_void_p)]


def pack_weight_tiles(w: torch.Tensor) -> torch.Tensor:
    """A [K, N] matrix (stored [in, out]) in the order in which the resident decode kernel's warps hold
    it: [N / 16 feature tiles][K / 16 k tiles][32 lanes][8 values], a lane's eight values being its
    registers of the 16 x 16 operand tile of mma.sync m16n8k16 (rows = features, columns = k)."""
    k, n = w.shape
    if k % 16 or n % 16:
        raise KernelError(f"pack_weight_tiles: both sizes must be multiples of 16, got {tuple(w.shape)}")
    lane = torch.arange(32, device=w.device)
    g, t = lane >> 2, lane & 3
    r, e = torch.arange(4, device=w.device), torch.arange(2, device=w.device)
    m_idx = (g[:, None, None] + 8 * (r[None, :, None] & 1) + 0 * e[None, None, :])      # feature within the tile
    k_idx = (2 * t[:, None, None] + e[None, None, :] + 8 * (r[None, :, None] >> 1))      # k within the tile
    tiles = w.reshape(k // 16, 16, n // 16, 16).permute(2, 0, 3, 1)                      # [feature tile, k tile, feature, k]
    return tiles[:, :, m_idx, k_idx].contiguous().view(-1)


def decode_resident_library(head_dim: int) -> C.CDLL:
    return _lib_for_head_dim("decode_resident", head_dim)


def decode_resident(head_dim: int, layers: torch.Tensor, shape: ResidentShapeC, buffers: ResidentBuffersC, page_shift: int,
                    device) -> bool:
    """All layers of a decode-only step in one launch; False where the kernel does not take the case."""
    status = decode_resident_library(head_dim).r2_decode_resident(
        _p(layers), C.byref(shape), C.byref(buffers), page_shift, sm_count(device), _stream())
    if status == -4:
        return False
    _check(status, "decode step (resident kernel)")
    _used("decode_resident")
    return True


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, key0: torch.Tensor,
           key1: torch.Tensor, sample_pos: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V] -> int32 [R]."""
    _need(logits, "logits", torch.float32, 2)
    n, vocab = logits.shape
    _need(temperature, "temperature", torch.float32, 1)
    _need(top_k, "top_k", torch.int32, 1)
    _need(sample_pos, "sample_pos", torch.int32, 1)
    for name, t in (("key0", key0), ("key1", key1)):
        if not t.is_cuda or t.dtype not in (torch.int32, torch.uint32) or t.dim() != 1:
            raise KernelError(f"{name} must be a 1-D CUDA tensor of 32-bit integers")
    if min(temperature.shape[0], top_k.shape[0], key0.shape[0], key1.shape[0], sample_pos.shape[0]) < n:
        raise KernelError("sample: a per-row parameter is shorter than the logits")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    status = _lib("sampling").r2_sample(_p(logits), _rows(logits, "logits"), n, vocab, _p(temperature), _p(top_k),
                                       _p(key0), _p(key1), _p(sample_pos), _p(out), _stream())
    _check(status, "sample")
    return out
