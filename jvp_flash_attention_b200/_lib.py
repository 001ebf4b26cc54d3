"""ctypes binding of libjvpfa.so (the C ABI declared in include/jvpfa.h).

The library is loaded lazily; there is no fallback of any kind: if the shared object is missing
or a call returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

F16, BF16, F32 = 0, 1, 2
MASK_NONE, MASK_BOOL, MASK_ADDITIVE = 0, 1, 2

OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CAUSAL_MASK, ERR_WORKSPACE, ERR_LAUNCH, ERR_DEVICE_TIMEOUT, ERR_NO_ALLOC_LIMIT = range(1, 8)

_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

EXPORTED_SYMBOLS = (
    "jvpfa_version",
    "jvpfa_error_string",
    "jvpfa_fwd_workspace_bytes",
    "jvpfa_bwd_workspace_bytes",
    "jvpfa_mask_summary_bytes",
    "jvpfa_mask_summary",
    "jvpfa_fwd",
    "jvpfa_bwd",
    "jvpfa_read_status",
    "jvpfa_bwd_marked",
    "jvpfa_selftest_timeout",
    "jvpfa_sm_clock_probe",
    "jvpfa_bwd_noalloc",
)


class Mask(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("kind", C.c_int32), ("dtype", C.c_int32), ("stride", C.c_int64 * 4)]


class Strides(C.Structure):
    _fields_ = [("b", C.c_int64), ("h", C.c_int64), ("n", C.c_int64)]


class FwdArgs(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("sm_scale", C.c_float),
        ("mask", Mask), ("mask_summary", C.c_void_p),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("tq", C.c_void_p), ("tk", C.c_void_p), ("tv", C.c_void_p),
        ("o", C.c_void_p), ("to", C.c_void_p), ("lse2", C.c_void_p), ("mu", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_strides", Strides), ("k_strides", Strides), ("v_strides", Strides),
        ("tq_strides", Strides), ("tk_strides", Strides), ("tv_strides", Strides),
        ("dropout_p", C.c_float), ("dropout_seed", C.c_uint64),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("sm_scale", C.c_float),
        ("mask", Mask), ("mask_summary", C.c_void_p),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("tq", C.c_void_p), ("tk", C.c_void_p), ("tv", C.c_void_p),
        ("o", C.c_void_p), ("to", C.c_void_p), ("lse2", C.c_void_p), ("mu", C.c_void_p),
        ("go", C.c_void_p), ("gto", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dtq", C.c_void_p), ("dtk", C.c_void_p), ("dtv", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_strides", Strides), ("k_strides", Strides), ("v_strides", Strides),
        ("tq_strides", Strides), ("tk_strides", Strides), ("tv_strides", Strides),
        ("go_strides", Strides), ("gto_strides", Strides),
        ("dropout_p", C.c_float), ("dropout_seed", C.c_uint64),
    ]


class JvpfaError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"libjvpfa status {status}: {text}")
        self.status = status


_lock = threading.Lock()
_lib = None


def library_path() -> Path:
    env = os.environ.get("JVPFA_LIBRARY")
    return Path(env) if env else Path(__file__).resolve().parent / "libjvpfa.so"


def lib():
    """Returns the loaded CDLL; raises if the shared object has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = library_path()
                if not path.exists():
                    raise RuntimeError(
                        f"{path} not found: build it with `python -m jvp_flash_attention_b200.build` "
                        "(there is no non-CUDA fallback)")
                L = C.CDLL(str(path))
                L.jvpfa_version.restype = C.c_int
                L.jvpfa_error_string.restype = C.c_char_p
                L.jvpfa_error_string.argtypes = [C.c_int]
                L.jvpfa_fwd_workspace_bytes.restype = C.c_size_t
                L.jvpfa_fwd_workspace_bytes.argtypes = [C.POINTER(FwdArgs)]
                L.jvpfa_bwd_workspace_bytes.restype = C.c_size_t
                L.jvpfa_bwd_workspace_bytes.argtypes = [C.POINTER(BwdArgs)]
                L.jvpfa_mask_summary_bytes.restype = C.c_size_t
                L.jvpfa_mask_summary_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
                L.jvpfa_mask_summary.restype = C.c_int
                L.jvpfa_mask_summary.argtypes = [C.POINTER(Mask), C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
                L.jvpfa_fwd.restype = C.c_int
                L.jvpfa_fwd.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
                L.jvpfa_bwd.restype = C.c_int
                L.jvpfa_bwd.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
                L.jvpfa_read_status.restype = C.c_int
                L.jvpfa_read_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
                L.jvpfa_sm_clock_probe.restype = C.c_int
                L.jvpfa_sm_clock_probe.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
                L.jvpfa_selftest_timeout.restype = C.c_int
                L.jvpfa_selftest_timeout.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
                L.jvpfa_bwd_marked.restype = C.c_int
                L.jvpfa_bwd_marked.argtypes = [C.POINTER(BwdArgs), C.c_void_p, C.POINTER(C.c_void_p), C.c_int32]
                L.jvpfa_bwd_noalloc.restype = C.c_int
                L.jvpfa_bwd_noalloc.argtypes = [C.POINTER(BwdArgs), C.c_void_p, C.c_void_p]
                _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise JvpfaError(status, lib().jvpfa_error_string(status).decode())


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise AssertionError(f"unsupported dtype {dt}; expected float16, bfloat16 or float32") from None


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def tensor_core_path(dtype: torch.dtype, D: int) -> bool:
    """Whether (dtype, head dimension) runs on the tensor-core kernels, which read strided inputs in place."""
    if dtype in (torch.float16, torch.bfloat16):
        return 8 <= D <= 128 and D % 8 == 0
    return dtype == torch.float32 and 8 <= D <= 64 and D % 8 == 0


def readable_in_place(t: torch.Tensor) -> bool:
    """A (B,H,N,D) input the tensor-core kernels can read as it is: last axis contiguous, every other stride (of an
    axis longer than 1) positive and a multiple of 16 bytes, 16-byte aligned storage."""
    if t.stride(-1) != 1:
        return False
    try:
        if t.data_ptr() % 16 != 0:
            return False
    except RuntimeError:
        pass        # a functorch wrapper without storage: the launch wrappers look again at the plain tensor inside
    es = t.element_size()
    for dim in range(3):
        if t.shape[dim] > 1 and (t.stride(dim) <= 0 or (t.stride(dim) * es) % 16 != 0):
            return False
    return (t.stride(2) * es) % 16 == 0 and t.stride(2) > 0


def as_input(t):
    """The tensor itself when the kernels can read it in place, else a contiguous copy (None stays None)."""
    if t is None or t.is_contiguous():
        return t
    if tensor_core_path(t.dtype, t.shape[-1]) and readable_in_place(t):
        return t
    return t.contiguous()


def _set_strides(field: Strides, t) -> None:
    if t is None or t.is_contiguous():
        field.b = field.h = field.n = 0
        return
    B, H, N, _ = t.shape
    # an axis of length 1 may carry any stride: give it the contiguous one
    field.n = t.stride(2) if N > 1 else t.shape[3]
    field.h = t.stride(1) if H > 1 else N * t.shape[3]
    field.b = t.stride(0) if B > 1 else H * N * t.shape[3]


def make_mask(mask, B, H, N) -> Mask:
    """Builds the C mask view of a tensor broadcastable to (B,H,N,N); None -> kind NONE."""
    m = Mask()
    if mask is None:
        m.ptr, m.kind, m.dtype = None, MASK_NONE, 0
        return m
    assert mask.dim() == 4, "The provided attention mask must have 4 dimensions (Z, H, N_CTX, N_CTX)."
    view = mask.expand(B, H, N, N)
    m.ptr = view.data_ptr()
    if mask.dtype == torch.bool:
        m.kind, m.dtype = MASK_BOOL, 0
    else:
        m.kind, m.dtype = MASK_ADDITIVE, dtype_code(mask.dtype)
    for i in range(4):
        m.stride[i] = view.stride(i)
    return m


def stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# Workspaces (status word + scratch), one per (device, stream), grown on demand. Kernels of calls that share a
# workspace must be ordered on one stream (the backward's per-row statistics live in it between its preprocess and
# family kernels), so every stream gets its own. A buffer that is outgrown is kept alive until the process ends:
# kernels already enqueued may still use it.
class _Workspace:
    def __init__(self, device, nbytes: int):
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.word = self.buf[:4].view(torch.int32)                       # device status word
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()       # its last copy on the host
        self.retired: list = []


_workspaces: dict = {}


def _ws_key(device):
    index = device.index if device.index is not None else torch.cuda.current_device()
    return index, torch.cuda.current_stream(index).cuda_stream


def _raise_timeout(ws: _Workspace, device) -> None:
    """Error path: waits for the stream, reads and clears the status word, raises."""
    torch.cuda.current_stream(device).synchronize()
    detail = int(ws.word.cpu().item())
    ws.word.zero_()
    ws.host.zero_()
    torch.cuda.current_stream(device).synchronize()
    raise JvpfaError(ERR_DEVICE_TIMEOUT, lib().jvpfa_error_string(ERR_DEVICE_TIMEOUT).decode() + f" (wait id {detail})")


def workspace(device, nbytes: int) -> torch.Tensor:
    """Workspace of the current stream of ``device`` with at least ``nbytes`` bytes. Before handing it out, looks at
    the host copy of the status word that the previous call on this stream left (no synchronisation): a device-side
    wait that gave up in an earlier call raises here."""
    key = _ws_key(device)
    ws = _workspaces.get(key)
    if ws is not None and int(ws.host[0]) != 0:
        _raise_timeout(ws, device)
    if ws is None or ws.buf.numel() < nbytes:
        new = _Workspace(device, max(nbytes, 1 << 20))
        if ws is not None:
            new.retired = ws.retired + [ws.buf]
        _workspaces[key] = ws = new
    return ws.buf


def post_launch(device) -> None:
    """Enqueues a copy of the status word to pinned host memory behind the kernels just launched."""
    ws = _workspaces.get(_ws_key(device))
    if ws is not None:
        ws.host.copy_(ws.word, non_blocking=True)


def read_status(device=None) -> None:
    """Synchronises the device and raises if a device-side wait gave up, on any stream, since the last read."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    index = device.index if device.index is not None else torch.cuda.current_device()
    torch.cuda.synchronize(index)
    for (dev_i, _), ws in list(_workspaces.items()):
        if dev_i != index:
            continue
        detail = C.c_int32(0)
        rc = lib().jvpfa_read_status(C.c_void_p(ws.buf.data_ptr()), stream_ptr(device), C.byref(detail))
        ws.host.zero_()
        if rc != OK:
            raise JvpfaError(rc, lib().jvpfa_error_string(rc).decode() + f" (wait id {detail.value})")


def sm_clock_probe(stream: "torch.cuda.Stream", duration_us: int) -> torch.Tensor:
    """Launches the clock probe on ``stream`` (one that the measured kernels do not use); returns the (1,) float
    device tensor that will hold the average SM clock in MHz over the next ``duration_us`` microseconds."""
    out = torch.zeros(1, dtype=torch.float32, device=stream.device)
    check(lib().jvpfa_sm_clock_probe(C.c_void_p(out.data_ptr()), int(duration_us), C.c_void_p(stream.cuda_stream)))
    return out


def selftest_timeout(device, budget_us: int = 2000) -> torch.Tensor:
    """Runs the library's failure-detection self-test on the current stream of ``device``: a bounded device-side wait
    that is made to run out. Returns the (4,) int32 device tensor with the two wait results and their durations in
    microseconds. The status word is then non-zero: the next call on this stream, or ``read_status``, raises."""
    ws = workspace(device, 256)
    out = torch.full((4,), -1, dtype=torch.int32, device=device)
    check(lib().jvpfa_selftest_timeout(C.c_void_p(ws.data_ptr()), int(budget_us), C.c_void_p(out.data_ptr()),
                                       stream_ptr(device)))
    post_launch(device)
    return out


def mask_summary(mask_c: Mask, mask_tensor, B, H, N):
    """Runs the tile-summary pre-pass; returns the uint8 tensor (kept alive by the caller)."""
    if mask_c.kind == MASK_NONE:
        return None
    Bm = 1 if mask_c.stride[0] == 0 else B
    Hm = 1 if mask_c.stride[1] == 0 else H
    n = lib().jvpfa_mask_summary_bytes(Bm, Hm, N)
    out = torch.empty(n, dtype=torch.uint8, device=mask_tensor.device)
    check(lib().jvpfa_mask_summary(C.byref(mask_c), B, H, N, C.c_void_p(out.data_ptr()), stream_ptr(mask_tensor.device)))
    return out


def dropout_supported(dtype: torch.dtype, D: int) -> bool:
    """Dropout runs in the tensor-core kernels: fp16 / bf16 with a head dimension that is a multiple of 8 up to 128, fp32
    up to 64."""
    return tensor_core_path(dtype, D)


def fwd(q, k, v, tq, tk, tv, mask_c: Mask, summary, causal: bool, sm_scale: float, dropout_p: float = 0.0,
        dropout_seed: int = 0):
    """Launches the dual forward; returns (o, to, lse2, mu). tq/tk/tv None -> primal only (to None). ``dropout_p`` > 0:
    dropout on the attention probabilities with the keep pattern of ``dropout_seed`` (pass both to ``bwd`` again)."""
    B, H, N, D = q.shape
    dual = tq is not None
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)        # outputs are always contiguous
    to = torch.empty(q.shape, dtype=q.dtype, device=q.device) if dual else None
    lse2 = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    mu = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    a = FwdArgs()
    a.B, a.H, a.N, a.D = B, H, N, D
    a.dtype, a.causal, a.sm_scale = dtype_code(q.dtype), int(bool(causal)), float(sm_scale)
    a.mask = mask_c
    a.mask_summary = None if summary is None else summary.data_ptr()
    a.dropout_p, a.dropout_seed = float(dropout_p), int(dropout_seed) & 0xFFFFFFFFFFFFFFFF
    q, k, v, tq, tk, tv = (as_input(t) for t in (q, k, v, tq, tk, tv))
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.tq, a.tk, a.tv = (tq.data_ptr(), tk.data_ptr(), tv.data_ptr()) if dual else (None, None, None)
    for name, t in (("q", q), ("k", k), ("v", v), ("tq", tq), ("tk", tk), ("tv", tv)):
        _set_strides(getattr(a, name + "_strides"), t)
    a.o, a.to = o.data_ptr(), (to.data_ptr() if dual else None)
    a.lse2, a.mu = lse2.data_ptr(), mu.data_ptr()
    need = lib().jvpfa_fwd_workspace_bytes(C.byref(a))
    ws = workspace(q.device, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    check(lib().jvpfa_fwd(C.byref(a), stream_ptr(q.device)))
    post_launch(q.device)
    return o, to, lse2, mu


def bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, go, gto, mask_c: Mask, summary, causal: bool, sm_scale: float,
        marks=None, dropout_p: float = 0.0, dropout_seed: int = 0):
    """Launches the backward. Dual form: returns (dq, dk, dv, dtq, dtk, dtv). With tq None (primal-only: tk, tv,
    to, gto are ignored) returns (dq, dk, dv). ``marks``: five ``torch.cuda.Event(enable_timing=True)`` that have
    been recorded once (so that they exist); they are recorded before the preprocess kernel, before each of the three
    family kernels and after the last one (head dimensions up to 64 in fp16 / bf16 run the key and value families as one
    kernel: the last two events are then recorded together)."""
    B, H, N, D = q.shape
    dual = tq is not None
    outs = [torch.empty(q.shape, dtype=q.dtype, device=q.device) for _ in range(6 if dual else 3)]
    q, k, v, tq, tk, tv, go, gto = (as_input(t) for t in (q, k, v, tq, tk, tv, go, gto))
    a = BwdArgs()
    a.B, a.H, a.N, a.D = B, H, N, D
    a.dtype, a.causal, a.sm_scale = dtype_code(q.dtype), int(bool(causal)), float(sm_scale)
    a.mask = mask_c
    a.mask_summary = None if summary is None else summary.data_ptr()
    a.dropout_p, a.dropout_seed = float(dropout_p), int(dropout_seed) & 0xFFFFFFFFFFFFFFFF
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.o, a.lse2, a.mu = o.data_ptr(), lse2.data_ptr(), mu.data_ptr()
    a.go = go.data_ptr()
    for name, t in (("q", q), ("k", k), ("v", v), ("go", go), ("tq", tq if dual else None), ("tk", tk if dual else None),
                    ("tv", tv if dual else None), ("gto", gto if dual else None)):
        _set_strides(getattr(a, name + "_strides"), t)
    a.dq, a.dk, a.dv = (t.data_ptr() for t in outs[:3])
    if dual:
        a.tq, a.tk, a.tv, a.to, a.gto = (t.data_ptr() for t in (tq, tk, tv, to, gto))
        a.dtq, a.dtk, a.dtv = (t.data_ptr() for t in outs[3:])
    else:
        a.tq = a.tk = a.tv = a.to = a.gto = a.dtq = a.dtk = a.dtv = None
    need = lib().jvpfa_bwd_workspace_bytes(C.byref(a))
    ws = workspace(q.device, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    if marks is None:
        check(lib().jvpfa_bwd(C.byref(a), stream_ptr(q.device)))
    else:
        handles = (C.c_void_p * 5)(*[C.c_void_p(e.cuda_event) for e in marks])
        check(lib().jvpfa_bwd_marked(C.byref(a), stream_ptr(q.device), handles, 5))
    post_launch(q.device)
    return tuple(outs)
