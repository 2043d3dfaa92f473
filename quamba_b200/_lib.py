"""ctypes binding of libquamba_b200.so.

The argument structs are generated from ``include/quamba_b200.h`` at import time (the
header keeps one ``type name;`` field per line for exactly this purpose), so the C ABI
has a single source of truth.  There is no CPU fallback: if the shared library is
missing, importing this module raises.
"""
import ctypes
import re
from pathlib import Path

_PKG = Path(__file__).resolve().parent
HEADER = _PKG.parent / "include" / "quamba_b200.h"
LIB_PATH = _PKG / "libquamba_b200.so"

_CTYPES = {
    "int64_t": ctypes.c_int64,
    "int32_t": ctypes.c_int32,
    "int": ctypes.c_int32,
    "uint32_t": ctypes.c_uint32,
    "float": ctypes.c_float,
}

QB_OK = 0
QB_ERR_INVALID_ARG = -1
QB_ERR_UNSUPPORTED = -2
QB_ERR_CUDA = -3
QB_ERR_TIMEOUT = -4
QB_ERR_TOO_LARGE = -5


def parse_header(text: str):
    """Return ({struct_name: [(field, ctype), ...]}, [function names])."""
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    defines = {k: int(v) for k, v in re.findall(r"^#define\s+(QB_\w+)\s+(\d+)\s*$", text, flags=re.M)}
    structs = {}
    for body, name in re.findall(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for line in body.strip().splitlines():
            line = line.strip()
            if not line:
                continue
            m = re.match(r"^(.*?)(\w+)\s*(?:\[(\w+)\])?\s*;$", line)
            ctype_txt, fname, count = m.group(1).strip(), m.group(2), m.group(3)
            if "*" in ctype_txt:
                ct = ctypes.c_void_p
            else:
                ct = _CTYPES[ctype_txt.replace("const", "").strip()]
            if count is not None:                     # a fixed-size array field: `type name[N];`, N a number or a #define
                ct = ct * (int(count) if count.isdigit() else defines[count])
            fields.append((fname, ct))
        structs[name] = fields
    funcs = re.findall(r"^\s*(?:const\s+char\s*\*|int64_t|int)\s+(qb_\w+)\s*\(", text, flags=re.M)
    return structs, funcs


_STRUCT_FIELDS, FUNCTIONS = parse_header(HEADER.read_text())
STRUCTS = {name: type(name, (ctypes.Structure,), {"_fields_": fields}) for name, fields in _STRUCT_FIELDS.items()}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m quamba_b200.build` (nvcc, sm_100a). "
                "quamba_b200 has no CPU or PyTorch fallback.")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.qb_last_error.restype = ctypes.c_char_p
        _lib.qb_sizeof.restype = ctypes.c_int64
        _lib.qb_sizeof.argtypes = [ctypes.c_char_p]
        _lib.qb_ssd_workspace_bytes.restype = ctypes.c_int64
        _lib.qb_ssd_workspace_bytes.argtypes = [ctypes.c_int32] * 7
        _lib.qb_read_device_status.argtypes = [ctypes.c_void_p]
        _lib.qb_ssd_static_scratch_bytes.restype = ctypes.c_int64
        for name, st in STRUCTS.items():
            got = _lib.qb_sizeof(name.encode())
            if got != ctypes.sizeof(st):
                raise RuntimeError(f"ABI mismatch for {name}: library {got} bytes, binding {ctypes.sizeof(st)}")
    return _lib


def make(struct_name: str, **kw):
    st = STRUCTS[struct_name]()
    names = {f for f, _ in st._fields_}
    for k, v in kw.items():
        if k not in names:
            raise KeyError(f"{struct_name} has no field {k}")
        setattr(st, k, v)
    return st


def check(status: int):
    if status != QB_OK:
        msg = lib().qb_last_error().decode(errors="replace")
        raise RuntimeError(f"quamba_b200 error {status}: {msg}")


# Optional per-call trace for benchmarks: when a list is installed with set_call_trace(), every C-ABI call appends
# (entry point, start, end) with two CUDA events recorded on the call's stream right around the launch.
_trace = None


def set_call_trace(sink):
    """``sink``: a list to append (fn, start_event, end_event) to, or None to switch tracing off."""
    global _trace
    _trace = sink


def call(fn: str, args, stream: int):
    f = getattr(lib(), fn)
    if _trace is None:
        check(f(ctypes.byref(args), ctypes.c_void_p(stream)))
        return
    import torch
    ext = torch.cuda.ExternalStream(stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    check(f(ctypes.byref(args), ctypes.c_void_p(stream)))
    e1.record(ext)
    _trace.append((fn, e0, e1))


PATH_SSD_PORTABLE, PATH_HADAMARD_SIMT, PATH_GEMM_SMALL_TILES, PATH_UPDATE_CTA_TILES = 1, 2, 4, 8


class path_override:
    """``with path_override(PATH_SSD_PORTABLE): ...`` runs the enclosed calls on the portable twin of an op (a
    cross-check facility of the library, see qb_set_path_override in the header)."""

    def __init__(self, mask):
        self.mask = mask

    def __enter__(self):
        self.prev = lib().qb_set_path_override(self.mask)
        return self

    def __exit__(self, *exc):
        lib().qb_set_path_override(self.prev)


class early_overlap:
    """``with early_overlap(): ...`` lets the prefill kernels launched inside start their successors early (see
    qb_set_early_overlap in the header).  Only this library's own launch sequences belong inside."""

    def __init__(self, on=True):
        self.on = on

    def __enter__(self):
        self.prev = lib().qb_set_early_overlap(int(self.on))
        return self

    def __exit__(self, *exc):
        lib().qb_set_early_overlap(self.prev)


def set_sm_budget(sms: int) -> int:
    """Cap the multiprocessors the library's kernels size their grids for (0 = all); returns the previous value.  See
    qb_set_sm_budget in the header: leaves a concurrent collective's CTAs room."""
    return lib().qb_set_sm_budget(int(sms))


def read_device_status(stream: int):
    check(lib().qb_read_device_status(ctypes.c_void_p(stream)))
