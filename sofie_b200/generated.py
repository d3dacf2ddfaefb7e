"""Drives the C++ generator the way a SOFIE user does and loads the result:

    ONNX file --RModelParser_ONNX::Parse / RModel::Generate / OutputGenerated-->  <name>.hxx + <name>.dat
    <name>.hxx --g++ (any C++17 compiler), -lSOFIE_cuda-->  shared object with the emitted Session

The emitted `Session(std::string)` / `std::vector<float> infer(float*)` are reached from Python through
three extern "C" trampolines compiled next to the header. Used by the tests and by the end-to-end leg
of the benchmark; nothing here computes anything itself.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import subprocess
from pathlib import Path

import numpy as np

from . import _build

ROOT = Path(__file__).resolve().parent.parent
HOST = Path(__file__).resolve().parent / "host"
LIBDIR = Path(__file__).resolve().parent / "lib"
WORK = ROOT / "build" / "generated"

TRAMPOLINE = r"""
#include "{header}"
#include <cstring>
#include <string>
using Session = SOFIE_{name}::Session;
static void set_err(char *err, int n, const char *msg) {{ if (err && n > 0) {{ std::strncpy(err, msg, n - 1); err[n - 1] = 0; }} }}
extern "C" void *sofie_session_create(const char *dat, char *err, int errlen) {{
   try {{ return new Session(dat); }} catch (const std::exception &e) {{ set_err(err, errlen, e.what()); return nullptr; }}
}}
extern "C" long sofie_session_infer(void *s, {in_type} **xs, {out_type} *y, long ny, char *err, int errlen) {{
   try {{
      auto out = static_cast<Session *>(s)->infer({args});
      if ((long)out.size() > ny) {{ set_err(err, errlen, "output buffer too small"); return -(long)out.size(); }}
      std::memcpy(y, out.data(), out.size() * sizeof({out_type}));
      return (long)out.size();
   }} catch (const std::exception &e) {{ set_err(err, errlen, e.what()); return -1; }}
}}
extern "C" void sofie_session_destroy(void *s) {{ delete static_cast<Session *>(s); }}
"""


def build_generator() -> Path:
    """make the generator libraries (libSOFIE_core, libSOFIE_parsers) and the sofie_emit tool."""
    r = subprocess.run(["make", "-C", str(HOST), f"OUT={LIBDIR}"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the SOFIE generator failed:\n{r.stdout}")
    return LIBDIR / "sofie_emit"


def emit(onnx_bytes: bytes, name: str, batch: int | None = None, workdir: Path | None = None, binary: bool = False,
         pipelined: bool = False) -> Path:
    """Parse -> Generate -> OutputGenerated. Returns the path of <name>.hxx (the .dat, or with binary=True the
    .bin, lies next to it)."""
    tool = build_generator()
    work = Path(workdir) if workdir else WORK / (name + ("_bin_" if binary else "_") + ("pipe_" if pipelined else "") +
                                                 hashlib.sha1(onnx_bytes).hexdigest()[:10])
    work.mkdir(parents=True, exist_ok=True)
    onnx_path, hxx = work / f"{name}.onnx", work / f"{name}.hxx"
    onnx_path.write_bytes(onnx_bytes)
    cmd = [str(tool), str(onnx_path), str(hxx)] + ([str(batch)] if batch else []) + (["--binary"] if binary else []) + (["--pipelined-upload"] if pipelined else [])
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"sofie_emit failed: {r.stdout.strip()}")
    return hxx


def count_inputs(hxx: Path) -> int:
    """Number of tensors the emitted infer() takes (one pointer argument each)."""
    import re
    m = re.search(r"std::vector<float>\s+infer\(([^)]*)\)", hxx.read_text())
    return max(1, m.group(1).count("tensor_")) if m else 1


def compile_session(hxx: Path, name: str, in_type="float", out_type="float") -> Path:
    """Compile the emitted header (plus the trampolines) and link it against libSOFIE_cuda."""
    lib = _build.build()
    so = hxx.with_suffix(".so")
    if so.exists() and so.stat().st_mtime >= max(hxx.stat().st_mtime, lib.stat().st_mtime, Path(__file__).stat().st_mtime):
        return so
    src = hxx.with_name(hxx.stem + "_trampoline.cxx")
    args = ", ".join(f"xs[{i}]" for i in range(count_inputs(hxx)))
    src.write_text(TRAMPOLINE.format(header=hxx.name, name=name, in_type=in_type, out_type=out_type, args=args))
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I", str(ROOT / "include"), "-I", str(hxx.parent), str(src), "-o", str(so),
           "-L", str(lib.parent), "-lSOFIE_cuda", f"-Wl,-rpath,{lib.parent}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling the emitted header failed:\n{r.stdout}")
    return so


class GeneratedSession:
    """The emitted Session of one model, loaded from its shared object."""

    def __init__(self, so: Path, dat: Path, out_elems: int, out_dtype=np.float32):
        self.lib = C.CDLL(str(so))
        self.lib.sofie_session_create.restype = C.c_void_p
        self.lib.sofie_session_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        self.lib.sofie_session_infer.restype = C.c_long
        self.lib.sofie_session_infer.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_char_p, C.c_int]
        self.lib.sofie_session_destroy.argtypes = [C.c_void_p]
        self.err = C.create_string_buffer(1024)
        self.handle = self.lib.sofie_session_create(str(dat).encode(), self.err, 1024)
        if not self.handle:
            raise RuntimeError(self.err.value.decode())
        self.out_elems, self.out_dtype = out_elems, out_dtype

    def infer(self, x, out: np.ndarray | None = None) -> np.ndarray:
        """x: one array, or a list of arrays for a model with several inputs (in the order of infer())."""
        xs = [np.ascontiguousarray(a) for a in (x if isinstance(x, (list, tuple)) else [x])]
        ptrs = (C.c_void_p * len(xs))(*[a.ctypes.data_as(C.c_void_p) for a in xs])
        y = out if out is not None else np.empty(self.out_elems, self.out_dtype)
        n = self.lib.sofie_session_infer(self.handle, ptrs, y.ctypes.data_as(C.c_void_p), self.out_elems, self.err, 1024)
        if n != self.out_elems:
            raise RuntimeError(f"infer failed ({n}): {self.err.value.decode()}")
        return y

    def infer_ptr(self, x_ptr: int, y_ptr: int) -> None:
        """infer() on raw host addresses (pinned buffers of the benchmark)."""
        ptrs = (C.c_void_p * 1)(C.c_void_p(x_ptr))
        n = self.lib.sofie_session_infer(self.handle, ptrs, C.c_void_p(y_ptr), self.out_elems, self.err, 1024)
        if n != self.out_elems:
            raise RuntimeError(f"infer failed ({n}): {self.err.value.decode()}")

    def close(self):
        if self.handle:
            self.lib.sofie_session_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def session_from_model(model, name: str | None = None, batch: int | None = None, binary: bool = False,
                       fp8_scales=None, pipelined: bool = False) -> GeneratedSession:
    """configs.Model -> ONNX bytes -> generator -> compiled Session."""
    from . import onnx_wire
    name = name or model.name
    hxx = emit(onnx_wire.model_to_onnx(model, fp8_scales), name, batch, binary=binary, pipelined=pipelined)
    so = compile_session(hxx, name)
    out_elems = None
    # output size from the emitted header: "std::vector<float> ret_0(<pointer>, <pointer> + N);"
    import re
    found = re.search(r"ret_0\([^;]*?\+ (\d+)\);", hxx.read_text())
    if found:
        out_elems = int(found.group(1))
    if out_elems is None:
        raise RuntimeError("cannot find the output size in the emitted header")
    return GeneratedSession(so, hxx.with_suffix(".bin" if binary else ".dat"), out_elems)
