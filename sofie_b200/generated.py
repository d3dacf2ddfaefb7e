"""Drives the C++ generator the way a SOFIE user does and loads the result:

    ONNX file --RModelParser_ONNX::Parse / RModel::Generate / OutputGenerated-->  <name>.hxx + <name>.dat
    <name>.hxx --g++ (any C++17 compiler), -lSOFIE_cuda-->  shared object with the emitted Session

The emitted `Session(std::string)` / `std::vector<float> infer(float*)` are reached from Python through
three extern "C" trampolines compiled next to the header. Used by the tests and by the end-to-end leg
of the benchmark; nothing here computes anything itself.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import fcntl
import hashlib
import os
import shutil
import subprocess
import tempfile
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
extern "C" void *sofie_session_ctx(void *s) {{ return static_cast<Session *>(s)->fCtx; }}
extern "C" int sofie_session_run_resident(void *s, char *err, int errlen) {{
   try {{ static_cast<Session *>(s)->RunResident(); return 0; }} catch (const std::exception &e) {{ set_err(err, errlen, e.what()); return -1; }}
}}
"""


@contextlib.contextmanager
def _locked(path: Path):
    """Exclusive advisory lock on `path` (created on demand). Several processes of one job -- the ranks of a
    multi-GPU run, test workers -- build the same generator, library and emitted Session; whoever holds the lock
    builds, the others wait and find the finished files."""
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "a+") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


_generator_built = False


def build_generator() -> Path:
    """make the generator libraries (libSOFIE_core, libSOFIE_parsers) and the sofie_emit tool (once per process,
    one process at a time)."""
    global _generator_built
    if not _generator_built:
        with _locked(LIBDIR / ".generator.lock"):
            r = subprocess.run(["make", "-C", str(HOST), f"OUT={LIBDIR}"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"building the SOFIE generator failed:\n{r.stdout}")
        _generator_built = True
    return LIBDIR / "sofie_emit"


def _toolchain_fingerprint() -> str:
    """Identifies everything an emitted Session depends on besides its ONNX bytes: the generator binaries, the
    library sources and this file's trampoline text."""
    h = hashlib.sha1()
    for f in ("sofie_emit", "libSOFIE_core.so", "libSOFIE_parsers.so"):
        h.update((LIBDIR / f).read_bytes())
    h.update(_build._fingerprint().encode())
    h.update(TRAMPOLINE.encode())
    h.update(TRAMPOLINE_DYN.encode())
    return h.hexdigest()


# A Session generated with a run-time batch parameter: Session(file, size_t bs) / infer(size_t bs, float*).
TRAMPOLINE_DYN = r"""
#include "{header}"
#include <cstring>
#include <string>
using Session = SOFIE_{name}::Session;
static void set_err(char *err, int n, const char *msg) {{ if (err && n > 0) {{ std::strncpy(err, msg, n - 1); err[n - 1] = 0; }} }}
extern "C" void *sofie_session_create_bs(const char *dat, long max_batch, char *err, int errlen) {{
   try {{ return new Session(dat, (size_t)max_batch); }} catch (const std::exception &e) {{ set_err(err, errlen, e.what()); return nullptr; }}
}}
extern "C" long sofie_session_infer_bs(void *s, long bs, {in_type} **xs, {out_type} *y, long ny, char *err, int errlen) {{
   try {{
      auto out = static_cast<Session *>(s)->infer((size_t)bs, {args});
      if ((long)out.size() > ny) {{ set_err(err, errlen, "output buffer too small"); return -(long)out.size(); }}
      std::memcpy(y, out.data(), out.size() * sizeof({out_type}));
      return (long)out.size();
   }} catch (const std::exception &e) {{ set_err(err, errlen, e.what()); return -1; }}
}}
extern "C" void sofie_session_destroy(void *s) {{ delete static_cast<Session *>(s); }}
extern "C" void *sofie_session_ctx(void *s) {{ return static_cast<Session *>(s)->fCtx; }}
"""


def is_dynamic(hxx: Path) -> bool:
    """True when the emitted infer() takes the batch as its first argument."""
    import re
    return re.search(r"std::vector<float>\s+infer\(size_t \w+,", hxx.read_text()) is not None


def _run_emit(tool: Path, onnx_bytes: bytes, name: str, batch, binary: bool, pipelined, work: Path) -> Path:
    work.mkdir(parents=True, exist_ok=True)
    onnx_path, hxx = work / f"{name}.onnx", work / f"{name}.hxx"
    onnx_path.write_bytes(onnx_bytes)
    cmd = [str(tool), str(onnx_path), str(hxx)] + ([str(batch)] if batch else []) + (["--binary"] if binary else []) + (["--pipelined-upload"] if pipelined is True else []) + (["--single-upload"] if pipelined is False else [])
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"sofie_emit failed: {r.stdout.strip()}")
    return hxx


def emit(onnx_bytes: bytes, name: str, batch: int | None = None, workdir: Path | None = None, binary: bool = False,
         pipelined: bool | None = None) -> Path:
    """Parse -> Generate -> OutputGenerated. Returns the path of <name>.hxx (the .dat, or with binary=True the
    .bin, lies next to it). pipelined: None = the generator's size gate decides whether the input is uploaded in
    parts, True = always (Options::kPipelinedUpload), False = never (Options::kSingleUpload).

    Without `workdir` the files go to a cache directory keyed by the ONNX bytes, the options and the generator
    build. The directory is filled under a temporary name and renamed into place, so a reader never sees a
    half-written header or weight file, and an existing directory is reused as it is: concurrent processes that
    ask for the same model (the ranks of a multi-GPU run) emit once."""
    tool = build_generator()
    if workdir:
        return _run_emit(tool, onnx_bytes, name, batch, binary, pipelined, Path(workdir))
    key = hashlib.sha1(onnx_bytes + f"|{name}|{batch}|{binary}|{pipelined}|{_toolchain_fingerprint()}".encode()).hexdigest()[:16]
    final = WORK / f"{name}_{key}"
    hxx = final / f"{name}.hxx"
    if hxx.exists():
        return hxx
    with _locked(WORK / f".{name}_{key}.lock"):
        if hxx.exists():
            return hxx
        tmp = Path(tempfile.mkdtemp(prefix=f".{name}_{key}.", dir=WORK))
        try:
            _run_emit(tool, onnx_bytes, name, batch, binary, pipelined, tmp)
            os.replace(tmp, final)
        except BaseException:
            shutil.rmtree(tmp, ignore_errors=True)
            raise
    return hxx


def count_inputs(hxx: Path) -> int:
    """Number of tensors the emitted infer() takes (one pointer argument each)."""
    import re
    m = re.search(r"std::vector<float>\s+infer\(([^)]*)\)", hxx.read_text())
    return m.group(1).count("tensor_") if m else 1   # 0 for a graph made of constants only


def compile_session(hxx: Path, name: str, in_type="float", out_type="float") -> Path:
    """Compile the emitted header (plus the trampolines) and link it against libSOFIE_cuda. The shared object is
    written under a temporary name and renamed into place; an up-to-date one is reused."""
    lib = _build.build()
    so = hxx.with_suffix(".so")

    def fresh():
        return so.exists() and so.stat().st_mtime >= max(hxx.stat().st_mtime, lib.stat().st_mtime)
    if fresh():
        return so
    with _locked(hxx.with_suffix(".lock")):
        if fresh():
            return so
        src = hxx.with_name(hxx.stem + "_trampoline.cxx")
        args = ", ".join(f"xs[{i}]" for i in range(count_inputs(hxx)))
        template = TRAMPOLINE_DYN if is_dynamic(hxx) else TRAMPOLINE
        src.write_text(template.format(header=hxx.name, name=name, in_type=in_type, out_type=out_type, args=args))
        tmp = so.with_name(f".{so.name}.{os.getpid()}.tmp")
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I", str(ROOT / "include"), "-I", str(hxx.parent), str(src), "-o", str(tmp),
               "-L", str(lib.parent), "-lSOFIE_cuda", f"-Wl,-rpath,{lib.parent}"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"compiling the emitted header failed:\n{r.stdout}")
        os.replace(tmp, so)
    return so


class DynamicSession:
    """An emitted Session with a run-time batch: built for `max_batch` samples, infer() takes any batch up to it."""

    def __init__(self, so: Path, dat: Path, max_batch: int, out_per_sample: int):
        self.lib = C.CDLL(str(so))
        self.lib.sofie_session_create_bs.restype = C.c_void_p
        self.lib.sofie_session_create_bs.argtypes = [C.c_char_p, C.c_long, C.c_char_p, C.c_int]
        self.lib.sofie_session_infer_bs.restype = C.c_long
        self.lib.sofie_session_infer_bs.argtypes = [C.c_void_p, C.c_long, C.c_void_p, C.c_void_p, C.c_long, C.c_char_p, C.c_int]
        self.lib.sofie_session_destroy.argtypes = [C.c_void_p]
        self.err = C.create_string_buffer(1024)
        self.handle = self.lib.sofie_session_create_bs(str(dat).encode(), max_batch, self.err, 1024)
        if not self.handle:
            raise RuntimeError(self.err.value.decode())
        self.max_batch, self.out_per_sample = max_batch, out_per_sample

    def infer(self, x: np.ndarray) -> np.ndarray:
        """x: [batch, ...] float32; returns batch * out_per_sample floats."""
        x = np.ascontiguousarray(x, np.float32)
        bs = x.shape[0]
        y = np.empty(max(1, bs * self.out_per_sample), np.float32)
        ptrs = (C.c_void_p * 1)(x.ctypes.data_as(C.c_void_p))
        n = self.lib.sofie_session_infer_bs(self.handle, bs, ptrs, y.ctypes.data_as(C.c_void_p), y.size, self.err, 1024)
        if n != bs * self.out_per_sample:
            raise RuntimeError(f"infer failed ({n}): {self.err.value.decode()}")
        return y[:n]

    def close(self):
        if self.handle:
            self.lib.sofie_session_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def dynamic_session_from_model(model, name: str, max_batch: int, param: str = "bs") -> DynamicSession:
    """configs.Model -> ONNX with the first input dimension written as the parameter `param` -> Generate() without a batch
    size -> compiled Session(file, max_batch)."""
    from . import onnx_wire
    hxx = emit(onnx_wire.model_to_onnx(model, batch_param=param), name)
    so = compile_session(hxx, name)
    sess = DynamicSession(so, hxx.with_suffix(".dat"), max_batch, int(np.prod(model_output_shape(model)[1:])))
    sess.hxx = hxx
    return sess


def model_output_shape(model):
    """Shape of the model's output for its configured batch, from a dry run of the shapes through the layers' weights (Gemm /
    QLinearMatMul chains end in [batch, N]); falls back to running nothing: only the per-sample size is needed."""
    last = model.layers[-1]
    w = model.weights
    for L in reversed(model.layers):
        if L["op"] in ("Gemm", "QLinearMatMul", "Fp8Gemm"):
            B = w[L["B"]]
            n = B.shape[0] if (L.get("transB") or L["op"] == "Fp8Gemm") else B.shape[1]
            return (model.batch(), n)
    raise ValueError(f"cannot tell the output width of a model ending in {last['op']}")


class GeneratedSession:
    """The emitted Session of one model, loaded from its shared object."""

    def __init__(self, so: Path, dat: Path, out_elems: int, out_dtype=np.float32):
        self.lib = C.CDLL(str(so))
        self.lib.sofie_session_create.restype = C.c_void_p
        self.lib.sofie_session_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        self.lib.sofie_session_infer.restype = C.c_long
        self.lib.sofie_session_infer.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_char_p, C.c_int]
        self.lib.sofie_session_destroy.argtypes = [C.c_void_p]
        self.lib.sofie_session_ctx.restype = C.c_void_p
        self.lib.sofie_session_ctx.argtypes = [C.c_void_p]
        self.lib.sofie_session_run_resident.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        self.err = C.create_string_buffer(1024)
        self.handle = self.lib.sofie_session_create(str(dat).encode(), self.err, 1024)
        if not self.handle:
            raise RuntimeError(self.err.value.decode())
        self.out_elems, self.out_dtype = out_elems, out_dtype

    def infer(self, x, out: np.ndarray | None = None) -> np.ndarray:
        """x: one array, or a list of arrays for a model with several inputs (in the order of infer())."""
        xs = [np.ascontiguousarray(a) for a in (x if isinstance(x, (list, tuple)) else [x])]
        ptrs = (C.c_void_p * max(1, len(xs)))(*[a.ctypes.data_as(C.c_void_p) for a in xs])
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

    @property
    def ctx(self) -> int:
        """The Session's sofie_cuda_ctx (its public member fCtx), for the ctx_* entry points of the C ABI."""
        return self.lib.sofie_session_ctx(self.handle)

    def run_resident(self) -> None:
        """Session::RunResident(): the kernels of one inference on the inputs the last infer() left on the device;
        enqueues only (no copies, no wait)."""
        if self.lib.sofie_session_run_resident(self.handle, self.err, 1024) != 0:
            raise RuntimeError(f"RunResident failed: {self.err.value.decode()}")

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
                       fp8_scales=None, pipelined: bool | None = None) -> GeneratedSession:
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
    sess = GeneratedSession(so, hxx.with_suffix(".bin" if binary else ".dat"), out_elems)
    sess.hxx = hxx
    return sess


def launch_plan(hxx: Path) -> list[dict]:
    """The operators of the emitted Launch() in execution order, read from the header text: for each the comment
    line the generator wrote above it, the libSOFIE_cuda entry points it calls and the multiply-accumulate work
    of its contraction descriptors (2 x M x N x K per product, 2 x N x oH x oW x Cout x C/g x kH x kW per convolution; 0 for
    everything else). The intervals sofie_cuda_ctx_timers_read returns are in this order."""
    import re
    text = hxx.read_text()
    body = text[text.index("void Launch() {"):]
    body = body[:body.index("\n}\n")]
    # one segment per mark; the text behind the last mark is the end of the function
    segs = re.split(r"\n\s*Check\(sofie_cuda_ctx_mark\(fCtx, \d+\), \"sofie_cuda_ctx_mark\"\);", "\n" + body)[1:-1]
    plan = []
    for seg in segs:
        calls = re.findall(r"Check\((sofie_cuda_\w+)\(", seg)   # none for an operator that is an alias (Flatten, Reshape)
        title = next((ln.strip(" /-") for ln in seg.splitlines() if ln.strip().startswith("//")), calls[0] if calls else "alias")
        flops = 0
        for kind, vals in re.findall(r"const (sofie_\w+_desc) \w+ = \{([^;]*)\};", seg):
            nums = [float(v.rstrip("f")) for v in re.findall(r"-?\d+\.?\d*(?:e[-+]?\d+)?f?", vals)]
            if kind in ("sofie_gemm_f32_desc", "sofie_qgemm_desc", "sofie_fp8_gemm_desc"):
                flops += 2 * nums[0] * nums[1] * nums[2]
            elif kind == "sofie_conv2d_desc":
                n, c, h, w, co, kh, kw, ph, pw, sh, sw, dh, dw, grp = nums[:14]
                oh = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
                ow = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
                flops += 2 * n * oh * ow * co * (c / grp) * kh * kw
            elif kind == "sofie_qconv2d_desc":
                n, c, h, w, co, kh, kw, ph, pw, sh, sw = nums[:11]
                oh = (h + 2 * ph - kh) // sh + 1
                ow = (w + 2 * pw - kw) // sw + 1
                flops += 2 * n * oh * ow * co * c * kh * kw
            elif kind == "sofie_mlp_desc":
                m, layers = int(nums[0]), int(nums[1])
                dims = nums[2:3 + layers]
                flops += 2 * m * sum(dims[i] * dims[i + 1] for i in range(layers))
        plan.append(dict(title=title, calls=calls, flops=int(flops)))
    return plan
