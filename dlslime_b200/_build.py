"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host runtime.

Two artefacts are produced next to the Python package so that they travel with a
source snapshot and are visible as loaded in-tree libraries:

* ``dlslime_b200/_C/libslime_cuda.so`` -- every ``csrc/kernels/*.cu`` compiled
  with ``-gencode arch=compute_100a,code=sm_100a``; a plain C API (ctypes).
* ``dlslime_b200/_slime_c*.so`` -- the pybind11 host runtime (assignment model,
  cache directory, counters, TCP endpoint, RPC session, control plane, ...).
* ``dlslime_b200/_C/nanoctrl`` -- the stand-alone control-plane server binary.

Objects are rebuilt only when a source or header is newer (mtime), and
independent translation units compile in parallel.
"""

from __future__ import annotations

import os
import sys

# Run as a script, this file's directory comes first on sys.path, where the package's own
# ``logging`` module would shadow the standard library's.
_here = os.path.dirname(os.path.abspath(__file__))
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != _here]

import concurrent.futures as cf  # noqa: E402
import re  # noqa: E402
import shutil  # noqa: E402
import subprocess  # noqa: E402
import sysconfig  # noqa: E402
from pathlib import Path  # noqa: E402

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
PKG = ROOT / "dlslime_b200"
OBJ = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O2", "-g0", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall", "-Wno-unused-function"]


def slime_option(name: str, default: bool) -> bool:
    """A build switch with an environment override, like the reference's ``slime_option`` CMake macro
    (cmake/utils.cmake:1-15 in the reference): ``ON|OFF|TRUE|FALSE`` (also ``1|0``, any case); anything else warns and
    keeps the default.

    ``BUILD_RDMA`` (ON)          the RDMA RC transport (context, endpoint, worker) and its bindings
    ``BUILD_NVLINK`` (ON)        the sm_100a kernel library (NVLink endpoint and every device op); OFF = host runtime only
    ``BUILD_PYTHON`` (ON)        the pybind11 module ``_slime_c``; OFF builds only the ``nanoctrl`` binary from the host tree
    ``BUILD_TORCH_PLUGIN`` (ON)  the C++ ``torch.distributed`` backend
    ``BUILD_ASCEND_DIRECT`` (OFF) accepted for parity; the transport is an interface stub either way
    ``BUILD_BENCH`` / ``BUILD_TEST`` (OFF) also build the sanitizer stress programs of the host runtime
    """
    raw = os.environ.get(name)
    if raw is None:
        return default
    v = raw.strip().upper()
    if v in ("ON", "TRUE", "1"):
        return True
    if v in ("OFF", "FALSE", "0"):
        return False
    print(f"warning: invalid value for {name}: {raw!r}, using default {'ON' if default else 'OFF'}", file=sys.stderr)
    return default


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the sm_100a kernels cannot be built")
    return cand


def _cuda_include() -> list[Path]:
    """The CUDA toolkit's include directory when there is one: the host runtime takes only the header-only NVTX 3 from it
    (csrc/host/core/nvtx.h) and builds without it."""
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "include" / "nvtx3" / "nvToolsExt.h").exists():
            return [Path(root) / "include"]
    return []


def _newest_header_mtime(dirs) -> float:
    newest = 0.0
    for d in dirs:
        for p in Path(d).rglob("*"):
            if p.suffix in (".h", ".hpp", ".cuh"):
                newest = max(newest, p.stat().st_mtime)
    return newest


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build command failed:\n{' '.join(str(c) for c in cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout.strip() or res.stderr.strip()):
        print(res.stdout, res.stderr, flush=True)
    return res


def _compile_many(jobs, verbose, workers):
    """jobs: list of (src, obj, cmd). Runs the stale ones in parallel."""
    stale = []
    for src, obj, cmd, dep_mtime in jobs:
        if (not obj.exists()) or obj.stat().st_mtime < max(src.stat().st_mtime, dep_mtime):
            stale.append((src, obj, cmd))
    if not stale:
        return False
    with cf.ThreadPoolExecutor(max_workers=workers) as ex:
        futs = [ex.submit(_run, cmd, verbose) for _, _, cmd in stale]
        for f in futs:
            f.result()
    return True


def cuda_lib_path() -> Path:
    return PKG / "_C" / "libslime_cuda.so"


def host_ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_slime_c{suffix}"


def nanoctrl_bin_path() -> Path:
    return PKG / "_C" / "nanoctrl"


def build_cuda(verbose: bool = False, ptxas_info: bool = False, workers: int | None = None) -> Path:
    nvcc = _nvcc()
    kdir = CSRC / "kernels"
    inc = [CSRC / "include", kdir]
    dep = _newest_header_mtime([CSRC / "include", kdir])
    (OBJ / "cuda").mkdir(parents=True, exist_ok=True)
    (PKG / "_C").mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    for src in sorted(kdir.glob("*.cu")):
        obj = OBJ / "cuda" / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if ptxas_info else []), *sum((["-I", i] for i in inc), []), "-c", src, "-o", obj]
        jobs.append((src, obj, cmd, dep))
        objs.append(obj)
    changed = _compile_many(jobs, verbose or ptxas_info, workers or min(8, os.cpu_count() or 4))
    out = cuda_lib_path()
    if changed or not out.exists():
        _run([nvcc, "-shared", "-o", out, *objs, "-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"], verbose)
    return out


def build_host(verbose: bool = False, workers: int | None = None, out_dir: Path | None = None) -> Path:
    """The host runtime. ``out_dir`` (default: the package directory) receives ``_slime_c*.so`` and ``_C/nanoctrl``;
    tests build switch combinations into a scratch directory with it."""
    import pybind11

    hdir = CSRC / "host"
    if not hdir.exists():
        return host_ext_path()
    with_rdma = slime_option("BUILD_RDMA", True)
    with_python = slime_option("BUILD_PYTHON", True)
    variant = "host" + ("" if with_rdma else "_nordma")
    feature_defs = [] if with_rdma else ["-DSLIME_NO_RDMA"]
    inc = [CSRC / "include", hdir, Path(pybind11.get_include()), Path(sysconfig.get_paths()["include"]), *_cuda_include()]
    dep = _newest_header_mtime([CSRC / "include", hdir])
    (OBJ / variant).mkdir(parents=True, exist_ok=True)
    # The system compiler links libstdc++ dynamically. Some environments export CXX as a wrapper that
    # links it statically, and a second, exported copy of the C++ runtime inside an extension clashes
    # with the one torch loads; --exclude-libs keeps any static archive private in either case.
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else os.environ.get("CXX", "g++")
    jobs, objs, main_objs = [], [], []
    for src in sorted(hdir.rglob("*.cpp")):
        parts = src.relative_to(hdir).parts
        if "stress" in parts:
            continue  # sanitizer stress programs are built by build_stress()
        if not with_rdma and ("rdma" in parts or src.name == "bind_rdma.cpp"):
            continue
        rel = "_".join(src.relative_to(hdir).with_suffix("").parts)
        obj = OBJ / variant / (rel + ".o")
        cmd = [cxx, *CXX_FLAGS, *feature_defs, *sum((["-I", i] for i in inc), []), "-c", src, "-o", obj]
        jobs.append((src, obj, cmd, dep))
        if src.name == "nanoctrl_main.cpp":
            main_objs.append(obj)
        else:
            objs.append(obj)
    changed = _compile_many(jobs, verbose, workers or min(8, os.cpu_count() or 4))
    out = host_ext_path() if out_dir is None else Path(out_dir) / host_ext_path().name
    stamp = OBJ / variant / ("linked_into_" + str(abs(hash(str(out)))))
    relink = changed or not out.exists() or not stamp.exists()  # another variant may have been linked to this path last
    if with_python and relink:
        _run([cxx, "-shared", "-o", out, *objs, "-Wl,--exclude-libs,ALL", "-pthread", "-ldl", "-lrt"], verbose)
        for other in OBJ.glob("host*/linked_into_" + str(abs(hash(str(out))))):
            other.unlink()
        stamp.write_text(str(out))
    if main_objs:
        exe = nanoctrl_bin_path() if out_dir is None else Path(out_dir) / "_C" / "nanoctrl"
        if relink or not exe.exists():
            exe.parent.mkdir(parents=True, exist_ok=True)
            core = [o for o in objs if not o.name.startswith("bind")]
            _run([cxx, "-o", exe, *main_objs, *core, "-pthread", "-ldl", "-lrt"], verbose)
    return out


def build_stress(sanitizer: str, verbose: bool = False) -> Path:
    """Builds csrc/host/stress/host_stress.cpp with the whole host runtime (minus the Python bindings) under a
    sanitizer: ``thread`` or ``address,undefined``. Returns the program's path."""
    hdir = CSRC / "host"
    tag = sanitizer.replace(",", "_")
    odir = OBJ / f"san_{tag}"
    odir.mkdir(parents=True, exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else os.environ.get("CXX", "g++")
    flags = ["-O1", "-g1", "-std=c++17", "-pthread", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer"]
    inc = [CSRC / "include", hdir]
    dep = _newest_header_mtime([CSRC / "include", hdir])
    jobs, objs = [], []
    for src in sorted(hdir.rglob("*.cpp")):
        parts = src.relative_to(hdir).parts
        if parts[0] == "bind" or src.name == "nanoctrl_main.cpp":
            continue
        obj = odir / ("_".join(src.relative_to(hdir).with_suffix("").parts) + ".o")
        jobs.append((src, obj, [cxx, *flags, *sum((["-I", i] for i in inc), []), "-c", src, "-o", obj], dep))
        objs.append(obj)
    changed = _compile_many(jobs, verbose, min(8, os.cpu_count() or 4))
    exe = odir / "host_stress"
    if changed or not exe.exists():
        _run([cxx, *flags, "-o", exe, *objs, "-ldl", "-lrt"], verbose)
    for obj in objs:  # instrumented objects are large and only the program is needed
        obj.unlink(missing_ok=True)
    return exe


def torch_plugin_path() -> Path:
    return PKG / ("_slime_torch" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_torch_plugin(verbose: bool = False) -> Path | None:
    """The C++ ``torch.distributed`` backend (csrc/torch/slime_backend.cpp): built against the installed torch with
    torch's own ABI settings. It reaches the runtime through the C table of ``slime_bridge.h`` only, so it links
    libtorch and nothing of this package. Returns None when torch is not importable."""
    src = CSRC / "torch" / "slime_backend.cpp"
    out = torch_plugin_path()
    if not src.exists():
        return None
    try:
        import torch
        from torch.utils import cpp_extension as ce
    except Exception:
        return None
    dep = max(src.stat().st_mtime, (CSRC / "include" / "slime_bridge.h").stat().st_mtime)
    stamp = OBJ / "torch" / "built_for"
    tag = f"{torch.__version__}"
    if out.exists() and out.stat().st_mtime >= dep and stamp.exists() and stamp.read_text() == tag:
        return out
    (OBJ / "torch").mkdir(parents=True, exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else os.environ.get("CXX", "g++")
    inc = [*ce.include_paths(), sysconfig.get_paths()["include"], str(CSRC / "include")]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = ["-DTORCH_EXTENSION_NAME=_slime_torch", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    for name in ("COMPILER_TYPE", "STDLIB", "BUILD_ABI"):
        val = getattr(torch._C, f"_PYBIND11_{name}", None)
        if val is not None:
            defs.append(f'-DPYBIND11_{name}="{val}"')
    libdirs = ce.library_paths()
    obj = OBJ / "torch" / "slime_backend.o"
    _run([cxx, "-O2", "-g0", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wno-unused-function", *defs,
          *sum((["-isystem", str(i)] for i in inc), []), "-c", str(src), "-o", str(obj)], verbose)
    _run([cxx, "-shared", "-o", str(out), str(obj), *sum((["-L", d] for d in libdirs), []),
          *sum(([f"-Wl,-rpath,{d}"] for d in libdirs), []), "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-pthread"], verbose)
    stamp.write_text(tag)
    return out


def build_all(verbose: bool = False) -> None:
    """Everything the switches ask for (see ``slime_option``); with no switch set: kernels, host runtime, torch plugin."""
    if slime_option("BUILD_NVLINK", True):
        build_cuda(verbose=verbose)
    build_host(verbose=verbose)
    if slime_option("BUILD_TORCH_PLUGIN", True) and slime_option("BUILD_PYTHON", True):
        build_torch_plugin(verbose=verbose)
    slime_option("BUILD_ASCEND_DIRECT", False)  # validated for parity; the Ascend transport is a stub in either setting
    if slime_option("BUILD_BENCH", False) or slime_option("BUILD_TEST", False):
        build_stress("thread", verbose=verbose)
        build_stress("address,undefined", verbose=verbose)


def generate_stubs(out_dir: Path | None = None) -> Path:
    """Type stubs of the host module (the reference generates them with pybind11-stubgen, scripts/gen_stubs.sh in
    the reference). Uses pybind11-stubgen when it is installed, else writes the signatures pybind11 puts into the
    docstrings: classes with their methods, and module-level functions. Returns the written file."""
    out_dir = Path(out_dir) if out_dir else PKG
    try:
        import pybind11_stubgen  # noqa: F401

        _run([sys.executable, "-m", "pybind11_stubgen", "dlslime_b200._slime_c", "--output-dir", str(out_dir.parent),
              "--ignore-unresolved-names", "json"], False)
        return out_dir / "_slime_c.pyi"
    except ImportError:
        pass
    import importlib
    import inspect

    sys.path.insert(0, str(ROOT))
    mod = importlib.import_module("dlslime_b200._slime_c")

    def sigs(obj, name, indent):
        doc = (getattr(obj, "__doc__", None) or "").strip().splitlines()
        lines = [ln.strip() for ln in doc if ln.strip().startswith(name + "(") or (ln.strip()[:3].rstrip(".").isdigit() and name + "(" in ln)]
        lines = [ln[ln.index(name + "("):] for ln in lines] or [f"{name}(*args, **kwargs)"]
        out = []
        for ln in lines:
            if len(lines) > 1:
                out.append(f"{indent}@typing.overload")
            ln = ln.replace("dlslime_b200._slime_c.", "").replace("json", "dict")
            ln = re.sub(r"[A-Za-z_][\w]*(?:::[\w<>, ]+)+", "typing.Any", ln)  # a C++ type pybind11 could not name
            out.append(f"{indent}def {ln}: ...")
        return out

    text = ["# Generated by dlslime_b200._build.generate_stubs() from the pybind11 signatures.", "import typing", ""]
    for name, obj in sorted(vars(mod).items()):
        if name.startswith("__"):
            continue
        if inspect.isclass(obj):
            text.append(f"class {name}:")
            body = []
            for mname, m in sorted(vars(obj).items()):
                if mname.startswith("__") and mname != "__init__":
                    continue
                if callable(m) or isinstance(m, (staticmethod, classmethod)):
                    body += sigs(m, mname, "    ")
            text += body or ["    ..."]
            text.append("")
        elif callable(obj):
            text += sigs(obj, name, "") + [""]
        elif inspect.ismodule(obj):
            continue
        else:
            text.append(f"{name}: {type(obj).__name__}")
    path = out_dir / "_slime_c.pyi"
    path.write_text("\n".join(text) + "\n")
    return path


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--ptxas" in sys.argv:
        build_cuda(verbose=True, ptxas_info=True)
    elif "--cuda" in sys.argv:
        build_cuda(verbose=v)
    elif "--host" in sys.argv:
        build_host(verbose=v)
    elif "--stubs" in sys.argv:
        print("stubs:", generate_stubs())
        sys.exit(0)
    elif "--torch" in sys.argv:
        print("built:", build_torch_plugin(verbose=True))
        sys.exit(0)
    else:
        build_all(verbose=v)
    print("built:", cuda_lib_path(), host_ext_path())
