"""Properties of the source tree that the design relies on, checked by reading the files."""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent
KERNELS = sorted((ROOT / "csrc" / "kernels").rglob("*.cu")) + sorted((ROOT / "csrc" / "kernels").rglob("*.cuh"))


def _code_lines(path):
    """(line number, text) without // comments (good enough for these checks: no block comments in the kernels)."""
    for i, line in enumerate(path.read_text().splitlines(), 1):
        yield i, line.split("//", 1)[0]


def test_no_load_uses_cluster_multicast():
    """Operand tiles are fetched by each CTA itself; the qualifier may only appear on tcgen05.commit."""
    needle = "multicast" + "::cluster"
    bad = [(p.name, i) for p in KERNELS for i, line in _code_lines(p) if needle in line and "tcgen05.commit" not in line]
    assert not bad, bad


def test_kernels_never_trap_or_assert():
    """Problems are reported through the status page and the kernel returns; nothing traps the GPU."""
    pat = re.compile(r"__trap\s*\(|(?<![_a-zA-Z])assert\s*\(")
    bad = [(p.name, i) for p in KERNELS for i, line in _code_lines(p) if pat.search(line)]
    assert not bad, bad


def test_tensor_core_path_is_tcgen05_only():
    text = "\n".join(line for p in KERNELS for _, line in _code_lines(p))
    assert "tcgen05.mma" in text and "cp.async.bulk.tensor" in text
    for legacy in ("wgmma", "mma.sync", "wmma::"):
        assert legacy not in text, legacy


def test_every_device_wait_goes_through_the_bounded_helpers():
    """Acquire loads in a loop live in ptx.cuh (wait_flag_ge, mbar_wait) or sit next to a globaltimer limit."""
    for p in KERNELS:
        lines = list(_code_lines(p))
        for idx, (i, line) in enumerate(lines):
            if re.search(r"while\s*\(", line) and "ld_acquire" in line:
                window = " ".join(t for _, t in lines[idx: idx + 8])
                assert "globaltimer_ns" in window or "limit" in window, f"{p.name}:{i}: unbounded wait"


def test_c_api_header_and_library_agree():
    """Every function declared in the public C headers is exported by the built kernel library."""
    from dlslime_b200 import _lib

    if not _lib.available():
        import pytest

        pytest.skip("kernel library not built")
    lib = _lib.load()
    names = set()
    for h in ("slime_cuda.h", "slime_noalloc.h"):
        text = (ROOT / "csrc" / "include" / h).read_text()
        text = re.sub(r"//[^\n]*", "", text)
        names.update(re.findall(r"\b(slime_[a-z0-9_]+)\s*\(", text))
    assert len(names) > 40
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing


def test_baseline_arms_import_nothing_of_the_package():
    """The reference arm and the tuned arm of bench.py must not load this repository's package or libraries: their
    modules import only the standard library, torch and each other, and bench.py imports the package inside run_ours
    only."""
    import ast

    for name in ("reference_arm.py", "tuned_arm.py", "torch_moe.py"):
        tree = ast.parse((ROOT / "baseline" / name).read_text())
        for node in ast.walk(tree):
            mods = []
            if isinstance(node, ast.Import):
                mods = [a.name for a in node.names]
            elif isinstance(node, ast.ImportFrom):
                mods = [node.module or ""]
            assert not any(m.split(".")[0] == "dlslime_b200" for m in mods), (name, mods)
    tree = ast.parse((ROOT / "bench.py").read_text())
    for fn in [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef))]:
        uses = [n for n in ast.walk(fn) if isinstance(n, ast.ImportFrom) and (n.module or "").startswith("dlslime_b200")]
        assert not uses or fn.name == "run_ours", fn.name
    top = [n for n in tree.body if isinstance(n, (ast.Import, ast.ImportFrom))]
    assert not any("dlslime_b200" in ast.dump(n) for n in top)
