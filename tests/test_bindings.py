"""The ctypes signatures against the C prototypes they bind (no GPU, no compiler needed): every function
of ``kernels/lib.py`` is exported by the source file of the library it names, with the same number of
arguments and the same kind of each (pointer, int, long long, float).  A drift between the two would not
fail to load: it would pass garbage to a kernel."""

import re
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest

from pyre_b200.kernels import build, lib

KIND = {c_void_p: "pointer", c_int: "int", c_longlong: "long long", c_float: "float"}


def prototypes(source: str) -> dict:
    """name -> list of argument kinds, for every ``PYRE_API <type> name(args)`` of a source file."""
    text = re.sub(r"//[^\n]*", "", (build.CSRC / source).read_text())
    out = {}
    for m in re.finditer(r"PYRE_API\s+[\w ]+?\s+(\w+)\s*\(([^)]*)\)", text):
        kinds = []
        for arg in (a.strip() for a in m.group(2).split(",")):
            if not arg or arg == "void":
                continue
            if "*" in arg or re.match(r"(const\s+)?cudaStream_t\b", arg):
                kinds.append("pointer")
            elif re.match(r"(const\s+)?long long\b", arg):
                kinds.append("long long")
            elif re.match(r"(const\s+)?float\b", arg):
                kinds.append("float")
            elif re.match(r"(const\s+)?int\b", arg):
                kinds.append("int")
            else:
                raise AssertionError(f"{source}: {m.group(1)} has an argument this test cannot classify: {arg!r}")
        out[m.group(1)] = kinds
    return out


def test_every_bound_function_matches_its_prototype():
    by_library = {name: prototypes(source) for name, source in build.LIBRARIES.items()}
    for fn, (library, argtypes) in lib.SIGNATURES.items():
        assert library in by_library, f"{fn} names the unknown library {library!r}"
        assert fn in by_library[library], f"{fn} is not exported by {build.LIBRARIES[library]}"
        want = by_library[library][fn]
        got = [KIND[t] for t in argtypes]
        assert got == want, f"{fn}: bound as {got}, declared as {want}"


def test_every_exported_launcher_is_bound_or_known():
    """An exported function that nothing binds is dead or forgotten; the few that are called by other means
    (the allocation-free attention entry and the size queries, through ctypes directly) are named here."""
    bound = set(lib.SIGNATURES)
    other = {"pyre_attention_mma_scratch_floats", "pyre_paged_attention_mma_noalloc",
             "pyre_paged_attention_mma_noalloc_capacity"}
    for name, source in build.LIBRARIES.items():
        for fn in prototypes(source):
            assert fn in bound or fn in other, f"{source} exports {fn}, which kernels/lib.py does not bind"


def test_every_call_site_passes_as_many_arguments_as_the_signature_has():
    """``lib.call("name", ...)`` in the package: the count of arguments at each call site (none of them starred)
    equals the signature's, and every name called is a bound one."""
    import ast
    from pathlib import Path

    import pyre_b200

    seen = set()
    for path in Path(pyre_b200.__file__).parent.rglob("*.py"):
        for node in ast.walk(ast.parse(path.read_text())):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr in ("call", "call_value")
                    and isinstance(node.func.value, ast.Name) and node.func.value.id == "lib"):
                continue
            name = node.args[0]
            assert isinstance(name, ast.Constant) and name.value in lib.SIGNATURES, f"{path}:{node.lineno}: unknown function"
            assert not any(isinstance(a, ast.Starred) for a in node.args) and not node.keywords, f"{path}:{node.lineno}"
            want = len(lib.SIGNATURES[name.value][1])
            assert len(node.args) - 1 == want, f"{path}:{node.lineno}: {name.value} takes {want} arguments, {len(node.args) - 1} given"
            seen.add(name.value)
    assert seen == set(lib.SIGNATURES), f"bound but never called: {sorted(set(lib.SIGNATURES) - seen)}"


def test_a_tensor_on_another_device_is_refused_on_the_host(monkeypatch):
    """Kernels launch on the current device's stream: a tensor of another device is refused before any launch
    (it would fault on the GPU), and the stepper makes its model's device current around everything it launches.
    Stand-ins play the devices here; nothing runs on a GPU."""
    import torch
    from pyre_b200.engine import step
    from pyre_b200.kernels import ops

    monkeypatch.setattr(ops, "_current_device", lambda: 0)
    ops.require_current_device(torch.device("cuda:0"))
    ops.require_current_device(torch.device("cuda"))          # no index: the current device
    with pytest.raises(ValueError, match=r"cuda:1 but the current device is cuda:0"):
        ops.require_current_device(torch.device("cuda:1"), "q")

    class FakeTensor:
        is_cuda, device, dtype = True, torch.device("cuda:1"), torch.float32

        def is_contiguous(self):
            return True

        def dim(self):
            return 2

    with pytest.raises(ValueError, match="x is on cuda:1"):
        ops._check(FakeTensor(), "x", torch.float32, 2)

    entered = []

    class FakeGuard:
        def __init__(self, device):
            self.device = device

        def __enter__(self):
            entered.append(self.device)

        def __exit__(self, *exc):
            return False

    monkeypatch.setattr(torch.cuda, "device", FakeGuard)
    with step.device_guard("cuda:1"):
        pass
    with step.device_guard("cpu"):          # the stand-ins' device: nothing to enter
        pass
    assert entered == [torch.device("cuda:1")]


def test_no_kernel_reads_through_the_read_only_path():
    """Kernels run under programmatic dependent launch: a CTA may live while earlier kernels still write what
    it will read, so no load may take the read-only path (``ld.global.nc``), which promises unchanging data for
    the kernel's whole life (csrc/common.cuh).  Every source is compiled to PTX here and searched; the only such
    load allowed reads the constant table inside ``sincosf``."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not shutil.which(nvcc):
        pytest.skip("no nvcc on this machine")
    sources = sorted(set(build.LIBRARIES.values()))
    assert sources
    for name in sources:
        text = (build.CSRC / name).read_text()
        assert "__restrict__" not in text and "__ldg(" not in text, f"{name}: a read-only qualifier or load"
    procs = {name: subprocess.Popen([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-I", str(build.CSRC),
                                     "-ptx", str(build.CSRC / name), "-o", "/dev/stdout"],
                                    stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for name in sources}
    for name, proc in procs.items():
        ptx, err = proc.communicate(timeout=600)
        assert proc.returncode == 0, f"{name}: {err[-500:]}"
        lines = ptx.splitlines()
        bad = []
        for n, line in enumerate(lines):
            if "ld.global.nc" in line:
                address = line.split("[")[-1].split("]")[0].split("+")[0].strip()
                origin = [prev for prev in lines[max(0, n - 40):n] if address + "," in prev and "mov." in prev]
                if not (origin and "__cudart_i2opi_f" in origin[-1]):
                    bad.append(line.strip())
        assert not bad, f"{name}: read-only loads in the PTX: {bad[:3]}"
