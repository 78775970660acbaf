"""Building the kernel libraries (no GPU needed: nvcc cross-compiles): a library is compiled on first
use into the build folder, is current until its source changes, and a compiler error comes back
as one BuildError with the compiler's message."""

import ctypes

import pytest

from pyre_b200.kernels import build


@pytest.fixture
def scratch_build(tmp_path, monkeypatch):
    try:
        build.find_nvcc()
    except build.BuildError:
        pytest.skip("nvcc is not installed")
    monkeypatch.setattr(build, "_build_dir", tmp_path / "out")
    (tmp_path / "out").mkdir()
    monkeypatch.setattr(build, "LIBRARIES", dict(build.LIBRARIES))
    return tmp_path


def test_build_on_first_use_staleness_and_errors(scratch_build, capfd):
    src = scratch_build / "toy.cu"
    src.write_text('extern "C" __attribute__((visibility("default"))) int toy_answer() { return 41; }\n')
    build.register_library("toy", str(src))
    assert not build.is_current("toy")
    build.ensure_built(["toy"])
    assert build.is_current("toy") and build.library_path("toy").parent == scratch_build / "out"
    assert "compiling 1 CUDA library" in capfd.readouterr().err          # progress goes to stderr, never to stdout
    assert ctypes.CDLL(str(build.library_path("toy"))).toy_answer() == 41
    build.ensure_built(["toy"])                                          # nothing to do: no message
    assert capfd.readouterr().err == ""
    src.write_text(src.read_text().replace("41", "42"))                  # the source changed: stale, rebuilt
    assert not build.is_current("toy")
    build.ensure_built(["toy"], verbose=False)
    assert build.is_current("toy")
    src.write_text("this is not CUDA\n")
    with pytest.raises(build.BuildError, match=r"nvcc failed on .*toy\.cu[\s\S]*expected a declaration"):
        build.ensure_built(["toy"], verbose=False)
    assert not build.is_current("toy")
    with pytest.raises(build.BuildError, match="unknown kernel library"):
        build.ensure_built(["no_such_library"])


def test_every_library_names_a_source_and_the_flags_target_sm_100a():
    for name, source in build.LIBRARIES.items():
        assert (build.CSRC / source).is_file(), name
    for header in build.HEADERS:
        assert (build.CSRC / header).is_file(), header
    flags = " ".join(build.NVCC_FLAGS)
    assert "arch=compute_100a,code=sm_100a" in flags and "-lineinfo" in flags
