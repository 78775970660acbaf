"""The debug build of the kernels (``PYRE_DEBUG_CHECKS=1``): device-side range checks of every cache page
and slot a kernel takes from a block table or a slot mapping.  Here: the host side of it on the CPU (which
build is chosen, what the error word means), and on the GPU a VALID trace replayed under the debug build,
whose logits must equal the normal build's bit for bit with the error word left clear.  No test feeds a
kernel a bad table: the checks' failing branch is three lines read by eye (csrc/common.cuh), and a bad
page on a GPU is what they exist to avoid."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import helpers as H

ROOT = Path(__file__).resolve().parent.parent


def test_the_debug_build_is_a_build_of_its_own(monkeypatch):
    from pyre_b200.kernels import build
    monkeypatch.setattr(build, "DEBUG_CHECKS", False)
    plain_path, plain_print = build.library_path("elementwise"), build._fingerprint("elementwise")
    assert "-DPYRE_DEBUG_CHECKS" not in build._flags()
    monkeypatch.setattr(build, "DEBUG_CHECKS", True)
    assert "-DPYRE_DEBUG_CHECKS" in build._flags()
    assert build.library_path("elementwise").name == "libpyre_elementwise_dbg.so" != plain_path.name
    assert build._fingerprint("elementwise") != plain_print          # the flag is part of what makes a build current


def test_every_kernel_that_reads_a_table_checks_it():
    """Each dereference of a block table or of the slot mapping in the kernels goes through the checking helpers."""
    import re
    from pyre_b200.kernels import build
    for source, helper, least in (("attention_generic.cu", "pyre_checked_page", 1), ("attention_mma.cu", "pyre_checked_page", 3),
                                  ("attention_tc.cu", "pyre_checked_page", 1), ("attention_prefill.cu", "pyre_checked_page", 1),
                                  ("elementwise.cu", "pyre_checked_slot", 2)):
        text = re.sub(r"//[^\n]*", "", (build.CSRC / source).read_text())
        assert text.count(helper + "(") >= least, source
        for m in re.finditer(r"\btable\[|slot_mapping\[", text):
            line = text[text.rfind("\n", 0, m.start()) + 1:text.find("\n", m.start())]
            assert "pyre_checked_" in line, f"{source}: unchecked read: {line.strip()}"


def test_the_error_word_names_a_bad_page():
    from pyre_b200.kernels import ops
    assert "page" in ops.device_error_message(6) and "debug checks" in ops.device_error_message(6)
    assert "bounded wait" in ops.device_error_message(2)
    assert "code 77" in ops.device_error_message(77)
    assert sorted(ops.DEVICE_ERROR_MESSAGES) == [1, 2, 3, 4, 5, 6]


def _replay(model_dir, dtype, steps, out, page_size, debug):
    env = dict(os.environ, PYRE_DEBUG_CHECKS="1" if debug else "0")
    res = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out),
                          "--max-tokens", str(H.max_live_tokens(steps, max(64, page_size))), "--page-size", str(page_size),
                          "--poison-freed-pages"],
                         input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stdout.count("done ") == len(steps)
    return res


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["tiny fp32", "tiny bf16", "head size 64 bf16"])
def test_a_valid_trace_under_the_debug_build(tmp_path, case):
    """Mixed steps with pages used again (so the tables hold -1 entries outside the live ranges and reused page
    numbers), through every attention kernel: the debug build raises nothing and changes no logit."""
    if case.startswith("tiny"):
        raw, page, dtype = H.TINY["B"], 8, "float32" if "fp32" in case else "bfloat16"
        H.make_model_dir(tmp_path / "m", raw, seed=5)
        reqs = {f"r{i}": H.random_ids(raw["vocab_size"], n, seed=i) for i, n in enumerate((40, 63, 100, 7, 131))}
        steps = H.trace_mixed(dict(reqs, **{k + "x": v for k, v in reqs.items()}), seed=2, max_live=4)
    else:
        from test_big_shape_gpu import SCALES, SHAPES
        raw, page, dtype = SHAPES["hd64"], 16, "bfloat16"
        H.make_model_dir(tmp_path / "m", raw, seed=5, **SCALES["hd64"])
        reqs = {f"r{i}": H.random_ids(raw["vocab_size"], n, seed=i) for i, n in enumerate((300, 170, 45, 420))}
        steps = H.trace_mixed(dict(reqs, **{k + "x": v for k, v in reqs.items()}), seed=3, max_live=4, prefill_head=0.85,
                              portion=(30, 200))
    res = _replay(tmp_path / "m", dtype, steps, tmp_path / "dbg", page, debug=True)
    assert "with debug checks" in res.stderr or "compiling" not in res.stderr      # if anything was compiled, it was the debug build
    _replay(tmp_path / "m", dtype, steps, tmp_path / "plain", page, debug=False)
    files = sorted(p.name for p in (tmp_path / "plain").iterdir())
    assert files and files == sorted(p.name for p in (tmp_path / "dbg").iterdir())
    for name in files:
        a, b = np.fromfile(tmp_path / "plain" / name, dtype="<f4"), np.fromfile(tmp_path / "dbg" / name, dtype="<f4")
        assert np.isfinite(a).all() and np.array_equal(a, b), name
