"""The plain implementation against outputs of the reference's own model code
(``pyre.model.PyreQwen2`` on the CPU in fp32), committed under tests/golden/ together with
the script that made them."""

import json
from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

from plain import qwen2_plain

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["tiny_untied", "tiny_tied"])
def test_plain_matches_reference_outputs(name):
    d = GOLDEN / name
    raw = json.loads((d / "config.json").read_text())
    w = load_file(str(d / "model.safetensors"))
    gold = load_file(str(d / "golden.safetensors"))
    with torch.inference_mode():
        logits = qwen2_plain.forward(gold["ids"].tolist(), w, raw)
    assert logits.shape == gold["logits"].shape
    # same formulas, same order of operations, same library on the same kind of machine:
    # the difference was 0.0 when the files were made; allow the last bit of other BLAS builds
    assert (logits - gold["logits"]).abs().max().item() <= 2e-6
    n = int(gold["greedy_prompt_len"][0])
    out = qwen2_plain.greedy_generate(gold["ids"][:n].tolist(), w, raw, len(gold["greedy_tokens"]))
    assert out == gold["greedy_tokens"].tolist()


def test_schedule_and_window_defaults_are_the_reference_model():
    d = GOLDEN / "tiny_untied"
    raw = json.loads((d / "config.json").read_text())
    w = load_file(str(d / "model.safetensors"))
    ids = load_file(str(d / "golden.safetensors"))["ids"].tolist()
    base = qwen2_plain.forward(ids, w, raw)
    L = raw["num_hidden_layers"]
    same = qwen2_plain.forward(ids, w, raw, schedule=[(i, None) for i in range(L)], windows=[None] * L)
    assert torch.equal(base, same)
    # a window as long as the sequence changes nothing; a short one does
    wide = qwen2_plain.forward(ids, w, raw, windows=[len(ids)] * L)
    assert torch.allclose(base, wide, atol=1e-6)
    narrow = qwen2_plain.forward(ids, w, raw, windows=[4] * L)
    assert torch.allclose(base[:4], narrow[:4], atol=1e-6)
    assert not torch.allclose(base[8:], narrow[8:], atol=1e-4)


def test_gumbel_sampler_statistics():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    assert qwen2_plain.sample(logits, 0.0, 0, 0) == 2
    counts = [0] * 4
    for i in range(3000):
        counts[qwen2_plain.sample(logits, 1.0, 5, i)] += 1
    p = torch.softmax(logits, 0)
    for c, q in zip(counts, p.tolist()):
        assert abs(c / 3000 - q) < 0.03
