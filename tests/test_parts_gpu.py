"""Each part of a layer alone against the plain implementation's function for it; the
schedule as data (a layer run twice, a layer that reads another layer's cache); layers
with a window beside layers without (two cache groups); and a toy mixer with state of
its own, defined here, registered, built and stepped without any change to the package."""

from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers as H
from plain import qwen2_plain

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype, roundings=1):
    """Largest error against the size of the part's output.  float32: sums in another order,
    1e-5 of the largest output.  bfloat16: every tensor the part rounds to bf16 on the way
    (``roundings`` of them) may be off by 2^-8 relative, so the bound is that many times
    0.4 % of the largest output."""
    bound = (1e-5 if dtype == torch.float32 else roundings * 2.0 ** -8) * float(want.abs().max())
    err = (got.float().cpu() - want).abs()
    assert float(err.max()) <= bound, f"max error {float(err.max()):.3e} > {bound:.3e} (output max {float(want.abs().max()):.3f})"


def mini_context(dtype, token_ids=None, positions=None):
    from pyre_b200.engine.context import StepContext
    n = len(positions if positions is not None else token_ids)
    z = torch.zeros(n, dtype=torch.int32, device="cuda")
    return StepContext(dtype=dtype, device=torch.device("cuda"), num_tokens=n, num_seqs=1, num_logit_rows=0,
                       token_ids=torch.tensor(token_ids or [0] * n, dtype=torch.int32, device="cuda"),
                       positions=torch.tensor(positions or list(range(n)), dtype=torch.int32, device="cuda"),
                       seq_of_token=z, cu_seqlens=torch.tensor([0, n], dtype=torch.int32, device="cuda"),
                       logit_rows=z[:0], cu_seqlens_host=np.array([0, n]),
                       start_pos_host=np.array([positions[0] if positions is not None else 0]),
                       error_flag=torch.zeros(1, dtype=torch.int32, device="cuda"))


def make(category, kind, dtype, **params):
    from pyre_b200.parts import PartSpec, make_part
    return make_part(category, PartSpec(kind, params), dtype, "cuda")


def load_random(part, seed, scale=0.3):
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, spec in part.tensors().items():
        t = torch.randn(spec.shape, generator=g) * scale
        if spec.role == "vector":
            tensors[name] = (t + (1.0 if name == "weight" else 0.0)).cuda()
        else:
            tensors[name] = t.to(part.dtype).cuda()
    part.load(dict(tensors))
    return {k: v.float().cpu() for k, v in tensors.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    norm = make("norm", "rms_norm", dtype, width=120, eps=3e-6)
    w = load_random(norm, 0)
    x = torch.randn(9, 120, device="cuda") * 2
    delta = torch.randn(9, 120, device="cuda").to(dtype)
    want = qwen2_plain.rms_norm((x + delta.float()).cpu(), w["weight"], 3e-6)
    got = norm.forward(mini_context(dtype, positions=list(range(9))), x, delta=delta)
    close(got, want, dtype)


@pytest.mark.parametrize("head_dim,theta", [(16, 1e4), (48, 5e4), (128, 1e6)])
def test_rotary_part(head_dim, theta):
    rot = make("position", "rotary", torch.float32, head_dim=head_dim, theta=theta)
    pos = [0, 1, 2, 77, 4095, 32767]
    ctx = mini_context(torch.float32, positions=pos)
    cos, sin = rot.tables(ctx)
    want_cos, want_sin = qwen2_plain.rope_tables(torch.tensor(pos), head_dim, theta, torch.float32)
    torch.testing.assert_close(cos.cpu(), want_cos[:, :head_dim // 2], rtol=1e-5, atol=2e-6)
    torch.testing.assert_close(sin.cpu(), want_sin[:, :head_dim // 2], rtol=1e-5, atol=2e-6)
    assert rot.tables(ctx)[0] is cos          # computed once per step, shared by the layers


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    ffn = make("ffn", "gated_mlp", dtype, width=72, intermediate=200)
    w = load_random(ffn, 1)
    h = torch.randn(11, 72, device="cuda").to(dtype)
    want = qwen2_plain.swiglu_mlp(h.float().cpu(), w, "")
    from pyre_b200.kernels import ops
    got = ops.materialize(ffn.forward(mini_context(dtype, positions=list(range(11))), h))
    close(got, want, dtype, roundings=4)      # input, gate/up, activation, output


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    emb = make("embed", "token_embedding", dtype, vocab=333, width=40)
    w = load_random(emb, 2)
    ids = [0, 332, 7, 7]
    x = emb.forward(mini_context(dtype, token_ids=ids))
    assert x.dtype == torch.float32 and torch.equal(x.cpu(), w["weight"][ids])
    head = make("head", "linear_head", dtype, vocab=333, width=40)
    wh = load_random(head, 3)
    h = torch.randn(3, 40, device="cuda").to(dtype)
    logits = head.forward(None, h)
    assert logits.dtype == torch.float32
    close(logits, h.float().cpu() @ wh["weight"].t(), torch.float32)      # fp32 logits from the accumulator in both modes


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (6, 3, 48, 7), (3, 1, 32, None)])
def test_attention_part(dtype, nh, nkv, hd, window):
    """The mixer alone, fed in two portions through its paged cache, against the plain
    projections + rotary + attention + output projection on the whole sequence."""
    from pyre_b200.cache import CacheManager
    from pyre_b200.engine.context import KVView
    from pyre_b200.kernels import ops
    from pyre_b200.parts import BoundCall, PartSpec
    width, S, page = 56, 29, 8
    att = make("mixer", "attention", dtype, width=width, n_heads=nh, n_kv_heads=nkv, head_dim=hd, window=window,
               position=PartSpec("rotary", {"head_dim": hd, "theta": 1e4}))
    w = load_random(att, 4, scale=0.15)
    h = torch.randn(S, width, device="cuda").to(dtype)

    hf = h.float().cpu()
    q, k, v = qwen2_plain.project_qkv(hf, w, "", nh, nkv, hd)
    cos, sin = qwen2_plain.rope_tables(torch.arange(S), hd, 1e4, torch.float32)
    a = qwen2_plain.attention(qwen2_plain.apply_rope(q, cos, sin), qwen2_plain.apply_rope(k, cos, sin), v, window)
    want = a @ w["o_proj.weight"].t()

    @dataclass(frozen=True)
    class G:
        spec: object
        n_layers: int
    cache = CacheManager([G(att.cache_spec(), 1)], [], page, 16, 2, dtype, "cuda")
    cache.begin("r")
    outs = []
    for start, n in ((0, 18), (18, 11)):
        assert cache.reserve("r", start + n)
        ctx = mini_context(dtype, positions=list(range(start, start + n)))
        table = torch.from_numpy(cache.block_table_rows(0, ["r"])).cuda()
        slots = torch.from_numpy(cache.slots_for(0, "r", start, n)).cuda()
        ctx.kv_groups.append(KVView(cache.groups[0].pool, table, slots, page, window))
        outs.append(ops.materialize(att.forward(ctx, h[start:start + n].contiguous(), BoundCall(0, 0, 0, 0, True))))
        cache.commit("r", start + n)
    got = torch.cat(outs).float().cpu()
    close(got, want, dtype, roundings=5)      # qkv, rotated q and k, v, attention output, result


# --------------------------------------------------------------------------- whole models from specs
def run_spec(spec, model_dir, dtype, ids, portions, page_size=8, max_tokens=256):
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import build
    from pyre_b200.models import Model
    model = Model(spec, dtype, "cuda")
    build.ensure_built(model.kernel_libraries())
    model.load_weights(model_dir)
    cache, stepper = runtime_for_model(model, max_tokens, page_size, poison=True)
    cache.begin("r")
    out, pos = [], 0
    for n in portions:
        out.append(stepper.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).cpu())
        pos += n
    assert pos == len(ids)
    cache.end("r")
    cache.check()
    return torch.cat(out).numpy(), cache


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_is_data(tmp_path, dtype):
    """Layer 0 runs twice (each run with a cache layer of its own) and the last entry runs
    layer 1's weights again on the keys and values that layer 1's first run stored."""
    from pyre_b200.config import architecture, config_from_dict
    from pyre_b200.models import LayerCall
    from pyre_b200.config import parse_dtype
    raw = H.TINY_A
    H.make_model_dir(tmp_path, raw, seed=21)
    cfg = config_from_dict(raw)
    spec = architecture("Qwen2ForCausalLM").build(cfg)
    spec.schedule = [LayerCall(0), LayerCall(1, cache="shared"), LayerCall(0), LayerCall(1, cache="shared", write=False)]
    ids = H.random_ids(raw["vocab_size"], 45, seed=4)
    got, cache = run_spec(spec, tmp_path, parse_dtype(dtype), ids, [20, 2, 23])
    assert cache.groups[0].n_layers == 3                     # three cache layers for four entries
    w = H.load_plain_weights(tmp_path, round_matrices_to_bf16=(dtype == "bfloat16"))
    with torch.inference_mode():
        want = qwen2_plain.forward(ids, w, raw, schedule=[(0, None), (1, None), (0, None), (1, 1)]).numpy()
    assert np.abs(got - want).max() <= (2e-4 if dtype == "float32" else 0.08)
    with pytest.raises(ValueError, match="before any entry wrote"):
        spec.schedule = [LayerCall(0, cache="x", write=False), LayerCall(1)]
        from pyre_b200.models import Model
        Model(spec, torch.float32, "cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_layers_beside_full_layers(tmp_path, dtype):
    """Layer 1 of three attends over a window of 11 keys: it gets a cache group of its own
    whose pages are given back as the window passes them; logits equal the plain
    implementation's with the same window, whole and in portions that straddle its edge."""
    from pyre_b200.config import architecture, config_from_dict, parse_dtype
    from pyre_b200.parts import PartSpec
    raw = H.TINY_B
    H.make_model_dir(tmp_path, raw, seed=22)
    spec = architecture("Qwen2ForCausalLM").build(config_from_dict(raw))
    b = spec.blocks[1]
    mixer = PartSpec("attention", dict(b.params["mixer"].params, window=11))
    spec.blocks[1] = PartSpec(b.kind, dict(b.params, mixer=mixer))
    ids = H.random_ids(raw["vocab_size"], 90, seed=5)
    w = H.load_plain_weights(tmp_path, round_matrices_to_bf16=(dtype == "bfloat16"))
    with torch.inference_mode():
        want = qwen2_plain.forward(ids, w, raw, windows=[None, 11, None]).numpy()
    bound = 2e-4 if dtype == "float32" else 0.08
    for portions in ([90], [40] + [1] * 50, [3, 9, 2, 30, 11, 12, 23]):
        got, cache = run_spec(spec, tmp_path, parse_dtype(dtype), ids, portions, page_size=4, max_tokens=128)
        err = np.abs(got - want).max(axis=1)
        assert err.max() <= bound, f"portions {portions[:4]}...: first wrong position {int(np.where(err > bound)[0][0])}"
        assert len(cache.groups) == 2 and cache.groups[1].spec.window == 11
    # while decoding, the windowed group holds only the pages its window touches
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.models import Model
    model = Model(spec, parse_dtype(dtype), "cuda")
    model.load_weights(tmp_path)
    cache, stepper = runtime_for_model(model, 128, 4)
    cache.begin("r")
    stepper.step([StepEntry("r", ids[:60], [])])
    assert cache.groups[0].pages_held("r") == 15 and cache.groups[1].pages_held("r") <= 4


# --------------------------------------------------------------------------- a toy mixer with state
def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A recurrent toy mixer with state of its own and an architecture of its own (``tests/toy_parts.py``),
    stepped in portions beside another request through the package's step function on the device."""
    import toy_parts
    toy_parts.toy_decay_model_scenario(tmp_path, "cuda")


# --------------------------------------------------------------------------- a toy routed feed-forward and a toy position encoding
def test_toy_routed_ffn_and_toy_positions_beside_real_attention(tmp_path):
    """A toy routed feed-forward and a toy position encoding (``tests/toy_parts.py``) in blocks beside the
    package's own attention part, stepped in portions on the device against a plain evaluation."""
    import toy_parts
    toy_parts.toy_routed_model_scenario(tmp_path, "cuda")


# --------------------------------------------------------------------------- a windowed group with a small pool, through the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_gives_a_windowed_group_a_smaller_pool(tmp_path, dtype):
    """An architecture of this test's own (the decoder with a window of 20 keys on its middle layer) generates through
    ``Engine``: the windowed layer's cache group gets a pool a fraction the size of the other group's, several
    requests decode far beyond what that pool could hold without a window, and the tokens are the plain
    implementation's with the same window."""
    from pyre_b200 import Engine, SamplingParams
    from pyre_b200.config import architecture, register_architecture
    from pyre_b200.config.model_config import Qwen2Config
    from pyre_b200.parts import PartSpec

    def build(cfg):
        spec = architecture("Qwen2ForCausalLM").build(cfg)
        b = spec.blocks[1]
        spec.blocks[1] = PartSpec(b.kind, dict(b.params, mixer=PartSpec("attention", dict(b.params["mixer"].params, window=20))))
        return spec

    @dataclass(frozen=True)
    class WindowedConfig(Qwen2Config):
        architecture = "ToyWindowedForCausalLM"

    register_architecture("ToyWindowedForCausalLM", WindowedConfig, build, replace=True)
    raw = dict(H.TINY_B, architectures=["ToyWindowedForCausalLM"])
    H.make_model_dir(tmp_path, raw, seed=31)
    prompts = [H.random_ids(raw["vocab_size"], n, seed=90 + n) for n in (50, 9, 33)]
    eng = Engine(tmp_path, dtype=dtype, page_size=4, num_pages=120, max_num_seqs=3, max_num_batched_tokens=32, prefill_chunk=16,
                 debug_poison_freed_pages=True)
    full, windowed = eng.cache.groups
    assert windowed.spec.window == 20 and full.num_pages == 120
    assert windowed.num_pages == 3 * (-(-(19 + 16) // 4) + 1) == 30          # 120 tokens for three requests of up to 110
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=60))
    assert eng.stats()["preempted"] == 0
    eng.cache.check()
    w = H.load_plain_weights(tmp_path, round_matrices_to_bf16=(dtype == "bfloat16"))
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 60
        with torch.inference_mode():
            logits = qwen2_plain.forward(list(p) + o.token_ids[:-1], w, raw, windows=[None, 20, None]).numpy()
        for k, tok in enumerate(o.token_ids):
            row = logits[len(p) - 1 + k]
            if dtype == "float32":
                assert tok == int(row.argmax()), f"token {k}"
            else:
                assert row[tok] >= row.max() - 0.08, f"token {k}: {row[tok]:.4f} against the best {row.max():.4f}"
