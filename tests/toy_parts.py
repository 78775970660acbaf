"""Toy parts that exist only in the tests: defined here, registered through the package's public
calls, built and stepped without a change to the package's files.  The scenarios take the device, so
the same code runs on a B200 with the kernels and on the CPU with the plain stand-ins."""

import json
from dataclasses import dataclass
from typing import ClassVar

import torch

import helpers as H
from plain import qwen2_plain


def toy_decay_model_scenario(tmp_path, device):
    """A mixer that is no attention at all: a per-request running state
    s_t = decay * s_{t-1} + h_t W_in, output s_t W_out.  It is defined, registered and given an
    architecture of its own right here; the package's files are untouched.  Its state
    lives in the cache manager's slots, so a sequence cut into portions (and mixed with
    another request) gives what the whole sequence gives."""
    from pyre_b200.config import ModelConfig, config_from_dict, register_architecture
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.models import Model, ModelSpec
    from pyre_b200.parts import Part, PartSpec, StateSpec, register_part
    from pyre_b200.weights import TensorSpec, write_random_model

    class ToyDecayMixer(Part):
        def __init__(self, dtype, device, width, state_width, decay):
            super().__init__(dtype, device)
            self.width, self.state_width, self.decay = width, state_width, decay

        def tensors(self):
            return {"in_proj.weight": TensorSpec((self.state_width, self.width), init=("normal", 0.0, 0.2)),
                    "out_proj.weight": TensorSpec((self.width, self.state_width), init=("normal", 0.0, 0.2))}

        def load(self, tensors):
            self.w_in, self.w_out = tensors["in_proj.weight"].float(), tensors["out_proj.weight"].float()

        def cache_spec(self):
            return None

        def state_spec(self):
            return StateSpec((self.state_width,), torch.float32)

        def forward(self, ctx, h, call):
            view = ctx.state_group(call.state_group)
            u = h.float() @ self.w_in.t()
            out = torch.empty_like(u)
            cu = ctx.cu_seqlens_host
            for b in range(ctx.num_seqs):                       # rows of one request in order
                s = view.buffer[call.state_layer, int(view.slots_host[b])]
                for t in range(cu[b], cu[b + 1]):
                    s.mul_(self.decay).add_(u[t])
                    out[t] = s
            return (out @ self.w_out.t()).to(self.dtype)

    register_part("mixer", "toy_decay", ToyDecayMixer, replace=True)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyDecayForCausalLM"
        width: int = 24
        layers: int = 2
        vocab: int = 50
        state_width: int = 10
        decays: tuple = (0.5, 0.9)

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["width"], raw["layers"], raw["vocab"], raw["state_width"], tuple(raw["decays"]))

    def build_toy(cfg):
        norm = PartSpec("rms_norm", {"width": cfg.width, "eps": 1e-5})
        blocks = [PartSpec("prenorm", {
            "norm1": norm, "norm2": norm,
            "mixer": PartSpec("toy_decay", {"width": cfg.width, "state_width": cfg.state_width, "decay": cfg.decays[i]}),
            "ffn": PartSpec("gated_mlp", {"width": cfg.width, "intermediate": 40}),
            "names": {"mixer": "mixer."}}) for i in range(cfg.layers)]
        return ModelSpec(embed=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": cfg.width}), blocks=blocks,
                         final_norm=norm, head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width}),
                         vocab_size=cfg.vocab, max_positions=4096)

    register_architecture("ToyDecayForCausalLM", ToyConfig, build_toy, replace=True)

    cfg = ToyConfig()
    write_random_model(tmp_path, cfg, seed=1)                    # the random-weights mode knows the new parts
    assert config_from_dict(json.loads((tmp_path / "config.json").read_text())) == cfg
    from safetensors.torch import load_file
    w = load_file(str(tmp_path / "model.safetensors"))
    assert "model.layers.1.mixer.in_proj.weight" in w and len(w) == 2 * 7 + 3

    def plain(ids):
        x = w["model.embed_tokens.weight"][ids]
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            h = qwen2_plain.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
            u = h @ w[p + "mixer.in_proj.weight"].t()
            s, rows = torch.zeros(cfg.state_width), []
            for t in range(len(ids)):
                s = cfg.decays[i] * s + u[t]
                rows.append(s)
            x = x + torch.stack(rows) @ w[p + "mixer.out_proj.weight"].t()
            h = qwen2_plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
            x = x + qwen2_plain.swiglu_mlp(h, w, p + "mlp.")
        return qwen2_plain.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].t()

    from pyre_b200.config import architecture_of
    model = Model(architecture_of(cfg).build(cfg), torch.float32, device)
    assert model.kv_groups == [] and len(model.state_groups) == 1 and model.state_groups[0].n_layers == 2
    model.load_weights(tmp_path)
    cache, stepper = runtime_for_model(model, 64, 16, max_requests=3)
    a, b = H.random_ids(50, 23, seed=1), H.random_ids(50, 9, seed=2)
    cache.begin("a"); cache.begin("b")
    got_a = [stepper.step([StepEntry("a", a[:7], list(range(7)))])]
    both = stepper.step([StepEntry("b", b[:4], list(range(4))), StepEntry("a", a[7:9], [0, 1])])
    got_b, got_a = [both[:4]], got_a + [both[4:]]
    both = stepper.step([StepEntry("a", a[9:], list(range(14))), StepEntry("b", b[4:], list(range(5)))])
    got_a.append(both[:14]); got_b.append(both[14:])
    torch.testing.assert_close(torch.cat(got_a).cpu(), plain(a), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(torch.cat(got_b).cpu(), plain(b), rtol=1e-4, atol=1e-5)
    # a slot is zeroed for its next owner
    cache.end("a"); cache.begin("c")
    got_c = stepper.step([StepEntry("c", b, list(range(9)))])
    torch.testing.assert_close(got_c.cpu(), plain(b), rtol=1e-4, atol=1e-5)


def toy_routed_model_scenario(tmp_path, device):
    """Three more parts that exist only here: a feed-forward that routes every token to the one of
    three small experts with the largest router logit (fp32 logits); a position encoding whose
    angles grow with the square root of the position (a rotation, through the package's fused kernel
    with tables of its own); and one that is no rotation at all (layer 1: queries and keys are
    multiplied, dimension by dimension, by a gain that depends on the position).  They are registered
    from this test, put into blocks beside the package's own attention part (which takes a position
    encoding as its ``position`` parameter and knows nothing about it) and norms, written as a random
    model, loaded and stepped in portions against a plain evaluation.  No file of the package changes."""
    from pyre_b200.config import ModelConfig, register_architecture, architecture_of
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.models import Model, ModelSpec
    from pyre_b200.kernels import ops
    from pyre_b200.parts import Part, PartSpec, PositionEncoding, register_part
    from pyre_b200.weights import TensorSpec, write_random_model

    class ToyRoutedFFN(Part):
        def __init__(self, dtype, device, width, inner, experts):
            super().__init__(dtype, device)
            self.width, self.inner, self.experts = width, inner, experts

        def tensors(self):
            t = {"router.weight": TensorSpec((self.experts, self.width), role="keep", init=("normal", 0.0, 1.0))}
            for e in range(self.experts):
                t[f"experts.{e}.up.weight"] = TensorSpec((self.inner, self.width), init=("normal", 0.0, 0.3))
                t[f"experts.{e}.down.weight"] = TensorSpec((self.width, self.inner), init=("normal", 0.0, 0.3))
            return t

        def load(self, tensors):
            self.router = tensors["router.weight"].float()
            self.up = [tensors[f"experts.{e}.up.weight"].float() for e in range(self.experts)]
            self.down = [tensors[f"experts.{e}.down.weight"].float() for e in range(self.experts)]

        def forward(self, ctx, h):
            x = h.float()
            choice = (x @ self.router.t()).argmax(dim=-1)            # router logits in fp32
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = torch.relu(x[rows] @ self.up[e].t()) @ self.down[e].t()
            return out.to(self.dtype)

    class ToySqrtPositions(PositionEncoding):
        """A rotation by sqrt(position) * inv_freq: tables of its own into the package's fused kernel."""
        def __init__(self, dtype, device, head_dim, theta):
            super().__init__(dtype, device)
            self.rotary_dim = head_dim
            self.inv_freq = (1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).to(self.device)

        def kernel_libraries(self):
            return ["elementwise"]

        def apply(self, ctx, qkv, bias, heads, kv, cache_layer):
            key = ("toy_sqrt", self.rotary_dim)
            if key not in ctx.scratch:
                ang = ctx.positions.float().sqrt()[:, None] * self.inv_freq[None, :]
                ctx.scratch[key] = (ang.cos().contiguous(), ang.sin().contiguous())
            cos, sin = ctx.scratch[key]
            return ops.qkv_rope_write(qkv, bias, cos, sin, cache_layer, kv.slot_mapping, heads.n_heads, heads.n_kv_heads,
                                      heads.head_dim, self.rotary_dim, kv.page_size)

    def toy_gain(positions, head_dim):
        """gain[t, d] = 1 + 0.4 sin(0.37 position + d): no rotation, nothing a cos/sin table could express."""
        d = torch.arange(head_dim, dtype=torch.float32, device=positions.device)
        return 1.0 + 0.4 * torch.sin(0.37 * positions.float()[:, None] + d[None, :])

    class ToyGainPositions(PositionEncoding):
        """Not a rotation: q and k are scaled per dimension by a gain that depends on the position.  It transforms
        the projections itself (plain torch: this is a test's part) and uses the base class's ``store``."""
        def __init__(self, dtype, device, head_dim):
            super().__init__(dtype, device)
            self.head_dim = head_dim

        def kernel_libraries(self):
            return ["elementwise"]

        def apply(self, ctx, qkv, bias, heads, kv, cache_layer):
            x = ops.materialize(qkv).float() + bias
            T = x.shape[0]
            x = x.view(T, heads.n_heads + 2 * heads.n_kv_heads, heads.head_dim)
            gain = toy_gain(ctx.positions, heads.head_dim)[:, None, :]
            x[:, :heads.n_heads + heads.n_kv_heads] *= gain                       # queries and keys; values pass
            return self.store(x.reshape(T, -1).to(self.dtype).contiguous(), None, heads, kv, cache_layer)

    register_part("ffn", "toy_routed", ToyRoutedFFN, replace=True)
    register_part("position", "toy_sqrt", ToySqrtPositions, replace=True)
    register_part("position", "toy_gain", ToyGainPositions, replace=True)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyRoutedForCausalLM"
        width: int = 40
        layers: int = 2
        vocab: int = 61
        heads: int = 5
        kv_heads: int = 1
        head_dim: int = 16
        experts: int = 3

        @classmethod
        def from_dict(cls, raw):
            return cls(*(raw[k] for k in ("width", "layers", "vocab", "heads", "kv_heads", "head_dim", "experts")))

    def build_toy(cfg):
        norm = PartSpec("rms_norm", {"width": cfg.width, "eps": 1e-5})
        blocks = [PartSpec("prenorm", {
            "norm1": norm, "norm2": norm,
            "mixer": PartSpec("attention", {"width": cfg.width, "n_heads": cfg.heads, "n_kv_heads": cfg.kv_heads,
                                            "head_dim": cfg.head_dim, "qkv_bias": True, "o_bias": False, "window": None,
                                            "position": PartSpec("toy_sqrt", {"head_dim": cfg.head_dim, "theta": 100.0}) if i == 0
                                            else PartSpec("toy_gain", {"head_dim": cfg.head_dim})}),
            "ffn": PartSpec("toy_routed", {"width": cfg.width, "inner": 24, "experts": cfg.experts})})
            for i in range(cfg.layers)]
        return ModelSpec(embed=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": cfg.width}), blocks=blocks,
                         final_norm=norm, head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width}),
                         vocab_size=cfg.vocab, max_positions=4096)

    register_architecture("ToyRoutedForCausalLM", ToyConfig, build_toy, replace=True)
    cfg = ToyConfig()
    write_random_model(tmp_path, cfg, seed=3)
    from safetensors.torch import load_file
    w = load_file(str(tmp_path / "model.safetensors"))
    assert "model.layers.1.mlp.experts.2.down.weight" in w and w["model.layers.0.mlp.router.weight"].dtype == torch.float32

    def plain(ids):
        T = len(ids)
        x = w["model.embed_tokens.weight"].float()[ids]
        inv = 1.0 / (100.0 ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        ang = torch.arange(T, dtype=torch.float32).sqrt()[:, None] * inv[None, :]
        cos, sin = torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1)
        rot = lambda v: torch.cat([-v[..., cfg.head_dim // 2:], v[..., :cfg.head_dim // 2]], -1)
        used = set()
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            h = qwen2_plain.rms_norm(x, w[p + "input_layernorm.weight"].float(), 1e-5)
            q = (h @ w[p + "self_attn.q_proj.weight"].float().t() + w[p + "self_attn.q_proj.bias"].float()).view(T, cfg.heads, cfg.head_dim)
            k = (h @ w[p + "self_attn.k_proj.weight"].float().t() + w[p + "self_attn.k_proj.bias"].float()).view(T, cfg.kv_heads, cfg.head_dim)
            v = (h @ w[p + "self_attn.v_proj.weight"].float().t() + w[p + "self_attn.v_proj.bias"].float()).view(T, cfg.kv_heads, cfg.head_dim)
            if i == 0:
                q, k = q * cos[:, None] + rot(q) * sin[:, None], k * cos[:, None] + rot(k) * sin[:, None]
            else:
                gain = toy_gain(torch.arange(T), cfg.head_dim)[:, None, :]
                q, k = q * gain, k * gain
            k, v = k.repeat_interleave(cfg.heads // cfg.kv_heads, 1), v.repeat_interleave(cfg.heads // cfg.kv_heads, 1)
            s = torch.einsum("qhd,khd->hqk", q, k) * cfg.head_dim ** -0.5
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, -1)
            x = x + a @ w[p + "self_attn.o_proj.weight"].float().t()
            h = qwen2_plain.rms_norm(x, w[p + "post_attention_layernorm.weight"].float(), 1e-5)
            choice = (h @ w[p + "mlp.router.weight"].float().t()).argmax(-1)
            used |= set(choice.tolist())
            y = torch.stack([torch.relu(h[t] @ w[p + f"mlp.experts.{int(c)}.up.weight"].float().t())
                             @ w[p + f"mlp.experts.{int(c)}.down.weight"].float().t() for t, c in enumerate(choice)])
            x = x + y
        return qwen2_plain.rms_norm(x, w["model.norm.weight"].float(), 1e-5) @ w["lm_head.weight"].float().t(), used

    model = Model(architecture_of(cfg).build(cfg), torch.float32, device)
    assert len(model.kv_groups) == 1 and model.state_groups == []
    model.load_weights(tmp_path)
    cache, stepper = runtime_for_model(model, 64, 16, max_requests=2)
    a, b = H.random_ids(cfg.vocab, 37, seed=5), H.random_ids(cfg.vocab, 11, seed=6)
    cache.begin("a"); cache.begin("b")
    got_a = [stepper.step([StepEntry("a", a[:18], list(range(18)))])]
    both = stepper.step([StepEntry("b", b, list(range(11))), StepEntry("a", a[18:20], [0, 1])])
    got_b, got_a = both[:11], got_a + [both[11:]]
    got_a.append(stepper.step([StepEntry("a", a[20:], list(range(17)))]))
    want_a, used = plain(a)
    want_b, _ = plain(b)
    assert len(used) >= 2                                              # the router really routes
    torch.testing.assert_close(torch.cat(got_a).cpu(), want_a, rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(got_b.cpu(), want_b, rtol=2e-4, atol=2e-5)
