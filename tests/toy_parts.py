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
