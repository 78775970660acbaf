"""Makes the golden files of this folder from the reference's own model code.

Run once, on the CPU, with the reference on the path (it is imported, never copied):

    PYTHONPATH=<checkout of Lalitaditya-tickoo/pyre> PYTHONDONTWRITEBYTECODE=1 HF_HUB_OFFLINE=1 \
        python tests/golden/make_golden.py

For each of two tiny random Qwen2 models it writes ``<name>/config.json``,
``<name>/model.safetensors`` (fp32, checkpoint names) and ``<name>/golden.safetensors``
with the token ids and the fp32 logits of ``pyre.model.PyreQwen2.forward`` on the whole
sequence (no cache), plus the tokens of ``generate_greedy``.  It also runs the plain
implementation of ``tests/plain`` on the same weights and prints the largest difference;
``tests/test_plain_vs_golden.py`` repeats that comparison from the committed files, so
the reference is not needed again.
"""

import json
import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

MODELS = {
    "tiny_untied": dict(hidden_size=40, intermediate_size=56, num_hidden_layers=2, num_attention_heads=2,
                        num_key_value_heads=1, head_dim=16, vocab_size=96, rms_norm_eps=1e-5, rope_theta=1e6,
                        tie_word_embeddings=False, max_position_embeddings=128),
    "tiny_tied": dict(hidden_size=48, intermediate_size=80, num_hidden_layers=3, num_attention_heads=3,
                      num_key_value_heads=3, vocab_size=70, rms_norm_eps=1e-6, rope_theta=10000.0,
                      tie_word_embeddings=True, max_position_embeddings=64),
}


def random_weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or H // nh

    def mat(*shape):
        return torch.randn(*shape, generator=g) * 0.05

    w = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = 1 + 0.1 * torch.randn(H, generator=g)
        w[p + "self_attn.q_proj.weight"] = mat(nh * hd, H)
        w[p + "self_attn.q_proj.bias"] = mat(nh * hd)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.k_proj.bias"] = mat(nkv * hd)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.v_proj.bias"] = mat(nkv * hd)
        w[p + "self_attn.o_proj.weight"] = mat(H, nh * hd)
        w[p + "post_attention_layernorm.weight"] = 1 + 0.1 * torch.randn(H, generator=g)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = 1 + 0.1 * torch.randn(H, generator=g)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, H)
    return w


def main():
    from pyre.loader import load_model  # the reference
    from plain import qwen2_plain

    for n, (name, cfg) in enumerate(MODELS.items()):
        out = HERE / name
        out.mkdir(exist_ok=True)
        raw = dict(cfg, architectures=["Qwen2ForCausalLM"])
        (out / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
        w = random_weights(cfg, 1234 + n)
        save_file(w, str(out / "model.safetensors"))
        model, _ = load_model(str(out), device="cpu", dtype=torch.float32)
        g = torch.Generator().manual_seed(99 + n)
        ids = torch.randint(0, cfg["vocab_size"], (1, 37), generator=g)
        with torch.inference_mode():
            logits = model(ids)[0].clone()
            greedy = model.generate_greedy(ids[:, :9], max_new_tokens=12)[0, 9:].clone()
        save_file({"ids": ids[0].to(torch.int32), "logits": logits.contiguous(),
                   "greedy_prompt_len": torch.tensor([9], dtype=torch.int32),
                   "greedy_tokens": greedy.to(torch.int32)}, str(out / "golden.safetensors"))
        mine = qwen2_plain.forward(ids[0], w, raw)
        print(f"{name}: reference logits {tuple(logits.shape)}, max |plain - reference| = "
              f"{(mine - logits).abs().max().item():.3e}, max |logit| = {logits.abs().max().item():.3f}")
        mine_greedy = qwen2_plain.greedy_generate(ids[0, :9].tolist(), w, raw, 12)
        print(f"{name}: greedy tokens equal: {mine_greedy == greedy.tolist()}")


if __name__ == "__main__":
    main()
