"""The packed W4A16 checkpoint format and a seeded synthetic checkpoint in that format.

Format (the reference defines it by its dequantiser, src/quant/checkpoint.py:23-36):

* ``<prefix>.weight_packed``      int32 [N, K/8]   weight k = 8j+i is nibble i (bits 4i..4i+3) of word j
* ``<prefix>.weight_zero_point``  int32 [N/8, K/G] row n lives in word n//8, nibble n%8
* ``<prefix>.weight_scale``       fp16  [N, K/G]
* ``<prefix>.weight_shape``       int64 [2] (ignored by the reference)
* ``w[n, k] = (q[n, k] - zp[n, k//G]) * scale[n, k//G]``

Real Qwen2.5-0.5B weights cannot be downloaded where this project is built and measured,
so every test and benchmark uses ``synthetic_checkpoint``: the Qwen2.5-0.5B architecture
with int4 values, zero points and scales drawn as the benchmark configuration prescribes.
"""

from __future__ import annotations

import json
import os

import torch

QUANT_SUFFIXES = (".weight_packed", ".weight_scale", ".weight_zero_point", ".weight_shape")

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, GROUP = 896, 14, 2, 64, 4864, 128

# (module name, N, K, has bias) of the seven linears of a decoder layer
LAYER_LINEARS = (
    ("self_attn.q_proj", HEADS * HEAD_DIM, HIDDEN, True),
    ("self_attn.k_proj", KV_HEADS * HEAD_DIM, HIDDEN, True),
    ("self_attn.v_proj", KV_HEADS * HEAD_DIM, HIDDEN, True),
    ("self_attn.o_proj", HIDDEN, HEADS * HEAD_DIM, False),
    ("mlp.gate_proj", INTER, HIDDEN, False),
    ("mlp.up_proj", INTER, HIDDEN, False),
    ("mlp.down_proj", HIDDEN, INTER, False),
)


def packed_prefixes(weights: dict) -> set:
    """Module names that carry packed int4 weights (same role as checkpoint.py:8)."""
    tail = ".weight_packed"
    return {name[: -len(tail)] for name in weights if name.endswith(tail)}


def detect_group_size(raw_config: dict, default: int = 32) -> int:
    """Group size from a ``quantization_config`` block; looks at the top level and at the
    compressed-tensors ``config_groups`` (same lookup order as checkpoint.py:12-20)."""
    qc = raw_config.get("quantization_config") or {}
    top = qc.get("group_size")
    if isinstance(top, int):
        return top
    for group in (qc.get("config_groups") or {}).values():
        inner = ((group or {}).get("weights") or {}).get("group_size")
        if isinstance(inner, int):
            return inner
    return default


def pack_layer(q: torch.Tensor, zp: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Packs int4 values q [N, K] and zero points zp [N, K/G] (both in 0..15) into the
    checkpoint's ``weight_packed`` [N, K/8] and ``weight_zero_point`` [N/8, K/G] words."""
    n, k = q.shape
    shifts = 4 * torch.arange(8, dtype=torch.int64)
    words = (q.to(torch.int64).reshape(n, k // 8, 8) << shifts).sum(-1)
    zwords = (zp.to(torch.int64).reshape(n // 8, 8, -1) << shifts[None, :, None]).sum(1)
    to_i32 = lambda t: ((t + 2**31) % 2**32 - 2**31).to(torch.int32)  # two's complement wrap
    return to_i32(words), to_i32(zwords)


def synthetic_layer(n: int, k: int, gen: torch.Generator, group: int = GROUP) -> dict:
    """One linear drawn as the linear-op benchmark prescribes: q and zp uniform in 0..15,
    scales |N(0, 0.01)| + 1e-3 in fp16."""
    q = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.int64)
    zp = torch.randint(0, 16, (n, k // group), generator=gen, dtype=torch.int64)
    scale = (torch.randn(n, k // group, generator=gen).abs() * 0.01 + 1e-3).to(torch.float16)
    packed, zpacked = pack_layer(q, zp)
    return {
        "weight_packed": packed,
        "weight_zero_point": zpacked,
        "weight_scale": scale,
        "weight_shape": torch.tensor([n, k], dtype=torch.int64),
    }


def synthetic_checkpoint(n_layers: int = 24, vocab: int = 151936, seed: int = 0) -> dict:
    """State dict of a Qwen2.5-0.5B-architecture model in the packed checkpoint format:
    all linears quantised as ``synthetic_layer``, q/k/v biases and the tied embedding fp16
    ~ N(0, 0.02), norm weights 1.  Deterministic in (n_layers, vocab, seed)."""
    gen = torch.Generator().manual_seed(seed)
    state: dict[str, torch.Tensor] = {}
    state["model.embed_tokens.weight"] = (torch.randn(vocab, HIDDEN, generator=gen) * 0.02).to(torch.float16)
    state["model.norm.weight"] = torch.ones(HIDDEN, dtype=torch.float16)
    for i in range(n_layers):
        base = f"model.layers.{i}"
        state[f"{base}.input_layernorm.weight"] = torch.ones(HIDDEN, dtype=torch.float16)
        state[f"{base}.post_attention_layernorm.weight"] = torch.ones(HIDDEN, dtype=torch.float16)
        for name, n, k, has_bias in LAYER_LINEARS:
            for key, value in synthetic_layer(n, k, gen).items():
                state[f"{base}.{name}.{key}"] = value
            if has_bias:
                state[f"{base}.{name}.bias"] = (torch.randn(n, generator=gen) * 0.02).to(torch.float16)
    return state


def synthetic_dense_checkpoint(n_layers: int = 24, vocab: int = 151936, seed: int = 0) -> dict:
    """State dict of the same architecture with UN-QUANTISED fp16 linears (``.weight`` [N, K]
    ~ N(0, 0.02)), the form of the reference's FP16 checkpoints (src/model.py:332-356 without
    packed tensors).  Deterministic in (n_layers, vocab, seed)."""
    gen = torch.Generator().manual_seed(seed)
    state: dict[str, torch.Tensor] = {}
    state["model.embed_tokens.weight"] = (torch.randn(vocab, HIDDEN, generator=gen) * 0.02).to(torch.float16)
    state["model.norm.weight"] = torch.ones(HIDDEN, dtype=torch.float16)
    for i in range(n_layers):
        base = f"model.layers.{i}"
        state[f"{base}.input_layernorm.weight"] = torch.ones(HIDDEN, dtype=torch.float16)
        state[f"{base}.post_attention_layernorm.weight"] = torch.ones(HIDDEN, dtype=torch.float16)
        for name, n, k, has_bias in LAYER_LINEARS:
            state[f"{base}.{name}.weight"] = (torch.randn(n, k, generator=gen) * 0.02).to(torch.float16)
            if has_bias:
                state[f"{base}.{name}.bias"] = (torch.randn(n, generator=gen) * 0.02).to(torch.float16)
    return state


def qwen_config_dict(n_layers: int = 24, vocab: int = 151936, group: int = GROUP,
                     max_position_embeddings: int = 32768) -> dict:
    """``config.json`` contents of the architecture (Qwen2.5-0.5B values)."""
    return {
        "architectures": ["Qwen2ForCausalLM"],
        "model_type": "qwen2",
        "hidden_size": HIDDEN,
        "intermediate_size": INTER,
        "num_hidden_layers": n_layers,
        "num_attention_heads": HEADS,
        "num_key_value_heads": KV_HEADS,
        "vocab_size": vocab,
        "max_position_embeddings": max_position_embeddings,
        "rms_norm_eps": 1e-6,
        "rope_theta": 1000000.0,
        "tie_word_embeddings": True,
        "hidden_act": "silu",
        "attention_dropout": 0.0,
        "use_sliding_window": False,
        "torch_dtype": "float16",
        "bos_token_id": 151643 if vocab > 151645 else 0,
        "eos_token_id": 151645 if vocab > 151645 else 1,
        "quantization_config": {
            "quant_method": "compressed-tensors",
            "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": group,
                                                      "symmetric": False, "strategy": "group"}}},
        },
    }


def write_checkpoint_dir(path: str, state: dict, config: dict) -> None:
    """Writes ``model.safetensors`` + ``config.json`` the way the reference's loaders expect
    them (src/model.py:332-338)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    save_file({k: v.contiguous() for k, v in state.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as handle:
        json.dump(config, handle, indent=1)
