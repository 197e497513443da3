"""The reference's dequantised-weight Hugging Face path (``hf_quant``) restated.

TEST INFRASTRUCTURE ONLY (see quic_ref.py).  Follows src/model_hf.py:36-45 of
hdahroug/quic.cu: dequantise every packed layer (src/quant/checkpoint.py:39-43), load the
result into ``transformers.Qwen2ForCausalLM`` and tie the embeddings.  The transformer
arithmetic itself lives in the third-party ``transformers`` package (the reference pins
``transformers<4.45.0``, requirements.txt:2; this image carries 5.5.0, whose default
attention is ``sdpa`` — ``eager`` is requested explicitly).

Used (a) in fp16 on the GPU as the correctness oracle of the CUDA path, (b) in fp32 on
the host cores as the CPU baseline and the ``--impl reference`` arm of bench.py (the
reference's HF eager CPU path of the benchmark configuration).
"""

from __future__ import annotations

import torch

from .quic_ref import dequantize

QUANT_SUFFIXES = (".weight_packed", ".weight_scale", ".weight_zero_point", ".weight_shape")


def dequantized_state_dict(state: dict, group: int = 128) -> dict:
    """fp32 ``.weight`` for every packed prefix, other tensors unchanged (checkpoint.py:39-43)."""
    out = {k: v for k, v in state.items() if not k.endswith(QUANT_SUFFIXES)}
    tail = ".weight_packed"
    for name in state:
        if name.endswith(tail):
            p = name[: -len(tail)]
            out[f"{p}.weight"] = torch.from_numpy(dequantize(
                state[f"{p}.weight_packed"].numpy(), state[f"{p}.weight_scale"].numpy(),
                state[f"{p}.weight_zero_point"].numpy(), group))
    return out


def build_hf_model(state: dict, config: dict, dtype=torch.float16, device="cpu"):
    """Qwen2ForCausalLM(config).to(dtype) <- dequantised weights, tied (model_hf.py:38-45)."""
    from transformers import Qwen2Config, Qwen2ForCausalLM

    keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "vocab_size", "max_position_embeddings", "rms_norm_eps",
            "rope_theta", "tie_word_embeddings", "hidden_act")
    cfg = Qwen2Config(**{k: config[k] for k in keys if k in config})
    cfg._attn_implementation = "eager"
    model = Qwen2ForCausalLM(cfg).to(dtype)
    missing, unexpected = model.load_state_dict(dequantized_state_dict(state), strict=False)
    if set(missing) - {"lm_head.weight"} or unexpected:
        raise RuntimeError(f"weight mismatch: missing={missing} unexpected={unexpected}")
    model.tie_weights()
    return model.to(device).eval()


@torch.inference_mode()
def greedy_with_logits(model, prompt_ids: torch.Tensor, n_new: int):
    """The reference's generation loop (run.py:49-61): prefill, then one token per forward
    with the cache.  Returns (tokens [n_new], logits of each generated position [n_new, V])."""
    out = model(prompt_ids, use_cache=True)
    cache = out.past_key_values
    logits = out.logits[:, -1, :]
    tokens, kept = [], []
    for _ in range(n_new):
        kept.append(logits[0].clone())
        nxt = logits.argmax(dim=-1, keepdim=True)
        tokens.append(int(nxt))
        out = model(nxt, past_key_values=cache, use_cache=True)
        logits = out.logits[:, -1, :]
    return tokens, torch.stack(kept)


@torch.inference_mode()
def teacher_forced_logits(model, prompt_ids: torch.Tensor, forced: list[int]) -> torch.Tensor:
    """Logits at every position where a token of ``forced`` is predicted, feeding ``forced``
    regardless of the model's own argmax: [len(forced), V]."""
    ids = torch.cat([prompt_ids, torch.tensor([forced[:-1]], dtype=prompt_ids.dtype,
                                              device=prompt_ids.device)], dim=1) if len(forced) > 1 else prompt_ids
    logits = model(ids).logits[0]
    return logits[prompt_ids.shape[1] - 1:]
