"""The check behind ``__graft_entry__.smoke()``: a 2-layer model decodes 4 tokens on cuda:0
through the C ABI and must reproduce the CPU oracle's tokens and logits."""

import torch


def run_smoke() -> None:
    from oracle.quic_ref import RefModel
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import qwen_config_dict, synthetic_checkpoint

    if not torch.cuda.is_available():
        raise RuntimeError("smoke() needs cuda:0")
    state = synthetic_checkpoint(n_layers=2, vocab=2048, seed=1234)
    net = qmodel.from_state_dict(state, qwen_config_dict(2, 2048), device="cuda:0")
    prompt = [11, 7, 1999, 42, 0, 512]
    ref_tokens, ref_logits = RefModel(state, 2).greedy(prompt, 4)

    cache = net.new_cache(n_slots=2, s_max=256)
    first, logits = net.prefill(cache, [1], [torch.tensor(prompt)])
    tokens = [int(first[0])] + net.decode(cache, [1], 3)[0]
    err = (logits[0].float().cpu() - ref_logits[0].float()).abs().max().item()
    print(f"smoke: tokens {tokens} oracle {ref_tokens} max|dlogit| {err:.4f}")
    assert tokens == ref_tokens, (tokens, ref_tokens)
    assert err < 5e-2
