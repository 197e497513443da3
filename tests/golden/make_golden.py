"""Generates the golden fixtures of tests/golden/ by running the REFERENCE's own Python.

Run in a container that has the reference checked out (read-only is fine):

    python tests/golden/make_golden.py [/path/to/reference]

It imports, unmodified, from the reference:
  * ``quant.checkpoint.dequantize``        (src/quant/checkpoint.py:23)  -> dequant_*.npz
  * ``scheduler.*AdmissionPolicy.decide``  (src/scheduler.py:28,49)      -> scheduler.json
  * ``model_hf.load``                      (src/model_hf.py:14)          -> hf_quant_logits.npz
and feeds them the seeded synthetic checkpoint of quic.cu_b200/checkpoint.py.  The
fixtures hold the reference's OUTPUTS (and small inputs); inputs that are large are
re-created from the seed by the tests.  The reference itself cannot travel to the GPU box,
which is why its outputs are committed.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
from collections import deque

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, REF)

import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from quic_cu_b200.checkpoint import (qwen_config_dict, synthetic_checkpoint, synthetic_layer,  # noqa: E402
                                     write_checkpoint_dir)

GOLDEN_MODEL = {"n_layers": 2, "vocab": 2048, "seed": 1234}
GOLDEN_PROMPT = [11, 7, 1999, 42, 0, 512, 77, 1023, 5, 300, 301, 302]
GOLDEN_NEW = 6


def golden_dequant():
    from quant.checkpoint import dequantize  # reference

    for tag, (n, k, seed) in {"a": (64, 256, 3), "b": (128, 896, 4)}.items():
        layer = synthetic_layer(n, k, torch.Generator().manual_seed(seed))
        weights = {f"l.{key}": value for key, value in layer.items()}
        ref = dequantize(weights, "l", 128)
        np.savez_compressed(os.path.join(HERE, f"dequant_{tag}.npz"),
                            weight_packed=layer["weight_packed"].numpy(),
                            weight_scale=layer["weight_scale"].numpy(),
                            weight_zero_point=layer["weight_zero_point"].numpy(),
                            reference=ref.numpy().astype(np.float32))


def golden_scheduler():
    from scheduler import ContinuousAdmissionPolicy, StaticAdmissionPolicy  # reference
    from sequence import SequenceState  # reference

    rng = np.random.default_rng(7)
    cases = []
    for _ in range(40):
        max_batch = int(rng.integers(1, 6))
        n_run, n_wait = int(rng.integers(0, max_batch + 1)), int(rng.integers(0, 7))
        running_desc = []
        for i in range(n_run):
            max_tokens = int(rng.integers(1, 5))
            running_desc.append({"id": i + 1, "max_tokens": max_tokens,
                                 "generated": int(rng.integers(0, max_tokens + 1)),
                                 "eos": bool(rng.integers(0, 4) == 0)})
        waiting_ids = [100 + j for j in range(n_wait)]
        case = {"max_batch": max_batch, "running": running_desc, "waiting": waiting_ids}
        for name, policy in (("static", StaticAdmissionPolicy()), ("continuous", ContinuousAdmissionPolicy())):
            running = []
            for d in running_desc:
                s = SequenceState(prompt_tokens=torch.tensor([[1]]), request_id=d["id"], max_tokens=d["max_tokens"])
                s.generated_tokens = [9] * d["generated"]
                if d["eos"] and d["generated"] > 0:
                    s.finished_at = d["generated"] - 1
                running.append(s)
            waiting = deque(SequenceState(prompt_tokens=torch.tensor([[2]]), request_id=w, max_tokens=4)
                            for w in waiting_ids)
            dec = policy.decide(running, waiting, max_batch)
            case[name] = {"release": [s.request_id for s in dec.release],
                          "admit": [s.request_id for s in dec.admit]}
        cases.append(case)
    with open(os.path.join(HERE, "scheduler.json"), "w") as handle:
        json.dump(cases, handle, indent=0)


def write_stub_tokenizer(path: str, vocab: int):
    from tokenizers import Tokenizer, models

    tok = Tokenizer(models.WordLevel({f"t{i}": i for i in range(vocab)}, unk_token="t0"))
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as handle:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "t0", "eos_token": "t1"}, handle)


def golden_hf_quant():
    import model_hf  # reference

    state = synthetic_checkpoint(**GOLDEN_MODEL)
    config = qwen_config_dict(GOLDEN_MODEL["n_layers"], GOLDEN_MODEL["vocab"])
    with tempfile.TemporaryDirectory() as tmp:
        write_checkpoint_dir(tmp, state, config)
        write_stub_tokenizer(tmp, GOLDEN_MODEL["vocab"])
        model, _ = model_hf.load(tmp)  # fp16 Qwen2ForCausalLM with dequantised weights, on CPU
    ids = torch.tensor([GOLDEN_PROMPT], dtype=torch.long)
    tokens, logits = [], []
    with torch.no_grad():  # the reference's greedy loop, run.py:49-61
        out = model(ids)
        cache = out.past_key_values
        cur = out.logits[:, -1:, :]
        for _ in range(GOLDEN_NEW):
            logits.append(cur[0, 0].float().numpy())
            nxt = cur.argmax(dim=-1)
            tokens.append(int(nxt))
            out = model(nxt, past_key_values=cache)
            cur = out.logits[:, -1:, :]
    np.savez_compressed(os.path.join(HERE, "hf_quant_logits.npz"),
                        model=json.dumps(GOLDEN_MODEL), prompt=np.array(GOLDEN_PROMPT),
                        tokens=np.array(tokens), logits=np.stack(logits).astype(np.float16),
                        dtype=str(next(model.parameters()).dtype))


if __name__ == "__main__":
    golden_dequant()
    golden_scheduler()
    golden_hf_quant()
    print("golden fixtures written to", HERE)
