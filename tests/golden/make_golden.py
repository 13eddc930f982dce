"""Generates tests/golden/cpu_reference_small.json by running the UNMODIFIED reference CPU executor
(oracle/_ref/libedge_ref.so, built from the reference's own sources by `make -C oracle ref`) as a verify loop.

    python tests/golden/make_golden.py

Needs the reference tree only to build oracle/_ref; the tests read the JSON, never the reference.
The model is Qwen2-style (q/k/v bias, no QK-norm): the one family the reference's CPU executor runs natively.
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

package = entry.load_package()
oracle = entry.load_oracle()

SHAPE = dict(vocab_size=640, n_layers=2, n_heads=4, n_kv_heads=2, hidden_size=256, intermediate_size=768,
             max_position_embeddings=96, qk_norm=False, qkv_bias=True)
SEED, CAPACITY, K, ROUNDS = 21, 80, 4, 8


def main() -> None:
    shape = package.Shape(**SHAPE)
    tensors = package.synthetic.make_model(shape, seed=SEED, vary_norms=True)
    ref = oracle.ReferenceCpu(shape, tensors, capacity=CAPACITY)
    prompt = package.synthetic.make_prompt(SEED, 17, shape.vocab_size)
    logits = ref.forward(prompt)
    pending = int(ref.greedy(logits[-1:])[0])
    record = {"shape": SHAPE, "seed": SEED, "capacity": CAPACITY, "prompt": [int(t) for t in prompt],
              "first_token": pending, "steps": []}
    # Greedy continuation of the reference itself, then corrupted drafts (p = 0.3), as the configs prescribe.
    probe = oracle.ReferenceCpu(shape, tensors, capacity=CAPACITY)
    probe.forward(prompt)
    continuation, token = [], pending
    for _ in range(ROUNDS * (K + 1) + K):
        token = int(probe.greedy(probe.forward([token]))[0])
        continuation.append(token)
    drafts_all = package.synthetic.corrupt_drafts(SEED, np.array(continuation, dtype=np.uint32), 0.3, shape.vocab_size)
    emitted_total = 0
    for _ in range(ROUNDS):
        drafts = drafts_all[emitted_total:emitted_total + K]
        inputs = np.concatenate([[pending], drafts]).astype(np.uint32)
        before = ref.size()
        logits = ref.forward(inputs)
        targets = ref.greedy(logits)
        emitted = oracle.accept(inputs, targets)
        ref.resize(before + emitted)
        rng = np.random.default_rng(len(record["steps"]))
        probes = [[int(rng.integers(0, len(inputs))), int(rng.integers(0, shape.vocab_size))] for _ in range(6)]
        bits = logits.view(np.uint32)
        record["steps"].append({
            "inputs": [int(t) for t in inputs], "targets": [int(t) for t in targets], "emitted": emitted,
            "probe_index": probes, "probe_bits": [int(bits[r, c]) for r, c in probes],
            "checksum": int(bits.astype(np.uint64).sum()),
            "top2_gap": [float(g) for g in oracle.top2_gap(logits)],
            "max_abs_logit": float(np.abs(logits).max()),
        })
        pending = int(targets[emitted - 1])
        emitted_total += emitted
    out = Path(__file__).resolve().parent / "cpu_reference_small.json"
    out.write_text(json.dumps(record, indent=1))
    print("wrote", out, "accept lengths:", [s["emitted"] for s in record["steps"]])


if __name__ == "__main__":
    main()
