"""Several sessions per forward: step time of ei_batch_verify against one session at a time.

The rows of S sessions are stacked into one forward of S * rows <= 16 rows, so the weights are streamed once
per step for all of them; attention, KV append and acceptance stay per session. Prints, per S, the time of
one batched step (host tokens in, results out, one synchronisation: the call a user makes) and the
session-steps per second it gives, next to S separate ei_session_verify calls.

    python edge-infer_b200/batchbench.py --shape qwen25_7b --rows 5 --prompt 512
"""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def main():
    import torch

    parser = argparse.ArgumentParser()
    parser.add_argument("--shape", default="qwen25_7b", choices=["qwen25_7b", "qwen3_8b"])
    parser.add_argument("--rows", type=int, default=5, help="tokens per session and step: pending + k drafts")
    parser.add_argument("--prompt", type=int, default=512)
    parser.add_argument("--steps", type=int, default=30)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("batchbench needs a CUDA device")
    package = entry.load_package()
    package.abi.load_library()
    syn = package.synthetic
    capacity = args.prompt + (args.steps + 8) * args.rows + 64
    factory = syn.qwen25_7b_awq if args.shape == "qwen25_7b" else syn.qwen3_8b_awq
    shape = factory() if args.shape == "qwen25_7b" else factory(max_position_embeddings=capacity)
    model = package.Model(shape, syn.make_device_model(shape, seed=0))
    torch.cuda.empty_cache()
    most = 16 // args.rows
    sessions = [model.new_session(capacity, graph=True) for _ in range(most)]
    for j, session in enumerate(sessions):
        session.prefill(syn.make_prompt(j, args.prompt, shape.vocab_size))
    rng = np.random.default_rng(0)

    def tokens(count):
        return rng.integers(0, shape.vocab_size, size=(count, args.rows)).tolist()

    def rewind():
        for session in sessions:
            session.truncate(args.prompt)

    def timed(call, count):
        rewind()
        for _ in range(3):
            call(tokens(count))
        torch.cuda.synchronize()
        start = time.perf_counter()
        for _ in range(args.steps):
            call(tokens(count))
        torch.cuda.synchronize()
        return (time.perf_counter() - start) / args.steps

    def one_at_a_time(rows_of_tokens):
        for session, row in zip(sessions, rows_of_tokens):
            session.verify(row)

    print(f"{args.shape}, {args.rows} rows per session, context {args.prompt}, weights {model.weight_bytes() / 1e9:.2f} GB")
    base = None
    for count in range(1, most + 1):
        batch = package.runtime.SessionBatch(sessions[:count])
        together = timed(batch.verify, count)
        apart = timed(one_at_a_time, count)
        batch.close()
        base = base or apart
        print(f"S={count}: batched {together * 1e3:7.3f} ms/step  {count / together:8.1f} session-steps/s   "
              f"separate {apart * 1e3:7.3f} ms  {count / apart:8.1f} session-steps/s   gain x{apart / together:.2f}", flush=True)


if __name__ == "__main__":
    main()
