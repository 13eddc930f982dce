"""Draft + verify rounds without host round trips (ei_speculative_*) against a host-driven round.

Target: the Qwen3-8B-shape AWQ model; draft: the Qwen3-0.6B-shape BF16 model (both random-init, so nearly every
draft is rejected: the figure of interest is the time of a round, not the acceptance). A round is k + 1 draft
decode steps, one verify forward of k + 1 rows and the hand-over between the two sessions. The device-resident
loop enqueues whole rounds and synchronises once per `--rounds` rounds; the host-driven round does what the
reference's loop does (runtime/src/speculative_decoder.cpp:176-224): one synchronisation and one token copy per
draft step, then the verify call.

    python edge-infer_b200/specbench.py --drafts 8 --prompt 2048
"""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def main():
    import torch

    parser = argparse.ArgumentParser()
    parser.add_argument("--drafts", type=int, default=8, help="k: drafts verified per round")
    parser.add_argument("--prompt", type=int, default=2048)
    parser.add_argument("--rounds", type=int, default=24)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("specbench needs a CUDA device")
    package = entry.load_package()
    package.abi.load_library()
    syn = package.synthetic
    rows = args.drafts + 1
    capacity = args.prompt + (2 * args.rounds + 8) * rows + 64
    target_shape = syn.qwen3_8b_awq(max_position_embeddings=capacity)
    draft_shape = syn.qwen3_0_6b(max_position_embeddings=capacity)
    target_model = package.Model(target_shape, syn.make_device_model(target_shape, seed=0))
    draft_model = package.Model(draft_shape, syn.make_device_model(draft_shape, seed=1))
    torch.cuda.empty_cache()
    prompt = syn.make_prompt(0, args.prompt, target_shape.vocab_size)

    # ---- device-resident rounds ----
    target, draft = target_model.new_session(capacity, graph=True), draft_model.new_session(capacity, graph=True)
    decoder = package.runtime.SpeculativeDecoder(target, draft, args.drafts)
    decoder.prefill(prompt)
    decoder.enqueue(3)
    decoder.drain()
    decoder.truncate(1)
    torch.cuda.synchronize()
    start = time.perf_counter()
    decoder.enqueue(args.rounds)
    produced = decoder.drain()
    resident = (time.perf_counter() - start) / args.rounds
    decoder.close()

    # ---- host-driven rounds: a synchronisation per draft token, as the reference's loop ----
    target, draft = target_model.new_session(capacity, graph=True), draft_model.new_session(capacity, graph=True)
    target.prefill(prompt)
    draft.prefill(prompt)
    pending = package.runtime.greedy_token(target.read_logits(1)[0])

    def host_round(pending):
        base = draft.context_size()
        tokens, token = [pending], pending
        for _ in range(rows):
            token = draft.verify([token]).tokens[-1]      # one decode step: greedy token back on the host
            tokens.append(token)
        out = target.verify(tokens[:rows])
        draft.truncate(base + out.emitted)
        return out.tokens[-1], out.emitted

    for _ in range(3):
        pending, _ = host_round(pending)
    torch.cuda.synchronize()
    start = time.perf_counter()
    emitted = 0
    for _ in range(args.rounds):
        pending, count = host_round(pending)
        emitted += count
    torch.cuda.synchronize()
    driven = (time.perf_counter() - start) / args.rounds

    print(f"target qwen3_8b_awq + draft qwen3_0_6b, k = {args.drafts}, prompt {args.prompt}: "
          f"device-resident round {resident * 1e3:.3f} ms ({(len(produced) - 1) / args.rounds:.2f} tokens per round), "
          f"host-driven round {driven * 1e3:.3f} ms ({emitted / args.rounds:.2f} tokens per round), "
          f"x{driven / resident:.2f}")


if __name__ == "__main__":
    main()
