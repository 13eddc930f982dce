"""Pins the CPU oracle (oracle/verify_oracle.cpp, FP32 mode) against the UNMODIFIED reference CPU executor
(oracle/_ref, compiled from the reference's own sources) and against the committed golden vectors that the
same reference produced (tests/golden/make_golden.py)."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def small_shape(package, **kw):
    base = dict(vocab_size=512, n_layers=2, n_heads=4, n_kv_heads=2, hidden_size=256, intermediate_size=512,
                max_position_embeddings=64, qk_norm=False, qkv_bias=True)
    base.update(kw)
    return package.Shape(**base)


def run_verify_loop(model, greedy, accept, prompt, rounds, k, seed, vocab, resize, size):
    """prefill, then `rounds` verify steps with random drafts; returns per-step records."""
    rng = np.random.default_rng(seed)
    logits = model(prompt)
    pending = int(greedy(logits[-1:])[0])
    records = []
    for _ in range(rounds):
        drafts = rng.integers(0, vocab, size=k, dtype=np.uint32)
        inputs = np.concatenate([[pending], drafts]).astype(np.uint32)
        before = size()
        logits = model(inputs)
        targets = greedy(logits)
        emitted = accept(inputs, targets)
        resize(before + emitted)
        records.append((inputs, logits, targets, emitted))
        pending = int(targets[emitted - 1])
    return records


@pytest.mark.skipif(not (Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libedge_ref.so").exists(),
                    reason="oracle/_ref not built (needs the reference tree)")
def test_fp32_mode_is_bit_identical_to_reference_cpu_executor(package, oracle):
    shape = small_shape(package)
    tensors = package.synthetic.make_model(shape, seed=3, vary_norms=True)
    ref = oracle.ReferenceCpu(shape, tensors, capacity=48)
    mine = oracle.OracleModel(shape, tensors, capacity=48)
    prompt = package.synthetic.make_prompt(3, 9, shape.vocab_size)
    a = run_verify_loop(ref.forward, ref.greedy, oracle.accept, prompt, 4, 4, 11, shape.vocab_size, ref.resize, ref.size)
    b = run_verify_loop(lambda t: mine.forward(t, 0), oracle.argmax, oracle.accept, prompt, 4, 4, 11, shape.vocab_size,
                        mine.resize, mine.size)
    for (ia, la, ta, ea), (ib, lb, tb, eb) in zip(a, b):
        assert np.array_equal(ia, ib)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)), "logits differ bitwise from the reference"
        assert np.array_equal(ta, tb) and ea == eb
    for layer in range(shape.n_layers):
        rk, rv = ref.read_kv(layer)
        mk, mv = mine.read_kv(layer)
        assert np.array_equal(rk.view(np.uint32), mk.view(np.uint32))
        assert np.array_equal(rv.view(np.uint32), mv.view(np.uint32))


def test_fp32_mode_matches_golden_vectors(package, oracle):
    golden = json.loads((GOLDEN / "cpu_reference_small.json").read_text())
    shape = package.Shape(**golden["shape"])
    tensors = package.synthetic.make_model(shape, seed=golden["seed"], vary_norms=True)
    mine = oracle.OracleModel(shape, tensors, capacity=golden["capacity"])
    logits = mine.forward(np.array(golden["prompt"], dtype=np.uint32), 0)
    assert int(oracle.argmax(logits[-1:])[0]) == golden["first_token"]
    for step in golden["steps"]:
        inputs = np.array(step["inputs"], dtype=np.uint32)
        before = mine.size()
        logits = mine.forward(inputs, 0)
        targets = oracle.argmax(logits)
        assert list(map(int, targets)) == step["targets"]
        assert oracle.accept(inputs, targets) == step["emitted"]
        # logits are pinned through their exact bit pattern at a few probes and a checksum
        probes = [int(logits.view(np.uint32)[r, c]) for r, c in step["probe_index"]]
        assert probes == step["probe_bits"]
        assert int(logits.view(np.uint32).astype(np.uint64).sum()) == step["checksum"]
        mine.resize(before + step["emitted"])


def test_staged_mode_close_to_fp32_mode(package, oracle):
    shape = small_shape(package, qk_norm=True, qkv_bias=False)
    tensors = package.synthetic.make_model(shape, seed=5, vary_norms=True)
    a = oracle.OracleModel(shape, tensors, capacity=32)
    b = oracle.OracleModel(shape, tensors, capacity=32)
    prompt = package.synthetic.make_prompt(5, 12, shape.vocab_size)
    fp32 = a.forward(prompt, 0)
    staged = b.forward(prompt, 1)
    assert np.abs(fp32 - staged).max() <= 2e-2 * np.abs(fp32).max()


def test_accept_rule():
    import __graft_entry__ as entry
    oracle = entry.load_oracle()
    # inputs = [pending, d1, d2, d3]; targets t0..t3
    assert oracle.accept([9, 1, 2, 3], [1, 2, 3, 4]) == 4      # all drafts accepted + bonus token
    assert oracle.accept([9, 1, 2, 3], [1, 7, 3, 4]) == 2      # d2 rejected: emit t0, t1
    assert oracle.accept([9, 1, 2, 3], [5, 2, 3, 4]) == 1      # d1 rejected: only the correction
    assert oracle.accept([9], [5]) == 1                        # k = 0 is ordinary decode


def test_argmax_rules(oracle):
    row = np.array([[1.0, np.nan, 3.0, 3.0, -np.inf]], dtype=np.float32)
    assert int(oracle.argmax(row)[0]) == 2                      # ties go to the lowest index, NaN never wins
    assert int(oracle.argmax(np.full((1, 4), np.nan, dtype=np.float32))[0]) == 0
