"""Size-independent properties at the benchmark's full shape (Qwen3-8B-shape AWQ: 36 layers, hidden 4096,
32 Q / 8 KV heads, FFN 12288, vocabulary 151936, k = 8), where no CPU oracle run is affordable:

  * exact greedy speculation reproduces ordinary greedy decoding whatever the drafts are (the reference's own
    acceptance property, inference_generation_test.cpp:604-647);
  * a row's logits do not depend on how many rows share the forward (1 row with the decode path, 9 rows with
    the verify path) nor on whether other sessions are stacked into it: same bits;
  * a replayed graph step equals the eager step.

Weights are generated on the device (4.85 GB), so the whole file costs well under a minute on a B200."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture
def full_model(cuda, package):
    syn = package.synthetic
    shape = syn.qwen3_8b_awq(max_position_embeddings=512)
    model = package.Model(shape, syn.make_device_model(shape, seed=7))
    cuda.cuda.empty_cache()
    return shape, model


def greedy(session, package, prompt, count):
    session.prefill(prompt)
    tokens = [package.runtime.greedy_token(session.read_logits(1)[0])]
    for _ in range(count - 1):
        session.decode(tokens[-1])
        tokens.append(package.runtime.greedy_token(session.read_logits(1)[0]))
    return tokens


def test_full_shape_speculation_equals_greedy_and_rows_are_independent(cuda, package, full_model):
    syn = package.synthetic
    shape, model = full_model
    prompt = syn.make_prompt(3, 48, shape.vocab_size)
    expected = greedy(model.new_session(256, graph=True), package, prompt, 40)
    corrupted = syn.corrupt_drafts(3, np.array(expected[1:] + [0] * 16, dtype=np.uint32), 0.2, shape.vocab_size)

    def noisy(position, count):
        i = position - len(prompt)
        return list(corrupted[i:i + count])

    def perfect(position, count):
        i = position - len(prompt)
        return (expected + [0] * 16)[i + 1:i + 1 + count]

    for drafts in (noisy, perfect):
        session = model.new_session(256, graph=True)
        emitted, accepts = package.runtime.speculative_generate(session, prompt, drafts, 40, 8)
        assert emitted[:40] == expected, drafts.__name__
        if drafts is perfect:
            assert max(accepts) == 9
        assert session.context_size() == len(prompt) + len(emitted) - 1

    # One row through decode against the same token as row 0 of a nine-row verify: identical logits.
    a, b = model.new_session(256, graph=True), model.new_session(256, graph=False)
    a.prefill(prompt)
    b.prefill(prompt)
    a.decode(expected[0])
    single = a.read_logits(1)[0].copy()
    out = b.verify([expected[0]] + list(corrupted[:8]))
    stacked = b.read_logits(9)
    assert np.array_equal(single, stacked[0])
    assert out.targets[0] == expected[1]

    # Graph replay equals the eager step, and stacking a second session into the forward changes nothing.
    c, d, e = (model.new_session(256, graph=True) for _ in range(3))
    for session in (c, d, e):
        session.prefill(prompt)
    first = [c.verify([expected[0]] + list(corrupted[:7])) for _ in range(1)][0]
    c.truncate(len(prompt))
    replay = c.verify([expected[0]] + list(corrupted[:7]))
    assert first.targets == replay.targets and first.emitted == replay.emitted
    batch = package.runtime.SessionBatch([d, e])
    both = batch.verify([[expected[0]] + list(corrupted[:7]), [expected[0]] + list(corrupted[:7])])
    assert both[0].targets == replay.targets == both[1].targets
    assert both[0].emitted == replay.emitted == both[1].emitted
    ka, va = c.read_kv(35)
    kb, vb = d.read_kv(35)
    assert np.array_equal(ka, kb) and np.array_equal(va, vb)
    batch.close()
