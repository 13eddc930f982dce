"""Several sessions verified in one forward (ei_batch_verify) must end exactly as if each had run its own
ei_session_verify: same greedy tokens, accept lengths and contexts, same KV bits. The GEMMs see the stacked rows
of all sessions, and a row's sums do not depend on the other rows of the tile, so the comparison is bit-exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def small_shapes(package):
    S = package.Shape
    return {
        "qwen3_awq": S(vocab_size=2048, n_layers=2, n_heads=8, n_kv_heads=2, hidden_size=1024, intermediate_size=2048,
                       quant_type=1, max_position_embeddings=512),
        "qwen25_awq_bias": S(vocab_size=1024, n_layers=2, n_heads=14, n_kv_heads=2, hidden_size=1792,
                             intermediate_size=2560, quant_type=1, qk_norm=False, qkv_bias=True,
                             max_position_embeddings=512),
        "qwen3_bf16_tied": S(vocab_size=1536, n_layers=3, n_heads=4, n_kv_heads=2, hidden_size=512,
                             intermediate_size=1536, tied_embeddings=True, max_position_embeddings=512),
    }


@pytest.mark.parametrize("name,sessions,rows,graph", [("qwen3_awq", 3, 5, True), ("qwen25_awq_bias", 2, 8, True),
                                                      ("qwen3_bf16_tied", 4, 4, False), ("qwen3_awq", 1, 9, True)])
def test_batched_verify_equals_individual_verify(cuda, package, name, sessions, rows, graph):
    syn = package.synthetic
    shape = small_shapes(package)[name]
    model = package.Model(shape, syn.make_model(shape, seed=21, vary_norms=True))
    prompts = [syn.make_prompt(100 + j, 20 + 7 * j, shape.vocab_size) for j in range(sessions)]   # ragged contexts

    def start():
        group = [model.new_session(128, graph=graph) for _ in range(sessions)]
        pendings = []
        for session, prompt in zip(group, prompts):
            session.prefill(prompt)
            pendings.append(package.runtime.greedy_token(session.read_logits(1)[0]))
        return group, pendings

    alone, pending_a = start()
    together, pending_b = start()
    assert pending_a == pending_b
    batch = package.runtime.SessionBatch(together)
    rng = np.random.default_rng(5)
    for step in range(4):                                   # the third and fourth steps replay the captured graph
        drafts = rng.integers(0, shape.vocab_size, size=(sessions, rows - 1))
        if step == 1:                                       # make some drafts right: the model's own next tokens
            for j, session in enumerate(alone):
                probe = session.verify([pending_a[j]] + list(drafts[j]))
                session.truncate(probe.context - probe.emitted)
                drafts[j, 0] = probe.targets[0]
        inputs = [[pending_a[j]] + list(drafts[j]) for j in range(sessions)]
        singles = [session.verify(tokens) for session, tokens in zip(alone, inputs)]
        batched = batch.verify(inputs)
        for j, (one, many) in enumerate(zip(singles, batched)):
            assert one.targets == many.targets, (step, j)
            assert one.emitted == many.emitted and one.context == many.context, (step, j)
            assert alone[j].context_size() == together[j].context_size()
        pending_a = [out.tokens[-1] for out in singles]
    for j in range(sessions):
        for layer in (0, shape.n_layers - 1):
            ka, va = alone[j].read_kv(layer)
            kb, vb = together[j].read_kv(layer)
            assert np.array_equal(ka, kb) and np.array_equal(va, vb), (j, layer)
    batch.close()


def test_batch_rejects_bad_requests(cuda, package):
    syn = package.synthetic
    shape = small_shapes(package)["qwen3_awq"]
    model = package.Model(shape, syn.make_model(shape, seed=3))
    other_model = package.Model(shape, syn.make_model(shape, seed=4))
    a, b, c = model.new_session(64), model.new_session(64), other_model.new_session(64)
    with pytest.raises(ValueError):
        package.runtime.SessionBatch([a, a])                # the same session twice
    with pytest.raises(ValueError):
        package.runtime.SessionBatch([a, c])                # different models
    with pytest.raises(ValueError):
        package.runtime.SessionBatch([a, model.new_session(32)])    # different capacities
    batch = package.runtime.SessionBatch([a, b])
    with pytest.raises(package.abi.LogicError):
        batch.verify([[1, 2], [3, 4]])                      # no prefill yet
    a.prefill([1, 2, 3])
    b.prefill([4, 5])
    with pytest.raises(ValueError):
        batch.verify([[1] * 9, [2] * 9])                    # 2 x 9 rows > 16
    with pytest.raises(ValueError):
        batch.verify([[1, shape.vocab_size], [2, 3]])       # token out of range: rejected before any work
    assert a.context_size() == 3 and b.context_size() == 2
    out = batch.verify([[1, 2, 3], [4, 5, 6]])
    assert [o.context for o in out] == [3 + out[0].emitted, 2 + out[1].emitted]
    batch.close()
