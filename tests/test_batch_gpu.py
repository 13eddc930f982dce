"""Several sessions verified in one forward (ei_batch_verify). Up to 16 stacked rows they must end exactly as if
each had run its own ei_session_verify: same greedy tokens, accept lengths and contexts, same KV bits (the GEMMs see
the stacked rows of all sessions, and a row's sums do not depend on the other rows of the tile). Above 16 stacked
rows the forward runs on the prompt GEMM and is compared within rounding (second test)."""
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


@pytest.mark.parametrize("name,sessions,rows", [("qwen3_awq", 9, 5), ("qwen25_awq_bias", 24, 3),
                                                ("qwen3_bf16_tied", 40, 9), ("qwen3_awq", 17, 1)])
def test_wide_batch_agrees_with_individual_verify(cuda, package, oracle, name, sessions, rows):
    """More than 16 stacked rows: one forward on the prompt GEMM for all sessions. Another summation order than the
    single-session kernels, so: greedy tokens equal wherever the single-session logits are decisive (top-2 gap above
    twice 1.5e-2 * sqrt(layers) of the logit scale), accept lengths equal whenever the emitted prefix is decisive,
    appended K / V rows within BF16 rounding of the single-session ones, and replays give the same bits."""
    syn = package.synthetic
    shape = small_shapes(package)[name]
    model = package.Model(shape, syn.make_model(shape, seed=23, vary_norms=True))
    prompts = [syn.make_prompt(300 + j, 9 + (11 * j) % 60, shape.vocab_size) for j in range(sessions)]   # ragged

    def start():
        group = [model.new_session(128, graph=True) for _ in range(sessions)]
        pendings = []
        for session, prompt in zip(group, prompts):
            session.prefill(prompt)
            pendings.append(package.runtime.greedy_token(session.read_logits(1)[0]))
        return group, pendings

    alone, pending = start()
    together, _ = start()
    again, _ = start()
    batch, batch_again = package.runtime.SessionBatch(together), package.runtime.SessionBatch(again)
    rng = np.random.default_rng(9)
    bound = 1.5e-2 * np.sqrt(shape.n_layers)
    checked = 0
    for step in range(3):
        drafts = rng.integers(0, shape.vocab_size, size=(sessions, rows - 1))
        if rows > 1:                                        # make the first draft of every other session right
            for j in range(0, sessions, 2):
                probe = alone[j].verify([pending[j]] + list(drafts[j]))
                alone[j].truncate(probe.context - probe.emitted)
                drafts[j, 0] = probe.targets[0]
        inputs = [[pending[j]] + list(drafts[j]) for j in range(sessions)]
        before = [s.context_size() for s in alone]
        singles, logits = [], []
        for session, tokens in zip(alone, inputs):
            singles.append(session.verify(tokens))
            logits.append(syn.bf16_to_float(session.read_logits(rows)))
        wide = batch.verify(inputs)
        replay = batch_again.verify(inputs)
        for j in range(sessions):
            assert wide[j].targets == replay[j].targets and wide[j].emitted == replay[j].emitted
            decisive = oracle.top2_gap(logits[j]) > 2 * bound * float(np.abs(logits[j]).max())
            for r in range(rows):
                if decisive[r]:
                    checked += 1
                    assert wide[j].targets[r] == singles[j].targets[r], (step, j, r)
            if decisive[:singles[j].emitted].all():
                assert wide[j].emitted == singles[j].emitted and wide[j].context == singles[j].context, (step, j)
        # Continue every group from the shortest accepted prefix (a near-tie may change an accept length): rows
        # up to there were accepted, and so written, in all three.
        pending = []
        for j in range(sessions):
            emitted = min(singles[j].emitted, wide[j].emitted, replay[j].emitted)
            for group in (alone, together, again):
                group[j].truncate(before[j] + emitted)
            pending.append(singles[j].targets[emitted - 1])
    assert checked >= sessions                               # the check was not vacuous
    for j in (0, sessions - 1):
        for layer in (0, shape.n_layers - 1):
            for a, b in zip(alone[j].read_kv(layer), together[j].read_kv(layer)):
                fa, fb = syn.bf16_to_float(a), syn.bf16_to_float(b)
                assert np.abs(fa - fb).max() <= 0.03 * max(1.0, float(np.abs(fa).max())), (j, layer)
                if layer == 0:
                    assert np.mean(a == b) > 0.97
    batch.close()
    batch_again.close()


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
        batch.verify([[1] * 17, [2] * 17])                  # more than 16 rows per session
    with pytest.raises(ValueError):
        batch.verify([[1, shape.vocab_size], [2, 3]])       # token out of range: rejected before any work
    assert a.context_size() == 3 and b.context_size() == 2
    out = batch.verify([[1, 2, 3], [4, 5, 6]])
    assert [o.context for o in out] == [3 + out[0].emitted, 2 + out[1].emitted]
    batch.close()
