"""The draft + verify loop that runs without host round trips (ei_speculative_*).

The property the reference's own tests demand of its SpeculativeDecoder (runtime/tests/inference_generation_test.cpp:
488-538 for windows 1 / 6 / 8, 580-647 for a draft that is always rejected): the speculative token sequence equals the
ordinary greedy sequence of the target model, whatever the draft proposes. Here the comparison is bit-exact: a
target row's logits do not depend on how many rows the step has."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def shapes(package):
    S = package.Shape
    target = S(vocab_size=2048, n_layers=2, n_heads=8, n_kv_heads=2, hidden_size=1024, intermediate_size=2048,
               quant_type=1, max_position_embeddings=512)
    draft = S(vocab_size=2048, n_layers=1, n_heads=4, n_kv_heads=2, hidden_size=512, intermediate_size=1024,
              max_position_embeddings=512)
    return target, draft


def greedy_reference(package, model, prompt, new_tokens, capacity):
    """Ordinary greedy decoding of the target alone: prefill, then one token per decode step."""
    session = model.new_session(capacity, graph=True)
    session.prefill(prompt)
    token = package.runtime.greedy_token(session.read_logits(1)[0])
    out = [token]
    while len(out) < new_tokens:
        session.decode(token)
        token = package.runtime.greedy_token(session.read_logits(1)[0])
        out.append(token)
    return out


@pytest.mark.parametrize("window", [1, 4, 8])
@pytest.mark.parametrize("draft_kind", ["same_model", "other_model"])
def test_speculative_tokens_equal_greedy_tokens(cuda, package, window, draft_kind):
    syn = package.synthetic
    target_shape, draft_shape = shapes(package)
    target_model = package.Model(target_shape, syn.make_model(target_shape, seed=11, vary_norms=True))
    if draft_kind == "same_model":      # every draft is accepted: rounds emit window + 1 tokens
        draft_model = target_model
    else:                               # a random smaller model: almost every draft is rejected
        draft_model = package.Model(draft_shape, syn.make_model(draft_shape, seed=12))
    prompt = syn.make_prompt(7, 37, target_shape.vocab_size)
    new_tokens, capacity = 48, 256
    expected = greedy_reference(package, target_model, prompt, new_tokens, capacity)

    target, draft = target_model.new_session(capacity, graph=True), draft_model.new_session(capacity, graph=True)
    decoder = package.runtime.SpeculativeDecoder(target, draft, window)
    first = decoder.prefill(prompt)
    assert first == expected[0]
    produced, rounds = [], 0
    while len(produced) < new_tokens:
        decoder.enqueue(3)              # several rounds per host synchronisation
        rounds += 3
        produced = decoder.drain()
    assert produced[:new_tokens] == expected
    per_round = (len(produced) - 1) / rounds
    if draft_kind == "same_model":
        assert per_round == window + 1  # full acceptance plus the target's own next token
    else:
        assert 1 <= per_round <= window + 1
    # Both sessions stand at the same boundary: everything generated but the pending token is in both caches.
    assert target.context_size() == draft.context_size() == len(prompt) + len(produced) - 1

    # Truncation (the reference's EOS handling) and continuation give the same sequence again.
    keep = new_tokens // 2
    decoder.truncate(keep)
    assert target.context_size() == draft.context_size() == len(prompt) + keep - 1
    again = []
    while len(again) < new_tokens:
        decoder.enqueue(2)
        again = decoder.drain()
    assert again[:new_tokens] == expected
    decoder.close()


def test_generate_stops_after_eos(cuda, package):
    syn = package.synthetic
    target_shape, draft_shape = shapes(package)
    target_model = package.Model(target_shape, syn.make_model(target_shape, seed=11, vary_norms=True))
    draft_model = package.Model(draft_shape, syn.make_model(draft_shape, seed=12))
    prompt = syn.make_prompt(9, 21, target_shape.vocab_size)
    expected = greedy_reference(package, target_model, prompt, 24, 128)
    eos = expected[10]
    stop = expected.index(eos)
    decoder = package.runtime.SpeculativeDecoder(target_model.new_session(128), draft_model.new_session(128), 4)
    out = decoder.generate(prompt, 24, eos=eos, rounds_per_drain=2)
    assert out == expected[:stop + 1]
    assert decoder.target.context_size() == len(prompt) + stop
    decoder.close()


def test_speculative_rejects_bad_requests(cuda, package):
    syn = package.synthetic
    target_shape, draft_shape = shapes(package)
    model = package.Model(target_shape, syn.make_model(target_shape, seed=3))
    a, b = model.new_session(64), model.new_session(64)
    with pytest.raises(ValueError):
        package.runtime.SpeculativeDecoder(a, a, 4)                 # one session twice
    with pytest.raises(ValueError):
        package.runtime.SpeculativeDecoder(a, b, 16)                # 17 rows
    other = package.Shape(vocab_size=1024, n_layers=1, n_heads=4, n_kv_heads=2, hidden_size=512, intermediate_size=1024,
                          max_position_embeddings=512)
    other_model = package.Model(other, syn.make_model(other, seed=4))
    with pytest.raises(ValueError):
        package.runtime.SpeculativeDecoder(a, other_model.new_session(64), 4)   # different vocabularies
    decoder = package.runtime.SpeculativeDecoder(a, b, 4)
    with pytest.raises(package.abi.LogicError):
        decoder.enqueue(1)                                          # no prefill yet
    decoder.prefill(syn.make_prompt(1, 30, target_shape.vocab_size))
    decoder.enqueue(6)                                              # 30 + 6 * 5 = 60 <= 64
    with pytest.raises(package.abi.LengthError):
        decoder.enqueue(1)                                          # the bound of full acceptance passes the capacity
    produced = decoder.drain()
    assert 7 <= len(produced) <= 31
    decoder.close()
