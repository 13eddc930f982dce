"""GPU parity of the long-prompt prefill (more than 32 rows: every projection one tcgen05 GEMM over all rows, one
attention launch over all rows; reference verb Qwen3Session::prefill, runtime/src/qwen3.cpp:547-550) against

  * the CPU oracle at the CUDA path's rounding points (last row's logits; rms / max relative to the logit scale,
    the bounds of tests/test_session_gpu.py), and every layer's K / V rows;
  * the same library's 16-rows-at-a-time prefill (taken when the caller asks for every row's logits), which is
    pinned against the reference's CUDA path in tests/test_reference_cuda_gpu.py;
  * itself: replays give the same bits, verify steps continue from either history, prompts longer than one
    segment of 2048 rows match, and a bounded wait that runs out inside the prompt GEMM is reported without
    losing the session.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def shapes(package):
    S = package.Shape
    return {
        "qwen3_awq": S(vocab_size=2048, n_layers=2, n_heads=8, n_kv_heads=2, hidden_size=1024, intermediate_size=2048,
                       quant_type=1, max_position_embeddings=4096),
        "qwen3_bf16_tied": S(vocab_size=1536, n_layers=3, n_heads=4, n_kv_heads=2, hidden_size=512,
                             intermediate_size=1536, tied_embeddings=True, max_position_embeddings=512),
        "qwen25_awq_bias": S(vocab_size=1024, n_layers=2, n_heads=14, n_kv_heads=2, hidden_size=1792,
                             intermediate_size=2560, quant_type=1, qk_norm=False, qkv_bias=True,
                             max_position_embeddings=512),
    }


def relative(a, b):
    scale = float(np.abs(b).max())
    error = np.abs(a - b)
    return float(np.sqrt((error ** 2).mean())) / scale, float(error.max()) / scale


def narrow_prefill(torch, session, prompt, vocab):
    """The 16-rows-at-a-time path: asking for every row's logits selects it."""
    everything = torch.empty((len(prompt), vocab), dtype=torch.bfloat16, device="cuda")
    session.prefill(prompt, all_logits=everything)
    return everything


@pytest.mark.parametrize("name", ["qwen3_awq", "qwen3_bf16_tied", "qwen25_awq_bias"])
@pytest.mark.parametrize("prompt_len", [33, 130, 300])
def test_long_prompt_against_oracle_and_narrow_path(cuda, package, oracle, name, prompt_len):
    torch, syn = cuda, package.synthetic
    shape = shapes(package)[name]
    tensors = syn.make_model(shape, seed=5, vary_norms=True)
    model = package.Model(shape, tensors)
    wide, narrow = model.new_session(512, graph=True), model.new_session(512, graph=True)
    prompt = syn.make_prompt(21, prompt_len, shape.vocab_size)
    wide.prefill(prompt)
    narrow_prefill(torch, narrow, prompt, shape.vocab_size)
    assert wide.context_size() == narrow.context_size() == prompt_len
    got = syn.bf16_to_float(wide.read_logits(1))[0]
    other = syn.bf16_to_float(narrow.read_logits(1))[0]
    staged = oracle.OracleModel(shape, tensors, capacity=512)
    ref = staged.forward(prompt, 1)[-1]
    bound = 1.5e-2 * np.sqrt(shape.n_layers)
    rms, worst = relative(got, ref)
    assert rms <= 1e-2 and worst <= bound, (rms, worst)
    rms, worst = relative(got, other)
    assert rms <= 1e-2 and worst <= bound, (rms, worst)
    # Every layer's appended K / V rows. The first layer's come from the embedding, one norm and one projection:
    # nearly all bits agree. Deeper rows inherit the rounding flips of the layers below.
    for layer in range(shape.n_layers):
        for a, b in zip(wide.read_kv(layer), narrow.read_kv(layer)):
            fa, fb = syn.bf16_to_float(a), syn.bf16_to_float(b)
            scale = max(1.0, float(np.abs(fb).max()))
            assert np.abs(fa - fb).max() <= 0.03 * scale, layer
            assert float(np.sqrt(((fa - fb) ** 2).mean())) <= 5e-3 * scale, layer
            if layer == 0:
                assert np.mean(a == b) > 0.97
    # The same bits on a replay, also after another prompt went through the shared workspace.
    first_bits = wide.read_logits(1).copy()
    narrow.prefill(syn.make_prompt(22, 64, shape.vocab_size))
    wide.prefill(prompt)
    assert np.array_equal(wide.read_logits(1), first_bits)
    # Verify steps continue from the long-prompt history as from the other one wherever the choice is decisive.
    narrow_prefill(torch, narrow, prompt, shape.vocab_size)
    drafts = [int(t) for t in syn.make_prompt(23, 5, shape.vocab_size)]
    out_w, out_n = wide.verify(drafts), narrow.verify(drafts)
    logits_n = syn.bf16_to_float(narrow.read_logits(5))
    decisive = oracle.top2_gap(logits_n) > 2 * bound * float(np.abs(logits_n).max())
    for r in range(5):
        if decisive[r]:
            assert out_w.targets[r] == out_n.targets[r]
    rms, worst = relative(syn.bf16_to_float(wide.read_logits(5)), logits_n)
    assert rms <= 1e-2 and worst <= bound


def test_prompt_longer_than_one_segment(cuda, package):
    """2048 + 77 rows: two segments, the second attending over the first one's rows."""
    torch, syn = cuda, package.synthetic
    shape = shapes(package)["qwen3_awq"]
    tensors = syn.make_model(shape, seed=6, vary_norms=True)
    model = package.Model(shape, tensors)
    wide, narrow = model.new_session(2200, graph=False), model.new_session(2200, graph=False)
    prompt = syn.make_prompt(31, 2048 + 77, shape.vocab_size)
    wide.prefill(prompt)
    narrow_prefill(torch, narrow, prompt, shape.vocab_size)
    assert wide.context_size() == len(prompt)
    rms, worst = relative(syn.bf16_to_float(wide.read_logits(1))[0], syn.bf16_to_float(narrow.read_logits(1))[0])
    assert rms <= 1e-2 and worst <= 1.5e-2 * np.sqrt(shape.n_layers), (rms, worst)
    for a, b in zip(wide.read_kv(1), narrow.read_kv(1)):
        fa, fb = syn.bf16_to_float(a[2048:]), syn.bf16_to_float(b[2048:])
        assert float(np.sqrt(((fa - fb) ** 2).mean())) <= 5e-3 * max(1.0, float(np.abs(fb).max()))


def test_prompt_that_fills_the_cache_exactly_and_one_that_does_not_fit(cuda, package):
    """Maximum sizes: a prompt of exactly `capacity` rows (one full segment of 2048) is taken and leaves no room for a
    verify step; one row more is refused before any write, and the history stays."""
    torch, syn, abi = cuda, package.synthetic, package.abi
    shape = shapes(package)["qwen3_awq"]
    model = package.Model(shape, syn.make_model(shape, seed=6, vary_norms=True))
    session, narrow = model.new_session(2048, graph=True), model.new_session(2048, graph=True)
    prompt = syn.make_prompt(33, 2048, shape.vocab_size)
    session.prefill(prompt)
    assert session.context_size() == 2048 == session.context_capacity()
    narrow_prefill(torch, narrow, prompt, shape.vocab_size)
    rms, worst = relative(syn.bf16_to_float(session.read_logits(1))[0], syn.bf16_to_float(narrow.read_logits(1))[0])
    assert rms <= 1e-2 and worst <= 1.5e-2 * np.sqrt(shape.n_layers), (rms, worst)
    kept = session.read_logits(1).copy()
    with pytest.raises(abi.LengthError):
        session.verify([1, 2, 3])
    with pytest.raises(abi.LengthError):
        session.prefill(syn.make_prompt(34, 2049, shape.vocab_size))
    assert session.context_size() == 2048 and np.array_equal(session.read_logits(1), kept)
    session.truncate(2040)
    out = session.verify([1, 2, 3])
    assert out.context == 2040 + out.emitted


def test_speculative_decoder_after_long_prompt_equals_greedy(cuda, package):
    """The speculative loop's output after a long prompt is the target's own greedy continuation."""
    syn = package.synthetic
    shape = shapes(package)["qwen3_awq"]
    tensors = syn.make_model(shape, seed=8, vary_norms=True)
    model = package.Model(shape, tensors)
    prompt = [int(t) for t in syn.make_prompt(41, 100, shape.vocab_size)]
    plain = model.new_session(256, graph=True)
    plain.prefill(prompt)
    expected = [int(np.argmax(syn.bf16_to_float(plain.read_logits(1))[0]))]
    for _ in range(11):
        plain.decode(expected[-1])
        expected.append(int(np.argmax(syn.bf16_to_float(plain.read_logits(1))[0])))
    target, draft = model.new_session(256, graph=True), model.new_session(256, graph=True)
    decoder = package.runtime.SpeculativeDecoder(target, draft, 4)
    got = decoder.generate(prompt, 12)
    assert got[:12] == expected


def test_bounded_wait_inside_the_prompt_gemm_is_reported(cuda, package):
    """The first copy of the prompt GEMM's first block of inputs is told to expect 16 bytes more than it delivers,
    with a short poll limit: every role of the kernel gives up, the tensor memory is released, the status bit
    is raised; the prefill reports a runtime error, and the same session then prefills the same prompt to the
    same bits."""
    syn = package.synthetic
    for name in ("qwen3_awq", "qwen3_bf16_tied"):
        shape = shapes(package)[name]
        model = package.Model(shape, syn.make_model(shape, seed=2))
        session = model.new_session(256, graph=True)
        prompt = syn.make_prompt(3, 200, shape.vocab_size)
        session.prefill(prompt)
        expected = session.read_logits(1).copy()
        session.inject_wait_timeout(2000)
        with pytest.raises(RuntimeError, match="bounded wait"):
            session.prefill(prompt)
        assert session.context_size() == 0
        session.prefill(prompt)
        assert np.array_equal(session.read_logits(1), expected)
