"""GPU parity against the reference's own CUDA path: the UNMODIFIED edge-infer library (oracle/_ref, compiled
from its sources for sm_100) runs Qwen3Session<bf16>::prefill_eager and op::cuda::sample on the same seeded
model and tokens. Skipped where oracle/_ref has not been built.

Logits: rms(a - ref) / max|ref| <= 1e-2. The residual is BF16 rounding-flip noise (one flipped rounding costs a
BF16 ulp and flips accumulate over layers), so the library must also be no farther from the reference than 1.5x
the distance of the exact-accumulation staged oracle, in the mean and in the maximum (+ 0.5e-2 for the tail of
a maximum over ~10^4 logits). Greedy tokens equal wherever the reference's top-2 gap exceeds twice the observed
maximum band; accept lengths equal when the emitted prefix is decisive."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def cases(package):
    S = package.Shape
    return {
        "qwen3_awq": (S(vocab_size=2048, n_layers=2, n_heads=8, n_kv_heads=2, hidden_size=1024, intermediate_size=2048,
                        quant_type=1, max_position_embeddings=512), 9),
        "qwen3_awq_deep": (S(vocab_size=2048, n_layers=8, n_heads=8, n_kv_heads=2, hidden_size=1024,
                             intermediate_size=2048, quant_type=1, max_position_embeddings=512), 9),
        "qwen3_bf16": (S(vocab_size=1536, n_layers=3, n_heads=4, n_kv_heads=2, hidden_size=512, intermediate_size=1536,
                         max_position_embeddings=512), 5),
        "qwen25_awq_bias": (S(vocab_size=1024, n_layers=2, n_heads=14, n_kv_heads=2, hidden_size=1792,
                              intermediate_size=2560, quant_type=1, qk_norm=False, qkv_bias=True,
                              max_position_embeddings=512), 5),
    }


@pytest.mark.parametrize("name", ["qwen3_awq", "qwen3_awq_deep", "qwen3_bf16", "qwen25_awq_bias"])
def test_verify_against_reference_cuda_path(cuda, package, oracle, name):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref not built")
    syn = package.synthetic
    shape, rows = cases(package)[name]
    tensors = syn.make_model(shape, seed=12, vary_norms=True)
    session = package.Model(shape, tensors).new_session(256, graph=True)
    reference = oracle.ReferenceCuda(shape, tensors, 256)
    staged = oracle.OracleModel(shape, tensors, 256)
    prompt = syn.make_prompt(12, 83, shape.vocab_size)
    session.prefill(prompt)
    ref_logits, ref_greedy = reference.forward(prompt)
    staged.forward(prompt, 1)
    max_bound = 1.5e-2 * np.sqrt(shape.n_layers)
    pending = int(ref_greedy[-1])
    compared = 0
    rng = np.random.default_rng(0)
    for step in range(5):
        # drafts: the reference's own greedy continuation with p = 0.3 substitution
        length = reference.size()
        continuation, token = [], pending
        for _ in range(rows - 1):
            token = int(reference.forward([token])[1][0])
            continuation.append(token)
        reference.resize(length)
        drafts = np.array(continuation, dtype=np.uint32)
        drafts = np.where(rng.random(len(drafts)) < 0.3, rng.integers(0, shape.vocab_size, len(drafts)), drafts)
        inputs = np.concatenate([[pending], drafts]).astype(np.uint32)
        out = session.verify(inputs)
        ref_logits, ref_greedy = reference.forward(inputs)
        staged_logits = staged.forward(inputs, 1)
        got = syn.bf16_to_float(session.read_logits(rows))
        scale = float(np.abs(ref_logits).max())
        mine, ideal = np.abs(got - ref_logits), np.abs(staged_logits - ref_logits)
        rms = float(np.sqrt((mine ** 2).mean())) / scale
        assert rms <= 1e-2, (step, rms)
        assert rms <= 1.5 * float(np.sqrt((ideal ** 2).mean())) / scale + 1e-4
        # Both maxima are extreme values over rows x vocabulary of equally distributed errors: a factor of two
        # between them is still noise.
        band = max(max_bound, 2.0 * float(ideal.max()) / scale + 0.5e-2)
        assert float(mine.max()) / scale <= band, (step, float(mine.max()) / scale, float(ideal.max()) / scale)
        gaps = oracle.top2_gap(ref_logits)
        decisive = gaps > 2 * band * scale
        for r in range(rows):
            if decisive[r]:
                assert out.targets[r] == int(ref_greedy[r]), (step, r)
                compared += 1
        emitted = oracle.accept(inputs, ref_greedy)
        if decisive[:emitted].all():
            assert out.emitted == emitted
        reference.resize(length + emitted)
        staged.resize(length + emitted)
        session.truncate(length + emitted)
        pending = int(ref_greedy[emitted - 1])
    assert compared >= 5
