"""Operators borrow everything and allocate nothing, and a session's steady path allocates nothing either (the
reference's alloc-probe tests; README.md:108-113 of the reference: scratch is caller-owned, the model owns weights,
the session owns stream, arenas and KV). Measured with the DRIVER's free-memory figure (cudaMemGetInfo) around the
second and later calls of every operator and around verify steps after their graphs exist: an allocation made inside
the library would not show in torch's own allocator statistics. The first call of a kernel may load its module, so
every probe follows a warm call."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def to_dev(torch, bits: np.ndarray):
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def probe(torch, call, repeats=3):
    """Free device bytes must not shrink over `repeats` calls that follow a warm one."""
    call()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(repeats):
        call()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before


def test_operators_allocate_nothing(cuda, package):
    torch, ops, syn = cuda, package.operators, package.synthetic
    ctx = ops.prepare_execution_context(0)
    n, k = 512, 1024
    q, s, z = syn.awq_triple(3, "probe", n, k)
    dq, ds, dz = torch.from_numpy(q).cuda(), to_dev(torch, s), torch.from_numpy(z).cuda()
    awq = ops.prepare_awq(dq, ds, dz, 128, k)
    dense_w = torch.randn((n, k), device="cuda").to(torch.bfloat16)
    dense = ops.prepare_dense(dense_w.t())
    for rows in (9, 300):                                   # the streaming kernels, and the tcgen05 prompt kernel
        x = torch.randn((rows, k), device="cuda").to(torch.bfloat16)
        out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(max(16, ops.linear_scratch_bytes(min(rows, 16), k, n)), dtype=torch.uint8, device="cuda")
        probe(torch, lambda: ops.awq_linear(ctx, x, awq, out, scratch))
        probe(torch, lambda: ops.linear(ctx, x, dense, out, scratch))
    gate_up = ops.prepare_awq(dq, ds, dz, 128, k)
    x = torch.randn((9, k), device="cuda").to(torch.bfloat16)
    act = torch.empty((9, n // 2), dtype=torch.bfloat16, device="cuda")
    probe(torch, lambda: ops.awq_gate_up_silu(ctx, x, gate_up, act))
    a, b = torch.randn((9, 4096), device="cuda").to(torch.bfloat16), torch.randn((9, 4096), device="cuda").to(torch.bfloat16)
    c = torch.empty_like(a)
    weight = torch.ones(4096, dtype=torch.bfloat16, device="cuda")
    probe(torch, lambda: ops.add(ctx, a, b, c))
    probe(torch, lambda: ops.silu_multiply(ctx, a, b, c))
    probe(torch, lambda: ops.rms_norm(ctx, a, weight, c, 9, 4096, 1e-6))
    heads, kv_heads, length, rows = 8, 2, 700, 9
    qv = torch.randn((rows, heads, 128), device="cuda").to(torch.bfloat16)
    kk = torch.randn((length, kv_heads, 128), device="cuda").to(torch.bfloat16)
    vv = torch.randn((length, kv_heads, 128), device="cuda").to(torch.bfloat16)
    ao = torch.empty_like(qv)
    attention_scratch = torch.empty(ops.attention_scratch_bytes(rows, heads, 128, length), dtype=torch.uint8, device="cuda")
    probe(torch, lambda: ops.attention_prefill(ctx, qv, kk, vv, ao, length - rows, attention_scratch))
    table = torch.from_numpy(ops.build_rope_table(1024, 128, 1e6)).cuda()
    probe(torch, lambda: ops.rope_precomputed(ctx, qv, table, 5))
    cache = torch.zeros((64, kv_heads * 128), dtype=torch.bfloat16, device="cuda")
    rows_kv = kk[:9].reshape(9, kv_heads * 128).contiguous()
    probe(torch, lambda: ops.store_kv(ctx, rows_kv, cache, 3))
    ids = torch.randint(0, 50, (9,), dtype=torch.int32, device="cuda")
    emb = torch.randn((50, 256), device="cuda").to(torch.bfloat16)
    gathered = torch.empty((9, 256), dtype=torch.bfloat16, device="cuda")
    probe(torch, lambda: ops.gather(ctx, ids, emb, gathered))
    logits = torch.randn((9, 5000), device="cuda").to(torch.bfloat16)
    tokens = torch.empty(9, dtype=torch.int32, device="cuda")
    sample_scratch = torch.empty(ops.sample_scratch_bytes(9, 5000), dtype=torch.uint8, device="cuda")
    probe(torch, lambda: ops.sample_greedy(ctx, logits, tokens, sample_scratch))


def test_session_steady_path_allocates_nothing(cuda, package):
    """Verify steps (graph replay and eager), one-row decodes and a repeated long-prompt prefill of the same length."""
    torch, syn = cuda, package.synthetic
    shape = package.Shape(vocab_size=2048, n_layers=2, n_heads=8, n_kv_heads=2, hidden_size=1024, intermediate_size=2048,
                          quant_type=1, max_position_embeddings=512)
    model = package.Model(shape, syn.make_model(shape, seed=3))
    prompt = syn.make_prompt(1, 120, shape.vocab_size)
    for graph in (True, False):
        session = model.new_session(256, graph=graph)
        session.prefill(prompt)

        def step():
            session.verify([5, 6, 7, 8, 9])
            session.truncate(120)

        step()                                              # warm run, and the capture of the graph
        probe(torch, step, repeats=5)
        probe(torch, lambda: (session.decode(3), session.truncate(120)), repeats=5)
        probe(torch, lambda: session.prefill(prompt), repeats=2)
