"""Paged-attention decode, KV-cache write / gather and greedy sampling kernels against the
contiguous fp32 reference (paged == contiguous is the reference's own functional test,
tests/MLFramework.Tests/Inference/PagedAttention/PagedAttentionFunctionalTests.cs:41-256)."""
import pytest
import torch

from ml_framework_b200.ops import native
from ml_framework_b200.ops.reference import paged_attention_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,Hq,Hkv,lens", [(3, 4, 1, [1, 16, 17]), (4, 8, 2, [128, 700, 33, 1500]), (2, 4, 4, [2560, 5]),
                                           (5, 32, 8, [40, 41, 600, 64, 1])])
def test_paged_decode_matches_contiguous(B, Hq, Hkv, lens):
    torch.manual_seed(0)
    bs, D = 16, 128
    max_len = max(lens)
    max_blocks = (max_len + bs - 1) // bs
    nb = sum((l + bs - 1) // bs for l in lens) + 3
    cache = torch.randn(nb, 2, bs, Hkv, D, device="cuda").to(torch.bfloat16)
    perm = torch.randperm(nb).tolist()
    table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    k = 0
    for b, l in enumerate(lens):
        n = (l + bs - 1) // bs
        table[b, :n] = torch.tensor(perm[k:k + n], dtype=torch.int32)
        k += n
    table = table.cuda()
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    out = native.paged_decode(q, cache, table, sl, max_len)
    ref = paged_attention_ref(q, cache, table.cpu(), lens)
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2 * (ref.abs().max().item() + 1e-3), err
    # a smaller split size exercises the merge kernel
    out2 = native.paged_decode(q, cache, table, sl, max_len, split_tokens=128)
    assert (out2.float() - ref).abs().max().item() < 2e-2 * (ref.abs().max().item() + 1e-3)
    # split count chosen from the batch size
    out3 = native.paged_decode(q, cache, table, sl, max_len, split_tokens=0)
    assert (out3.float() - ref).abs().max().item() < 2e-2 * (ref.abs().max().item() + 1e-3)
    # splits merged by the last split inside the same launch (twice: the counters must come back to zero)
    for _ in range(2):
        out4 = native.paged_decode(q, cache, table, sl, max_len, split_tokens=128, fused_merge=True)
        assert (out4.float() - ref).abs().max().item() < 2e-2 * (ref.abs().max().item() + 1e-3)


def test_kv_cache_write_gather_and_argmax():
    torch.manual_seed(1)
    nb, bs, Hkv, D, T = 10, 16, 2, 128, 37
    cache = torch.zeros(nb, 2, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    kv = torch.randn(T, 2 * Hkv * D, device="cuda").to(torch.bfloat16)
    k = kv[:, :Hkv * D].view(T, Hkv, D)
    v = kv[:, Hkv * D:].view(T, Hkv, D)
    blocks = [7, 2, 5]
    slots = torch.tensor([blocks[t // bs] * bs + t % bs for t in range(T)], device="cuda")
    slots[3] = -1
    native.kv_cache_write(cache, k, v, slots)
    gk, gv = native.kv_gather(cache, torch.tensor(blocks, dtype=torch.int32, device="cuda"), T)
    mask = torch.ones(T, dtype=torch.bool, device="cuda"); mask[3] = False
    assert torch.equal(gk[mask], k[mask]) and torch.equal(gv[mask], v[mask]) and gk[3].abs().max().item() == 0
    logits = torch.randn(9, 1024, device="cuda").to(torch.bfloat16)
    assert torch.equal(native.argmax_rows(logits, 1000), logits[:, :1000].float().argmax(-1))


def test_executor_cuda_graph_decode_matches_eager():
    """Continuous batching over the paged cache: decode steps replayed from captured CUDA graphs (batch padded to a
    power of two) generate the same tokens as the eager path."""
    from ml_framework_b200.modelzoo.zoo import build_model, default_registry
    from ml_framework_b200.serving.executor import ExecutorConfig, PagedLlamaExecutor
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.scheduler import (BatchConstraints, CompletionConfiguration, ContinuousBatchScheduler, Request,
                                                     SchedulerConfiguration)
    torch.manual_seed(0)
    model = build_model(default_registry().get("llama-tiny"), "cuda", torch.bfloat16).eval()
    mc = model.cfg
    prompts = [[(7 * i + 3 * j) % (mc.vocab_size - 1) + 1 for j in range(20 + 5 * i)] for i in range(5)]
    outs = {}
    for graphs in (False, True):
        kv = KVCacheBlockManager(256, 16, mc.head_dim, mc.n_layers, mc.n_kv_heads, device="cuda", dtype=torch.bfloat16)
        ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=8, max_seq_len=256, prefill_chunk=64, use_cuda_graphs=graphs,
                                                          graph_warmup_steps=1))
        sched = ContinuousBatchScheduler(ex, kv, SchedulerConfiguration(max_batch_size=8, warmup_iterations=0), BatchConstraints(max_batch_size=8),
                                         completion=CompletionConfiguration(eos_token_id=-1, default_max_tokens=12))
        futs = [sched.enqueue(Request(list(p), max_tokens=12)) for p in prompts]
        sched.run_until_idle()
        outs[graphs] = [f.result(1).tokens for f in futs]
        if graphs:
            st = ex._graphs.stats()
            assert st["graphs"] >= 1 and st["replays"] >= 5, st
    same = sum(a == b for x, y in zip(outs[False], outs[True]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs[False])
    assert all(len(x) == 12 for x in outs[True]) and same >= 0.9 * total, (same, total)


def test_batched_prefill_matches_one_by_one():
    """First chunks of equal length prefilled in one pass give the tokens of request-by-request prefill."""
    from ml_framework_b200.modelzoo.zoo import build_model, default_registry
    from ml_framework_b200.serving.executor import ExecutorConfig, PagedLlamaExecutor
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.scheduler import (BatchConstraints, CompletionConfiguration, ContinuousBatchScheduler, Request,
                                                     SchedulerConfiguration)
    torch.manual_seed(0)
    model = build_model(default_registry().get("llama-tiny"), "cuda", torch.bfloat16).eval()
    mc = model.cfg
    prompts = [[(11 * i + 5 * j) % (mc.vocab_size - 1) + 1 for j in range(40 if i < 4 else 23)] for i in range(6)]
    outs = {}
    for budget in (1, 8192):         # 1: every request on its own
        kv = KVCacheBlockManager(256, 16, mc.head_dim, mc.n_layers, mc.n_kv_heads, device="cuda", dtype=torch.bfloat16)
        ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=8, max_seq_len=256, prefill_chunk=64, use_cuda_graphs=False,
                                                          max_prefill_tokens=budget))
        sched = ContinuousBatchScheduler(ex, kv, SchedulerConfiguration(max_batch_size=8, warmup_iterations=0), BatchConstraints(max_batch_size=8),
                                         completion=CompletionConfiguration(eos_token_id=-1, default_max_tokens=6))
        futs = [sched.enqueue(Request(list(p), max_tokens=6)) for p in prompts]
        sched.run_until_idle()
        outs[budget] = [f.result(1).tokens for f in futs]
    same = sum(a == b for x, y in zip(outs[1], outs[8192]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs[1])
    assert all(len(x) == 6 for x in outs[8192]) and same >= 0.9 * total, (same, total)


def test_chunked_prefill_matches_single_chunk():
    """A prompt prefilled in chunks (later chunks attend to the cached prefix through the prefix-attention kernel)
    generates the tokens of the same prompt prefilled at once."""
    from ml_framework_b200.modelzoo.zoo import build_model, default_registry
    from ml_framework_b200.serving.executor import ExecutorConfig, PagedLlamaExecutor
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.scheduler import (BatchConstraints, CompletionConfiguration, ContinuousBatchScheduler, Request,
                                                     SchedulerConfiguration)
    torch.manual_seed(0)
    model = build_model(default_registry().get("llama-tiny"), "cuda", torch.bfloat16).eval()
    mc = model.cfg
    prompts = [[(13 * i + 7 * j) % (mc.vocab_size - 1) + 1 for j in range(150 + 31 * i)] for i in range(3)]
    outs = {}
    for chunk in (512, 64):
        kv = KVCacheBlockManager(256, 16, mc.head_dim, mc.n_layers, mc.n_kv_heads, device="cuda", dtype=torch.bfloat16)
        ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=8, max_seq_len=512, prefill_chunk=chunk, use_cuda_graphs=False))
        sched = ContinuousBatchScheduler(ex, kv, SchedulerConfiguration(max_batch_size=8, warmup_iterations=0), BatchConstraints(max_batch_size=8),
                                         completion=CompletionConfiguration(eos_token_id=-1, default_max_tokens=6))
        futs = [sched.enqueue(Request(list(p), max_tokens=6)) for p in prompts]
        sched.run_until_idle()
        outs[chunk] = [f.result(1).tokens for f in futs]
    same = sum(a == b for x, y in zip(outs[512], outs[64]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs[512])
    assert all(len(x) == 6 for x in outs[64]) and same >= 0.9 * total, (same, total)


def test_fused_rope_and_cache_write_matches_separate_kernels():
    torch.manual_seed(3)
    nb, bs, Hq, Hkv, D, T = 12, 16, 4, 2, 128, 45
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    pos = torch.randint(0, 3000, (T,), device="cuda")
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int64)
    slots[5] = -1
    ref = qkv.clone()
    q = ref[:, :Hq * D].view(T, Hq, D)
    k = ref[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = ref[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    native.rope_(q, pos, 500000.0)
    native.rope_(k, pos, 500000.0)
    cache_ref = torch.zeros(nb, 2, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    native.kv_cache_write(cache_ref, k, v, slots)
    cache = torch.zeros_like(cache_ref)
    native.rope_kv_write_(qkv, pos, slots, cache, Hq, Hkv, 500000.0)
    torch.cuda.synchronize()
    assert torch.equal(qkv, ref) and torch.equal(cache, cache_ref)


def test_paged_attention_layer_native_matches_reference_layer():
    """The standalone layer on the native kernels (bf16, head dimension 128) against the same layer in fp32 PyTorch:
    prefill in two chunks (the second attends to the cached prefix), then two decode steps."""
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.paged_attention_layer import AttentionPhase, PagedAttentionLayer
    torch.manual_seed(0)
    d, hq, hkv, D = 512, 4, 2, 128
    gpu = PagedAttentionLayer(d, hq, hkv, D, rope_theta=10000.0, dtype=torch.bfloat16, device="cuda")
    cpu = PagedAttentionLayer(d, hq, hkv, D, rope_theta=10000.0)
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    kv_g = KVCacheBlockManager(total_blocks=64, block_size=16, head_dim=D, num_layers=1, num_kv_heads=hkv, dtype=torch.bfloat16, device="cuda")
    kv_c = KVCacheBlockManager(total_blocks=64, block_size=16, head_dim=D, num_layers=1, num_kv_heads=hkv, dtype=torch.float32, device="cpu")
    x = (torch.randn(200, d) * 0.5)
    xg = x.cuda().to(torch.bfloat16)
    xc = xg.float().cpu()
    steps = [(slice(0, 128), AttentionPhase.PREFILL), (slice(128, 198), AttentionPhase.PREFILL), (slice(198, 199), AttentionPhase.DECODE),
             (slice(199, 200), AttentionPhase.DECODE)]
    for sl, ph in steps:
        og = gpu(xg[sl], kv_g, [3], ph)
        oc = cpu(xc[sl], kv_c, [3], ph)
        assert torch.allclose(og.float().cpu(), oc, atol=3e-2, rtol=3e-2), (sl, (og.float().cpu() - oc).abs().max())


@pytest.mark.parametrize("Sq,Skv,Hq,Hkv", [(128, 128, 4, 2), (70, 198, 4, 1), (256, 700, 8, 2), (300, 300, 2, 2)])
def test_prefill_attention_through_the_block_table_matches_gathered_attention(Sq, Skv, Hq, Hkv):
    """Queries = the last Sq positions of a sequence of Skv cached tokens; K / V fetched page by page through a
    shuffled block table inside the tcgen05 kernel, against fp32 attention over the gathered pages."""
    from ml_framework_b200.ops import native, reference
    torch.manual_seed(0)
    B, bs, D = 2, 16, 128
    pages = (Skv + bs - 1) // bs
    nb = B * pages + 5
    cache = torch.zeros(nb, 2, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(nb)[: B * pages].reshape(B, pages)
    table = torch.full((B, pages + 3), -1, dtype=torch.int32)
    table[:, :pages] = perm.to(torch.int32)
    k = (torch.randn(B, Skv, Hkv, D, device="cuda") * 0.5).to(torch.bfloat16)
    v = (torch.randn(B, Skv, Hkv, D, device="cuda") * 0.5).to(torch.bfloat16)
    for b in range(B):
        for pg in range(pages):
            lo, hi = pg * bs, min((pg + 1) * bs, Skv)
            cache[perm[b, pg], 0, : hi - lo] = k[b, lo:hi]
            cache[perm[b, pg], 1, : hi - lo] = v[b, lo:hi]
    q = (torch.randn(B * Sq, Hq, D, device="cuda") * 0.5).to(torch.bfloat16)
    out = native.flash_fwd_paged(q, cache, table.cuda(), B, Sq, Skv, causal=True)
    ref, _ = reference.attention_ref(q.view(B, Sq, Hq, D).float(), k.float(), v.float(), causal=True, start_pos=Skv - Sq)
    assert torch.allclose(out.view(B, Sq, Hq, D).float(), ref, atol=2e-2, rtol=2e-2), (out.view(B, Sq, Hq, D).float() - ref).abs().max()
