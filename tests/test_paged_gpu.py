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
