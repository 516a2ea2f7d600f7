"""CPU checks of the oracle's op restatements against closed forms, torch
built-ins and the worked example in the reference kernel's comment."""
import numpy as np
import torch

from oracle import tp_layer_oracle as O


def test_moe_align_kernel_comment_example():
    # csrc/moe_align_block_size_kernels.cu:88-93 (reference): 9 slots, 5 experts, block 4
    ids = torch.tensor([0, 1, 2, 1, 2, 3, 0, 3, 4])
    s, e, n = O.moe_align_block_size(ids, 4, 5)
    P = 9
    assert int(n) == 20
    assert s[:20].tolist() == [0, 6, P, P, 1, 3, P, P, 2, 4, P, P, 5, 7, P, P, 8, P, P, P]
    assert e[:5].tolist() == [0, 1, 2, 3, 4]


def test_moe_align_properties():
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 8, (1024, 2), generator=g)
    s, e, n = O.moe_align_block_size(ids, 64, 8)
    n = int(n)
    assert n % 64 == 0 and s.numel() == 2048 + 8 * 63
    valid = s[:n][s[:n] < 2048]
    assert sorted(valid.tolist()) == list(range(2048))  # a permutation of the slots
    flat = ids.reshape(-1)
    for b in range(n // 64):
        blk = s[b * 64:(b + 1) * 64]
        real = blk[blk < 2048]
        assert torch.all(flat[real.long()] == e[b])
        assert torch.all(real[1:] > real[:-1])  # stable: ascending slot index inside an expert


def test_topk_softmax_against_torch():
    g = torch.Generator().manual_seed(1)
    for E in (8, 64, 6):
        logits = torch.randn(300, E, generator=g)
        w, ids, src = O.topk_softmax(logits, 2)
        p = torch.softmax(logits, -1)
        tw, ti = torch.topk(p, 2, dim=-1)
        assert torch.equal(ids.long(), ti)
        assert torch.allclose(w, tw, rtol=1e-5, atol=1e-7)
        assert src[5, 1].item() == 1 * 300 + 5
    w, _, _ = O.topk_softmax(logits, 2, renormalize=True)
    assert torch.allclose(w.sum(-1), torch.ones(300))


def test_rms_norm_and_silu_closed_form():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(9, 64, generator=g)
    w = torch.randn(64, generator=g)
    ref = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(O.rms_norm(x, w, 1e-5), ref, rtol=1e-5, atol=1e-6)
    y = torch.randn(9, 128, generator=g)
    assert torch.allclose(O.silu_and_mul(y), torch.nn.functional.silu(y[:, :64]) * y[:, 64:], rtol=1e-5, atol=1e-6)
    assert torch.allclose(O.gelu_new(x), torch.nn.functional.gelu(x, approximate="tanh"), rtol=1e-4, atol=1e-5)
    assert torch.allclose(O.gelu_fast(x), torch.nn.functional.gelu(x, approximate="tanh"), rtol=1e-4, atol=1e-5)


def test_rotary_is_a_rotation():
    """Norm-preserving and equal to the complex-multiplication form, both styles."""
    g = torch.Generator().manual_seed(3)
    cache = O.cos_sin_cache(64, 64, 128, 10000.0, torch.float32)
    pos = torch.randint(0, 128, (11,), generator=g)
    for neox in (True, False):
        q = torch.randn(11, 4 * 64, generator=g)
        k = torch.randn(11, 2 * 64, generator=g)
        q0, k0 = q.clone(), k.clone()
        O.rotary_embedding(pos, q, k, 64, cache, neox)
        assert torch.allclose(q.view(11, 4, 64).norm(dim=-1), q0.view(11, 4, 64).norm(dim=-1), rtol=1e-5)
        v0 = q0.view(11, 4, 64)
        if neox:
            z = torch.complex(v0[..., :32], v0[..., 32:])
        else:
            z = torch.complex(v0[..., 0::2], v0[..., 1::2])
        ang = torch.complex(cache[pos][:, None, :32], cache[pos][:, None, 32:])
        zr = z * ang
        got = q.view(11, 4, 64)
        gz = torch.complex(got[..., :32], got[..., 32:]) if neox else torch.complex(got[..., 0::2], got[..., 1::2])
        assert torch.allclose(torch.view_as_real(gz), torch.view_as_real(zr), rtol=1e-5, atol=1e-6)


def test_fused_experts_matches_dense_evaluation():
    g = torch.Generator().manual_seed(4)
    T, H, I, E = 13, 32, 48, 4
    x = torch.randn(T, H, generator=g)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.1
    w2 = torch.randn(E, H, I, generator=g) * 0.1
    w, ids, _ = O.topk_softmax(torch.randn(T, E, generator=g), 2, renormalize=True)
    out = O.fused_experts(x, w13, w2, w, ids)
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(2):
            e = int(ids[t, j])
            gu = w13[e] @ x[t]
            a = torch.nn.functional.silu(gu[:I]) * gu[I:]
            ref[t] += w[t, j] * (w2[e] @ a)
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-5)


def test_vocab_parallel_embedding_equals_the_full_table_lookup():
    g = torch.Generator().manual_seed(3)
    table = torch.randn(96, 40, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 96, (57,), generator=g)
    for tp in (1, 2, 4, 8):
        shards = list(table.chunk(tp, dim=0))
        assert torch.equal(O.vocab_parallel_embedding(ids, shards), table[ids])


def test_kv_cache_append_oracle_on_a_hand_worked_batch():
    """Two requests, pages of 4 slots: request 0 holds 3 tokens and appends 3 (positions 3, 4, 5: the last
    slot of its first page, then two slots of its second page), request 1 appends its first token."""
    page = 4
    kv_indices = [7, 2, 5]       # request 0 owns pages 7 and 2, request 1 page 5
    kv_indptr = [0, 2, 3]
    batch_indices = [0, 0, 0, 1, -1]
    positions = [3, 4, 5, 0, 0]
    s = O.kv_cache_slots(batch_indices, positions, kv_indices, kv_indptr, page)
    assert s.tolist() == [7 * 8 + 3, 2 * 8 + 0, 2 * 8 + 1, 5 * 8 + 0, -1]
    cache = torch.zeros(8, 2, page, 1, 2)
    k = torch.arange(10, dtype=torch.float32).view(5, 1, 2) + 1
    v = -k
    O.append_paged_kv_cache(k, v, batch_indices, positions, cache, kv_indices, kv_indptr)
    assert torch.equal(cache[7, 0, 3], k[0]) and torch.equal(cache[7, 1, 3], v[0])
    assert torch.equal(cache[2, 0, 0], k[1]) and torch.equal(cache[2, 1, 1], v[2])
    assert torch.equal(cache[5, 0, 0], k[3]) and torch.equal(cache[5, 1, 0], v[3])
    assert float(cache.abs().sum()) == float(k[:4].abs().sum() * 2)  # the padding entry stored nothing
