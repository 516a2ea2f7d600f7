"""Paged KV-cache append (cache layout [pages, 2, page_size, kv_heads, head_dim]): the standalone kernels and the
append fused into the qkv + rotary GEMM epilogue, against the CPU oracle and -- where the installed flashinfer
can run it -- against flashinfer's own append_paged_kv_cache, the call the reference makes
(sarathi/model_executor/attention/flashinfer_attention_wrapper.py:253-270).  Copies: bit for bit."""
import pytest
import torch

from oracle import tp_layer_oracle as O

pytestmark = pytest.mark.gpu


def _batch(seed, page_size, lens_before, lens_new, num_pages, pad=0):
    """A Sarathi-style step: request r already holds lens_before[r] tokens and appends lens_new[r] (a prefill
    chunk or one decode token).  Pages are handed out in a shuffled order."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    kv_indices, kv_indptr, batch_indices, positions = [], [0], [], []
    for r, (a, n) in enumerate(zip(lens_before, lens_new)):
        need = -(-(a + n) // page_size)
        kv_indices += [perm.pop() for _ in range(need)]
        kv_indptr.append(len(kv_indices))
        batch_indices += [r] * n
        positions += list(range(a, a + n))
    batch_indices += [-1] * pad  # padding tokens of the batch are not stored
    positions += [0] * pad
    t = lambda v: torch.tensor(v, dtype=torch.int32)
    return t(batch_indices), t(positions), t(kv_indices), t(kv_indptr)


CASES = [(16, [0, 37, 512, 5, 1000], [448, 1, 1, 1, 1], 200, 4), (16, [0], [1], 4, 0), (8, [3, 0, 15], [13, 8, 1], 16, 7)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("case", CASES)
def test_slots_and_append_against_oracle(dtype, case):
    from sarathi_serve_b200 import kv_cache_ops
    page, before, new, pages, pad = case
    bi, pos, ki, kp = _batch(1, page, before, new, pages, pad)
    n, nkv, hd = bi.numel(), 2, 128
    s_ref = O.kv_cache_slots(bi, pos, ki, kp, page)
    s = kv_cache_ops.slots(bi.cuda(), pos.cuda(), ki.cuda(), kp.cuda(), page)
    assert torch.equal(s.cpu(), s_ref)
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(n, (4 + 2 * nkv) * hd, generator=g).to(dtype)
    k, v = qkv[:, 4 * hd:(4 + nkv) * hd], qkv[:, (4 + nkv) * hd:]   # strided views, as the layer has them
    cache0 = torch.randn(pages, 2, page, nkv, hd, generator=g).to(dtype)
    ref = cache0.clone()
    O.append_paged_kv_cache(k, v, bi, pos, ref, ki, kp)
    cache = cache0.clone().cuda()
    qkv_d = qkv.cuda()
    kv_cache_ops.append_paged_kv_cache(qkv_d[:, 4 * hd:(4 + nkv) * hd], qkv_d[:, (4 + nkv) * hd:], bi.cuda(), pos.cuda(),
                                       cache, ki.cuda(), kp.cuda(), None)
    assert torch.equal(cache.cpu(), ref)
    assert not torch.equal(ref, cache0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_append_matches_flashinfer(dtype):
    """The dependency's own kernel on the same inputs (it is what the reference calls)."""
    try:
        from flashinfer.page import append_paged_kv_cache as fi_append
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"flashinfer not importable: {exc}")
    from sarathi_serve_b200 import kv_cache_ops
    page, before, new, pages, _ = CASES[0]
    bi, pos, ki, kp = _batch(3, page, before, new, pages, 0)
    n, nkv, hd = bi.numel(), 8, 128
    g = torch.Generator().manual_seed(4)
    k = torch.randn(n, nkv, hd, generator=g).to(dtype).cuda()
    v = torch.randn(n, nkv, hd, generator=g).to(dtype).cuda()
    cache0 = torch.randn(pages, 2, page, nkv, hd, generator=g).to(dtype).cuda()
    theirs, ours = cache0.clone(), cache0.clone()
    last = torch.tensor([((a + m - 1) % page) + 1 for a, m in zip(before, new)], dtype=torch.int32).cuda()
    try:
        fi_append(k, v, bi.cuda(), pos.cuda(), theirs, ki.cuda(), kp.cuda(), last, kv_layout="NHD")
        torch.cuda.synchronize()
    except Exception as exc:  # its JIT needs a compiler cache / network it may not have on this box
        pytest.skip(f"flashinfer's append_paged_kv_cache cannot run here: {type(exc).__name__}: {str(exc)[:120]}")
    kv_cache_ops.append_paged_kv_cache(k, v, bi.cuda(), pos.cuda(), ours, ki.cuda(), kp.cuda(), last)
    assert torch.equal(ours, theirs)
    ref = cache0.cpu().clone()
    O.append_paged_kv_cache(k.cpu(), v.cpu(), bi, pos, ref, ki, kp)
    assert torch.equal(theirs.cpu(), ref), "the oracle restates flashinfer's addressing"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tile_n", [0, 64, 3064, 128, 3256, 203128, 2256])
@pytest.mark.parametrize("nq,nkv,hd", [(4, 1, 128), (8, 2, 64)])
def test_qkv_rotary_epilogue_appends_to_the_cache(dtype, tile_n, nq, nkv, hd):
    """qkv GEMM + rotary + KV-cache append in one kernel = the unfused sequence (GEMM + rotary, then append)."""
    from sarathi_serve_b200 import dense_ops, kv_cache_ops
    if tile_n and (tile_n % 1000) % hd and not (tile_n % 1000 == 64 and hd > 64):
        pytest.skip("tile configuration does not fit this head size")
    page, before, new, pages, pad = CASES[2] if hd == 64 else CASES[0]
    bi, pos_in_req, ki, kp = _batch(5, page, before, new, pages, pad)
    T, K = bi.numel(), 512
    N = (nq + 2 * nkv) * hd
    g = torch.Generator().manual_seed(6)
    x = torch.randn(T, K, generator=g).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) * 0.03).to(dtype).cuda()
    positions = pos_in_req.to(torch.int64).cuda()
    cs = O.cos_sin_cache(hd, hd, 2048, 10000.0, dtype).cuda()
    cache0 = torch.randn(pages, 2, page, nkv, hd, generator=g).to(dtype).cuda()
    slots = kv_cache_ops.slots(bi.cuda(), pos_in_req.cuda(), ki.cuda(), kp.cuda(), page)
    # unfused: GEMM + rotary, then the append kernel on the k / v views
    qkv_ref = dense_ops.linear_rotary(x, w, positions, cs, hd, (nq + nkv) * hd, True, tile_n=tile_n)
    want = cache0.clone()
    kv_cache_ops.append_rows(want, qkv_ref[:, nq * hd:(nq + nkv) * hd], qkv_ref[:, (nq + nkv) * hd:], slots)
    # fused
    got = cache0.clone()
    qkv = dense_ops.linear_rotary(x, w, positions, cs, hd, (nq + nkv) * hd, True, tile_n=tile_n, kv_cache=got,
                                  kv_slots=slots, num_kv_heads=nkv)
    dense_ops.check_status(torch.device("cuda", torch.cuda.current_device()))
    assert torch.equal(qkv, qkv_ref)
    assert torch.equal(got, want)
    assert not torch.equal(got, cache0)
