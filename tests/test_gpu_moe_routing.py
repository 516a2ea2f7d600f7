"""GPU parity of the MoE routing kernels through the C ABI: ids and the block
alignment must be BIT-EXACT against the oracle and against the reference's own
kernels (oracle/_ref) on identical inputs."""
import pytest
import torch

import ref_kernels
from oracle import tp_layer_oracle as O

pytestmark = pytest.mark.gpu


def _topk(gating, k, renorm=False):
    from sarathi_serve_b200 import moe_ops
    T = gating.shape[0]
    w = torch.empty(T, k, dtype=torch.float32, device="cuda")
    ids = torch.empty(T, k, dtype=torch.int32, device="cuda")
    src = torch.empty(T, k, dtype=torch.int32, device="cuda")
    moe_ops.topk_softmax(w, ids, src, gating, renormalize=renorm)
    return w, ids, src


@pytest.mark.parametrize("E", [1, 2, 4, 8, 16, 32, 64, 128, 256, 6, 48, 300])
@pytest.mark.parametrize("T,k", [(1, 1), (7, 2), (64, 2), (1024, 2), (1000, 4)])
def test_topk_softmax(E, T, k):
    if k > E:
        pytest.skip("k > E")
    g = torch.Generator().manual_seed(E * 100 + T)
    logits = torch.randn(T, E, generator=g)
    w, ids, src = _topk(logits.cuda(), k)
    ow, oids, osrc = O.topk_softmax(logits, k)
    assert torch.equal(ids.cpu(), oids), "expert ids differ from the oracle"
    assert torch.equal(src.cpu(), osrc)
    assert torch.allclose(w.cpu(), ow, rtol=1e-5, atol=1e-7)
    ref = ref_kernels.load("moe_ops")
    if ref is not None:
        rw = torch.empty(T, k, dtype=torch.float32, device="cuda")
        rids = torch.empty(T, k, dtype=torch.int32, device="cuda")
        rsrc = torch.empty(T, k, dtype=torch.int32, device="cuda")
        ref.topk_softmax(rw, rids, rsrc, logits.cuda())
        assert torch.equal(ids, rids), "expert ids differ from the reference kernel"
        assert torch.equal(src, rsrc)
        assert torch.equal(w, rw), "softmax weights differ from the reference kernel (same evaluation order expected)"


def test_topk_ties_pick_lowest_index():
    logits = torch.zeros(5, 8)
    logits[1, 3] = logits[1, 6] = 2.0
    _, ids, _ = _topk(logits.cuda(), 2)
    assert ids.cpu().tolist() == [[0, 1], [3, 6], [0, 1], [0, 1], [0, 1]]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_topk_low_precision_logits_and_renorm(dtype):
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(1024, 8, generator=g).to(dtype)
    w, ids, _ = _topk(logits.cuda(), 2, renorm=True)
    ow, oids, _ = O.topk_softmax(logits.float(), 2, renormalize=True)
    assert torch.equal(ids.cpu(), oids)
    assert torch.allclose(w.cpu(), ow, rtol=1e-5, atol=1e-7)
    assert torch.allclose(w.sum(-1), torch.ones(1024, device="cuda"), atol=1e-6)


def _align(ids, E, block, scratch=False):
    from sarathi_serve_b200 import moe_ops
    n = ids.numel()
    cap = n + E * (block - 1)
    sorted_ids = torch.full((cap,), -7, dtype=torch.int32, device="cuda")  # NOT pre-filled with the pad value
    nblk = (cap + block - 1) // block
    expert_ids = torch.full((nblk,), -1, dtype=torch.int32, device="cuda")
    npp = torch.zeros(1, dtype=torch.int32, device="cuda")
    scr = None
    if scratch:
        scr = torch.empty(moe_ops.moe_align_scratch_bytes(n, E), dtype=torch.uint8, device="cuda")
    moe_ops.moe_align_block_size(ids, E, block, sorted_ids, expert_ids, npp, scratch=scr)
    return sorted_ids, expert_ids, npp


def test_align_kernel_comment_example():
    """The worked example in the reference kernel's comment
    (csrc/moe_align_block_size_kernels.cu:88-93)."""
    ids = torch.tensor([0, 1, 2, 1, 2, 3, 0, 3, 4], dtype=torch.int32)
    s, e, n = _align(ids.cuda(), 5, 4)
    P = 9
    assert int(n) == 20
    assert s[:20].cpu().tolist() == [0, 6, P, P, 1, 3, P, P, 2, 4, P, P, 5, 7, P, P, 8, P, P, P]
    assert e[:5].cpu().tolist() == [0, 1, 2, 3, 4]


@pytest.mark.parametrize("itype", [torch.int32, torch.int64, torch.int16, torch.uint8])
@pytest.mark.parametrize("T,k,E,block", [(1, 2, 8, 64), (7, 2, 8, 16), (1024, 2, 8, 64), (1000, 4, 64, 32),
                                         (77, 2, 8, 64), (5000, 2, 8, 128), (20000, 2, 16, 64), (300, 1, 3, 5)])
@pytest.mark.parametrize("scratch", [False, True])
def test_moe_align_block_size(itype, T, k, E, block, scratch):
    g = torch.Generator().manual_seed(T + E)
    ids = torch.randint(0, E, (T, k), generator=g).to(itype)
    if E > 2:
        ids[ids == 1] = 0  # leave one expert empty
    s, e, n = _align(ids.cuda(), E, block, scratch)
    os_, oe, on = O.moe_align_block_size(ids.to(torch.int64), block, E)
    npp = int(on)
    assert int(n) == npp
    assert torch.equal(s.cpu(), os_), "sorted_token_ids (including the pad fill) differ from the oracle"
    assert torch.equal(e[:npp // block].cpu(), oe[:npp // block])
    ref = ref_kernels.load("moe_ops")
    if ref is not None and itype != torch.uint8 or (ref is not None and E <= 255):
        rs = torch.full_like(s, T * k)
        re_ = torch.empty_like(e)
        rn = torch.empty(1, dtype=torch.int32, device="cuda")
        ref.moe_align_block_size(ids.cuda(), E, block, rs, re_, rn)
        assert int(rn) == int(n)
        assert torch.equal(rs, s), "sorted_token_ids differ from the reference kernel"
        assert torch.equal(re_[:npp // block], e[:npp // block])


def test_align_empty():
    ids = torch.empty(0, 2, dtype=torch.int32, device="cuda")
    s, e, n = _align(ids, 8, 64)
    assert int(n) == 0 and torch.all(s == 0)
