"""The allocation-free variant of the block-aligned expert sort, called through the C ABI.

Some callers cannot allocate device memory where they route tokens (all GPU memory already
belongs to the KV cache; an allocation would stall every stream of the device), and cannot
pass a scratch buffer either.  `sb200_moe_align_block_size_noalloc` keeps its counters in a
fixed array inside the library.  This test checks that it produces exactly what the regular
entry point produces (integer outputs: bit for bit), on two calls in a row -- the second call
finds the array holding the first call's counters, which must not leak into its result -- and
that it refuses inputs beyond its stated limits.  It is collected last so that a run that
stops at the first failure has already run everything else; it also passes on its own in a
fresh process (the first call on the device sets the array's address up)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(n, E, block):
    cap = n + E * (block - 1)
    return (torch.full((cap,), -3, dtype=torch.int32, device="cuda"),
            torch.full(((cap + block - 1) // block,), -1, dtype=torch.int32, device="cuda"),
            torch.zeros(1, dtype=torch.int32, device="cuda"))


def _compare(ids, E, block):
    from sarathi_serve_b200 import moe_ops
    n = ids.numel()
    s0, e0, n0 = _outputs(n, E, block)
    moe_ops.moe_align_block_size(ids, E, block, s0, e0, n0)          # existing entry point
    s1, e1, n1 = _outputs(n, E, block)
    moe_ops.moe_align_block_size_noalloc(ids, E, block, s1, e1, n1)  # the one that allocates nothing
    torch.cuda.synchronize()
    npp = int(n0)
    assert int(n1) == npp
    assert torch.equal(s1, s0), "sorted_token_ids differ between the two entry points"
    assert torch.equal(e1[:npp // block], e0[:npp // block]), "expert_ids differ between the two entry points"
    # and directly against the CPU oracle of the reference's kernel (not only through the other entry point)
    from oracle import tp_layer_oracle as O
    so, eo, no = O.moe_align_block_size(ids.cpu(), block, E)
    assert int(no) == int(n1)
    assert torch.equal(s1.cpu()[:npp], so[:npp].to(torch.int32)), "sorted_token_ids differ from the oracle"
    assert torch.equal(e1.cpu()[:npp // block], eo[:npp // block].to(torch.int32)), "expert_ids differ from the oracle"


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    g = torch.Generator().manual_seed(11)
    # first call: many slots, every expert busy -> leaves large counters behind in the shared array
    ids_a = torch.randint(0, 64, (30000, 2), generator=g, dtype=torch.int32).cuda()
    _compare(ids_a, 64, 64)
    # second call right after: fewer slots, fewer experts, one expert empty
    ids_b = torch.randint(0, 8, (1024, 2), generator=g, dtype=torch.int32)
    ids_b[ids_b == 5] = 4
    _compare(ids_b.cuda(), 8, 64)
    # and once more with int64 ids and an odd block size
    ids_c = torch.randint(0, 16, (777, 4), generator=g, dtype=torch.int64).cuda()
    _compare(ids_c, 16, 24)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from sarathi_serve_b200 import moe_ops
    ids = torch.zeros(moe_ops.NOALLOC_MAX_SLOTS + 1, dtype=torch.int32, device="cuda")
    s, e, n = _outputs(ids.numel(), 8, 16)
    with pytest.raises(RuntimeError, match="exceed the built-in scratch"):
        moe_ops.moe_align_block_size_noalloc(ids, 8, 16, s, e, n)
    ids = torch.zeros(64, dtype=torch.int32, device="cuda")
    s, e, n = _outputs(64, moe_ops.NOALLOC_MAX_EXPERTS + 1, 4)
    with pytest.raises(RuntimeError, match="exceed the built-in scratch"):
        moe_ops.moe_align_block_size_noalloc(ids, moe_ops.NOALLOC_MAX_EXPERTS + 1, 4, s, e, n)
