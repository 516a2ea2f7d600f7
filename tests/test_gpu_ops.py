"""GPU parity of the bandwidth kernels, called through the C ABI (ctypes):
against the CPU oracle, and -- when oracle/_ref was built -- against the
reference's own CUDA kernels on identical inputs (bit-exact where the kernel has
no reduction-order freedom)."""
import pytest
import torch

import ref_kernels
from helpers import TOL, rel_err
from oracle import tp_layer_oracle as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]
TS = [1, 7, 8, 63, 64, 65, 288, 512]


def _same(a, b, dtype, what):
    """Element-wise kernels without a reduction: for the 16-bit types every operator result is
    rounded explicitly, so results must agree bit for bit; in fp32 the compiler is free to
    contract a*b+c into an fma, so only a few ulps are allowed there."""
    if dtype == torch.float32:
        assert rel_err(a, b) <= 2e-6, what
    else:
        assert torch.equal(a, b), what + " (bit-exact expected)"


def _canary(shape, dtype, pad=64):
    """Output buffer with guard elements on both sides; returns (view, check())."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * pad,), 777.0, dtype=dtype, device="cuda")
    view = buf[pad:pad + n].view(*shape)

    def check():
        assert torch.all(buf[:pad] == 777.0) and torch.all(buf[pad + n:] == 777.0), "kernel wrote outside its output"
    return view, check


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("H", [1024, 4096, 8192, 100])
def test_rms_norm(dtype, T, H):
    from sarathi_serve_b200 import layernorm_ops
    g = torch.Generator().manual_seed(T * 1000 + H)
    x = torch.randn(T, H, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    out, check = _canary((T, H), dtype)
    layernorm_ops.rms_norm(out, x.cuda(), w.cuda(), 1e-5)
    check()
    assert rel_err(out, O.rms_norm(x, w, 1e-5)) <= TOL[dtype]
    ref = ref_kernels.load("layernorm_ops")
    if ref is not None:
        r = torch.empty(T, H, dtype=dtype, device="cuda")
        ref.rms_norm(r, x.cuda(), w.cuda(), 1e-5)
        # the block reduction order differs, so allow the last bit of the statistic to move
        assert rel_err(out, r) <= (1e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 4096), (65, 1024), (512, 4096), (9, 72)])
def test_fused_add_rms_norm(dtype, T, H):
    from sarathi_serve_b200 import layernorm_ops
    g = torch.Generator().manual_seed(T + H)
    x = torch.randn(T, H, generator=g).to(dtype)
    r = torch.randn(T, H, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    out, c1 = _canary((T, H), dtype)
    z, c2 = _canary((T, H), dtype)
    layernorm_ops.fused_add_rms_norm(out, z, x.cuda(), r.cuda(), w.cuda(), 1e-5)
    c1(); c2()
    ro, rz = O.add_rms_norm(x, r, w, 1e-5)
    assert torch.equal(z.cpu(), rz)  # a single rounded add: bit-exact
    assert rel_err(out, ro) <= TOL[dtype]
    # in-place on the residual
    rc = r.cuda().clone()
    out2 = torch.empty(T, H, dtype=dtype, device="cuda")
    layernorm_ops.fused_add_rms_norm(out2, rc, x.cuda(), rc, w.cuda(), 1e-5)
    assert torch.equal(rc, z) and torch.equal(out2, out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("d", [1408, 1792, 14336, 33])
def test_silu_and_mul(dtype, T, d):
    from sarathi_serve_b200 import activation_ops
    if T * d > 3_000_000:
        pytest.skip("covered by the smaller row counts")
    g = torch.Generator().manual_seed(T + d)
    x = (2 * torch.randn(T, 2 * d, generator=g)).to(dtype)
    out, check = _canary((T, d), dtype)
    activation_ops.silu_and_mul(out, x.cuda())
    check()
    assert rel_err(out, O.silu_and_mul(x)) <= TOL[dtype]
    ref = ref_kernels.load("activation_ops")
    if ref is not None:
        r = torch.empty(T, d, dtype=dtype, device="cuda")
        ref.silu_and_mul(r, x.cuda())
        _same(out, r, dtype, "silu_and_mul vs the reference kernel")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fn", ["gelu_new", "gelu_fast"])
@pytest.mark.parametrize("T,d", [(7, 4096), (64, 1000), (1, 3)])
def test_gelu(dtype, fn, T, d):
    from sarathi_serve_b200 import activation_ops
    g = torch.Generator().manual_seed(T + d)
    x = (2 * torch.randn(T, d, generator=g)).to(dtype)
    out, check = _canary((T, d), dtype)
    getattr(activation_ops, fn)(out, x.cuda())
    check()
    assert rel_err(out, getattr(O, fn)(x)) <= TOL[dtype]
    closed = torch.nn.functional.gelu(x.float(), approximate="tanh")
    assert rel_err(out.float(), closed) <= 2e-2
    ref = ref_kernels.load("activation_ops")
    if ref is not None:
        r = torch.empty(T, d, dtype=dtype, device="cuda")
        getattr(ref, fn)(r, x.cuda())
        _same(out, r, dtype, f"{fn} vs the reference kernel")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("T,nq,nkv,hd,rot", [(1, 4, 1, 128, 128), (65, 16, 4, 64, 64), (288, 8, 2, 64, 64),
                                             (512, 4, 1, 128, 128), (33, 3, 3, 80, 40), (9, 2, 1, 256, 256)])
def test_rotary_embedding(dtype, neox, T, nq, nkv, hd, rot):
    from sarathi_serve_b200 import pos_encoding_ops
    g = torch.Generator().manual_seed(T + nq)
    max_pos = 4096
    cache = O.cos_sin_cache(hd, rot, max_pos, 10000.0, dtype)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, generator=g).to(dtype)
    pos = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int64)
    ref_qkv = qkv.clone()
    rq, rk, _ = ref_qkv.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    O.rotary_embedding(pos, rq, rk, hd, cache, neox)
    dev = qkv.cuda()
    q, k, v = dev.split([nq * hd, nkv * hd, nkv * hd], dim=-1)  # strided views, as in the model
    pos_encoding_ops.rotary_embedding(pos.cuda(), q, k, hd, cache.cuda(), neox)
    _same(dev.cpu(), ref_qkv, dtype, "rotary vs the oracle")
    ref = ref_kernels.load("pos_encoding_ops")
    if ref is not None:
        dev2 = qkv.cuda()
        q2, k2, _ = dev2.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
        ref.rotary_embedding(pos.cuda(), q2, k2, hd, cache.cuda(), neox)
        _same(dev, dev2, dtype, "rotary vs the reference kernel")


def test_empty_inputs():
    from sarathi_serve_b200 import activation_ops, layernorm_ops
    x = torch.empty(0, 4096, dtype=torch.bfloat16, device="cuda")
    layernorm_ops.rms_norm(torch.empty_like(x), x, torch.ones(4096, dtype=torch.bfloat16, device="cuda"), 1e-5)
    activation_ops.silu_and_mul(torch.empty(0, 2048, dtype=torch.bfloat16, device="cuda"), x)


def test_cpu_tensors_are_rejected():
    from sarathi_serve_b200 import layernorm_ops
    x = torch.randn(4, 64)
    with pytest.raises(RuntimeError):
        layernorm_ops.rms_norm(torch.empty_like(x), x, torch.ones(64), 1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,H,V", [(512, 4096, 1024), (7, 40, 96), (1, 8, 16), (300, 1000, 333), (0, 64, 32)])
def test_vocab_embedding_slices(dtype, T, H, V):
    """Every rank's masked lookup (any slice of the vocabulary) is bit-exact, and the slices add up to the
    full-table lookup of the oracle."""
    from sarathi_serve_b200 import embedding_ops
    g = torch.Generator().manual_seed(T + H + V)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g)
    total = torch.zeros(T, H, dtype=torch.float32)
    bounds = [0, V // 3, V // 3, (2 * V) // 3, V]  # includes an empty slice
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        out = torch.full((T, H), 7.0, dtype=dtype, device="cuda")
        embedding_ops.vocab_embedding(out, ids.cuda(), table[lo:hi].contiguous().cuda(), lo, hi)
        mask = (ids >= lo) & (ids < hi)
        ref = torch.zeros(T, H, dtype=dtype)
        ref[mask] = table[ids[mask]]
        assert torch.equal(out.cpu(), ref)
        total += out.float().cpu()
    if T:
        assert torch.equal(total.to(dtype), O.vocab_parallel_embedding(ids, [table]))


def test_vocab_parallel_embedding_module_tp1():
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.tp_layers import VocabParallelEmbedding
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    try:
        emb = VocabParallelEmbedding(1000, 256, params_dtype=torch.bfloat16)
        assert emb.weight.shape == (1000, 256) and emb.vocab_start_index == 0 and emb.vocab_end_index == 1000
        g = torch.Generator().manual_seed(0)
        w = torch.randn(1000, 256, generator=g).to(torch.bfloat16)
        emb.weight.data.copy_(w)
        ids = torch.randint(0, 1000, (5, 13), generator=g)
        out = emb(ids.cuda())
        assert out.shape == (5, 13, 256) and torch.equal(out.cpu(), w[ids])
    finally:
        ps.destroy_model_parallel()
