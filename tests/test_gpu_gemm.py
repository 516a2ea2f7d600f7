"""GPU parity of the dense projections (tcgen05 GEMM for bf16/fp16, FFMA for
fp32) through the C ABI, against a plain fp32 torch matmul of the same operands
and against the CPU oracle for the fused epilogues."""
import pytest
import torch

from helpers import rel_err
from oracle import tp_layer_oracle as O

pytestmark = pytest.mark.gpu

GEMM_TOL = {torch.float32: 2e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# Per-rank shapes of the 70B-shaped layer at TP=8 (hidden 8192, 64 q / 8 kv heads, intermediate 28672;
# T = 512): qkv N=1280, o_proj K=1024, gate_up N=7168 (d=3584), down K=3584.
def test_70b_shaped_tp8_shard_projections():
    from sarathi_serve_b200 import dense_ops
    T, H = 512, 8192
    dtype = torch.bfloat16
    x = _rand((T, H), dtype, 11)
    # qkv + rotary: 8 q heads + 1 k head rotated, 1 v head untouched
    wqkv = _rand((1280, H), dtype, 12, 0.02)
    pos = torch.arange(T, dtype=torch.int64) * 5 % 4096
    cache = O.cos_sin_cache(128, 128, 8192, 500000.0, dtype)
    ref = (x.float() @ wqkv.float().t()).to(dtype)
    q, k = ref[:, :1024].clone(), ref[:, 1024:1152].clone()
    O.rotary_embedding(pos, q, k, 128, cache, True)
    out = dense_ops.linear_rotary(x.cuda(), wqkv.cuda(), pos.cuda(), cache.cuda(), 128, 1152, True)
    _check_status()
    assert rel_err(out[:, :1024].float().cpu(), q.float()) <= 2e-2
    assert rel_err(out[:, 1024:1152].float().cpu(), k.float()) <= 2e-2
    assert rel_err(out[:, 1152:].float().cpu(), ref[:, 1152:].float()) <= 2e-2
    # gate_up + SiLU*mul
    wgu = _rand((7168, H), dtype, 13, 0.02)
    gu = (x.float() @ wgu.float().t()).to(dtype)
    act_ref = O.silu_and_mul(gu)
    act = dense_ops.linear_silu_mul(x.cuda(), wgu.cuda())
    _check_status()
    assert rel_err(act.float().cpu(), act_ref.float()) <= 2e-2
    # o_proj / down shards (K = 1024, 3584), output rows of 16 KiB
    for K, seed in ((1024, 14), (3584, 15)):
        a, w = _rand((T, K), dtype, seed), _rand((H, K), dtype, seed + 10, 0.02)
        y = dense_ops.linear(a.cuda(), w.cuda())
        _check_status()
        assert rel_err(y.float().cpu(), a.float() @ w.float().t()) <= 2e-2


def _check_status():
    from sarathi_serve_b200 import dense_ops
    dense_ops.check_status(torch.device("cuda", torch.cuda.current_device()))


# tile configuration = BN + 1000*MI + 100000*splitK (0 = chosen by the library)
TILE_CFGS = [0, 64, 96, 128, 160, 224, 256, 2064, 2128, 2256, 301128, 402256, 1602128, 200032,
             3064, 3128, 3192, 3256, 203256, 503128, 4064, 4128, 4256, 304256,  # 3xxx/4xxx = CTA pairs (cta_group::2)
             205256, 205128, 405128, 205064, 405064, 405192]  # 5xxx = a cluster of 2 / 4 CTA pairs splits the K of every tile


def _skip_unless_planned(epi, T, N, K, cfg, head_size=128):
    """Cluster K-split configurations are only accepted for problems with few tiles (one cluster per tile)."""
    from sarathi_serve_b200 import dense_ops
    if (cfg // 1000) % 100 == 5:
        try:
            dense_ops.gemm_plan(epi, T, N, K, head_size, cfg)
        except RuntimeError:
            pytest.skip("this problem does not fit the cluster K-split configuration")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("tile_n", TILE_CFGS)
@pytest.mark.parametrize("T,N,K", [(128, 128, 64), (128, 256, 128), (512, 768, 4096), (288, 768, 1024), (1, 256, 512),
                                   (65, 200, 264), (300, 1000, 1000), (512, 6144, 512), (1024, 8, 4096)])
def test_linear(dtype, tile_n, T, N, K):
    from sarathi_serve_b200 import dense_ops
    if dtype == torch.float32 and tile_n not in (0,):
        pytest.skip("tile shape applies to the tensor-core path only")
    if tile_n // 100000 > (K + 63) // 64:
        pytest.skip("more splits than k-blocks")
    _skip_unless_planned(0, T, N, K, tile_n)
    x, w = _rand((T, K), dtype, T + N + K), _rand((N, K), dtype, 7 * N + K, 0.05)
    b = _rand((N,), dtype, 3)
    ref = x.float().cuda() @ w.float().cuda().t()
    out = dense_ops.linear(x.cuda(), w.cuda(), tile_n=tile_n)
    _check_status()
    assert rel_err(out.float(), ref) <= GEMM_TOL[dtype]
    outb = dense_ops.linear(x.cuda(), w.cuda(), b.cuda(), tile_n=tile_n)
    assert rel_err(outb.float(), ref + b.float().cuda()) <= GEMM_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tile_n", [0, 128, 3256, 203128, 2064, 205256, 405128])
@pytest.mark.parametrize("T,N,K", [(512, 4096, 512), (65, 200, 264), (300, 1000, 1000), (1, 256, 512)])
def test_linear_with_residual_in_the_epilogue(dtype, tile_n, T, N, K):
    """out = residual + round(x w^T + b): the reference's `hidden_states = residual + hidden_states` after a
    row-parallel projection (models/llama.py:248,254) fused into the plain GEMM (what runs at TP = 1)."""
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import dense_ops
    if tile_n // 100000 > (K + 63) // 64:
        pytest.skip("more splits than k-blocks")
    _skip_unless_planned(0, T, N, K, tile_n)
    x, w = _rand((T, K), dtype, T + N + K), _rand((N, K), dtype, 7 * N + K, 0.05)
    b, r = _rand((N,), dtype, 3), _rand((T, N), dtype, 4)
    ref = r + O.linear(x.float(), w.float(), b.float()).to(dtype)
    out = dense_ops.linear(x.cuda(), w.cuda(), b.cuda(), tile_n=tile_n, residual=r.cuda())
    _check_status()
    assert rel_err(out.float(), ref.float()) <= GEMM_TOL[dtype]
    # strided residual view and a caller-provided output
    big = torch.zeros(T, N + 64, dtype=dtype, device="cuda")
    big[:, 32:32 + N] = r.cuda()
    out2 = torch.empty(T, N, dtype=dtype, device="cuda")
    dense_ops.linear(x.cuda(), w.cuda(), b.cuda(), out=out2, tile_n=tile_n, residual=big[:, 32:32 + N])
    assert torch.equal(out2, out)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_linear_strided_operands(dtype):
    """A and the output may be row-strided views (q view of the fused qkv buffer feeding o_proj)."""
    from sarathi_serve_b200 import dense_ops
    big = _rand((130, 1536), dtype, 1).cuda()
    x = big[:, 256:256 + 512]  # row stride 1536, 16-byte aligned start
    w = _rand((384, 512), dtype, 2, 0.05).cuda()
    outbuf = torch.zeros(130, 1024, dtype=dtype, device="cuda")
    out = outbuf[:, 128:128 + 384]
    dense_ops.linear(x, w, out=out)
    _check_status()
    assert rel_err(out.float(), x.float() @ w.float().t()) <= GEMM_TOL[dtype]
    assert torch.all(outbuf[:, :128] == 0) and torch.all(outbuf[:, 512:] == 0)


def test_linear_rejects_misaligned_stride():
    from sarathi_serve_b200 import dense_ops
    x = torch.randn(16, 100, dtype=torch.bfloat16, device="cuda")[:, :68]  # 68*2 bytes rows of a 100-wide buffer
    w = torch.randn(32, 68, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        dense_ops.linear(x[:, 1:65], w[:, :64].contiguous())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("tile_n", [0, 256, 2256, 401256, 302256, 3256, 303256, 4256, 204128,
                                    # 64-column tiles: for NeoX heads wider than 64 a tile holds 32 + 32 columns of
                                    # the two halves of a head, so that every rotation pair sits in one accumulator
                                    64, 2064, 3064, 4064, 303064, 600064,
                                    205128, 405128, 205064, 405256])
@pytest.mark.parametrize("T,nq,nkv,hd,K", [(512, 4, 1, 128, 4096), (288, 8, 2, 64, 1024), (65, 2, 2, 128, 512),
                                           (7, 1, 1, 256, 256)])
def test_linear_rotary(dtype, neox, tile_n, T, nq, nkv, hd, K):
    from sarathi_serve_b200 import dense_ops
    N = (nq + 2 * nkv) * hd
    x, w = _rand((T, K), dtype, T + K), _rand((N, K), dtype, N, 0.03)
    g = torch.Generator().manual_seed(5)
    pos = torch.randint(0, 2048, (T,), generator=g, dtype=torch.int64)
    cache = O.cos_sin_cache(hd, hd, 2048, 10000.0, dtype)
    split_head = neox and tile_n % 1000 == 64 and hd > 64
    if tile_n // 100000 > (K + 63) // 64 or (tile_n and (tile_n % 1000) % hd and not split_head):
        pytest.skip("tile configuration does not fit this case")
    _skip_unless_planned(1, T, (nq + 2 * nkv) * hd, K, tile_n, hd)
    out = dense_ops.linear_rotary(x.cuda(), w.cuda(), pos.cuda(), cache.cuda(), hd, (nq + nkv) * hd, neox,
                                  tile_n=tile_n)
    _check_status()
    # oracle: GEMM rounded to the dtype (GPU fp32 matmul of the same operands), then the rotary restatement
    ref = (x.float().cuda() @ w.float().cuda().t()).to(dtype).cpu()
    q, k, _ = ref.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    O.rotary_embedding(pos, q, k, hd, cache, neox)
    assert rel_err(out, ref) <= GEMM_TOL[dtype]
    # v columns are a plain GEMM
    assert rel_err(out[:, (nq + nkv) * hd:], ref[:, (nq + nkv) * hd:]) <= GEMM_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tile_n", [0, 64, 128, 192, 256, 2128, 2256, 501256, 402128, 3064, 3128, 3256, 403256, 4128, 4256, 304256,
                                    205256, 405128, 205064])
@pytest.mark.parametrize("T,d,K", [(512, 1792, 4096), (288, 1408, 1024), (65, 96, 512), (1, 64, 64)])
def test_linear_silu_mul(dtype, tile_n, T, d, K):
    from sarathi_serve_b200 import dense_ops
    if tile_n // 100000 > (K + 63) // 64:
        pytest.skip("more splits than k-blocks")
    _skip_unless_planned(2, T, 2 * d, K, tile_n)
    x, w = _rand((T, K), dtype, T + K), _rand((2 * d, K), dtype, d, 0.05)
    out = dense_ops.linear_silu_mul(x.cuda(), w.cuda(), tile_n=tile_n)
    _check_status()
    gate_up = (x.float().cuda() @ w.float().cuda().t()).to(dtype).cpu()
    ref = O.silu_and_mul(gate_up)
    assert out.shape == (T, d)
    assert rel_err(out, ref) <= 2e-2


def test_gemm_linearity_full_size():
    """Size-independent property at the headline shapes: (a*x) W^T == a * (x W^T) for a power of two."""
    from sarathi_serve_b200 import dense_ops
    x = _rand((512, 4096), torch.bfloat16, 1).cuda()
    w = _rand((3584 * 2, 4096), torch.bfloat16, 2, 0.02).cuda()
    y1 = dense_ops.linear(x, w)
    y2 = dense_ops.linear(x * 4, w)
    _check_status()
    assert torch.equal(y1 * 4, y2)


def test_mma_rate_diagnostic_runs_and_orders_the_two_modes():
    """The planner's two constants, re-measured: a CTA pair completes a 256-row MMA of N = 128 in fewer clocks than
    one CTA needs for its 128-row MMA, and N = 256 on a pair takes about twice as long as N = 128."""
    from sarathi_serve_b200 import mma_rate
    one = mma_rate.measure(False, 128, iters=256)
    pair128 = mma_rate.measure(True, 128, iters=256)
    pair256 = mma_rate.measure(True, 256, iters=256)
    for r in (one, pair128, pair256):
        assert 8 < r["clk_per_mma_complete"] < 2000, r
    assert pair128["clk_per_mma_complete"] < one["clk_per_mma_complete"]
    assert 1.5 < pair256["clk_per_mma_complete"] / pair128["clk_per_mma_complete"] < 2.5
