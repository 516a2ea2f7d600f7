"""GPU parity of the mixture-of-experts path (routing -> block alignment -> gather -> two grouped
tcgen05 GEMMs -> sum over the k slots) against the CPU oracle, through the package's
reference-shaped API (fused_topk / fused_experts / fused_moe / FusedMoE / MixtralMoE)."""
import pytest
import torch

from helpers import rel_err
from oracle import tp_layer_oracle as O
from sarathi_serve_b200 import synthetic as S

pytestmark = pytest.mark.gpu


def _check_status():
    from sarathi_serve_b200 import dense_ops
    dense_ops.check_status(torch.device("cuda", torch.cuda.current_device()))


@pytest.mark.parametrize("case_name,world", [("mini_moe", 1), ("mini_moe", 2), ("config5", 8)])
def test_fused_experts_and_routing(case_name, world):
    """One rank's shard of the experts (TP-sharded along the intermediate dimension)."""
    from sarathi_serve_b200 import fused_moe as FM
    case = S.MOE_CASES[case_name]
    d = S.generate_moe(case, world=world, rank=0)
    x, w13, w2, logits = d["x"], d["w13"], d["w2"], d["logits"]
    # routing: ids bit-exact against the oracle
    wts, ids = FM.fused_topk(x.cuda(), logits.cuda(), case.top_k, True)
    ow, oids, _ = O.topk_softmax(logits, case.top_k, renormalize=True)
    assert torch.equal(ids.cpu(), oids)
    assert torch.allclose(wts.cpu(), ow, rtol=1e-5, atol=1e-7)
    # block alignment with the GEMM's block: bit-exact
    s_ids, e_ids, npp = FM.moe_align_block_size(ids, FM.block_rows(), case.num_experts)
    os_, oe, on = O.moe_align_block_size(oids.long(), FM.block_rows(), case.num_experts)
    n = int(on)
    assert int(npp) == n and torch.equal(s_ids.cpu(), os_) and torch.equal(e_ids[:n // FM.block_rows()].cpu(), oe[:n // FM.block_rows()])
    # experts
    out = FM.fused_experts(x.cuda(), w13.cuda(), w2.cuda(), wts, ids, inplace=False)
    _check_status()
    ref = O.fused_experts(x, w13, w2, ow, oids.long())
    assert rel_err(out, ref) <= 2e-2
    # in place + the one-call form
    xin = x.cuda().clone()
    out2 = FM.fused_moe(xin, w13.cuda(), w2.cuda(), logits.cuda(), case.top_k, renormalize=True, inplace=True)
    assert out2 is xin and torch.equal(out2, out)


@pytest.mark.parametrize("T", [1, 7, 129, 300])
def test_fused_experts_token_counts(T):
    """Ragged token counts, an expert that receives nothing, fp16."""
    from sarathi_serve_b200 import fused_moe as FM
    g = torch.Generator().manual_seed(T)
    H, I, E, k = 256, 384, 8, 2
    x = torch.randn(T, H, generator=g).to(torch.float16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.float16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.float16)
    logits = torch.randn(T, E, generator=g)
    logits[:, 3] = -30.0  # expert 3 is never chosen
    wts, ids = FM.fused_topk(x.cuda(), logits.cuda(), k, True)
    assert not bool((ids == 3).any())
    out = FM.fused_experts(x.cuda(), w13.cuda(), w2.cuda(), wts, ids)
    _check_status()
    ow, oids, _ = O.topk_softmax(logits, k, renormalize=True)
    assert rel_err(out, O.fused_experts(x, w13, w2, ow, oids.long())) <= 2e-2


@pytest.mark.parametrize("T", [1, 129, 300, 1024])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_expert_gemms_on_cta_pair_tiles_equal_single_cta_tiles(T, dtype):
    """The grouped GEMMs on CTA-pair tiles (256-row expert blocks) against the single-CTA tiles (128-row blocks) and
    the oracle: the alignment differs, the per-slot results must not."""
    from sarathi_serve_b200 import fused_moe as FM
    g = torch.Generator().manual_seed(T + 1)
    H, I, E, k = 256, 384, 8, 2
    x = torch.randn(T, H, generator=g).to(dtype).cuda()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(dtype).cuda()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(dtype).cuda()
    logits = torch.randn(T, E, generator=g)
    logits[:, 5] = -30.0
    wts, ids = FM.fused_topk(x, logits.cuda(), k, True)
    single = FM._expert_slots(x, w13, w2, wts, ids, True, pairs=False)
    pair = FM._expert_slots(x, w13, w2, wts, ids, True, pairs=True)
    _check_status()
    assert torch.equal(pair, single)
    ow, oids, _ = O.topk_softmax(logits, k, renormalize=True)
    ref = O.fused_experts(x.cpu(), w13.cpu(), w2.cpu(), ow, oids.long())
    assert rel_err(pair.view(T, k, H).float().sum(1), ref.float()) <= 2e-2
    assert FM.use_pair_tiles(2048, 8) and not FM.use_pair_tiles(154, 8)


def test_mixtral_moe_block_tp1():
    """MixtralMoE module (gate + FusedMoE) at tensor-parallel size 1 against the oracle's MoE layer."""
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.decoder_layer import MixtralMoE
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    try:
        case = S.MOE_CASES["mini_moe"]
        d = S.generate_moe(case)
        g = torch.Generator().manual_seed(5)
        gate_w = (torch.randn(case.num_experts, case.hidden_size, generator=g) * 0.05).to(case.dtype)
        old = torch.get_default_dtype()
        torch.set_default_dtype(case.dtype)
        try:
            moe = MixtralMoE(case.num_experts, case.top_k, case.hidden_size, case.intermediate_size)
        finally:
            torch.set_default_dtype(old)
        sd = moe.state_dict()
        assert set(sd) == {"gate.weight", "experts.w13_weight", "experts.w2_weight"}
        with torch.no_grad():
            sd["gate.weight"].copy_(gate_w)
            sd["experts.w13_weight"].copy_(d["w13"])
            sd["experts.w2_weight"].copy_(d["w2"])
        x = d["x"].cuda()
        out = moe(x.clone())
        _check_status()
        ref = O.moe_layer(d["x"], gate_w, [d["w13"]], [d["w2"]], case.top_k)
        assert rel_err(out, ref) <= 2e-2
    finally:
        ps.destroy_model_parallel()


def test_fused_experts_against_the_reference_fixture_fp16():
    """The committed output of the reference's own fused_experts (its Triton kernel, fp16,
    tests/golden/fused_experts_f16.npz) -- ragged sizes: H=96, per-expert intermediate 80."""
    import os
    import numpy as np
    from sarathi_serve_b200 import fused_moe as FM
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "fused_experts_f16.npz"))
    h = lambda name: torch.from_numpy(g[name]).view(torch.float16)
    out = FM.fused_experts(h("x").cuda(), h("w1").cuda(), h("w2").cuda(), torch.from_numpy(g["topk_weights"]).cuda(),
                           torch.from_numpy(g["topk_ids"]).cuda(), inplace=False)
    _check_status()
    assert rel_err(out, h("out")) <= 2e-3


def test_mixtral_decoder_layer_tp1_against_oracle_and_reference_fixture():
    """MixtralDecoderLayer (attention block with the fused o_proj tail + MoE block), fp16, one rank: against the
    oracle's layer and against the output of the reference's own layer (tests/golden/mixtral_layer_f16_tp2.npz,
    made over two ranks -- the layer output does not depend on the tensor-parallel size beyond rounding)."""
    import os
    import sys
    import numpy as np
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from make_golden import mixtral_case
    from test_oracle_golden import _mixtral_oracle
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.decoder_layer import MixtralDecoderLayer

    class Q:
        def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
            return q

    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    try:
        cfg, full, shard = mixtral_case(1, 0)
        old = torch.get_default_dtype()
        torch.set_default_dtype(torch.float16)
        try:
            layer = MixtralDecoderLayer(cfg, layer_id=0)
        finally:
            torch.set_default_dtype(old)
        sd = layer.state_dict()
        with torch.no_grad():
            for name, value in shard.items():
                sd[name].copy_(value)
        with torch.inference_mode():
            out = layer(full["positions"].cuda(), full["x"].cuda(), 0, Q())
        _check_status()
        ps.get_tensor_model_parallel_comm().check_status()
        _, _, ref = _mixtral_oracle(1)
        assert rel_err(out, ref) <= 5e-3
        g = np.load(os.path.join(os.path.dirname(__file__), "golden", "mixtral_layer_f16_tp2.npz"))
        assert rel_err(out, torch.from_numpy(g["out"]).view(torch.float16)) <= 5e-3
    finally:
        ps.destroy_model_parallel()
