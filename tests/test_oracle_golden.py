"""The CPU oracle against fixtures produced by the reference's own Python layer
code (tests/golden/make_golden.py).  Pins oracle/tp_layer_oracle.decoder_layer."""
import pytest
import torch

from helpers import TOL, load_golden, rel_err
from oracle import tp_layer_oracle as O
from sarathi_serve_b200 import synthetic as S

RUNS = [("mini_f32", 1), ("mini_f32", 2), ("mini_bf16", 1), ("mini_bf16", 2), ("mini_f16", 1), ("mini_f16", 2),
        ("config1", 2)]
NAMES = ["input_norm", "qkv_pre_rotary", "o_proj", "post_attn_norm", "gate_up", "act", "down_proj", "out"]


def run_oracle(case_name, world):
    case = S.CASES[case_name]
    t = S.generate(case)
    params = [S.shard(t, r, world) for r in range(world)]
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    out = O.decoder_layer(params, t.x.to(case.dtype), t.positions, num_heads=case.num_heads,
                          num_kv_heads=case.num_kv_heads, head_dim=case.head_dim, eps=case.rms_norm_eps, cache=cache)
    return case, out, cache


@pytest.mark.parametrize("case_name,world", RUNS)
def test_oracle_matches_reference_layer(case_name, world):
    gold, sums, step, dtype = load_golden(case_name, world)
    case, out, cache = run_oracle(case_name, world)
    nq = case.num_heads // world * case.head_dim
    nkv = case.num_kv_heads // world * case.head_dim
    out["q_rot"], out["k_rot"], out["v"] = out["qkv"].split([nq, nkv, nkv], dim=-1)
    # The oracle repeats the reference's op sequence with the same CPU kernels: the only
    # freedom is the GEMM blocking of differently shaped calls, so allow a few ulps.
    tol = {torch.float32: 2e-6, torch.bfloat16: 1e-2, torch.float16: 2e-3}[dtype]
    for name in NAMES + ["q_rot", "k_rot", "v"]:
        got = out[name]
        assert rel_err(got[::step], gold[name]) <= tol, name
        s = got.double()
        ref = sums[name]
        assert abs(s.sum().item() - ref[0]) <= 1e-3 * max(1.0, ref[1]) * (tol * 50), name
        assert abs(s.pow(2).sum().item() - ref[2]) <= ref[2] * tol * 50 + 1e-9, name


@pytest.mark.parametrize("case_name", ["mini_f32", "mini_bf16", "mini_f16", "config1"])
def test_cos_sin_cache_matches_reference(case_name):
    world = 2 if case_name == "config1" else 1
    gold, _, _, dtype = load_golden(case_name, world)
    case = S.CASES[case_name]
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    got = torch.cat([cache[:24], cache[-8:]])
    assert torch.equal(got.view(torch.int16) if got.element_size() == 2 else got,
                       gold["cos_sin_cache"].view(torch.int16) if got.element_size() == 2 else gold["cos_sin_cache"])


def test_tp_invariance():
    """TP=1 and TP=2 of the oracle agree (fp32: summation order only)."""
    _, o1, _ = run_oracle("mini_f32", 1)
    _, o2, _ = run_oracle("mini_f32", 2)
    assert rel_err(o2["out"], o1["out"]) < 1e-5


def test_vocab_parallel_embedding_matches_the_reference_module():
    """Fixture made by the reference's own VocabParallelEmbedding over two gloo ranks
    (tests/golden/make_golden.py): the oracle's masked lookups + sum reproduce it bit for bit."""
    import os
    import numpy as np
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "vocab_embedding_tp2.npz"))
    table = torch.from_numpy(g["table"]).view(torch.bfloat16)
    out = torch.from_numpy(g["out"]).view(torch.bfloat16)
    ids = torch.from_numpy(g["ids"])
    world = int(g["world"][0])
    got = O.vocab_parallel_embedding(ids, list(table.chunk(world, dim=0)))
    assert torch.equal(got, out)
    assert torch.equal(out, table[ids])  # the sharded lookup is the full-table lookup


def test_fused_experts_matches_the_reference_triton_kernel():
    """Fixture made by the reference's own fused_experts with its Triton grouped-GEMM kernel executed by the
    Triton interpreter on the CPU (fp16; tests/golden/make_golden.py).  The oracle's restatement -- GEMM1 with
    fp32 accumulation -> T, SiLU*mul -> T, GEMM2 * routed weight -> T, sum over the k slots -> T -- agrees bit
    for bit except where the order of the fp32 additions along K (the kernel adds 32-wide blocks) moves a value
    across a rounding boundary: under 2 % of the elements, by one unit in the last place.  (A restatement with
    different rounding points, e.g. none between the stages, differs in about 65 % of the elements.)"""
    import os
    import numpy as np
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "fused_experts_f16.npz"))
    h = lambda name: torch.from_numpy(g[name]).view(torch.float16)
    got = O.fused_experts(h("x"), h("w1"), h("w2"), torch.from_numpy(g["topk_weights"]),
                          torch.from_numpy(g["topk_ids"]).long())
    ref = h("out")
    assert float((got != ref).float().mean()) <= 0.02
    assert rel_err(got, ref) <= 5e-4


def test_moe_block_matches_the_reference_mixtral_moe_over_two_ranks():
    """Fixture made by the reference's own MixtralMoE (replicated gate, fused_topk with renormalisation, FusedMoE
    with its Triton kernel in the Triton interpreter, gloo SUM all-reduce over two ranks; fp16).  The oracle's
    moe_layer agrees bit for bit except for one-ulp differences in well under 2 % of the elements (order of the
    fp32 additions along K inside the kernel)."""
    import os
    import numpy as np
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_block_f16_tp2.npz"))
    h = lambda name: torch.from_numpy(g[name]).view(torch.float16)
    world, k = int(g["world"][0]), int(g["top_k"][0])
    wg, wu, wd = h("w_gate"), h("w_up"), h("w_down")
    ish = wg.shape[1] // world
    w13 = [torch.cat([wg[:, r * ish:(r + 1) * ish], wu[:, r * ish:(r + 1) * ish]], dim=1).contiguous()
           for r in range(world)]
    w2 = [wd[:, :, r * ish:(r + 1) * ish].contiguous() for r in range(world)]
    got = O.moe_layer(h("x"), h("gate_w"), w13, w2, k)
    ref = h("out")
    assert float((got != ref).float().mean()) <= 0.02
    assert rel_err(got, ref) <= 5e-4


def test_rope_variant_tables_match_the_reference():
    """cos|sin tables of the reference's RotaryEmbedding, LinearScaling, DynamicNTKScaling and YaRN variants
    (layers/rotary_embedding.py:33-345; fixture rows from tests/golden/make_golden.py): this package's get_rope
    builds the same tables bit for bit (fp32)."""
    import os
    import sys
    import numpy as np
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from make_golden import ROPE_VARIANTS
    from sarathi_serve_b200.nn_layers import get_rope
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_variants.npz"))
    for name, (hs, rot, max_pos, base, scaling) in ROPE_VARIANTS.items():
        ours = get_rope(hs, rot, max_pos, base, True, scaling).cos_sin_cache.float().cpu()
        assert tuple(ours.shape) == tuple(g[name + "__shape"]), name
        assert torch.equal(ours[torch.from_numpy(g[name + "__rows"])], torch.from_numpy(g[name])), name


def _mixtral_oracle(world):
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from make_golden import mixtral_case
    cfg, full, _ = mixtral_case(1, 0)
    shards = [mixtral_case(world, r)[2] for r in range(world)]
    hd = cfg.hidden_size // cfg.num_attention_heads
    cache = O.cos_sin_cache(hd, hd, cfg.max_position_embeddings, cfg.rope_theta, torch.float16)
    out = O.mixtral_decoder_layer(shards, full["gate"], [s["block_sparse_moe.experts.w13_weight"] for s in shards],
                                  [s["block_sparse_moe.experts.w2_weight"] for s in shards], full["x"], full["positions"],
                                  num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads, head_dim=hd,
                                  eps=cfg.rms_norm_eps, cache=cache, top_k=cfg.num_experts_per_tok)
    return cfg, full, out


def test_mixtral_decoder_layer_matches_the_reference_over_two_ranks():
    """Fixture made by the reference's own MixtralDecoderLayer over two gloo ranks (fp16, Triton interpreter for its
    grouped GEMM; attention stand-in attn_out = q): the oracle's mixtral_decoder_layer agrees up to one-ulp
    differences in a small fraction of the elements."""
    import os
    import numpy as np
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "mixtral_layer_f16_tp2.npz"))
    ref = torch.from_numpy(g["out"]).view(torch.float16)
    _, _, got = _mixtral_oracle(int(g["world"][0]))
    assert float((got != ref).float().mean()) <= 0.03
    assert rel_err(got, ref) <= 1e-3


def test_model_stack_chain_matches_the_reference_llama_model():
    """Fixture made by the reference's own LlamaModel (VocabParallelEmbedding, two decoder layers, final RMSNorm)
    over two gloo ranks: the oracle's chain embedding -> decoder_layer x 2 -> rms_norm reproduces it (bf16; the
    same chain is what the GPU model-stack test compares the fused stack with)."""
    import dataclasses
    import os
    import sys
    import numpy as np
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    from make_golden import model_stack_inputs
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "llama_model_mini_bf16_tp2.npz"))
    world = int(g["world"][0])
    case = S.CASES["mini_bf16"]
    t = S.generate(case)
    table, final_w, _head, ids = model_stack_inputs(case)
    h = O.vocab_parallel_embedding(ids, list(table.chunk(world, dim=0)))
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    for _ in range(2):
        tt = dataclasses.replace(t, x=h.float())
        h = O.decoder_layer([S.shard(tt, r, world) for r in range(world)], h, t.positions, num_heads=case.num_heads,
                            num_kv_heads=case.num_kv_heads, head_dim=case.head_dim, eps=case.rms_norm_eps,
                            cache=cache)["out"]
    got = O.rms_norm(h, final_w, case.rms_norm_eps)
    ref = torch.from_numpy(g["out"]).view(torch.bfloat16)
    assert torch.equal(got, ref)
