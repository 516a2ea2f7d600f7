"""GPU parity of the decoder layer built from this package's modules (tensor
parallel size 1: one GPU, the row-parallel kernel runs its reduce / residual /
norm phases locally) against the CPU oracle and the reference fixtures."""
import dataclasses

import pytest
import torch

from helpers import TOL, load_golden, rel_err
from oracle import tp_layer_oracle as O
from sarathi_serve_b200 import synthetic as S

pytestmark = pytest.mark.gpu


class QAttention:
    """Attention stand-in shared with the oracle and the fixtures: attn_out = q (after rotary)."""

    def __init__(self):
        self.seen = {}

    def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
        self.seen = {"q_rot": q.clone(), "k_rot": k.clone(), "v": v.clone()}
        return q  # a strided view: the o_proj GEMM reads it in place


@pytest.fixture(scope="module")
def tp1():
    from sarathi_serve_b200 import parallel_state as ps
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    yield ps
    ps.destroy_model_parallel()


def build_layer(case, rank=0, world=1):
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer
    old = torch.get_default_dtype()
    torch.set_default_dtype(case.dtype)
    try:
        layer = LlamaDecoderLayer(case.hf_config(), layer_id=0)
    finally:
        torch.set_default_dtype(old)
    t = S.generate(case)
    S.load_layer(layer, S.shard(t, rank, world))
    return layer, t


def oracle_out(case, t, next_norm=None):
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    return O.decoder_layer([S.shard(t, 0, 1)], t.x.to(case.dtype), t.positions, num_heads=case.num_heads,
                           num_kv_heads=case.num_kv_heads, head_dim=case.head_dim, eps=case.rms_norm_eps,
                           cache=cache, next_norm_weight=next_norm)


@pytest.mark.parametrize("case_name", ["mini_f32", "mini_bf16", "mini_f16", "config1"])
@pytest.mark.parametrize("path", ["fused", "unfused"])
def test_layer_matches_oracle_and_fixture(tp1, case_name, path):
    case = S.CASES[case_name]
    layer, t = build_layer(case)
    attn = QAttention()
    x = t.x.to(case.dtype).cuda()
    pos = t.positions.cuda()
    with torch.inference_mode():
        fn = layer.forward if path == "fused" else layer.forward_unfused
        out = fn(pos, x.clone(), 0, attn)
    tp1.get_tensor_model_parallel_comm().check_status()
    ref = oracle_out(case, t)
    tol = TOL[case.dtype]
    assert rel_err(out, ref["out"]) <= tol
    nq = case.num_heads * case.head_dim
    assert rel_err(attn.seen["q_rot"], ref["qkv"][:, :nq]) <= tol
    assert rel_err(attn.seen["k_rot"], ref["qkv"][:, nq:nq + case.num_kv_heads * case.head_dim]) <= tol
    world = 2 if case_name == "config1" else 1
    gold, _, step, _ = load_golden(case_name, world)
    assert rel_err(out[::step], gold["out"]) <= tol  # the reference's own layer output (TP-invariant)


def test_layer_carry_path(tp1):
    """(normed, residual) -> (normed', residual') equals the oracle's layer followed by the next norm."""
    from sarathi_serve_b200.nn_layers import RMSNorm
    case = S.CASES["mini_bf16"]
    layer, t = build_layer(case)
    x = t.x.to(case.dtype).cuda()
    next_norm = RMSNorm(case.hidden_size, eps=case.rms_norm_eps)
    next_norm.weight.data = t.ln2.to(case.dtype).cuda()
    with torch.inference_mode():
        normed = layer.input_layernorm(x)
        y, z = layer.forward_carry(t.positions.cuda(), normed, x, 0, QAttention(), next_norm)
    tp1.get_tensor_model_parallel_comm().check_status()
    ref = oracle_out(case, t, next_norm=t.ln2.to(case.dtype))
    assert rel_err(z, ref["out"]) <= TOL[case.dtype]
    assert rel_err(y, ref["out_normed"]) <= TOL[case.dtype]


def test_layer_config2_full_size(tp1):
    """Headline shapes (Llama-3-8B layer, 512-token mixed chunk), TP=1, against the CPU oracle."""
    case = S.CASES["config2"]
    layer, t = build_layer(case)
    with torch.inference_mode():
        out = layer(t.positions.cuda(), t.x.to(case.dtype).cuda(), 0, QAttention())
    tp1.get_tensor_model_parallel_comm().check_status()
    ref = oracle_out(case, t)
    assert rel_err(out, ref["out"]) <= TOL[case.dtype]


def test_layer_graph_replay_equals_eager(tp1):
    """A layer captured in a CUDA graph (graph_runner.LayerGraph) and fed from pinned host buffers returns
    exactly what the eager call returns, for two different inputs in a row."""
    from sarathi_serve_b200.graph_runner import LayerGraph

    class Q:
        def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
            return q

    case = S.CASES["mini_bf16"]
    layer, t = build_layer(case)
    runner = LayerGraph(layer, case.num_tokens, Q())
    pos_host = t.positions.pin_memory()
    for scale in (1.0, -0.5):
        x_host = (t.x * scale).to(case.dtype).pin_memory()
        out = runner(pos_host, x_host).clone()
        with torch.inference_mode():
            eager = layer(t.positions.cuda(), x_host.cuda(), 0, Q())
        assert torch.equal(out, eager)
    with pytest.raises(RuntimeError, match="captured for"):
        runner(pos_host[:3], x_host[:3])
    # host buffers owned by the graph: the copies are graph nodes, a step is one launch
    io = LayerGraph(layer, case.num_tokens, Q(), host_io=True)
    io.host_positions.copy_(t.positions)
    for scale in (1.0, 0.25):
        io.host_hidden_states.copy_((t.x * scale).to(case.dtype))
        out = io.replay_host_io()
        torch.cuda.synchronize()
        with torch.inference_mode():
            eager = layer(t.positions.cuda(), (t.x * scale).to(case.dtype).cuda(), 0, Q())
        assert torch.equal(out, eager.cpu())
    tp1.get_tensor_model_parallel_comm().check_status()


def test_host_pipeline_returns_every_steps_result_in_order(tp1):
    """graph_runner.HostPipeline (uploads and downloads on copy streams under the neighbouring steps' kernels):
    with three steps in flight every collected result equals the eager layer on that step's input."""
    from sarathi_serve_b200.graph_runner import HostPipeline, LayerGraph

    class Q:
        def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
            return q

    case = S.CASES["mini_bf16"]
    layer, t = build_layer(case)
    slots = [LayerGraph(layer, case.num_tokens, Q(), host_io=True, copies_in_graph=False) for _ in range(3)]
    with pytest.raises(RuntimeError, match="copies_in_graph"):
        HostPipeline([LayerGraph(layer, case.num_tokens, Q(), host_io=True)] * 2)
    pipe = HostPipeline(slots)
    scales = [1.0, -0.5, 0.25, 2.0, -1.5, 0.75, 1.25]
    with torch.inference_mode():
        eager = [layer(t.positions.cuda(), (t.x * sc).to(case.dtype).cuda(), 0, Q()).cpu() for sc in scales]
    got = []
    for sc in scales:
        g = pipe.next_slot()
        g.host_positions.copy_(t.positions)
        g.host_hidden_states.copy_((t.x * sc).to(case.dtype))
        pipe.submit()
        if pipe.in_flight >= 3:
            got.append(pipe.collect().clone())
    while pipe.in_flight:
        got.append(pipe.collect().clone())
    assert len(got) == len(scales)
    for i, (a, b) in enumerate(zip(got, eager)):
        assert torch.equal(a, b), i
    with pytest.raises(RuntimeError, match="nothing in flight"):
        pipe.collect()
    # the serial call of such a graph (copies enqueued around the replay) gives the same
    slots[0].host_hidden_states.copy_((t.x * scales[1]).to(case.dtype))
    out = slots[0].replay_host_io()
    torch.cuda.synchronize()
    assert torch.equal(out, eager[1])
    tp1.get_tensor_model_parallel_comm().check_status()


def test_model_stack_embedding_layers_norm_logits(tp1):
    """Token ids -> VocabParallelEmbedding -> two decoder layers chained through forward_carry -> final norm
    (applied by the last layer's kernel) -> lm_head logits, against the oracle's op-by-op chain."""
    from sarathi_serve_b200.decoder_layer import LlamaForCausalLM

    class Q:
        def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
            return q

    case = S.CASES["mini_bf16"]
    cfg = case.hf_config()
    cfg.num_hidden_layers, cfg.vocab_size = 2, 1000
    old = torch.get_default_dtype()
    torch.set_default_dtype(case.dtype)
    try:
        lm = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    t = S.generate(case)
    for layer in lm.model.layers:
        S.load_layer(layer, S.shard(t, 0, 1))
    g = torch.Generator().manual_seed(21)
    table = torch.randn(1024, case.hidden_size, generator=g).to(case.dtype)
    final_w = (1 + 0.1 * torch.randn(case.hidden_size, generator=g)).to(case.dtype)
    head = (torch.randn(1024, case.hidden_size, generator=g) * 0.05).to(case.dtype)
    lm.model.embed_tokens.weight.data.copy_(table)
    lm.model.norm.weight.data.copy_(final_w)
    lm.lm_head.weight.data.copy_(head)
    ids = torch.randint(0, 1000, (case.num_tokens,), generator=g)
    with torch.inference_mode():
        hidden = lm(ids.cuda(), t.positions.cuda(), Q())
        logits = lm.compute_logits(hidden)
    tp1.get_tensor_model_parallel_comm().check_status()
    h = table[ids]
    for _ in range(2):
        h = oracle_out(case, dataclasses.replace(t, x=h.float()))["out"]
    ref_hidden = O.rms_norm(h, final_w, case.rms_norm_eps)
    assert hidden.shape == (case.num_tokens, case.hidden_size)
    assert rel_err(hidden, ref_hidden) <= TOL[case.dtype] * 1.5
    assert logits.shape == (case.num_tokens, 1000)
    assert rel_err(logits, O.linear(ref_hidden, head)[:, :1000]) <= TOL[case.dtype] * 1.5


def test_model_graph_runner_whole_stack_per_batch_size_bucket(tp1):
    """prepare_inputs lays a mixed batch out as the reference does (prefill chunks, then decodes, zero padding to
    a multiple of 8); ModelGraphRunner captures the whole stack (embedding, two layers, final norm) once per
    padded size and its replays equal the eager model on the same padded batch."""
    from sarathi_serve_b200.decoder_layer import LlamaModel
    from sarathi_serve_b200.model_runner import ModelGraphRunner, prepare_inputs

    class Q:
        def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
            return q

    case = S.CASES["mini_bf16"]
    cfg = case.hf_config()
    cfg.num_hidden_layers, cfg.vocab_size = 2, 1000
    old = torch.get_default_dtype()
    torch.set_default_dtype(case.dtype)
    try:
        model = LlamaModel(cfg)
    finally:
        torch.set_default_dtype(old)
    t = S.generate(case)
    for layer in model.layers:
        S.load_layer(layer, S.shard(t, 0, 1))
    g = torch.Generator().manual_seed(3)
    model.embed_tokens.weight.data.copy_(torch.randn(1024, case.hidden_size, generator=g).to(case.dtype))
    tok, pos, n = prepare_inputs([([5, 6, 7, 8, 9], 0), ([11, 12, 13], 40)], [(21, 100), (22, 7)], "cuda")
    assert n == 10 and tok.tolist() == [5, 6, 7, 8, 9, 11, 12, 13, 21, 22, 0, 0, 0, 0, 0, 0]
    assert pos.tolist() == [0, 1, 2, 3, 4, 40, 41, 42, 99, 6, 0, 0, 0, 0, 0, 0]
    runner = ModelGraphRunner(model, Q(), buckets=(16, 32, 64))
    assert runner.bucket_for(1) == 16 and runner.bucket_for(17) == 32
    for n_tok in (10, 16, 29, 64, 10):
        ids = torch.randint(0, 1000, (n_tok,), generator=g).cuda()
        p_ = torch.randint(0, 1000, (n_tok,), generator=g).cuda()
        out = runner.run(ids, p_).clone()
        size = runner.bucket_for(n_tok)
        ids_p = torch.zeros(size, dtype=torch.long, device="cuda"); ids_p[:n_tok] = ids
        pos_p = torch.zeros(size, dtype=torch.long, device="cuda"); pos_p[:n_tok] = p_
        with torch.inference_mode():
            eager = model(ids_p, pos_p, Q())[:n_tok]
        assert out.shape == (n_tok, case.hidden_size) and torch.equal(out, eager), n_tok
    assert sorted(runner._graphs) == [16, 32, 64]
    tp1.get_tensor_model_parallel_comm().check_status()
    with pytest.raises(RuntimeError, match="largest bucket"):
        runner.run(torch.zeros(65, dtype=torch.long, device="cuda"), torch.zeros(65, dtype=torch.long, device="cuda"))


@pytest.mark.parametrize("case_name", ["mini_bf16", "mini_f32"])
def test_layer_appends_to_the_paged_kv_cache_through_the_wrapper_hook(tp1, case_name):
    """An attention wrapper that offers fused_kv_append gets this step's rotated keys and values stored into its
    paged cache by the qkv GEMM's epilogue (bf16) or by the append kernel (fp32): the cache then holds exactly
    the k / v the wrapper's forward receives."""
    from sarathi_serve_b200 import kv_cache_ops
    case = S.CASES[case_name]
    layer, t = build_layer(case)
    T, page = case.num_tokens, 16
    nkv, hd = case.num_kv_heads, case.head_dim
    pages = -(-T // page) + 3
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    # one request whose tokens 0..T-1 are this step's tokens
    bi = torch.zeros(T, dtype=torch.int32, device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    ki, kp = perm[: -(-T // page)].cuda(), torch.tensor([0, -(-T // page)], dtype=torch.int32, device="cuda")

    class Wrapper(QAttention):
        def __init__(self):
            super().__init__()
            self.cache = torch.zeros(pages, 2, page, nkv, hd, dtype=case.dtype, device="cuda")
            self.slots = kv_cache_ops.slots(bi, pos, ki, kp, page)   # what begin_forward would compute

        def fused_kv_append(self, layer_cache_idx):
            return self.cache, self.slots

    w = Wrapper()
    with torch.inference_mode():
        layer(t.positions.cuda(), t.x.to(case.dtype).cuda(), 0, w)
    want = torch.zeros_like(w.cache)
    kv_cache_ops.append_rows(want, w.seen["k_rot"], w.seen["v"], w.slots)
    assert torch.equal(w.cache, want) and float(w.cache.abs().sum()) > 0
    ref = torch.zeros(pages, 2, page, nkv, hd, dtype=case.dtype)
    O.append_paged_kv_cache(w.seen["k_rot"].cpu(), w.seen["v"].cpu(), bi.cpu(), pos.cpu(), ref, ki.cpu(), kp.cpu())
    assert torch.equal(w.cache.cpu(), ref)
