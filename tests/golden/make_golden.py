"""Generate golden fixtures by running the REFERENCE's own Python modules on CPU/gloo.

    python tests/golden/make_golden.py [--reference <checkout of microsoft/sarathi-serve>]

The unmodified reference package is imported from its checkout (never copied).
What it needs to run without a GPU is shimmed here:
  * stub modules for plotting / sketch packages its metrics code imports;
  * its four CUDA extension modules (`sarathi.layernorm_ops`, `activation_ops`,
    `pos_encoding_ops`, `moe_ops`) are replaced by the CPU restatements in
    oracle/tp_layer_oracle.py (those restatements are pinned separately, on the
    GPU, against the reference's compiled kernels);
  * `torch.cuda.current_device` -> "cpu" and `device="cuda"` -> "cpu" in
    torch.arange, because the reference allocates on the current CUDA device;
  * a disabled MetricsStore, a plain-namespace model config, and an attention
    stand-in (attn_out = q after rotary; attention is outside the path).
Everything else -- ColumnParallelLinear, RowParallelLinear, the all-reduce in
mappings._reduce over a gloo group, RMSNorm, RotaryEmbedding (incl. its cos/sin
cache), SiluAndMul, LlamaAttention, LlamaMLP, LlamaDecoderLayer -- is the
reference's code.  Inputs come from sarathi_serve_b200.synthetic (seeded).

Outputs: tests/golden/<case>_tp<world>.npz with rank 0's intermediates (16-bit
tensors as raw int16 bit patterns).  Larger cases store a strided subset of rows
plus float64 checksums (sum, sum |.|, sum of squares) of the full tensors.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

RUNS = [("mini_f32", 1), ("mini_f32", 2), ("mini_bf16", 1), ("mini_bf16", 2), ("mini_f16", 1), ("mini_f16", 2),
        ("config1", 2)]
ROW_SUBSET = {"config1": 18, "mini_f16": 4}  # keep every n-th row of the larger cases


def _install_shims(reference: str) -> None:
    sys.path.insert(0, reference)
    from oracle import tp_layer_oracle as O

    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    stub("plotly"); stub("plotly.express"); stub("plotly_express")
    stub("ddsketch"); stub("ddsketch.ddsketch", DDSketch=object)

    def silu_and_mul(out, x): out.copy_(O.silu_and_mul(x))
    def gelu_new(out, x): out.copy_(O.gelu_new(x))
    def gelu_fast(out, x): out.copy_(O.gelu_fast(x))
    def rms_norm(out, x, w, eps): out.copy_(O.rms_norm(x, w, eps))
    def rotary_embedding(positions, q, k, head_size, cache, is_neox):
        O.rotary_embedding(positions, q, k, head_size, cache, is_neox)

    stub("sarathi.activation_ops", silu_and_mul=silu_and_mul, gelu_new=gelu_new, gelu_fast=gelu_fast)
    stub("sarathi.layernorm_ops", rms_norm=rms_norm)
    stub("sarathi.pos_encoding_ops", rotary_embedding=rotary_embedding)
    stub("sarathi.moe_ops")
    torch.cuda.current_device = lambda: "cpu"
    _arange = torch.arange

    def arange(*a, **k):
        if k.get("device") == "cuda":
            k["device"] = "cpu"
        return _arange(*a, **k)

    torch.arange = arange


def _worker(rank: int, world: int, case_name: str, port: int, reference: str, out_path: str) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _install_shims(reference)
    from sarathi_serve_b200 import synthetic as S
    from sarathi.config import MetricsConfig
    from sarathi.metrics.metrics_store import MetricsStore
    MetricsStore.get_or_create_instance(None, None, MetricsConfig(write_metrics=False))
    from sarathi.model_executor.parallel_utils import parallel_state as ps
    ps.initialize_model_parallel(world, 1)
    from sarathi.model_executor.attention.base_attention_wrapper import BaseAttentionWrapper
    from sarathi.model_executor.models.llama import LlamaDecoderLayer

    case = S.CASES[case_name]
    torch.set_default_dtype(case.dtype)
    layer = LlamaDecoderLayer(case.hf_config(), layer_id=0)
    tensors = S.generate(case)
    S.load_layer(layer, S.shard(tensors, rank, world))

    captured = {}

    def keep(name):
        def hook(_m, _inp, outp):
            t = outp[0] if isinstance(outp, tuple) else outp
            captured[name] = t.detach().clone()
        return hook

    layer.input_layernorm.register_forward_hook(keep("input_norm"))
    layer.self_attn.qkv_proj.register_forward_hook(keep("qkv_pre_rotary"))
    layer.self_attn.o_proj.register_forward_hook(keep("o_proj"))
    layer.post_attention_layernorm.register_forward_hook(keep("post_attn_norm"))
    layer.mlp.gate_up_proj.register_forward_hook(keep("gate_up"))
    layer.mlp.act_fn.register_forward_hook(keep("act"))
    layer.mlp.down_proj.register_forward_hook(keep("down_proj"))

    class Attn(BaseAttentionWrapper):
        def __init__(self): pass
        def init_gpu_cache(self, n): pass
        def get_cache_block(self, n, **k): pass
        def begin_forward(self, l): pass
        def end_forward(self): pass
        def forward(self, q, k, v, idx, softmax_scale=1.0, layer_id=None):
            captured["q_rot"] = q.detach().clone()
            captured["k_rot"] = k.detach().clone()
            captured["v"] = v.detach().clone()
            return q.contiguous()

    with torch.inference_mode():
        out = layer(tensors.positions, tensors.x.to(case.dtype).clone(), 0, Attn())
    captured["out"] = out.clone()
    captured["cos_sin_cache"] = layer.self_attn.rotary_emb.cos_sin_cache.clone()
    if rank == 0:
        step = ROW_SUBSET.get(case_name, 1)
        arrays = {}
        for name, t in captured.items():
            if name == "cos_sin_cache":
                t = torch.cat([t[:24], t[-8:]])  # a few table rows are enough to pin the cache builder
            else:
                tf = t.double()
                arrays[f"{name}__sum"] = np.array([tf.sum().item(), tf.abs().sum().item(), tf.pow(2).sum().item()])
                t = t[::step]
            # 16-bit dtypes are stored as their raw bit patterns (exact, half the size of fp32)
            arrays[name] = t.contiguous().view(torch.int16).numpy() if t.element_size() == 2 else t.numpy()
        arrays["__row_step"] = np.array([step])
        arrays["__dtype"] = np.array([str(case.dtype)])
        np.savez_compressed(out_path, **arrays)
        print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")
    dist.destroy_process_group()


def _worker_embedding(rank: int, world: int, port: int, reference: str, out_path: str) -> None:
    """The reference's VocabParallelEmbedding (tensor_parallel/layers.py:72-177) over gloo ranks."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _install_shims(reference)
    from sarathi.config import MetricsConfig
    from sarathi.metrics.metrics_store import MetricsStore
    MetricsStore.get_or_create_instance(None, None, MetricsConfig(write_metrics=False))
    from sarathi.model_executor.parallel_utils import parallel_state as ps
    ps.initialize_model_parallel(world, 1)
    from sarathi.model_executor.parallel_utils.tensor_parallel.layers import VocabParallelEmbedding
    V, H = 256, 48
    g = torch.Generator().manual_seed(17)
    table = torch.randn(V, H, generator=g).to(torch.bfloat16)
    ids = torch.cat([torch.tensor([0, V // world - 1, V // world, V - 1]), torch.randint(0, V, (60,), generator=g)])
    emb = VocabParallelEmbedding(V, H, params_dtype=torch.bfloat16)
    emb.weight.data.copy_(table[emb.vocab_start_index:emb.vocab_end_index])
    with torch.inference_mode():
        out = emb(ids)
    if rank == 0:
        np.savez_compressed(out_path, table=table.view(torch.int16).numpy(), ids=ids.numpy(),
                            out=out.contiguous().view(torch.int16).numpy(), world=np.array([world]))
        print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")
    dist.destroy_process_group()


def _worker_fused_experts(rank: int, reference: str, out_path: str) -> None:
    """The reference's fused_experts (layers/fused_moe/fused_moe.py:411-544) with its own Triton kernel
    (:15-148) executed by the Triton interpreter on CPU tensors.  fp16 only: the interpreter of the installed
    Triton mishandles bf16.  The CUDA ops it calls are shimmed with the oracle's restatements (they are pinned
    separately against the reference's compiled kernels)."""
    os.environ["TRITON_INTERPRET"] = "1"  # before triton is imported
    _install_shims(reference)
    from oracle import tp_layer_oracle as O
    import importlib

    def moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, experts, num_post_pad):
        s_, e_, n_ = O.moe_align_block_size(topk_ids, block_size, num_experts)
        sorted_ids.copy_(s_); experts.copy_(e_.clamp(min=0)); num_post_pad.copy_(n_)

    sys.modules["sarathi.moe_ops"].moe_align_block_size = moe_align_block_size
    torch.cuda.get_device_name = lambda *a, **k: "CPU"  # no tuned tile file: the reference's default tiles
    FM = importlib.import_module("sarathi.model_executor.layers.fused_moe.fused_moe")
    g = torch.Generator().manual_seed(23)
    T, E, H, I, k = 40, 4, 96, 80, 2
    x = torch.randn(T, H, generator=g).to(torch.float16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.1).to(torch.float16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.1).to(torch.float16)
    tw, ti, _ = O.topk_softmax(torch.randn(T, E, generator=g), k, True)
    out = FM.fused_experts(x, w1, w2, tw, ti.to(torch.int32), inplace=False)
    np.savez_compressed(out_path, x=x.view(torch.int16).numpy(), w1=w1.view(torch.int16).numpy(),
                        w2=w2.view(torch.int16).numpy(), topk_weights=tw.numpy(), topk_ids=ti.numpy().astype(np.int32),
                        out=out.view(torch.int16).numpy())
    print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")


def _worker_moe_block(rank: int, world: int, port: int, reference: str, out_path: str) -> None:
    """The reference's MixtralMoE block (models/mixtral.py:58-108: replicated gate, FusedMoE with the experts
    sharded along the intermediate dimension, SUM all-reduce) over gloo ranks, fp16, its Triton kernel run
    by the Triton interpreter."""
    os.environ["TRITON_INTERPRET"] = "1"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _install_shims(reference)
    from oracle import tp_layer_oracle as O

    def moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, experts, num_post_pad):
        s_, e_, n_ = O.moe_align_block_size(topk_ids, block_size, num_experts)
        sorted_ids.copy_(s_); experts.copy_(e_.clamp(min=0)); num_post_pad.copy_(n_)

    def topk_softmax(topk_weights, topk_ids, token_expert_indices, gating_output):
        w_, i_, _ = O.topk_softmax(gating_output, topk_weights.shape[1], False)
        topk_weights.copy_(w_); topk_ids.copy_(i_)

    sys.modules["sarathi.moe_ops"].moe_align_block_size = moe_align_block_size
    sys.modules["sarathi.moe_ops"].topk_softmax = topk_softmax
    torch.cuda.get_device_name = lambda *a, **k: "CPU"
    from sarathi.config import MetricsConfig
    from sarathi.metrics.metrics_store import MetricsStore
    MetricsStore.get_or_create_instance(None, None, MetricsConfig(write_metrics=False))
    from sarathi.model_executor.parallel_utils import parallel_state as ps
    ps.initialize_model_parallel(world, 1)
    from sarathi.model_executor.models.mixtral import MixtralMoE
    g = torch.Generator().manual_seed(29)
    T, E, H, I, k = 40, 4, 96, 160, 2
    x = torch.randn(T, H, generator=g).to(torch.float16)
    gate_w = (torch.randn(E, H, generator=g) * 0.3).to(torch.float16)
    w_gate = (torch.randn(E, I, H, generator=g) * 0.1).to(torch.float16)
    w_up = (torch.randn(E, I, H, generator=g) * 0.1).to(torch.float16)
    w_down = (torch.randn(E, H, I, generator=g) * 0.1).to(torch.float16)
    moe = MixtralMoE(E, k, H, I, params_dtype=torch.float16)
    Ish = I // world
    sl = slice(rank * Ish, (rank + 1) * Ish)
    with torch.no_grad():
        moe.gate.weight.copy_(gate_w)
        moe.experts.w13_weight.copy_(torch.cat([w_gate[:, sl], w_up[:, sl]], dim=1))
        moe.experts.w2_weight.copy_(w_down[:, :, sl])
    with torch.inference_mode():
        out = moe(x.clone())
    if rank == 0:
        i16 = lambda t: t.contiguous().view(torch.int16).numpy()
        np.savez_compressed(out_path, x=i16(x), gate_w=i16(gate_w), w_gate=i16(w_gate), w_up=i16(w_up), w_down=i16(w_down),
                            out=i16(out), world=np.array([world]), top_k=np.array([k]))
        print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")
    dist.destroy_process_group()


def model_stack_inputs(case):
    """Seeded extra tensors of the two-layer model stack used by the fixture and the tests: embedding table
    (vocabulary 1000 padded to 1024), final norm weight, lm_head, token ids."""
    g = torch.Generator().manual_seed(21)
    f32 = dict(generator=g, dtype=torch.float32)  # independent of the default dtype in force
    table = torch.randn(1024, case.hidden_size, **f32).to(case.dtype)
    final_w = (1 + 0.1 * torch.randn(case.hidden_size, **f32)).to(case.dtype)
    head = (torch.randn(1024, case.hidden_size, **f32) * 0.05).to(case.dtype)
    ids = torch.randint(0, 1000, (case.num_tokens,), generator=g)
    return table, final_w, head, ids


def _worker_model_stack(rank: int, world: int, port: int, reference: str, out_path: str) -> None:
    """The reference's LlamaModel (models/llama.py:258-314: VocabParallelEmbedding, two LlamaDecoderLayers, final
    RMSNorm) over gloo ranks, mini_bf16 shapes."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _install_shims(reference)
    from sarathi_serve_b200 import synthetic as S
    from sarathi.config import MetricsConfig
    from sarathi.metrics.metrics_store import MetricsStore
    MetricsStore.get_or_create_instance(None, None, MetricsConfig(write_metrics=False))
    from sarathi.model_executor.parallel_utils import parallel_state as ps
    ps.initialize_model_parallel(world, 1)
    from sarathi.model_executor.attention.base_attention_wrapper import BaseAttentionWrapper
    from sarathi.model_executor.models.llama import LlamaModel
    case = S.CASES["mini_bf16"]
    cfg = case.hf_config()
    cfg.num_hidden_layers, cfg.vocab_size, cfg.pad_token_id = 2, 1000, None
    torch.set_default_dtype(case.dtype)
    model = LlamaModel(cfg)
    tensors = S.generate(case)
    for layer in model.layers:
        S.load_layer(layer, S.shard(tensors, rank, world))
    table, final_w, _head, ids = model_stack_inputs(case)
    with torch.no_grad():
        emb = model.embed_tokens
        emb.weight.copy_(table[emb.vocab_start_index:emb.vocab_end_index])
        model.norm.weight.copy_(final_w)

    class Attn(BaseAttentionWrapper):
        def __init__(self): pass
        def init_gpu_cache(self, n): pass
        def get_cache_block(self, n, **k): pass
        def begin_forward(self, l): pass
        def end_forward(self): pass
        def forward(self, q, k, v, idx, softmax_scale=1.0, layer_id=None):
            return q.contiguous()

    with torch.inference_mode():
        out = model(ids, tensors.positions, Attn())
    if rank == 0:
        np.savez_compressed(out_path, out=out.contiguous().view(torch.int16).numpy(), world=np.array([world]))
        print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")
    dist.destroy_process_group()


def mixtral_case(world: int, rank: int):
    """Seeded tensors of the small Mixtral-shaped layer used by the fixture and by the tests (fp16): returns
    (config namespace, full-size tensors, this rank's shards)."""
    from types import SimpleNamespace
    H, nq, nkv, hd, I, E, k, T = 128, 2, 2, 64, 160, 4, 2, 40
    cfg = SimpleNamespace(hidden_size=H, num_attention_heads=nq, num_key_value_heads=nkv, intermediate_size=I,
                          num_local_experts=E, num_experts_per_tok=k, rms_norm_eps=1e-5, rope_theta=10000.0,
                          rope_scaling=None, max_position_embeddings=256)
    g = torch.Generator().manual_seed(31)
    r = lambda *shape, s=1.0: (torch.randn(*shape, generator=g, dtype=torch.float32) * s).to(torch.float16)
    full = dict(x=r(T, H), positions=torch.randint(0, 256, (T,), generator=g), wq=r(nq * hd, H, s=0.1), wk=r(nkv * hd, H, s=0.1),
                wv=r(nkv * hd, H, s=0.1), wo=r(H, nq * hd, s=0.1), gate=r(E, H, s=0.3), w_gate=r(E, I, H, s=0.1),
                w_up=r(E, I, H, s=0.1), w_down=r(E, H, I, s=0.1), ln1=(1 + 0.05 * torch.randn(H, generator=g, dtype=torch.float32)).to(torch.float16),
                ln2=(1 + 0.05 * torch.randn(H, generator=g, dtype=torch.float32)).to(torch.float16))
    ch = lambda t_, dim: t_.chunk(world, dim=dim)[rank]
    ish = slice(rank * (I // world), (rank + 1) * (I // world))
    shard = {"input_layernorm.weight": full["ln1"], "post_attention_layernorm.weight": full["ln2"],
             "self_attn.qkv_proj.weight": torch.cat([ch(full["wq"], 0), ch(full["wk"], 0), ch(full["wv"], 0)]).contiguous(),
             "self_attn.o_proj.weight": ch(full["wo"], 1).contiguous(),
             "block_sparse_moe.gate.weight": full["gate"],
             "block_sparse_moe.experts.w13_weight": torch.cat([full["w_gate"][:, ish], full["w_up"][:, ish]], dim=1).contiguous(),
             "block_sparse_moe.experts.w2_weight": full["w_down"][:, :, ish].contiguous()}
    return cfg, full, shard


def _worker_mixtral_layer(rank: int, world: int, port: int, reference: str, out_path: str) -> None:
    """The reference's MixtralDecoderLayer (models/mixtral.py:194-258) over gloo ranks, fp16, Triton interpreter."""
    os.environ["TRITON_INTERPRET"] = "1"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _install_shims(reference)
    from oracle import tp_layer_oracle as O

    def moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, experts, num_post_pad):
        s_, e_, n_ = O.moe_align_block_size(topk_ids, block_size, num_experts)
        sorted_ids.copy_(s_); experts.copy_(e_.clamp(min=0)); num_post_pad.copy_(n_)

    def topk_softmax(topk_weights, topk_ids, token_expert_indices, gating_output):
        w_, i_, _ = O.topk_softmax(gating_output, topk_weights.shape[1], False)
        topk_weights.copy_(w_); topk_ids.copy_(i_)

    sys.modules["sarathi.moe_ops"].moe_align_block_size = moe_align_block_size
    sys.modules["sarathi.moe_ops"].topk_softmax = topk_softmax
    torch.cuda.get_device_name = lambda *a, **k: "CPU"
    from sarathi.config import MetricsConfig
    from sarathi.metrics.metrics_store import MetricsStore
    MetricsStore.get_or_create_instance(None, None, MetricsConfig(write_metrics=False))
    from sarathi.model_executor.parallel_utils import parallel_state as ps
    ps.initialize_model_parallel(world, 1)
    from sarathi.model_executor.attention.base_attention_wrapper import BaseAttentionWrapper
    from sarathi.model_executor.models.mixtral import MixtralDecoderLayer
    cfg, full, shard = mixtral_case(world, rank)
    torch.set_default_dtype(torch.float16)
    layer = MixtralDecoderLayer(cfg, layer_id=0)
    sd = layer.state_dict()
    with torch.no_grad():
        for name, value in shard.items():
            sd[name].copy_(value)

    class Attn(BaseAttentionWrapper):
        def __init__(self): pass
        def init_gpu_cache(self, n): pass
        def get_cache_block(self, n, **k): pass
        def begin_forward(self, l): pass
        def end_forward(self): pass
        def forward(self, q, k, v, idx, softmax_scale=1.0, layer_id=None):
            return q.contiguous()

    with torch.inference_mode():
        out = layer(full["positions"], full["x"].clone(), 0, Attn())
    if rank == 0:
        np.savez_compressed(out_path, out=out.contiguous().view(torch.int16).numpy(), world=np.array([world]))
        print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")
    dist.destroy_process_group()


ROPE_VARIANTS = {
    "plain": (64, 64, 128, 10000, None),
    "partial": (64, 32, 128, 10000, None),
    "linear": (64, 64, 128, 10000, {"type": "linear", "factor": 2.0}),
    "dynamic": (64, 64, 128, 10000, {"type": "dynamic", "factor": 2.0}),
    "yarn": (64, 64, 256, 10000, {"type": "yarn", "factor": 2.0, "original_max_position_embeddings": 128}),
    "yarn_opts": (128, 128, 512, 500000, {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 128,
                                          "beta_fast": 16, "beta_slow": 2, "attn_factor": 0.9}),
}


def _worker_rope(rank: int, reference: str, out_path: str) -> None:
    """cos|sin tables of the reference's RotaryEmbedding variants (layers/rotary_embedding.py:33-345), fp32."""
    _install_shims(reference)
    from sarathi.model_executor.layers.rotary_embedding import get_rope
    torch.set_default_dtype(torch.float32)
    arrays = {}
    for name, (hs, rot, max_pos, base, scaling) in ROPE_VARIANTS.items():
        cache = get_rope(hs, rot, max_pos, base, True, scaling).cos_sin_cache.float()
        rows = sorted(set(range(8)) | set(range(cache.shape[0] - 8, cache.shape[0])) | set(range(0, cache.shape[0], 9)))
        arrays[name] = cache[rows].numpy()
        arrays[name + "__rows"] = np.array(rows)
        arrays[name + "__shape"] = np.array(cache.shape)
    np.savez_compressed(out_path, **arrays)
    print(f"wrote {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SARATHI_REFERENCE"), required="SARATHI_REFERENCE" not in os.environ,
                    help="checkout of microsoft/sarathi-serve (or $SARATHI_REFERENCE)")
    ap.add_argument("--only", default=None)
    a = ap.parse_args()
    import torch.multiprocessing as mp
    port = 29610
    for case_name, world in RUNS:
        if a.only and a.only != case_name:
            continue
        out_path = os.path.join(HERE, f"{case_name}_tp{world}.npz")
        mp.spawn(_worker, args=(world, case_name, port, a.reference, out_path), nprocs=world)
        port += 1
    if not a.only or a.only == "fused_experts":
        mp.spawn(_worker_fused_experts, args=(a.reference, os.path.join(HERE, "fused_experts_f16.npz")), nprocs=1)
    if not a.only or a.only == "moe_block":
        mp.spawn(_worker_moe_block, args=(2, port + 1, a.reference, os.path.join(HERE, "moe_block_f16_tp2.npz")), nprocs=2)
    if not a.only or a.only == "model_stack":
        mp.spawn(_worker_model_stack, args=(2, port + 3, a.reference, os.path.join(HERE, "llama_model_mini_bf16_tp2.npz")),
                 nprocs=2)
    if not a.only or a.only == "mixtral_layer":
        mp.spawn(_worker_mixtral_layer, args=(2, port + 2, a.reference, os.path.join(HERE, "mixtral_layer_f16_tp2.npz")),
                 nprocs=2)
    if not a.only or a.only == "rope":
        mp.spawn(_worker_rope, args=(a.reference, os.path.join(HERE, "rope_variants.npz")), nprocs=1)
    if not a.only or a.only == "vocab_embedding":
        mp.spawn(_worker_embedding, args=(2, port, a.reference, os.path.join(HERE, "vocab_embedding_tp2.npz")), nprocs=2)


if __name__ == "__main__":
    main()
