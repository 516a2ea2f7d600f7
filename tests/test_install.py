"""``sarathi_serve_b200.install()``: the reference's OWN model file on top of this library.

The reference package is imported from its checkout ($SARATHI_REFERENCE) or from the git-ignored
``baseline/_ref`` install; without either the tests skip.  Each test runs in a child process, because
``install()`` rebinds names inside the imported ``sarathi`` modules.

CPU test: after ``install()`` the reference's ``LlamaDecoderLayer`` is built from this package's layer classes,
keeps the reference's state-dict names and shapes, and the four ops modules resolve to the ctypes stubs.
GPU tests: the reference's own ``LlamaDecoderLayer.forward`` / ``MixtralDecoderLayer.forward`` -- its op
sequence, its residual adds, its RMSNorm / rotary / activation wrappers -- run on the installed library and match
the committed fixtures of the unmodified reference (made on CPU/gloo) and the oracle.
"""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def reference_root():
    """Directory to put on sys.path so that ``import sarathi`` finds the reference, or None."""
    cands = [os.environ.get("SARATHI_REFERENCE"), os.path.join(ROOT, "baseline", "_ref")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "sarathi", "model_executor", "models", "llama.py")):
            return c
    return None


def _child(body: str, timeout: int = 600) -> str:
    ref = reference_root()
    if ref is None:
        pytest.skip("no reference checkout (set SARATHI_REFERENCE) and no baseline/_ref install")
    env = dict(os.environ, SB200_TEST_REFERENCE=ref, MASTER_ADDR="127.0.0.1", MASTER_PORT="29871")
    r = subprocess.run([sys.executable, "-c", _PRELUDE + body], cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=timeout)
    if r.returncode != 0:
        print(r.stdout[-4000:])
        print(r.stderr[-8000:])
    assert r.returncode == 0, f"child failed:\n{r.stderr[-3000:]}"
    return r.stdout


# What the reference needs around it to import and build a layer outside its engine: stub modules for the
# plotting / sketch packages its metrics code imports (and for its protobuf module when that is missing), a disabled MetricsStore, a one-rank process group with
# its parallel state initialised, and -- without a GPU -- its device choices mapped to the CPU.
_PRELUDE = r'''
import os, sys, types
import torch
ROOT = os.getcwd()
sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
sys.path.insert(0, os.environ["SB200_TEST_REFERENCE"])
for name, attrs in (("plotly", {}), ("plotly.express", {}), ("plotly_express", {}), ("ddsketch", {}),
                    ("ddsketch.ddsketch", {"DDSketch": object})):
    try:
        __import__(name)
    except Exception:
        m = types.ModuleType(name); m.__dict__.update(attrs); sys.modules[name] = m
if not os.path.isfile(os.path.join(os.environ["SB200_TEST_REFERENCE"], "sarathi", "core", "proto", "datatypes_pb2.py")):
    # a pip-installed copy of the reference lacks its protobuf module (the directory has no __init__.py, so the
    # reference's own setup.py leaves it out); only the engine's wire format uses it
    class _AnyAttr(types.ModuleType):
        def __getattr__(self, name):
            if name.startswith("__"):
                raise AttributeError(name)
            return object
    sys.modules["sarathi.core.proto"] = _AnyAttr("sarathi.core.proto")
    sys.modules["sarathi.core.proto.datatypes_pb2"] = sys.modules["sarathi.core.proto"].datatypes_pb2 = _AnyAttr("sarathi.core.proto.datatypes_pb2")
HAVE_GPU = torch.cuda.is_available()
if not HAVE_GPU:
    torch.cuda.current_device = lambda: "cpu"
    _arange = torch.arange
    def arange(*a, **k):
        if k.get("device") == "cuda": k["device"] = "cpu"
        return _arange(*a, **k)
    torch.arange = arange
else:
    torch.cuda.set_device(0)
import torch.distributed as dist
dist.init_process_group("gloo", rank=0, world_size=1)
import sarathi_serve_b200
from sarathi_serve_b200.install import install, uninstall
counts = install()
from sarathi.config import MetricsConfig
from sarathi.metrics.metrics_store import MetricsStore
MetricsStore.get_or_create_instance(None, None, MetricsConfig(write_metrics=False))
from sarathi.model_executor.parallel_utils import parallel_state as ref_ps
ref_ps.initialize_model_parallel(1, 1)
from sarathi.model_executor.attention.base_attention_wrapper import BaseAttentionWrapper
class Attn(BaseAttentionWrapper):
    def __init__(self): pass
    def init_gpu_cache(self, n): pass
    def get_cache_block(self, n, **k): pass
    def begin_forward(self, l): pass
    def end_forward(self): pass
    def forward(self, q, k, v, idx, softmax_scale=1.0, layer_id=None):
        return q.contiguous()
'''


def test_install_swaps_ops_and_layers_under_the_reference_model_file():
    out = _child(r'''
import sarathi
from sarathi_serve_b200 import tp_layers, layernorm_ops, activation_ops, pos_encoding_ops, moe_ops, fused_moe, mappings
from sarathi_serve_b200 import parallel_state as ps
assert counts["ops_modules"] == 4 and counts["definitions"] >= 8, counts
# 1. the four compiled-module names resolve to the ctypes stubs, by every route the reference uses
import sarathi.layernorm_ops as a1
from sarathi import activation_ops as a2, pos_encoding_ops as a3, moe_ops as a4
assert a1 is layernorm_ops and a2 is activation_ops and a3 is pos_encoding_ops and a4 is moe_ops
import sarathi.model_executor.layers.layernorm as ref_ln
import importlib
ref_fm = importlib.import_module("sarathi.model_executor.layers.fused_moe.fused_moe")
assert ref_ln.layernorm_ops is layernorm_ops and ref_fm.moe_ops is moe_ops and ref_fm.activation_ops is activation_ops
# 2. the model files see the replacement classes whatever the import order was
import sarathi.model_executor.models.llama as ref_llama
import sarathi.model_executor.models.mixtral as ref_mixtral
import sarathi.model_executor.parallel_utils.tensor_parallel as ref_tp
for mod in (ref_llama, ref_mixtral, ref_tp, ref_tp.layers):
    for name in ("ColumnParallelLinear", "RowParallelLinear", "VocabParallelEmbedding", "ReplicatedLinear"):
        if hasattr(mod, name):
            assert getattr(mod, name) is getattr(tp_layers, name), (mod.__name__, name)
assert ref_mixtral.FusedMoE is fused_moe.FusedMoE
assert ref_tp.reduce_from_tensor_model_parallel_region is mappings.reduce_from_tensor_model_parallel_region
# 3. this package's parallel state follows the reference's
assert ps.model_parallel_is_initialized() and ps.get_tensor_model_parallel_world_size() == 1
assert ps.get_tensor_model_parallel_group() is ref_ps.get_tensor_model_parallel_group()
# 4. the reference's own decoder layer, built from the replacement layers, with the reference's parameter names
from sarathi_serve_b200 import synthetic as S
case = S.CASES["mini_bf16"]
torch.set_default_dtype(case.dtype)
layer = ref_llama.LlamaDecoderLayer(case.hf_config(), layer_id=0)
assert type(layer).__module__ == "sarathi.model_executor.models.llama"
assert type(layer.self_attn.qkv_proj) is tp_layers.ColumnParallelLinear
assert type(layer.self_attn.o_proj) is tp_layers.RowParallelLinear
assert type(layer.mlp.gate_up_proj) is tp_layers.ColumnParallelLinear
assert type(layer.mlp.down_proj) is tp_layers.RowParallelLinear
H, I, hd = case.hidden_size, case.intermediate_size, case.head_dim
shapes = {k: tuple(v.shape) for k, v in layer.state_dict().items()}
assert shapes == {"self_attn.qkv_proj.weight": ((case.num_heads + 2 * case.num_kv_heads) * hd, H),
                  "self_attn.o_proj.weight": (H, case.num_heads * hd),
                  "mlp.gate_up_proj.weight": (2 * I, H), "mlp.down_proj.weight": (H, I),
                  "input_layernorm.weight": (H,), "post_attention_layernorm.weight": (H,)}, shapes
S.load_layer(layer, S.shard(S.generate(case), 0, 1))  # the loader contract: copy into layer.<name>.weight
mcfg = types.SimpleNamespace(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=512,
                             num_local_experts=8, num_experts_per_tok=2, rms_norm_eps=1e-5, rope_theta=10000.0,
                             max_position_embeddings=512, sliding_window=None)
ml = ref_mixtral.MixtralDecoderLayer(mcfg, layer_id=0)
names = set(ml.state_dict().keys())
assert {"block_sparse_moe.gate.weight", "block_sparse_moe.experts.w13_weight", "block_sparse_moe.experts.w2_weight",
        "self_attn.qkv_proj.weight", "self_attn.o_proj.weight"} <= names, names
assert type(ml.block_sparse_moe.experts) is fused_moe.FusedMoE and type(ml.block_sparse_moe.gate) is tp_layers.ReplicatedLinear
# 5. and back
uninstall()
assert ref_llama.ColumnParallelLinear is not tp_layers.ColumnParallelLinear
assert ref_llama.ColumnParallelLinear.__module__.startswith("sarathi.")
assert not ps.model_parallel_is_initialized()
print("INSTALL-OK", counts)
''')
    assert "INSTALL-OK" in out


@pytest.mark.gpu
def test_reference_llama_decoder_layer_forward_on_installed_library():
    out = _child(r'''
from helpers import TOL, load_golden, rel_err
from oracle import tp_layer_oracle as O
from sarathi_serve_b200 import synthetic as S, parallel_state as ps, dense_ops
import sarathi.model_executor.models.llama as ref_llama
for case_name in ("mini_f32", "mini_bf16", "mini_f16"):
    case = S.CASES[case_name]
    torch.set_default_dtype(case.dtype)
    layer = ref_llama.LlamaDecoderLayer(case.hf_config(), layer_id=0).cuda()
    torch.set_default_dtype(torch.float32)
    t = S.generate(case)
    S.load_layer(layer, S.shard(t, 0, 1))
    with torch.inference_mode():
        out = layer(t.positions.cuda(), t.x.to(case.dtype).cuda(), 0, Attn())
    torch.cuda.synchronize()
    dense_ops.check_status(torch.device("cuda", 0))
    gold, _, step, _ = load_golden(case_name, 1)
    err_fix = rel_err(out[::step], gold["out"])
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    ref = O.decoder_layer([S.shard(t, 0, 1)], t.x.to(case.dtype), t.positions, num_heads=case.num_heads,
                          num_kv_heads=case.num_kv_heads, head_dim=case.head_dim, eps=case.rms_norm_eps, cache=cache)["out"]
    err_or = rel_err(out, ref)
    print(case_name, "fixture", err_fix, "oracle", err_or)
    assert err_fix <= TOL[case.dtype] and err_or <= TOL[case.dtype], (case_name, err_fix, err_or)
print("FORWARD-OK")
''')
    assert "FORWARD-OK" in out


@pytest.mark.gpu
def test_reference_mixtral_decoder_layer_forward_on_installed_library():
    out = _child(r'''
import numpy as np
from helpers import rel_err
from make_golden import mixtral_case
from test_oracle_golden import _mixtral_oracle
from sarathi_serve_b200 import dense_ops
import sarathi.model_executor.models.mixtral as ref_mixtral
cfg, full, shard = mixtral_case(1, 0)
torch.set_default_dtype(torch.float16)
layer = ref_mixtral.MixtralDecoderLayer(cfg, layer_id=0).cuda()
torch.set_default_dtype(torch.float32)
sd = layer.state_dict()
with torch.no_grad():
    for name, value in shard.items():
        sd[name].copy_(value)
with torch.inference_mode():
    out = layer(full["positions"].cuda(), full["x"].cuda(), 0, Attn())
torch.cuda.synchronize()
dense_ops.check_status(torch.device("cuda", 0))
_, _, ref = _mixtral_oracle(1)
g = np.load(os.path.join(ROOT, "tests", "golden", "mixtral_layer_f16_tp2.npz"))
e1, e2 = rel_err(out, ref), rel_err(out, torch.from_numpy(g["out"]).view(torch.float16))
print("oracle", e1, "fixture", e2)
assert e1 <= 5e-3 and e2 <= 5e-3
print("FORWARD-OK")
''')
    assert "FORWARD-OK" in out
