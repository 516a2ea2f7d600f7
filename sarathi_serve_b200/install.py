"""``install()``: run the reference's own model_executor on this library.

The reference's layer wrappers import four compiled ops modules by name
(``from sarathi import layernorm_ops`` -- sarathi/model_executor/layers/layernorm.py:8,
``activation_ops`` -- layers/activation.py:6, ``pos_encoding_ops`` --
layers/rotary_embedding.py:30, ``moe_ops`` -- layers/fused_moe/fused_moe.py:12) and its model
files take the tensor-parallel layer classes from
``sarathi.model_executor.parallel_utils.tensor_parallel`` (models/llama.py:48-52,
models/mixtral.py).  ``install()``

  1. registers this package's ctypes-backed ops modules under those four names, so the reference's
     ``RMSNorm`` / ``SiluAndMul`` / ``RotaryEmbedding`` / ``fused_topk`` / ``moe_align_block_size``
     call this library's kernels through the unchanged pybind signatures;
  2. replaces ``ColumnParallelLinear``, ``RowParallelLinear``, ``ReplicatedLinear``,
     ``VocabParallelEmbedding`` and ``reduce_from_tensor_model_parallel_region`` (and, optionally,
     ``FusedMoE``, ``RMSNorm``, ``SiluAndMul``, ``get_rope``) in the modules that define them AND in every
     already imported ``sarathi.*`` module that holds a reference to the original, so the order of
     imports does not matter;
  3. makes this package's ``parallel_state`` follow the reference's (group, rank and size come from
     ``sarathi.model_executor.parallel_utils.parallel_state`` once that is initialised).

After it, ``sarathi.model_executor.models.llama.LlamaDecoderLayer(config)`` -- the reference's own class,
untouched -- builds its projections from this package's layers (same parameter names and shapes, so the
reference's weight loaders keep working) and its forward runs on the tcgen05 GEMMs, the fused
GEMM + all-reduce kernel and the element-wise kernels of this library.  ``uninstall()`` undoes it.
"""
from __future__ import annotations

import importlib
import sys
from typing import Any, Dict, List, Tuple

_OPS = ("layernorm_ops", "activation_ops", "pos_encoding_ops", "moe_ops")
_TP = "sarathi.model_executor.parallel_utils.tensor_parallel"
_STATE: Dict[str, Any] = {}


def _replacements(fused_moe: bool, nn_layers: bool) -> List[Tuple[str, str, Any]]:
    """(defining module of the reference, attribute, replacement)."""
    from . import mappings, tp_layers
    out = [(_TP + ".layers", n, getattr(tp_layers, n))
           for n in ("ColumnParallelLinear", "RowParallelLinear", "ReplicatedLinear", "VocabParallelEmbedding")]
    out += [(_TP + ".mappings", n, getattr(mappings, n))
            for n in ("reduce_from_tensor_model_parallel_region", "gather_from_tensor_model_parallel_region",
                      "scatter_to_tensor_model_parallel_region", "copy_to_tensor_model_parallel_region")]
    if fused_moe:
        from . import fused_moe as fm
        out.append(("sarathi.model_executor.layers.fused_moe.layer", "FusedMoE", fm.FusedMoE))
    if nn_layers:
        from . import nn_layers as nl
        out += [("sarathi.model_executor.layers.layernorm", "RMSNorm", nl.RMSNorm),
                ("sarathi.model_executor.layers.activation", "SiluAndMul", nl.SiluAndMul),
                ("sarathi.model_executor.layers.rotary_embedding", "get_rope", nl.get_rope)]
    return out


def install(*, fused_moe: bool = True, nn_layers: bool = False) -> Dict[str, int]:
    """See the module docstring.  ``fused_moe``: also replace the reference's ``FusedMoE`` (Triton grouped GEMM)
    by this package's (tcgen05 grouped GEMM); ``nn_layers``: also replace ``RMSNorm`` / ``SiluAndMul`` /
    ``get_rope`` by this package's module wrappers (the reference's own wrappers already run on this library's
    kernels through the ops modules, so this is optional).  Returns how many names were rebound.  The ``sarathi``
    package has to be importable (with whatever its own imports need); calling it twice is harmless."""
    if _STATE.get("installed"):
        return dict(_STATE["counts"])
    from . import _native
    _native.lib()  # fail now, loudly, if the CUDA library is missing
    saved: List[Tuple[Any, str, Any]] = []   # (module, attribute, original value or _MISSING)
    counts = {"ops_modules": 0, "definitions": 0, "rebound_references": 0}

    # 1. the ops modules.  `from sarathi import layernorm_ops` finds a sys.modules entry named
    #    "sarathi.layernorm_ops" (and the attribute on the package once it is imported).
    for name in _OPS:
        mod = importlib.import_module(f"{__package__}.{name}")
        full = "sarathi." + name
        saved.append((sys.modules, full, sys.modules.get(full, _MISSING)))
        sys.modules[full] = mod
        counts["ops_modules"] += 1
    import sarathi  # noqa: F401  (the reference package; its compiled ops modules are the ones registered above)
    for name in _OPS:
        saved.append((sarathi, name, getattr(sarathi, name, _MISSING)))
        setattr(sarathi, name, sys.modules["sarathi." + name])

    # 2. classes and functions: in their defining modules, in the package namespaces that re-export them, and in
    #    every imported sarathi.* module that already bound the original
    originals: Dict[int, Any] = {}
    for mod_name, attr, repl in _replacements(fused_moe, nn_layers):
        mod = importlib.import_module(mod_name)
        orig = getattr(mod, attr)
        if orig is repl:
            continue
        originals[id(orig)] = (orig, repl)
        saved.append((mod, attr, orig))
        setattr(mod, attr, repl)
        counts["definitions"] += 1
    for mname, mod in list(sys.modules.items()):
        if mod is None or not (mname == "sarathi" or mname.startswith("sarathi.")):
            continue
        for attr, val in list(vars(mod).items()):
            hit = originals.get(id(val))
            if hit is not None and hit[0] is val:
                saved.append((mod, attr, val))
                setattr(mod, attr, hit[1])
                counts["rebound_references"] += 1

    # 3. group / rank / size follow the reference's parallel state
    from . import parallel_state as ps
    ref_ps = importlib.import_module("sarathi.model_executor.parallel_utils.parallel_state")
    ps.follow(ref_ps)

    _STATE.update(installed=True, saved=saved, counts=counts)
    return dict(counts)


class _Missing:
    pass


_MISSING = _Missing()


def uninstall() -> None:
    """Put every name ``install()`` changed back."""
    if not _STATE.get("installed"):
        return
    for holder, attr, orig in reversed(_STATE["saved"]):
        if isinstance(holder, dict):
            if orig is _MISSING:
                holder.pop(attr, None)
            else:
                holder[attr] = orig
        elif orig is _MISSING:
            if hasattr(holder, attr):
                delattr(holder, attr)
        else:
            setattr(holder, attr, orig)
    from . import parallel_state as ps
    ps.follow(None)
    _STATE.clear()
