"""CPU oracle of the tensor-parallel decoder-layer path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this module, and only as the checker or the timed CPU baseline: the product
(sarathi_serve_b200) never imports it and has no CPU path.

Each function restates, with torch/numpy on the CPU, what one piece of the
reference (microsoft/sarathi-serve) computes, citing the file:line it follows.
The reference's 16-bit scalar types compute every binary operator in fp32 and
round the result to the type; torch's CPU kernels for bf16/fp16 tensors do the
same per operator, so expressions are written operator by operator on tensors
of the model dtype.

Pinning:
  * layer-level functions are checked against fixtures produced by running the
    reference's own Python modules (ColumnParallelLinear, RowParallelLinear,
    LlamaDecoderLayer, RMSNorm, RotaryEmbedding, VocabParallelEmbedding, ... imported from the reference
    checkout, CPU/gloo) -- tests/golden/make_golden.py, tests/golden/*.npz;
  * op-level functions (rms_norm, silu_and_mul, gelu_*, rotary_embedding,
    topk_softmax, moe_align_block_size) are checked on the GPU against the
    reference's own CUDA kernels compiled into oracle/_ref/ (oracle/build_ref.py);
  * moe_align_block_size is also checked against the worked example in the
    reference's kernel comment (csrc/moe_align_block_size_kernels.cu:88-93);
  * fused_experts() (the reference's Triton grouped GEMMs, layers/fused_moe/fused_moe.py:15-148,411-544) is
    checked against a fixture made by running the reference's own kernel in the Triton interpreter on the CPU
    (fp16 only -- the installed interpreter mishandles bf16; tests/golden/make_golden.py): equal except for
    one-ulp differences where the order of the fp32 additions along K decides a rounding; moe_layer() likewise
    against the reference's MixtralMoE block over two gloo ranks.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------- ops
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """csrc/layernorm_kernels.cu:10-35: fp32 sum of squares, inv = rsqrt(var/H + eps),
    out = ((T)(x * inv)) * w with the product rounded to T before the weight multiply."""
    xf = x.float()
    var = xf.pow(2).sum(-1, keepdim=True) / x.shape[-1]
    inv = torch.rsqrt(var + eps)
    return (xf * inv).to(x.dtype) * w


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    """models/llama.py:248,251-252: z = residual + x in the model dtype, then rms_norm(z)."""
    z = residual + x
    return rms_norm(z, w, eps), z


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """csrc/activation_kernels.cu:8-25: (T)(g / (1 + expf(-g))) * u."""
    d = x.shape[-1] // 2
    g = x[..., :d].float()
    return (g / (1.0 + torch.exp(-g))).to(x.dtype) * x[..., d:]


def gelu_new(x: torch.Tensor) -> torch.Tensor:
    """csrc/activation_kernels.cu:86-91."""
    T = x.dtype
    x3 = (x * x * x).float()
    inner = (x + (0.044715 * x3).to(T)).float()
    t = torch.tanh((0.79788456 * inner).to(T).float()).to(T)
    half, one = torch.tensor(0.5, dtype=T), torch.tensor(1.0, dtype=T)
    return half * x * (one + t)


def gelu_fast(x: torch.Tensor) -> torch.Tensor:
    """csrc/activation_kernels.cu:93-98."""
    T = x.dtype
    f = x.float()
    one, half = torch.tensor(1.0, dtype=T), torch.tensor(0.5, dtype=T)
    a = (f * 0.79788456).to(T)
    b = one + (0.044715 * f).to(T) * x
    t = torch.tanh((a * b).float()).to(T)
    return half * x * (one + t)


def cos_sin_cache(head_dim: int, rot_dim: int, max_pos: int, base: float, dtype: torch.dtype) -> torch.Tensor:
    """layers/rotary_embedding.py:55-84 (+ the cast of :51-53): inv_freq = base^(-2i/rot),
    cache[p] = cos(p*inv_freq) | sin(p*inv_freq), computed in fp32 then cast."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(dtype)


def rotary_embedding(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor, head_size: int,
                     cache: torch.Tensor, is_neox: bool) -> None:
    """csrc/pos_encoding_kernels.cu:8-76, in place on (possibly strided) 2-D views."""
    rot = cache.shape[1]
    half = rot // 2
    cs = cache[positions]
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    for t in (query, key):
        if t.shape[1] == 0:
            continue
        v = t.unflatten(1, (-1, head_size))
        if is_neox:
            x, y = v[..., :half].clone(), v[..., half:rot].clone()
            v[..., :half] = x * cos - y * sin
            v[..., half:rot] = y * cos + x * sin
        else:
            x, y = v[..., 0:rot:2].clone(), v[..., 1:rot:2].clone()
            v[..., 0:rot:2] = x * cos - y * sin
            v[..., 1:rot:2] = y * cos + x * sin


# ---------------------------------------------------------------- MoE routing
def _pow2_row_sum(e: np.ndarray) -> np.ndarray:
    """Row sums of exp values in the evaluation order of the reference's warp-level
    kernel (csrc/moe_topk_softmax_kernels.cu:259-301): each thread sums its VPT values
    in order, then an xor-butterfly over the THREADS_PER_ROW threads of the row."""
    T, E = e.shape
    ldg = min(4, E)
    vecs = max(1, E // (ldg * 32))
    vpt = vecs * ldg
    tpr = E // vpt
    # thread g holds, for ldg group l, columns l*ldg*tpr + g*ldg .. +ldg
    cols = np.empty((tpr, vpt), dtype=np.int64)
    for g in range(tpr):
        for l in range(vecs):
            for j in range(ldg):
                cols[g, l * ldg + j] = l * ldg * tpr + g * ldg + j
    part = np.zeros((T, tpr), dtype=np.float32)
    for i in range(vpt):
        part = (part + e[:, cols[:, i]]).astype(np.float32)
    m = tpr // 2
    idx = np.arange(tpr)
    while m > 0:
        part = (part + part[:, idx ^ m]).astype(np.float32)
        m //= 2
    return part[:, 0]


def topk_softmax(gating: torch.Tensor, k: int, renormalize: bool = False):
    """fused_moe.py:346-373 + csrc/moe_topk_softmax_kernels.cu:182-380: fp32 softmax
    (max, expf(x - max), sum, multiply by the reciprocal), then k rounds of arg-max
    with the lowest index winning ties.  Returns (weights f32 [T,k], ids i32 [T,k],
    token_expert_indices i32 [T,k])."""
    g = gating.float().numpy().astype(np.float32)
    T, E = g.shape
    mx = g.max(axis=1, keepdims=True)
    e = np.exp((g - mx).astype(np.float32)).astype(np.float32)
    if E & (E - 1) == 0 and E <= 256:
        s = _pow2_row_sum(e)
    else:
        s = e.sum(axis=1, dtype=np.float32)
    rcp = (np.float32(1.0) / s).astype(np.float32)
    p = (e * rcp[:, None]).astype(np.float32)
    w = np.empty((T, k), dtype=np.float32)
    ids = np.empty((T, k), dtype=np.int32)
    work = p.copy()
    rows = np.arange(T)
    for j in range(k):
        best = work.argmax(axis=1)  # numpy returns the first maximum: lowest index wins
        w[:, j] = work[rows, best]
        ids[:, j] = best
        work[rows, best] = -10000.0
    src = (np.arange(k, dtype=np.int32)[None, :] * T + np.arange(T, dtype=np.int32)[:, None]).astype(np.int32)
    wt = torch.from_numpy(w)
    if renormalize:
        wt = wt / wt.sum(dim=-1, keepdim=True)
    return wt, torch.from_numpy(ids), torch.from_numpy(src)


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """fused_moe.py:151-204 + csrc/moe_align_block_size_kernels.cu:23-109: stable counting
    sort of flat slot indices by expert; each expert's run padded to a multiple of
    block_size with the value numel.  Returns (sorted_ids [numel + E*(block-1)],
    expert_ids [ceil(that / block)] (only the first num_post_pad/block are defined; the
    rest is filled with -1 here), num_tokens_post_pad [1])."""
    flat = topk_ids.reshape(-1).numpy().astype(np.int64)
    n = flat.size
    cap = n + num_experts * (block_size - 1)
    sorted_ids = np.full(cap, n, dtype=np.int32)
    expert_ids = np.full((cap + block_size - 1) // block_size, -1, dtype=np.int32)
    pos = 0
    for e in range(num_experts):
        idx = np.nonzero(flat == e)[0]
        padded = (len(idx) + block_size - 1) // block_size * block_size
        sorted_ids[pos:pos + len(idx)] = idx
        expert_ids[pos // block_size:(pos + padded) // block_size] = e
        pos += padded
    return torch.from_numpy(sorted_ids), torch.from_numpy(expert_ids), torch.tensor([pos], dtype=torch.int32)


def fused_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                  topk_ids: torch.Tensor) -> torch.Tensor:
    """fused_moe.py:411-544 with the rounding points of the Triton kernel (:15-148):
    GEMM1 (fp32 accumulate) -> T, silu_and_mul -> T, GEMM2 * routed weight (fp32) -> T,
    sum over the k slots -> T.  Pinned for fp16 by tests/golden/fused_experts_f16.npz (see the module docstring)."""
    T_, H = x.shape
    k = topk_ids.shape[1]
    out3 = torch.zeros(T_, k, w2.shape[1], dtype=x.dtype)
    for e in range(w13.shape[0]):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        c1 = (x[tok].float() @ w13[e].float().t()).to(x.dtype)
        a = silu_and_mul(c1)
        c3 = (a.float() @ w2[e].float().t()) * topk_weights[tok, slot].float()[:, None]
        out3[tok, slot] = c3.to(x.dtype)
    return torch.sum(out3, dim=1)


# ------------------------------------------------------------------- layers
def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tensor_parallel/layers.py:278-284,421-423: F.linear on the local shard."""
    return F.linear(x, w, b)


def vocab_parallel_embedding(ids: torch.Tensor, weight_shards: Sequence[torch.Tensor]) -> torch.Tensor:
    """tensor_parallel/layers.py:147-177 over len(weight_shards) simulated ranks: each rank looks up the ids of
    its vocabulary slice (zeros elsewhere), then the SUM all-reduce."""
    per = weight_shards[0].shape[0]
    parts = []
    for r, w in enumerate(weight_shards):
        lo, hi = r * per, (r + 1) * per
        mask = (ids < lo) | (ids >= hi)
        local = (ids - lo).masked_fill(mask, 0)
        o = w[local].clone()
        o[mask] = 0
        parts.append(o)
    return sum_over_ranks(parts)


def sum_over_ranks(parts: Sequence[torch.Tensor]) -> torch.Tensor:
    """tensor_parallel/mappings.py:16-26: element-wise SUM all-reduce in the tensor dtype,
    evaluated here in rank order."""
    acc = parts[0].clone()
    for p in parts[1:]:
        acc = acc + p
    return acc


def kv_cache_slots(batch_indices, positions, kv_indices, kv_indptr, page_size: int) -> torch.Tensor:
    """Row of the cache, seen as [pages * 2 * page_size, kv_heads * head_dim], that receives each token's key
    (-1 for a negative batch index): page = kv_indices[kv_indptr[b] + p // page_size], slot = p % page_size --
    the addressing of flashinfer's append_paged_kv_cache (flashinfer-python, pinned 0.4.1 in the reference's
    requirements.txt:18; not vendored), which the reference calls at
    attention/flashinfer_attention_wrapper.py:261-270."""
    b = np.asarray(batch_indices, dtype=np.int64)
    p = np.asarray(positions, dtype=np.int64)
    ki = np.asarray(kv_indices, dtype=np.int64)
    kp = np.asarray(kv_indptr, dtype=np.int64)
    out = np.full(b.shape, -1, dtype=np.int64)
    ok = b >= 0
    page = ki[kp[b[ok]] + p[ok] // page_size]
    out[ok] = page * (2 * page_size) + p[ok] % page_size
    return torch.from_numpy(out)


def append_paged_kv_cache(key: torch.Tensor, value: torch.Tensor, batch_indices, positions, cache: torch.Tensor,
                          kv_indices, kv_indptr) -> None:
    """In place on ``cache`` [pages, 2, page_size, kv_heads, head_dim] (attention/flashinfer_attention_wrapper.py:69-77):
    cache[page, 0, slot] = key[i], cache[page, 1, slot] = value[i]."""
    page_size = cache.shape[2]
    s = kv_cache_slots(batch_indices, positions, kv_indices, kv_indptr, page_size)
    flat = cache.view(cache.shape[0] * 2 * page_size, -1)
    n = s.numel()
    k2, v2 = key.reshape(n, -1), value.reshape(n, -1)
    for i in range(n):
        if s[i] >= 0:
            flat[s[i]] = k2[i]
            flat[s[i] + page_size] = v2[i]


def decoder_layer(params: Sequence[Dict[str, torch.Tensor]], x: torch.Tensor, positions: torch.Tensor, *,
                  num_heads: int, num_kv_heads: int, head_dim: int, eps: float, cache: torch.Tensor,
                  all_reduce: Optional[Callable[[List[torch.Tensor]], torch.Tensor]] = None,
                  next_norm_weight: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """models/llama.py:232-255 (LlamaDecoderLayer.forward) with LlamaAttention.forward
    (:168-188) and LlamaMLP.forward (:101-106) over `len(params)` simulated ranks.

    params[r] is rank r's state dict (synthetic.shard).  Attention itself is outside the
    path: the stand-in is attn_out = q (after rotary, contiguous), as in the fixtures.
    Returns rank 0's intermediates plus the (rank-independent) layer output."""
    world = len(params)
    reduce = all_reduce or sum_over_ranks
    nq, nkv = num_heads // world, num_kv_heads // world
    q_size, kv_size = nq * head_dim, nkv * head_dim
    out: Dict[str, torch.Tensor] = {}
    residual = x
    o_parts, per_rank = [], []
    for r, p in enumerate(params):
        h = rms_norm(x, p["input_layernorm.weight"], eps)
        qkv = linear(h, p["self_attn.qkv_proj.weight"])
        if r == 0:
            out["input_norm"] = h
            out["qkv_pre_rotary"] = qkv.clone()
        q, k, v = qkv.split([q_size, kv_size, kv_size], dim=-1)
        rotary_embedding(positions, q, k, head_dim, cache, True)
        if r == 0:
            out["qkv"] = qkv.clone()
        attn = q.contiguous()
        o_parts.append(linear(attn, p["self_attn.o_proj.weight"]))
        per_rank.append(p)
    o = reduce(o_parts)
    out["o_proj"] = o
    hidden = residual + o
    out["residual_mid"] = hidden
    residual = hidden
    d_parts = []
    for r, p in enumerate(params):
        h2 = rms_norm(hidden, p["post_attention_layernorm.weight"], eps)
        gate_up = linear(h2, p["mlp.gate_up_proj.weight"])
        act = silu_and_mul(gate_up)
        if r == 0:
            out["post_attn_norm"] = h2
            out["gate_up"] = gate_up
            out["act"] = act
        d_parts.append(linear(act, p["mlp.down_proj.weight"]))
    d = reduce(d_parts)
    out["down_proj"] = d
    out["out"] = residual + d
    if next_norm_weight is not None:
        out["out_normed"] = rms_norm(out["out"], next_norm_weight, eps)
    return out


def decoder_layer_distributed(p: Dict[str, torch.Tensor], x: torch.Tensor, positions: torch.Tensor, *,
                              num_heads: int, num_kv_heads: int, head_dim: int, eps: float, cache: torch.Tensor,
                              world: int, group=None) -> torch.Tensor:
    """The same layer for ONE real rank of a torch.distributed (gloo) group: the all-reduce is
    torch.distributed.all_reduce, as in tensor_parallel/mappings.py:24."""
    import torch.distributed as dist

    def ar(t):
        if world > 1:
            dist.all_reduce(t, group=group)
        return t

    nq, nkv = num_heads // world, num_kv_heads // world
    q_size, kv_size = nq * head_dim, nkv * head_dim
    residual = x
    h = rms_norm(x, p["input_layernorm.weight"], eps)
    qkv = linear(h, p["self_attn.qkv_proj.weight"])
    q, k, v = qkv.split([q_size, kv_size, kv_size], dim=-1)
    rotary_embedding(positions, q, k, head_dim, cache, True)
    o = ar(linear(q.contiguous(), p["self_attn.o_proj.weight"]))
    hidden = residual + o
    h2 = rms_norm(hidden, p["post_attention_layernorm.weight"], eps)
    act = silu_and_mul(linear(h2, p["mlp.gate_up_proj.weight"]))
    d = ar(linear(act, p["mlp.down_proj.weight"]))
    return hidden + d


def moe_layer(x: torch.Tensor, gate_w: torch.Tensor, w13: Sequence[torch.Tensor], w2: Sequence[torch.Tensor],
              top_k: int, renormalize: bool = True) -> torch.Tensor:
    """models/mixtral.py:102-108 + layers/fused_moe/layer.py:122-134 over len(w13) simulated ranks:
    router logits from the replicated gate (F.linear), fused_topk, each rank's fused_experts on its
    shard of every expert (w13[r]: [E, 2I/tp, H], w2[r]: [E, H, I/tp]), then the SUM all-reduce."""
    logits = linear(x, gate_w)
    wts, ids, _ = topk_softmax(logits, top_k, renormalize)
    parts = [fused_experts(x, w13[r], w2[r], wts, ids.long()) for r in range(len(w13))]
    return sum_over_ranks(parts)


def mixtral_decoder_layer(attn_params: Sequence[Dict[str, torch.Tensor]], gate_w: torch.Tensor,
                          w13: Sequence[torch.Tensor], w2: Sequence[torch.Tensor], x: torch.Tensor,
                          positions: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, eps: float,
                          cache: torch.Tensor, top_k: int) -> torch.Tensor:
    """models/mixtral.py:235-258 (MixtralDecoderLayer.forward) over len(attn_params) simulated ranks: the
    attention block of the Llama layer (qkv, rotary, stand-in attn_out = q, o_proj + SUM all-reduce, residual
    add), post-attention norm, then the MoE block (moe_layer) and the second residual add.
    attn_params[r]: rank r's "input_layernorm.weight", "post_attention_layernorm.weight",
    "self_attn.qkv_proj.weight", "self_attn.o_proj.weight"."""
    world = len(attn_params)
    nq, nkv = num_heads // world, max(1, num_kv_heads // world)
    q_size, kv_size = nq * head_dim, nkv * head_dim
    o_parts = []
    for p in attn_params:
        h = rms_norm(x, p["input_layernorm.weight"], eps)
        qkv = linear(h, p["self_attn.qkv_proj.weight"])
        q, k, _v = qkv.split([q_size, kv_size, kv_size], dim=-1)
        rotary_embedding(positions, q, k, head_dim, cache, True)
        o_parts.append(linear(q.contiguous(), p["self_attn.o_proj.weight"]))
    hidden = x + sum_over_ranks(o_parts)
    h2 = rms_norm(hidden, attn_params[0]["post_attention_layernorm.weight"], eps)
    return hidden + moe_layer(h2, gate_w, w13, w2, top_k)


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """The parity measure used everywhere: max|a - ref| / max|ref| (element-wise relative
    error is meaningless near zero)."""
    denom = float(ref.double().abs().max())
    return float((a.double() - ref.double()).abs().max()) / (denom if denom > 0 else 1.0)
