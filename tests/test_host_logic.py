"""Host-side logic that needs no GPU: sharding, layer construction (API surface,
parameter names and shapes), tensor-parallel group bookkeeping over gloo with
two processes, the distributed oracle, and a threaded model of the device-side
push / reduce / finish counter protocol including a rank that never arrives."""
import os
import threading
import time

import pytest
import torch
import torch.multiprocessing as mp

from oracle import tp_layer_oracle as O
from sarathi_serve_b200 import synthetic as S


def test_divide_and_shard_shapes():
    from sarathi_serve_b200.mappings import divide
    assert divide(12, 4) == 3
    with pytest.raises(AssertionError):
        divide(10, 4)
    t = S.generate(S.CASES["mini_bf16"])
    for world in (1, 2):
        p = S.shard(t, world - 1, world)
        assert p["self_attn.qkv_proj.weight"].shape == ((4 + 2 * 2) * 128 // world, 512)
        assert p["self_attn.o_proj.weight"].shape == (512, 4 * 128 // world)
        assert p["mlp.gate_up_proj.weight"].shape == (2 * 1024 // world, 512)
        assert p["mlp.down_proj.weight"].shape == (512, 1024 // world)
    # shards tile the full matrices
    p0, p1 = S.shard(t, 0, 2, torch.float32), S.shard(t, 1, 2, torch.float32)
    assert torch.equal(torch.cat([p0["self_attn.o_proj.weight"], p1["self_attn.o_proj.weight"]], 1), t.wo)
    assert torch.equal(torch.cat([p0["mlp.gate_up_proj.weight"][:512], p1["mlp.gate_up_proj.weight"][:512]]), t.wgate)


def test_generator_is_deterministic_and_dtype_independent():
    a = S.generate(S.CASES["mini_f32"])
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        b = S.generate(S.CASES["mini_f32"])
    finally:
        torch.set_default_dtype(old)
    assert torch.equal(a.x, b.x) and torch.equal(a.wdown, b.wdown) and torch.equal(a.positions, b.positions)
    c = S.CASES["config2"]
    assert c.num_tokens == 512 and c.prefill_tokens == 448 and c.decode_tokens == 64


def test_layer_api_surface_on_cpu():
    """Constructor keywords, attributes and state-dict names/shapes of the reference's layers."""
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer
    from sarathi_serve_b200.tp_layers import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    ps.set_tensor_model_parallel_world_size(4)
    ps.set_tensor_model_parallel_rank(1)
    try:
        col = ColumnParallelLinear(64, 256, bias=True, gather_output=False, skip_bias_add=True,
                                   params_dtype=torch.bfloat16, linear_metric_name="x",
                                   communication_metric_name="y", layer_id=3)
        assert col.weight.shape == (64, 64) and col.bias.shape == (64,) and col.output_size_per_partition == 64
        assert col.weight.dtype == torch.bfloat16 and col.world_size == 4
        row = RowParallelLinear(256, 64, bias=False, input_is_parallel=True, reduce_results=True, layer_id=0)
        assert row.weight.shape == (64, 64) and row.bias is None and row.input_size_per_partition == 64
        rep = ReplicatedLinear(64, 8, bias=False, params_dtype=torch.float16, metric_name="g")
        assert rep.weight.shape == (8, 64)
        with pytest.raises(AssertionError):
            ColumnParallelLinear(64, 30)  # 30 not divisible by 4
        with pytest.raises(AssertionError):
            RowParallelLinear(64, 64, perform_initialization=True)
        case = S.CASES["config1"]
        layer = LlamaDecoderLayer(case.hf_config(), layer_id=0)
        sd = layer.state_dict()
        assert sd["self_attn.qkv_proj.weight"].shape == ((16 + 8) * 64 // 4, 1024)
        assert sd["self_attn.o_proj.weight"].shape == (1024, 1024 // 4)
        assert sd["mlp.gate_up_proj.weight"].shape == (2 * 2816 // 4, 1024)
        assert sd["mlp.down_proj.weight"].shape == (1024, 2816 // 4)
        assert set(sd) == {"self_attn.qkv_proj.weight", "self_attn.o_proj.weight", "mlp.gate_up_proj.weight",
                           "mlp.down_proj.weight", "input_layernorm.weight", "post_attention_layernorm.weight"}
        with pytest.raises(RuntimeError):  # no CPU fallback: a CPU tensor is refused
            col(torch.randn(4, 64, dtype=torch.bfloat16))
    finally:
        ps.destroy_model_parallel()


def test_rope_variants_build_tables():
    from sarathi_serve_b200.nn_layers import get_rope
    base = get_rope(64, 64, 128, 10000, True, None)
    assert base.cos_sin_cache.shape == (128, 64)
    assert torch.allclose(base.cos_sin_cache.float().cpu(), O.cos_sin_cache(64, 64, 128, 10000.0, torch.float32))
    lin = get_rope(64, 64, 128, 10000, True, {"type": "linear", "factor": 2.0})
    assert lin.cos_sin_cache.shape == (256, 64)
    assert torch.allclose(lin.cos_sin_cache[2].float(), base.cos_sin_cache[1].float())
    dyn = get_rope(64, 64, 128, 10000, True, {"type": "dynamic", "factor": 2.0})
    assert dyn.cos_sin_cache.shape == (256, 64)
    yarn = get_rope(64, 64, 256, 10000, True, {"type": "yarn", "factor": 2.0, "original_max_position_embeddings": 128})
    assert yarn.cos_sin_cache.shape == (256, 64)
    with pytest.raises(ValueError):
        get_rope(64, 64, 128, 10000, True, {"type": "nope", "factor": 2.0})


# ---------------------------------------------------------------- gloo, 2 ranks
def _gloo_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.mappings import gather_from_tensor_model_parallel_region, scatter_to_tensor_model_parallel_region
    ps.initialize_model_parallel(world)
    assert ps.get_tensor_model_parallel_world_size() == world
    assert ps.get_tensor_model_parallel_rank() == rank
    x = torch.arange(12.0).view(3, 4)
    mine = scatter_to_tensor_model_parallel_region(x)
    assert torch.equal(mine, x[:, rank * 2:(rank + 1) * 2])
    assert torch.equal(gather_from_tensor_model_parallel_region(mine), x)
    # distributed oracle == single-process simulated-rank oracle
    case = S.CASES["mini_f32"]
    t = S.generate(case)
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    kw = dict(num_heads=case.num_heads, num_kv_heads=case.num_kv_heads, head_dim=case.head_dim,
              eps=case.rms_norm_eps, cache=cache)
    out = O.decoder_layer_distributed(S.shard(t, rank, world), t.x, t.positions, world=world,
                                      group=ps.get_tensor_model_parallel_group(), **kw)
    sim = O.decoder_layer([S.shard(t, r, world) for r in range(world)], t.x, t.positions, **kw)["out"]
    assert O.rel_err(out, sim) < 1e-6
    ps.destroy_model_parallel()
    dist.destroy_process_group()


def test_two_rank_gloo_groups_and_distributed_oracle():
    mp.spawn(_gloo_worker, args=(2, 29731, None), nprocs=2)


def _pipeline_worker(rank, world, port, tp, pp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.pipeline_mappings import recv, send
    ps.initialize_model_parallel(tp, pp)
    # the reference's layout (parallel_state.py:147-178): tensor-parallel groups are consecutive ranks, the stages
    # of a pipeline are world / pp apart
    assert ps.get_tensor_model_parallel_world_size() == tp and ps.get_tensor_model_parallel_rank() == rank % tp
    assert ps.get_pipeline_model_parallel_world_size() == pp
    stage = rank // (world // pp)
    assert ps.get_pipeline_model_parallel_rank() == stage
    assert ps.is_pipeline_first_stage() == (stage == 0) and ps.is_pipeline_last_stage() == (stage == pp - 1)
    assert ps.get_pipeline_model_parallel_next_rank() == (rank + world // pp) % world
    assert ps.get_pipeline_model_parallel_prev_rank() == (rank - world // pp) % world
    # hidden states travel down the pipeline, every stage adds its mark (models/llama.py:347-359)
    h = torch.zeros(5, 8)
    if not ps.is_pipeline_first_stage():
        h = recv(h)
        assert torch.equal(h, torch.full((5, 8), float(sum(range(1, stage + 1)))) + (rank % (world // pp)))
    else:
        h = h + (rank % (world // pp))  # pipelines carry different data
    if not ps.is_pipeline_last_stage():
        send(h + (stage + 1))
    ps.destroy_model_parallel()
    assert ps.get_pipeline_model_parallel_world_size() == 1
    dist.destroy_process_group()


def test_pipeline_parallel_groups_and_stage_hand_off_two_stages():
    mp.spawn(_pipeline_worker, args=(2, 29741, 1, 2), nprocs=2)


def test_pipeline_parallel_groups_with_tensor_parallel_pairs():
    mp.spawn(_pipeline_worker, args=(4, 29743, 2, 2), nprocs=4)


def test_single_stage_hand_off_is_a_no_op():
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.pipeline_mappings import recv, send
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    x = torch.ones(2, 3)
    assert send(x) is x and recv(x) is x
    assert ps.is_pipeline_first_stage() and ps.is_pipeline_last_stage()
    ps.destroy_model_parallel()


# --------------------------------------------- host model of the flag protocol
class _Rank:
    """Control words of one rank's heap: per-source flags (written by peers) and local arrival counters."""

    def __init__(self, world):
        self.push_flag = [[0] * world, [0] * world]
        self.done_flag = [[0] * world, [0] * world]
        self.local_push = [0] * world
        self.local_done = 0
        self.epoch = [0, 0]
        self.lock = threading.Lock()


def _wait(get, limit_s):
    t0 = time.perf_counter()
    while not get():
        if time.perf_counter() - t0 > limit_s:
            return False
        time.sleep(0.0005)
    return True


def _run_protocol(world, calls, absent=None, limit_s=0.3, workers=3, one_shot=False):
    """Each rank = `workers` threads (its CTAs) running `calls` collectives with the device protocol:
    a worker counts its arrival per owner locally, the arrival that completes the count stores the
    epoch into the owner's flag; the owner waits for every source's flag, 'reduces', and the last of
    its workers stores the done flag on every rank; everybody waits for every done flag; the last
    worker to leave closes the call (epoch += 1, local counters cleared).  Returns per-rank status."""
    ranks = [_Rank(world) for _ in range(world)]
    status = [0] * world
    barriers = [threading.Barrier(workers) for _ in range(world)]

    def body(r, w):
        me = ranks[r]
        for c in range(calls):
            s = c & 1
            if absent == (r, c):
                return
            epoch = me.epoch[s] + 1
            if one_shot:  # one counter; the arrival that completes it flags every rank
                with me.lock:
                    me.local_push[0] += 1
                    last = me.local_push[0] == workers
                if last:
                    for o in range(world):
                        ranks[o].push_flag[s][r] = epoch
            for o in range(world if not one_shot else 0):  # this worker's share for every owner
                with me.lock:
                    me.local_push[o] += 1
                    last = me.local_push[o] == workers
                if last:
                    ranks[o].push_flag[s][r] = epoch
            ok = _wait(lambda: all(f == epoch for f in me.push_flag[s]), limit_s)
            if not ok:
                status[r] = 2
            with me.lock:  # reduce done: count locally, last worker tells everyone
                me.local_done += 1
                last = me.local_done == workers
            if last and not one_shot:
                for o in range(world):
                    ranks[o].done_flag[s][r] = epoch
            if ok and not one_shot and not _wait(lambda: all(f == epoch for f in me.done_flag[s]), limit_s):
                status[r] = 3
            try:
                if barriers[r].wait(timeout=5) == 0:  # "last CTA": close the call
                    me.epoch[s] = epoch
                    me.local_push = [0] * world
                    me.local_done = 0
                barriers[r].wait(timeout=5)
            except threading.BrokenBarrierError:
                return
            if status[r]:
                return

    th = [threading.Thread(target=body, args=(r, w)) for r in range(world) for w in range(workers)]
    [t.start() for t in th]
    [t.join() for t in th]
    return status


def test_flag_protocol_completes_with_skewed_ranks():
    assert _run_protocol(4, 25) == [0, 0, 0, 0]
    assert _run_protocol(2, 40) == [0, 0]


def test_one_shot_protocol_completes_and_reports_a_lost_rank():
    assert _run_protocol(4, 25, one_shot=True) == [0, 0, 0, 0]
    st = _run_protocol(2, 6, absent=(1, 2), workers=1, one_shot=True)
    assert st[1] == 0 and st[0] == 2


def test_flag_protocol_reports_a_lost_rank_instead_of_hanging():
    st = _run_protocol(4, 6, absent=(2, 3), workers=1)
    assert st[2] == 0  # the absent rank just stops
    assert all(s_ in (2, 3) for i, s_ in enumerate(st) if i != 2), st


# ------------------------------------- host model of the K-range partition of the GEMM scheduler
def _sk_unit_of(W, Gs, x):
    return ((x + 1) * Gs - 1) // W


def _sk_segments(R, KB, Gs, p):
    """Mirror of segment_of() in csrc/gemm_sm100.cuh for the remaining tiles: (tile, kb0, kb1, parts, part, slot)."""
    W = R * KB
    b0, b1 = p * W // Gs, (p + 1) * W // Gs
    out = []
    e = 0
    while True:
        rt = b0 // KB + e
        if rt >= R:
            break
        t0 = rt * KB
        lo, hi = max(b0, t0), min(b1, t0 + KB)
        if lo >= hi:
            break
        pf = _sk_unit_of(W, Gs, rt * KB)
        pl = _sk_unit_of(W, Gs, (rt + 1) * KB - 1)
        out.append((rt, lo - t0, hi - t0, pl - pf + 1, p - pf, p + rt, pf + rt))
        e += 1
    return out


@pytest.mark.parametrize("R,KB,Gs", [(96, 64, 148), (4, 64, 32), (4, 64, 148), (1, 8, 4), (147, 7, 148), (12, 64, 148),
                                     (64, 28, 148), (56, 64, 74), (5, 3, 7), (3, 224, 74), (10, 10, 10)])
def test_k_range_partition_covers_every_k_block_once(R, KB, Gs):
    cover = {}
    slots = set()
    for p in range(Gs):
        segs = _sk_segments(R, KB, Gs, p)
        assert 1 <= len(segs) <= 2
        for rt, k0, k1, parts, part, slot, first_slot in segs:
            assert 0 <= part < parts and slot == first_slot + part
            assert slot not in slots and slot < Gs + R
            slots.add(slot)
            for k in range(k0, k1):
                assert (rt, k) not in cover
                cover[(rt, k)] = (p, parts)
    assert len(cover) == R * KB
    for rt in range(R):  # the units of a tile are consecutive and agree on how many they are
        units = sorted({cover[(rt, k)][0] for k in range(KB)})
        assert units == list(range(units[0], units[0] + len(units)))
        assert {cover[(rt, k)][1] for k in range(KB)} == {len(units)}


# --------------------------------------------------------- tile planner (host-only entry point)
@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_planner_gives_valid_schedules_for_the_layer_shapes(tp):
    """sb200_gemm_plan needs no GPU (148 SMs assumed): the schedules it returns for the four projections of
    the headline layer are self-consistent."""
    from sarathi_serve_b200 import dense_ops as D
    H, I, T = 4096, 14336, 512
    shapes = (("qkv", 1, 6144 // tp, H), ("o_proj", 3, H, 4096 // tp), ("gate_up", 2, 2 * I // tp, H),
              ("down", 3, H, I // tp))
    for name, epi, N, K in shapes:
        for cfg in (0, 3256, 203256, 1128, 301128):
            try:
                p = D.gemm_plan(epi, T, N, K, tile_cfg=cfg)
            except RuntimeError:
                continue  # a forced configuration may not exist for a shape
            bm = (256 if p["cta_pairs"] else 128) * p["accumulators"]
            cols = p["bn"] // 2 if epi == 2 else p["bn"]
            out_cols = N // 2 if epi == 2 else N
            assert p["m_tiles"] == -(-T // bm) and p["n_tiles"] == -(-out_cols // cols), (name, cfg, p)
            assert p["k_blocks"] == -(-K // 64)
            tiles = p["m_tiles"] * p["n_tiles"]
            units_max = 74 if p["cta_pairs"] else 148
            assert 1 <= p["units"] <= units_max
            assert p["tiles_full"] % p["units"] == 0 and p["tiles_full"] <= tiles
            rem = tiles - p["tiles_full"]
            assert rem < units_max or p["tiles_full"] == 0
            if rem:
                assert rem <= p["rem_units"] <= p["units"], (name, cfg, p)
                assert p["rem_units"] <= rem * p["k_blocks"]  # at least one k-block per unit
            assert 2 <= p["stages"] <= 8


def test_planner_rules_for_the_cluster_k_split():
    """Tile mode 5 (a cluster of S CTA pairs per tile): one cluster per tile, at least S k-blocks, room for the
    exchanged accumulator shares in the stage ring; with the row-parallel epilogue, whose CTAs wait for one another,
    only two pairs per cluster and only as many clusters as can be resident together."""
    from sarathi_serve_b200 import dense_ops as D
    p = D.gemm_plan(0, 512, 768, 4096, tile_cfg=405128)
    assert p["cluster_split"] == 4 and p["cta_pairs"] == 1 and p["units"] == p["tiles_full"] == 12 and p["rem_units"] == 0
    p = D.gemm_plan(0, 288, 1024, 704, tile_cfg=205256)
    assert p["cluster_split"] == 2 and p["units"] == 8
    with pytest.raises(RuntimeError):
        D.gemm_plan(0, 512, 4096, 64, tile_cfg=205256)      # one k-block cannot be split
    with pytest.raises(RuntimeError):
        D.gemm_plan(0, 2048, 4096, 4096, tile_cfg=205256)   # 128 tiles x 4 CTAs do not fit the GPU
    with pytest.raises(RuntimeError):
        D.gemm_plan(1, 512, 6144, 4096, 128, tile_cfg=205256)  # 48 tiles x 4 CTAs do not fit either
    assert D.gemm_plan(3, 288, 1024, 704, tile_cfg=205256)["cluster_split"] == 2
    with pytest.raises(RuntimeError):
        D.gemm_plan(3, 288, 1024, 704, tile_cfg=405128)     # row-parallel epilogue: two pairs only


def test_tuned_configuration_cache_round_trip(tmp_path):
    from sarathi_serve_b200 import dense_ops as D
    saved = dict(D._tuned)
    try:
        D._tuned.clear()
        D._tuned[("silu", 512, 28672, 4096, torch.bfloat16)] = 303256
        D._tuned[("push", 512, 4096, 2048, torch.float16)] = 101128
        path = str(tmp_path / "tuned.json")
        D.save_tuned(path)
        D._tuned.clear()
        assert D.load_tuned(path) == 2
        assert D.tuned_cfg("silu", 512, 28672, 4096, torch.bfloat16) == 303256
        assert D.tuned_cfg("push", 512, 4096, 2048, torch.float16) == 101128
        assert D.tuned_cfg("push", 512, 4096, 2048, torch.bfloat16) == 0  # unknown problem: library default
    finally:
        D._tuned.clear()
        D._tuned.update(saved)


def test_vocab_parallel_embedding_api_surface_on_cpu():
    """Constructor keywords, attributes and the weight shard shape of the reference (layers.py:72-145)."""
    from sarathi_serve_b200.tp_layers import VocabParallelEmbedding
    emb = VocabParallelEmbedding(128256, 64, params_dtype=torch.bfloat16, linear_metric_name="x",
                                 communication_metric_name="y", reduce_results=True, world_size=8, rank=3)
    assert emb.num_embeddings == 128256 and emb.embedding_dim == 64
    assert emb.tensor_model_parallel_size == 8 and emb.rank == 3
    assert (emb.vocab_start_index, emb.vocab_end_index) == (3 * 16032, 4 * 16032)
    assert emb.num_embeddings_per_partition == 16032 and emb.weight.shape == (16032, 64)
    assert emb.weight.dtype == torch.bfloat16 and not emb.weight.requires_grad
    with pytest.raises(AssertionError):
        VocabParallelEmbedding(100, 8, world_size=3, rank=0)  # the vocabulary must divide evenly


# ------------------------- arrivals the row-parallel kernel reports vs what the host tells it to expect
def _model_arrivals(p, T, lo, hi):
    """What the device does (csrc/gemm_sm100.cuh, epilogue of EPI_PUSH): for every tile and every group of 32
    rows of it that holds a valid row, the epilogue warps that drain those rows (two per group with one
    accumulator, one with two) report once per owner whose rows the group overlaps -- once per part for a
    tile that is cut along K, because every part finishes a share of it."""
    bm = (256 if p["cta_pairs"] else 128) * p["accumulators"]
    warps_per_group = 2 if p["accumulators"] == 1 else 1
    tiles = p["m_tiles"] * p["n_tiles"]
    rem = tiles - p["tiles_full"]
    total = 0
    for tile in range(tiles):
        mt = tile % p["m_tiles"]
        parts = 1
        if tile >= p["tiles_full"]:
            rt, KB, Gs = tile - p["tiles_full"], p["k_blocks"], p["rem_units"]
            W = rem * KB
            parts = _sk_unit_of(W, Gs, (rt + 1) * KB - 1) - _sk_unit_of(W, Gs, rt * KB) + 1
        for g0 in range(mt * bm, min(T, mt * bm + bm), 32):
            g1 = min(T, g0 + 32)
            if g0 < hi and g1 > lo:
                total += warps_per_group * parts
    return total


@pytest.mark.parametrize("T,N,K", [(512, 4096, 4096), (512, 4096, 1792), (65, 256, 64), (1, 128, 512), (130, 4096, 7168),
                                   (300, 1024, 704), (96, 8192, 256)])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_expected_arrivals_match_the_kernels_reporting_rule(T, N, K, world):
    from sarathi_serve_b200 import _native as N_, dense_ops as D
    ws = 64 << 20
    rpr = -(-T // world)
    for cfg in (0, 128, 2256, 302128, 3256, 203256, 4256, 803128):
        try:
            p = D.gemm_plan(3, T, N, K, tile_cfg=cfg, workspace_bytes=ws)
        except RuntimeError:
            continue
        for o in range(world):
            lo, hi = o * rpr, min(T, o * rpr + rpr)
            got = N_.lib().sb200_gemm_rowpar_arrivals(T, N, K, cfg, ws, lo, hi)
            want = _model_arrivals(p, T, lo, hi) if hi > lo else 0
            assert got == want, (cfg, o, p)
        # one-shot calls count every finished (tile, 32-row group, part) once
        assert N_.lib().sb200_gemm_rowpar_arrivals(T, N, K, cfg, ws, 0, T) == _model_arrivals(p, T, 0, T)


def test_model_stack_api_surface_on_cpu():
    """LlamaModel / LlamaForCausalLM keep the reference's module tree and parameter names
    (models/llama.py:258-345), so its weight loader addresses the same state-dict keys."""
    from types import SimpleNamespace
    from sarathi_serve_b200 import parallel_state as ps
    from sarathi_serve_b200.decoder_layer import LlamaForCausalLM
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1)
    try:
        cfg = SimpleNamespace(hidden_size=128, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
                              rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, max_position_embeddings=64,
                              hidden_act="silu", num_hidden_layers=2, vocab_size=1000, pad_token_id=None)
        lm = LlamaForCausalLM(cfg)
        keys = set(lm.state_dict().keys())
        for k in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight",
                  "model.layers.0.self_attn.qkv_proj.weight", "model.layers.1.self_attn.o_proj.weight",
                  "model.layers.0.mlp.gate_up_proj.weight", "model.layers.1.mlp.down_proj.weight",
                  "model.layers.0.input_layernorm.weight", "model.layers.1.post_attention_layernorm.weight"):
            assert k in keys, k
        assert lm.model.embed_tokens.weight.shape == (1024, 128)  # vocabulary padded to a multiple of 64
        assert lm.lm_head.weight.shape == (1024, 128) and lm.lm_head.bias is None
    finally:
        ps.destroy_model_parallel()


def test_prepare_inputs_lays_a_mixed_batch_out_like_the_reference():
    """Prefill chunks first (positions continue where the prompt stopped), then one token per decoding request at
    position context_len - 1, then zeros up to a multiple of 8 (sarathi/model_executor/model_runner.py:67-117)."""
    from sarathi_serve_b200.model_runner import pad_to_alignment, prepare_inputs
    tok, pos, n = prepare_inputs([([5, 6, 7], 0), ([9], 4)], [(21, 100)], "cpu")
    assert n == 5 and tok.dtype == torch.long and pos.dtype == torch.long
    assert tok.tolist() == [5, 6, 7, 9, 21, 0, 0, 0] and pos.tolist() == [0, 1, 2, 4, 99, 0, 0, 0]
    tok, pos, n = prepare_inputs([], [(1, 1)] * 8, "cpu")
    assert n == 8 and tok.numel() == 8 and pos.tolist() == [0] * 8
    assert pad_to_alignment([], 8) == [] and len(pad_to_alignment([1] * 9, 8)) == 16
    tok, pos, n = prepare_inputs([], [], "cpu")
    assert n == 0 and tok.numel() == 0
