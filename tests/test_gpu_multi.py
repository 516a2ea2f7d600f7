"""Multi-GPU parity (2, 4 and 8 GPUs, as many as the box has): the standalone all-reduce,
the fused row-parallel GEMM + all-reduce (+bias, +residual, +RMSNorm) and the
whole tensor-parallel decoder layer, one process per GPU, against torch sums and
the CPU oracle.  torch.distributed (gloo) carries only the IPC handles and host
barriers.  Also: a rank that does not join a collective makes the peer's bounded
device-side wait run out and report SB200_ERR_PEER_TIMEOUT instead of hanging."""
import os
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

WORLDS = (2, 4, 8)


def _need_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


def _rel(a, ref):
    d = float(ref.double().abs().max())
    return float((a.double().cpu() - ref.double().cpu()).abs().max()) / (d if d > 0 else 1.0)


def _host_barrier():
    """The ranks prepare their inputs on the host at different speeds (seconds apart for the large cases); the
    device-side waits are bounded, so the ranks meet here before they launch collectives."""
    import torch.distributed as dist
    torch.cuda.synchronize()
    dist.barrier()


def _entry(rank, world, port, fn_name, ret, nvls):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["SB200_NVLS"] = "1" if nvls else "0"  # heaps bound to an NVSwitch multicast range, or plain peer mappings
        # a wait on a peer that cannot succeed ends after about a second (the library's default is ten): a protocol
        # error then fails the test quickly instead of stalling every following collective for long
        os.environ.setdefault("SB200_WAIT_LIMIT_CYCLES", "3000000000")
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        import datetime
        # a rank that fails leaves the others in a host barrier: it gives up after a minute and a half
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=90))
        from sarathi_serve_b200 import parallel_state as ps
        ps.initialize_model_parallel(world)
        try:
            globals()[fn_name](rank, world)
            torch.cuda.synchronize()
            dist.barrier()  # nobody unbinds its heap while a peer's kernels may still touch it
            mc = ps._TP_COMM is not None and ps._TP_COMM.multicast
        finally:
            ps.destroy_model_parallel()
            dist.destroy_process_group()
        ret[rank] = "ok" if (mc or not nvls) else "ok-without-multicast"
    except Exception:  # report the traceback to the parent instead of a bare exit code
        ret[rank] = traceback.format_exc()


def _run(fn_name, port, world, nvls=True):
    _need_gpus(world)
    port += 10 * world + (100 if nvls else 0)
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn_name, ret, nvls)) for r in range(world)]
    [p.start() for p in procs]
    import time
    deadline = time.time() + 240
    [p.join(timeout=max(1.0, deadline - time.time())) for p in procs]
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail(f"{fn_name}: a rank did not finish within the time limit")
    if nvls and all(ret.get(r) == "ok-without-multicast" for r in range(world)):
        pytest.skip("the heaps could not be bound to an NVSwitch multicast range on this box: this run repeated the "
                    "peer-mapping variant")
    bad = {r: ret.get(r) for r in range(world) if ret.get(r) != "ok"}
    if bad:  # the children's tracebacks, in full, on stdout as well (the assertion message gets truncated)
        for r, text in bad.items():
            print(f"---- {fn_name} world={world} rank {r} ----\n{text}", flush=True)
    assert not bad, f"{fn_name} world={world}: ranks {sorted(bad)} failed; first: {next(iter(bad.values()))}"


# ------------------------------------------------------------------ bodies
def _body_all_reduce(rank, world):
    from sarathi_serve_b200 import parallel_state as ps
    comm = ps.get_tensor_model_parallel_comm(64 << 20)
    for dtype, tol, one_shot in ((torch.bfloat16, 1e-2, None), (torch.bfloat16, 1e-2, 0), (torch.float32, 1e-5, None),
                                 (torch.float16, 2e-3, None), (torch.float16, 2e-3, 1 << 30)):
        if world > 2 and dtype == torch.float16:
            continue  # larger groups: a reduced set keeps the multi-GPU run short
        # both schemes whatever the size: None = the library's threshold, 0 = never one-shot, 1 GiB = always
        comm.set_one_shot_bytes((4 << 20) if one_shot is None else one_shot)
        for T, H in ((512, 4096), (288, 1024), (7, 256), (1, 64), (65, 8192)):
            g = torch.Generator().manual_seed(T * 7 + H)
            parts = [torch.randn(T, H, generator=g).to(dtype) for _ in range(world)]
            bias = torch.randn(H, generator=g).to(dtype)
            resid = torch.randn(T, H, generator=g).to(dtype)
            w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
            x = parts[rank].cuda()
            total = sum(p.float() for p in parts)
            _host_barrier()
            # plain sum, result in a heap view
            y, z = comm.all_reduce(x)
            assert z is None and _rel(y, total) <= tol, ("sum", dtype, T, H)
            # in place (reduce_from_tensor_model_parallel_region semantics)
            from sarathi_serve_b200.mappings import reduce_from_tensor_model_parallel_region
            xin = x.clone()
            out = reduce_from_tensor_model_parallel_region(xin)
            assert out is xin and _rel(xin, total) <= tol
            # bias + residual + norm; both results copied to caller tensors
            yo, zo = torch.empty_like(x), torch.empty_like(x)
            y2, z2 = comm.all_reduce(x, bias=bias.cuda(), residual=resid.cuda(), norm_weight=w.cuda(), eps=1e-5,
                                     out=yo, resid_out=zo)
            zref = (resid.float() + (total.to(dtype).float() + bias.float()).to(dtype).float()).to(dtype)
            zf = zref.float()
            yref = ((zf * torch.rsqrt(zf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dtype) * w)
            # (the in-switch reduction of the multicast scheme rounds the fp32 sum to the 16-bit type with its own
            #  tie rule: about 5e-5 of the sums differ from round-to-nearest-even by one unit in the last place,
            #  which the bias and residual adds can carry to two units -- the bound is twice the plain sum's)
            assert _rel(z2, zref) <= max(tol, 1e-4) * 2, ("z", dtype, T, H)
            assert _rel(y2, yref) <= max(tol, 1e-4) * 2, ("y", dtype, T, H)
            # heap views of the same call agree with the copies
            y3, z3 = comm.all_reduce(x, bias=bias.cuda(), residual=resid.cuda(), norm_weight=w.cuda(), eps=1e-5)
            assert torch.equal(y3, yo) and torch.equal(z3, zo)
    comm.check_status()


def _body_rowpar(rank, world):
    from sarathi_serve_b200 import parallel_state as ps
    comm = ps.get_tensor_model_parallel_comm(64 << 20)
    for dtype, tol, one_shot in ((torch.bfloat16, 1e-2, 4 << 20), (torch.bfloat16, 1e-2, 0), (torch.float16, 2e-3, 1 << 30),
                                 (torch.float32, 2e-5, 4 << 20)):
        comm.set_one_shot_bytes(one_shot)  # the library's threshold / never one-shot / always one-shot
        for T, H, K in ((512, 4096, 1024), (288, 1024, 704), (65, 256, 64), (1, 128, 512), (130, 4096, 7168), (96, 8192, 256)):
            for tile_n in (0, 128, 2256, 302128, 3256, 203128, 4256, 204128, 205256, 405128):
                if dtype == torch.float32 and tile_n != 0:
                    continue
                if world > 2 and (dtype == torch.float16 or tile_n not in (0, 302128, 3256, 203128, 205256)):
                    continue  # larger groups: a reduced set keeps the multi-GPU run short
                if tile_n // 100000 > (K + 63) // 64:
                    continue
                if (tile_n // 1000) % 100 == 5:  # cluster K-split: only problems with one cluster per tile
                    from sarathi_serve_b200 import dense_ops
                    try:
                        dense_ops.gemm_plan(3, T, H, K, 128, tile_n)
                    except RuntimeError:
                        continue
                g = torch.Generator().manual_seed(T + H + K)
                X = torch.randn(T, K * world, generator=g).to(dtype)
                W = (torch.randn(H, K * world, generator=g) * 0.05).to(dtype)
                resid = torch.randn(T, H, generator=g).to(dtype)
                nw = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
                x = X[:, rank * K:(rank + 1) * K].contiguous().cuda()
                w = W[:, rank * K:(rank + 1) * K].contiguous().cuda()
                ref = sum((X[:, r * K:(r + 1) * K].float().cuda() @ W[:, r * K:(r + 1) * K].float().cuda().t())
                          for r in range(world)).cpu()
                _host_barrier()
                y, _ = comm.rowpar_linear(x, w, tile_n=tile_n)
                assert _rel(y, ref) <= tol, ("plain", dtype, T, H, K, tile_n)
                y, z = comm.rowpar_linear(x, w, residual=resid.cuda(), norm_weight=nw.cuda(), eps=1e-5, tile_n=tile_n)
                zref = (resid.float() + ref.to(dtype).float()).to(dtype)
                zf = zref.float()
                yref = (zf * torch.rsqrt(zf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dtype) * nw
                assert _rel(z, zref) <= tol * 2 and _rel(y, yref) <= tol * 2, ("fused", dtype, T, H, K, tile_n)
                try:  # a wait that ran out is reported with the configuration it happened in
                    comm.check_status()
                except RuntimeError as e:
                    raise AssertionError(f"status after {(dtype, one_shot, T, H, K, tile_n)}: {e}") from e
    comm.check_status()


def _body_layer(rank, world):
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import parallel_state as ps, synthetic as S
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer
    from helpers import TOL, load_golden

    class QAttention:
        def forward(self, q, k, v, idx, scale=1.0, layer_id=None):
            return q

    for case_name in ("mini_f32", "mini_bf16", "mini_f16", "config1", "config2"):
        case = S.CASES[case_name]
        if case.num_kv_heads % world or case.intermediate_size % world:
            continue  # the reference shards whole kv heads (tensor_parallel/layers.py): this case does not split that far
        old = torch.get_default_dtype()
        torch.set_default_dtype(case.dtype)
        try:
            layer = LlamaDecoderLayer(case.hf_config(), layer_id=0)
        finally:
            torch.set_default_dtype(old)
        t = S.generate(case)
        S.load_layer(layer, S.shard(t, rank, world))
        x = t.x.to(case.dtype).cuda()
        _host_barrier()
        with torch.inference_mode():
            out = layer(t.positions.cuda(), x.clone(), 0, QAttention())
            out_u = layer.forward_unfused(t.positions.cuda(), x.clone(), 0, QAttention())
        ps.get_tensor_model_parallel_comm().check_status()
        if rank == 0 or (case_name != "config2" and world == 2):
            cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
            ref = O.decoder_layer([S.shard(t, r, world) for r in range(world)], t.x.to(case.dtype), t.positions,
                                  num_heads=case.num_heads, num_kv_heads=case.num_kv_heads, head_dim=case.head_dim,
                                  eps=case.rms_norm_eps, cache=cache)["out"]
            assert _rel(out, ref) <= TOL[case.dtype], (case_name, "fused")
            assert _rel(out_u, ref) <= TOL[case.dtype], (case_name, "unfused")
        if case_name != "config2" and world == 2:
            gold, _, step, _ = load_golden(case_name, 2)
            assert _rel(out[::step], gold["out"]) <= TOL[case.dtype], (case_name, "fixture")


def _body_carry(rank, world):
    """Two layers chained through forward_carry with the residual stream kept sharded by rows, under both
    all-reduce schemes, against two oracle layers."""
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import parallel_state as ps, synthetic as S
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer
    from helpers import TOL

    class QAttention:
        def forward(self, q, k, v, idx, scale=1.0, layer_id=None):
            return q

    case = S.CASES["mini_bf16" if world <= 2 else "mini8_bf16"]  # (kv heads must divide over the ranks)
    old = torch.get_default_dtype()
    torch.set_default_dtype(case.dtype)
    try:
        layers = [LlamaDecoderLayer(case.hf_config(), layer_id=i) for i in range(2)]
    finally:
        torch.set_default_dtype(old)
    t = S.generate(case)
    for l in layers:
        S.load_layer(l, S.shard(t, rank, world))
    x = t.x.to(case.dtype).cuda()
    pos = t.positions.cuda()
    shards = [S.shard(t, r, world) for r in range(world)]
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    kw = dict(num_heads=case.num_heads, num_kv_heads=case.num_kv_heads, head_dim=case.head_dim, eps=case.rms_norm_eps,
              cache=cache)
    ref1 = O.decoder_layer(shards, t.x.to(case.dtype), t.positions, **kw)
    ref2 = O.decoder_layer(shards, ref1["out"], t.positions, next_norm_weight=t.ln1.to(case.dtype), **kw)
    comm = ps.get_tensor_model_parallel_comm()
    T = case.num_tokens
    rpr = -(-T // world)
    lo, hi = rank * rpr, min(T, rank * rpr + rpr)
    for one_shot in (4 << 20, 0):
        comm.set_one_shot_bytes(one_shot)
        _host_barrier()
        with torch.inference_mode():
            normed = layers[0].input_layernorm(x)
            y1, z1 = layers[0].forward_carry(pos, normed, x, 0, QAttention(), layers[1].input_layernorm, shard_residual=True)
            y2, z2 = layers[1].forward_carry(pos, y1, z1, 0, QAttention(), layers[0].input_layernorm, shard_residual=True)
        comm.check_status()
        assert _rel(y2, ref2["out_normed"]) <= TOL[case.dtype] * 1.5, ("normed", one_shot)
        assert _rel(z2[lo:hi], ref2["out"][lo:hi]) <= TOL[case.dtype] * 1.5, ("own rows of the residual", one_shot)


def _body_embedding(rank, world):
    """VocabParallelEmbedding: each rank's masked lookup summed by the all-reduce = the full-table lookup."""
    from sarathi_serve_b200.tp_layers import VocabParallelEmbedding
    for dtype in (torch.bfloat16, torch.float32):
        V, H = 1024, 512
        g = torch.Generator().manual_seed(9)
        table = torch.randn(V, H, generator=g).to(dtype)
        emb = VocabParallelEmbedding(V, H, params_dtype=dtype)
        emb.weight.data.copy_(table[emb.vocab_start_index:emb.vocab_end_index])
        for shape in ((300,), (5, 13), (1,)):
            ids = torch.randint(0, V, shape, generator=g)
            _host_barrier()
            out = emb(ids.cuda())
            assert out.shape == (*shape, H) and torch.equal(out.cpu(), table[ids]), (dtype, shape)


def _body_moe(rank, world):
    """Tensor-parallel MoE block: experts sharded along the intermediate dimension, k-slot sum fused
    into the all-reduce."""
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import parallel_state as ps, synthetic as S
    from sarathi_serve_b200.decoder_layer import MixtralMoE
    for case_name in ("mini_moe", "config5"):
        case = S.MOE_CASES[case_name]
        if case.intermediate_size % world:
            continue
        if case_name == "config5" and world > 2:
            continue  # the CPU oracle of the full-size block takes minutes; its shard shapes run at world 2
        if case_name == "config5":  # a slice of the 8-way sharded experts keeps the CPU oracle affordable
            shards = [S.generate_moe(case, world=8, rank=r) for r in range(world)]
        else:
            shards = [S.generate_moe(case, world=world, rank=r) for r in range(world)]
        g = torch.Generator().manual_seed(5)
        gate_w = (torch.randn(case.num_experts, case.hidden_size, generator=g) * 0.05).to(case.dtype)
        old = torch.get_default_dtype()
        torch.set_default_dtype(case.dtype)
        try:
            moe = MixtralMoE(case.num_experts, case.top_k, case.hidden_size,
                             shards[0]["w2"].shape[2] * world)
        finally:
            torch.set_default_dtype(old)
        sd = moe.state_dict()
        with torch.no_grad():
            sd["gate.weight"].copy_(gate_w)
            sd["experts.w13_weight"].copy_(shards[rank]["w13"])
            sd["experts.w2_weight"].copy_(shards[rank]["w2"])
        x = shards[0]["x"]
        _host_barrier()
        out = moe(x.cuda().clone())
        ps.get_tensor_model_parallel_comm().check_status()
        if rank == 0:
            ref = O.moe_layer(x, gate_w, [s_["w13"] for s_ in shards], [s_["w2"] for s_ in shards], case.top_k)
            assert _rel(out, ref) <= 2e-2, case_name


def _body_lost_peer(rank, world):
    """Rank 1 sits one collective out; rank 0's wait is bounded and reports a timeout."""
    import torch.distributed as dist
    from sarathi_serve_b200 import parallel_state as ps
    comm = ps.get_tensor_model_parallel_comm(16 << 20)
    x = torch.ones(64, 256, dtype=torch.bfloat16, device="cuda")
    y, _ = comm.all_reduce(x)
    torch.cuda.synchronize()
    assert float(y[0, 0]) == world
    dist.barrier()
    if rank == 0:
        comm.set_wait_limit_cycles(400_000_000)  # ~0.2 s
        comm.all_reduce(x)  # nobody else joins this one
        with pytest.raises(RuntimeError, match="timed out"):
            comm.check_status()
        assert comm.status_code() == 0  # cleared by check_status
        with pytest.raises(RuntimeError, match="out of step"):
            comm.all_reduce(x)  # the context refuses further collectives until it is reset
    dist.barrier()  # rank 1 was idle on the host the whole time: nothing of it was in flight
    comm.reset()  # collective: control words back to their initial state on every rank
    y, _ = comm.all_reduce(x)
    torch.cuda.synchronize()
    assert float(y[0, 0]) == world
    comm.check_status()


def _body_graph_odd(rank, world):
    """A CUDA graph that holds ONE collective, replayed three times in a row, then an eager call, then the
    graph again: the buffers and flags a call uses alternate with a counter kept on the device, so an odd
    number of collectives per replay must neither corrupt a peer's reads nor stall."""
    from sarathi_serve_b200 import parallel_state as ps
    comm = ps.get_tensor_model_parallel_comm(16 << 20)
    T, H = 256, 2048
    for one_shot in (4 << 20, 0):
        comm.set_one_shot_bytes(one_shot)
        g = torch.Generator().manual_seed(11 + one_shot % 7)
        parts = [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(world)]
        x = parts[rank].cuda()
        xs = x.clone()
        out = torch.empty_like(x)
        comm.all_reduce(xs, out=out)
        _host_barrier()
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(st):
            with torch.cuda.graph(graph, stream=st):
                comm.all_reduce(xs, out=out)
        torch.cuda.current_stream().wait_stream(st)
        for rep in range(7):
            scale = float(rep + 1)
            xs.copy_(x * scale)
            if rep == 4:
                y, _ = comm.all_reduce(xs)  # an eager call between replays
                res = y.clone()
            else:
                graph.replay()
                res = out.clone()
            total = sum((p * scale).to(torch.bfloat16).float() for p in parts)
            assert _rel(res, total) <= 1e-2, (one_shot, rep)
    comm.check_status()


def _body_all_gather(rank, world):
    """All-gather of row blocks: every rank contributes its rows, every rank ends up with all of them --
    exact copies -- also for batches with fewer rows than ranks and for ragged last blocks."""
    from sarathi_serve_b200 import parallel_state as ps
    comm = ps.get_tensor_model_parallel_comm(16 << 20)
    for dtype in (torch.bfloat16, torch.float32):
        for T, H in ((512, 4096), (65, 1024), (7, 256), (1, 64), (world, 128)):
            g = torch.Generator().manual_seed(T + H)
            full = torch.randn(T, H, generator=g).to(dtype)
            rpr = -(-T // world)
            lo, hi = min(T, rank * rpr), min(T, rank * rpr + rpr)
            rows = full[lo:hi].contiguous().cuda()
            _host_barrier()
            y = comm.all_gather_rows(rows, T)
            assert torch.equal(y.cpu(), full), ("heap view", dtype, T, H)
            out = torch.empty(T, H, dtype=dtype, device="cuda")
            y2 = comm.all_gather_rows(rows, T, out=out)
            assert y2 is out and torch.equal(out.cpu(), full), ("caller tensor", dtype, T, H)
            # interleaved with a sum: the two kinds of collective share the flags and the call counter
            s_, _ = comm.all_reduce(out)
            assert _rel(s_, full.float() * world) <= 1e-2
    # gather_from_tensor_model_parallel_region: shards concatenated along the LAST dimension (the logits gather of
    # the sampler, layers/sampler.py:89-97), through the same kernel
    from sarathi_serve_b200.mappings import gather_from_tensor_model_parallel_region
    for shape in ((13, 16032), (5, 3, 64), (1, 8)):
        g = torch.Generator().manual_seed(sum(shape))
        shards = [torch.randn(*shape, generator=g).to(torch.bfloat16) for _ in range(world)]
        _host_barrier()
        got = gather_from_tensor_model_parallel_region(shards[rank].cuda())
        assert torch.equal(got.cpu(), torch.cat(shards, dim=-1)), shape
    comm.check_status()


def _body_graph_io(rank, world):
    """LayerGraph with host buffers sharded by token rows: upload this rank's rows, all-gather inside the graph,
    the layer, download this rank's rows of the result; replayed with fresh inputs."""
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import parallel_state as ps, synthetic as S
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer
    from sarathi_serve_b200.graph_runner import LayerGraph
    from helpers import TOL

    class QAttention:
        def forward(self, q, k, v, idx, scale=1.0, layer_id=None):
            return q

    case = S.CASES["mini_bf16" if world <= 2 else "mini8_bf16"]  # (kv heads must divide over the ranks)
    old = torch.get_default_dtype()
    torch.set_default_dtype(case.dtype)
    try:
        layer = LlamaDecoderLayer(case.hf_config(), layer_id=0)
    finally:
        torch.set_default_dtype(old)
    t = S.generate(case)
    S.load_layer(layer, S.shard(t, rank, world))
    _host_barrier()
    runner = LayerGraph(layer, case.num_tokens, QAttention(), host_io=True, shard_host_io=True)
    lo, hi = runner.row_range
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    shards = [S.shard(t, r, world) for r in range(world)]
    for rep in range(3):
        x = (t.x * (1.0 + 0.25 * rep)).to(case.dtype)
        runner.host_positions.copy_(t.positions)
        runner.host_hidden_states.copy_(x[lo:hi])
        _host_barrier()
        out = runner.replay_host_io()
        torch.cuda.current_stream().synchronize()
        ref = O.decoder_layer(shards, x, t.positions, num_heads=case.num_heads, num_kv_heads=case.num_kv_heads,
                              head_dim=case.head_dim, eps=case.rms_norm_eps, cache=cache)["out"]
        err = float((out.double() - ref[lo:hi].double()).abs().max()) / float(ref.double().abs().max())
        assert err <= TOL[case.dtype], (rep, err)
    ps.get_tensor_model_parallel_comm().check_status()
    # the same through HostPipeline: three steps in flight, copies on their own streams, kernels on one
    from sarathi_serve_b200.graph_runner import HostPipeline
    slots = [LayerGraph(layer, case.num_tokens, QAttention(), host_io=True, shard_host_io=True, copies_in_graph=False)
             for _ in range(3)]
    pipe = HostPipeline(slots)
    xs = [(t.x * (1.0 - 0.2 * rep)).to(case.dtype) for rep in range(5)]
    got = []
    _host_barrier()
    for x in xs:
        g = pipe.next_slot()
        g.host_positions.copy_(t.positions)
        g.host_hidden_states.copy_(x[lo:hi])
        pipe.submit()
        if pipe.in_flight >= 3:
            got.append(pipe.collect().clone())
    while pipe.in_flight:
        got.append(pipe.collect().clone())
    for rep, (x, out) in enumerate(zip(xs, got)):
        ref = O.decoder_layer(shards, x, t.positions, num_heads=case.num_heads, num_kv_heads=case.num_kv_heads,
                              head_dim=case.head_dim, eps=case.rms_norm_eps, cache=cache)["out"]
        err = float((out.double() - ref[lo:hi].double()).abs().max()) / float(ref.double().abs().max())
        assert err <= TOL[case.dtype], ("pipelined", rep, err)
    ps.get_tensor_model_parallel_comm().check_status()


# -------------------------------------------------------------------- tests
SCHEMES = pytest.mark.parametrize("nvls", (False, True), ids=("peer-loads", "nvls"))


@SCHEMES
@pytest.mark.parametrize("world", WORLDS)
def test_all_reduce_multi_gpu(world, nvls):
    _run("_body_all_reduce", 29801, world, nvls)


@SCHEMES
@pytest.mark.parametrize("world", WORLDS)
def test_rowpar_linear_multi_gpu(world, nvls):
    _run("_body_rowpar", 29802, world, nvls)


@SCHEMES
@pytest.mark.parametrize("world", WORLDS)
def test_decoder_layer_multi_gpu(world, nvls):
    _run("_body_layer", 29803, world, nvls)


@SCHEMES
@pytest.mark.parametrize("world", WORLDS)
def test_layer_stack_with_sharded_residual_multi_gpu(world, nvls):
    _run("_body_carry", 29806, world, nvls)


@SCHEMES
@pytest.mark.parametrize("world", (2, 4))
def test_graph_with_an_odd_number_of_collectives_replays(world, nvls):
    _run("_body_graph_odd", 29808, world, nvls)


@SCHEMES
@pytest.mark.parametrize("world", WORLDS)
def test_all_gather_rows_multi_gpu(world, nvls):
    _run("_body_all_gather", 29809, world, nvls)


@SCHEMES
@pytest.mark.parametrize("world", (2, 8))
def test_layer_graph_with_row_sharded_host_buffers(world, nvls):
    _run("_body_graph_io", 29810, world, nvls)


@pytest.mark.parametrize("world", WORLDS)
def test_vocab_parallel_embedding_multi_gpu(world):
    _run("_body_embedding", 29807, world)


@pytest.mark.parametrize("world", WORLDS)
def test_moe_block_multi_gpu(world):
    _run("_body_moe", 29805, world)


@pytest.mark.parametrize("world", (2, 4))
def test_lost_peer_reports_timeout(world):
    # peer mappings only: a rank must not leave while its memory is bound to a multicast object
    _run("_body_lost_peer", 29804, world, nvls=False)
