"""Worker of the multi-GPU tests: one process per GPU (torch.distributed.run), NCCL for bootstrap only.

Checks, on every rank, against the CPU oracle:
  1. plain peer-memory all-reduce (one-shot and two-shot, staged and registered input) on several sizes;
  2. the fused k-slot-sum + all-reduce;
  3. the whole tensor-parallel MoE block (I sharded as the reference's weight_loader does);
  4. a graph-captured all-reduce; 5. the all-reduce that ends in the next layer's add + RMSNorm, also behind
     the row-parallel linear (o_proj).
Prints "TP_WORKER_OK rank=<r>" on success; any failure raises.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from layered_prefill_b200 import fused_moe, ops
    from layered_prefill_b200.custom_all_reduce import CustomAllreduce
    from layered_prefill_b200.layer import FusedMoE
    from oracle import moe_oracle as O

    comm = CustomAllreduce(group=dist.new_group(backend="gloo"), device=dev)
    assert not comm.disabled, "peer-memory all-reduce did not initialise"

    # ---- 1. plain all-reduce
    for numel in (8, 2048, 64 * 2048, 256 * 2048 + 8, 3 * 1024 * 1024):
        for dtype in (torch.bfloat16, torch.float32):
            for algo in (1, 2):
                parts = []
                for r in range(world):
                    g = torch.Generator().manual_seed(numel + 17 * r)
                    parts.append(torch.randn(numel, generator=g).to(dtype))
                want = O.all_reduce(parts)
                mine = parts[rank].to(dev)
                out = comm.all_reduce(mine, registered=False, algo=algo)
                torch.cuda.synchronize()
                assert torch.equal(out.cpu(), want), f"all_reduce numel={numel} {dtype} algo={algo}"
    # default dispatch through the reference-shaped entry
    t = torch.full((64, 2048), float(rank + 1), dtype=torch.bfloat16, device=dev)
    got = comm.custom_all_reduce(t)
    assert got is not None and torch.all(got == sum(range(1, world + 1)))
    assert ops.read_status(dev) == 0

    # ---- 2. fused k-slot sum + all-reduce (both algorithms)
    from layered_prefill_b200._lib import check, lib
    # algo 0 / 1: decode-sized tensors take the flag-in-data kernel (no barrier); 3: one-shot with barriers
    # (the one-barrier kernel on its alternating halves); 2: two-shot
    for T, k, H, algo in ((64, 8, 2048, 1), (64, 8, 2048, 2), (64, 8, 2048, 3), (300, 4, 512, 2), (1, 2, 64, 1),
                          (1, 2, 64, 3), (17, 8, 2048, 0), (64, 8, 2048, 0)):
        c3s = []
        for r in range(world):
            g = torch.Generator().manual_seed(T * 7 + r)
            c3s.append(torch.randn(T, k, H, generator=g).to(torch.bfloat16))
        want = O.all_reduce([O.moe_sum(c) for c in c3s])
        c3 = c3s[rank].to(dev)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        check(lib.moe_b200_ar_moe_sum_all_reduce(comm._ptr, c3.data_ptr(), out.data_ptr(), T, k, H,
                                                 comm.buffer_ptrs[rank], comm.max_size, algo,
                                                 ops.status_word(dev).data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), want), f"moe_sum_all_reduce T={T} algo={algo}"
    assert ops.read_status(dev) == 0

    # ---- 3. whole block, tensor parallel, through the FusedMoE mirror
    g = torch.Generator().manual_seed(5)
    T, H, E, k, I = 96, 512, 16, 4, 64 * world
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g).to(torch.bfloat16)
    want = O.moe_block_tp(x, logits, w13, w2, k, world)
    layer = FusedMoE(E, k, H, I, params_dtype=torch.bfloat16, reduce_results=True).to(dev)
    assert layer.tp_size == world and layer.intermediate_size_per_partition == I // world
    for e in range(E):  # checkpoint tensors are per expert: gate, up, down
        layer.weight_loader(layer.w13_weight, w13[e, :I].to(dev), "experts.w13_weight", "w1", e)
        layer.weight_loader(layer.w13_weight, w13[e, I:].to(dev), "experts.w13_weight", "w3", e)
        layer.weight_loader(layer.w2_weight, w2[e].to(dev), "experts.w2_weight", "w2", e)
    sh13, sh2 = O.shard_expert_weights(w13, w2, world, rank)
    assert torch.equal(layer.w13_weight.cpu(), sh13) and torch.equal(layer.w2_weight.cpu(), sh2)
    import layered_prefill_b200.custom_all_reduce as car
    car._ar_comm = comm
    out = layer(x.to(dev).clone(), logits.to(dev))
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    rl, ma = O.rel_l2(out.cpu(), want), O.max_abs(out.cpu(), want)
    assert rl <= 5e-3 and ma <= 2e-2, (rl, ma)
    # every rank holds identical bits
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    assert all(torch.equal(gathered[0], t) for t in gathered)
    # unfused route: forward (no reduction) then the reference-shaped all-reduce call
    layer.reduce_results = False
    part = layer(x.to(dev).clone(), logits.to(dev))
    red = layer.maybe_all_reduce_tensor_model_parallel(part)
    assert torch.equal(red, out)

    # ---- 3b. benchmark shapes at full size: the decode configuration (T=64, H=2048, E=128, top-8, I=768; at 8 ranks
    # I/tp = 96, one 96-column gate_up tile per expert) and the 235B layer's widths (H=4096, I=1536: I/tp = 192 at 8
    # ranks; 32 of its 128 experts, to bound host memory) through the one-call block with the fused reduction
    from layered_prefill_b200 import workload as W
    cases = [W.WORKLOADS["qwen3-30b-a3b-decode-t64"]]
    if world == 8:
        cases.append(W.MoeWorkload("qwen3-235b-a22b-widths-e32-t64", 64, 4096, 32, 8, 1536))
    for wl in cases:
        inp = W.make_inputs(wl, seed=0)
        want = O.moe_block_tp(inp["x"], inp["router_logits"], inp["w13"], inp["w2"], wl.top_k, world)
        sh13, sh2 = O.shard_expert_weights(inp["w13"], inp["w2"], world, rank)
        xd, lgd, w13d, w2d = inp["x"].to(dev), inp["router_logits"].to(dev), sh13.to(dev), sh2.to(dev)
        outs = []
        for rep in range(3):  # repeated calls alternate the halves of the fused buffer
            outs.append(fused_moe.fused_moe_forward(xd, lgd, w13d, w2d, wl.top_k, True, inplace=False, comm=comm))
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        rl, ma = O.rel_l2(outs[0].cpu(), want), O.max_abs(outs[0].cpu(), want)
        assert rl <= 5e-3 and ma <= 2e-2, (wl.name, rl, ma)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        gathered = [torch.empty_like(outs[0]) for _ in range(world)]
        dist.all_gather(gathered, outs[0])
        assert all(torch.equal(gathered[0], t) for t in gathered), wl.name
        del inp, sh13, sh2, w13d, w2d

    # ---- 4. CUDA-graph capture of the all-reduce on an unregistered tensor: the address met during capture
    # is registered with the peers when the capture() context ends (custom_all_reduce.py:206-239)
    inp = torch.full((128, 1024), float(rank + 1), dtype=torch.bfloat16, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with car.capture():
            warm = car.tensor_model_parallel_all_reduce(inp)  # warm-up outside capture: allocation pattern only
            assert warm.shape == inp.shape
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                res = car.tensor_model_parallel_all_reduce(inp)
    torch.cuda.current_stream().wait_stream(side)
    dist.barrier()
    for rep in range(3):
        inp.fill_(float(rank + 1 + rep))
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.all(res == sum(r + 1 + rep for r in range(world))), f"graph replay {rep}"
        dist.barrier()
    assert ops.read_status(dev) == 0

    # ---- 5. all-reduce that ends in the next layer's residual add + RMSNorm: same bits as the two steps, for a
    # decode-sized tensor (one fused launch) and one above every one-shot limit (all-reduce + norm kernel)
    for T, H in ((64, 2048), (1, 512), (33, 1024), (3000, 2048)):
        parts, g = [], None
        for r in range(world):
            g = torch.Generator().manual_seed(T + 31 * r)
            parts.append(torch.randn(T, H, generator=g).to(torch.bfloat16))
        g = torch.Generator().manual_seed(T + 1000)
        res0 = (torch.randn(T, H, generator=g) * 2).to(torch.bfloat16)
        wn = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(dev)
        # the two separate steps
        red = comm.all_reduce(parts[rank].to(dev), registered=False)
        res_a, norm_a = res0.to(dev).clone(), torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        ops.add_rms_norm(norm_a, res_a, red, wn, 1e-6)
        # one call
        res_b = res0.to(dev).clone()
        norm_b, res_b2 = comm.all_reduce_add_rms_norm(parts[rank].to(dev), res_b, wn, 1e-6)
        torch.cuda.synchronize()
        assert res_b2.data_ptr() == res_b.data_ptr()
        assert torch.equal(res_a, res_b), f"residual T={T}"
        assert torch.equal(norm_a, norm_b), f"normed T={T}"
        assert torch.equal(red.cpu(), O.all_reduce(parts))
    assert ops.read_status(dev) == 0
    # the same tail behind the k-slot sum (decode shapes), ranks deliberately out of step and calls back to back
    # without host synchronisation: a block of a lagging peer must never be read before it wrote its rows
    T, k, H, reps = 64, 8, 2048, 40
    c3s, res0s = [], []
    for variant in range(2):
        per_rank = []
        for r in range(world):
            g = torch.Generator().manual_seed(900 + 10 * variant + r)
            per_rank.append(torch.randn(T, k, H, generator=g).to(torch.bfloat16))
        c3s.append(per_rank)
        res0s.append((torch.randn(T, H, generator=torch.Generator().manual_seed(950 + variant)) * 2).to(torch.bfloat16))
    wn = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(960))).to(torch.bfloat16)
    mine = [per_rank[rank].to(dev) for per_rank in c3s]
    wnd = wn.to(dev)
    wants = []  # the separate steps, each synchronised: k-slot sum, all-reduce, add + norm
    for variant in range(2):
        part = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        ops.moe_sum(mine[variant], part)
        red = comm.all_reduce(part, registered=False)
        torch.cuda.synchronize()
        assert torch.equal(red.cpu(), O.all_reduce([O.moe_sum(c) for c in c3s[variant]]))
        res_w, norm_w = res0s[variant].to(dev).clone(), torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        ops.add_rms_norm(norm_w, res_w, red, wnd, 1e-6)
        torch.cuda.synchronize()
        wants.append((norm_w.cpu(), res_w.cpu()))
        dist.barrier()
    res_bufs = torch.stack([res0s[i % 2] for i in range(reps)]).to(dev)
    norm_bufs = torch.empty(reps, T, H, dtype=torch.bfloat16, device=dev)
    scratch = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    dist.barrier()
    for i in range(reps):
        if (i + rank) % 5 == 0:
            torch.cuda._sleep(300_000 * (1 + rank % 3))
        check(lib.moe_b200_ar_moe_sum_all_reduce_add_rms_norm(
            comm._ptr, mine[i % 2].data_ptr(), scratch.data_ptr(), res_bufs[i].data_ptr(), wnd.data_ptr(), 1e-6,
            norm_bufs[i].data_ptr(), T, k, H, comm.buffer_ptrs[rank], comm.max_size, 0,
            ops.status_word(dev).data_ptr(), stream))
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    for i in range(reps):
        want_norm, want_res = wants[i % 2]
        assert torch.equal(res_bufs[i].cpu(), want_res), f"norm-tailed fused reduction, residual of call {i}"
        assert torch.equal(norm_bufs[i].cpu(), want_norm), f"norm-tailed fused reduction, call {i}"

    # the block with that tail, through the FusedMoE mirror: same bits as block -> all-reduce -> add_rms_norm
    layer.reduce_results = True
    res0 = (torch.randn(T := 96, H := 512, generator=torch.Generator().manual_seed(77)) * 2).to(torch.bfloat16)
    wn = torch.ones(H, dtype=torch.bfloat16, device=dev)
    blk = layer(x.to(dev).clone(), logits.to(dev))
    res_a, norm_a = res0.to(dev).clone(), torch.empty_like(blk)
    ops.add_rms_norm(norm_a, res_a, blk, wn, 1e-6)
    res_b = res0.to(dev).clone()
    norm_b, _ = layer.forward_reduce_norm(x.to(dev).clone(), logits.to(dev), res_b, wn, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(res_a, res_b) and torch.equal(norm_a, norm_b)
    assert ops.read_status(dev) == 0

    # ---- 5b. the row-parallel linear (o_proj, nanovllm/layers/linear.py:155-201) through the same tail: product
    # written into the peer-visible buffer, reduction + residual add + norm in one call; same bits as
    # forward() followed by add_rms_norm, and close to the unsharded fp32 product
    from layered_prefill_b200.linear import RowParallelLinear
    for T, K, Nout, use_bias in ((64, 4096, 2048, False), (5, 512, 256, True), (700, 1024, 2048, False)):
        g = torch.Generator().manual_seed(T + K)
        w_full = (torch.randn(Nout, K, generator=g) * 0.03).to(torch.bfloat16)
        b_full = torch.randn(Nout, generator=g).to(torch.bfloat16)
        x_full = torch.randn(T, K, generator=g).to(torch.bfloat16)
        res0 = torch.randn(T, Nout, generator=g).to(torch.bfloat16)
        wn = (1 + 0.1 * torch.randn(Nout, generator=g)).to(torch.bfloat16).to(dev)
        lin = RowParallelLinear(K, Nout, bias=use_bias).to(dev).to(torch.bfloat16)
        assert lin.weight.shape == (Nout, K // world) and lin.tp_size == world
        lin.weight_loader(lin.weight, w_full.to(dev))
        if use_bias:
            lin.bias.data.zero_()
            lin.weight_loader(lin.bias, b_full.to(dev))
        kp = K // world
        x_shard = x_full[:, rank * kp:(rank + 1) * kp].contiguous().to(dev)
        y = lin(x_shard)
        res_a, norm_a = res0.to(dev).clone(), torch.empty(T, Nout, dtype=torch.bfloat16, device=dev)
        ops.add_rms_norm(norm_a, res_a, y, wn, 1e-6)
        res_b = res0.to(dev).clone()
        norm_b, res_b2 = lin.forward_reduce_norm(x_shard, res_b, wn, 1e-6)
        torch.cuda.synchronize()
        assert res_b2.data_ptr() == res_b.data_ptr()
        assert torch.equal(res_a, res_b) and torch.equal(norm_a, norm_b), f"row-parallel linear tail T={T}"
        full = x_full.float() @ w_full.float().t() + (b_full.float() if use_bias else 0.0)
        assert O.rel_l2(y.cpu(), full.to(torch.bfloat16)) <= 1e-2
    assert ops.read_status(dev) == 0

    # ---- 6. fp8 experts, tensor parallel with I/tp = 192 (slices split the 128-wide scale blocks), k-slot sum fused
    # with the all-reduce: against the all-reduced per-rank CPU emulations
    g = torch.Generator().manual_seed(91)
    T, H, E, k, I = 48, 256, 4, 2, 192 * world
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.03).to(torch.bfloat16)
    q13, s13 = O.quant_weight_block_fp8(w13)
    q2, s2 = O.quant_weight_block_fp8(w2)
    tw, ti, _ = O.fused_topk(x, torch.randn(T, E, generator=g), k, True)
    ip = I // world
    b13, b2 = q13.view(torch.uint8), q2.view(torch.uint8)

    def shard(r):
        lo, hi = r * ip, (r + 1) * ip
        return (torch.cat([b13[:, lo:hi], b13[:, I + lo:I + hi]], dim=1).contiguous().view(torch.float8_e4m3fn),
                b2[:, :, lo:hi].contiguous().view(torch.float8_e4m3fn))

    want = O.all_reduce([O.fused_experts_fp8(x, *[t for t in (shard(r)[0], s13, shard(r)[1], s2)], tw, ti,
                                             i_offset=r * ip, i_total=I) for r in range(world)])
    q13r, q2r = shard(rank)
    got = fused_moe.fused_experts_fp8_shard(x.to(dev), q13r.to(dev), s13.to(dev), q2r.to(dev), s2.to(dev), tw.to(dev),
                                            ti.to(dev), rank * ip, I, comm=comm)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    assert O.rel_l2(got.cpu(), want) <= 5e-3, O.rel_l2(got.cpu(), want)
    gathered = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(gathered, got)
    assert all(torch.equal(gathered[0], t) for t in gathered)

    # ---- 7. the fused k-slot-sum + one-shot all-reduce keeps no closing barrier (it alternates between two
    # registered halves): many calls back to back without host synchronisation, ranks deliberately out of step,
    # every result checked afterwards; then the same from a replayed CUDA graph
    T, k, H, reps = 64, 8, 2048, 120
    c3s = []
    for variant in range(3):
        per_rank = []
        for r in range(world):
            g = torch.Generator().manual_seed(400 + 10 * variant + r)
            per_rank.append(torch.randn(T, k, H, generator=g).to(torch.bfloat16))
        c3s.append(per_rank)
    wants = [O.all_reduce([O.moe_sum(c) for c in per_rank]) for per_rank in c3s]
    mine = [per_rank[rank].to(dev) for per_rank in c3s]
    outs = torch.empty(reps, T, H, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for algo in (0, 3):  # the flag-in-data kernel, then the one-barrier kernel
        outs.zero_()
        dist.barrier()
        for i in range(reps):
            if (i + rank) % 7 == 0:
                torch.cuda._sleep(200_000 * (1 + rank))   # this rank falls behind its peers for a while
            check(lib.moe_b200_ar_moe_sum_all_reduce(comm._ptr, mine[i % 3].data_ptr(), outs[i].data_ptr(), T, k, H,
                                                     comm.buffer_ptrs[rank], comm.max_size, algo,
                                                     ops.status_word(dev).data_ptr(), stream))
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        for i in range(reps):
            assert torch.equal(outs[i].cpu(), wants[i % 3]), f"barrier-free / one-barrier all-reduce (algo {algo}), call {i}"
    c3_buf = mine[0].clone()
    out_g = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            check(lib.moe_b200_ar_moe_sum_all_reduce(comm._ptr, c3_buf.data_ptr(), out_g.data_ptr(), T, k, H,
                                                     comm.buffer_ptrs[rank], comm.max_size, 0,
                                                     ops.status_word(dev).data_ptr(), side.cuda_stream))
    torch.cuda.current_stream().wait_stream(side)
    dist.barrier()
    for i in range(9):   # the same graph replayed back to back: the half in use is chosen on the device
        c3_buf.copy_(mine[i % 3])
        graph.replay()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out_g.cpu(), wants[i % 3]), f"one-barrier all-reduce, graph replay {i}"
        dist.barrier()
    assert ops.read_status(dev) == 0

    # ---- 8. inside the reference's own caller: its Qwen3MoeSparseMoeBlock (gate linear -> FusedMoE -> reduce,
    # nanovllm/models/qwen3_moe.py:66-116) built tensor-parallel on these ranks from the staged copy of the reference,
    # run as it is (its Triton experts; its reduction's arithmetic carried by NCCL) and with this library's fused_topk / fused_experts /
    # tensor_model_parallel_all_reduce patched into its modules; then the patched block captured into a CUDA graph
    # under capture() as the reference's model runner does (qwen3_moe.py:710-759) and replayed on new tokens
    from oracle.build_ref import load_reference_package
    if load_reference_package() is not None:
        import nanovllm.layers.for_moe.fused_moe as rfm
        import nanovllm.layers.fused_moe as rlayer
        import nanovllm.models.qwen3_moe as rmodel
        from transformers import Qwen3MoeConfig
        cfg = Qwen3MoeConfig(hidden_size=1024, num_experts=32, num_experts_per_tok=4, moe_intermediate_size=96 * world,
                             norm_topk_prob=True)
        saved = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            with torch.device(dev):
                blk = rmodel.Qwen3MoeSparseMoeBlock(cfg)
        finally:
            torch.set_default_dtype(saved)
        E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
        assert blk.experts.tp_size == world and blk.experts.w13_weight.shape == (E, 2 * I // world, H)
        g = torch.Generator().manual_seed(123)
        for e in range(E):
            gate = (torch.randn(I, H, generator=g) * 0.05).to(torch.bfloat16).to(dev)
            up = (torch.randn(I, H, generator=g) * 0.05).to(torch.bfloat16).to(dev)
            down = (torch.randn(H, I, generator=g) * 0.05).to(torch.bfloat16).to(dev)
            blk.experts.weight_loader(blk.experts.w13_weight, gate, "experts.w13_weight", "w1", e)
            blk.experts.weight_loader(blk.experts.w13_weight, up, "experts.w13_weight", "w3", e)
            blk.experts.weight_loader(blk.experts.w2_weight, down, "experts.w2_weight", "w2", e)
        blk.gate.weight.data.copy_((torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16))
        xs = [torch.randn(T_, H, generator=g).to(torch.bfloat16).to(dev) for T_ in (64, 64, 1536)]

        def nccl_sum(t):
            # the arithmetic of the reference's own all-reduce kernel (fp32 sum in rank order, one rounding,
            # csrc/custom_all_reduce.cuh:288-296), carried by NCCL: gather the partial sums, add them here
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            acc = parts[0].float()
            for part in parts[1:]:
                acc += part.float()
            return acc.to(t.dtype)

        stock_fns = (rfm.fused_topk, blk.experts.quant_method.fused_experts, rlayer.tensor_model_parallel_all_reduce)
        try:
            rlayer.tensor_model_parallel_all_reduce = nccl_sum
            wants = [blk(x_.clone()) for x_ in xs]
            torch.cuda.synchronize()
            rfm.fused_topk = fused_moe.fused_topk
            blk.experts.quant_method.fused_experts = fused_moe.fused_experts
            rlayer.tensor_model_parallel_all_reduce = car.tensor_model_parallel_all_reduce
            l0 = ops.launch_count()
            gots = [blk(x_.clone()) for x_ in xs]
            torch.cuda.synchronize()
            assert ops.launch_count() - l0 >= 4 * len(xs), "the patched block did not run this library's kernels"
            for got, want in zip(gots, wants):
                rl, ma = O.rel_l2(got.cpu(), want.cpu()), O.max_abs(got.cpu(), want.cpu())
                assert rl <= 5e-3 and ma <= max(2e-2, 2 ** -7 * float(want.float().abs().max())), (rl, ma)
            # graph capture of the patched block on a fixed input buffer
            x_buf = xs[0].clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with car.capture():
                    blk(x_buf.clone())  # warm-up outside the capture
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        res = blk(x_buf.clone())
            torch.cuda.current_stream().wait_stream(side)
            dist.barrier()
            for i in (1, 0):
                x_buf.copy_(xs[i])
                torch.cuda.synchronize()
                dist.barrier()
                graph.replay()
                torch.cuda.synchronize()
                assert torch.equal(res, gots[i]), f"graph replay of the patched block, input {i}"
                dist.barrier()
        finally:
            rfm.fused_topk, blk.experts.quant_method.fused_experts, rlayer.tensor_model_parallel_all_reduce = stock_fns
        assert ops.read_status(dev) == 0
        print(f"TP_WORKER_REFERENCE_CALLER_OK rank={rank}", flush=True)

    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"TP_WORKER_OK rank={rank}", flush=True)


if __name__ == "__main__":
    main()
