"""Host-side logic of the tensor-parallel path with two gloo ranks on the CPU: sharding through
FusedMoE.weight_loader, the partial sums' reduction, and the IPC handle exchange of CustomAllreduce
(with the device calls replaced by fakes -- there is no GPU here)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from layered_prefill_b200 import custom_all_reduce as car
        from layered_prefill_b200.layer import FusedMoE
        from oracle import moe_oracle as O

        g = torch.Generator().manual_seed(0)
        T, H, E, k, I = 10, 64, 8, 2, 64
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.1).to(torch.bfloat16)
        w2 = (torch.randn(E, H, I, generator=g) * 0.1).to(torch.bfloat16)
        b13 = torch.randn(E, 2 * I, generator=g).to(torch.bfloat16)
        b2 = torch.randn(E, H, generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, generator=g)

        layer = FusedMoE(E, k, H, I, params_dtype=torch.bfloat16)
        assert (layer.tp_size, layer.tp_rank) == (world, rank)
        assert layer.w13_weight.shape == (E, 2 * I // world, H) and layer.w2_weight.shape == (E, H, I // world)
        for e in range(E):  # Qwen3-MoE checkpoints: one tensor per expert and projection
            layer.weight_loader(layer.w13_weight, w13[e, :I], "model.layers.0.mlp.experts.0.gate_proj.weight", "w1", e)
            layer.weight_loader(layer.w13_weight, w13[e, I:], "model.layers.0.mlp.experts.0.up_proj.weight", "w3", e)
            layer.weight_loader(layer.w2_weight, w2[e], "model.layers.0.mlp.experts.0.down_proj.weight", "w2", e)
        sh13, sh2 = O.shard_expert_weights(w13, w2, world, rank)
        assert torch.equal(layer.w13_weight.data, sh13) and torch.equal(layer.w2_weight.data, sh2)
        ip = I // world

        # gpt-oss checkpoints: all-expert tensors, gate/up rows interleaved and fused ("w13"), biases beside them
        # (utils/loader.py:41-49; layers/fused_moe.py:388-392,647-654): a rank takes a contiguous slice of the
        # fused rows and of the fused bias, w2_bias lives on rank 0 only
        goss = FusedMoE(E, k, H, I, params_dtype=torch.bfloat16, activation="swigluoai", has_bias=True)
        goss.weight_loader(goss.w13_weight, w13.clone(), "model.layers.0.mlp.experts.gate_up_proj_blocks", "w13", 0)
        goss.weight_loader(goss.w2_weight, w2.clone(), "model.layers.0.mlp.experts.down_proj_blocks", "w2", 0)
        goss.weight_loader(goss.w13_bias, b13.clone(), "model.layers.0.mlp.experts.gate_up_proj_bias", "w13", 0)
        goss.weight_loader(goss.w2_bias, b2.clone(), "model.layers.0.mlp.experts.down_proj_bias", "w2", 0)
        g13, g2 = O.shard_expert_weights(w13, w2, world, rank, "swigluoai")
        assert torch.equal(goss.w13_weight.data, g13) and torch.equal(goss.w2_weight.data, g2)
        assert torch.equal(goss.w13_bias.data, b13[:, 2 * rank * ip:2 * (rank + 1) * ip])
        assert torch.equal(goss.w2_bias.data, b2 if rank == 0 else torch.zeros_like(b2))  # rank 0 only
        whole = FusedMoE(E, k, H, I, params_dtype=torch.bfloat16, has_bias=True)
        whole.weight_loader(whole.w13_bias, goss.w13_bias.data.clone(), "experts.gate_up_proj_bias", "all", 0)
        assert torch.equal(whole.w13_bias.data, goss.w13_bias.data)
        try:
            layer.weight_loader(layer.w2_weight, w2[0], "model.layers.0.mlp.experts.0.down_proj", "w2", 0)
            raise AssertionError("a name without weight / block / bias must be refused, as the reference refuses it")
        except ValueError:
            pass

        # partial block on this rank's shard (CPU oracle), reduced over the ranks == the full block
        tw, ti, _ = O.fused_topk(x, logits, k, True)
        part = O.fused_experts(x, goss.w13_weight.data, goss.w2_weight.data, tw, ti, "swigluoai", mode="exact",
                               w13_bias=goss.w13_bias.data, w2_bias=goss.w2_bias.data).float()
        dist.all_reduce(part)
        full = O.fused_experts(x, w13, w2, tw, ti, "swigluoai", mode="exact", w13_bias=b13, w2_bias=b2).float()
        assert O.rel_l2(part, full) < 8e-3

        # fp8 shards: sliced like the bf16 weights, scales of the unsharded tensors; I / world = 192 puts rank 1's
        # slice in the middle of a 128-wide scale block. The ranks' partial sums add up to the unsharded emulation
        # (up to the finer quantisation groups of a split block).
        from layered_prefill_b200 import fused_moe as fm
        g8 = torch.Generator().manual_seed(3)
        I8, H8 = 192 * world, 128
        x8 = torch.randn(T, H8, generator=g8).to(torch.bfloat16)
        q13, s13 = O.quant_weight_block_fp8((torch.randn(E, 2 * I8, H8, generator=g8) * 0.05).to(torch.bfloat16))
        q2, s2 = O.quant_weight_block_fp8((torch.randn(E, H8, I8, generator=g8) * 0.05).to(torch.bfloat16))
        q13r, q2r, off = fm.shard_fp8_expert_weights(q13, q2, rank, world)
        assert off == rank * 192 and q13r.shape == (E, 384, H8) and q2r.shape == (E, H8, 192)
        ref13, ref2 = O.shard_expert_weights(q13.view(torch.uint8), q2.view(torch.uint8), world, rank)
        assert torch.equal(q13r.view(torch.uint8), ref13) and torch.equal(q2r.view(torch.uint8), ref2)
        part8 = O.fused_experts_fp8(x8, q13r, s13, q2r, s2, tw, ti, i_offset=off, i_total=I8).float()
        dist.all_reduce(part8)
        full8 = O.fused_experts_fp8(x8, q13, s13, q2, s2, tw, ti).float()
        assert O.rel_l2(part8, full8) < 3e-2

        # the row-parallel linear (o_proj): weight sharded on its input dimension, bias on rank 0 only, partial
        # products summed over the ranks (nanovllm/layers/linear.py:155-201)
        from layered_prefill_b200.linear import RowParallelLinear
        car._ar_comm = None
        gl = torch.Generator().manual_seed(11)
        w_full = torch.randn(24, 16 * world, generator=gl)
        b_full = torch.randn(24, generator=gl)
        x_full = torch.randn(5, 16 * world, generator=gl)
        lin = RowParallelLinear(16 * world, 24, bias=True)
        assert lin.weight.shape == (24, 16) and (lin.tp_rank, lin.tp_size) == (rank, world)
        lin.bias.data.zero_()
        lin.weight_loader(lin.weight, w_full)
        lin.weight_loader(lin.bias, b_full)
        assert torch.equal(lin.weight.data, w_full[:, 16 * rank:16 * (rank + 1)])
        assert torch.equal(lin.bias.data, b_full if rank == 0 else torch.zeros(24))
        y = lin(x_full[:, 16 * rank:16 * (rank + 1)].contiguous())
        assert torch.allclose(y, x_full @ w_full.t() + b_full, atol=1e-4)

        # mapping of checkpoint names to (param, shard) as the loader uses it
        m = FusedMoE.make_expert_params_mapping("gate_proj", "down_proj", "up_proj", num_experts=E)
        assert len(m) == 3 * E and m[0] == ("experts.w13_", "experts.0.gate_proj.", 0, "w1")
        assert m[1] == ("experts.w2_", "experts.0.down_proj.", 0, "w2")

        # without CUDA the communicator disables itself and the all-reduce entry falls back to the process group
        comm = car.CustomAllreduce(group=dist.new_group(backend="gloo"))
        assert comm.disabled and comm.world_size == world
        car._ar_comm = comm
        t = torch.full((4, 8), float(rank + 1))
        out = car.tensor_model_parallel_all_reduce(t)
        assert torch.all(out == sum(range(1, world + 1)))
        with car.capture():
            pass

        # handle exchange with fake device calls: every rank ends up with its own pointer at [rank]
        # and the pointers "opened" from its peers' handles elsewhere
        class FakeOps:
            @staticmethod
            def allocate_shared_buffer_and_handle(size):
                return 1000 + rank, bytes([rank]) * 64

            @staticmethod
            def open_mem_handle(h):
                return 2000 + h[0]
        real = car.ops
        car.ops = FakeOps
        try:
            ptrs = car.CustomAllreduce.create_shared_buffer(1 << 20, group=comm.gloo_group)
        finally:
            car.ops = real
        assert ptrs == [1000 + r if r == rank else 2000 + r for r in range(world)]
        # close(): every mapping of a peer's buffer is closed, the ranks meet, then each frees its own three buffers
        calls = []

        class FakeLifecycleOps:
            dispose = staticmethod(lambda p: calls.append(("dispose", p)))
            close_mem_handle = staticmethod(lambda p: calls.append(("close", p)))
            free_shared_buffer = staticmethod(lambda p: calls.append(("free", p)))
        c2 = car.CustomAllreduce.__new__(car.CustomAllreduce)
        c2.disabled, c2._ptr, c2.rank, c2.gloo_group = False, 77, rank, comm.gloo_group
        c2.meta_ptrs = [10 + r for r in range(world)]
        c2.buffer_ptrs = [20 + r for r in range(world)]
        c2.fused_ptrs = [30 + r for r in range(world)]
        c2.ll_ptrs = [40 + r for r in range(world)]
        car.ops = FakeLifecycleOps
        try:
            c2.close()
            c2.close()  # idempotent
        finally:
            car.ops = real
        assert calls[0] == ("dispose", 77) and c2.disabled and c2._ptr == 0
        closes = [c for c in calls if c[0] == "close"]
        frees = [c for c in calls if c[0] == "free"]
        assert sorted(p for _, p in closes) == sorted(b + r for b in (10, 20, 30, 40) for r in range(world) if r != rank)
        assert [p for _, p in frees] == [10 + rank, 20 + rank, 30 + rank, 40 + rank]
        assert max(calls.index(c) for c in closes) < min(calls.index(f) for f in frees)
        assert not car.is_weak_contiguous(torch.zeros(4, 4)[:, :2]) and car.is_weak_contiguous(torch.zeros(4, 4)[2:])
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))


@pytest.mark.parametrize("world", [2])
def test_tp_host_logic_two_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
