"""Tensor-parallel NVFP4 MLP (column-parallel fc1 -> row-parallel fc2, sequence parallel,
quantized all-gather) on two GPUs over NCCL against the same layers on one GPU. Skipped on
boxes with a single GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _emulate_rank(x, w1_shard, w2_shard, dy, recipe):
    """What rank r computes before its collectives, run without any process group: fc1 and fc2
    built from r's weight shards, applied to the full (gathered) activations. The partial outputs
    y_r and dx_r of all ranks are then summed, which is what the reduce-scatters do."""
    from minitransformer_b200.module import config
    from minitransformer_b200.module.linear import Linear
    p = config.get_qlinear_params_from_predefined(recipe)
    kw = dict(bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=p)
    fc1, fc2 = Linear(x.shape[1], w1_shard.shape[0], **kw), Linear(w2_shard.shape[1], w2_shard.shape[0], **kw)
    with torch.no_grad():
        fc1.weight.copy_(w1_shard)
        fc2.weight.copy_(w2_shard)
    xd = x.clone().requires_grad_(True)
    h = fc1(xd)
    y = fc2(h)
    y.backward(dy)
    return y.detach().float(), xd.grad.float(), fc1.weight.grad, fc2.weight.grad, h.detach()


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from minitransformer_b200 import kernels as K
        from minitransformer_b200.module import config
        from minitransformer_b200.module.linear import Linear
        recipe = config.QuantizeRecipe.FP4_SUB_CHANNEL
        g = torch.Generator().manual_seed(3)
        T, H, Fd = 512, 256, 768
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        w1 = (torch.randn(Fd, H, generator=g) * 0.02).to(torch.bfloat16).cuda()
        w2 = (torch.randn(H, Fd, generator=g) * 0.02).to(torch.bfloat16).cuda()
        dy = (torch.randn(T, H, generator=g) * 1e-3).to(torch.bfloat16).cuda()
        emu = [_emulate_rank(x, w1.chunk(world, 0)[r], w2.chunk(world, 1)[r], dy, recipe) for r in range(world)]
        y_ref = sum(e[0] for e in emu)
        dx_ref = sum(e[1] for e in emu)

        p = config.get_qlinear_params_from_predefined(recipe)
        assert p.allgather_quantize
        kw = dict(bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=p, tp_group=dist.group.WORLD,
                  sequence_parallel=True)
        fc1 = Linear(H, Fd, parallel_mode="column", **kw)
        fc2 = Linear(Fd, H, parallel_mode="row", **kw)
        with torch.no_grad():
            fc1.weight.copy_(w1.chunk(world, 0)[rank])
            fc2.weight.copy_(w2.chunk(world, 1)[rank])
        xd = x.chunk(world, 0)[rank].clone().requires_grad_(True)
        h = fc1(xd)
        y = fc2(h)
        y.backward(dy.chunk(world, 0)[rank])
        torch.cuda.synchronize()

        def relf(a, b):
            return float((a.float() - b.float()).norm() / b.float().norm())

        errs = {
            "h": relf(h, emu[rank][4]),
            "y": relf(y, y_ref.chunk(world, 0)[rank]),          # bf16 partials summed by the reduce-scatter
            "dx": relf(xd.grad, dx_ref.chunk(world, 0)[rank]),
            "dw1": relf(fc1.weight.grad, emu[rank][2]),
            "dw2": relf(fc2.weight.grad, emu[rank][3]),
        }
        # quantized gather == quantize(gathered): check the activation codes directly
        from minitransformer_b200.module.linear import _QuantizedLinear
        qg = _QuantizedLinear.quantize_optionally_allgather(p.quantize_op, x.chunk(world, 0)[rank].contiguous(), p.x_params,
                                                            True, True, True, dist.group.WORLD)
        qf = p.quantize_op.quantize(x, p.x_params, return_transpose=True)
        same = (torch.equal(qg.data, qf.data) and torch.equal(qg.scale.view(torch.uint8), qf.scale.view(torch.uint8))
                and torch.equal(qg.data_t, qf.data_t)
                and torch.equal(qg.scale_t.view(torch.uint8), qf.scale_t.view(torch.uint8)[: H])
                and float(qg.global_amax_row) == float(qf.global_amax_row)
                and float(qg.global_amax_col) == float(qf.global_amax_col))
        # the copy-free form of the same gather: codes concatenated in place, GEMM-layout scales,
        # transposed copies left as per-rank K slabs that the GEMM walks directly
        qs = _QuantizedLinear.quantize_optionally_allgather(p.quantize_op, x.chunk(world, 0)[rank].contiguous(), p.x_params,
                                                            True, True, True, dist.group.WORLD, weight_shape=(Fd, H))
        assert qs.data_t.dim() == 3 and qs.data_t.shape[0] == world
        same = (same and torch.equal(qs.data, qf.data) and torch.equal(qs.scale_swz.view(-1), qf.scale_swz.view(-1))
                and torch.equal(qs.data_t.permute(1, 0, 2).reshape(H, -1), qf.data_t))
        d_plain = K.gemm_nvfp4(qf.data_t, qf.scale_t_swz, qf.global_amax_col, qf.data_t, qf.scale_t_swz,
                               qf.global_amax_col, out_dtype=torch.float32)
        d_slab = K.gemm_nvfp4(qf.data_t, qf.scale_t_swz, qf.global_amax_col, qs.data_t, qs.scale_t_swz,
                              qs.global_amax_col, out_dtype=torch.float32)
        d_slab2 = K.gemm_nvfp4(qs.data_t, qs.scale_t_swz, qs.global_amax_col, qs.data_t, qs.scale_t_swz,
                               qs.global_amax_col, out_dtype=torch.float32)
        same = same and torch.equal(d_plain, d_slab) and torch.equal(d_plain, d_slab2)
        result[rank] = (errs, bool(same), K.read_device_status())
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_nvfp4_mlp_matches_single_gpu():
    world = 2
    mgr = mp.Manager()
    result = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), result), nprocs=world, join=True)
    for rank in range(world):
        errs, same, status = result[rank]
        assert same, "gathered quantized shards differ from quantizing the gathered tensor"
        assert status == 0
        # local GEMMs see identical quantized operands; the two reduce-scattered results add one
        # bf16 rounding of the partial sums
        assert errs["h"] <= 1e-3 and errs["dw1"] <= 1e-3 and errs["dw2"] <= 1e-3, errs
        assert errs["y"] <= 1e-2 and errs["dx"] <= 1e-2, errs
