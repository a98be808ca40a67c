"""Tensor-parallel wiring of `Linear` on two CPU ranks (gloo): column-parallel fc1 followed by
row-parallel fc2 under sequence parallelism, with the quantized all-gather, the abs-max
MAX all-reduce, the async dgrad reduce-scatter and the memory-saving re-gather. The CUDA
kernels cannot run here, so a stand-in backend defined in this file plays the quantize
operator: it keeps values in fp32 and multiplies exactly, which makes the expected result a
plain matmul on the gathered tensors."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from minitransformer_b200.distributed.distributed import (allreduce_max_, gather_packed_along_first_dim)
from minitransformer_b200.module import config
from minitransformer_b200.module.linear import Linear
from minitransformer_b200.ops import quantization as Q


class _StandInOp(Q.QuantizeOpBase):
    """Test double: 'codes' are the fp32 values, 'scales' are per-block abs-max (unused by the
    product), the per-tensor abs-max goes through the same reduce path as the real backends."""
    calls = []

    @property
    def supports_allgather(self):
        return True

    def quantize(self, x, qparams, return_transpose=False, reduce_amax=False, tp_group=None, input_meta=None):
        x = x.reshape(-1, x.shape[-1]).float().contiguous()
        amax = torch.stack([x.abs().max(), x.abs().max()])
        if reduce_amax:
            allreduce_max_(amax, tp_group)
            _StandInOp.calls.append("reduce_amax")
        blk = 16
        scale = x.abs().reshape(x.shape[0], -1, blk).amax(-1)
        r = Q.QuantizeResult(x.clone(), scale, None, None, amax[0:1], amax[1:2])
        if return_transpose:
            xt = x.t().contiguous()
            r.data_t, r.scale_t = xt, xt.abs().reshape(xt.shape[0], -1, blk).amax(-1)
        return r

    def qgemm(self, qx, qw, m_params, out_dtype, sx, sw, bias=None, out=None, accumulate=False,
              global_amax_qx=None, global_amax_qw=None, qparams_x=None, qparams_w=None):
        assert sx.shape[0] >= qx.shape[0] and sx.shape[1] * 16 == qx.shape[1]
        y = qx @ qw.t()
        if accumulate:
            out.add_(y.to(out.dtype))
            return out
        if out is not None:
            out.copy_(y.to(out.dtype))
            return out
        return y.to(out_dtype)


def _params(allgather_quantize, memory_saving):
    qp = Q.QParams(quant_tile_shape=(1, 16))
    return config.QLinearParams(quantize=True, x_params=qp, w_params=qp, g_params=qp, quantize_op=_StandInOp(),
                                allgather_quantize=allgather_quantize, memory_saving=memory_saving)


def _worker(rank, world, port, allgather_quantize, memory_saving, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        T, H, Fd = 64, 32, 96
        x_full = torch.randn(T, H)
        w1_full = torch.randn(Fd, H) * 0.1
        w2_full = torch.randn(H, Fd) * 0.1
        dy_full = torch.randn(T, H)
        p = _params(allgather_quantize, memory_saving)
        kw = dict(bias=False, params_dtype=torch.float32, device="cpu", qlinear_params=p, tp_group=dist.group.WORLD,
                  sequence_parallel=True)
        fc1 = Linear(H, Fd, parallel_mode="column", **kw)
        fc2 = Linear(Fd, H, parallel_mode="row", **kw)
        assert fc1.out_features == Fd // world and fc2.in_features == Fd // world
        assert fc1.weight.tensor_model_parallel and fc1.weight.partition_dim == 0 and fc2.weight.partition_dim == 1
        with torch.no_grad():
            fc1.weight.copy_(w1_full.chunk(world, 0)[rank])
            fc2.weight.copy_(w2_full.chunk(world, 1)[rank])
        x = x_full.chunk(world, 0)[rank].clone().requires_grad_(True)
        y = fc2(fc1(x))
        y.backward(dy_full.chunk(world, 0)[rank])

        h_ref = x_full @ w1_full.t()
        y_ref = h_ref @ w2_full.t()
        dh_ref = dy_full @ w2_full
        ok = torch.allclose(y, y_ref.chunk(world, 0)[rank], atol=1e-4)
        ok &= torch.allclose(x.grad, (dh_ref @ w1_full).chunk(world, 0)[rank], atol=1e-4)
        ok &= torch.allclose(fc1.weight.grad, (dh_ref.t() @ x_full).chunk(world, 0)[rank], atol=1e-4)
        ok &= torch.allclose(fc2.weight.grad, (dy_full.t() @ h_ref).chunk(world, 1)[rank], atol=1e-4)
        if allgather_quantize:
            ok &= "reduce_amax" in _StandInOp.calls
        # the packed gather returns every piece in rank order
        a = torch.full((2, 3), float(rank))
        b = torch.full((2, 1), float(10 + rank)).to(torch.float64)
        ga, gb = gather_packed_along_first_dim([a, b], dist.group.WORLD)
        ok &= ga.shape == (2 * world, 3) and gb.dtype == torch.float64
        ok &= torch.equal(ga[:, 0], torch.arange(world).repeat_interleave(2).float())
        ok &= torch.equal(gb[:, 0], (10 + torch.arange(world)).repeat_interleave(2).double())
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("allgather_quantize,memory_saving", [(True, False), (False, False), (True, True)])
def test_column_then_row_parallel_linear_on_two_gloo_ranks(allgather_quantize, memory_saving):
    world = 2
    mgr = mp.Manager()
    result = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), allgather_quantize, memory_saving, result), nprocs=world, join=True)
    assert dict(result) == {0: True, 1: True}


def _grouped_worker(rank, world, port, result):
    """Tensor-parallel GroupedLinear on the non-quantized path: column-parallel experts followed
    by row-parallel experts; the output of the row-parallel layer and the input gradient of the
    column-parallel layer are all-reduced (there is no sequence parallelism for experts)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from minitransformer_b200.module.group_linear import GroupedLinear
        torch.manual_seed(1)
        G, H, Fd = 3, 128, 256
        m_splits = [5, 0, 9]
        R = sum(m_splits)
        x_full = torch.randn(R, H)
        w1 = [torch.randn(Fd, H) * 0.1 for _ in range(G)]
        w2 = [torch.randn(H, Fd) * 0.1 for _ in range(G)]
        dy = torch.randn(R, H)
        p = config.QLinearParams(quantize=False)
        kw = dict(bias=False, params_dtype=torch.float32, device="cpu", qlinear_params=p, tp_group=dist.group.WORLD,
                  tp_size=world)
        fc1 = GroupedLinear(G, H, Fd, parallel_mode="column", **kw)
        fc2 = GroupedLinear(G, Fd, H, parallel_mode="row", **kw)
        assert fc1.out_features == Fd // world and fc2.in_features == Fd // world
        with torch.no_grad():
            for g in range(G):
                getattr(fc1, f"weight{g}").copy_(w1[g].chunk(world, 0)[rank])
                getattr(fc2, f"weight{g}").copy_(w2[g].chunk(world, 1)[rank])
        x = x_full.clone().requires_grad_(True)
        y = fc2(fc1(x, m_splits), m_splits)
        y.backward(dy)

        xs, dys = torch.split(x_full, m_splits), torch.split(dy, m_splits)
        hs = [a @ w.t() for a, w in zip(xs, w1)]
        y_ref = torch.cat([h @ w.t() for h, w in zip(hs, w2)])
        dhs = [d @ w for d, w in zip(dys, w2)]
        dx_ref = torch.cat([d @ w for d, w in zip(dhs, w1)])
        ok = torch.allclose(y, y_ref, atol=1e-4) and torch.allclose(x.grad, dx_ref, atol=1e-4)
        for g in range(G):
            ok &= torch.allclose(getattr(fc1, f"weight{g}").grad, (dhs[g].t() @ xs[g]).chunk(world, 0)[rank], atol=1e-4)
            ok &= torch.allclose(getattr(fc2, f"weight{g}").grad, (dys[g].t() @ hs[g]).chunk(world, 1)[rank], atol=1e-4)
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_grouped_linear_on_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    result = mgr.dict()
    mp.spawn(_grouped_worker, args=(world, _free_port(), result), nprocs=world, join=True)
    assert dict(result) == {0: True, 1: True}
