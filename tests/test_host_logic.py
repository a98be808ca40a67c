"""Host-side logic that needs no GPU: shape rules of the tensor-parallel exchange paths, sizes of a
rank's quantized shard, the quantized-weight cache as checkpoint state, the flop count of the
decoder configuration."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from minitransformer_b200 import kernels
from minitransformer_b200.module import linear as L
from minitransformer_b200.ops import quantization as Q


def test_copy_free_gather_shape_rules():
    ok = L._QuantizedLinear._gemm_ready_shapes
    assert ok("nvfp4", 1024, 8192, 8, True) and ok("mxfp8", 1024, 4096, 8, True)
    assert not ok("nvfp4", 100, 8192, 8, True)            # shards of whole 128-row scale chunks
    assert not ok("nvfp4", 128, 8192, 8, True)            # transposed rows of 64 bytes: not whole K steps
    assert ok("nvfp4", 128, 8192, 8, False)               # ... which only matter when x^T is gathered
    assert ok("mxfp8", 128, 8192, 8, True)
    assert not ok("nvfp4", 1024, 128, 8, True)            # a shape the tile kernel does not take


def test_scatter_rules_and_link_bound_estimate():
    class _PG:      # only its presence matters to the shape rule
        pass
    pg = _PG()
    assert L._scatter_possible(pg, 8192, 8192, torch.bfloat16, None, 8)
    assert not L._scatter_possible(pg, 8192, 8192, torch.float32, None, 8)     # bf16 partial sums only
    assert not L._scatter_possible(pg, 8192, 8192, torch.bfloat16, torch.zeros(1), 8)   # no bias inside the GEMM
    assert not L._scatter_possible(pg, 1024, 8192, torch.bfloat16, None, 8)    # slices of whole 256-row tiles
    assert not L._scatter_possible(None, 8192, 8192, torch.bfloat16, None, 8)
    # configuration 4: link-bound on 8 ranks (117 MB against 0.1 ms of tensor work), not on 2 or 4
    assert L._scatter_is_link_bound(8192, 8192, 28672 // 8, 8)
    assert not L._scatter_is_link_bound(8192, 8192, 28672 // 4, 4)
    assert not L._scatter_is_link_bound(8192, 8192, 28672 // 2, 2)


def test_quantized_shard_bytes():
    q, s, qt, st = kernels.quantized_shard_bytes("nvfp4", 1024, 8192)
    assert (q, qt) == (1024 * 4096, 8192 * 512)
    assert s == kernels.swizzled_scale_bytes(1024, 512) and st == kernels.swizzled_scale_bytes(8192, 64)
    q, s, qt, st = kernels.quantized_shard_bytes("mxfp8", 1024, 4096)
    assert (q, qt) == (1024 * 4096, 4096 * 1024) and s == kernels.swizzled_scale_bytes(1024, 128)


def test_quantized_weight_cache_round_trips_through_checkpoint_state():
    cache = Q.QuantizeResultCache()
    r = Q.QuantizeResult(torch.arange(12, dtype=torch.uint8).view(3, 4), torch.ones(3, 1).to(torch.float8_e4m3fn),
                         torch.arange(12, dtype=torch.uint8).view(4, 3), torch.ones(4, 1).to(torch.float8_e4m3fn),
                         torch.tensor([2.5]), torch.tensor([3.5]), torch.zeros(512, dtype=torch.uint8),
                         torch.ones(512, dtype=torch.uint8))
    cache.store(r)
    state = cache.state()
    assert all(t.dtype in (torch.uint8, torch.float32) for t, _ in state.values())
    other = Q.QuantizeResultCache()
    other.load_state(state)
    back = other.to_qresult()
    assert back.scale.dtype == torch.float8_e4m3fn and torch.equal(back.data, r.data)
    assert torch.equal(back.scale.view(torch.uint8), r.scale.view(torch.uint8))
    assert float(back.global_amax_col) == 3.5 and back.scale._mt_swz is back.scale_swz
    other.clear()
    assert other.data is None and other.scale_t_swz is None


def test_pad_offsets_remember_their_split_sizes():
    pad = kernels.PadOffsets([0, 128, 128, 256])
    pad.splits = (3, 0, 5)
    assert list(pad) == [0, 128, 128, 256] and pad[-1] == 256 and pad.splits == (3, 0, 5)


def test_decoder_flop_count_matches_the_configuration():
    import bench
    f_layers = bench.llama_linear_flops(bench.C5, with_head=False)
    # 2 * 8192 tokens * 4096 * (6144 + 4096 + 28672 + 14336) per layer forward, x 3 GEMMs x 8 layers
    assert abs(f_layers - 3 * 8 * 2.0 * 8192 * 4096 * (6144 + 4096 + 28672 + 14336)) < 1e6
    assert abs(f_layers / 1e12 - 85.8) < 0.1
    assert abs((bench.llama_linear_flops(bench.C5) - f_layers) / 1e12 - 6.44) < 0.01
