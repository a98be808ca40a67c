"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --profile-case gemm|gemm_mxfp8|quant|quant_mxfp8|grouped

One step = one forward + backward of the NVFP4 Linear of the reference recipe (Hadamard
transform on the transposed activation / gradient copies) on synthetic data:
quantize x, quantize w (every step: the "first microbatch" case), fprop GEMM, quantize dy,
dgrad GEMM, wgrad GEMM (fp32). At N = 1 the shape is the Llama-style MLP up-projection of
the benchmark configuration (tokens 8192, in 4096, out 14336); at N > 1 it is the
tensor-parallel MLP (tokens 8192, hidden 8192, ffn 28672; column-parallel fc1 then
row-parallel fc2, sequence parallel, quantized all-gather) strong-scaled over N ranks.

`value` = GEMM flops of the step (2*M*N*K per GEMM, all ranks) / device time of the step
with inputs resident in HBM (the per-kernel events behind `roofline` are recorded on every
fourth timed step). `e2e` = the same metric through the public `Linear` module with
pinned host inputs copied to the device and a checksum read back inside every timed step (the
copies of step i + 1 are issued on a copy stream while step i computes).
`--impl reference` times the CPU restatement of the reference's PyTorch emulation on a
bounded sample of the same workload on the host cores.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "nvfp4_linear_fwd_bwd_tflops"
UNIT = "TFLOP/s"

C2 = dict(tokens=8192, in_features=4096, out_features=14336)
# DRAM bytes (read + write) per GEMM launch of this workload, average of fprop / dgrad / wgrad,
# from a one-pass ncu capture of this script (dram__bytes_read.sum + dram__bytes_write.sum:
# 275.3, 165.9 and 279.0 MB). Slightly below the algorithmic bytes because part of each output
# is still in L2 when the kernel ends.
GEMM_DRAM_BYTES_PER_LAUNCH = 240.0e6
# sm__pipe_tensor_cycles_active of the NVFP4 pair kernel under ncu (4096 x 9472 x 4096 case,
# profiles/gemm_nvfp4_pair_4096x9472x4096.md)
GEMM_TENSOR_PIPE_ACTIVE_PCT = 59.7
C3 = dict(experts=128, rows=131072, hidden=2048, ffn=768)
C4 = dict(tokens=8192, hidden=8192, ffn=28672)
CPU_SAMPLE = dict(tokens=512, in_features=4096, out_features=3584)
CPU_SAMPLE_MLP = dict(tokens=512, hidden=2048, ffn=3584)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=float(p["hbm_gbs"]), bf16_burst=float(p["bf16_tflops"]),
                    bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------
# CPU arm: numpy restatement of the reference emulation on a bounded sample
# ---------------------------------------------------------------------------------------------
def _cpu_layers(n_gpus):
    """(tokens, in, out) of the layers one CPU sample step runs: a slice of the headline Linear
    at N = 1, a slice of the fc1 + fc2 pair of the tensor-parallel MLP otherwise."""
    if n_gpus == 1:
        s = CPU_SAMPLE
        return [(s["tokens"], s["in_features"], s["out_features"])]
    s = CPU_SAMPLE_MLP
    return [(s["tokens"], s["hidden"], s["ffn"]), (s["tokens"], s["ffn"], s["hidden"])]


def _cpu_step_inputs(n_gpus=1, seed=0):
    import numpy as np
    from oracle import formats as F
    rng = np.random.default_rng(seed)
    layers = []
    for t, k, n in _cpu_layers(n_gpus):
        x = F.bf16_round(rng.standard_normal((t, k)).astype(np.float32))
        w = F.bf16_round((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        dy = F.bf16_round((rng.standard_normal((t, n)) * 1e-3).astype(np.float32))
        layers.append((x, w, dy))
    return layers


def _cpu_sample_flops(n_gpus=1):
    return sum(3 * 2.0 * t * k * n for t, k, n in _cpu_layers(n_gpus))


def _reference_emulation():
    """The reference's own PyTorch emulation from oracle/_ref/ (placed there by oracle/make_ref.py),
    or None when that folder has not been made."""
    try:
        from oracle import make_ref
        return make_ref.load()
    except Exception:
        return None


def cpu_kind():
    return "reference" if _reference_emulation() is not None else "port"


def cpu_run(steps, warmup, n_gpus=1):
    """Times `steps` passes of the NVFP4 linear fwd+bwd on the sample with all host cores:
    the reference's _QuantizedLinear (forward + backward on CPU tensors) when oracle/_ref/
    exists, otherwise the numpy restatement. Returns (TFLOP/s, seconds per sample step)."""
    layers = _cpu_step_inputs(n_gpus)
    ref = _reference_emulation()
    if ref is not None:
        import torch
        torch.set_num_threads(os.cpu_count() or 1)
        params = ref.get_params(ref.QuantizeRecipe.FP4_SUB_CHANNEL_REF)
        tl = [tuple(torch.from_numpy(a).to(torch.bfloat16) for a in layer) for layer in layers]

        def one():
            for x, w, dy in tl:
                xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
                y = ref.QuantizedLinear.apply(xr, None, wr, ref.QuantizeResultCache(), None, False, None, 1, None,
                                              params, torch.bfloat16, True, None, False)
                y.backward(dy)
    else:
        from oracle import linear

        def one():
            for x, w, dy in layers:
                linear.nvfp4_linear_fwd_bwd(x, w, dy, with_rht=True, fused=True)

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / max(1, steps)
    return _cpu_sample_flops(n_gpus) / dt / 1e12, dt


def _cpu_sample_text(n_gpus=1):
    what = ("the reference's own _QuantizedLinear forward + backward (PyTorch emulation, recipe FP4_SUB_CHANNEL_REF) "
            "on CPU tensors" if cpu_kind() == "reference" else
            "numpy restatement of the reference emulation, single-sgemm GEMM variant")
    if n_gpus == 1:
        s = CPU_SAMPLE
        return (f"NVFP4 linear fwd+bwd on tokens={s['tokens']} in={s['in_features']} out={s['out_features']} "
                f"(1/64 of the GEMM flops of the 8192x4096x14336 workload, scaled linearly), {what}")
    s = CPU_SAMPLE_MLP
    return (f"NVFP4 fc1 + fc2 fwd+bwd on tokens={s['tokens']} hidden={s['hidden']} ffn={s['ffn']} (1/512 of the GEMM "
            f"flops of the 8192x8192x28672 MLP; the two layers timed with independent seeded inputs), {what}, "
            f"no sharding (one host)")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    tf, dt = cpu_run(args.steps, args.warmup, args.gpus)
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
        "config": _workload_config(args.gpus),
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": cores, "kind": cpu_kind(), "sample": _cpu_sample_text(args.gpus)},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def _workload_config(n):
    if n == 1:
        return {"workload": "NVFP4 Linear fwd+bwd (fprop, dgrad, wgrad), Llama-style MLP up-projection",
                **C2, "recipe": "1x16 E2M1 + E4M3 block scales + fp32 per-tensor scale, RHT on x^T/dy^T, "
                                "weights re-quantized every step",
                "l2": "inputs (x 64 MiB, w 112 MiB, dy 224 MiB) exceed the 126 MB L2"}
    return {"workload": "tensor-parallel NVFP4 MLP fwd+bwd: column-parallel fc1 -> row-parallel fc2, "
                        "sequence parallel, quantized all-gather, bf16 reduce-scatter",
            **C4, "parallelism": f"tp{n}", "l2": "per-rank operands exceed the 126 MB L2",
            "exchange": ("NVLink peer memory by this library's kernels (pull all-gather, GEMM epilogue that scatters rows + "
                         "local reduce)" if os.environ.get("MT_BENCH_TP_EXCHANGE", "peer") != "nccl" else "NCCL collectives"),
            "cuda_graph": os.environ.get("MT_BENCH_CUDA_GRAPH", "1") != "0"}   # intent; see line["cuda_graph"]


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.05)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def _physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def _tp_workload_single_gpu(torch, Linear, params, dev, kernels, steps=10, warmup=5):
    """The workload the N > 1 runs shard (tensor-parallel MLP, fc1 then fc2, fwd+bwd), unsharded on
    one GPU: the base of the strong-scaling series, reported beside the N = 1 headline."""
    T, H, Fd = C4["tokens"], C4["hidden"], C4["ffn"]
    gen = torch.Generator(device="cpu").manual_seed(4321)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16).to(dev)
    dy = (torch.randn(T, H, generator=gen) * 1e-3).to(torch.bfloat16).to(dev)
    init = lambda t: torch.nn.init.normal_(t, std=0.02)
    fc1 = Linear(H, Fd, bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                 fuse_wgrad_accumulation=True, init_method=init)
    fc2 = Linear(Fd, H, bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                 fuse_wgrad_accumulation=True, init_method=init)
    for m in (fc1, fc2):
        m.weight.main_grad = torch.zeros_like(m.weight, dtype=torch.float32)

    def step():
        xd = x.detach().requires_grad_(True)
        fc1.prefetch_quantized_weight()      # the same calls as the sharded step makes
        fc2.prefetch_quantized_weight()
        y = fc2(fc1(xd, is_first_microbatch=True), is_first_microbatch=True)
        y.backward(dy)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    flops = 6 * 2.0 * T * H * Fd
    return {"value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps,
            "workload": f"NVFP4 MLP fc1+fc2 fwd+bwd, tokens={T}, hidden={H}, ffn={Fd}, no sharding"}


class _HostInputPipeline:
    """Pinned host inputs of the end-to-end step, double-buffered on the device: `take()` hands out
    the buffers of the current step (waiting on the copy stream's event for them) and starts the
    copies of the next step's inputs into the other pair, so that they cross PCIe under the
    current step's kernels. Every step's inputs are still copied once per step inside the timed
    region; the pair that a step reads was last read two steps earlier, whose result the host has
    already read back."""

    def __init__(self, torch, dev, host_tensors):
        self.torch, self.host = torch, host_tensors
        self.stream = torch.cuda.Stream(device=dev)
        self.slots = [[torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host_tensors] for _ in range(2)]
        self.ready = [[torch.cuda.Event() for _ in host_tensors] for _ in range(2)]
        self.step = 0
        self._issue(0)

    def _issue(self, slot):
        with self.torch.cuda.stream(self.stream):
            for dst, src, ev in zip(self.slots[slot], self.host, self.ready[slot]):
                dst.copy_(src, non_blocking=True)
                ev.record(self.stream)

    def take(self):
        """-> list of (device tensor, event to wait for before reading it)."""
        slot = self.step & 1
        self.step += 1
        self._issue(slot ^ 1)
        return list(zip(self.slots[slot], self.ready[slot]))

    @property
    def bytes_per_step(self):
        return sum(t.numel() * t.element_size() for t in self.host)


def _timed_loop(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _other_configs_single_gpu(torch, dev, steps=5, warmup=3):
    """The two MXFP8 configurations beside the headline one, on one GPU: the dense forward
    (4096^3) and the grouped (MoE expert) fc1 + fc2 forward+backward through GroupedLinear."""
    import numpy as np
    from minitransformer_b200.module import config as mt_config
    from minitransformer_b200.module.group_linear import GroupedLinear
    out = {}
    params = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    op = params.quantize_op
    gen = torch.Generator(device="cpu").manual_seed(99)

    # dense MXFP8 forward: quantize x and w (row-wise), one GEMM
    M = N = Kd = 4096
    x = torch.randn(M, Kd, generator=gen).to(torch.bfloat16).to(dev)
    w = (torch.randn(N, Kd, generator=gen) * 0.02).to(torch.bfloat16).to(dev)

    def fwd():
        qx = op.quantize(x, params.x_params, return_transpose=False)
        qw = op.quantize(w, params.w_params, return_transpose=False)
        return op.qgemm(qx.data, qw.data, params.mm_fprop, torch.bfloat16, qx.scale, qw.scale)

    ms = _timed_loop(torch, fwd, 20, warmup)
    qx = op.quantize(x, params.x_params, return_transpose=False)
    qw = op.quantize(w, params.w_params, return_transpose=False)
    ms_g = _timed_loop(torch, lambda: op.qgemm(qx.data, qw.data, params.mm_fprop, torch.bfloat16, qx.scale, qw.scale),
                       20, warmup)
    out["mxfp8_linear_fwd_4096"] = {"value": 2.0 * M * N * Kd / (ms * 1e-3) / 1e12, "unit": UNIT, "ms": ms,
                                    "gemm_only_tflops": 2.0 * M * N * Kd / (ms_g * 1e-3) / 1e12,
                                    "workload": "MXFP8 quantize(x) + quantize(w) + GEMM, M=N=K=4096"}
    del x, w, qx, qw

    # grouped MXFP8: 128 experts, 131072 rows, Zipf(1.1) group sizes, hidden 2048, ffn 768
    G, R, H, Fd = C3["experts"], C3["rows"], C3["hidden"], C3["ffn"]
    rng = np.random.default_rng(1234)
    p = 1.0 / np.arange(1, G + 1) ** 1.1
    m_splits = np.bincount(rng.choice(G, size=R, p=p / p.sum()), minlength=G).tolist()
    init = lambda t: torch.nn.init.normal_(t, std=0.02)
    kw = dict(bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params, init_method=init)
    fused = os.environ.get("MT_BENCH_MOE_FUSED", "1") != "0"
    kw["fuse_wgrad_accumulation"] = fused
    fc1, fc2 = GroupedLinear(G, H, Fd, **kw), GroupedLinear(G, Fd, H, **kw)
    if fused:
        # Megatron-style fp32 main_grad buffers, one block per layer
        for m in (fc1, fc2):
            block = torch.zeros(G, m.out_features, m.in_features, dtype=torch.float32, device=dev)
            for i in range(G):
                getattr(m, f"weight{i}").main_grad = block[i]
    xg = torch.randn(R, H, generator=gen).to(torch.bfloat16).to(dev)
    dyg = (torch.randn(R, H, generator=gen) * 1e-3).to(torch.bfloat16).to(dev)

    def moe_step(first=True):
        if not fused:
            for m in (fc1, fc2):
                for prm in m.parameters():
                    prm.grad = None
        xd = xg.detach().requires_grad_(True)
        y = fc2(fc1(xd, m_splits, is_first_microbatch=first), m_splits, is_first_microbatch=first)
        y.backward(dyg)

    ms = _timed_loop(torch, moe_step, steps, warmup)
    # later microbatches of a step: quantized expert weights kept, wgrad accumulated into main_grad
    ms_steady = _timed_loop(torch, lambda: moe_step(False), steps, 1)
    # host time to enqueue one step (the GPU still busy with earlier ones)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(3):
        moe_step()
    host_ms = (time.perf_counter() - t0) / 3 * 1e3
    torch.cuda.synchronize()
    flops = 6 * 2.0 * R * H * Fd
    q_bytes = (2 * R * (H + Fd) + 2 * 2 * G * H * Fd) * 4.0625   # x, h, dy, dh and both weight blocks, row + transposed
    out["mxfp8_grouped_linear_fwd_bwd"] = {
        "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms,
        "steady_microbatch_weights_cached": {"value": flops / (ms_steady * 1e-3) / 1e12, "ms_per_step": ms_steady},
        "host_enqueue_ms_per_step": host_ms,
        "frac_of_nominal_4500": flops / (ms * 1e-3) / 1e12 / 4500.0,
        "quantize_algorithmic_bytes_per_step": q_bytes,
        "workload": f"GroupedLinear fc1+fc2 fwd+bwd, {G} experts, {R} rows (Zipf 1.1 sizes), hidden {H}, ffn {Fd}"}
    return out


def tp_parity_check(group, T=2048, H=1024, Fd=4096, recipe="fp4_subchannel_scaling", peer=True):
    """Parity of the tensor-parallel path on the ranks of `group` (one GPU each), run in-process
    before the timed loop of `--gpus N` and by tests/test_gpu_tp.py:
      * bit-exact: the quantized all-gather (codes, GEMM-layout scales, per-tensor abs-max)
        equals quantizing the gathered tensor, and the wgrad GEMM over gathered K slabs equals
        the GEMM on the interleaved transposed copy;
      * within tolerance: column-parallel fc1 -> row-parallel fc2 forward + backward against
        the same layers built from this rank's weight shards and run without any collective on
        the full activations (partial sums reduced in fp32), once more with memory_saving.
    The shape takes the copy-free gather on every world size up to 8. peer=True builds the layers
    with ub_overlap_ag / ub_overlap_rs (exchanges over NVLink peer memory by this library's own
    kernels, what the benchmark times); peer=False keeps them on the process group. Returns a
    dict; raises nothing, the caller decides."""
    import torch
    import torch.distributed as dist
    from minitransformer_b200 import kernels as K
    from minitransformer_b200.module import config
    from minitransformer_b200.module.linear import Linear, _QuantizedLinear
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rcp = config.QuantizeRecipe(recipe)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    w1 = (torch.randn(Fd, H, generator=g) * 0.02).to(torch.bfloat16).cuda()
    w2 = (torch.randn(H, Fd, generator=g) * 0.02).to(torch.bfloat16).cuda()
    dy = (torch.randn(T, H, generator=g) * 1e-3).to(torch.bfloat16).cuda()
    w1s, w2s = w1.chunk(world, 0)[rank].contiguous(), w2.chunk(world, 1)[rank].contiguous()

    def relf(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))

    # this rank's share of the work, with no process group: full activations, sharded weights
    p0 = config.get_qlinear_params_from_predefined(rcp)
    kw = dict(bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=p0)
    e1, e2 = Linear(H, w1s.shape[0], **kw), Linear(w2s.shape[1], H, **kw)
    with torch.no_grad():
        e1.weight.copy_(w1s)
        e2.weight.copy_(w2s)
    xe = x.clone().requires_grad_(True)
    he = e1(xe)
    ye = e2(he)
    ye.backward(dy)
    y_sum, dx_sum = ye.detach().float(), xe.grad.float()
    dist.all_reduce(y_sum, group=group)
    dist.all_reduce(dx_sum, group=group)

    errs, exact = {}, True
    runs = {}
    for mem_saving in (False, True):
        p = config.get_qlinear_params_from_predefined(rcp)
        p.memory_saving = mem_saving
        kw = dict(bias=False, params_dtype=torch.bfloat16, device="cuda", qlinear_params=p, tp_group=group,
                  sequence_parallel=True, ub_overlap_ag=peer, ub_overlap_rs=peer)
        fc1 = Linear(H, Fd, parallel_mode="column", ub_name="parity_fc1", **kw)
        fc2 = Linear(Fd, H, parallel_mode="row", ub_name="parity_fc2", **kw)
        with torch.no_grad():
            fc1.weight.copy_(w1s)
            fc2.weight.copy_(w2s)
        xd = x.chunk(world, 0)[rank].clone().requires_grad_(True)
        h = fc1(xd)
        y = fc2(h)
        y.backward(dy.chunk(world, 0)[rank].contiguous())
        torch.cuda.synchronize()
        tag = "_memory_saving" if mem_saving else ""
        errs["h" + tag] = relf(h, he)
        errs["y" + tag] = relf(y, y_sum.chunk(world, 0)[rank])
        errs["dx" + tag] = relf(xd.grad, dx_sum.chunk(world, 0)[rank])
        errs["dw1" + tag] = relf(fc1.weight.grad, e1.weight.grad)
        errs["dw2" + tag] = relf(fc2.weight.grad, e2.weight.grad)
        runs[mem_saving] = (h.detach(), fc1.weight.grad, fc2.weight.grad)
    # the local GEMMs see identical operands in both modes
    exact &= all(torch.equal(a, b) for a, b in zip(runs[False], runs[True]))
    exact &= torch.equal(runs[False][0], he.detach())

    # quantized gather == quantize(gathered), in the form the GEMMs read
    p = config.get_qlinear_params_from_predefined(rcp)
    xs = x.chunk(world, 0)[rank].contiguous()
    qf = p.quantize_op.quantize(x, p.x_params, return_transpose=True)
    pg = None
    if peer:
        from minitransformer_b200.distributed.peer import get_peer_group
        pg = get_peer_group(group, x.device)
    qs = _QuantizedLinear.quantize_optionally_allgather(p.quantize_op, xs, p.x_params, True, True, True, group,
                                                        weight_shape=(Fd, H), peer_group=pg, site="parity:x")
    for hnd in tuple(getattr(qs, "_pending_handles", ())) + tuple(getattr(qs, "_pending_handles_t", ())):
        hnd.wait()
    copy_free = qs.data_t is not None and qs.data_t.dim() == 3
    exact &= torch.equal(qs.data.view(torch.uint8), qf.data.view(torch.uint8))
    if copy_free:
        exact &= torch.equal(qs.scale_swz.view(-1), qf.scale_swz.view(-1))
        exact &= torch.equal(qs.data_t.view(torch.uint8).permute(1, 0, 2).reshape(H, -1), qf.data_t.view(torch.uint8))
        if qf.global_amax_row is not None:
            args = lambda q: (q.data_t, q.scale_t_swz, q.global_amax_col)
            d_plain = K.gemm_nvfp4(*args(qf), *args(qf), out_dtype=torch.float32)
            d_slab = K.gemm_nvfp4(*args(qf), *args(qs), out_dtype=torch.float32)
            d_slab2 = K.gemm_nvfp4(*args(qs), *args(qs), out_dtype=torch.float32)
        else:
            args = lambda q: (q.data_t.view(torch.uint8), q.scale_t_swz)
            d_plain = K.gemm_mxfp8(*args(qf), *args(qf), out_dtype=torch.float32)
            d_slab = K.gemm_mxfp8(*args(qf), *args(qs), out_dtype=torch.float32)
            d_slab2 = K.gemm_mxfp8(*args(qs), *args(qs), out_dtype=torch.float32)
        exact &= torch.equal(d_plain, d_slab) and torch.equal(d_plain, d_slab2)
    else:
        exact &= torch.equal(qs.scale.view(torch.uint8), qf.scale.view(torch.uint8)[: qs.scale.shape[0]])
        exact &= torch.equal(qs.data_t.view(torch.uint8), qf.data_t.view(torch.uint8))
    if qf.global_amax_row is not None:
        exact &= float(qs.global_amax_row) == float(qf.global_amax_row)
        exact &= float(qs.global_amax_col) == float(qf.global_amax_col)
    status = K.read_device_status()

    # local GEMMs see identical quantized operands (1e-3); the two reduce-scattered results carry
    # the rounding of bf16 partial sums (1e-2)
    tight = max(v for k, v in errs.items() if k.split("_")[0] in ("h", "dw1", "dw2"))
    loose = max(v for k, v in errs.items() if k.split("_")[0] in ("y", "dx"))
    ok = bool(exact) and tight <= 1e-3 and loose <= 1e-2 and status == 0
    flags = torch.tensor([1.0 if ok else 0.0, 1.0 if exact else 0.0, -tight, -loose], device="cuda")
    dist.all_reduce(flags, op=dist.ReduceOp.MIN, group=group)
    return {"tp": world, "ok": bool(flags[0] > 0.5), "bit_exact": bool(flags[1] > 0.5),
            "max_rel_frob": float(-flags[2]), "max_rel_frob_reduced_outputs": float(-flags[3]),
            "tolerance": {"local_gemms": 1e-3, "reduce_scattered": 1e-2}, "copy_free_gather": bool(copy_free),
            "shape": {"tokens": T, "hidden": H, "ffn": Fd}, "recipe": recipe, "memory_saving_checked": True,
            "exchange": "peer memory (own kernels)" if pg is not None else "process group (NCCL)",
            "rank_errors": errs if rank == 0 else None}


# ---------------------------------------------------------------------------------------------
# Configuration 5: Llama-style decoder step with every Linear swapped for the drop-in module
# ---------------------------------------------------------------------------------------------
C5 = dict(layers=8, hidden=4096, heads=32, kv_heads=8, ffn=14336, vocab=32000, seq=4096, micro_batch=2)


def build_llama_decoder(torch, dims, params, tp_group=None, peer=True, device="cuda"):
    """Llama-style decoder (RMSNorm, grouped-query attention through torch SDPA, gated SiLU MLP)
    whose linears are the drop-in Linear under `params`. With a tensor-parallel group: Megatron
    layout with sequence parallelism (qkv and the gated fc1 column-parallel with their heads /
    ffn columns sharded, proj and fc2 row-parallel, token-sharded activations between blocks, a
    vocabulary-parallel head and loss). Input ids [micro_batch, seq]; returns the mean loss."""
    import torch.distributed as dist
    from minitransformer_b200.module.linear import Linear
    tp = dist.get_world_size(tp_group) if tp_group is not None else 1
    rank = dist.get_rank(tp_group) if tp_group is not None else 0
    H, heads, kvh, ffn, vocab = dims["hidden"], dims["heads"], dims["kv_heads"], dims["ffn"], dims["vocab"]
    hd = H // heads
    assert heads % tp == 0 and kvh % tp == 0 and ffn % tp == 0 and vocab % tp == 0
    init = lambda t: torch.nn.init.normal_(t, std=0.02)

    def lin(i, o, mode, name):
        kw = dict(bias=False, params_dtype=torch.bfloat16, device=device, qlinear_params=params, init_method=init)
        if tp > 1:
            kw.update(parallel_mode=mode, sequence_parallel=True, tp_group=tp_group, ub_overlap_ag=peer,
                      ub_overlap_rs=peer, ub_name=name)
        return Linear(i, o, **kw)

    class RMSNorm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(H, dtype=torch.bfloat16, device=device))

        def forward(self, x):
            v = x.float()
            return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * self.weight

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2 = RMSNorm(), RMSNorm()
            self.qkv = lin(H, (heads + 2 * kvh) * hd, "column", "qkv")   # this rank: its heads' [q | k | v]
            self.proj = lin(H, H, "row", "proj")
            self.fc1 = lin(H, 2 * ffn, "column", "fc1")                   # this rank: [gate shard | up shard]
            self.fc2 = lin(ffn, H, "row", "fc2")

        def forward(self, x, B, S):                                       # x [B*S / tp, H] (token shard)
            nh, nkv = heads // tp, kvh // tp
            qkv = self.qkv(self.norm1(x))                                 # [B*S, (nh + 2 nkv) hd]
            q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
            q = q.view(B, S, nh, hd).transpose(1, 2)
            k = k.view(B, S, nkv, hd).transpose(1, 2).repeat_interleave(nh // nkv, 1)
            v = v.view(B, S, nkv, hd).transpose(1, 2).repeat_interleave(nh // nkv, 1)
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.proj(a.transpose(1, 2).reshape(B * S, nh * hd))
            g, u = self.fc1(self.norm2(x)).chunk(2, dim=-1)
            return x + self.fc2(torch.nn.functional.silu(g) * u)

    class Decoder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(vocab, H, dtype=torch.bfloat16, device=device)
            self.blocks = torch.nn.ModuleList([Block() for _ in range(dims["layers"])])
            self.norm = RMSNorm()
            self.head = lin(H, vocab, "column", "head")

        def forward(self, ids, targets):
            B, S = ids.shape
            x = self.emb(ids).view(B * S, H)
            if tp > 1:
                x = x.chunk(tp, 0)[rank]
            for b in self.blocks:
                x = b(x, B, S)
            logits = self.head(self.norm(x)).float()                      # [B*S, vocab / tp]
            t = targets.view(-1)
            if tp == 1:
                return torch.nn.functional.cross_entropy(logits, t)
            # vocabulary-parallel cross entropy
            import torch.distributed.nn.functional as dfn
            vs = vocab // tp
            m = logits.max(dim=-1).values.detach()
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=tp_group)
            z = dfn.all_reduce((logits - m[:, None]).exp().sum(-1), group=tp_group)
            local = (t >= rank * vs) & (t < (rank + 1) * vs)
            idx = (t - rank * vs).clamp(0, vs - 1)
            picked = torch.where(local, logits.gather(1, idx[:, None])[:, 0] - m, torch.zeros_like(m))
            picked = dfn.all_reduce(picked, group=tp_group)
            return (z.log() - picked).mean()

    return Decoder()


def llama_linear_flops(dims, with_head=True):
    """GEMM flops of one forward + backward step: 2 M N K per GEMM, three GEMMs per Linear."""
    T, H, hd = dims["seq"] * dims["micro_batch"], dims["hidden"], dims["hidden"] // dims["heads"]
    per_layer = (dims["heads"] + 2 * dims["kv_heads"]) * hd + H + 2 * dims["ffn"]
    f = 3 * 2.0 * T * H * per_layer * dims["layers"] + 3 * 2.0 * T * H * dims["ffn"] * dims["layers"]
    return f + (3 * 2.0 * T * H * dims["vocab"] if with_head else 0.0)


def _llama_step_bench(torch, dims, tp_group, dev, steps=3, warmup=2, peer=True):
    """Times forward + backward of the decoder (MXFP8 recipe); returns the `other_configs` entry."""
    import torch.distributed as dist
    from minitransformer_b200.module import config as mt_config
    params = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
    n = dist.get_world_size(tp_group) if tp_group is not None else 1
    torch.manual_seed(1234)
    model = build_llama_decoder(torch, dims, params, tp_group, peer=peer, device=dev)
    g = torch.Generator(device="cpu").manual_seed(77)
    ids = torch.randint(0, dims["vocab"], (dims["micro_batch"], dims["seq"]), generator=g).to(dev)
    tgt = torch.randint(0, dims["vocab"], (dims["micro_batch"], dims["seq"]), generator=g).to(dev)
    loss = None

    def step():
        nonlocal loss
        for p_ in model.parameters():
            p_.grad = None
        loss = model(ids, tgt)
        # every rank holds the same loss; the autograd-aware all-reduces of the vocabulary-parallel
        # loss sum the ranks' gradients, so each rank back-propagates its 1/n share
        (loss / n).backward()

    graph_env = os.environ.get("MT_BENCH_CUDA_GRAPH", "")
    graphed = tp_group is not None and (graph_env == "1" or (graph_env != "0" and peer))   # as for the MLP step
    # warm-up on a side stream, as graph capture of a backward pass wants it (the gradient
    # accumulation nodes remember the stream they first ran on)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(max(warmup, 3 if graphed else 0)):
            step()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize()
    if tp_group is not None:
        dist.barrier()
    run = step
    if graphed:
        # the sharded step is a few hundred short kernels: replayed from a CUDA graph, like the MLP step
        for p_ in model.parameters():
            p_.grad = None
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loss = model(ids, tgt)
            (loss / n).backward()
        run = graph.replay
        run()
        torch.cuda.synchronize()
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if tp_group is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=tp_group)
    ms = float(ms.item())
    flops = llama_linear_flops(dims)
    return {"ms_per_step": ms, "linear_tflops_per_gpu": flops / n / (ms * 1e-3) / 1e12, "unit": UNIT,
            "linear_flops_per_step": flops, "loss": float(loss.item()), "steps": steps, "tp": n, "cuda_graph": graphed,
            "workload": (f"{dims['layers']}-layer Llama-style decoder fwd+bwd, MXFP8 recipe on every Linear (LM head "
                         f"included), hidden {dims['hidden']}, {dims['heads']} heads / {dims['kv_heads']} KV heads, "
                         f"ffn {dims['ffn']}, vocab {dims['vocab']}, seq {dims['seq']} x micro-batch "
                         f"{dims['micro_batch']}, torch SDPA, sequence-parallel TP={n}, random-init weights, uniform ids")}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from minitransformer_b200 import kernels
    from minitransformer_b200.module import config as mt_config
    from minitransformer_b200.module.linear import Linear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        tp_group = dist.group.WORLD
    n = world
    assert n == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    params = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.FP4_SUB_CHANNEL)
    op = params.quantize_op
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)

    def randn_bf16(shape, std, pin=False):
        t = (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
        return t.pin_memory() if pin else t

    gemm_ms, quant_ms = [], []
    parity = base = None
    quick = os.environ.get("MT_BENCH_QUICK", "0") == "1"    # A/B timing runs: only the timed loop of the sharded step
    if n > 1 and not quick:
        # parity first: the sharded path must reproduce the per-rank emulation before it is timed
        parity = tp_parity_check(tp_group, peer=os.environ.get("MT_BENCH_TP_EXCHANGE", "peer") != "nccl")
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": n, "parity": parity, "error": "tensor-parallel parity failed"}),
                      flush=True)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(3)
        # base of the strong-scaling series: the same MLP unsharded, timed on rank 0 alone. The
        # other ranks block on the rendezvous store meanwhile (a socket wait): waiting in an NCCL
        # barrier would spin one host thread per rank beside rank 0's enqueue loop.
        store = dist.distributed_c10d._get_default_store()
        if rank == 0:
            base = _tp_workload_single_gpu(torch, Linear, params, dev, kernels)
            torch.cuda.empty_cache()
            store.set("mt_bench_base_done", "1")
        else:
            store.wait(["mt_bench_base_done"])
        dist.barrier()

    if n == 1:
        T, K_in, N_out = C2["tokens"], C2["in_features"], C2["out_features"]
        x_h, dy_h = randn_bf16((T, K_in), 1.0, pin=True), randn_bf16((T, N_out), 1e-3, pin=True)
        w = randn_bf16((N_out, K_in), 0.02).to(dev)
        x, dy = x_h.to(dev), dy_h.to(dev)
        flops_step = 3 * 2.0 * T * K_in * N_out
        gemm_flops_each = 2.0 * T * K_in * N_out
        dw = torch.empty((N_out, K_in), dtype=torch.float32, device=dev)

        def timed(fn, bucket):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn()
            e1.record()
            bucket.append((e0, e1))
            return r

        def step(record):
            tq = (lambda fn: timed(fn, quant_ms)) if record else (lambda fn: fn())
            tg = (lambda fn: timed(fn, gemm_ms)) if record else (lambda fn: fn())
            qx = op.quantize(x, params.x_params, return_transpose=True)
            qw = op.quantize(w, params.w_params, return_transpose=True)
            y = tg(lambda: op.qgemm(qx.data, qw.data, params.mm_fprop, torch.bfloat16, qx.scale, qw.scale,
                                    global_amax_qx=qx.global_amax_row, global_amax_qw=qw.global_amax_row))
            qg = tq(lambda: op.quantize(dy, params.g_params, return_transpose=True))
            dx = tg(lambda: op.qgemm(qg.data, qw.data_t, params.mm_dgrad, torch.bfloat16, qg.scale, qw.scale_t,
                                     global_amax_qx=qg.global_amax_row, global_amax_qw=qw.global_amax_col))
            tg(lambda: op.qgemm(qg.data_t, qx.data_t, params.mm_wgrad, torch.float32, qg.scale_t, qx.scale_t,
                                out=dw, global_amax_qx=qg.global_amax_col, global_amax_qw=qx.global_amax_col))
            return y, dx

        def variant_step(p_, qw_cached=None):
            """The same three GEMMs with another recipe, or with the weight's quantized copies kept
            from an earlier microbatch (the module's weight_qresult_cache)."""
            o_ = p_.quantize_op
            qx = o_.quantize(x, p_.x_params, return_transpose=True)
            qw = qw_cached if qw_cached is not None else o_.quantize(w, p_.w_params, return_transpose=True)
            o_.qgemm(qx.data, qw.data, p_.mm_fprop, torch.bfloat16, qx.scale, qw.scale,
                     global_amax_qx=qx.global_amax_row, global_amax_qw=qw.global_amax_row)
            qg = o_.quantize(dy, p_.g_params, return_transpose=True)
            o_.qgemm(qg.data, qw.data_t, p_.mm_dgrad, torch.bfloat16, qg.scale, qw.scale_t,
                     global_amax_qx=qg.global_amax_row, global_amax_qw=qw.global_amax_col)
            o_.qgemm(qg.data_t, qx.data_t, p_.mm_wgrad, torch.float32, qg.scale_t, qx.scale_t, out=dw,
                     global_amax_qx=qg.global_amax_col, global_amax_qw=qx.global_amax_col)

        def library_comparator():
            """cuBLASLt's block-scaled NVFP4 GEMM (through torch._scaled_mm) on the same quantized
            operands and shapes: a measured ceiling for the GEMM kernels, not a product path.
            Its result lacks the per-tensor factor, which does not change the timing."""
            try:
                f4, f8 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
                qx = op.quantize(x, params.x_params, return_transpose=True)
                qw = op.quantize(w, params.w_params, return_transpose=True)
                qg = op.quantize(dy, params.g_params, return_transpose=True)
                cases = {"fprop": (qx.data, qx.scale_swz, qw.data, qw.scale_swz, torch.bfloat16),
                         "dgrad": (qg.data, qg.scale_swz, qw.data_t, qw.scale_t_swz, torch.bfloat16),
                         "wgrad": (qg.data_t, qg.scale_t_swz, qx.data_t, qx.scale_t_swz, torch.float32)}
                out = {}
                for name, (a_, sa_, b_, sb_, dt) in cases.items():
                    fn = lambda: torch._scaled_mm(a_.view(f4), b_.view(f4).t(), scale_a=sa_.view(f8),
                                                  scale_b=sb_.view(f8), out_dtype=dt)
                    try:
                        ms = _timed_loop(torch, fn, 10, 3)
                        out[name] = {"tflops": gemm_flops_each / (ms * 1e-3) / 1e12, "ms": ms}
                    except Exception as e:   # a shape / dtype combination the library does not take
                        out[name] = {"unavailable": repr(e)[:120]}
                return out
            except Exception as e:
                return {"unavailable": repr(e)[:200]}

        def measure_variants():
            """Variants and the headline recipe timed in alternating bursts of 5 steps, so that all
            of them see the same clocks (a long run settles at lower SM clocks under the power cap
            than the headline's short timed region)."""
            qw_keep = op.quantize(w, params.w_params, return_transpose=True)
            p_norht = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.FP4_SUB_CHANNEL_NO_RHT)
            p_mx = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
            cases = {
                "headline_recipe_again": lambda: variant_step(params),
                "steady_microbatch_weights_cached": lambda: variant_step(params, qw_keep),
                "without_rht": lambda: variant_step(p_norht),
                "mxfp8_same_shape": lambda: variant_step(p_mx),
            }
            total = {k: 0.0 for k in cases}
            for fn in cases.values():
                fn()
            rounds, burst = 4, 5
            for _ in range(rounds):
                for k, fn in cases.items():
                    total[k] += _timed_loop(torch, fn, burst, 1) * burst
            return {k: {"value": flops_step / (t / (rounds * burst) * 1e-3) / 1e12, "unit": UNIT,
                        "ms_per_step": t / (rounds * burst)} for k, t in total.items()}

        lin = Linear(K_in, N_out, bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                     fuse_wgrad_accumulation=True)
        with torch.no_grad():
            lin.weight.copy_(w)
        lin.weight.main_grad = torch.zeros((N_out, K_in), dtype=torch.float32, device=dev)

        def module_step():
            """The same step through the public Linear module with inputs resident in HBM: autograd,
            the weight cache protocol and main_grad fusion inside the timed region."""
            xd = x.detach().requires_grad_(True)
            lin(xd, is_first_microbatch=True).backward(dy)

        inputs = _HostInputPipeline(torch, dev, [x_h, dy_h])

        def e2e_step():
            # this step's x and dy were sent while the previous step ran; the next step's start now
            main = torch.cuda.current_stream(dev)
            (xb, x_ready), (dyb, dy_ready) = inputs.take()
            main.wait_event(x_ready)
            xd = xb.detach().requires_grad_(True)
            y = lin(xd, is_first_microbatch=True)
            main.wait_event(dy_ready)
            y.backward(dyb)
            chk = torch.stack([y.sum(dtype=torch.float32), xd.grad.sum(dtype=torch.float32), lin.weight.main_grad.sum()])
            return chk.cpu()

        h2d = inputs.bytes_per_step
        d2h = 12
        launches_per_step = None
    else:
        T, H, Fd = C4["tokens"], C4["hidden"], C4["ffn"]
        assert T % n == 0 and Fd % n == 0
        peer = os.environ.get("MT_BENCH_TP_EXCHANGE", "peer") != "nccl"   # "nccl": the process-group exchanges, for comparison
        x_h, dy_h = randn_bf16((T // n, H), 1.0, pin=True), randn_bf16((T // n, H), 1e-3, pin=True)
        fc1 = Linear(H, Fd, bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                     parallel_mode="column", sequence_parallel=True, tp_group=tp_group, fuse_wgrad_accumulation=True,
                     init_method=lambda t: torch.nn.init.normal_(t, std=0.02), ub_overlap_ag=peer, ub_overlap_rs=peer,
                     ub_name="fc1")
        fc2 = Linear(Fd, H, bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                     parallel_mode="row", sequence_parallel=True, tp_group=tp_group, fuse_wgrad_accumulation=True,
                     init_method=lambda t: torch.nn.init.normal_(t, std=0.02), ub_overlap_ag=peer, ub_overlap_rs=peer,
                     ub_name="fc2")
        for m in (fc1, fc2):
            m.weight.main_grad = torch.zeros_like(m.weight, dtype=torch.float32)
        x, dy = x_h.to(dev), dy_h.to(dev)
        flops_step = 6 * 2.0 * T * H * Fd  # whole job: fc1 + fc2, fprop + dgrad + wgrad
        gemm_flops_each = 2.0 * T * H * Fd / n

        def mlp(xd, dyd):
            # the step's weights are final: both layers quantize theirs on a side stream, beside the
            # gather of x, instead of between the GEMMs
            if os.environ.get("MT_BENCH_PREFETCH", "1") != "0":
                fc1.prefetch_quantized_weight()
                fc2.prefetch_quantized_weight()
            # no activation between fc1 and fc2: the benchmark configuration names none
            y = fc2(fc1(xd, is_first_microbatch=True), is_first_microbatch=True)
            y.backward(dyd)
            return y

        def eager_step(record):
            xd = x.detach().requires_grad_(True)
            y = mlp(xd, dy)
            return y, xd.grad

        # The sharded step holds ~50 short kernels: at 8 ranks it would be bound by the host
        # enqueueing them (about 1.6 ms of Python per step), so the whole forward + backward is
        # captured once into a CUDA graph and replayed (MT_BENCH_CUDA_GRAPH=0 times the eager step).
        # Replay is for the peer-memory exchanges (this library's own kernels). With the process
        # group's collectives (MT_BENCH_TP_EXCHANGE=nccl, or no peer access on this box) the step is
        # timed eagerly unless MT_BENCH_CUDA_GRAPH=1 asks for capture: NCCL collectives and their
        # side streams inside a capture are not something this benchmark should depend on.
        from minitransformer_b200.distributed.peer import get_peer_group
        peer_active = peer and get_peer_group(tp_group, dev) is not None
        graph_env = os.environ.get("MT_BENCH_CUDA_GRAPH", "")
        use_graph = graph_env == "1" or (graph_env != "0" and peer_active)
        step = eager_step
        if use_graph:
            x_static = x.detach().clone().requires_grad_(True)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(3):                      # warm-up: one-time setup, shared-buffer allocation
                    x_static.grad = None
                    mlp(x_static, dy)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            x_static.grad = None
            before = kernels.LAUNCH_COUNT
            try:
                with torch.cuda.graph(graph):
                    y_static = mlp(x_static, dy)
            except RuntimeError as e:       # the same on every rank: time the eager step instead
                use_graph = False
                if rank == 0:
                    print(f"[bench] graph capture failed ({str(e)[:200]}); timing the eager step", file=sys.stderr)
                torch.cuda.synchronize()
            launches_per_replay = kernels.LAUNCH_COUNT - before

            def graph_step(record):
                graph.replay()
                kernels.LAUNCH_COUNT += launches_per_replay
                return y_static, x_static.grad

            if use_graph:
                step = graph_step

        inputs = _HostInputPipeline(torch, dev, [x_h, dy_h])

        def e2e_step():
            main = torch.cuda.current_stream(dev)
            (xb, x_ready), (dyb, dy_ready) = inputs.take()
            main.wait_event(x_ready)
            main.wait_event(dy_ready)
            if use_graph:
                # the captured step reads fixed buffers: refill them (device-to-device) and replay
                with torch.no_grad():
                    x_static.copy_(xb)
                    dy.copy_(dyb)
                y, xgrad = graph_step(True)
            else:
                xd = xb.detach().requires_grad_(True)
                y = mlp(xd, dyb)
                xgrad = xd.grad
            chk = torch.stack([y.sum(dtype=torch.float32), xgrad.sum(dtype=torch.float32)])
            return chk.cpu()

        h2d = inputs.bytes_per_step
        d2h = 8

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run_timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kernels.LAUNCH_COUNT = 0
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = kernels.LAUNCH_COUNT
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, launches

    sampler = ClockSampler(_physical_gpu_index(local_rank)) if rank == 0 else None
    if sampler:
        sampler.start()
    # Per-kernel events (the roofline's launch durations) are recorded inside the timed region on
    # every fourth step only, the first timed step included: an event between two kernels costs a
    # few microseconds and keeps the second from being launched ahead of the first one's end.
    calls = {"n": 0}

    def timed_step():
        i = calls["n"] - args.warmup      # index inside the timed region (warm-up steps come first)
        calls["n"] += 1
        return step(i >= 0 and i % 4 == 0)

    ms_step, launches = run_timed(timed_step, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    # every recorded event pair lies in the timed region
    torch.cuda.synchronize()
    g_ms = [a.elapsed_time(b) for a, b in gemm_ms] if n == 1 else []
    q_ms = [a.elapsed_time(b) for a, b in quant_ms] if n == 1 else []
    e2e_ms = float("nan") if quick and n > 1 else run_timed(e2e_step, max(2, min(args.steps, 10)), 2)[0]

    c5 = None
    if n > 1 and not quick and all(C5[k] % n == 0 for k in ("heads", "kv_heads", "ffn", "vocab")):
        # configuration 5 on the same ranks (every rank takes part; reported in the N > 1 line)
        del fc1, fc2
        torch.cuda.empty_cache()
        c5 = _llama_step_bench(torch, C5, tp_group, dev, peer=peer_active)

    status = kernels.read_device_status()
    if status != 0:
        raise SystemExit(f"device status word is {status}: a bounded device-side wait expired")

    if rank == 0:
        peaks = _peaks()
        value = flops_step / (ms_step * 1e-3) / 1e12
        e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if n == 1 else "strong",
            "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic", "config": _workload_config(n),
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
        }
        if n > 1:
            line["cuda_graph"] = bool(use_graph)
        if n > 1 and not quick:
            line["parity"] = parity
            line["scaling_base_ms"] = base["ms_per_step"]
            line["scaling_base"] = base["workload"] + ", timed on rank 0 before the sharded run"
            line["efficiency_vs_tp1"] = base["ms_per_step"] / (n * ms_step)
            line["other_configs"] = {"llama8_mxfp8_tp_step": c5}
        if n == 1:
            g_avg = sum(g_ms) / len(g_ms)
            T_, H_, F_ = C2["tokens"], C2["in_features"], C2["out_features"]
            # codes (0.5 B/elt) and scales (one byte per 16 elements) of both operands, plus the output
            gemm_alg_bytes = ((T_ * H_ + F_ * H_) * 0.5625 + T_ * F_ * 2          # fprop, bf16 out
                              + (T_ * F_ + H_ * F_) * 0.5625 + T_ * H_ * 2        # dgrad, bf16 out
                              + (F_ * T_ + H_ * T_) * 0.5625 + F_ * H_ * 4) / 3   # wgrad, fp32 out
            achieved = gemm_flops_each / (g_avg * 1e-3) / 1e12
            # the timed region is short (tens of ms at full clocks): the burst figure is the denominator
            peak = 4.0 * peaks["bf16_burst"]
            line["roofline"] = {
                "bound": "tensor", "kernel": "gemm_blockscaled_pair_kernel<NVFP4> (fprop/dgrad/wgrad average)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": GEMM_DRAM_BYTES_PER_LAUNCH, "traffic_unit": "bytes per launch (DRAM read + write, ncu)",
                "algorithmic_bytes": gemm_alg_bytes,
                "peak_source": f"4 x {peaks['source']} burst bf16 cuBLAS rate ({peaks['bf16_burst']} TFLOP/s): no FP4 "
                               "figure is measured on this pool, so this is a convention; the nominal dense NVFP4 "
                               "figure is 9000 TFLOP/s",
                "frac_of_nominal_9000": achieved / 9000.0,
                "frac_of_4x_sustained_bf16": achieved / (4.0 * peaks["bf16_sustained"]),
                "tensor_pipe_active_pct_ncu": GEMM_TENSOR_PIPE_ACTIVE_PCT,
                "whole_step_frac_of_nominal_9000": value / 9000.0,
                "avg_launch_ms": g_avg,
            }
            # dy: the abs-max pass reads 2 B/elt; the cast reads 2 B/elt and writes two 0.5 B/elt code
            # copies plus two 1/16 B/elt scale copies. The per-tensor scale makes the first read
            # unavoidable for a tensor larger than L2, so the sequence moves 5.125 B/elt.
            q_avg = sum(q_ms) / len(q_ms)
            elts = C2["tokens"] * C2["out_features"]
            q_bytes = elts * 3.125          # the input once, every output once; the abs-max pre-pass is overhead
            q_gbs = q_bytes / (q_avg * 1e-3) / 1e9
            line["roofline_quantize"] = {
                "bound": "hbm", "kernel": "amax_tiled_kernel<RHT> + quantize_nvfp4_kernel on dy (row + transposed, RHT)",
                "achieved": q_gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": q_gbs / peaks["hbm"],
                "algorithmic_bytes": q_bytes, "avg_sequence_ms": q_avg,
                "achieved_counting_both_reads": elts * 5.125 / (q_avg * 1e-3) / 1e9,
                "frac_of_nominal_8000": q_gbs / 8000.0,
                "peak_source": f"{peaks['source']} copy bandwidth"}
            m_ms = _timed_loop(torch, module_step, 10, 3)
            line["module_level_device_resident"] = {
                "value": flops_step / (m_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": m_ms,
                "what": "the headline step through Linear (autograd, weight cache, main_grad fusion), inputs in HBM"}
            line["tp_workload_on_1_gpu"] = _tp_workload_single_gpu(torch, Linear, params, dev, kernels)
            line["roofline"]["library_comparator"] = {"what": "torch._scaled_mm (cuBLASLt NVFP4 block-scaled GEMM), same "
                                                      "operands, per GEMM", **library_comparator()}
            line["variants"] = measure_variants()
            line["other_configs"] = _other_configs_single_gpu(torch, dev)
            tf, dt = cpu_run(4, 1)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": cpu_kind(),
                                    "sample": _cpu_sample_text(), "s_per_sample_step": dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _profile_tp_step() -> None:
    import torch
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile
    from minitransformer_b200 import kernels as K
    from minitransformer_b200.module import config as mt_config
    from minitransformer_b200.module.linear import Linear
    rank, lr = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    g, n = dist.group.WORLD, dist.get_world_size()
    peer = os.environ.get("MT_BENCH_TP_EXCHANGE", "peer") != "nccl"
    params = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.FP4_SUB_CHANNEL)
    T, H, Fd = C4["tokens"], C4["hidden"], C4["ffn"]
    x = torch.randn(T // n, H, device=dev).to(torch.bfloat16)
    dy = (torch.randn(T // n, H, device=dev) * 1e-3).to(torch.bfloat16)
    kw = dict(bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params, sequence_parallel=True,
              tp_group=g, fuse_wgrad_accumulation=True, init_method=lambda t: torch.nn.init.normal_(t, std=0.02),
              ub_overlap_ag=peer, ub_overlap_rs=peer)
    fc1 = Linear(H, Fd, parallel_mode="column", ub_name="fc1", **kw)
    fc2 = Linear(Fd, H, parallel_mode="row", ub_name="fc2", **kw)
    for m in (fc1, fc2):
        m.weight.main_grad = torch.zeros_like(m.weight, dtype=torch.float32)

    def step():
        xd = x.detach().requires_grad_(True)
        fc2(fc1(xd, is_first_microbatch=True), is_first_microbatch=True).backward(dy)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        step()
    e1.record()
    torch.cuda.synchronize()
    # host time to enqueue one step (the GPU is kept busy by a long queue, so this is pure CPU time)
    t0 = time.perf_counter()
    for _ in range(10):
        step()
    host_ms = (time.perf_counter() - t0) / 10 * 1e3
    torch.cuda.synchronize()
    if rank == 0:
        print(f"tp{n} exchange={'peer' if peer else 'nccl'} ms/step {e0.elapsed_time(e1) / 5:.3f} "
              f"host enqueue ms/step {host_ms:.3f}")
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    if rank == 0:
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=24, max_name_column_width=64))
        evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
        names = [e.name for e in evs]
        per_step = len(evs) // 3
        last = evs[-per_step:]
        t0 = last[0].time_range.start
        print("timeline of the last step (start us, duration us, kernel):")
        for e in last:
            print(f"{e.time_range.start - t0:8.0f} {e.time_range.end - e.time_range.start:7.0f}  {e.name[:90]}")
    print("rank", rank, "device status", K.read_device_status()) if rank == 0 else K.read_device_status()
    dist.barrier()
    dist.destroy_process_group()


def run_profile_case(what: str) -> None:
    """Small, self-contained kernel workloads for `ncu` captures (one kernel family each, a few
    launches, a few hundred MB on the device; the quantize inputs exceed the 126 MB L2):
      gemm         NVFP4 pair GEMM 4096x9472x4096 (8 full waves), 3 launches
      gemm_mxfp8   MXFP8 pair GEMM, same shape
      quant        abs-max + NVFP4 cast/transpose (RHT) of 8192x14336
      quant_mxfp8  MXFP8 cast/transpose of 8192x14336
      grouped      MXFP8 GroupedLinear fc1+fc2 fwd+bwd, 128 experts, 2 steps
      tp_step      (under torchrun, N ranks) the tensor-parallel MLP step of `--gpus N` under the torch
                   profiler: per-kernel device time of three steps and the timeline of the last one"""
    import torch
    from minitransformer_b200 import kernels as K
    if what == "tp_step":
        return _profile_tp_step()
    dev = "cuda"
    torch.manual_seed(0)
    if what in ("gemm", "gemm_mxfp8"):
        M, N, Kd = 4096, 9472, 4096   # 16 x 37 pair tiles = 8 x 74: no partial last wave
        x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, Kd, device=dev) * 0.02).to(torch.bfloat16)
        if what == "gemm":
            a, b = K.quantize_nvfp4(x, return_transpose=False), K.quantize_nvfp4(w, return_transpose=False)
            for _ in range(3):
                K.gemm_nvfp4(a.data, a.scale_swz, a.amax_row, b.data, b.scale_swz, b.amax_row)
        else:
            a, b = K.quantize_mxfp8(x, return_transpose=False), K.quantize_mxfp8(w, return_transpose=False)
            for _ in range(3):
                K.gemm_mxfp8(a.data, a.scale_swz, b.data, b.scale_swz)
    elif what == "quant":
        x = (torch.randn(8192, 14336, device=dev) * 1e-3).to(torch.bfloat16)
        for _ in range(3):
            K.quantize_nvfp4(x, with_rht=True)
    elif what == "quant_mxfp8":
        x = torch.randn(8192, 14336, device=dev).to(torch.bfloat16)
        for _ in range(3):
            K.quantize_mxfp8(x)
    elif what == "grouped":
        # GroupedLinear fc1 + fc2 forward+backward: 128 experts, 131072 rows, Zipf(1.1) group sizes
        import numpy as np
        from minitransformer_b200.module import config as mt_config
        from minitransformer_b200.module.group_linear import GroupedLinear
        params = mt_config.get_qlinear_params_from_predefined(mt_config.QuantizeRecipe.MXFP8_SUB_CHANNEL)
        G, R, H, Fd = 128, 131072, 2048, 768
        rng = np.random.default_rng(1234)
        p = 1.0 / np.arange(1, G + 1) ** 1.1
        m_splits = np.bincount(rng.choice(G, size=R, p=p / p.sum()), minlength=G).tolist()
        kw = dict(bias=False, params_dtype=torch.bfloat16, device=dev, qlinear_params=params,
                  fuse_wgrad_accumulation=True, init_method=lambda t: torch.nn.init.normal_(t, std=0.02))
        fc1, fc2 = GroupedLinear(G, H, Fd, **kw), GroupedLinear(G, Fd, H, **kw)
        for m in (fc1, fc2):
            block = torch.zeros(G, m.out_features, m.in_features, dtype=torch.float32, device=dev)
            for i in range(G):
                getattr(m, f"weight{i}").main_grad = block[i]
        x = torch.randn(R, H, device=dev).to(torch.bfloat16)
        dy = (torch.randn(R, H, device=dev) * 1e-3).to(torch.bfloat16)
        for _ in range(2):
            xd = x.detach().requires_grad_(True)
            fc2(fc1(xd, m_splits, is_first_microbatch=True), m_splits, is_first_microbatch=True).backward(dy)
    else:
        raise SystemExit(f"unknown case {what!r}")
    torch.cuda.synchronize()
    print("done, device status", K.read_device_status())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--profile-case", default=None,
                    help="run one small kernel workload for a profiler capture and exit (see run_profile_case)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
