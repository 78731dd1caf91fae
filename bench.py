"""Headline benchmark: BERT-large encoder forward (24 layers, fp32 tensors, TF32 tensor-core mode),
batch 1024 x seq 384 sharded by sequence across the GPUs of one node, outputs all-gathered.

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference ...                      # the CPU restatement of the
                                                              # reference's pure expansion, timed
                                                              # on the host cores (bounded sample)

Prints ONE JSON line (rank 0). Inputs are synthetic: weights ~ N(0, 0.02^2), biases 0,
LayerNorm gamma 1 / beta 0, embeddings ~ N(0, 1), all from fixed seeds.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (layers, hidden, heads, ffn, batch, seq, math mode)
    "bert_large_x24_b1024_s384_tf32": (24, 1024, 16, 4096, 1024, 384, "tf32"),
    "bert_base_x1_b64_s512_fp32x3": (1, 768, 12, 3072, 64, 512, "fp32x3"),
    "bert_base_x1_b64_s512_tf32": (1, 768, 12, 3072, 64, 512, "tf32"),
}
DEFAULT_WORKLOAD = "bert_large_x24_b1024_s384_tf32"
METRIC = "bert_encoder_seqs_per_s"
UNIT = "seqs/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [s.strip() for s in line.split(",")]
            if len(parts) >= 9:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz = sorted(int(float(s[1])) for s in self.samples if s[1].replace(".", "").isdigit())
        mx = [int(float(s[2])) for s in self.samples if s[2].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def cpu_baseline_sample(layers, hidden, heads, ffn, seq, sample_seqs, reps, warmup):
    """Times oracle/pure_oracle.py (one encoder layer on `sample_seqs` sequences) on all host cores
    and scales to `layers` layers. Returns (seqs_per_s, cores, description, seconds_per_rep)."""
    from oracle import pure_oracle as po
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    params = po.make_bert_layer_params(hidden, ffn, seed=1)
    x = torch.randn(sample_seqs, seq, hidden, generator=torch.Generator().manual_seed(2))
    for _ in range(warmup):
        po.bert_layer_forward(x, params, heads)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        po.bert_layer_forward(x, params, heads)
        times.append(time.perf_counter() - t0)
    times.sort()
    t_layer = times[len(times) // 2]
    value = sample_seqs / (t_layer * layers)
    sample = ("1 of %d layers x %d of the batch's sequences (seq %d, hidden %d), median of %d, "
              "scaled linearly in layers" % (layers, sample_seqs, seq, hidden, reps))
    return value, cores, sample, t_layer


def run_reference(args, wl):
    layers, hidden, heads, ffn, batch, seq, mode = WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_seqs = 8
    t_start = time.perf_counter()
    value, cores, sample, t_layer = cpu_baseline_sample(layers, hidden, heads, ffn, seq, sample_seqs,
                                                        max(args.steps, 1), max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * layers * (batch / sample_seqs) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "layers": layers, "hidden": hidden, "heads": heads, "ffn": ffn,
                   "global_batch": batch, "seq_len": seq,
                   "note": "CPU restatement of the reference's pure expansions (the reference needs DaCe, which "
                           "is not installable here); each step is a bounded sample scaled to the full workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_start,
    }
    print(json.dumps(line), flush=True)


def run_b200(args, wl):
    import torch.distributed as dist
    from dace_onnx_b200 import _lib, sharding
    from dace_onnx_b200.encoder import BertEncoderB200, synthetic_layer_params

    layers, hidden, heads, ffn, batch, seq, mode = WORKLOADS[wl]
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    rank, world, local_rank = sharding.init_from_env("nccl")
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch one rank per GPU with torch.distributed.run"
                         % (args.gpus, world))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _lib.load()

    # replicated weights from the same seeds on every rank (no broadcast needed)
    params = [synthetic_layer_params(hidden, ffn, seed=100 + i) for i in range(layers)]
    enc = BertEncoderB200(params, heads, device=device, math_mode=mode, micro_batch=args.micro_batch)
    del params
    lo, hi = sharding.shard_bounds(batch, world, rank)
    local = hi - lo
    x_host = torch.randn(local, seq, hidden, generator=torch.Generator().manual_seed(7 + rank)).pin_memory()
    y_host = torch.empty(local, seq, hidden).pin_memory()
    x_dev = x_host.to(device)
    y_local = torch.empty_like(x_dev)
    y_full = torch.empty(batch, seq, hidden, device=device) if world > 1 else None

    def step_device():
        enc.forward_device(x_dev, out=y_local)
        if world > 1:
            sharding.all_gather_batch(y_local, batch, out=y_full)

    def step_e2e():
        # pinned host input -> device -> layers -> pinned host output, micro-batch copies overlapped
        # with compute; the local result also stays on the device for the all-gather
        enc.forward_host(x_host, y_host, out_device=y_local)
        if world > 1:
            sharding.all_gather_batch(y_local, batch, out=y_full)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step_device()
    sampler = ClockSampler(local_rank)
    sampler.start()
    enc.timeline = []
    launches0 = enc.launches
    ms_step = timed(step_device, args.steps)
    launches = enc.launches - launches0
    timeline, enc.timeline = enc.timeline, None
    clocks = sampler.stop()
    for _ in range(min(args.warmup, 1)):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    _lib.device_status()

    # per-kernel-class totals from the events recorded around every launch of the timed steps
    per_kind = {}
    for kind, flops, nbytes, s, e in timeline:
        d = per_kind.setdefault(kind, [0.0, 0.0, 0.0, 0])
        d[0] += s.elapsed_time(e) * 1e-3
        d[1] += flops
        d[2] += nbytes
        d[3] += 1
    peaks = measured_peaks()
    tf32_peak = peaks["bf16_sustained"] / 2.0  # no TF32 figure is measured; half the sustained bf16 rate
    ops_report = {}
    for kind, (sec, flops, nbytes, n) in sorted(per_kind.items()):
        entry = {"launches": n, "ms_per_step": sec * 1e3 / args.steps, "share": None}
        if flops and kind == "gemm":
            entry.update(tflops=flops / sec / 1e12, frac_tensor=flops / sec / 1e12 / tf32_peak)
        elif nbytes:
            entry.update(gbs=nbytes / sec / 1e9, frac_hbm=nbytes / sec / 1e9 / peaks["hbm_gbs"])
            if flops:
                entry["tflops"] = flops / sec / 1e12
        ops_report[kind] = entry
    total_sec = sum(v[0] for v in per_kind.values()) or 1.0
    for kind in ops_report:
        ops_report[kind]["share"] = per_kind[kind][0] / total_sec
    g = per_kind.get("gemm", [1.0, 0.0, 0.0, 1])
    # DRAM traffic of the dense GEMM kernel: ncu measured dram read+write = 0.83 x the algorithmic bytes
    # 4(MK+NK+MN) on the captured small case (profiles/gemm_tc_tf32_qkv_16384x3072x1024.txt: 232.7 MB vs
    # 281.0 MB; part of the output is still in L2 when the kernel ends). Traffic grows in proportion to M,
    # so the per-launch figure here is that ratio times the average algorithmic bytes of a bench launch.
    t_tok = min(args.micro_batch, local) * seq
    gemm_shapes = [(3 * hidden, hidden), (hidden, hidden), (ffn, hidden), (hidden, ffn)]
    alg_bytes = sum(4 * (t_tok * k + n * k + t_tok * n) for n, k in gemm_shapes) / len(gemm_shapes)
    traffic = 0.83 * alg_bytes
    achieved = g[1] / g[0] / 1e12
    roofline = {"bound": "tensor", "kernel": "gemm_tc_pair_kernel<256, K-major> (TF32 dense projections, CTA pairs)",
                "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak,
                "peak_source": "%s bf16 sustained / 2 (TF32 runs at half the bf16 rate)" % peaks["source"],
                "avg_launch_ms": g[0] * 1e3 / max(g[3], 1), "traffic": traffic,
                "traffic_unit": "bytes per launch (scaled from an ncu capture of a smaller launch)",
                "algorithmic_bytes": alg_bytes}

    line = None
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            cb_value, cores, sample, _ = cpu_baseline_sample(layers, hidden, heads, ffn, seq, 8, 3, 1)
            cpu_baseline = {"value": cb_value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        else:
            cpu_baseline = None
        bytes_io = local * seq * hidden * 4
        line = {
            "metric": METRIC, "value": batch / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "tf32" if mode == "tf32" else "f32", "data": "synthetic",
            "config": {"workload": wl, "layers": layers, "hidden": hidden, "heads": heads, "ffn": ffn,
                       "global_batch": batch, "seq_len": seq, "parallelism": "batch-sharded x%d, output all-gather" % world,
                       "math_mode": mode, "micro_batch": enc.micro_batch,
                       "l2": "inputs larger than L2 (every activation tensor of a micro-batch exceeds 126 MB)"},
            "e2e": {"value": batch / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": bytes_io,
                    "d2h_bytes_per_step": bytes_io, "ms_per_step": ms_e2e},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_baseline,
            "ops": ops_report,
            "tflops_algorithmic": enc.flops_per_sequence(seq) * batch / (ms_step * 1e-3) / 1e12 / world,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# single-kernel cases: the bandwidth microbenchmarks of the specification and one launch shape of
# each contraction, small enough (a few hundred MB) to profile under ncu
# ---------------------------------------------------------------------------------------------
def kernel_cases(device):
    from dace_onnx_b200 import ops
    from dace_onnx_b200._lib import EPI_BIAS, EPI_BIAS_GELU, EPI_SCALE
    g = torch.Generator(device=device).manual_seed(0)
    rn = lambda *s, std=1.0: torch.randn(*s, device=device, generator=g) * std  # noqa: E731

    def softmax_c4():
        x = rn(768, 512, 512, std=2.0)
        y = torch.empty_like(x)
        return (lambda: ops.softmax(x, -1, out=y)), 0, 8 * x.numel(), "hbm"

    def layernorm_c4():
        x = rn(65536, 1024)
        gamma, beta = torch.ones(1024, device=device), torch.zeros(1024, device=device)
        y = torch.empty_like(x)
        return (lambda: ops.layernorm(x, gamma, beta, 1e-12, out=y)), 0, 8 * x.numel(), "hbm"

    def gemm(m, n, k, mode, epi=EPI_BIAS):
        def make():
            a, w, b = rn(m, k), rn(n, k, std=0.02), rn(n, std=0.02)
            y = torch.empty(m, n, device=device)
            return (lambda: ops.matmul(a, w, out=y, trans_b=True, epilogue=epi, bias=b, math_mode=mode)), \
                2 * m * n * k, 4 * (m * k + n * k + m * n), "tensor"
        return make

    def gemm_no_workspace(m, n, k, mode, epi=EPI_BIAS):
        # the plain entry point (b200_gemm_f32): in 3xTF32 mode the single-CTA kernel that splits B in shared memory
        def make():
            import ctypes
            from dace_onnx_b200 import _lib
            a, w, b = rn(m, k), rn(n, k, std=0.02), rn(n, std=0.02)
            y = torch.empty(m, n, device=device)
            d = _lib.GemmDesc(1, 1, m, n, k, k, k, n, 0, 0, 0, 0, 0, 0, 1, epi, 1.0, _lib.MATH_MODES[mode])
            lib = _lib.load()
            ptr = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
            fn = lambda: _lib.check(lib.b200_gemm_f32(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),  # noqa
                                                      ctypes.byref(d), ptr(a), ptr(w), ptr(b), None, ptr(y)))
            return fn, 2 * m * n * k, 4 * (m * k + n * k + m * n), "tensor"
        return make

    def attn_qk(b, h, s, d, mode):
        def make():
            qkv = rn(b, s, 3 * h * d)
            sc = torch.empty(b, h, s, s, device=device)
            hid = h * d
            fn = lambda: ops.gemm_raw(qkv, qkv[..., hid:], sc, batch_outer=b, batch_inner=h, M=s, N=s, K=d,  # noqa
                                      lda=3 * hid, ldb=3 * hid, ldy=s, a_strides=(s * 3 * hid, d),
                                      b_strides=(s * 3 * hid, d), y_strides=(h * s * s, s * s), trans_b=True,
                                      epilogue=EPI_SCALE, scale=0.125, math_mode=mode)
            return fn, 2 * b * h * s * s * d, 4 * (2 * b * s * hid + b * h * s * s), "hbm"
        return make

    def attn_pv(b, h, s, d, mode):
        def make():
            qkv = rn(b, s, 3 * h * d)
            pr = torch.rand(b, h, s, s, device=device, generator=g)
            hid = h * d
            ctx = torch.empty(b, s, hid, device=device)
            fn = lambda: ops.gemm_raw(pr, qkv[..., 2 * hid:], ctx, batch_outer=b, batch_inner=h, M=s, N=d, K=s,  # noqa
                                      lda=s, ldb=3 * hid, ldy=hid, a_strides=(h * s * s, s * s),
                                      b_strides=(s * 3 * hid, d), y_strides=(s * hid, d), trans_b=False,
                                      math_mode=mode)
            return fn, 2 * b * h * s * s * d, 4 * (2 * b * s * hid + b * h * s * s), "hbm"
        return make

    def attn_fused(b, h, s, d):
        def make():
            qkv = rn(b, s, 3 * h * d)
            ctx = torch.empty(b, s, h * d, device=device)
            v4 = qkv.view(b, s, 3 * h, d)
            fn = lambda: ops.attention_views(v4[:, :, :h], v4[:, :, h:2 * h], v4[:, :, 2 * h:], ctx.view(b, s, h, d),  # noqa
                                             0.125, math_mode="tf32")
            return fn, 4 * b * h * s * s * d, 16 * b * s * h * d, "tensor"
        return make

    def attn_fused_headmajor(b, h, s, d):
        def make():
            q, k, v = (rn(b, h, s, d) for _ in range(3))  # each head's [s, d] block contiguous
            ctx = torch.empty(b, s, h * d, device=device)
            fn = lambda: ops.attention_views(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),  # noqa
                                             ctx.view(b, s, h, d), 0.125, math_mode="tf32")
            return fn, 4 * b * h * s * s * d, 16 * b * s * h * d, "tensor"
        return make

    def conv(n, c, hw, m, mode):
        def make():
            x = torch.rand(n, c, hw, hw, device=device, generator=g)
            bound = 1.0 / (c * 9) ** 0.5
            w = (torch.rand(m, c, 3, 3, device=device, generator=g) * 2 - 1) * bound
            b = (torch.rand(m, device=device, generator=g) * 2 - 1) * bound
            y = torch.empty(n, m, hw, hw, device=device)
            ws = torch.empty(2 * x.numel() * 4 + (1 << 20), device=device, dtype=torch.uint8)
            fn = lambda: ops.conv2d(x, w, b, out=y, pads=(1, 1, 1, 1), relu=True, workspace=ws, math_mode=mode)  # noqa
            return fn, 2 * n * hw * hw * m * c * 9, 4 * (x.numel() + y.numel()), "tensor"
        return make

    def frontdoor_bert_layer(b, s, hidden, heads, ffn, mode):
        # transformers.BertLayer exported to ONNX and run through the graph front door (49 nodes -> 6 fused)
        def make():
            from transformers import BertConfig, BertLayer
            from dace_onnx_b200.torch_module import B200Module
            torch.manual_seed(0)
            cfg = BertConfig(hidden_size=hidden, num_attention_heads=heads, intermediate_size=ffn,
                             hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
            cfg._attn_implementation = "eager"
            mod = B200Module(BertLayer(cfg).eval(), dummy_inputs=(torch.zeros(b, s, hidden),), math_mode=mode)
            x = rn(b, s, hidden)
            t = b * s
            flops = 2 * t * hidden * (4 * hidden + 2 * ffn) + 4 * b * heads * s * s * (hidden // heads)
            return (lambda: mod(x)), flops, 0, "tensor"
        return make

    def encoder_bert_layer(b, s, hidden, heads, ffn, mode):
        # the hand-written runner on the same layer shape, for comparison with the front door
        def make():
            from dace_onnx_b200.encoder import BertEncoderB200, synthetic_layer_params
            enc = BertEncoderB200([synthetic_layer_params(hidden, ffn, 0)], heads, device=str(device),
                                  math_mode=mode, micro_batch=b)
            x = rn(b, s, hidden)
            y = torch.empty_like(x)
            t = b * s
            flops = 2 * t * hidden * (4 * hidden + 2 * ffn) + 4 * b * heads * s * s * (hidden // heads)
            return (lambda: enc.forward_device(x, out=y)), flops, 0, "tensor"
        return make

    def frontdoor_mlp_c1(cuda_graph=False, mode="fp32x3"):
        # configuration 1: Linear 784-120-32-10 + ReLU + LogSoftmax, batch 4096, exported and run from the graph
        def make():
            from dace_onnx_b200.torch_module import B200Module
            torch.manual_seed(0)
            net = torch.nn.Sequential(torch.nn.Linear(784, 120), torch.nn.ReLU(), torch.nn.Linear(120, 32),
                                      torch.nn.ReLU(), torch.nn.Linear(32, 10), torch.nn.LogSoftmax(dim=1)).eval()
            mod = B200Module(net, dummy_inputs=(torch.zeros(4096, 784),), math_mode=mode, cuda_graph=cuda_graph)
            x = rn(4096, 784)
            if cuda_graph:  # the serving pattern: fill the captured input buffer in place, replay
                mod(x)
                x = mod.onnx_model.static_inputs(x.shape)[0].copy_(x)
            return (lambda: mod(x)), 2 * 4096 * (784 * 120 + 120 * 32 + 32 * 10), 13.40e6, "hbm"
        return make

    return {
        "frontdoor_bert_large_layer_tf32": frontdoor_bert_layer(64, 384, 1024, 16, 4096, "tf32"),
        "encoder_bert_large_layer_tf32": encoder_bert_layer(64, 384, 1024, 16, 4096, "tf32"),
        "frontdoor_mlp_c1": frontdoor_mlp_c1(), "frontdoor_mlp_c1_cudagraph": frontdoor_mlp_c1(True),
        "frontdoor_mlp_c1_cudagraph_fp32": frontdoor_mlp_c1(True, "fp32"),
        "frontdoor_mlp_c1_cudagraph_tf32": frontdoor_mlp_c1(True, "tf32"),
        "conv_c2_fp32x3": conv(256, 64, 56, 64, "fp32x3"), "conv_c2_tf32": conv(256, 64, 56, 64, "tf32"),
        "softmax_c4": softmax_c4, "layernorm_c4": layernorm_c4,
        "gemm_tf32_qkv": gemm(16384, 3072, 1024, "tf32"), "gemm_tf32_ffn1": gemm(16384, 4096, 1024, "tf32", EPI_BIAS_GELU),
        "gemm_tf32_ffn2": gemm(16384, 1024, 4096, "tf32"), "gemm_tf32_proj": gemm(16384, 1024, 1024, "tf32"),
        "gemm_fp32x3_ffn1": gemm(16384, 3072, 768, "fp32x3", EPI_BIAS_GELU), "gemm_fp32x3_proj": gemm(16384, 768, 768, "fp32x3"),
        "gemm_fp32x3_ffn1_no_workspace": gemm_no_workspace(16384, 3072, 768, "fp32x3", EPI_BIAS_GELU),
        "attn_qk_tf32": attn_qk(32, 16, 384, 64, "tf32"), "attn_pv_tf32": attn_pv(32, 16, 384, 64, "tf32"),
        "attention_fused_tf32": attn_fused(32, 16, 384, 64),
        "attention_stream_tf32_s512": attn_fused(64, 12, 512, 64), "attention_stream_tf32_s2048": attn_fused(8, 16, 2048, 64),
        "attention_fused_tf32_headmajor": attn_fused_headmajor(32, 16, 384, 64),
    }


def run_kernel_case(args):
    from dace_onnx_b200 import _lib
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    cases = kernel_cases(device)
    names = sorted(cases) if args.kernel == "all" else [args.kernel]
    peaks = measured_peaks()
    flush = torch.empty(64 * 1024 * 1024, device=device)  # 256 MB > L2, rewritten between iterations
    for name in names:
        fn, flops, nbytes, bound = cases[name]()
        for _ in range(args.warmup):
            fn()
        times = []
        for _ in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        _lib.device_status()
        ms = sorted(times)[len(times) // 2]
        if bound == "tensor":
            peak = peaks["bf16"] / 2.0  # a kernel timed alone: burst figure
            achieved, unit = flops / (ms * 1e-3) / 1e12, "TFLOP/s"
        else:
            peak, achieved, unit = peaks["hbm_gbs"], nbytes / (ms * 1e-3) / 1e9, "GB/s"
        print(json.dumps({"kernel_case": name, "ms": ms, "steps": args.steps, "warmup": args.warmup,
                          "l2": "flushed (256 MB memset) before every timed launch",
                          "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                                       "frac": achieved / peak, "peak_source": peaks["source"]},
                          "tflops": flops / (ms * 1e-3) / 1e12 if flops else None,
                          "gbs": nbytes / (ms * 1e-3) / 1e9}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default=None, help="run one single-kernel case (or 'all') instead of the encoder")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--micro-batch", type=int, default=256)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.kernel:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args, args.workload)
    else:
        run_b200(args, args.workload)


if __name__ == "__main__":
    main()
