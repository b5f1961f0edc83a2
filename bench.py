"""Throughput of the LFM2 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step.  The default run uses the layer sizes of LFM2-1.2B (16
layers: 10 gated short-convolution, 6 attention at [2,5,8,10,12,14]; hidden 2048; 32
query heads, 8 KV heads, head size 64; feed-forward 12288 adjusted to 8192; filter
length 3; vocabulary 65536; tied head) with random bfloat16 weights, a batch of 8 and
a context of 4,096 tokens: every request is prefilled so that after the W warm-up
steps it holds 4096 - K tokens, then K steps are timed with CUDA events and end at
4,096.  The one JSON line printed holds

  value      decoded tokens a second over the K timed steps, tokens fed back on the
             device (no host round trip inside the timed region)
  e2e        the same through the Python entry point (`Engine.step`): every step copies
             its index arrays from pinned host memory and reads the sampled ids back
  prefill    one step over a 2,048-token prompt: tokens a second, and its FLOPs / time /
             the bfloat16 peak
  roofline   the decode step's bytes (every weight once, the live requests' keys and
             values and convolution states) / its time, against the HBM peak
  points     decoded tokens a second at batch 1 and batch 64 (context 2,048 + steps), each
             with its bytes / time as a fraction of the HBM peak (`decode_b1_frac`, ...)
  workloads  two scheduler runs through `Engine.step` with requests that come and go
             (`--workloads none` leaves them out; `--only workload --workload NAME` runs one):
             350m-mixed      LFM2-350M sizes, 32 requests, prompts U[128, 2048], prompt
                             portions of 512 beside the running decodes, 256 new tokens each
             700m-staggered  LFM2-700M sizes, 64 requests arriving four steps apart, prompts
                             U[512, 8192], 512 new tokens each, a page pool of 90 % of the
                             free device memory
             each after one untimed run of the same requests: output and total tokens a
             second, steps, preemptions, the share of steps replayed from a captured graph,
             and per step the host time of `Engine.step` against the device time between
             events recorded around it (`gpu_idle_frac`: the share of the run's wall time in
             which the device waited for the host)

RVLLM_BENCH_PAGE sets the tokens per cache page (16; 64 measured the same).

Peaks come from MEASURED_PEAKS.json beside this file when it exists ("of measured"),
else from the fallback figures 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LFM2_1_2B = {
    "architectures": ["Lfm2ForCausalLM"],
    "num_hidden_layers": 16, "full_attn_idxs": [2, 5, 8, 10, 12, 14],
    "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 65536, "rope_theta": 1000000.0,
    "max_position_embeddings": 4096, "norm_eps": 1e-5, "tie_embedding": True,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 7,
}
# The other published sizes differ in these keys only.
SIZES = {
    "1.2b": {},
    "700m": {"hidden_size": 1536, "num_attention_heads": 24, "block_ff_dim": 10240},
    "350m": {"hidden_size": 1024, "num_attention_heads": 16, "block_ff_dim": 6656},
}
WORKLOADS = {
    "350m-mixed": {"size": "350m", "requests": 32, "prompt": (128, 2048), "new": 256,
                   "chunk": 512, "arrival_gap": 0, "pool": "fit", "positions": 4096},
    "700m-staggered": {"size": "700m", "requests": 64, "prompt": (512, 8192), "new": 512,
                       "chunk": 2048, "arrival_gap": 4, "pool": "90% of free HBM",
                       "positions": 16384},
    # not one of the two that the default run reports: the mixed workload at the headline's sizes
    "1.2b-mixed": {"size": "1.2b", "requests": 32, "prompt": (128, 2048), "new": 256,
                   "chunk": 512, "arrival_gap": 2, "pool": "fit", "positions": 4096},
}
DEFAULT_WORKLOADS = ("350m-mixed", "700m-staggered")
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = int(os.environ.get("RVLLM_BENCH_PAGE", "16"))      # tokens per cache page


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            m = json.load(f)
        return {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi samples during the timed region: SM clock and throttle reasons."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    @staticmethod
    def _device_id() -> str:
        """What nvidia-smi calls the device CUDA runs on: its UUID when torch can tell it
        (CUDA_VISIBLE_DEVICES may renumber the devices), else index 0."""
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            return "0"

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self._device_id(), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6:
                    continue
                try:
                    clocks.append(float(parts[0]))
                    mx = float(parts[1])
                except ValueError:
                    continue
                for name, val in zip(names, parts[2:6]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.remove(self.path)
        if clocks:
            clocks.sort()
            out["sm_mhz"] = clocks[len(clocks) // 2]
            out["sm_max_mhz"] = mx
        out["reasons"] = sorted(reasons)
        return out


def model_bytes_and_flops(cfg, spec_decls):
    """Bytes of every weight a step reads once, and matrix FLOPs per token."""
    weight_bytes = 0
    matmul_params = 0
    for name, decl in spec_decls.items():
        n = 1
        for d in decl.shape:
            n *= d
        weight_bytes += n * 2
        if len(decl.shape) == 2 and "embed_tokens" not in name and "conv.conv" not in name:
            matmul_params += n
    return weight_bytes, matmul_params


def run_ours(args):
    import torch

    from rvllm_b200.config import architecture, config_from_dict
    from rvllm_b200.engine import (Engine, ModelRunner, Request, SchedulerConfig, StepEntry,
                                   graphs_default, load_model, make_cache)
    from rvllm_b200.parts.model import param_decls
    from rvllm_b200.sampling import SamplingParams
    from rvllm_b200.weights import write_random_model

    pk = peaks()
    layers_full = LFM2_1_2B["num_hidden_layers"]
    data = dict(LFM2_1_2B)
    data.update(SIZES[args.size])
    cfg = config_from_dict(data)
    K, W, B = args.steps, args.warmup, args.batch
    if K + W > CONTEXT - 64:
        raise SystemExit(f"--steps + --warmup must stay below {CONTEXT - 64}")
    tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
    t0 = time.time()
    try:
        folder = write_random_model(os.path.join(tmp, "lfm2_1_2b"), cfg, seed=0)
        model, cfg = load_model(folder, "bfloat16", "cuda")
    finally:                     # gigabytes of weights: never leave them behind
        shutil.rmtree(tmp, ignore_errors=True)
    setup_s = time.time() - t0
    ops = model.ops
    spec = architecture(cfg.architecture).build_spec(cfg)
    weight_bytes, matmul_params = model_bytes_and_flops(cfg, param_decls(spec))
    n_attn = len(cfg.full_attn_idxs)
    n_conv = cfg.num_hidden_layers - n_attn
    kv_bytes_per_token = n_attn * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    conv_state_bytes = n_conv * (cfg.conv_L_cache - 1) * cfg.hidden_size * 4 * 2   # read + write
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def fresh_runner(batch):
        pages = batch * (CONTEXT // PAGE)
        cache = make_cache(model, PAGE, pages, batch)
        return ModelRunner(model, cache, ops, use_graphs=graphs_default())

    def do_prefill(runner, ids_list, chunk=2048):
        for i, ids in enumerate(ids_list):
            runner.add_request(i)
            for a in range(0, len(ids), chunk):
                runner.step([StepEntry(i, ids[a:a + chunk], ())])

    def timed_decode(batch, start_ctx, steps, warmup):
        """Device-timed greedy decode: tokens fed back on the device."""
        runner = fresh_runner(batch)
        do_prefill(runner, prompts(batch, start_ctx - warmup))
        reqs = list(range(batch))
        first = [1] * batch
        out = runner.decode_greedy(reqs, first, warmup)
        first = out[-1].tolist() if warmup else first
        torch.cuda.synchronize()
        launches0 = ops.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.decode_greedy(reqs, first, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        return batch * steps / (ms / 1e3), ms / steps, ops.launches - launches0

    if args.only == "prefill":
        return run_prefill_only(torch, fresh_runner, prompts, StepEntry)

    # ---- the headline: batch B, K steps ending at the full context ------------------
    sampler = ClockSampler()
    sampler.start()
    value, ms_per_step, launches = timed_decode(B, CONTEXT - K, K, W)
    clocks = sampler.stop()
    mean_ctx = CONTEXT - K / 2
    step_bytes = weight_bytes + B * mean_ctx * kv_bytes_per_token + B * conv_state_bytes
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    if args.only == "breakdown":
        return run_breakdown(torch, fresh_runner, do_prefill, prompts, B, ops)

    if args.only == "decode":
        print(json.dumps({"only": "decode", "value": round(value, 1),
                          "ms_per_step": round(ms_per_step, 4), "gpu_launches": launches,
                          "roofline_gbs": round(achieved, 1), "clocks": clocks}))
        return 0

    # ---- end to end through Engine.step ------------------------------------------------
    runner = fresh_runner(B)
    sched = SchedulerConfig(block_size=PAGE, num_blocks=B * (CONTEXT // PAGE),
                            max_num_batched_tokens=8192, prefill_chunk=2048)
    engine = Engine(runner, sched, CONTEXT, lookahead=True)
    e2e_steps = min(K, 512)
    budget = e2e_steps + W + 16          # requests start decoding a few steps apart
    for i, ids in enumerate(prompts(B, CONTEXT - budget)):
        engine.add_request(Request(i, ids, budget, (), SamplingParams()))
    seqs = list(engine.scheduler.seqs.values())
    while min(len(s.generated) for s in seqs) < W:
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    done = 0
    for _ in range(e2e_steps):
        done += len(engine.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e = {"value": round(done / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": runner.builder.last_h2d_bytes, "d2h_bytes_per_step": 4 * B}
    del engine, runner

    # ---- prefill of 2,048 tokens -----------------------------------------------------
    runner = fresh_runner(1)
    ids = prompts(1, PREFILL_TOKENS)[0]
    times = []
    for it in range(5):
        runner.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("p", ids, (PREFILL_TOKENS - 1,))])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.end_request("p")
    pre_ms = sorted(times[2:])[len(times[2:]) // 2]
    T = PREFILL_TOKENS
    flops = 2.0 * T * matmul_params + 2.0 * cfg.vocab_size * cfg.hidden_size \
        + n_attn * 4.0 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    del runner

    # ---- other batch sizes -------------------------------------------------------------
    points = {}
    for b in (1, 64):
        # 2,048 prompt tokens, then 8 untimed steps: the padded block-table width grows at
        # 2,049 tokens, and the graph of the new width is captured there, outside the timing
        v, ms, _ = timed_decode(b, 2048 + 8, 256, 8)
        points[f"decode_b{b}"] = round(v, 1)
        nbytes = weight_bytes + b * (2048 + 8 + 128) * kv_bytes_per_token + b * conv_state_bytes
        points[f"decode_b{b}_frac"] = round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    del model
    workloads = {}
    if args.workloads != "none":
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for name in (DEFAULT_WORKLOADS if args.workloads == "both" else [args.workloads]):
            workloads[name] = run_workload(name)

    line = {
        "metric": f"decode tok/s at batch {B} (LFM2-{args.size.upper()} sizes, context to 4,096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights (seed 0), "
        "uniform random token ids", "impl": "ours",
        "config": {"model": f"LFM2-{args.size.upper()} sizes", "layers": cfg.num_hidden_layers,
                   "layers_full": layers_full, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size,
                   "conv_taps": cfg.conv_L_cache, "attn_layers": n_attn,
                   "global_batch": B, "seq_len": CONTEXT, "page": PAGE,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (2.3 GB weights)",
                   "peaks": pk["source"]},
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "workloads": workloads, "gpu_launches": launches, "clocks": clocks,
        "setup_s": round(setup_s, 1),
    }
    print(json.dumps(line))
    return 0


def run_prefill_only(torch, fresh_runner, prompts, StepEntry):
    runner = fresh_runner(1)
    ids = prompts(1, PREFILL_TOKENS)[0]
    times = []
    for it in range(3):
        runner.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("p", ids, (PREFILL_TOKENS - 1,))])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.end_request("p")
    print(json.dumps({"only": "prefill", "ms": [round(t, 3) for t in times]}))
    return 0


def run_breakdown(torch, fresh_runner, do_prefill, prompts, B, ops, ctx=3000, steps=20):
    """Per-kernel device time inside replayed decode steps (torch.profiler over `steps`
    steps at context `ctx`), the wall time of a step, and the host time of an engine step.
    With programmatic dependent launch a kernel's time includes its wait for the previous
    kernel, so the kernel times can add up to more than the wall time."""
    import collections
    import re

    from torch.profiler import ProfilerActivity, profile
    runner = fresh_runner(B)
    do_prefill(runner, prompts(B, ctx))
    reqs = list(range(B))
    runner.decode_greedy(reqs, [1] * B, 8)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.decode_greedy(reqs, [1] * B, 50)
    e1.record()
    torch.cuda.synchronize()
    wall_us = e0.elapsed_time(e1) / 50 * 1e3
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        runner.decode_greedy(reqs, [1] * B, steps)
        torch.cuda.synchronize()
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            name = re.sub(r"<.*", "", ev.name).replace("void ", "")[:48]
            agg[name][0] += 1
            agg[name][1] += ev.device_time
    ops.check_status()
    kernels = {k: {"per_step": round(n / steps, 1), "us_each": round(t / n, 2),
                   "us_per_step": round(t / steps, 1)}
               for k, (n, t) in sorted(agg.items(), key=lambda x: -x[1][1])[:16]}
    print(json.dumps({"only": "breakdown", "batch": B, "context": ctx,
                      "wall_us_per_step": round(wall_us, 1), "kernels": kernels}))
    return 0


def run_kernels(args):
    """Single kernels at LFM2-1.2B sizes, timed as launches captured in one CUDA graph (no
    host gaps), over operands larger than L2.  One JSON line."""
    import math
    from types import SimpleNamespace

    import torch

    from rvllm_b200.kernels import cuda_ops
    ops = cuda_ops()
    pk = peaks()
    nh, nkv, hd, ps = args.kernel_heads, 8, 64, args.kernel_page
    out = {"only": "kernels", "peaks": pk["source"]}

    def graph_time(fns, reps=5):
        for f in fns[:2]:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / len(fns))
        return sorted(ts)[len(ts) // 2]

    if args.kernel == "copy_rate":
        # the copy probe (csrc/copy_probe.cu): what one SM, a quarter of the SMs and all of
        # them can copy into shared memory, as tensor-map boxes and as contiguous bulk copies
        import ctypes
        K, iters = 2048, 512
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        rows = sms * iters * 16384 // (K * 2) + 128
        w = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)      # 1.2 GB: larger than L2
        status = ops.status_word("cuda")
        for mode, name, chunk in ((0, "box", 16384), (1, "bulk", 16384), (1, "bulk32k", 32768),
                                  (1, "bulk64k", 65536)):
            for grid in (sms, sms // 4, 1):
                for stages in (3, 4, 10):
                    if stages * chunk > 200 * 1024:
                        continue

                    def call():
                        ops._check(ops.lib.rv_copy_probe(
                            ctypes.c_void_p(w.data_ptr()), ctypes.c_longlong(rows), ctypes.c_int(K),
                            ctypes.c_int(mode), ctypes.c_int(grid), ctypes.c_int(iters * 16384 // chunk),
                            ctypes.c_int(stages), ctypes.c_int(chunk), ctypes.c_void_p(status.data_ptr()),
                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "copy_probe")
                    call()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    call()
                    e1.record()
                    torch.cuda.synchronize()
                    gbs = grid * (iters * 16384 // chunk) * chunk / (e0.elapsed_time(e1) * 1e-3) / 1e9
                    out[f"copy_{name}_sms{grid}_stages{stages}"] = {
                        "GB/s": round(gbs, 1), "GB/s_per_sm": round(gbs / grid, 1)}
        ops.check_status()
        print(json.dumps(out))
        return 0
    if args.kernel in ("all", "attn_decode"):
        B, ctx = args.kernel_batch, args.kernel_ctx
        blocks = -(-ctx // ps)
        layers = max(2, min(6, (400 << 20) // (B * ctx * nkv * hd * 4)))   # distinct caches > L2
        caches = [(torch.randn(B * blocks, ps, nkv, hd, device="cuda", dtype=torch.bfloat16),
                   torch.randn(B * blocks, ps, nkv, hd, device="cuda", dtype=torch.bfloat16))
                  for _ in range(layers)]
        table = torch.randperm(B * blocks, device="cuda").to(torch.int32).view(B, blocks)
        q = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
        o = torch.empty(B, nh * hd, device="cuda", dtype=torch.bfloat16)
        cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        qs = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        scale = 1 / math.sqrt(hd)
        nbytes = B * ctx * nkv * hd * 2 * 2
        for name, fn in (("mma", lambda k, v: ops.paged_attention_decode_mma(
                q, nh, nkv, hd, k, v, table, qs, cl, B, ctx, ps, scale, None, o)),
                         ("simt", lambda k, v: ops.paged_attention_decode(
                q, nh, nkv, hd, k, v, table, cl, B, ctx, ps, scale, None, o))):
            us = graph_time([(lambda k=k, v=v: fn(k, v)) for k, v in caches])
            out[f"attn_decode_{name}_b{B}_ctx{ctx}"] = {
                "us": round(us, 1), "GB/s": round(nbytes / us / 1e3, 1),
                "frac_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
    if args.kernel in ("all", "attn_prefill"):
        # the whole prompt in one portion, and (--kernel-ctx above the portion) its last portion:
        # the same number of query tokens at the end of a longer context
        T = args.kernel_tokens
        for C in sorted({T, max(T, args.kernel_ctx if args.kernel == "attn_prefill" else T)}):
            blocks = -(-C // ps)
            kc = torch.randn(blocks, ps, nkv, hd, device="cuda", dtype=torch.bfloat16)
            vc = torch.randn_like(kc)
            table = torch.randperm(blocks, device="cuda").to(torch.int32).view(1, blocks)
            q = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
            o = torch.empty(T, nh * hd, device="cuda", dtype=torch.bfloat16)
            ctx = SimpleNamespace(n_tokens=T, n_reqs=1, n_decode=0, max_ctx_len=C, max_q_len=T,
                                  q_start=torch.tensor([0, T], dtype=torch.int32, device="cuda"),
                                  ctx_lens=torch.tensor([C], dtype=torch.int32, device="cuda"),
                                  token_req=torch.zeros(T, dtype=torch.int32, device="cuda"))
            group = SimpleNamespace(block_table=table, max_blocks=blocks, page_size=ps, window=None)
            us = graph_time([lambda: ops.paged_attention(q, nh, nkv, hd, kc, vc, ctx, group,
                                                         1 / math.sqrt(hd), None, o)] * 4)
            flops = 4 * nh * hd * (T * (C - T) + T * (T + 1) / 2)
            name = f"attn_prefill_t{T}" + (f"_ctx{C}" if C != T else "")
            out[name] = {"us": round(us, 1), "TFLOP/s": round(flops / us / 1e6, 1),
                         "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}
    if args.kernel == "elementwise":
        # the memory-bound kernels between the products of a 2,048-token prompt portion, each on
        # buffers in rotation that together exceed the L2 (bytes = what the kernel has to move)
        T = PREFILL_TOKENS
        cfgd = dict(LFM2_1_2B)
        cfgd.update(SIZES[args.size])
        from rvllm_b200.config import config_from_dict
        mc = config_from_dict(cfgd)
        H, F, taps = mc.hidden_size, mc.ffn_dim, mc.conv_L_cache
        bf = torch.bfloat16
        n = 6
        res = {}

        def timed(name, fns, nbytes):
            us = graph_time(fns)
            res[name] = {"us": round(us, 1), "GB/s": round(nbytes / us / 1e3, 1),
                         "frac_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}

        gu = [torch.randn(T, 2 * F, device="cuda", dtype=bf) for _ in range(n)]
        act = [torch.empty(T, F, device="cuda", dtype=bf) for _ in range(n)]
        timed("swiglu", [(lambda a=a, b=b: ops.swiglu(a, b)) for a, b in zip(gu, act)], T * F * 6)
        del gu, act
        resid = [torch.randn(T, H, device="cuda", dtype=torch.float32) for _ in range(n * 2)]
        delta = [torch.randn(T, H, device="cuda", dtype=bf) for _ in range(n * 2)]
        outs = [torch.empty(T, H, device="cuda", dtype=bf) for _ in range(n * 2)]
        wn = torch.ones(H, device="cuda", dtype=torch.float32)
        timed("add_rmsnorm", [(lambda r=r, d=d, o=o: ops.add_rmsnorm(r, d, wn, 1e-5, o))
                              for r, d, o in zip(resid, delta, outs)], T * H * 12)
        del resid, delta
        proj = [torch.randn(T, 3 * H, device="cuda", dtype=bf) for _ in range(n * 2)]
        filt = torch.randn(H, taps, device="cuda", dtype=torch.float32)
        state = torch.zeros(2, taps - 1, H, device="cuda", dtype=torch.float32)
        cctx = SimpleNamespace(n_reqs=1, max_q_len=T,
                               q_start=torch.tensor([0, T], dtype=torch.int32, device="cuda"),
                               state_slot=torch.tensor([1], dtype=torch.int32, device="cuda"),
                               start_pos=torch.tensor([0], dtype=torch.int32, device="cuda"))
        timed("short_conv", [(lambda a=a, o=o: ops.short_conv(a, filt, None, None, state, cctx, o))
                             for a, o in zip(proj, outs)], T * H * 8)
        del proj
        qkv = [torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=bf) for _ in range(n * 3)]
        blocks = -(-T // ps)
        kcs = [torch.empty(blocks, ps, nkv, hd, device="cuda", dtype=bf) for _ in range(n * 3)]
        vcs = [torch.empty_like(k) for k in kcs]
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        slots = torch.randperm(blocks * ps, device="cuda").to(torch.int32)[:T].contiguous()
        qw = torch.ones(hd, device="cuda", dtype=torch.float32)
        inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
        ang = pos.float()[:, None] * inv[None, :]
        table = (ang.cos().contiguous(), ang.sin().contiguous())
        timed("qk_norm_rope_write",
              [(lambda a=a, k=k, v=v: ops.qk_norm_rope_write(a, nh, nkv, hd, qw, qw, 1e-5, table, pos,
                                                            slots, k, v))
               for a, k, v in zip(qkv, kcs, vcs)],
              T * hd * 2 * ((nh + nkv) * 2 + nkv + 2 * nkv))
        print(json.dumps({"only": "kernels", "peaks": pk["source"], "tokens": T, **res}))
        return 0
    if args.kernel == "all" or args.kernel.startswith("gemm"):
        M = args.kernel_m
        x = torch.randn(M, 8192, device="cuda", dtype=torch.bfloat16)
        shapes = ((6144, 2048), (2048, 2048), (3072, 2048), (16384, 2048), (2048, 8192),
                  (65536, 2048))
        if ":" in args.kernel:                       # gemm:NxK, one shape (for profiling)
            shapes = (tuple(int(v) for v in args.kernel.split(":")[1].split("x")),)
        for N, K in shapes:
            copies = max(4, min(48, (300 << 20) // (N * K * 2)))
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
            xs = x[:, :K].contiguous()
            t_lib = graph_time([(lambda w=w: torch.mm(xs, w.t())) for w in ws])
            t_own = graph_time([(lambda w=w: ops.linear_tcgen05(xs, w, torch.bfloat16)) for w in ws])
            out[f"gemm_m{M}_n{N}_k{K}"] = {
                "cublas_us": round(t_lib, 1), "tcgen05_us": round(t_own, 1),
                "tcgen05_GB/s": round(N * K * 2 / t_own / 1e3, 1),
                "frac_hbm": round(N * K * 2 / t_own / 1e3 / pk["hbm_gbs"], 3)}
            del ws
        ops.check_status()
    print(json.dumps(out))
    return 0


def run_workload(name, verbose=False):
    """One scheduler workload through `Engine.step`, after two untimed runs of the same
    requests (the reference's bench discards a warm-up run too, src/bin/bench.rs:215-232;
    prompts are seeded uniform random ids like its own, src/bin/bench.rs:93-109; random
    weights never produce a meaningful stop token, so none is set and every request
    generates its full length)."""
    import random

    import torch

    from rvllm_b200.config import config_from_dict
    import gc

    from rvllm_b200.engine import (Engine, ModelRunner, Request, SchedulerConfig, graphs_default,
                                   load_model, make_cache, settled_heap)
    from rvllm_b200.sampling import SamplingParams
    from rvllm_b200.weights import write_random_model

    w = WORKLOADS[name]
    data = dict(LFM2_1_2B)
    data.update(SIZES[w["size"]])
    data["max_position_embeddings"] = w["positions"]
    cfg = config_from_dict(data)
    tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=0)
        model, cfg = load_model(folder, "bfloat16", "cuda")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    rng = random.Random(17)
    lengths = [rng.randint(*w["prompt"]) for _ in range(w["requests"])]
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lengths]
    per_token = 2 * len(cfg.full_attn_idxs) * cfg.num_key_value_heads * cfg.head_dim * 2
    if w["pool"] == "fit":
        pages = sum(-(-(n + w["new"]) // PAGE) for n in lengths)
    else:
        torch.cuda.synchronize()
        free, _ = torch.cuda.mem_get_info()
        pages = int(0.9 * free) // (per_token * PAGE)
    cache = make_cache(model, PAGE, pages, w["requests"])
    runner = ModelRunner(model, cache, model.ops, use_graphs=graphs_default())
    sched = SchedulerConfig(block_size=PAGE, num_blocks=pages,
                            max_num_batched_tokens=w["chunk"] + w["requests"],
                            prefill_chunk=w["chunk"])

    def one_run(timed):
        engine = Engine(runner, sched, cfg.max_position_embeddings, lookahead=True)
        for i, ids in enumerate(prompts):
            engine.add_request(Request(i, ids, w["new"], (), SamplingParams(),
                                       arrival_step=i * w["arrival_gap"]))
        steps0, graph0 = runner.steps, runner.graph_steps
        captures0 = runner.captures
        marks, host = [], []
        out_tokens = 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while engine.has_work():
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            h0 = time.perf_counter()
            out_tokens += len(engine.step())
            host.append(time.perf_counter() - h0)
            b.record()
            marks.append((a, b))
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        model.ops.check_status()
        if not timed:
            return None
        device = [a.elapsed_time(b) for a, b in marks]
        if os.environ.get("RVLLM_BENCH_STEPS"):              # the slowest steps, for a look
            worst = sorted(range(len(device)), key=lambda i: -host[i])[:12]
            print("slowest steps (index, host ms, device ms):",
                  [(i, round(1e3 * host[i], 2), round(device[i], 2)) for i in sorted(worst)],
                  file=sys.stderr)
        st = engine.scheduler.stats
        n_steps = runner.steps - steps0
        busy = sum(device) / 1e3
        return {
            "model": f"LFM2-{w['size'].upper()} sizes", "requests": w["requests"],
            "prompt_tokens": sum(lengths), "new_tokens": out_tokens,
            "pool_pages": pages, "pool": w["pool"],
            "wall_s": round(wall, 3),
            "output_tok_s": round(out_tokens / wall, 1),
            "total_tok_s": round((sum(lengths) + out_tokens) / wall, 1),
            "steps": n_steps, "preemptions": st.preemptions,
            "graph_step_share": round((runner.graph_steps - graph0) / max(1, n_steps), 3),
            "host_ms_per_step": round(1e3 * sum(host) / len(host), 3),
            "device_ms_per_step": round(sum(device) / len(device), 3),
            "gpu_idle_frac": round(max(0.0, 1.0 - busy / wall), 3),
            "graphs_captured_meanwhile": runner.captures - captures0,
        }

    # two untimed runs: sizes that come once per run are met in the first and captured in the
    # second, so that the timed run, like steady traffic, replays (a capture costs 4 - 5 ms and
    # now and then 30 - 130 ms on this shared machine)
    one_run(False)
    one_run(False)
    # what earlier parts of the benchmark left on the Python heap is not walked again by the
    # garbage collector during the timed run, as in `rvllm_b200.engine.run`
    with settled_heap():
        result = one_run(True)
    del runner, cache, model
    gc.collect()
    torch.cuda.empty_cache()
    return result


def run_further(args):
    """Speed at further sizes, one JSON line: decode at batch 8 with 16,384 and 32,768 tokens of
    context, a prompt of 8,192 tokens taken in portions of 2,048 (convolution state and attention
    across portion boundaries at the real widths), and the samplers over 65,536 logits."""
    import torch

    from rvllm_b200.config import architecture, config_from_dict
    from rvllm_b200.engine import ModelRunner, StepEntry, graphs_default, load_model, make_cache
    from rvllm_b200.parts.model import param_decls
    from rvllm_b200.weights import write_random_model

    pk = peaks()
    data = dict(LFM2_1_2B)
    data["max_position_embeddings"] = 32768
    cfg = config_from_dict(data)
    tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=0)
        model, cfg = load_model(folder, "bfloat16", "cuda")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    ops = model.ops
    spec = architecture(cfg.architecture).build_spec(cfg)
    weight_bytes, matmul_params = model_bytes_and_flops(cfg, param_decls(spec))
    n_attn = len(cfg.full_attn_idxs)
    kv_per_token = n_attn * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    gen = torch.Generator().manual_seed(0)
    out = {"only": "further", "peaks": pk["source"]}

    def ids(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    B, steps = 8, 128
    for ctx in (16384, 32768):
        cache = make_cache(model, PAGE, B * (ctx // PAGE), B)
        runner = ModelRunner(model, cache, ops, use_graphs=graphs_default())
        for i in range(B):
            runner.add_request(i)
            toks = ids(ctx - steps - 8)
            for a in range(0, len(toks), 2048):
                runner.step([StepEntry(i, toks[a:a + 2048], ())])
        first = runner.decode_greedy(list(range(B)), [1] * B, 8)[-1].tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.decode_greedy(list(range(B)), first, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        nbytes = weight_bytes + B * (ctx - steps / 2) * kv_per_token
        out[f"decode_b{B}_ctx{ctx}"] = {"tok_s": round(B / (ms / 1e3), 1), "ms_per_step": round(ms, 4),
                                         "frac_hbm": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
        del runner, cache

    # a prompt of 8,192 tokens in portions of 2,048
    T, portion = 8192, 2048
    cache = make_cache(model, PAGE, T // PAGE, 1)
    runner = ModelRunner(model, cache, ops, use_graphs=False)
    toks = ids(T)
    times = []
    for it in range(4):
        runner.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for a in range(0, T, portion):
            runner.step([StepEntry("p", toks[a:a + portion], (portion - 1,) if a + portion == T else ())])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.end_request("p")
    ms = sorted(times[1:])[1]
    flops = 2.0 * T * matmul_params + 2.0 * cfg.vocab_size * cfg.hidden_size \
        + n_attn * 4.0 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2
    out["prefill_8192_in_portions_of_2048"] = {
        "tok_s": round(T / (ms / 1e3), 1), "ms": round(ms, 3),
        "frac_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    del runner, cache

    # the samplers over [rows, 65,536] float32 logits
    for rows in (8, 64):
        logits = torch.randn(rows, cfg.vocab_size, device="cuda", generator=None) * 3
        temp = torch.full((rows,), 0.8, device="cuda")
        seed = torch.arange(rows, dtype=torch.int64, device="cuda")
        counter = torch.zeros(rows, dtype=torch.int64, device="cuda")

        def timed(fn, reps=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return round(e0.elapsed_time(e1) * 1e3 / reps, 1)
        entry = {"argmax_us": timed(lambda: ops.argmax(logits))}
        for top_p in (1.0, 0.9):
            tp = torch.full((rows,), top_p, device="cuda")
            entry[f"sample_top_p_{top_p}_us"] = timed(lambda: ops.sample(logits, temp, tp, seed, counter))
        entry["logits_MB"] = round(rows * cfg.vocab_size * 4 / 1e6, 1)
        out[f"sampling_rows{rows}"] = entry
    ops.check_status()
    print(json.dumps(out))
    return 0


def run_reference(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "ermolushka/rvllm is a Rust crate (no setup.py/pyproject.toml: pip says "
                       "'not installable'); no cargo/rustc and no vendored crates offline"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="1.2b", choices=sorted(SIZES),
                    help="layer sizes: LFM2-1.2B (the default and the headline), 700M or 350M")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "kernels", "breakdown", "workload", "further"],
                    help="run one part only (for profiling); the JSON line then lacks the rest")
    ap.add_argument("--workloads", default="both", choices=["both", "none"] + sorted(WORKLOADS),
                    help="scheduler workloads to add to the line (default: both)")
    ap.add_argument("--workload", default="350m-mixed", choices=sorted(WORKLOADS),
                    help="with --only workload: which one")
    ap.add_argument("--kernel", default="all",
                    help="with --only kernels: attn_decode, attn_prefill, gemm, gemm:NxK, elementwise, copy_rate or all")
    ap.add_argument("--kernel-batch", type=int, default=64)
    ap.add_argument("--kernel-m", type=int, default=8, help="tokens of the gemm micro-benchmark")
    ap.add_argument("--kernel-ctx", type=int, default=4096)
    ap.add_argument("--kernel-tokens", type=int, default=PREFILL_TOKENS,
                    help="query tokens of the prefill attention micro-benchmark")
    ap.add_argument("--kernel-heads", type=int, default=32,
                    help="query heads of the attention micro-benchmarks (8 key/value heads)")
    ap.add_argument("--kernel-page", type=int, default=PAGE, help="page size of the attention micro-benchmarks")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only == "kernels":
        return run_kernels(args)
    if args.only == "further":
        return run_further(args)
    if args.only == "workload":
        print(json.dumps({"only": "workload", args.workload: run_workload(args.workload)}))
        return 0
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
