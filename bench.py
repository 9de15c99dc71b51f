#!/usr/bin/env python
"""Decode-throughput benchmark of the sm_100a backend.

  python bench.py --gpus N --steps K --warmup W            (our arm; torchrun for N > 1)
  python bench.py --impl reference --gpus N --steps K --warmup W   (CPU arm: the reference's C kernels)

Workload at every N: a Ministral-3B-shaped W4A16 (group-128) GQA decoder, batch 64 requests per
GPU, prompts of 2048 random token ids prefilled through the engine, then greedy decode; a "step"
is one decode step of the whole batch (64 tokens per GPU). Requests are independent, so ranks
share nothing on the data path (request-partitioned, weak scaling).
Prints ONE JSON line on rank 0.

The default line also carries sub-records measured after it in the same process (switch them off with --no-extras):
"gpt2_fp32" (N = 1: the reference's CPU-runnable case, one sequence), "dp512" (512 ragged requests bin-packed over the
ranks and served in waves: total work fixed, so its figures scale strongly with N) and, for N > 1, "tp" (one batch of 64
over a tensor-parallel group of all ranks, with a check that its greedy ids equal a single-rank engine's).

Other modes (none of them the default line): --workload gpt2-fp32 (the reference's CPU-runnable case: one sequence,
f32 weights), --workload dp512 (512 requests with prompt lengths U{256..4096}, 256 decode steps each, bin-packed over the
ranks and served in waves of 64: total work fixed, strong scaling), --weights w8a16, --parallelism tp (one batch over a
tensor-parallel group), --microbench
attention | attention-ragged | gemv | gemv-lm-head | gemm64 | quant-linear (single kernels, CUDA-graph timed; used for ncu captures)
| prefill (a few 2048-token prompts through the engine's chunked prefill; --steps = number of prompts).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = "ministral3b-shaped W4A16-g128 decode, batch 64/GPU, 2048-token prompts prefilled, greedy"
PROMPT_LEN = 2048
BATCH = 64
OUT = [sys.stdout]  # the stream that receives the one JSON line (see main)


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str | None):
        self.uuid, self.rows, self.proc = uuid, [], None

    def start(self):
        cmd = ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"]
        if self.uuid:
            cmd += ["-i", self.uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_model(gm, torch, dev, steps_total: int, use_pdl: int, prefill_chunk: int, tp_size: int = 1, tp_rank: int = 0, nccl_id=None,
                weight_mode=None, max_context=None):
    ctx = (((max_context or PROMPT_LEN + steps_total + 64) + 15) // 16) * 16
    pages_per_seq = ctx // 16
    cfg = gm.ModelConfig.ministral_3b(context_length=ctx, weight_mode=weight_mode or gm.MODE_W4A16, max_seqs=BATCH,
                                      max_tokens=prefill_chunk, max_logit_rows=BATCH,
                                      kv_pages=BATCH * pages_per_seq + 8, max_pages_per_seq=pages_per_seq, use_pdl=use_pdl,
                                      tp_size=tp_size, tp_rank=tp_rank)
    model = gm.LoadedModel(cfg, namespace=0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    for name, shape in cfg.param_shapes().items():
        if name.endswith("gamma"):
            w = torch.ones(shape, dtype=torch.float32, device=dev)
        else:
            w = torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, 0.02, generator=gen)
        model.load_param(name, w)
        del w
    if tp_size > 1:
        model.init_tensor_parallel(nccl_id)
    model.finalize(drop_f32_leaves=True)
    torch.cuda.empty_cache()
    return model, cfg


def _tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text()).get("bf16_tflops") or 0) or None
    return 1590.0


def time_attention_kernel(ops, torch, dev, ctx_len: int, launches: int = 20, ragged_seed=None):
    """CUDA-event time of the dominant kernel (paged decode attention of ONE layer) on a synthetic
    pool of the bench geometry; every launch streams the whole pool (> L2). With `ragged_seed` the
    context lengths are drawn uniformly from 512..ctx_len and the physical pages are a random permutation."""
    n_q, n_kv = 32, 8
    pages_per = (ctx_len + 15) // 16
    if ragged_seed is None:
        lens_host = [ctx_len] * BATCH
    else:
        import numpy as np
        lens_host = [int(v) for v in np.random.default_rng(ragged_seed).integers(512, ctx_len + 1, size=BATCH)]
    total = BATCH * pages_per
    pool = torch.randn(total * n_kv * 2 * 16 * 128, dtype=torch.bfloat16, device=dev).view(torch.uint8)
    table = torch.randperm(total, device=dev, dtype=torch.int32).view(BATCH, pages_per).contiguous()
    q = torch.randn((BATCH, n_q, 128), dtype=torch.bfloat16, device=dev)
    slot = torch.arange(BATCH, dtype=torch.int32, device=dev)
    lens = torch.tensor(lens_host, dtype=torch.int32, device=dev)
    bucket = ((ctx_len + 511) // 512) * 512
    from gptrs_b200 import lib
    chunk = lib().gptrs_cuda_attention_chunk_pages(bucket, BATCH, n_kv)
    out = torch.empty((BATCH, n_q * 128), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nbytes = lib().gptrs_cuda_attention_scratch_bytes(BATCH, n_q, min(bucket, pages_per * 16), chunk)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)

    def launch():
        from gptrs_b200 import check
        check(lib().gptrs_cuda_paged_attention_decode(
            q.data_ptr(), pool.data_ptr(), table.data_ptr(), pages_per, slot.data_ptr(), lens.data_ptr(), out.data_ptr(),
            scratch.data_ptr(), nbytes, status.data_ptr(), BATCH, n_q, n_kv, 128, min(bucket, pages_per * 16), chunk,
            torch.cuda.current_stream().cuda_stream))

    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph.capture_begin()
        for _ in range(launches):
            launch()
        graph.capture_end()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / launches
    alg_bytes = sum(lens_host) * 4096 + 2 * BATCH * n_q * 128 * 2 + sum((v + 15) // 16 for v in lens_host) * 4
    del pool
    return ms, alg_bytes, chunk


def time_prefill_attention(ops, torch, dev, ctx_len: int, n_seq: int = 4, launches: int = 5):
    """CUDA-event time of the prefill attention of ONE layer over whole prompts of `ctx_len` tokens (row t of a
    sequence sees keys 0..t; 32 query / 8 kv heads of 128, random page permutation): the tensor-core kernel and the
    grouped mma.sync kernel on the same inputs. FLOPs counted: 4 x head_dim per visible (query, key) pair and head."""
    n_q, n_kv = 32, 8
    ctx_len = (ctx_len + 63) // 64 * 64   # every prompt starts a new 64-token tile of the tensor-core kernel
    pages_per = (ctx_len + 15) // 16
    total = n_seq * pages_per
    pool = (torch.randn(total * n_kv * 2 * 16 * 128, device=dev) * 0.5).to(torch.bfloat16).view(torch.uint8)
    table = torch.randperm(total, device=dev, dtype=torch.int32).view(n_seq, pages_per).contiguous()
    q = torch.randn((n_seq * ctx_len, n_q, 128), device=dev).to(torch.bfloat16)
    slot = torch.arange(n_seq, dtype=torch.int32, device=dev).repeat_interleave(ctx_len).contiguous()
    ctx = torch.arange(1, ctx_len + 1, dtype=torch.int32, device=dev).repeat(n_seq).contiguous()
    flops = 4.0 * 128 * n_q * n_seq * ctx_len * (ctx_len + 1) / 2
    res = {}
    for name, mode in (("paged_prefill_tc_kernel", "tc"), ("paged_attention_kernel<2,1>", True)):
        for _ in range(2):
            out, st = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, ctx_len, prefill=mode)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(launches):
            out, st = ops.paged_attention_decode(q, pool, table, slot, ctx, n_q, n_kv, ctx_len, prefill=mode)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / launches
        res[name] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "status": int(st.item())}
    return res, flops


def time_gemv(ops, torch, dev, n=9216, k=3072, m=1, n_mats=64, iters=3, bits=4, pdl=True):
    """W4A16 / W8A16 matmul over a rotating set of distinct weight matrices (working set >> L2)."""
    if bits == 4:
        nbytes = ops.w4a16_packed_bytes(n, k)
        mats = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev) for _ in range(n_mats)]
        half = n * k // 2 + n * (k // 128) * 2  # the buffer holds two layouts, each weights then fp16 scales
        for mt in mats:  # keep the fp16 scale bits finite
            mt[n * k // 2:half] = 0x1C
            mt[half + n * k // 2:] = 0x1C
        run = ops.quant_matmul_w4a16
        weight_bytes = nbytes // 2  # a launch reads ONE of the two weight layouts
    else:
        nbytes = ops.w8a16_packed_bytes(n, k)
        mats = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev) for _ in range(n_mats)]
        for mt in mats:  # per-channel fp16 scales of both layouts: finite bit patterns
            mt[n * k:n * k + 2 * n] = 0x1C
            mt[nbytes - 2 * ((n + 127) // 128) * 128:] = 0x1C
        run = ops.quant_matmul_w8a16
        weight_bytes = n * k + 2 * n  # a launch reads ONE of the two weight layouts
    x = torch.randn((m, k), dtype=torch.bfloat16, device=dev)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    for mt in mats[:4]:
        run(x, mt, m, n, k, out=y)
    torch.cuda.synchronize()
    # one CUDA graph over all matrices: the timing sees the device, not the Python launch rate
    # ... and the launches carry programmatic dependent launch edges, as in the engine's recorded decode step
    from gptrs_b200 import lib as _lib
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    before = _lib().gptrs_cuda_set_thread_pdl(1 if pdl else 0)
    try:
        with torch.cuda.stream(side):
            graph.capture_begin()
            for mt in mats:
                run(x, mt, m, n, k, out=y)
            graph.capture_end()
    finally:
        _lib().gptrs_cuda_set_thread_pdl(before)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (iters * n_mats)
    alg = weight_bytes + 2 * m * k + 2 * m * n
    return us, alg


def run_reference_arm(args):
    """CPU arm: the gpt.rs C backend's kernel library (oracle/_ref) driving the restated f32 decode
    step on the host. The reference's kernels are single-threaded and requests are independent, so one
    process per host core (at most 64) runs its share of the batch at once; each step is one bounded
    sample taken by all processes together. The GPT-2 workload is one sequence, hence one thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cbaseline as cb
    lib = cb.load(prefer_reference=True)
    if args.workload == "gpt2-fp32":
        res = cb.time_gpt2_decode(lib, n_tokens=max(4, min(args.steps, 32)))
        v = res["tokens_per_s"]
        print(json.dumps({"impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": GPT2_WORKLOAD},
                          "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]},
                          "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}), file=OUT[0])
        return
    procs = cb.host_processes(min(64, BATCH))  # requests are independent: one share of the batch per host core
    res = cb.time_ministral_step_parallel(lib, procs, reps=args.warmup + args.steps, batch=BATCH, ctx_len=PROMPT_LEN, sample_rows=1)
    vals = res["rep_tokens_per_s"][args.warmup:]
    v = sum(vals) / len(vals)
    n = args.gpus
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * BATCH / v, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU arm: f32 weights (the reference has no quantised path), host cores only, one process per core (at most 64)"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=OUT[0])


GPT2_PUBLISHED_TOKENS_PER_S = 74.71  # the reference README's GPT-2 small row (C backend, single thread)
GPT2_WORKLOAD = "gpt2-small fp32, one sequence, 32-token prompt, greedy decode with the dense-cache f32 kernels (one cooperative kernel per token)"


def run_gpt2(args, out, gm, torch, np):
    if args.path == "run_program":
        print(json.dumps(measure_gpt2_run_program(args, torch, np)), file=out)
        return
    print(json.dumps(measure_gpt2(args, gm, torch, np, cpu_baseline=not args.no_cpu_baseline)), file=out)


def measure_gpt2_run_program(args, torch, np):
    """GPT-2 small decode driven ONLY through PortableBackend::run_program: the captured one-token decode program (the
    op sequence gpt.rs' functionals emit, capacity bucket 128), its weights as parameter handles, the previous step's
    K/V handles in and fresh ones out every step, the next id picked by the backend's decode sampler. Timed on the host
    clock around the loop (every step ends with the synchronous read of the sampled id)."""
    from types import SimpleNamespace
    from gptrs_b200 import ptir
    from gptrs_b200 import lib as _lib
    from gptrs_b200.backend import CudaBackend
    torch.cuda.set_device(0)
    cfg = SimpleNamespace(kind="gpt", n_layers=12, d_model=768, n_q=12, n_kv=12, hd=64, d_mlp=3072, vocab=50257, ctx=1024, eps=1e-5, rot=0)
    cap = 128
    be = CudaBackend()
    builder, names = ptir.decode_step_program(cfg, cap)
    prog = be.prepare(builder.to_json())
    rng = np.random.default_rng(0)
    weights = {}
    shapes = {p.id: p.dims for p in builder.params}
    for n, p in zip(names, builder.params):
        if n.startswith("@"):
            continue
        if n.endswith("gamma"):
            w = np.ones(p.dims, np.float32)
        elif n.endswith("beta") or ".b_" in n:
            w = np.zeros(p.dims, np.float32)
        else:
            w = rng.normal(0.0, 0.02, size=p.dims).astype(np.float32)
        weights[n] = be.materialize(w)
    caches = [(be.materialize_zeroed(np.float32, [cfg.n_kv, cap, cfg.hd]), be.materialize_zeroed(np.float32, [cfg.n_kv, cap, cfg.hd]))
              for _ in range(cfg.n_layers)]
    state = {"tok": 0, "pos": 0}

    def step():
        tok, pos = state["tok"], state["pos"]
        small = {"@tokens": np.array([tok], np.int32), "@positions": np.array([pos], np.int32),
                 "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
        hs = []
        for n in names:
            if n in small:
                hs.append(be.materialize(small[n]))
            elif n.startswith("@k"):
                hs.append(caches[int(n[2:])][0])
            elif n.startswith("@v"):
                hs.append(caches[int(n[2:])][1])
            else:
                hs.append(weights[n])
        res = prog.run(hs)
        state["replays"] = state.get("replays", 0) + int(_lib().gptrs_cuda_last_run_replayed_graph())
        for l in range(cfg.n_layers):
            caches[l] = (res[1 + 2 * l], res[2 + 2 * l])
        state["tok"] = be.sample_decode_token(res[0], 0.0)
        state["pos"] = pos + 1

    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=32)
    for t in prompt[:-1]:    # the prompt, one token per call (set-up, not timed)
        state["tok"] = int(t)
        step()
    state["tok"] = int(prompt[-1])
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    allocs0 = be.alloc_stats()["driver_allocs"]
    state["replays"] = 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st, al = be.run_program_stats(), be.alloc_stats()
    weight_bytes = 4 * sum(int(np.prod(p.dims)) for n, p in zip(names, builder.params) if not n.startswith("@") and "embeddings" not in n)
    peak, peak_kind = _peaks()
    return {"metric": "decode_tokens_per_s", "value": args.steps / dt, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": args.steps / dt / GPT2_PUBLISHED_TOKENS_PER_S, "dtype": "f32", "data": "synthetic",
            "config": {"workload": GPT2_WORKLOAD.replace("the dense-cache f32 kernels (one cooperative kernel per token)", "every step one PortableBackend::run_program call"),
                       "path": "run_program", "capacity_bucket": cap, "l2": "494 MB of f32 weights streamed per token (> L2)",
                       "program_instructions": len(builder.body)},
            "e2e": {"value": args.steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": 32, "d2h_bytes_per_step": 8,
                    "note": "the timed loop is the end-to-end loop: host arguments in, sampled id out, every step"},
            "gpu_launches": int(st["last_launches"]) * args.steps, "launches_per_token": int(st["last_launches"]),
            "fused_rewrites": int(st["last_fused"]), "driver_allocs_in_timed_region": int(al["driver_allocs"] - allocs0),
            "pool_hits": int(al["pool_hits"]), "graph_replays_in_timed_region": int(state["replays"]),
            "roofline": {"kernel": "all weight matrices of a step", "bound": "hbm", "achieved": weight_bytes / dt * args.steps / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": weight_bytes / dt * args.steps / 1e9 / peak, "traffic": None,
                         "peak_kind": peak_kind}}


def measure_gpt2(args, gm, torch, np, cpu_baseline: bool, device_index: int = 0):
    """The reference's CPU-runnable case on one GPU: GPT-2 small, f32 weights N(0, 0.02) seed 0, a 32-token
    random prompt, greedy decode; a step is one generated token."""
    torch.cuda.set_device(device_index)
    dev = torch.device("cuda", device_index)
    cfg = gm.ModelConfig.gpt2_small(weight_mode=gm.MODE_F32, max_seqs=1, max_tokens=32, max_logit_rows=32, use_pdl=args.pdl)
    model = gm.LoadedModel(cfg, namespace=7)
    gen_t = torch.Generator(device=dev)
    gen_t.manual_seed(0)
    for name, shape in cfg.param_shapes().items():
        if name.endswith("gamma"):
            w = torch.ones(shape, dtype=torch.float32, device=dev)
        elif name.endswith("beta") or ".b_" in name:
            w = torch.zeros(shape, dtype=torch.float32, device=dev)
        else:
            w = torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, 0.02, generator=gen_t)
        model.load_param(name, w)
    model.finalize()
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=32)
    model.reset_sequence(0)
    _, first = model.prefill(0, prompt)
    gen = gm.Generator(model, [first], use_graph=True)
    stream = torch.cuda.ExternalStream(lib_stream(model), device=dev)
    for _ in range(args.warmup):
        gen.step(read_back=False)
    gen.sync()
    sampler = ClockSampler(None)
    launches0 = model.stats()["kernel_launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.start()
    e0.record(stream)
    for _ in range(args.steps):
        gen.step(read_back=False)
    e1.record(stream)
    gen.sync()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = model.stats()["kernel_launches"] - launches0
    tok = int(gen.step()[0])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = int(gen.step(tokens_in=[tok])[0])
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    weight_bytes = 4 * sum(int(np.prod(sh)) for n, sh in cfg.param_shapes().items() if "embeddings" not in n)
    peak, peak_kind = _peaks()
    line = {"metric": "decode_tokens_per_s", "value": args.steps / ms * 1e3, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": args.steps / ms * 1e3 / GPT2_PUBLISHED_TOKENS_PER_S,
            "dtype": "f32", "data": "synthetic", "config": {"workload": GPT2_WORKLOAD, "cuda_graph": True, "pdl": bool(args.pdl),
            "published_baseline": "74.71 tokens/s, gpt.rs C backend, one thread, Ryzen 9 9950X3D, pretrained weights (random weights of the same shapes here)",
            "l2": "494 MB of f32 weights streamed per token (> L2)"},
            "e2e": {"value": args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "clocks": clocks,
            "roofline": {"kernel": "gpt_decode_mega_kernel (all weight matrices of a step)", "bound": "hbm", "achieved": weight_bytes / (ms / args.steps) / 1e6,
                         "peak": peak, "unit": "GB/s", "frac": weight_bytes / (ms / args.steps) / 1e6 / peak, "traffic": None,
                         "peak_kind": peak_kind, "note": "whole-step figure: f32 weight bytes of one token over the step time"}}
    line["launches_per_token"] = launches / max(args.steps, 1)
    if cpu_baseline:
        from oracle import cbaseline as cb
        res = cb.time_gpt2_decode(cb.load(prefer_reference=True), n_tokens=8)
        line["cpu_baseline"] = {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]}
    model.close()
    return line


def run_dp512(args, out, gm, torch, np):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    line = measure_dp512(args, gm, torch, np, dist, world, rank, dev)
    if rank == 0:
        print(json.dumps(line), file=out)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def measure_dp512(args, gm, torch, np, dist, world, rank, dev):
    """512 requests with prompt lengths U{256..4096} (seed 0), 256 greedy decode steps each: the requests are
    bin-packed over the ranks by token count, every rank serves its shard in waves of 64 on its own engine and
    KV pool, and the only exchange is the host-side gather of the generated ids. Times are CUDA events on each
    engine's stream around every phase, summed per rank, max over ranks (and the mean, for the imbalance).
    Returns the JSON line (every rank computes it; rank 0's is the one to print)."""
    from gptrs_b200 import parallel
    lo, hi = 256, 4096
    lens = np.random.default_rng(0).integers(lo, hi + 1, size=args.requests)
    assign, cost = parallel.partition_requests(lens, args.decode_steps, world)
    mine = parallel.shard_of(assign, rank)
    model, cfg = build_model(gm, torch, dev, 0, args.pdl, args.prefill_chunk, max_context=hi + args.decode_steps + 16)
    rng = np.random.default_rng(2000)
    all_prompts = [rng.integers(0, cfg.vocab, size=int(n)) for n in lens]  # same arrays on every rank
    prompts = {int(i): all_prompts[int(i)] for i in mine}
    stream = torch.cuda.ExternalStream(lib_stream(model), device=dev)
    # warm-up: one short wave, so that graph capture and first-launch costs stay outside the timed region
    parallel.run_requests(model, {int(i): all_prompts[int(i)][:64] for i in mine[:BATCH]}, max(args.warmup, 3), BATCH, args.prefill_chunk)
    spans = {"prefill": [], "decode": []}
    wall = {"prefill": 0.0, "decode": 0.0}

    def timed(name, wave, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record(stream)
        fn()
        e1.record(stream)
        torch.cuda.synchronize()
        wall[name] += time.perf_counter() - t0
        spans[name].append(e0.elapsed_time(e1))

    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid)
    launches0 = model.stats()["kernel_launches"]
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    ids = parallel.run_requests(model, prompts, args.decode_steps, BATCH, args.prefill_chunk, on_phase=timed)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop()
    launches = model.stats()["kernel_launches"] - launches0
    merged = parallel.gather_generated(ids, world)
    t = torch.tensor([sum(spans["decode"]), sum(spans["prefill"]), wall["decode"] * 1e3, (wall["decode"] + wall["prefill"]) * 1e3],
                     dtype=torch.float64, device=dev)
    t_sum = t.clone()
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_sum, op=dist.ReduceOp.SUM)
    dec_ms, pre_ms, dec_wall_ms, job_ms = (float(x) for x in t)
    job_mean_ms = float(t_sum[3]) / world
    tokens = args.requests * args.decode_steps
    waves = len(spans["decode"])
    model.close()
    assert sorted(merged) == list(range(args.requests)) and all(len(v) == args.decode_steps + 1 for v in merged.values())
    line = {"metric": "decode_tokens_per_s", "value": tokens / (dec_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": waves * args.decode_steps, "warmup": max(args.warmup, 3), "ms_per_step": dec_ms / max(waves * args.decode_steps, 1),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 activations x int4 weights, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"Ministral-3B-shaped W4A16-g128, {args.requests} requests, prompt lengths U{{{lo}..{hi}}} (seed 0), "
                                   f"{args.decode_steps} greedy decode steps each, waves of {BATCH} per GPU",
                       "parallelism": f"dp{world} (requests bin-packed by token count, no collective)",
                       "rank_token_cost": [int(c) for c in cost], "waves_on_rank0": waves,
                       "l2": "inputs larger than L2 (1.8 GB weights + KV of the wave streamed per step)",
                       "cuda_graph": True, "pdl": bool(args.pdl), "kv_cache": "paged bf16, 16-token pages",
                       "prefill_seconds": round(pre_ms * 1e-3, 2), "prefill_tokens": int(lens.sum()),
                       "prefill_tokens_per_s": float(lens.sum()) / (pre_ms * 1e-3),
                       "job_seconds": round(job_ms * 1e-3, 2), "requests_per_s": args.requests / (job_ms * 1e-3),
                       "rank_time_max_over_mean": job_ms / max(job_mean_ms, 1e-9),
                       "token_step_cost_per_rank": [int(c) for c in cost]},
            "e2e": {"value": tokens / (dec_wall_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": BATCH * 4,
                    "d2h_bytes_per_step": BATCH * 4, "note": "host ids in and sampled ids out on every step; value is the same loop timed with CUDA events"},
            "gpu_launches": int(launches), "clocks": clocks}
    return line


def measure_tp(args, gm, torch, np, dist, world, rank, dev, single_rank_model, single_cfg):
    """One batch of 64 requests (2048-token prompts) over a tensor-parallel group of all ranks: ms per decode step and
    tokens/s, CUDA events, max over ranks. `check`: the single-rank engine of rank 0 prefills 24 48-token prompts and
    decodes eight greedy steps; the tensor-parallel engine does the same, fed the single-rank ids at every step; the
    216 ids are compared one by one (the weights are random, so a few exact near-ties between the two summation orders
    are possible: the count is reported)."""
    steps_total = args.warmup + args.steps + 32
    NP = 24   # more than 16 rows: the decode steps of the check run the tensor-core matmuls, like the timed batch
    short = [np.random.default_rng(77 + i).integers(0, 131072, size=48) for i in range(NP)]

    GAP = 0.1   # logits of this model have a standard deviation of about 1.1; two engines agree to a few hundredths

    def reference_run(m):
        """The single-rank engine: first id from every prompt, then eight eager decode steps with the logits read back.
        Returns the ids per step and, per id, whether the top-2 gap of its logits row makes it a decided choice."""
        for s_ in range(NP):
            m.reset_sequence(s_)
        cur = list(m.prefill_many(list(range(NP)), short, chunk=args.prefill_chunk))
        ids, sure = [cur], [[False] * NP]   # the first ids come without logits: compared but reported apart
        for k in range(8):
            pos = [48 + k] * NP
            lg, tok = m.forward_with_decode_cache(cur, list(range(NP)), pos, list(range(NP)))
            top = np.sort(lg, axis=1)
            ids.append([int(t) for t in tok])
            sure.append([bool(g) for g in (top[:, -1] - top[:, -2]) > GAP])
            cur = ids[-1]
        for s_ in range(NP):
            m.reset_sequence(s_)
        return ids, sure

    def forced_run(m, ref_ids):
        """The tensor-parallel engine, fed the reference's ids at every step (one near-tie cannot change what follows)."""
        for s_ in range(NP):
            m.reset_sequence(s_)
        first = m.prefill_many(list(range(NP)), short, chunk=args.prefill_chunk)
        g = gm.Generator(m, ref_ids[0], use_graph=True)
        ids = [[int(t) for t in first]]
        for k in range(8):
            ids.append(g.step(tokens_in=ref_ids[k]).tolist())
        for s_ in range(NP):
            m.reset_sequence(s_)
        return ids

    ref_box = [reference_run(single_rank_model) if rank == 0 else None]
    dist.broadcast_object_list(ref_box, src=0)
    ref_ids, ref_sure = ref_box[0]

    def one(collective):
        """Builds the tensor-parallel engine with the given collective, checks it, times it."""
        os.environ["GPTRS_TP_ALLREDUCE"] = collective
        box = [gm.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        model, cfg = build_model(gm, torch, dev, steps_total, args.pdl, args.prefill_chunk, world, rank, box[0])
        kind = model.tp_allreduce_kind()
        tp_ids = forced_run(model, ref_ids)
        differ = sum(int(a != b) for ra, rb in zip(tp_ids, ref_ids) for a, b in zip(ra, rb))
        decided = sum(int(a != b and ok) for ra, rb, rs in zip(tp_ids, ref_ids, ref_sure) for a, b, ok in zip(ra, rb, rs))
        flags = torch.tensor([differ, decided], dtype=torch.int32, device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MAX)
        rng = np.random.default_rng(1000)
        prompts = [rng.integers(0, cfg.vocab, size=PROMPT_LEN) for _ in range(BATCH)]
        first = model.prefill_many(list(range(BATCH)), prompts, chunk=args.prefill_chunk)
        gen = gm.Generator(model, first, use_graph=True)
        stream = torch.cuda.ExternalStream(lib_stream(model), device=dev)
        for _ in range(args.warmup):
            gen.step(read_back=False)
        gen.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            gen.step(read_back=False)
        e1.record(stream)
        gen.sync()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del gen
        model.close()
        os.environ.pop("GPTRS_TP_ALLREDUCE", None)
        return float(t[0]) / args.steps, (int(flags[0]), int(flags[1])), kind

    # the engine's default collective for this group size first, the other one for comparison
    first, second = ("peer", "nccl") if world <= 2 else ("nccl", "peer")
    ms, (differ, decided), kind = one(first)
    ms_other, (differ_other, decided_other), kind_other = one(second)
    n_collectives = 2 * 26
    n_sure = sum(int(ok) for rs in ref_sure for ok in rs)
    return {"parallelism": f"tp{world}", "batch": BATCH, "ms_per_step": ms, "tokens_per_s": BATCH / (ms * 1e-3),
            "collective": f"{kind}: all-reduce(sum, f32 [64, 3072]) after o_proj and down_proj, {n_collectives} per step, inside the decode graph"
                          + ("; the matmul epilogue stores its tile into the peers' receive slots, the norm kernel that follows waits for the marks and adds the tiles"
                             if kind.startswith("peer") else ""),
            "other_collective": {"collective": kind_other, "ms_per_step": ms_other, "ids_that_differ": differ_other,
                                 "decided_ids_that_differ": decided_other,
                                 "us_per_collective_vs_default": (ms_other - ms) * 1e3 / n_collectives},
            "check": {"same_greedy_ids_as_single_rank": decided == 0, "decided_ids_compared": n_sure, "decided_ids_that_differ": decided,
                      "ids_compared": 9 * NP, "ids_that_differ": differ,
                      "rule": f"teacher-forced; an id is decided when the single-rank logits' top-2 gap exceeds {GAP}", "prompts": NP, "steps": 8}}


def main():
    # Libraries (NCCL banners, warnings) may write to stdout; the contract is ONE JSON line there.
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    try:
        _main(real_stdout)
    finally:
        real_stdout.flush()


def _main(out):
    OUT[0] = out
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill-chunk", type=int, default=1536,
                    help="rows per prefill pass: 1536 = 6 tiles of 256 rows, so the 24-column-tile projections launch 144 CTAs (one wave of 148 SMs)")
    ap.add_argument("--pdl", type=int, default=int(os.environ.get("GPTRS_PDL", "1")))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the kernel microbenchmarks")
    ap.add_argument("--microbench", default=None, choices=["attention", "attention-ragged", "gemv", "gemv-lm-head", "gemm64", "quant-linear", "prefill", "prefill-attention"],
                    help="run only one kernel microbenchmark (used for ncu captures) and print its JSON")
    ap.add_argument("--ctx", type=int, default=PROMPT_LEN + 20, help="context length for --microbench attention")
    ap.add_argument("--workload", default="ministral3b-w4", choices=["ministral3b-w4", "gpt2-fp32", "dp512"],
                    help="gpt2-fp32 = the reference's CPU-runnable case (one sequence, 32-token prompt, 64 greedy tokens); "
                         "dp512 = 512 requests with prompt lengths U{256..4096}, 256 decode steps each, partitioned over the ranks "
                         "(total work fixed: strong scaling; not the default line)")
    ap.add_argument("--path", default="engine", choices=["engine", "run_program"],
                    help="gpt2-fp32 only: engine = the model-level ABI (default); run_program = every decode step one "
                         "PortableBackend::run_program call on the captured decode program")
    ap.add_argument("--requests", type=int, default=512, help="dp512: number of requests")
    ap.add_argument("--decode-steps", type=int, default=256, help="dp512: decode steps per request")
    ap.add_argument("--weights", default="w4a16", choices=["w4a16", "w8a16"],
                    help="w8a16 = the same workload with per-channel int8 weights (not the default line)")
    ap.add_argument("--sub", default="tp,dp512,gpt2", help="sub-records measured after the default line (comma list of tp, dp512, gpt2)")
    ap.add_argument("--parallelism", default="dp", choices=["dp", "tp"],
                    help="dp: every rank decodes its own 64 requests (default); tp: all ranks share ONE batch of 64 "
                         "(tensor parallel, NCCL all-reduce after the row-parallel projections)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import numpy as np
    import torch
    import __graft_entry__ as entry
    entry.load_package()
    from gptrs_b200 import model as gm
    from gptrs_b200 import ops

    if args.workload == "gpt2-fp32":
        run_gpt2(args, out, gm, torch, np)
        return
    if args.workload == "dp512":
        run_dp512(args, out, gm, torch, np)
        return
    if args.microbench == "prefill":
        # chunked prefill of a few 2048-token prompts through the engine (used for the ncu launch list of the prefill path)
        torch.cuda.set_device(0)
        dev = torch.device("cuda", 0)
        model, cfg = build_model(gm, torch, dev, 0, args.pdl, args.prefill_chunk)
        stream = torch.cuda.ExternalStream(lib_stream(model), device=dev)
        rng = np.random.default_rng(1000)
        n_seq = max(args.steps, 1) if args.steps != 64 else 4
        model.prefill(0, rng.integers(0, cfg.vocab, size=PROMPT_LEN), chunk=args.prefill_chunk)  # warm-up
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for s_ in range(1, 1 + n_seq):
            model.prefill(s_, rng.integers(0, cfg.vocab, size=PROMPT_LEN), chunk=args.prefill_chunk)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        qkv_w = (cfg.n_q_heads + 2 * cfg.n_kv_heads) * cfg.head_dim
        per_layer = cfg.d_model * qkv_w + cfg.n_q_heads * cfg.head_dim * cfg.d_model + 3 * cfg.d_model * cfg.d_mlp
        flops = 2.0 * cfg.n_layers * per_layer * PROMPT_LEN * n_seq  # projections only (attention and the one lm_head row left out)
        print(json.dumps({"microbench": "prefill", "sequences": n_seq, "prompt_tokens": PROMPT_LEN, "chunk": args.prefill_chunk,
                          "ms": ms, "tokens_per_s": n_seq * PROMPT_LEN / ms * 1e3, "matmul_tflops": flops / ms / 1e9}), file=out)
        return

    if args.microbench:
        torch.cuda.set_device(0)
        dev = torch.device("cuda", 0)
        peak, _ = _peaks()
        if args.microbench == "attention":
            ms, nbytes, chunk = time_attention_kernel(ops, torch, dev, args.ctx, launches=5)
            print(json.dumps({"kernel": "paged_attention_kernel", "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6,
                              "frac": nbytes / ms / 1e6 / peak, "chunk_pages": chunk, "ctx": args.ctx}), file=out)
        elif args.microbench == "prefill-attention":
            res, flops = time_prefill_attention(ops, torch, dev, args.ctx)
            tf_peak = _tensor_peak()
            print(json.dumps({"microbench": "prefill-attention", "workload": f"4 prompts of {(args.ctx + 63) // 64 * 64} tokens, causal, 32 q / 8 kv heads of 128, one layer",
                              "flops": flops, "bf16_peak_tflops": tf_peak, "kernels": res,
                              "frac_of_bf16_peak": round(res["paged_prefill_tc_kernel"]["tflops"] / tf_peak, 3) if tf_peak else None}), file=out)
        elif args.microbench == "attention-ragged":
            ms, nbytes, chunk = time_attention_kernel(ops, torch, dev, 8192, launches=5, ragged_seed=0)
            print(json.dumps({"kernel": "paged_attention_kernel", "workload": "batch 64, context lengths U{512..8192} (seed 0), 32 q / 8 kv heads of 128, random page permutation",
                              "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak,
                              "chunk_pages": chunk}), file=out)
        elif args.microbench == "quant-linear":
            rows = []
            tf_peak = _tensor_peak()
            for bits in (4, 8):
                for n in (3072, 9216):
                    for m in (1, 16, 64, 256):
                        per = n * 3072 * bits // 8
                        n_mats = max(8, min(64, (400 << 20) // per))  # rotating working set of about 400 MB (> L2)
                        us, alg = time_gemv(ops, torch, dev, n=n, k=3072, m=m, n_mats=n_mats, iters=3, bits=bits)
                        tf = 2.0 * m * n * 3072 / us / 1e6
                        rows.append({"bits": bits, "M": m, "N": n, "K": 3072, "us": round(us, 2), "algorithmic_bytes": alg,
                                     "gbs": round(alg / us / 1e3, 1), "frac_of_hbm_peak": round(alg / us / 1e3 / peak, 3),
                                     "tflops": round(tf, 1), "frac_of_bf16_peak": round(tf / tf_peak, 3) if tf_peak else None})
            print(json.dumps({"microbench": "quant-linear", "hbm_peak_gbs": peak, "bf16_peak_tflops": tf_peak,
                              "note": "rotating distinct weight matrices (> L2), back-to-back launches in one CUDA graph, CUDA events",
                              "rows": rows}), file=out)
        elif args.microbench == "gemv":
            us, nbytes = time_gemv(ops, torch, dev, n_mats=16, iters=1)
            print(json.dumps({"kernel": "w4_gemv_kernel<1,2> M=1 N=9216 K=3072", "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}), file=out)
        elif args.microbench == "gemv-lm-head":
            us, nbytes = time_gemv(ops, torch, dev, n=131072, k=3072, n_mats=4, iters=1)
            print(json.dumps({"kernel": "w4_gemv_kernel<1,4> M=1 N=131072 K=3072", "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}), file=out)
        else:
            us, nbytes = time_gemv(ops, torch, dev, n=6144, k=3072, m=64, n_mats=16, iters=1)
            print(json.dumps({"kernel": "umma_w4a16_kernel<64>", "us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3}), file=out)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    steps_total = args.warmup + 2 * args.steps + 8  # device-resident loop, then the end-to-end loop
    t_setup = time.perf_counter()
    tp = args.parallelism == "tp" and world > 1
    nccl_id = None
    if tp:
        box = [gm.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        nccl_id = box[0]
    w8 = args.weights == "w8a16"
    model, cfg = build_model(gm, torch, dev, steps_total, args.pdl, args.prefill_chunk, world if tp else 1, rank if tp else 0, nccl_id,
                             gm.MODE_W8A16 if w8 else gm.MODE_W4A16)
    t_weights = time.perf_counter() - t_setup

    rng = np.random.default_rng(1000 + (0 if tp else rank))  # a tensor-parallel group shares ONE batch
    t0 = time.perf_counter()
    prompts = [rng.integers(0, cfg.vocab, size=PROMPT_LEN) for _ in range(BATCH)]
    first = model.prefill_many(list(range(BATCH)), prompts, chunk=args.prefill_chunk)  # rows packed across prompts
    t_prefill = time.perf_counter() - t0

    gen = gm.Generator(model, first, use_graph=True)
    stream = torch.cuda.ExternalStream(lib_stream(model), device=dev)
    for _ in range(args.warmup):
        gen.step(read_back=False)
    gen.sync()

    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid)
    # ---- device-resident timed region ---------------------------------------------------------
    launches0 = model.stats()["kernel_launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    e0.record(stream)
    for _ in range(args.steps):
        gen.step(read_back=False)
    e1.record(stream)
    gen.sync()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = model.stats()["kernel_launches"] - launches0
    ctx_mid = PROMPT_LEN + args.warmup + args.steps // 2

    # ---- end-to-end timed region: host token ids in, sampled ids out, every step ----------------
    cur = gen.step()  # brings the current ids to the host
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cur = gen.step(tokens_in=cur)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop()

    t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    tokens = (1 if tp else world) * BATCH * args.steps
    value = tokens / (ms * 1e-3)
    e2e_value = tokens / (e2e_ms * 1e-3)

    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if tp else "weak",
        "vs_baseline": None, "dtype": f"bf16 activations x {'int8' if w8 else 'int4'} weights, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD.replace("W4A16-g128", "W8A16 per-channel") if w8 else WORKLOAD, "parallelism": (f"tp{world} (one batch of 64; all-reduce of [64,3072] f32 after o_proj and down_proj: {model.tp_allreduce_kind()})" if tp
                                   else f"dp{world} (request-partitioned, no collective)"),
                   "context_tokens_during_timing": [PROMPT_LEN + args.warmup, PROMPT_LEN + args.warmup + args.steps],
                   "l2": "inputs larger than L2 (1.8 GB weights + >14 GB KV streamed per step)",
                   "cuda_graph": True, "pdl": bool(args.pdl), "lm_head": "W8A16" if w8 else "W4A16", "kv_cache": "paged bf16, 16-token pages",
                   "prefill_seconds": round(t_prefill, 2), "weight_setup_seconds": round(t_weights, 2)},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": BATCH * 4, "d2h_bytes_per_step": BATCH * 4,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }

    if rank == 0:
        peak, peak_kind = _peaks()
        # whole-step roofline: weight + KV bytes per step
        w_bytes = model_weight_bytes(cfg, w8)
        kv_bytes = cfg.n_layers * BATCH * ctx_mid * 4096
        step_bytes = (w_bytes + kv_bytes) // (world if tp else 1)  # per GPU
        line["step_roofline"] = {"bytes_per_step_per_gpu": step_bytes, "achieved_gbs": step_bytes / (ms / args.steps * 1e-3) / 1e9,
                                 "peak_gbs": peak, "frac": step_bytes / (ms / args.steps * 1e-3) / 1e9 / peak,
                                 "peak_kind": peak_kind}
    if rank == 0 and not args.no_extras:
        peak, peak_kind = _peaks()
        del gen
        a_ms, a_bytes, chunk = time_attention_kernel(ops, torch, dev, ctx_mid)
        ach = a_bytes / (a_ms * 1e-3) / 1e9
        cap = ncu_traffic("paged_attention_kernel")
        line["roofline"] = {"kernel": "paged_attention_kernel", "bound": "hbm", "achieved": ach, "peak": peak,
                            "unit": "GB/s", "frac": ach / peak, "traffic": int(cap["bytes"] * ctx_mid / cap["ctx"]) if cap else None,
                            "traffic_source": (f"dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture at context {cap['ctx']} "
                                               f"({cap['source']}), scaled by the tokens of this launch") if cap else None,
                            "peak_kind": f"{peak_kind} copy bandwidth", "us_per_launch": a_ms * 1e3,
                            "algorithmic_bytes_per_launch": a_bytes, "chunk_pages": chunk,
                            "units": f"{BATCH} sequences x {ctx_mid} tokens x 4096 B KV (one layer)"}
        g_us, g_bytes = time_gemv(ops, torch, dev)
        line["gemv_w4a16"] = {"shape": "M=1 N=9216 K=3072", "us_per_launch": g_us, "achieved_gbs": g_bytes / (g_us * 1e-6) / 1e9,
                              "frac_of_peak": g_bytes / (g_us * 1e-6) / 1e9 / peak, "frac_of_nominal_8tbs": g_bytes / (g_us * 1e-6) / 8e12,
                              "note": "64 distinct weight matrices in rotation (0.94 GB working set), back-to-back launches in one CUDA graph with programmatic dependent launch edges, as in the engine's recorded step"}
        g_us, g_bytes = time_gemv(ops, torch, dev, n=131072, k=3072, n_mats=4, iters=3)
        line["gemv_w4a16_lm_head"] = {"shape": "M=1 N=131072 K=3072", "us_per_launch": g_us,
                                      "achieved_gbs": g_bytes / (g_us * 1e-6) / 1e9, "frac_of_peak": g_bytes / (g_us * 1e-6) / 1e9 / peak}
    if not args.no_extras and not tp:
        # sub-records: measured after the headline figures, in the same process group
        subs = set(args.sub.split(","))
        if world > 1 and "tp" in subs:
            try:
                line["tp"] = measure_tp(args, gm, torch, np, dist, world, rank, dev, model, cfg)
            except Exception as e:  # noqa: BLE001  (every rank runs the same shapes, so a refusal is raised on all of them alike)
                line["tp"] = {"parallelism": f"tp{world}", "error": f"{type(e).__name__}: {e}"[:400]}
        model.close()
        del model
        torch.cuda.empty_cache()
        sub = argparse.Namespace(**vars(args))
        sub.warmup = 3
        if "dp512" in subs:
            line["dp512"] = strip_sub(measure_dp512(sub, gm, torch, np, dist, world, rank, dev))
        if rank == 0 and world == 1 and "gpt2" in subs:
            g2 = argparse.Namespace(**vars(args))
            g2.steps, g2.warmup = 64, 4
            line["gpt2_fp32"] = strip_sub(measure_gpt2(g2, gm, torch, np, cpu_baseline=not args.no_cpu_baseline, device_index=local))
            rp = measure_gpt2_run_program(g2, torch, np)
            line["gpt2_fp32"]["run_program_path"] = {k: rp[k] for k in ("value", "ms_per_step", "launches_per_token", "fused_rewrites",
                                                                        "driver_allocs_in_timed_region", "graph_replays_in_timed_region")}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import cbaseline as cb
        # the CPU arm forks one process per host core: run it as its own interpreter, apart from this CUDA process
        res = None
        try:
            r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "8", "--warmup", "3"],
                               capture_output=True, text=True, timeout=600, env={**os.environ, "RANK": "0", "WORLD_SIZE": "1"})
            ref = json.loads([ln for ln in r.stdout.splitlines() if ln.strip()][-1])["cpu_baseline"]
            res = {"tokens_per_s": ref["value"], "cores": ref["cores"], "kind": ref["kind"], "sample": ref["sample"]}
        except Exception as e:  # noqa: BLE001  (fall back to the single-process sample)
            print(f"cpu_baseline: parallel run failed ({e}); timing one process", file=sys.stderr)
        if res is None:
            res = cb.time_ministral_step_sample(cb.load(prefer_reference=True), batch=BATCH, ctx_len=PROMPT_LEN)
        line["cpu_baseline"] = {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": res["kind"],
                                "sample": res["sample"], "host_cores_available": os.cpu_count()}
    if rank == 0:
        print(json.dumps(line), file=out)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def ncu_traffic(kernel: str):
    """DRAM traffic per launch of a kernel as one committed ncu capture recorded it: reads the summary under profiles/
    (the lines `dram__bytes_read.sum` / `dram__bytes_write.sum` of its first captured launch and the context length in
    its file name). Returns {"bytes", "ctx", "source"} or None when the summary is missing."""
    import re
    for path in sorted((ROOT / "profiles").glob(f"{kernel}_*ctx*.md")):
        text = path.read_text()
        m_ctx = re.search(r"ctx(\d+)", path.name)
        rd = re.search(r"dram__bytes_read\.sum\s*\|\s*([0-9.]+)\s*\|\s*(\w+)", text)
        wr = re.search(r"dram__bytes_write\.sum\s*\|\s*([0-9.]+)\s*\|\s*(\w+)", text)
        if not (m_ctx and rd and wr):
            continue
        unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
        total = float(rd.group(1)) * unit.get(rd.group(2), 1.0) + float(wr.group(1)) * unit.get(wr.group(2), 1.0)
        return {"bytes": total, "ctx": int(m_ctx.group(1)), "source": f"profiles/{path.name}"}
    return None


def strip_sub(rec: dict) -> dict:
    """A sub-record keeps its figures and drops what only a top-level line needs."""
    return {k: v for k, v in rec.items() if k not in ("n_gpus", "higher_is_better", "vs_baseline", "data", "warmup")}


def lib_stream(model):
    from gptrs_b200 import lib
    return lib().gptrs_cuda_model_stream(model._h)


def model_weight_bytes(cfg, w8: bool = False) -> int:
    d, qkv, qd, mlp = cfg.d_model, (cfg.n_q_heads + 2 * cfg.n_kv_heads) * cfg.head_dim, cfg.n_q_heads * cfg.head_dim, cfg.d_mlp
    per_layer = d * qkv + qd * d + 2 * d * mlp + mlp * d
    elems = cfg.n_layers * per_layer + d * cfg.vocab
    if w8:  # int8 + one fp16 scale per output channel
        return elems + 2 * (cfg.n_layers * (qkv + d + 2 * mlp + d) + cfg.vocab)
    return elems // 2 + elems // 128 * 2


if __name__ == "__main__":
    main()
