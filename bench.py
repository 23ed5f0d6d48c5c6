"""Benchmark of the muGraph executor's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (BASELINE config "GQA incremental decode", fp16): batch 1, 32 query heads, 8 KV
heads (group 4), head_dim 128, KV length 4096; the muGraph is two customized operators (split-KV
partials over 16 blocks with a for-loop over KV tiles of 64, then the cross-block reduction and
division).  One STEP = `calls_per_step` evaluations of that muGraph, each on a different resident
K/V/Q buffer set so that no call finds its inputs in L2 (the sets together exceed 2x the L2 size);
the step is replayed from a CUDA graph.  `value` = microseconds per call (whole muGraph, both
operators).  With N GPUs the 8 KV heads are sharded N ways (strong scaling, no collective on the
data path).

Also measured in the same run and reported as extra keys:
  roofline            the split-KV kernel alone: algorithmic bytes (Q+K+V read once) / event time
  fingerprint         the verification sweep: the same muGraph evaluated in fingerprint mode on
                      independent seeded input sets, sharded over ranks, result fingerprints
                      all-gathered over NCCL; evals/s over all ranks
  e2e                 the same call through the public API with host buffers: pinned H2D of Q,K,V,
                      both operators, D2H of the output, per call
  cpu_baseline        the fp32 host evaluator of the same muGraph (oracle/f32_oracle.c) on this box
All inputs are synthetic (seeded), shaped and distributed as the configuration names them.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# ---- workload constants (BASELINE configs 2 and 5) ----------------------------------------------
KV_HEADS, GROUP, HEAD_DIM, KV_LEN, SPLITS, FORLOOP = 8, 4, 128, 4096, 16, 4
L2_BYTES = 126 * 1024 * 1024
SWEEP_SETS = 4096


def per_call_bytes(heads):
    q = heads * GROUP * HEAD_DIM * 2
    kv = heads * HEAD_DIM * KV_LEN * 2
    return q, kv, kv, q  # Q, K, V, O


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured (MEASURED_PEAKS.json)"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback (6.65 TB/s)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# =================================================================================================
# our arm
# =================================================================================================
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import attention_superoptimizer_b200 as mg
    from oracle import fp_oracle, mugraph_oracle as mo

    rank, local_rank, world = dist_env()
    if args.streams <= 0:
        args.streams = 8 if world == 1 else (16 if world == 2 else 32)
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert KV_HEADS % world == 0, "KV heads shard evenly over 1, 2, 4 or 8 GPUs"
    heads = KV_HEADS // world

    qb, kb, vb, ob = per_call_bytes(heads)
    set_bytes = qb + kb + vb
    nsets = max(16, -(-(5 * L2_BYTES // 2) // set_bytes))          # > 2.5x L2 of distinct inputs
    calls = args.calls_per_step if args.calls_per_step > 0 else max(nsets, 64)
    arena = nsets * (2 * set_bytes + (1 << 20)) + (1 << 28) + (3 << 29)   # + room for the other configs' graphs
    rt = mg.Runtime.get(device=local_rank, arena_bytes=arena)
    rt.set_specialisation(0 if args.interpreter_only else args.specialisation)
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream

    # ---- decode graphs: one per resident buffer set ---------------------------------------------
    plan1, plan2 = mg.gqa_decode_plans(heads, GROUP, HEAD_DIM, KV_LEN, SPLITS, FORLOOP)
    k_layout = mg.DmemColumnMajor if args.k_layout == "col" else mg.DmemRowMajor
    v_layout = mg.DmemColumnMajor if args.v_layout == "col" else mg.DmemRowMajor
    graphs = []
    for s in range(nsets):
        g = mg.PyGraph(rt)
        Q = g.new_input((heads, GROUP, HEAD_DIM), mg.float16)
        K = g.new_input((heads, HEAD_DIM, KV_LEN), mg.float16, k_layout)
        V = g.new_input((heads, KV_LEN, HEAD_DIM), mg.float16, v_layout)
        parts = g.customized([Q, K, V], plan1)
        out = g.customized(parts, plan2)
        seed = 2024 + 1000 * rank + s
        Q.fill_data_seeded(3 * seed, HEAD_DIM ** -0.5)   # 1/sqrt(d) folded into Q
        K.fill_data_seeded(3 * seed + 1, 1.0)
        V.fill_data_seeded(3 * seed + 2, 1.0)
        graphs.append((g, (Q, K, V), out[0]))
    info = graphs[0][0].customized_info(3)
    info2 = graphs[0][0].customized_info(4)

    # one un-captured pass (sets function attributes), then capture
    for g, _, _ in graphs:
        g.run(stream=sh, sync=False)
    torch.cuda.synchronize()

    # Independent calls (different buffer sets) may be put on several streams inside the captured step so that
    # more than one call is in flight; --streams 1 keeps strict stream order (each call after the previous one).
    lanes = [stream] + [torch.cuda.Stream() for _ in range(max(0, args.streams - 1))]

    def fan_out():
        if len(lanes) > 1:
            ev = torch.cuda.Event()
            ev.record(stream)
            for s in lanes[1:]:
                s.wait_event(ev)

    def fan_in():
        for s in lanes[1:]:
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)

    def record_calls():
        fan_out()
        for c in range(calls):
            graphs[c % nsets][0].run(stream=lanes[c % len(lanes)].cuda_stream, sync=False)
        fan_in()

    def record_op1():
        fan_out()
        for c in range(calls):
            graphs[c % nsets][0].run_op(3, stream=lanes[c % len(lanes)].cuda_stream)
        fan_in()

    # The headline protocol keeps `--streams` independent calls in flight and sizes launches for throughput;
    # the stream-ordered protocol (one stream, each call after the previous one, launches sized for latency) is
    # captured first and reported beside it.
    all_lanes, lanes = lanes, [stream]
    rt.set_launch_policy(mg.POLICY_LATENCY)
    ordered_graph = mg.CapturedSequence(sh, record_calls)
    lanes = all_lanes
    rt.set_launch_policy(mg.POLICY_THROUGHPUT if args.streams > 1 else mg.POLICY_LATENCY)
    step_graph = mg.CapturedSequence(sh, record_calls)
    op1_graph = mg.CapturedSequence(sh, record_op1)
    rt.set_launch_policy(mg.POLICY_LATENCY)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        """`warmup` untimed then exactly `steps` timed calls of fn; CUDA events on the launching stream;
        returns the max over ranks of the elapsed milliseconds."""
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = mg.launch_count()
    total_ms = timed(step_graph.launch, args.steps, args.warmup)
    # nvidia-smi samples every 100 ms and the timed region can be shorter: keep replaying the same step
    # (untimed) for about a second so that the sampler sees the clocks under this load
    t_end = time.perf_counter() + 1.0
    while time.perf_counter() < t_end:
        for _ in range(20):
            step_graph.launch()
        stream.synchronize()
    clocks = sampler.stop() if rank == 0 else {}
    ms_per_step = total_ms / args.steps
    us_per_call = ms_per_step * 1000.0 / calls
    gpu_launches = args.steps * step_graph.kernels

    # ---- dominant kernel alone: roofline ----------------------------------------------------------
    ordered_us = timed(ordered_graph.launch, max(3, args.steps // 2), 3) / max(3, args.steps // 2) * 1000.0 / calls
    op1_ms = timed(op1_graph.launch, max(3, args.steps // 2), 3) / max(3, args.steps // 2)
    # Single call, not captured: events around one evaluation of the muGraph (a different buffer set each time),
    # median of 200; and the reference's own protocol (KNCustomizedOp::profile: 1024 untimed + 1024 timed launches
    # of op1 on the same buffers, so K and V stay in L2).
    singles = []
    for c in range(0 if args.no_latency_probes else 210):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graphs[c % nsets][0].run(stream=sh, sync=False)
        e1.record(stream)
        stream.synchronize()
        if c >= 10:
            singles.append(e0.elapsed_time(e1) * 1000.0)
    single_us = statistics.median(singles) if singles else float("nan")
    l2_resident_us = float("nan") if args.no_latency_probes else graphs[0][0].profile_op(3) * 1000.0
    op1_us = op1_ms * 1000.0 / calls
    peaks, peak_src = load_peaks()
    op1_bytes = qb + kb + vb
    achieved = op1_bytes / (op1_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "kernel": "split-KV attention operator (op1)", "achieved": round(achieved, 1),
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                "peak_source": peak_src,
                "traffic": 16853248 if world == 1 else None,
                "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture "
                                  "profiles/attn_split_fp16_gqa_decode.md (same shapes, N = 1)",
                "bytes_per_launch": op1_bytes,
                "us_per_launch": round(op1_us, 3)}

    # ---- end to end through the public API with host buffers -----------------------------------------
    g0, (Q0, K0, V0), O0 = graphs[0]
    host_in = [torch.empty(t.num_elements, dtype=torch.float16).pin_memory() for t in (Q0, K0, V0)]
    host_out = torch.empty(O0.num_elements, dtype=torch.float16).pin_memory()
    for h, t in zip(host_in, (Q0, K0, V0)):
        h.copy_(torch.from_numpy(t.download_data().view(np.float16)))
    lib, rth = rt.lib, rt.handle
    import ctypes

    def e2e_call():
        for h, t in zip(host_in, (Q0, K0, V0)):
            mg.check(lib.mg_tensor_upload_data_async(rth, ctypes.byref(t.pod), h.data_ptr(), sh))
        g0.run(stream=sh, sync=False)
        mg.check(lib.mg_tensor_download_data_async(rth, ctypes.byref(O0.pod), host_out.data_ptr(), sh))
        stream.synchronize()   # the caller reads the result

    e2e_calls = max(5, min(50, args.steps))
    e2e_ms = timed(e2e_call, e2e_calls, 3) / e2e_calls
    e2e = {"value": round(e2e_ms * 1000.0, 2), "unit": "us/call", "h2d_bytes_per_step": qb + kb + vb,
           "d2h_bytes_per_step": ob, "note": "one call per e2e step: pinned H2D of Q,K,V + both operators + D2H of O"}

    # ---- fingerprint verification sweep ----------------------------------------------------------------
    fingerprint = run_fingerprint_sweep(args, mg, mo, fp_oracle, rt, torch, dist, np, rank, world, stream, timed)
    others = None
    if world == 1 and not args.no_other_configs:
        others = measure_other_configs(mg, rt, stream, timed, load_peaks()[0])

    # ---- CPU baseline (rank 0, N = 1 only) ----------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_float_baseline(mo, fp_oracle, np, budget_s=12.0)

    if rank == 0:
        line = {
            "metric": "gqa_decode_customized_op_us_per_call", "value": round(us_per_call, 3), "unit": "us/call",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp16",
            "data": "synthetic (seeded N(0,1) K/V, Q pre-scaled by 1/sqrt(d); fingerprints uniform in [0,227))",
            "config": {"workload": "GQA incremental decode muGraph (BASELINE config 2): batch 1, 32 q heads, 8 kv heads, "
                                   "head_dim 128, kv_len 4096, 16 KV splits x for-loop 4 (tiles of 64), 2 customized ops",
                       "kv_heads_per_gpu": heads, "calls_per_step": calls, "resident_buffer_sets": nsets,
                       "l2_defeat": "each call reads a different buffer set; sets total %.0f MB > 2x L2" % (nsets * set_bytes / 1e6),
                       "replay": "CUDA graph of calls_per_step muGraph evaluations; the calls of a step are independent "
                                 "(distinct buffer sets) and spread over %d streams, launches sized for throughput" % args.streams,
                       "streams": args.streams,
                       "kernel_op1": info["kernel_float"], "kernel_op2": info2["kernel_float"],
                       "k_layout": args.k_layout, "v_layout": args.v_layout,
                       "parallelism": "kv-heads sharded x%d, no collective" % world},
            "hbm_gbs": round(sum(per_call_bytes(heads)) / (us_per_call * 1e-6) / 1e9, 1),
            "stream_ordered_us_per_call": round(ordered_us, 3),
            "single_call_us_median": None if args.no_latency_probes else round(single_us, 3),
            "l2_resident_profile_us": None if args.no_latency_probes else round(l2_resident_us, 3),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(gpu_launches),
            "clocks": clocks, "fingerprint": fingerprint, "other_configs": others,
        }
        print(json.dumps(line))
    step_graph.close()
    op1_graph.close()
    ordered_graph.close()
    for g, _, _ in reversed(graphs):
        g.close()
    if world > 1:
        dist.destroy_process_group()


def run_fingerprint_sweep(args, mg, mo, fp_oracle, rt, torch, dist, np, rank, world, stream, timed):
    """BASELINE config 5: the decode muGraph in fingerprint mode over independent seeded input sets
    (uniform in [0, 227)), sets sharded over ranks, processed in resident chunks; result fingerprints
    all-gathered.  A few sets are checked bit-exactly against the CPU oracle."""
    import ctypes
    sh = stream.cuda_stream
    total_sets = args.sweep_sets
    my_sets = total_sets // world
    chunk = min(args.sweep_chunk, my_sets)
    nchunks = my_sets // chunk
    B, M, D, L = KV_HEADS, GROUP, HEAD_DIM, KV_LEN
    with mg.PyGraph(rt) as g:
        Q = g.new_input((B, M, D))
        K = g.new_input((B, D, L), layout=mg.DmemColumnMajor)
        V = g.new_input((B, L, D), layout=mg.DmemColumnMajor)
        p1, p2 = mg.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
        parts = g.customized([Q, K, V], p1)
        out = g.customized(parts, p2)
        elems = [t.num_elements for t in (Q, K, V)]
        # All input sets of this rank stay resident when they fit (4096 sets = 69 GB on one GPU): the evaluation
        # launches then go out back to back and the device time has no host gaps in it.  Otherwise one chunk is
        # resident at a time and refilled (outside the timed regions) between evaluations.
        free_bytes, _ = torch.cuda.mem_get_info()
        resident = my_sets * 2 * sum(elems) < 0.7 * free_bytes
        held = my_sets if resident else chunk
        bufs = [torch.empty(held * n, dtype=torch.int16, device="cuda") for n in elems]
        result = torch.zeros(my_sets * out[0].num_elements, dtype=torch.int16, device="cuda")
        wbytes = g.fingerprint_batched_workspace(chunk)
        work = torch.empty(max(wbytes, 256), dtype=torch.uint8, device="cuda")

        def fill_chunk(c):
            # set s (global index) uses seed 2024 + s; tensor id 0,1,2 = Q,K,V
            slot0 = c * chunk if resident else 0
            for i, (buf, n) in enumerate(zip(bufs, elems)):
                for s in range(chunk):
                    gs = rank * my_sets + c * chunk + s
                    pod = mg.mg_tensor()
                    pod.data_type, pod.num_dims, pod.dim[0] = mg.float16, 1, n
                    pod.fp_ptr = buf.data_ptr() + 2 * (slot0 + s) * n
                    mg.check(rt.lib.mg_tensor_fill_fingerprint_seeded(rt.handle, ctypes.byref(pod), 3 * (2024 + gs) + i, mg.FP_P))

        def eval_chunk(c):
            slot0 = c * chunk if resident else 0
            g.fingerprint_batched(chunk, [b.data_ptr() + 2 * slot0 * n for b, n in zip(bufs, elems)],
                                  result.data_ptr() + 2 * c * chunk * out[0].num_elements, work.data_ptr(), wbytes, stream=sh)

        fill_chunk(0)
        eval_chunk(0)
        torch.cuda.synchronize()
        if resident:
            for c in range(1, nchunks):
                fill_chunk(c)
            t_eval = timed(lambda: [eval_chunk(c) for c in range(nchunks)], 1, 0)
        else:
            t_eval = 0.0
            for c in range(nchunks):
                if c > 0:
                    fill_chunk(c)
                t_eval += timed(lambda: eval_chunk(c), 1, 0)
        # all-gather of the result fingerprints (8 KB per set) for dedup / comparison on every rank
        gathered = result
        t_gather = 0.0
        if world > 1:
            from attention_superoptimizer_b200 import sharding
            local = result.view(my_sets, -1)
            gathered = torch.empty((world * my_sets, local.shape[1]), dtype=local.dtype, device=local.device)
            t_gather = timed(lambda: sharding.all_gather_fingerprints(local, world, out=gathered), 1, 2)  # 2 warm-ups
        # compare on every rank: which of all the sets has the fingerprint of set 0 (the search's verify step)
        from attention_superoptimizer_b200 import sharding as _sh
        all_rows = gathered.view(-1, out[0].num_elements)
        box = {}
        t_compare = timed(lambda: box.__setitem__("m", _sh.matches_reference_on_device(all_rows, all_rows[0])), 1, 1)
        equal_to_first = int(box["m"].sum().item())
        evals_per_s = (nchunks * chunk * world) / ((t_eval + t_gather + t_compare) * 1e-3)
        # bit-exact check of a sample against the CPU oracle
        checked, ok = 0, True
        if rank == 0:
            specs, op1, op2 = mo.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
            g1 = mo.build_customized(specs, op1)
            g2 = mo.build_customized(mo.output_specs(g1), op2)
            host = gathered.cpu().numpy().view(np.uint16).reshape(-1, out[0].num_elements)
            for gs in sorted({0, my_sets - 1, (total_sets // world) * (world - 1)}):
                x = [host_seeded(np, 3 * (2024 + gs) + i, n, mg.FP_P).reshape(s.dims) for i, (n, s) in enumerate(zip(elems, specs))]
                o1, _ = fp_oracle.run(g1, x)
                o2, _ = fp_oracle.run(g2, o1)
                ok = ok and gs < host.shape[0] and np.array_equal(host[gs], o2[0].ravel())
                checked += 1
        info = g.customized_info(3)
    return {"metric": "fingerprint_evals_per_s", "value": round(evals_per_s, 1), "unit": "evals/s",
            "sets": nchunks * chunk * world, "sets_per_gpu": nchunks * chunk, "chunk_sets": chunk,
            "inputs_resident": bool(resident),
            "eval_ms": round(t_eval, 3), "allgather_ms": round(t_gather, 3), "compare_ms": round(t_compare, 3),
            "sets_equal_to_first": equal_to_first,
            "bytes_per_eval": 16793600, "hbm_gbs_per_gpu": round(16793600 * nchunks * chunk / (t_eval * 1e-3) / 1e9, 1),
            "kernel_op1": info["kernel_fingerprint"], "oracle_checked_sets": checked, "bit_exact": bool(ok)}


def run_one_config(args):
    """`--only-config`: one of the other BASELINE configs alone (profiling, tuning); prints {"other_configs": {...}}."""
    import torch
    import attention_superoptimizer_b200 as mg

    torch.cuda.set_device(0)
    rt = mg.Runtime.get(device=0, arena_bytes=3 << 30)
    rt.set_specialisation(0 if args.interpreter_only else args.specialisation)
    stream = torch.cuda.Stream()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    out = measure_other_configs(mg, rt, stream, timed, load_peaks()[0], only=args.only_config)
    print(json.dumps({"other_configs": out}))


def measure_other_configs(mg, rt, stream, timed, peaks, only=None):
    """Device-timed numbers for the remaining BASELINE configs (N = 1 only), each replayed from a CUDA graph:
    config 3 (speculative decode with the causal draft window, fp16), config 4 (dense prefill, bf16, tcgen05)
    and config 1 (matmul chain, both modes on the generic interpreters).  `only` = "c1" | "c3" | "c4" runs one."""
    sh = stream.cuda_stream
    out = {}

    def replay_us(graphs, reps):
        for g in graphs:
            g.run(stream=sh, sync=False)
        stream.synchronize()
        seq = mg.CapturedSequence(sh, lambda: [graphs[i % len(graphs)].run(stream=sh, sync=False) for i in range(reps)])
        # the clocks of an idle GPU take a while to come up: replay untimed for 0.3 s, then time 20 replays
        t_end = time.perf_counter() + 0.3
        while time.perf_counter() < t_end:
            for _ in range(10):
                seq.launch()
            stream.synchronize()
        ms = timed(seq.launch, 20, 3) / 20
        seq.close()
        return ms * 1000.0 / reps

    # ---- config 3: batch 4 x 8 KV heads = 32 units, 8 draft tokens x group 4 = 32 rows, KV 8192 -------------
    def config3():
        units, rows, d, kv, splits, fr, window = 32, 32, 128, 8192, 16, 8, 8
        graphs = []
        for s in range(2):  # two buffer sets of 135 MB each: consecutive calls never share L2 contents
            g = mg.PyGraph(rt)
            Q = g.new_input((units, rows, d)); K = g.new_input((units, d, kv), layout=mg.DmemColumnMajor)
            V = g.new_input((units, kv, d), layout=mg.DmemRowMajor)
            p1, p2 = mg.gqa_decode_plans(units, rows, d, kv, splits, fr)
            parts = g.customized([Q, K, V], p1); g.customized(parts, p2)
            g.set_causal_window(3, window)
            Q.fill_data_seeded(900 + s, d ** -0.5); K.fill_data_seeded(910 + s, 1.0); V.fill_data_seeded(920 + s, 1.0)
            graphs.append(g)
        us = replay_us(graphs, 8)
        nbytes = 2 * units * rows * d * 2 + 2 * units * d * kv * 2
        out["spec_decode_c3"] = {"us_per_call": round(us, 2), "hbm_gbs": round(nbytes / us / 1e3, 1),
                                 "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4), "bytes": nbytes,
                                 "kernel": graphs[0].customized_info(3)["kernel_float"], "dtype": "fp16",
                                 "note": "32 rows x KV 8192, 16 splits x for-loop 8, causal draft window 8, fused merge"}
        for g in reversed(graphs):
            g.close()

    # ---- config 4: 32 heads, 2048 x 2048, head_dim 128, bf16 ----------------------------------------------------
    def config4():
        d = 128
        H, SQ, L = 32, 2048, 2048
        g = mg.PyGraph(rt)
        Q = g.new_input((H, SQ, d), mg.bfloat16); K = g.new_input((H, d, L), mg.bfloat16, mg.DmemColumnMajor)
        V = g.new_input((H, L, d), mg.bfloat16, mg.DmemColumnMajor)
        p1, p2 = mg.attention_prefill_plans(H, SQ, d, L)
        acc = g.customized([Q, K, V], p1); g.customized(acc, p2)
        Q.fill_data_seeded(930, d ** -0.5); K.fill_data_seeded(931, 1.0); V.fill_data_seeded(932, 1.0)
        us = replay_us([g], 10)
        flops = 4.0 * H * SQ * L * d
        out["prefill_c4"] = {"us_per_call": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                             "frac_of_bf16_peak": round(flops / us / 1e6 / peaks["bf16_tflops"], 4), "flops": flops,
                             "kernel": g.customized_info(3)["kernel_float"], "dtype": "bf16",
                             "note": "both customized ops in one launch (division fused into the tcgen05 kernel's epilogue)"}
        g.close()

    # ---- config 1: X[16,1024] W1[1024,1024] W2[1024,1024], fingerprint mode, generic interpreter -------------------
    def config1():
        g = mg.PyGraph(rt)
        X = g.new_input((16, 1024)); W1 = g.new_input((1024, 1024)); W2 = g.new_input((1024, 1024))
        chain = mg.ExecutionPlan(ops=[(mg.TB_MATMUL_OP, [(0, 0), (1, 0)]), (mg.TB_MATMUL_OP, [(3, 0), (2, 0)])],
                                 input_map=[(-1, -1, -1), (1, -1, -1), (0, -1, -1)], forloop_dim=[1, 0, -1],
                                 input_smem_layouts=[mg.SmemRowMajor] * 3, output_map=(1, -1, -1), forloop_range=16,
                                 grid_dim=(16, 1, 1), reduction_dimx=1024)
        part = g.customized([X, W1, W2], chain)
        reduce_plan = mg.ExecutionPlan(ops=[(mg.TB_REDUCTION_1_TO_DIMX_OP, [(0, 0)])], input_map=[(0, -1, -1)],
                                       forloop_dim=[-1], input_smem_layouts=[mg.SmemRowMajor], output_map=(0, -1, -1),
                                       forloop_range=1, grid_dim=(16, 1, 1), reduction_dimx=1024)
        g.customized(part, reduce_plan)
        for t, sd in ((X, 940), (W1, 941), (W2, 942)):
            t.fill_fingerprint_seeded(sd, mg.FP_P)
        g.fingerprint()
        import time as _t
        t0 = _t.perf_counter()
        for _ in range(20):
            g.fingerprint()
        fp_us = (_t.perf_counter() - t0) / 20 * 1e6
        X.fill_data_seeded(943, 1.0); W1.fill_data_seeded(944, 1.0 / 32); W2.fill_data_seeded(945, 1.0 / 32)
        float_us = replay_us([g], 10)
        out["matmul_chain_c1"] = {"float_us_per_call": round(float_us, 1), "fingerprint_us_per_call": round(fp_us, 1),
                                  "kernel": g.customized_info(3)["kernel_fingerprint"], "dtype": "fp16",
                                  "bytes": 4259840, "flops": 67108864,
                                  "note": "two customized ops (16 blocks over the intermediate columns, for-loop 16 over K "
                                          "tiles of 64; then the cross-block reduction), generic interpreters; float: CUDA "
                                          "graph replay; fingerprint: host-synchronised calls"}
        g.close()

    for name, fn in (("c3", config3), ("c4", config4), ("c1", config1)):
        if only in (None, name):
            fn()
    return out


def host_seeded(np, seed, n, modulus):
    """Host twin of mg_rng_uniform (include/mugraph_rng.h): splitmix64 finaliser over (seed, index)."""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64)
        z = np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + idx * np.uint64(0xD1B54A32D192ED03) + np.uint64(0x632BE59BD9B4E019)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(32)) % np.uint64(modulus)).astype(np.uint16)


def cpu_float_baseline(mo, fp_oracle, np, budget_s, threads=0):
    """Times the fp32 host evaluator (oracle/f32_oracle.c, OpenMP) on whole C2 calls for about
    `budget_s` seconds.  Returns the cpu_baseline object."""
    B, M, D, L = KV_HEADS, GROUP, HEAD_DIM, KV_LEN
    rng = np.random.default_rng(2024)
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
    g1 = mo.build_customized(specs, p1)
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    q = (rng.standard_normal((B, M, D)) / np.sqrt(D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, L, D)).astype(np.float16).astype(np.float32)   # memory image, column-major
    v = rng.standard_normal((B, D, L)).astype(np.float16).astype(np.float32)
    used = 1
    fp_oracle.run_float(g1, [q, k, v], threads)  # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        o1, used = fp_oracle.run_float(g1, [q, k, v], threads)
        fp_oracle.run_float(g2, o1, threads)
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50000:
            break
    dt = time.perf_counter() - t0
    return {"value": round(dt / n * 1e6, 1), "unit": "us/call", "cores": int(used), "kind": "port",
            "sample": "%d whole C2 muGraph calls (both operators) by the fp32 host evaluator oracle/f32_oracle.c in %.1f s" % (n, dt)}


# =================================================================================================
# reference arm: the CPU implementation of the same path, on the box's host cores
# =================================================================================================
def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    import numpy as np
    from oracle import fp_oracle, mugraph_oracle as mo
    # each step = one bounded sample: `calls` whole C2 muGraph evaluations by the fp32 host evaluator
    B, M, D, L = KV_HEADS, GROUP, HEAD_DIM, KV_LEN
    rng = np.random.default_rng(2024)
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
    g1 = mo.build_customized(specs, p1)
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    q = (rng.standard_normal((B, M, D)) / np.sqrt(D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, L, D)).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((B, D, L)).astype(np.float16).astype(np.float32)
    calls = 4
    used = 1

    def step():
        nonlocal used
        for _ in range(calls):
            o1, used = fp_oracle.run_float(g1, [q, k, v], 0)
            fp_oracle.run_float(g2, o1, 0)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    us = dt / (args.steps * calls) * 1e6
    sample = "%d steps x %d whole C2 muGraph calls, fp32 host evaluator (oracle/f32_oracle.c, OpenMP)" % (args.steps, calls)
    line = {"impl": "reference", "metric": "gqa_decode_customized_op_us_per_call", "value": round(us, 1), "unit": "us/call",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
            "data": "synthetic (seeded)",
            "config": {"workload": "GQA incremental decode muGraph (BASELINE config 2), CPU evaluation",
                       "calls_per_step": calls,
                       "note": "the reference has no CPU evaluation path and its GPU float interpreter does not compute "
                               "correct values; this arm times the fp32 host evaluator of the same graph semantics"},
            "cpu_baseline": {"value": round(us, 1), "unit": "us/call", "cores": int(used), "kind": "port", "sample": sample},
            "e2e": {"value": round(us, 1), "unit": "us/call", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--calls-per-step", type=int, default=0, help="muGraph evaluations per step (0 = auto)")
    ap.add_argument("--sweep-sets", type=int, default=SWEEP_SETS, help="input sets of the fingerprint sweep (all ranks)")
    ap.add_argument("--sweep-chunk", type=int, default=128, help="sets resident per chunk and rank")
    ap.add_argument("--k-layout", default="col", choices=["row", "col"],
                    help="DmemLayout of K[heads, d, kv]: col = memory [kv][d] (KV-cache order), row = memory [d][kv]")
    ap.add_argument("--v-layout", default="row", choices=["row", "col"],
                    help="DmemLayout of V[heads, kv, d]: row = memory [kv][d] (KV-cache order), col = memory [d][kv]")
    ap.add_argument("--streams", type=int, default=0,
                    help="streams the independent calls of a step are spread over (0 = 8 per rank at N = 1, 16 at N = 2, "
                         "32 from N = 4: the fewer KV heads a rank holds, the more calls fit on the GPU at once)")
    ap.add_argument("--interpreter-only", action="store_true", help="disable the specialised kernels")
    ap.add_argument("--specialisation", type=int, default=2, choices=[0, 1, 2],
                    help="0 = interpreters, 1 = specialised kernels without operator fusion, 2 = with fusion (default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the extra measurements of configs 1, 3 and 4")
    ap.add_argument("--no-latency-probes", action="store_true",
                    help="skip the single-call latency and the 1024 + 1024 launch L2-resident measurement (short launch lists)")
    ap.add_argument("--only-config", default=None, choices=["c1", "c3", "c4"],
                    help="measure just this other config on one GPU and print its entry (no headline line)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.only_config:
        run_one_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
