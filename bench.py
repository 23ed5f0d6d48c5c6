"""Benchmark of the muGraph executor's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (GQA incremental decode, fp16): batch 1, 32 query heads, 8 KV heads (group 4), head_dim 128,
KV length 4096; the muGraph is two customized operators (split-KV partials over 16 blocks with a for-loop over KV
tiles of 64, then the cross-block reduction and division).  A CALL is one evaluation of that muGraph on one
Q/K/V set.  One STEP = `calls_per_step` independent calls, each on its own resident Q/K/V set, issued as batched
launches (`--batch` calls per kernel: split-KV and merge of all the batch's calls in ONE launch) that run back to
back on one stream; the sets a step reads exceed 2.5x the L2 size, so no call finds its inputs there.  `value` =
microseconds per call.  With N GPUs the 8 KV heads are sharded N ways (strong scaling, no collective on the data
path).

Reported beside it:
  roofline            the batched kernel: algorithmic bytes per launch (Q + K + V read once, O written) / mean launch
                      duration inside the timed region / measured HBM peak
  per_call_launch     one kernel launch per call: `calls` launches spread over several streams (throughput sizing),
                      strictly one after the other on one stream (latency sizing), one un-captured call, and the
                      reference's own profile protocol (same buffers, K/V stay in L2)
  fingerprint         the verification sweep: the same muGraph in fingerprint mode on 4096 seeded input sets,
                      sharded over ranks, fingerprints all-gathered (NCCL) and compared row by row on the device
                      with reference fingerprints; every row is also checked against digests of the reference's
                      own host code
  e2e                 one call through the public API with host buffers: pinned H2D of Q,K,V, the muGraph, D2H of O
  cpu_baseline        CPU evaluation of the same work on this box (float: fp32 port; fingerprints: the reference's
                      own fingerprinter classes), one core and all cores
All inputs are synthetic (seeded), shaped and distributed as the configuration names them.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# ---- workload constants (decode muGraph and verification sweep) ------------------------------------------
KV_HEADS, GROUP, HEAD_DIM, KV_LEN, SPLITS, FORLOOP = 8, 4, 128, 4096, 16, 4
L2_BYTES = 126 * 1024 * 1024
SWEEP_SETS = 4096
SWEEP_DIGESTS = os.path.join(ROOT, "tests", "golden", "sweep_digests_gqa_decode.json")
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "attn_split_fp16_gqa_decode_batched.json")


def per_call_bytes(heads):
    q = heads * GROUP * HEAD_DIM * 2
    kv = heads * HEAD_DIM * KV_LEN * 2
    return q, kv, kv, q  # Q, K, V, O


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured (MEASURED_PEAKS.json)"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback (6.65 TB/s, 1.59 PFLOP/s)"


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
            time.sleep(0.15)  # let the first sample land before the region starts
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
    nsets = max(16, -(-(5 * L2_BYTES // 2) // set_bytes))          # per-call-launch protocols: > 2.5x L2 of inputs
    arena = nsets * (2 * set_bytes + (1 << 20)) + (1 << 28) + (3 << 29)   # + room for the other configs' graphs
    rt = mg.Runtime.get(device=local_rank, arena_bytes=arena)
    rt.set_specialisation(0 if args.interpreter_only else args.specialisation)
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    peaks, peak_src = load_peaks()

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

    plan1, plan2 = mg.gqa_decode_plans(heads, GROUP, HEAD_DIM, KV_LEN, SPLITS, FORLOOP)
    k_layout = mg.DmemColumnMajor if args.k_layout == "col" else mg.DmemRowMajor
    v_layout = mg.DmemColumnMajor if args.v_layout == "col" else mg.DmemRowMajor

    # ---- headline: batched launches over dense resident sets -------------------------------------------------
    batch = args.batch
    nbatches = max(2, -(-(5 * L2_BYTES // 2) // (batch * set_bytes)))     # distinct batches a replay walks through
    elems = [qb // 2, kb // 2, vb // 2]
    dense = [torch.empty(nbatches * batch * n, dtype=torch.int16, device="cuda") for n in elems]
    dense_out = torch.zeros(nbatches * batch * (ob // 2), dtype=torch.int16, device="cuda")
    for i, (buf, n) in enumerate(zip(dense, elems)):
        for s in range(nbatches * batch):
            mg.fill_data_seeded_raw(rt, buf.data_ptr() + 2 * s * n, n, 3 * (2024 + 1000 * rank + s) + i,
                                    HEAD_DIM ** -0.5 if i == 0 else 1.0)   # 1/sqrt(d) folded into Q
    bg = mg.PyGraph(rt)
    bQ = bg.new_input((heads, GROUP, HEAD_DIM), mg.float16)
    bK = bg.new_input((heads, HEAD_DIM, KV_LEN), mg.float16, k_layout)
    bV = bg.new_input((heads, KV_LEN, HEAD_DIM), mg.float16, v_layout)
    b_out = bg.customized(bg.customized([bQ, bK, bV], plan1), plan2)
    wbytes = bg.run_batched_workspace(batch)
    bwork = torch.empty(max(wbytes, 256), dtype=torch.uint8, device="cuda")

    def launch_batch(b, on=sh):
        bg.run_batched(batch, [d.data_ptr() + 2 * b * batch * n for d, n in zip(dense, elems)],
                       dense_out.data_ptr() + b * batch * ob, bwork.data_ptr(), wbytes, stream=on)

    for b in range(nbatches):
        launch_batch(b)
    mg.synchronize()
    before = mg.launch_count()
    batched_graph = mg.CapturedSequence(sh, lambda: [launch_batch(b) for b in range(nbatches)])
    kernels_per_replay = batched_graph.kernels
    calls_per_replay = nbatches * batch
    # a step long enough for the clock sampler to see it: about 30 ms of back-to-back launches
    replays = args.replays_per_step if args.replays_per_step > 0 else max(1, round(30e3 / (calls_per_replay * 2.9 * heads / KV_HEADS + 20)))
    calls = replays * calls_per_replay

    def step():
        for _ in range(replays):
            batched_graph.launch()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms = timed(step, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else {}
    mg.synchronize()   # reads the device status word: a bounded wait that gave up would raise here
    ms_per_step = total_ms / args.steps
    us_per_call = ms_per_step * 1000.0 / calls
    gpu_launches = args.steps * replays * kernels_per_replay
    us_per_launch = ms_per_step * 1000.0 / (replays * kernels_per_replay)
    launch_bytes = batch * (qb + kb + vb + ob)
    achieved = launch_bytes / (us_per_launch * 1e-6) / 1e9
    traffic, traffic_src = None, None
    if os.path.exists(TRAFFIC_FILE):
        with open(TRAFFIC_FILE) as f:
            t = json.load(f)
        # the capture's DRAM bytes per call, scaled to this launch (traffic grows in proportion to the calls)
        traffic = int(t["dram_bytes_per_call_per_kv_head"] * heads * batch)
        traffic_src = t["source"]
    roofline = {"bound": "hbm", "kernel": "attn_split_kernel<fp16,128> over %d calls (split-KV partials + fused merge)" % batch,
                "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peak_src,
                "traffic": traffic, "traffic_source": traffic_src,
                "bytes_per_launch": launch_bytes, "us_per_launch": round(us_per_launch, 3),
                "launches_timed": int(gpu_launches)}

    # ---- the same with the work per GPU and launch held constant (N > 1): 64 x N calls per launch, so that a GPU's
    # launch carries the 8 x 64 (KV head, call) units it carries at N = 1.  Reported beside the headline, which
    # keeps 64 calls per launch at every N (a GPU's launch shrinks with N there).
    fixed_work = None
    if world > 1:
        wb = batch * world
        wdense = [torch.empty(2 * wb * n, dtype=torch.int16, device="cuda") for n in elems]
        wout = torch.zeros(2 * wb * (ob // 2), dtype=torch.int16, device="cuda")
        for i, (buf, n) in enumerate(zip(wdense, elems)):
            for s in range(2 * wb):
                mg.fill_data_seeded_raw(rt, buf.data_ptr() + 2 * s * n, n, 3 * (90000 + 4000 * rank + s) + i,
                                        HEAD_DIM ** -0.5 if i == 0 else 1.0)
        ww = bg.run_batched_workspace(wb)
        wwork = torch.empty(max(ww, 256), dtype=torch.uint8, device="cuda")

        def launch_wide(b):
            bg.run_batched(wb, [d.data_ptr() + 2 * b * wb * n for d, n in zip(wdense, elems)],
                           wout.data_ptr() + b * wb * ob, wwork.data_ptr(), ww, stream=sh)

        for b in range(2):
            launch_wide(b)
        mg.synchronize()
        wide_graph = mg.CapturedSequence(sh, lambda: [launch_wide(b) for b in range(2)])
        wreps = max(1, round(10e3 / (2 * wb * 2.9 * heads / KV_HEADS + 20)))
        wide_ms = timed(lambda: [wide_graph.launch() for _ in range(wreps)], 5, 3) / 5
        wide_graph.close()
        mg.synchronize()
        w_launch_us = wide_ms * 1000.0 / (wreps * 2)
        fixed_work = {"calls_per_launch": wb, "us_per_call": round(wide_ms * 1000.0 / (wreps * 2 * wb), 3),
                      "us_per_launch": round(w_launch_us, 2),
                      "frac_of_hbm_peak_per_gpu": round(wb * (qb + kb + vb + ob) / (w_launch_us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
                      "note": "64 x N calls per launch: every GPU's launch keeps the size it has at N = 1"}
        del wdense, wout, wwork

    # output check of the timed protocol: a few calls of the last replay against the fp32 evaluation
    checked_calls, worst = 0, 0.0
    if rank == 0:
        from tests.helpers import assert_close, from_bits
        host_out = dense_out.cpu().numpy().view(np.uint16).reshape(nbatches * batch, heads, GROUP, HEAD_DIM)
        for s in sorted({0, batch - 1, nbatches * batch - 1}):
            q, k, v = (from_bits(d[s * n:(s + 1) * n].cpu().numpy().view(np.uint16), mg.float16) for d, n in zip(dense, elems))
            q = q.reshape(heads, GROUP, HEAD_DIM)
            k = k.reshape(heads, KV_LEN, HEAD_DIM).transpose(0, 2, 1) if args.k_layout == "col" else k.reshape(heads, HEAD_DIM, KV_LEN)
            v = v.reshape(heads, KV_LEN, HEAD_DIM) if args.v_layout == "row" else v.reshape(heads, HEAD_DIM, KV_LEN).transpose(0, 2, 1)
            worst = max(worst, assert_close(from_bits(host_out[s], mg.float16), mo.attention_fp32(q, k, v), mg.float16,
                                            "timed call %d" % s))
            checked_calls += 1

    per_call_launch, ordered_us, single_us, graphs = None, None, None, []
    call_bytes = qb + kb + vb + ob
    streams_graph = ordered_graph = None
    if not args.no_per_call_launch:
        # ---- one kernel launch per call: resident graphs, several protocols ------------------------------------------
        graphs = []
        for s in range(nsets):
            g = mg.PyGraph(rt)
            Q = g.new_input((heads, GROUP, HEAD_DIM), mg.float16)
            K = g.new_input((heads, HEAD_DIM, KV_LEN), mg.float16, k_layout)
            V = g.new_input((heads, KV_LEN, HEAD_DIM), mg.float16, v_layout)
            parts = g.customized([Q, K, V], plan1)
            out = g.customized(parts, plan2)
            seed = 5000 + 1000 * rank + s
            Q.fill_data_seeded(3 * seed, HEAD_DIM ** -0.5)
            K.fill_data_seeded(3 * seed + 1, 1.0)
            V.fill_data_seeded(3 * seed + 2, 1.0)
            graphs.append((g, (Q, K, V), out[0]))
        info = graphs[0][0].customized_info(3)
        info2 = graphs[0][0].customized_info(4)
        for g, _, _ in graphs:
            g.run(stream=sh, sync=False)
        torch.cuda.synchronize()
        pc_calls = max(nsets, 64)
        lanes = [stream] + [torch.cuda.Stream() for _ in range(max(0, args.streams - 1))]

        def record_calls(use):
            """pc_calls launches; a graph always goes to the same lane, so two launches of one graph (they share the
            graph's ticket counters and output buffers) are ordered by their stream."""
            if len(use) > 1:
                ev = torch.cuda.Event()
                ev.record(stream)
                for s in use[1:]:
                    s.wait_event(ev)
            for c in range(pc_calls):
                gi = c % nsets
                graphs[gi][0].run(stream=use[gi % len(use)].cuda_stream, sync=False)
            for s in use[1:]:
                ev = torch.cuda.Event()
                ev.record(s)
                stream.wait_event(ev)

        rt.set_launch_policy(mg.POLICY_LATENCY)
        ordered_graph = mg.CapturedSequence(sh, lambda: record_calls([stream]))
        rt.set_launch_policy(mg.POLICY_THROUGHPUT if args.streams > 1 else mg.POLICY_LATENCY)
        streams_graph = mg.CapturedSequence(sh, lambda: record_calls(lanes))
        rt.set_launch_policy(mg.POLICY_LATENCY)
        reps = 40
        ordered_us = timed(lambda: [ordered_graph.launch() for _ in range(reps)], 3, 2) / 3 / reps * 1000.0 / pc_calls
        streams_us = timed(lambda: [streams_graph.launch() for _ in range(reps)], 3, 2) / 3 / reps * 1000.0 / pc_calls
        mg.synchronize()
        singles = []
        for c in range(0 if args.no_latency_probes else 210):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graphs[c % nsets][0].run(stream=sh, sync=False)
            e1.record(stream)
            stream.synchronize()
            if c >= 10:
                singles.append(e0.elapsed_time(e1) * 1000.0)
        single_us = statistics.median(singles) if singles else None
        l2_resident_us = None if args.no_latency_probes else graphs[0][0].profile_op(3) * 1000.0
        call_bytes = qb + kb + vb + ob

        def frac_of(us):
            return None if not us else round(call_bytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)

        per_call_launch = {
            "streams_us_per_call": round(streams_us, 3), "streams": args.streams, "streams_frac_of_hbm_peak": frac_of(streams_us),
            "stream_ordered_us_per_call": round(ordered_us, 3), "stream_ordered_frac_of_hbm_peak": frac_of(ordered_us),
            "single_call_us_median": None if single_us is None else round(single_us, 3),
            "single_call_frac_of_hbm_peak": frac_of(single_us),
            "l2_resident_profile_us": None if l2_resident_us is None else round(l2_resident_us, 3),
            "calls": pc_calls, "resident_buffer_sets": nsets, "kernel_op1": info["kernel_float"], "kernel_op2": info2["kernel_float"],
            "note": "one fused kernel per call; streams: calls spread over lanes inside a captured step, blocks sized for "
                    "throughput; stream_ordered: one stream, each call after the previous one (programmatic dependent "
                    "launch), blocks sized for latency; single: events around one un-captured call, median of 200; "
                    "l2_resident: the reference's profile protocol (1024 + 1024 launches of op1 on the same buffers)"}

    # ---- end to end through the public API with host buffers -----------------------------------------
    host_in = torch.empty(sum(elems), dtype=torch.int16).pin_memory()
    host_in.copy_(torch.cat([d[:n] for d, n in zip(dense, elems)]).cpu())
    host_out_pinned = torch.empty(ob // 2, dtype=torch.int16).pin_memory()
    dev_in = torch.empty(sum(elems), dtype=torch.int16, device="cuda")
    dev_out = torch.empty(ob // 2, dtype=torch.int16, device="cuda")
    w1 = bg.run_batched_workspace(1)
    work1 = torch.empty(max(w1, 256), dtype=torch.uint8, device="cuda")
    offs = [0, elems[0], elems[0] + elems[1]]

    def e2e_call():
        with torch.cuda.stream(stream):
            dev_in.copy_(host_in, non_blocking=True)                      # one pinned H2D copy of Q | K | V
            mg.stream_inputs_written(sh)                                  # torch's copy is work the library cannot see
            bg.run_batched(1, [dev_in.data_ptr() + 2 * o for o in offs], dev_out.data_ptr(), work1.data_ptr(), w1, stream=sh)
            host_out_pinned.copy_(dev_out, non_blocking=True)             # D2H of O
        stream.synchronize()                                              # the caller reads the result

    e2e_calls = max(5, min(50, args.steps))
    e2e_ms = timed(e2e_call, e2e_calls, 3) / e2e_calls
    # the same set through the batched launch of the timed protocol (another block shape, so equal up to rounding)
    from tests.helpers import from_bits as _fb
    e2e_diff = float(np.abs(_fb(host_out_pinned.numpy().view(np.uint16).ravel(), mg.float16) -
                            _fb(dense_out[:ob // 2].cpu().numpy().view(np.uint16).ravel(), mg.float16)).max())
    e2e = {"value": round(e2e_ms * 1000.0, 2), "unit": "us/call", "h2d_bytes_per_step": qb + kb + vb,
           "d2h_bytes_per_step": ob, "pcie_gbs": round((qb + kb + vb) / (e2e_ms * 1e-3) / 1e9, 1),
           "max_abs_diff_vs_device_resident_result": round(e2e_diff, 6),
           "note": "one call per e2e step through mg_graph_run_batched with caller-owned buffers: one pinned H2D copy of "
                   "Q|K|V, the fused kernel, D2H of O, stream synchronisation"}

    # ---- fingerprint verification sweep ----------------------------------------------------------------
    fingerprint = run_fingerprint_sweep(args, mg, mo, rt, torch, dist, np, rank, world, stream, timed, barrier)
    candidates = None if args.no_other_configs else run_candidate_verification(mg, rt, torch, dist, np, rank, world, stream)
    others = None
    if not args.no_other_configs:
        # N = 1: all three other configurations; N > 1: the speculative decode, its batch x KV-head units sharded
        others = measure_other_configs(mg, rt, stream, timed, peaks, only=None if world == 1 else "c3", world=world, rank=rank)

    # ---- the reference's own GPU fingerprint kernel on the same box (rank 0, N = 1 only) -------------------------
    if rank == 0 and world == 1 and not args.no_reference_gpu:
        fingerprint["reference_gpu"] = reference_gpu_fingerprint(mo, np, torch, mg, rt, fingerprint["value"])

    # ---- CPU baselines (rank 0, N = 1 only) ----------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_float_baseline(mo, fp_oracle, np, budget_s=8.0)
        fingerprint["cpu_baseline"] = cpu_fingerprint_baseline(mo, np, budget_s=8.0)

    if rank == 0:
        line = {
            "metric": "gqa_decode_customized_op_us_per_call", "value": round(us_per_call, 3), "unit": "us/call",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp16",
            "data": "synthetic (seeded N(0,1) K/V, Q pre-scaled by 1/sqrt(d); fingerprints uniform in [0,227))",
            "config": {"workload": "GQA incremental decode muGraph: batch 1, 32 q heads, 8 kv heads, head_dim 128, kv_len 4096, "
                                   "16 KV splits x for-loop 4 (tiles of 64), 2 customized ops",
                       "kv_heads_per_gpu": heads, "calls_per_step": calls, "calls_per_launch": batch,
                       "launches_per_step": replays * kernels_per_replay, "resident_sets": nbatches * batch,
                       "l2_defeat": "every call reads its own resident set; a replay walks %.0f MB of inputs (> 2.5x L2) before "
                                    "any set is read again" % (nbatches * batch * set_bytes / 1e6),
                       "replay": "CUDA graph of %d batched launches (split-KV + merge of %d independent calls in one kernel), "
                                 "replayed %d times per step on one stream" % (nbatches, batch, replays),
                       "k_layout": args.k_layout, "v_layout": args.v_layout,
                       "parallelism": "kv-heads sharded x%d, no collective" % world},
            "hbm_gbs": round(call_bytes / (us_per_call * 1e-6) / 1e9, 1),
            "output_check": {"calls_checked": checked_calls, "worst_rel_err_vs_fp32": round(worst, 6), "tolerance": 2e-3},
            "per_call_launch": per_call_launch,
            "stream_ordered_us_per_call": None if ordered_us is None else round(ordered_us, 3),
            "single_call_us_median": None if single_us is None else round(single_us, 3),
            "roofline": roofline, "fixed_work_per_gpu": fixed_work, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(gpu_launches),
            "clocks": clocks, "fingerprint": fingerprint, "candidates": candidates, "other_configs": others,
        }
        print(json.dumps(line))
    batched_graph.close()
    if streams_graph is not None:
        streams_graph.close()
        ordered_graph.close()
    for g, _, _ in reversed(graphs):
        g.close()
    bg.close()
    if world > 1:
        dist.destroy_process_group()


def fnv1a64_rows(np, rows):
    """FNV-1a-64 of every row of a [n, m] uint16 array (the digest of tests/golden/sweep_digests_gqa_decode.json),
    vectorised over the rows."""
    h = np.full(rows.shape[0], 1469598103934665603, dtype=np.uint64)
    prime = np.uint64(1099511628211)
    cols = np.ascontiguousarray(rows.T).astype(np.uint64)
    with np.errstate(over="ignore"):
        for c in range(cols.shape[0]):
            h = (h ^ cols[c]) * prime
    return h


def run_fingerprint_sweep(args, mg, mo, rt, torch, dist, np, rank, world, stream, timed, barrier):
    """The verification sweep: the decode muGraph in fingerprint mode over independent seeded input sets (uniform in
    [0, 227)), sets sharded over ranks.  Timed region: evaluation of this rank's sets in chunks, one all-gather of the
    fingerprints, row-wise comparison of all gathered fingerprints with reference fingerprints on the device.  The reference fingerprints are those of an untimed
    first pass, every row of which is checked on the host against the digests produced by the reference's own host
    code (tests/golden/sweep_digests_gqa_decode.json)."""
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
        out = g.customized(g.customized([Q, K, V], p1), p2)
        elems = [t.num_elements for t in (Q, K, V)]
        row = out[0].num_elements
        # All input sets of this rank stay resident when they fit (4096 sets = 69 GB on one GPU); otherwise one
        # chunk is resident at a time and refilled (outside the timed regions) between evaluations.
        free_bytes, _ = torch.cuda.mem_get_info()
        resident = my_sets * 2 * sum(elems) < 0.7 * free_bytes
        held = my_sets if resident else chunk
        bufs = [torch.empty(held * n, dtype=torch.int16, device="cuda") for n in elems]
        # this rank's fingerprints [chunk index][set in chunk][row]; gathered [rank][chunk index][set in chunk][row], i.e.
        # in global set order: set (r, c, s) is global set r * my_sets + c * chunk + s
        local = torch.zeros((nchunks, chunk, row), dtype=torch.int16, device="cuda")
        gathered = torch.zeros((world, nchunks, chunk, row), dtype=torch.int16, device="cuda") if world > 1 else local.view(1, nchunks, chunk, row)
        wbytes = g.fingerprint_batched_workspace(chunk)
        work = torch.empty(max(wbytes, 256), dtype=torch.uint8, device="cuda")
        flags = torch.zeros(nchunks * world * chunk, dtype=torch.int32, device="cuda")
        mismatches = torch.zeros(1, dtype=torch.int32, device="cuda")

        def fill_chunk(c):
            slot0 = c * chunk if resident else 0
            for i, (buf, n) in enumerate(zip(bufs, elems)):
                for s in range(chunk):
                    gs = rank * my_sets + c * chunk + s
                    mg.fill_fingerprint_seeded_raw(rt, buf.data_ptr() + 2 * (slot0 + s) * n, n, 3 * (2024 + gs) + i, mg.FP_P)

        def eval_chunk(c):
            slot0 = c * chunk if resident else 0
            g.fingerprint_batched(chunk, [b.data_ptr() + 2 * slot0 * n for b, n in zip(bufs, elems)],
                                  local[c].data_ptr(), work.data_ptr(), wbytes, stream=sh)

        def gather_all():
            """One all-gather of this rank's fingerprints behind the last evaluation.  (A gather per chunk on a second
            stream, under the next chunk's evaluation, was slower: the evaluation kernel fills every SM with resident
            blocks, so each small collective waited for a gap between two launches and lengthened the chain.)"""
            if world > 1:
                with torch.cuda.stream(stream):
                    dist.all_gather_into_tensor(gathered.view(torch.uint8).view(-1), local.view(torch.uint8).view(-1))

        # ---- untimed first pass: produces the reference fingerprints, checked on the host against the digests
        for c in range(nchunks):
            fill_chunk(c)
            eval_chunk(c)
            if not resident:
                torch.cuda.synchronize()   # the next fill reuses the chunk's input buffers
        gather_all()
        barrier()
        reference = gathered.clone()
        checked, ok = 0, True
        if rank == 0 and os.path.exists(SWEEP_DIGESTS) and total_sets <= SWEEP_SETS:
            with open(SWEEP_DIGESTS) as f:
                want = np.array([int(x) for x in json.load(f)["digests"]], dtype=np.uint64)
            host = reference.cpu().numpy().view(np.uint16)                       # [world, nchunks, chunk, row]
            got = fnv1a64_rows(np, host.reshape(-1, row)).reshape(world, nchunks * chunk)
            for r in range(world):
                first = r * my_sets
                ok = ok and bool(np.array_equal(got[r], want[first:first + nchunks * chunk]))
                checked += nchunks * chunk
        # ---- timed pass
        gathered.zero_() if world > 1 else local.zero_()
        barrier()

        def sweep():
            for c in range(nchunks):
                eval_chunk(c)
            gather_all()
            mg.compare_fingerprint_rows(rt, gathered.data_ptr(), reference.data_ptr(), nchunks * world * chunk, row,
                                        flags.data_ptr(), mismatches.data_ptr(), stream=sh)

        if resident:
            t_total = timed(sweep, 1, 0)
            # the evaluation alone, for the per-GPU bandwidth figure
            t_eval = timed(lambda: [eval_chunk(c) for c in range(nchunks)], 1, 0)
        else:
            t_total, t_eval = 0.0, 0.0
            for c in range(nchunks):
                fill_chunk(c)
                t = timed(lambda: eval_chunk(c), 1, 0)
                t_eval += t
                t_total += t
            t_total += timed(gather_all, 1, 0)
            t_total += timed(lambda: mg.compare_fingerprint_rows(rt, gathered.data_ptr(), reference.data_ptr(), nchunks * world * chunk,
                                                                 row, flags.data_ptr(), mismatches.data_ptr(), stream=sh), 1, 0)
        mg.synchronize()
        rows_equal = int(flags.sum().item())
        evals_per_s = (nchunks * chunk * world) / (t_total * 1e-3)
        info = g.customized_info(3)
    return {"metric": "fingerprint_evals_per_s", "value": round(evals_per_s, 1), "unit": "evals/s",
            "sets": nchunks * chunk * world, "sets_per_gpu": nchunks * chunk, "chunk_sets": chunk,
            "inputs_resident": bool(resident),
            "sweep_ms": round(t_total, 3), "eval_only_ms": round(t_eval, 3),
            "timed_region": "evaluation of all chunks + one all-gather of the fingerprints + row-wise device "
                            "comparison of all gathered fingerprints with the reference fingerprints",
            "rows_equal_to_reference": rows_equal, "rows_compared": nchunks * chunk * world,
            "mismatches": int(mismatches.item()),
            "bytes_per_eval": 16793600, "hbm_gbs_per_gpu": round(16793600 * nchunks * chunk / (t_eval * 1e-3) / 1e9, 1),
            "frac_of_hbm_peak_per_gpu": round(16793600 * nchunks * chunk / (t_eval * 1e-3) / 1e9 / load_peaks()[0]["hbm_gbs"], 4),
            "kernel_op1": info["kernel_fingerprint"], "oracle_checked_sets": checked,
            "oracle": "FNV-1a-64 digests of the reference's own host code (oracle/_ref), tests/golden/sweep_digests_gqa_decode.json",
            "bit_exact": bool(ok and checked > 0 and rows_equal == nchunks * chunk * world)}


def run_candidate_verification(mg, rt, torch, dist, np, rank, world, stream):
    """The search's verify step on independent candidate graphs: the 69 muGraphs of the reference's own search
    checkpoint for the speculative-decode attention graph (tests/golden/spec_decode_candidates.json.gz), dealt
    round-robin over the ranks; every rank evaluates its candidates' fingerprint kernels and compares each result
    with the computation graph's fingerprint on the device (one synchronisation per rank), then the verdicts are
    all-gathered.  Wall clock around the whole step, max over ranks."""
    import contextlib
    import gzip
    from attention_superoptimizer_b200 import sharding
    path = os.path.join(ROOT, "tests", "golden", "spec_decode_candidates.json.gz")
    if not os.path.exists(path):
        return None
    with gzip.open(path) as f:
        fx = json.loads(f.read().decode())
    docs = fx["generated_graphs"]
    sh = stream.cuda_stream

    def inputs_of(g):
        return [g.operator(i)[1][0] for i in range(g.num_operators) if g.operator(i)[0] == 1001]

    with contextlib.ExitStack() as stack:
        ref = stack.enter_context(mg.PyGraph.from_json(fx["computation_graph"], rt))
        for i, t in enumerate(inputs_of(ref)):
            t.fill_fingerprint_seeded(700 + i, mg.FP_PQ)
        ref.fingerprint()
        ref_out = ref.operator(ref.num_operators - 1)[1][0]
        mine = sharding.candidate_shard(len(docs), rank, world)
        batch = []
        for n in mine:
            g = stack.enter_context(mg.PyGraph.from_json(docs[n], rt))
            for i, t in enumerate(inputs_of(g)):
                t.fill_fingerprint_seeded(700 + i, mg.FP_PQ)
            batch.append((g, g.operator(g.num_operators - 1)[1][0]))

        def step():
            return sharding.verify_candidates_sharded(len(docs), lambda idx: mg.verify_candidates(ref_out, batch, stream=sh),
                                                      world, rank, device=torch.device("cuda") if world > 1 else None)

        step()
        times = []
        for _ in range(5):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            flags, _ = step()
            times.append(time.perf_counter() - t0)
        ms = torch.tensor([statistics.median(times) * 1e3], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return {"candidates": len(docs), "candidates_per_gpu": len(mine), "all_equal_to_computation_graph": bool(all(flags)),
            "ms_per_batch": round(float(ms.item()), 3), "candidates_per_s": round(len(docs) / (float(ms.item()) * 1e-3), 1),
            "note": "69 candidate muGraphs of the reference's search checkpoint, round-robin over ranks, fingerprint kernels + "
                    "on-device comparison per candidate, all-gather of the verdicts; wall clock, median of 5"}


def run_one_config(args):
    """`--only-config`: one of the other configurations alone (profiling, tuning); prints {"other_configs": {...}}."""
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

    out = measure_other_configs(mg, rt, stream, timed, load_peaks()[0], only=args.only_config, quick=args.quick)
    print(json.dumps({"other_configs": out}))


def measure_other_configs(mg, rt, stream, timed, peaks, only=None, quick=False, world=1, rank=0):
    """Device-timed numbers for the remaining configurations (N = 1 only), each replayed from a CUDA graph:
    speculative decode with the causal draft window (fp16), dense prefill (bf16, tcgen05) and the matmul chain (both
    modes).  `only` = "c1" | "c3" | "c4" runs one; `quick` = few replays (profiling)."""
    sh = stream.cuda_stream
    out = {}

    def replay_us(launch_all, reps):
        launch_all(1)
        stream.synchronize()
        seq = mg.CapturedSequence(sh, lambda: launch_all(reps))
        if quick:
            ms = timed(seq.launch, 2, 1) / 2
        else:
            # the clocks of an idle GPU take a while to come up: replay untimed for 0.3 s, then time 20 replays
            t_end = time.perf_counter() + 0.3
            while time.perf_counter() < t_end:
                for _ in range(10):
                    seq.launch()
                stream.synchronize()
            ms = timed(seq.launch, 20, 3) / 20
        seq.close()
        mg.synchronize()
        return ms * 1000.0 / reps

    def graphs_runner(graphs):
        return lambda reps: [graphs[i % len(graphs)].run(stream=sh, sync=False) for i in range(max(reps, len(graphs)) if reps == 1 else reps)]

    def hbm_roofline(nbytes, us, kernel):
        gbs = nbytes / us / 1e3
        return {"bound": "hbm", "kernel": kernel, "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(gbs / peaks["hbm_gbs"], 4), "bytes_per_call": nbytes}

    # ---- speculative decode: batch 4 x 8 KV heads = 32 units, 8 draft tokens x group 4 = 32 rows, KV 8192 -------------
    def config3():
        units, rows, d, kv, splits, fr, window = 32 // world, 32, 128, 8192, 16, 8, 8   # units sharded over the ranks
        graphs = []
        for s in range(2):  # two buffer sets of 135 MB each: consecutive calls never share L2 contents
            g = mg.PyGraph(rt)
            Q = g.new_input((units, rows, d)); K = g.new_input((units, d, kv), layout=mg.DmemColumnMajor)
            V = g.new_input((units, kv, d), layout=mg.DmemRowMajor)
            p1, p2 = mg.gqa_decode_plans(units, rows, d, kv, splits, fr)
            parts = g.customized([Q, K, V], p1); g.customized(parts, p2)
            g.set_causal_window(3, window)
            Q.fill_data_seeded(900 + s + 50 * rank, d ** -0.5); K.fill_data_seeded(910 + s + 50 * rank, 1.0); V.fill_data_seeded(920 + s + 50 * rank, 1.0)
            graphs.append((g, [Q, K, V]))
        import torch
        # the batched entry point with one set per call: caller-owned result and workspace, partials are scratch
        g0 = graphs[0][0]
        wbytes = g0.run_batched_workspace(1)
        work = torch.empty(max(wbytes, 256), dtype=torch.uint8, device="cuda")
        res = torch.zeros(units * rows * d, dtype=torch.int16, device="cuda")
        ptrs = [[t.pod.data_ptr for t in ins] for _, ins in graphs]
        batched = lambda reps: [g0.run_batched(1, ptrs[i % 2], res.data_ptr(), work.data_ptr(), wbytes, stream=sh)
                                for i in range(max(reps, 2) if reps == 1 else reps)]
        us = replay_us(batched, 8)
        us_graph = replay_us(graphs_runner([g for g, _ in graphs]), 8)
        graphs = [g for g, _ in graphs]
        nbytes = 2 * units * rows * d * 2 + 2 * units * d * kv * 2
        out["spec_decode_c3"] = {"us_per_call": round(us, 2), "us_per_call_graph_run": round(us_graph, 2), "units_per_gpu": units, "n_gpus": world,
                                 "hbm_gbs": round(nbytes / us / 1e3, 1),
                                 "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4), "bytes": nbytes,
                                 "roofline": hbm_roofline(nbytes, us, "attn_split_tc_kernel + attn_merge_rows_kernel"),
                                 "kernel": graphs[0].customized_info(3)["kernel_float"], "dtype": "fp16",
                                 "note": "32 rows x KV 8192, 16 splits x for-loop 8, causal draft window 8, merge kernel behind "
                                         "the tcgen05 split-KV kernel (programmatic dependent launch); us_per_call: through "
                                         "mg_graph_run_batched (one set per call; the partials are scratch, blocks take single tiles "
                                         "and sum what they hold of a head); us_per_call_graph_run: through mg_graph_run (every "
                                         "split's partial is a tensor of the graph: items dealt whole, 3 or 4 per block)"}
        for g in reversed(graphs):
            g.close()

    # ---- prefill: 32 heads, 2048 x 2048, head_dim 128, bf16 ----------------------------------------------------
    def config4():
        d = 128
        H, SQ, L = 32, 2048, 2048
        g = mg.PyGraph(rt)
        Q = g.new_input((H, SQ, d), mg.bfloat16); K = g.new_input((H, d, L), mg.bfloat16, mg.DmemColumnMajor)
        V = g.new_input((H, L, d), mg.bfloat16, mg.DmemColumnMajor)
        p1, p2 = mg.attention_prefill_plans(H, SQ, d, L)
        acc = g.customized([Q, K, V], p1); g.customized(acc, p2)
        Q.fill_data_seeded(930, d ** -0.5); K.fill_data_seeded(931, 1.0); V.fill_data_seeded(932, 1.0)
        # a stream of 40 calls per replayed graph: a call's blocks take the SMs that the call in front leaves idle in
        # its second round of blocks (programmatic dependent launch; 256 blocks on 148 SMs); one call at a time beside it
        us = replay_us(graphs_runner([g]), 40)
        us_single = replay_us(graphs_runner([g]), 1)
        flops = 4.0 * H * SQ * L * d
        tf = flops / us / 1e6
        sustained = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        out["prefill_c4"] = {"us_per_call": round(us, 2), "us_single_call": round(us_single, 2),
                             "tflops_single_call": round(flops / us_single / 1e6, 1), "tflops": round(tf, 1),
                             "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
                             "frac_of_sustained_bf16_peak": round(tf / sustained, 4), "flops": flops,
                             # timed inside a long loop (0.3 s of replays, then 800 calls) at the end of a long run: the
                             # GPU sits at its power cap, which is what the sustained cuBLAS figure was measured under
                             "roofline": {"bound": "tensor", "kernel": "attn_rows_pp_kernel<bf16>", "achieved": round(tf, 1),
                                          "peak": sustained, "peak_kind": "sustained (kernel timed inside a long loop)",
                                          "unit": "TFLOP/s", "frac": round(tf / sustained, 4),
                                          "frac_of_burst_peak": round(tf / peaks["bf16_tflops"], 4),
                                          "flops_per_call": flops},
                             "kernel": g.customized_info(3)["kernel_float"], "dtype": "bf16",
                             "note": "both customized ops in one launch (division fused into the tcgen05 kernel's epilogue); us_per_call: calls back "
                                     "to back on one stream, 40 per replayed CUDA graph, each launched with programmatic stream "
                                     "serialisation so that its first blocks run beside the last blocks of the call in front; "
                                     "us_single_call: one call per graph replay, nothing overlaps"}
        g.close()

    # ---- matmul chain: X[16,1024] W1[1024,1024] W2[1024,1024], generic interpreters, both modes -------------------
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
        lib, h = g.lib, g.handle
        fp_us = replay_us(lambda reps: [mg.check(lib.mg_graph_fingerprint_enqueue(h, sh)) for _ in range(reps)], 10)
        X.fill_data_seeded(943, 0.02); W1.fill_data_seeded(944, 0.02); W2.fill_data_seeded(945, 0.02)
        float_us = replay_us(graphs_runner([g]), 10)
        nbytes = 4259840
        info = g.customized_info(3)
        names = {0: "generic interpreter", 4: "chain_kernel + tile_reduce_kernel"}
        out["matmul_chain_c1"] = {"float_us_per_call": round(float_us, 1), "fingerprint_us_per_call": round(fp_us, 1),
                                  "kernel": info["kernel_fingerprint"], "kernel_float": info["kernel_float"], "dtype": "fp16",
                                  "bytes": nbytes, "flops": 67108864,
                                  "roofline_float": hbm_roofline(nbytes, float_us, names.get(info["kernel_float"], "?") + " (fp16)"),
                                  "roofline_fingerprint": hbm_roofline(nbytes, fp_us, names.get(info["kernel_fingerprint"], "?") + " (fingerprints)"),
                                  "note": "two customized ops (16 blocks over the intermediate columns, for-loop 16 over K "
                                          "tiles of 64; then the cross-block reduction); inputs N(0, 0.02) / uniform [0,227); both "
                                          "modes replayed from a CUDA graph; the HBM floor of 0.65 us is not the binding limit of a "
                                          "16-block plan (two dependent launches and the latency of one block's 290 KB of tiles are); "
                                          "--interpreter-only times the generic interpreters on the same plan"}
        g.close()

    for name, fn in (("c3", config3), ("c4", config4), ("c1", config1)):
        if only in (None, name):
            fn()
    return out


def reference_gpu_fingerprint(mo, np, torch, mg, rt, our_evals_per_s):
    """The reference's compute_customizedop_fingerprint built for sm_100a (oracle/_ref/libref_gpu.so) on evaluations
    of the sweep, launched the way the reference launches it (`for op: op->fingerprint()`: one kernel and one
    device synchronisation per operator, one input set at a time).  Its result for a seeded set is compared with
    the committed digest of that set."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        return {"unavailable": "oracle/_ref/libref_gpu.so has not been built (needs the reference checkout)"}
    B, M, D, L = KV_HEADS, GROUP, HEAD_DIM, KV_LEN
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
    op1 = ref_gpu.CustomizedOp(specs, p1)
    op2 = ref_gpu.CustomizedOp(None, p2, producer=op1)
    try:
        s = 7
        bufs = []
        for i, sp in enumerate(specs):
            n = int(np.prod(sp.dims))
            b = torch.empty(n, dtype=torch.int16, device="cuda")
            mg.fill_fingerprint_seeded_raw(rt, b.data_ptr(), n, 3 * (2024 + s) + i, mg.FP_P)
            op1.set_input_from_device(i, b.data_ptr())
            bufs.append(b)
        op1.fingerprint()
        op2.fingerprint()
        ok = None
        if os.path.exists(SWEEP_DIGESTS):
            with open(SWEEP_DIGESTS) as f:
                ok = str(mo.fnv1a64(op2.output(0))) == json.load(f)["digests"][s]
        ref_gpu.time_pair(op1, op2, 20)
        iters = 300
        ms = ref_gpu.time_pair(op1, op2, iters)
    finally:
        op2.destroy()
        op1.destroy()
    return {"value": round(1000.0 / ms, 1), "unit": "evals/s", "ms_per_eval": round(ms, 4), "evaluations_timed": iters,
            "matches_committed_digest": ok, "ratio_ours_over_reference_gpu": round(our_evals_per_s * ms / 1000.0, 1),
            "kernel": "compute_customizedop_fingerprint (src/kernel/cuda/customized_kernel.cu:307-603), sm_100a build",
            "protocol": "the reference's: per input set, one launch and one cudaDeviceSynchronize per customized operator "
                        "(customized_kernel.cu:655-678); wall clock"}


def decode_float_inputs(mo, np):
    B, M, D, L = KV_HEADS, GROUP, HEAD_DIM, KV_LEN
    rng = np.random.default_rng(2024)
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
    g1 = mo.build_customized(specs, p1)
    g2 = mo.build_customized(mo.output_specs(g1), p2)
    q = (rng.standard_normal((B, M, D)) / np.sqrt(D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, L, D)).astype(np.float16).astype(np.float32)   # memory image, column-major
    v = rng.standard_normal((B, D, L)).astype(np.float16).astype(np.float32)
    return g1, g2, [q, k, v]


def time_loop(fn, budget_s, max_n=50000):
    fn()  # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        fn()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= max_n:
            break
    return (time.perf_counter() - t0) / n, n


def cpu_float_baseline(mo, fp_oracle, np, budget_s):
    """Times the fp32 host evaluator (oracle/f32_oracle.c, OpenMP) on whole decode calls: all cores the process may
    use, and one core.  Returns the cpu_baseline object (value = all cores)."""
    g1, g2, x = decode_float_inputs(mo, np)
    cores = host_cores()

    def call(threads):
        o1, _ = fp_oracle.run_float(g1, x, threads)
        fp_oracle.run_float(g2, o1, threads)

    t_all, n_all = time_loop(lambda: call(cores), budget_s * 0.6)
    t_one, n_one = time_loop(lambda: call(1), budget_s * 0.4)
    return {"value": round(t_all * 1e6, 1), "unit": "us/call", "cores": cores, "kind": "port",
            "value_1core": round(t_one * 1e6, 1),
            "sample": "%d (all cores) + %d (one core) whole decode muGraph calls, both operators, by the fp32 host evaluator "
                      "oracle/f32_oracle.c (the reference has no CPU float path)" % (n_all, n_one)}


def cpu_fingerprint_baseline(mo, np, budget_s):
    """Times one fingerprint evaluation of the decode muGraph (both operators, one input set of the sweep) by the
    reference's own fingerprinter classes compiled for the host (oracle/_ref), falling back to the plain-C port when
    that library is absent: all cores and one core.  Reported as evaluations per second."""
    from oracle import fp_oracle, ref_host
    B, M, D, L = KV_HEADS, GROUP, HEAD_DIM, KV_LEN
    specs, p1, p2 = mo.gqa_decode_plans(B, M, D, L, SPLITS, FORLOOP)
    x = mo.sweep_inputs(0, specs)
    cores = host_cores()
    if ref_host.available():
        kind, what = "reference", "the reference's host serialiser + fingerprinter classes (oracle/_ref/libref_host.so)"

        def call(threads):
            ref_host.set_threads(threads)
            o1, _ = ref_host.customized_fingerprint(specs, p1, x)
            ref_host.customized_fingerprint([mo.DTensorSpec(o.shape) for o in o1], p2, o1)
    else:
        kind, what = "port", "oracle/fp_oracle.c"
        g1 = mo.build_customized(specs, p1)
        g2 = mo.build_customized(mo.output_specs(g1), p2)

        def call(threads):
            o1, _ = fp_oracle.run(g1, x, 1, threads)
            fp_oracle.run(g2, o1, 1, threads)

    t_all, n_all = time_loop(lambda: call(cores), budget_s * 0.5, 2000)
    t_one, n_one = time_loop(lambda: call(1), budget_s * 0.5, 2000)
    return {"value": round(1.0 / t_all, 2), "unit": "evals/s", "cores": cores, "kind": kind,
            "value_1core": round(1.0 / t_one, 2),
            "sample": "%d (all cores) + %d (one core) evaluations of input set 0 of the sweep (33.5 M modular multiply-adds "
                      "each) by %s; the full sweep is 4096 such evaluations" % (n_all, n_one, what)}


# =================================================================================================
# reference arm: the CPU implementation of the same path, on the box's host cores
# =================================================================================================
def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    import numpy as np
    from oracle import fp_oracle, mugraph_oracle as mo
    # each step = one bounded sample: `calls` whole decode muGraph evaluations by the fp32 host evaluator.
    # The thread count is set explicitly: a launcher may export OMP_NUM_THREADS=1.
    g1, g2, x = decode_float_inputs(mo, np)
    cores = host_cores()
    calls = 4
    used = cores

    def step():
        nonlocal used
        for _ in range(calls):
            o1, used = fp_oracle.run_float(g1, x, cores)
            fp_oracle.run_float(g2, o1, cores)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    us = dt / (args.steps * calls) * 1e6
    sample = "%d steps x %d whole decode muGraph calls, fp32 host evaluator (oracle/f32_oracle.c, OpenMP, %d threads)" % (args.steps, calls, used)
    line = {"impl": "reference", "metric": "gqa_decode_customized_op_us_per_call", "value": round(us, 1), "unit": "us/call",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
            "data": "synthetic (seeded)",
            "config": {"workload": "GQA incremental decode muGraph: batch 1, 32 q heads, 8 kv heads, head_dim 128, kv_len 4096, "
                                   "16 KV splits x for-loop 4 (tiles of 64), 2 customized ops; CPU evaluation",
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
    ap.add_argument("--batch", type=int, default=64, help="independent calls per batched launch of the headline protocol")
    ap.add_argument("--replays-per-step", type=int, default=0,
                    help="replays of the captured launch sequence per step (0 = about 30 ms per step)")
    ap.add_argument("--sweep-sets", type=int, default=SWEEP_SETS, help="input sets of the fingerprint sweep (all ranks)")
    ap.add_argument("--sweep-chunk", type=int, default=128, help="sets per evaluation launch and rank")
    ap.add_argument("--k-layout", default="col", choices=["row", "col"],
                    help="DmemLayout of K[heads, d, kv]: col = memory [kv][d] (KV-cache order), row = memory [d][kv]")
    ap.add_argument("--v-layout", default="row", choices=["row", "col"],
                    help="DmemLayout of V[heads, kv, d]: row = memory [kv][d] (KV-cache order), col = memory [d][kv]")
    ap.add_argument("--streams", type=int, default=0,
                    help="per-call-launch protocol: streams the calls are spread over (0 = 8 per rank at N = 1, 16 at N = 2, "
                         "32 from N = 4)")
    ap.add_argument("--interpreter-only", action="store_true", help="disable the specialised kernels")
    ap.add_argument("--specialisation", type=int, default=2, choices=[0, 1, 2],
                    help="0 = interpreters, 1 = specialised kernels without operator fusion, 2 = with fusion (default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the reference's own GPU fingerprint kernel")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the extra measurements of the other configurations")
    ap.add_argument("--no-per-call-launch", action="store_true",
                    help="skip the protocols that launch one kernel per call (short launch lists for the profiler)")
    ap.add_argument("--no-latency-probes", action="store_true",
                    help="skip the single-call latency and the 1024 + 1024 launch L2-resident measurement (short launch lists)")
    ap.add_argument("--only-config", default=None, choices=["c1", "c3", "c4"],
                    help="measure just this other configuration on one GPU and print its entry (no headline line)")
    ap.add_argument("--quick", action="store_true", help="with --only-config: a handful of replays only (profiler runs)")
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
