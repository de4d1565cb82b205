"""Benchmark of the decoder token loop: decoded tokens/s at batch 64 with weight-only int8 (BASELINE config 3).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" of this benchmark is one pass of the hot path over one batch: 64 sequences (encoder lengths uniform in
[50, 375], 10-token prompts) decoded for 448 new tokens each = 457 CUDA-graph replays of the decoding step. K passes
are timed after W warm-up passes.

  value      decoded tokens/s over all GPUs with the inputs resident in HBM: the timed region is the token loop
             (admit + 457 replays) on the decoder stream, CUDA events, max over ranks.
  e2e        the same metric through the public API from host buffers: pinned host encoder memory -> device,
             fill_cross (cross-K/V prefill), admit, 457 replays, finished rows read back to the host.
  roofline   the dominant kernel (attention over the bf16 KV cache): algorithmic KV bytes per launch / its launch
             duration measured here with CUDA events, against the measured HBM copy bandwidth; `step` gives the same
             for the whole decoding step (weights + KV bytes / replay time) and `classes` splits the step's time into
             attention, layer projections and the rest (whole passes that launch only those kernels).
  stream     BASELINE configs 4 and 5 as extra keys: the seeded request stream through 128 slots per GPU with the 2:4
             feed-forward weights, admitted and evicted between graph replays (config 5: 8000 requests dealt
             round-robin over the ranks).
  cpu_baseline / --impl reference   the reference's CPU arithmetic (transformers fp32 decoder, else the numpy port) on
             the host cores, on a bounded sample of the same workload.
With --gpus N (launched by torchrun, one rank per GPU) every rank decodes its own batch: replicas, no collective on
the token loop; NCCL only for the barriers, the max over ranks and one stats gather.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, PROMPT, NEW, FRAMES = 64, 10, 448, (50, 375)
FALLBACK_HBM_GBS = 6650.0
KV_PREFETCH_MB = 0


def measured_peak() -> tuple[float, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region (read-only queries)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i].lower().startswith("active")
                                                         for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


_RESULT_OUT = None


def emit(text: str, flush: bool = True) -> None:
    """The result line, on the process's original stdout (see main: everything else is sent to stderr)."""
    out = _RESULT_OUT or sys.stdout
    out.write(text + "\n")
    out.flush()


def make_inputs(seed: int):
    rng = np.random.default_rng(seed)
    lens = rng.integers(FRAMES[0], FRAMES[1] + 1, BATCH).tolist()
    memory = torch.from_numpy(rng.standard_normal((sum(lens), 1024), dtype=np.float32))
    prompts = [torch.from_numpy(rng.integers(0, 16384, PROMPT).astype(np.int64)) for _ in range(BATCH)]
    return lens, memory, prompts


def classes_in_child() -> tuple[dict, str | None]:
    """The per-class passes in a process of their own: this command line again with --classes-only. Returns
    ({mask: ms per pass}, None) or ({}, why not)."""
    import subprocess
    cmd = [sys.executable, os.path.abspath(__file__), *sys.argv[1:], "--classes-only", "--no-cpu", "--no-stream"]
    # a plain single process whatever launched this one: none of a distributed launcher's variables go along
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "MASTER_ADDR",
                        "MASTER_PORT") and not k.startswith("TORCHELASTIC_")}
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600, env=env)
    except subprocess.TimeoutExpired:
        return {}, "the class passes did not end within 600 s"
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    if r.returncode != 0 or not lines:
        sys.stderr.write(r.stderr[-2000:])
        return {}, f"the class passes ended with exit code {r.returncode}"
    got = json.loads(lines[-1])["class_ms"]
    return {int(k): float(v) for k, v in got.items()}, None


def run_ours(args) -> None:
    from cohere_inference_b200 import StreamDecoder, dataparallel as dp, native as nv, synthetic_model
    rank, local, world = dp.init()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch N > 1 with torch.distributed.run)"
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    model = synthetic_model(0).to(dev)
    dec = StreamDecoder(model, slots=BATCH, max_new_tokens=NEW, max_prompt=16, max_audio_s=30.0, buckets=(BATCH,),
                        int8=not args.fp16_weights, fp16_weights=args.fp16_weights, eos=-1,
                        pdl=0 if args.no_pdl else args.pdl, chains=args.chains, attn_ring=args.attn_ring,
                        head_split=not args.no_head_split, head_umma=not args.no_head_umma, kv_int8=args.kv_int8,
                        proj_umma=False if args.no_proj_umma else (args.proj_umma or True), kv_prefetch_mb=args.kv_prefetch)
    digest = dec.weights_digest()
    dp.check_identical(digest, dev)  # replicas: the same packed bits on every GPU, before anything is timed
    lens, memory_host, prompts = make_inputs(1000 + rank)
    memory_host = memory_host.pin_memory()
    memory_dev = memory_host.to(dev)
    slots = list(range(BATCH))
    steps_per_pass = PROMPT - 1 + NEW
    out_host = torch.zeros(BATCH, dec.out.shape[1], dtype=torch.long).pin_memory()
    step_events: list = []

    def token_loop(record: bool):
        dec.admit(slots, prompts, lens)
        b = dec.set_active(slots)
        for _ in range(steps_per_pass):
            dec.step(b)
            if record:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(dec.stream)
                step_events.append(ev)

    def resident_pass(record=False):
        """Inputs in HBM: cross K/V already in the slot caches; the timed region is the token loop."""
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(dec.stream)
        if record:
            step_events.append(s)
        token_loop(record)
        e.record(dec.stream)
        return s, e

    prefill_pairs = []

    def e2e_pass():
        """Host buffers in, host tokens out, everything on the decoder stream."""
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(dec.stream):
            s.record(dec.stream)
            mem = memory_host.to(dev, non_blocking=True)
            dec.fill_cross(mem, lens, slots)
            f.record(dec.stream)
        prefill_pairs.append((s, f))
        token_loop(False)
        with torch.cuda.stream(dec.stream):
            out_host.copy_(dec.out[:BATCH], non_blocking=True)
            e.record(dec.stream)
        return s, e

    with torch.cuda.stream(dec.stream):
        dec.fill_cross(memory_dev, lens, slots)
    for _ in range(args.warmup):
        resident_pass()
    dec.stream.synchronize()
    if args.classes_only:  # the child of classes_in_child(): the three partial passes, one line, nothing else
        class_ms = {}
        for mask in (1, 3, 5):
            dec.capture_classes(mask)
            resident_pass()
            dec.stream.synchronize()
            s, e = resident_pass()
            dec.stream.synchronize()
            dec.check_status()
            print(f"[bench] class pass {mask}: done", file=sys.stderr, flush=True)
            class_ms[str(mask)] = s.elapsed_time(e)
        emit(json.dumps({"class_ms": class_ms}))
        return
    dp.barrier(dev)
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        t_wall = time.perf_counter()
        pairs = [resident_pass(record=True) for _ in range(args.steps)]
        dec.stream.synchronize()
        t_wall = time.perf_counter() - t_wall
        dp.barrier(dev)
        torch.cuda.synchronize()
    dec.check_status()
    my_ms = sum(s.elapsed_time(e) for s, e in pairs)  # this rank's own device time
    ms = dp.max_over_ranks(my_ms, dev)
    tokens = BATCH * NEW * args.steps
    value = world * tokens / (ms / 1e3)
    # drop the gaps between passes (admit + set_active): keep intervals that end at a step event of the same pass
    per_pass = steps_per_pass + 1
    step_ms = [a.elapsed_time(b) for i, (a, b) in enumerate(zip(step_events[:-1], step_events[1:]))
               if (i + 1) % per_pass != 0]
    p50 = statistics.median(step_ms)

    # ---- the step's time by class of kernel: whole passes that launch only the embedding / vocabulary projection /
    # pick (1), those plus the layer projections (1 | 2), those plus the attention kernels (1 | 4). The pick runs in
    # all three, so positions advance as in a real pass and every launch moves the bytes it moves there (the values
    # are meaningless). One pass each after one warm-up pass. These passes run kernel sequences no real step has, so
    # they run in a child process of their own (1 GPU only): whatever happens there, this process still holds its
    # measurements and prints its line.
    class_ms, class_note = {}, None
    if not args.no_classes and world == 1:
        class_ms, class_note = classes_in_child()
    elif not args.no_classes:
        class_note = "measured at 1 GPU only"

    # ---- algorithmic bytes of the passes (exact positions and lengths) and the step's roofline
    total_bytes = sum(dec.step_bytes([min(t, steps_per_pass)] * BATCH, lens) for t in range(steps_per_pass))
    peak, peak_kind = measured_peak()
    loop_ms = sum(step_ms) / args.steps
    step_gbs = total_bytes / (loop_ms / 1e3) / 1e9

    # ---- the dominant kernel alone: cross-attention over all rows, cycling the layers so no launch finds its
    # cache in L2 (one layer's cross K/V is ~56 MB, the eight together ~450 MB > the 126 MB L2)
    lib, L = nv.lib(), len(dec.layers)
    attn_fn = lib.b200dec_attention_ring if args.attn_ring else lib.b200dec_attention
    kv_bytes = int(sum(lens) * 2 * 1024 * ((1 + 4 / dec.d) if args.kv_int8 else 2))
    reps = 10

    def attn_launches():
        for i in range(reps * L):
            ly = i % L
            if args.attn_ring:
                nv.check(attn_fn(0, nv.ptr(dec.active), nv.ptr(dec.cq), 1024, nv.ptr(dec.cross_k[ly]),
                                 nv.ptr(dec.cross_v[ly]), nv.ptr(dec.cross_len), dec.slots, dec.h, dec.d,
                                 dec.frames, dec.scale, nv.ptr(dec.att), nv.OUT_F16, BATCH,
                                 nv.ptr(dec.attn_part), nv.ptr(dec.attn_count), nv.ptr(dec.status),
                                 1 if args.pdl & 2 else 0, nv.stream_ptr(dec.stream)))
            elif args.kv_int8:
                nv.check(lib.b200dec_attention_paired_q8(0, nv.ptr(dec.sched_cross), nv.ptr(dec.cq), 1024,
                                                         nv.ptr(dec.cross_k[ly]), nv.ptr(dec.cross_v[ly]),
                                                         nv.ptr(dec.cross_ks[ly]), nv.ptr(dec.cross_vs[ly]), dec.h,
                                                         dec.d, dec.frames, dec.scale, nv.ptr(dec.att), nv.OUT_F16,
                                                         BATCH, 1 if args.pdl & 2 else 0, nv.stream_ptr(dec.stream)))
            else:  # what the step launches at this batch size: the paired kernel on the step's own row schedule
                nv.check(lib.b200dec_attention_paired(0, nv.ptr(dec.sched_cross), nv.ptr(dec.cq), 1024,
                                                      nv.ptr(dec.cross_k[ly]), nv.ptr(dec.cross_v[ly]), dec.h, dec.d,
                                                      dec.frames, dec.scale, nv.ptr(dec.att), nv.OUT_F16, BATCH,
                                                      1 if args.pdl & 2 else 0, nv.stream_ptr(dec.stream)))

    # launched from a CUDA graph, as in the step (from Python the loop would be bound by the host's launch rate)
    attn_graph = torch.cuda.CUDAGraph()
    ks, ke = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(dec.stream):
        attn_launches()
        with torch.cuda.graph(attn_graph, stream=dec.stream):
            attn_launches()
        attn_graph.replay()
        ks.record(dec.stream)
        attn_graph.replay()
        ke.record(dec.stream)
    dec.stream.synchronize()
    attn_us = ks.elapsed_time(ke) * 1e3 / (reps * L)
    attn_gbs = kv_bytes / (attn_us / 1e6) / 1e9

    # ---- the same launch with nothing but its loads (b200dec_read_probe): one CTA per (row, head) as above, each reading
    # its share of the launch's bytes from the cross caches, six disjoint regions in turn (333 MB > L2), replayed from a
    # graph with the same launch attribute. What a launch of this size can read at all: ramp-up and tail included.
    items = BATCH * dec.h
    per_cta = (kv_bytes // items) // 16 * 16
    region = -(-items * per_cta // (1 << 20)) + 4 << 20  # bytes between the starts of two regions
    flat = dec.cross_k.view(torch.uint8).reshape(-1)
    n_regions = min(6, (flat.numel() - items * per_cta) // region + 1)
    bare_us = None
    if n_regions >= 3:
        def probe_launches():
            for i in range(reps * L):
                nv.check(lib.b200dec_read_probe(flat.data_ptr() + (i % n_regions) * region, items, per_cta, None,
                                                1 if args.pdl & 2 else 0, nv.stream_ptr(dec.stream)))
        probe_graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(dec.stream):
            probe_launches()
            with torch.cuda.graph(probe_graph, stream=dec.stream):
                probe_launches()
            probe_graph.replay()
            ks.record(dec.stream)
            probe_graph.replay()
            ke.record(dec.stream)
        dec.stream.synchronize()
        bare_us = ks.elapsed_time(ke) * 1e3 / (reps * L)

    # ---- end to end through the public API, host buffers
    for _ in range(min(args.warmup, 2)):
        e2e_pass()
    dec.stream.synchronize()
    dp.barrier(dev)
    torch.cuda.synchronize()
    pairs = [e2e_pass() for _ in range(args.steps)]
    dec.stream.synchronize()
    dp.barrier(dev)
    e2e_ms = dp.max_over_ranks(sum(s.elapsed_time(e) for s, e in pairs), dev)
    e2e_value = world * tokens / (e2e_ms / 1e3)
    prefill_ms = sum(s.elapsed_time(f) for s, f in prefill_pairs[-args.steps:]) / args.steps
    assert (out_host[:, PROMPT:PROMPT + NEW] != dec.pad).any()

    all_stats = dp.gather_stats(dict(steps=steps_per_pass * args.steps, new_tokens=tokens, bytes=total_bytes * args.steps,
                                     gpu_us=int(my_ms * 1e3), p50_step_ns=int(p50 * 1e6)), dev)
    chains_per_step, launches_per_step = len(dec.row_ranges(BATCH)), dec.launches(BATCH)
    weight_bytes, head_bytes = dec.weight_bytes, dec.head.stream_bytes()
    # ---- BASELINE configs 4 / 5: the request stream (extra keys of the line)
    stream = {}
    if not args.no_stream:
        del dec
        torch.cuda.empty_cache()
        if world == 1:
            stream["config4"] = stream_workload(args, dev, rank, local, world, 2000)
        stream["config5"] = stream_workload(args, dev, rank, local, world, args.stream_requests)
        dec = None
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import cpu_baseline
        r = cpu_baseline.time_cpu(synthetic_model(0), BATCH, args.cpu_steps)
        cpu = {"value": round(r["tokens_per_s"], 1), "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"],
               "sample": r["sample"], "ms_per_step": round(r["ms_per_step"], 2)}
    if rank == 0:
        classes = {"unavailable": class_note} if class_note else None
        if class_ms:
            # bytes of a pass by class: the attention kernels' keys, values and appends; the layer projections' weights;
            # the vocabulary projection's weights and the embedding rows
            head_b = head_bytes + BATCH * 2 * 1024 * 2
            proj_b = weight_bytes - head_bytes
            kv_b = total_bytes / steps_per_pass - proj_b - head_b
            t1, t12, t14 = class_ms[1], class_ms[3], class_ms[5]

            def entry(b_step, ms_pass):
                us = ms_pass * 1e3 / steps_per_pass
                return {"bytes_per_step": int(b_step), "us_per_step": round(us, 1),
                        "frac": round(b_step / (us / 1e6) / 1e9 / peak, 4) if us > 0 else None}
            classes = {"attention": entry(kv_b, t14 - t1), "projections": entry(proj_b, t12 - t1),
                       "embed_head_pick": entry(head_b, t1),
                       "sum_us": round((t14 + t12 - t1) * 1e3 / steps_per_pass, 1),
                       "how": "in a child process: whole passes (457 replays, real positions) that launch only the class's kernels beside "
                              "the embedding / vocabulary projection / pick; time of a class = its pass minus the pass "
                              "of those three alone; bytes and fraction of the measured HBM peak per step"}
        line = {
            "metric": "decoded tokens/s at batch 64, " + ("fp16 weights (not the benchmark's mode)" if args.fp16_weights else
                                                          "weight-only int8") + (", int8 KV caches" if args.kv_int8 else ""),
            "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": ("fp16 weights" if args.fp16_weights else "int8 weights") + " x fp16, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "BASELINE config 3: 8 layers x 1024, 16 heads x 64, GELU, vocab 16384; batch 64 per GPU, "
                                   "encoder lengths U[50,375], 10-token prompts + 448 new tokens, one CUDA graph per "
                                   "decoding step; a bench step = one pass = 457 replays",
                       "batch_per_gpu": BATCH, "new_tokens": NEW,
                       "kv_cache": "int8 + fp32 scale per head vector" if args.kv_int8 else "bf16",
                       "parallelism": f"dp{world} replicas", "chains_per_step": chains_per_step,
                       "kv_prefetch_mb": args.kv_prefetch,
                       "l2": "inputs larger than L2: each replay streams ~0.2-1.9 GB of KV cache and weights",
                       "weights": "seed-0 random init N(0, 0.02)", "packed_weights_sha256": digest[:16]},
            "p50_step_ms": round(p50, 4),
            "tokens_per_s_per_gpu": round(value / world, 1),
            # every row advances one position per replay, the 9 prompt-feeding steps of a sequence included
            "row_steps_per_s": round(world * BATCH * steps_per_pass * args.steps / (ms / 1e3), 1),
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(memory_host.numel() * 4),
                    "d2h_bytes_per_step": int(out_host.numel() * 8 + steps_per_pass * (BATCH + 1)),
                    "ms_per_step": round(e2e_ms / args.steps, 3),
                    # host -> device copy of the encoder memory + fill_cross (cross-K/V prefill), this rank
                    "prefill_ms": round(prefill_ms, 3)},
            "gpu_launches": launches_per_step * steps_per_pass * args.steps,
            "roofline": {"bound": "hbm", "kernel": ("attention_ring" if args.attn_ring else "attention_pair") + " kernel <64, cross> (64 rows x 16 heads), replayed from a CUDA graph",
                         "achieved": round(attn_gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(attn_gbs / peak, 4),
                         "peak_source": peak_kind, "bytes_per_launch": kv_bytes, "us_per_launch": round(attn_us, 2),
                         # dram__bytes_read.sum + dram__bytes_write.sum of one such launch from an ncu capture of the
                         # same kernel on the same 64 rows: a stored figure, scaled by bytes, not measured by this run
                         # (no number taken under a profiler is a bench value, and ncu is not run from here)
                         "traffic": int(kv_bytes * (ATTN_TRAFFIC_PER_BYTE_Q8 if args.kv_int8 else ATTN_TRAFFIC_PER_BYTE)),
                         "traffic_source": "stored: ncu capture of this kernel, scaled by bytes; not re-measured by this run",
                         "step": {"bytes_per_step_mean": int(total_bytes / steps_per_pass),
                                  "achieved": round(step_gbs, 1), "frac": round(step_gbs / peak, 4),
                                  "frac_of_8TBs": round(step_gbs / 8000, 4)},
                         # a launch of the same grid that only loads the same number of bytes (b200dec_read_probe):
                         # the kernel's time against it says how much of the distance to `peak` is the size of the
                         # launch (ramp-up and tail of 55 MB) rather than the kernel
                         "bare_read": None if bare_us is None else {
                             "us_per_launch": round(bare_us, 2), "achieved": round(items * per_cta / (bare_us / 1e6) / 1e9, 1),
                             "unit": "GB/s", "bytes_per_launch": items * per_cta,
                             "kernel_time_over_bare_read": round(attn_us / bare_us, 3)},
                         "classes": classes},
            "stream": stream or None,
            "cpu_baseline": cpu,
            "clocks": clocks.summary(),
            "per_rank_tokens_per_s": [round(s["new_tokens"] / (s["gpu_us"] / 1e6), 1) for s in all_stats],
            "per_rank_p50_step_ms": [round(s["p50_step_ns"] / 1e6, 4) for s in all_stats],
            "wall_s": round(t_wall, 3),
        }
        emit(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


# measured DRAM traffic (ncu dram__bytes_read.sum + dram__bytes_write.sum of one cross-attention launch over the
# benchmark's 64 rows) / algorithmic key and value bytes of that launch: bf16 caches, int8 caches with their scales
ATTN_TRAFFIC_PER_BYTE = (55.73 + 0.28) / 55.44
ATTN_TRAFFIC_PER_BYTE_Q8 = 30.04 / 29.45


def run_profile(args) -> None:
    """A short run for a profiler: the config-3 batch at a mid-sequence position, kernels launched directly (no graph),
    3 warm-up steps, then `--profile N` steps between cudaProfilerStart/Stop (use ncu --profile-from-start off).
    --profile-slots / --profile-pos size the case (a capture with many passes wants a small one)."""
    from cohere_inference_b200 import StreamDecoder, synthetic_model
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = args.profile_slots
    dec = StreamDecoder(synthetic_model(0).to(dev), slots=B, max_new_tokens=NEW, max_prompt=16, max_audio_s=30.0,
                        buckets=(B,), int8=True, eos=-1, graphs=False, ffn_sparse=args.sparse, chains=args.chains,
                        attn_ring=args.attn_ring, kv_prefetch_mb=args.kv_prefetch, kv_int8=args.kv_int8)
    rng = np.random.default_rng(1000)
    lens = rng.integers(FRAMES[0], FRAMES[1] + 1, B).tolist()
    prompts = [torch.from_numpy(rng.integers(0, 16384, PROMPT).astype(np.int64)) for _ in range(B)]
    slots = list(range(B))
    with torch.cuda.stream(dec.stream):
        dec.fill_cross(torch.randn(sum(lens), 1024, device=dev), lens, slots)
    dec.admit(slots, prompts, lens)
    b = dec.set_active(slots)
    with torch.cuda.stream(dec.stream):
        dec.pos[:B] = args.profile_pos  # the self cache below this position holds zeros: same bytes, same time
        dec.plen[:B] = 1
    for _ in range(3):
        dec.step(b)
    dec.stream.synchronize()
    torch.cuda.profiler.start()
    for _ in range(args.profile):
        dec.step(b)
    dec.stream.synchronize()
    torch.cuda.profiler.stop()
    dec.check_status()
    kv = sum(lens) * 2 * 1024 * 2
    emit(json.dumps({"profile_steps": args.profile, "rows": B, "pos": args.profile_pos + 3, "sum_frames": sum(lens),
                      "cross_kv_bytes_per_launch": kv, "self_kv_bytes_per_launch": B * (args.profile_pos + 4) * 4096,
                      "weight_bytes": dec.weight_bytes, "launches_per_step": dec.launches_per_step}))


def run_profile_prefill(args) -> None:
    """A short run for a profiler: fill_cross (the two tcgen05 products of the cross-K/V prefill) on `--profile-frames`
    encoder frames in pieces of up to 375, 2 warm-up calls, then `--profile-prefill N` calls between
    cudaProfilerStart/Stop; prints the frames, the FLOPs of one call and its CUDA-event time without a profiler."""
    from cohere_inference_b200 import StreamDecoder, synthetic_model
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dec = StreamDecoder(synthetic_model(0).to(dev), slots=64, max_new_tokens=NEW, max_prompt=16, max_audio_s=30.0,
                        buckets=(1,), int8=True, eos=-1, kv_int8=args.kv_int8)
    lens, left = [], args.profile_frames
    while left > 0:
        lens.append(min(left, FRAMES[1]))
        left -= lens[-1]
    assert len(lens) <= 64
    hidden = torch.randn(sum(lens), 1024, device=dev)
    slots = list(range(len(lens)))
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(dec.stream):
        for _ in range(2):
            dec.fill_cross(hidden, lens, slots)
        s.record(dec.stream)
        dec.fill_cross(hidden, lens, slots)
        e.record(dec.stream)
    dec.stream.synchronize()
    torch.cuda.profiler.start()
    with torch.cuda.stream(dec.stream):
        for _ in range(args.profile_prefill):
            dec.fill_cross(hidden, lens, slots)
    dec.stream.synchronize()
    torch.cuda.profiler.stop()
    dec.check_status()
    m = sum(lens)
    flops = 2 * 2 * m * 1024 * (1024 + 16384)  # both bf16 halves of the rows against both weight matrices
    emit(json.dumps({"profile_prefill_calls": args.profile_prefill, "frames": m, "pieces": len(lens), "flops_per_call": flops,
                     "ms_per_call": round(s.elapsed_time(e), 4),
                     "tflops": round(flops / (s.elapsed_time(e) / 1e3) / 1e12, 1)}))


def stream_workload(args, dev, rank: int, local: int, world: int, n_requests: int) -> dict | None:
    """BASELINE configs 4 / 5: continuous batching, 128 slots per GPU, 2:4 int8 feed-forward weights, a seeded Poisson
    stream of n_requests requests dealt round-robin over the ranks, admitted and evicted between graph replays by
    DecodeScheduler. Device time of the whole run (max over ranks), delivered new tokens, occupancy (whole run, and
    over the steady part between ramp-up and drain), and the run's algorithmic bytes against the measured HBM peak.
    Every rank calls this; rank 0 gets the summary."""
    from cohere_inference_b200 import DecodeScheduler, StreamDecoder, synthetic_model, synthetic_requests
    from cohere_inference_b200 import dataparallel as dp
    SLOTS = 128
    dec = StreamDecoder(synthetic_model(0).to(dev), slots=SLOTS, max_new_tokens=NEW, max_prompt=16, max_audio_s=30.0,
                        int8=True, ffn_sparse=True, eos=-1, pdl=args.pdl, attn_ring=args.attn_ring,
                        head_umma=not args.no_head_umma, kv_prefetch_mb=args.kv_prefetch, device_sched=args.device_sched)
    mine = dp.partition(synthetic_requests(n_requests, seed=0, slots=SLOTS * world, fill=args.fill), rank, world)
    # encoder memory in pinned host memory: 16 seeded N(0, 1) blocks of the longest length, a request takes the first
    # `frames` rows of one of them (the scheduler copies them to the device at admission); drawing every request's own
    # block would make the host the bottleneck of the run without changing a byte the GPU moves
    g = torch.Generator().manual_seed(1234 + rank)
    pool = torch.randn(16, FRAMES[1], 1024, generator=g).pin_memory()
    sched = DecodeScheduler(dec, lambda r: pool[r.mem_seed % 16, :r.frames], account_bytes=True)
    dp.barrier(dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(dec.stream)
    out = sched.run(mine)
    e1.record(dec.stream)
    torch.cuda.synchronize()
    dp.barrier(dev)
    wall = time.perf_counter() - t0
    dec.check_status()
    st = sched.stats
    ms = dp.max_over_ranks(e0.elapsed_time(e1), dev)
    times = sched.step_time_summary()
    stats = dp.gather_stats(dict(steps=st.steps, row_steps=st.row_steps, padded_row_steps=st.padded_row_steps,
                                 slot_steps=st.slot_steps, admitted=st.admitted, evicted=st.evicted,
                                 new_tokens=st.new_tokens, delivered_tokens=st.delivered_tokens, bytes=st.bytes,
                                 gpu_us=int(e0.elapsed_time(e1) * 1e3), steady_row_steps=st.steady_row_steps,
                                 steady_slot_steps=st.steady_slot_steps,
                                 p50_step_ns=int(times.get("p50_ms", 0) * 1e6)), dev)
    assert all(o is not None for o in out) and st.evicted == len(mine)
    del sched, dec
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    tokens = sum(s["new_tokens"] for s in stats)
    gbs = sum(s["bytes"] for s in stats) / world / (ms / 1e3) / 1e9
    return {"workload": f"{n_requests} requests (encoder lengths U[50,375], targets U[16,448], Poisson arrivals at "
                        f"{args.fill:.2f} x the service rate) dealt round-robin over {world} GPU(s), 128 slots each, 2:4 "
                        "int8 feed-forward weights; host memory -> prefill -> decode -> tokens on the host",
            "tokens_per_s": round(tokens / (ms / 1e3), 1), "n_gpus": world,
            "per_rank_tokens_per_s": [round(s["new_tokens"] / (s["gpu_us"] / 1e6), 1) for s in stats],
            "steps": [s["steps"] for s in stats], "ms_per_step": round(ms / max(s["steps"] for s in stats), 4),
            "p50_step_ms": [round(s["p50_step_ns"] / 1e6, 4) for s in stats],
            "occupancy": round(sum(s["row_steps"] for s in stats) / max(1, sum(s["slot_steps"] for s in stats)), 4),
            "occupancy_steady": round(sum(s["steady_row_steps"] for s in stats) /
                                      max(1, sum(s["steady_slot_steps"] for s in stats)), 4),
            "padding": round(sum(s["padded_row_steps"] for s in stats) / max(1, sum(s["row_steps"] for s in stats)), 4),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(gbs / peak, 4), "peak_source": peak_kind,
                         "what": "whole run incl. host scheduling, per GPU"},
            "wall_s": round(wall, 2)}


def run_stream(args) -> None:
    """`--workload stream`: only the request stream (configs 4 / 5), one JSON line."""
    from cohere_inference_b200 import dataparallel as dp
    rank, local, world = dp.init()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    with ClockSampler(local) as clocks:
        r = stream_workload(args, dev, rank, local, world, args.requests)
    if rank == 0:
        emit(json.dumps({"metric": "decoded tokens/s, continuous batching, 128 slots per GPU, 2:4 int8 feed-forward",
                         "impl": "ours", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                         "higher_is_better": True, "scaling": "strong", "data": "synthetic",
                         "config": {"workload": f"BASELINE config {'4' if world == 1 else '5'}: " + r["workload"]},
                         **{k: v for k, v in r.items() if k not in ("workload", "tokens_per_s", "n_gpus")},
                         "clocks": clocks.summary()}), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def run_reference(args) -> None:
    """The reference's own CPU implementation of the path (transformers, FAST=0 arithmetic) on the host cores, on a
    bounded sample of the same workload. Rank 0 alone runs it."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    from cohere_inference_b200 import synthetic_model
    from oracle import cpu_baseline
    model = synthetic_model(0)
    runs = []
    for i in range(args.warmup + args.steps):
        r = cpu_baseline.time_cpu(model, BATCH, args.cpu_steps, seed=1000)
        if i >= args.warmup:
            runs.append(r)
        if i == 0 and r["seconds"] + r["prefill_s"] > 60:  # slow host: one sample is the bounded budget
            runs = [r]
            break
    secs, toks = sum(r["seconds"] for r in runs), sum(r["batch"] * r["steps"] for r in runs)
    value = toks / secs
    r = runs[-1]
    line = {"impl": "reference", "metric": "decoded tokens/s at batch 64, weight-only int8", "value": round(value, 1),
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(runs), "warmup": args.warmup,
            "ms_per_step": round(1e3 * secs / len(runs), 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32 (CPU)", "data": "synthetic",
            "config": {"workload": "BASELINE config 3 shapes on the host CPU: batch 64, encoder lengths U[50,375]; each "
                                   f"step a bounded sample of {args.cpu_steps} cached greedy decoding steps",
                       "batch_per_gpu": BATCH},
            "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"],
                             "sample": r["sample"]},
            "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-steps", type=int, default=32, help="decoding steps of the bounded CPU sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-pdl", action="store_true", help="launch the step's kernels without programmatic dependent launch")
    ap.add_argument("--pdl", type=int, default=7, help="which launches are programmatic: 1 projection after projection, "
                    "2 attention, 4 projection after attention (sum them)")
    ap.add_argument("--no-proj-umma", action="store_true", help="the layer projections on mma.sync instead of tcgen05")
    ap.add_argument("--proj-umma", default="", help="all, or a subset of qkv,o,cq,co,fc1,fc2 on tcgen05 (default: qkv,fc1)")
    ap.add_argument("--no-head-umma", action="store_true", help="vocabulary projection on mma.sync instead of tcgen05")
    ap.add_argument("--no-head-split", action="store_true", help="vocabulary projection on a single fp16 operand")
    ap.add_argument("--fp16-weights", action="store_true", help="the 16-bit weight mode (fp16 image of the bf16 weights) "
                    "instead of int8: a separate row, not the benchmark's configuration")
    ap.add_argument("--kv-int8", action="store_true", help="int8 KV caches with per-vector scales (the reference's int8 "
                    "mode); a separate row, the headline keeps bf16 caches")
    ap.add_argument("--attn-ring", action="store_true", help="use the persistent bulk-copy attention kernel")
    ap.add_argument("--chains", type=int, default=1, help="concurrent kernel chains a step's rows are split into")
    ap.add_argument("--profile", type=int, default=0, help="profiler mode: this many directly launched steps")
    ap.add_argument("--profile-prefill", type=int, default=0, help="profiler mode: this many fill_cross calls")
    ap.add_argument("--profile-frames", type=int, default=2048, help="encoder frames of a profiled fill_cross call")
    ap.add_argument("--profile-slots", type=int, default=BATCH)
    ap.add_argument("--profile-pos", type=int, default=225)
    ap.add_argument("--sparse", action="store_true", help="profiler mode: 2:4 feed-forward weights")
    ap.add_argument("--workload", default="batch64", choices=["batch64", "stream"],
                    help="batch64: BASELINE config 3 (the headline line); stream: configs 4 / 5, continuous batching")
    ap.add_argument("--requests", type=int, default=2000, help="stream workload: requests in the whole stream")
    ap.add_argument("--stream-requests", type=int, default=8000, help="requests of the config-5 stream run by the default "
                    "invocation (dealt round-robin over the ranks)")
    ap.add_argument("--fill", type=float, default=1.05, help="stream workloads: arrival rate as a multiple of the rate "
                    "at which 128 slots per GPU serve requests")
    ap.add_argument("--no-stream", action="store_true", help="skip the stream workloads of the default invocation")
    ap.add_argument("--no-classes", action="store_true", help="skip the per-class passes")
    ap.add_argument("--classes-only", action="store_true", help="run only the per-class passes and print their times "
                    "(what the default invocation starts as a child process)")
    ap.add_argument("--kv-prefetch", type=int, default=KV_PREFETCH_MB, help="MB of an attention launch's keys and values "
                    "that the projections before it start towards L2 (0: off)")
    ap.add_argument("--device-sched", action="store_true", help="stream workloads: the active list lives on the device")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: libraries that write to file descriptor 1 themselves (NCCL's
    # version banner, for one) are pointed at stderr, the result goes to a copy of the original descriptor
    global _RESULT_OUT
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.profile_prefill:
        run_profile_prefill(args)
    elif args.profile:
        run_profile(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "stream":
        run_stream(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
