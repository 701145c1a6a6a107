"""Throughput of the token loop on B200s: NCP coarse-to-fine generate + decode.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps 2 --warmup 1     # the reference's CPU build

Workload (default "c2"): the mid NCP configuration -- 12 layers, d=512, 8 query /
2 KV heads, SwiGLU, prefix 256, levels 1-4-16-32 over 4096-entry codebooks, CFG
1.5, temperature 0.8, top-k 50, top-p 0.9, frequency penalty 0.2 -- on 256
sequences per GPU with seeded N(0, 0.02) weights and Zipf(1.1) prefixes.  One
step = one ncp_generate over the batch plus decoding the codes to token ids.
Sequences are independent: each rank runs its own 256 (weak scaling), no
collective on the data path.  "tokens" are nominal: 512 target tokens per
sequence (32 concepts x 16 tokens), as the configuration states.

One JSON line is printed by rank 0:
  value      device-timed (CUDA events) whole-job tokens/s, ids already in HBM
  e2e        the same through the host C API: host prefix ids in, host token ids out
  roofline   the GEMM kernel class: FLOPs executed / event-timed duration vs measured peak
  cpu_baseline  the reference CPU build (oracle/_ref) or the oracle port on a bounded sample
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "saphira-cncm_b200"))

import capi  # noqa: E402
import synth  # noqa: E402

NOMINAL_TOKENS = {"c2": 512, "c5": 512, "c1": 81, "c1b": 81, "c2s": 512}


def workload(name: str):
    if name == "c2":
        return synth.spec_c2(), 256
    if name == "c2s":                      # C2 widths at 2 layers: quick functional runs
        return synth.spec_c2(n_layer=2, name="c2s"), 32
    if name == "c5":
        return synth.spec_c5(), 1024
    if name == "c1":
        return synth.spec_c1(), 64
    if name == "c1b":
        return synth.spec_c1((1, 3, 9, 81)), 64
    raise SystemExit(f"unknown workload {name}")


def gen_kwargs(spec):
    g = spec.gen
    kw = dict(temp=float(g.get("temperature", 0.0)), top_k=int(g.get("top_k", 0)), top_p=float(g.get("top_p", 1.0)),
              cfg=float(g.get("cfg_scale", 0.0)), freq=float(g.get("freq", 0.0)), mu=float(g.get("mu", 0.0)))
    if spec.token_unigram:
        kw["allow"] = np.full(max(spec.vocab), 1.0 / max(spec.vocab))
    return kw


def algorithmic_flops_per_row(spec) -> float:
    """MACs * 2 per model row with the prefix processed once (attention included)."""
    C_, H, nkv = spec.n_embd, spec.n_head, spec.n_kv_heads
    hd = C_ // H
    g = 3 if (spec.swiglu or spec.geglu) else 2
    Hh = spec.mlp_hidden if spec.mlp_hidden else 4 * C_
    lin = C_ * (C_ + 2 * nkv * hd) + C_ * C_ + g * C_ * Hh
    P, Ls = spec.prefix_len, spec.levels
    lv = Ls if spec.query_level0 else Ls[1:]
    vs = spec.vocab if spec.query_level0 else spec.vocab[1:]
    mac = spec.n_layer * lin * (P + sum(lv))
    mac += spec.n_layer * (2 * P * P * C_ + sum(2 * l * (P + l) * C_ for l in lv))
    mac += sum(l * v * C_ for l, v in zip(lv, vs)) + (P + sum(lv)) * C_ * spec.vq_dim
    return 2.0 * mac


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
            t0 = time.time()                      # the tool needs a moment to start: wait for its first line, so that
            while not self.rows and time.time() - t0 < 3.0:      # the samples that follow fall inside the region
                time.sleep(0.01)
            self.rows.clear()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.th.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(sm)[len(sm) // 2:] if sm else []          # upper half: samples under load
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm

def cpu_sample_run(spec, conf, w, rows: int, steps: int, warmup: int, seed: int, keep: "dict | None" = None):
    """Times the reference's CPU build (oracle/_ref) -- or, where that build is not
    present, the CPU oracle port -- on `rows` sequences of the workload per step.
    Returns (kind, cores, [seconds per step]); `keep` receives the prefixes, seed, codes and
    token ids of the last step so that the caller can check its own results against them."""
    cores = os.cpu_count() or 1
    kw = gen_kwargs(spec)
    pre = synth.ncp_prefixes(spec, rows, seed)
    if keep is not None:
        keep.update(prefix=pre, seed=seed)
    ref_lib = os.path.join(ROOT, "oracle", "_ref", "libcncm_ref.so")
    times = []
    if os.path.exists(ref_lib):
        os.environ["NCM_THREADS"] = str(cores)
        os.environ["OMP_NUM_THREADS"] = str(cores)      # torchrun presets 1; the reference build reads it when it loads
        ref = capi.NcmLib(ref_lib)
        m = capi.NcpModel(ref, conf, w, arena_mb=2048)
        L, D, Vp, nl = spec.L, spec.vq_dim, spec.in_vocab, len(spec.levels)
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            codes = m.generate(pre, seed=seed, **kw)
            # decode as the reference CLI does (src/main.c:863-879): zhats -> decoder -> host argmax
            ref.arena_reset()
            zh = [ref.arena_alloc(rows * L * D) for _ in range(nl)]
            lg = ref.arena_alloc(rows * L * Vp)
            ref.vq_idx_to_zhats(m.vq, codes.ctypes.data, rows, (C.c_void_p * nl)(*zh))
            ref.vqvae_decode(m.vqvae, zh[-1], lg, rows)
            toks = ref.to_host(lg, (rows, L, Vp)).argmax(axis=-1)
            dt = time.perf_counter() - t0
            if it >= warmup:
                times.append(dt)
            if keep is not None:
                keep.update(codes=codes, tokens=toks.astype(np.int32))
        return "reference", cores, times
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    m = orc.Model(conf, w)
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        codes = m.generate(pre, seed=seed, **kw)
        toks = m.decode_tokens(codes)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
        if keep is not None:
            keep.update(codes=codes, tokens=toks)
    return "port", min(cores, rows * (2 if kw["cfg"] > 0 else 1)), times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec, B = workload(args.workload)
    tok = NOMINAL_TOKENS[args.workload]
    rows = args.cpu_rows
    with tempfile.TemporaryDirectory() as tmp:
        conf, w = synth.write_ncp(spec, tmp)
        kind, cores, times = cpu_sample_run(spec, conf, w, rows, args.steps, args.warmup, 7)
    total = sum(times)
    value = rows * tok * len(times) / total
    sample = f"{rows} of the {B} sequences per step (cost is linear in sequences: the reference loops rows)"
    line = {
        "impl": "reference", "metric": "generated tokens/sec", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * total / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (fp64 accumulate)", "data": "synthetic",
        "config": workload_config(args.workload, spec, B, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(name, spec, B, n_gpus):
    return {
        "workload": f"{name}: NCP {spec.n_layer}x{spec.n_embd}, {spec.n_head}q/{spec.n_kv_heads}kv heads, "
                    f"prefix {spec.prefix_len}, levels {'-'.join(map(str, spec.levels))}, codebooks {spec.vocab[0]}x{spec.vq_dim}, "
                    f"{'CFG %.1f, ' % spec.gen.get('cfg_scale', 0) if spec.gen.get('cfg_scale', 0) else ''}"
                    f"temp {spec.gen.get('temperature', 0)}, top-k {spec.gen.get('top_k', 0)}, top-p {spec.gen.get('top_p', 1.0)}; "
                    f"generate + decode to token ids",
        "sequences_per_gpu": B, "global_sequences": B * n_gpus,
        "nominal_tokens_per_sequence": NOMINAL_TOKENS[name], "codes_per_sequence": sum(spec.levels),
        "parallelism": f"independent sequences sharded over {n_gpus} GPU(s), no collective",
        "l2_policy": "working set (K/V cache + activations, > 1 GB) exceeds the 126 MB L2 between iterations",
    }


# --------------------------------------------------------------------------- sharding helpers

def shard_plan(rank: int, world: int, per_gpu: int) -> dict:
    """Weak scaling over independent sequences: rank r owns global rows [r*per_gpu, (r+1)*per_gpu),
    draws its own prefixes (seed 1000 + r) and keys the counter-based sampler by global row."""
    assert 0 <= rank < world
    return {"rows": per_gpu, "row_offset": rank * per_gpu, "prefix_seed": 1000 + rank,
            "global_rows": world * per_gpu, "rng_mode": 1}


def token_checksum(tokens) -> int:
    """CRC-32 of a rank's decoded token ids (int32, row-major): printed per rank so that runs can be compared"""
    import zlib
    return zlib.crc32(np.ascontiguousarray(tokens, dtype=np.int32).tobytes())


def max_over_ranks(values, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity without a process group)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


# --------------------------------------------------------------------------- GPU arm

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the library has no CPU path)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib_path = os.path.join(ROOT, "saphira-cncm_b200", "libncm_b200.so")
    if not os.path.exists(lib_path):
        raise SystemExit("bench.py: libncm_b200.so is not built (python saphira-cncm_b200/build.py)")
    lib = capi.NcmLib(lib_path)
    if args.gemm is not None:
        lib.ncmb_set_gemm_mode(args.gemm)
    stream = torch.cuda.current_stream()
    lib.ncmb_set_stream(C.c_void_p(stream.cuda_stream))

    spec, B = workload(args.workload)
    if args.batch:
        B = args.batch
    tok = NOMINAL_TOKENS[args.workload]
    kw = gen_kwargs(spec)
    tmp = tempfile.TemporaryDirectory()
    conf, w = synth.write_ncp(spec, tmp.name)
    model = capi.NcpModel(lib, conf, w, arena_mb=64)
    # each rank owns a distinct block of sequences; pinned host buffers for the end-to-end path
    plan = shard_plan(rank, world, B)
    prefix = torch.from_numpy(synth.ncp_prefixes(spec, B, plan["prefix_seed"])).pin_memory()
    tokens_host = torch.empty((B, spec.L), dtype=torch.int32).pin_memory()
    tokens_dev = torch.empty((B, spec.L), dtype=torch.int32, device="cuda")
    allow = kw.get("allow")
    allow_p = allow.ctypes.data if allow is not None else None
    # timed runs draw from the counter-based stream keyed by the global sequence index: a sequence's codes do not
    # depend on which rank, batch or wave it runs in (the reference's batch-ordered stream is used for the parity
    # check against the CPU run further down)
    lib.ncmb_set_rng_mode(plan["rng_mode"])
    lib.ncmb_set_row_offset(plan["row_offset"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_device(seed):
        """ids already resident: plan + upload outside the timed events, all device work inside."""
        g = lib.ncp_gen_begin(model.ncp, None, prefix.data_ptr(), B, kw["temp"], kw["top_k"], kw["top_p"], kw["cfg"],
                              kw["freq"], kw["mu"], 0.0, 0, 1.0, allow_p, seed)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        marks = [e0]                                   # one event per stepper step (a level): the step latencies
        e0.record(stream)
        while lib.ncp_gen_step(g, None, None) == 0:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            marks.append(ev)
        lib.ncmb_decode_tokens_dev(model.vqvae, lib.ncmb_gen_codes_dev(g), B, tokens_dev.data_ptr())
        e1.record(stream)
        level_marks.append(marks)
        return g, e0, e1

    level_marks = []

    def step_e2e(seed):
        """host prefix ids in, host token ids out, through the public C API."""
        out = lib.ncp_generate(model.ncp, None, prefix.data_ptr(), B, kw["temp"], kw["top_k"], kw["top_p"], kw["cfg"],
                               kw["freq"], kw["mu"], 0.0, 0, 1.0, allow_p, seed)
        lib.ncmb_decode_tokens(model.vqvae, out, B, tokens_host.data_ptr())
        capi._libc.free(out)

    for i in range(args.warmup):
        g, _, _ = step_device(100 + i)
        torch.cuda.synchronize()
        lib.ncp_gen_abort(g)
        step_e2e(100 + i)

    # ---- device-timed steps (value): the library's per-kernel event timers are OFF here -- two extra event
    # records around each of ~2800 launches cost about 4% of a step ----
    n0 = lib.ncmb_launch_count()
    barrier()
    dev_ms = 0.0
    with ClockSampler(local) as clk:
        t_wall0 = time.perf_counter()
        for i in range(args.steps):
            g, e0, e1 = step_device(200 + i)
            e1.synchronize()
            dev_ms += e0.elapsed_time(e1)
            lib.ncp_gen_abort(g)
        barrier()
        t_wall = time.perf_counter() - t_wall0
    launches = lib.ncmb_launch_count() - n0
    # latency of a stepper step (the prefix pass + level 0, then one refinement level each) over the timed steps
    lvl_ms = [[a.elapsed_time(b) for a, b in zip(mk[:-1], mk[1:])] for mk in level_marks[-args.steps:]]
    flat = sorted(x for row in lvl_ms for x in row)
    p50_level = flat[len(flat) // 2] if flat else None
    by_level = [float(np.median([row[i] for row in lvl_ms])) for i in range(len(lvl_ms[0]))] if lvl_ms else []
    # ---- the same steps again with the per-kernel timers on: kernel classes and the roofline's launch times ----
    lib.ncmb_prof_reset()
    lib.ncmb_prof_enable(1)
    prof_ms = 0.0
    for i in range(args.steps):
        g, e0, e1 = step_device(200 + i)
        e1.synchronize()
        prof_ms += e0.elapsed_time(e1)
        lib.ncp_gen_abort(g)
    barrier()
    lib.ncmb_prof_enable(0)
    top = None
    tn, tms, tfl, tby = C.c_longlong(), C.c_double(), C.c_double(), C.c_double()
    if lib.ncmb_prof_top_shape(0, C.byref(tn), C.byref(tms), C.byref(tfl), C.byref(tby)) == 0 and tn.value > 0:
        top = {"launches": tn.value, "ms": tms.value, "flops": tfl.value, "bytes": tby.value}
    if os.environ.get("NCM_B200_PROF_SHAPES") and rank == 0:
        lib.ncmb_prof_dump_shapes()          # per-call-shape table on stderr (diagnostic)
    prof = {}
    for name, k in (("gemm", 0), ("attention", 1), ("norm", 2), ("sampling", 3), ("elementwise", 4), ("quantizer", 5)):
        n, ms, fl, by = C.c_longlong(), C.c_double(), C.c_double(), C.c_double()
        lib.ncmb_prof_read(k, C.byref(n), C.byref(ms), C.byref(fl), C.byref(by))
        prof[name] = {"launches": n.value, "ms": ms.value, "flops": fl.value, "bytes": by.value}

    # ---- end-to-end steps through the host API ----
    h0, d0 = C.c_ulonglong(), C.c_ulonglong()
    lib.ncmb_copy_bytes(C.byref(h0), C.byref(d0))
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step_e2e(300 + i)
    barrier()
    e2e_s = time.perf_counter() - t0
    h1, d1 = C.c_ulonglong(), C.c_ulonglong()
    lib.ncmb_copy_bytes(C.byref(h1), C.byref(d1))

    dev_s, e2e_max, _ = max_over_ranks([dev_ms / 1000.0, e2e_s, t_wall], device="cuda")
    # checksum of the token ids of the last end-to-end step, one per rank
    sums = torch.zeros(world, dtype=torch.int64, device="cuda")
    sums[rank] = token_checksum(tokens_host.numpy())
    if world > 1:
        dist.all_reduce(sums)
    checksums = [int(v) for v in sums.tolist()]
    if rank == 0:
        peaks = {}
        pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(pk):
            peaks = json.load(open(pk))
        peak_tf = peaks.get("bf16_tflops_sustained", 1400.0)
        gm = prof["gemm"]
        ach_class = gm["flops"] / (gm["ms"] * 1e-3) / 1e12 if gm["ms"] > 0 else 0.0
        # roofline of the dominant kernel: the GEMM call shape with the largest total time in the timed steps
        roof_kernel, ach, traffic, roof_ms, roof_n = "gemm (all linear layers)", ach_class, None, gm["ms"] / max(gm["launches"], 1), gm["launches"]
        if top:
            roof_ms, roof_n = top["ms"] / top["launches"], top["launches"]
            ach = top["flops"] / (roof_ms * 1e-3) / 1e12
            roof_kernel, traffic = describe_gemm_shape(spec, top["flops"])
        total_tok = world * B * tok * args.steps
        mode = lib.ncmb_get_gemm_mode()
        line = {
            "metric": "generated tokens/sec", "value": total_tok / dev_s, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * dev_s / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": {0: "f32", 1: "tf32 (fp32 accumulate)", 2: "3xtf32 (fp32 accumulate)",
                      3: "f16 pairs x3 (fp32-grade operands, fp32 accumulate)"}.get(mode, "f32"),
            "data": "synthetic",
            "config": workload_config(args.workload, spec, B, world),
            "codes_per_sec": world * B * sum(spec.levels) * args.steps / dev_s,
            # step = one call of the level stepper: the prefix pass with level 0, then one refinement level each
            "p50_step_latency_ms": p50_level, "step_latency_ms_by_level": by_level,
            "e2e": {"value": total_tok / e2e_max, "unit": "tokens/s",
                    "h2d_bytes_per_step": (h1.value - h0.value) // args.steps,
                    "d2h_bytes_per_step": (d1.value - d0.value) // args.steps},
            "gpu_launches": launches,
            "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "kernel": roof_kernel, "achieved": ach, "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": ach / peak_tf if peak_tf else None, "traffic": traffic,
                         "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained" if peaks else "fallback",
                         "launches": roof_n, "avg_launch_ms": roof_ms,
                         "mma_passes": 3 if mode >= 2 else 1,
                         "note": "achieved counts algorithmic flops (2MNK); fp32-grade operands cost 3 tensor-core "
                                 "MMAs per algorithmic MMA, so the tensor pipe runs at mma_passes x achieved",
                         "all_gemm_launches": {"achieved": ach_class, "launches": gm["launches"],
                                               "ms_per_step": gm["ms"] / args.steps}},
            "algorithmic_tflop_per_step": algorithmic_flops_per_row(spec) * B * (2 if kw["cfg"] > 0 else 1) / 1e12,
            "kernel_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items()},
            "profiled_ms_per_step": prof_ms / args.steps,
        }
        line["rng"] = "counter-based, keyed by (seed, global sequence index, level, position)"
        line["token_checksums"] = checksums
        if world == 1 and not args.no_cpu_baseline:
            got = {}
            kind, cores, times = cpu_sample_run(spec, conf, w, args.cpu_rows, 1, 0, 7, keep=got)
            line["cpu_baseline"] = {
                "value": args.cpu_rows * tok / times[0], "unit": "tokens/s", "cores": cores, "kind": kind,
                "sample": f"{args.cpu_rows} of the {B} sequences, one pass (reference cost is linear in sequences)"}
            # result check: the same prefixes and seed through the library, on the reference's own sampling stream
            lib.ncmb_set_rng_mode(0)
            lib.ncmb_set_row_offset(0)
            codes = model.generate(got["prefix"], seed=got["seed"], **kw)
            toks = model.decode_tokens(codes, spec.L)
            lib.ncmb_set_rng_mode(plan["rng_mode"])
            line["parity_check"] = {
                "rows": int(codes.shape[0]), "against": kind,
                "codes_equal": bool(np.array_equal(codes, got["codes"])),
                "tokens_equal": bool(np.array_equal(toks, got["tokens"])),
                "codes_differing": int((codes != got["codes"]).sum()), "codes_total": int(codes.size),
                "tensor_core_timeouts": int(lib.ncmb_gemm_tc_check())}
        if world == 1 and args.workload == "c2" and not args.no_workloads:
            line["workloads"] = other_workloads(lib, args)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    tmp.cleanup()


def describe_gemm_shape(spec, flops):
    """Names the transformer GEMM whose 2*M*N*K equals `flops` and, for the gated up-projection, scales the
    DRAM traffic of one captured launch of that kernel (dram bytes read + written: 293.3 MB at M=32896, N=4096,
    K=512, i.e. 8916 bytes per token row; input and output bytes are per row and the 8 MB weight pair is read
    once, so traffic is proportional to M at fixed N, K)."""
    C_ = spec.n_embd
    Hh = spec.mlp_hidden if spec.mlp_hidden else 4 * C_
    kvd = (spec.n_kv_heads or spec.n_head) * (C_ // spec.n_head)
    gated = bool(spec.mlp_hidden)
    shapes = [("MLP up-projection" + (" with fused gated SiLU, fp16-pair output" if gated else ""), (2 * Hh if gated else Hh), C_),
              ("MLP down-projection + residual", C_, Hh), ("QKV projection", C_ + 2 * kvd, C_),
              ("attention output projection + residual", C_, C_)]
    for name, N, K in shapes:
        M = flops / (2.0 * N * K)
        if abs(M - round(M)) < 1e-6 and M >= 1:
            traffic = None
            if gated and name.startswith("MLP up") and (N, K) == (4096, 512):
                traffic = 8916.0 * round(M)
            return f"k_gemm_h3: {name}, M={int(round(M))} N={N} K={K}", traffic
    return "k_gemm_h3 (largest GEMM call shape)", None


# --------------------------------------------------------------------------- decoder LMs / quantizer sweep

def lm_workload(name):
    if name == "c3":
        return synth.spec_gpt2_124m(), dict(prompt=128, n_new=256, temp=0.0, top_k=0, top_p=1.0, batch=1)
    if name == "c4":
        return synth.spec_qwen_05b(), dict(prompt=512, n_new=512, temp=0.7, top_k=0, top_p=0.95, batch=1)
    if name == "c3t":
        return synth.spec_gpt2_tiny(), dict(prompt=9, n_new=12, temp=0.0, top_k=0, top_p=1.0, batch=2)
    raise SystemExit(f"unknown workload {name}")


def _peaks():
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return json.load(open(pk)) if os.path.exists(pk) else {}


# Dense TF32 throughput of one B200 of this pool: torch.matmul on 8192^3 fp32 operands with TF32 allowed, best of
# 10, measured once with a scratch script in the way the bf16 figure of MEASURED_PEAKS.json is measured (that file
# has no TF32 entry). Used as the denominator of the quantizer sweep, whose distance GEMM runs on the TF32 pipe.
TF32_PEAK_TFLOPS_MEASURED = 752.7      # burst; 611.5 in a 4-second loop under the power cap


def tf32_peak():
    p = _peaks()
    if "tf32_tflops" in p:
        return p["tf32_tflops"], "MEASURED_PEAKS.json tf32_tflops"
    if TF32_PEAK_TFLOPS_MEASURED:
        return TF32_PEAK_TFLOPS_MEASURED, "torch.matmul TF32 8192^3 on this pool (builder-measured)"
    return p.get("bf16_tflops", 1590.0) / 2.0, "half of the measured bf16 burst peak (no TF32 measurement)"


def lm_bytes_per_step(spec, B, mean_ctx):
    """Algorithmic bytes of one decode step: every parameter once plus the K/V cache of B sequences at the mean
    context, at the storage width the configuration states (fp32 for the GPT-2 shape; 2-byte weights and 2-byte
    K/V for the bf16 Qwen2 shape)."""
    C_, hd = spec.n_embd, spec.n_embd // spec.n_head
    kvd = spec.n_kv_heads * hd
    per_layer = C_ * (C_ + 2 * kvd) + C_ * C_ + (3 if spec.kind == "qwen" else 2) * C_ * spec.n_inner
    params = spec.n_layer * per_layer + spec.vocab * C_
    width = 2.0 if spec.bf16_round else 4.0
    return width * params + B * spec.n_layer * 2 * kvd * width * mean_ctx


def measure_lm(lib, stream, name, batches, steps, warmup, local, n_new=0):
    """GPT-2 / Qwen2 shaped decoding with a KV cache, one line per batch size: tokens/s (prefill included) and
    achieved HBM GB/s per decode step. The model is opened once for all batch sizes."""
    import torch
    spec, w = lm_workload(name)
    if n_new > 0:
        w = dict(w, n_new=n_new)                               # shorter generations: profiler captures of a few decode steps
    tmp = tempfile.TemporaryDirectory()
    conf, wt = synth.write_lm(spec, tmp.name)
    cfg = lib.load_config(conf)
    m = lib.ncmb_lm_open(cfg, wt.encode(), int(spec.kind == "qwen"), int(spec.bf16_round))
    os.remove(wt)                                              # up to 2 GB; the model holds its own copy
    peak = _peaks().get("hbm_gbs", 6650.0)
    lines = []
    for B in batches:
        prompts = np.ascontiguousarray(synth.lm_prompts(spec, B, w["prompt"], 5))
        out = np.zeros((B, w["n_new"]), np.int32)

        def step(seed):
            lib.ncmb_lm_generate(m, prompts.ctypes.data, B, w["prompt"], w["n_new"], w["temp"], w["top_k"], w["top_p"],
                                 seed, -1, out.ctypes.data)

        for i in range(warmup):
            step(1 + i)
        n0 = lib.ncmb_launch_count()
        torch.cuda.synchronize()
        with ClockSampler(local) as clk:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record(stream)
            for i in range(steps):
                step(100 + i)
            e1.record(stream)
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
        dev_s = e0.elapsed_time(e1) / 1000.0
        launches = lib.ncmb_launch_count() - n0
        bytes_step = lm_bytes_per_step(spec, B, w["prompt"] + w["n_new"] / 2.0)
        steps_total = steps * w["n_new"]
        ach = bytes_step * steps_total / dev_s / 1e9
        lines.append({
            "metric": "generated tokens/sec", "value": B * steps_total / dev_s, "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": 1000.0 * dev_s / steps,
            "token_latency_ms": 1000.0 * dev_s / steps_total, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (2-byte weight copies streamed by the decode steps)" if spec.bf16_round else "f32",
            "data": "synthetic",
            "config": {"workload": f"{name}: {spec.kind} {spec.n_layer}x{spec.n_embd}, vocab {spec.vocab}, prompt {w['prompt']}, "
                                   f"+{w['n_new']} tokens, batch {B}, temp {w['temp']}, top-p {w['top_p']}; KV-cached decode incl. prefill"},
            "e2e": {"value": B * steps_total / wall, "unit": "tokens/s", "h2d_bytes_per_step": int(prompts.nbytes),
                    "d2h_bytes_per_step": int(out.nbytes)},
            "gpu_launches": launches, "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "kernel": "decode step (weights + KV cache streamed once per token)", "achieved": ach,
                         "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "algorithmic_bytes_per_step": bytes_step,
                         "note": "token latency here is the mean over the run (prefill included); bytes per step count "
                                 + ("2 B per parameter and 2 B per cached K/V element" if spec.bf16_round else "4 B per parameter and per cached K/V element")},
        })
    assert lib.ncmb_gemm_tc_check() == 0
    lib.ncmb_lm_close(m)
    tmp.cleanup()
    return lines


def _lm_setup(args):
    import torch
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    lib = capi.NcmLib(os.path.join(ROOT, "saphira-cncm_b200", "libncm_b200.so"))
    if args.gemm is not None:
        lib.ncmb_set_gemm_mode(args.gemm)
    stream = torch.cuda.current_stream()
    lib.ncmb_set_stream(C.c_void_p(stream.cuda_stream))
    return lib, stream, local


def run_lm_arm(args):
    lib, stream, local = _lm_setup(args)
    _, w = lm_workload(args.workload)
    for line in measure_lm(lib, stream, args.workload, [args.batch or w["batch"]], args.steps, args.warmup, local, args.n_new):
        print(json.dumps(line), flush=True)


def measure_quantizer(lib, stream, n, steps, warmup):
    """Flat nearest-code search: N(0,1) 64-d vectors against a 16384 x 64 codebook (config-5 sweep)."""
    import torch
    spec = synth.spec_c2(n_layer=1, vocab=16384, name="c5q")
    tmp = tempfile.TemporaryDirectory()
    conf, wt = synth.write_ncp(spec, tmp.name)
    model = capi.NcpModel(lib, conf, wt, arena_mb=64)
    x = torch.randn((n, 64), device="cuda", dtype=torch.float32, generator=torch.Generator(device="cuda").manual_seed(3))
    idx = torch.empty((n,), device="cuda", dtype=torch.int32)
    for _ in range(warmup):
        lib.ncmb_vq_nearest_dev(model.vq, 3, x.data_ptr(), n, idx.data_ptr())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        lib.ncmb_vq_nearest_dev(model.vq, 3, x.data_ptr(), n, idx.data_ptr())
    e1.record(stream)
    torch.cuda.synchronize()
    dev_s = e0.elapsed_time(e1) / 1000.0 / steps
    flops = 2.0 * n * 16384 * 64
    peak, src = tf32_peak()
    line = {"metric": "quantized vectors/sec", "value": n / dev_s, "unit": "vectors/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": 1000 * dev_s, "higher_is_better": True,
            "dtype": "3xtf32 (fp32-grade distances)", "data": "synthetic",
            "config": {"workload": f"c5q: {n} fp32 N(0,1) 64-d vectors vs 16384 x 64 codebook, nearest code"},
            "roofline": {"bound": "tensor", "achieved": flops / dev_s / 1e12, "peak": peak, "unit": "TFLOP/s",
                         "frac": flops / dev_s / 1e12 / peak, "traffic": None, "peak_source": src, "mma_passes": 3}}
    lib.ncp_free(model.ncp)
    lib.vqvae_free(model.vqvae)
    lib.weights_free(C.byref(model.ws))
    tmp.cleanup()
    return line


def run_quantizer_arm(args):
    lib, stream, _ = _lm_setup(args)
    print(json.dumps(measure_quantizer(lib, stream, args.batch or (1 << 20), args.steps, args.warmup)), flush=True)


def measure_ncp_brief(lib, stream, name, B, steps, warmup, local):
    """A short device-timed run of another NCP configuration (ids resident, stepper + device decode): throughput,
    level latencies and the algorithmic tensor-core fraction of the whole step."""
    import torch
    spec, B0 = workload(name)
    B = B or B0
    kw = gen_kwargs(spec)
    tmp = tempfile.TemporaryDirectory()
    conf, w = synth.write_ncp(spec, tmp.name)
    model = capi.NcpModel(lib, conf, w, arena_mb=64)
    os.remove(w)
    prefix = torch.from_numpy(synth.ncp_prefixes(spec, B, 1000)).pin_memory()
    tokens_dev = torch.empty((B, spec.L), dtype=torch.int32, device="cuda")
    allow = kw.get("allow")
    allow_p = allow.ctypes.data if allow is not None else None
    lat, total_ms = [], 0.0

    def step(seed, timed):
        nonlocal total_ms
        g = lib.ncp_gen_begin(model.ncp, None, prefix.data_ptr(), B, kw["temp"], kw["top_k"], kw["top_p"], kw["cfg"],
                              kw["freq"], kw["mu"], 0.0, 0, 1.0, allow_p, seed)
        marks = [torch.cuda.Event(enable_timing=True)]
        marks[0].record(stream)
        while lib.ncp_gen_step(g, None, None) == 0:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            marks.append(ev)
        lib.ncmb_decode_tokens_dev(model.vqvae, lib.ncmb_gen_codes_dev(g), B, tokens_dev.data_ptr())
        end = torch.cuda.Event(enable_timing=True)
        end.record(stream)
        end.synchronize()
        lib.ncp_gen_abort(g)
        if timed:
            total_ms += marks[0].elapsed_time(end)
            lat.extend(a.elapsed_time(b) for a, b in zip(marks[:-1], marks[1:]))

    for i in range(warmup):
        step(100 + i, False)
    n0 = lib.ncmb_launch_count()
    with ClockSampler(local) as clk:
        for i in range(steps):
            step(200 + i, True)
    launches = lib.ncmb_launch_count() - n0
    tok = NOMINAL_TOKENS[name]
    flop = algorithmic_flops_per_row(spec) * B * (2 if kw["cfg"] > 0 else 1)
    peak = _peaks().get("bf16_tflops_sustained", 1400.0)
    ach = flop * steps / (total_ms * 1e-3) / 1e12
    line = {"metric": "generated tokens/sec", "value": B * tok * steps / (total_ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": total_ms / steps,
            "p50_step_latency_ms": sorted(lat)[len(lat) // 2], "higher_is_better": True, "scaling": "weak",
            "dtype": "f16 pairs x3 (fp32-grade operands, fp32 accumulate)", "data": "synthetic",
            "config": workload_config(name, spec, B, 1), "gpu_launches": launches, "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "kernel": "whole step (all kernels)", "achieved": ach, "peak": peak,
                         "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                         "algorithmic_tflop_per_step": flop / 1e12,
                         "note": "algorithmic flops of the step (prefix once per model row) over the device time of "
                                 "the whole step, not of one kernel"}}
    assert lib.ncmb_gemm_tc_check() == 0
    lib.ncp_free(model.ncp)
    lib.vqvae_free(model.vqvae)
    lib.weights_free(C.byref(model.ws))
    tmp.cleanup()
    return line


def other_workloads(lib, args):
    """Short runs of the other stated configurations on the same GPU, appended to the default 1-GPU line: the small
    NCP (c1), the GPT-2 shape at batch 1 / 64 (c3), the Qwen2 shape at batch 1 / 32 / 256 (c4), the box-scale NCP on
    1 024 sequences (c5) and the 2^20-vector quantizer sweep (c5q). Config 2 stays the headline."""
    import torch
    stream = torch.cuda.current_stream()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    lib.ncmb_set_rng_mode(1)
    lib.ncmb_set_row_offset(0)
    out = {}
    t0 = time.perf_counter()
    out["c1"] = measure_ncp_brief(lib, stream, "c1", 64, 5, 3, local)
    for ln, B in zip(measure_lm(lib, stream, "c3", [1, 64], 2, 1, local), (1, 64)):
        out[f"c3_b{B}"] = ln
    for ln, B in zip(measure_lm(lib, stream, "c4", [1, 32, 256], 1, 1, local), (1, 32, 256)):
        out[f"c4_b{B}"] = ln
    out["c5_1024seq"] = measure_ncp_brief(lib, stream, "c5", 1024, 1, 1, local)
    out["c5q"] = measure_quantizer(lib, stream, 1 << 20, 5, 3)
    out["seconds"] = time.perf_counter() - t0
    return out


def run_box_arm(args):
    """Config 5 at its stated size: 65 536 independent sequences (strong scaling: the total is fixed and split over
    the ranks), each rank calling ncp_generate + ncmb_decode_tokens through the host API. A rank's share does not fit
    the GPU in one pass; the library runs it as waves of rows. Timed with the wall clock around the calls (each wave
    ends in a device-to-host copy, so wall time is device time plus the host's part), max over ranks."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = capi.NcmLib(os.path.join(ROOT, "saphira-cncm_b200", "libncm_b200.so"))
    stream = torch.cuda.current_stream()
    lib.ncmb_set_stream(C.c_void_p(stream.cuda_stream))
    spec, _ = workload("c5")
    total = args.batch or 65536
    B = total // world
    kw = gen_kwargs(spec)
    tmp = tempfile.TemporaryDirectory()
    conf, w = synth.write_ncp(spec, tmp.name)
    model = capi.NcpModel(lib, conf, w, arena_mb=64)
    os.remove(w)
    prefix = synth.ncp_prefixes(spec, B, 1000 + rank)
    lib.ncmb_set_rng_mode(1)
    lib.ncmb_set_row_offset(rank * B)
    allow = kw.get("allow")
    warm = synth.ncp_prefixes(spec, 64, 5)
    model.decode_tokens(model.generate(warm, seed=1, **kw), spec.L)          # kernels loaded, weights converted
    tokens = np.zeros((B, spec.L), np.int32)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    n0 = lib.ncmb_launch_count()
    with ClockSampler(local) as clk:
        t0 = time.perf_counter()
        codes = model.generate(prefix, seed=7, **kw)
        for r0 in range(0, B, 4096):
            tokens[r0:r0 + 4096] = model.decode_tokens(codes[r0:r0 + 4096], spec.L)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    launches = lib.ncmb_launch_count() - n0
    (dt_max,) = max_over_ranks([dt], device="cuda")
    sums = torch.zeros(world, dtype=torch.int64, device="cuda")
    sums[rank] = token_checksum(tokens)
    if world > 1:
        dist.all_reduce(sums)
    if rank == 0:
        flop = algorithmic_flops_per_row(spec) * total * 2
        peak = _peaks().get("bf16_tflops_sustained", 1400.0) * world
        ach = flop / dt_max / 1e12
        print(json.dumps({
            "metric": "generated tokens/sec", "value": total * NOMINAL_TOKENS["c5"] / dt_max, "unit": "tokens/s",
            "n_gpus": world, "steps": 1, "warmup": 0, "ms_per_step": 1000.0 * dt_max, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 pairs x3 (fp32-grade operands, fp32 accumulate)",
            "data": "synthetic", "config": workload_config("c5", spec, B, world),
            "e2e": {"value": total * NOMINAL_TOKENS["c5"] / dt_max, "unit": "tokens/s",
                    "h2d_bytes_per_step": int(prefix.nbytes), "d2h_bytes_per_step": int(codes.nbytes + tokens.nbytes)},
            "gpu_launches": launches, "clocks": clk.summary(), "token_checksums": [int(v) for v in sums.tolist()],
            "tensor_core_timeouts": int(lib.ncmb_gemm_tc_check()),
            "roofline": {"bound": "tensor", "kernel": "whole job (all kernels, all waves)", "achieved": ach, "peak": peak,
                         "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                         "algorithmic_tflop": flop / 1e12}}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    tmp.cleanup()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (default: the workload's)")
    ap.add_argument("--gemm", type=int, default=None, help="GEMM engine override (0 fp32, 1 tf32, 2 3xtf32, 3 fp16 pairs)")
    ap.add_argument("--cpu-rows", type=int, default=1, help="sequences in the CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--n-new", type=int, default=0, help="decoder-LM workloads: tokens to generate (default: the configuration's)")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the short runs of the other configurations that the default 1-GPU run appends")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours" and args.workload == "c2":
        args.warmup = 3
    if args.workload in ("c3", "c4", "c3t"):
        run_lm_arm(args)
    elif args.workload == "c5q":
        run_quantizer_arm(args)
    elif args.workload == "c5box":
        run_box_arm(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
