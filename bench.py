#!/usr/bin/env python
"""Benchmark of the packed ragged step on B200.

Workload (N = 1): the 27B-shape 4-bit model, 8 decoding sessions with seeded contexts of
36K-42K tokens, each verifying an 8-token draft block: one 64-row packed step, KV cache int8,
all rows accepted after each step as the reference's context benchmark does
(Sources/SploshCLI/GenerateCommand.swift:375-469). Weights are seeded synthetic (quantised
N(0, 0.02) stand-ins), KV pages hold pseudo-random codes with scale 0.01 and the recurrent state
U(-0.5, 0.5), as the reference's Engine.debugFillKV and its tests fill them.

With --gpus N each rank runs the same 8-session workload on its own GPU (sessions shard across
GPUs with weights replicated and no collective on the data path): weak scaling.

`--impl reference` times the CPU restatement of the step (oracle/) on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SESSIONS, BLOCK = 8, 8
CONTEXT_LOW, CONTEXT_HIGH = 36 * 1024, 42 * 1024
PREFILL_PROMPT, PREFILL_CHUNK = 54500, 2048        # BASELINE configuration 2: one 54.5K-token prompt in 2,048-row chunks
RIDER_PROMPT, RIDER_ROWS = 21000, 64               # configuration 3's prefilling session: 64 prompt rows ride in every 64-row decode step
GGUF_CONTEXT, GGUF_BLOCK = 171000, 16              # configuration 4: one session at 171K context verifying 16-token blocks on GGUF weights
# DRAM bytes the GEMM kernel moves per algorithmic byte: measured per tensor shape with ncu (reads + writes), 15.06 GB
# for the 14.41 GB of a full step's 257 launches.
GEMM_DRAM_PER_ALGORITHMIC_BYTE = 1.044
SPAN_TARGET = 608      # scan blocks per step the table builder aims for (engine configuration)
WEIGHT_SEED, TOKEN_SEED = 0x5EED6D17, 0xC0FFEE00


def splitmix_at(seed, n):
    mask = (1 << 64) - 1
    z = (seed + (n + 1) * 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    return z ^ (z >> 31)


def contexts(rank):
    return [CONTEXT_LOW + splitmix_at(TOKEN_SEED + rank, s) % (CONTEXT_HIGH - CONTEXT_LOW) for s in range(SESSIONS)]


def weights_per_step(g):
    """Weights streamed by one step (every block plus the head), and their bytes at 0.5625 B/weight."""
    H, I = g.hidden, g.inter
    C = (2 * g.gdn_key_heads + g.gdn_value_heads) * g.gdn_head_dim
    VD, VH = g.gdn_value_heads * g.gdn_head_dim, g.gdn_value_heads
    AD, KV = g.heads * g.head_dim, g.kv_heads * g.head_dim
    mlp = 3 * H * I
    linear = (C + VD + 2 * VH) * H + H * VD + mlp
    full = (2 * AD + 2 * KV) * H + H * AD + mlp
    n_full = g.layers // 4
    total = (g.layers - n_full) * linear + n_full * full + g.vocab * H
    return total, total * 0.5625


def algorithmic_bytes(g, ctx, rows_per_session):
    """HBM bytes one decode step must move: weights once, each session's KV once, its recurrent state in and out."""
    _, wbytes = weights_per_step(g)
    n_full = g.layers // 4
    kv_per_token = n_full * 2 * g.kv_heads * (g.head_dim + 4)
    kv = sum(ctx) * kv_per_token
    state = len(ctx) * (g.layers - n_full) * g.gdn_value_heads * 128 * 128 * 4 * 2
    return wbytes + kv + state, dict(weights=wbytes, kv=kv, state=state)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], False
        self.max_mhz = None

    def run(self):
        query = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
                "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={query}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                self.samples.append([f.strip() for f in out])
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        ok = [s for s in self.samples if len(s) == 6 and s[0].isdigit()]
        if not ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in ok)]
        return {"sm_mhz": float(np.median([int(s[0]) for s in ok])), "sm_max_mhz": float(ok[0][1]), "reasons": reasons}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, an earlier measurement on this pool)"


class CpuSample:
    """The oracle on a bounded sample of the same step: `layers` blocks of the 27B shape (3 gated-delta + 1 attention per 4)
    and a head of `vocab` columns, 64 rows at `context` tokens of synthetic KV; extrapolated to 64 blocks and the full head."""

    def __init__(self, rows_per_session=BLOCK, sessions=SESSIONS, layers=4, vocab=32768):
        from oracle import oracle as O
        from oracle import tables as T
        self.O, self.T = O, T
        self.sessions, self.block, self.layers, self.vocab = sessions, rows_per_session, layers, vocab
        ctx = contexts(0)[:sessions]              # the benchmark's own contexts: the attention block sees what the GPU arm sees
        g = O.b27_geometry().with_(layers=layers, vocab=vocab)
        self.model = O.Model(g, WEIGHT_SEED)
        pages = sum(c // 256 + 4 for c in ctx)
        self.host = T.Host(max_slots=sessions, max_rows=sessions * rows_per_session, kv_pages=pages, max_context=max(ctx) + 1024,
                           vocab=vocab, kv_heads=g.kv_heads, last_layer_full=True)
        self.engine = O.Engine(self.model, sessions, pages, self.host.max_pages, self.host.state_units)
        # Allocate each slot's pages with a throwaway row at the end of its context, then fill KV and state.
        tb = self.host.build([T.Row(s, 1000, ctx[s] - 1, False) for s in range(sessions)])
        self.engine.step(tb); self.host.finish_step(tb)
        rng = np.random.default_rng(1)
        for index in range(layers // 4):
            for which in ("k_codes", "v_codes"):
                buf = self.engine.buffer(which, index); buf[:] = rng.integers(-127, 128, buf.size, dtype=np.int8)
            for which in ("k_scale", "v_scale"):
                self.engine.buffer(which, index)[:] = 0.01
        for index in range(layers - layers // 4):
            st = self.engine.buffer("state", index); st[:] = rng.uniform(-0.5, 0.5, st.size).astype(np.float32)
        self.position = list(ctx)
        self.cores = O.lib().orc_threads()
        self.sample = (f"{layers} blocks (3 gated-delta : 1 attention) of the 27B shape + a {vocab}-column head, {sessions * rows_per_session} rows, "
                       f"{sessions} sessions at the benchmark's contexts ({min(ctx)}-{max(ctx)} tokens of synthetic KV); time = blocks x{64 / layers:g} + head x{248320 / vocab:.2f}")

    def step(self):
        """One 64-row verify step; returns the extrapolated seconds of a full 64-block step."""
        T = self.T
        rows = [T.Row(s, int(splitmix_at(TOKEN_SEED, s * 100 + i + self.position[s]) % self.vocab), self.position[s] + i, True, True)
                for s in range(self.sessions) for i in range(self.block)]
        tb = self.host.build(rows)
        t0 = time.perf_counter(); self.engine.step(tb, max_layers=self.layers); t_blocks = time.perf_counter() - t0
        self.host.finish_step(tb)
        for s in range(self.sessions):
            self.position[s] += self.block
            self.host.accept_verify(s, self.block, self.position[s])
        # The head on the same rows: final norm + head GEMM = a step of zero blocks is not expressible, so time it as a bare GEMM.
        packed, scales, biases = self.model.q4(-1, "head")
        a = np.zeros((self.sessions * self.block, 5120), np.float32) + 0.5
        t0 = time.perf_counter(); self.O.gemm_q4(packed, scales, biases, a); t_head = time.perf_counter() - t0
        return t_blocks * (64 / self.layers) + t_head * (248320 / self.vocab)


def cpu_baseline(steps=1):
    sample = CpuSample()
    seconds = float(np.mean([sample.step() for _ in range(steps)]))
    return SESSIONS * BLOCK / seconds, sample.cores, sample.sample


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the step on all host threads, rank 0 only."""
    if rank != 0:
        return
    # A launcher that starts one process per GPU sets OMP_NUM_THREADS=1 for its workers; this arm is a CPU job and takes
    # every host core (the OpenMP runtime reads the variable when the oracle's library loads, below).
    if os.environ.get("OMP_NUM_THREADS") == "1" and ("TORCHELASTIC_RUN_ID" in os.environ or "LOCAL_RANK" in os.environ):
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    sample = CpuSample()
    for _ in range(max(args.warmup, 0)):
        sample.step()
    t0 = time.perf_counter()
    seconds = [sample.step() for _ in range(args.steps)]
    value = SESSIONS * BLOCK / float(np.mean(seconds))
    line = {"metric": "packed_step_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * float(np.mean(seconds)), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 x int4 -> fp32 (int8 KV, fp32 state)", "data": "synthetic", "impl": "reference",
            "config": {"workload": "27B-shape MLX 4-bit g64, 8 sessions x 8-row verify blocks = 64 rows per step (bounded sample, extrapolated)",
                       "parallelism": "host cores", "sample_wall_seconds": time.perf_counter() - t0},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": sample.cores, "kind": "port", "sample": sample.sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="splosh_b200")
    ap.add_argument("--layers", type=int, default=64, help="blocks of the 27B shape (64 is the benchmark; fewer for ncu captures)")
    ap.add_argument("--context-scale", type=float, default=1.0, help="scales the session contexts (1.0 is the benchmark)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-draft", action="store_true", help="leave out the drafter's measurement")
    ap.add_argument("--no-prefill", action="store_true", help="leave out the prefill, rider, strong-scaling and GGUF measurements that follow the timed region")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    args.warmup = max(args.warmup, 3)

    import torch
    import splosh_b200 as S
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)

    g = S.b27_geometry(layers=args.layers)
    ctx = [int(c * args.context_scale) for c in contexts(rank)]
    steps_total = args.warmup + 4 * args.steps + 8
    extras = not args.no_prefill
    prompt_tokens = int(PREFILL_PROMPT * args.context_scale)
    rider_prompt = int(RIDER_PROMPT * args.context_scale)
    gguf_context = int(GGUF_CONTEXT * args.context_scale)
    pages = sum((c + BLOCK * steps_total) // 256 + 2 for c in ctx) + (prompt_tokens // 256 + 4 if extras else 0)
    # The engine's span target (how many scan blocks a step should make; the reference tunes it to its GPU, 592 there): one
    # scan block fills an SM here; 608 gives this workload 19 spans of 9 pages, which packs the 148 SMs best.
    cfg = S.EngineConfig(max_slots=SESSIONS + 1, max_rows=max(SESSIONS * BLOCK + RIDER_ROWS, PREFILL_CHUNK) if extras else SESSIONS * BLOCK, kv_pages=pages,
                         max_context=max(max(ctx) + BLOCK * steps_total, (prompt_tokens if extras else 0), (gguf_context + GGUF_BLOCK * (args.steps + 4) if extras else 0)) + 256, device=local, span_target=SPAN_TARGET,
                         max_logit_rows=SESSIONS * BLOCK + 8)
    engine = S.Engine(g, cfg)
    from splosh_b200 import synthetic
    synthetic.load_vectors(engine, WEIGHT_SEED)
    engine.synthesize_q4(WEIGHT_SEED)

    # Contexts: one throwaway row at the end of each allocates its pages; then KV and state are filled.
    engine.step([S.EngineRow(s, 1000, ctx[s] - 1, False) for s in range(SESSIONS)])
    for s in range(SESSIONS):
        engine.debug_fill_kv(s)
        engine.debug_fill_state(s, 0x5747 + s)
    position = list(ctx)

    def rows_for(step):
        return [S.EngineRow(s, int(splitmix_at(TOKEN_SEED + rank, 1000003 * step + 97 * s + i) % g.vocab), position[s] + i, True, True)
                for s in range(SESSIONS) for i in range(BLOCK)]

    def one_step(step, read_ids):
        stats = engine.step(rows_for(step))
        ids = engine.argmax(248077 if g.vocab == 248320 else g.vocab) if read_ids else None
        for s in range(SESSIONS):
            position[s] += BLOCK
            engine.accept_verify(s, BLOCK, position[s])
        return stats, ids

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # Every rank first runs the same seeded session (slot 8 is free of the timed work): the token ids it decodes have to be
    # rank 0's, or the replicas are not replicas.
    if dist is not None:
        probe = []
        engine.step([S.EngineRow(SESSIONS, int(splitmix_at(TOKEN_SEED, 7000 + i) % g.vocab), i, i == 23) for i in range(24)])
        probe += [int(x) for x in engine.argmax(g.vocab)]
        engine.step([S.EngineRow(SESSIONS, int(splitmix_at(TOKEN_SEED, 8000 + i) % g.vocab), 24 + i, True, True) for i in range(8)])
        probe += [int(x) for x in engine.argmax(g.vocab)]
        engine.reset_slot(SESSIONS)
        gathered = [None] * world
        dist.all_gather_object(gathered, probe)
        if any(ids != gathered[0] for ids in gathered):
            raise SystemExit(f"rank {rank}: the ranks decode different tokens from the same session: {gathered}")

    step_index = 0
    for _ in range(args.warmup):
        one_step(step_index, True); step_index += 1

    sampler = ClockSampler(local); sampler.start()
    # Timed region 1: end to end through the C ABI with host rows in and token ids out.
    barrier(); t0 = time.perf_counter()
    gpu_seconds, launches = 0.0, 0
    for _ in range(args.steps):
        stats, ids = one_step(step_index, True); step_index += 1
        gpu_seconds += stats.gpu_seconds; launches += stats.launches
    barrier(); wall = time.perf_counter() - t0
    sampler.stop_flag = True; sampler.join()
    clocks = sampler.summary()

    times = torch.tensor([wall, gpu_seconds], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    wall_max, gpu_max = float(times[0]), float(times[1])
    per_rank = [1000.0 * gpu_seconds / args.steps]
    if dist is not None:
        per_rank = [None] * world
        dist.all_gather_object(per_rank, 1000.0 * gpu_seconds / args.steps)
    rows_per_step = SESSIONS * BLOCK
    total_rows = world * rows_per_step * args.steps

    # Profiled pass (events around every launch): the dominant kernel's share and achieved bandwidth.
    engine.debug_profile(True)
    for _ in range(args.steps):
        one_step(step_index, False); step_index += 1
    prof = engine.profile_read()
    engine.debug_profile(False)

    PREFILL_SLOT = SESSIONS

    def prompt_token(i):
        return int(splitmix_at(TOKEN_SEED ^ 0x9F1E, i) % g.vocab)

    def prefill_pass(tokens, chunk):
        """One prompt of `tokens` tokens through slot 8 in steps of `chunk` rows; returns (device seconds, launches)."""
        engine.reset_slot(PREFILL_SLOT)
        fed, seconds, count = 0, 0.0, 0
        while fed < tokens:
            n = min(chunk, tokens - fed)
            stats = engine.step([S.EngineRow(PREFILL_SLOT, prompt_token(fed + i), fed + i, fed + i == tokens - 1) for i in range(n)])
            seconds += stats.gpu_seconds; count += stats.launches; fed += n
        return seconds, count

    prefill = rider = strong = None
    if extras and world == 1:
        # Configuration 2: a 54.5K-token prompt in 2,048-row chunks. One chunk warms the wide kernels, one pass is timed,
        # a third runs with events around every launch for the classes' shares.
        prefill_pass(min(prompt_tokens, PREFILL_CHUNK), PREFILL_CHUNK)
        seconds, count = prefill_pass(prompt_tokens, PREFILL_CHUNK)
        engine.debug_profile(True)
        prefill_pass(prompt_tokens, PREFILL_CHUNK)
        shares = engine.profile_read()
        engine.debug_profile(False)
        weights, _ = weights_per_step(g)
        gemm_flops = 2.0 * (weights - g.vocab * g.hidden) * prompt_tokens
        peaks = {}
        if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        tensor_peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        gemm_tflops = gemm_flops / (shares["gemm_q4"]["ms"] * 1e-3) / 1e12 if shares["gemm_q4"]["ms"] > 0 else 0.0
        prefill = {"workload": f"one session, {prompt_tokens}-token prompt in {PREFILL_CHUNK}-row chunks, {g.layers} blocks", "tok_per_s": prompt_tokens / seconds,
                   "seconds": seconds, "steps": -(-prompt_tokens // PREFILL_CHUNK), "gpu_launches": count,
                   "gemm": {"kernel": "spl_gemm_q4_narrow_kernel<128, true> (the pair form of the 128-row block)", "tflops": gemm_tflops, "peak_tflops": tensor_peak, "frac": gemm_tflops / tensor_peak,
                            "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if peaks else "fallback (1.4 PFLOP/s sustained, an earlier measurement on this pool)",
                            "flops": "2 x the blocks' weights per prompt token (the head runs for the prompt's last token only)"},
                   "class_ms": {k: v["ms"] for k, v in shares.items()}}
        # Configuration 3's rider: the 8 decoding sessions' 64 verify rows and 64 rows of a 21K-token prompt in every step,
        # the prompt half fed (its pages hold synthetic KV, its state is seeded).
        engine.reset_slot(PREFILL_SLOT)
        start = rider_prompt // 2
        engine.step([S.EngineRow(PREFILL_SLOT, 1000, start - 1, False)])
        engine.debug_fill_kv(PREFILL_SLOT); engine.debug_fill_state(PREFILL_SLOT, 0x7777)
        seconds = 0.0
        for n in range(args.steps + 2):
            rows = rows_for(step_index) + [S.EngineRow(PREFILL_SLOT, prompt_token(start + i), start + i, False) for i in range(RIDER_ROWS)]
            stats = engine.step(rows)
            engine.argmax(248077 if g.vocab == 248320 else g.vocab)
            for s_ in range(SESSIONS):
                position[s_] += BLOCK
                engine.accept_verify(s_, BLOCK, position[s_])
            start += RIDER_ROWS; step_index += 1
            if n >= 2:
                seconds += stats.gpu_seconds
        rider = {"workload": f"64 verify rows of the 8 decoding sessions + {RIDER_ROWS} rows of a {rider_prompt}-token prompt (half fed) per step",
                 "ms_per_step": 1000.0 * seconds / args.steps, "decode_tok_per_s": rows_per_step * args.steps / seconds,
                 "prefill_tok_per_s": RIDER_ROWS * args.steps / seconds}
    if extras:
        # Strong scaling of configuration 3 as written: its 8 sessions split over the GPUs, 8 / N each, weights replicated.
        share = [s_ for s_ in range(SESSIONS) if s_ % world == rank]
        seconds = 0.0
        for n in range(args.steps + 2):
            rows = [r for r in rows_for(step_index) if r.slot in share]
            stats = engine.step(rows)
            engine.argmax(248077 if g.vocab == 248320 else g.vocab)
            for s_ in share:
                position[s_] += BLOCK
                engine.accept_verify(s_, BLOCK, position[s_])
            step_index += 1
            if n >= 2:
                seconds += stats.gpu_seconds
        slowest = torch.tensor([seconds], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        strong = {"workload": f"the 8 sessions split over {world} GPU(s), {len(share)} per GPU, 8-row verify blocks", "ms_per_step": 1000.0 * float(slowest[0]) / args.steps,
                  "tok_per_s": rows_per_step * args.steps / float(slowest[0])}
    draft = None
    if extras and world == 1 and not args.no_draft:
        # The DFlash 2 drafter beside the target (DraftModel.swift): 5 layers, 32 query and 8 kv heads of 128, the target's
        # width, its linear layers quantised to MLX affine-4 (MLX's range rule here: seconds instead of a minute of host
        # time for the fitted ranges), random weights of the checkpoint's shapes (one array a shape, used by every layer).
        # Context: the feature rows of one 64-row step pushed at consecutive positions until every slot's window of 2,048
        # is full; then a draft pass of one block a session.
        taps = [l for l in (5, 19, 33, 47, 61) if l < g.layers - 1] or [0]
        engine.enable_features(taps)
        dconfig = S.DraftConfig(mask_token=min(248070, g.vocab - 1), minmax_ranges=True)
        dm = S.DraftModel(engine, dconfig)
        rng = np.random.default_rng(WEIGHT_SEED & 0xFFFFFFFF)

        def bf16_of(shape, deviation, mean=0.0):
            x = rng.standard_normal(shape, dtype=np.float32) * np.float32(deviation) + np.float32(mean)
            b = x.view(np.uint32)
            return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)

        H, I, A, KV, GR = g.hidden, g.inter, dconfig.heads * 128, dconfig.kv_heads * 128, g.hidden // dconfig.group_size
        per_layer = {"input_layernorm.weight": bf16_of(H, 0.02, 1.0), "post_attention_layernorm.weight": bf16_of(H, 0.02, 1.0),
                     "self_attn.q_norm.weight": bf16_of(128, 0.02, 1.0), "self_attn.k_norm.weight": bf16_of(128, 0.02, 1.0),
                     "attention_conv.base_kernel": bf16_of((4, H), 0.2, 0.5), "mlp_conv.base_kernel": bf16_of((4, H), 0.2, 0.5),
                     "self_attn.q_proj.weight": bf16_of((A, H), 0.02), "self_attn.k_proj.weight": bf16_of((KV, H), 0.02),
                     "self_attn.o_proj.weight": bf16_of((H, A), 0.02), "mlp.gate_proj.weight": bf16_of((I, H), 0.02),
                     "mlp.down_proj.weight": bf16_of((H, I), 0.02), "attention_conv.kernel_projection.weight": bf16_of((4 * GR, H), 0.01)}
        per_layer["self_attn.v_proj.weight"] = per_layer["self_attn.k_proj.weight"]
        per_layer["mlp.up_proj.weight"] = per_layer["mlp.gate_proj.weight"]
        per_layer["mlp_conv.kernel_projection.weight"] = per_layer["attention_conv.kernel_projection.weight"]
        for layer in range(dconfig.layers):
            for name, bits in per_layer.items():
                dm.set_tensor(f"layers.{layer}.{name}", bits)
        dm.set_tensor("fc.weight", bf16_of((H, H * len(taps)), 0.01))
        dm.set_tensor("hidden_norm.weight", per_layer["input_layernorm.weight"])
        dm.set_tensor("norm.weight", per_layer["input_layernorm.weight"])
        dm.set_tensor("candidate_selector.hidden_projection.weight", bf16_of((dconfig.rank, H), 0.05))
        codebook = bf16_of((g.vocab, dconfig.rank), 0.5)
        dm.set_tensor("candidate_selector.predecessor_codebook", codebook)
        dm.set_tensor("candidate_selector.successor_codebook", codebook)
        del per_layer, codebook
        one_step(step_index, False); step_index += 1
        pushes = dconfig.window // BLOCK
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for n in range(pushes):
            dm.push_context([(s_, n * BLOCK + i, s_ * BLOCK + i) for s_ in range(SESSIONS) for i in range(BLOCK)])
        push_ms = 1000.0 * (time.perf_counter() - t0) / pushes
        at = pushes * BLOCK
        passes = {}
        for block, isolate in ((8, False), (16, True)):
            requests = [S.DraftRequest(s_, int(splitmix_at(TOKEN_SEED ^ 0xD4AF, s_) % 200000), at, block, isolate) for s_ in range(SESSIONS)]
            for _ in range(2):
                dm.propose(requests, vocab_limit=min(248077, g.vocab))
            t0 = time.perf_counter()
            for _ in range(args.steps):
                dm.propose(requests, vocab_limit=min(248077, g.vocab))
            passes[block] = 1000.0 * (time.perf_counter() - t0) / args.steps
        draft = {"workload": f"DFlash 2 drafter ({dconfig.layers} layers, {dconfig.heads}/{dconfig.kv_heads} heads of 128, MLX 4-bit g64, random weights) beside the target: "
                             f"{SESSIONS} sessions, every context window full ({dconfig.window} positions), one block a session per pass; wall time through "
                             "spl_draft_propose (block pass, top-16 on the device, selector on the host)",
                 "ms_per_pass_8_row_blocks": passes[8], "ms_per_pass_16_row_blocks": passes[16], "context_push_ms_per_64_rows": push_ms, "taps": taps}
        dm.close()
        engine.enable_features(enabled=False)
    gguf = None
    if extras and world == 1 and g.hidden % 256 == 0:
        # Configuration 4: Q5_K_M-style weights (Q5_K blocks, Q6_K embedding and head; pseudo-random blocks made on the device),
        # one session at 171K context verifying 16-token blocks. One way: the MLX tensors are freed as the GGUF ones arrive,
        # so this comes last. The session's pages hold synthetic KV, its state is seeded.
        for s_ in range(SESSIONS + 1):
            engine.reset_slot(s_)
        engine.step([S.EngineRow(0, 1000, gguf_context - 1, False)])
        engine.debug_fill_kv(0); engine.debug_fill_state(0, 0x6660)
        engine.synthesize_gguf(WEIGHT_SEED, "Q5_K", "Q6_K")
        at, seconds = gguf_context, 0.0
        for n in range(args.steps + 2):
            rows = [S.EngineRow(0, int(splitmix_at(TOKEN_SEED ^ 0x66, at + i) % g.vocab), at + i, True, True) for i in range(GGUF_BLOCK)]
            stats = engine.step(rows)
            engine.argmax(248077 if g.vocab == 248320 else g.vocab)
            at += GGUF_BLOCK
            engine.accept_verify(0, GGUF_BLOCK, at)
            if n >= 2:
                seconds += stats.gpu_seconds
        # Two more steps with events around every launch, for the classes' shares.
        engine.debug_profile(True)
        for n in range(2):
            rows = [S.EngineRow(0, int(splitmix_at(TOKEN_SEED ^ 0x66, at + i) % g.vocab), at + i, True, True) for i in range(GGUF_BLOCK)]
            engine.step(rows)
            at += GGUF_BLOCK
            engine.accept_verify(0, GGUF_BLOCK, at)
        gguf_shares = engine.profile_read()
        engine.debug_profile(False)
        wcount, _ = weights_per_step(g)
        head_weights = g.vocab * g.hidden
        gguf_bytes = (wcount - head_weights) * 176 / 256 + head_weights * 210 / 256
        device_bytes = (wcount - head_weights) * 272 / 256 + head_weights * 288 / 256      # the library's layout: a byte a code for Q5_K and Q6_K
        n_full = g.layers // 4
        kv_bytes = gguf_context * n_full * 2 * g.kv_heads * (g.head_dim + 4)
        gguf = {"workload": f"one session at {gguf_context} tokens of context, {GGUF_BLOCK}-row verify blocks, every block tensor Q5_K, embedding and head Q6_K "
                            "(GGUF super-blocks), plain norms, unfused SiLU gate",
                "ms_per_step": 1000.0 * seconds / args.steps, "tok_per_s": GGUF_BLOCK * args.steps / seconds, "weights_gb": gguf_bytes / 1e9, "weights_read_gb": device_bytes / 1e9, "kv_gb": kv_bytes / 1e9,
                "hbm_gbs": (gguf_bytes + kv_bytes) / (seconds / args.steps) / 1e9,
                "class_ms_per_step": {k: v["ms"] / 2 for k, v in gguf_shares.items()}}
    if rank == 0:
        peak, peak_source = measured_peak_gbs()
        gemm = prof["gemm_q4"]
        gemm_gbs = gemm["bytes"] / (gemm["ms"] * 1e-3) / 1e9 if gemm["ms"] > 0 else 0.0
        step_bytes, parts = algorithmic_bytes(g, ctx, BLOCK)
        step_ms = 1000.0 * gpu_max / args.steps
        tables_bytes = (rows_per_step * 5 + SESSIONS * 5 + rows_per_step + rows_per_step // 4 + SESSIONS * engine.host.max_pages) * 4
        line = {
            "metric": "packed_step_tok_per_s", "value": total_rows / gpu_max, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 x int4 -> fp32 (int8 KV, fp32 state)", "data": "synthetic",
            "config": {"workload": f"27B-shape ({g.layers} blocks) MLX 4-bit g64, 8 sessions x 8-row verify blocks = 64 rows per step, contexts "
                                   f"{min(ctx)}-{max(ctx)} tokens, int8 paged KV, all rows accepted each step", "sessions_per_gpu": SESSIONS,
                       "rows_per_step": rows_per_step, "span_target": SPAN_TARGET, "parallelism": f"sessions sharded, {world} replica(s)",
                       "l2": "inputs larger than L2: 14.4 GB of weights and the KV pool stream every step"},
            "e2e": {"value": total_rows / wall_max, "unit": "tok/s", "h2d_bytes_per_step": tables_bytes, "d2h_bytes_per_step": rows_per_step * 4},
            "gpu_launches": launches,
            "ms_per_step_by_rank": per_rank,
            "clocks": clocks,
            "step": {"algorithmic_gb": step_bytes / 1e9, "weights_gb": parts["weights"] / 1e9, "kv_gb": parts["kv"] / 1e9, "state_gb": parts["state"] / 1e9,
                     "hbm_gbs": step_bytes / (step_ms * 1e-3) / 1e9, "frac_of_peak": step_bytes / (step_ms * 1e-3) / 1e9 / peak,
                     "class_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items()},
                     "class_launches_per_step": {k: v["launches"] / args.steps for k, v in prof.items()}},
            "roofline": {"kernel": "spl_gemm_q4_narrow_kernel", "bound": "hbm", "achieved": gemm_gbs, "peak": peak, "unit": "GB/s",
                         "frac": gemm_gbs / peak, "traffic": GEMM_DRAM_PER_ALGORITHMIC_BYTE * gemm["bytes"] / max(gemm["launches"], 1),
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of the 4-block case, per tensor shape, scaled by launches (profiles/gemm_q4_narrow_kernel_27b_64rows.md)",
                         "peak_source": peak_source,
                         "per_launch": {"algorithmic_bytes": gemm["bytes"] / max(gemm["launches"], 1), "ms": gemm["ms"] / max(gemm["launches"], 1)}},
        }
        if prefill is not None:
            line["prefill"] = prefill
        if rider is not None:
            line["rider"] = rider
        if strong is not None:
            line["strong"] = strong
        if gguf is not None:
            line["gguf"] = gguf
        if draft:
            line["draft"] = draft
        if not args.no_cpu_baseline and world == 1:
            value, cores, sample = cpu_baseline()
            line["cpu_baseline"] = {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    engine.close()
    if dist is not None:
        dist.barrier(); dist.destroy_process_group()


if __name__ == "__main__":
    main()
