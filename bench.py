"""Benchmark of the batch-1 greedy decode path (fp16 weights, fp16 KV cache) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: a 4096-token random prompt
is prefilled once (not timed; the metric is decode throughput), then each step decodes 256 greedy
tokens from position 4095 through ONE call of the ``generate_nosync`` op (= one persistent-kernel
launch).  Under torchrun every rank runs an independent replica on its own GPU (no collective on the
data path); the value is all ranks' tokens divided by the slowest rank's time.

Prints one JSON line (rank 0).  ``value`` is timed with CUDA events around the op calls with every
input resident in HBM; ``e2e`` is the same call sequence as ``Decoder.generate_ids`` uses after
prefill (token log cleared, op call, device->host copy of the log into pinned memory, host-side
trimming), timed on the host clock.  ``--impl reference`` times the CPU oracle instead.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "qwen3-0.6b-megakernel-rtx-5090_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

import synthetic as S  # noqa: E402

PROMPT_LEN = 4096
DECODE_TOKENS = 256
MAX_SEQ_LEN = 4352
METRIC = "batch-1 decode tok/s"
UNIT = "tok/s"
WORKLOAD = ("configs[1]: Qwen3-0.6B fp16, batch 1 per GPU, 4096 random prompt tokens prefilled (untimed), "
            "256 greedy decode tokens per step, KV cache fp16 [layer][kv_head][pos][128]")


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def step_bytes(prompt_len: int = PROMPT_LEN, decode_tokens: int = DECODE_TOKENS, weights: str = "fp16") -> int:
    """Algorithmic HBM bytes of one step: sum over its tokens of weights + KV read + KV write."""
    total = sum(S.decode_step_bytes(prompt_len + i) for i in range(decode_tokens))
    if weights == "fp8":
        import quantize
        total += decode_tokens * (quantize.weight_bytes_fp8() - S.weight_bytes_fp16())
    return total


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def aggregate(tokens_per_rank: int, seconds_max: float, world: int) -> float:
    """Whole-job throughput of independent replicas: all ranks' tokens over the slowest rank's time."""
    return tokens_per_rank * world / seconds_max


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


# --------------------------------------------------------------------------- CPU oracle legs
def cpu_decode_rate(n_tokens: int, threads: int):
    """tok/s of the CPU oracle at the benchmark's context length.  The KV cache is filled with seeded
    random fp16 values instead of a real 4096-token prefill (step time does not depend on the values)."""
    from oracle.decoder_ref import Decoder as Oracle
    torch.set_num_threads(threads)
    w = S.make_weights(seed=0, max_seq_len=16)
    o = Oracle(w, max_seq_len=PROMPT_LEN + n_tokens + 2)
    g = torch.Generator("cpu").manual_seed(1)
    o.k_cache[:, :, :PROMPT_LEN] = torch.randn(o.k_cache[:, :, :PROMPT_LEN].shape, generator=g).to(o.kv_dtype)
    o.v_cache[:, :, :PROMPT_LEN] = torch.randn(o.v_cache[:, :, :PROMPT_LEN].shape, generator=g).to(o.kv_dtype)
    o._position = PROMPT_LEN - 1
    tok = o.step(17)  # warm-up step (also brings weights into cache/TLB)
    o._position = PROMPT_LEN - 1
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        tok = o.step(tok)
    dt = time.perf_counter() - t0
    return n_tokens / dt, dt, o


def run_reference(args):
    """The reference has no CPU implementation of this path (its only implementation is sm_120 CUDA and
    its Python layer needs that extension to import), so this arm times the CPU oracle port."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample_tokens = 8
    from oracle.decoder_ref import Decoder as Oracle
    torch.set_num_threads(threads)
    w = S.make_weights(seed=0, max_seq_len=16)
    o = Oracle(w, max_seq_len=PROMPT_LEN + sample_tokens + 2)
    g = torch.Generator("cpu").manual_seed(1)
    o.k_cache[:, :, :PROMPT_LEN] = torch.randn(o.k_cache[:, :, :PROMPT_LEN].shape, generator=g).to(o.kv_dtype)
    o.v_cache[:, :, :PROMPT_LEN] = torch.randn(o.v_cache[:, :, :PROMPT_LEN].shape, generator=g).to(o.kv_dtype)

    def one_step():
        o._position = PROMPT_LEN - 1
        tok = 17
        for _ in range(sample_tokens):
            tok = o.step(tok)

    for _ in range(args.warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    dt = time.perf_counter() - t0
    value = args.steps * sample_tokens / dt
    sample = (f"each step = {sample_tokens} greedy tokens at context {PROMPT_LEN} (bounded sample of the 256-token "
              f"step; KV cache pre-filled with random values); oracle port, torch fp32, {threads} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# --------------------------------------------------------------------------- the engine arm
def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU path (use --impl reference for the oracle)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    import build
    build.build()
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import Decoder

    PROMPT_LEN, DECODE_TOKENS = args.prompt_len, args.decode_tokens   # defaults: the benchmark configuration
    MAX_SEQ_LEN = PROMPT_LEN + DECODE_TOKENS
    host_weights = S.make_weights(seed=0, max_seq_len=16)
    expanded = False              # quantised weights stored as fp16 (engines without a packed path)
    if args.weights != "fp16" and args.batch > 4:
        import quantize
        host_weights, _ = (quantize.expand_weights_fp8 if args.weights == "fp8" else quantize.expand_weights_nvfp4)(host_weights)
        expanded = True
    elif args.weights == "nvfp4":
        raise SystemExit("bench.py: --weights nvfp4 needs --batch > 4 (expanded to fp16 on the tensor-core path)")
    elif args.weights == "fp8":   # BASELINE.json configs[2] weight format, packed rows (batch <= 4)
        import quantize
        host_weights, _ = quantize.quantize_weights_fp8(host_weights)
    engine_format = "fp16" if expanded else args.weights
    weights = S.weights_to(host_weights, str(device))
    B = args.batch
    if B == 1:
        eng = Decoder(weights=weights, tokenizer=S.StubTokenizer(-1), verbose=False, max_seq_len=MAX_SEQ_LEN,
                      device=str(device), weight_format=engine_format)
        prompt = S.make_prompt(PROMPT_LEN, seed=rank)   # each replica serves its own stream
        eng.reset()
        eng.prefill_ids(prompt[:-1])                    # untimed; fills 4095 cache rows
        start_pos = eng.position
        first = prompt[-1]
        log = eng._output_log[:DECODE_TOKENS]
        host_log = eng._output_log_cpu[:DECODE_TOKENS]

        def op_call():
            eng._gen(first, DECODE_TOKENS, *eng._common(), log, eng.num_layers, start_pos, eng.max_seq_len,
                     eng._attn_scale, -1)

        def api_call():
            # what Decoder.generate_ids does after prefill, with host buffers on both sides
            log.fill_(-1)
            op_call()
            host_log.copy_(log)
            out = []
            for t in host_log.tolist():
                if t == -1:
                    break
                out.append(t)
            return out
    else:
        # B sequences per launch (multi-sequence kernel), every one at the benchmark context length
        from Model.Qwen06B_architecture import BatchDecoder
        eng = BatchDecoder(weights=weights, tokenizer=S.StubTokenizer(-1), num_sequences=B, max_seq_len=MAX_SEQ_LEN,
                           device=str(device), weight_format=engine_format,
                           prefill_mode="tensor" if engine_format == "fp16" else "serial")
        persistent = eng.engine == "persistent"
        prompts = [S.make_prompt(PROMPT_LEN, seed=rank * 16 + b) for b in range(B)]
        for b in range(B):
            eng._prefill_slot(b, prompts[b][:-1])       # untimed
        firsts = [p[-1] for p in prompts]
        starts = list(eng.positions)
        logs = [eng._logs[b][:DECODE_TOKENS] for b in range(B)]
        host_logs = eng._logs_cpu[:, :DECODE_TOKENS]
        base = eng._base

        def op_call():
            eng._gen_batch(firsts, starts, DECODE_TOKENS, base._embed_weight, base._layer_weights_packed,
                           base._final_norm_weight, base._lm_head_weight, base._cos_table, base._sin_table,
                           eng._k_caches, eng._v_caches, logs, base.num_layers, eng.max_seq_len, base._attn_scale)

        def api_call():
            out = []
            for b in range(B):
                logs[b].fill_(-1)
            op_call()
            for b in range(B):
                host_logs[b].copy_(logs[b])
                for t in host_logs[b].tolist():
                    if t == -1:
                        break
                    out.append(t)
            return out

    for _ in range(max(args.warmup, 0)):
        op_call()
    ref_tokens = api_call()
    assert len(ref_tokens) == DECODE_TOKENS * B

    # ---- device-timed region: K steps, one launch each
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier(world)
    with ClockSampler(local) as clocks:
        t_begin = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_begin.record()
        for a, b in ev:
            a.record()
            op_call()
            b.record()
        t_end.record()
        barrier(world)
    total_s = t_begin.elapsed_time(t_end) / 1e3
    launch_ms = [a.elapsed_time(b) for a, b in ev]
    total_s = max_over_ranks(total_s, world, device)
    value = aggregate(args.steps * DECODE_TOKENS * B, total_s, world)

    # ---- end-to-end region through the host API
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = api_call()
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device)
    assert out == ref_tokens, "decode is not reproducible run to run"
    e2e_value = aggregate(args.steps * DECODE_TOKENS * B, e2e_s, world)

    peak, peak_kind = measured_peak_gbs()
    avg_launch_s = statistics.mean(launch_ms) / 1e3
    # algorithmic bytes of a launch: weights once per step, KV of every sequence
    kv_only = step_bytes(PROMPT_LEN, DECODE_TOKENS, "fp16") - DECODE_TOKENS * S.weight_bytes_fp16()
    launch_bytes = step_bytes(PROMPT_LEN, DECODE_TOKENS, "fp16" if expanded else args.weights) + (B - 1) * kv_only
    achieved = launch_bytes / avg_launch_s / 1e9
    traffic = None   # DRAM bytes per launch from the committed ncu capture, scaled by tokens per launch
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            per_token = json.load(f).get("qwen3_decode_megakernel_dram_bytes_per_token")
        if per_token and args.weights == "fp16" and B == 1:
            traffic = per_token * DECODE_TOKENS
    except Exception:
        pass

    if rank == 0:
        line = {
            "metric": METRIC if B == 1 else f"batch-{B} decode tok/s (all sequences)", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * total_s / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16" if (args.weights == "fp16" or expanded) else "fp8-e4m3 weights, fp32 math",
            "data": "synthetic",
            "config": {"weights": args.weights + (" (quantised values, stored expanded as fp16)" if expanded else ""), "workload": WORKLOAD if (PROMPT_LEN, DECODE_TOKENS) == (4096, 256) else
                       f"profiling case: {PROMPT_LEN} prompt tokens, {DECODE_TOKENS} decode tokens per step",
                       "tokens_per_step": DECODE_TOKENS * B, "sequences_per_launch": B,
                       "engine": "persistent megakernel" if (B == 1 or persistent) else "tcgen05 GEMM path", "replicas": world,
                       "l2": "no flush needed: each token streams 1.19 GB of weights + 0.47 GB of KV, > 126 MB L2",
                       "grid_ctas": C.num_ctas()},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_kind": f"of {peak_kind}",
                         "bytes_per_launch": launch_bytes, "launch_ms": statistics.mean(launch_ms),
                         "frac_of_nominal_8TBs": achieved / 8000.0},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * B,
                    "d2h_bytes_per_step": 4 * DECODE_TOKENS * B},
            "gpu_launches": args.steps if (B == 1 or persistent) else args.steps * DECODE_TOKENS * (7 * 28 + 4),
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            n = 16
            rate, dt, _ = cpu_decode_rate(n, threads)
            line["cpu_baseline"] = {
                "value": rate, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"{n} greedy tokens at context {PROMPT_LEN} (KV pre-filled with random values), "
                          f"oracle torch fp32, {dt:.1f} s"}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_continuous(args):
    """Continuous-batching job (the multi-replica serving configuration, scaled by --continuous): N requests
    per GPU, prompt lengths uniform in [64, 2048], 128 greedy tokens each, up to --batch live sequences.
    Wall-clock of the whole job, prefill included; one JSON line with its own metric name."""
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    import build
    build.build()
    from Model.Qwen06B_architecture import BatchDecoder
    from scheduler import ContinuousBatcher
    slots = max(args.batch, 2)
    new_tokens = 128
    weights = S.weights_to(S.make_weights(seed=0, max_seq_len=16), str(device))
    eng = BatchDecoder(weights=weights, tokenizer=S.StubTokenizer(-1), num_sequences=slots, max_seq_len=2048 + new_tokens,
                       device=str(device), prefill_mode=args.prefill)
    gen = torch.Generator("cpu").manual_seed(rank)             # a different request stream per replica
    lens = torch.randint(64, 2049, (args.continuous,), generator=gen).tolist()
    prompts = [S.make_prompt(L, seed=1000 * rank + i) for i, L in enumerate(lens)]
    prefill_s = [0.0]
    inner = eng.prefill_slot

    def timed_prefill(b, ids):
        t = time.perf_counter()
        inner(b, ids)
        prefill_s[0] += time.perf_counter() - t
    eng.prefill_slot = timed_prefill
    sch = ContinuousBatcher(eng, eos_token_id=None, quantum=32,
                            overlap_prefill=bool(args.overlap) and getattr(eng, "supports_overlap", False))
    sch.submit(prompts[0][:64], 8)                             # warm-up: both kernels, all buffers
    sch.run_until_idle()
    prefill_s[0] = 0.0
    launches0 = sch.launches
    barrier(world)
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        futs = [sch.submit(p, new_tokens) for p in prompts]
        sch.run_until_idle()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    n_out = sum(len(f.result().tokens) for f in futs)
    assert n_out == args.continuous * new_tokens
    wall = max_over_ranks(wall, world, device)
    if rank == 0:
        print(json.dumps({
            "metric": "continuous-batching generated tok/s (prefill included)", "value": world * n_out / wall,
            "unit": UNIT, "n_gpus": world, "requests_per_gpu": args.continuous, "live_sequences": slots,
            "new_tokens_per_request": new_tokens, "prompt_tokens": sum(lens), "wall_s": wall,
            "prefill_s": prefill_s[0], "decode_s": wall - prefill_s[0],
            "decode_only_tok_s": n_out / max(wall - prefill_s[0], 1e-9), "launches": sch.launches - launches0,
            "prefill": args.prefill, "overlap_prefill": sch.overlap_prefill, "prompt_tok_s": sum(lens) / max(prefill_s[0], 1e-9),
            "scaling": "weak", "data": "synthetic", "dtype": "fp16", "clocks": clocks.summary(),
            "note": "rank 0's own prefill/decode split; value uses the slowest replica's wall time"}))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle leg (profiling runs)")
    ap.add_argument("--weights", choices=["fp16", "fp8", "nvfp4"], default="fp16",
                    help="weight format (default fp16 = the benchmark configuration)")
    ap.add_argument("--batch", type=int, default=1,
                    help="sequences per GPU decoded together (default 1: the headline batch-1 configuration; 2-3 (4 with fp8): one "
                         "persistent launch; above: tensor-core batched decode)")
    ap.add_argument("--continuous", type=int, default=0, metavar="N",
                    help="instead of the headline workload: N requests per GPU through the continuous-batching "
                         "scheduler (prompt lengths 64..2048, 128 new tokens each, --batch live sequences)")
    ap.add_argument("--overlap", type=int, default=1,
                    help="--continuous only: 1 = prefill the next request while the live ones decode (tensor-core engines)")
    ap.add_argument("--prefill", choices=["serial", "tensor"], default="tensor",
                    help="--continuous only: token-serial prefill op or the tensor-core chunked prefill")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prefilled context (default: benchmark config)")
    ap.add_argument("--decode-tokens", type=int, default=DECODE_TOKENS,
                    help="greedy tokens per step (default: benchmark config; smaller for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.continuous > 0:
        run_continuous(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
