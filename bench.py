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
GOLDEN_CTX4096 = os.path.join(ROOT, "tests", "golden", "full_seed0_prompt4096.json")


def kv_bytes(context_lens, decode_tokens: int) -> int:
    """Algorithmic KV bytes of `decode_tokens` steps of sequences that start with these many cached positions:
    per step and sequence 114,688 B per position attended (the new one included) + one new row written."""
    per_pos = S.decode_step_bytes(1) - S.decode_step_bytes(0)
    total = 0
    for L in context_lens:
        total += sum(per_pos * (L + i + 1) + per_pos for i in range(decode_tokens))
    return total


def weight_bytes(kind: str) -> int:
    if kind == "fp8":
        import quantize
        return quantize.weight_bytes_fp8()
    if kind == "nvfp4":
        import quantize
        return quantize.weight_bytes_nvfp4()
    return S.weight_bytes_fp16()


def decode_case(device, rank, world, fp16_weights, weights_kind, B, prompt_lens, decode_tokens, steps, warmup,
                check_golden=False):
    """One decode configuration on this rank's GPU: prompts prefilled (untimed), then `steps` timed launches of
    `decode_tokens` greedy tokens for all B sequences, then the same through the host API.  Returns a dict with the
    device-timed and end-to-end rates (max over ranks), per-launch times and the HBM roofline of the launch."""
    import qwen_megakernel_C as C
    from Model.Qwen06B_architecture import BatchDecoder, Decoder
    max_seq = max(prompt_lens) + decode_tokens
    expanded = False
    weights = fp16_weights
    if weights_kind != "fp16":
        import quantize
        # packed rows in HBM on every path: the persistent kernels read FP8 rows directly, the tensor-core path
        # expands FP8 / NVFP4 K blocks to fp16 tiles inside its GEMMs
        if weights_kind == "fp8":
            weights, _ = quantize.quantize_weights_fp8(fp16_weights)
        elif B > 3:
            weights, _ = quantize.quantize_weights_nvfp4(fp16_weights)
        else:
            raise SystemExit("bench.py: nvfp4 needs --batch > 3 (only the tensor-core path reads NVFP4 rows)")
    engine_format = "fp16" if (expanded or weights_kind == "fp16") else weights_kind
    parity = None
    if B == 1:
        eng = Decoder(weights=weights, tokenizer=S.StubTokenizer(-1), verbose=False, max_seq_len=max_seq,
                      device=str(device), weight_format=engine_format)
        prompt = S.make_prompt(prompt_lens[0], seed=rank)   # each replica serves its own stream
        eng.reset()
        eng.prefill_ids(prompt[:-1])                        # untimed
        start_pos = eng.position
        first = prompt[-1]
        log = eng._output_log[:decode_tokens]
        host_log = eng._output_log_cpu[:decode_tokens]
        engine_name = "persistent megakernel"

        def op_call():
            eng._gen(first, decode_tokens, *eng._common(), log, eng.num_layers, start_pos, eng.max_seq_len,
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
        eng = BatchDecoder(weights=weights, tokenizer=S.StubTokenizer(-1), num_sequences=B, max_seq_len=max_seq,
                           device=str(device), weight_format=engine_format,
                           prefill_mode="serial" if (engine_format == "fp8" and B <= 3) else "tensor")
        engine_name = "persistent megakernel" if eng.engine == "persistent" else "tcgen05 GEMM path"
        prompts = [S.make_prompt(prompt_lens[b], seed=rank * 128 + b) for b in range(B)]
        for b in range(B):
            eng._prefill_slot(b, prompts[b][:-1])           # untimed
        firsts = [p[-1] for p in prompts]
        starts = list(eng.positions)
        logs = [eng._logs[b][:decode_tokens] for b in range(B)]
        host_logs = eng._logs_cpu[:, :decode_tokens]
        base = eng._base

        def op_call():
            eng._gen_batch(firsts, starts, decode_tokens, base._embed_weight, base._layer_weights_packed,
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

    for _ in range(max(warmup, 0)):
        op_call()
    ref_tokens = api_call()
    assert len(ref_tokens) == decode_tokens * B
    if check_golden and rank == 0:
        # parity of the benchmarked configuration itself (outside the timed region): rank 0's prompt is the golden
        # file's, its first tokens must be the CPU oracle's
        with open(GOLDEN_CTX4096) as f:
            g = json.load(f)
        n = len(g["tokens"])
        parity = (prompt_lens[0] == g["prompt_len"] and ref_tokens[:n] == g["tokens"])
        if not parity:
            raise SystemExit(f"bench.py: decode does not reproduce the golden tokens: {ref_tokens[:n]} vs {g['tokens']}")

    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier(world)
    with ClockSampler(device.index) as clocks:
        t_begin = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_begin.record()
        for a, b in ev:
            a.record()
            op_call()
            b.record()
        t_end.record()
        barrier(world)
    own_s = t_begin.elapsed_time(t_end) / 1e3
    launch_ms = [a.elapsed_time(b) for a, b in ev]
    total_s = max_over_ranks(own_s, world, device)

    barrier(world)
    t0 = time.perf_counter()
    for _ in range(steps):
        out = api_call()
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device)
    assert out == ref_tokens, "decode is not reproducible run to run"

    per_rank = [statistics.mean(launch_ms)]
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor(per_rank, dtype=torch.float64, device=device)
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        per_rank = [float(x.item()) for x in gathered]
    tokens = steps * decode_tokens * B
    launch_bytes = decode_tokens * weight_bytes("fp16" if expanded else weights_kind) + kv_bytes(
        [L - 1 for L in prompt_lens], decode_tokens)
    peak, peak_kind = measured_peak_gbs()
    achieved = launch_bytes / (statistics.mean(launch_ms) / 1e3) / 1e9
    res = dict(value=aggregate(tokens, total_s, world), e2e=aggregate(tokens, e2e_s, world),
               ms_per_step=1e3 * total_s / steps, launch_ms=statistics.mean(launch_ms),
               per_rank_launch_ms={"min": min(per_rank), "median": statistics.median(per_rank), "max": max(per_rank)},
               bytes_per_launch=launch_bytes, achieved_gbs=achieved, frac=achieved / peak, peak=peak, peak_kind=peak_kind,
               engine=engine_name, expanded=expanded,
               stored={"fp16": "fp16", "fp8": "packed FP8-E4M3 rows (fp32 row scales)",
                       "nvfp4": "packed NVFP4 rows (e2m1 pairs, e4m3 block-16 scales, fp32 tensor scale)"}[weights_kind], clocks=clocks.summary(), grid=C.num_ctas(), parity=parity,
               launches=steps if engine_name == "persistent megakernel" else steps * decode_tokens * (7 * 28 + 4))
    del eng
    torch.cuda.empty_cache()
    return res


def continuous_case(device, rank, world, fp16_weights, requests, slots, prefill="tensor", overlap=1):
    """BASELINE.json's serving configuration on this rank's GPU: `requests` requests, prompt lengths uniform in
    [64, 2048], 128 greedy tokens each, continuous batching with up to `slots` live sequences; wall clock of the
    whole job (prefill included), slowest replica."""
    from Model.Qwen06B_architecture import BatchDecoder
    from scheduler import ContinuousBatcher
    new_tokens = 128
    # `slots` sequences decode together; half as many extra cache slots hold requests that are prefilled already, so
    # that a seat which frees up is taken in the next round (ContinuousBatcher(live_limit=...))
    spare = min(slots // 2, 128 - slots) if prefill == "tensor" and overlap else 0
    eng = BatchDecoder(weights=fp16_weights, tokenizer=S.StubTokenizer(-1), num_sequences=slots + spare,
                       max_seq_len=2048 + new_tokens, device=str(device), prefill_mode=prefill)
    gen = torch.Generator("cpu").manual_seed(rank)             # a different request stream per replica
    lens = torch.randint(64, 2049, (requests,), generator=gen).tolist()
    prompts = [S.make_prompt(L, seed=1000 * rank + i) for i, L in enumerate(lens)]
    prefill_s = [0.0]
    inner = eng.prefill_slot

    def timed_prefill(b, ids):
        t = time.perf_counter()
        inner(b, ids)
        prefill_s[0] += time.perf_counter() - t
    eng.prefill_slot = timed_prefill
    if hasattr(eng, "prefill_slots"):                          # several waiting requests in one pass
        inner_many = eng.prefill_slots

        def timed_prefill_many(bs, many):
            t = time.perf_counter()
            inner_many(bs, many)
            prefill_s[0] += time.perf_counter() - t
        eng.prefill_slots = timed_prefill_many
    sch = ContinuousBatcher(eng, eos_token_id=None, quantum=32,
                            overlap_prefill=bool(overlap) and getattr(eng, "supports_overlap", False), live_limit=slots)
    sch.submit(prompts[0][:64], 8)                             # warm-up: both kernels, all buffers
    sch.run_until_idle()
    prefill_s[0] = 0.0
    launches0 = sch.launches
    barrier(world)
    with ClockSampler(device.index) as clocks:
        t0 = time.perf_counter()
        futs = [sch.submit(p, new_tokens) for p in prompts]
        sch.run_until_idle()
        torch.cuda.synchronize()
        own_wall = time.perf_counter() - t0
    n_out = sum(len(f.result().tokens) for f in futs)
    assert n_out == requests * new_tokens
    wall = max_over_ranks(own_wall, world, device)
    res = dict(value=world * n_out / wall, wall_s=wall, own_wall_s=own_wall, requests_per_gpu=requests, live_sequences=slots,
               new_tokens_per_request=new_tokens, prompt_tokens=sum(lens), prefill_s=prefill_s[0],
               decode_s=own_wall - prefill_s[0], decode_only_tok_s=n_out / max(own_wall - prefill_s[0], 1e-9),
               prompt_tok_s=sum(lens) / max(prefill_s[0], 1e-9), launches=sch.launches - launches0, prefill=prefill,
               overlap_prefill=sch.overlap_prefill, prefilled_ahead_slots=spare, max_live=sch.max_live, clocks=clocks.summary())
    del sch, eng
    torch.cuda.empty_cache()
    return res


def init_engine_arm():
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
    return rank, world, device


def finish_engine_arm(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_ours(args):
    rank, world, device = init_engine_arm()
    weights = S.weights_to(S.make_weights(seed=0, max_seq_len=16), str(device))
    B = args.batch
    headline = (args.prompt_len, args.decode_tokens, args.weights, B) == (PROMPT_LEN, DECODE_TOKENS, "fp16", 1)
    r = decode_case(device, rank, world, weights, args.weights, B, [args.prompt_len] * B, args.decode_tokens, args.steps,
                    args.warmup, check_golden=headline)
    traffic = None   # DRAM bytes per launch from the committed ncu capture, scaled by tokens per launch
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            per_token = json.load(f).get("qwen3_decode_megakernel_dram_bytes_per_token")
        if per_token and headline:
            traffic = per_token * args.decode_tokens
    except Exception:
        pass
    line = {
        "metric": METRIC if B == 1 else f"batch-{B} decode tok/s (all sequences)", "value": r["value"], "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16" if (args.weights == "fp16" or r["expanded"]) else f"{args.weights} weights, fp32 accumulation", "data": "synthetic",
        "config": {"weights": args.weights + (" (quantised values, stored expanded as fp16)" if r["expanded"] else ""),
                   "workload": WORKLOAD if (args.prompt_len, args.decode_tokens) == (PROMPT_LEN, DECODE_TOKENS) else
                   f"profiling case: {args.prompt_len} prompt tokens, {args.decode_tokens} decode tokens per step",
                   "tokens_per_step": args.decode_tokens * B, "sequences_per_launch": B, "engine": r["engine"], "replicas": world,
                   "l2": "no flush needed: each token streams 1.19 GB of weights + 0.47 GB of KV, > 126 MB L2",
                   "grid_ctas": r["grid"]},
        "roofline": {"bound": "hbm", "achieved": r["achieved_gbs"], "peak": r["peak"], "unit": "GB/s", "frac": r["frac"],
                     "traffic": traffic, "peak_kind": f"of {r['peak_kind']}", "bytes_per_launch": r["bytes_per_launch"],
                     "launch_ms": r["launch_ms"], "frac_of_nominal_8TBs": r["achieved_gbs"] / 8000.0},
        "e2e": {"value": r["e2e"], "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * args.decode_tokens * B},
        "gpu_launches": r["launches"], "clocks": r["clocks"], "per_rank_launch_ms": r["per_rank_launch_ms"],
    }
    if r["parity"] is not None:
        line["parity_checked"] = bool(r["parity"])
    if headline and not args.no_extra:
        # the other BASELINE.json configurations, each with its own algorithmic-bytes roofline; every rank runs them
        def brief(c):
            return {"value": c["value"], "unit": UNIT, "e2e": c["e2e"], "ms_per_step": c["ms_per_step"], "engine": c["engine"],
                    "roofline_frac": c["frac"], "achieved_gbs": c["achieved_gbs"], "bytes_per_launch": c["bytes_per_launch"],
                    "weights_stored_as": c["stored"],
                    "per_rank_launch_ms": c["per_rank_launch_ms"]}
        extra = {}
        c3 = {}
        for b3 in (1, 4, 16):
            c3[f"batch{b3}"] = brief(decode_case(device, rank, world, weights, "fp8", b3, [1024] * b3, 128, 2, 1))
        extra["config3"] = {"workload": "configs[2]: FP8-E4M3 weights (per-row fp32 scale), 1024-token prompts, 128 decode steps",
                            **c3}
        gen = torch.Generator("cpu").manual_seed(0)
        lens4 = torch.randint(128, 2049, (64,), generator=gen).tolist()
        extra["config4"] = {"workload": "configs[3]: NVFP4 weight values, batch 64, prompt lengths uniform in [128, 2048], 128 decode steps",
                            **brief(decode_case(device, rank, world, weights, "nvfp4", 64, lens4, 128, 2, 1))}
        c5 = continuous_case(device, rank, world, weights, 256, 32)
        extra["config5"] = {"workload": "configs[4]: 256 requests per GPU, prompts uniform in [64, 2048], 128 greedy tokens each, "
                                        "continuous batching, <= 32 live sequences", "unit": UNIT,
                            **{k: c5[k] for k in ("value", "wall_s", "prefill_s", "decode_s", "decode_only_tok_s", "prompt_tok_s",
                                                  "launches", "overlap_prefill")}}
        line["extra"] = extra
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            n = 16
            rate, dt, _ = cpu_decode_rate(n, threads)
            line["cpu_baseline"] = {
                "value": rate, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"{n} greedy tokens at context {PROMPT_LEN} (KV pre-filled with random values), "
                          f"oracle torch fp32, {dt:.1f} s"}
        print(json.dumps(line))
    finish_engine_arm(world)


def run_continuous(args):
    """Continuous-batching job (the multi-replica serving configuration, scaled by --continuous): N requests
    per GPU, prompt lengths uniform in [64, 2048], 128 greedy tokens each, up to --batch live sequences.
    Wall-clock of the whole job, prefill included; one JSON line with its own metric name."""
    rank, world, device = init_engine_arm()
    weights = S.weights_to(S.make_weights(seed=0, max_seq_len=16), str(device))
    c = continuous_case(device, rank, world, weights, args.continuous, max(args.batch, 2), args.prefill, args.overlap)
    if rank == 0:
        print(json.dumps({
            "metric": "continuous-batching generated tok/s (prefill included)", "unit": UNIT, "n_gpus": world,
            "scaling": "weak", "data": "synthetic", "dtype": "fp16",
            "note": "rank 0's own prefill/decode split; value uses the slowest replica's wall time", **c}))
    finish_engine_arm(world)


def run_prefill_only(args):
    """Chunked tensor-core prefill alone (the step before the decode path): N prompt tokens through
    ``Decoder(prefill_mode="tensor").prefill_ids``, timed with CUDA events; prompt tok/s and dense fp16 TFLOP/s
    (2 x the matrix weights a token actually passes - every layer but the last in full, of the last one the q / k / v
    projection; the LM head is not part of a prefill - + causal attention in the layers that run it)."""
    rank, world, device = init_engine_arm()
    from Model.Qwen06B_architecture import Decoder
    n = args.prefill_only
    weights = S.weights_to(S.make_weights(seed=0, max_seq_len=16), str(device))
    eng = Decoder(weights=weights, tokenizer=S.StubTokenizer(-1), verbose=False, max_seq_len=n + 8, device=str(device),
                  prefill_mode="tensor")
    prompt = S.make_prompt(n, seed=rank)
    for _ in range(max(args.warmup, 1)):
        eng.reset()
        eng.prefill_ids(prompt)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier(world)
    for a, b in ev:
        eng.reset()
        a.record()
        eng.prefill_ids(prompt)
        b.record()
    barrier(world)
    ms = statistics.mean(a.elapsed_time(b) for a, b in ev)
    ms = max_over_ranks(ms, world, device)
    # Work the pass executes: a prefill leaves only cache rows behind, so the last layer stops after its q / k / v
    # projection (its K and V rows); attention, O and the MLP run in the layers before it.
    per_layer_w = sum(S.math.prod(shape) for _, shape in S.LAYER_FIELDS if len(shape) == 2)
    qkv_w = sum(S.math.prod(shape) for name, shape in S.LAYER_FIELDS if name in ("q_proj", "k_proj", "v_proj"))
    full_layers = S.NUM_LAYERS - 1
    flops = n * 2.0 * (full_layers * per_layer_w + qkv_w) + full_layers * 4.0 * 16 * 128 * n * (n + 1) / 2
    if rank == 0:
        print(json.dumps({"metric": "chunked tensor-core prefill, prompt tok/s", "value": world * n / (ms / 1e3), "unit": UNIT,
                          "n_gpus": world, "prompt_tokens": n, "ms_per_prefill": ms, "tflops": flops / (ms / 1e3) / 1e12,
                          "steps": args.steps, "warmup": args.warmup, "dtype": "fp16", "data": "synthetic"}))
    finish_engine_arm(world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true",
                    help="headline workload only: skip the FP8 / NVFP4 / continuous-batching configurations of `extra`")
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
    ap.add_argument("--prefill-only", type=int, default=0, metavar="N",
                    help="instead of the headline workload: time the chunked tensor-core prefill of N prompt tokens")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prefilled context (default: benchmark config)")
    ap.add_argument("--decode-tokens", type=int, default=DECODE_TOKENS,
                    help="greedy tokens per step (default: benchmark config; smaller for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.prefill_only > 0:
        run_prefill_only(args)
    elif args.continuous > 0:
        run_continuous(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
