"""Regenerates the golden vectors under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py [--only tiny|full]

The reference project has no fixtures for the decode path, so these files pin
the oracle itself (tests/test_oracle.py re-derives them) and give the GPU parity
tests inputs and answers that do not need the oracle at full size.  Models are
the seeded synthetic ones of ``synthetic.make_weights``; nothing here reads the
reference checkout.

Files written:
  full_seed0_prompt32.json   Qwen3-0.6B shape (28 layers, vocab 151936), seed 0,
                             prompt = make_prompt(32, seed 0); 32 greedy tokens,
                             per-step top-8 logits, greedy margins (fp16 KV cache,
                             the oracle default), and the tokens / max logit shift
                             of the same run with an fp32 cache.
  full_seed0_prompt4096.json the benchmarked configuration: same model, prompt = make_prompt(4096,
                             seed 0) (4095 tokens prefilled in chunks, decode from the last one);
                             8 greedy tokens, per-step top-8 logits and greedy margins.
  tiny_l2_v4096.npz          2 layers, vocab 4096, norm_std 0.1, seed 3:
                             prompt 12 tokens, 8 greedy tokens, logits per step,
                             and the per-phase trace of the first decode step.
"""

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "qwen3-0.6b-megakernel-rtx-5090_b200"))

import synthetic as S  # noqa: E402
from oracle.decoder_ref import Decoder  # noqa: E402

TINY = dict(seed=3, num_layers=2, vocab_size=4096, norm_std=0.1, prompt_len=12, prompt_seed=5, steps=8,
            max_seq_len=64)
FULL = dict(seed=0, num_layers=28, vocab_size=151936, norm_std=0.0, prompt_len=32, prompt_seed=0, steps=32,
            max_seq_len=128)


FULL4096 = dict(seed=0, num_layers=28, vocab_size=151936, norm_std=0.0, prompt_len=4096, prompt_seed=0, steps=8,
                max_seq_len=4352)


def run(cfg, kv_dtype=torch.float16, trace_first=False):
    w = S.make_weights(seed=cfg["seed"], num_layers=cfg["num_layers"], vocab_size=cfg["vocab_size"],
                       norm_std=cfg["norm_std"], max_seq_len=cfg["max_seq_len"])
    ids = S.make_prompt(cfg["prompt_len"], seed=cfg["prompt_seed"], vocab_size=cfg["vocab_size"])
    d = Decoder(w, max_seq_len=cfg["max_seq_len"], kv_dtype=kv_dtype)
    d.prefill(ids[:-1])
    toks, logits, trace = [], [], None
    cur = ids[-1]
    for s in range(cfg["steps"]):
        cur = d.step(cur, trace=(trace_first and s == 0))
        if trace_first and s == 0:
            trace = d.trace
        toks.append(cur)
        logits.append(d.last_logits.clone())
    return ids, toks, torch.stack(logits), trace


def make_tiny():
    ids, toks, logits, trace = run(TINY, trace_first=True)
    out = dict(prompt=np.array(ids, np.int64), tokens=np.array(toks, np.int64),
               logits=logits.numpy().astype(np.float32))
    for li, tr in trace.items():
        for k, v in tr.items():
            out[f"l{li}_{k}"] = v[0].numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "tiny_l2_v4096.npz"), **out)
    print("tiny tokens", toks)


def make_full():
    ids, toks, logits, _ = run(FULL)
    top = torch.topk(logits, 8, dim=-1)
    margins = (top.values[:, 0] - top.values[:, 1]).tolist()
    ids32, toks32, logits32, _ = run(FULL, kv_dtype=torch.float32)
    doc = dict(config=FULL, prompt=ids, tokens=toks,
               top8_values=[[float(x) for x in r] for r in top.values.tolist()],
               top8_indices=top.indices.tolist(), margins=margins, min_margin=min(margins),
               fp32_kv_tokens=toks32,
               fp32_kv_max_abs_logit_diff=float((logits32 - logits).abs().max()))
    with open(os.path.join(HERE, "full_seed0_prompt32.json"), "w") as f:
        json.dump(doc, f, indent=1)
    print("full tokens", toks)
    print("min margin", min(margins), "fp32-kv same ids:", toks32 == toks,
          "max logit diff", doc["fp32_kv_max_abs_logit_diff"])


def make_full_ctx4096():
    ids, toks, logits, _ = run(FULL4096)
    top = torch.topk(logits, 8, dim=-1)
    margins = (top.values[:, 0] - top.values[:, 1]).tolist()
    doc = dict(config=FULL4096, prompt_seed=FULL4096["prompt_seed"], prompt_len=len(ids), prompt_head=ids[:8],
               prompt_tail=ids[-8:], tokens=toks,
               top8_values=[[float(x) for x in r] for r in top.values.tolist()],
               top8_indices=top.indices.tolist(), margins=margins, min_margin=min(margins))
    with open(os.path.join(HERE, "full_seed0_prompt4096.json"), "w") as f:
        json.dump(doc, f, indent=1)
    print("ctx4096 tokens", toks, "margins", margins)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", choices=["tiny", "full", "ctx4096"])
    a = ap.parse_args()
    if a.only in (None, "tiny"):
        make_tiny()
    if a.only in (None, "full"):
        make_full()
    if a.only in (None, "ctx4096"):
        make_full_ctx4096()
